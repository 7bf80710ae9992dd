"""Host-side mirror of the peer-memory hand-off between two stages (libb200kq.so does the work).

The receiving stage owns an `Endpoint` (a ring of landing slots in its HBM); the sending stage holds
a `Sender` mapped onto it, either inside one process (`Endpoint.local_sender()`) or from another
process through the 64-byte handle (`Endpoint.handle()` -> `Sender.open(handle, ...)`).  Payloads are
numbered 0, 1, 2, ... on both sides.  What this replaces in the reference: the activation's trip
through ggml-RPC between two workers (third_party/llama.cpp/patches/0002 lines 544-735).
"""
from __future__ import annotations

import ctypes as C

from .capi import check, cur_stream, lib, ptr


class HandoffTimeout(RuntimeError):
    pass


class _Base:
    h = None

    def status(self):
        """0 ok; 1 a send found no free slot in time; 2 a wait saw no payload in time.  Synchronise first."""
        v = C.c_int32()
        check(lib().b200_handoff_status(self.h, C.byref(v)))
        return v.value

    def raise_on_timeout(self):
        s = self.status()
        if s:
            raise HandoffTimeout({1: "hand-off: no free landing slot in time", 2: "hand-off: payload did not arrive in time"}.get(s, str(s)))

    def close(self):
        if self.h:
            lib().b200_handoff_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Endpoint(_Base):
    def __init__(self, slot_bytes, n_slots=16):
        self.slot_bytes, self.n_slots, self.next = slot_bytes, n_slots, 0
        h = C.c_void_p()
        check(lib().b200_handoff_create(slot_bytes, n_slots, C.byref(h)))
        self.h = h

    def handle(self):
        buf = C.create_string_buffer(64)
        check(lib().b200_handoff_export(self.h, buf))
        return buf.raw

    def local_sender(self):
        return Sender(_local=self)

    def wait(self, dst, limit_ns=0):
        """next payload -> dst (a contiguous device tensor)"""
        nbytes = dst.numel() * dst.element_size()
        check(lib().b200_handoff_wait(self.h, ptr(dst), nbytes, self.next, limit_ns, None, cur_stream()))
        self.next += 1

    def wait_in_place(self, nbytes, limit_ns=0):
        """-> (device address of the next payload, its number); call release(number) after reading it"""
        slot = C.c_void_p()
        check(lib().b200_handoff_wait(self.h, None, nbytes, self.next, limit_ns, C.byref(slot), cur_stream()))
        self.next += 1
        return slot.value, self.next - 1

    def release(self, seqno):
        check(lib().b200_handoff_release(self.h, seqno, cur_stream()))


class Sender(_Base):
    def __init__(self, _local=None, _handle=None, slot_bytes=0, n_slots=0):
        h = C.c_void_p()
        if _local is not None:
            check(lib().b200_handoff_open_local(_local.h, C.byref(h)))
            self._keep = _local  # the mapping points into the endpoint's memory
        else:
            check(lib().b200_handoff_open(_handle, slot_bytes, n_slots, C.byref(h)))
        self.h, self.next = h, 0

    @classmethod
    def open(cls, handle, slot_bytes, n_slots):
        return cls(_handle=handle, slot_bytes=slot_bytes, n_slots=n_slots)

    def send(self, src, limit_ns=0):
        nbytes = src.numel() * src.element_size()
        check(lib().b200_handoff_send(self.h, ptr(src), nbytes, self.next, limit_ns, cur_stream()))
        self.next += 1
