"""Test client for the worker front end: the ggml RPC wire protocol as the reference's own test
client speaks it (third_party/llama.cpp/patches/0002 lines 1172-1490)."""
from __future__ import annotations

import ctypes as C
import socket
import struct

from mesh_llm_b200.capi import Tensor, check, lib

(ALLOC_BUFFER, GET_ALIGNMENT, GET_MAX_SIZE, BUFFER_GET_BASE, FREE_BUFFER, BUFFER_CLEAR, SET_TENSOR,
 SET_TENSOR_HASH, GET_TENSOR, COPY_TENSOR, GRAPH_COMPUTE, GET_DEVICE_MEMORY, INIT_TENSOR, GET_ALLOC_SIZE,
 HELLO, DEVICE_COUNT, GRAPH_RECOMPUTE, SET_TENSOR_GGUF, REGISTER_PEER, PUSH_TENSOR_TO_PEER,
 PEER_TENSOR_DATA) = range(21)


class Server:
    """in-process server on a free port"""

    def __init__(self, gguf_path=None):
        h = C.c_void_p()
        check(lib().b200_rpc_server_start(b"127.0.0.1", 0, str(gguf_path).encode() if gguf_path else None, C.byref(h)))
        self.h = h
        self.port = lib().b200_rpc_server_port(h)
        self.endpoint = f"127.0.0.1:{self.port}"

    def stop(self):
        if self.h:
            lib().b200_rpc_server_stop(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.stop()


class Client:
    def __init__(self, port, hello=True):
        self.s = socket.create_connection(("127.0.0.1", port), timeout=20)
        self.s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        if hello:
            major, minor, patch = self.hello()
            assert major == 4 and minor >= 1

    def close(self):
        self.s.close()

    def send(self, cmd, payload=b""):
        self.s.sendall(struct.pack("<BQ", cmd, len(payload)) + payload)

    def recv_exact(self, n):
        out = bytearray()
        while len(out) < n:
            chunk = self.s.recv(min(1 << 20, n - len(out)))
            if not chunk:
                raise ConnectionError("server closed the connection")
            out += chunk
        return bytes(out)

    def recv(self):
        (n,) = struct.unpack("<Q", self.recv_exact(8))
        return self.recv_exact(n)

    def call(self, cmd, payload=b""):
        self.send(cmd, payload)
        return self.recv()

    # ---- commands
    def hello(self):
        r = self.call(HELLO, bytes(24))
        assert len(r) == 28
        return r[0], r[1], r[2]

    def device_count(self):
        return struct.unpack("<I", self.call(DEVICE_COUNT))[0]

    def alloc_buffer(self, device, size):
        return struct.unpack("<QQ", self.call(ALLOC_BUFFER, struct.pack("<IQ", device, size)))

    def buffer_get_base(self, handle):
        return struct.unpack("<Q", self.call(BUFFER_GET_BASE, struct.pack("<Q", handle)))[0]

    def free_buffer(self, handle):
        return self.call(FREE_BUFFER, struct.pack("<Q", handle)) == b""

    def buffer_clear(self, handle, value):
        return self.call(BUFFER_CLEAR, struct.pack("<QB", handle, value)) == b""

    def set_tensor(self, tensor, offset, data):
        self.send(SET_TENSOR, bytes(tensor) + struct.pack("<Q", offset) + bytes(data))  # no response

    def get_tensor(self, tensor, offset, size):
        return self.call(GET_TENSOR, bytes(tensor) + struct.pack("<QQ", offset, size))

    def copy_tensor(self, src, dst):
        return self.call(COPY_TENSOR, bytes(src) + bytes(dst))[0]

    def register_peer(self, peer_id, endpoint):
        ep = endpoint.encode()[:127]
        return self.call(REGISTER_PEER, struct.pack("<I128s", peer_id, ep))[0]

    def push_tensor_to_peer(self, peer_id, src, dst, offset, size):
        return self.call(PUSH_TENSOR_TO_PEER, struct.pack("<I", peer_id) + bytes(src) + bytes(dst) +
                         struct.pack("<QQ", offset, size))[0]

    def set_tensor_gguf(self, tensor, offset=0):
        return self.call(SET_TENSOR_GGUF, bytes(tensor) + struct.pack("<Q", offset))[0]

    def graph_compute(self, device, node_ids, tensors):
        payload = struct.pack("<II", device, len(node_ids)) + b"".join(struct.pack("<Q", i) for i in node_ids)
        payload += struct.pack("<I", len(tensors)) + b"".join(bytes(t) for t in tensors)
        self.send(GRAPH_COMPUTE, payload)  # no response

    def graph_recompute(self, device):
        self.send(GRAPH_RECOMPUTE, struct.pack("<I", device))


def make_tensor(buffer, data, ne, type_=0, nb0=4, name="t", id_=0, op=0, src=()):
    """row-major tensor record in a remote buffer (strides in bytes, ne[0] contiguous)"""
    t = Tensor()
    t.id, t.type, t.buffer, t.data, t.op = id_, type_, buffer, data, op
    ne = list(ne) + [1] * (4 - len(ne))
    for i in range(4):
        t.ne[i] = ne[i]
    t.nb[0] = nb0
    stride = nb0 * ne[0]
    for i in range(1, 4):
        t.nb[i] = stride
        stride *= ne[i]
    for i, s in enumerate(src):
        t.src[i] = s
    t.name = name.encode()
    return t
