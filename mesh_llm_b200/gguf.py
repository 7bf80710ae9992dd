"""Host-side view of the library's GGUF reader: header scan, tensor index, selective reads.

Mirrors the scanner mesh-llm plans deployments with (mesh-client/src/models/gguf.rs) and the
worker-side load of a stage's own tensors from its local file (llama.cpp patches/0001,
SET_TENSOR_GGUF).  All parsing happens in libb200kq.so; this module only wraps the handles.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from .capi import GgufByteProfile, GgufMeta, GgufTensor, StageConfig, check, lib


class GgufFile:
    def __init__(self, path):
        h = C.c_void_p()
        check(lib().b200_gguf_open(str(path).encode(), C.byref(h)))
        self.h = h
        self.path = str(path)

    def close(self):
        if getattr(self, "h", None):
            lib().b200_gguf_close(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def meta(self):
        m = GgufMeta()
        check(lib().b200_gguf_get_meta(self.h, C.byref(m)))
        out = {name: getattr(m, name) for name, _ in GgufMeta._fields_}
        out["architecture"] = m.architecture.decode()
        out["tokenizer_model"] = m.tokenizer_model.decode()
        return out

    def tensors(self):
        out = []
        for i in range(lib().b200_gguf_tensor_count(self.h)):
            t = GgufTensor()
            check(lib().b200_gguf_tensor_info(self.h, i, C.byref(t)))
            out.append(dict(name=t.name.decode(), type=t.type, n_dims=t.n_dims, ne=list(t.ne),
                            file_offset=t.file_offset, nbytes=t.nbytes))
        return out

    def find(self, name):
        return lib().b200_gguf_find_tensor(self.h, name.encode())

    def read(self, name):
        i = self.find(name)
        if i < 0:
            raise KeyError(name)
        t = GgufTensor()
        check(lib().b200_gguf_tensor_info(self.h, i, C.byref(t)))
        buf = np.empty(t.nbytes, np.uint8)
        check(lib().b200_gguf_read_tensor(self.h, i, buf.ctypes.data, buf.size))
        return buf

    def byte_profile(self):
        p = GgufByteProfile()
        check(lib().b200_gguf_byte_profile(self.h, C.byref(p)))
        return {name: getattr(p, name) for name, _ in GgufByteProfile._fields_}

    def stage_config(self, layer_begin=0, layer_end=-1, n_ctx=4096, n_seq=1, n_ubatch=512, device=0):
        cfg = StageConfig()
        check(lib().b200_gguf_stage_config(self.h, layer_begin, layer_end, n_ctx, n_seq, n_ubatch, device,
                                           C.byref(cfg)))
        return cfg

    def write_expert_shard(self, expert_ids, dst_path):
        """trunk + the listed experts (router rows gathered, counts rewritten) -> bytes written"""
        ids = np.ascontiguousarray(expert_ids, dtype=np.int32)
        n = C.c_uint64()
        check(lib().b200_gguf_write_expert_shard(self.h, ids.ctypes.data, ids.size, str(dst_path).encode(), C.byref(n)))
        return n.value


def moe_assign(ranking, n_nodes, min_experts, overlap=1, mode=0):
    """Expert ids per node -> list of dict(experts, n_shared, n_unique); mode 0 = shared core +
    round-robin with overlap, mode 1 = shared core + snake draft"""
    rk = np.ascontiguousarray(ranking, dtype=np.uint32)
    out = []
    for node in range(max(1, n_nodes)):
        buf = np.zeros(rk.size, np.uint32)
        n, ns, nu = C.c_int32(), C.c_int32(), C.c_int32()
        check(lib().b200_moe_assign(rk.ctypes.data, rk.size, n_nodes, min_experts, overlap, mode, node,
                                    buf.ctypes.data, buf.size, C.byref(n), C.byref(ns), C.byref(nu)))
        out.append(dict(experts=buf[: n.value].tolist(), n_shared=ns.value, n_unique=nu.value))
    return out
