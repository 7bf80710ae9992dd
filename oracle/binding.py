"""ctypes binding of the CPU oracle (oracle/kquant_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs import this module; the
product package never does.  Arrays are numpy, row-major, shaped as the C header documents.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libkquant_oracle.so")

TYPE_F32, TYPE_F16, TYPE_Q4_0, TYPE_Q8_0, TYPE_Q4_K, TYPE_Q6_K = 0, 1, 2, 8, 12, 14
Q4K_BYTES, Q6K_BYTES, QK_K = 144, 210, 256


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "kquant_oracle.c")
    hdr = os.path.join(_HERE, "kquant_oracle.h")
    stale = (not os.path.exists(_SO)) or any(
        os.path.exists(p) and os.path.getmtime(p) > os.path.getmtime(_SO) for p in (src, hdr)
    )
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-s"] + (["-B"] if force else []))
    return _SO


class Config(C.Structure):
    _fields_ = [
        ("n_layer", C.c_int32), ("layer_begin", C.c_int32), ("layer_end", C.c_int32),
        ("n_embd", C.c_int32), ("n_head", C.c_int32), ("n_head_kv", C.c_int32),
        ("head_dim", C.c_int32), ("n_ff", C.c_int32), ("n_vocab", C.c_int32),
        ("n_expert", C.c_int32), ("n_expert_used", C.c_int32), ("n_ff_exp", C.c_int32),
        ("n_ctx", C.c_int32), ("n_seq", C.c_int32),
        ("rope_neox", C.c_int32), ("qkv_bias", C.c_int32), ("qk_norm", C.c_int32),
        ("has_embd", C.c_int32), ("has_output", C.c_int32),
        ("rms_eps", C.c_float), ("rope_theta", C.c_float),
        ("kv_type_k", C.c_int32), ("kv_type_v", C.c_int32),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        vp, i64, i32 = C.c_void_p, C.c_int64, C.c_int32
        L.orc_dequant_q4k.argtypes = [vp, i64, vp]
        L.orc_dequant_q6k.argtypes = [vp, i64, vp]
        L.orc_quantize_q4k.argtypes = [vp, i64, vp]
        L.orc_quantize_q6k.argtypes = [vp, i64, vp]
        L.orc_row_bytes.argtypes = [i32, i64]
        L.orc_row_bytes.restype = i64
        L.orc_quantize_act.argtypes = [vp, i64, i64, vp, vp, vp]
        L.orc_block_sums.argtypes = [i32, vp, vp, vp, i64, i64, i64, vp, vp]
        L.orc_mul_mat.argtypes = [i32, vp, vp, i64, i64, i64, vp]
        L.orc_mul_mat_q8.argtypes = [i32, vp, vp, vp, vp, i64, i64, i64, vp]
        L.orc_rms_norm.argtypes = [vp, vp, i64, i64, C.c_float, vp]
        L.orc_rope.argtypes = [vp, vp, i64, i64, i64, C.c_float, i32]
        L.orc_rope_inv_freq.argtypes = [C.c_float, i64, vp]
        L.orc_swiglu.argtypes = [vp, vp, i64, vp]
        L.orc_f32_to_f16.argtypes = [vp, i64, vp]
        L.orc_f16_to_f32.argtypes = [vp, i64, vp]
        L.orc_attention.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, vp]
        L.orc_get_rows.argtypes = [i32, vp, vp, i64, i64, vp]
        L.orc_quantize_q8_0.argtypes = [vp, i64, vp]
        L.orc_quantize_q4_0.argtypes = [vp, i64, vp]
        L.orc_dequant_q8_0.argtypes = [vp, i64, vp]
        L.orc_dequant_q4_0.argtypes = [vp, i64, vp]
        L.orc_kv_round_trip.argtypes = [i32, vp, i64, vp]
        L.orc_argmax.argtypes = [vp, i64, i64, vp]
        L.orc_moe_route.argtypes = [vp, i64, i64, i64, vp, vp]
        L.orc_moe_route_masked.argtypes = [vp, i64, i64, i64, vp, vp, vp]
        L.orc_model_set_expert_mask.argtypes = [vp, vp, i32]
        L.orc_model_set_expert_mask.restype = i32
        L.orc_model_create.argtypes = [C.POINTER(Config)]
        L.orc_model_create.restype = vp
        L.orc_model_free.argtypes = [vp]
        L.orc_model_generate.argtypes = [vp, C.c_uint64]
        L.orc_model_get_tensor.argtypes = [vp, C.c_char_p, C.POINTER(i32), C.POINTER(vp),
                                           C.POINTER(i64), C.POINTER(i64 * 3)]
        L.orc_model_get_tensor.restype = i32
        L.orc_model_set_tensor.argtypes = [vp, C.c_char_p, i32, vp, i64]
        L.orc_model_set_tensor.restype = i32
        L.orc_model_n_tensors.argtypes = [vp]
        L.orc_model_n_tensors.restype = i32
        L.orc_model_tensor_name.argtypes = [vp, i32]
        L.orc_model_tensor_name.restype = C.c_char_p
        L.orc_model_forward.argtypes = [vp, i32, vp, vp, i64, i64, vp, vp]
        L.orc_model_forward.restype = i32
        L.orc_set_threads.argtypes = [i32]
        L.orc_get_threads.restype = i32
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def row_bytes(type_, k):
    return int(lib().orc_row_bytes(type_, k))


def dequantize(type_, blocks):
    blocks = _c(blocks, np.uint8).reshape(-1)
    bpb = Q4K_BYTES if type_ == TYPE_Q4_K else Q6K_BYTES
    nb = blocks.size // bpb
    out = np.empty(nb * 256, np.float32)
    (lib().orc_dequant_q4k if type_ == TYPE_Q4_K else lib().orc_dequant_q6k)(_p(blocks), nb, _p(out))
    return out


def quantize_weights(type_, x):
    """x: [..., K] f32 (K % 256 == 0) -> uint8 [..., K/256*bytes]"""
    x = _c(x, np.float32)
    bpb = Q4K_BYTES if type_ == TYPE_Q4_K else Q6K_BYTES
    out = np.empty(x.shape[:-1] + (x.shape[-1] // 256 * bpb,), np.uint8)
    (lib().orc_quantize_q4k if type_ == TYPE_Q4_K else lib().orc_quantize_q6k)(_p(x), x.size, _p(out))
    return out


def quantize_act(x):
    """x: [M, K] f32 -> (q int8 [M,K], d f32 [M,K/256], bsum16 int16 [M,K/16])"""
    x = _c(x, np.float32)
    M, K = x.shape
    q = np.empty((M, K), np.int8)
    d = np.empty((M, K // 256), np.float32)
    bs = np.empty((M, K // 16), np.int16)
    lib().orc_quantize_act(_p(x), M, K, _p(q), _p(d), _p(bs))
    return q, d, bs


def block_sums(type_, W, q, bs, N, K):
    W = _c(W, np.uint8)
    M = q.shape[0]
    sumi = np.empty((M, N, K // 256), np.int32)
    summ = np.zeros((M, N, K // 256), np.int32)
    lib().orc_block_sums(type_, _p(W), _p(_c(q, np.int8)), _p(_c(bs, np.int16)), M, N, K,
                         _p(sumi), _p(summ))
    return sumi, summ


def mul_mat(type_, W, x, N, K):
    W = _c(W, np.uint8)
    x = _c(x, np.float32).reshape(-1, K)
    M = x.shape[0]
    y = np.empty((M, N), np.float32)
    lib().orc_mul_mat(type_, _p(W), _p(x), M, N, K, _p(y))
    return y


def rms_norm(x, w, eps):
    x = _c(x, np.float32)
    T, h = x.shape
    y = np.empty_like(x)
    w = None if w is None else _c(w, np.float32)
    lib().orc_rms_norm(_p(x), _p(w), T, h, eps, _p(y))
    return y


def rope(x, pos, theta, neox):
    """x: [T, n_head, hd]"""
    x = _c(x, np.float32).copy()
    T, nh, hd = x.shape
    pos = _c(pos, np.int32)
    lib().orc_rope(_p(x), _p(pos), T, nh, hd, theta, int(neox))
    return x


def rope_inv_freq(theta, hd):
    out = np.empty(hd // 2, np.float32)
    lib().orc_rope_inv_freq(theta, hd, _p(out))
    return out


def swiglu(g, u):
    g, u = _c(g, np.float32), _c(u, np.float32)
    y = np.empty_like(g)
    lib().orc_swiglu(_p(g), _p(u), g.size, _p(y))
    return y


def f32_to_f16(x):
    x = _c(x, np.float32)
    y = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_f16(_p(x), x.size, _p(y))
    return y


def attention(q, kc, vc, pos0):
    """q: [T, n_head, hd] f32; kc/vc: [n_ctx, n_kv, hd] uint16 (f16 bits)"""
    q = _c(q, np.float32)
    kc, vc = _c(kc, np.uint16), _c(vc, np.uint16)
    T, nh, hd = q.shape
    out = np.empty_like(q)
    lib().orc_attention(_p(q), _p(kc), _p(vc), T, pos0, nh, kc.shape[1], hd, _p(out))
    return out


def kv_quantize(type_, x):
    """x: [..., n] f32 (n % 32 == 0) -> ggml q8_0 / q4_0 blocks, uint8 [..., n/32 * (34 | 18)]"""
    x = _c(x, np.float32)
    bpb = 34 if type_ == TYPE_Q8_0 else 18
    out = np.empty(x.shape[:-1] + (x.shape[-1] // 32 * bpb,), np.uint8)
    (lib().orc_quantize_q8_0 if type_ == TYPE_Q8_0 else lib().orc_quantize_q4_0)(_p(x), x.size, _p(out))
    return out


def kv_dequantize(type_, blocks):
    blocks = _c(blocks, np.uint8)
    bpb = 34 if type_ == TYPE_Q8_0 else 18
    nb = blocks.size // bpb
    out = np.empty(nb * 32, np.float32)
    (lib().orc_dequant_q8_0 if type_ == TYPE_Q8_0 else lib().orc_dequant_q4_0)(_p(blocks), nb, _p(out))
    return out.reshape(blocks.shape[:-1] + (blocks.shape[-1] // bpb * 32,))


def kv_round_trip(type_, x):
    """the f16 values attention sees for rows stored in a cache of `type_` (F16, Q8_0 or Q4_0)"""
    x = _c(x, np.float32)
    y = np.empty(x.shape, np.uint16)
    lib().orc_kv_round_trip(type_, _p(x), x.size, _p(y))
    return y


def get_rows(type_, W, ids, K):
    W = _c(W, np.uint8)
    ids = _c(ids, np.int32)
    y = np.empty((ids.size, K), np.float32)
    lib().orc_get_rows(type_, _p(W), _p(ids), ids.size, K, _p(y))
    return y


def argmax(x):
    x = _c(x, np.float32)
    idx = np.empty(x.shape[0], np.int32)
    lib().orc_argmax(_p(x), x.shape[0], x.shape[1], _p(idx))
    return idx


def moe_route(logits, k, mask=None):
    """mask: one entry per expert, nonzero = allowed (the reference's expert mask); None = all"""
    logits = _c(logits, np.float32)
    T, E = logits.shape
    ids = np.empty((T, k), np.int32)
    w = np.empty((T, k), np.float32)
    if mask is None:
        lib().orc_moe_route(_p(logits), T, E, k, _p(ids), _p(w))
    else:
        mask = _c(np.asarray(mask) != 0, np.uint8)
        assert mask.size == E
        lib().orc_moe_route_masked(_p(logits), T, E, k, _p(mask), _p(ids), _p(w))
    return ids, w


class Model:
    """One stage (layer range) of a synthetic Q4_K_M model held in host memory."""

    def __init__(self, **kw):
        cfg = Config()
        defaults = dict(n_expert=0, n_expert_used=0, n_ff_exp=0, n_seq=1, rope_neox=1, qkv_bias=0,
                        qk_norm=0, has_embd=1, has_output=1, rms_eps=1e-6, rope_theta=1e6,
                        layer_begin=0)
        defaults.update(kw)
        if "layer_end" not in defaults:
            defaults["layer_end"] = defaults["n_layer"]
        for k, v in defaults.items():
            setattr(cfg, k, v)
        self.cfg = cfg
        self.h = lib().orc_model_create(C.byref(cfg))

    def close(self):
        if self.h:
            lib().orc_model_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def generate(self, seed):
        lib().orc_model_generate(self.h, seed)

    def tensor_names(self):
        n = lib().orc_model_n_tensors(self.h)
        return [lib().orc_model_tensor_name(self.h, i).decode() for i in range(n)]

    def tensor(self, name):
        """-> (type, uint8 view of the bytes, ne[3])"""
        ty, ptr, nb, ne = C.c_int32(), C.c_void_p(), C.c_int64(), (C.c_int64 * 3)()
        ok = lib().orc_model_get_tensor(self.h, name.encode(), C.byref(ty), C.byref(ptr),
                                        C.byref(nb), C.byref(ne))
        if not ok:
            raise KeyError(name)
        buf = (C.c_uint8 * nb.value).from_address(ptr.value)
        return ty.value, np.frombuffer(buf, np.uint8), tuple(ne)

    def set_tensor(self, name, type_, data):
        data = _c(data, np.uint8).reshape(-1)
        if not lib().orc_model_set_tensor(self.h, name.encode(), type_, _p(data), data.size):
            raise ValueError(f"set_tensor({name}) rejected")

    def set_expert_mask(self, mask):
        """mask: one entry per expert (nonzero = allowed) or None to clear; -> 0, or -1 on a wrong length"""
        if mask is None:
            return lib().orc_model_set_expert_mask(self.h, None, 0)
        mask = _c(np.asarray(mask) != 0, np.uint8)
        return lib().orc_model_set_expert_mask(self.h, _p(mask), mask.size)

    def forward(self, tokens=None, hidden_in=None, pos0=0, seq=0, want_logits=True):
        c = self.cfg
        if tokens is not None:
            tokens = _c(tokens, np.int32)
            T = tokens.size
        else:
            hidden_in = _c(hidden_in, np.float32)
            T = hidden_in.shape[0]
        hidden = np.empty((T, c.n_embd), np.float32)
        logits = np.empty((T, c.n_vocab), np.float32) if (c.has_output and want_logits) else None
        rc = lib().orc_model_forward(self.h, seq, _p(tokens), _p(hidden_in), T, pos0, _p(hidden),
                                     _p(logits))
        if rc != 0:
            raise RuntimeError(f"orc_model_forward -> {rc}")
        return hidden, logits
