"""Host-side mirror of the op surface: thin wrappers that hand torch CUDA tensors to the C ABI.

Every function launches hand-written sm_100a kernels from libb200kq.so on the current torch
stream.  Tensors follow ggml's convention with the contiguous dimension last in torch terms:
weights [N, K-bytes] uint8, activations [M, K] float32.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import capi
from .capi import TYPE_F32, TYPE_Q4_K, TYPE_Q6_K, check, lib, ptr, cur_stream

Q4K_BYTES, Q6K_BYTES = 144, 210


def _dev(t):
    if not t.is_cuda:
        raise ValueError("expected a CUDA tensor: this library has no CPU path")
    return t


def row_bytes(type_, k):
    return lib().b200_row_bytes(type_, k)


def device_row_bytes(type_, k):
    return lib().b200_device_row_bytes(type_, k)


def upload_weights(type_, gguf_rows, n_rows, k, device="cuda"):
    """GGUF-layout rows (numpy/torch uint8) -> device-layout uint8 tensor [n_rows, device_row_bytes]."""
    src = torch.as_tensor(gguf_rows).reshape(-1).to(device=device, dtype=torch.uint8)
    if type_ != TYPE_Q6_K:
        return src.reshape(n_rows, -1).contiguous()
    pad = torch.zeros(16, dtype=torch.uint8, device=device)  # keep u16 reads of the tail in bounds
    src = torch.cat([src, pad])
    out = torch.zeros((n_rows, device_row_bytes(type_, k)), dtype=torch.uint8, device=device)
    check(lib().b200_repack_q6k(ptr(src), ptr(out), n_rows, k, cur_stream()))
    return out


def download_weights(type_, dev_rows, n_rows, k):
    """inverse of upload_weights -> uint8 tensor of GGUF bytes on the device"""
    if type_ != TYPE_Q6_K:
        return dev_rows.reshape(-1).clone()
    out = torch.empty(n_rows * row_bytes(type_, k), dtype=torch.uint8, device=dev_rows.device)
    check(lib().b200_unpack_q6k(ptr(dev_rows), ptr(out), n_rows, k, cur_stream()))
    return out


def quantize_act(x):
    x = _dev(x).contiguous().float()
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    d = torch.empty((M, K // 256), dtype=torch.float32, device=x.device)
    bs = torch.empty((M, K // 16), dtype=torch.int16, device=x.device)
    check(lib().b200_quantize_act(ptr(x), M, K, ptr(q), ptr(d), ptr(bs), cur_stream()))
    return q, d, bs


def mul_mat(type_, W, x, N, K, scratch=None):
    x = _dev(x).contiguous().float().reshape(-1, K)
    M = x.shape[0]
    need = lib().b200_mul_mat_scratch_bytes(M, K)
    if scratch is None or scratch.numel() < need:
        scratch = torch.empty(need, dtype=torch.uint8, device=x.device)
    y = torch.empty((M, N), dtype=torch.float32, device=x.device)
    check(lib().b200_mul_mat(type_, ptr(W), ptr(x), M, N, K, ptr(y), ptr(scratch), scratch.numel(),
                             cur_stream()))
    return y


def mul_mat_q8(type_, W, q, d, bs, N, K, bias=None, residual=None, out=None):
    M = q.shape[0]
    y = out if out is not None else torch.empty((M, N), dtype=torch.float32, device=q.device)
    check(lib().b200_mul_mat_q8(type_, ptr(W), ptr(q), ptr(d), ptr(bs), M, N, K, ptr(y), ptr(bias),
                                ptr(residual), cur_stream()))
    return y


def probe_int8_mma(n_mma=65536, repeats=5):
    """(TOP/s, ms) of a bare tcgen05.mma kind::i8 loop on every SM of the current device"""
    import ctypes as C

    tops, ms = C.c_double(0.0), C.c_double(0.0)
    check(lib().b200_probe_int8_mma(n_mma, repeats, C.byref(tops), C.byref(ms)))
    return tops.value, ms.value


def block_sums(type_, W, q, bs, N, K):
    M = q.shape[0]
    sumi = torch.empty((M, N, K // 256), dtype=torch.int32, device=q.device)
    summ = torch.empty((M, N, K // 256), dtype=torch.int32, device=q.device)
    check(lib().b200_block_sums(type_, ptr(W), ptr(q), ptr(bs), M, N, K, ptr(sumi), ptr(summ),
                                cur_stream()))
    return sumi, summ


def rms_norm(x, w, eps):
    x = _dev(x).contiguous().float()
    T, h = x.shape
    y = torch.empty_like(x)
    check(lib().b200_rms_norm(ptr(x), ptr(w), T, h, eps, ptr(y), cur_stream()))
    return y


def rope(x, pos, theta, neox):
    """x: [T, n_head, hd] f32 (copied), pos: [T] int32"""
    x = _dev(x).contiguous().float().clone()
    T, nh, hd = x.shape
    pos = pos.to(device=x.device, dtype=torch.int32).contiguous()
    check(lib().b200_rope(ptr(x), ptr(pos), T, nh, hd, theta, int(neox), cur_stream()))
    return x


def swiglu(g, u):
    y = torch.empty_like(g)
    check(lib().b200_swiglu(ptr(g), ptr(u), g.numel(), ptr(y), cur_stream()))
    return y


def add(a, b):
    y = torch.empty_like(a)
    check(lib().b200_add(ptr(a), ptr(b), a.numel(), ptr(y), cur_stream()))
    return y


def cpy_f32_f16(x):
    y = torch.empty(x.shape, dtype=torch.float16, device=x.device)
    check(lib().b200_cpy_f32_f16(ptr(x), x.numel(), ptr(y), cur_stream()))
    return y


def attention(q, k_cache, v_cache, pos0):
    """q: [T, n_head, hd] f32; caches: [n_ctx, n_kv, hd] f16 holding rows [0, pos0+T)"""
    q = _dev(q).contiguous().float()
    T, nh, hd = q.shape
    n_ctx, nkv, _ = k_cache.shape
    need = lib().b200_attention_scratch_bytes(T, nh, hd, n_ctx)
    scratch = torch.empty(need, dtype=torch.uint8, device=q.device)
    out = torch.empty_like(q)
    check(lib().b200_attention(ptr(q), ptr(k_cache), ptr(v_cache), T, pos0, nh, nkv, hd, ptr(out),
                               ptr(scratch), need, cur_stream()))
    return out


def kv_row_bytes(type_, hd):
    return int(lib().b200_kv_row_bytes(type_, hd))


def kv_types_for_model_bytes(model_bytes):
    """(k_type, v_type) mesh-llm starts a server with for a model file of this size"""
    k, v = C.c_uint32(), C.c_uint32()
    lib().b200_kv_types_for_model_bytes(int(model_bytes), C.byref(k), C.byref(v))
    return k.value, v.value


def kv_cache(type_, n_ctx, n_kv, hd, device="cuda"):
    """zeroed cache of n_ctx positions: uint8 [n_ctx, n_kv, row bytes]"""
    return torch.zeros((n_ctx, n_kv, kv_row_bytes(type_, hd)), dtype=torch.uint8, device=device)


def kv_store(k, v, pos, k_cache, v_cache, k_type, v_type, theta, neox):
    """k, v: [T, n_kv, hd] f32 rows of the new tokens; k is rotated at pos[t]; both are written at
    those positions into caches made by kv_cache()"""
    k = _dev(k).contiguous().float()
    v = _dev(v).contiguous().float()
    T, nkv, hd = k.shape
    pos = pos.to(device=k.device, dtype=torch.int32).contiguous()
    check(lib().b200_kv_store(ptr(k), ptr(v), ptr(pos), T, nkv, hd, theta, int(neox), k_type, v_type,
                              ptr(k_cache), ptr(v_cache), cur_stream()))


def attention_kv(q, k_cache, v_cache, k_type, v_type, pos0):
    """attention() over caches of the given row types (made by kv_cache / kv_store)"""
    q = _dev(q).contiguous().float()
    T, nh, hd = q.shape
    n_ctx, nkv, _ = k_cache.shape
    need = lib().b200_attention_scratch_bytes(T, nh, hd, n_ctx)
    scratch = torch.empty(need, dtype=torch.uint8, device=q.device)
    out = torch.empty_like(q)
    check(lib().b200_attention_kv(ptr(q), ptr(k_cache), ptr(v_cache), k_type, v_type, T, pos0, nh, nkv, hd,
                                  ptr(out), ptr(scratch), need, cur_stream()))
    return out


def get_rows(type_, W, ids, K):
    ids = ids.to(device=W.device, dtype=torch.int32).contiguous()
    y = torch.empty((ids.numel(), K), dtype=torch.float32, device=W.device)
    check(lib().b200_get_rows(type_, ptr(W), ptr(ids), ids.numel(), K, ptr(y), cur_stream()))
    return y


def argmax(x):
    x = _dev(x).contiguous().float()
    idx = torch.empty(x.shape[0], dtype=torch.int32, device=x.device)
    check(lib().b200_argmax(ptr(x), x.shape[0], x.shape[1], ptr(idx), cur_stream()))
    return idx


def logit_signals(logits, chosen=None):
    """-> dict of device tensors: entropy [T] (bits), margin [T], p_chosen [T], top_p [T][5], top_id [T][5],
    argmax [T]; the statistics the reference's server takes from the full-vocabulary softmax per token"""
    logits = _dev(logits).contiguous().float()
    T, n = logits.shape
    nb = lib().b200_logit_signals_scratch_bytes(T)
    scratch = torch.zeros(nb, dtype=torch.uint8, device=logits.device)
    sig = torch.empty((T, 13), dtype=torch.float32, device=logits.device)  # 3 + 5 floats, 5 int32
    am = torch.empty(T, dtype=torch.int32, device=logits.device)
    ch = None if chosen is None else _dev(chosen).to(torch.int32).contiguous()
    check(lib().b200_logit_signals(ptr(logits), T, n, ptr(ch), ptr(sig), ptr(am), ptr(scratch), nb, cur_stream()))
    return dict(entropy=sig[:, 0], margin=sig[:, 1], p_chosen=sig[:, 2], top_p=sig[:, 3:8],
                top_id=sig[:, 8:13].contiguous().view(torch.int32), argmax=am)


def mul_mat_id(type_, W, n_expert, x, ids, N, K):
    """MUL_MAT_ID: W [n_expert * N, row bytes] device layout, x [rows, K] f32, ids [n_pairs] int32 (n_pairs a
    multiple of rows: pair p uses row p // (n_pairs // rows)) -> y [n_pairs, N]"""
    x = _dev(x).contiguous().float().reshape(-1, K)
    ids = _dev(ids).contiguous().to(torch.int32).reshape(-1)
    rows, pairs = x.shape[0], ids.numel()
    need = lib().b200_mul_mat_id_scratch_bytes(rows, pairs, K, n_expert)
    scratch = torch.empty(need, dtype=torch.uint8, device=x.device)
    y = torch.empty((pairs, N), dtype=torch.float32, device=x.device)
    check(lib().b200_mul_mat_id(type_, ptr(W), n_expert, ptr(x), rows, ptr(ids), pairs, N, K, ptr(y), ptr(scratch), need,
                                cur_stream()))
    return y


def moe_route(logits, k, mask=None):
    logits = _dev(logits).contiguous().float()
    T, E = logits.shape
    ids = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    if mask is not None:  # uint8 device tensor, one entry per expert, nonzero = allowed
        mask = (_dev(mask) != 0).to(torch.uint8).contiguous()
        if mask.numel() != E:
            raise ValueError("expert mask needs one entry per expert")
    check(lib().b200_moe_route_masked(ptr(logits), T, E, k, ptr(mask), ptr(ids), ptr(w), cur_stream()))
    return ids, w
