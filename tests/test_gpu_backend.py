"""The ggml-shaped boundary on the GPU: buffers, set/get with the Q6_K repack, the stage hand-off
copy, and graph_compute over hot-path ops, all through the C ABI.

The hand-off cases mirror the reference's own exactness test for direct tensor pushes
(third_party/llama.cpp/patches/0002, test_direct_push lines 1612-1745 and test_large_push): a
byte-exact full copy, a partial window (offset 1024, size 2048) that must leave the rest of the
destination untouched, the reverse direction, and a 16 MB transfer.
"""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import binding as orc

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")

OP = dict(NONE=0, MUL_MAT=1, MUL_MAT_ID=2, RMS_NORM=3, MUL=4, ADD=5, ROPE=6, SWIGLU=7, GET_ROWS=8, CPY=9,
          ATTN=10, MOE_ROUTE=11, ARGMAX=12)
F32, F16, Q4K, Q6K, I32 = 0, 1, 12, 14, 26


class Buf:
    def __init__(self, dev, size):
        from mesh_llm_b200.capi import check, lib

        self.h = C.c_void_p()
        check(lib().b200_buffer_alloc(dev, size, C.byref(self.h)))
        self.base = lib().b200_buffer_get_base(self.h)
        self.size, self.off, self.next_id = size, 0, 1

    def tensor(self, type_, ne, name="t"):
        from mesh_llm_b200.capi import Tensor, check, lib

        ne = list(ne) + [1] * (4 - len(ne))
        t = Tensor()
        t.id = id(self) % 100000 * 1000 + self.next_id
        self.next_id += 1
        t.type = type_
        t.buffer = self.h.value
        for i in range(4):
            t.ne[i] = ne[i]
        t.name = name.encode()
        t.data = self.base + self.off
        sz = lib().b200_buft_alloc_size(type_, C.byref((C.c_uint32 * 4)(*ne)))
        self.off += sz
        assert self.off <= self.size
        check(lib().b200_buffer_init_tensor(self.h, C.byref(t)))
        return t

    def set(self, t, data, offset=0):
        from mesh_llm_b200.capi import check, lib

        data = np.ascontiguousarray(data)
        check(lib().b200_buffer_set_tensor(self.h, C.byref(t), data.ctypes.data, offset, data.nbytes))

    def get(self, t, nbytes, offset=0, dtype=np.uint8):
        from mesh_llm_b200.capi import check, lib

        out = np.empty(nbytes, np.uint8)
        check(lib().b200_buffer_get_tensor(self.h, C.byref(t), out.ctypes.data, offset, nbytes))
        return out.view(dtype)

    def free(self):
        from mesh_llm_b200.capi import lib

        lib().b200_buffer_free(self.h)


def test_registry_and_buffer_type():
    from mesh_llm_b200.capi import lib

    L = lib()
    assert L.b200_reg_name() == b"B200" and L.b200_reg_device_count() >= 1
    name = C.create_string_buffer(32)
    assert L.b200_dev_name(0, name, 32) == 0 and name.value == b"B200_0"
    free, total = C.c_size_t(), C.c_size_t()
    assert L.b200_dev_memory(0, C.byref(free), C.byref(total)) == 0 and 0 < free.value <= total.value
    assert L.b200_buft_alignment() == 256
    assert L.b200_dev_supports_op(OP["MUL_MAT"], Q4K, F32) == 1
    assert L.b200_dev_supports_op(OP["MUL_MAT"], 2, F32) == 0  # Q4_0 is not on the path
    ne = (C.c_uint32 * 4)(5120, 3, 1, 1)
    assert L.b200_buft_alloc_size(Q6K, C.byref(ne)) >= 3 * 4208
    assert L.b200_buft_alloc_size(Q4K, C.byref(ne)) == (3 * 2880 + 255) // 256 * 256


def test_set_get_round_trips_including_partial_q6k_windows():
    rng = np.random.default_rng(0)
    buf = Buf(0, 1 << 20)
    for ty, rb in ((Q4K, 144 * 3), (Q6K, 210 * 3), (F32, 768 * 4)):
        t = buf.tensor(ty, (768, 11))
        data = rng.integers(0, 256, 11 * rb, dtype=np.uint8)
        buf.set(t, data)
        np.testing.assert_array_equal(buf.get(t, data.size), data)
        # partial window that starts and ends inside rows
        patch = rng.integers(0, 256, 1000, dtype=np.uint8)
        buf.set(t, patch, offset=777)
        data[777:1777] = patch
        np.testing.assert_array_equal(buf.get(t, data.size), data)
        np.testing.assert_array_equal(buf.get(t, 333, offset=1500), data[1500:1833])
    buf.free()


def test_bounds_are_enforced():
    from mesh_llm_b200.capi import B200Error, Tensor, check, lib

    buf = Buf(0, 4096)
    t = buf.tensor(F32, (256,))
    with pytest.raises(B200Error):
        buf.set(t, np.zeros(2048, np.uint8))  # larger than the tensor
    with pytest.raises(B200Error):
        buf.get(t, 16, offset=1020)
    bad = Tensor()
    C.memmove(C.byref(bad), C.byref(t), C.sizeof(Tensor))
    bad.ne[0] = 4096  # would run past the end of the buffer
    assert lib().b200_buffer_init_tensor(buf.h, C.byref(bad)) == -5
    other = Buf(0, 4096)
    with pytest.raises(B200Error):
        other.set(t, np.zeros(16, np.uint8))  # tensor of another buffer
    buf.free()
    other.free()


@pytest.mark.parametrize("two_devices", [False, True])
def test_stage_handoff_copy_is_byte_exact(two_devices):
    import torch
    from mesh_llm_b200.capi import lib

    if two_devices and torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    g = np.load(os.path.join(GOLD, "handoff_pattern.npz"))
    n = g["forward"].size
    a, b = Buf(0, 1 << 25), Buf(1 if two_devices else 0, 1 << 25)
    ta, tb = a.tensor(F32, (n // 4,)), b.tensor(F32, (n // 4,))
    L = lib()
    a.set(ta, g["forward"])
    assert L.b200_buffer_cpy_tensor(C.byref(ta), C.byref(tb), 0, n) == 1
    np.testing.assert_array_equal(b.get(tb, n), g["forward"])
    # partial push: offset 1024, size 2048; everything else stays zero
    b.set(tb, np.zeros(n, np.uint8))
    off, size = int(g["partial_offset"]), int(g["partial_size"])
    assert L.b200_buffer_cpy_tensor(C.byref(ta), C.byref(tb), off, size) == 1
    got = b.get(tb, n)
    assert not got[:off].any() and not got[off + size:].any()
    np.testing.assert_array_equal(got[off:off + size], g["forward"][off:off + size])
    # reverse direction
    b.set(tb, g["reverse"])
    assert L.b200_buffer_cpy_tensor(C.byref(tb), C.byref(ta), 0, n) == 1
    np.testing.assert_array_equal(a.get(ta, n), g["reverse"])
    # 16 MB
    big = int(g["large_bytes"])
    la, lb = a.tensor(F32, (big // 4,)), b.tensor(F32, (big // 4,))
    payload = np.random.default_rng(1).integers(0, 256, big, dtype=np.uint8)
    a.set(la, payload)
    assert L.b200_buffer_cpy_tensor(C.byref(la), C.byref(lb), 0, big) == 1
    np.testing.assert_array_equal(b.get(lb, big), payload)
    # a window past the end is refused (the caller then falls back to get + set)
    assert L.b200_buffer_cpy_tensor(C.byref(ta), C.byref(tb), n - 8, 64) == 0
    a.free()
    b.free()


def _f32bits(x):
    return int(np.float32(x).view(np.int32))


def test_graph_compute_runs_a_dense_ffn_block_like_the_oracle():
    """norm -> mul(weight) -> {gate, up} mul_mat -> swiglu -> down mul_mat -> add(residual) -> argmax"""
    from mesh_llm_b200.capi import Tensor, check, lib

    rng = np.random.default_rng(2)
    h, ff, T = 512, 1024, 5
    buf = Buf(0, 1 << 24)
    x = rng.standard_normal((T, h)).astype(np.float32)
    wn = (1 + 0.02 * rng.standard_normal(h)).astype(np.float32)
    Wg = orc.quantize_weights(orc.TYPE_Q4_K, (rng.standard_normal((ff, h)) * 0.02).astype(np.float32))
    Wu = orc.quantize_weights(orc.TYPE_Q4_K, (rng.standard_normal((ff, h)) * 0.02).astype(np.float32))
    Wd = orc.quantize_weights(orc.TYPE_Q6_K, (rng.standard_normal((h, ff)) * 0.02).astype(np.float32))
    t_x, t_wn = buf.tensor(F32, (h, T), "x"), buf.tensor(F32, (h,), "wn")
    t_g, t_u, t_d = buf.tensor(Q4K, (h, ff), "Wg"), buf.tensor(Q4K, (h, ff), "Wu"), buf.tensor(Q6K, (ff, h), "Wd")
    for t, d in ((t_x, x), (t_wn, wn), (t_g, Wg), (t_u, Wu), (t_d, Wd)):
        buf.set(t, d)

    def node(op, type_, ne, srcs, name, params=()):
        t = buf.tensor(type_, ne, name)
        t.op = OP[op]
        for i, s in enumerate(srcs):
            t.src[i] = s.id
        for i, p in enumerate(params):
            t.op_params[i] = p
        return t

    n1 = node("RMS_NORM", F32, (h, T), [t_x], "norm", [_f32bits(1e-6)])
    n2 = node("MUL", F32, (h, T), [n1, t_wn], "normw")
    n3 = node("MUL_MAT", F32, (ff, T), [t_g, n2], "gate")
    n4 = node("MUL_MAT", F32, (ff, T), [t_u, n2], "up")
    n5 = node("SWIGLU", F32, (ff, T), [n3, n4], "act")
    n6 = node("MUL_MAT", F32, (h, T), [t_d, n5], "down")
    n7 = node("ADD", F32, (h, T), [n6, t_x], "out")
    n8 = node("ARGMAX", I32, (T,), [n7], "amax")
    nodes = [n1, n2, n3, n4, n5, n6, n7, n8]
    table = (Tensor * 13)(t_x, t_wn, t_g, t_u, t_d, *nodes)
    ids = (C.c_uint64 * len(nodes))(*[n.id for n in nodes])
    be = C.c_void_p()
    check(lib().b200_backend_init(0, C.byref(be)))
    check(lib().b200_backend_graph_compute(be, ids, len(nodes), table, 13))
    got = buf.get(n7, T * h * 4, dtype=np.float32).reshape(T, h)
    xn = orc.rms_norm(x, wn, 1e-6)
    act = orc.swiglu(orc.mul_mat(orc.TYPE_Q4_K, Wg, xn, ff, h), orc.mul_mat(orc.TYPE_Q4_K, Wu, xn, ff, h))
    ref = orc.mul_mat(orc.TYPE_Q6_K, Wd, act, h, ff) + x
    assert np.abs(got - ref).max() <= 1e-3 * np.abs(ref).max()
    np.testing.assert_array_equal(buf.get(n8, T * 4, dtype=np.int32), got.argmax(-1))
    # an op outside the hot path is reported, not emulated
    bad = node("NONE", F32, (h, T), [t_x], "bad")
    bad.op = 99
    table2 = (Tensor * 2)(t_x, bad)
    assert lib().b200_backend_graph_compute(be, (C.c_uint64 * 1)(bad.id), 1, table2, 2) == -4
    lib().b200_backend_free(be)
    buf.free()


def test_graph_compute_mul_mat_id_matches_per_expert_oracle():
    from mesh_llm_b200.capi import Tensor, check, lib

    rng = np.random.default_rng(3)
    K, N, E, k, T = 512, 256, 6, 2, 4
    buf = Buf(0, 1 << 24)
    W = orc.quantize_weights(orc.TYPE_Q4_K, (rng.standard_normal((E * N, K)) * 0.02).astype(np.float32))
    x = rng.standard_normal((T, K)).astype(np.float32)
    ids = rng.integers(0, E, (T, k)).astype(np.int32)
    t_w, t_x, t_i = buf.tensor(Q4K, (K, N, E), "exps"), buf.tensor(F32, (K, 1, T), "x"), buf.tensor(I32, (k, T), "ids")
    buf.set(t_w, W)
    buf.set(t_x, x)
    buf.set(t_i, ids)
    out = buf.tensor(F32, (N, k, T), "y")
    out.op = OP["MUL_MAT_ID"]
    out.src[0], out.src[1], out.src[2] = t_w.id, t_x.id, t_i.id
    be = C.c_void_p()
    check(lib().b200_backend_init(0, C.byref(be)))
    table = (Tensor * 4)(t_w, t_x, t_i, out)
    check(lib().b200_backend_graph_compute(be, (C.c_uint64 * 1)(out.id), 1, table, 4))
    got = buf.get(out, T * k * N * 4, dtype=np.float32).reshape(T, k, N)
    Wr = W.reshape(E, N, -1)
    for t in range(T):
        for s in range(k):
            ref = orc.mul_mat(orc.TYPE_Q4_K, Wr[ids[t, s]], x[t:t + 1], N, K)[0]
            assert np.abs(got[t, s] - ref).max() <= 1e-3 * np.abs(ref).max()
    lib().b200_backend_free(be)
    buf.free()


def test_graph_compute_rejects_outputs_too_small_for_what_the_op_writes():
    """A graph that arrives over the wire may name a destination smaller than the op's result.  Every op
    checks the node's own shape and type before it launches: the call answers out-of-bounds (or invalid
    for a wrong type), launches nothing for that node, and the bytes after the small tensor stay as
    they were."""
    from mesh_llm_b200.capi import Tensor, lib

    h, T = 512, 6
    buf = Buf(0, 1 << 22)
    rng = np.random.default_rng(4)
    x = rng.standard_normal((T, h)).astype(np.float32)
    t_x = buf.tensor(F32, (h, T), "x")
    t_pos = buf.tensor(I32, (T,), "pos")
    t_ids = buf.tensor(I32, (T,), "ids")
    buf.set(t_x, x)
    buf.set(t_pos, np.arange(T, dtype=np.int32))
    buf.set(t_ids, np.zeros(T, np.int32))
    small = buf.tensor(F32, (h, 1), "small")       # one row where T rows would be written
    guard = buf.tensor(F32, (h, T), "guard")       # sits right behind it in the buffer
    sentinel = np.full((T, h), 7.25, np.float32)
    buf.set(guard, sentinel)
    be = C.c_void_p()
    assert lib().b200_backend_init(0, C.byref(be)) == 0

    def run(op, type_, srcs, params=(), ne=None):
        t = Tensor()
        C.memmove(C.byref(t), C.byref(small), C.sizeof(Tensor))
        t.id = 990000 + run.n
        run.n += 1
        t.type = type_
        if ne:
            for i in range(4):
                t.ne[i] = (list(ne) + [1] * 4)[i]
        t.op = OP[op]
        for i, s in enumerate(srcs):
            t.src[i] = s.id
        for i, p in enumerate(params):
            t.op_params[i] = p
        table = (Tensor * (len(srcs) + 1))(*srcs, t)
        return lib().b200_backend_graph_compute(be, (C.c_uint64 * 1)(t.id), 1, table, len(srcs) + 1)

    run.n = 0
    launches_before = lib().b200_backend_synchronize(be)
    assert launches_before == 0
    assert run("RMS_NORM", F32, [t_x], [_f32bits(1e-6)]) == -5
    assert run("ADD", F32, [t_x, t_x]) == -5
    assert run("MUL", F32, [t_x, t_x]) == -5
    assert run("SWIGLU", F32, [t_x, t_x]) == -5
    assert run("CPY", F32, [t_x]) == -5
    assert run("CPY", F16, [t_x]) == -5
    assert run("GET_ROWS", F32, [t_x, t_ids]) == -5
    assert run("ARGMAX", I32, [t_x], ne=(1,)) == -5
    assert run("ARGMAX", F32, [t_x], ne=(T,)) == -1          # the op writes i32
    q = buf.tensor(F32, (128, 4, T), "q")
    kc = buf.tensor(F16, (128, 2, 16), "kc")
    vc = buf.tensor(F16, (128, 2, 16), "vc")
    vbad = buf.tensor(F16, (64, 2, 16), "vbad")
    assert run("ROPE", F32, [q, t_pos], [128, 2, _f32bits(1e6)]) == -5
    assert run("ATTN", F32, [q, kc, vc], [_f32bits(0.088), 0]) == -5
    full_ne = (128, 4, T)
    assert run("ATTN", F32, [q, kc, vbad], [_f32bits(0.088), 0], ne=full_ne) == -1  # V of another head_dim
    logits = buf.tensor(F32, (8, T), "logits")
    idsout = buf.tensor(I32, (2, T), "idsout")
    assert run("MOE_ROUTE", F32, [logits, idsout], [2], ne=(2, 1)) == -5
    assert run("MOE_ROUTE", F32, [logits, idsout], [9], ne=(9, T)) == -1       # k above the expert count
    # extents whose product does not fit are refused before any size is computed from them
    huge = Tensor()
    C.memmove(C.byref(huge), C.byref(small), C.sizeof(Tensor))
    for i in range(4):
        huge.ne[i] = 0xFFFFFFFF
    assert lib().b200_buffer_init_tensor(buf.h, C.byref(huge)) == -5
    assert lib().b200_backend_synchronize(be) == 0
    np.testing.assert_array_equal(buf.get(guard, T * h * 4, dtype=np.float32).reshape(T, h), sentinel)
    lib().b200_backend_free(be)
    buf.free()


Q4_0, Q8_0 = 2, 8


@pytest.mark.parametrize("kt, vt", [(Q8_0, Q4_0), (Q4_0, Q4_0), (F16, Q8_0)], ids=["q8_0-q4_0", "q4_0-q4_0", "f16-q8_0"])
@pytest.mark.parametrize("T, pos0", [(1, 77), (40, 0), (70, 58)])
def test_graph_attention_over_a_quantised_cache_in_ggml_block_layout(kt, vt, T, pos0):
    """The caches mesh-llm starts large models with (mesh-llm/src/inference/launch.rs:568-591), as llama.cpp
    holds them: tensors of type q8_0 / q4_0 in ggml's 34 / 18-byte blocks.  A CPY node quantises f32 rows
    into such a tensor (the bytes must be the pinned CPU quantiser's), and ATTN reads K and V from them in
    place; the result is compared with the oracle's attention over the f16 decode of the same bytes."""
    from mesh_llm_b200.capi import Tensor, check, lib

    rng = np.random.default_rng(100 * T + pos0)
    hd, n_head, n_kv = 128, 8, 2
    L = pos0 + T
    buf = Buf(0, 1 << 24)
    k = (rng.standard_normal((L, n_kv, hd)) * rng.uniform(0.05, 2.0, (L, n_kv, 1))).astype(np.float32)
    v = (rng.standard_normal((L, n_kv, hd)) * rng.uniform(0.05, 4.0, (L, n_kv, 1))).astype(np.float32)
    q = rng.standard_normal((T, n_head, hd)).astype(np.float32)
    t_k, t_v, t_q = buf.tensor(F32, (hd, n_kv, L), "k"), buf.tensor(F32, (hd, n_kv, L), "v"), buf.tensor(F32, (hd, n_head, T), "q")
    for t, d in ((t_k, k), (t_v, v), (t_q, q)):
        buf.set(t, d)

    def node(op, type_, ne, srcs, name, params=()):
        t = buf.tensor(type_, ne, name)
        t.op = OP[op]
        for i, s in enumerate(srcs):
            t.src[i] = s.id
        for i, p in enumerate(params):
            t.op_params[i] = p
        return t

    c_k = node("CPY", kt, (hd, n_kv, L + 5), [t_k], "cache_k")
    c_v = node("CPY", vt, (hd, n_kv, L + 5), [t_v], "cache_v")
    att = node("ATTN", F32, (hd, n_head, T), [t_q, c_k, c_v], "att", [_f32bits(hd ** -0.5), pos0])
    nodes = [c_k, c_v, att]
    table = (Tensor * 6)(t_k, t_v, t_q, *nodes)
    be = C.c_void_p()
    check(lib().b200_backend_init(0, C.byref(be)))
    check(lib().b200_backend_graph_compute(be, (C.c_uint64 * 3)(*[n.id for n in nodes]), 3, table, 6))

    def as_f16(t, type_, src):
        if type_ == F16:
            got = buf.get(t, L * n_kv * hd * 2, dtype=np.uint16).reshape(L, n_kv, hd)
            np.testing.assert_array_equal(got, orc.f32_to_f16(src))
            return got
        bb = 34 if type_ == Q8_0 else 18
        blocks = buf.get(t, L * n_kv * 4 * bb).reshape(L, n_kv, 4 * bb)
        np.testing.assert_array_equal(blocks, orc.kv_quantize(type_, src))  # the pinned quantiser's bytes
        return orc.kv_dequantize(type_, blocks).astype(np.float16).view(np.uint16)

    kc, vc = as_f16(c_k, kt, k), as_f16(c_v, vt, v)
    got = buf.get(att, T * n_head * hd * 4, dtype=np.float32).reshape(T, n_head, hd)
    ref = orc.attention(q * np.float32(1.0), kc, vc, pos0)
    assert np.abs(got - ref).max() <= 1e-3 * np.abs(ref).max()
    lib().b200_backend_free(be)
    buf.free()
