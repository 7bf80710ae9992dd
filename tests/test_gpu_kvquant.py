"""Quantised KV cache (q8_0 / q4_0 rows) on the GPU against the CPU oracle.

mesh-llm starts its servers with --cache-type-k q8_0 --cache-type-v q4_0 for models of 5-50 GB and
q4_0 / q4_0 above (mesh-llm/src/inference/launch.rs:568-591).  The row quantisers are ggml's and are
integer work, so the stored bytes must equal the oracle's (which tests/test_oracle_formats.py pins to
gguf-py's); attention over identical cache bytes is held to the f16 path's tolerance.
"""
import numpy as np
import pytest

from oracle import binding as orc

pytestmark = pytest.mark.gpu

HD = 128
PAIRS = [(orc.TYPE_Q8_0, orc.TYPE_Q4_0), (orc.TYPE_Q4_0, orc.TYPE_Q4_0), (orc.TYPE_F16, orc.TYPE_Q8_0),
         (orc.TYPE_Q8_0, orc.TYPE_F16)]
PAIR_IDS = ["q8_0-q4_0", "q4_0-q4_0", "f16-q8_0", "q8_0-f16"]


def device_rows_to_blocks(rows, type_, hd=HD):
    """[..., row bytes] uint8 in the device layout (codes, then f16 scales, then padding) -> ggml blocks
    [..., hd / 32 * (34 | 18)]"""
    nb = hd // 32
    cb = 32 if type_ == orc.TYPE_Q8_0 else 16
    lead = rows.shape[:-1]
    codes = rows[..., : nb * cb].reshape(lead + (nb, cb))
    scales = rows[..., nb * cb: nb * cb + 2 * nb].reshape(lead + (nb, 2))
    return np.concatenate([scales, codes], axis=-1).reshape(lead + (nb * (cb + 2),))


def cache_as_f16(cache, type_):
    """what attention reads from a cache tensor made by ops.kv_cache: uint16 [n_ctx, n_kv, hd]"""
    a = cache.cpu().numpy()
    if type_ == orc.TYPE_F16:
        return a.view(np.uint16).reshape(a.shape[0], a.shape[1], HD)
    f = orc.kv_dequantize(type_, device_rows_to_blocks(a, type_))
    return f.astype(np.float16).view(np.uint16)


def mixed_rows(rng, *shape):
    x = rng.standard_normal(shape) * rng.uniform(0.05, 8.0, size=shape[:-1] + (1,))
    return x.astype(np.float32)


def test_row_bytes_and_size_tiers():
    from mesh_llm_b200 import ops
    from mesh_llm_b200.capi import TYPE_F16, TYPE_Q4_0, TYPE_Q8_0

    assert ops.kv_row_bytes(TYPE_F16, 128) == 256
    assert ops.kv_row_bytes(TYPE_Q8_0, 128) == 144 and ops.kv_row_bytes(TYPE_Q4_0, 128) == 80
    assert ops.kv_row_bytes(TYPE_Q8_0, 64) == 80 and ops.kv_row_bytes(TYPE_Q4_0, 64) == 48
    assert ops.kv_row_bytes(12, 128) == 0
    assert ops.kv_types_for_model_bytes(4_999_999_999) == (TYPE_F16, TYPE_F16)
    assert ops.kv_types_for_model_bytes(19_850_000_000) == (TYPE_Q8_0, TYPE_Q4_0)   # Qwen2.5-32B Q4_K_M
    assert ops.kv_types_for_model_bytes(50_000_000_000) == (TYPE_Q4_0, TYPE_Q4_0)


@pytest.mark.parametrize("type_", [orc.TYPE_Q8_0, orc.TYPE_Q4_0], ids=["q8_0", "q4_0"])
def test_stored_rows_are_the_oracles_bytes(type_):
    """V rows are not rotated: every stored byte equals ggml's quantiser output.  Includes an all-zero
    block, a constant block, a single outlier and ties for the largest magnitude."""
    import torch
    from mesh_llm_b200 import ops

    rng = np.random.default_rng(3)
    T, n_kv = 37, 3
    v = mixed_rows(rng, T, n_kv, HD)
    v[0, 0, :32] = 0.0
    v[1, 0, 32:64] = 1.0
    v[2, 1, 5] = -300.0
    v[3, 2, 64:96] = np.where(np.arange(32) % 2 == 0, 2.5, -2.5)   # ties: the first (positive) one sets the sign
    v[4, 2, 96:128] = -v[3, 2, 64:96]
    pos = rng.permutation(64)[:T].astype(np.int32)
    kc = ops.kv_cache(orc.TYPE_F16, 64, n_kv, HD)
    vc = ops.kv_cache(type_, 64, n_kv, HD)
    ops.kv_store(torch.from_numpy(v).cuda(), torch.from_numpy(v).cuda(), torch.from_numpy(pos), kc, vc,
                 orc.TYPE_F16, type_, 1e6, 1)
    got = device_rows_to_blocks(vc.cpu().numpy()[pos], type_)
    np.testing.assert_array_equal(got, orc.kv_quantize(type_, v))
    # untouched positions stay zero
    rest = np.setdiff1d(np.arange(64), pos)
    assert not vc.cpu().numpy()[rest].any()


@pytest.mark.parametrize("neox", [1, 0], ids=["neox", "interleaved"])
@pytest.mark.parametrize("type_", [orc.TYPE_Q8_0, orc.TYPE_Q4_0], ids=["q8_0", "q4_0"])
def test_stored_k_rows_follow_the_rotation(type_, neox):
    """K rows are rotated before they are quantised.  cosf / sinf differ from the host's by an ulp, so a
    value within an ulp of a code boundary may take the neighbouring code: at position 0 (angle 0) the
    bytes are exact, elsewhere all but a handful of codes agree and none differs by more than one step."""
    import torch
    from mesh_llm_b200 import ops

    rng = np.random.default_rng(5)
    T, n_kv, theta = 48, 2, 1e4
    k = mixed_rows(rng, T, n_kv, HD)
    pos = np.arange(T, dtype=np.int32)
    kc = ops.kv_cache(type_, T, n_kv, HD)
    vc = ops.kv_cache(orc.TYPE_F16, T, n_kv, HD)
    ops.kv_store(torch.from_numpy(k).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(pos), kc, vc,
                 type_, orc.TYPE_F16, theta, neox)
    want_rot = orc.rope(k, pos, theta, neox)
    want = orc.kv_quantize(type_, want_rot)
    got = device_rows_to_blocks(kc.cpu().numpy(), type_)
    np.testing.assert_array_equal(got[0], want[0])
    assert (got != want).mean() < 2e-3
    step = np.abs(want_rot).reshape(T, n_kv, 4, 32).max(-1, keepdims=True) / (127 if type_ == orc.TYPE_Q8_0 else 8)
    diff = np.abs(orc.kv_dequantize(type_, got) - orc.kv_dequantize(type_, want)).reshape(T, n_kv, 4, 32)
    assert (diff <= step * 1.01 + 1e-6).all()
    # the f16 V cache written by the same call
    np.testing.assert_array_equal(vc.cpu().numpy().view(np.uint16).reshape(T, n_kv, HD), orc.f32_to_f16(k))


@pytest.mark.parametrize("kt, vt", PAIRS, ids=PAIR_IDS)
@pytest.mark.parametrize("T, pos0, n_head, n_kv", [(1, 0, 4, 2), (1, 200, 8, 1), (5, 59, 5, 1), (40, 0, 4, 4), (130, 70, 16, 2)])
def test_attention_over_quantised_rows(kt, vt, T, pos0, n_head, n_kv):
    """Attention over caches written by the store kernel, against the oracle's attention over the f16
    decode of the very same bytes (tolerance of the f16 tensor-core path: q and the probabilities are
    rounded to f16)."""
    import torch
    from mesh_llm_b200 import ops

    rng = np.random.default_rng(T * 1000 + pos0)
    L = pos0 + T
    k = mixed_rows(rng, L, n_kv, HD) * 0.3
    v = mixed_rows(rng, L, n_kv, HD)
    q = rng.standard_normal((T, n_head, HD)).astype(np.float32)
    kc = ops.kv_cache(kt, L + 3, n_kv, HD)
    vc = ops.kv_cache(vt, L + 3, n_kv, HD)
    ops.kv_store(torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), torch.arange(L, dtype=torch.int32), kc, vc,
                 kt, vt, 1e6, 1)
    got = ops.attention_kv(torch.from_numpy(q).cuda(), kc, vc, kt, vt, pos0).cpu().numpy()
    ref = orc.attention(q, cache_as_f16(kc, kt), cache_as_f16(vc, vt), pos0)
    assert np.abs(got - ref).max() <= 1e-3 * np.abs(ref).max()


CFG = dict(n_layer=3, n_embd=512, n_head=4, n_head_kv=2, head_dim=128, n_ff=512, n_vocab=1024, n_ctx=320,
           qkv_bias=1, rope_neox=1, rope_theta=1e6, rms_eps=1e-6)
LLAMA = dict(n_layer=2, n_embd=1024, n_head=8, n_head_kv=1, head_dim=128, n_ff=768, n_vocab=1024, n_ctx=192,
             qkv_bias=0, rope_neox=0, rope_theta=5e5, rms_eps=1e-5)


def _stage_pair(cfg, full, l0, l1, kt, vt, **kw):
    from mesh_llm_b200.stage import Stage

    extra = dict(layer_begin=l0, layer_end=l1, has_embd=0, has_output=0, kv_type_k=kt, kv_type_v=vt)
    st = Stage(**cfg, **extra, **kw)
    om = orc.Model(**cfg, **extra)
    for n in om.tensor_names():
        ty, data, _ = full.tensor(n)
        om.set_tensor(n, ty, data)
        st.set_tensor(n, ty, data)
    return om, st


def _row_errs(got, ref):
    return np.abs(np.asarray(got, np.float64) - ref).max(-1) / np.abs(ref).max()


@pytest.mark.parametrize("kt, vt", PAIRS[:2], ids=PAIR_IDS[:2])
@pytest.mark.parametrize("cfg", [CFG, LLAMA], ids=["qwen2", "llama"])
def test_layer_outputs_with_a_quantised_cache(cfg, kt, vt):
    """Each layer gets the oracle's input: a prefill of 150 tokens (tensor-core attention, two cache
    chunks), a 3-token batch at position 150, then decode steps through the one-launch kernel (which
    decodes the raw rows it fetched by TMA and quantises the new row itself).

    Batches go through the f16 tensor-core attention whatever the cache type; its 2-4e-4 error flips int8
    codes of the re-quantised attention output, which at these toy widths moves a row by 3-7e-3 (the f16
    cache shows the same figures), so batch rows are held to 2e-2.  Decode steps run their products on
    mma.m16n8k16 too, but with q and the probabilities as hi + lo pairs of f16, i.e. to f32 accuracy over the
    same cache bytes: they must be near exact unless a cache code sat on a boundary (see above), which may
    touch a minority of them."""
    import torch

    full = orc.Model(**cfg)
    full.generate(21)
    rng = np.random.default_rng(1)
    n_pre, n_mid, n_dec = 150, 3, 4
    prompt = rng.integers(0, cfg["n_vocab"], n_pre + n_mid + n_dec).astype(np.int32)
    emb = orc.get_rows(*full.tensor("token_embd.weight")[:2], prompt, cfg["n_embd"])
    cuts = [0, n_pre, n_pre + n_mid] + [n_pre + n_mid + i + 1 for i in range(n_dec)]
    hs = [emb[a:b] for a, b in zip(cuts[:-1], cuts[1:])]
    batch_worst, dec = 0.0, []
    for l in range(cfg["n_layer"]):
        om, st = _stage_pair(cfg, full, l, l + 1, kt, vt, n_ubatch=256)
        nxt = []
        for h, p0 in zip(hs, cuts[:-1]):
            ref, _ = om.forward(hidden_in=h, pos0=p0)
            got, _, _ = st.forward(hidden_in=torch.from_numpy(h).cuda(), pos0=p0)
            e = _row_errs(got.cpu().numpy(), ref)
            assert e.max() <= 2e-2, (l, p0, e)
            if len(h) == 1:
                dec.append(e[0])
            else:
                batch_worst = max(batch_worst, e.max())
            nxt.append(ref)
        hs = nxt
        st.close()
    dec = np.array(dec)
    print(f"batch rows worst {batch_worst:.2e}; decode rows {np.array2string(dec, precision=1)}")
    assert dec.max() <= 2e-2 and np.median(dec) <= 1e-4, dec


def test_decode_equals_prefill_on_the_gpu_cache():
    """The same 140 tokens as one batch and token by token (the last 12 through the decode kernel, over
    a cache whose earlier rows were written by the prefill store).  Both read identical cache bytes; the
    batch goes through the f16 tensor-core attention, so the two are compared the way the long-prefill
    test of the f16 cache compares with the oracle: KL of the output distributions and relative error."""
    import torch
    from mesh_llm_b200.stage import Stage

    kw = dict(CFG, kv_type_k=orc.TYPE_Q8_0, kv_type_v=orc.TYPE_Q4_0, n_ubatch=256, n_seq=2)
    st = Stage(**kw)
    st.generate(9)
    toks = torch.from_numpy(np.random.default_rng(2).integers(0, CFG["n_vocab"], 140).astype(np.int32)).cuda()
    _, all_lg, _ = st.forward(tokens=toks, all_logits=True)
    st.forward(tokens=toks[:128], seq0=1)
    rows = []
    for i in range(128, 140):
        _, lg, _ = st.forward(tokens=toks[i:i + 1], pos0=i, seq0=1)
        rows.append(lg[0].cpu().numpy())
    st.close()
    got, ref = np.stack(rows).astype(np.float64), all_lg[128:140].cpu().numpy().astype(np.float64)
    assert np.abs(got - ref).max() <= 5e-2 * np.abs(ref).max()
    la = ref - ref.max(-1, keepdims=True)
    la -= np.log(np.exp(la).sum(-1, keepdims=True))
    lb = got - got.max(-1, keepdims=True)
    lb -= np.log(np.exp(lb).sum(-1, keepdims=True))
    kl = (np.exp(la) * (la - lb)).sum(-1).mean()
    print(f"decode vs batch: rel {np.abs(got - ref).max() / np.abs(ref).max():.2e} KL {kl:.2e}")
    assert kl < 1e-4


def test_batched_decode_and_unsupported_shapes():
    import torch
    from mesh_llm_b200.stage import Stage
    from mesh_llm_b200.capi import B200Error

    kw = dict(CFG, kv_type_k=orc.TYPE_Q8_0, kv_type_v=orc.TYPE_Q4_0, n_ubatch=64, n_seq=3)
    st = Stage(**kw)
    st.generate(4)
    rng = np.random.default_rng(6)
    toks = torch.from_numpy(rng.integers(0, CFG["n_vocab"], (3, 20)).astype(np.int32)).cuda()
    # three sequences prefilled together, then one batched decode step == each sequence on its own
    st.forward(tokens=toks.reshape(-1), n_seq=3)
    nxt = torch.from_numpy(rng.integers(0, CFG["n_vocab"], 3).astype(np.int32)).cuda()
    _, lg3, _ = st.forward(tokens=nxt, n_seq=3, pos0=20)
    single = Stage(**dict(kw, n_seq=1))
    single.generate(4)
    for s in range(3):
        single.forward(tokens=toks[s])
        _, lg1, _ = single.forward(tokens=nxt[s:s + 1], pos0=20)
        assert np.abs(lg3[s].cpu().numpy() - lg1[0].cpu().numpy()).max() <= 2e-3 * lg1.abs().max().item()
    st.close()
    single.close()
    with pytest.raises(B200Error):
        Stage(**dict(CFG, head_dim=64, n_head=8, kv_type_k=orc.TYPE_Q8_0, kv_type_v=orc.TYPE_Q4_0))
    with pytest.raises(B200Error):
        Stage(**dict(CFG, kv_type_k=12))
