"""Whole-stage behaviour of the CPU oracle (no GPU): layer-range split and expert models."""
import numpy as np

from oracle import binding as orc

DENSE = dict(n_layer=4, n_embd=256, n_head=4, n_head_kv=2, head_dim=64, n_ff=512, n_vocab=512,
             n_ctx=32, qkv_bias=1)
MOE = dict(n_layer=2, n_embd=256, n_head=4, n_head_kv=2, head_dim=64, n_ff=0, n_vocab=512,
           n_ctx=32, n_expert=8, n_expert_used=2, n_ff_exp=256, qk_norm=1)


def test_q4km_mix_and_determinism():
    m = orc.Model(**DENSE)
    m.generate(1)
    names = m.tensor_names()
    assert "token_embd.weight" in names and "output.weight" in names
    assert m.tensor("blk.0.attn_v.weight")[0] == orc.TYPE_Q4_K
    assert m.tensor("blk.1.attn_v.weight")[0] == orc.TYPE_Q6_K
    assert m.tensor("blk.1.ffn_down.weight")[0] == orc.TYPE_Q6_K
    assert m.tensor("blk.2.ffn_down.weight")[0] == orc.TYPE_Q4_K
    assert m.tensor("output.weight")[0] == orc.TYPE_Q6_K
    m2 = orc.Model(**DENSE)
    m2.generate(1)
    np.testing.assert_array_equal(m.tensor("blk.3.ffn_up.weight")[1], m2.tensor("blk.3.ffn_up.weight")[1])
    w = orc.dequantize(orc.TYPE_Q4_K, m.tensor("blk.0.attn_q.weight")[1])
    assert abs(w.std() - 0.02) < 0.002 and abs(w.mean()) < 1e-3


def test_two_stages_equal_one_stage_bit_for_bit():
    """The stage hand-off is a bit copy of the residual stream, so splitting the layer range
    must not change a single bit (the reference only warns on a difference:
    third_party/llama.cpp/patches/0002 lines 961-969; here it is a hard assert)."""
    full = orc.Model(**DENSE)
    full.generate(42)
    s0 = orc.Model(**DENSE, layer_end=2, has_output=0)
    s1 = orc.Model(**DENSE, layer_begin=2, layer_end=4, has_embd=0)
    s0.generate(42)
    s1.generate(42)
    toks = np.random.default_rng(0).integers(0, 512, 9)
    _, logits = full.forward(tokens=toks[:8])
    h0, _ = s0.forward(tokens=toks[:8])
    _, logits2 = s1.forward(hidden_in=h0)
    np.testing.assert_array_equal(logits, logits2)
    # one decode step continues from the KV cache in both
    _, l1 = full.forward(tokens=toks[8:], pos0=8)
    h0, _ = s0.forward(tokens=toks[8:], pos0=8)
    _, l2 = s1.forward(hidden_in=h0, pos0=8)
    np.testing.assert_array_equal(l1, l2)


def test_prefill_equals_token_by_token():
    m = orc.Model(**DENSE)
    m.generate(5)
    toks = np.random.default_rng(1).integers(0, 512, 6)
    _, all_at_once = m.forward(tokens=toks)
    m2 = orc.Model(**DENSE)
    m2.generate(5)
    rows = [m2.forward(tokens=toks[i:i + 1], pos0=i)[1][0] for i in range(6)]
    np.testing.assert_allclose(all_at_once, np.stack(rows), rtol=0, atol=1e-6)


def test_moe_forward_runs_and_is_finite():
    m = orc.Model(**MOE)
    m.generate(3)
    assert m.tensor("blk.0.ffn_gate_exps.weight")[2] == (256, 256, 8)
    assert m.tensor("blk.0.ffn_gate_inp.weight")[0] == orc.TYPE_F32
    toks = np.random.default_rng(2).integers(0, 512, 5)
    h, logits = m.forward(tokens=toks)
    assert np.isfinite(logits).all() and np.isfinite(h).all()
    assert logits.shape == (5, 512)


def test_quantised_kv_cache_changes_little_and_keeps_prefill_equal_to_decode():
    """q8_0 K / q4_0 V (what mesh-llm launches 5-50 GB models with) perturbs the logits slightly
    and, like the f16 cache, gives the same result token by token as in one batch."""
    kw = dict(DENSE, head_dim=128, n_embd=512)
    toks = np.arange(1, 13, dtype=np.int32)
    ref = orc.Model(**kw)
    ref.generate(3)
    want = ref.forward(tokens=toks)[1]
    m = orc.Model(**kw, kv_type_k=orc.TYPE_Q8_0, kv_type_v=orc.TYPE_Q4_0)
    m.generate(3)
    got = m.forward(tokens=toks)[1]
    err = np.abs(got - want).max() / np.abs(want).max()
    assert 0 < err < 0.3  # random weights: no trained redundancy to absorb the 4-bit V rows
    m2 = orc.Model(**kw, kv_type_k=orc.TYPE_Q8_0, kv_type_v=orc.TYPE_Q4_0)
    m2.generate(3)
    rows = [m2.forward(tokens=toks[i:i + 1], pos0=i)[1][0] for i in range(len(toks))]
    np.testing.assert_allclose(np.stack(rows), got, rtol=0, atol=1e-6)


def test_oracle_expert_mask_equals_routing_without_the_masked_experts():
    """selection_probs = probs + (0 | -inf), weights from the unmasked probs renormalised over the
    selection (third_party/llama.cpp/patches/0003 lines 82-108): with at least k experts allowed that
    is the routing of the same logits with the masked experts' logits at -inf."""
    rng = np.random.default_rng(3)
    for E, k in ((128, 8), (16, 4)):
        logits = rng.standard_normal((21, E)).astype(np.float32)
        mask = np.zeros(E, np.uint8)
        mask[rng.permutation(E)[: E // 2]] = 1
        ids, w = orc.moe_route(logits, k, mask)
        cut = logits.copy()
        cut[:, mask == 0] = -np.inf
        ids2, w2 = orc.moe_route(cut, k)
        assert np.array_equal(ids, ids2) and np.abs(w - w2).max() < 1e-6
        assert mask[ids].all() and np.allclose(w.sum(-1), 1, atol=1e-6)
    m = orc.Model(n_layer=1, n_embd=256, n_head=2, n_head_kv=1, head_dim=128, n_ff=0, n_vocab=256, n_ctx=8,
                  n_expert=8, n_expert_used=2, n_ff_exp=256)
    assert m.set_expert_mask(np.ones(7)) == -1 and m.set_expert_mask(np.ones(8)) == 0 and m.set_expert_mask(None) == 0
