"""Output-distribution statistics on the device against a float64 restatement of what the
reference's server computes per token on the CPU (third_party/llama.cpp/patches/0005:
full-vocabulary softmax sorted by probability, mesh_compute_entropy = -sum p log2 p over p > 0,
margin = p[0] - p[1], probability of the sampled token, five most likely tokens)."""
import numpy as np
import pytest
import torch

from mesh_llm_b200 import ops

pytestmark = pytest.mark.gpu


def reference(logits, chosen):
    x = logits.astype(np.float64)
    p = np.exp(x - x.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    ent = -(np.where(p > 0, p * np.log2(np.where(p > 0, p, 1.0)), 0.0)).sum(-1)
    order = np.lexsort((np.arange(x.shape[1])[None, :].repeat(x.shape[0], 0), -x), axis=-1)[:, :5]
    top_p = np.take_along_axis(p, order, -1)
    margin = top_p[:, 0] - top_p[:, 1] if x.shape[1] >= 2 else np.ones(x.shape[0])
    return ent, margin, p[np.arange(x.shape[0]), chosen], top_p, order


@pytest.mark.parametrize("T,n,scale", [(1, 152064, 3.0), (3, 151936, 8.0), (5, 4097, 1.0), (2, 7, 2.0), (4, 128256, 0.01)])
def test_signals_match_float64_softmax(T, n, scale):
    rng = np.random.default_rng(T * 1000 + n)
    logits = (rng.standard_normal((T, n)) * scale).astype(np.float32)
    chosen = rng.integers(0, n, T).astype(np.int32)
    out = ops.logit_signals(torch.from_numpy(logits).cuda(), torch.from_numpy(chosen).cuda())
    ent, margin, pc, top_p, top_id = reference(logits, chosen)
    k = min(5, n)
    assert np.array_equal(out["top_id"].cpu().numpy()[:, :k], top_id[:, :k])
    assert np.array_equal(out["argmax"].cpu().numpy(), logits.argmax(-1))
    np.testing.assert_allclose(out["entropy"].cpu().numpy(), ent, rtol=2e-4, atol=2e-4)
    np.testing.assert_allclose(out["margin"].cpu().numpy(), margin, rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(out["p_chosen"].cpu().numpy(), pc, rtol=1e-4, atol=1e-9)
    np.testing.assert_allclose(out["top_p"].cpu().numpy()[:, :k], top_p[:, :k], rtol=1e-4, atol=1e-9)


def test_ties_take_the_lowest_index_and_default_chosen_is_argmax():
    logits = np.zeros((2, 70000), np.float32)
    logits[0, [9, 40000, 69999]] = 5.0
    logits[1, :] = -3.0
    out = ops.logit_signals(torch.from_numpy(logits).cuda())
    assert out["top_id"].cpu().numpy()[0, :4].tolist() == [9, 40000, 69999, 0]
    assert out["argmax"].cpu().numpy().tolist() == [9, 0]
    assert out["margin"].cpu().numpy()[0] == pytest.approx(0.0, abs=1e-7)
    assert out["entropy"].cpu().numpy()[1] == pytest.approx(np.log2(70000), rel=1e-5)  # uniform row
    assert out["p_chosen"].cpu().numpy()[1] == pytest.approx(1 / 70000, rel=1e-4)


def test_repeated_calls_reuse_scratch_and_stay_identical():
    x = torch.randn(4, 152064, device="cuda") * 4
    a = ops.logit_signals(x)
    b = ops.logit_signals(x)
    for k in a:
        assert torch.equal(a[k], b[k]), k


def test_rejects_small_scratch():
    from mesh_llm_b200.capi import B200Error, check, lib, ptr, cur_stream
    x = torch.randn(1, 1000, device="cuda")
    s = torch.zeros(64, dtype=torch.uint8, device="cuda")
    with pytest.raises(B200Error, match="scratch"):
        check(lib().b200_logit_signals(ptr(x), 1, 1000, None, None, None, ptr(s), 64, cur_stream()))
