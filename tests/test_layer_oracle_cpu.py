"""No GPU: the step-by-step oracle layer used by the strict layer parity test (tests/layer_oracle.py)
reproduces oracle.binding.Model.forward -- bit for bit on dense layers, to f32 rounding of the router's
dot products on an expert layer -- for a prefill and a following decode step."""
import numpy as np
import pytest

from oracle import binding as orc

from layer_oracle import LayerOracle

DENSE = dict(n_layer=2, n_embd=512, n_head=4, n_head_kv=2, head_dim=128, n_ff=1024, n_vocab=256,
             n_ctx=32, qkv_bias=1, rope_neox=1, rope_theta=1e6, rms_eps=1e-6)
LLAMA = dict(n_layer=2, n_embd=1024, n_head=8, n_head_kv=1, head_dim=128, n_ff=768, n_vocab=256,
             n_ctx=32, qkv_bias=0, rope_neox=0, rope_theta=5e5, rms_eps=1e-5)
MOE = dict(n_layer=2, n_embd=512, n_head=8, n_head_kv=2, head_dim=64, n_ff=0, n_vocab=256, n_ctx=32,
           n_expert=16, n_expert_used=4, n_ff_exp=256, qk_norm=1)


@pytest.mark.parametrize("cfg", [DENSE, LLAMA, MOE], ids=["qwen2-dense", "llama-dense", "qwen3-moe"])
def test_step_by_step_layer_equals_the_model_forward(cfg):
    full = orc.Model(**cfg, has_embd=0, has_output=0)
    full.generate(5)
    x = (np.random.default_rng(1).standard_normal((12, cfg["n_embd"])) * 0.02).astype(np.float32)
    for l in range(2):
        one = orc.Model(**cfg, layer_begin=l, layer_end=l + 1, has_embd=0, has_output=0)
        for n in one.tensor_names():
            ty, data, _ = full.tensor(n)
            one.set_tensor(n, ty, data)
        L = LayerOracle(full, cfg, l)
        ref_pre, _ = one.forward(hidden_in=x[:11])
        ref_dec, _ = one.forward(hidden_in=x[11:], pos0=11)
        got_pre = L.forward(x[:11], 0)["out"]
        got_dec = L.forward(x[11:], 11)["out"]
        if cfg.get("n_expert", 0):
            for got, ref in ((got_pre, ref_pre), (got_dec, ref_dec)):
                assert np.abs(got - ref).max() <= 2e-6 * np.abs(ref).max()
        else:
            assert np.array_equal(got_pre, ref_pre) and np.array_equal(got_dec, ref_dec)
        x = np.concatenate([ref_pre, ref_dec])
