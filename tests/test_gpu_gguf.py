"""Per-stage selective load from a GGUF file (SET_TENSOR_GGUF semantics, llama.cpp patches/0001
lines 179-266): a stage created from the file's metadata reads exactly its own tensors by name,
holds the same bytes as a stage fed through set_tensor, and computes the same result."""
import os

import numpy as np
import pytest
import torch

from oracle import binding as orc
from mesh_llm_b200.gguf import GgufFile
from mesh_llm_b200.stage import Stage
from gguf_util import write_model_gguf

pytestmark = pytest.mark.gpu

CFG = dict(n_layer=2, n_embd=512, n_head=4, n_head_kv=2, head_dim=128, n_ff=1024, n_vocab=2048, n_ctx=96,
           qkv_bias=1, rope_neox=1, rope_theta=1e6, rms_eps=1e-6)
MOE = dict(n_layer=2, n_embd=512, n_head=4, n_head_kv=2, head_dim=128, n_ff=0, n_vocab=2048, n_ctx=96,
           qkv_bias=0, rope_neox=1, rope_theta=1e6, rms_eps=1e-6, n_expert=8, n_expert_used=2, n_ff_exp=256)


def make(tmp_path, cfg, arch):
    m = orc.Model(**cfg)
    m.generate(23)
    path = tmp_path / "model.gguf"
    write_model_gguf(path, m, arch=arch)
    return m, path


@pytest.mark.parametrize("cfg,arch", [(CFG, "qwen2"), (MOE, "qwen3moe")])
def test_stage_from_gguf_matches_set_tensor_stage(tmp_path, cfg, arch):
    m, path = make(tmp_path, cfg, arch)
    with GgufFile(path) as g:
        st, n_loaded, nbytes = Stage.from_gguf(g, n_ctx=cfg["n_ctx"], n_ubatch=32)
        infos = {t["name"]: t for t in g.tensors()}
    names = [n for n, _, _ in st.tensor_names()]
    assert n_loaded == len(names) == len(m.tensor_names())
    assert nbytes == sum(infos[n]["nbytes"] for n in names)
    for key in ("n_layer", "n_embd", "n_head", "n_head_kv", "head_dim", "n_ff", "n_vocab", "qkv_bias", "rope_neox",
                "n_expert", "n_expert_used", "n_ff_exp"):
        assert getattr(st.cfg, key) == cfg.get(key, 0), key
    ref = Stage(**cfg, n_ubatch=32)
    ref.load((n,) + m.tensor(n)[:2] for n in m.tensor_names())
    for n in names:  # same bytes back out of both (inverse of the device repack)
        ty, data, _ = m.tensor(n)
        assert np.array_equal(st.get_tensor(n, data.size), data), n
    toks = torch.from_numpy(np.random.default_rng(1).integers(0, cfg["n_vocab"], 19).astype(np.int32)).cuda()
    _, lg_a, _ = st.forward(tokens=toks, all_logits=True)
    _, lg_b, _ = ref.forward(tokens=toks, all_logits=True)
    assert torch.equal(lg_a, lg_b)
    _, ref_logits = m.forward(tokens=toks.cpu().numpy())
    assert (lg_a.cpu().numpy().argmax(-1) == ref_logits.argmax(-1)).mean() >= 0.9


def test_two_stages_read_only_their_own_tensors(tmp_path):
    m, path = make(tmp_path, CFG, "qwen2")
    size = os.path.getsize(path)
    with GgufFile(path) as g:
        s0, n0, b0 = Stage.from_gguf(g, layer_begin=0, layer_end=1, n_ctx=CFG["n_ctx"], n_ubatch=32)
        s1, n1, b1 = Stage.from_gguf(g, layer_begin=1, layer_end=2, n_ctx=CFG["n_ctx"], n_ubatch=32)
        whole, nw, bw = Stage.from_gguf(g, n_ctx=CFG["n_ctx"], n_ubatch=32)
    names0 = {n for n, _, _ in s0.tensor_names()}
    names1 = {n for n, _, _ in s1.tensor_names()}
    assert "token_embd.weight" in names0 and "output.weight" in names1 and not (names0 & names1)
    assert all(n.startswith("blk.0.") or n == "token_embd.weight" for n in names0)
    assert n0 + n1 == nw and b0 + b1 == bw and b0 < size and b1 < size
    toks = torch.from_numpy(np.random.default_rng(2).integers(0, CFG["n_vocab"], 11).astype(np.int32)).cuda()
    hid, _, _ = s0.forward(tokens=toks)
    _, lg2, nx2 = s1.forward(hidden_in=hid, all_logits=True)
    _, lg1, nx1 = whole.forward(tokens=toks, all_logits=True)
    assert torch.equal(lg1, lg2) and torch.equal(nx1, nx2)


def test_missing_tensor_and_unsupported_type_are_reported(tmp_path):
    import gguf
    from mesh_llm_b200.capi import B200Error

    m, path = make(tmp_path, CFG, "qwen2")
    # a file that lacks one tensor the stage owns
    path2 = tmp_path / "partial.gguf"
    w = gguf.GGUFWriter(str(path2), "qwen2")
    for k, v in (("block_count", 2), ("embedding_length", 512), ("attention.head_count", 4),
                 ("attention.head_count_kv", 2), ("feed_forward_length", 1024), ("attention.key_length", 128)):
        w.add_uint32(f"qwen2.{k}", v)
    w.add_tensor("token_embd.weight", np.zeros((2048, 2 * 144), np.uint8), raw_dtype=gguf.GGMLQuantizationType.Q4_K)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    with GgufFile(path2) as g:
        with pytest.raises(B200Error, match="has no tensor"):
            Stage.from_gguf(g, n_ctx=64, n_ubatch=16)


def test_expert_shard_stage_matches_oracle_on_the_same_shard(tmp_path):
    """A shard file written by the library, loaded as a stage, against the CPU oracle holding the same
    experts (router rows gathered in the same order): the shard is a complete model of its own."""
    m, path = make(tmp_path, MOE, "qwen3moe")
    ids = [5, 0, 3, 6]
    shard_path = tmp_path / "shard.gguf"
    with GgufFile(path) as g:
        g.write_expert_shard(ids, shard_path)
    cfg = dict(MOE, n_expert=len(ids), n_expert_used=min(MOE["n_expert_used"], len(ids)))
    ref = orc.Model(**cfg)
    for name in m.tensor_names():
        ty, data, ne = m.tensor(name)
        if any(k in name for k in ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps", "ffn_gate_inp")):
            per = data.size // MOE["n_expert"]
            data = np.concatenate([data[e * per:(e + 1) * per] for e in ids])
        ref.set_tensor(name, ty, data)
    with GgufFile(shard_path) as s:
        st, n_loaded, _ = Stage.from_gguf(s, n_ctx=MOE["n_ctx"], n_ubatch=32)
    assert st.cfg.n_expert == 4 and st.cfg.n_expert_used == 2 and n_loaded == len(m.tensor_names())
    toks = np.random.default_rng(4).integers(0, MOE["n_vocab"], 13).astype(np.int32)
    hid = torch.empty((13, MOE["n_embd"]), device="cuda")
    _, lg, _ = st.forward(tokens=torch.from_numpy(toks).cuda(), all_logits=True, hidden_out=hid)
    href, lref = ref.forward(tokens=toks)
    # Two layers end to end: a single activation code that rounds the other way (or one f16 cache element)
    # moves every later row by up to about 1e-2 (see tests/layer_oracle.py), while a wrong expert or a
    # router row out of place moves them by 1e-1 and more.  The strict per-segment bound is checked at
    # full width in tests/test_gpu_real_widths.py; here the question is whether the shard is the model.
    err = np.abs(hid.cpu().numpy() - href).max(-1) / np.abs(href).max()
    assert err.max() <= 3e-2 and np.median(err) <= 1e-2, err
    got, a, b = lg.cpu().numpy().astype(np.float64), None, None
    a = lref.astype(np.float64) - lref.max(-1, keepdims=True)
    b = got - got.max(-1, keepdims=True)
    pa = np.exp(a) / np.exp(a).sum(-1, keepdims=True)
    kl = (pa * ((a - np.log(np.exp(a).sum(-1, keepdims=True))) - (b - np.log(np.exp(b).sum(-1, keepdims=True))))).sum(-1).mean()
    assert kl < 1e-4, kl
    assert (lg.cpu().numpy().argmax(-1) == lref.argmax(-1)).mean() >= 0.9
