"""Expert assignment against the reference's own cases (mesh-llm/src/inference/moe.rs:841-889,
1156-1260) and the expert-shard writer against numpy slices of the source file (llama-moe-split
semantics, llama.cpp patches/0003 lines 1040-1113, 1142-1191).  Host code only."""
import numpy as np
import pytest

from oracle import binding as orc
from mesh_llm_b200.capi import B200Error
from mesh_llm_b200.gguf import GgufFile, moe_assign
from gguf_util import write_model_gguf

MOE = dict(n_layer=2, n_embd=512, n_head=4, n_head_kv=2, head_dim=128, n_ff=0, n_vocab=512, n_ctx=64,
           qkv_bias=0, rope_neox=1, rope_theta=1e6, rms_eps=1e-6, n_expert=8, n_expert_used=4, n_ff_exp=256)


def test_assignments_2_nodes():
    a = moe_assign(range(10), 2, 4)
    assert [len(x["experts"]) for x in a] == [7, 7] and a[0]["n_shared"] == 4 and a[0]["n_unique"] == 3
    assert all(set(range(4)) <= set(x["experts"]) for x in a)
    assert sorted(set(a[0]["experts"]) | set(a[1]["experts"])) == list(range(10))
    assert a[0]["experts"] == [0, 1, 2, 3, 4, 6, 8] and a[1]["experts"] == [0, 1, 2, 3, 5, 7, 9]


def test_assignments_3_nodes_and_single_node():
    a = moe_assign(range(128), 3, 46)
    assert [len(x["experts"]) for x in a] == [74, 73, 73]
    assert sorted(set().union(*[x["experts"] for x in a])) == list(range(128))
    one = moe_assign(range(8), 1, 4)
    assert len(one) == 1 and one[0]["experts"] == list(range(8))


def test_overlap_cases():
    a = moe_assign(range(128), 3, 46, overlap=2)
    count = np.zeros(128, int)
    for x in a:
        count[x["experts"]] += 1
    assert (count[:46] == 3).all() and (count[46:] >= 2).all()
    assert [len(x["experts"]) for x in moe_assign(range(10), 2, 4, overlap=2)] == [10, 10]
    assert [x["experts"] for x in moe_assign(range(128), 3, 46, overlap=1)] == [x["experts"] for x in moe_assign(range(128), 3, 46)]
    assert all(len(x["experts"]) == 20 for x in moe_assign(range(20), 3, 5, overlap=10))  # capped at the node count
    g = moe_assign(range(256), 10, 96, overlap=2)
    count = np.zeros(256, int)
    for x in g:
        count[x["experts"]] += 1
    assert (count > 0).all() and (count[96:] >= 2).all()


def test_snake_draft_and_ranking_order():
    ranking = [7, 3, 5, 0, 1, 2, 4, 6, 9, 8]
    a = moe_assign(ranking, 3, 2, mode=1)
    # core {7, 3}; remaining 5 0 1 | 6 4 2 (reversed) | 9 8 dealt in snake order
    assert a[0]["experts"] == sorted([7, 3, 5, 6, 9]) and a[1]["experts"] == sorted([7, 3, 0, 4, 8])
    assert a[2]["experts"] == sorted([7, 3, 1, 2]) and a[0]["n_shared"] == 2 and a[0]["n_unique"] == 3
    assert moe_assign(ranking, 1, 2)[0]["experts"] == ranking  # a single node keeps the ranking order


def test_shard_writer_slices_experts_and_router(tmp_path):
    import gguf

    m = orc.Model(**MOE)
    m.generate(3)
    src = tmp_path / "moe.gguf"
    write_model_gguf(src, m, arch="qwen3moe", extra_kv={"qwen3moe.vocab_size": MOE["n_vocab"]})
    ids = [6, 1, 4]
    dst = tmp_path / "shard.gguf"
    with GgufFile(src) as g:
        written = g.write_expert_shard(ids, dst)
        src_t = {t["name"]: t for t in g.tensors()}
        src_bytes = {n: g.read(n) for n in src_t}
    assert written == dst.stat().st_size
    with GgufFile(dst) as s:
        meta = s.meta()
        assert meta["expert_count"] == 3 and meta["expert_used_count"] == 3  # clamped from 4
        assert meta["embedding_length"] == MOE["n_embd"] and meta["vocab_size"] == MOE["n_vocab"]
        shard_t = {t["name"]: t for t in s.tensors()}
        assert list(shard_t) == list(src_t)
        for name, t in shard_t.items():
            got = s.read(name)
            packed = any(k in name for k in ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps", "ffn_gate_inp"))
            if packed:
                per = src_t[name]["nbytes"] // MOE["n_expert"]
                want = np.concatenate([src_bytes[name][e * per:(e + 1) * per] for e in ids])
                assert t["ne"][t["n_dims"] - 1] == 3 and t["nbytes"] == 3 * per
                assert t["ne"][: t["n_dims"] - 1] == src_t[name]["ne"][: t["n_dims"] - 1]
            else:
                want = src_bytes[name]
                assert t["ne"] == src_t[name]["ne"]
            assert np.array_equal(got, want), name
            assert t["file_offset"] % 32 == 0
    # an independent reader accepts the file and sees the same shapes
    r = gguf.GGUFReader(str(dst))
    assert int(r.fields["qwen3moe.expert_count"].parts[-1][0]) == 3
    shapes = {t.name: [int(x) for x in t.shape] for t in r.tensors}
    assert shapes["blk.0.ffn_gate_exps.weight"][-1] == 3 and shapes["blk.1.ffn_gate_inp.weight"][-1] == 3


def test_shard_writer_rejects_bad_requests(tmp_path):
    m = orc.Model(**MOE)
    m.generate(3)
    src = tmp_path / "moe.gguf"
    write_model_gguf(src, m, arch="qwen3moe")
    with GgufFile(src) as g:
        for ids, msg in (([8], "out of range"), ([1, 1], "twice"), ([], "experts of")):
            with pytest.raises(B200Error, match=msg):
                g.write_expert_shard(ids, tmp_path / "x.gguf")
    dense = orc.Model(n_layer=1, n_embd=512, n_head=4, n_head_kv=2, head_dim=128, n_ff=512, n_vocab=512, n_ctx=64)
    dense.generate(1)
    write_model_gguf(tmp_path / "dense.gguf", dense, arch="qwen2")
    with GgufFile(tmp_path / "dense.gguf") as g:
        with pytest.raises(B200Error, match="not a mixture"):
            g.write_expert_shard([0], tmp_path / "y.gguf")
