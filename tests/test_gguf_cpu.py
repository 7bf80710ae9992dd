"""GGUF reader of the library against the known-answer cases of the reference's own scanner
(mesh-client/src/models/gguf.rs:621-758) and against files written by gguf-py.  Host code only."""
import struct

import numpy as np
import pytest

from mesh_llm_b200.capi import B200Error
from mesh_llm_b200.gguf import GgufFile
from gguf_util import (ARRAY, U8, align, array_header, gstr, header, kv_f32, kv_i32, kv_str, kv_u32,
                       tensor_info)


def write(tmp_path, name, data):
    p = tmp_path / name
    p.write_bytes(data)
    return p


def test_rejects_bad_magic_and_old_version(tmp_path):
    with pytest.raises(B200Error, match="not a GGUF file"):
        GgufFile(write(tmp_path, "a.gguf", b"GGML" + bytes(32)))
    with pytest.raises(B200Error, match="version"):
        GgufFile(write(tmp_path, "b.gguf", header(0, 0, version=1)))
    with pytest.raises(B200Error, match="cannot open"):
        GgufFile(tmp_path / "missing.gguf")


def test_rejects_nested_array_bomb(tmp_path):
    # gguf.rs:652-669: 65 levels of array nesting inside general.architecture
    data = header(0, 1) + gstr("general.architecture") + struct.pack("<I", ARRAY)
    for _ in range(64):
        data += array_header(ARRAY, 1)
    data += array_header(U8, 1) + b"\0"
    with pytest.raises(B200Error):
        GgufFile(write(tmp_path, "bomb.gguf", data))
    # the same under a key the scanner skips: the depth limit itself
    data = header(0, 1) + gstr("some.other.key") + struct.pack("<I", ARRAY)
    for _ in range(64):
        data += array_header(ARRAY, 1)
    data += array_header(U8, 1) + b"\0"
    with pytest.raises(B200Error, match="nesting too deep"):
        GgufFile(write(tmp_path, "deep.gguf", data))


def test_rejects_oversized_array_and_string(tmp_path):
    data = header(0, 1) + gstr("x.list") + struct.pack("<I", ARRAY) + array_header(U8, 1_000_001)
    with pytest.raises(B200Error, match="array too long"):
        GgufFile(write(tmp_path, "arr.gguf", data))
    data = header(0, 1) + struct.pack("<Q", 1_000_001)
    with pytest.raises(B200Error, match="string too long"):
        GgufFile(write(tmp_path, "str.gguf", data))


def test_rejects_negative_and_excessive_counts(tmp_path):
    with pytest.raises(B200Error, match="negative KV count"):
        GgufFile(write(tmp_path, "neg.gguf", header(0, -1)))
    with pytest.raises(B200Error, match="tensor count too large"):
        GgufFile(write(tmp_path, "big.gguf", header(1_000_001, 0)))
    with pytest.raises(B200Error, match="end of file"):
        GgufFile(write(tmp_path, "trunc.gguf", header(0, 3) + kv_u32("llama.block_count", 4)))


def test_rejects_negative_int_for_unsigned_field(tmp_path):
    data = header(0, 1) + kv_i32("llama.block_count", -4)  # gguf.rs:716-726
    with pytest.raises(B200Error, match="negative value"):
        GgufFile(write(tmp_path, "negint.gguf", data))


def test_value_length_from_kv_heads_without_head_count(tmp_path):
    data = header(0, 2) + kv_u32("llama.embedding_length", 4096) + kv_u32("llama.attention.head_count_kv", 8)
    with GgufFile(write(tmp_path, "kvheads.gguf", data)) as g:
        m = g.meta()
    assert (m["head_count"], m["key_length"], m["value_length"]) == (0, 0, 512)  # gguf.rs:672-687


def test_compact_meta_fields(tmp_path):
    kvs = [kv_str("general.architecture", "qwen3moe"), kv_str("tokenizer.ggml.model", "gpt2"),
           kv_u32("qwen3moe.context_length", 40960), kv_u32("qwen3moe.embedding_length", 2048),
           kv_u32("qwen3moe.attention.head_count", 32), kv_u32("qwen3moe.attention.head_count_kv", 4),
           kv_u32("qwen3moe.block_count", 48), kv_u32("qwen3moe.feed_forward_length", 6144),
           kv_u32("qwen3moe.expert_feed_forward_length", 768), kv_u32("qwen3moe.attention.key_length", 128),
           kv_u32("qwen3moe.expert_count", 128), kv_u32("qwen3moe.expert_used_count", 8),
           kv_f32("qwen3moe.rope.freq_base", 1e6), kv_f32("qwen3moe.attention.layer_norm_rms_epsilon", 1e-6),
           kv_u32("qwen3moe.vocab_size", 151936),
           gstr("tokenizer.ggml.tokens") + struct.pack("<I", ARRAY) + array_header(8, 2) + gstr("a") + gstr("b")]
    with GgufFile(write(tmp_path, "meta.gguf", header(0, len(kvs)) + b"".join(kvs))) as g:
        m = g.meta()
    assert m["architecture"] == "qwen3moe" and m["tokenizer_model"] == "gpt2"
    assert (m["context_length"], m["embedding_length"], m["head_count"], m["head_count_kv"]) == (40960, 2048, 32, 4)
    assert (m["block_count"], m["feed_forward_length"], m["expert_feed_forward_length"]) == (48, 6144, 768)
    assert (m["key_length"], m["value_length"]) == (128, 512)  # value length derived: 2048 / 4 kv heads
    assert (m["expert_count"], m["expert_used_count"], m["vocab_size"]) == (128, 8, 151936)
    assert m["rope_freq_base"] == pytest.approx(1e6) and m["rms_epsilon"] == pytest.approx(1e-6)


def test_byte_profile_splits_base_and_expert_bytes(tmp_path):
    # gguf.rs:728-757: expert tensor at offset 0, attention tensor at 64, 96 bytes of data
    data = header(2, 3) + kv_u32("general.alignment", 32) + kv_u32("llama.expert_count", 8) + \
        kv_u32("llama.expert_used_count", 2) + tensor_info("blk.0.ffn_up_exps.weight", 0) + \
        tensor_info("blk.0.attn_q.weight", 64)
    data = data.ljust(align(len(data)), b"\0") + bytes(96)
    with GgufFile(write(tmp_path, "prof.gguf", data)) as g:
        p = g.byte_profile()
        t = g.tensors()
    assert (p["expert_count"], p["expert_used_count"]) == (8, 2)
    assert (p["expert_tensor_bytes"], p["base_resident_bytes"]) == (64, 32)
    assert p["full_model_bytes"] == len(data)
    assert p["full_model_bytes"] == p["base_resident_bytes"] + p["expert_tensor_bytes"] + p["file_overhead_bytes"]
    assert [x["name"] for x in t] == ["blk.0.ffn_up_exps.weight", "blk.0.attn_q.weight"]
    assert t[1]["file_offset"] == len(data) - 96 + 64 and t[1]["nbytes"] == 16


def test_empty_tensor_table_profile(tmp_path):
    data = header(0, 1) + kv_u32("llama.expert_count", 4)
    with GgufFile(write(tmp_path, "empty.gguf", data)) as g:
        p = g.byte_profile()
    assert p["file_overhead_bytes"] == len(data) == p["full_model_bytes"] and p["base_resident_bytes"] == 0


def test_rejects_tensor_outside_file(tmp_path):
    data = header(1, 0) + tensor_info("blk.0.attn_q.weight", 0, dims=(256, 64), ggml_type=12)
    data = data.ljust(align(len(data)), b"\0") + bytes(100)  # 64 rows x 144 bytes do not fit
    with pytest.raises(B200Error, match="outside the file"):
        GgufFile(write(tmp_path, "short.gguf", data))


def test_against_gguf_py_writer(tmp_path):
    import gguf

    rng = np.random.default_rng(5)
    path = tmp_path / "w.gguf"
    w = gguf.GGUFWriter(str(path), "llama")
    w.add_uint32("llama.block_count", 2)
    w.add_uint32("llama.embedding_length", 512)
    w.add_uint32("llama.attention.head_count", 4)
    w.add_uint32("llama.feed_forward_length", 1024)
    w.add_float32("llama.rope.freq_base", 5e5)
    w.add_array("tokenizer.ggml.tokens", ["<s>", "</s>", "x"])
    tensors = {
        "token_embd.weight": (rng.integers(0, 256, (64, 2 * 144), dtype=np.uint8), gguf.GGMLQuantizationType.Q4_K),
        "blk.0.attn_norm.weight": (rng.standard_normal(512).astype(np.float32), None),
        "blk.1.ffn_down.weight": (rng.integers(0, 256, (512, 4 * 210), dtype=np.uint8), gguf.GGMLQuantizationType.Q6_K),
        "blk.1.ffn_up_exps.weight": (rng.integers(0, 256, (3, 256, 2 * 144), dtype=np.uint8), gguf.GGMLQuantizationType.Q4_K),
    }
    for name, (arr, qt) in tensors.items():
        w.add_tensor(name, arr, raw_dtype=qt)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    ref = {t.name: t for t in gguf.GGUFReader(str(path)).tensors}
    with GgufFile(path) as g:
        m = g.meta()
        assert (m["architecture"], m["block_count"], m["embedding_length"], m["head_count"]) == ("llama", 2, 512, 4)
        assert m["vocab_size"] == 64  # taken from token_embd when the key is absent
        infos = {t["name"]: t for t in g.tensors()}
        assert set(infos) == set(tensors)
        for name, (arr, qt) in tensors.items():
            t, r = infos[name], ref[name]
            assert t["type"] == int(r.tensor_type) and t["nbytes"] == arr.nbytes == int(r.n_bytes)
            assert t["file_offset"] == int(r.data_offset)
            assert t["ne"][: t["n_dims"]] == [int(x) for x in r.shape]
            assert np.array_equal(g.read(name), arr.view(np.uint8).reshape(-1))
        assert g.find("nope") == -1
        cfg = g.stage_config(layer_begin=1, layer_end=-1, n_ctx=128, n_seq=2, n_ubatch=16)
        assert (cfg.n_layer, cfg.layer_begin, cfg.layer_end, cfg.has_embd, cfg.has_output) == (2, 1, 2, 0, 1)
        assert (cfg.n_embd, cfg.n_head, cfg.n_head_kv, cfg.head_dim, cfg.n_ff) == (512, 4, 4, 128, 1024)
        assert cfg.rope_neox == 0 and cfg.qkv_bias == 0 and cfg.rope_theta == pytest.approx(5e5)
        p = g.byte_profile()
        assert p["expert_tensor_bytes"] >= tensors["blk.1.ffn_up_exps.weight"][0].nbytes
