"""Test helpers: GGUF files written byte by byte (the shapes the reference's own scanner tests
use, mesh-client/src/models/gguf.rs:600-758) and with the gguf-py writer of the image."""
from __future__ import annotations

import struct

import numpy as np

U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 = range(13)


def gstr(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def kv_u32(key, v):
    return gstr(key) + struct.pack("<II", U32, v)


def kv_i32(key, v):
    return gstr(key) + struct.pack("<Ii", I32, v)


def kv_f32(key, v):
    return gstr(key) + struct.pack("<If", F32, v)


def kv_str(key, v):
    return gstr(key) + struct.pack("<I", STRING) + gstr(v)


def array_header(elem_type, count):
    return struct.pack("<IQ", elem_type, count)


def header(n_tensors, n_kv, version=2):
    return b"GGUF" + struct.pack("<Iqq", version, n_tensors, n_kv)


def tensor_info(name, offset, dims=(16,), ggml_type=24):  # default: 16 x I8, as the reference's tests use
    out = gstr(name) + struct.pack("<I", len(dims))
    for d in dims:
        out += struct.pack("<Q", d)
    return out + struct.pack("<IQ", ggml_type, offset)


def align(n, a=32):
    return (n + a - 1) // a * a


def write_model_gguf(path, model, arch="qwen2", extra_kv=None):
    """Writes every tensor of an oracle model (names, types and bytes as the oracle holds them) with
    the metadata keys a loader needs, using the gguf-py writer."""
    import gguf

    c = model.cfg
    w = gguf.GGUFWriter(str(path), arch)
    w.add_uint32(f"{arch}.block_count", c.n_layer)
    w.add_uint32(f"{arch}.context_length", 4096)
    w.add_uint32(f"{arch}.embedding_length", c.n_embd)
    w.add_uint32(f"{arch}.attention.head_count", c.n_head)
    w.add_uint32(f"{arch}.attention.head_count_kv", c.n_head_kv)
    w.add_uint32(f"{arch}.attention.key_length", c.head_dim)
    w.add_uint32(f"{arch}.attention.value_length", c.head_dim)
    w.add_float32(f"{arch}.attention.layer_norm_rms_epsilon", c.rms_eps)
    w.add_float32(f"{arch}.rope.freq_base", c.rope_theta)
    if c.n_expert:
        w.add_uint32(f"{arch}.expert_count", c.n_expert)
        w.add_uint32(f"{arch}.expert_used_count", c.n_expert_used)
        w.add_uint32(f"{arch}.expert_feed_forward_length", c.n_ff_exp)
    else:
        w.add_uint32(f"{arch}.feed_forward_length", c.n_ff)
    for k, v in (extra_kv or {}).items():
        w.add_uint32(k, v)
    qt = {0: gguf.GGMLQuantizationType.F32, 12: gguf.GGMLQuantizationType.Q4_K, 14: gguf.GGMLQuantizationType.Q6_K}
    for name in model.tensor_names():
        ty, data, ne = model.tensor(name)
        rows = ne[1] * ne[2]
        if ty == 0:
            arr = np.frombuffer(data.tobytes(), np.float32).reshape((ne[2], ne[1], ne[0]) if ne[2] > 1 else
                                                                    ((ne[1], ne[0]) if ne[1] > 1 else (ne[0],)))
            w.add_tensor(name, arr)
        else:
            rb = data.size // rows
            shape = (ne[2], ne[1], rb) if ne[2] > 1 else (ne[1], rb)
            w.add_tensor(name, np.frombuffer(data.tobytes(), np.uint8).reshape(shape), raw_dtype=qt[ty])
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
