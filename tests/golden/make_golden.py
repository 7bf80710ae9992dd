"""Generates the committed golden vectors under tests/golden/.

Run once in a container that has the third-party `gguf` Python package (gguf-py), which holds
an independent decoder for Q4_K / Q6_K blocks:

    python tests/golden/make_golden.py

Outputs (small .npz files):
  kquant_blocks.npz  random valid Q4_K / Q6_K blocks (every scale/min code reachable) and their
                     f32 decode as computed by gguf.quants.dequantize -- pins the block layout.
  kv_rows.npz        f32 rows (mixed magnitudes, an all-zero block, a constant block, an outlier) with
                     their ggml q8_0 / q4_0 blocks and decodes from gguf.quants.quantize /
                     dequantize -- pins the KV-cache row quantisers.
  handoff_pattern.npz the byte patterns of the stage hand-off exactness cases that
                     third_party/llama.cpp/patches/0002 (test_direct_push, lines 1612-1745)
                     pushes between two servers: i & 0xFF and 0xFF - (i & 0xFF) over 4096 bytes,
                     and the partial window offset 1024 / size 2048.
"""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def random_q4k(rng, n):
    blk = rng.integers(0, 256, size=(n, 144), dtype=np.uint8)
    d = rng.uniform(1e-4, 2e-2, size=n).astype(np.float16)
    dmin = rng.uniform(0, 2e-2, size=n).astype(np.float16)
    blk[:, 0:2] = d.view(np.uint8).reshape(n, 2)
    blk[:, 2:4] = dmin.view(np.uint8).reshape(n, 2)
    return blk


def random_q6k(rng, n):
    blk = rng.integers(0, 256, size=(n, 210), dtype=np.uint8)
    d = (rng.uniform(1e-5, 2e-3, size=n) * rng.choice([-1, 1], size=n)).astype(np.float16)
    blk[:, 208:210] = d.view(np.uint8).reshape(n, 2)
    return blk


def main():
    from gguf import GGMLQuantizationType as T
    from gguf.quants import dequantize

    rng = np.random.default_rng(20251125)
    q4 = random_q4k(rng, 64)
    q6 = random_q6k(rng, 64)
    # edge blocks: all-zero payload, all-ones payload
    q4[0, 4:] = 0
    q4[1, 4:] = 0xFF
    q6[0, :208] = 0
    q6[1, :208] = 0xFF
    np.savez_compressed(
        os.path.join(HERE, "kquant_blocks.npz"),
        q4k_blocks=q4, q4k_f32=dequantize(q4.reshape(-1), T.Q4_K).reshape(64, 256).astype(np.float32),
        q6k_blocks=q6, q6k_f32=dequantize(q6.reshape(-1), T.Q6_K).reshape(64, 256).astype(np.float32),
    )
    i = np.arange(4096)
    np.savez_compressed(
        os.path.join(HERE, "handoff_pattern.npz"),
        forward=(i & 0xFF).astype(np.uint8), reverse=(0xFF - (i & 0xFF)).astype(np.uint8),
        partial_offset=np.int64(1024), partial_size=np.int64(2048), large_bytes=np.int64(16 << 20),
    )
    from gguf.quants import quantize

    x = (rng.standard_normal((48, 128)) * rng.uniform(0.01, 10.0, size=(48, 1))).astype(np.float32)
    x[0] = 0.0
    x[1, :32] = 1.0
    x[2, 5] = -100.0
    x[3, 40] = 64.0
    q8 = quantize(x, T.Q8_0)
    q4 = quantize(x, T.Q4_0)
    np.savez_compressed(
        os.path.join(HERE, "kv_rows.npz"), x=x,
        q8_0=q8, q8_0_f32=dequantize(q8, T.Q8_0).astype(np.float32),
        q4_0=q4, q4_0_f32=dequantize(q4, T.Q4_0).astype(np.float32),
    )
    print("wrote golden vectors to", HERE)


if __name__ == "__main__":
    main()
