"""The matmul kernels at the full sizes of the benchmark configurations, through properties that do
not need the oracle to process the whole matrix: sampled rows must equal the oracle run on exactly
those rows; the output is linear in the activation scales (a power-of-two factor must come through
bit-exactly); a launch is deterministic; and the per-token results of the batch and tensor-core
paths agree with the single-token path on the same token."""
import numpy as np
import pytest
import torch

from oracle import binding as orc
from test_gpu_kernels import _weights, rel_err

pytestmark = pytest.mark.gpu

SHAPES = [(5120, 27648), (27648, 5120), (8192, 28672), (28672, 8192), (151936, 2048)]


@pytest.fixture(scope="module")
def ops():
    from mesh_llm_b200 import ops as o

    return o


@pytest.mark.parametrize("ty", [orc.TYPE_Q4_K, orc.TYPE_Q6_K])
@pytest.mark.parametrize("N,K", SHAPES)
def test_full_size_matmul_properties(ops, ty, N, K):
    W = _weights(ty, N, K, N % 97 + ty, random_bytes=True)
    dev = ops.upload_weights(ty, W, N, K)
    rng = np.random.default_rng(N + K)
    rows = np.sort(rng.choice(N, 48, replace=False))
    rows[0], rows[-1] = 0, N - 1
    sub = np.ascontiguousarray(W[rows])
    x = rng.standard_normal((8, K)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    q, d, bs = ops.quantize_act(xd)
    ref = orc.mul_mat(ty, sub, x, len(rows), K)  # [8][48]
    # decode paths: 1 token (streaming kernel), 2 tokens, 8 tokens (tensor-core form for Q4_K)
    y1 = ops.mul_mat_q8(ty, dev, q[:1], d[:1], bs[:1], N, K)
    y2 = ops.mul_mat_q8(ty, dev, q[:2], d[:2], bs[:2], N, K)
    y8 = ops.mul_mat_q8(ty, dev, q, d, bs, N, K)
    for y, m in ((y1, 1), (y2, 2), (y8, 8)):
        got = y.cpu().numpy()[:, rows]
        assert rel_err(got, ref[:m]) <= 1e-3, (m, rel_err(got, ref[:m]))
    # the same token through the three paths
    assert rel_err(y2[:1].cpu().numpy(), y1.cpu().numpy()) <= 1e-5
    assert rel_err(y8[:1].cpu().numpy(), y1.cpu().numpy()) <= 1e-5
    # deterministic
    assert torch.equal(ops.mul_mat_q8(ty, dev, q[:1], d[:1], bs[:1], N, K), y1)
    assert torch.equal(ops.mul_mat_q8(ty, dev, q, d, bs, N, K), y8)
    # linear in the activation scales: an exact factor of 4 comes through bit for bit
    y1s = ops.mul_mat_q8(ty, dev, q[:1], d[:1] * 4, bs[:1], N, K)
    assert torch.equal(y1s, y1 * 4)
    y8s = ops.mul_mat_q8(ty, dev, q, d * 0.5, bs, N, K)
    assert torch.equal(y8s, y8 * 0.5)


@pytest.mark.parametrize("ty,N,K", [(orc.TYPE_Q4_K, 27648, 5120), (orc.TYPE_Q6_K, 5120, 27648), (orc.TYPE_Q6_K, 151936, 2048)])
def test_full_size_prefill_gemm_sampled_rows(ops, ty, N, K):
    M = 512
    W = _weights(ty, N, K, 5 + ty, random_bytes=True)
    dev = ops.upload_weights(ty, W, N, K)
    rng = np.random.default_rng(K)
    rows = np.sort(rng.choice(N, 24, replace=False))
    rows[0], rows[-1] = 0, N - 1
    x = rng.standard_normal((M, K)).astype(np.float32)
    q, d, bs = ops.quantize_act(torch.from_numpy(x).cuda())
    y = ops.mul_mat_q8(ty, dev, q, d, bs, N, K)
    ref = orc.mul_mat(ty, np.ascontiguousarray(W[rows]), x, len(rows), K)
    assert rel_err(y.cpu().numpy()[:, rows], ref) <= 1e-3
    assert torch.equal(ops.mul_mat_q8(ty, dev, q, d, bs, N, K), y)  # deterministic
    # a token of the batch equals the same token through the single-token kernel
    y1 = ops.mul_mat_q8(ty, dev, q[37:38], d[37:38], bs[37:38], N, K)
    assert rel_err(y[37:38].cpu().numpy(), y1.cpu().numpy()) <= 1e-5
    assert torch.equal(ops.mul_mat_q8(ty, dev, q, d * 2, bs, N, K), y * 2)
