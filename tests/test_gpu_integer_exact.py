"""Bit-exact integer sums through the production matmul kernels, with no instrumentation.

The hot-path specification asks for the per-block integer dot sums to be bit-exact.  The kernels
return f32, so the test makes every floating-point factor exactly 1: weight blocks carry d = 1.0
(Q4_K: dmin = 0; a second case has d = 0, dmin = 1 to isolate the min term), and every 256-block of
the activations holds integers in [-127, 127] with at least one +-127, so that the Q8 scale is
127 / 127 = 1 and the codes are the values themselves.  The f32 result is then the integer
sum_blocks sum_j sc_j sum_i q_ij a_ij itself (kept below 2^24, where f32 is exact under any order of
accumulation), and it must equal the CPU oracle's int32 block sums bit for bit.

Token counts select the kernels: M = 1, 2 the streaming decode GEMV (gemv_block_kernel<type, 1|2>),
M = 3..8 its mma.m16n8k32 batch form (Q4_K) or the dp4a kernel (Q6_K), M > 8 the tcgen05 prefill
GEMM with its two-plane recombination (from 384 tokens on in its form with pre-unpacked operand images).
"""
import numpy as np
import pytest

from oracle import binding as orc

pytestmark = pytest.mark.gpu

F16_ONE = np.array([1.0], np.float16).view(np.uint8)
F16_ZERO = np.array([0.0], np.float16).view(np.uint8)


@pytest.fixture(scope="module")
def ops():
    import torch

    assert torch.cuda.is_available()
    from mesh_llm_b200 import ops as o

    return o


def unit_blocks(ty, N, K, seed, min_only=False):
    """random valid blocks whose f16 scale factors are exactly 1 (or 0)"""
    rng = np.random.default_rng(seed)
    nblk = N * K // 256
    if ty == orc.TYPE_Q4_K:
        blk = rng.integers(0, 256, size=(nblk, 144), dtype=np.uint8)
        blk[:, 0:2] = F16_ZERO if min_only else F16_ONE  # d
        blk[:, 2:4] = F16_ONE if min_only else F16_ZERO  # dmin
    else:
        blk = rng.integers(0, 256, size=(nblk, 210), dtype=np.uint8)
        blk[:, 208:210] = F16_ONE
        # int8 scales of both signs, kept within +-48 so that sums over 2048 elements stay below 2^24
        blk[:, 192:208] = rng.integers(-48, 49, size=(nblk, 16)).astype(np.int8).view(np.uint8)
    return blk.reshape(N, -1)


def unit_scale_activations(M, K, seed):
    """integers in [-127, 127], one +-127 per 256-block: Q8 scale 1.0, codes = values"""
    rng = np.random.default_rng(seed)
    x = rng.integers(-127, 128, size=(M, K)).astype(np.float32)
    for b in range(K // 256):
        x[np.arange(M), b * 256 + rng.integers(0, 256, M)] = rng.choice([-127.0, 127.0], M)
    return x


CASES = [(256, 256), (100, 512), (264, 512), (64, 2048)]


@pytest.mark.parametrize("ty", [orc.TYPE_Q4_K, orc.TYPE_Q6_K], ids=["q4_k", "q6_k"])
@pytest.mark.parametrize("M", [1, 2, 3, 8, 9, 130, 390])
@pytest.mark.parametrize("N,K", CASES)
def test_matmul_output_is_the_integer_sum(ops, ty, M, N, K):
    import torch

    W = unit_blocks(ty, N, K, 100 + K)
    x = unit_scale_activations(M, K, 200 + M)
    q, d, bs = orc.quantize_act(x)
    assert np.all(d == 1.0) and np.array_equal(q.astype(np.float32), x)
    si, _ = orc.block_sums(ty, W, q, bs, N, K)
    want = si.astype(np.int64).sum(-1)  # [M][N]
    assert np.abs(si.astype(np.int64)).cumsum(-1).max() < 2 ** 24  # every partial sum is exact in f32
    dev = ops.upload_weights(ty, W, N, K)
    y = ops.mul_mat(ty, dev, torch.from_numpy(x).cuda(), N, K).cpu().numpy()
    assert y.dtype == np.float32
    np.testing.assert_array_equal(y.astype(np.int64), want)
    assert np.array_equal(y, want.astype(np.float32))


@pytest.mark.parametrize("M", [1, 2, 3, 8, 9, 130, 390])
@pytest.mark.parametrize("N,K", CASES)
def test_q4k_min_term_is_the_integer_sum(ops, M, N, K):
    """d = 0, dmin = 1: the output is minus sum_blocks sum_j m_j sum_i a_ij"""
    import torch

    ty = orc.TYPE_Q4_K
    W = unit_blocks(ty, N, K, 300 + K, min_only=True)
    x = unit_scale_activations(M, K, 400 + M)
    q, d, bs = orc.quantize_act(x)
    _, sm = orc.block_sums(ty, W, q, bs, N, K)
    want = -sm.astype(np.int64).sum(-1)
    assert np.abs(sm.astype(np.int64)).cumsum(-1).max() < 2 ** 24
    dev = ops.upload_weights(ty, W, N, K)
    y = ops.mul_mat(ty, dev, torch.from_numpy(x).cuda(), N, K).cpu().numpy()
    assert np.array_equal(y, want.astype(np.float32))
