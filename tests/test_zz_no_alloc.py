"""b200_mul_mat_static: the MUL_MAT entry point for callers that cannot allocate.

Some users of this library may not call cudaMalloc once they are running: a stage whose VRAM was
budgeted exactly before launch, a decode loop that cannot take cudaMalloc's device-wide stall, a
host with its own device allocator.  For them the Q8 scratch lives in a fixed array inside the
library.  This test calls the entry point through the C ABI twice in a row and checks each result
against the ordinary entry point (b200_mul_mat with caller-provided scratch) and against the CPU
oracle.  The second call uses a smaller, different problem, so anything left in the shared array
by the first call would show up as a wrong answer.  Further cases sit at the advertised limits
(8 tokens of 32768 elements, which fill the array to its last byte, and one such token), and one
checks with cudaMemGetInfo that a call leaves the device's free memory as it found it.  It is collected last so that a run stopping at the first failure has
already covered everything else, and it stands alone in a fresh process as well.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _problem(ty, M, N, K, seed):
    """random but valid blocks in GGUF layout (finite, small f16 scales), uploaded to the device"""
    import torch
    from mesh_llm_b200 import ops

    rng = np.random.default_rng(seed)
    nblk = N * K // 256
    if ty == 12:
        blk = rng.integers(0, 256, (nblk, 144), dtype=np.uint8)
        blk[:, 0:4] = np.array([0.01, 0.005], np.float16).view(np.uint8)
    else:
        blk = rng.integers(0, 256, (nblk, 210), dtype=np.uint8)
        blk[:, 208:210] = np.array([0.001], np.float16).view(np.uint8)
    W = ops.upload_weights(ty, blk.reshape(N, -1), N, K)
    x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).cuda()
    return W, x, blk.reshape(N, -1)


def _check(ty, M, N, K, seed):
    import torch
    from mesh_llm_b200 import ops
    from mesh_llm_b200.capi import check, cur_stream, lib, ptr
    from oracle import binding as orc

    W, x, host_blocks = _problem(ty, M, N, K, seed)
    want = ops.mul_mat(ty, W, x, N, K)
    got = torch.full((M, N), float("nan"), device="cuda")
    check(lib().b200_mul_mat_static(ty, ptr(W), ptr(x), M, N, K, ptr(got), cur_stream()))
    torch.cuda.synchronize()
    ref = want.cpu().numpy()
    err = np.abs(got.cpu().numpy() - ref).max() / np.abs(ref).max()
    assert err <= 1e-3, (M, N, K, err)
    cpu = orc.mul_mat(ty, host_blocks, x.cpu().numpy(), N, K)
    err = np.abs(got.cpu().numpy() - cpu).max() / np.abs(cpu).max()
    assert err <= 1e-3, ("against the CPU oracle", M, N, K, err)


@pytest.mark.parametrize("ty", [12, 14], ids=["q4_k", "q6_k"])
def test_static_scratch_entry_matches_the_allocating_one_twice_in_a_row(ty):
    for (M, N, K, seed) in ((8, 320, 8192, 1), (3, 77, 1024, 2)):
        _check(ty, M, N, K, seed)


@pytest.mark.parametrize("ty", [12, 14], ids=["q4_k", "q6_k"])
@pytest.mark.parametrize("M", [8, 1])
def test_static_scratch_entry_at_its_limits(ty, M):
    """K = 32768 with 8 tokens uses the whole array; the row is too long for the streaming kernel's
    8- and 4-token forms, and with one token it takes that kernel's whole-SM layout."""
    _check(ty, M, 40, 32768, 3 + M)


def test_static_scratch_entry_leaves_free_memory_unchanged():
    import torch
    from mesh_llm_b200.capi import check, cur_stream, lib, ptr

    W, x, _ = _problem(12, 4, 64, 2048, 9)
    y = torch.empty((4, 64), device="cuda")
    check(lib().b200_mul_mat_static(12, ptr(W), ptr(x), 4, 64, 2048, ptr(y), cur_stream()))  # set-up call
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        check(lib().b200_mul_mat_static(12, ptr(W), ptr(x), 4, 64, 2048, ptr(y), cur_stream()))
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0


def test_static_scratch_entry_rejects_oversize_calls():
    import torch
    from mesh_llm_b200.capi import B200Error, check, cur_stream, lib, ptr

    W = torch.zeros(16, dtype=torch.uint8, device="cuda")
    x = torch.zeros(16, device="cuda")
    y = torch.zeros(16, device="cuda")
    with pytest.raises(B200Error, match="exceed the built-in scratch"):
        check(lib().b200_mul_mat_static(12, ptr(W), ptr(x), 9, 4, 256, ptr(y), cur_stream()))
    with pytest.raises(B200Error, match="exceed the built-in scratch"):
        check(lib().b200_mul_mat_static(12, ptr(W), ptr(x), 1, 4, 32768 + 256, ptr(y), cur_stream()))
