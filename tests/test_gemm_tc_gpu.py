"""GPU: the tcgen05 batched GEMM (more than 8 activation rows) against the oracle.

Tolerance: max|y - y_ref| / max|y_ref| <= 1e-3 (operands are rounded once to f16 on this path).
"""
import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-3


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run(ctx, kb, torch, dtype, blocks, x, M, N, K):
    y = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    fn = ctx.gemm_q8_0 if dtype == kb.DTYPE_Q8_0 else ctx.gemm_q4_k
    fn(dev(torch, blocks), dev(torch, x), y, M, N, K, kb.ACT_F32)
    ctx.sync()
    return y.cpu().numpy()


@pytest.mark.parametrize("M,N,K", [(16, 128, 256), (9, 320, 1024), (32, 960, 960), (100, 200, 2560),
                                   (128, 1000, 512), (256, 384, 768), (300, 136, 256),
                                   (64, 2560, 960)])
def test_q8_0_gemm(ctx, kb, oracle, torch_cuda, M, N, K):
    rng = np.random.Generator(np.random.PCG64(0xB2000800 + M * 7 + N * 3 + K))
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    blocks = oracle.quantize_weights_q8_0(w)
    got = run(ctx, kb, torch_cuda, kb.DTYPE_Q8_0, blocks, x, M, N, K)
    assert rel_err(got, oracle.gemm_q8_0(blocks, x, M, N, K)) <= TOL


@pytest.mark.parametrize("M,N,K", [(16, 128, 256), (12, 320, 1024), (32, 1024, 4096),
                                   (128, 264, 512), (200, 130, 768), (512, 256, 1024)])
def test_q4_k_gemm(ctx, kb, oracle, torch_cuda, M, N, K):
    rng = np.random.Generator(np.random.PCG64(0xB2000900 + M * 7 + N * 3 + K))
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    blocks = oracle.quantize_weights_q4_k(w)
    got = run(ctx, kb, torch_cuda, kb.DTYPE_Q4_K, blocks, x, M, N, K)
    assert rel_err(got, oracle.gemm_q4_k(blocks, x, M, N, K)) <= TOL


def test_gemm_rows_equal_gemv_rows(ctx, kb, oracle, torch_cuda):
    """Every row of the batched result is the GEMV of that activation row (the reference's
    forward_batch == per-sequence check, tests/test_batched_forward.rs:52-201), here between
    the tensor-core path and the streaming path, within twice the tolerance."""
    torch = torch_cuda
    rng = np.random.Generator(np.random.PCG64(0xB2000A00))
    M, N, K = 40, 512, 1024
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    b4 = oracle.quantize_weights_q4_k(w)
    big = run(ctx, kb, torch, kb.DTYPE_Q4_K, b4, x, M, N, K)
    for m in (0, 17, 39):
        one = run(ctx, kb, torch, kb.DTYPE_Q4_K, b4, x[m:m + 1], 1, N, K)
        assert rel_err(big[m], one[0]) <= 2 * TOL
