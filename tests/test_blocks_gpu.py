"""GPU: block-level kernels against the oracle — bit-exact where the arithmetic is pinned."""
import numpy as np
import pytest

from conftest import golden

pytestmark = pytest.mark.gpu


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_dequantize_q8_0_bit_exact(ctx, oracle, torch_cuda):
    torch = torch_cuda
    g = golden("gguf_blocks.npz")
    blocks = g["q8_0"]
    nb = blocks.size // 34
    out = torch.empty(nb * 32, dtype=torch.float32, device="cuda")
    ctx.dequantize_q8_0(dev(torch, blocks), out, nb)
    ctx.sync()
    got = out.cpu().numpy()
    assert got.tobytes() == g["q8_0_dequant"].tobytes()
    # random bytes: every f16 scale pattern that is finite, every int8 value
    rng = np.random.Generator(np.random.PCG64(1))
    raw = rng.integers(0, 256, size=4096 * 34, dtype=np.uint8)
    raw.reshape(-1, 34)[:, 1] &= 0x7B  # keep the f16 exponent below inf/nan
    ref = oracle.dequantize_q8_0(raw)
    out = torch.empty(4096 * 32, dtype=torch.float32, device="cuda")
    ctx.dequantize_q8_0(dev(torch, raw), out, 4096)
    ctx.sync()
    assert out.cpu().numpy().tobytes() == ref.tobytes()


def test_dequantize_q4_k_bit_exact(ctx, oracle, torch_cuda):
    torch = torch_cuda
    g = golden("gguf_blocks.npz")
    blocks = g["q4_k"]
    nb = blocks.size // 144
    out = torch.empty(nb * 256, dtype=torch.float32, device="cuda")
    ctx.dequantize_q4_k(dev(torch, blocks), out, nb)
    ctx.sync()
    assert out.cpu().numpy().tobytes() == g["q4_k_dequant"].tobytes()
    rng = np.random.Generator(np.random.PCG64(2))
    raw = rng.integers(0, 256, size=2048 * 144, dtype=np.uint8)
    r = raw.reshape(-1, 144)
    r[:, 1] &= 0x7B
    r[:, 3] &= 0x7B
    ref = oracle.dequantize_q4_k(raw)
    out = torch.empty(2048 * 256, dtype=torch.float32, device="cuda")
    ctx.dequantize_q4_k(dev(torch, raw), out, 2048)
    ctx.sync()
    assert out.cpu().numpy().tobytes() == ref.tobytes()
    # the reference's own block pattern (tests/test_neon_simd_gemv.rs:72-101) in the f16 layout
    k = golden("q4_k_kat.npz")
    blk = np.zeros(144, np.uint8)
    blk[0:2] = np.frombuffer(np.float16(k["dot_d"]).tobytes(), np.uint8)
    blk[2:4] = np.frombuffer(np.float16(k["dot_dmin"]).tobytes(), np.uint8)
    blk[4:16] = k["dot_scales"]
    blk[16:] = k["dot_qs"]
    out = torch.empty(256, dtype=torch.float32, device="cuda")
    ctx.dequantize_q4_k(dev(torch, blk), out, 1)
    ctx.sync()
    assert out.cpu().numpy().tobytes() == oracle.dequantize_q4_k(blk).tobytes()


def test_unpack_scales_q4_k_bit_exact(ctx, oracle, torch_cuda):
    torch = torch_cuda
    rng = np.random.Generator(np.random.PCG64(3))
    raw = rng.integers(0, 256, size=1000 * 144, dtype=np.uint8)
    out = torch.empty(1000 * 16, dtype=torch.uint8, device="cuda")
    ctx.unpack_scales_q4_k(dev(torch, raw), out, 1000)
    ctx.sync()
    assert np.array_equal(out.cpu().numpy().reshape(1000, 16), oracle.unpack_scales_q4_k(raw))


def test_quantize_row_q8_0_bit_exact(ctx, oracle, torch_cuda):
    torch = torch_cuda
    g = golden("q8_0_kat.npz")
    rng = np.random.Generator(np.random.PCG64(4))
    cases = [g["quant_x"], g["dot_x"], rng.standard_normal(4096).astype(np.float32),
             np.zeros(64, np.float32),
             # ties and the +/-128 edge of the clamp
             (np.arange(-64, 64).astype(np.float32) * 0.5).astype(np.float32),
             (rng.standard_normal(960) * 1e-30).astype(np.float32)]
    for x in cases:
        d_ref, q_ref = oracle.quantize_row_q8_0(x)
        d = torch.empty(x.size // 32, dtype=torch.float32, device="cuda")
        q = torch.empty(x.size, dtype=torch.int8, device="cuda")
        ctx.quantize_row_q8_0(dev(torch, x), d, q, x.size)
        ctx.sync()
        assert d.cpu().numpy().tobytes() == d_ref.tobytes()
        assert np.array_equal(q.cpu().numpy(), q_ref)


def test_block_isums_q8_0_bit_exact(ctx, oracle, torch_cuda):
    torch = torch_cuda
    rng = np.random.Generator(np.random.PCG64(5))
    for rows, cols in [(12, 512), (64, 960), (7, 32)]:
        raw = rng.integers(0, 256, size=rows * (cols // 32) * 34, dtype=np.uint8)
        xq = rng.integers(-128, 128, size=cols, dtype=np.int8)
        ref = oracle.block_isums_q8_0(raw, xq, rows, cols)
        out = torch.empty(rows * (cols // 32), dtype=torch.int32, device="cuda")
        ctx.block_isums_q8_0(dev(torch, raw), dev(torch, xq), out, rows, cols)
        ctx.sync()
        assert np.array_equal(out.cpu().numpy().reshape(rows, -1), ref)


def test_shape_errors(ctx, kb, torch_cuda):
    torch = torch_cuda
    buf = torch.zeros(1024, dtype=torch.float32, device="cuda")
    with pytest.raises(kb.KansoError) as e:
        ctx.quantize_row_q8_0(buf, buf, buf, 33)
    assert e.value.code == kb.ERR_SHAPE
    with pytest.raises(kb.KansoError) as e:
        ctx.gemv_q8_0(buf, buf, buf, 4, 48)
    assert e.value.code == kb.ERR_SHAPE
    with pytest.raises(kb.KansoError) as e:
        ctx.gemv_q4_k(buf, buf, buf, 4, 128)  # cols % 256 != 0
    assert e.value.code == kb.ERR_SHAPE
    with pytest.raises(kb.KansoError) as e:
        ctx.gemm_q4_k(buf, buf, buf, 2, 4, 256, kb.ACT_Q8)
    assert e.value.code == kb.ERR_UNSUPPORTED
