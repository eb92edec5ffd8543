"""dot_general on bf16 / f16 operands through the native 16-bit kernels (tensor-core tiles fed by TMA for M > 8,
the HBM-bound skinny kernels for M <= 8) against the oracle: exact products, fp32 accumulation, one rounding.
Layouts follow the reference's matmul cases (tests/configs/matmul.py:19-249 of the reference: transposed operands,
batch dimensions, several free dimensions) at sizes that reach every tile width, the K split, ragged edges, the
row repack of operands whose row stride is not a multiple of 16 bytes, and the result rows that start off a 16-byte
line."""
import numpy as np
import pytest

import b200
from b200.shlo.builder import Builder
from util import compare, run_gpu
from oracle import interp

pytestmark = pytest.mark.gpu


def _rand(shape, seed, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


# (lhs shape, rhs shape, contracting dims, batch dims, result dtype or None)
GEMM_CASES = [
    ((256, 128), (128, 192), ((1,), (0,)), ((), ()), None),               # A k-contiguous, B n-contiguous
    ((128, 256), (128, 192), ((0,), (0,)), ((), ()), None),               # A m-contiguous (a weight gradient)
    ((256, 128), (192, 128), ((1,), (1,)), ((), ()), None),               # B k-contiguous (an input gradient)
    ((128, 256), (192, 128), ((0,), (1,)), ((), ()), None),               # both transposed
    ((300, 200), (200, 100), ((1,), (0,)), ((), ()), None),               # ragged in m, n and k
    ((1024, 768), (768, 1536), ((1,), (0,)), ((), ()), None),             # 128-wide tiles
    ((2048, 512), (512, 2560), ((1,), (0,)), ((), ()), "f32"),            # f32 result, several tiles per CTA
    ((4096, 256), (256, 3072), ((1,), (0,)), ((), ()), None),             # 256-wide tiles, several per CTA
    ((3072, 256), (4096, 256), ((1,), (1,)), ((), ()), None),             # 256-wide tiles with B k-contiguous
    ((4096, 64), (4096, 96), ((0,), (0,)), ((), ()), None),               # deep K, few tiles: K split
    ((640, 136), (136, 250), ((1,), (0,)), ((), ()), None),               # N = 250: result rows start off 16-byte lines
    ((96, 250), (250, 136), ((1,), (0,)), ((), ()), None),                # K = 250 contiguous in A: row repack
    ((250, 96), (250, 136), ((0,), (0,)), ((), ()), None),                # K = 250 rows, both n-contiguous
    ((96, 40), (136, 40), ((1,), (1,)), ((), ()), "f32"),                 # K = 40 < one k-tile
    ((6, 128, 64), (6, 128, 64), ((2,), (2,)), ((0,), (0,)), None),       # batched q k^T
    ((6, 128, 128), (6, 128, 64), ((2,), (1,)), ((0,), (0,)), None),      # batched p v
    ((6, 128, 128), (6, 128, 64), ((1,), (1,)), ((0,), (0,)), None),      # batched p^T dv (A m-contiguous)
    ((2, 3, 72, 40), (2, 3, 40, 56), ((3,), (2,)), ((0, 1), (0, 1)), None),   # two batch dims
    ((3, 5, 16, 48), (48, 24), ((3,), (0,)), ((), ()), None),             # several free dims collapse to one
    ((12, 5, 8), (5, 8, 24), ((1, 2), (0, 1)), ((), ()), None),           # two contracting dims collapse to one
]


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("ls,rs,contract,batch,out", GEMM_CASES)
def test_dot_general_16bit(client, ls, rs, contract, batch, out, dtype):
    if dtype == "f16" and ls[0] > 1024:
        pytest.skip("large shapes are covered in bf16")
    b = Builder()
    x, y = b.arg(ls, dtype), b.arg(rs, dtype)
    z = b.dot_general(x, y, contract, batch, out_dtype=out)
    text = b.module([z])
    plan, _ = b200.compile_to_plan(text)
    assert "gemm16" in plan and "igemm" not in plan, plan
    args = [_rand(ls, 1), _rand(rs, 2)]
    got, _ = run_gpu(client, text, args, dtypes=[dtype, dtype])
    want = interp.run_text(text, args)
    # one rounding of an exactly accumulated sum: half a unit in the last place of the result type, plus fp32
    # accumulation error relative to the largest partial sums
    rtol = 2e-6 if out == "f32" else (4e-3 if dtype == "bf16" else 5e-4)
    compare(got[0], want[0], rtol=rtol, atol=2e-6 if out == "f32" else rtol, scale_atol=True)


SKINNY_CASES = [
    ((1, 2048), (2048, 640), ((1,), (0,)), ((), ()), None),               # n contiguous, K split over CTAs
    ((1, 256), (256, 4096), ((1,), (0,)), ((), ()), None),                # n contiguous, many panels
    ((1, 1000), (1000, 250), ((1,), (0,)), ((), ()), "f32"),              # ragged panel, unaligned rows
    ((8, 640), (640, 256), ((1,), (0,)), ((), ()), None),                 # eight rows (heads against a value cache)
    ((5, 333), (333, 77), ((1,), (0,)), ((), ()), None),                  # odd everything
    ((1, 512), (3000, 512), ((1,), (1,)), ((), ()), None),                # k contiguous (tied-embedding logits)
    ((1, 2048), (20000, 2048), ((1,), (1,)), ((), ()), "f32"),            # k contiguous, four columns per warp
    ((8, 256), (640, 256), ((1,), (1,)), ((), ()), None),                 # heads against a key cache
    ((3, 4, 64), (3, 64, 40), ((2,), (1,)), ((0,), (0,)), None),          # batched skinny
]


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("ls,rs,contract,batch,out", SKINNY_CASES)
def test_skinny_dot_general_16bit(client, ls, rs, contract, batch, out, dtype):
    b = Builder()
    x, y = b.arg(ls, dtype), b.arg(rs, dtype)
    text = b.module([b.dot_general(x, y, contract, batch, out_dtype=out)])
    plan, _ = b200.compile_to_plan(text)
    assert "gemv16" in plan and "igemm" not in plan, plan
    args = [_rand(ls, 3), _rand(rs, 4)]
    got, _ = run_gpu(client, text, args, dtypes=[dtype, dtype])
    want = interp.run_text(text, args)
    rtol = 2e-6 if out == "f32" else (4e-3 if dtype == "bf16" else 5e-4)
    compare(got[0], want[0], rtol=rtol, atol=2e-6 if out == "f32" else rtol, scale_atol=True)


def test_16bit_contractions_are_reproducible(client):
    """Bit equality from run to run for a product whose K splits meet at a counter (the last CTA adds the splits in a
    fixed order) and for a tensor-core product with a K split."""
    for ls, rs, contract in [((1, 4096), (4096, 512), ((1,), (0,))), ((4096, 128), (4096, 96), ((0,), (0,)))]:
        b = Builder()
        x, y = b.arg(ls, "bf16"), b.arg(rs, "bf16")
        exe = client.compile(b.module([b.dot_general(x, y, contract, out_dtype="f32")]))
        bufs = [client.buffer_from_host(_rand(ls, 5), dtype="bf16"), client.buffer_from_host(_rand(rs, 6), dtype="bf16")]
        ref = exe.execute(bufs)[0].to_numpy()
        for _ in range(8):
            np.testing.assert_array_equal(exe.execute(bufs)[0].to_numpy(), ref)


def test_f32_result_is_exact_to_fp32_accumulation(client):
    """bf16 products are exact in fp32, so an f32 result may differ from a float64 sum of the same products only by
    fp32 accumulation: far below plain-TF32 or bf16-rounded accumulation."""
    m, k, n = 384, 1024, 320
    a, w = _rand((m, k), 7), _rand((k, n), 8)
    b = Builder()
    x, y = b.arg((m, k), "bf16"), b.arg((k, n), "bf16")
    text = b.module([b.dot_general(x, y, ((1,), (0,)), out_dtype="f32")])
    got, _ = run_gpu(client, text, [a, w], dtypes=["bf16", "bf16"])
    import torch
    ab = torch.from_numpy(a).to(torch.bfloat16).to(torch.float64)
    wb = torch.from_numpy(w).to(torch.bfloat16).to(torch.float64)
    want = (ab @ wb).numpy()
    err = np.max(np.abs(got[0] - want)) / np.max(np.abs(want))
    assert err < 2e-6, err
