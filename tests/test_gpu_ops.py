"""Operation-level parity on the GPU: every case builds a StableHLO module,
runs it through the C ABI on the B200 and through the CPU oracle, and compares
(integers, booleans and indices bit-exact; fp32 at rtol = atol = 1e-5, the
reference's own bar in tests/test_ops.py:91-105). Case shapes follow the
reference's catalogue (tests/configs/{conv,matmul,slice,reduction,control_flow}.py)."""
import math

import numpy as np

import b200
import pytest

from b200.shlo.builder import Builder
from oracle import interp
from tests.util import check, compare, run_gpu

pytestmark = pytest.mark.gpu
rng = np.random.default_rng(42)


def f32(*shape, lo=-1.0, hi=1.0):
    return rng.uniform(lo, hi, shape).astype(np.float32)


# ---------------------------------------------------------------------------
# elementwise
# ---------------------------------------------------------------------------
UNARY_F = ["exp", "log", "sqrt", "rsqrt", "neg", "abs", "floor", "ceil", "sin", "cos", "tanh", "tan", "logistic",
           "sign", "log1p", "expm1", "cbrt", "round_even", "round_afz"]


@pytest.mark.parametrize("name", UNARY_F)
def test_unary_float(client, name):
    b = Builder()
    x = b.arg((33, 65), "f32")
    y = getattr(b, name)(x)
    pos = name in ("log", "sqrt", "rsqrt", "log1p")
    a = f32(33, 65, lo=0.05 if pos else -4.0, hi=4.0)
    if name in ("round_even", "round_afz"):
        a = np.concatenate([a.reshape(-1)[:-8], np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 3.5, -3.5], np.float32)]).reshape(33, 65)
    check(client, b.module([y]), [a], rtol=2e-5, atol=1e-5)


CHLO_UNARY = {"sinh": (-4, 4), "cosh": (-4, 4), "asin": (-1, 1), "acos": (-1, 1), "atan": (-8, 8), "asinh": (-8, 8), "acosh": (1, 8),
              "atanh": (-0.99, 0.99), "erf": (-3, 3), "erf_inv": (-0.999, 0.999), "tan": (-1.4, 1.4)}


@pytest.mark.parametrize("form", ["op", "custom_call"])
@pytest.mark.parametrize("name", sorted(CHLO_UNARY))
def test_chlo_unary(client, name, form):
    """The functions jax emits as chlo operations, as custom calls to @mhlo.<name> or as composites
    (src/pjrt_plugin/ops/control_flow.cc:53-66 of the reference lists them)."""
    lo, hi = CHLO_UNARY[name]
    b = Builder()
    x = b.arg((17, 33), "f32")
    check(client, b.module([b.chlo_unary(name, x, form)]), [f32(17, 33, lo=lo, hi=hi)], rtol=3e-5, atol=1e-5)


def test_chlo_composite_runs_as_the_named_operation(client):
    """A composite named after a chlo function is that function, whatever its decomposition says (here: a wrong one),
    as in the reference (src/pjrt_plugin/ops/control_flow.cc:2206-2222)."""
    text = """
module @test {
  func.func private @chlo.asin.impl(%arg0: tensor<4xf32>) -> tensor<4xf32> {
    %0 = stablehlo.negate %arg0 : tensor<4xf32>
    return %0 : tensor<4xf32>
  }
  func.func @main(%arg0: tensor<4xf32>) -> tensor<4xf32> {
    %0 = stablehlo.composite "chlo.asin" %arg0 {decomposition = @chlo.asin.impl} : (tensor<4xf32>) -> tensor<4xf32>
    return %0 : tensor<4xf32>
  }
}
"""
    x = np.array([0.0, 0.5, -0.5, 0.9], np.float32)
    got, _ = run_gpu(client, text, [x])
    np.testing.assert_allclose(got[0], np.arcsin(x), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("name", ["add", "sub", "mul", "div", "max", "min", "pow", "rem", "atan2"])
def test_binary_float(client, name):
    b = Builder()
    x, y = b.arg((7, 129), "f32"), b.arg((7, 129), "f32")
    z = getattr(b, name)(x, y)
    a0 = f32(7, 129, lo=0.1 if name == "pow" else -3, hi=3)
    a1 = f32(7, 129, lo=-3, hi=3)
    a1[np.abs(a1) < 0.05] = 0.5
    check(client, b.module([z]), [a0, a1], rtol=2e-5, atol=1e-5)


def test_float_specials(client):
    """NaN propagation of maximum/minimum/sign, is_finite, total-order compare."""
    b = Builder()
    x, y = b.arg((8,), "f32"), b.arg((8,), "f32")
    outs = [b.max(x, y), b.min(x, y), b.sign(x), b.is_finite(x), b.compare(x, y, "LT", "TOTALORDER"),
            b.compare(x, y, "EQ"), b.compare(x, y, "NE")]
    a0 = np.array([np.nan, 1.0, -0.0, 0.0, np.inf, -np.inf, 2.0, -np.nan], np.float32)
    a1 = np.array([1.0, np.nan, 0.0, -0.0, np.inf, 1.0, 2.0, np.nan], np.float32)
    check(client, b.module(outs), [a0, a1])


@pytest.mark.parametrize("dt", ["i32", "ui32", "i8", "i64", "ui8", "i16"])
def test_integer_arithmetic(client, dt):
    """Truncating division, remainder with the dividend's sign, division by
    zero, INT_MIN / -1, shifts by out-of-range amounts, popcnt, clz."""
    from b200.shlo.builder import _NP
    npdt = _NP[dt]
    info = np.iinfo(npdt)
    b = Builder()
    x, y = b.arg((64,), dt), b.arg((64,), dt)
    outs = [b.add(x, y), b.sub(x, y), b.mul(x, y), b.div(x, y), b.rem(x, y), b.max(x, y), b.min(x, y), b.and_(x, y),
            b.or_(x, y), b.xor(x, y), b.shl(x, y), b.shr_logical(x, y), b.shr_arith(x, y), b.not_(x), b.popcnt(x),
            b.clz(x), b.neg(x), b.abs(x), b.sign(x), b.compare(x, y, "LT"), b.compare(x, y, "GE")]
    a0 = rng.integers(info.min, info.max, 64, dtype=npdt, endpoint=True)
    a1 = rng.integers(max(info.min, -9), 9, 64).astype(npdt)
    a0[:4] = [info.min, info.max, 0, 7]
    a1[:4] = [-1 if info.min < 0 else 1, 0, 0, info.max]
    a1[4:8] = [info.max, 31, 33, 8]     # shift amounts beyond the width
    check(client, b.module(outs), [a0, a1])


def test_integer_power(client):
    b = Builder()
    x, y = b.arg((16,), "i32"), b.arg((16,), "i32")
    a0 = np.array([2, 3, -2, 1, -1, -1, 0, 5, 7, 2, 2, 10, -3, 4, 6, 9], np.int32)
    a1 = np.array([10, 5, 3, -4, -3, -2, 0, 0, 2, 31, 30, 9, 3, -1, 1, 2], np.int32)
    check(client, b.module([b.pow(x, y)]), [a0, a1])


def test_select_clamp_convert(client):
    b = Builder()
    p, x, y = b.arg((5, 9), "i1"), b.arg((5, 9), "f32"), b.arg((5, 9), "f32")
    lo, hi = b.arg((), "f32"), b.arg((), "f32")
    outs = [b.select(p, x, y), b.clamp(lo, x, hi), b.convert(x, "i32"), b.convert(x, "ui8"), b.convert(x, "i1"),
            b.convert(b.convert(x, "i32"), "f32"), b.convert(p, "f32"), b.convert(x, "bf16"), b.convert(x, "f16"),
            b.convert(b.convert(x, "bf16"), "f32"), b.convert(x, "i64"), b.convert(b.convert(x, "i8"), "i32")]
    a = f32(5, 9, lo=-300, hi=300)
    a[0, :4] = [np.nan, np.inf, -np.inf, 3e9]
    check(client, b.module(outs), [rng.integers(0, 2, (5, 9)).astype(bool), a, f32(5, 9), np.float32(-10), np.float32(99.5)])


def test_bitcast_and_threefry_style_bits(client):
    """u32 shift/or/xor chains and bitcast to float, the building blocks of
    the threefry generator the reference runs bit-exactly (tests/configs/random.py:54-74)."""
    b = Builder()
    k = b.arg((256,), "ui32")
    x = b.add(k, b.full((256,), 0x9E3779B9, "ui32"))
    rot = b.or_(b.shl(x, b.full((256,), 13, "ui32")), b.shr_logical(x, b.full((256,), 19, "ui32")))
    y = b.xor(rot, k)
    mant = b.or_(b.shr_logical(y, b.full((256,), 9, "ui32")), b.full((256,), 0x3F800000, "ui32"))
    f = b.sub(b.bitcast_convert(mant, "f32"), b.full((256,), 1.0, "f32"))
    check(client, b.module([y, f, b.bitcast_convert(f, "i32")]), [rng.integers(0, 2**32, 256, dtype=np.uint32)], rtol=0, atol=0)


def test_bf16_elementwise(client):
    b = Builder()
    x, y = b.arg((40, 64), "bf16"), b.arg((40, 64), "bf16")
    z = b.add(b.mul(x, y), b.tanh(x))
    s = b.convert(b.reduce_sum(b.convert(z, "f32"), (1,)), "bf16")
    a0, a1 = f32(40, 64), f32(40, 64)
    check(client, b.module([z, s]), [a0, a1], rtol=2e-2, atol=1e-2, dtypes=["bf16", "bf16"])


# ---------------------------------------------------------------------------
# data movement
# ---------------------------------------------------------------------------
def test_broadcast_iota_reshape_transpose(client):
    b = Builder()
    x, v = b.arg((4, 5, 6), "f32"), b.arg((5,), "f32")
    t = b.transpose(x, (2, 0, 1))
    outs = [b.add(x, b.broadcast_in_dim(v, (4, 5, 6), (1,))), t, b.reshape(t, (6, 20)), b.reshape(x, (20, 6)),
            b.iota((3, 7), "i32", 1), b.iota((3, 7), "f32", 0), b.reverse(x, (0, 2)),
            b.add(b.reshape(b.transpose(x, (1, 0, 2)), (5, 24)), b.full((5, 24), 1.0, "f32")),
            b.broadcast_in_dim(b.reshape(v, (5, 1)), (2, 5, 3), (1, 2))]
    check(client, b.module(outs), [f32(4, 5, 6), f32(5)])


def test_big_transpose(client):
    b = Builder()
    x = b.arg((96, 200, 33), "f32")
    check(client, b.module([b.transpose(x, (2, 1, 0)), b.transpose(x, (1, 0, 2))]), [f32(96, 200, 33)])


@pytest.mark.parametrize("shape,perm,dt", [
    ((1000, 520), (1, 0), "f32"), ((1000, 520), (1, 0), "bf16"), ((514, 300), (1, 0), "i32"),
    ((6, 200, 136), (0, 2, 1), "f32"), ((6, 200, 136), (0, 2, 1), "bf16"),
    ((4, 16, 64, 40), (0, 1, 3, 2), "f32"),           # two batch dimensions
    ((40, 8, 512), (2, 0, 1), "bf16"),                # [X0, X1, Y] -> [Y, X0, X1]
    ((512, 40, 8), (1, 2, 0), "f32"),                 # [X, Y0, Y1] -> [Y0, Y1, X]
])
def test_tiled_transpose(client, shape, perm, dt):
    """Large transposes that move the innermost dimension go through the shared-memory tile kernel (plan step
    `transpose`); values must be the input's, bit for bit."""
    b = Builder()
    x = b.arg(shape, dt)
    text = b.module([b.transpose(x, perm)])
    plan, _ = b200.compile_to_plan(text)
    assert "transpose batch=" in plan and "kernel " not in plan, plan
    a = (np.random.default_rng(5).standard_normal(shape) * 100).astype(np.float32)
    if dt == "i32":
        a = a.astype(np.int32)
    got, _ = run_gpu(client, text, [a], dtypes=[dt])
    want = interp.run_text(text, [a])
    np.testing.assert_array_equal(got[0], want[0])


def test_transposes_concatenated_along_rows(client):
    """concatenate(transpose(a), transpose(b)) along dimension 0 (the form the weights of a decode loop take): each
    part is one tiled transpose into its rows of the result."""
    b = Builder()
    x, y = b.arg((256, 384), "bf16"), b.arg((256, 130), "bf16")
    text = b.module([b.concatenate([b.transpose(x, (1, 0)), b.transpose(y, (1, 0))], 0)])
    plan, _ = b200.compile_to_plan(text)
    assert plan.count("transpose batch=") == 2 and "kernel " not in plan, plan
    a0, a1 = f32(256, 384), f32(256, 130)
    got, _ = run_gpu(client, text, [a0, a1], dtypes=["bf16", "bf16"])
    want = interp.run_text(text, [a0, a1])
    np.testing.assert_array_equal(got[0], want[0])


def test_collectives_on_one_partition_are_identities(client):
    """all_reduce, all_gather and partition_id with one partition (src/pjrt_plugin/ops/collectives.cc:41-78)."""
    b = Builder()
    x = b.arg((7, 3), "f32")
    outs = [b.all_gather(x, 1, 1), b.all_reduce_sum([x], 1)[0], b.convert(b.partition_id(), "i32")]
    got, _ = run_gpu(client, b.module(outs), [f32(7, 3)])
    want = interp.run_text(b.module(outs), [f32(7, 3)])
    a = f32(7, 3)
    got, _ = run_gpu(client, b.module(outs), [a])
    np.testing.assert_array_equal(got[0], a)
    np.testing.assert_array_equal(got[1], a)
    assert int(got[2]) == 0


def test_slice_pad_concat(client):
    """Negative and interior padding (src/pjrt_plugin/ops/slice.cc:202-276)."""
    b = Builder()
    x, y = b.arg((6, 10), "f32"), b.arg((3, 10), "f32")
    z = b.const(-7.0, "f32")
    outs = [b.slice(x, (1, 2), (5, 9), (2, 3)), b.pad(x, z, (1, 2), (0, 3), (0, 0)), b.pad(x, z, (-1, 0), (2, -3), (0, 0)),
            b.pad(x, z, (0, 1), (0, 0), (2, 1)), b.pad(x, z, (-2, -1), (1, -2), (1, 2)),
            b.concatenate([x, y, x], 0), b.concatenate([b.slice(x, (0, 0), (6, 4)), b.mul(x, x)], 1)]
    check(client, b.module(outs), [f32(6, 10), f32(3, 10)])


def test_dynamic_slice_update_clamp(client):
    """Start indices are clamped into range (src/pjrt_plugin/ops/slice.cc:80-107)."""
    b = Builder()
    x, u = b.arg((8, 12), "f32"), b.arg((3, 4), "f32")
    i, j = b.arg((), "i32"), b.arg((), "i32")
    outs = [b.dynamic_slice(x, [i, j], (3, 4)), b.dynamic_update_slice(x, u, [i, j])]
    text = b.module(outs)
    for ii, jj in [(0, 0), (2, 5), (7, 11), (-3, 100), (6, -1)]:
        check(client, text, [f32(8, 12), f32(3, 4), np.int32(ii), np.int32(jj)])


def test_gather_rows_and_take_along(client):
    """Embedding lookup and take_along_axis forms, with out-of-range indices
    clamped (src/pjrt_plugin/ops/gather_scatter.cc:233-239)."""
    b = Builder()
    tab, idx = b.arg((50, 16), "f32"), b.arg((4, 7), "i32")
    x, lab = b.arg((9, 11), "f32"), b.arg((9,), "i32")
    outs = [b.take_rows(tab, idx), b.take_along_last(x, lab)]
    ids = rng.integers(0, 50, (4, 7)).astype(np.int32)
    ids[0, :3] = [-5, 49, 77]
    check(client, b.module(outs), [f32(50, 16), ids, f32(9, 11), rng.integers(0, 11, 9).astype(np.int32)])


# ---------------------------------------------------------------------------
# reductions
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("shape,dims", [((128, 10), (1,)), ((64, 8, 8, 32), (0, 1, 2)), ((16, 6, 6, 48), (1, 2)),
                                        ((3, 5000), (1,)), ((70000,), (0,)), ((33, 17, 9), (0, 2)), ((4, 7), (0, 1)),
                                        ((2, 300000), (1,)), ((5, 1, 3), (1,))])
def test_reduce_sum_max(client, shape, dims):
    b = Builder()
    x = b.arg(shape, "f32")
    outs = [b.reduce_sum(x, dims), b.reduce_max(x, dims), b.reduce_sum(b.mul(x, x), dims)]
    check(client, b.module(outs), [f32(*shape)], rtol=2e-5, atol=2e-5)


def test_reduce_other_bodies(client):
    b = Builder()
    x, p, n = b.arg((9, 40), "f32"), b.arg((9, 40), "i1"), b.arg((9, 40), "i32")
    one, t, f_, big = b.const(1.0, "f32"), b.const(True, "i1"), b.const(False, "i1"), b.const(2**31 - 1, "i32")
    outs = [b.reduce([x], [one], (1,), lambda s, a, c: s.mul(a, c))[0],
            b.reduce([x], [b.const(math.inf, "f32")], (0,), lambda s, a, c: s.min(a, c))[0],
            b.reduce([p], [t], (1,), lambda s, a, c: s.and_(a, c))[0],
            b.reduce([p], [f_], (0,), lambda s, a, c: s.or_(a, c))[0],
            b.reduce([n], [big], (1,), lambda s, a, c: s.min(a, c))[0],
            b.reduce([n], [b.const(0, "i32")], (0, 1), lambda s, a, c: s.add(a, c))[0]]
    check(client, b.module(outs), [f32(9, 40, lo=0.8, hi=1.2), rng.integers(0, 2, (9, 40)).astype(bool),
                                   rng.integers(-1000, 1000, (9, 40)).astype(np.int32)], rtol=2e-5)


@pytest.mark.parametrize("shape,dim", [((6, 1000), 1), ((1, 256000), 1), ((50, 7), 0)])
def test_argmax_first_index_on_ties(client, shape, dim):
    b = Builder()
    x = b.arg(shape, "f32")
    a = np.round(f32(*shape) * 4) / 4          # many ties
    got, _ = check(client, b.module([b.argmax(x, dim)]), [a])
    np.testing.assert_array_equal(got[0], np.argmax(a, axis=dim).astype(np.int32))


# ---------------------------------------------------------------------------
# dot_general (case shapes: tests/configs/matmul.py of the reference)
# ---------------------------------------------------------------------------
DOT_CASES = [
    ((32, 64), (64, 48), ((1,), (0,)), ((), ())),
    ((64, 32), (64, 48), ((0,), (0,)), ((), ())),            # lhs transposed
    ((32, 64), (48, 64), ((1,), (1,)), ((), ())),            # rhs transposed
    ((4, 16, 32), (4, 32, 24), ((2,), (1,)), ((0,), (0,))),  # batch
    ((4, 16, 32), (4, 24, 32), ((2,), (2,)), ((0,), (0,))),
    ((3, 5, 7, 11), (11, 13), ((3,), (0,)), ((), ())),       # several free dims
    ((6, 5, 8), (5, 8, 9), ((1, 2), (0, 1)), ((), ())),      # two contracting dims
    ((17,), (17,), ((0,), (0,)), ((), ())),                  # vector . vector
    ((128, 512), (512, 10), ((1,), (0,)), ((), ())),
    ((10, 300), (10, 7), ((0,), (0,)), ((), ())),
    ((2, 3, 40, 8), (2, 3, 8, 40), ((3,), (2,)), ((0, 1), (0, 1))),
    ((1, 2048), (2048, 300), ((1,), (0,)), ((), ())),        # GEMV shape
    ((200, 3000), (3000, 70), ((1,), (0,)), ((), ())),       # deep K (split-K path)
]


def test_strided_convolution_input_gradient_with_skipped_k_tiles(client):
    """Input gradient of stride-2 convolutions with 32-aligned channels: an input-dilated convolution whose rows
    are visited phase by phase and whose dead k-tiles (window positions that only meet dilation holes) are
    skipped; 3x3 and 1x1 kernels, odd and even extents."""
    for (n, h, w, ci, co, k, pad) in [(4, 16, 16, 64, 64, 3, 1), (2, 15, 13, 32, 96, 3, 1), (8, 8, 8, 64, 128, 1, 0),
                                      (96, 16, 16, 64, 64, 3, 1)]:
        b = Builder()
        x, wt = b.arg((n, h, w, ci), "f32"), b.arg((k, k, ci, co), "f32")
        y = b.conv(x, wt, strides=(2, 2), padding=((pad, pad), (pad, pad)))
        g = b.arg(y.shape, "f32")
        dx, dw = b.grad(b.reduce_sum(b.mul(y, g), (0, 1, 2, 3)), [x, wt])
        check(client, b.module([dx, dw]), [f32(n, h, w, ci), f32(k, k, ci, co), f32(*y.shape)],
              rtol=1e-5, atol=1e-5, scale_atol=True)


@pytest.mark.parametrize("n,h,w,ci,co,k,pad,rdil", [
    (4, 32, 32, 64, 64, 3, 1, 1),        # four output rows per tile
    (6, 16, 16, 32, 96, 3, 1, 1),        # eight rows per tile
    (3, 8, 8, 64, 128, 3, 1, 1),         # two images per tile, a ragged last tile (192 rows)
    (20, 4, 4, 96, 64, 3, 1, 1),         # eight images per tile
    (5, 16, 16, 64, 32, 1, 0, 1),        # 1 x 1
    (2, 16, 16, 32, 64, 5, 2, 1),        # 5 x 5
    (2, 16, 16, 32, 64, 3, 2, 2),        # kernel dilation 2, same size
    (4, 18, 18, 32, 64, 3, 0, 1),        # no padding: 16 x 16 outputs from an 18 x 18 input (its input gradient has 18-pixel rows: gathered)
])
def test_stride_one_convolution_with_tma_fed_operand(client, n, h, w, ci, co, k, pad, rdil):
    """Stride-1 convolutions over NHWC inputs with a multiple of 32 channels whose 128-row tiles are whole output rows:
    the A operand arrives by TMA boxes (plan tag `tmaA`), forward and input gradient, against the oracle."""
    b = Builder()
    x, wt = b.arg((n, h, w, ci), "f32"), b.arg((k, k, ci, co), "f32")
    y = b.conv(x, wt, padding=((pad, pad), (pad, pad)), rhs_dilation=(rdil, rdil))
    g = b.arg(y.shape, "f32")
    dx, dw = b.grad(b.reduce_sum(b.mul(y, g), (0, 1, 2, 3)), [x, wt])
    text = b.module([y, dx, dw])
    plan, _ = b200.compile_to_plan(text)
    assert plan.count("tmaA") == (1 if pad == 0 and k > 1 else 2), plan
    check(client, text, [f32(n, h, w, ci), f32(k, k, ci, co), f32(*y.shape)], rtol=1e-5, atol=1e-5, scale_atol=True)


@pytest.mark.parametrize("ci", [1, 3, 5, 7])
def test_small_channel_convolution_and_gradients(client, ci):
    """Convolutions whose input has a few channels (not a multiple of 4): forward, input gradient and weight
    gradient; the compiler pads the channels with zeros to reach the 16-byte gather paths."""
    b = Builder()
    x, wt = b.arg((6, 10, 9, ci), "f32"), b.arg((3, 3, ci, 24), "f32")
    y = b.conv(x, wt, padding=((1, 1), (1, 1)))
    g = b.arg(y.shape, "f32")
    dx, dw = b.grad(b.reduce_sum(b.mul(y, g), (0, 1, 2, 3)), [x, wt])
    check(client, b.module([y, dx, dw]), [f32(6, 10, 9, ci), f32(3, 3, ci, 24), f32(*y.shape)], rtol=1e-5, atol=1e-5, scale_atol=True)


def test_contraction_results_are_reproducible(client):
    """Run-to-run bit equality on a split-K convolution with many k-tiles per CTA (the shape on which reading the
    accumulator before the last MMAs had retired once showed up as sporadic errors in single output tiles)."""
    b = Builder()
    x, w = b.arg((128, 4, 4, 512), "f32"), b.arg((3, 3, 512, 512), "f32")
    exe = client.compile(b.module([b.conv(x, w, padding=((1, 1), (1, 1)))]))
    bufs = [client.buffer_from_host(f32(128, 4, 4, 512)), client.buffer_from_host(f32(3, 3, 512, 512))]
    ref = exe.execute(bufs)[0].to_numpy()
    for _ in range(12):
        np.testing.assert_array_equal(exe.execute(bufs)[0].to_numpy(), ref)


def test_bf16_contractions(client):
    """bf16 dot_general and convolution: bf16 products accumulated in fp32 and rounded once (what a CPU backend
    computes); compared at bf16 resolution."""
    b = Builder()
    x, w = b.arg((96, 160), "bf16"), b.arg((160, 72), "bf16")
    img, ker = b.arg((4, 12, 12, 32), "bf16"), b.arg((3, 3, 32, 48), "bf16")
    outs = [b.matmul(x, w), b.dot_general(x, w, ((1,), (0,)), out_dtype="f32"), b.conv(img, ker, padding=((1, 1), (1, 1)))]
    check(client, b.module(outs), [f32(96, 160), f32(160, 72), f32(4, 12, 12, 32), f32(3, 3, 32, 48)],
          rtol=1e-2, atol=1e-2, scale_atol=True, dtypes=["bf16"] * 4)


@pytest.mark.parametrize("ls,rs,contract,batch", DOT_CASES)
def test_dot_general(client, ls, rs, contract, batch):
    b = Builder()
    x, y = b.arg(ls, "f32"), b.arg(rs, "f32")
    z = b.dot_general(x, y, contract, batch)
    # atol scales with the largest output: a sum of K products carries absolute error ~ eps * sqrt(K) * |terms|
    check(client, b.module([z]), [f32(*ls), f32(*rs)], rtol=1e-5, atol=1e-5, scale_atol=True)


# ---------------------------------------------------------------------------
# convolution (case shapes: tests/configs/conv.py:9-224 of the reference)
# ---------------------------------------------------------------------------
def _same(size, k, s, d=1):
    kd = (k - 1) * d + 1
    out = -(-size // s)
    tot = max((out - 1) * s + kd - size, 0)
    return (tot // 2, tot - tot // 2)


CONV_CASES = {
    "nhwc-same": dict(x=(2, 8, 8, 3), w=(3, 3, 3, 8), pad="SAME"),
    "nchw-oihw-same": dict(x=(1, 3, 8, 8), w=(16, 3, 3, 3), pad="SAME", dn=("bf01", "oi01", "bf01")),
    "1d-nwc-stride2": dict(x=(2, 16, 3), w=(3, 3, 4), stride=(2,), pad="SAME", dn=("b0f", "0io", "b0f")),
    "stride2-same": dict(x=(2, 8, 8, 3), w=(3, 3, 3, 8), stride=(2, 2), pad="SAME"),
    "stride2-asymmetric": dict(x=(2, 8, 8, 3), w=(3, 3, 3, 8), stride=(2, 2), pad=((1, 0), (1, 0))),
    "5x5-stride2": dict(x=(2, 16, 16, 3), w=(5, 5, 3, 8), stride=(2, 2), pad="SAME"),
    "stride2-dilated": dict(x=(2, 16, 16, 3), w=(3, 3, 3, 8), stride=(2, 2), pad="SAME", rdil=(2, 2)),
    "stride2-valid": dict(x=(2, 16, 16, 3), w=(3, 3, 3, 8), stride=(2, 2), pad=((0, 0), (0, 0))),
    "1d-stride2-dilated": dict(x=(2, 32, 3), w=(3, 3, 4), stride=(2,), pad="SAME", rdil=(2,), dn=("b0f", "0io", "b0f")),
    "lhs_dilation-neg_padding": dict(x=(1, 6, 7, 4), w=(1, 2, 4, 2), pad=((0, -1), (0, 0)), ldil=(2, 1)),
    "lhs_dilation-only": dict(x=(1, 6, 7, 4), w=(1, 2, 4, 2), pad=((0, 0), (0, 0)), ldil=(2, 1)),
    "large-kernel": dict(x=(1, 4, 4, 3), w=(8, 8, 3, 16), pad="SAME"),
    "batch_group_2": dict(x=(4, 1, 6, 7), w=(2, 1, 1, 2), pad=((0, 0), (0, 0)), dn=("bf01", "oi01", "bf01"), bg=2),
    "batch_group_2-lhs_dil-neg_pad": dict(x=(2, 6, 7, 4), w=(1, 2, 4, 2), pad=((0, -1), (0, 0)), ldil=(2, 1), bg=2),
    "batch_group_3-multi_filter": dict(x=(6, 5, 5, 2), w=(3, 3, 2, 6), pad=((1, 1), (1, 1)), bg=3),
    "feature_group_4": dict(x=(2, 9, 9, 8), w=(3, 3, 2, 12), pad="SAME", fg=4),
    "resnet-stage1": dict(x=(8, 32, 32, 64), w=(3, 3, 64, 64), pad="SAME"),
    "resnet-proj-1x1-stride2": dict(x=(8, 32, 32, 64), w=(1, 1, 64, 128), stride=(2, 2), pad="SAME"),
    "small-map-stride2": dict(x=(16, 4, 4, 64), w=(3, 3, 64, 128), stride=(2, 2), pad="SAME"),
    "small-map-proj-stride2": dict(x=(16, 4, 4, 64), w=(1, 1, 64, 128), stride=(2, 2), pad="SAME"),
    "narrow-stride2": dict(x=(32, 16, 16, 16), w=(3, 3, 16, 32), stride=(2, 2), pad="SAME"),
    "narrow-proj-stride2": dict(x=(32, 16, 16, 16), w=(1, 1, 16, 32), stride=(2, 2), pad="SAME"),
    "tiny-map-3x3": dict(x=(16, 2, 2, 128), w=(3, 3, 128, 128), pad="SAME"),
}


def _build_conv(case, grads=False):
    dn = case.get("dn", ("b01f", "01io", "b01f"))
    nsp = len(dn[0]) - 2
    stride = case.get("stride", (1,) * nsp)
    rdil = case.get("rdil", (1,) * nsp)
    ldil = case.get("ldil", (1,) * nsp)
    b = Builder()
    x, w = b.arg(case["x"], "f32"), b.arg(case["w"], "f32")
    pad = case["pad"]
    if pad == "SAME":
        pad = [_same(case["x"][dn[0].index(str(s))], case["w"][dn[1].index(str(s))], stride[s], rdil[s]) for s in range(nsp)]
    y = b.conv(x, w, strides=stride, padding=pad, lhs_dilation=ldil, rhs_dilation=rdil, dn=dn,
               feature_group_count=case.get("fg", 1), batch_group_count=case.get("bg", 1))
    outs = [y]
    if grads:
        loss = b.reduce_sum(b.mul(y, y), tuple(range(y.ndim)))
        outs += b.grad(loss, [x, w])
    return b.module(outs)


@pytest.mark.parametrize("name", list(CONV_CASES))
def test_convolution(client, name):
    case = CONV_CASES[name]
    check(client, _build_conv(case), [f32(*case["x"]), f32(*case["w"])], rtol=1e-5, atol=1e-5, scale_atol=True)


@pytest.mark.parametrize("name", ["nhwc-same", "stride2-same", "stride2-asymmetric", "5x5-stride2", "stride2-dilated",
                                  "resnet-stage1", "resnet-proj-1x1-stride2", "small-map-stride2",
                                  "small-map-proj-stride2", "narrow-stride2", "narrow-proj-stride2", "tiny-map-3x3"])
def test_convolution_gradients(client, name):
    """Input and kernel gradients as jax emits them: convolutions with
    lhs_dilation / rhs_dilation, negative padding and permuted dimension numbers."""
    case = CONV_CASES[name]
    check(client, _build_conv(case, grads=True), [f32(*case["x"]), f32(*case["w"])], rtol=1e-4, atol=1e-5, wide=True,
          scale_atol=True)


# ---------------------------------------------------------------------------
# control flow
# ---------------------------------------------------------------------------
def test_counted_while(client):
    """fori_loop of 130 iterations (tests/configs/control_flow.py:426-435 of the reference)."""
    b = Builder()
    x = b.arg((16,), "f32")
    def cond(s, i, v): return s.compare(i, s.const(130, "i32"), "LT")
    def body(s, i, v): return [s.add(i, s.const(1, "i32")), s.add(s.mul(v, s.full((16,), 0.99, "f32")), s.full((16,), 0.01, "f32"))]
    i0 = b.const(0, "i32")
    outs = b.while_([i0, x], cond, body)
    got, exe = check(client, b.module(outs), [f32(16)], rtol=1e-4)
    assert int(got[0]) == 130


def test_dynamic_while_and_zero_trip(client):
    """Data-dependent trip count; zero iterations returns the inputs."""
    b = Builder()
    x, lim = b.arg((), "f32"), b.arg((), "f32")
    def cond(s, v, l): return s.compare(v, l, "LT")
    def body(s, v, l): return [s.mul(v, s.const(2.0, "f32")), l]
    text = b.module(b.while_([x, lim], cond, body))
    for start, limit in [(1.0, 100.0), (5.0, 1.0), (3.0, 3.0)]:
        check(client, text, [np.float32(start), np.float32(limit)])


def test_data_dependent_loop_and_case_run_on_the_device(client):
    """A `while` with a data-dependent trip count and a `case` run as conditional CUDA-graph nodes from their second
    execution on: the host reads no predicate back (the client's counter of stream synchronisations inside executions
    stands still), trip counts and branches still follow the data (zero trips, out-of-range index -> last branch)."""
    b = Builder()
    x, lim = b.arg((64,), "f32"), b.arg((), "f32")
    def cond(s, v, l): return s.compare(s.reduce_max(v, (0,)), l, "LT")
    def body(s, v, l): return [s.add(s.mul(v, s.full((64,), 1.5, "f32")), s.full((64,), 0.25, "f32")), l]
    text = b.module(b.while_([x, lim], cond, body))
    exe = client.compile(text)
    v0 = np.linspace(0.1, 1.0, 64).astype(np.float32)
    settled = None
    for limit in [50.0, 400.0, 0.5, 3.0, 1e4]:                      # 0.5: zero trips
        args = [v0, np.float32(limit)]
        before = client.host_syncs()
        got = [o.to_numpy() for o in exe.execute([client.buffer_from_host(a) for a in args])]
        want = interp.run_text(text, args)
        np.testing.assert_allclose(got[0], want[0], rtol=1e-5)
        if settled is not None:
            assert client.host_syncs() == before, "a recorded loop must not read its predicate back"
        if limit == 50.0:
            assert client.host_syncs() > before                     # the first execution goes through the host
            settled = True
    b = Builder()
    i, u = b.arg((), "i32"), b.arg((6, 5), "f32")
    idx = b.max(i, b.const(-7, "i32"))                              # computed on the device: the index lives in the arena
    outs = b.case(idx, [lambda s: [s.add(u, u)], lambda s: [s.mul(u, u)], lambda s: [s.tanh(u)]], [((6, 5), "f32")])
    text = b.module([b.exp(outs[0])])
    exe = client.compile(text)
    ub = f32(6, 5)
    for n, sel in enumerate([1, 0, 2, 9, -3, 1]):
        before = client.host_syncs()
        got = exe.execute([client.buffer_from_host(np.int32(sel)), client.buffer_from_host(ub)])[0].to_numpy()
        want = interp.run_text(text, [np.int32(sel), ub])[0]
        np.testing.assert_allclose(got, want, rtol=1e-5)
        if n > 0:
            assert client.host_syncs() == before, "a recorded case must not read its index back"


def test_scan_with_dynamic_slices(client):
    """A scan body: read xs[t] with dynamic_slice, update a carry, write ys[t]
    with dynamic_update_slice (the shape of lax.scan lowerings)."""
    T, N = 12, 8
    b = Builder()
    xs, h0 = b.arg((T, N), "f32"), b.arg((N,), "f32")
    ys0 = b.full((T, N), 0.0, "f32")
    def cond(s, t, h, ys): return s.compare(t, s.const(T, "i32"), "LT")
    def body(s, t, h, ys):
        z = s.const(0, "i32")
        xt = s.reshape(s.dynamic_slice(xs, [t, z], (1, N)), (N,))
        h2 = s.tanh(s.add(s.mul(h, s.full((N,), 0.5, "f32")), xt))
        ys2 = s.dynamic_update_slice(ys, s.reshape(h2, (1, N)), [t, z])
        return [s.add(t, s.const(1, "i32")), h2, ys2]
    outs = b.while_([b.const(0, "i32"), h0, ys0], cond, body)
    _, exe = check(client, b.module(outs), [f32(T, N), f32(N)], rtol=2e-5)
    assert ".window" in exe.plan_text()      # ys is updated in place, one window per iteration


def test_in_place_window_update_clamps(client):
    """A loop-carried tensor updated in place through a two-row window whose start runs from below zero to past
    the end: the start is clamped like the general dynamic_update_slice (src/pjrt_plugin/ops/slice.cc:80-107)."""
    T, N = 9, 40
    b = Builder()
    ys0, u0 = b.arg((T, N), "f32"), b.arg((2, N), "f32")
    def cond(s, t, u, ys): return s.compare(t, s.const(8, "i32"), "LT")
    def body(s, t, u, ys):
        start = s.sub(s.mul(t, s.const(2, "i32")), s.const(3, "i32"))
        u2 = s.add(u, s.full((2, N), 1.0, "f32"))
        ys2 = s.dynamic_update_slice(ys, s.mul(u, s.full((2, N), 0.5, "f32")), [start, s.const(0, "i32")])
        return [s.add(t, s.const(1, "i32")), u2, ys2]
    outs = b.while_([b.const(0, "i32"), u0, ys0], cond, body)
    _, exe = check(client, b.module(outs), [f32(T, N), f32(2, N)], rtol=1e-6)
    assert ".window" in exe.plan_text()


def test_loop_state_pointer_exchange(client):
    """Carried values trade buffers with their next values instead of being copied. The body reads a carried
    value late (after temporaries have come and gone), returns one value at two positions and passes one through;
    odd and even trip counts leave the final values in either buffer."""
    N = 4096
    for trips in (1, 6, 7):
        b = Builder()
        x, y = b.arg((N,), "f32"), b.arg((N,), "f32")
        def cond(s, i, a, c, d, e): return s.compare(i, s.const(trips, "i32"), "LT")
        def body(s, i, a, c, d, e):
            t1 = s.tanh(s.add(a, c))
            t2 = s.reduce_sum(s.mul(t1, t1), [0])
            t3 = s.mul(t1, s.broadcast_in_dim(t2, (N,), []))
            # (the factor keeps the map contractive: rounding differences of the sum must not grow over the iterations)
            a2 = s.add(s.mul(t3, s.full((N,), 1e-4, "f32")), c)
            c2 = s.sub(a2, s.mul(a, s.full((N,), 0.5, "f32")))       # reads the old state after a2 exists
            return [s.add(i, s.const(1, "i32")), a2, c2, c2, e]
        outs = b.while_([b.const(0, "i32"), x, y, y, x], cond, body)
        _, exe = check(client, b.module(outs), [f32(N), f32(N)], rtol=1e-4)
        assert "exchanged=" in exe.plan_text()


def test_bundled_pointwise_kernels(client):
    """Independent pointwise results of different shapes leave as one launch; a later kernel that reads one of
    them stays separate. Values must equal the unbundled evaluation (the oracle)."""
    b = Builder()
    x, y, z = b.arg((1000,), "f32"), b.arg((7, 33), "f32"), b.arg((5000,), "f32")
    a1 = b.tanh(x)
    a2 = b.mul(y, y)
    a3 = b.add(z, b.full((5000,), 2.0, "f32"))
    s1 = b.reduce_sum(a3, [0])                       # forces a3 into memory before the dependent kernel
    a4 = b.mul(a3, b.broadcast_in_dim(s1, (5000,), []))
    _, exe = check(client, b.module([a1, a2, a3, a4]), [f32(1000), f32(7, 33), f32(5000)], rtol=1e-5)
    plan = exe.plan_text()
    assert "bundle_" in plan and plan.count("kernel ") < 6


def test_counted_loop_graph_replay_odd_and_even(client):
    """Counted loops of four or more iterations replay a recorded pair of iterations; odd counts run the last
    iteration directly. Executing twice reuses the recorded graph."""
    for trips in (4, 5, 11, 130):
        b = Builder()
        x = b.arg((300,), "f32")
        def cond(s, i, v, w): return s.compare(i, s.const(trips, "i32"), "LT")
        def body(s, i, v, w):
            v2 = s.add(s.mul(v, s.full((300,), 0.9, "f32")), w)
            return [s.add(i, s.const(1, "i32")), v2, s.mul(w, s.full((300,), 1.01, "f32"))]
        text = b.module(b.while_([b.const(0, "i32"), x, x], cond, body))
        xin = f32(300)
        got, exe = check(client, text, [xin], rtol=1e-4)
        assert int(got[0]) == trips
        again = [o.to_numpy() for o in exe.execute([client.buffer_from_host(xin)])]
        for g, a in zip(got, again):
            assert np.array_equal(np.asarray(g), a)


def test_results_share_blocks_and_outlive_their_siblings(client):
    """The results of one execution come out of two shared allocations (small and large results). A result that is
    kept while its siblings are deleted stays valid, later executions do not disturb it, and the accounted bytes
    return to where they were once everything is deleted."""
    b = Builder()
    x = b.arg((40000,), "f32")
    big1 = b.add(x, b.full((40000,), 1.0, "f32"))
    big2 = b.mul(x, b.full((40000,), 2.0, "f32"))
    s1 = b.reduce_sum(x, [0])
    s2 = b.reduce_sum(b.mul(x, x), [0])
    exe = client.compile(b.module([big1, big2, s1, s2]))
    xin = f32(40000)
    import gc
    gc.collect()                                         # buffers of earlier tests go first
    before = client.memory_stats().bytes_in_use
    xb = client.buffer_from_host(xin)
    outs = exe.execute([xb])
    keep_big, keep_small = outs[1], outs[2]
    outs[0].delete(); outs[3].delete()
    del outs
    for _ in range(3):                                   # further executions reuse the pool
        for o in exe.execute([xb]):
            o.delete()
    np.testing.assert_allclose(keep_big.to_numpy(), xin * 2.0, rtol=1e-6)
    np.testing.assert_allclose(float(keep_small.to_numpy()), float(xin.astype(np.float64).sum()), rtol=1e-4, atol=1e-3)
    keep_big.delete(); keep_small.delete(); xb.delete()
    client.synchronize()
    assert client.memory_stats().bytes_in_use == before


def test_row_scatter(client):
    """Row scatter with repeated and out-of-range indices: add in f32 and bf16 (update order, fp32 accumulator),
    multiply / minimum / maximum / set, i64 indices, and the embedding-gradient form."""
    rng = np.random.default_rng(3)
    idx = rng.integers(0, 12, (5, 7)).astype(np.int32)
    idx[0, 0], idx[1, 1] = 40, -2                      # dropped
    for dt, tol in [("f32", 1e-6), ("bf16", 1e-2)]:
        for op in ["add", "multiply", "minimum", "maximum", "set"]:
            b = Builder()
            t, i, u = b.arg((12, 3, 10), dt), b.arg((5, 7), "i32"), b.arg((5, 7, 3, 10), dt)
            if op == "set":                            # duplicates make "set" order-dependent: keep indices unique
                ii = np.arange(35, dtype=np.int32).reshape(5, 7) % 12
                ii[2:] = 100
                args = [f32(12, 3, 10), ii, f32(5, 7, 3, 10)]
            else:
                args = [f32(12, 3, 10), idx, f32(5, 7, 3, 10)]
            check(client, b.module([b.scatter_rows(t, i, u, op)]), args, rtol=tol, atol=tol, dtypes=[dt, None, dt])
    b = Builder()
    t, i, u = b.arg((9, 4), "i32"), b.arg((6,), "i64"), b.arg((6, 4), "i32")
    check(client, b.module([b.scatter_rows(t, i, u, "add")]),
          [rng.integers(-5, 5, (9, 4)).astype(np.int32), np.array([3, 3, 0, 8, 3, 0], np.int64), rng.integers(-5, 5, (6, 4)).astype(np.int32)])
    b = Builder()
    table, ids, g = b.arg((50, 8), "f32"), b.arg((3, 4), "i32"), b.arg((3, 4, 8), "f32")
    y = b.take_rows(table, ids)
    (dtab,) = b.grad(b.reduce_sum(b.mul(y, g), (0, 1, 2)), [table])
    check(client, b.module([y, dtab]), [f32(50, 8), rng.integers(0, 50, (3, 4)).astype(np.int32), f32(3, 4, 8)], rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("dt,out", [("i32", None), ("i8", "i32"), ("ui8", None), ("i64", None), ("ui32", None), ("i16", "i32")])
def test_integer_dot_general_is_exact(client, dt, out):
    """dot_general on integers: exact integer products and sums (wrapping in the result type), the layouts of the
    reference's matmul cases (tests/configs/matmul.py:19-141 of the reference): plain, transposed, batched, several
    free and several contracting dimensions, and a contraction of length 300 whose partial sums pass 2^24 (where the
    reference's cast through f32, src/pjrt_plugin/ops/linalg.cc:110-119, stops being exact)."""
    rng = np.random.default_rng(5)
    npdt = {"i32": np.int32, "i8": np.int8, "ui8": np.uint8, "i64": np.int64, "ui32": np.uint32, "i16": np.int16}[dt]
    lo, hi = (0, 200) if dt.startswith("u") else (-100, 100)
    big = dt in ("i32", "i64", "ui32")
    cases = [((6, 5), (5, 7), ((1,), (0,)), ((), ())),
             ((5, 6), (7, 5), ((0,), (1,)), ((), ())),
             ((3, 4, 9), (3, 9, 5), ((2,), (1,)), ((0,), (0,))),
             ((2, 3, 4, 6), (6, 5), ((3,), (0,)), ((), ())),
             ((4, 3, 5), (3, 5, 6), ((1, 2), (0, 1)), ((), ())),
             ((8, 300), (300, 9), ((1,), (0,)), ((), ())),
             ((7,), (7,), ((0,), (0,)), ((), ()))]
    for ls, rs, contract, batch in cases:
        b = Builder()
        x, y = b.arg(ls, dt), b.arg(rs, dt)
        text = b.module([b.dot_general(x, y, contract, batch, out_dtype=out)])
        scale = 20000 if big and ls == (8, 300) else 1
        args = [(rng.integers(lo, hi, ls) * scale).astype(npdt), (rng.integers(lo, hi, rs) * scale).astype(npdt)]
        check(client, text, args)


def test_boolean_dot_general(client):
    """dot_general on i1: and / or."""
    rng = np.random.default_rng(6)
    b = Builder()
    x, y = b.arg((9, 40), "i1"), b.arg((40, 11), "i1")
    text = b.module([b.dot_general(x, y, ((1,), (0,)))])
    check(client, text, [rng.random((9, 40)) < 0.05, rng.random((40, 11)) < 0.05])


def test_row_scatter_with_many_updates(client):
    """Above 1024 updates the (row, update number) ranking is a stable radix sort: one, two and three 8-bit passes
    (rows below 2^8, 2^16, 2^24), heavy duplication, dropped indices, i64 indices; integer results are exact, the
    f32 sums follow update order (one accumulator per row), and two executions agree bit for bit."""
    rng = np.random.default_rng(11)
    for rows, U, idt in [(200, 5000, "i32"), (30522, 4096, "i32"), (70000, 3000, "i64"), (300, 2049, "i32")]:
        idx = rng.integers(0, rows, (U,)).astype(np.int64 if idt == "i64" else np.int32)
        idx[::97] = rows + 5                            # dropped
        idx[1::131] = -1                                # dropped
        b = Builder()
        t, i, u = b.arg((rows, 8), "i32"), b.arg((U,), idt), b.arg((U, 8), "i32")
        check(client, b.module([b.scatter_rows(t, i, u, "add")]),
              [rng.integers(-9, 9, (rows, 8)).astype(np.int32), idx, rng.integers(-9, 9, (U, 8)).astype(np.int32)])
        b = Builder()
        t, i, u = b.arg((rows, 8), "f32"), b.arg((U,), idt), b.arg((U, 8), "f32")
        text = b.module([b.scatter_rows(t, i, u, "add")])
        args = [f32(rows, 8), idx, f32(U, 8)]
        check(client, text, args, rtol=1e-6, atol=1e-5)
        exe = client.compile(text)
        bufs = [client.buffer_from_host(a) for a in args]
        first = exe.execute(bufs)[0].to_numpy()
        np.testing.assert_array_equal(exe.execute(bufs)[0].to_numpy(), first)


GENERAL_SCATTERS = [
    # operand shape, indices shape, updates shape, dimension numbers: the forms x.at[i, j].add(v), x.at[i, 2:5].add(rows),
    # x.at[:, j].add(cols), windows of a rank-3 operand, batching dimensions, a scalar index
    ((9, 7), (20, 2), (20,), dict(update_window_dims=(), inserted_window_dims=(0, 1), scatter_dims_to_operand_dims=(0, 1), index_vector_dim=1)),
    ((9, 7), (12, 2), (12, 1, 3), dict(update_window_dims=(1, 2), inserted_window_dims=(), scatter_dims_to_operand_dims=(0, 1), index_vector_dim=1)),
    ((9, 7), (15,), (9, 15), dict(update_window_dims=(0,), inserted_window_dims=(1,), scatter_dims_to_operand_dims=(1,), index_vector_dim=1)),
    ((6, 5, 8), (4, 10, 2), (4, 10, 5), dict(update_window_dims=(2,), inserted_window_dims=(0, 2), scatter_dims_to_operand_dims=(0, 2), index_vector_dim=2)),
    ((4, 6, 5), (4, 7, 1), (4, 7, 5), dict(update_window_dims=(2,), inserted_window_dims=(1,), scatter_dims_to_operand_dims=(1,), index_vector_dim=2,
                                           input_batching_dims=(0,), scatter_indices_batching_dims=(0,))),
    ((30,), (1,), (4,), dict(update_window_dims=(0,), inserted_window_dims=(), scatter_dims_to_operand_dims=(0,), index_vector_dim=0)),
    ((3000, 6), (5000, 2), (5000,), dict(update_window_dims=(), inserted_window_dims=(0, 1), scatter_dims_to_operand_dims=(0, 1), index_vector_dim=1)),
]


POINT_1D = dict(update_window_dims=(), inserted_window_dims=(0,), scatter_dims_to_operand_dims=(0,), index_vector_dim=1)
SCATTER_BODIES = {
    "apply_sin": (lambda s, a, u: s.sin(a), "f32"),                           # lax.scatter_apply(x, idx, jnp.sin)
    "apply_mul2": (lambda s, a, u: s.mul(a, s.const(2.0, "f32")), "f32"),
    "subtract": ("subtract", "f32"),
    "decay_then_add": (lambda s, a, u: s.add(s.mul(a, s.const(0.5, "f32")), u), "f32"),      # depends on the order of duplicates
    "add_ui8": ("add", "ui8"),
    "add_i64": ("add", "i64"),
    "add_f64": ("add", "f64"),
    "max_i16": ("maximum", "i16"),
}


@pytest.mark.parametrize("name", sorted(SCATTER_BODIES))
def test_scatter_with_any_update_computation(client, name):
    """Update computations and element types beyond the built-in five run through the compiled region
    (tests/configs/slice.py:500-535 of the reference: lax.scatter_apply with sin and with x * 2;
    src/pjrt_plugin/ops/gather_scatter.cc:79-120). Duplicate destinations are folded in update order."""
    from b200.shlo.builder import _NP
    op, dt = SCATTER_BODIES[name]
    rng = np.random.default_rng(11)
    for n, idx in [(6, np.array([[0], [2], [4]], np.int32)), (5, np.array([[1], [3]], np.int32)),
                   (40, rng.integers(-2, 42, (300, 1)).astype(np.int32))]:
        if name.startswith("apply") and len(idx) > 3:
            idx = np.unique(idx, axis=0)                # the reference applies a function once per index
        b = Builder()
        t, i, u = b.arg((n,), dt), b.arg(idx.shape, "i32"), b.arg((len(idx),), dt)
        text = b.module([b.scatter(t, i, u, op, **POINT_1D)])
        plan, _ = b200.compile_to_plan(text)
        assert "scatter_apply" in plan, plan
        if dt in ("f32", "f64"):
            args = [rng.standard_normal(n).astype(_NP[dt]), idx, rng.standard_normal(len(idx)).astype(_NP[dt])]
        elif dt == "i64":
            args = [rng.integers(-2**40, 2**40, n), idx, rng.integers(-2**40, 2**40, len(idx))]
        else:
            info = np.iinfo(_NP[dt])
            args = [rng.integers(info.min, info.max, n).astype(_NP[dt]), idx, rng.integers(info.min, info.max, len(idx)).astype(_NP[dt])]
        check(client, text, args, rtol=1e-5, atol=1e-5, dtypes=[dt, "i32", dt])


@pytest.mark.parametrize("os_,is_,us_,dn", GENERAL_SCATTERS)
def test_general_scatter(client, os_, is_, us_, dn):
    """stablehlo.scatter beyond the row form (point updates, partial windows, batching dimensions;
    src/pjrt_plugin/ops/gather_scatter.cc:296-699): duplicates accumulate in update order, a window that does not fit is
    dropped as a whole, integer results are exact and two executions agree bit for bit."""
    rng = np.random.default_rng(8)
    sdo = dn["scatter_dims_to_operand_dims"]
    ivd = dn["index_vector_dim"]
    comps = is_[ivd] if ivd < len(is_) else 1
    idx = np.zeros(is_, np.int32)
    for k in range(comps):
        hi = os_[sdo[k]]
        col = rng.integers(-1, hi + 1, [n for d, n in enumerate(is_) if d != ivd] if ivd < len(is_) else is_)     # some out of range
        if ivd < len(is_):
            np.moveaxis(idx, ivd, -1)[..., k] = col
        else:
            idx[...] = col
    for op, dt in [("add", "i32"), ("add", "f32"), ("maximum", "f32"), ("set", "i32")]:
        b = Builder()
        t, i, u = b.arg(os_, dt), b.arg(is_, "i32"), b.arg(us_, dt)
        text = b.module([b.scatter(t, i, u, op, **dn)])
        plan, _ = b200.compile_to_plan(text)
        assert "scatter keys" in plan or "scatter_keys" in plan, plan
        if dt == "i32":
            args = [rng.integers(-9, 9, os_).astype(np.int32), idx, rng.integers(-9, 9, us_).astype(np.int32)]
        else:
            args = [f32(*os_), idx, f32(*us_)]
        if op == "set":                       # duplicates make "set" order-dependent in the oracle: compare sums only where unique
            continue
        check(client, text, args, rtol=1e-5, atol=1e-5)
        exe = client.compile(text)
        bufs = [client.buffer_from_host(a) for a in args]
        first = exe.execute(bufs)[0].to_numpy()
        np.testing.assert_array_equal(exe.execute(bufs)[0].to_numpy(), first)


def test_case_branches(client):
    """lax.cond / lax.switch lowerings: branches capture outer values; an index outside [0, n) runs the last
    branch; a case inside a while body."""
    b = Builder()
    idx, x, y = b.arg((), "i32"), b.arg((6, 5), "f32"), b.arg((6, 5), "f32")
    outs = b.case(idx, [lambda s: [s.add(x, y), s.reduce_sum(x, (0,))],
                        lambda s: [s.mul(x, y), s.reduce_sum(y, (0,))],
                        lambda s: [s.tanh(s.sub(x, y)), s.reduce_max(x, (0,))]],
                  [((6, 5), "f32"), ((5,), "f32")])
    text = b.module([outs[0], b.exp(outs[1])])
    for i in [0, 1, 2, 7, -3]:
        check(client, text, [np.int32(i), f32(6, 5), f32(6, 5)])
    b = Builder()
    v = b.arg((4,), "f32")
    def cond(s, i, a): return s.compare(i, s.const(5, "i32"), "LT")
    def body(s, i, a):
        r = s.case(s.rem(i, s.const(2, "i32")), [lambda q: [q.add(a, q.full((4,), 1.0, "f32"))],
                                                  lambda q: [q.mul(a, q.full((4,), 2.0, "f32"))]], [((4,), "f32")])
        return [s.add(i, s.const(1, "i32")), r[0]]
    check(client, b.module(b.while_([b.const(0, "i32"), v], cond, body)), [f32(4)])


def test_loop_carried_swap(client):
    """Body hands carried values to other positions; copies must not clobber."""
    b = Builder()
    x, y = b.arg((4,), "f32"), b.arg((4,), "f32")
    def cond(s, i, a, c): return s.compare(i, s.const(3, "i32"), "LT")
    def body(s, i, a, c): return [s.add(i, s.const(1, "i32")), c, a]
    check(client, b.module(b.while_([b.const(0, "i32"), x, y], cond, body)), [f32(4), f32(4)])


# ---------------------------------------------------------------------------
# BatchNorm forward + backward (reductions with fused producers, split over blocks)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(16, 2, 2, 128), (16, 4, 4, 64), (16, 8, 8, 32), (32, 16, 16, 16), (16, 16, 16, 8),
                                   (128, 8, 8, 48)])
def test_batch_norm_relu_gradients(client, shape):
    from b200.shlo.programs import _batch_norm, _relu
    b = Builder()
    x, scale, bias, g = b.arg(shape, "f32"), b.arg(shape[-1:], "f32"), b.arg(shape[-1:], "f32"), b.arg(shape, "f32")
    y = _relu(b, _batch_norm(b, x, scale, bias))
    loss = b.reduce_sum(b.mul(y, g), (0, 1, 2, 3))
    grads = b.grad(loss, [x, scale, bias])
    check(client, b.module([y, loss] + grads), [f32(*shape, lo=-2, hi=3), f32(shape[-1], lo=0.5, hi=1.5), f32(shape[-1]),
                                                f32(*shape)], rtol=1e-4, atol=1e-5, wide=True, scale_atol=True)
