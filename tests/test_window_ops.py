"""reduce_window and select_and_scatter (pooling, cumulative reductions, the gradient of max pooling): the oracle is
pinned against PyTorch on the CPU, the GPU path against the oracle. The reference handles these in
src/pjrt_plugin/ops/reduction.cc:165-626 (pooling with max / sum / min / prod, cumulative forms, select_and_scatter with
an add scatter and padding that is never selected)."""
import numpy as np
import pytest
import torch

import b200
from b200.shlo.builder import Builder
from oracle import interp


def _x(shape, seed=0):
    return np.random.default_rng(seed).standard_normal(shape).astype(np.float32)


NHWC_POOL = [((1, 3, 3, 1), (1, 2, 2, 1), ((0, 0), (1, 1), (1, 1), (0, 0))),      # ResNet stem pooling
             ((1, 2, 2, 1), (1, 2, 2, 1), None),
             ((1, 3, 2, 1), (1, 1, 2, 1), ((0, 0), (1, 0), (0, 1), (0, 0)))]


@pytest.mark.parametrize("window,strides,padding", NHWC_POOL)
def test_oracle_pooling_matches_torch(window, strides, padding):
    x = _x((2, 9, 10, 3))
    pad = padding or ((0, 0),) * 4
    b = Builder()
    xv = b.arg(x.shape, "f32")
    fwd = b.reduce_window(xv, -np.inf, "maximum", window, strides, padding)
    src = b.arg(fwd.shape, "f32")
    bwd = b.select_and_scatter(xv, src, 0.0, window, strides, padding, select="GE")
    text = b.module([fwd, bwd])
    g = _x(fwd.shape, 1)
    got = interp.run_text(text, [x, g])
    xt = torch.from_numpy(x).permute(0, 3, 1, 2).clone().requires_grad_(True)
    xp = torch.nn.functional.pad(xt, (pad[2][0], pad[2][1], pad[1][0], pad[1][1]), value=float("-inf"))
    out = torch.nn.functional.max_pool2d(xp, (window[1], window[2]), (strides[1], strides[2]))
    out.backward(torch.from_numpy(g).permute(0, 3, 1, 2))
    np.testing.assert_array_equal(got[0], out.detach().permute(0, 2, 3, 1).numpy())
    np.testing.assert_allclose(got[1], xt.grad.permute(0, 2, 3, 1).numpy(), atol=1e-6)


def test_oracle_cumulative_and_sum_pool():
    v = _x((5, 7), 2)
    b = Builder()
    xv = b.arg(v.shape, "f32")
    text = b.module([b.reduce_window(xv, 0.0, "add", (1, 7), (1, 1), ((0, 0), (6, 0))),
                     b.reduce_window(xv, -np.inf, "maximum", (5, 1), (1, 1), ((4, 0), (0, 0))),
                     b.reduce_window(xv, 0.0, "add", (2, 2), (2, 2), None)])
    got = interp.run_text(text, [v])
    np.testing.assert_allclose(got[0], np.cumsum(v, 1), atol=1e-5)
    np.testing.assert_array_equal(got[1], np.maximum.accumulate(v, 0))
    np.testing.assert_allclose(got[2], v[:4, :6].reshape(2, 2, 3, 2).sum((1, 3)), atol=1e-6)


def test_window_ops_compile_to_one_kernel_each():
    b = Builder()
    xv = b.arg((2, 9, 10, 3), "f32")
    fwd = b.reduce_window(xv, -np.inf, "maximum", (1, 3, 3, 1), (1, 2, 2, 1), ((0, 0), (1, 1), (1, 1), (0, 0)))
    bwd = b.select_and_scatter(xv, b.mul(fwd, fwd), 0.0, (1, 3, 3, 1), (1, 2, 2, 1), ((0, 0), (1, 1), (1, 1), (0, 0)))
    plan, _ = b200.compile_to_plan(b.module([fwd, bwd]), validate=True)
    assert plan.count("window_") == 2 and "reduce_window" in plan and "select_and_scatter" in plan, plan


GPU_CASES = [
    # (shape, dtype, op, init, window, strides, padding, base_dilations, window_dilations)
    ((2, 9, 10, 3), "f32", "maximum", -np.inf, (1, 3, 3, 1), (1, 2, 2, 1), ((0, 0), (1, 1), (1, 1), (0, 0)), None, None),
    ((2, 9, 10, 3), "f32", "minimum", np.inf, (1, 2, 2, 1), (1, 2, 2, 1), None, None, None),
    ((4, 16, 16, 8), "f32", "add", 0.0, (1, 2, 2, 1), (1, 2, 2, 1), None, None, None),
    ((3, 11, 7), "f32", "add", 0.0, (1, 3, 2), (1, 2, 1), ((0, 0), (2, 1), (1, 1)), (1, 2, 1), (1, 1, 2)),   # both dilations
    ((6, 33), "f32", "add", 0.0, (1, 33), (1, 1), ((0, 0), (32, 0)), None, None),                               # cumulative sum
    ((6, 33), "f32", "multiply", 1.0, (6, 1), (1, 1), ((5, 0), (0, 0)), None, None),                            # cumulative product
    ((6, 33), "f32", "maximum", -np.inf, (1, 33), (1, 1), ((0, 0), (0, 32)), None, None),                       # reverse cumulative max
    ((5, 12), "f32", "add", 0.0, (2, 3), (1, 1), ((0, 0), (-1, -2)), None, None),                               # negative padding crops
    ((2, 9, 10, 3), "bf16", "maximum", -np.inf, (1, 3, 3, 1), (1, 2, 2, 1), ((0, 0), (1, 1), (1, 1), (0, 0)), None, None),
    ((7, 9), "i32", "add", 0, (3, 3), (2, 2), ((1, 1), (1, 1)), None, None),
]


@pytest.mark.gpu
@pytest.mark.parametrize("shape,dt,op,init,window,strides,padding,bdil,wdil", GPU_CASES)
def test_reduce_window_on_the_gpu(client, shape, dt, op, init, window, strides, padding, bdil, wdil):
    from util import run_gpu
    b = Builder()
    xv = b.arg(shape, dt)
    text = b.module([b.reduce_window(xv, init, op, window, strides, padding, bdil, wdil)])
    x = _x(shape, 3)
    if dt == "i32":
        x = (x * 10).astype(np.int32)
    got, _ = run_gpu(client, text, [x], dtypes=[dt])
    want = interp.run_text(text, [x])
    if dt == "i32" or op in ("maximum", "minimum"):
        np.testing.assert_array_equal(got[0], want[0])
    else:
        np.testing.assert_allclose(got[0], want[0], rtol=1e-5, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("select", ["GE", "GT", "LE"])
@pytest.mark.parametrize("window,strides,padding", NHWC_POOL + [((1, 3, 3, 1), (1, 1, 1, 1), ((0, 0), (1, 1), (1, 1), (0, 0)))])
def test_select_and_scatter_on_the_gpu(client, select, window, strides, padding):
    """Overlapping windows, padding, and ties (the operand is rounded to few distinct values): GE / LE give a tie to the
    first element of the window, GT to the last; every element's sum is accumulated in the row-major order of the windows."""
    from util import run_gpu
    shape = (2, 9, 10, 3)
    x = np.round(_x(shape, 4) * 2) / 2
    b = Builder()
    xv = b.arg(shape, "f32")
    probe = b.reduce_window(xv, 0.0, "add", window, strides, padding)
    src = b.arg(probe.shape, "f32")
    text = b.module([b.select_and_scatter(xv, src, 0.0, window, strides, padding, select=select)])
    g = _x(probe.shape, 5)
    got, _ = run_gpu(client, text, [x, g])
    want = interp.run_text(text, [x, g])
    np.testing.assert_allclose(got[0], want[0], rtol=1e-6, atol=1e-6)
    assert abs(float(got[0].sum()) - float(g.sum())) < 1e-3 * max(1.0, float(np.abs(g).sum()))      # every window gives its value once
