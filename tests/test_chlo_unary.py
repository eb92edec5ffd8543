"""The chlo unary functions on the CPU: both forms compile to one generated kernel whose source passes NVRTC, and
the oracle's values are NumPy's / SciPy's (the reference's table: src/pjrt_plugin/ops/control_flow.cc:53-66)."""
import numpy as np
import pytest
import scipy.special

import b200
from b200.shlo.builder import Builder
from oracle import interp

FUNCS = {"sinh": np.sinh, "cosh": np.cosh, "asin": np.arcsin, "acos": np.arccos, "atan": np.arctan, "asinh": np.arcsinh,
         "acosh": lambda a: np.arccosh(a + 2.0), "atanh": np.arctanh, "erf": scipy.special.erf, "erf_inv": scipy.special.erfinv,
         "tan": np.tan}


@pytest.mark.parametrize("form", ["op", "custom_call"])
@pytest.mark.parametrize("name", sorted(FUNCS))
def test_chlo_unary_compiles_and_oracle_matches_numpy(name, form):
    x = np.linspace(-0.95, 0.95, 39).astype(np.float32).reshape(3, 13)
    b = Builder()
    xv = b.arg(x.shape, "f32")
    arg = b.add(xv, b.full(x.shape, 2.0, "f32")) if name == "acosh" else xv
    text = b.module([b.chlo_unary(name, arg, form)])
    plan, src = b200.compile_to_plan(text, validate=True)
    assert plan.count("kernel ") == 1, plan
    (got,) = interp.run_text(text, [x])
    np.testing.assert_allclose(got, FUNCS[name](x.astype(np.float64)), rtol=1e-6, atol=1e-6)


def test_mhlo_topk_custom_call_is_top_k():
    x = np.random.default_rng(0).standard_normal((4, 9)).astype(np.float32)
    b = Builder()
    xv = b.arg(x.shape, "f32")
    text = b.module(b.custom_call("mhlo.topk", [xv], [((4, 3), "f32"), ((4, 3), "i32")]))
    plan, _ = b200.compile_to_plan(text, validate=True)
    assert "sort_tile" in plan
    vals, idx = interp.run_text(text, [x])
    np.testing.assert_array_equal(vals, -np.sort(-x, axis=-1)[:, :3])
    np.testing.assert_array_equal(np.take_along_axis(x, idx.astype(np.int64), -1), vals)
