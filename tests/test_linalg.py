"""stablehlo.cholesky and stablehlo.triangular_solve. The reference hands both to LAPACK on the host
(src/pjrt_plugin/ops/linalg.cc:553-660); the oracle does the same in float64 and is pinned by the defining identities
(L L^T = A, op(A) X = B), the GPU path is held to the oracle. Shapes follow the reference's cases
(tests/configs/linalg.py:150-260: 2x2 to 4x4, one and several right-hand sides, both triangles, transposed, unit
diagonal, a singular matrix) plus batches and sizes that span several blocks."""
import numpy as np
import pytest

import b200
from b200.shlo.builder import Builder
from oracle import interp


def _posdef(batch, n, seed=0):
    m = np.random.default_rng(seed).standard_normal(batch + (n, n))
    return (m @ np.swapaxes(m, -1, -2) + n * np.eye(n)).astype(np.float32)


def _tri(batch, n, lower, seed=0, unit=False):
    m = np.random.default_rng(seed).standard_normal(batch + (n, n)) / (np.sqrt(n) if n > 8 else 1.0)     # large ones stay well conditioned
    t = np.tril(m) if lower else np.triu(m)
    eye = np.eye(n)
    t = t * (1 - eye) + (eye if unit else (np.abs(t * eye) + eye))
    return t.astype(np.float32)


@pytest.mark.parametrize("lower", [True, False])
@pytest.mark.parametrize("batch,n", [((), 2), ((), 3), ((), 4), ((3, 2), 5), ((), 33)])
def test_oracle_cholesky_factors_its_input(batch, n, lower):
    a = _posdef(batch, n)
    junk = a + np.where(np.tril(np.ones((n, n)), -1).T if lower else np.tril(np.ones((n, n)), -1), 7.0, 0.0).astype(np.float32)
    b = Builder()
    text = b.module([b.cholesky(b.arg(a.shape, "f32"), lower)])
    (l,) = interp.run_text(text, [junk])                 # the other triangle is never read
    prod = l @ np.swapaxes(l, -1, -2) if lower else np.swapaxes(l, -1, -2) @ l
    np.testing.assert_allclose(prod, a, rtol=1e-5, atol=1e-5)
    assert np.all((np.triu(l, 1) if lower else np.tril(l, -1)) == 0)


def test_oracle_cholesky_of_an_indefinite_matrix_is_nan():
    b = Builder()
    text = b.module([b.cholesky(b.arg((2, 2), "f32"))])
    (l,) = interp.run_text(text, [np.array([[-1, 0], [0, 1]], np.float32)])
    assert np.isnan(l).any()


SOLVES = [  # batch, n, k, left, lower, unit, transpose
    ((), 2, 1, True, True, False, "NO_TRANSPOSE"), ((), 3, 1, True, False, False, "NO_TRANSPOSE"),
    ((), 4, 3, True, True, False, "NO_TRANSPOSE"), ((), 4, 3, True, False, False, "NO_TRANSPOSE"),
    ((), 3, 1, True, True, False, "TRANSPOSE"), ((), 3, 1, True, False, False, "TRANSPOSE"),
    ((), 3, 1, True, True, True, "NO_TRANSPOSE"), ((2, 3), 5, 4, False, True, False, "NO_TRANSPOSE"),
    ((2,), 5, 4, False, False, False, "ADJOINT"), ((), 40, 300, True, True, False, "NO_TRANSPOSE"),
    ((), 40, 7, False, False, True, "TRANSPOSE")]


def _solve_case(batch, n, k, left, lower, unit, tr):
    a = _tri(batch, n, lower, 1, unit)
    rhs = np.random.default_rng(2).standard_normal(batch + ((n, k) if left else (k, n))).astype(np.float32)
    b = Builder()
    text = b.module([b.triangular_solve(b.arg(a.shape, "f32"), b.arg(rhs.shape, "f32"), left_side=left, lower=lower,
                                        unit_diagonal=unit, transpose_a=tr)])
    return text, a, rhs


@pytest.mark.parametrize("batch,n,k,left,lower,unit,tr", SOLVES)
def test_oracle_triangular_solve_satisfies_its_equation(batch, n, k, left, lower, unit, tr):
    text, a, rhs = _solve_case(batch, n, k, left, lower, unit, tr)
    (x,) = interp.run_text(text, [a, rhs])
    m = a.astype(np.float64)
    if tr != "NO_TRANSPOSE":
        m = np.swapaxes(m, -1, -2)
    back = m @ x if left else x @ m
    np.testing.assert_allclose(back, rhs, rtol=1e-4, atol=1e-4)


def test_oracle_singular_solve_is_nan_per_matrix():
    a = np.stack([np.array([[1.0, 0.0], [1.0, 0.0]], np.float32), np.array([[1.0, 0.0], [1.0, 2.0]], np.float32)])
    rhs = np.ones((2, 2, 1), np.float32)
    b = Builder()
    text = b.module([b.triangular_solve(b.arg(a.shape, "f32"), b.arg(rhs.shape, "f32"))])
    (x,) = interp.run_text(text, [a, rhs])
    assert np.isnan(x[0]).all() and np.isfinite(x[1]).all()


def test_linalg_plans_compile():
    b = Builder()
    a = b.arg((3, 6, 6), "f32")
    l = b.cholesky(a)
    x = b.triangular_solve(l, b.arg((3, 6, 2), "f32"), transpose_a="TRANSPOSE")
    plan, _ = b200.compile_to_plan(b.module([l, x]), validate=True)
    assert "cholesky_" in plan and "triangular_solve_" in plan, plan
    b = Builder()
    plan, _ = b200.compile_to_plan(b.module([b.cholesky(b.arg((4, 4), "f64"), False)]), validate=True)
    with pytest.raises(Exception, match="not supported"):
        b = Builder()
        b200.compile_to_plan(b.module([b.cholesky(b.arg((4, 4), "bf16"))]))


@pytest.mark.gpu
@pytest.mark.parametrize("lower", [True, False])
@pytest.mark.parametrize("batch,n", [((), 2), ((), 3), ((), 4), ((3, 2), 5), ((), 33), ((2,), 300)])
def test_cholesky_on_the_gpu(client, batch, n, lower):
    from util import run_gpu
    a = _posdef(batch, n, 3)
    b = Builder()
    text = b.module([b.cholesky(b.arg(a.shape, "f32"), lower)])
    got, _ = run_gpu(client, text, [a])
    want = interp.run_text(text, [a])
    np.testing.assert_allclose(got[0], want[0], rtol=2e-4, atol=2e-4 * float(np.abs(want[0]).max()))
    l = got[0].astype(np.float64)
    prod = l @ np.swapaxes(l, -1, -2) if lower else np.swapaxes(l, -1, -2) @ l
    np.testing.assert_allclose(prod, a, rtol=1e-4, atol=1e-4 * float(np.abs(a).max()))


@pytest.mark.gpu
def test_cholesky_of_an_indefinite_matrix_on_the_gpu(client):
    from util import run_gpu
    b = Builder()
    got, _ = run_gpu(client, b.module([b.cholesky(b.arg((2, 2), "f32"))]), [np.array([[-1, 0], [0, 1]], np.float32)])
    assert np.isnan(got[0]).any()


@pytest.mark.gpu
@pytest.mark.parametrize("batch,n,k,left,lower,unit,tr", SOLVES)
def test_triangular_solve_on_the_gpu(client, batch, n, k, left, lower, unit, tr):
    from util import run_gpu
    text, a, rhs = _solve_case(batch, n, k, left, lower, unit, tr)
    got, _ = run_gpu(client, text, [a, rhs])
    want = interp.run_text(text, [a, rhs])
    np.testing.assert_allclose(got[0], want[0], rtol=2e-3, atol=2e-3 * float(np.abs(want[0]).max()))
    m = a.astype(np.float64)
    if tr != "NO_TRANSPOSE":
        m = np.swapaxes(m, -1, -2)
    x = got[0].astype(np.float64)
    back = m @ x if left else x @ m
    np.testing.assert_allclose(back, rhs, rtol=1e-3, atol=1e-3 * max(1.0, float(np.abs(x).max())))


@pytest.mark.gpu
def test_singular_solve_is_nan_per_matrix_on_the_gpu(client):
    from util import run_gpu
    a = np.stack([np.array([[1.0, 0.0], [1.0, 0.0]], np.float32), np.array([[1.0, 0.0], [1.0, 2.0]], np.float32)])
    rhs = np.ones((2, 2, 1), np.float32)
    b = Builder()
    got, _ = run_gpu(client, b.module([b.triangular_solve(b.arg(a.shape, "f32"), b.arg(rhs.shape, "f32"))]), [a, rhs])
    assert np.isnan(got[0][0]).all()
    np.testing.assert_allclose(got[0][1], [[1.0], [0.0]], atol=1e-6)
