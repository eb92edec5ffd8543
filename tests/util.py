"""Helpers shared by the parity tests: run a StableHLO module on the GPU
through the C ABI and on the CPU oracle, and compare with the reference's
rule (tests/test_ops.py:91-105 of the reference: exact for integers and
booleans, tolerance for floats)."""
import numpy as np

from oracle import interp

# fp32 bar of the plugin: rtol 1e-4 / atol 1e-5 end to end; single ops are held to the reference's 1e-5
RTOL, ATOL = 1e-5, 1e-5


def run_gpu(client, text, args, dtypes=None):
    exe = client.compile(text)
    bufs = [client.buffer_from_host(a, dtype=(dtypes[i] if dtypes else None)) for i, a in enumerate(args)]
    return [o.to_numpy() for o in exe.execute(bufs)], exe


def compare(got, want, rtol=RTOL, atol=ATOL, what="", scale_atol=False):
    """`scale_atol` multiplies atol by max|want| (>= 1): sums of many O(1) terms carry an absolute
    rounding error proportional to the magnitude of the terms, not of the (possibly cancelling) result."""
    got, want = np.asarray(got), np.asarray(want)
    if scale_atol and want.size and want.dtype.kind == "f":
        atol = atol * max(1.0, float(np.max(np.abs(want))))
    assert got.shape == want.shape, (what, got.shape, want.shape)
    if want.dtype.kind in "iub":
        np.testing.assert_array_equal(got, want.astype(got.dtype), err_msg=what)
    else:
        np.testing.assert_allclose(got.astype(np.float64), want.astype(np.float64), rtol=rtol, atol=atol,
                                   equal_nan=True, err_msg=what)


def check(client, text, args, rtol=RTOL, atol=ATOL, wide=False, dtypes=None, scale_atol=False):
    got, exe = run_gpu(client, text, args, dtypes)
    want = interp.run_text(text, args, wide=wide)
    assert len(got) == len(want)
    for i, (g, w) in enumerate(zip(got, want)):
        compare(g, w, rtol, atol, what=f"result {i}", scale_atol=scale_atol)
    return got, exe
