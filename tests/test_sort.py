"""stablehlo.sort and chlo.top_k. The oracle's sort is defined by all-pairs ranks with the comparator region and is
pinned against NumPy's stable sort; its merging form for long rows is pinned against the rank form; the GPU path is
held bit-exact to the oracle. Shapes follow the reference's cases (tests/configs/sort.py:13-205: jnp.sort over every
axis of 1-D to 3-D inputs, descending, lax.sort_key_val with several operands, lax.top_k for k from 1 to the axis
size); the reference's handlers are src/pjrt_plugin/ops/sort_fft_complex.cc:41-250."""
import numpy as np
import pytest

import b200
from b200.shlo.builder import Builder
from oracle import interp


def _x(shape, seed=0, ties=False):
    x = np.random.default_rng(seed).standard_normal(shape).astype(np.float32)
    return np.round(x * 2) / 2 + 0.0 if ties else x            # + 0.0: no negative zeros, which the total order tells apart


SORT_CASES = [((16,), 0), ((4, 8), 0), ((4, 8), 1), ((2, 4, 8), 0), ((2, 4, 8), 1), ((2, 4, 8), 2), ((3, 1000), 1),
              ((37, 5, 3), 0)]


@pytest.mark.parametrize("shape,dim", SORT_CASES)
@pytest.mark.parametrize("descending", [False, True])
def test_oracle_sort_matches_numpy(shape, dim, descending):
    x = _x(shape, 1, ties=True)
    tag = np.arange(x.size, dtype=np.int32).reshape(shape)
    b = Builder()
    xv, tv = b.arg(shape, "f32"), b.arg(shape, "i32")
    text = b.module(b.sort([xv, tv], dim, descending=descending))
    got = interp.run_text(text, [x, tag])
    order = np.argsort(-x if descending else x, axis=dim, kind="stable")
    np.testing.assert_array_equal(got[0], np.take_along_axis(x, order, dim))
    np.testing.assert_array_equal(got[1], np.take_along_axis(tag, order, dim))       # equal keys keep their order


def test_oracle_sort_total_order_of_floats():
    x = np.array([np.nan, 1.0, -0.0, 0.0, -np.inf, np.inf, -1.0, -np.nan], np.float32)
    x[7] = np.frombuffer(np.uint32(0xFFC00000).tobytes(), np.float32)[0]                # NaN with the sign bit set
    b = Builder()
    text = b.module(b.sort([b.arg(x.shape, "f32")], 0))
    (got,) = interp.run_text(text, [x])
    bits = got.view(np.uint32)
    assert bits[0] == 0xFFC00000 and np.isnan(got[7]) and not np.signbit(got[7])
    np.testing.assert_array_equal(got[1:7], np.array([-np.inf, -1.0, -0.0, 0.0, 1.0, np.inf], np.float32))
    assert np.signbit(got[3]) and not np.signbit(got[4])


def test_oracle_merging_form_equals_rank_form():
    x = _x((3, 1500), 2, ties=True)
    y = np.random.default_rng(3).integers(0, 4, x.shape).astype(np.int32)
    tag = np.arange(x.size, dtype=np.int32).reshape(x.shape)
    b = Builder()
    vs = [b.arg(x.shape, "f32"), b.arg(x.shape, "i32"), b.arg(x.shape, "i32")]
    text = b.module(b.sort(vs, 1, num_keys=2))
    want = interp.run_text(text, [x, y, tag])
    old = interp.Interp.SORT_RANK_MAX
    interp.Interp.SORT_RANK_MAX = 0
    try:
        got = interp.run_text(text, [x, y, tag])
    finally:
        interp.Interp.SORT_RANK_MAX = old
    for g, w in zip(got, want):
        np.testing.assert_array_equal(g, w)
    order = np.lexsort((y, x), axis=1)
    np.testing.assert_array_equal(want[2], np.take_along_axis(tag, order, 1))


TOP_K_CASES = [((16,), 3), ((4, 8), 1), ((4, 8), 3), ((4, 8), 5), ((2, 4, 8), 2), ((2, 2, 4, 8), 3), ((4, 8), 8), ((5, 3000), 40)]


@pytest.mark.parametrize("shape,k", TOP_K_CASES)
def test_oracle_top_k(shape, k):
    x = _x(shape, 4, ties=True)
    b = Builder()
    text = b.module(b.top_k(b.arg(shape, "f32"), k))
    vals, idx = interp.run_text(text, [x])
    assert idx.dtype == np.int32 and vals.shape == shape[:-1] + (k,)
    np.testing.assert_array_equal(vals, -np.sort(-x, axis=-1)[..., :k])
    np.testing.assert_array_equal(np.take_along_axis(x, idx.astype(np.int64), -1), vals)
    same = vals[..., 1:] == vals[..., :-1]
    assert np.all(idx[..., 1:][same] > idx[..., :-1][same])                              # ties by ascending position


def test_sort_plans():
    """A row that fits one tile is one launch; a longer row adds one launch per doubling of the sorted runs, all but the
    last sharing a kernel; chlo.top_k is a sort of the values with their positions followed by slices. The generated
    source compiles."""
    b = Builder()
    x = b.arg((6, 1000), "f32")
    plan, _ = b200.compile_to_plan(b.module(b.sort([x], 1)), validate=True)
    assert plan.count("sort_tile") == 1 and "sort_merge" not in plan, plan
    b = Builder()
    x, t = b.arg((5000, 3), "bf16"), b.arg((5000, 3), "i32")
    plan, src = b200.compile_to_plan(b.module(b.sort([x, t], 0, descending=True)), validate=True)
    lines = [l for l in plan.splitlines() if "sort" in l]
    assert sum("sort_tile" in l for l in lines) == 1 and sum("sort_merge" in l for l in lines) == 3, plan      # runs of 1024, 2048, 4096
    assert sum("sort_merge_out" in l for l in lines) == 1
    b = Builder()
    plan, _ = b200.compile_to_plan(b.module(b.top_k(b.arg((4, 8), "f32"), 3)), validate=True)
    assert "sort_tile" in plan, plan


def test_sort_of_unsupported_width_is_a_compile_error():
    b = Builder()
    vs = [b.arg((4, 2000), "i64") for _ in range(5)]
    with pytest.raises(Exception, match="36 bytes"):
        b200.compile_to_plan(b.module(b.sort(vs, 1)))


GPU_SORT = [((16,), 0, "f32", 1), ((4, 8), 0, "f32", 1), ((4, 8), 1, "f32", 1), ((2, 4, 8), 1, "f32", 1), ((2, 4, 8), 2, "bf16", 1),
            ((3, 1000), 1, "f32", 1), ((37, 5, 3), 0, "i32", 1), ((7, 1024), 1, "f32", 1), ((2, 1025), 1, "f32", 1),
            ((3, 5000), 1, "f32", 2), ((5000, 3), 0, "f32", 1), ((2, 70001), 1, "i32", 1), ((1, 1 << 20), 1, "f32", 1),
            ((300, 33), 1, "ui8", 1), ((0, 5), 1, "f32", 1)]


@pytest.mark.gpu
@pytest.mark.parametrize("shape,dim,dt,keys", GPU_SORT)
@pytest.mark.parametrize("descending", [False, True])
def test_sort_on_the_gpu(client, shape, dim, dt, keys, descending):
    """Keys with many ties and a position operand riding along: the result is the one stable order, bit for bit."""
    from util import run_gpu
    rng = np.random.default_rng(5)
    if dt in ("f32", "bf16"):
        x = _x(shape, 6, ties=True)
        if x.size > 4:
            x.reshape(-1)[[1, 3]] = [np.nan, -0.0]
    elif dt == "ui8":
        x = rng.integers(0, 256, shape).astype(np.uint8)
    else:
        x = rng.integers(-50, 50, shape).astype(np.int32)
    y = rng.integers(0, 3, shape).astype(np.int32)
    tag = np.arange(x.size, dtype=np.int32).reshape(shape)
    b = Builder()
    vs = [b.arg(shape, dt), b.arg(shape, "i32"), b.arg(shape, "i32")]
    text = b.module(b.sort(vs, dim, descending=descending, num_keys=keys))
    got, _ = run_gpu(client, text, [x, y, tag], dtypes=[dt, "i32", "i32"])
    want = interp.run_text(text, [x, y, tag])
    for g, w in zip(got[1:], want[1:]):
        np.testing.assert_array_equal(g, w)
    np.testing.assert_array_equal(np.asarray(got[0], np.float64) if dt == "bf16" else got[0], np.asarray(want[0], np.float64) if dt == "bf16" else want[0])


@pytest.mark.gpu
def test_sort_with_a_comparator_of_its_own(client):
    """The comparator region is compiled as written: here by absolute value, descending, through arithmetic ops."""
    from util import run_gpu
    x = _x((4, 300), 7)
    b = Builder()
    xv = b.arg(x.shape, "f32")
    text = b.module(b.sort([xv], 1, comparator=lambda s, a, c: s.compare(s.mul(a, a), s.mul(c, c), "GT")))
    got, _ = run_gpu(client, text, [x])
    want = interp.run_text(text, [x])
    np.testing.assert_array_equal(got[0], want[0])
    assert np.all(np.diff(np.abs(got[0]), axis=1) <= 0)


@pytest.mark.gpu
@pytest.mark.parametrize("shape,k", TOP_K_CASES + [((3, 50000), 64)])
def test_top_k_on_the_gpu(client, shape, k):
    from util import run_gpu
    x = _x(shape, 8, ties=True)
    b = Builder()
    text = b.module(b.top_k(b.arg(shape, "f32"), k))
    got, _ = run_gpu(client, text, [x])
    want = interp.run_text(text, [x])
    np.testing.assert_array_equal(got[0], want[0])
    np.testing.assert_array_equal(got[1], want[1])
