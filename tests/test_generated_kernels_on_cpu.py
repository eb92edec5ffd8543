"""The plan compiler's generated CUDA kernels, executed on the CPU: the emitted source is compiled with g++ against a
shim of the CUDA execution model (tests/cuda_emu: a host thread per CUDA thread, block and warp barriers, shuffles,
shared memory) and run step by step over NumPy buffers, then compared with the interpreter under oracle/. This holds
the generated code itself, not only its plan, to the oracle without a GPU: index arithmetic, wide accesses, warp and
block reductions, the row chains, window operations, the merge sort, Philox, the factorizations and the split-position
attention kernel with its last-block combine. Hand-written kernels (contractions, transposes, the built-in scatter)
are outside its reach and stay with the GPU tests."""
import shutil

import numpy as np
import pytest

if shutil.which("g++") is None:
    pytest.skip("needs g++ to build the generated kernels for the host", allow_module_level=True)

from b200.shlo import programs
from b200.shlo.builder import Builder
from cuda_emu import Unsupported, run_plan_on_cpu
from oracle import interp

rng = np.random.default_rng(3)


def f32(*shape):
    return rng.standard_normal(shape).astype(np.float32)


def _check(text, inputs, rtol=1e-5, atol=1e-5):
    got = run_plan_on_cpu(text, inputs)
    want = interp.run_text(text, inputs)
    assert len(got) == len(want)
    for g, w in zip(got, want):
        w = np.asarray(w)
        assert g.shape == w.shape
        if g.dtype.kind in "iub":
            np.testing.assert_array_equal(g, w.astype(g.dtype))
        else:
            np.testing.assert_allclose(g.astype(np.float64), w.astype(np.float64), rtol=rtol, atol=atol, equal_nan=True)
    return got


def test_pointwise_fusions_scalar_and_wide():
    for shape, dt, tol in [((33, 65), "f32", 1e-5), ((64, 256), "f32", 1e-5), ((64, 256), "bf16", 2e-2)]:
        b = Builder()
        x, y, s = b.arg(shape, dt), b.arg(shape, dt), b.arg((shape[1],), dt)
        z = b.max(b.add(b.mul(x, b.broadcast_in_dim(s, shape, (1,))), b.tanh(y)), b.full(shape, 0.0, dt))
        _check(b.module([z, b.select(b.compare(x, y, "LT"), x, y)]), [f32(*shape), f32(*shape), f32(shape[1])], rtol=tol, atol=tol)


def test_integer_kernels_are_exact():
    b = Builder()
    x, y = b.arg((1000,), "i32"), b.arg((1000,), "i32")
    outs = [b.add(x, y), b.mul(x, y), b.div(x, y), b.rem(x, y), b.shl(x, y), b.shr_arith(x, y), b.popcnt(x), b.clz(x)]
    a0 = rng.integers(-2**31, 2**31 - 1, 1000).astype(np.int32)
    a1 = rng.integers(-40, 40, 1000).astype(np.int32)
    _check(b.module(outs), [a0, a1])


def test_reductions_rows_columns_and_argmax():
    b = Builder()
    x = b.arg((300, 70), "f32")
    _check(b.module([b.reduce_sum(x, [1]), b.reduce_max(x, [0]), b.reduce_sum(b.mul(x, x), [0, 1]), b.argmax(x, 1)]), [f32(300, 70)],
           rtol=1e-5, atol=1e-4)
    b = Builder()
    x = b.arg((4096, 128), "f32")                                       # the four-columns-per-thread form with its second pass
    _check(b.module([b.reduce_sum(x, [0]), b.reduce_sum(b.mul(x, x), [0])]), [f32(4096, 128)], rtol=1e-5, atol=2e-3)


@pytest.mark.parametrize("rows,n", [(40, 100), (3, 1500), (70, 32)])
def test_softmax_row_chain(rows, n):
    b = Builder()
    x = b.arg((rows, n), "f32")
    m = b.reduce_max(x, (1,))
    e = b.exp(b.sub(x, b.broadcast_in_dim(m, x.shape, (0,))))
    p = b.div(e, b.broadcast_in_dim(b.reduce_sum(e, (1,)), x.shape, (0,)))
    _check(b.module([p]), [f32(rows, n)], rtol=1e-5, atol=1e-6)


def test_window_operations():
    b = Builder()
    x = b.arg((2, 9, 10, 3), "f32")
    win, st, pad = (1, 3, 3, 1), (1, 2, 2, 1), ((0, 0), (1, 1), (1, 1), (0, 0))
    fwd = b.reduce_window(x, -np.inf, "maximum", win, st, pad)
    src = b.arg(fwd.shape, "f32")
    bwd = b.select_and_scatter(x, src, 0.0, win, st, pad, select="GE")
    cum = b.reduce_window(b.reshape(x, (18, 30)), 0.0, "add", (1, 30), (1, 1), ((0, 0), (29, 0)))
    xv = np.round(f32(2, 9, 10, 3) * 2) / 2
    _check(b.module([fwd, bwd, cum]), [xv, f32(*fwd.shape)], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("shape,dim,desc", [((5, 700), 1, False), ((3, 3000), 1, True), ((1500, 3), 0, False)])
def test_sort_and_top_k(shape, dim, desc):
    keys = (np.round(f32(*shape) * 2) / 2 + 0.0).astype(np.float32)
    tag = np.arange(keys.size, dtype=np.int32).reshape(shape)
    b = Builder()
    _check(b.module(b.sort([b.arg(shape, "f32"), b.arg(shape, "i32")], dim, descending=desc)), [keys, tag])
    if dim == 1:
        b = Builder()
        _check(b.module(b.top_k(b.arg(shape, "f32"), 7)), [keys])


def test_random_bits_and_factorizations():
    b = Builder()
    _check(b.module(b.rng_bit_generator(b.arg((2,), "ui64"), (1000, 3), "ui16")), [np.array([5, (1 << 64) - 2], np.uint64)])
    m = rng.standard_normal((3, 6, 6))
    a = (m @ np.swapaxes(m, 1, 2) + 6 * np.eye(6)).astype(np.float32)
    b = Builder()
    av = b.arg(a.shape, "f32")
    l = b.cholesky(av)
    x = b.triangular_solve(l, b.arg((3, 6, 2), "f32"), transpose_a="TRANSPOSE")
    y = b.triangular_solve(l, b.arg((3, 4, 6), "f32"), left_side=False)
    _check(b.module([l, x, y]), [a, f32(3, 6, 2), f32(3, 4, 6)], rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("G,M,T,D,N,upto", [(None, 8, 100, 64, 64, 70), (2, 3, 24, 64, 32, 11), (None, 4, 70, 128, 64, 3)])
def test_decode_attention_kernel(G, M, T, D, N, upto):
    """Several chunks with the last block's combine, one chunk, and chunks that the mask empties."""
    text = programs.decode_attention(G, M, T, D, N)
    lead = () if G is None else (G,)
    args = [f32(*lead, M, D), f32(*lead, T, D), f32(*lead, T, N), np.array(upto, np.int32)]
    _check(text, args, rtol=2e-2, atol=2e-2)


def test_plans_with_hand_written_steps_are_reported():
    b = Builder()
    x, w = b.arg((64, 64), "f32"), b.arg((64, 64), "f32")
    with pytest.raises(Unsupported):
        run_plan_on_cpu(b.module([b.matmul(x, w)]), [f32(64, 64), f32(64, 64)])


@pytest.mark.parametrize("rows,n,dt,tol", [(48, 96, "f32", 2e-4), (5, 1536, "f32", 2e-4), (64, 256, "bf16", 4e-2)])
def test_layer_norm_forward_and_backward_row_chains(rows, n, dt, tol):
    """LayerNorm with its gradient (reductions and pointwise stages that share rows fuse into row kernels: a warp per
    row for short rows, a block per row for long ones, 16-byte accesses for bf16), next to the column reductions of
    the scale and shift gradients."""
    b = Builder()
    x, gamma, beta, w = b.arg((rows, n), dt), b.arg((n,), dt), b.arg((n,), dt), b.arg((rows, n), dt)
    xf = b.convert(x, "f32") if dt != "f32" else x
    mu = b.mean(xf, (1,))
    xc = b.sub(xf, b.bcast(mu, xf.shape, (0,)))
    var = b.mean(b.mul(xc, xc), (1,))
    inv = b.rsqrt(b.add(var, b.full(var.shape, 1e-5, "f32")))
    y = b.mul(xc, b.bcast(inv, xf.shape, (0,)))
    gf = b.convert(gamma, "f32") if dt != "f32" else gamma
    bf = b.convert(beta, "f32") if dt != "f32" else beta
    y = b.add(b.mul(y, b.bcast(gf, xf.shape, (1,))), b.bcast(bf, xf.shape, (1,)))
    yo = b.convert(y, dt) if dt != "f32" else y
    wf = b.convert(w, "f32") if dt != "f32" else w
    loss = b.reduce_sum(b.mul(b.convert(yo, "f32") if dt != "f32" else yo, wf), (0, 1))
    grads = b.grad(loss, [x, gamma, beta])
    import b200
    assert "row_" in b200.compile_to_plan(b.module([yo, loss] + list(grads)))[0]
    _check(b.module([yo, loss] + list(grads)), [f32(rows, n), 1 + 0.1 * f32(n), 0.1 * f32(n), f32(rows, n)], rtol=tol, atol=tol * 5)


def test_indexing_operations_inside_fused_kernels():
    """transpose, reverse, strided slice, pad with negative-free interior padding, concatenate, broadcast of a reduction,
    row gather, and dynamic_slice / dynamic_update_slice whose start is clamped into range."""
    b = Builder()
    x = b.arg((7, 9, 5), "f32")
    outs = [b.transpose(x, (2, 0, 1)), b.reverse(x, [1]), b.slice(x, (1, 2, 0), (6, 9, 5), (2, 3, 1)),
            b.pad(x, b.const(1.5, "f32"), [1, 0, 2], [0, 3, 1], [1, 0, 2]), b.concatenate([x, x], 1),
            b.bcast(b.reduce_sum(x, (1,)), x.shape, (0, 2))]
    _check(b.module(outs), [f32(7, 9, 5)])
    b = Builder()
    t, i = b.arg((50, 12), "f32"), b.arg((33,), "i32")
    _check(b.module([b.take_rows(t, i)]), [f32(50, 12), rng.integers(0, 50, 33).astype(np.int32)])
    b = Builder()
    x, s = b.arg((5000,), "f32"), b.arg((), "i32")
    _check(b.module([b.dynamic_slice(x, [s], (100,)), b.dynamic_update_slice(x, b.full((7,), 2.0, "f32"), [s])]),
           [f32(5000), np.array(4950, np.int32)])


@pytest.mark.parametrize("dt", ["i8", "ui8", "i16", "i64", "ui32", "f64"])
def test_arithmetic_in_every_element_type(dt):
    from b200.shlo.builder import _NP
    b = Builder()
    x, y = b.arg((999,), dt), b.arg((999,), dt)
    if dt == "f64":
        a0, a1 = rng.standard_normal(999), rng.standard_normal(999)
    else:
        info = np.iinfo(_NP[dt])
        a0 = rng.integers(info.min, info.max, 999).astype(_NP[dt])
        a1 = rng.integers(max(info.min, -50), min(info.max, 50), 999).astype(_NP[dt])
    _check(b.module([b.add(x, y), b.mul(x, y), b.div(x, y), b.max(x, y), b.convert(x, "f32")]), [a0, a1], rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("rows,n", [(1, 1), (3, 31), (65, 33), (3, 129), (1, 1025), (3, 5000)])
def test_softmax_rows_around_the_warp_and_block_sizes(rows, n):
    b = Builder()
    x = b.arg((rows, n), "f32")
    m = b.reduce_max(x, (1,))
    e = b.exp(b.sub(x, b.broadcast_in_dim(m, x.shape, (0,))))
    p = b.div(e, b.broadcast_in_dim(b.reduce_sum(e, (1,)), x.shape, (0,)))
    _check(b.module([p]), [f32(rows, n)], rtol=1e-5, atol=1e-6)


def _random_fusion_graph(seed):
    """A random graph of pointwise operations, row / column broadcasts and reductions over one [R, C] shape: what the
    fusion, sibling-reduction and row-chain logic has to cut into kernels."""
    r = np.random.default_rng(seed)
    R = int(r.choice([1, 2, 3, 7, 16, 31, 33, 64, 70, 130, 300, 1100]))
    C = int(r.choice([1, 2, 5, 8, 31, 32, 33, 64, 100, 128, 257, 1030]))
    if R * C > 40000:
        C = max(1, 40000 // R)
    b = Builder()
    full = [b.arg((R, C), "f32"), b.arg((R, C), "f32")]
    rows, cols = [b.arg((C,), "f32")], [b.arg((R,), "f32")]
    inputs = [r.standard_normal((R, C)).astype(np.float32), r.standard_normal((R, C)).astype(np.float32),
              r.standard_normal((C,)).astype(np.float32), r.standard_normal((R,)).astype(np.float32)]
    for _ in range(int(r.integers(3, 14))):
        k = int(r.integers(0, 12))
        x, y = full[int(r.integers(0, len(full)))], full[int(r.integers(0, len(full)))]
        if k == 0: full.append(b.tanh(b.add(x, y)))
        elif k == 1: full.append(b.mul(x, b.tanh(y)))
        elif k == 2: full.append(b.max(x, b.neg(y)))
        elif k == 3: full.append(b.add(x, b.bcast(rows[int(r.integers(0, len(rows)))], (R, C), (1,))))
        elif k == 4: full.append(b.mul(x, b.bcast(cols[int(r.integers(0, len(cols)))], (R, C), (0,))))
        elif k == 5: rows.append(b.tanh(b.reduce_sum(x, (0,))))
        elif k == 6: cols.append(b.tanh(b.reduce_sum(x, (1,))))
        elif k == 7: cols.append(b.reduce_max(x, (1,)))
        elif k == 8: full.append(b.select(b.compare(x, y, "GT"), x, b.exp(b.neg(b.abs(y)))))
        elif k == 9: full.append(b.sub(x, b.bcast(b.mean(x, (1,)), (R, C), (0,))))
        elif k == 10: full.append(b.tanh(b.div(x, b.add(b.abs(y), b.full((R, C), 1.0, "f32")))))
        else: full.append(b.add(x, b.tanh(b.bcast(b.reduce_sum(b.mul(x, y), (0, 1)), (R, C)))))
    pool = full[2:] + rows[1:] + cols[1:]
    outs = [pool[int(i)] for i in r.choice(len(pool), size=min(len(pool), int(r.integers(1, 4))), replace=False)]
    return b.module(outs), inputs


@pytest.mark.parametrize("seed", [0, 3, 17, 41, 77, 102, 150, 211])
def test_random_fusion_graphs(seed):
    """Seeds from a sweep of 220 such graphs (all of which agreed with the interpreter)."""
    text, inputs = _random_fusion_graph(seed)
    got = run_plan_on_cpu(text, inputs)
    want = interp.run_text(text, inputs)
    for g, w in zip(got, want):
        w = np.asarray(w, np.float64)
        np.testing.assert_allclose(g.astype(np.float64), w, rtol=2e-4, atol=2e-4 * max(1.0, float(np.max(np.abs(w))) if w.size else 1.0))


@pytest.mark.parametrize("seed", [2, 5, 9, 23, 38, 47])
def test_random_window_geometries(seed):
    """reduce_window with random windows, strides, paddings (negative too) and both dilations, and select_and_scatter
    where it applies; seeds from a sweep of 60 geometries."""
    r = np.random.default_rng(seed)
    rank = int(r.integers(1, 5))
    shape = tuple(int(r.integers(1, 9)) for _ in range(rank))
    win = tuple(int(r.integers(1, min(4, s + 1) + 1)) for s in shape)
    st = tuple(int(r.integers(1, 4)) for _ in range(rank))
    pad = tuple((int(r.integers(-1, 3)), int(r.integers(-1, 3))) for _ in range(rank))
    bd = tuple(int(r.integers(1, 3)) for _ in range(rank))
    wd = tuple(int(r.integers(1, 3)) for _ in range(rank))
    op, init = [("add", 0.0), ("maximum", -np.inf), ("minimum", np.inf), ("multiply", 1.0)][int(r.integers(0, 4))]
    x = (np.round(r.standard_normal(shape) * 4) / 4).astype(np.float32)
    b = Builder()
    xv = b.arg(shape, "f32")
    y = b.reduce_window(xv, init, op, win, st, pad, bd, wd)
    if any(d <= 0 for d in y.shape):
        pytest.skip("empty result")
    outs, inputs = [y], [x]
    if all(d == 1 for d in bd + wd) and all(p[0] >= 0 and p[1] >= 0 for p in pad):
        src = b.arg(y.shape, "f32")
        outs.append(b.select_and_scatter(xv, src, 0.0, win, st, pad, select=["GE", "GT", "LE"][int(r.integers(0, 3))]))
        inputs.append(r.standard_normal(y.shape).astype(np.float32))
    _check(b.module(outs), inputs)


def test_threefry_bits_are_exact():
    """The 20 rounds of Threefry-2x32 as one generated integer kernel: word for word what the interpreter gives (which
    tests/test_threefry.py holds to the published known answers)."""
    p = programs.threefry_bits(4096)
    args = [np.array([0x13198a2e, 0x03707344], np.uint32)]
    got, want = run_plan_on_cpu(p.text, args), interp.run_text(p.text, args)
    assert len(got) == len(want) == 1
    np.testing.assert_array_equal(got[0], want[0])


GENERAL_SCATTERS = [
    ((9, 7), (20, 2), (20,), dict(update_window_dims=(), inserted_window_dims=(0, 1), scatter_dims_to_operand_dims=(0, 1), index_vector_dim=1)),
    ((9, 7), (12, 2), (12, 1, 3), dict(update_window_dims=(1, 2), inserted_window_dims=(), scatter_dims_to_operand_dims=(0, 1), index_vector_dim=1)),
    ((6, 5, 8), (4, 10, 2), (4, 10, 5), dict(update_window_dims=(2,), inserted_window_dims=(0, 2), scatter_dims_to_operand_dims=(0, 2), index_vector_dim=2)),
    ((4, 6, 5), (4, 7, 1), (4, 7, 5), dict(update_window_dims=(2,), inserted_window_dims=(1,), scatter_dims_to_operand_dims=(1,), index_vector_dim=2,
                                           input_batching_dims=(0,), scatter_indices_batching_dims=(0,))),
    ((30,), (1,), (4,), dict(update_window_dims=(0,), inserted_window_dims=(), scatter_dims_to_operand_dims=(0,), index_vector_dim=0)),
]


@pytest.mark.parametrize("os_,is_,us_,dn", GENERAL_SCATTERS)
def test_general_scatter_key_and_apply_kernels(os_, is_, us_, dn):
    """The generated halves of a general scatter: the kernel that maps every update element to its destination (point
    updates, partial windows, batching dimensions, windows that do not fit) and, for update computations of their own,
    the kernel that folds each run of equal destinations in update order. The radix sort between them is hand-written
    CUDA and is restated by the harness."""
    sdo, ivd = dn["scatter_dims_to_operand_dims"], dn["index_vector_dim"]
    comps = is_[ivd] if ivd < len(is_) else 1
    idx = np.zeros(is_, np.int32)
    for k in range(comps):
        col = rng.integers(-1, os_[sdo[k]] + 1, [n for d, n in enumerate(is_) if d != ivd] if ivd < len(is_) else is_)   # some out of range
        if ivd < len(is_):
            np.moveaxis(idx, ivd, -1)[..., k] = col
        else:
            idx[...] = col
    for op, dt in [("add", "i32"), ("maximum", "f32"), (lambda s, a, u: s.add(s.mul(a, s.const(0.5, "f32")), u), "f32"), ("subtract", "i32")]:
        b = Builder()
        text = b.module([b.scatter(b.arg(os_, dt), b.arg(is_, "i32"), b.arg(us_, dt), op, **dn)])
        if dt == "i32":
            args = [rng.integers(-9, 9, os_).astype(np.int32), idx, rng.integers(-9, 9, us_).astype(np.int32)]
        else:
            args = [f32(*os_), idx, f32(*us_)]
        _check(text, args)


def _random_indexing_graph(seed):
    """A chain of transposes, reversals, strided slices, pads (negative too), concatenations, reshapes, broadcast
    reductions, row gathers, clamped dynamic slices and selects over a random shape and element type."""
    r = np.random.default_rng(seed)
    dt = str(r.choice(["f32", "f32", "bf16", "i32"]))
    shape = tuple(int(v) for v in r.integers(1, 12, int(r.integers(2, 5))))
    b = Builder()
    vals = [b.arg(shape, dt)]
    inputs = [r.integers(-20, 20, shape).astype(np.int32) if dt == "i32" else (np.round(r.standard_normal(shape) * 8) / 8).astype(np.float32)]
    for _ in range(int(r.integers(2, 9))):
        x = vals[int(r.integers(0, len(vals)))]
        k, rank = int(r.integers(0, 11)), x.ndim
        if k == 0:
            vals.append(b.transpose(x, tuple(int(v) for v in r.permutation(rank))))
        elif k == 1:
            dims = [int(d) for d in range(rank) if r.random() < 0.5]
            vals.append(b.reverse(x, dims) if dims else x)
        elif k == 2:
            lo = [int(r.integers(0, s)) for s in x.shape]
            hi = [int(r.integers(l + 1, s + 1)) for l, s in zip(lo, x.shape)]
            vals.append(b.slice(x, lo, hi, [int(r.integers(1, 3)) for _ in x.shape]))
        elif k == 3:
            lo, hi = [int(r.integers(-1, 3)) for _ in x.shape], [int(r.integers(-1, 3)) for _ in x.shape]
            it = [int(r.integers(0, 2)) for _ in x.shape]
            if all(max(0, (s - 1) * (i + 1) + 1 + l + h) > 0 for s, l, h, i in zip(x.shape, lo, hi, it)):
                vals.append(b.pad(x, b.const(3 if dt == "i32" else 0.5, dt), lo, hi, it))
        elif k == 4:
            vals.append(b.concatenate([x, x], int(r.integers(0, rank))))
        elif k == 5:
            n = int(np.prod(x.shape))
            f = int(r.choice([f for f in range(1, n + 1) if n % f == 0]))
            vals.append(b.reshape(x, (f, n // f)))
        elif k == 6 and rank >= 2:
            d = int(r.integers(0, rank))
            red = b.reduce_sum(x, (d,)) if dt != "bf16" else b.reduce_max(x, (d,))
            vals.append(b.bcast(red, x.shape, tuple(i for i in range(rank) if i != d)))
        elif k == 7:
            vals.append(b.add(x, x) if dt == "i32" else b.mul(x, b.full(x.shape, 0.5, dt)))
        elif k == 8 and x.shape[0] > 1:
            idx = b.arg((5,), "i32")
            inputs.append(r.integers(0, x.shape[0], 5).astype(np.int32))
            vals.append(b.take_rows(b.reshape(x, (x.shape[0], int(np.prod(x.shape[1:])))), idx))
        elif k == 9:
            s = b.arg((), "i32")
            inputs.append(np.array(int(r.integers(-2, x.shape[0] + 2)), np.int32))
            vals.append(b.dynamic_slice(x, [s] + [b.const(0, "i32")] * (rank - 1), (max(1, x.shape[0] // 2),) + tuple(x.shape[1:])))
        elif k == 10:
            vals.append(b.select(b.compare(x, b.reverse(x, [rank - 1]), "LT"), x, b.neg(x)))
    return b.module(vals[1:][-3:]), inputs, dt


@pytest.mark.parametrize("seed", [6, 31, 103, 106, 240, 377])
def test_random_indexing_graphs(seed):
    """Seeds from a sweep of 520 such graphs (all of which agreed with the interpreter)."""
    text, inputs, dt = _random_indexing_graph(seed)
    tol = 2e-2 if dt == "bf16" else 1e-5
    _check(text, inputs, rtol=tol, atol=tol)


def _random_gather_or_scatter(seed, scatter):
    """stablehlo.gather / stablehlo.scatter with random dimension numbers: every operand dimension is collapsed
    (inserted), a window or a batching dimension; a random subset of the others is indexed, in random order; the index
    vector sits at a random position; window positions in the result (updates) are random; indices reach out of range."""
    from b200.shlo.builder import _i64arr
    r = np.random.default_rng(seed)
    R = int(r.integers(1, 5))
    oshape = [int(r.integers(1, 7)) for _ in range(R)]
    cat = [str(r.choice(["collapsed", "window", "window", "batch"])) for _ in range(R)]
    batch_dims = [d for d in range(R) if cat[d] == "batch"]
    collapsed = [d for d in range(R) if cat[d] == "collapsed"]
    window = [d for d in range(R) if cat[d] == "window"]
    sizes = [1 if cat[d] != "window" else int(r.integers(1, oshape[d] + 1)) for d in range(R)]
    sim = [d for d in range(R) if cat[d] != "batch" and r.random() < 0.7]
    r.shuffle(sim)
    sim = [int(d) for d in sim]
    if not sim:
        return None
    extra = [int(r.integers(1, 5)) for _ in range(int(r.integers(0, 3)))]
    bshape = [oshape[d] for d in batch_dims] + extra
    order = list(r.permutation(len(bshape)))
    bshape_p = [bshape[i] for i in order]
    ivd = int(r.integers(0, len(bshape_p) + 1))
    ishape = bshape_p[:ivd] + [len(sim)] + bshape_p[ivd:]
    sib = [order.index(q) if order.index(q) < ivd else order.index(q) + 1 for q in range(len(batch_dims))]
    rank = len(bshape_p) + len(window)
    wpos = sorted(int(v) for v in r.choice(rank, size=len(window), replace=False)) if window else []
    shape, bi, wi = [], 0, 0
    for p in range(rank):
        if p in wpos:
            shape.append(sizes[window[wi]]); wi += 1
        else:
            shape.append(bshape_p[bi]); bi += 1
    ids = np.zeros(ishape, np.int32)
    for c, d in enumerate(sim):
        np.moveaxis(ids, ivd, -1)[..., c] = r.integers(-2, oshape[d] + 2, [s for k, s in enumerate(ishape) if k != ivd])
    b = Builder()
    if not scatter:
        dn = f"#stablehlo.gather<offset_dims = {wpos}, collapsed_slice_dims = {collapsed}, "
        if batch_dims:
            dn += f"operand_batching_dims = {batch_dims}, start_indices_batching_dims = {sib}, "
        dn += f"start_index_map = {sim}, index_vector_dim = {ivd}>"
        x, idx = b.arg(tuple(oshape), "f32"), b.arg(tuple(ishape), "i32")
        (y,) = b.emit("stablehlo.gather", [x, idx], [(tuple(shape), "f32")],
                      props={"dimension_numbers": dn, "indices_are_sorted": "false", "slice_sizes": _i64arr(sizes)})
        return b.module([b.add(y, y)]), [r.standard_normal(oshape).astype(np.float32), ids]
    dn = dict(update_window_dims=tuple(wpos), inserted_window_dims=tuple(collapsed), scatter_dims_to_operand_dims=tuple(sim), index_vector_dim=ivd)
    if batch_dims:
        dn.update(input_batching_dims=tuple(batch_dims), scatter_indices_batching_dims=tuple(sib))
    body = lambda s, a, u: s.add(s.mul(a, s.const(0.5, "f32")), u)              # depends on the order of duplicates
    text = b.module([b.scatter(b.arg(tuple(oshape), "f32"), b.arg(tuple(ishape), "i32"), b.arg(tuple(shape), "f32"), body, **dn)])
    return text, [r.standard_normal(oshape).astype(np.float32), ids, r.standard_normal(shape).astype(np.float32)]


@pytest.mark.parametrize("seed", [0, 7, 13, 29, 58, 77])
@pytest.mark.parametrize("scatter", [False, True])
def test_random_gather_and_scatter_dimension_numbers(seed, scatter):
    """Seeds from sweeps of 300 gathers and 150 scatters (all of which agreed with the interpreter)."""
    made = _random_gather_or_scatter(seed, scatter)
    if made is None:
        pytest.skip("nothing indexed")
    try:
        _check(*made)
    except Unsupported:
        pytest.skip("row form: hand-written kernels")
