"""Generates tests/golden/known_answers_more_ops.json: sort, top_k, rng_bit_generator, cholesky, triangular_solve
and scatter with an update computation of its own, with the results a brute-force evaluation gives. Run from the repo
root:

    python tests/golden/make_known_answers_more_ops.py

The expected values come from the plain-Python loops in this file (an insertion sort, Cholesky-Banachiewicz,
forward / backward substitution, Philox-4x32-10 on Python integers, a sequential scatter), written from the operation
definitions alone: no NumPy sorting or linear algebra, no use of the interpreter under oracle/ or of the plugin. The
reference's handlers for these operations: src/pjrt_plugin/ops/sort_fft_complex.cc:41-250,
src/pjrt_plugin/ops/control_flow.cc:2301-2362, src/pjrt_plugin/ops/linalg.cc:553-660,
src/pjrt_plugin/ops/gather_scatter.cc:79-120; its cases: tests/configs/sort.py, tests/configs/linalg.py:150-320,
tests/configs/slice.py:500-535, tests/test_ops.py:337-363.
"""
import json
import math
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "jax-mps_b200"))
HERE = Path(__file__).resolve().parent

from b200.shlo.builder import Builder  # noqa: E402


def insertion_sort_rows(keys, riders, descending=False):
    """Stable sort of every row of `keys` [R, n] (a list of key arrays compared lexicographically), `riders` moved
    along; returns the permuted arrays. Insertion sort moves an element left only past strictly later elements."""
    def before(a, b):
        for x, y in zip(a, b):
            if x != y:
                return x > y if descending else x < y
        return False
    R, n = keys[0].shape
    outs = [np.array(a) for a in keys + riders]
    for r in range(R):
        order = []
        for i in range(n):
            j = len(order)
            ki = tuple(float(k[r, i]) for k in keys)
            while j > 0 and before(ki, tuple(float(k[r, order[j - 1]]) for k in keys)):
                j -= 1
            order.insert(j, i)
        for a, o in zip(keys + riders, outs):
            for pos, i in enumerate(order):
                o[r, pos] = a[r, i]
    return outs


def cholesky_loops(a):
    n = a.shape[0]
    l = [[0.0] * n for _ in range(n)]
    for i in range(n):
        for j in range(i + 1):
            s = float(a[i, j]) - sum(l[i][k] * l[j][k] for k in range(j))
            l[i][j] = math.sqrt(s) if i == j else s / l[j][j]
    return np.array(l)


def solve_loops(m, b, lower, unit):
    """m x = b for a triangular m [n, n] and b [n, k] by substitution."""
    n, k = b.shape
    x = [[0.0] * k for _ in range(n)]
    rows = range(n) if lower else range(n - 1, -1, -1)
    for c in range(k):
        for i in rows:
            cols = range(i) if lower else range(i + 1, n)
            s = float(b[i, c]) - sum(float(m[i, j]) * x[j][c] for j in cols)
            x[i][c] = s if unit else s / float(m[i, i])
    return np.array(x)


def philox_words(key, counter, blocks):
    """Philox-4x32-10 (Salmon et al., SC 2011) on Python integers: 4 words per counter value."""
    mask = 0xFFFFFFFF
    out = []
    for j in range(blocks):
        c = (counter + j) & ((1 << 128) - 1)
        c0, c1, c2, c3 = c & mask, (c >> 32) & mask, (c >> 64) & mask, (c >> 96) & mask
        k0, k1 = key & mask, (key >> 32) & mask
        for _ in range(10):
            p0, p1 = 0xD2511F53 * c0, 0xCD9E8D57 * c2
            c0, c1, c2, c3 = (p1 >> 32) ^ c1 ^ k0, p1 & mask, (p0 >> 32) ^ c3 ^ k1, p0 & mask
            k0, k1 = (k0 + 0x9E3779B9) & mask, (k1 + 0xBB67AE85) & mask
        out += [c0, c1, c2, c3]
    return out


def main():
    rng = np.random.default_rng(20241126)
    cases = []

    def add(name, text, inputs, expected, rtol=1e-5, atol=1e-5):
        cases.append({"name": name, "mlir": text,
                      "inputs": [{"dtype": str(a.dtype), "shape": list(a.shape), "data": np.asarray(a).reshape(-1).tolist()} for a in inputs],
                      "expected": [{"dtype": str(np.asarray(e).dtype), "shape": list(np.asarray(e).shape),
                                    "data": np.asarray(e).reshape(-1).tolist()} for e in expected],
                      "rtol": rtol, "atol": atol})

    # --- sort: one key with many ties and a rider, both directions; two keys; along the first dimension -----------------
    keys = (np.round(rng.standard_normal((3, 17)) * 2) / 2 + 0.0).astype(np.float32)
    tag = np.arange(keys.size, dtype=np.int32).reshape(keys.shape)
    for desc in (False, True):
        b = Builder()
        text = b.module(b.sort([b.arg(keys.shape, "f32"), b.arg(keys.shape, "i32")], 1, descending=desc))
        add(f"sort_rows_with_rider_{'descending' if desc else 'ascending'}", text, [keys, tag], insertion_sort_rows([keys], [tag], desc))
    k2 = rng.integers(0, 3, keys.shape).astype(np.int32)
    b = Builder()
    text = b.module(b.sort([b.arg(keys.shape, "i32"), b.arg(keys.shape, "f32"), b.arg(keys.shape, "i32")], 1, num_keys=2))
    add("sort_two_keys", text, [k2, keys, tag], insertion_sort_rows([k2, keys], [tag]))
    cols = (np.round(rng.standard_normal((9, 4)) * 2) / 2 + 0.0).astype(np.float32)
    ctag = np.arange(cols.size, dtype=np.int32).reshape(cols.shape)
    b = Builder()
    text = b.module(b.sort([b.arg(cols.shape, "f32"), b.arg(cols.shape, "i32")], 0))
    want = insertion_sort_rows([np.ascontiguousarray(cols.T)], [np.ascontiguousarray(ctag.T)])
    add("sort_along_first_dimension", text, [cols, ctag], [w.T for w in want])

    # --- top_k: the k largest, ties by position ---------------------------------------------------------------------------
    for k in (1, 3, 8):
        x = (np.round(rng.standard_normal((4, 8)) * 2) / 2 + 0.0).astype(np.float32)
        pos = np.broadcast_to(np.arange(8, dtype=np.int32), x.shape).copy()
        vals, idx = insertion_sort_rows([x], [pos], descending=True)
        b = Builder()
        add(f"top_k_{k}_of_8", b.module(b.top_k(b.arg(x.shape, "f32"), k)), [x], [vals[:, :k], idx[:, :k]])

    # --- rng_bit_generator: the Philox stream of the key from the counter on, the counter advanced per 16 bytes -------
    for name, key, ctr, shape, dt in [("zero_state_8_words", 0, 0, (8,), "uint32"), ("key_and_counter_5_bytes", 0x0123456789ABCDEF, 41, (5,), "uint8"),
                                      ("counter_wraps_64_bits", 7, (1 << 64) - 1, (3, 2), "uint64")]:
        n_bytes = int(np.prod(shape)) * np.dtype(dt).itemsize
        blocks = (n_bytes + 15) // 16
        words = philox_words(key, ctr, blocks)
        raw = b"".join(int(w).to_bytes(4, "little") for w in words)[:n_bytes]
        out = np.frombuffer(raw, dtype=dt).reshape(shape)
        state = np.array([key, ctr & ((1 << 64) - 1)], np.uint64)
        new_state = np.array([key, (ctr + blocks) & ((1 << 64) - 1)], np.uint64)
        b = Builder()
        text = b.module(b.rng_bit_generator(b.arg((2,), "ui64"), shape, {"uint32": "ui32", "uint8": "ui8", "uint64": "ui64"}[dt]))
        add(f"rng_bit_generator_{name}", text, [state], [new_state, out])

    # --- cholesky: both triangles, a batch ---------------------------------------------------------------------------------
    for name, lower in (("lower", True), ("upper", False)):
        m = rng.standard_normal((2, 4, 4))
        a = (m @ np.swapaxes(m, 1, 2) + 4 * np.eye(4)).astype(np.float32)
        want = np.stack([cholesky_loops(a[g]) for g in range(2)])
        if not lower:
            want = np.swapaxes(want, 1, 2)
        b = Builder()
        add(f"cholesky_{name}_batch_of_4x4", b.module([b.cholesky(b.arg(a.shape, "f32"), lower)]), [a], [want.astype(np.float32)], rtol=1e-4, atol=1e-5)

    # --- triangular_solve: every combination of side, triangle, transposition on a 4x4 system, and a unit diagonal -------
    for left in (True, False):
        for lower in (True, False):
            for trans in (False, True):
                t = rng.standard_normal((4, 4))
                t = (np.tril(t) if lower else np.triu(t)) * (1 - np.eye(4)) + np.eye(4) * (np.abs(np.diag(t)) + 1.0)
                t = t.astype(np.float32)
                rhs = rng.standard_normal((4, 3) if left else (3, 4)).astype(np.float32)
                m = t.T if trans else t
                m_lower = lower != trans
                if left:
                    want = solve_loops(m, rhs, m_lower, False)
                else:                                                  # x m = b  <=>  m^T x^T = b^T
                    want = solve_loops(m.T, rhs.T, not m_lower, False).T
                b = Builder()
                text = b.module([b.triangular_solve(b.arg(t.shape, "f32"), b.arg(rhs.shape, "f32"), left_side=left, lower=lower,
                                                    transpose_a="TRANSPOSE" if trans else "NO_TRANSPOSE")])
                add(f"triangular_solve_{'left' if left else 'right'}_{'lower' if lower else 'upper'}{'_transposed' if trans else ''}",
                    text, [t, rhs], [want.astype(np.float32)], rtol=1e-4, atol=1e-5)
    t = np.tril(rng.standard_normal((4, 4))).astype(np.float32)        # the diagonal is ignored
    rhs = rng.standard_normal((4, 2)).astype(np.float32)
    b = Builder()
    text = b.module([b.triangular_solve(b.arg(t.shape, "f32"), b.arg(rhs.shape, "f32"), unit_diagonal=True)])
    add("triangular_solve_unit_diagonal", text, [t, rhs], [solve_loops(t, rhs, True, True).astype(np.float32)], rtol=1e-4, atol=1e-5)

    # --- scatter with an update computation of its own, applied to duplicates in update order ------------------------------
    point = dict(update_window_dims=(), inserted_window_dims=(0,), scatter_dims_to_operand_dims=(0,), index_vector_dim=1)
    x = rng.standard_normal(6).astype(np.float32)
    idx = np.array([[0], [2], [4]], np.int32)
    want = x.astype(np.float64).copy()
    for i in idx[:, 0]:
        want[i] = math.sin(want[i])
    b = Builder()
    text = b.module([b.scatter(b.arg((6,), "f32"), b.arg(idx.shape, "i32"), b.arg((3,), "f32"), lambda s, a, u: s.sin(a), **point)])
    add("scatter_apply_sin", text, [x, idx, np.zeros(3, np.float32)], [want.astype(np.float32)])
    idx = np.array([[1], [3], [1], [7], [1], [-1]], np.int32)          # duplicates, two out of range
    upd = rng.standard_normal(6).astype(np.float32)
    want = x.copy()
    for i, u in zip(idx[:, 0], upd):
        if 0 <= i < 6:
            want[i] = np.float32(np.float32(want[i] * np.float32(0.5)) + u)
    b = Builder()
    text = b.module([b.scatter(b.arg((6,), "f32"), b.arg(idx.shape, "i32"), b.arg((6,), "f32"),
                               lambda s, a, u: s.add(s.mul(a, s.const(0.5, "f32")), u), **point)])
    add("scatter_decay_then_add_in_update_order", text, [x, idx, upd], [want])

    body = ",\n".join(json.dumps(c, separators=(",", ":")) for c in cases)                  # one case per line
    (HERE / "known_answers_more_ops.json").write_text('{"cases":[\n' + body + "\n]}\n")
    print(f"{len(cases)} cases written")


if __name__ == "__main__":
    main()
