"""Generates tests/golden/known_answers.json: small StableHLO programs with inputs and the results a brute-force
evaluation gives. Run from the repo root:

    python tests/golden/make_known_answers.py

The expected values come from the nested-loop functions in this file, written from the StableHLO operation
definitions alone: no torch convolution, no use of the interpreter under oracle/ or of the plugin. They pin the corner
rules the reference documents in its handlers and exercises in its own case tables:
  convolution: dilate the input first, then pad (negative padding trims), batch_group_count
      src/pjrt_plugin/ops/linalg.cc:339-362,508-532; cases tests/configs/conv.py:124-223
  dot_general with several free dimensions         tests/configs/matmul.py:129-141
  case with an index outside [0, branches)         src/pjrt_plugin/ops/control_flow.cc:672-675
  a counted loop of 130 iterations                 tests/configs/control_flow.py:426-435
  dynamic_update_slice with clamped start indices  src/pjrt_plugin/ops/slice.cc:167-177
  scatter-add with repeated and out-of-range rows  src/pjrt_plugin/ops/gather_scatter.cc:296-699
  pad with negative and interior padding           src/pjrt_plugin/ops/slice.cc:202-276
"""
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "jax-mps_b200"))
HERE = Path(__file__).resolve().parent

from b200.shlo.builder import Builder  # noqa: E402


def conv_nhwc_brute(x, w, strides=(1, 1), padding=((0, 0), (0, 0)), lhs_dilation=(1, 1), rhs_dilation=(1, 1),
                    feature_group_count=1, batch_group_count=1):
    """x [N,H,W,C], w [KH,KW,C/fg,O] -> [N/bg,OH,OW,O], float64, loops over every output element."""
    x, w = np.asarray(x, np.float64), np.asarray(w, np.float64)
    N, H, W, C = x.shape
    KH, KW, Cg, O = w.shape
    # 1. dilate the input
    Hd, Wd = (H - 1) * lhs_dilation[0] + 1, (W - 1) * lhs_dilation[1] + 1
    xd = np.zeros((N, Hd, Wd, C))
    xd[:, ::lhs_dilation[0], ::lhs_dilation[1], :] = x
    # 2. pad (negative: trim)
    def pad_axis(a, axis, lo, hi):
        if lo < 0:
            a = np.take(a, range(-lo, a.shape[axis]), axis=axis); lo = 0
        if hi < 0:
            a = np.take(a, range(0, a.shape[axis] + hi), axis=axis); hi = 0
        widths = [(0, 0)] * a.ndim
        widths[axis] = (lo, hi)
        return np.pad(a, widths)
    xd = pad_axis(xd, 1, *padding[0])
    xd = pad_axis(xd, 2, *padding[1])
    Hp, Wp = xd.shape[1], xd.shape[2]
    ekh, ekw = (KH - 1) * rhs_dilation[0] + 1, (KW - 1) * rhs_dilation[1] + 1
    OH, OW = (Hp - ekh) // strides[0] + 1, (Wp - ekw) // strides[1] + 1
    G, BG = feature_group_count, batch_group_count
    Nb = N // BG
    out = np.zeros((Nb, OH, OW, O))
    for n in range(Nb):
        for oh in range(OH):
            for ow in range(OW):
                for o in range(O):
                    fg = o // (O // G)                    # feature group of this output channel
                    bg = o // (O // BG)                   # batch group of this output channel
                    acc = 0.0
                    for kh in range(KH):
                        for kw in range(KW):
                            for c in range(Cg):
                                ih, iw = oh * strides[0] + kh * rhs_dilation[0], ow * strides[1] + kw * rhs_dilation[1]
                                acc += xd[bg * Nb + n, ih, iw, fg * Cg + c] * w[kh, kw, c, o]
                    out[n, oh, ow, o] = acc
    return out


def rand(rng, *shape):
    return rng.uniform(-1.0, 1.0, shape).astype(np.float32)


def main():
    rng = np.random.default_rng(20240607)
    cases = []

    def add(name, text, inputs, expected, rtol=1e-5, atol=1e-5):
        cases.append({"name": name, "mlir": text,
                      "inputs": [{"dtype": str(a.dtype), "shape": list(a.shape), "data": np.asarray(a).reshape(-1).tolist()} for a in inputs],
                      "expected": [{"dtype": str(np.asarray(e).dtype), "shape": list(np.asarray(e).shape),
                                    "data": np.asarray(e).reshape(-1).tolist()} for e in expected],
                      "rtol": rtol, "atol": atol})

    # --- convolutions ------------------------------------------------------------------------------------------
    def conv_case(name, xs, ws, **kw):
        b = Builder()
        x, w = b.arg(xs, "f32"), b.arg(ws, "f32")
        bkw = dict(kw)
        bkw["padding"] = kw.get("padding", ((0, 0), (0, 0)))
        y = b.conv(x, w, strides=kw.get("strides", (1, 1)), padding=bkw["padding"], lhs_dilation=kw.get("lhs_dilation", (1, 1)),
                   rhs_dilation=kw.get("rhs_dilation", (1, 1)), feature_group_count=kw.get("feature_group_count", 1),
                   batch_group_count=kw.get("batch_group_count", 1))
        xv, wv = rand(rng, *xs), rand(rng, *ws)
        add(name, b.module([y]), [xv, wv], [conv_nhwc_brute(xv, wv, **kw).astype(np.float32)])
    conv_case("conv_lhs_dilation_negative_padding", (1, 6, 7, 4), (1, 2, 4, 2), padding=((0, -1), (0, 0)), lhs_dilation=(2, 1))
    conv_case("conv_lhs_dilation_only", (1, 6, 7, 4), (1, 2, 4, 2), lhs_dilation=(2, 1))
    conv_case("conv_batch_group_2_lhs_dilation_negative_padding", (2, 6, 7, 4), (1, 2, 4, 2), padding=((0, -1), (0, 0)),
              lhs_dilation=(2, 1), batch_group_count=2)
    conv_case("conv_batch_group_3_two_filters_per_group", (6, 5, 5, 2), (3, 3, 2, 6), padding=((1, 1), (1, 1)), batch_group_count=3)
    conv_case("conv_feature_group_2_stride_2_rhs_dilation", (2, 9, 8, 4), (2, 3, 2, 6), strides=(2, 2), padding=((1, 2), (0, 1)),
              rhs_dilation=(2, 1), feature_group_count=2)
    # NCHW / OIHW with batch groups (tests/configs/conv.py:175-188): expected through the NHWC loops on transposed data
    b = Builder()
    x, w = b.arg((4, 1, 6, 7), "f32"), b.arg((2, 1, 1, 2), "f32")
    y = b.conv(x, w, dn=("bf01", "oi01", "bf01"), batch_group_count=2)
    xv, wv = rand(rng, 4, 1, 6, 7), rand(rng, 2, 1, 1, 2)
    ref = conv_nhwc_brute(xv.transpose(0, 2, 3, 1), wv.transpose(2, 3, 1, 0), batch_group_count=2).transpose(0, 3, 1, 2)
    add("conv_nchw_batch_group_2", b.module([y]), [xv, wv], [ref.astype(np.float32)])

    # --- dot_general with two free dimensions on each side -----------------------------------------------------------
    b = Builder()
    x, y = b.arg((2, 3, 4, 5), "f32"), b.arg((2, 5, 6, 7), "f32")
    z = b.dot_general(x, y, ((3,), (1,)), ((0,), (0,)))
    xv, yv = rand(rng, 2, 3, 4, 5), rand(rng, 2, 5, 6, 7)
    ref = np.zeros((2, 3, 4, 6, 7))
    for bb in range(2):
        for i in range(3):
            for j in range(4):
                for p in range(6):
                    for q in range(7):
                        ref[bb, i, j, p, q] = sum(float(xv[bb, i, j, k]) * float(yv[bb, k, p, q]) for k in range(5))
    add("dot_general_two_free_dims_each_side", b.module([z]), [xv, yv], [ref.astype(np.float32)])

    # --- case: an index outside the branches selects the last one ------------------------------------------------------
    for idx, want in [(-1, 5.0 - 3.0), (100, 5.0 - 3.0), (1, 10.0), (0, 6.0)]:
        b = Builder()
        sel, v = b.arg((), "i32"), b.arg((), "f32")
        (r,) = b.case(sel, [lambda s: [s.add(v, s.const(1.0, "f32"))], lambda s: [s.mul(v, s.const(2.0, "f32"))],
                           lambda s: [s.sub(v, s.const(3.0, "f32"))]], [((), "f32")])
        add(f"case_index_{idx}", b.module([r]), [np.array(idx, np.int32), np.array(5.0, np.float32)], [np.array(want, np.float32)])

    # --- fori_loop(0, 130, val * 0.99 + i * 0.001) -----------------------------------------------------------------
    b = Builder()
    v0 = b.arg((), "f32")
    outs = b.while_([b.const(0, "i32"), v0], lambda s, i, v: s.compare(i, s.const(130, "i32"), "LT"),
                    lambda s, i, v: [s.add(i, s.const(1, "i32")),
                                     s.add(s.mul(v, s.const(0.99, "f32")), s.mul(s.convert(i, "f32"), s.const(0.001, "f32")))])
    val = np.float32(1.0)
    for i in range(130):
        val = np.float32(val * np.float32(0.99) + np.float32(i) * np.float32(0.001))
    add("counted_loop_130_iterations", b.module([outs[1]]), [np.array(1.0, np.float32)], [np.array(val, np.float32)], rtol=1e-5)

    # --- dynamic_update_slice: runtime start indices, clamped to keep the window inside ------------------------------
    for start in [(1, 2), (5, 9), (-3, 0)]:
        b = Builder()
        t, u = b.arg((6, 10), "f32"), b.arg((2, 3), "f32")
        i0, i1 = b.arg((), "i32"), b.arg((), "i32")
        tv, uv = rand(rng, 6, 10), rand(rng, 2, 3)
        ref = tv.copy()
        r0, c0 = min(max(start[0], 0), 6 - 2), min(max(start[1], 0), 10 - 3)
        ref[r0:r0 + 2, c0:c0 + 3] = uv
        add(f"dynamic_update_slice_start_{start[0]}_{start[1]}", b.module([b.dynamic_update_slice(t, u, [i0, i1])]),
            [tv, uv, np.array(start[0], np.int32), np.array(start[1], np.int32)], [ref])

    # --- scatter-add of rows with repeated and out-of-range indices ----------------------------------------------------
    b = Builder()
    t, i, u = b.arg((7, 5), "f32"), b.arg((9,), "i32"), b.arg((9, 5), "f32")
    tv, uv = rand(rng, 7, 5), rand(rng, 9, 5)
    iv = np.array([3, 0, 3, 6, 3, 7, -1, 0, 6], np.int32)       # 7 and -1 are out of range: dropped
    ref = tv.astype(np.float64).copy()
    for k, row in enumerate(iv):
        if 0 <= row < 7:
            ref[row] += uv[k]
    add("scatter_add_rows_with_duplicates", b.module([b.scatter_rows(t, i, u, "add")]), [tv, iv, uv], [ref.astype(np.float32)])

    # --- pad with negative edges and interior padding ----------------------------------------------------------------
    b = Builder()
    x, pv = b.arg((4, 5), "f32"), b.arg((), "f32")
    xv = rand(rng, 4, 5)
    lo, hi, interior = (1, -1), (-1, 2), (1, 2)
    # interior first, then edges
    big = np.full(((4 - 1) * 2 + 1, (5 - 1) * 3 + 1), np.float32(-7.5))
    big[::2, ::3] = xv
    rows = [np.full(big.shape[1], np.float32(-7.5))] * lo[0] + [r for r in big]
    rows = rows[:len(rows) + hi[0]]
    ref = np.array(rows)[:, -lo[1]:]
    ref = np.concatenate([ref, np.full((ref.shape[0], hi[1]), np.float32(-7.5))], 1)
    add("pad_negative_and_interior", b.module([b.pad(x, pv, lo, hi, interior)]), [xv, np.array(-7.5, np.float32)], [ref.astype(np.float32)])

    # --- argmax: the first index wins a tie --------------------------------------------------------------------------
    b = Builder()
    x = b.arg((3, 8), "f32")
    xv = np.array([[1, 5, 5, 2, 5, 0, 0, 0], [7, 1, 7, 7, 0, 0, 0, 0], [-1, -1, -1, -1, -1, -1, -1, -1]], np.float32)
    add("argmax_first_index_on_ties", b.module([b.argmax(x, 1)]), [xv], [np.array([1, 0, 0], np.int32)])

    (HERE / "known_answers.json").write_text(json.dumps({"cases": cases}, indent=0))
    print(f"wrote {len(cases)} cases")


if __name__ == "__main__":
    main()
