"""TEST INFRASTRUCTURE — CPU oracle for the plugin's hot path. Never imported
by the product; only tests, the smoke check and the bench's CPU-baseline leg
use it.

A NumPy (plus torch-CPU for convolution) interpreter of StableHLO modules in
text form. It restates, op by op, the semantics the reference's handlers
implement on top of MLX (file:line below are paths inside the reference
project), which are the StableHLO semantics jaxlib's CPU backend implements —
the backend the reference's own tests compare against
(tests/test_ops.py:108-161, atol = rtol = 1e-5, integers exact).

PARITY PINNING: the reference stores no golden vectors for this path and
cannot run on Linux; jaxlib is not installable here. The interpreter is
pinned against (1) the literal expectations of the reference's raw-MLIR test
(tests/test_ops.py:216-281, arcsin / sinh decompositions vs numpy), (2) the
literal expectations in tests/test_control_flow_compile.py:114-133, and (3)
PyTorch autograd twins of the benchmark models (oracle/twins.py), an
independent implementation of the same mathematics. Everything else is
"parity unpinned" by reference data.

Values are numpy arrays; bf16 is carried as float32 rounded to bf16 after
every op. Floating-point reductions accumulate in float64.
"""
from __future__ import annotations

import math

import numpy as np

from . import mlir_text as mt
from .mlir_text import Block, Module, Op, TType, attr_i64s, attr_int, enum_word, struct_fields

FLOATS = ("f32", "bf16", "f16", "f64")


def round_bf16(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = (u + (0x7FFF + ((u >> 16) & 1))) & np.uint32(0xFFFF0000)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = np.where(nan, u | 0x00400000, r).astype(np.uint32)
    return r.view(np.float32)


def cast(a, dt: str) -> np.ndarray:
    """Round/wrap `a` into element type `dt`."""
    a = np.asarray(a)
    if dt == "bf16":
        return round_bf16(a.astype(np.float32))
    if dt == "token":
        return np.zeros((), np.bool_)
    return a.astype(mt.np_dtype(dt), copy=False)


# --------------------------------------------------------------------------
# elementwise rules
# --------------------------------------------------------------------------

def _bits(dt): return np.dtype(mt.np_dtype(dt)).itemsize * 8


def _int_div(a, b):
    """Truncating integer division (src/pjrt_plugin/ops/arithmetic.cc:492-513);
    division by zero gives -1 / all-ones, INT_MIN / -1 gives INT_MIN, as XLA."""
    with np.errstate(all="ignore"):
        bz = b == 0
        bs = np.where(bz, 1, b)
        if np.issubdtype(a.dtype, np.signedinteger):
            ovf = (a == np.iinfo(a.dtype).min) & (bs == -1)
            bs = np.where(ovf, 1, bs)
            q = np.abs(a.astype(object)) // np.abs(bs.astype(object))
            q = np.where((a < 0) != (bs < 0), -q, q).astype(a.dtype) if a.size else a
            q = np.where(ovf, a, q)
            return np.where(bz, a.dtype.type(-1), q).astype(a.dtype)
        q = a // bs
        return np.where(bz, np.iinfo(a.dtype).max, q).astype(a.dtype)


def _int_rem(a, b):
    """C remainder: sign follows the dividend (arithmetic.cc:45-83); x % 0 = x."""
    with np.errstate(all="ignore"):
        bz = b == 0
        bs = np.where(bz, 1, b)
        if np.issubdtype(a.dtype, np.signedinteger):
            bs = np.where((a == np.iinfo(a.dtype).min) & (bs == -1), 1, bs)
            r = np.fmod(a, bs)
        else:
            r = a % bs
        return np.where(bz, a, r).astype(a.dtype)


def _shift(kind):
    def f(a, b):
        """Out-of-range amounts: logical shifts give 0, arithmetic gives the
        sign fill (src/pjrt_plugin/mlx_executable.cc:272-304, arithmetic.cc:113-144)."""
        nb = a.dtype.itemsize * 8
        bu = b.astype(np.int64) if np.issubdtype(b.dtype, np.signedinteger) else b.astype(np.uint64)
        oor = (bu < 0) | (bu >= nb)
        sh = np.where(oor, 0, bu).astype(a.dtype)
        if kind == "l":
            return np.where(oor, 0, np.left_shift(a, sh)).astype(a.dtype)
        if kind == "rl":
            ua = a.view(np.dtype(f"uint{nb}"))
            return np.where(oor, 0, np.right_shift(ua, sh.view(ua.dtype))).astype(ua.dtype).view(a.dtype)
        sa = a.view(np.dtype(f"int{nb}"))
        fill = np.where(sa < 0, -1, 0).astype(sa.dtype)
        return np.where(oor, fill, np.right_shift(sa, sh.view(sa.dtype))).astype(sa.dtype).view(a.dtype)
    return f


def _sign(a):
    if np.issubdtype(a.dtype, np.floating):
        return np.where(np.isnan(a), a, np.sign(a)).astype(a.dtype)      # NaN propagates (arithmetic.cc:515-531)
    return np.sign(a).astype(a.dtype)


def _round_afz(a):
    return (np.sign(a) * np.floor(np.abs(a) + 0.5)).astype(a.dtype)


def _popcnt(a):
    u = a.view(np.dtype(f"uint{a.dtype.itemsize * 8}"))
    out = np.zeros(a.shape, np.uint64)
    v = u.astype(np.uint64)
    for _ in range(a.dtype.itemsize * 8):
        out += v & 1
        v >>= 1
    return out.astype(a.dtype)


def _clz(a):
    nb = a.dtype.itemsize * 8
    v = a.view(np.dtype(f"uint{nb}")).astype(np.uint64)
    out = np.full(a.shape, nb, np.int64)
    for k in range(nb):
        out = np.where((v >> np.uint64(k)) != 0, nb - 1 - k, out)
    return out.astype(a.dtype)


def _total_order_key(a):
    """Sign-magnitude key giving -NaN < -inf < ... < -0 < +0 < ... < +inf < +NaN
    (arithmetic.cc:236-283)."""
    nb = a.dtype.itemsize * 8
    it = np.dtype(f"int{nb}")
    i = np.ascontiguousarray(a).view(it)
    mask = (i >> (nb - 1)) & it.type((1 << (nb - 1)) - 1)
    return i ^ mask


_UNARY = {
    "exponential": np.exp, "log": np.log, "sqrt": np.sqrt, "rsqrt": lambda a: 1.0 / np.sqrt(a),
    "negate": np.negative, "abs": np.abs, "floor": np.floor, "ceil": np.ceil, "sine": np.sin, "cosine": np.cos,
    "tanh": np.tanh, "tan": np.tan, "logistic": lambda a: 1.0 / (1.0 + np.exp(-a)), "sign": _sign,
    "log_plus_one": np.log1p, "exponential_minus_one": np.expm1, "cbrt": np.cbrt,
    "round_nearest_even": np.rint, "round_nearest_afz": _round_afz, "popcnt": _popcnt,
    "count_leading_zeros": _clz,
    "sinh": np.sinh, "cosh": np.cosh, "asin": np.arcsin, "acos": np.arccos, "atan": np.arctan, "asinh": np.arcsinh,
    "acosh": np.arccosh, "atanh": np.arctanh,
}
_BINARY_F = {
    "add": np.add, "subtract": np.subtract, "multiply": np.multiply, "divide": np.divide,
    "maximum": np.maximum, "minimum": np.minimum, "power": np.power, "remainder": np.fmod, "atan2": np.arctan2,
}
_BINARY_I = {
    "add": np.add, "subtract": np.subtract, "multiply": np.multiply, "divide": _int_div,
    "maximum": np.maximum, "minimum": np.minimum, "remainder": _int_rem,
    "and": np.bitwise_and, "or": np.bitwise_or, "xor": np.bitwise_xor,
    "shift_left": _shift("l"), "shift_right_logical": _shift("rl"), "shift_right_arithmetic": _shift("ra"),
}
_CMP = {"EQ": np.equal, "NE": np.not_equal, "LT": np.less, "LE": np.less_equal, "GT": np.greater,
        "GE": np.greater_equal}


def _int_pow(a, b):
    out = np.ones_like(a)
    base, e = a.copy(), b.astype(np.int64).copy()
    neg = e < 0
    e = np.where(neg, 0, e)
    with np.errstate(all="ignore"):
        while np.any(e > 0):
            out = np.where(e & 1, out * base, out)
            base = base * base
            e >>= 1
    # negative exponent: 1 for base 1, +-1 for base -1, else 0
    negv = np.where(a == 1, 1, np.where(a == -1, np.where(b & 1, -1, 1), 0)).astype(a.dtype)
    return np.where(neg, negv, out).astype(a.dtype)


class Interp:
    def __init__(self, module: Module | str, collective=None, partition_id: int = 0, conv_f64: bool = False,
                 wide: bool = False, gather=None):
        self.m = mt.parse_module(module) if isinstance(module, str) else module
        self.collective = collective          # callable(list[np.ndarray]) -> list (sum over partitions)
        self.gather = gather                  # callable(np.ndarray) -> list of every partition's array, in partition order
        self.partition_id = partition_id
        self.conv_f64 = conv_f64 or wide
        self.wide = wide
        self._vector = 0          # >0 while a combiner region is evaluated on whole arrays

    def cast(self, a, dt: str) -> np.ndarray:
        """Element-type rounding; with `wide` every f32 value is carried in
        float64 (ground truth for ill-conditioned comparisons)."""
        if self.wide and dt == "f32":
            return np.asarray(a).astype(np.float64, copy=False)
        return cast(a, dt)

    # ---- entry ----------------------------------------------------------
    def run(self, args, func: str = "main") -> list:
        f = self.m.funcs[func]
        assert len(args) == len(f.args), (len(args), len(f.args))
        env = {}
        for (n, t), a in zip(f.args, args):
            a = np.asarray(a)
            assert tuple(a.shape) == tuple(t.shape), (n, a.shape, t.shape)
            env[n] = self.cast(a, t.dtype)
        return self.block(f.body, env)

    def block(self, blk: Block, env: dict) -> list:
        for op in blk.ops:
            if op.name in ("func.return", "stablehlo.return"):
                return [env[o] for o in op.operands]
            outs = self.op(op, env)
            for n, t, v in zip(op.results, op.result_types, outs):
                v = np.asarray(v)
                if t.dtype != "token" and not self._vector:
                    assert tuple(v.shape) == tuple(t.shape), (op.name, v.shape, t.shape)
                env[n] = self.cast(v, t.dtype)
        return []

    def region(self, blk: Block, env: dict, args) -> list:
        e = dict(env)
        for (n, t), a in zip(blk.args, args):
            e[n] = a
        return self.block(blk, e)

    # ---- dispatch ----------------------------------------------------------
    def op(self, op: Op, env: dict) -> list:
        name = op.name.split(".", 1)[1] if "." in op.name else op.name
        x = [env[o] for o in op.operands]
        rt = op.result_types[0] if op.result_types else None
        fn = getattr(self, "op_" + name, None)
        if fn is not None:
            return fn(op, x, env)
        if name in _UNARY and len(x) == 1:
            a = x[0]
            with np.errstate(all="ignore"):
                if rt.dtype in FLOATS:
                    w = a.astype(np.float64) if rt.dtype != "f64" else a
                    return [_UNARY[name](w)]
                return [_UNARY[name](a)]
        if name in _BINARY_F or name in _BINARY_I:
            a, b = x
            with np.errstate(all="ignore"):
                if rt.dtype in FLOATS:
                    if rt.dtype == "bf16":
                        return [_BINARY_F[name](a.astype(np.float32), b.astype(np.float32))]
                    return [_BINARY_F[name](a, b)]
                if rt.dtype == "i1":
                    return [{"and": np.logical_and, "or": np.logical_or, "xor": np.logical_xor,
                             "maximum": np.logical_or, "minimum": np.logical_and, "add": np.logical_or,
                             "multiply": np.logical_and}[name](a, b)]
                if name == "power":
                    return [_int_pow(a, b)]
                return [_BINARY_I[name](a, b)]
        raise NotImplementedError(f"oracle: unsupported op {op.name}")

    # ---- elementwise specials -------------------------------------------------
    def op_constant(self, op, x, env):
        return [mt.dense_array(op.attrs["value"])]

    def op_not(self, op, x, env):
        a = x[0]
        return [np.logical_not(a) if a.dtype == np.bool_ else np.invert(a)]     # arithmetic.cc:99-110

    def op_is_finite(self, op, x, env):
        return [np.isfinite(x[0])]

    def op_convert(self, op, x, env):
        a, dt = x[0], op.result_types[0].dtype
        with np.errstate(all="ignore"):
            if dt == "i1":
                return [a != 0]
            if a.dtype.kind == "f" and dt not in FLOATS:
                info = np.iinfo(mt.np_dtype(dt))
                t = np.trunc(np.nan_to_num(a.astype(np.float64), nan=0.0, posinf=float(info.max), neginf=float(info.min)))
                t = np.clip(t, float(info.min), float(info.max))
                out = np.where(t >= float(info.max), info.max, t.astype(np.int64 if info.min < 0 else np.uint64))
                return [out.astype(mt.np_dtype(dt))]
            return [a]

    def op_bitcast_convert(self, op, x, env):
        a, t = x[0], op.result_types[0]
        src = op_operand_dtype(a)
        if t.dtype == "bf16" or src == "bf16":
            raise NotImplementedError("bf16 bitcast")
        out = np.ascontiguousarray(a).view(mt.np_dtype(t.dtype))
        return [out.reshape(t.shape)]

    def op_compare(self, op, x, env):
        a, b = x
        d = enum_word(op.attrs["comparison_direction"])
        ct = enum_word(op.attrs["compare_type"]) if "compare_type" in op.attrs else ""
        if ct == "TOTALORDER" and a.dtype.kind == "f":
            a, b = _total_order_key(a), _total_order_key(b)
        return [_CMP[d](a, b)]

    def op_select(self, op, x, env):
        p, a, b = x
        return [np.where(p, a, b)]

    def op_clamp(self, op, x, env):
        lo, a, hi = x                      # (min, operand, max) order, arithmetic.cc:34-43
        return [np.minimum(np.maximum(a, lo), hi)]

    def op_reduce_precision(self, op, x, env):
        eb, mb = attr_int(op.attrs["exponent_bits"]), attr_int(op.attrs["mantissa_bits"])
        a = x[0].astype(np.float32)
        if eb >= 8 and mb >= 23:
            return [a]
        if eb == 8 and mb == 7:
            return [round_bf16(a)]
        if eb == 5 and mb == 10:
            return [a.astype(np.float16).astype(np.float32)]
        raise NotImplementedError("reduce_precision format")

    def op_erf_inv(self, op, x, env):
        from scipy.special import erfinv
        return [erfinv(x[0].astype(np.float64))]

    def op_erf(self, op, x, env):
        from scipy.special import erf
        return [erf(x[0].astype(np.float64))]

    # ---- shape ops ---------------------------------------------------------------
    def op_broadcast_in_dim(self, op, x, env):
        t = op.result_types[0]
        dims = attr_i64s(op.attrs["broadcast_dimensions"])
        a = x[0]
        shape = [1] * len(t.shape)
        for i, d in enumerate(dims):
            shape[d] = a.shape[i]
        return [np.broadcast_to(a.reshape(shape), t.shape)]

    def op_reshape(self, op, x, env):
        return [np.ascontiguousarray(x[0]).reshape(op.result_types[0].shape)]

    def op_transpose(self, op, x, env):
        return [np.transpose(x[0], attr_i64s(op.attrs["permutation"]))]

    def op_reverse(self, op, x, env):
        return [np.flip(x[0], tuple(attr_i64s(op.attrs["dimensions"])))]

    def op_iota(self, op, x, env):
        t = op.result_types[0]
        d = attr_int(op.attrs["iota_dimension"])
        shape = [1] * len(t.shape)
        shape[d] = t.shape[d]
        return [np.broadcast_to(np.arange(t.shape[d]).reshape(shape), t.shape)]

    def op_concatenate(self, op, x, env):
        return [np.concatenate(x, axis=attr_int(op.attrs["dimension"]))]

    def op_slice(self, op, x, env):
        st, li, sd = (attr_i64s(op.attrs[k]) for k in ("start_indices", "limit_indices", "strides"))
        return [x[0][tuple(slice(s, l, d) for s, l, d in zip(st, li, sd))]]

    def op_pad(self, op, x, env):
        """Interior padding first, then (possibly negative) edges
        (src/pjrt_plugin/ops/slice.cc:14-52,202-276)."""
        a, pv = x
        lo, hi, it = (attr_i64s(op.attrs[k]) for k in ("edge_padding_low", "edge_padding_high", "interior_padding"))
        t = op.result_types[0]
        out = np.full(t.shape, pv, dtype=a.dtype)
        src, dst = [], []
        for d in range(a.ndim):
            n = a.shape[d]
            pos = lo[d] + np.arange(n) * (it[d] + 1)
            ok = (pos >= 0) & (pos < t.shape[d])
            src.append(np.nonzero(ok)[0]); dst.append(pos[ok])
        if all(len(s) for s in src) or a.ndim == 0:
            out[np.ix_(*dst)] = a[np.ix_(*src)]
        return [out]

    def _starts(self, starts, full, size):
        """Clamp each start into [0, dim - size] (slice.cc:80-107)."""
        return [int(min(max(int(s), 0), f - z)) for s, f, z in zip(starts, full, size)]

    def op_dynamic_slice(self, op, x, env):
        a = x[0]
        sizes = attr_i64s(op.attrs["slice_sizes"])
        st = self._starts(x[1:], a.shape, sizes)
        return [a[tuple(slice(s, s + z) for s, z in zip(st, sizes))]]

    def op_dynamic_update_slice(self, op, x, env):
        a, u = x[0], x[1]
        st = self._starts(x[2:], a.shape, u.shape)
        out = a.copy()
        out[tuple(slice(s, s + z) for s, z in zip(st, u.shape))] = u
        return [out]

    # ---- reductions -----------------------------------------------------------------
    def _simple_body(self, blk: Block):
        """A body made of one binary op on (acc, value) -> its name."""
        real = [o for o in blk.ops if o.name != "stablehlo.return"]
        if len(real) == 1 and len(blk.args) == 2 and set(real[0].operands) == {blk.args[0][0], blk.args[1][0]}:
            return real[0].name.split(".", 1)[1]
        return None

    def op_reduce(self, op, x, env):
        n = len(x) // 2
        ins, inits = x[:n], x[n:]
        dims = tuple(attr_i64s(op.attrs["dimensions"]))
        blk = op.regions[0]
        kind = self._simple_body(blk) if n == 1 else None
        a, dt = ins[0], op.result_types[0].dtype
        with np.errstate(all="ignore"):
            if kind in ("add", "multiply") and dt in FLOATS:
                w = a.astype(np.float64)
                r = w.sum(dims) if kind == "add" else w.prod(dims)
                r = r + inits[0] if kind == "add" else r * inits[0]
                return [r]
            if kind in ("maximum", "minimum") and a.size:
                f = np.max if kind == "maximum" else np.min
                r = f(a, axis=dims)
                return [(np.maximum if kind == "maximum" else np.minimum)(r, inits[0])]
            if kind in ("add",) and dt not in FLOATS and dt != "i1":
                return [(a.sum(dims, dtype=a.dtype) + inits[0]).astype(a.dtype)]
            if kind in ("and", "or") and dt == "i1":
                r = a.all(dims) if kind == "and" else a.any(dims)
                return [(np.logical_and if kind == "and" else np.logical_or)(r, inits[0])]
        # generic: move reduced dims last, flatten, fold pairwise with the body
        kept = [d for d in range(a.ndim) if d not in dims]
        perm = kept + list(dims)
        R = int(np.prod([a.shape[d] for d in dims])) if dims else 1
        cur = [np.transpose(v, perm).reshape([v.shape[d] for d in kept] + [R]) for v in ins]
        kshape = cur[0].shape[:-1]
        while cur[0].shape[-1] > 1:
            L = cur[0].shape[-1]
            h = L // 2
            lo = [c[..., :h] for c in cur]
            hi = [c[..., h:2 * h] for c in cur]
            rest = [c[..., 2 * h:] for c in cur]
            self._vector += 1
            outs = self.region(blk, env, lo + hi)
            self._vector -= 1
            outs = [self.cast(o, t.dtype) for o, t in zip(outs, op.result_types)]
            cur = [np.concatenate([o, r], axis=-1) for o, r in zip(outs, rest)]
        if R == 0:
            return [np.broadcast_to(i, kshape) for i in inits]
        acc = [c[..., 0] for c in cur]
        self._vector += 1
        outs = self.region(blk, env, [np.broadcast_to(i, kshape) for i in inits] + acc)
        self._vector -= 1
        return outs

    # ---- contractions -----------------------------------------------------------------
    def op_dot_general(self, op, x, env):
        a, b = x
        f = struct_fields(op.attrs["dot_dimension_numbers"])
        lb, rb = f.get("lhs_batching_dimensions", []), f.get("rhs_batching_dimensions", [])
        lc, rc = f.get("lhs_contracting_dimensions", []), f.get("rhs_contracting_dimensions", [])
        lf = [i for i in range(a.ndim) if i not in lb and i not in lc]
        rf = [i for i in range(b.ndim) if i not in rb and i not in rc]
        dt = op.result_types[0].dtype
        wt = np.float64 if dt in FLOATS else (np.int64 if not dt.startswith("ui") else np.uint64)
        if dt == "i1":
            wt = np.int64
        A = np.transpose(a, lb + lf + lc).astype(wt)
        B = np.transpose(b, rb + rc + rf).astype(wt)
        bs = [a.shape[i] for i in lb]
        m = int(np.prod([a.shape[i] for i in lf])) if lf else 1
        k = int(np.prod([a.shape[i] for i in lc])) if lc else 1
        n = int(np.prod([b.shape[i] for i in rf])) if rf else 1
        nb = int(np.prod(bs)) if bs else 1
        C = np.matmul(A.reshape(nb, m, k), B.reshape(nb, k, n))
        C = C.reshape(bs + [a.shape[i] for i in lf] + [b.shape[i] for i in rf])
        if dt == "i1":
            C = C != 0
        return [C]

    def op_convolution(self, op, x, env):
        """Dilate the input, then pad (negative pad crops), then correlate
        with the dilated kernel (src/pjrt_plugin/ops/linalg.cc:508-532);
        batch_group_count folds into feature groups (linalg.cc:339-362)."""
        import torch
        lhs, rhs = x
        dn = op.attrs["dimension_numbers"]
        inner = dn[dn.index("<") + 1:dn.rindex(">")]
        ls, rest = inner.split("]x[")
        rs, os_ = rest.split("]->[")
        ls, rs, os_ = ([t.strip() for t in s.strip("[] ").split(",")] for s in (ls, rs, os_))
        nsp = len(ls) - 2
        assert nsp in (1, 2), "oracle convolution: 1 or 2 spatial dims"
        if nsp == 1:        # run 1-D as 2-D with a unit second spatial dim
            lhs, rhs = lhs[..., None], rhs[..., None]
            ls, rs, os1 = ls + ["1"], rs + ["1"], os_ + ["1"]
            op2 = mt.Op(op.name, op.operands, op.results,
                        [mt.TType(tuple(op.result_types[0].shape) + (1,), op.result_types[0].dtype)], dict(op.attrs), [])
            spec = lambda s: "[" + ", ".join(s) + "]"
            op2.attrs["dimension_numbers"] = f"#stablehlo.conv<{spec(ls)}x{spec(rs)}->{spec(os1)}>"
            for k, d in (("window_strides", 1), ("lhs_dilation", 1), ("rhs_dilation", 1)):
                v = attr_i64s(op.attrs[k]) if k in op.attrs else [d]
                op2.attrs[k] = "array<i64: " + ", ".join(str(q) for q in v + [1]) + ">"
            pd = [int(q) for q in np.array(mt.dense_array(op.attrs["padding"])).reshape(-1)] if "padding" in op.attrs else [0, 0]
            op2.attrs["padding"] = f"dense<[[{pd[0]}, {pd[1]}], [0, 0]]> : tensor<2x2xi64>"
            return [self.op_convolution(op2, [lhs, rhs], env)[0][..., 0]]
        def get(name, default):
            return attr_i64s(op.attrs[name]) if name in op.attrs else default
        stride = get("window_strides", [1] * nsp)
        ldil = get("lhs_dilation", [1] * nsp)
        rdil = get("rhs_dilation", [1] * nsp)
        pad = np.array(mt.dense_array(op.attrs["padding"])).reshape(nsp, 2) if "padding" in op.attrs else np.zeros((nsp, 2), int)
        G = attr_int(op.attrs.get("feature_group_count", "1"))
        BG = attr_int(op.attrs.get("batch_group_count", "1"))
        if "window_reversal" in op.attrs and any(mt.dense_array(op.attrs["window_reversal"]).reshape(-1)):
            raise NotImplementedError("window_reversal")
        # to NCHW / OIHW
        L = np.transpose(lhs, [ls.index("b"), ls.index("f")] + [ls.index(str(s)) for s in range(nsp)])
        K = np.transpose(rhs, [rs.index("o"), rs.index("i")] + [rs.index(str(s)) for s in range(nsp)])
        wt = torch.float64 if (self.conv_f64 or op.result_types[0].dtype == "f64") else torch.float32
        Lt = torch.from_numpy(np.ascontiguousarray(L).astype(np.float64)).to(wt)
        Kt = torch.from_numpy(np.ascontiguousarray(K).astype(np.float64)).to(wt)
        if BG > 1:
            # batch groups: split batch into BG groups, each feeding O/BG output features
            n, c = Lt.shape[0], Lt.shape[1]
            Lt = Lt.reshape(BG, n // BG, c, *Lt.shape[2:]).permute(1, 0, 2, 3, 4).reshape(n // BG, BG * c, *Lt.shape[2:])
            G = BG
        # lhs dilation
        if any(d != 1 for d in ldil):
            n, c, h, w = Lt.shape
            hd = 0 if h == 0 else (h - 1) * ldil[0] + 1
            wd = 0 if w == 0 else (w - 1) * ldil[1] + 1
            Z = torch.zeros((n, c, hd, wd), dtype=wt)
            Z[:, :, ::ldil[0], ::ldil[1]] = Lt
            Lt = Z
        # padding (negative crops)
        for s in range(nsp):
            lo, hi = int(pad[s][0]), int(pad[s][1])
            if lo < 0:
                Lt = Lt.narrow(2 + s, -lo, Lt.shape[2 + s] + lo); lo = 0
            if hi < 0:
                Lt = Lt.narrow(2 + s, 0, Lt.shape[2 + s] + hi); hi = 0
            if lo or hi:
                padspec = [0, 0, 0, 0]
                padspec[(nsp - 1 - s) * 2] = lo; padspec[(nsp - 1 - s) * 2 + 1] = hi
                Lt = torch.nn.functional.pad(Lt, padspec)
        out = torch.nn.functional.conv2d(Lt.contiguous(), Kt.contiguous(), None, stride=tuple(stride),
                                         padding=0, dilation=tuple(rdil), groups=G).numpy()
        cur = ["b", "f"] + [str(s) for s in range(nsp)]
        return [np.transpose(out, [cur.index(c) for c in os_])]

    # ---- gather / scatter -------------------------------------------------------------------
    def op_gather(self, op, x, env):
        """Per-output-element index arithmetic of stablehlo.gather with clamped
        starts and batching dims (src/pjrt_plugin/ops/gather_scatter.cc:200-294)."""
        operand, idx = x
        f = struct_fields(op.attrs["dimension_numbers"])
        offset_dims = f.get("offset_dims", [])
        collapsed = f.get("collapsed_slice_dims", [])
        obatch = f.get("operand_batching_dims", [])
        ibatch = f.get("start_indices_batching_dims", [])
        smap = f.get("start_index_map", [])
        ivd = f.get("index_vector_dim", idx.ndim)
        sizes = attr_i64s(op.attrs["slice_sizes"])
        t = op.result_types[0]
        out_rank = len(t.shape)
        batch_dims = [d for d in range(out_rank) if d not in offset_dims]
        oi = np.indices(t.shape).reshape(out_rank, -1) if t.shape else np.zeros((0, 1), int)
        nel = oi.shape[1]
        # batch index into start_indices
        idx_m = np.moveaxis(idx, ivd, -1) if ivd < idx.ndim else idx[..., None]
        bidx = tuple(oi[d] for d in batch_dims)
        starts = idx_m[bidx].astype(np.int64).reshape(nel, -1) if batch_dims else np.broadcast_to(idx_m.reshape(1, -1), (nel, idx_m.size))
        full = np.zeros((operand.ndim, nel), np.int64)
        for k, od in enumerate(smap):
            full[od] = np.clip(starts[:, k], 0, operand.shape[od] - sizes[od])
        # batching dims: operand batch coordinate = index batch coordinate
        idx_batch_dims_in_out = [d for d in range(idx.ndim) if d != ivd]
        for od, ib in zip(obatch, ibatch):
            pos = idx_batch_dims_in_out.index(ib)
            full[od] = oi[batch_dims[pos]]
        window_dims = [d for d in range(operand.ndim) if d not in collapsed and d not in obatch]
        for k, wd in enumerate(window_dims):
            full[wd] += oi[offset_dims[k]]
        return [operand[tuple(full)].reshape(t.shape)]

    @staticmethod
    def _window_geometry(op, rank):
        def lst(name, dflt):
            v = attr_i64s(op.attrs[name]) if name in op.attrs else []
            return list(v) if len(v) else [dflt] * rank
        win, stride = lst("window_dimensions", 1), lst("window_strides", 1)
        bdil, wdil = lst("base_dilations", 1), lst("window_dilations", 1)
        pad = [(0, 0)] * rank
        if "padding" in op.attrs:
            dv = mt.dense_array(op.attrs["padding"])
            pad = [tuple(int(v) for v in row) for row in np.asarray(dv).reshape(rank, 2)]
        return win, stride, pad, bdil, wdil

    def op_reduce_window(self, op, x, env):
        """stablehlo.reduce_window: the input is dilated, then padded, both with the init value
        (src/pjrt_plugin/ops/reduction.cc:165-458 handles the pooling and cumulative forms); every window offset is
        folded into the accumulator with the body, offsets in row-major order."""
        n = len(x) // 2
        ins, inits = x[:n], x[n:]
        rank = ins[0].ndim
        win, stride, pad, bdil, wdil = self._window_geometry(op, rank)
        oshape = op.result_types[0].shape
        padded = []
        for a, i in zip(ins, inits):
            dil = tuple((a.shape[d] - 1) * bdil[d] + 1 if a.shape[d] else 0 for d in range(rank))
            full = np.full(tuple(max(0, dil[d] + pad[d][0] + pad[d][1]) for d in range(rank)), i, dtype=a.dtype)
            # negative padding crops: place the dilated input through index arithmetic
            src = np.full(dil, i, dtype=a.dtype)
            src[tuple(slice(None, None, bdil[d]) for d in range(rank))] = a
            sl_dst, sl_src = [], []
            for d in range(rank):
                lo = pad[d][0]
                s0, d0 = max(0, -lo), max(0, lo)
                ln = min(dil[d] - s0, full.shape[d] - d0)
                sl_src.append(slice(s0, s0 + max(ln, 0)))
                sl_dst.append(slice(d0, d0 + max(ln, 0)))
            full[tuple(sl_dst)] = src[tuple(sl_src)]
            padded.append(full)
        acc = [np.broadcast_to(np.asarray(i, dtype=a.dtype), oshape).copy() for a, i in zip(ins, inits)]
        for off in np.ndindex(*win):
            sl = tuple(slice(off[d] * wdil[d], off[d] * wdil[d] + (oshape[d] - 1) * stride[d] + 1, stride[d]) if oshape[d] else slice(0, 0)
                       for d in range(rank))
            vals = [p[sl] for p in padded]
            self._vector += 1
            outs = self.region(op.regions[0], env, acc + vals)
            self._vector -= 1
            acc = [self.cast(o, t.dtype) for o, t in zip(outs, op.result_types)]
        return acc

    def op_select_and_scatter(self, op, x, env):
        """stablehlo.select_and_scatter: per window the in-bounds element chosen by the select body (scanned in row-major
        order, the current choice stays while select(current, candidate) holds; padding is never chosen:
        src/pjrt_plugin/ops/reduction.cc:531-549) receives the window's source value through the scatter body."""
        operand, source, init = x
        rank = operand.ndim
        win, stride, pad, _, _ = self._window_geometry(op, rank)
        sshape = source.shape
        have = np.zeros(sshape, dtype=bool)
        cur = np.zeros(sshape, dtype=operand.dtype)
        cur_at = np.full(sshape + (rank,), -1, dtype=np.int64)
        grids = np.meshgrid(*[np.arange(n) for n in sshape], indexing="ij") if rank else []
        for off in np.ndindex(*win):
            pos = [grids[d] * stride[d] + off[d] - pad[d][0] for d in range(rank)]
            ok = np.ones(sshape, dtype=bool)
            for d in range(rank):
                ok &= (pos[d] >= 0) & (pos[d] < operand.shape[d])
            cand = operand[tuple(np.clip(pos[d], 0, max(operand.shape[d] - 1, 0)) for d in range(rank))] if rank else operand
            self._vector += 1
            keep = np.asarray(self.region(op.regions[0], env, [cur, cand])[0]).astype(bool)
            self._vector -= 1
            take = ok & (~have | ~keep)
            cur = np.where(take, cand, cur)
            for d in range(rank):
                cur_at[..., d] = np.where(take, pos[d], cur_at[..., d])
            have |= take
        out = np.broadcast_to(np.asarray(init, dtype=operand.dtype), operand.shape).copy()
        for sidx in np.ndindex(*sshape):                       # windows in row-major order
            if not have[sidx]:
                continue
            at = tuple(int(v) for v in cur_at[sidx])
            r = self.region(op.regions[1], env, [out[at], source[sidx]])[0]
            out[at] = self.cast(np.asarray(r), op.result_types[0].dtype)
        return [out]

    def op_scatter(self, op, x, env):
        """stablehlo.scatter, one operand. Out-of-bounds windows are skipped.
        Body classification as in gather_scatter.cc:13-53."""
        operand, idx, upd = x
        f = struct_fields(op.attrs["scatter_dimension_numbers"])
        uwd = f.get("update_window_dims", [])
        iwd = f.get("inserted_window_dims", [])
        ibd = f.get("input_batching_dims", [])
        sbd = f.get("scatter_indices_batching_dims", [])
        sdo = f.get("scatter_dims_to_operand_dims", [])
        ivd = f.get("index_vector_dim", idx.ndim)
        kind = self._simple_body(op.regions[0])
        real = [o for o in op.regions[0].ops if o.name != "stablehlo.return"]
        if not real:
            kind = "update"
        ui = np.indices(upd.shape).reshape(upd.ndim, -1) if upd.shape else np.zeros((0, 1), int)
        nel = ui.shape[1]
        scatter_dims = [d for d in range(upd.ndim) if d not in uwd]
        idx_m = np.moveaxis(idx, ivd, -1) if ivd < idx.ndim else idx[..., None]
        sidx = tuple(ui[d] for d in scatter_dims)
        starts = idx_m[sidx].astype(np.int64).reshape(nel, -1) if scatter_dims else np.broadcast_to(idx_m.reshape(1, -1), (nel, idx_m.size))
        full = np.zeros((operand.ndim, nel), np.int64)
        for k, od in enumerate(sdo):
            full[od] = starts[:, k]
        idx_batch_dims = [d for d in range(idx.ndim) if d != ivd]
        for od, ib in zip(ibd, sbd):
            full[od] = ui[scatter_dims[idx_batch_dims.index(ib)]]
        window_dims = [d for d in range(operand.ndim) if d not in iwd and d not in ibd]
        # window bounds check uses the window start (whole window must fit)
        wsize = {wd: upd.shape[uwd[k]] for k, wd in enumerate(window_dims)}
        ok = np.ones(nel, bool)
        for d in range(operand.ndim):
            sz = wsize.get(d, 1)
            ok &= (full[d] >= 0) & (full[d] + sz <= operand.shape[d])
        for k, wd in enumerate(window_dims):
            full[wd] = full[wd] + ui[uwd[k]]
        tgt = tuple(full[:, ok])
        vals = upd.reshape(-1)[ok]
        dt = op.result_types[0].dtype
        if kind == "add" and dt in FLOATS:
            acc = operand.astype(np.float64)
            np.add.at(acc, tgt, vals.astype(np.float64))
            return [acc]
        out = operand.copy()
        if kind == "update":
            out[tgt] = vals
        elif kind in ("add", "subtract", "multiply", "maximum", "minimum"):
            {"add": np.add, "subtract": np.subtract, "multiply": np.multiply, "maximum": np.maximum,
             "minimum": np.minimum}[kind].at(out, tgt, vals)
        else:
            flat_t = np.stack(tgt, 0) if tgt else np.zeros((0, len(vals)), int)
            for j in range(len(vals)):
                pos = tuple(flat_t[:, j])
                out[pos] = self.region(op.regions[0], env, [out[pos], vals[j]])[0]
        return [out]

    # ---- control flow ----------------------------------------------------------------------------
    def op_while(self, op, x, env):
        cur = list(x)
        cond, body = op.regions
        it = 0
        while bool(self.region(cond, env, cur)[0]):
            cur = self.region(body, env, cur)
            cur = [self.cast(v, t.dtype) for v, t in zip(cur, op.result_types)]
            it += 1
            if it > 10_000_000:
                raise RuntimeError("oracle while: iteration limit")
        return cur

    # ---- dense linear algebra --------------------------------------------------------------------------
    def op_cholesky(self, op, x, env):
        """stablehlo.cholesky through LAPACK in float64, as the reference runs it on the host
        (src/pjrt_plugin/ops/linalg.cc:553-570); only the named triangle is read, the other triangle of the result is
        zero, a matrix that is not positive definite gives NaN."""
        a = np.asarray(x[0], np.float64)
        lower = mt.attr_bool(op.attrs["lower"]) if "lower" in op.attrs else True
        n = a.shape[-1]
        flat = a.reshape(-1, n, n)
        out = np.empty_like(flat)
        for g, m in enumerate(flat):
            tri = np.tril(m) if lower else np.triu(m).T
            sym = tri + np.tril(tri, -1).T
            try:
                l = np.linalg.cholesky(sym)
            except np.linalg.LinAlgError:
                l = np.full((n, n), np.nan)
            out[g] = l if lower else l.T
        return [out.reshape(a.shape)]

    def op_triangular_solve(self, op, x, env):
        """stablehlo.triangular_solve by substitution in float64 (scipy.linalg.solve_triangular); a matrix with a zero on
        a diagonal that counts gives NaN for its whole solution (src/pjrt_plugin/ops/linalg.cc:596-628)."""
        from scipy.linalg import solve_triangular
        a, b = np.asarray(x[0], np.float64), np.asarray(x[1], np.float64)
        flag = lambda k, d: mt.attr_bool(op.attrs[k]) if k in op.attrs else d
        left, lower, unit = flag("left_side", True), flag("lower", True), flag("unit_diagonal", False)
        trans = enum_word(op.attrs["transpose_a"]) in ("TRANSPOSE", "ADJOINT") if "transpose_a" in op.attrs else False
        n = a.shape[-1]
        fa, fb = a.reshape(-1, n, n), b.reshape((-1,) + b.shape[-2:])
        out = np.empty_like(fb)
        for g in range(fa.shape[0]):
            m = np.tril(fa[g]) if lower else np.triu(fa[g])
            if not unit and np.any(np.diagonal(m) == 0):
                out[g] = np.nan
                continue
            with np.errstate(all="ignore"):
                if left:
                    out[g] = solve_triangular(m, fb[g], lower=lower, trans=1 if trans else 0, unit_diagonal=unit, check_finite=False)
                else:       # X op(A) = B  <=>  op(A)^T X^T = B^T
                    out[g] = solve_triangular(m, fb[g].T, lower=lower, trans=0 if trans else 1, unit_diagonal=unit, check_finite=False).T
        return [out.reshape(b.shape)]

    # ---- random bits -----------------------------------------------------------------------------------
    @staticmethod
    def philox4x32_10(ctr, key):
        """Philox-4x32 with ten rounds (Salmon, Moraes, Dror, Shaw, SC 2011) on arrays of 32-bit words held in uint64:
        ctr = four arrays, key = two scalars; returns the four output words."""
        mask = np.uint64(0xFFFFFFFF)
        c = [np.asarray(v, np.uint64) for v in ctr]
        k = [np.uint64(key[0]), np.uint64(key[1])]
        for _ in range(10):
            p0 = np.uint64(0xD2511F53) * c[0]
            p1 = np.uint64(0xCD9E8D57) * c[2]
            c = [(p1 >> np.uint64(32)) ^ c[1] ^ k[0], p1 & mask, (p0 >> np.uint64(32)) ^ c[3] ^ k[1], p0 & mask]
            k = [(k[0] + np.uint64(0x9E3779B9)) & mask, (k[1] + np.uint64(0xBB67AE85)) & mask]
        return c

    def op_rng_bit_generator(self, op, x, env):
        """stablehlo.rng_bit_generator: the state is a 64-bit key and a 64- or 128-bit counter; the output bytes are the
        Philox-4x32-10 stream of the key from the counter on, 16 bytes per counter value, and the returned counter has
        advanced by one per 16 bytes (src/pjrt_plugin/ops/control_flow.cc:2346-2356 advances it the same way; the bits
        themselves differ between backends there too)."""
        state = np.ascontiguousarray(x[0])
        words = state.view(np.uint32).reshape(-1).astype(np.uint64)
        if words.size not in (4, 6):
            raise ValueError("rng_bit_generator: the state must be 16 or 24 bytes")
        ot = op.result_types[1]
        dt = np.dtype(mt.np_dtype(ot.dtype))
        nbytes = int(np.prod(ot.shape, dtype=np.int64)) * dt.itemsize
        blocks = (nbytes + 15) // 16
        lo64 = int(words[2]) | int(words[3]) << 32
        hi64 = (int(words[4]) | int(words[5]) << 32) if words.size == 6 else 0
        j = np.arange(blocks, dtype=np.uint64)
        with np.errstate(over="ignore"):
            lo = np.uint64(lo64) + j
        hi = (np.uint64(hi64) + (lo < np.uint64(lo64)).astype(np.uint64)) if blocks else np.zeros(0, np.uint64)
        mask = np.uint64(0xFFFFFFFF)
        r = self.philox4x32_10([lo & mask, lo >> np.uint64(32), hi & mask, hi >> np.uint64(32)], (words[0], words[1]))
        stream = np.stack([v.astype(np.uint32) for v in r], axis=-1).reshape(-1)
        out = stream.view(np.uint8)[:nbytes].copy().view(dt).reshape(ot.shape)
        nlo = (lo64 + blocks) & ((1 << 64) - 1)
        nhi = (hi64 + (1 if nlo < lo64 else 0)) & ((1 << 64) - 1)
        nw = [int(words[0]), int(words[1]), nlo & 0xFFFFFFFF, nlo >> 32] + ([nhi & 0xFFFFFFFF, nhi >> 32] if words.size == 6 else [])
        new_state = np.array(nw, np.uint32).view(state.dtype).reshape(state.shape)
        return [new_state, out]

    # ---- sorting ---------------------------------------------------------------------------------------
    SORT_RANK_MAX = 2048                    # rows up to this length are sorted by the all-pairs definition

    def _sort_before(self, blk, env, lhs, rhs):
        """The comparator region on arrays: lhs[k] goes before rhs[k] (elementwise over broadcast shapes)."""
        args = []
        for a, b in zip(lhs, rhs):
            shape = np.broadcast_shapes(a.shape, b.shape)
            args += [np.broadcast_to(a, shape), np.broadcast_to(b, shape)]
        self._vector += 1
        (r,) = self.region(blk, env, args)
        self._vector -= 1
        return np.asarray(r).astype(bool)

    def _sort_positions_by_rank(self, blk, env, rows):
        """Position of every element in the stable order, from the definition: the elements that go before it plus the
        equivalent elements (neither before the other) in front of it. rows: one [R, n] array per operand."""
        R, n = rows[0].shape
        pos = np.empty((R, n), np.int64)
        chunk = max(1, (1 << 22) // max(1, n * n))
        earlier = np.tril(np.ones((n, n), bool), -1)           # [i, j]: j < i
        for r0 in range(0, R, chunk):
            sl = slice(r0, min(R, r0 + chunk))
            xi = [v[sl, :, None] for v in rows]
            xj = [v[sl, None, :] for v in rows]
            j_before_i = self._sort_before(blk, env, xj, xi)    # [c, i, j]
            i_before_j = self._sort_before(blk, env, xi, xj)
            tie = ~j_before_i & ~i_before_j & earlier[None]
            pos[sl] = j_before_i.sum(-1) + tie.sum(-1)
        return pos

    def _sort_positions_by_merging(self, blk, env, rows):
        """The same order for long rows: runs of one element are merged pairwise, every element finding its place in
        the sibling run by bisection with the comparator (left-run elements go in front of equivalent right-run ones)."""
        R, n = rows[0].shape
        perm = np.broadcast_to(np.arange(n), (R, n)).copy()
        ar = np.arange(n)
        rr = np.arange(R)[:, None]
        w = 1
        while w < n:
            run = ar // (2 * w) * (2 * w)
            right = (ar - run) >= w
            lo = np.where(right, run, np.minimum(run + w, n))
            hi = np.minimum(np.where(right, run + w, run + 2 * w), n)
            lo = np.minimum(lo, hi)
            me = [np.take_along_axis(v, perm, 1) for v in rows]
            l = np.broadcast_to(lo, (R, n)).copy()
            h = np.broadcast_to(hi, (R, n)).copy()
            while True:
                open_ = l < h
                if not open_.any():
                    break
                mid = np.where(open_, (l + h) // 2, 0)
                other = [v[rr, perm[rr, mid]] for v in rows]
                first = np.where(right[None], ~self._sort_before(blk, env, me, other), self._sort_before(blk, env, other, me))
                l = np.where(open_ & first, mid + 1, l)
                h = np.where(open_ & ~first, mid, h)
            dest = run[None] + np.where(right, ar - run - w, ar - run)[None] + (l - lo[None])
            nxt = np.empty_like(perm)
            nxt[rr, dest] = perm
            perm = nxt
            w *= 2
        pos = np.empty_like(perm)
        pos[rr, perm] = ar[None]
        return pos

    def op_sort(self, op, x, env):
        """stablehlo.sort along `dimension` with the comparator region; always stable, which is_stable = false permits
        (src/pjrt_plugin/ops/sort_fft_complex.cc:135-250 sorts by the direction it reads out of the comparator)."""
        rank = x[0].ndim
        dim = attr_int(op.attrs["dimension"]) if "dimension" in op.attrs else rank - 1
        dim %= rank
        n = x[0].shape[dim]
        if x[0].size == 0:
            return [np.array(v) for v in x]
        moved = [np.moveaxis(np.asarray(v), dim, -1) for v in x]
        lead = moved[0].shape[:-1]
        rows = [np.ascontiguousarray(m).reshape(-1, n) for m in moved]
        blk = op.regions[0]
        pos = (self._sort_positions_by_rank if n <= self.SORT_RANK_MAX else self._sort_positions_by_merging)(blk, env, rows)
        outs = []
        rr = np.arange(rows[0].shape[0])[:, None]
        for v in rows:
            o = np.empty_like(v)
            o[rr, pos] = v
            outs.append(np.moveaxis(o.reshape(lead + (n,)), -1, dim))
        return outs

    def op_top_k(self, op, x, env):
        """chlo.top_k: the k largest along the last dimension, descending, equal values by ascending position, NaN
        after every number (src/pjrt_plugin/ops/sort_fft_complex.cc:41-88 sorts the negated values stably)."""
        a = np.asarray(x[0])
        k = op.result_types[0].shape[-1]
        if a.dtype.kind == "f":
            nan = np.isnan(a)
            order = np.lexsort((np.where(nan, 0.0, -a.astype(np.float64)), nan), axis=-1)      # stable; NaN last
        else:
            order = np.argsort(~a, axis=-1, kind="stable")          # bitwise not reverses integer order without overflow
        order = order[..., :k]
        return [np.take_along_axis(a, order, -1), order.astype(np.int32)]

    def op_case(self, op, x, env):
        i = int(x[0])
        n = len(op.regions)
        if i < 0 or i >= n:
            i = n - 1                       # src/pjrt_plugin/ops/control_flow.cc:672-675
        return self.region(op.regions[i], env, [])

    def op_call(self, op, x, env):
        callee = op.attrs["callee"].strip().lstrip("@")
        return Interp(self.m, self.collective, self.partition_id, self.conv_f64, self.wide, self.gather).run(x, callee)

    def op_composite(self, op, x, env):
        callee = op.attrs["decomposition"].strip().lstrip("@")
        return Interp(self.m, self.collective, self.partition_id, self.conv_f64, self.wide, self.gather).run(x, callee)

    def op_optimization_barrier(self, op, x, env):
        return list(x)

    def op_create_token(self, op, x, env):
        return [np.zeros((), np.bool_)]

    def op_after_all(self, op, x, env):
        return [np.zeros((), np.bool_)]

    def op_custom_call(self, op, x, env):
        tgt = mt.attr_str(op.attrs["call_target_name"])
        if tgt in ("Sharding", "SPMDFullToShardShape", "SPMDShardToFullShape"):
            return [x[0].reshape(op.result_types[0].shape)]         # control_flow.cc:1426-1438
        if tgt.startswith("mhlo.") and len(x) == 1:             # control_flow.cc:1440-1477: the chlo operation of that name
            fn = tgt[5:]
            if fn == "topk":
                return self.op_top_k(op, x, env)
            if fn in _UNARY:
                with np.errstate(all="ignore"):
                    return [_UNARY[fn](x[0].astype(np.float64))]
            if hasattr(self, "op_" + fn):
                return getattr(self, "op_" + fn)(op, x, env)
        raise NotImplementedError(f"oracle: custom_call {tgt}")

    # ---- collectives ---------------------------------------------------------------------------------
    def op_all_reduce(self, op, x, env):
        if self.collective is None:
            return list(x)                  # one partition: identity (src/pjrt_plugin/ops/collectives.cc:41-47)
        return self.collective(list(x))

    def op_all_gather(self, op, x, env):
        # every partition's operand, concatenated along all_gather_dim in partition order
        dim = mt.attr_int(op.attrs["all_gather_dim"])
        if self.gather is None:
            return list(x)                  # one partition
        return [np.concatenate(self.gather(v), axis=dim) for v in x]

    def op_partition_id(self, op, x, env):
        return [np.uint32(self.partition_id)]

    def op_replica_id(self, op, x, env):
        return [np.uint32(0)]


def op_operand_dtype(a: np.ndarray) -> str:
    return {np.dtype(v): k for k, v in mt._NPDT.items() if k != "bf16"}[a.dtype]


def run_text(text: str, args, **kw) -> list:
    return Interp(text, **kw).run(args)
