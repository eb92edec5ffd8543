"""StableHLO text builder with tape-based reverse-mode differentiation.

JAX is not installable next to this plugin's build, so the programs the plugin
is exercised with are produced here: a small eager tracer whose primitives
print the StableHLO operations `jax.jit(...).lower()` prints for the same
`lax` primitive (generic operation form, `func.func` in its custom form), and
whose VJP rules emit the operations JAX's transpose rules emit
(`stablehlo.convolution` with `lhs_dilation`/`rhs_dilation` and permuted
dimension numbers for the two convolution gradients, `select` for ReLU,
`broadcast_in_dim` for reduced sums, `scatter` for gathered rows).

The text is the plugin's compile input (the reference takes the same module
as `args->program->code`, src/pjrt_plugin/pjrt_client.cc:179-257).
"""
from __future__ import annotations

import math
import struct
from typing import Callable, Sequence

import numpy as np

_NP = {
    "f32": np.float32, "f16": np.float16, "f64": np.float64,
    "i8": np.int8, "i16": np.int16, "i32": np.int32, "i64": np.int64,
    "ui8": np.uint8, "ui16": np.uint16, "ui32": np.uint32, "ui64": np.uint64,
    "i1": np.bool_,
}
FLOATS = ("f32", "bf16", "f16", "f64")


def ttype(shape: Sequence[int], dtype: str) -> str:
    return "tensor<" + "".join(f"{d}x" for d in shape) + dtype + ">"


def _fmt_scalar(v, dtype: str) -> str:
    if dtype == "i1":
        return "true" if v else "false"
    if dtype in FLOATS:
        v = float(v)
        if math.isinf(v):
            bits = {"f32": (0x7F800000, 0xFF800000), "bf16": (0x7F80, 0xFF80),
                    "f16": (0x7C00, 0xFC00),
                    "f64": (0x7FF0000000000000, 0xFFF0000000000000)}[dtype]
            return hex(bits[0] if v > 0 else bits[1]).upper().replace("X", "x")
        if math.isnan(v):
            return {"f32": "0x7FC00000", "bf16": "0x7FC0", "f16": "0x7E00",
                    "f64": "0x7FF8000000000000"}[dtype]
        return f"{v:.9e}" if dtype != "f64" else f"{v:.17e}"
    return str(int(v))


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + (0x7FFF + ((u >> 16) & 1))) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


class Val:
    """An SSA value. Arithmetic operators follow jax.numpy broadcasting for
    scalars and equal-shape tensors (no implicit rank promotion)."""

    __slots__ = ("b", "name", "shape", "dtype")
    __array_priority__ = 100

    def __init__(self, b: "Builder", name: str, shape, dtype: str):
        self.b, self.name, self.shape, self.dtype = b, name, tuple(int(d) for d in shape), dtype

    @property
    def type(self) -> str:
        return ttype(self.shape, self.dtype)

    @property
    def size(self) -> int:
        return int(np.prod(self.shape)) if self.shape else 1

    @property
    def ndim(self) -> int:
        return len(self.shape)

    def __repr__(self):
        return f"Val({self.name}: {self.type})"

    def _co(self, o):
        return self.b.as_val(o, like=self)

    def __add__(self, o): return self.b.add(self, self._co(o))
    def __radd__(self, o): return self.b.add(self._co(o), self)
    def __sub__(self, o): return self.b.sub(self, self._co(o))
    def __rsub__(self, o): return self.b.sub(self._co(o), self)
    def __mul__(self, o): return self.b.mul(self, self._co(o))
    def __rmul__(self, o): return self.b.mul(self._co(o), self)
    def __truediv__(self, o): return self.b.div(self, self._co(o))
    def __rtruediv__(self, o): return self.b.div(self._co(o), self)
    def __neg__(self): return self.b.neg(self)
    def astype(self, dt): return self.b.convert(self, dt)
    def reshape(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = shape[0]
        return self.b.reshape(self, shape)


class Builder:
    """Accumulates the body of one function; sub-builders (regions) share the
    SSA counter of their parent."""

    def __init__(self, parent: "Builder | None" = None):
        self.parent = parent
        self.root = parent.root if parent else self
        self.lines: list[str] = []
        self.args: list[Val] = []
        self.tape: list[tuple] = []
        self.indent = (parent.indent + 2) if parent else 2
        if parent is None:
            self._n = 0
            self.taping = True
            self.arg_attrs: dict[str, str] = {}

    # ---- plumbing -------------------------------------------------------
    def fresh(self) -> str:
        self.root._n += 1
        return f"%{self.root._n}"

    def arg(self, shape, dtype: str, attrs: str = "") -> Val:
        v = Val(self, f"%arg{len(self.root.args)}" if self is self.root else self.fresh(), shape, dtype)
        self.args.append(v)
        if attrs:
            self.root.arg_attrs[v.name] = attrs
        return v

    def emit(self, opname: str, operands: Sequence[Val], results: Sequence[tuple],
             props: dict | None = None, regions: Sequence[str] = (), attrs: dict | None = None):
        """Print one operation in MLIR's generic form and return its results."""
        outs = [Val(self, self.fresh(), s, d) for s, d in results]
        lhs = ""
        if outs:
            lhs = (outs[0].name if len(outs) == 1 else f"{outs[0].name}:{len(outs)}") + " = "
            if len(outs) > 1:
                base = outs[0].name
                for i, o in enumerate(outs):
                    o.name = f"{base}#{i}"
        s = f'{lhs}"{opname}"({", ".join(o.name for o in operands)})'
        if props:
            s += " <{" + ", ".join(f"{k} = {v}" for k, v in sorted(props.items())) + "}>"
        if regions:
            s += " (" + ", ".join(regions) + ")"
        if attrs:
            s += " {" + ", ".join(f"{k} = {v}" for k, v in sorted(attrs.items())) + "}"
        s += " : (" + ", ".join(o.type for o in operands) + ") -> "
        s += outs[0].type if len(outs) == 1 else "(" + ", ".join(o.type for o in outs) + ")"
        self.lines.append(" " * self.indent + s)
        return outs

    def region(self, arg_types: Sequence[tuple], body: Callable) -> str:
        """Build a single-block region; `body(sub, *args)` returns the values
        handed to stablehlo.return."""
        sub = Builder(self)
        sub.indent = self.indent + 4
        args = [sub.arg(s, d) for s, d in arg_types]
        rets = body(sub, *args)
        if isinstance(rets, Val):
            rets = [rets]
        sub.emit("stablehlo.return", list(rets), [])
        if not args:                   # a region without block arguments has no block header
            return "{\n" + "\n".join(sub.lines) + "\n" + " " * self.indent + "}"
        head = " " * (self.indent + 2) + "^bb0(" + ", ".join(f"{a.name}: {a.type}" for a in args) + "):"
        return "{\n" + head + "\n" + "\n".join(sub.lines) + "\n" + " " * self.indent + "}"

    def record(self, outs, ins, vjp):
        if self.root.taping:
            self.tape.append((list(outs), list(ins), vjp))

    # ---- constants -------------------------------------------------------
    def const(self, value, dtype: str, shape=()) -> Val:
        """Splat constant of `shape` (scalar by default)."""
        lit = _fmt_scalar(value, dtype)
        return self.emit("stablehlo.constant", [], [(shape, dtype)],
                         props={"value": f"dense<{lit}> : {ttype(shape, dtype)}"})[0]

    def const_array(self, arr: np.ndarray, dtype: str | None = None) -> Val:
        """Dense constant from a numpy array (hex blob form)."""
        arr = np.asarray(arr)
        if dtype is None:
            dtype = {v: k for k, v in _NP.items()}[arr.dtype.type]
        if dtype == "bf16":
            raw = f32_to_bf16_bits(arr.astype(np.float32)).tobytes()
        elif dtype == "i1":
            raw = np.ascontiguousarray(arr, dtype=np.uint8).tobytes()
        else:
            raw = np.ascontiguousarray(arr, dtype=_NP[dtype]).tobytes()
        return self.emit("stablehlo.constant", [], [(arr.shape, dtype)],
                         props={"value": f'dense<"0x{raw.hex().upper()}"> : {ttype(arr.shape, dtype)}'})[0]

    def as_val(self, o, like: Val) -> Val:
        if isinstance(o, Val):
            return o
        return self.full(like.shape, o, like.dtype)

    def full(self, shape, value, dtype: str) -> Val:
        c = self.const(value, dtype)
        return c if not shape else self.broadcast_in_dim(c, shape, ())

    def zeros_like(self, x: Val) -> Val:
        return self.full(x.shape, 0, x.dtype)

    # ---- elementwise -----------------------------------------------------
    def _unary(self, op: str, x: Val, vjp=None) -> Val:
        (y,) = self.emit(f"stablehlo.{op}", [x], [(x.shape, x.dtype)])
        if vjp is not None and x.dtype in FLOATS:
            self.record([y], [x], lambda g, y=y: [vjp(g[0], x, y)])
        return y

    def _binary(self, op: str, a: Val, b: Val, vjp=None) -> Val:
        assert a.shape == b.shape and a.dtype == b.dtype, (op, a, b)
        (y,) = self.emit(f"stablehlo.{op}", [a, b], [(a.shape, a.dtype)])
        if vjp is not None and a.dtype in FLOATS:
            self.record([y], [a, b], lambda g, y=y: vjp(g[0], a, b, y))
        return y

    def add(self, a, b): return self._binary("add", a, b, lambda g, a, b, y: [g, g])
    def sub(self, a, b): return self._binary("subtract", a, b, lambda g, a, b, y: [g, self.neg(g)])
    def mul(self, a, b): return self._binary("multiply", a, b, lambda g, a, b, y: [self.mul(g, b), self.mul(g, a)])

    def div(self, a, b):
        def vjp(g, a, b, y):
            ga = self.div(g, b)
            return [ga, self.neg(self.mul(ga, y))]
        return self._binary("divide", a, b, vjp)

    def max(self, a, b):
        def vjp(g, a, b, y):
            # jax: balanced split on ties
            half = self.full(a.shape, 0.5, a.dtype)
            one = self.full(a.shape, 1.0, a.dtype)
            zero = self.zeros_like(a)
            ma = self.select(self.compare(a, b, "GT"), one, self.select(self.compare(a, b, "EQ"), half, zero))
            return [self.mul(g, ma), self.mul(g, self.sub(one, ma))]
        return self._binary("maximum", a, b, vjp)

    def min(self, a, b): return self._binary("minimum", a, b)
    def pow(self, a, b): return self._binary("power", a, b)
    def rem(self, a, b): return self._binary("remainder", a, b)
    def and_(self, a, b): return self._binary("and", a, b)
    def or_(self, a, b): return self._binary("or", a, b)
    def xor(self, a, b): return self._binary("xor", a, b)
    def shl(self, a, b): return self._binary("shift_left", a, b)
    def shr_logical(self, a, b): return self._binary("shift_right_logical", a, b)
    def shr_arith(self, a, b): return self._binary("shift_right_arithmetic", a, b)
    def atan2(self, a, b): return self._binary("atan2", a, b)

    def neg(self, x): return self._unary("negate", x, lambda g, x, y: self.neg(g))
    def exp(self, x): return self._unary("exponential", x, lambda g, x, y: self.mul(g, y))
    def log(self, x): return self._unary("log", x, lambda g, x, y: self.div(g, x))
    def sqrt(self, x): return self._unary("sqrt", x, lambda g, x, y: self.div(g, self.mul(y, self.full(y.shape, 2.0, y.dtype))))
    def rsqrt(self, x): return self._unary("rsqrt", x, lambda g, x, y: self.mul(g, self.mul(self.div(y, x), self.full(y.shape, -0.5, y.dtype))))
    def tanh(self, x): return self._unary("tanh", x, lambda g, x, y: self.mul(g, self.sub(self.full(y.shape, 1.0, y.dtype), self.mul(y, y))))
    def logistic(self, x): return self._unary("logistic", x, lambda g, x, y: self.mul(g, self.mul(y, self.sub(self.full(y.shape, 1.0, y.dtype), y))))
    def sin(self, x): return self._unary("sine", x, lambda g, x, y: self.mul(g, self.cos(x)))
    def cos(self, x): return self._unary("cosine", x, lambda g, x, y: self.neg(self.mul(g, self.sin(x))))
    def abs(self, x): return self._unary("abs", x, lambda g, x, y: self.mul(g, self.sign(x)))
    def sign(self, x): return self._unary("sign", x)
    def floor(self, x): return self._unary("floor", x)
    def ceil(self, x): return self._unary("ceil", x)
    def not_(self, x): return self._unary("not", x)
    def log1p(self, x): return self._unary("log_plus_one", x, lambda g, x, y: self.div(g, self.add(x, self.full(x.shape, 1.0, x.dtype))))
    def expm1(self, x): return self._unary("exponential_minus_one", x, lambda g, x, y: self.mul(g, self.add(y, self.full(y.shape, 1.0, y.dtype))))
    def is_finite(self, x): return self.emit("stablehlo.is_finite", [x], [(x.shape, "i1")])[0]
    def popcnt(self, x): return self._unary("popcnt", x)
    def clz(self, x): return self._unary("count_leading_zeros", x)
    def round_even(self, x): return self._unary("round_nearest_even", x)
    def round_afz(self, x): return self._unary("round_nearest_afz", x)
    def cbrt(self, x): return self._unary("cbrt", x)
    def tan(self, x): return self._unary("tan", x)

    def chlo_unary(self, name: str, x: Val, form: str = "op") -> Val:
        """One of the chlo unary functions (sinh, cosh, asin, acos, atan, asinh, acosh, atanh, erf, erf_inv, tan) in the
        form jax emits it: the chlo operation itself ("op") or a custom call to @mhlo.<name> ("custom_call"). No gradient."""
        if form == "custom_call":
            return self.custom_call(f"mhlo.{name}", [x], [(x.shape, x.dtype)])[0]
        return self.emit(f"chlo.{name}", [x], [(x.shape, x.dtype)])[0]

    def square(self, x): return self.mul(x, x)

    def compare(self, a: Val, b: Val, direction: str, ctype: str | None = None) -> Val:
        assert a.shape == b.shape and a.dtype == b.dtype, (a, b)
        if ctype is None:
            ctype = "FLOAT" if a.dtype in FLOATS else ("UNSIGNED" if a.dtype.startswith("ui") or a.dtype == "i1" else "SIGNED")
        return self.emit("stablehlo.compare", [a, b], [(a.shape, "i1")],
                         props={"comparison_direction": f"#stablehlo<comparison_direction {direction}>",
                                "compare_type": f"#stablehlo<comparison_type {ctype}>"})[0]

    def select(self, p: Val, a: Val, b: Val) -> Val:
        assert a.shape == b.shape and a.dtype == b.dtype and p.shape in (a.shape, ()), (p, a, b)
        (y,) = self.emit("stablehlo.select", [p, a, b], [(a.shape, a.dtype)])
        if a.dtype in FLOATS:
            def vjp(g):
                z = self.zeros_like(g[0])
                return [None, self.select(p, g[0], z), self.select(p, z, g[0])]
            self.record([y], [p, a, b], vjp)
        return y

    def clamp(self, lo: Val, x: Val, hi: Val) -> Val:
        return self.emit("stablehlo.clamp", [lo, x, hi], [(x.shape, x.dtype)])[0]

    def convert(self, x: Val, dtype: str) -> Val:
        if x.dtype == dtype:
            return x
        (y,) = self.emit("stablehlo.convert", [x], [(x.shape, dtype)])
        if x.dtype in FLOATS and dtype in FLOATS:
            self.record([y], [x], lambda g: [self.convert(g[0], x.dtype)])
        return y

    def bitcast_convert(self, x: Val, dtype: str) -> Val:
        return self.emit("stablehlo.bitcast_convert", [x], [(x.shape, dtype)])[0]

    def stop_gradient(self, x: Val) -> Val:
        return x if not self.root.taping else _Stopped(x)

    # ---- shape ops -------------------------------------------------------
    def broadcast_in_dim(self, x: Val, shape, dims) -> Val:
        shape, dims = tuple(shape), tuple(dims)
        (y,) = self.emit("stablehlo.broadcast_in_dim", [x], [(shape, x.dtype)],
                         props={"broadcast_dimensions": _i64arr(dims)})
        if x.dtype in FLOATS:
            def vjp(g):
                red = [d for d in range(len(shape)) if d not in dims]
                r = self.reduce_sum(g[0], red) if red else g[0]
                # dims that were size-1 expanded
                exp = [i for i, d in enumerate(dims) if x.shape[i] == 1 and shape[d] != 1]
                if exp:
                    r = self.reduce_sum(r, exp)
                return [self.reshape(r, x.shape)]
            self.record([y], [x], vjp)
        return y

    def bcast(self, x: Val, shape, dims=None) -> Val:
        """Broadcast trailing-aligned (numpy style) unless `dims` given."""
        shape = tuple(shape)
        if dims is None:
            dims = tuple(range(len(shape) - x.ndim, len(shape)))
        if x.shape == shape:
            return x
        return self.broadcast_in_dim(x, shape, dims)

    def reshape(self, x: Val, shape) -> Val:
        shape = tuple(int(s) for s in shape)
        if shape == x.shape:
            return x
        assert int(np.prod(shape)) == x.size, (x, shape)
        (y,) = self.emit("stablehlo.reshape", [x], [(shape, x.dtype)])
        self.record([y], [x], lambda g: [self.reshape(g[0], x.shape)])
        return y

    def transpose(self, x: Val, perm) -> Val:
        perm = tuple(perm)
        if perm == tuple(range(x.ndim)):
            return x
        shape = tuple(x.shape[p] for p in perm)
        (y,) = self.emit("stablehlo.transpose", [x], [(shape, x.dtype)], props={"permutation": _i64arr(perm)})
        inv = tuple(int(i) for i in np.argsort(perm))
        self.record([y], [x], lambda g: [self.transpose(g[0], inv)])
        return y

    def reverse(self, x: Val, dims) -> Val:
        (y,) = self.emit("stablehlo.reverse", [x], [(x.shape, x.dtype)], props={"dimensions": _i64arr(dims)})
        self.record([y], [x], lambda g: [self.reverse(g[0], dims)])
        return y

    def iota(self, shape, dtype: str, dim: int) -> Val:
        return self.emit("stablehlo.iota", [], [(tuple(shape), dtype)], props={"iota_dimension": f"{dim} : i64"})[0]

    def slice(self, x: Val, start, limit, strides=None) -> Val:
        strides = tuple(strides) if strides else (1,) * x.ndim
        shape = tuple((l - s + st - 1) // st for s, l, st in zip(start, limit, strides))
        (y,) = self.emit("stablehlo.slice", [x], [(shape, x.dtype)],
                         props={"start_indices": _i64arr(start), "limit_indices": _i64arr(limit), "strides": _i64arr(strides)})
        if x.dtype in FLOATS:
            def vjp(g):
                hi = [x.shape[i] - (start[i] + (shape[i] - 1) * strides[i] + 1) if shape[i] else x.shape[i] - start[i]
                      for i in range(x.ndim)]
                return [self.pad(g[0], self.const(0, x.dtype), list(start), hi, [s - 1 for s in strides])]
            self.record([y], [x], vjp)
        return y

    def pad(self, x: Val, pv: Val, lo, hi, interior=None) -> Val:
        interior = list(interior) if interior else [0] * x.ndim
        shape = tuple(max(0, l + h + d + max(d - 1, 0) * i) for d, l, h, i in zip(x.shape, lo, hi, interior))
        (y,) = self.emit("stablehlo.pad", [x, pv], [(shape, x.dtype)],
                         props={"edge_padding_low": _i64arr(lo), "edge_padding_high": _i64arr(hi),
                                "interior_padding": _i64arr(interior)})
        if x.dtype in FLOATS:
            def vjp(g):
                # inverse: negative edge padding then strided slice
                z = self.const(0, x.dtype)
                t = self.pad(g[0], z, [-l for l in lo], [-h for h in hi], [0] * x.ndim)
                t = self.slice(t, [0] * x.ndim, t.shape, [i + 1 for i in interior])
                return [t, None]
            self.record([y], [x, pv], vjp)
        return y

    def concatenate(self, xs: Sequence[Val], dim: int) -> Val:
        xs = list(xs)
        shape = list(xs[0].shape)
        shape[dim] = sum(x.shape[dim] for x in xs)
        (y,) = self.emit("stablehlo.concatenate", xs, [(shape, xs[0].dtype)], props={"dimension": f"{dim} : i64"})
        if xs[0].dtype in FLOATS:
            def vjp(g):
                outs, off = [], 0
                for x in xs:
                    st = [0] * len(shape); li = list(shape)
                    st[dim] = off; li[dim] = off + x.shape[dim]
                    outs.append(self.slice(g[0], st, li)); off += x.shape[dim]
                return outs
            self.record([y], xs, vjp)
        return y

    def dynamic_slice(self, x: Val, starts: Sequence[Val], sizes) -> Val:
        (y,) = self.emit("stablehlo.dynamic_slice", [x, *starts], [(tuple(sizes), x.dtype)],
                         props={"slice_sizes": _i64arr(sizes)})
        if x.dtype in FLOATS:
            def vjp(g):
                return [self.dynamic_update_slice(self.zeros_like(x), g[0], starts)] + [None] * len(starts)
            self.record([y], [x, *starts], vjp)
        return y

    def dynamic_update_slice(self, x: Val, upd: Val, starts: Sequence[Val]) -> Val:
        (y,) = self.emit("stablehlo.dynamic_update_slice", [x, upd, *starts], [(x.shape, x.dtype)])
        if x.dtype in FLOATS:
            def vjp(g):
                gx = self.dynamic_update_slice(g[0], self.zeros_like(upd), starts)
                gu = self.dynamic_slice(g[0], starts, upd.shape)
                return [gx, gu] + [None] * len(starts)
            self.record([y], [x, upd, *starts], vjp)
        return y

    # ---- reductions ------------------------------------------------------
    def reduce(self, xs: Sequence[Val], inits: Sequence[Val], dims, body: Callable) -> list[Val]:
        xs, inits = list(xs), list(inits)
        dims = tuple(sorted(int(d) for d in dims))
        shape = tuple(s for i, s in enumerate(xs[0].shape) if i not in dims)
        targs = [((), x.dtype) for x in xs] * 2
        reg = self.region(targs, body)
        return self.emit("stablehlo.reduce", xs + inits, [(shape, x.dtype) for x in xs],
                         props={"dimensions": _i64arr(dims)}, regions=[reg])

    def reduce_sum(self, x: Val, dims) -> Val:
        dims = tuple(sorted(d % x.ndim for d in dims))
        (y,) = self.reduce([x], [self.const(0, x.dtype)], dims, lambda s, a, b: s.add(a, b))
        if x.dtype in FLOATS:
            kept = tuple(i for i in range(x.ndim) if i not in dims)
            self.record([y], [x], lambda g: [self.broadcast_in_dim(g[0], x.shape, kept)])
        return y

    def reduce_max(self, x: Val, dims) -> Val:
        dims = tuple(sorted(d % x.ndim for d in dims))
        init = self.const(-math.inf, x.dtype) if x.dtype in FLOATS else self.const(np.iinfo(_NP[x.dtype]).min, x.dtype)
        (y,) = self.reduce([x], [init], dims, lambda s, a, b: s.max(a, b))
        if x.dtype in FLOATS:
            kept = tuple(i for i in range(x.ndim) if i not in dims)
            def vjp(g):
                yb = self.broadcast_in_dim(y, x.shape, kept)
                loc = self.convert(self.compare(x, yb, "EQ"), x.dtype)
                cnt = self.reduce_sum(loc, dims)
                return [self.mul(self.broadcast_in_dim(self.div(g[0], cnt), x.shape, kept), loc)]
            self.record([y], [x], vjp)
        return y

    def mean(self, x: Val, dims) -> Val:
        n = int(np.prod([x.shape[d] for d in dims]))
        s = self.reduce_sum(x, dims)
        return self.div(s, self.full(s.shape, float(n), s.dtype))

    def argmax(self, x: Val, dim: int, index_dtype: str = "i32") -> Val:
        """jnp.argmax lowering: variadic (value, index) reduce; NaNs win, first
        index wins ties."""
        idx = self.iota(x.shape, index_dtype, dim)
        def body(s, av, ai, bv, bi):
            gt = s.compare(av, bv, "GT")
            nan = s.compare(av, av, "NE")
            pick = s.or_(gt, nan)
            eq = s.compare(av, bv, "EQ")
            lt = s.compare(ai, bi, "LT")
            pick_i = s.or_(pick, s.and_(eq, lt))
            return [s.select(pick, av, bv), s.select(pick_i, ai, bi)]
        init_v = self.const(-math.inf, x.dtype)
        init_i = self.const(0, index_dtype)
        return self.reduce([x, idx], [init_v, init_i], [dim], body)[1]

    # ---- contractions ----------------------------------------------------
    def dot_general(self, a: Val, b: Val, contract, batch=((), ()), out_dtype: str | None = None) -> Val:
        (lc, rc), (lb, rb) = contract, batch
        lc, rc, lb, rb = tuple(lc), tuple(rc), tuple(lb), tuple(rb)
        lfree = [i for i in range(a.ndim) if i not in lc and i not in lb]
        rfree = [i for i in range(b.ndim) if i not in rc and i not in rb]
        shape = tuple([a.shape[i] for i in lb] + [a.shape[i] for i in lfree] + [b.shape[i] for i in rfree])
        od = out_dtype or a.dtype
        dn = (f"#stablehlo.dot<lhs_batching_dimensions = {list(lb)}, rhs_batching_dimensions = {list(rb)}, "
              f"lhs_contracting_dimensions = {list(lc)}, rhs_contracting_dimensions = {list(rc)}>")
        (y,) = self.emit("stablehlo.dot_general", [a, b], [(shape, od)],
                         props={"dot_dimension_numbers": dn,
                                "precision_config": "[#stablehlo<precision DEFAULT>, #stablehlo<precision DEFAULT>]"})
        if a.dtype in FLOATS:
            nb = len(lb)
            def vjp(g):
                g0 = self.convert(g[0], a.dtype) if g[0].dtype != a.dtype else g[0]
                # d/da: contract g's rfree dims with b's rfree dims; result order batch, lfree, (b's contract dims)
                g_rfree = tuple(range(nb + len(lfree), nb + len(lfree) + len(rfree)))
                da = self.dot_general(g0, b, (g_rfree, tuple(rfree)), (tuple(range(nb)), rb))
                # da dims: batch..., lfree..., rc-ordered dims -> permute to a's layout
                src = list(lb) + lfree + [lc[i] for i in np.argsort(rc)]
                da = self.transpose(da, tuple(int(i) for i in np.argsort(src)))
                g_lfree = tuple(range(nb, nb + len(lfree)))
                db = self.dot_general(a, g0, (tuple(lfree), g_lfree), (lb, tuple(range(nb))))
                # db dims: batch..., (a's contract dims sorted by a index -> matching rc), rfree...
                srcb = list(rb) + [rc[i] for i in np.argsort(lc)] + rfree
                db = self.transpose(db, tuple(int(i) for i in np.argsort(srcb)))
                return [da, db]
            self.record([y], [a, b], vjp)
        return y

    def matmul(self, a: Val, b: Val) -> Val:
        """[..., m, k] @ [k, n]"""
        return self.dot_general(a, b, ((a.ndim - 1,), (0,)))

    def conv(self, x: Val, w: Val, strides=(1, 1), padding=((0, 0), (0, 0)), lhs_dilation=(1, 1),
             rhs_dilation=(1, 1), dn=("b01f", "01io", "b01f"), feature_group_count=1, batch_group_count=1) -> Val:
        """stablehlo.convolution, 2 spatial dims. `dn` strings use b/f/0/1 for
        input and output and i/o/0/1 for the kernel."""
        ls, rs, os_ = dn
        nsp = len(ls) - 2
        def dim(spec, c): return spec.index(c)
        padding = [tuple(p) for p in padding]
        out = [0] * (nsp + 2)
        n = x.shape[dim(ls, "b")] // batch_group_count
        o = w.shape[dim(rs, "o")]
        out[dim(os_, "b")] = n
        out[dim(os_, "f")] = o
        for s in range(nsp):
            i = x.shape[dim(ls, str(s))]
            k = w.shape[dim(rs, str(s))]
            idil = 0 if i == 0 else 1 + lhs_dilation[s] * (i - 1)
            kdil = 0 if k == 0 else 1 + rhs_dilation[s] * (k - 1)
            tot = idil + padding[s][0] + padding[s][1]
            out[dim(os_, str(s))] = 0 if tot < kdil else (tot - kdil) // strides[s] + 1
        def spec(s): return "[" + ", ".join(s) + "]"
        props = {
            "batch_group_count": f"{batch_group_count} : i64",
            "feature_group_count": f"{feature_group_count} : i64",
            "dimension_numbers": f"#stablehlo.conv<{spec(ls)}x{spec(rs)}->{spec(os_)}>",
            "lhs_dilation": _i64arr(lhs_dilation), "rhs_dilation": _i64arr(rhs_dilation),
            "window_strides": _i64arr(strides),
            "padding": f"dense<{[list(p) for p in padding]}> : tensor<{nsp}x2xi64>",
            "precision_config": "[#stablehlo<precision DEFAULT>, #stablehlo<precision DEFAULT>]",
        }
        (y,) = self.emit("stablehlo.convolution", [x, w], [(tuple(out), x.dtype)], props=props)
        if x.dtype in FLOATS:
            def dil(n, d): return 0 if n == 0 else 1 + d * (n - 1)
            def vjp(g):
                assert feature_group_count == 1 and batch_group_count == 1, "grouped conv VJP not provided"
                g0 = g[0]
                isp = [x.shape[dim(ls, str(s))] for s in range(nsp)]
                ksp = [w.shape[dim(rs, str(s))] for s in range(nsp)]
                osp = [y.shape[dim(os_, str(s))] for s in range(nsp)]
                # input gradient (jax _conv_general_dilated_transpose_lhs)
                pads = []
                for s in range(nsp):
                    before = dil(ksp[s], rhs_dilation[s]) - padding[s][0] - 1
                    after = dil(isp[s], lhs_dilation[s]) + dil(ksp[s], rhs_dilation[s]) - 1 - dil(osp[s], strides[s]) - before
                    pads.append((before, after))
                t_rs = rs.replace("i", "#").replace("o", "i").replace("#", "o")
                wr = self.reverse(w, [dim(rs, str(s)) for s in range(nsp)])
                dx = self.conv(g0, wr, strides=lhs_dilation, padding=pads, lhs_dilation=strides,
                               rhs_dilation=rhs_dilation, dn=(os_, t_rs, ls))
                # kernel gradient (jax _conv_general_dilated_transpose_rhs)
                pads = []
                for s in range(nsp):
                    lo = padding[s][0]
                    hi = dil(osp[s], strides[s]) - dil(isp[s], lhs_dilation[s]) + dil(ksp[s], rhs_dilation[s]) - lo - 1
                    pads.append((lo, hi))
                sw = lambda sp, a, b_: sp.replace(a, "#").replace(b_, a).replace("#", b_)
                l_t = sw(ls, "b", "f")
                r_t = os_.replace("b", "i").replace("f", "o")   # g as kernel: batch contracts, features are outputs
                o_t = rs.replace("i", "b").replace("o", "f")
                dw = self.conv(x, g0, strides=rhs_dilation, padding=pads, lhs_dilation=lhs_dilation,
                               rhs_dilation=strides, dn=(l_t, r_t, o_t))
                return [dx, dw]
            self.record([y], [x, w], vjp)
        return y

    # ---- indexing --------------------------------------------------------
    def take_rows(self, table: Val, idx: Val) -> Val:
        """table[idx] for a 2-D table and integer idx of any shape (the
        `jnp.take(table, idx, axis=0)` gather)."""
        assert table.ndim == 2
        d = table.shape[1]
        idx2 = self.reshape(idx, (*idx.shape, 1))
        n = idx.ndim
        dn = (f"#stablehlo.gather<offset_dims = [{n}], collapsed_slice_dims = [0], "
              f"start_index_map = [0], index_vector_dim = {n}>")
        (y,) = self.emit("stablehlo.gather", [table, idx2], [((*idx.shape, d), table.dtype)],
                         props={"dimension_numbers": dn, "indices_are_sorted": "false",
                                "slice_sizes": _i64arr((1, d))})
        if table.dtype in FLOATS:
            def vjp(g):
                sdn = (f"#stablehlo.scatter<update_window_dims = [{n}], inserted_window_dims = [0], "
                       f"scatter_dims_to_operand_dims = [0], index_vector_dim = {n}>")
                reg = self.region([((), table.dtype)] * 2, lambda s, a, b_: s.add(a, b_))
                (dt,) = self.emit("stablehlo.scatter", [self.zeros_like(table), idx2, g[0]],
                                  [(table.shape, table.dtype)],
                                  props={"scatter_dimension_numbers": sdn, "indices_are_sorted": "false",
                                         "unique_indices": "false"}, regions=[reg])
                return [dt, None]
            self.record([y], [table, idx], vjp)
        return y

    def scatter_rows(self, operand: Val, idx: Val, updates: Val, op: str = "add") -> Val:
        """operand.at[idx].<op>(updates) for integer idx of any shape and updates of shape idx.shape + operand.shape[1:]
        (`op` in add, multiply, minimum, maximum, or "set"); no gradient."""
        n = idx.ndim
        idx2 = self.reshape(idx, (*idx.shape, 1))
        win = list(range(n, n + operand.ndim - 1))
        sdn = (f"#stablehlo.scatter<update_window_dims = {win}, inserted_window_dims = [0], "
               f"scatter_dims_to_operand_dims = [0], index_vector_dim = {n}>")
        if callable(op):
            body = op                          # any update computation: body(sub, current element, update element)
        else:
            body = (lambda s, a, u: u) if op == "set" else (lambda s, a, u: s._binary(op, a, u))
        reg = self.region([((), operand.dtype)] * 2, body)
        (y,) = self.emit("stablehlo.scatter", [operand, idx2, updates], [(operand.shape, operand.dtype)],
                         props={"scatter_dimension_numbers": sdn, "indices_are_sorted": "false",
                                "unique_indices": "false"}, regions=[reg])
        return y

    @staticmethod
    def _window_props(rank, window, strides, padding, base_dilations=None, window_dilations=None):
        strides = tuple(strides or (1,) * rank)
        padding = tuple(tuple(p) for p in (padding or ((0, 0),) * rank))
        props = {"window_dimensions": "array<i64: " + ", ".join(str(int(v)) for v in window) + ">",
                 "window_strides": "array<i64: " + ", ".join(str(int(v)) for v in strides) + ">",
                 "padding": "dense<[" + ", ".join(f"[{int(a)}, {int(b)}]" for a, b in padding) + f"]> : tensor<{rank}x2xi64>"}
        if base_dilations is not None:
            props["base_dilations"] = "array<i64: " + ", ".join(str(int(v)) for v in base_dilations) + ">"
        if window_dilations is not None:
            props["window_dilations"] = "array<i64: " + ", ".join(str(int(v)) for v in window_dilations) + ">"
        return props, strides, padding

    def reduce_window(self, x: Val, init, op: str, window, strides=None, padding=None, base_dilations=None,
                      window_dilations=None) -> Val:
        """stablehlo.reduce_window with the body `op` (add, maximum, minimum, multiply, and, or): what lax.reduce_window,
        pooling and cumulative sums lower to. `init` is a scalar Val or a Python number. No gradient."""
        rank = x.ndim
        props, strides, padding = self._window_props(rank, window, strides, padding, base_dilations, window_dilations)
        bd = tuple(base_dilations or (1,) * rank)
        wd = tuple(window_dilations or (1,) * rank)
        shape = []
        for d in range(rank):
            padded = (x.shape[d] - 1) * bd[d] + 1 + padding[d][0] + padding[d][1] if x.shape[d] else 0
            win = (window[d] - 1) * wd[d] + 1
            shape.append(0 if padded < win else (padded - win) // strides[d] + 1)
        if not isinstance(init, Val):
            init = self.const(init, x.dtype)
        reg = self.region([((), x.dtype)] * 2, lambda s, a, b: s._binary(op, a, b))
        (y,) = self.emit("stablehlo.reduce_window", [x, init], [(tuple(shape), x.dtype)], props=props, regions=[reg])
        return y

    def select_and_scatter(self, operand: Val, source: Val, init, window, strides=None, padding=None,
                           select: str = "GE", scatter: str = "add") -> Val:
        """stablehlo.select_and_scatter (the gradient of max / min pooling): per window the element chosen by
        compare(a, b, `select`) receives the window's `source` value, combined with `scatter`. No gradient."""
        rank = operand.ndim
        props, _, _ = self._window_props(rank, window, strides, padding)
        if not isinstance(init, Val):
            init = self.const(init, operand.dtype)
        sel = self.region([((), operand.dtype)] * 2, lambda s, a, b: s.compare(a, b, select))
        sc = self.region([((), operand.dtype)] * 2, lambda s, a, b: s._binary(scatter, a, b))
        (y,) = self.emit("stablehlo.select_and_scatter", [operand, source, init], [(operand.shape, operand.dtype)],
                         props=props, regions=[sel, sc])
        return y

    def sort(self, xs: Sequence[Val], dim: int = -1, comparator: Callable | None = None, *, descending: bool = False,
             num_keys: int = 1, stable: bool = True) -> list[Val]:
        """stablehlo.sort of several operands of one shape along `dim`. `comparator(sub, a0, b0, a1, b1, ...)` returns
        the i1 "a goes before b"; by default what jnp.sort / lax.sort_key_val emit: the first `num_keys` operands
        compared lexicographically, floats in their total order (-NaN < -inf < ... < -0 < +0 < ... < inf < NaN).
        No gradient."""
        xs = list(xs)
        dim = dim % xs[0].ndim
        assert all(x.shape == xs[0].shape for x in xs)

        def default(sub, *ab):
            direction = "GT" if descending else "LT"
            out = None
            for k in reversed(range(num_keys)):
                a, b = ab[2 * k], ab[2 * k + 1]
                ctype = "TOTALORDER" if a.dtype in FLOATS else None
                first = sub.compare(a, b, direction, ctype)
                if out is None:
                    out = first
                else:
                    out = sub.or_(first, sub.and_(sub.compare(a, b, "EQ", ctype), out))
            return out

        targs = []
        for x in xs:
            targs += [((), x.dtype)] * 2
        reg = self.region(targs, comparator or default)
        return list(self.emit("stablehlo.sort", xs, [(x.shape, x.dtype) for x in xs],
                              props={"dimension": f"{dim} : i64", "is_stable": "true" if stable else "false"}, regions=[reg]))

    def rng_bit_generator(self, state: Val, shape, dtype: str = "ui32", algorithm: str = "DEFAULT") -> list[Val]:
        """stablehlo.rng_bit_generator: (new state, random bits of `shape` and integer `dtype`) from a state of two
        (or three) 64-bit words or as many 32-bit ones, what lax.rng_bit_generator emits."""
        return list(self.emit("stablehlo.rng_bit_generator", [state], [(state.shape, state.dtype), (tuple(shape), dtype)],
                              props={"rng_algorithm": f"#stablehlo<rng_algorithm {algorithm}>"}))

    def cholesky(self, a: Val, lower: bool = True) -> Val:
        """stablehlo.cholesky of a batch of symmetric positive definite matrices. No gradient."""
        return self.emit("stablehlo.cholesky", [a], [(a.shape, a.dtype)], props={"lower": "true" if lower else "false"})[0]

    def triangular_solve(self, a: Val, b: Val, *, left_side: bool = True, lower: bool = True, unit_diagonal: bool = False,
                         transpose_a: str = "NO_TRANSPOSE") -> Val:
        """stablehlo.triangular_solve: op(a) x = b (left_side) or x op(a) = b. No gradient."""
        tf = lambda v: "true" if v else "false"
        return self.emit("stablehlo.triangular_solve", [a, b], [(b.shape, b.dtype)],
                         props={"left_side": tf(left_side), "lower": tf(lower), "unit_diagonal": tf(unit_diagonal),
                                "transpose_a": f"#stablehlo<transpose {transpose_a}>"})[0]

    def top_k(self, x: Val, k: int) -> list[Val]:
        """chlo.top_k: the k largest values along the last dimension in descending order and their positions (i32);
        equal values keep the order of their positions. No gradient."""
        assert 0 <= k <= x.shape[-1]
        shape = x.shape[:-1] + (k,)
        return list(self.emit("chlo.top_k", [x], [(shape, x.dtype), (shape, "i32")], props={"k": f"{k} : i64"}))

    def scatter(self, operand: Val, indices: Val, updates: Val, op: str = "add", *, update_window_dims=(),
                inserted_window_dims=(), scatter_dims_to_operand_dims=(), index_vector_dim=None, input_batching_dims=(),
                scatter_indices_batching_dims=()) -> Val:
        """stablehlo.scatter with explicit dimension numbers (`op` names a binary operation, or "set", or is a function
        building the update computation); no gradient."""
        ivd = indices.ndim if index_vector_dim is None else index_vector_dim
        sdn = (f"#stablehlo.scatter<update_window_dims = {list(update_window_dims)}, inserted_window_dims = {list(inserted_window_dims)}, "
               + (f"input_batching_dims = {list(input_batching_dims)}, scatter_indices_batching_dims = {list(scatter_indices_batching_dims)}, "
                  if input_batching_dims else "")
               + f"scatter_dims_to_operand_dims = {list(scatter_dims_to_operand_dims)}, index_vector_dim = {ivd}>")
        if callable(op):
            body = op                          # any update computation: body(sub, current element, update element)
        else:
            body = (lambda s, a, u: u) if op == "set" else (lambda s, a, u: s._binary(op, a, u))
        reg = self.region([((), operand.dtype)] * 2, body)
        (y,) = self.emit("stablehlo.scatter", [operand, indices, updates], [(operand.shape, operand.dtype)],
                         props={"scatter_dimension_numbers": sdn, "indices_are_sorted": "false",
                                "unique_indices": "false"}, regions=[reg])
        return y

    def take_along_last(self, x: Val, idx: Val) -> Val:
        """x[i, idx[i]] for 2-D x and 1-D idx (jnp.take_along_axis on the last
        axis, lowered with operand batching dims)."""
        assert x.ndim == 2 and idx.ndim == 1
        idx2 = self.reshape(idx, (idx.shape[0], 1))
        dn = ("#stablehlo.gather<collapsed_slice_dims = [1], operand_batching_dims = [0], "
              "start_indices_batching_dims = [0], start_index_map = [1], index_vector_dim = 1>")
        (y,) = self.emit("stablehlo.gather", [x, idx2], [((x.shape[0],), x.dtype)],
                         props={"dimension_numbers": dn, "indices_are_sorted": "false",
                                "slice_sizes": _i64arr((1, 1))})
        if x.dtype in FLOATS:
            def vjp(g):
                oh = self.compare(self.iota(x.shape, idx.dtype, 1), self.broadcast_in_dim(idx, x.shape, (0,)), "EQ")
                return [self.select(oh, self.broadcast_in_dim(g[0], x.shape, (0,)), self.zeros_like(x)), None]
            self.record([y], [x, idx], vjp)
        return y

    # ---- control flow / collectives ---------------------------------------
    def while_(self, init: Sequence[Val], cond: Callable, body: Callable) -> list[Val]:
        init = list(init)
        types = [(v.shape, v.dtype) for v in init]
        was = self.root.taping
        self.root.taping = False
        try:
            rc = self.region(types, cond)
            rb = self.region(types, body)
        finally:
            self.root.taping = was
        return self.emit("stablehlo.while", init, types, regions=[rc, rb])

    def case(self, index: Val, branches: Sequence[Callable], result_types) -> list[Val]:
        was = self.root.taping
        self.root.taping = False
        try:
            regs = [self.region([], br) for br in branches]
        finally:
            self.root.taping = was
        return self.emit("stablehlo.case", [index], list(result_types), regions=regs)

    def all_reduce_sum(self, xs: Sequence[Val], n_devices: int, channel: int = 1) -> list[Val]:
        """psum over all partitions of a fully-manual shard_map body."""
        xs = list(xs)
        groups = f"dense<[{list(range(n_devices))}]> : tensor<1x{n_devices}xi64>"
        outs = []
        for i, x in enumerate(xs):
            reg = self.region([((), x.dtype)] * 2, lambda s, a, b_: s.add(a, b_))
            (y,) = self.emit("stablehlo.all_reduce", [x], [(x.shape, x.dtype)],
                             props={"replica_groups": groups, "use_global_device_ids": "unit",
                                    "channel_handle": f"#stablehlo.channel_handle<handle = {channel + i}, type = 1>"},
                             regions=[reg])
            self.record([y], [x], lambda g: [g[0]])
            outs.append(y)
        return outs

    def all_gather(self, x: Val, n_devices: int, dim: int = 0, channel: int = 100) -> Val:
        """lax.all_gather(..., tiled=True) over all partitions of a fully-manual shard_map body: the operands of the
        partitions concatenated along `dim` in partition order."""
        groups = f"dense<[{list(range(n_devices))}]> : tensor<1x{n_devices}xi64>"
        shape = tuple(d * n_devices if i == dim else d for i, d in enumerate(x.shape))
        (y,) = self.emit("stablehlo.all_gather", [x], [(shape, x.dtype)],
                         props={"all_gather_dim": f"{dim} : i64", "replica_groups": groups, "use_global_device_ids": "unit",
                                "channel_handle": f"#stablehlo.channel_handle<handle = {channel}, type = 1>"})
        return y

    def partition_id(self) -> Val:
        return self.emit("stablehlo.partition_id", [], [((), "ui32")])[0]

    def custom_call(self, target: str, xs: Sequence[Val], result_types, attrs: dict | None = None) -> list[Val]:
        props = {"call_target_name": f'"{target}"'}
        props.update(attrs or {})
        return self.emit("stablehlo.custom_call", list(xs), list(result_types), props=props)

    def optimization_barrier(self, xs: Sequence[Val]) -> list[Val]:
        xs = list(xs)
        return self.emit("stablehlo.optimization_barrier", xs, [(x.shape, x.dtype) for x in xs])

    # ---- differentiation ---------------------------------------------------
    def grad(self, loss: Val, wrt: Sequence[Val], seed: Val | None = None) -> list[Val]:
        """Cotangents of `loss` with respect to `wrt` by walking the tape in
        reverse; nothing emitted during the walk is taped."""
        ct: dict[str, Val] = {loss.name: seed if seed is not None else self.const(1.0, loss.dtype, loss.shape)}
        was = self.root.taping
        self.root.taping = False
        try:
            for outs, ins, vjp in reversed(self.tape):
                if not any(o.name in ct for o in outs):
                    continue
                gs = [ct.get(o.name) for o in outs]
                gs = [g if g is not None else self.zeros_like(o) for g, o in zip(gs, outs)]
                for i, gi in zip(ins, vjp(gs)):
                    if gi is None or isinstance(i, _Stopped):
                        continue
                    assert gi.shape == i.shape, (i, gi)
                    ct[i.name] = self.add(ct[i.name], gi) if i.name in ct else gi
        finally:
            self.root.taping = was
        return [ct[w.name] if w.name in ct else self.zeros_like(w) for w in wrt]

    # ---- module text -------------------------------------------------------
    def module(self, results: Sequence[Val], name: str = "jit_step", num_partitions: int = 1,
               num_replicas: int = 1) -> str:
        assert self is self.root
        results = list(results)
        sig = ", ".join(f"{a.name}: {a.type}" + (f" {{{self.arg_attrs[a.name]}}}" if a.name in self.arg_attrs else "")
                        for a in self.args)
        rt = ", ".join(r.type for r in results)
        body = list(self.lines)
        body.append(f'    "func.return"({", ".join(r.name for r in results)}) : ({rt}) -> ()')
        head = (f"module @{name} attributes {{mhlo.num_partitions = {num_partitions} : i32, "
                f"mhlo.num_replicas = {num_replicas} : i32}} {{\n"
                f"  func.func public @main({sig}) -> ({rt}) {{\n")
        return head + "\n".join("  " + l for l in body) + "\n  }\n}\n"


class _Stopped(Val):
    """A value whose uses do not propagate cotangents (lax.stop_gradient)."""

    def __init__(self, v: Val):
        super().__init__(v.b, v.name, v.shape, v.dtype)


def _i64arr(xs) -> str:
    xs = [int(x) for x in xs]
    return "array<i64: " + ", ".join(str(x) for x in xs) + ">" if xs else "array<i64>"
