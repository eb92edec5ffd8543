"""TEST INFRASTRUCTURE (oracle side): a small reader for StableHLO modules in
MLIR text form, independent of the C++ parser in the product so that the two
cross-check each other.

Accepts the generic operation form (`%r = "stablehlo.add"(%a, %b) : (...) ->
...`, with `<{properties}>`, regions and `{attributes}`) plus the custom
("pretty") form of the operations that appear in the reference's own raw-MLIR
test (tests/test_ops.py:216-269: constant, unary/binary elementwise,
composite, return) and a few more common ones.
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field

import numpy as np


@dataclass
class TType:
    shape: tuple
    dtype: str          # 'f32', 'bf16', 'i32', 'ui32', 'i1', 'token', ...

    def __str__(self):
        return "tensor<" + "".join(f"{d}x" for d in self.shape) + self.dtype + ">"


@dataclass
class Op:
    name: str
    operands: list
    results: list            # names
    result_types: list       # TType
    attrs: dict              # name -> raw text
    regions: list            # list[Block]


@dataclass
class Block:
    args: list = field(default_factory=list)        # [(name, TType)]
    ops: list = field(default_factory=list)


@dataclass
class Func:
    name: str
    args: list
    arg_attrs: list
    result_types: list
    body: Block
    private: bool = False


@dataclass
class Module:
    name: str
    attrs: dict
    funcs: dict


_ID = re.compile(r"[A-Za-z_][\w.$]*")
_SSA = re.compile(r"%[\w.$#-]+")
_NUM = re.compile(r"[-+]?(0x[0-9A-Fa-f]+|(\d+\.?\d*([eE][-+]?\d+)?|inf|nan))")

_SAME_TYPE_PRETTY = {
    "add", "subtract", "multiply", "divide", "maximum", "minimum", "power", "remainder", "atan2", "and", "or",
    "xor", "shift_left", "shift_right_logical", "shift_right_arithmetic", "exponential", "log", "sqrt", "rsqrt",
    "negate", "abs", "floor", "ceil", "sine", "cosine", "tanh", "tan", "logistic", "sign", "log_plus_one",
    "exponential_minus_one", "cbrt", "not", "popcnt", "count_leading_zeros", "round_nearest_even",
    "round_nearest_afz",
}


class Parser:
    def __init__(self, text: str):
        self.s = text
        self.i = 0

    # -- low level ---------------------------------------------------------
    def ws(self):
        s, n = self.s, len(self.s)
        while self.i < n:
            c = s[self.i]
            if c in " \t\r\n":
                self.i += 1
            elif s.startswith("//", self.i):
                j = s.find("\n", self.i)
                self.i = n if j < 0 else j
            else:
                break

    def peek(self, lit: str) -> bool:
        self.ws()
        return self.s.startswith(lit, self.i)

    def accept(self, lit: str) -> bool:
        if self.peek(lit):
            self.i += len(lit)
            return True
        return False

    def expect(self, lit: str):
        if not self.accept(lit):
            raise SyntaxError(f"expected {lit!r} at {self.i}: {self.s[self.i:self.i + 60]!r}")

    def rx(self, pat) -> str:
        self.ws()
        m = pat.match(self.s, self.i)
        if not m:
            raise SyntaxError(f"expected {pat.pattern} at {self.i}: {self.s[self.i:self.i + 60]!r}")
        self.i = m.end()
        return m.group(0)

    def string(self) -> str:
        self.ws()
        assert self.s[self.i] == '"', self.s[self.i:self.i + 40]
        j = self.i + 1
        while self.s[j] != '"':
            j += 2 if self.s[j] == "\\" else 1
        out = self.s[self.i + 1:j]
        self.i = j + 1
        return out

    def balanced(self, stops: str) -> str:
        """Raw text up to (not including) the first top-level char in `stops`."""
        self.ws()
        depth, j, s = 0, self.i, self.s
        while True:
            c = s[j]
            if c == '"':
                j += 1
                while s[j] != '"':
                    j += 2 if s[j] == "\\" else 1
            elif c in "([{<":
                depth += 1
            elif c in ")]}>":
                if depth == 0 and c in stops:
                    break
                if c == ">" and s[j - 1] == "-":
                    pass            # '->'
                else:
                    depth -= 1
            elif depth == 0 and c in stops:
                break
            j += 1
        out = s[self.i:j].strip()
        self.i = j
        return out

    # -- types ----------------------------------------------------------------
    def type(self) -> TType:
        self.ws()
        if self.accept("tensor<"):
            dims = []
            while True:
                m = re.compile(r"(\d+)x").match(self.s, self.i)
                if not m:
                    break
                dims.append(int(m.group(1)))
                self.i = m.end()
            dt = self.rx(_ID)
            self.expect(">")
            return TType(tuple(dims), dt)
        if self.accept("!stablehlo.token"):
            return TType((), "token")
        raise SyntaxError(f"type at {self.s[self.i:self.i + 40]!r}")

    def type_list(self) -> list:
        if self.accept("("):
            out = []
            if not self.accept(")"):
                while True:
                    out.append(self.type())
                    if not self.accept(","):
                        break
                self.expect(")")
            return out
        return [self.type()]

    # -- attributes -------------------------------------------------------------
    def attr_dict(self, close: str) -> dict:
        out = {}
        if self.accept(close):
            return out
        while True:
            self.ws()
            key = self.string() if self.s[self.i] == '"' else self.rx(_ID)
            if self.accept("="):
                out[key] = self.balanced("," + close[0])
            else:
                out[key] = "unit"
            if not self.accept(","):
                break
        self.expect(close)
        return out

    # -- module / function ------------------------------------------------------
    def module(self) -> Module:
        name, attrs = "", {}
        wrapped = False
        self.skip_location_aliases()
        if self.accept("module"):
            wrapped = True
            if self.peek("@"):
                self.i += 1
                name = self.rx(_ID)
            if self.accept("attributes"):
                self.expect("{")
                attrs = self.attr_dict("}")
            self.expect("{")
        funcs = {}
        while self.peek("func.func"):
            f = self.func()
            funcs[f.name] = f
        if wrapped:
            self.expect("}")
        self.skip_loc()
        self.skip_location_aliases()
        return Module(name, attrs, funcs)

    def skip_loc(self):
        if self.accept("loc("):
            self.balanced(")"); self.expect(")")

    def skip_location_aliases(self):
        """'#loc3 = loc(...)' lines of a module printed with debug information."""
        while self.peek("#loc"):
            j = self.s.find("\n", self.i)
            self.i = len(self.s) if j < 0 else j

    def func(self) -> Func:
        self.expect("func.func")
        private = False
        for vis in ("public", "private"):
            if self.accept(vis):
                private = vis == "private"
        self.expect("@")
        name = self.rx(re.compile(r"[\w.$]+"))
        self.expect("(")
        args, arg_attrs = [], []
        if not self.accept(")"):
            while True:
                n = self.rx(_SSA)
                self.expect(":")
                t = self.type()
                a = {}
                if self.accept("{"):
                    a = self.attr_dict("}")
                if self.accept("loc("):
                    self.balanced(")"); self.expect(")")
                args.append((n, t)); arg_attrs.append(a)
                if not self.accept(","):
                    break
            self.expect(")")
        rts = []
        if self.accept("->"):
            if self.accept("("):
                if not self.accept(")"):
                    while True:
                        rts.append(self.type())
                        if self.accept("{"):
                            self.attr_dict("}")
                        if not self.accept(","):
                            break
                    self.expect(")")
            else:
                rts = [self.type()]
        if self.accept("attributes"):
            self.expect("{"); self.attr_dict("}")
        self.expect("{")
        body = Block(args=list(args))
        self.ops_until(body, "}")
        self.expect("}")
        self.skip_loc()
        return Func(name, args, arg_attrs, rts, body, private)

    def ops_until(self, block: Block, close: str):
        while not self.peek(close):
            block.ops.append(self.op())

    def region(self) -> Block:
        self.expect("{")
        blk = Block()
        if self.accept("^"):
            self.rx(_ID)
            if self.accept("("):
                while True:
                    n = self.rx(_SSA)
                    self.expect(":")
                    blk.args.append((n, self.type()))
                    if self.accept("loc("):
                        self.balanced(")"); self.expect(")")
                    if not self.accept(","):
                        break
                self.expect(")")
            self.expect(":")
        self.ops_until(blk, "}")
        self.expect("}")
        return blk

    # -- operations ---------------------------------------------------------------
    def op(self) -> Op:
        self.ws()
        results = []
        if self.s[self.i] == "%":
            while True:
                n = self.rx(_SSA)
                if ":" in n:
                    raise SyntaxError(n)
                if self.accept(":"):
                    k = int(self.rx(re.compile(r"\d+")))
                    results.extend(f"{n}#{j}" for j in range(k))
                else:
                    results.append(n)
                if not self.accept(","):
                    break
            self.expect("=")
        self.ws()
        if self.s[self.i] == '"':
            op = self.generic(results)
        else:
            op = self.pretty(results)
        if self.accept("loc("):
            self.balanced(")"); self.expect(")")
        return op

    def operands(self, close=")") -> list:
        out = []
        if self.accept(close):
            return out
        while True:
            out.append(self.rx(_SSA))
            if not self.accept(","):
                break
        self.expect(close)
        return out

    def generic(self, results) -> Op:
        name = self.string()
        self.expect("(")
        operands = self.operands()
        attrs = {}
        if self.accept("<{"):
            attrs.update(self.attr_dict("}>"))
        regions = []
        if self.peek("("):
            self.expect("(")
            while True:
                regions.append(self.region())
                if not self.accept(","):
                    break
            self.expect(")")
        if self.accept("{"):
            attrs.update(self.attr_dict("}"))
        self.expect(":")
        self.type_list()
        self.expect("->")
        rts = self.type_list()
        if len(results) == 1 and len(rts) > 1:
            raise SyntaxError("result arity")
        return Op(name, operands, results, rts, attrs, regions)

    def pretty(self, results) -> Op:
        name = self.rx(re.compile(r"[\w.]+"))
        short = name.split(".", 1)[1] if name.startswith("stablehlo.") else name
        if name in ("return", "func.return", "stablehlo.return"):
            ops = []
            if self.peek("%"):
                while True:
                    ops.append(self.rx(_SSA))
                    if not self.accept(","):
                        break
                self.expect(":")
                while True:
                    self.type()
                    if not self.accept(","):
                        break
            return Op("func.return" if name != "stablehlo.return" else name, ops, [], [], {}, [])
        if short == "constant":
            raw = self.balanced("\n")
            # 'dense<...> : tensor<..>'
            t = Parser(raw[raw.rindex(": ") + 2:]).type()
            return Op("stablehlo.constant", [], results, [t], {"value": raw}, [])
        if short in _SAME_TYPE_PRETTY or (short == "clamp"):
            ops = [self.rx(_SSA)]
            while self.accept(","):
                ops.append(self.rx(_SSA))
            attrs = {}
            if self.accept("{"):
                attrs = self.attr_dict("}")
            self.expect(":")
            if self.peek("("):                     # (operand types) -> result type: clamp with scalar bounds
                self.type_list(); self.expect("->")
                return Op(name, ops, results, self.type_list(), attrs, [])
            t = self.type()
            while self.accept(","):
                t = self.type()
            return Op(name, ops, results, [t], attrs, [])
        if short == "composite":
            target = self.string()
            ops = []
            while self.peek("%"):
                ops.append(self.rx(_SSA))
                self.accept(",")
            attrs = {"name": f'"{target}"'}
            if self.accept("{"):
                attrs.update(self.attr_dict("}"))
            self.expect(":")
            self.type_list(); self.expect("->")
            return Op("stablehlo.composite", ops, results, self.type_list(), attrs, [])
        if short in ("convert", "reshape", "bitcast_convert", "is_finite", "optimization_barrier"):
            ops = [self.rx(_SSA)]
            while self.accept(","):
                ops.append(self.rx(_SSA))
            self.expect(":")
            if not self.peek("("):                 # results typed like the operands
                ts = [self.type()]
                while self.accept(","):
                    ts.append(self.type())
                if self.accept("->"):
                    ts = self.type_list()
                return Op(name, ops, results, ts, {}, [])
            self.type_list(); self.expect("->")
            return Op(name, ops, results, self.type_list(), {}, [])
        if short == "compare":
            d = self.rx(_ID); self.expect(",")
            a = self.rx(_SSA); self.expect(",")
            b = self.rx(_SSA)
            attrs = {"comparison_direction": f"#stablehlo<comparison_direction {d}>"}
            if self.accept(","):
                attrs["compare_type"] = f"#stablehlo<comparison_type {self.rx(_ID)}>"
            self.expect(":"); self.type_list(); self.expect("->")
            return Op(name, [a, b], results, self.type_list(), attrs, [])
        if short == "select":
            ops = [self.rx(_SSA)]
            while self.accept(","):
                ops.append(self.rx(_SSA))
            self.expect(":")
            ts = [self.type()]
            while self.accept(","):
                ts.append(self.type())
            return Op(name, ops, results, [ts[-1]], {}, [])
        if short in ("broadcast_in_dim", "transpose"):
            a = self.rx(_SSA); self.expect(","); self.expect("dims"); self.expect("=")
            self.expect("["); dims = self.balanced("]"); self.expect("]")
            key = "broadcast_dimensions" if short == "broadcast_in_dim" else "permutation"
            self.expect(":"); self.type_list(); self.expect("->")
            return Op(name, [a], results, self.type_list(), {key: f"array<i64: {dims}>" if dims else "array<i64>"}, [])
        if short == "reduce":
            # stablehlo.reduce(%a init: %i) applies stablehlo.add across dimensions = [1] : (..) -> ..
            self.expect("(")
            ins, inits = [], []
            while True:
                ins.append(self.rx(_SSA)); self.expect("init:"); inits.append(self.rx(_SSA))
                if self.accept(","):
                    continue
                self.expect(")")
                save = self.i
                if self.accept(",") and self.accept("("):      # (%a init: %i), (%b init: %j)
                    continue
                self.i = save
                break
            if not self.accept("applies"):
                # across dimensions = [..] : types reducer(%a: t, %b: t) (%c: t, %d: t) { ... }
                self.expect("across"); self.expect("dimensions"); self.expect("=")
                self.expect("["); dims = self.balanced("]"); self.expect("]")
                self.expect(":"); self.type_list(); self.expect("->")
                rts = self.type_list()
                self.expect("reducer")
                firsts, seconds = [], []
                while self.accept("("):
                    n1 = self.rx(_SSA); self.expect(":"); t1 = self.type(); self.expect(",")
                    n2 = self.rx(_SSA); self.expect(":"); t2 = self.type(); self.expect(")")
                    firsts.append((n1, t1)); seconds.append((n2, t2))
                blk = Block(args=firsts + seconds)
                self.expect("{")
                self.ops_until(blk, "}")
                self.expect("}")
                return Op(name, ins + inits, results, rts,
                          {"dimensions": f"array<i64: {dims}>" if dims else "array<i64>"}, [blk])
            body = self.rx(re.compile(r"[\w.]+"))
            self.expect("across"); self.expect("dimensions"); self.expect("=")
            self.expect("["); dims = self.balanced("]"); self.expect("]")
            self.expect(":"); self.type_list(); self.expect("->")
            rts = self.type_list()
            st = TType((), rts[0].dtype)
            blk = Block(args=[("%acc", st), ("%val", st)],
                        ops=[Op(body, ["%acc", "%val"], ["%red"], [st], {}, []),
                             Op("stablehlo.return", ["%red"], [], [], {}, [])])
            return Op(name, ins + inits, results, rts,
                      {"dimensions": f"array<i64: {dims}>" if dims else "array<i64>"}, [blk])
        if name in ("call", "func.call"):
            self.expect("@")
            callee = self.rx(re.compile(r"[\w.$]+"))
            self.expect("(")
            ops = self.operands()
            self.expect(":"); self.type_list(); self.expect("->")
            return Op("func.call", ops, results, self.type_list(), {"callee": "@" + callee}, [])
        def functional(ops, attrs, regions=()):
            self.expect(":"); self.type_list(); self.expect("->")
            return Op(name, ops, results, self.type_list(), attrs, list(regions))

        def bracket() -> str:
            self.expect("["); d = self.balanced("]"); self.expect("]")
            return f"array<i64: {d}>" if d else "array<i64>"

        def keyword(kw) -> str:
            self.expect(","); self.expect(kw); self.expect("=")
            return bracket()
        if short == "iota":
            self.expect("dim"); self.expect("=")
            d = self.rx(re.compile(r"\d+"))
            self.expect(":")
            return Op(name, [], results, [self.type()], {"iota_dimension": f"{d} : i64"}, [])
        if short == "concatenate":
            ops = []
            while self.peek("%"):
                ops.append(self.rx(_SSA)); self.expect(",")
            self.expect("dim"); self.expect("=")
            d = self.rx(re.compile(r"\d+"))
            return functional(ops, {"dimension": f"{d} : i64"})
        if short == "slice":
            a = self.rx(_SSA)
            self.expect("["); spec = self.balanced("]"); self.expect("]")
            lo, hi, st = [], [], []
            for part in [x.strip() for x in spec.split(",")] if spec else []:
                f = part.split(":")
                lo.append(f[0]); hi.append(f[1]); st.append(f[2] if len(f) > 2 else "1")
            arr = lambda v: "array<i64: " + ", ".join(v) + ">" if v else "array<i64>"
            return functional([a], {"start_indices": arr(lo), "limit_indices": arr(hi), "strides": arr(st)})
        if short in ("dynamic_slice", "dynamic_update_slice"):
            ops = [self.rx(_SSA)]
            attrs = {}
            while self.accept(","):
                if self.accept("sizes"):
                    self.expect("=")
                    attrs["slice_sizes"] = bracket()
                    break
                ops.append(self.rx(_SSA))
            return functional(ops, attrs)
        if short == "dot_general":
            a = self.rx(_SSA); self.expect(","); b = self.rx(_SSA)
            dims = {"batching_dims": ("[]", "[]"), "contracting_dims": ("[]", "[]")}
            attrs = {}
            while self.accept(","):
                key = self.rx(_ID); self.expect("=")
                if key in dims:
                    self.expect("["); l = self.balanced("]"); self.expect("]"); self.expect("x")
                    self.expect("["); r = self.balanced("]"); self.expect("]")
                    dims[key] = (f"[{l}]", f"[{r}]")
                else:
                    attrs[key] = self.balanced(",:")
            attrs["dot_dimension_numbers"] = (
                f"#stablehlo.dot<lhs_batching_dimensions = {dims['batching_dims'][0]}, rhs_batching_dimensions = {dims['batching_dims'][1]}, "
                f"lhs_contracting_dimensions = {dims['contracting_dims'][0]}, rhs_contracting_dimensions = {dims['contracting_dims'][1]}>")
            return functional([a, b], attrs)
        if short == "while":
            # stablehlo.while(%iterArg = %x, ...) : types [attributes {..}] cond { } do { }
            self.expect("(")
            names, ops = [], []
            if not self.accept(")"):
                while True:
                    names.append(self.rx(_SSA)); self.expect("="); ops.append(self.rx(_SSA))
                    if not self.accept(","):
                        break
                self.expect(")")
            types = []
            if self.accept(":"):
                types.append(self.type())
                while self.accept(","):
                    types.append(self.type())
            attrs = {}
            if self.accept("attributes"):
                self.expect("{"); attrs = self.attr_dict("}")
            regions = []
            for kw in ("cond", "do"):
                self.expect(kw); self.expect("{")
                blk = Block(args=list(zip(names, types)))
                self.ops_until(blk, "}")
                self.expect("}")
                regions.append(blk)
            return Op(name, ops, results, types, attrs, regions)
        if short == "pad":
            a = self.rx(_SSA); self.expect(","); v = self.rx(_SSA)
            attrs = {"edge_padding_low": keyword("low"), "edge_padding_high": keyword("high"), "interior_padding": keyword("interior")}
            return functional([a, v], attrs)
        if short == "reverse":
            a = self.rx(_SSA)
            attrs = {"dimensions": keyword("dims")}
            self.expect(":")
            return Op(name, [a], results, [self.type()], attrs, [])
        if short == "reduce_precision":
            a = self.rx(_SSA); self.expect(","); self.expect("format"); self.expect("=")
            m = re.compile(r"e(\d+)m(\d+)").match(self.rx(_ID))
            self.expect(":")
            return Op(name, [a], results, [self.type()], {"exponent_bits": f"{m.group(1)} : i32", "mantissa_bits": f"{m.group(2)} : i32"}, [])
        if short == "cholesky":
            a = self.rx(_SSA)
            attrs = {}
            if self.accept(","):
                self.expect("lower"); self.expect("=")
                attrs["lower"] = self.rx(_ID)
            self.expect(":")
            return Op(name, [a], results, [self.type()], attrs, [])
        if short == "rng_bit_generator":
            a = self.rx(_SSA); self.expect(","); self.expect("algorithm"); self.expect("=")
            return functional([a], {"rng_algorithm": f"#stablehlo<rng_algorithm {self.rx(_ID)}>"})
        if short == "custom_call":
            self.expect("@")
            self.ws()
            target = self.string() if self.s[self.i] == '"' else self.rx(re.compile(r"[\w.$]+"))
            self.expect("(")
            ops = self.operands()
            attrs = {"call_target_name": f'"{target}"'}
            if self.accept("{"):
                attrs.update(self.attr_dict("}"))
            return functional(ops, attrs)
        if short in ("after_all", "create_token", "partition_id", "replica_id"):
            ops = []
            while self.peek("%"):
                ops.append(self.rx(_SSA)); self.accept(",")
            self.expect(":")
            return Op(name, ops, results, [self.type()], {}, [])
        if short == "convolution":
            self.expect("(")
            ops = self.operands()
            self.expect("dim_numbers"); self.expect("=")
            dn = ""
            for part in range(3):
                self.expect("["); dn += "[" + self.balanced("]") + "]"; self.expect("]")
                if part == 0:
                    self.expect("x"); dn += "x"
                if part == 1:
                    self.expect("->"); dn += "->"
            attrs = {"dimension_numbers": f"#stablehlo.conv<{dn}>"}
            self.expect(","); self.expect("window"); self.expect("="); self.expect("{")
            if not self.accept("}"):
                while True:
                    key = self.rx(_ID); self.expect("=")
                    self.expect("["); body = self.balanced("]"); self.expect("]")
                    if key == "pad":
                        attrs["padding"] = f"dense<[{body}]> : tensor<{body.count('[')}x2xi64>"
                    elif key == "reverse":
                        attrs["window_reversal"] = f"array<i1: {body}>"
                    else:
                        attrs[{"stride": "window_strides", "lhs_dilate": "lhs_dilation", "rhs_dilate": "rhs_dilation"}[key]] = f"array<i64: {body}>"
                    if not self.accept(","):
                        break
                self.expect("}")
            if self.accept("{"):
                attrs.update(self.attr_dict("}"))
            return functional(ops, attrs)
        if name == "chlo.top_k":
            self.expect("("); a = self.rx(_SSA); self.expect(","); self.expect("k"); self.expect("=")
            k = self.rx(re.compile(r"\d+"))
            self.expect(")"); self.expect(":"); self.type(); self.expect("->")
            return Op(name, [a], results, self.type_list(), {"k": f"{k} : i64"}, [])
        if name.startswith("chlo.") and self.peek("%"):
            a = self.rx(_SSA)
            self.expect(":"); self.type(); self.expect("->")
            return Op(name, [a], results, self.type_list(), {}, [])
        raise SyntaxError(f"custom assembly of {name!r} is not supported; print the module in generic form")


def parse_module(text: str) -> Module:
    p = Parser(text)
    m = p.module()
    p.ws()
    if p.i != len(p.s):
        raise SyntaxError(f"trailing text at {p.i}: {p.s[p.i:p.i + 60]!r}")
    return m


# ---- attribute decoding helpers ----------------------------------------------

def attr_int(raw: str) -> int:
    return int(raw.split(":")[0].strip())


def attr_bool(raw: str) -> bool:
    return raw.strip().split(":")[0].strip() in ("true", "unit", "1")


def attr_i64s(raw: str) -> list:
    raw = raw.strip()
    if raw.startswith("array<"):
        inner = raw[raw.index("<") + 1:raw.rindex(">")]
        if ":" not in inner:
            return []
        body = inner.split(":", 1)[1]
        return [int(x) for x in body.split(",") if x.strip()]
    if raw.startswith("dense<"):
        return [int(x) for x in dense_array(raw).reshape(-1)]
    if raw.startswith("["):
        return [int(x.split(":")[0]) for x in raw[1:-1].split(",") if x.strip()]
    raise ValueError(raw)


def attr_str(raw: str) -> str:
    raw = raw.strip()
    return raw[1:-1] if raw.startswith('"') else raw


def enum_word(raw: str) -> str:
    """'#stablehlo<comparison_direction GT>' -> 'GT'"""
    return raw.strip().rstrip(">").split()[-1]


def struct_fields(raw: str) -> dict:
    """'#stablehlo.dot<a = [0], b = 1>' -> {'a': [0], 'b': 1}"""
    inner = raw[raw.index("<") + 1:raw.rindex(">")]
    out = {}
    for m in re.finditer(r"(\w+)\s*=\s*(\[[^\]]*\]|-?\d+)", inner):
        v = m.group(2)
        out[m.group(1)] = [int(x) for x in v[1:-1].split(",") if x.strip()] if v.startswith("[") else int(v)
    return out


_NPDT = {"f32": np.float32, "f16": np.float16, "f64": np.float64, "bf16": np.float32,
         "i8": np.int8, "i16": np.int16, "i32": np.int32, "i64": np.int64,
         "ui8": np.uint8, "ui16": np.uint16, "ui32": np.uint32, "ui64": np.uint64, "i1": np.bool_}


def np_dtype(dt: str):
    return _NPDT[dt]


def bf16_bits_to_f32(u16: np.ndarray) -> np.ndarray:
    return (u16.astype(np.uint32) << 16).view(np.float32)


def dense_array(raw: str) -> np.ndarray:
    """Decode 'dense<...> : tensor<...>' into a numpy array (bf16 as float32
    holding bf16-representable values)."""
    raw = raw.strip()
    assert raw.startswith("dense<"), raw[:40]
    p = Parser(raw)
    p.i = len("dense<")
    body = p.balanced(">")
    p.expect(">")
    p.expect(":")
    t = p.type()
    dt = np_dtype(t.dtype)
    n = int(np.prod(t.shape)) if t.shape else 1
    if body.startswith('"0x'):
        rawb = bytes.fromhex(body[3:-1])
        if t.dtype == "bf16":
            a = bf16_bits_to_f32(np.frombuffer(rawb, np.uint16))
        elif t.dtype == "i1":
            b = np.frombuffer(rawb, np.uint8)
            if len(b) == n:
                a = b != 0
            else:               # bit-packed legacy form
                a = np.unpackbits(b, bitorder="little")[:n].astype(bool)
        else:
            a = np.frombuffer(rawb, dt)
        if a.size == 1 and n != 1:
            a = np.broadcast_to(a, (n,))
        return np.array(a).reshape(t.shape)
    toks = re.findall(r"true|false|[-+]?0x[0-9A-Fa-f]+|[-+]?(?:\d+\.?\d*(?:[eE][-+]?\d+)?|inf|nan)", body)
    def conv(tok):
        if tok == "true": return True
        if tok == "false": return False
        if "0x" in tok:
            bits = int(tok, 16)
            if t.dtype == "f32": return np.array([bits], np.uint32).view(np.float32)[0]
            if t.dtype == "bf16": return bf16_bits_to_f32(np.array([bits], np.uint16))[0]
            if t.dtype == "f16": return np.array([bits], np.uint16).view(np.float16)[0]
            if t.dtype == "f64": return np.array([bits], np.uint64).view(np.float64)[0]
            return bits
        if t.dtype in ("f32", "f16", "f64", "bf16"):
            return float(tok)
        return int(tok)
    vals = [conv(x) for x in toks]
    if t.dtype == "i1":
        a = np.array([bool(v) for v in vals], bool)
    elif t.dtype.startswith("ui") or t.dtype.startswith("i"):
        a = np.array([int(v) for v in vals], dtype=object).astype(dt) if vals else np.zeros(0, dt)
    else:
        a = np.array(vals, dtype=np.float64).astype(dt)
    if a.size == 1 and n != 1:
        a = np.broadcast_to(a, (n,)).copy()
    return a.reshape(t.shape)
