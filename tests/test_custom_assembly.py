"""The custom assembly jax prints for StableHLO (`jax.jit(f).lower(x).as_text()`) against the generic form of the same
program: the plan compiler must make the same plan from both. The reference reads MLIR bytecode through the MLIR
libraries (src/pjrt_plugin/stablehlo_parser.cc:187-285), so every printed form reaches it; the text reader here has
to know each operation's custom form. Covered: pad, reverse, clamp with scalar bounds, convolution with its
`dim_numbers` / `window` clauses, reduce_precision, custom_call, after_all / create_token, partition_id, cholesky,
rng_bit_generator, the chlo unary functions, chlo.top_k, and location aliases of a module printed with debug
information."""
import numpy as np
import pytest

import b200
from b200.shlo.builder import Builder


def _module(body, sig):
    return "module @jit_f {\n  func.func public @main" + sig + " {\n" + body + "\n  }\n}\n"


def _same_plan(pretty, generic, inputs=None):
    """Both texts give the plan compiler the same plan and, where inputs are given, the interpreter (which has a reader
    of its own) the same numbers."""
    p1, _ = b200.compile_to_plan(pretty, validate=True)
    p0, _ = b200.compile_to_plan(generic, validate=True)
    body = lambda p: p.splitlines()[1:]
    assert body(p1) == body(p0), (p1, p0)
    if inputs is not None:
        from oracle import interp
        a, b_ = interp.run_text(pretty, inputs), interp.run_text(generic, inputs)
        assert len(a) == len(b_)
        for x, y in zip(a, b_):
            np.testing.assert_array_equal(np.asarray(x), np.asarray(y))
    return p1


def _f32(*shape, seed=0):
    return np.random.default_rng(seed).standard_normal(shape).astype(np.float32)


def test_pad_reverse_and_clamp():
    b = Builder()
    x = b.arg((4, 5), "f32")
    y = b.pad(x, b.const(0.5, "f32"), [1, 0], [0, 2], [1, 0])
    z = b.reverse(y, [0, 1])
    w = b.clamp(b.const(-0.25, "f32"), z, b.const(0.75, "f32"))
    generic = b.module([w])
    pretty = _module("""    %cst = stablehlo.constant dense<5.000000e-01> : tensor<f32>
    %0 = stablehlo.pad %arg0, %cst, low = [1, 0], high = [0, 2], interior = [1, 0] : (tensor<4x5xf32>, tensor<f32>) -> tensor<8x7xf32>
    %1 = stablehlo.reverse %0, dims = [0, 1] : tensor<8x7xf32>
    %cst_0 = stablehlo.constant dense<-2.500000e-01> : tensor<f32>
    %cst_1 = stablehlo.constant dense<7.500000e-01> : tensor<f32>
    %2 = stablehlo.clamp %cst_0, %1, %cst_1 : (tensor<f32>, tensor<8x7xf32>, tensor<f32>) -> tensor<8x7xf32>
    return %2 : tensor<8x7xf32>""", "(%arg0: tensor<4x5xf32>) -> (tensor<8x7xf32>)")
    _same_plan(pretty, generic)


@pytest.mark.parametrize("window,kw", [
    ("window = {stride = [2, 1], pad = [[1, 0], [2, 2]], lhs_dilate = [1, 2], rhs_dilate = [2, 1]}",
     dict(strides=(2, 1), padding=((1, 0), (2, 2)), lhs_dilation=(1, 2), rhs_dilation=(2, 1))),
    ("window = {pad = [[1, 1], [1, 1]]}", dict(padding=((1, 1), (1, 1)))),
    ("window = {}", dict()),
])
def test_convolution(window, kw):
    b = Builder()
    x, w = b.arg((2, 9, 8, 4), "f32"), b.arg((3, 3, 4, 8), "f32")
    y = b.conv(x, w, **kw)
    generic = b.module([y])
    out = "x".join(str(d) for d in y.shape)
    pretty = _module(f"""    %0 = stablehlo.convolution(%arg0, %arg1) dim_numbers = [b, 0, 1, f]x[0, 1, i, o]->[b, 0, 1, f], {window} {{batch_group_count = 1 : i64, feature_group_count = 1 : i64, precision_config = [#stablehlo<precision DEFAULT>, #stablehlo<precision DEFAULT>]}} : (tensor<2x9x8x4xf32>, tensor<3x3x4x8xf32>) -> tensor<{out}xf32>
    return %0 : tensor<{out}xf32>""", f"(%arg0: tensor<2x9x8x4xf32>, %arg1: tensor<3x3x4x8xf32>) -> (tensor<{out}xf32>)")
    plan = _same_plan(pretty, generic, [_f32(2, 9, 8, 4), _f32(3, 3, 4, 8, seed=1)])
    assert "igemm" in plan


def test_cholesky_rng_top_k_and_chlo_functions():
    b = Builder()
    a = b.arg((3, 3), "f32")
    generic = b.module([b.cholesky(a, lower=False), b.chlo_unary("erf_inv", a), b.chlo_unary("asinh", a)] + b.top_k(a, 2))
    pretty = _module("""    %0 = stablehlo.cholesky %arg0, lower = false : tensor<3x3xf32>
    %1 = chlo.erf_inv %arg0 : tensor<3x3xf32> -> tensor<3x3xf32>
    %2 = chlo.asinh %arg0 : tensor<3x3xf32> -> tensor<3x3xf32>
    %values, %indices = chlo.top_k(%arg0, k = 2) : tensor<3x3xf32> -> (tensor<3x2xf32>, tensor<3x2xi32>)
    return %0, %1, %2, %values, %indices : tensor<3x3xf32>, tensor<3x3xf32>, tensor<3x3xf32>, tensor<3x2xf32>, tensor<3x2xi32>""",
                     "(%arg0: tensor<3x3xf32>) -> (tensor<3x3xf32>, tensor<3x3xf32>, tensor<3x3xf32>, tensor<3x2xf32>, tensor<3x2xi32>)")
    m = _f32(3, 3) * 0.3
    _same_plan(pretty, generic, [(m @ m.T + np.eye(3) * 0.5).astype(np.float32) * 0.5])
    b = Builder()
    generic = b.module(b.rng_bit_generator(b.arg((2,), "ui64"), (5, 3), "ui16", "THREE_FRY"))
    pretty = _module("""    %output_state, %output = stablehlo.rng_bit_generator %arg0, algorithm = THREE_FRY : (tensor<2xui64>) -> (tensor<2xui64>, tensor<5x3xui16>)
    return %output_state, %output : tensor<2xui64>, tensor<5x3xui16>""", "(%arg0: tensor<2xui64>) -> (tensor<2xui64>, tensor<5x3xui16>)")
    _same_plan(pretty, generic, [np.array([11, 12], np.uint64)])


def test_custom_calls_tokens_partition_id_and_reduce_precision():
    b = Builder()
    x = b.arg((4,), "f32")
    (s,) = b.custom_call("Sharding", [x], [((4,), "f32")])
    (e,) = b.custom_call("mhlo.erf", [s], [((4,), "f32")])
    generic = b.module([e])
    pretty = _module("""    %0 = stablehlo.custom_call @Sharding(%arg0) {mhlo.sharding = "{replicated}"} : (tensor<4xf32>) -> tensor<4xf32>
    %1 = stablehlo.custom_call @mhlo.erf(%0) {mhlo.attributes = {}, mhlo.version = 1 : i64} : (tensor<4xf32>) -> tensor<4xf32>
    %2 = stablehlo.create_token : !stablehlo.token
    %3 = stablehlo.after_all %2 : !stablehlo.token
    %4 = stablehlo.after_all  : !stablehlo.token
    return %1 : tensor<4xf32>""", "(%arg0: tensor<4xf32>) -> (tensor<4xf32>)")
    _same_plan(pretty, generic, [_f32(4)])
    pretty = _module("""    %0 = stablehlo.partition_id : tensor<ui32>
    %1 = stablehlo.reduce_precision %arg0, format = e5m10 : tensor<4xf32>
    return %0, %1 : tensor<ui32>, tensor<4xf32>""", "(%arg0: tensor<4xf32>) -> (tensor<ui32>, tensor<4xf32>)")
    generic = _module("""    %0 = "stablehlo.partition_id"() : () -> tensor<ui32>
    %1 = "stablehlo.reduce_precision"(%arg0) <{exponent_bits = 5 : i32, mantissa_bits = 10 : i32}> : (tensor<4xf32>) -> tensor<4xf32>
    return %0, %1 : tensor<ui32>, tensor<4xf32>""", "(%arg0: tensor<4xf32>) -> (tensor<ui32>, tensor<4xf32>)")
    _same_plan(pretty, generic, [_f32(4)])


def test_module_printed_with_debug_information():
    text = """#loc = loc(unknown)
#loc1 = loc("x")
module @jit_f attributes {mhlo.num_partitions = 1 : i32, mhlo.num_replicas = 1 : i32} {
  func.func public @main(%arg0: tensor<4x4xf32> loc("x")) -> (tensor<4x4xf32> {jax.result_info = ""}) {
    %0 = stablehlo.add %arg0, %arg0 : tensor<4x4xf32> loc(#loc3)
    return %0 : tensor<4x4xf32> loc(#loc)
  } loc(#loc)
} loc(#loc)
#loc2 = loc("a.py":1:2)
#loc3 = loc("jit(f)/add"(#loc2))
"""
    plan, _ = b200.compile_to_plan(text, validate=True)
    assert plan.count("kernel ") == 1


def test_unknown_custom_assembly_is_still_an_error():
    text = _module("    %0 = chlo.broadcast_add %arg0, %arg0 : (tensor<4xf32>, tensor<4xf32>) -> tensor<4xf32>\n    return %0 : tensor<4xf32>",
                   "(%arg0: tensor<4xf32>) -> (tensor<4xf32>)")
    with pytest.raises(b200.B200Error, match="several operands|not supported"):
        b200.compile_to_plan(text)


def test_reduce_with_several_inputs_in_its_printed_form():
    """jnp.argmax as jax prints it: each (input init: value) pair in parentheses of its own and a `reducer` region."""
    pretty = _module("""    %0 = stablehlo.iota dim = 1 : tensor<4x8xi32>
    %cst = stablehlo.constant dense<0xFF800000> : tensor<f32>
    %c = stablehlo.constant dense<0> : tensor<i32>
    %1:2 = stablehlo.reduce(%arg0 init: %cst), (%0 init: %c) across dimensions = [1] : (tensor<4x8xf32>, tensor<4x8xi32>, tensor<f32>, tensor<i32>) -> (tensor<4xf32>, tensor<4xi32>)
     reducer(%arg1: tensor<f32>, %arg3: tensor<f32>) (%arg2: tensor<i32>, %arg4: tensor<i32>)  {
      %2 = stablehlo.compare  GT, %arg1, %arg3,  FLOAT : (tensor<f32>, tensor<f32>) -> tensor<i1>
      %3 = stablehlo.compare  NE, %arg1, %arg1,  FLOAT : (tensor<f32>, tensor<f32>) -> tensor<i1>
      %4 = stablehlo.or %2, %3 : tensor<i1>
      %5 = stablehlo.compare  EQ, %arg1, %arg3,  FLOAT : (tensor<f32>, tensor<f32>) -> tensor<i1>
      %6 = stablehlo.compare  LT, %arg2, %arg4,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>
      %7 = stablehlo.and %5, %6 : tensor<i1>
      %8 = stablehlo.or %4, %7 : tensor<i1>
      %9 = stablehlo.select %4, %arg1, %arg3 : tensor<i1>, tensor<f32>
      %10 = stablehlo.select %8, %arg2, %arg4 : tensor<i1>, tensor<i32>
      stablehlo.return %9, %10 : tensor<f32>, tensor<i32>
    }
    return %1#0, %1#1 : tensor<4xf32>, tensor<4xi32>""", "(%arg0: tensor<4x8xf32>) -> (tensor<4xf32>, tensor<4xi32>)")
    plan, _ = b200.compile_to_plan(pretty, validate=True)
    assert "reduce" in plan


def test_short_type_forms_and_attribute_dictionaries():
    """`convert` to the same type prints one type, `optimization_barrier` prints its operands' types without an arrow,
    and an elementwise operation may carry an attribute dictionary in front of its type."""
    pretty = _module("""    %0 = stablehlo.convert %arg0 : tensor<4xf32>
    %1:2 = stablehlo.optimization_barrier %0, %arg0 : tensor<4xf32>, tensor<4xf32>
    %2 = stablehlo.add %1#0, %1#1 {mhlo.frontend_attributes = {origin = "x"}} : tensor<4xf32>
    return %2 : tensor<4xf32>""", "(%arg0: tensor<4xf32>) -> (tensor<4xf32>)")
    plan, _ = b200.compile_to_plan(pretty, validate=True)
    assert plan.count("kernel ") == 1 and "add" in plan


def test_interpreter_reads_the_printed_forms_of_a_small_jax_program():
    """A loop, a batched product, iota, concatenate, strided slice, dynamic_slice and an argmax in the forms jax prints:
    the interpreter's own reader gives what NumPy gives, and the plan compiler accepts the same text."""
    from oracle import interp
    text = """#loc = loc(unknown)
module @jit_f attributes {mhlo.num_partitions = 1 : i32, mhlo.num_replicas = 1 : i32} {
  func.func public @main(%arg0: tensor<2x4x8xf32> loc(unknown), %arg1: tensor<2x8x3xf32> loc(unknown)) -> (tensor<2x4x3xf32> {jax.result_info = "[0]"}, tensor<6xi32> {jax.result_info = "[1]"}, tensor<2x4xi32> {jax.result_info = "[2]"}) {
    %0 = stablehlo.dot_general %arg0, %arg1, batching_dims = [0] x [0], contracting_dims = [2] x [1], precision = [DEFAULT, DEFAULT] : (tensor<2x4x8xf32>, tensor<2x8x3xf32>) -> tensor<2x4x3xf32> loc(#loc)
    %c = stablehlo.constant dense<0> : tensor<i32> loc(#loc)
    %1:2 = stablehlo.while(%iterArg = %c, %iterArg_0 = %0) : tensor<i32>, tensor<2x4x3xf32>
     cond {
      %c_1 = stablehlo.constant dense<3> : tensor<i32>
      %9 = stablehlo.compare  LT, %iterArg, %c_1,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>
      stablehlo.return %9 : tensor<i1>
    } do {
      %9 = stablehlo.add %iterArg_0, %iterArg_0 : tensor<2x4x3xf32>
      %c_1 = stablehlo.constant dense<1> : tensor<i32>
      %10 = stablehlo.add %iterArg, %c_1 : tensor<i32>
      stablehlo.return %10, %9 : tensor<i32>, tensor<2x4x3xf32>
    }
    %2 = stablehlo.iota dim = 0 : tensor<8xi32>
    %3 = stablehlo.slice %2 [1:8:3] : (tensor<8xi32>) -> tensor<3xi32>
    %c_2 = stablehlo.constant dense<5> : tensor<i32>
    %4 = stablehlo.dynamic_slice %2, %c_2, sizes = [3] : (tensor<8xi32>, tensor<i32>) -> tensor<3xi32>
    %5 = stablehlo.concatenate %3, %4, dim = 0 : (tensor<3xi32>, tensor<3xi32>) -> tensor<6xi32>
    %6 = stablehlo.iota dim = 2 : tensor<2x4x8xi32>
    %cst = stablehlo.constant dense<0xFF800000> : tensor<f32>
    %7:2 = stablehlo.reduce(%arg0 init: %cst), (%6 init: %c) across dimensions = [2] : (tensor<2x4x8xf32>, tensor<2x4x8xi32>, tensor<f32>, tensor<i32>) -> (tensor<2x4xf32>, tensor<2x4xi32>)
     reducer(%arg2: tensor<f32>, %arg4: tensor<f32>) (%arg3: tensor<i32>, %arg5: tensor<i32>)  {
      %9 = stablehlo.compare  GT, %arg2, %arg4,  FLOAT : (tensor<f32>, tensor<f32>) -> tensor<i1>
      %10 = stablehlo.compare  EQ, %arg2, %arg4,  FLOAT : (tensor<f32>, tensor<f32>) -> tensor<i1>
      %11 = stablehlo.compare  LT, %arg3, %arg5,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>
      %12 = stablehlo.and %10, %11 : tensor<i1>
      %13 = stablehlo.or %9, %12 : tensor<i1>
      %14 = stablehlo.select %9, %arg2, %arg4 : tensor<i1>, tensor<f32>
      %15 = stablehlo.select %13, %arg3, %arg5 : tensor<i1>, tensor<i32>
      stablehlo.return %14, %15 : tensor<f32>, tensor<i32>
    }
    return %1#1, %5, %7#1 : tensor<2x4x3xf32>, tensor<6xi32>, tensor<2x4xi32> loc(#loc)
  } loc(#loc)
} loc(#loc)
#loc1 = loc("f.py":3:0)
"""
    x, y = _f32(2, 4, 8), _f32(2, 8, 3, seed=1)
    out = interp.run_text(text, [x, y])
    np.testing.assert_allclose(out[0], 8 * np.einsum("bik,bkj->bij", x.astype(np.float64), y.astype(np.float64)), rtol=1e-5, atol=1e-5)
    np.testing.assert_array_equal(out[1], [1, 4, 7, 5, 6, 7])
    np.testing.assert_array_equal(out[2], np.argmax(x, axis=2))
    plan, _ = b200.compile_to_plan(text, validate=True)
    assert "while trip=3" in plan and "igemm" in plan
