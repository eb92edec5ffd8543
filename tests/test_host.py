"""CPU: host-side logic — the C-ABI library loads and exports every declared
symbol, the parser and the plan compiler behave (fusion shape, error text for
unsupported operations, custom assembly), and nothing computes without a GPU."""
import os
import re
from pathlib import Path

import numpy as np
import pytest

import b200
from b200.shlo.builder import Builder
from b200.shlo import programs

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "b200_core.h").read_text()
    declared = set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", header)) - {"b200_event_callback"}
    lib = b200.load_library()
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, missing
    assert declared == set(b200.SIGNATURES), declared ^ set(b200.SIGNATURES)


def test_no_cpu_fallback():
    """Without a CUDA device the client refuses to exist (no silent CPU path)."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(b200.B200Error) as e:
        b200.Client()
    assert e.value.code == b200.FAILED_PRECONDITION
    assert "no CPU fallback" in str(e.value)


def test_unsupported_op_is_a_compile_error_naming_all_ops():
    """Like the reference (src/pjrt_plugin/stablehlo_parser.cc:167-184): one error listing every unsupported op."""
    text = """
module @m { func.func public @main(%arg0: tensor<4xf32>) -> tensor<4xf32> {
  %0 = "stablehlo.fft"(%arg0) : (tensor<4xf32>) -> tensor<4xf32>
  %1 = "stablehlo.batch_norm_inference"(%0) : (tensor<4xf32>) -> tensor<4xf32>
  "func.return"(%1) : (tensor<4xf32>) -> ()
} }"""
    with pytest.raises(b200.B200Error) as e:
        b200.compile_to_plan(text)
    assert "stablehlo.fft" in str(e.value) and "stablehlo.batch_norm_inference" in str(e.value)
    assert e.value.code == b200.INVALID_ARGUMENT


def test_parse_errors_carry_a_line_number():
    with pytest.raises(b200.B200Error) as e:
        b200.compile_to_plan("module @m {\n func.func public @main() -> tensor<f32> {\n  %0 = stablehlo.bogus\n } }")
    assert "line 3" in str(e.value)


def test_elementwise_chain_is_one_kernel():
    b = Builder()
    x, y = b.arg((256, 64), "f32"), b.arg((64,), "f32")
    z = b.tanh(b.add(b.mul(x, x), b.bcast(y, x.shape)))
    w = b.select(b.compare(z, b.zeros_like(z), "GT"), z, b.neg(z))
    plan, src = b200.compile_to_plan(b.module([w]), validate=True)
    assert plan.count("kernel ") == 1, plan
    assert "op_tanh" in src


def test_multi_output_fusion_of_optimizer_update():
    """m' = 0.9 m + g and w' = w - 0.1 m' leave one kernel with two outputs."""
    b = Builder()
    w, m, g = (b.arg((1000,), "f32") for _ in range(3))
    m2 = b.add(b.mul(m, b.full((1000,), 0.9, "f32")), g)
    w2 = b.sub(w, b.mul(m2, b.full((1000,), 0.1, "f32")))
    plan, _ = b200.compile_to_plan(b.module([w2, m2]))
    assert plan.count("kernel ") == 1, plan


def test_fusion_can_be_disabled():
    b = Builder()
    x = b.arg((64,), "f32")
    y = b.exp(b.neg(b.mul(x, x)))
    assert b200.compile_to_plan(b.module([y]))[0].count("kernel ") == 1
    assert b200.compile_to_plan(b.module([y]), disable_fusion=True)[0].count("kernel ") == 3


def test_resnet_plan_shape():
    prog = programs.resnet18_train_step(batch=4, image=8, width=8)
    plan, src = b200.compile_to_plan(prog.text, validate=True)
    assert plan.count("igemm ") == 20 + 19 + 20 + 3        # 20 convs fwd, 19 input grads, 20 kernel grads, dense fwd + 2 grads
    assert "all_reduce" not in plan
    dp = programs.resnet18_train_step(batch=4, image=8, width=8, n_partitions=2)
    os.environ["B200_NO_ALL_REDUCE_OVERLAP"] = "1"
    try:
        plan2, _ = b200.compile_to_plan(dp.text, num_processes=2, process_index=1)
    finally:
        del os.environ["B200_NO_ALL_REDUCE_OVERLAP"]
    assert plan2.count("all_reduce") == 63                  # 62 gradient leaves + the loss
    assert "join" not in plan2 and "overlapped" not in plan2
    check_runs(plan2, overlapped=False)
    plan3, _ = b200.compile_to_plan(dp.text, num_processes=2, process_index=1)       # the default: buckets inside the backward pass
    assert plan3.count("all_reduce") == 63
    check_runs(plan3, overlapped=True)


def check_runs(plan2, overlapped):
    # Each run of consecutive all-reduces lies back to back in 256-byte granules (inputs in one block, outputs in
    # another): the runtime reduces a run with one call over the flat buffer. Runs whose gradients exist early are
    # moved up into the backward pass and issued on the collective stream; a join follows the last run.
    lines = plan2.splitlines()
    runs, prev = [], None
    for i, l in enumerate(lines):
        m = re.search(r"all_reduce (\d+) bytes in@(\d+) out@(\d+)", l)
        if not m:
            continue
        assert ("overlapped" in l) == overlapped
        if prev != i - 1:
            runs.append([])
        runs[-1].append(tuple(int(g) for g in m.groups()))
        prev = i
    assert len(runs) >= 2 if overlapped else len(runs) == 1
    for run in runs:
        for (b0, i0, o0), (_, i1, o1) in zip(run, run[1:]):
            step = (b0 + 255) // 256 * 256
            assert i1 == i0 + step and o1 == o0 + step
    join = [i for i, l in enumerate(lines) if l.strip().startswith("join")]
    if overlapped:
        assert len(join) == 1 and join[0] == prev + 1


def test_counted_loop_is_recognised():
    b = Builder()
    x = b.arg((4,), "f32")
    outs = b.while_([b.const(0, "i32"), x], lambda s, i, v: s.compare(i, s.const(130, "i32"), "LT"),
                    lambda s, i, v: [s.add(i, s.const(1, "i32")), s.mul(v, v)])
    plan, _ = b200.compile_to_plan(b.module(outs))
    assert "while trip=130" in plan


def test_scan_body_plan_has_no_copies():
    """The LSTM scan step: stacked carries are updated through a window in place, every other carried value trades
    pointers with its next value, independent pointwise kernels of a body share a launch, and the generated
    source of the whole plan compiles."""
    prog = programs.lstm_scan_train_step(steps=6, batch=8, in_dim=8, hidden=16)
    plan, _ = b200.compile_to_plan(prog.text, validate=True)
    loops = [l for l in plan.splitlines() if l.strip().startswith("while trip=6")]
    assert len(loops) == 2
    assert "exchanged=5/9" in loops[0] and "exchanged=9/9" in loops[1]
    assert plan.count(".window") >= 4 and "bundle_" in plan and "memcpy" not in plan


@pytest.mark.parametrize("dt", ["f32", "f64", "i32", "bf16"])
def test_column_reduction_source_compiles(dt):
    """The four-indices-per-thread column reduction and its block-per-output second pass are generated for every
    element type and pass NVRTC (compile only, no device)."""
    b = Builder()
    x = b.arg((4096, 128), dt)
    plan, src = b200.compile_to_plan(b.module([b.reduce_sum(x, [0]), b.reduce_sum(b.mul(x, x), [0])]), validate=True)
    assert "block=32x8" in plan and ".final" in plan
    assert "acc0[q]" in src


def _split_at_while(plan):
    lines = plan.splitlines()
    w = next(i for i, l in enumerate(lines) if l.strip().startswith("while"))
    return lines[1:w], [l for l in lines[w + 1:] if l.startswith("    ")]


def test_weight_widening_is_hoisted_out_of_the_decode_loop():
    """Where the native 16-bit kernels do not apply (here: switched off), bf16 contractions run as f32 contractions
    of widened operands. Weights come from outside the decode loop: their widened copies are made once in front of
    the `while`, not in every iteration."""
    prog = programs.gemma_greedy_decode(vocab=64, dim=32, layers=2, heads=2, head_dim=16, hidden=64, prompt_len=4,
                                        new_tokens=4, cache_len=8)
    os.environ["B200_NO_GEMM16"] = "1"
    try:
        before, body = _split_at_while(b200.compile_to_plan(prog.text, validate=True)[0])
        os.environ["B200_NO_HOIST"] = "1"
        os.environ["B200_NO_LICM"] = "1"               # general loop-invariant code motion would move them as well
        before0, body0 = _split_at_while(b200.compile_to_plan(prog.text)[0])
    finally:
        os.environ.pop("B200_NO_HOIST", None)
        os.environ.pop("B200_NO_LICM", None)
        del os.environ["B200_NO_GEMM16"]
    count = lambda ls: sum(l.count("convert") for l in ls)
    assert count(before) > count(before0) and count(body) < count(body0)


def test_bf16_decode_loop_reads_its_weights_in_place():
    """With the native 16-bit kernels the decode loop multiplies by the bf16 weights as they are: no widened copy in
    front of the loop, every product of the body a skinny 16-bit kernel, the key-value caches updated in their
    windows, one copy of the normalised activation for the projections that share it, and the attention over the
    cache (two products and a softmax) one kernel per layer."""
    prog = programs.gemma_decode_loop(vocab=64, dim=32, layers=2, heads=2, head_dim=16, hidden=64, start=4, new_tokens=4,
                                      cache_len=8)
    plan = b200.compile_to_plan(prog.text, validate=True)[0]
    before, body = _split_at_while(plan)
    assert not any("fusion{convert}" in l for l in before) and "igemm" not in plan      # no widened copy of a weight
    assert sum("gemv16" in l for l in body) == 2 * 7 + 1 and sum("attention_" in l for l in body) == 2
    assert sum(l.count(".window") for l in body) >= 2 * 2
    # q, k and v projections read one converted activation (args[0] of three consecutive products is one slot)
    prods = [l for l in body if "gemv16" in l]
    first = [l.split("args=[")[1].split(",")[0] for l in prods[:3]]
    assert len(set(first)) == 1


def test_loop_invariant_weights_of_skinny_products_are_transposed_once_and_merged():
    """Weights large enough to matter are transposed (and, for products sharing their left operand, concatenated) in
    front of the decode loop; the loop then runs one k-contiguous product for q / k / v and one for gate / up."""
    prog = programs.gemma_decode_loop(vocab=512, dim=256, layers=2, heads=2, head_dim=256, hidden=512, start=4, new_tokens=4,
                                      cache_len=8)
    plan = b200.compile_to_plan(prog.text, validate=True)[0]
    before, body = _split_at_while(plan)
    assert sum(l.count("transpose batch=") for l in before) == 2 * 7       # seven weights per layer, tiled kernel
    prods = [l for l in body if "gemv16" in l]
    assert sum("N=1024 K=256" in l and "gemv16_kc" in l for l in prods) == 2 * 2   # q | k | v (512 + 256 + 256) and gate | up
    assert len(prods) == 2 * 4 + 1 and sum("attention_" in l for l in body) == 2
    os.environ["B200_NO_WEIGHT_HOIST"] = "1"
    try:
        plan0 = b200.compile_to_plan(prog.text)[0]
    finally:
        del os.environ["B200_NO_WEIGHT_HOIST"]
    assert sum("gemv16" in l for l in plan0.splitlines()) == 2 * 7 + 1


def test_common_subexpressions_are_computed_once():
    b = Builder()
    x = b.arg((64, 32), "f32")
    w1, w2 = b.arg((32, 16), "bf16"), b.arg((32, 8), "bf16")
    y1 = b.matmul(b.convert(b.tanh(x), "bf16"), w1)
    y2 = b.matmul(b.convert(b.tanh(x), "bf16"), w2)
    plan = b200.compile_to_plan(b.module([y1, y2]))[0]
    assert plan.count("kernel ") == 1, plan


def test_custom_assembly_and_generic_form_give_the_same_plan():
    pretty = """
module @m { func.func public @main(%arg0: tensor<8x4xf32>, %arg1: tensor<4xf32>) -> tensor<8xf32> {
  %0 = stablehlo.broadcast_in_dim %arg1, dims = [1] : (tensor<4xf32>) -> tensor<8x4xf32>
  %1 = stablehlo.multiply %arg0, %0 : tensor<8x4xf32>
  %cst = stablehlo.constant dense<0.000000e+00> : tensor<f32>
  %2 = stablehlo.reduce(%1 init: %cst) applies stablehlo.add across dimensions = [1] : (tensor<8x4xf32>, tensor<f32>) -> tensor<8xf32>
  return %2 : tensor<8xf32>
} }"""
    b = Builder()
    x, y = b.arg((8, 4), "f32"), b.arg((4,), "f32")
    generic = b.module([b.reduce_sum(b.mul(x, b.broadcast_in_dim(y, (8, 4), (1,))), (1,))])
    p1, s1 = b200.compile_to_plan(pretty)
    p2, s2 = b200.compile_to_plan(generic)
    strip = lambda p: re.sub(r"program \S+:", "program:", p)
    assert strip(p1) == strip(p2)
    from oracle import interp
    a, v = np.arange(32, dtype=np.float32).reshape(8, 4), np.array([1, 2, 3, 4], np.float32)
    np.testing.assert_allclose(interp.run_text(pretty, [a, v])[0], (a * v).sum(1))


def test_sharding_custom_calls_are_pass_through():
    text = """
module @m attributes {mhlo.num_partitions = 1 : i32} { func.func public @main(%arg0: tensor<4xf32>) -> tensor<4xf32> {
  %0 = "stablehlo.custom_call"(%arg0) <{call_target_name = "Sharding"}> {mhlo.sharding = "{replicated}"} : (tensor<4xf32>) -> tensor<4xf32>
  %1 = "stablehlo.add"(%0, %0) : (tensor<4xf32>, tensor<4xf32>) -> tensor<4xf32>
  "func.return"(%1) : (tensor<4xf32>) -> ()
} }"""
    plan, _ = b200.compile_to_plan(text)
    assert plan.count("kernel ") == 1


def test_lstm_scan_program_matches_autograd_twin():
    """The LSTM-by-scan training step (forward while, reverse while with per-step recomputation, Adam) run in
    the float64 oracle against PyTorch autograd on the same weights: pins the program the GPU tests execute."""
    from b200.shlo import programs
    from oracle import interp, twins
    prog = programs.lstm_scan_train_step(steps=6, batch=4, in_dim=5, hidden=8)
    args = programs.lstm_inputs(prog, seed=2)
    outs = interp.run_text(prog.text, args, wide=True)
    loss, new_p, ms, vs = twins.lstm_train_step(args[:4], args[-2], args[-1])
    assert abs(float(outs[0]) - loss) < 1e-9
    for k in range(4):
        np.testing.assert_allclose(outs[1 + k], new_p[k], rtol=1e-6, atol=1e-9)
        np.testing.assert_allclose(outs[5 + k], ms[k], rtol=1e-6, atol=1e-12)
        np.testing.assert_allclose(outs[9 + k], vs[k], rtol=1e-6, atol=1e-15)


def test_distilbert_program_gradients_match_finite_differences():
    """The DistilBERT-shaped masked-language-model step in f32, run in the float64 oracle: the program's
    gradients against central differences of its own loss on a few leaves of every kind."""
    from b200.shlo import programs
    from oracle import interp
    prog = programs.distilbert_mlm_step(batch=2, seq=8, vocab=96, dim=32, layers=2, heads=4, ffn=64, dtype="f32")
    args = [a.astype(np.float64) if a.dtype == np.float32 else a for a in programs.distilbert_inputs(prog, weight_std=0.1, mask_rate=0.4)]
    outs = interp.run_text(prog.text, args, wide=True)
    names = [n for n, _, _ in prog.args]
    for nm in ["word_emb", "pos_emb", "layer0.q.w", "layer1.ff2.b", "head_ln.scale", "vocab_bias"]:
        k = names.index(nm)
        idx = tuple(np.unravel_index(3, args[k].shape))
        h = 1e-5
        up, dn = [x.copy() for x in args], [x.copy() for x in args]
        up[k][idx] += h
        dn[k][idx] -= h
        fd = (float(interp.run_text(prog.text, up, wide=True)[0]) - float(interp.run_text(prog.text, dn, wide=True)[0])) / (2 * h)
        assert abs(fd - float(outs[1 + k][idx])) < 1e-6 * max(1.0, abs(fd)), nm


def test_plans_of_case_scatter_and_half_precision_contractions():
    """Compile-only checks (no GPU): a case becomes one step with a sub-plan per branch, the row scatter one
    scatter step, a bf16 dot_general an f32 implicit GEMM between converts; an unsupported scatter form is a
    compile error that names the restriction."""
    b = Builder()
    idx, x = b.arg((), "i32"), b.arg((4, 4), "f32")
    outs = b.case(idx, [lambda s: [s.exp(x)], lambda s: [s.neg(x)]], [((4, 4), "f32")])
    plan, _ = b200.compile_to_plan(b.module(outs))
    assert "case branches=2" in plan

    b = Builder()
    t, i, u = b.arg((12, 8), "bf16"), b.arg((5,), "i32"), b.arg((5, 8), "bf16")
    plan, _ = b200.compile_to_plan(b.module([b.scatter_rows(t, i, u, "add")]))
    assert "scatter rows=12 row_elems=8 updates=5" in plan

    b = Builder()
    p, q = b.arg((64, 64), "bf16"), b.arg((64, 64), "bf16")
    plan, src = b200.compile_to_plan(b.module([b.matmul(p, q)]))
    assert "gemm16 M=64 N=64 K=64" in plan and "convert" not in plan          # native 16-bit tiles, no widened copies
    # a bf16 operand against an f32 one has no native kernel: both sides go through f32
    b = Builder()
    p, q = b.arg((64, 64), "bf16"), b.arg((64, 64), "f32")
    plan, src = b200.compile_to_plan(b.module([b.dot_general(b.convert(p, "f32"), q, ((1,), (0,)))]))
    assert "igemm M=64 N=64 K=64" in plan
    # an operand whose row stride is not a multiple of 16 bytes is copied into padded rows first
    b = Builder()
    p, q = b.arg((64, 100), "bf16"), b.arg((100, 30), "bf16")
    plan, src = b200.compile_to_plan(b.module([b.matmul(p, q)]))
    assert plan.count("repack16") == 2 and "ld 100->104" in plan and "ld 30->32" in plan and "gemm16 M=64 N=30 K=100" in plan

    b = Builder()
    t, i, u = b.arg((12, 8), "f32"), b.arg((5, 2), "i32"), b.arg((5,), "f32")
    sdn = ("#stablehlo.scatter<update_window_dims = [], inserted_window_dims = [0, 1], "
           "scatter_dims_to_operand_dims = [0, 1], index_vector_dim = 1>")
    reg = b.region([((), "f32")] * 2, lambda s, a, c: s.add(a, c))
    (y,) = b.emit("stablehlo.scatter", [t, i, u], [((12, 8), "f32")],
                  props={"scatter_dimension_numbers": sdn, "indices_are_sorted": "false", "unique_indices": "false"}, regions=[reg])
    plan, _ = b200.compile_to_plan(b.module([y]))          # any other form: key kernel + sorted apply
    assert "scatter keys" in plan and "row_elems=1" in plan, plan


def test_device_assignment_proto_round_trip():
    """The hand-encoded xla.DeviceAssignmentProto (src/proto/device_assignment.proto:9-17 of the reference) decodes back
    to what went in; the single-device case is byte for byte what protobuf writes for the reference's 1 x 1 assignment
    (pjrt_executable.cc:290-313: replica_count 1, computation_count 1, one ComputationDevice [0])."""
    assert b200.encode_device_assignment([[0]]) == bytes([0x08, 1, 0x10, 1, 0x1A, 3, 0x0A, 1, 0])
    for ids in ([[0, 1, 2, 3, 4, 5, 6, 7]], [[k] for k in range(8)], [[0, 1], [2, 3], [300, 70000]]):
        data = b200.encode_device_assignment(ids)
        reps, comps, rows = b200.decode_device_assignment(data)
        assert (reps, comps) == (len(ids[0]), len(ids)) and rows == [list(r) for r in ids]


def test_profiler_stub_accepts_a_session_and_returns_an_empty_trace():
    """Like the reference's stub (src/pjrt_plugin/pjrt_profiler.cc:17-125): create, start, stop, collect nothing."""
    p = b200.Profiler(b"options")
    p.start()
    with pytest.raises(b200.B200Error):
        p.start()
    p.stop()
    with pytest.raises(b200.B200Error):
        p.stop()
    assert p.collect() == b""


def test_all_gather_plans_and_oracle():
    """stablehlo.all_gather over all partitions: one NCCL step per operand (with a staging buffer when the gathered
    dimension is not the outermost); one partition is the identity; the interpreter concatenates what its `gather`
    callable returns."""
    from oracle import interp
    b = Builder()
    x = b.arg((6, 5), "f32")
    text = b.module([b.all_gather(x, 4, 0), b.all_gather(x, 4, 1)], num_partitions=4)
    plan = b200.compile_to_plan(text, num_processes=4, process_index=1)[0]
    assert plan.count("all_gather 120 bytes per partition") == 2 and "rows=1" in plan and "rows=6" in plan
    with pytest.raises(b200.B200Error):
        b200.compile_to_plan(text, num_processes=2)           # the group must span the job
    shards = [np.arange(30, dtype=np.float32).reshape(6, 5) + 100 * r for r in range(4)]
    outs = interp.Interp(text, gather=lambda v: shards, partition_id=1).run([shards[1]])
    np.testing.assert_array_equal(outs[0], np.concatenate(shards, 0))
    np.testing.assert_array_equal(outs[1], np.concatenate(shards, 1))
    b = Builder()
    x = b.arg((6, 5), "f32")
    one = b.module([b.all_gather(x, 1, 1)])
    np.testing.assert_array_equal(interp.run_text(one, [shards[0]])[0], shards[0])
