"""Attention of a few query rows over a cache (a decode step): dot_general -> scale / mask -> softmax -> dot_general is
recognised and runs as one kernel (the reference has the same chain as its fused attention call,
src/pjrt_plugin/ops/control_flow.cc:1484-1533). The oracle interprets the unfused operations; the GPU result is held to
it at the tolerance of the 16-bit element type."""
import os

import numpy as np
import pytest

import b200
from b200.shlo.builder import Builder
from b200.shlo.programs import decode_attention as attention_program
from oracle import interp


def _inputs(G, M, T, D, N, seed=0):
    rng = np.random.default_rng(seed)
    lead = () if G is None else (G,)
    f = lambda *s: rng.standard_normal(lead + s).astype(np.float32)
    return [f(M, D), f(T, D), f(T, N)]


def test_attention_chain_becomes_one_kernel():
    text = attention_program(None, 8, 640, 256, 256)
    plan, _ = b200.compile_to_plan(text, validate=True)
    assert plan.count("attention_") == 1 and "gemv16" not in plan and "row_" not in plan, plan
    assert "grid=20x1" in plan                                       # 640 positions in chunks of 32
    os.environ["B200_NO_ATTENTION_FUSION"] = "1"
    try:
        plan0, _ = b200.compile_to_plan(text)
    finally:
        del os.environ["B200_NO_ATTENTION_FUSION"]
    assert "attention_" not in plan0 and plan0.count("gemv16") == 2
    # a batch of groups, one chunk, f16
    plan, _ = b200.compile_to_plan(attention_program(3, 2, 24, 64, 32, dt="f16"), validate=True)
    assert plan.count("attention_") == 1 and "grid=1x3" in plan, plan


def test_keepdims_spelling_of_the_softmax_is_recognised():
    """jax.nn.softmax keeps the reduced dimension ([..., 1]) and broadcasts over all dimensions; both spellings give the
    same fused plan, and the interpreter gives the same numbers for both."""
    plain = attention_program(2, 4, 70, 64, 32)
    kd = attention_program(2, 4, 70, 64, 32, keepdims=True)
    assert "reshape" in kd and kd != plain
    p0, _ = b200.compile_to_plan(plain, validate=True)
    p1, _ = b200.compile_to_plan(kd, validate=True)
    assert p1.count("attention_") == 1 and "row_" not in p1 and "gemv16" not in p1, p1
    strip = lambda p: [l.split("args=")[0] for l in p.splitlines()[1:]]
    assert strip(p0) == strip(p1)
    args = _inputs(2, 4, 70, 64, 32) + [np.array(50, np.int32)]
    np.testing.assert_array_equal(interp.run_text(plain, args)[0], interp.run_text(kd, args)[0])


def test_attention_is_left_alone_where_the_kernel_does_not_apply():
    for args in [dict(G=None, M=16, T=64, D=64, N=64),           # more than eight query rows
                 dict(G=None, M=4, T=64, D=512, N=64),           # features beyond the staged row size
                 dict(G=None, M=4, T=64, D=60, N=64)]:           # rows that are not whole 16-byte pieces
        plan, _ = b200.compile_to_plan(attention_program(**args))
        assert "attention_" not in plan, plan
    # a second reader of the probabilities keeps the chain apart
    b = Builder()
    q, k, v = b.arg((4, 64), "bf16"), b.arg((96, 64), "bf16"), b.arg((96, 64), "bf16")
    sc = b.convert(b.dot_general(q, k, ((1,), (1,))), "f32")
    m = b.reduce_max(sc, (1,))
    e = b.exp(b.sub(sc, b.bcast(m, sc.shape, (0,))))
    pr = b.div(e, b.bcast(b.reduce_sum(e, (1,)), sc.shape, (0,)))
    att = b.dot_general(b.convert(pr, "bf16"), v, ((1,), (0,)))
    plan, _ = b200.compile_to_plan(b.module([att, pr]))
    assert "attention_" not in plan, plan


GPU_CASES = [  # G, M, T, D, N, dtype, masked, out_f32, upto
    (None, 8, 640, 256, 256, "bf16", True, True, 517),
    (None, 8, 640, 256, 256, "bf16", True, True, 3),             # most chunks fully masked
    (None, 1, 33, 64, 64, "bf16", True, True, 32),
    (None, 5, 100, 128, 64, "bf16", False, False, 0),
    (3, 2, 24, 64, 32, "f16", True, True, 11),                    # one chunk, groups
    (2, 8, 257, 64, 128, "bf16", True, False, 200),
    (4, 3, 2048, 128, 128, "bf16", True, True, 2047),
]


@pytest.mark.gpu
@pytest.mark.parametrize("G,M,T,D,N,dt,masked,out_f32,upto", GPU_CASES)
def test_decode_attention_on_the_gpu(client, G, M, T, D, N, dt, masked, out_f32, upto):
    from util import run_gpu
    text = attention_program(G, M, T, D, N, dt, masked, out_f32)
    args = _inputs(G, M, T, D, N) + [np.array(upto, np.int32)]
    got, _ = run_gpu(client, text, args, dtypes=[dt, dt, dt, "i32"])
    want = interp.run_text(text, [np.asarray(a) for a in args])
    # the probabilities are not rounded to 16 bits inside the kernel: agreement to the rounding of the element type
    np.testing.assert_allclose(np.asarray(got[0], np.float64), np.asarray(want[0], np.float64), rtol=2e-2, atol=2e-2)
    os.environ["B200_NO_ATTENTION_FUSION"] = "1"
    try:
        ref, _ = run_gpu(client, text, args, dtypes=[dt, dt, dt, "i32"])
    finally:
        del os.environ["B200_NO_ATTENTION_FUSION"]
    np.testing.assert_allclose(np.asarray(got[0], np.float64), np.asarray(ref[0], np.float64), rtol=2e-2, atol=1e-2)


@pytest.mark.gpu
def test_decode_attention_replays(client):
    """The counter that elects a group's last block is back at zero after every launch: a second and a third execution
    of the same program give the same bits."""
    text = attention_program(2, 8, 257, 64, 128)
    args = _inputs(2, 8, 257, 64, 128, seed=1) + [np.array(100, np.int32)]
    exe = client.compile(text)
    bufs = [client.buffer_from_host(a, dtype=d) for a, d in zip(args, ["bf16", "bf16", "bf16", "i32"])]
    outs = [exe.execute(bufs)[0].to_numpy() for _ in range(3)]
    np.testing.assert_array_equal(outs[0], outs[1])
    np.testing.assert_array_equal(outs[0], outs[2])
