"""Program-level parity on the GPU: the committed golden fixtures (literal
expectations of the reference's own tests; PyTorch float64 twin of the
ResNet18 step) and the training step against the oracle, through the C ABI."""
import json

import numpy as np
import pytest

import b200
from b200.shlo import programs
from oracle import interp
from tests.test_oracle_golden import LITERALS, check_resnet_against_golden, literal_inputs, resnet_tiny_args
from tests.util import compare, run_gpu

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", LITERALS, ids=[c["name"] for c in LITERALS])
def test_reference_literals_on_gpu(client, case):
    """The reference's raw-MLIR injection test (tests/test_ops.py:245-281): compile text, execute, compare."""
    outs, _ = run_gpu(client, case["mlir"], literal_inputs(case))
    for i, (o, e) in enumerate(zip(outs, case["expected"])):
        if i in case["skip"]:
            continue
        np.testing.assert_allclose(o, np.array(e, np.float32), rtol=case["rtol"], atol=case["atol"])


def test_resnet_step_matches_torch_twin_golden(client):
    g, prog, args = resnet_tiny_args()
    outs, exe = run_gpu(client, prog.text, args)
    check_resnet_against_golden(g, prog, outs, rtol=1e-4, atol_scale=1e-5)
    assert exe.launches_per_execute > 0


@pytest.mark.parametrize("batch,image,width", [(16, 16, 16), (32, 32, 8)])
def test_resnet_step_matches_oracle(client, batch, image, width):
    """Loss, every updated parameter and every momentum buffer against the
    float64 oracle at the plugin's fp32 bar (rtol 1e-4; atol 1e-5 scaled by the
    leaf's magnitude, since each gradient is a sum over batch * pixels terms)."""
    prog = programs.resnet18_train_step(batch=batch, image=image, width=width)
    args = programs.resnet18_inputs(prog)
    outs, _ = run_gpu(client, prog.text, args)
    ref = interp.run_text(prog.text, args, wide=True)
    for (name, _, _), o, r in zip(prog.results, outs, ref):
        compare(o, r, rtol=1e-4, atol=1e-5, what=name, scale_atol=True)


def test_resnet_two_steps_feed_outputs_back(client):
    """Outputs of step k are the arguments of step k+1 (device-resident), as in the training loop."""
    prog = programs.resnet18_train_step(batch=8, image=16, width=8)
    args = programs.resnet18_inputs(prog)
    exe = client.compile(prog.text)
    bufs = [client.buffer_from_host(a) for a in args]
    n = (len(args) - 2) // 2
    cur = list(args)
    for _ in range(2):
        outs = exe.execute(bufs)
        bufs = outs[1:] + bufs[-2:]
        ref = interp.run_text(prog.text, cur, wide=True)
        cur = [np.asarray(r, np.float32) for r in ref[1:]] + cur[-2:]
        compare(outs[0].to_numpy(), ref[0], rtol=1e-4, atol=1e-5, what="loss")
    compare(outs[1 + n].to_numpy(), ref[1 + n], rtol=1e-3, atol=1e-5, what="momentum leaf", scale_atol=True)


def test_same_program_text_hits_the_plan_cache(client):
    prog = programs.resnet18_train_step(batch=4, image=8, width=8)
    e1 = client.compile(prog.text)
    import time
    t = time.time()
    e2 = client.compile(prog.text)
    assert time.time() - t < 0.2 and e1.fingerprint == e2.fingerprint


def test_argument_checks(client):
    from b200.shlo.builder import Builder
    b = Builder()
    x = b.arg((4,), "f32")
    exe = client.compile(b.module([b.add(x, x)]))
    with pytest.raises(b200.B200Error):
        exe.execute([client.buffer_from_host(np.zeros(5, np.float32))])
    with pytest.raises(b200.B200Error):
        exe.execute([client.buffer_from_host(np.zeros(4, np.int32))])
    with pytest.raises(b200.B200Error):
        exe.execute([])
    buf = client.buffer_from_host(np.ones(4, np.float32))
    buf.delete()
    assert buf.is_deleted()
    with pytest.raises(b200.B200Error):
        exe.execute([buf])


def test_strided_and_zero_size_host_arrays(client):
    """Non-row-major host arrays are packed (src/pjrt_plugin/mlx_buffer.cc:151-201); zero-size arrays need no data."""
    a = np.arange(60, dtype=np.float32).reshape(5, 12)
    np.testing.assert_array_equal(client.buffer_from_host(a.T).to_numpy(), a.T)
    np.testing.assert_array_equal(client.buffer_from_host(a[::2, 1::3]).to_numpy(), a[::2, 1::3])
    z = client.buffer_from_host(np.zeros((0, 3), np.float32))
    assert z.shape == (0, 3) and z.to_numpy().shape == (0, 3)


def test_memory_stats_and_device_info(client):
    st = client.memory_stats()
    assert st.bytes_limit_is_set and st.bytes_limit > 100e9
    assert st.peak_bytes_in_use >= st.bytes_in_use >= 0
    assert "B200" in client.device_kind() and client.platform == "b200"
