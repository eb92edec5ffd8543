"""Events, completion callbacks, buffer copies, donation and the failure path of bounded device-side waits, through
the C ABI on the GPU (the reference's counterparts: PJRT_Event_* and the completion thread src/pjrt_plugin/
pjrt_event.cc:28-193, PJRT_Buffer_CopyToDevice pjrt_buffer.cc:101-131, donation mlx_executable.cc:306-336)."""
import threading

import numpy as np
import pytest

import b200
from b200.shlo.builder import Builder

pytestmark = pytest.mark.gpu


def _matmul_program(n=256):
    b = Builder()
    x, w = b.arg((n, n), "f32"), b.arg((n, n), "f32")
    return b.module([b.tanh(b.matmul(x, w))])


def test_completion_event_callback_and_error_query(client):
    exe = client.compile(_matmul_program())
    rng = np.random.default_rng(0)
    a, w = rng.standard_normal((256, 256)).astype(np.float32), rng.standard_normal((256, 256)).astype(np.float32)
    outs, done = exe.execute([client.buffer_from_host(a), client.buffer_from_host(w)], with_event=True)
    fired = threading.Event()
    seen = []
    done.on_ready(lambda err: (seen.append(err), fired.set()))
    assert fired.wait(30.0), "completion callback did not fire"
    assert seen == [None]
    done.wait()
    assert done.is_ready() and done.error() is None
    np.testing.assert_allclose(outs[0].to_numpy(), np.tanh(a @ w), rtol=1e-4, atol=1e-4)
    # a callback registered on an event that is already complete fires too
    again = threading.Event()
    done.on_ready(lambda err: again.set())
    assert again.wait(30.0)


def test_buffer_copy_is_independent_of_its_source(client):
    a = np.arange(4096, dtype=np.float32).reshape(64, 64)
    src = client.buffer_from_host(a)
    cp = src.copy()
    assert cp.device_pointer() != src.device_pointer() and cp.shape == (64, 64)
    src.delete()
    np.testing.assert_array_equal(cp.to_numpy(), a)
    with pytest.raises(b200.B200Error):
        src.copy()


def test_expired_device_wait_reaches_the_execution_event_and_its_outputs(client):
    """A bounded wait that runs out inside an execution (test hook: a barrier nothing arrives at, a budget of a
    thousand polls) is reported by that execution's completion event, by reads of its outputs and once by
    synchronize; the context stays usable and the next execution is clean."""
    exe = client.compile(_matmul_program())
    rng = np.random.default_rng(1)
    a, w = rng.standard_normal((256, 256)).astype(np.float32), rng.standard_normal((256, 256)).astype(np.float32)
    bufs = [client.buffer_from_host(a), client.buffer_from_host(w)]
    client.synchronize()
    client.debug_arm_wait_expiry(1000)
    outs, done = exe.execute(bufs, with_event=True)
    with pytest.raises(b200.B200Error) as ei:
        done.wait()
    assert ei.value.code == 13 and "bounded" in str(ei.value)
    assert done.error() is not None
    with pytest.raises(b200.B200Error):
        outs[0].to_numpy()
    got = []
    fired = threading.Event()
    done.on_ready(lambda err: (got.append(err), fired.set()))
    assert fired.wait(30.0) and isinstance(got[0], b200.B200Error)
    with pytest.raises(b200.B200Error):
        client.synchronize()
    client.synchronize()                                   # reported once
    outs2, done2 = exe.execute(bufs, with_event=True)
    done2.wait()
    assert done2.error() is None
    np.testing.assert_allclose(outs2[0].to_numpy(), np.tanh(a @ w), rtol=1e-4, atol=1e-4)


def test_donated_arguments_are_consumed(client):
    """tf.aliasing_output marks the parameter as donated: after an execution with donation its buffer is deleted and
    its memory is back in the pool; the result is right and the bytes in use do not grow from step to step."""
    b = Builder()
    p = b.arg((1024, 256), "f32", attrs="tf.aliasing_output = 0 : i32")
    g = b.arg((1024, 256), "f32")
    text = b.module([b.sub(p, b.mul(g, b.full((1024, 256), 0.1, "f32")))])
    exe = client.compile(text)
    rng = np.random.default_rng(2)
    p0, g0 = rng.standard_normal((1024, 256)).astype(np.float32), rng.standard_normal((1024, 256)).astype(np.float32)
    pb, gb = client.buffer_from_host(p0), client.buffer_from_host(g0)
    want = p0.copy()
    in_use = []
    for _ in range(4):
        (nb,) = exe.execute([pb, gb], donate=True)
        assert pb.is_deleted() and not gb.is_deleted()
        with pytest.raises(b200.B200Error):
            pb.to_numpy()
        pb = nb
        want = want - g0 * np.float32(0.1)
        client.synchronize()
        in_use.append(client.memory_stats().bytes_in_use)
    np.testing.assert_allclose(pb.to_numpy(), want, rtol=1e-6, atol=1e-6)
    assert len(set(in_use)) == 1, in_use
    # without donation the argument stays
    (nb,) = exe.execute([pb, gb])
    assert not pb.is_deleted()


def test_memory_spaces_topology_and_device_assignment(client):
    """The descriptors jaxlib asks a plugin for at start-up (pjrt_memory.cc:10-48, pjrt_device.cc:88-109,
    pjrt_topology.cc:10-70, pjrt_client.cc:259-265, pjrt_executable.cc:66-99,290-313 of the reference)."""
    mems = client.memories()
    assert len(mems) == 1 and mems[0]["kind"] == "device" and mems[0]["devices"] == [0] and mems[0]["id"] == 0
    assert "HBM" in mems[0]["debug_string"] and "kind=device" in mems[0]["to_string"]
    topo = client.topology()
    assert topo["platform_name"] == "b200" and topo["platform_version"] == client.platform_version
    assert [d["id"] for d in topo["devices"]] == [0] and "B200" in topo["devices"][0]["kind"]
    assert topo["fingerprint"] == client.topology()["fingerprint"] != 0
    assert client.default_device_assignment(1, 1) == [[0]]
    with pytest.raises(b200.B200Error):
        client.default_device_assignment(2, 1)              # one device in this job
    lib = b200.load_library()
    import ctypes as C
    out, size = C.c_void_p(), C.c_size_t(0)
    err = lib.b200_topology_serialize(client._h, C.byref(out), C.byref(size))
    assert err and lib.b200_error_get_code(err) == 12        # UNIMPLEMENTED, as in the reference
    lib.b200_error_destroy(err)
    exe = client.compile(_matmul_program(64))
    assert exe.device_assignment() == (1, 1, [[0]])
    assert exe.output_memory_kinds() == ["device"]
    buf = client.buffer_from_host(np.zeros(4, np.float32))
    assert lib.b200_buffer_memory(buf._h) == 0 == lib.b200_buffer_device(buf._h)
