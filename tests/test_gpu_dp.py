"""Two GPUs, one process each: the data-parallel ResNet step (per-shard body with stablehlo.all_reduce over
NCCL) against single-device steps on the two shards. With zero initial momentum the update is linear in the
gradient, so the data-parallel parameters equal the mean of the two single-device results, the loss is the
mean of the shard losses, and both replicas must hold identical bits afterwards. Skipped with fewer than 2 GPUs."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
CFG = dict(batch=8, image=16, width=8)
pytestmark = pytest.mark.gpu


def _stop(procs):
    """Ends children that are still running (between steps nothing of theirs is in flight that a peer waits for:
    the test is over either way), so that a failed or timed-out test cannot keep its process tree alive."""
    for p in procs:
        if p.is_alive():
            p.terminate()
            p.join(timeout=20)
        if p.is_alive():
            p.kill()


def _rank_main(rank, world, id_pipe, q, overlap):
    sys.path.insert(0, str(ROOT / "jax-mps_b200"))
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    if not overlap:
        os.environ["B200_NO_ALL_REDUCE_OVERLAP"] = "1"  # one all-reduce after the last gradient instead of buckets inside the backward pass
    try:
        import b200
        from b200.shlo import programs
        if rank == 0:
            nccl_id = b200.nccl_unique_id()
            for p in id_pipe:
                p.send(nccl_id)
        else:
            nccl_id = id_pipe.recv()
        dp = b200.Client(device_ordinal=rank, process_index=rank, num_processes=world, nccl_id=nccl_id)
        prog = programs.resnet18_train_step(n_partitions=world, **CFG)
        args = programs.resnet18_inputs(prog, rank=rank)
        outs = [o.to_numpy() for o in dp.compile(prog.text).execute([dp.buffer_from_host(a) for a in args])]
        dp.synchronize()
        single = b200.Client(device_ordinal=rank)
        prog1 = programs.resnet18_train_step(n_partitions=1, **CFG)
        outs1 = [o.to_numpy() for o in single.compile(prog1.text).execute([single.buffer_from_host(a) for a in args])]
        single.synchronize()
        q.put((rank, outs, outs1))
    except Exception as e:          # surface the failure instead of leaving the parent to time out
        q.put((rank, repr(e), None))


@pytest.mark.parametrize("overlap", [False, True])
def test_two_gpu_step_is_the_mean_of_the_shard_steps(overlap):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    recv, send = ctx.Pipe(duplex=False)
    # daemonic children: a rank that waits for a peer that died goes down with the test instead of outliving it
    procs = [ctx.Process(target=_rank_main, args=(0, world, [send], q, overlap), daemon=True),
             ctx.Process(target=_rank_main, args=(1, world, recv, q, overlap), daemon=True)]
    for p in procs:
        p.start()
    got = {}
    try:
        for _ in range(world):
            r, a, b = q.get(timeout=180)
            assert not isinstance(a, str), f"rank {r} failed: {a}"
            got[r] = (a, b)
        for p in procs:
            p.join(timeout=60)
    finally:
        _stop(procs)
    n_leaves = (len(got[0][0]) - 1) // 2
    np.testing.assert_allclose(got[0][0][0], (got[0][1][0] + got[1][1][0]) / 2, rtol=1e-5)
    for i in range(1, len(got[0][0])):
        np.testing.assert_array_equal(got[0][0][i], got[1][0][i], err_msg=f"replicas differ at result {i}")
        want = (got[0][1][i].astype(np.float64) + got[1][1][i].astype(np.float64)) / 2
        scale = max(1.0, float(np.max(np.abs(want))))
        np.testing.assert_allclose(got[0][0][i], want, rtol=1e-4, atol=1e-5 * scale, err_msg=f"result {i}")
    assert n_leaves == 62


def _group_main(q):
    """One process driving both GPUs through a device group (run in a child so that NVLS stays off for it)."""
    sys.path.insert(0, str(ROOT / "jax-mps_b200"))
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    try:
        import b200
        from b200.shlo import programs
        world = 2
        group = b200.DeviceGroup(num_devices=world)
        prog = programs.resnet18_train_step(n_partitions=world, **CFG)
        exes = group.compile(prog.text)
        shard_args = [programs.resnet18_inputs(prog, rank=d) for d in range(world)]
        arg_lists = [[group.devices[d].buffer_from_host(a) for a in shard_args[d]] for d in range(world)]
        outs, events = group.execute(exes, arg_lists)
        for e in events:
            e.wait()
        dp = [[o.to_numpy() for o in outs[d]] for d in range(world)]
        devs = [outs[d][1].client is group.devices[d] for d in range(world)]
        assign = exes[0].device_assignment()
        topo = [d["id"] for d in group.devices[0].topology()["devices"]]
        prog1 = programs.resnet18_train_step(n_partitions=1, **CFG)
        single = b200.Client(device_ordinal=0)
        exe1 = single.compile(prog1.text)
        ones = [[o.to_numpy() for o in exe1.execute([single.buffer_from_host(a) for a in shard_args[d]])] for d in range(world)]
        q.put((dp, ones, devs, assign, topo))
    except Exception as e:
        import traceback
        q.put((repr(e) + traceback.format_exc(), None, None, None, None))


def test_one_process_drives_two_devices_through_per_device_argument_lists():
    """Both GPUs as devices of one process: argument_lists[d] / output_lists[d] / one completion event per device. The
    result must be the mean of the two single-device shard steps and identical on both devices."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_group_main, args=(q,), daemon=True)
    p.start()
    try:
        dp, ones, devs, assign, topo = q.get(timeout=180)
        p.join(timeout=60)
    finally:
        _stop([p])
    assert not isinstance(dp, str), dp
    assert devs == [True, True] and topo == [0, 1]
    assert assign == (1, 2, [[0], [1]])
    np.testing.assert_allclose(dp[0][0], (ones[0][0] + ones[1][0]) / 2, rtol=1e-5)
    for i in range(1, len(dp[0])):
        np.testing.assert_array_equal(dp[0][i], dp[1][i], err_msg=f"devices differ at result {i}")
        want = (ones[0][i].astype(np.float64) + ones[1][i].astype(np.float64)) / 2
        scale = max(1.0, float(np.max(np.abs(want))))
        np.testing.assert_allclose(dp[0][i], want, rtol=1e-4, atol=1e-5 * scale, err_msg=f"result {i}")


def _gather_main(q):
    sys.path.insert(0, str(ROOT / "jax-mps_b200"))
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    try:
        import b200
        from b200.shlo.builder import Builder
        world = 2
        group = b200.DeviceGroup(num_devices=world)
        b = Builder()
        x, y = b.arg((6, 5), "f32"), b.arg((4, 3, 8), "bf16")
        s_ = b.all_reduce_sum([x], world)[0]
        text = b.module([b.all_gather(x, world, 0), b.all_gather(x, world, 1), b.all_gather(y, world, 1), s_], num_partitions=world)
        exes = group.compile(text)
        xs = [np.arange(30, dtype=np.float32).reshape(6, 5) + 100 * d for d in range(world)]
        ys = [(np.arange(96, dtype=np.float32).reshape(4, 3, 8) - 40 * d) for d in range(world)]
        args = [[group.devices[d].buffer_from_host(xs[d]), group.devices[d].buffer_from_host(ys[d], dtype="bf16")] for d in range(world)]
        outs, events = group.execute(exes, args)
        for e in events:
            e.wait()
        q.put(([[o.to_numpy() for o in outs[d]] for d in range(world)], xs, ys))
    except Exception as e:
        import traceback
        q.put((repr(e) + traceback.format_exc(), None, None))


def test_all_gather_over_two_devices():
    """stablehlo.all_gather over NCCL: along the outermost dimension (gathered in place) and along inner dimensions
    (gathered into a staging buffer and laid out by strided copies), f32 and bf16, beside an all_reduce of the same job;
    both devices must hold the concatenation in partition order."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_gather_main, args=(q,), daemon=True)
    p.start()
    try:
        outs, xs, ys = q.get(timeout=180)
        p.join(timeout=60)
    finally:
        _stop([p])
    assert not isinstance(outs, str), outs
    for d in range(2):
        np.testing.assert_array_equal(outs[d][0], np.concatenate(xs, 0))
        np.testing.assert_array_equal(outs[d][1], np.concatenate(xs, 1))
        np.testing.assert_array_equal(outs[d][2], np.concatenate(ys, 1))
        np.testing.assert_array_equal(outs[d][3], xs[0] + xs[1])
