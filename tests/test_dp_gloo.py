"""CPU, two gloo ranks: the data-parallel program (per-shard body with
stablehlo.all_reduce) run in the oracle with a gloo all-reduce must agree with
the PyTorch twin stepping on both shards and averaging the gradients — the
host-side contract of the N > 1 path (one process per GPU, gradients and loss
summed over ranks, divided by N, then the SGD-momentum update)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
CFG = dict(batch=4, image=8, width=8)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
    sys.path.insert(0, str(ROOT / "jax-mps_b200"))
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    from b200.shlo import programs
    from oracle import interp
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    prog = programs.resnet18_train_step(n_partitions=world, **CFG)
    args = programs.resnet18_inputs(prog, rank=rank)

    def all_reduce(xs):
        out = []
        for x in xs:
            t = torch.from_numpy(np.array(x, dtype=np.float64).reshape(-1))
            dist.all_reduce(t)
            out.append(t.numpy().reshape(np.shape(x)))
        return out

    try:
        outs = interp.Interp(prog.text, collective=all_reduce, partition_id=rank, wide=True).run(args)
        q.put((rank, [np.asarray(o) for o in outs]))
        dist.barrier()
    except Exception as e:                       # surface the failure instead of leaving the parent to time out
        q.put((rank, repr(e)))
    dist.destroy_process_group()


def test_two_rank_data_parallel_step_matches_averaged_twin():
    import torch
    import torch.multiprocessing as mp
    sys.path.insert(0, str(ROOT / "jax-mps_b200"))
    from b200.shlo import programs
    from oracle import twins
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=300) for _ in range(world))
    for r, v in got.items():
        assert not isinstance(v, str), f"rank {r} failed: {v}"
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # expected: per-shard gradients from the twin, averaged, one shared update
    prog = programs.resnet18_train_step(n_partitions=world, **CFG)
    shard = [programs.resnet18_inputs(prog, rank=r) for r in range(world)]
    names = [n for n, _, _ in prog.args]
    P = {n[2:]: a for n, a in zip(names, shard[0]) if n.startswith("p.")}
    M = {n[2:]: a for n, a in zip(names, shard[0]) if n.startswith("m.")}
    grads, losses = [], []
    for r in range(world):
        loss, _, _, g = twins.resnet18_train_step(P, M, shard[r][-2], shard[r][-1], dtype=torch.float64)
        grads.append(g); losses.append(loss)
    mean_loss = float(np.mean(losses))
    for r in range(world):
        outs = got[r]
        assert abs(float(outs[0]) - mean_loss) < 1e-9 * max(1, abs(mean_loss))
        for (name, _, _), o in zip(prog.results[1:], outs[1:]):
            key = name[2:]
            g = sum(gr[key] for gr in grads) / world
            m = 0.9 * M[key].astype(np.float64) + g
            want = m if name.startswith("m.") else P[key].astype(np.float64) - 0.1 * m
            np.testing.assert_allclose(o, want, rtol=1e-6, atol=1e-7, err_msg=name)
    # both ranks hold identical replicas after the step
    for a, b in zip(got[0][1:], got[1][1:]):
        np.testing.assert_array_equal(a, b)
