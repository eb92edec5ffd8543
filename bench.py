"""Benchmark of the hot path: ResNet18 (CIFAR variant) training steps per
second, fp32, batch 128 per GPU, through the B200 plugin's C ABI.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one jitted value_and_grad + SGD-momentum update of the
reference's example model (examples/resnet/model.py, examples/resnet/main.py)
on one synthetic batch. With N > 1 (launched by torchrun, one process per
GPU) every rank trains on its own shard of a global batch of 128*N and the
program averages gradients with stablehlo.all_reduce over NCCL (weak scaling).

`--impl reference` times the CPU baseline instead: the reference's own
comparison backend (jaxlib CPU) is not installable here and the reference's
Metal path cannot run on Linux, so the PyTorch-CPU twin of the same step
(oracle/twins.py) is timed on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "jax-mps_b200"))
sys.path.insert(0, str(ROOT))

METRIC = "resnet18_cifar_train_steps_per_s"
UNIT = "steps/s (batch 128 per step and GPU)"
BATCH = 128
# convolution + dense multiply-adds of one training step at batch 128: forward 555 422 720 MAC per image,
# training = 3x forward minus the input gradient of the first convolution (1 769 472 MAC)
FLOP_PER_STEP = 2.0 * (3 * 555_422_720 - 1_769_472) * BATCH


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops_sustained", 1400.0), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def count(self, t0: float, t1: float) -> int:
        return sum(1 for t, _ in self.lines if t0 <= t <= t1)

    def stop(self, t0: float, t1: float) -> dict:
        """Summary of the samples that arrived between t0 and t1 (perf_counter times)."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for t, ln in self.lines:
            if not (t0 <= t <= t1):
                continue
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx = float(f[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_twin_steps(steps: int, warmup: int, threads: int):
    """Times the PyTorch-CPU twin of the training step. Returns (steps/s, ms/step)."""
    import torch
    from b200.shlo import programs
    from oracle import twins
    torch.set_num_threads(threads)
    w = programs.init_resnet18(0)
    rng = np.random.default_rng(1)
    x = rng.standard_normal((BATCH, 32, 32, 3)).astype(np.float32)
    y = rng.integers(0, 10, BATCH).astype(np.int32)
    st = twins.ResNet18Stepper(w, threads=threads)
    for _ in range(warmup):
        st.step(x, y)
    t0 = time.perf_counter()
    for _ in range(steps):
        st.step(x, y)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return 1.0 / dt, dt * 1e3


def extra_configs(client, hbm_gbs, tensor_tflops, which):
    """The other single-GPU configurations of the benchmark, beside the headline: Gemma-2B-shaped greedy decoding
    (tokens per second of the 128-step loop, bf16 weights resident in HBM; its roofline is the bytes of weights a
    token has to read over the measured copy bandwidth) and the DistilBERT-base-shaped masked-LM step (bf16)."""
    from b200 import bench_ops
    out = {}
    try:
        g = bench_ops.gemma_decode(client, reps=3, hbm_gbs=hbm_gbs)
        per_token = g["weight_bytes_per_token"]
        ach = per_token / (g["ms_per_token"] * 1e-3) / 1e9
        out["gemma_decode_tok_s"] = {
            "value": g["tok_s"], "unit": "tokens/s (batch 1, greedy, 128 new tokens after a 512-token prompt)",
            "ms_per_token": g["ms_per_token"], "decode_ms_all": g["decode_ms_all"], "prefill_ms": g["prefill_ms"],
            "launches_per_token": g["launches_per_token"], "dtype": "bf16",
            "config": {"workload": "gemma_2b_shaped_decode_18l_d2048_h8kv1_hd256_ffn16384_v256000_prompt512_new128"},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": hbm_gbs, "unit": "GB/s", "frac": ach / hbm_gbs, "traffic": None,
                         "bytes_per_token": per_token, "peak_source": f"copy bandwidth, {which}",
                         "note": "algorithmic bytes = every bf16 weight once per token (2 506 M parameters); the whole "
                                 "token step is timed, not one kernel"}}
    except Exception as e:
        out["gemma_decode_tok_s"] = {"error": str(e)[:300]}
    try:
        d = bench_ops.distilbert_step(client, reps=5)
        ach = d["tflops"]
        out["distilbert_step_ms"] = {
            "value": d["step_ms"], "unit": "ms per masked-LM step (batch 32 x 128 tokens, forward + backward)",
            "step_ms_all": d["step_ms_all"], "launches": d["launches"], "dtype": "bf16", "loss": d["loss"],
            "config": {"workload": "distilbert_base_shaped_mlm_step_6l_d768_h12_ffn3072_v30522_b32_s128"},
            "roofline": {"bound": "tensor", "achieved": ach, "peak": tensor_tflops, "unit": "TFLOP/s", "frac": ach / tensor_tflops,
                         "traffic": None, "flop_per_step": d["flop"], "peak_source": f"bf16 sustained, {which}"}}
    except Exception as e:
        out["distilbert_step_ms"] = {"error": str(e)[:300]}
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    steps, warm = max(1, args.steps), max(0, args.warmup)
    world = max(1, args.gpus)
    sps, ms = cpu_twin_steps(steps, warm, threads)
    # The unit counts steps of one batch-128 shard. With N GPUs the job's step is a global batch of 128 * N, which this
    # one host runs as N shard steps one after the other: its rate in shard steps per second is the same at every N
    # (the timed sample is one shard's step), and a global step takes N times as long.
    value = sps
    sample = (f"{steps} steps after {warm} warm-up of one batch-{BATCH} shard, PyTorch-CPU twin, {threads} threads" +
              (f"; a global step of {world} shards counted as {world} such steps" if world > 1 else ""))
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": ms * world, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "resnet18_cifar_b128_fp32_sgd_momentum_train_step", "batch_per_gpu": BATCH,
                   "global_batch": BATCH * world, "parallelism": f"dp{world}",
                   "note": "CPU arm: the reference's Metal path cannot run on Linux and jaxlib "
                   "(its CPU comparison backend) is not installable here; PyTorch-CPU stand-in of the same step"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_b200(args):
    import torch
    import b200
    from b200.shlo import programs

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with torch.distributed.run (one process per GPU)")
    import torch.distributed as dist
    nccl_id = None
    if world > 1:
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        box = [b200.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        nccl_id = box[0]
    client = b200.Client(device_ordinal=local, process_index=rank, num_processes=world, nccl_id=nccl_id)
    prog = programs.resnet18_train_step(batch=BATCH, n_partitions=world)
    host_args = programs.resnet18_inputs(prog, seed_w=0, seed_x=1, rank=rank)
    exe = client.compile(prog.text)
    n_state = len(host_args) - 2

    stream = torch.cuda.ExternalStream(client.compute_stream(), device=torch.device("cuda", local))

    def barrier():
        client.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(local)

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=torch.device("cuda", local), dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident loop: parameters and momentum stay in HBM, outputs feed the next step -------
    bufs = [client.buffer_from_host(a) for a in host_args]
    state, xy = bufs[:n_state], bufs[n_state:]
    # the sampler starts ahead of the warm-up so that nvidia-smi is up and reporting when the timed region begins;
    # only samples that arrive inside the window below are used
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        outs = exe.execute(state + xy)
        state = outs[1:]
    barrier()
    t_begin = time.perf_counter()
    # the timed region (exactly `steps` steps between two events on the launching stream, a barrier on both sides)
    # is repeated; the reported figure is the median repeat, every repeat is listed
    repeats_ms, own_ms = [], []
    for rep in range(max(1, args.repeats)):
        launches0 = client.launch_count()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            ev0.record()
        for _ in range(args.steps):
            outs = exe.execute(state + xy)
            state = outs[1:]
        with torch.cuda.stream(stream):
            ev1.record()
        barrier()
        own_ms.append(ev0.elapsed_time(ev1))
        repeats_ms.append(max_over_ranks(own_ms[-1]))
        launches = client.launch_count() - launches0
    ms_total = statistics.median(repeats_ms)
    loss = float(outs[0].to_numpy())
    # replicas must agree: every rank holds the same parameter bits after the same number of steps
    consistency = None
    if world > 1:
        import hashlib
        h = hashlib.sha256()
        for buf in state[:8] + state[n_state // 2 - 4:n_state // 2]:
            h.update(buf.to_numpy().tobytes())
        digests = [None] * world
        dist.all_gather_object(digests, (h.hexdigest(), loss, statistics.median(own_ms)))
        if len({d[0] for d in digests}) != 1 or len({d[1] for d in digests}) != 1:
            raise SystemExit(f"replicas diverged: {digests}")
        consistency = {"replicas_bit_identical": True, "leaves_hashed": 12, "loss_identical": True,
                       "rank_ms_per_step": [round(d[2] / args.steps, 4) for d in digests]}
    # A short timed region (30 steps are 0.16 s) can end before nvidia-smi has reported a few times: every rank then
    # keeps running the same steps, untimed, until 0.6 s of load have passed since the region began, and the
    # sampling window covers them too (ms_total is the maximum over ranks, so all ranks run the same count).
    window = "all repeats of the timed region"
    if sum(repeats_ms) < 600.0:
        for _ in range(int((600.0 - sum(repeats_ms)) / (ms_total / args.steps)) + 1):
            o2 = exe.execute(state + xy)
            state = o2[1:]
        window = "all repeats of the timed region and further identical steps, untimed, up to 0.6 s of load"
    barrier()
    clocks = None
    if rank == 0:
        clocks = sampler.stop(t_begin, time.perf_counter())
        clocks["window"] = window
    ms_step = ms_total / args.steps
    value = world * args.steps / (ms_total / 1e3)

    # ---- end to end: every step copies its batch from pinned host memory and reads the loss back ----
    x_pin = torch.from_numpy(host_args[-2]).pin_memory()
    y_pin = torch.from_numpy(host_args[-1]).pin_memory()
    loss_pin = torch.zeros((), dtype=torch.float32).pin_memory()
    for _ in range(2):
        xb, yb = client.buffer_from_host(x_pin.numpy()), client.buffer_from_host(y_pin.numpy())
        outs = exe.execute(state + [xb, yb])
        state = outs[1:]
        outs[0].to_host_async(loss_pin.numpy()).wait()
    barrier()
    t0 = time.perf_counter()
    # input double-buffering, as a training loop's loader does it: the copy of the next step's batch is issued
    # (copy stream) before the loss of the current step is awaited; every step still copies its own batch up and
    # reads its own loss back inside the timed region
    nxt = (client.buffer_from_host(x_pin.numpy()), client.buffer_from_host(y_pin.numpy()))
    for i in range(args.steps):
        xb, yb = nxt
        outs = exe.execute(state + [xb, yb])
        state = outs[1:]
        pending = outs[0].to_host_async(loss_pin.numpy())
        if i + 1 < args.steps:
            nxt = (client.buffer_from_host(x_pin.numpy()), client.buffer_from_host(y_pin.numpy()))
        pending.wait()
    barrier()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3)
    e2e_value = world * args.steps / (e2e_ms / 1e3)

    # ---- per-kernel-class device time of the same steps (CUDA events around every plan step) ----------
    client.set_profiling(True)
    psteps = min(args.steps, 5)
    for _ in range(psteps):
        outs = exe.execute(state + xy)
        state = outs[1:]
    client.set_profiling(False)
    rep = client.profile_report()
    by_kind = {}
    for r in rep:
        k = by_kind.setdefault(r["kind"], {"ms": 0.0, "count": 0})
        k["ms"] += r["ms"] / psteps
        k["count"] += r["count"] // psteps
    igemm_ms = by_kind.get("igemm", {}).get("ms", 0.0)
    hbm, tens, which = measured_peaks()
    family = FLOP_PER_STEP / (igemm_ms * 1e-3) / 1e12 if igemm_ms else 0.0
    # the dominant launch class: the 3x3 stride-1 convolutions of stage 1 (forward and input gradient,
    # M = 128*32*32 output pixels, N = 64 channels, K = 9*64), eight launches of one kernel per step
    dom = [r for r in rep if r["kind"] == "igemm" and " M=131072 N=64 K=576 " in r["key"] + " "]
    dom_ms = sum(r["ms"] for r in dom)
    dom_n = sum(r["count"] for r in dom)
    dom_flop = 2.0 * 131072 * 64 * 576
    achieved = dom_flop * dom_n / (dom_ms * 1e-3) / 1e12 if dom_ms else 0.0
    try:
        tf32_rate = client.probe_tf32_mma_rate()
    except Exception as e:          # the probe is an aid, not part of the measurement
        tf32_rate = None
    roofline = {"bound": "tensor", "achieved": achieved, "peak": tens, "unit": "TFLOP/s", "frac": achieved / tens,
                # DRAM bytes of one such launch (input 33.6 MB read once, the 33.6 MB output still in L2 when the kernel
                # ends); algorithmic bytes are 67.3 MB
                "traffic": 37.6e6,
                "traffic_source": "ncu capture of this kernel on this shape, profiles/igemm_tf32x3_ta_kernel_conv3x3_stage1_stage3.md "
                                  "(dram__bytes_read.sum + dram__bytes_write.sum per launch); not re-measured by this run",
                "own_ceiling": {"tf32_mma_tflops": tf32_rate, "fp32_accurate_tflops": tf32_rate / 3.0 if tf32_rate else None,
                                "frac": achieved / (tf32_rate / 3.0) if tf32_rate else None,
                                "how": "tcgen05.mma.kind::tf32 issue loop, one CTA per SM, measured in this run; the kernel "
                                       "issues three such MMAs per fp32 product"},
                "kernel": "igemm_tf32x3_ta_kernel<64,...> on M=131072 N=64 K=576 (stage-1 3x3 convolutions, forward "
                          "and input gradient), algorithmic fp32 flop 2*M*N*K per launch",
                "launches_per_step": dom_n // psteps, "us_per_launch": 1e3 * dom_ms / max(dom_n, 1),
                "peak_source": f"bf16 sustained, {which}; the fp32-accurate path issues three TF32 MMAs per product, "
                               "so its own ceiling is the TF32 rate / 3 (about 360 TFLOP/s measured issue rate)",
                "all_contractions": {"achieved": family, "frac": family / tens, "ms_per_step": igemm_ms,
                                     "flop_per_step": FLOP_PER_STEP},
                "ms_per_step_by_kind": {k: round(v["ms"], 4) for k, v in by_kind.items()},
                "launches_by_kind": {k: v["count"] for k, v in by_kind.items()}}

    # ---- strong scaling: a global batch of 1024 split over the GPUs (an extra key beside the weak-scaling headline) ----
    strong = None
    if args.strong:
        per = 1024 // world
        sprog = programs.resnet18_train_step(batch=per, n_partitions=world)
        sargs = programs.resnet18_inputs(sprog, seed_w=0, seed_x=1, rank=rank)
        sexe = client.compile(sprog.text)
        sb = [client.buffer_from_host(a) for a in sargs]
        sstate, sxy = sb[:len(sargs) - 2], sb[len(sargs) - 2:]
        for _ in range(3):
            o = sexe.execute(sstate + sxy)
            sstate = o[1:]
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record()
        ssteps = max(5, args.steps // 2)
        for _ in range(ssteps):
            o = sexe.execute(sstate + sxy)
            sstate = o[1:]
        with torch.cuda.stream(stream):
            e1.record()
        barrier()
        sms = max_over_ranks(e0.elapsed_time(e1)) / ssteps
        strong = {"global_batch": 1024, "batch_per_gpu": per, "ms_per_step": sms, "steps_per_s": 1e3 / sms,
                  "images_per_s": 1024 * 1e3 / sms, "steps": ssteps}
        del sb, sstate, sxy, o

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        sps, cms = cpu_twin_steps(4, 1, threads)
        cpu = {"value": sps, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"4 steps after 1 warm-up of the same batch-{BATCH} step, PyTorch-CPU twin (jaxlib CPU stand-in)",
               "ms_per_step": cms}
    h2d = int(host_args[-2].nbytes + host_args[-1].nbytes)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "resnet18_cifar_b128_fp32_sgd_momentum_train_step", "batch_per_gpu": BATCH,
                   "global_batch": BATCH * world, "parallelism": f"dp{world}", "params": prog.meta["params"],
                   "l2": "no flush: the step's working set (about 0.8 GB of activations plus 90 MB of parameters "
                         "and momentum) is larger than the 126 MB L2",
                   "temp_bytes": exe.temp_bytes, "generated_kernels": exe.num_kernels},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": int(launches), "launches_per_step": exe.launches_per_execute,
        "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu, "final_loss": loss,
        "repeats": {"count": len(repeats_ms), "ms_per_step_all": [round(m / args.steps, 4) for m in repeats_ms],
                    "reported": "median"},
        "comm_ms_per_step": by_kind.get("all_reduce", {}).get("ms") if world > 1 else 0.0,
        "replica_consistency": consistency,
    }
    if strong is not None:
        line["strong_scaling"] = strong
    if world == 1 and not args.no_extras:
        line.update(extra_configs(client, hbm, tens, which))
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--repeats", type=int, default=5, help="repeats of the timed region; the median is reported")
    ap.add_argument("--no-extras", action="store_true", help="skip the Gemma decode and DistilBERT extra keys (N = 1)")
    ap.add_argument("--no-strong", dest="strong", action="store_false", help="skip the strong-scaling extra measurement")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
