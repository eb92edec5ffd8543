"""Single-operation timings through the public client API (used for the ncu
captures summarised under profiles/, and handy when tuning a kernel):

    python -m b200.bench_ops conv --case s1 [--reps 10]
    python -m b200.bench_ops reduce --shape 128,32,32,64 --dims 0,1,2
    python -m b200.bench_ops scan [--reps 10]

`scan` times the full-size LSTM-by-scan training step (100 time steps, batch 64, 32 -> 256 -> 256, Adam: a forward
and a reverse counted loop, 200 dependent iterations) and, beside it, the floor of one dependent kernel launch
inside a replayed loop (a counted loop of 2000 iterations whose body is one tiny kernel).

Convolution cases are the ResNet18 (batch 128) layer shapes: s1..s4 = the 3x3
stride-1 convolution of stage 1..4 (forward form).
"""
from __future__ import annotations

import argparse
import time

import numpy as np

import b200
from b200.shlo.builder import Builder

CONV_CASES = {"s1": ((128, 32, 32, 64), (3, 3, 64, 64)), "s2": ((128, 16, 16, 128), (3, 3, 128, 128)),
              "s3": ((128, 8, 8, 256), (3, 3, 256, 256)), "s4": ((128, 4, 4, 512), (3, 3, 512, 512))}


def time_program(client, text, arrays, reps):
    exe = client.compile(text)
    bufs = [client.buffer_from_host(a) for a in arrays]
    for _ in range(3):
        exe.execute(bufs)
    client.synchronize()
    client.set_profiling(True)
    for _ in range(reps):
        exe.execute(bufs)
    client.set_profiling(False)
    rep = client.profile_report()
    return sum(r["ms"] for r in rep) / reps, rep


def wall_ms(client, exe, bufs, reps):
    for _ in range(3):
        exe.execute(bufs)
    client.synchronize()
    t0 = time.perf_counter()
    for _ in range(reps):
        exe.execute(bufs)
    client.synchronize()
    return (time.perf_counter() - t0) * 1e3 / reps


def scan(client, reps):
    from b200.shlo import programs
    prog = programs.lstm_scan_train_step()
    exe = client.compile(prog.text)
    bufs = [client.buffer_from_host(a) for a in programs.lstm_inputs(prog, seed=0)]
    ms = wall_ms(client, exe, bufs, reps)
    print(f"lstm scan step: {ms:.2f} ms = {ms * 1e3 / 200:.1f} us per scan iteration (200 dependent iterations, "
          f"{exe.launches_per_execute} launches per step)")
    b = Builder()
    x = b.arg((16,), "f32")
    trips = 2000
    outs = b.while_([b.const(0, "i32"), x], lambda s, i, v: s.compare(i, s.const(trips, "i32"), "LT"),
                    lambda s, i, v: [s.add(i, s.const(1, "i32")),
                                     s.add(s.mul(v, s.full((16,), 0.99, "f32")), s.full((16,), 0.01, "f32"))])
    e2 = client.compile(b.module(outs))
    ms2 = wall_ms(client, e2, [client.buffer_from_host(np.ones(16, np.float32))], reps)
    per = e2.launches_per_execute / trips
    print(f"dependent-kernel floor: {ms2 * 1e3 / e2.launches_per_execute:.2f} us per launch "
          f"({per:.0f} launch per iteration, {trips} iterations)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["conv", "reduce", "scan"])
    ap.add_argument("--case", default="s1")
    ap.add_argument("--shape", default="128,32,32,64")
    ap.add_argument("--dims", default="0,1,2")
    ap.add_argument("--reps", type=int, default=10)
    a = ap.parse_args()
    client = b200.Client()
    rng = np.random.default_rng(0)
    b = Builder()
    if a.what == "scan":
        scan(client, a.reps)
        return
    if a.what == "conv":
        xs, ws = CONV_CASES[a.case]
        x, w = b.arg(xs, "f32"), b.arg(ws, "f32")
        text = b.module([b.conv(x, w, padding=((1, 1), (1, 1)))])
        ms, _ = time_program(client, text, [rng.standard_normal(xs).astype(np.float32),
                                            rng.standard_normal(ws).astype(np.float32)], a.reps)
        flop = 2.0 * np.prod(xs[:3]) * np.prod(ws)
        print(f"conv {a.case}: {ms * 1e3:.1f} us per launch, {flop / ms / 1e9:.1f} TFLOP/s (algorithmic fp32 flop)")
    else:
        shape = tuple(int(v) for v in a.shape.split(","))
        dims = tuple(int(v) for v in a.dims.split(","))
        x = b.arg(shape, "f32")
        text = b.module([b.reduce_sum(x, dims)])
        ms, _ = time_program(client, text, [rng.standard_normal(shape).astype(np.float32)], a.reps)
        print(f"reduce_sum {shape} over {dims}: {ms * 1e3:.1f} us, {np.prod(shape) * 4 / ms / 1e6:.0f} GB/s read")
    client.synchronize()


if __name__ == "__main__":
    main()
