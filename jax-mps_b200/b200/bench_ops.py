"""Single-operation timings through the public client API (used for the ncu
captures summarised under profiles/, and handy when tuning a kernel):

    python -m b200.bench_ops conv --case s1 [--reps 10]
    python -m b200.bench_ops reduce --shape 128,32,32,64 --dims 0,1,2
    python -m b200.bench_ops scan [--reps 10]
    python -m b200.bench_ops gemma [--layers 18] [--reps 3] [--profile]
    python -m b200.bench_ops distilbert [--reps 5] [--profile]
    python -m b200.bench_ops gemm --shape M,N,K [--reps 20]
    python -m b200.bench_ops gemv --shape M,N,K --layout kc|nc [--reps 50]
    python -m b200.bench_ops pointwise | transpose | softmax | gather | scatter [--dtype f32|bf16] [--reps 20]

`pointwise` is a batch-norm apply + residual + ReLU over a stage-1 activation (three tensors read, one written);
`transpose` a 2-D transpose of 8192 x 6144 elements (the tiled shared-memory kernel); `softmax` the attention softmax
of the DistilBERT-shaped step (49 152 rows of 128, one generated row kernel); `gather` / `scatter` the word-embedding
lookup of 4096 rows of 768 and its gradient (deterministic scatter-add into 30 522 rows).

`gemma` times the Gemma-2B-shaped prefill (512 prompt tokens in one pass) and the 128-step greedy decode loop (bf16
weights resident in HBM); `distilbert` the DistilBERT-base-shaped masked-LM step (forward + backward, bf16); `gemm` one
bf16 product [M,K] x [K,N]. `--profile` prints the device time per kernel class from CUDA events around every plan step.

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


def _events(client):
    """(record, elapsed_ms) timing with CUDA events on the client's own compute stream."""
    import torch
    stream = torch.cuda.ExternalStream(client.compute_stream())
    def record():
        ev = torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            ev.record()
        return ev
    return record


def _by_kind(rep, reps=1):
    out = {}
    for r in rep:
        k = out.setdefault(r["kind"], {"ms": 0.0, "count": 0})
        k["ms"] += r["ms"] / reps
        k["count"] += r["count"] // reps
    return out


def gemma_decode(client, reps=3, profile=False, hbm_gbs=6546.2, verbose=False, **shape):
    """Prefill once, then the decode loop `reps` times from the prefilled caches. Returns times, tokens per second and
    the fraction of the HBM roofline (bytes of weights read per token / time per token / copy bandwidth)."""
    from b200.shlo import programs
    pre = programs.gemma_prefill(**{k: v for k, v in shape.items() if k not in ("start", "new_tokens")})
    kw = dict(shape)
    kw.pop("prompt_len", None)
    dec = programs.gemma_decode_loop(start=pre.meta["prompt_len"], **kw)
    n_w = len(pre.args) - 1
    weights = programs.gemma_weights([(n, s) for n, s, _ in pre.args[:n_w]], seed=0, as_bits=True)
    wb = [client.buffer_from_host(w, dtype="bf16") for w in weights]
    del weights
    prompt = np.random.default_rng(1).integers(0, pre.meta["vocab"], pre.meta["prompt_len"]).astype(np.int32)
    pb = client.buffer_from_host(prompt)
    e_pre, e_dec = client.compile(pre.text), client.compile(dec.text)
    record = _events(client)
    outs = e_pre.execute(wb + [pb])
    client.synchronize()
    a = record()
    outs = e_pre.execute(wb + [pb])
    b = record()
    client.synchronize()
    prefill_ms = a.elapsed_time(b)
    tok, caches = outs[0], outs[2:]
    d = e_dec.execute(wb + [tok] + caches)          # first run records the loop's graph
    client.synchronize()
    times = []
    for _ in range(reps):
        a = record()
        d = e_dec.execute(wb + [tok] + caches)
        b = record()
        client.synchronize()
        times.append(a.elapsed_time(b))
    n_new = dec.meta["new_tokens"]
    ms = sorted(times)[len(times) // 2]
    res = {"prefill_ms": prefill_ms, "decode_ms": ms, "decode_ms_all": times, "new_tokens": n_new,
           "tok_s": n_new / (ms * 1e-3), "ms_per_token": ms / n_new, "weight_bytes_per_token": dec.meta["weight_bytes"],
           "hbm_frac": dec.meta["weight_bytes"] / (ms / n_new * 1e-3) / (hbm_gbs * 1e9),
           "launches_per_token": e_dec.launches_per_execute / n_new, "tokens": d[0].to_numpy().tolist()}
    if profile:
        client.set_profiling(True)
        e_dec.execute(wb + [tok] + caches)
        client.set_profiling(False)
        rep = client.profile_report()
        res["decode_by_kind"] = {k: {"ms_per_token": v["ms"] / n_new, "per_token": v["count"] / n_new} for k, v in _by_kind(rep).items()}
        if verbose:
            for r in sorted(rep, key=lambda r: -r["ms"])[:25]:
                print(f"  {r['ms'] / n_new * 1e3:9.1f} us/token x{r['count'] // n_new:<3d} {r['kind']:8s} {r['key'][:110]}")
        client.set_profiling(True)
        e_pre.execute(wb + [pb])
        client.set_profiling(False)
        rep = client.profile_report()
        res["prefill_by_kind"] = {k: {"ms": v["ms"], "count": v["count"]} for k, v in _by_kind(rep).items()}
        if verbose:
            for r in sorted(rep, key=lambda r: -r["ms"])[:20]:
                print(f"  {r['ms'] * 1e3:9.1f} us x{r['count']:<3d} {r['kind']:8s} {r['key'][:110]}")
    return res


def distilbert_step(client, reps=5, profile=False, verbose=False, **shape):
    """The DistilBERT-base-shaped masked-LM step (loss and every gradient, bf16). FLOP: 2 * 3 * 67.7 M multiply-adds per
    token over 4096 tokens (six layers and the tied-projector head, forward and two backward products)."""
    from b200.shlo import programs
    prog = programs.distilbert_mlm_step(**shape)
    args = programs.distilbert_inputs(prog, seed=0)
    dtypes = [d for _, _, d in prog.args]
    bufs = [client.buffer_from_host(a, dtype=(d if d == "bf16" else None)) for a, d in zip(args, dtypes)]
    exe = client.compile(prog.text)
    record = _events(client)
    for _ in range(3):
        outs = exe.execute(bufs)
    client.synchronize()
    times = []
    for _ in range(reps):
        a = record()
        outs = exe.execute(bufs)
        b = record()
        client.synchronize()
        times.append(a.elapsed_time(b))
    ms = sorted(times)[len(times) // 2]
    m = prog.meta
    tokens = m["batch"] * m["seq"]
    layers, dim, vocab = shape.get("layers", 6), m["dim"], m["vocab"]
    ffn, seq = shape.get("ffn", 3072), m["seq"]
    mac_per_token = layers * (4 * dim * dim + 2 * dim * ffn + 2 * seq * dim) + dim * dim + dim * vocab
    flop = 2.0 * 3 * mac_per_token * tokens
    res = {"step_ms": ms, "step_ms_all": times, "flop": flop, "tflops": flop / (ms * 1e-3) / 1e12,
           "loss": float(outs[0].to_numpy()), "launches": exe.launches_per_execute}
    if profile:
        client.set_profiling(True)
        exe.execute(bufs)
        client.set_profiling(False)
        rep = client.profile_report()
        res["by_kind"] = {k: {"ms": v["ms"], "count": v["count"]} for k, v in _by_kind(rep).items()}
        if verbose:
            for r in sorted(rep, key=lambda r: -r["ms"])[:40]:
                print(f"  {r['ms'] * 1e3:9.1f} us x{r['count']:<3d} {r['kind']:8s} {r['key'][:120]}")
    return res


def gemm(client, m, n, k, reps):
    b = Builder()
    x, w = b.arg((m, k), "bf16"), b.arg((k, n), "bf16")
    text = b.module([b.matmul(x, w)])
    rng = np.random.default_rng(0)
    exe = client.compile(text)
    bufs = [client.buffer_from_host(rng.standard_normal((m, k)).astype(np.float32), dtype="bf16"),
            client.buffer_from_host(rng.standard_normal((k, n)).astype(np.float32), dtype="bf16")]
    record = _events(client)
    for _ in range(3):
        exe.execute(bufs)
    client.synchronize()
    a = record()
    for _ in range(reps):
        exe.execute(bufs)
    e = record()
    client.synchronize()
    ms = a.elapsed_time(e) / reps
    print(f"gemm bf16 {m}x{n}x{k}: {ms * 1e3:.1f} us, {2.0 * m * n * k / ms / 1e9:.1f} TFLOP/s; plan: "
          + " | ".join(l.strip()[:90] for l in exe.plan_text().splitlines()[1:]))


def gemv(client, m, n, k, layout, reps, hbm_gbs=6546.2):
    """One skinny bf16 product x[m,k] . W with W stored [k,n] (`nc`) or [n,k] (`kc`), timed over `reps` launches that
    rotate through enough distinct weight buffers to exceed the 126 MB L2 (so every launch streams from HBM)."""
    b = Builder()
    x = b.arg((m, k), "bf16")
    w = b.arg((k, n) if layout == "nc" else (n, k), "bf16")
    text = b.module([b.dot_general(x, w, ((1,), (0,) if layout == "nc" else (1,)))])
    exe = client.compile(text)
    rng = np.random.default_rng(0)
    nbuf = max(2, int(300e6 // (2 * n * k)) + 1)
    wshape = (k, n) if layout == "nc" else (n, k)
    ws = [client.buffer_from_host(rng.integers(0, 1 << 14, wshape, dtype=np.uint16), dtype="bf16") for _ in range(min(nbuf, 64))]
    xb = client.buffer_from_host(rng.standard_normal((m, k)).astype(np.float32), dtype="bf16")
    record = _events(client)
    for i in range(3):
        exe.execute([xb, ws[i % len(ws)]])
    client.synchronize()
    a = record()
    for i in range(reps):
        exe.execute([xb, ws[i % len(ws)]])
    e = record()
    client.synchronize()
    us = a.elapsed_time(e) * 1e3 / reps
    gbs = 2.0 * n * k / us / 1e3
    print(f"gemv bf16 {layout} M={m} N={n} K={k}: {us:.1f} us per launch, {gbs:.0f} GB/s of weights = {gbs / hbm_gbs:.2f} of the "
          f"measured copy bandwidth ({len(ws)} rotating weight buffers); plan: " +
          " | ".join(l.strip()[:80] for l in exe.plan_text().splitlines()[1:]))


def simple(client, what, dtype, reps):
    """One-operation programs of the HBM-bound kernel classes; prints microseconds per execution and the algorithmic
    bytes (inputs read once + outputs written once) per second."""
    rng = np.random.default_rng(0)
    b = Builder()
    es = 4 if dtype == "f32" else 2
    f = lambda shape: rng.standard_normal(shape).astype(np.float32)
    if what == "pointwise":
        shape = (128, 32, 32, 64)
        x, r, sc, sh = b.arg(shape, dtype), b.arg(shape, dtype), b.arg((64,), dtype), b.arg((64,), dtype)
        y = b.add(b.mul(x, b.broadcast_in_dim(sc, shape, (3,))), b.broadcast_in_dim(sh, shape, (3,)))
        y = b.max(b.add(y, r), b.full(shape, 0.0, dtype))
        text, arrays = b.module([y]), [f(shape), f(shape), f((64,)), f((64,))]
        nbytes = 3 * int(np.prod(shape)) * es
    elif what == "transpose":
        shape = (8192, 6144)
        x = b.arg(shape, dtype)
        text, arrays = b.module([b.transpose(x, (1, 0))]), [f(shape)]
        nbytes = 2 * int(np.prod(shape)) * es
    elif what == "softmax":
        shape = (32 * 12 * 128, 128)
        x = b.arg(shape, dtype)
        xf = b.convert(x, "f32") if dtype != "f32" else x
        m = b.reduce_max(xf, (1,))
        e = b.exp(b.sub(xf, b.broadcast_in_dim(m, shape, (0,))))
        p = b.div(e, b.broadcast_in_dim(b.reduce_sum(e, (1,)), shape, (0,)))
        text, arrays = b.module([b.convert(p, dtype) if dtype != "f32" else p]), [f(shape)]
        nbytes = 2 * int(np.prod(shape)) * es
    elif what == "gather":
        table, idx = b.arg((30522, 768), dtype), b.arg((4096,), "i32")
        text = b.module([b.take_rows(table, idx)])
        arrays = [f((30522, 768)), rng.integers(0, 30522, (4096,)).astype(np.int32)]
        nbytes = 2 * 4096 * 768 * es
    elif what == "attention":
        # the decode step of the Gemma-2B-shaped model: 8 query heads on one key / value head, 640 cached positions
        from b200.shlo import programs
        G, M, T, D = None, 8, 640, 256
        text = programs.decode_attention(G, M, T, D, D, dt="bf16")
        arrays = [f((M, D)), f((T, D)), f((T, D)), np.array(T - 3, np.int32)]
        dtype, es = "bf16", 2
        nbytes = (2 * T * D + 2 * M * D) * es + M * D * 4
    elif what == "sort":
        shape = (4096, 1024)
        x = b.arg(shape, dtype)
        text, arrays = b.module(b.sort([x], 1)), [f(shape)]
        nbytes = 2 * int(np.prod(shape)) * es
    else:
        table, idx, upd = b.arg((30522, 768), dtype), b.arg((4096,), "i32"), b.arg((4096, 768), dtype)
        text = b.module([b.scatter_rows(table, idx, upd, "add")])
        arrays = [f((30522, 768)), rng.integers(0, 30522, (4096,)).astype(np.int32), f((4096, 768))]
        nbytes = (2 * 30522 * 768 + 2 * 4096 * 768) * es          # operand copied to the result, updates read and added
    exe = client.compile(text)
    dts = [dtype if a.dtype == np.float32 else "i32" for a in arrays]
    arrays = [np.asarray(a) for a in arrays]
    bufs = [client.buffer_from_host(a, dtype=d) for a, d in zip(arrays, dts)]
    record = _events(client)
    for _ in range(3):
        exe.execute(bufs)
    client.synchronize()
    a = record()
    for _ in range(reps):
        exe.execute(bufs)
    e = record()
    client.synchronize()
    us = a.elapsed_time(e) * 1e3 / reps
    print(f"{what} {dtype}: {us:.1f} us per execution, {nbytes / us / 1e3:.0f} GB/s of algorithmic bytes ({nbytes / 1e6:.1f} MB); plan: "
          + " | ".join(l.strip()[:100] for l in exe.plan_text().splitlines()[1:]))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["conv", "reduce", "scan", "gemma", "distilbert", "gemm", "gemv", "pointwise", "transpose",
                                     "softmax", "gather", "scatter", "attention", "sort"])
    ap.add_argument("--dtype", default="f32", choices=["f32", "bf16"])
    ap.add_argument("--layout", default="kc", choices=["kc", "nc"])
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--profile", action="store_true")
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
    if a.what in ("pointwise", "transpose", "softmax", "gather", "scatter", "attention", "sort"):
        simple(client, a.what, a.dtype, a.reps)
        return
    if a.what == "gemma":
        import json
        kw = {"layers": a.layers} if a.layers else {}
        res = gemma_decode(client, reps=min(a.reps, 5), profile=a.profile, verbose=True, **kw)
        res.pop("tokens")
        print(json.dumps(res))
        return
    if a.what == "distilbert":
        import json
        kw = {"layers": a.layers} if a.layers else {}
        print(json.dumps(distilbert_step(client, reps=a.reps, profile=a.profile, verbose=True, **kw)))
        return
    if a.what == "gemv":
        m, n, k = (int(v) for v in a.shape.split(","))
        gemv(client, m, n, k, a.layout, a.reps)
        return
    if a.what == "gemm":
        m, n, k = (int(v) for v in a.shape.split(","))
        gemm(client, m, n, k, a.reps)
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
