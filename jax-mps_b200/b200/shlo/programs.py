"""StableHLO programs of the benchmark configurations.

Each generator returns a `Program`: the module text, the flat argument list
(name, shape, dtype) and result list. Architectures follow the reference's
example models; data and weights are synthetic (see `init_*`).

  * ResNet18 (CIFAR variant): examples/resnet/model.py:6-163, training step
    examples/resnet/main.py:22-38 (softmax cross-entropy, value_and_grad),
    SGD with momentum 0.9, lr 0.1.
  * Data-parallel ResNet18: the same body as a fully-manual shard_map over
    `n` partitions, gradients and loss averaged with stablehlo.all_reduce.
"""
from __future__ import annotations

import dataclasses
import math

import numpy as np

from .builder import Builder, Val


@dataclasses.dataclass
class Program:
    name: str
    text: str
    args: list            # [(name, shape, dtype)]
    results: list         # [(name, shape, dtype)]
    num_partitions: int = 1
    meta: dict = dataclasses.field(default_factory=dict)


# --------------------------------------------------------------------------
# ResNet18
# --------------------------------------------------------------------------

def resnet18_param_spec(num_classes: int = 10, width: int = 64, in_ch: int = 3):
    """62 leaves for width 64: 20 conv kernels (HWIO), 20 BatchNorm
    (scale, bias) pairs, dense kernel and bias."""
    spec = []
    def conv(n, k, ci, co): spec.append((n + ".kernel", (k, k, ci, co)))
    def bn(n, c): spec.extend([(n + ".scale", (c,)), (n + ".bias", (c,))])
    conv("conv_init", 3, in_ch, width); bn("bn_init", width)
    cin = width
    for stage in range(4):
        cout = width * 2 ** stage
        for blk in range(2):
            stride = 2 if (stage > 0 and blk == 0) else 1
            p = f"stage{stage + 1}_block{blk + 1}"
            conv(p + ".conv1", 3, cin, cout); bn(p + ".bn1", cout)
            conv(p + ".conv2", 3, cout, cout); bn(p + ".bn2", cout)
            if cin != cout or stride != 1:
                conv(p + ".conv_proj", 1, cin, cout); bn(p + ".bn_proj", cout)
            cin = cout
    spec.append(("dense.kernel", (cin, num_classes)))
    spec.append(("dense.bias", (num_classes,)))
    return spec


def init_resnet18(seed: int = 0, **kw) -> dict:
    """He-normal conv and dense kernels, BatchNorm scale 1 / bias 0, dense
    bias 0 (float32)."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in resnet18_param_spec(**kw):
        if name.endswith(".kernel"):
            fan_in = int(np.prod(shape[:-1]))
            out[name] = (rng.standard_normal(shape) * math.sqrt(2.0 / fan_in)).astype(np.float32)
        elif name.endswith(".scale"):
            out[name] = np.ones(shape, np.float32)
        else:
            out[name] = np.zeros(shape, np.float32)
    return out


def _same_pad(size: int, k: int, s: int):
    out = -(-size // s)
    tot = max((out - 1) * s + k - size, 0)
    return (tot // 2, tot - tot // 2)


_CONV_TAPS = None      # debugging aid: when a list, every convolution output is appended to it


def _conv_same(b: Builder, x: Val, w: Val, stride: int) -> Val:
    pads = [_same_pad(x.shape[1], w.shape[0], stride), _same_pad(x.shape[2], w.shape[1], stride)]
    y = b.conv(x, w, strides=(stride, stride), padding=pads)
    if _CONV_TAPS is not None:
        _CONV_TAPS.append(y)
    return y


def _batch_norm(b: Builder, x: Val, scale: Val, bias: Val, eps: float = 1e-5) -> Val:
    """Training-mode BatchNorm over (N, H, W) as flax computes it: mean and
    mean of squares, var = max(0, E[x^2] - E[x]^2), y = (x - mean) *
    (rsqrt(var + eps) * scale) + bias."""
    c = x.shape[-1]
    mean = b.mean(x, (0, 1, 2))
    mean2 = b.mean(b.mul(x, x), (0, 1, 2))
    var = b.max(b.full((c,), 0.0, x.dtype), b.sub(mean2, b.mul(mean, mean)))
    y = b.sub(x, b.bcast(mean, x.shape))
    mul = b.mul(b.rsqrt(b.add(var, b.full((c,), eps, x.dtype))), scale)
    y = b.mul(y, b.bcast(mul, x.shape))
    return b.add(y, b.bcast(bias, x.shape))


def _relu(b: Builder, x: Val) -> Val:
    """jax.nn.relu: maximum(x, 0) with gradient select(x > 0, g, 0)."""
    y = b.emit("stablehlo.maximum", [x, b.zeros_like(x)], [(x.shape, x.dtype)])[0]
    b.record([y], [x], lambda g: [b.select(b.compare(x, b.zeros_like(x), "GT"), g[0], b.zeros_like(x))])
    return y


def resnet18_logits(b: Builder, p: dict, x: Val, taps: list | None = None) -> Val:
    y = _relu(b, _batch_norm(b, _conv_same(b, x, p["conv_init.kernel"], 1), p["bn_init.scale"], p["bn_init.bias"]))
    cin = y.shape[-1]
    for stage in range(4):
        for blk in range(2):
            n = f"stage{stage + 1}_block{blk + 1}"
            stride = 2 if (stage > 0 and blk == 0) else 1
            res = y
            z = _conv_same(b, y, p[n + ".conv1.kernel"], stride)
            z = _relu(b, _batch_norm(b, z, p[n + ".bn1.scale"], p[n + ".bn1.bias"]))
            z = _conv_same(b, z, p[n + ".conv2.kernel"], 1)
            z = _batch_norm(b, z, p[n + ".bn2.scale"], p[n + ".bn2.bias"])
            if (n + ".conv_proj.kernel") in p:
                res = _conv_same(b, res, p[n + ".conv_proj.kernel"], stride)
                res = _batch_norm(b, res, p[n + ".bn_proj.scale"], p[n + ".bn_proj.bias"])
            y = _relu(b, b.add(res, z))
            if taps is not None:
                taps.append((n, y))
    y = b.mean(y, (1, 2))
    y = b.matmul(y, p["dense.kernel"])
    return b.add(y, b.bcast(p["dense.bias"], y.shape))


def softmax_cross_entropy_int(b: Builder, logits: Val, labels: Val) -> Val:
    """mean over the batch of -sum(one_hot(labels) * log_softmax(logits)).
    One-hot through iota + compare; log_softmax subtracts a stop-gradient
    row maximum (jax.nn.log_softmax)."""
    n, k = logits.shape
    m = b.stop_gradient(b.reduce_max(logits, (1,)))
    sh = b.sub(logits, b.broadcast_in_dim(m, (n, k), (0,)))
    lse = b.log(b.reduce_sum(b.exp(sh), (1,)))
    logp = b.sub(sh, b.broadcast_in_dim(lse, (n, k), (0,)))
    oh = b.convert(b.compare(b.iota((n, k), "i32", 1), b.broadcast_in_dim(labels, (n, k), (0,)), "EQ"), logits.dtype)
    per = b.neg(b.reduce_sum(b.mul(oh, logp), (1,)))
    return b.mean(per, (0,))


def resnet18_train_step(batch: int = 128, image: int = 32, num_classes: int = 10, width: int = 64,
                        lr: float = 0.1, momentum: float = 0.9, n_partitions: int = 1) -> Program:
    """value_and_grad + SGD-momentum step. Arguments: params (62), momentum
    buffers (62), images f32[batch,image,image,3], labels i32[batch]. Results:
    loss, new params, new momentum. `batch` is the per-partition batch; with
    n_partitions > 1 the gradients and the loss are averaged over partitions
    by all_reduce (the psum/n of a shard_map body)."""
    spec = resnet18_param_spec(num_classes, width)
    b = Builder()
    params, moms = {}, {}
    for i, (n, s) in enumerate(spec):
        params[n] = b.arg(s, "f32", f"tf.aliasing_output = {1 + i} : i32")
    for i, (n, s) in enumerate(spec):
        moms[n] = b.arg(s, "f32", f"tf.aliasing_output = {1 + len(spec) + i} : i32")
    x = b.arg((batch, image, image, 3), "f32")
    y = b.arg((batch,), "i32")
    logits = resnet18_logits(b, params, x)
    loss = softmax_cross_entropy_int(b, logits, y)
    grads = b.grad(loss, [params[n] for n, _ in spec])
    b.root.taping = False
    if n_partitions > 1:
        red = b.all_reduce_sum(grads + [loss], n_partitions)
        inv = 1.0 / n_partitions
        grads = [b.mul(g, b.full(g.shape, inv, "f32")) for g in red[:-1]]
        loss = b.mul(red[-1], b.const(inv, "f32"))
    new_p, new_m = [], []
    for (n, s), g in zip(spec, grads):
        m = b.add(b.mul(moms[n], b.full(s, momentum, "f32")), g)
        new_m.append(m)
        new_p.append(b.sub(params[n], b.mul(m, b.full(s, lr, "f32"))))
    results = [loss] + new_p + new_m
    text = b.module(results, name="jit_train_step", num_partitions=n_partitions)
    args = ([("p." + n, s, "f32") for n, s in spec] + [("m." + n, s, "f32") for n, s in spec]
            + [("x", (batch, image, image, 3), "f32"), ("y", (batch,), "i32")])
    res = [("loss", (), "f32")] + [("p." + n, s, "f32") for n, s in spec] + [("m." + n, s, "f32") for n, s in spec]
    return Program("resnet18_train_step", text, args, res, n_partitions,
                   {"batch": batch, "image": image, "width": width, "params": sum(int(np.prod(s)) for _, s in spec)})


def resnet18_inputs(prog: Program, seed_w: int = 0, seed_x: int = 1, rank: int = 0) -> list:
    """Synthetic arguments in program order: He-normal weights (seed_w), zero
    momentum, images ~N(0,1) and labels uniform in [0, classes) (seed_x,
    offset by rank so shards differ)."""
    w = init_resnet18(seed_w, width=prog.meta["width"])
    rng = np.random.default_rng(seed_x + 1000 * rank)
    out = []
    for n, s, d in prog.args:
        if n.startswith("p."):
            out.append(w[n[2:]])
        elif n.startswith("m."):
            out.append(np.zeros(s, np.float32))
        elif n == "x":
            out.append(rng.standard_normal(s).astype(np.float32))
        else:
            out.append(rng.integers(0, 10, s).astype(np.int32))
    return out


# --------------------------------------------------------------------------
# Gemma-shaped greedy decoding
# --------------------------------------------------------------------------

def gemma_param_spec(vocab: int, dim: int, layers: int, heads: int, head_dim: int, hidden: int):
    """Leaves of the decoder (examples/gemma/model.py:118-296): tied embedding, per layer two RMSNorm weights,
    q / k / v / o projections with one shared key-value head, and the GeGLU feed-forward."""
    spec = [("embed", (vocab, dim))]
    for i in range(layers):
        p = f"layer{i}."
        spec += [(p + "attn_norm", (dim,)), (p + "wq", (dim, heads * head_dim)), (p + "wk", (dim, head_dim)),
                 (p + "wv", (dim, head_dim)), (p + "wo", (heads * head_dim, dim)), (p + "mlp_norm", (dim,)),
                 (p + "w_gate", (dim, hidden)), (p + "w_up", (dim, hidden)), (p + "w_down", (hidden, dim))]
    spec.append(("final_norm", (dim,)))
    return spec


def gemma_greedy_decode(vocab: int = 256000, dim: int = 2048, layers: int = 18, heads: int = 8, head_dim: int = 256,
                        hidden: int = 16384, prompt_len: int = 512, new_tokens: int = 128, cache_len: int = 640,
                        dtype: str = "bf16") -> Program:
    """Prompt consumption and greedy generation in one stablehlo.while (the loop of examples/gemma/main.py:109-134
    moved inside the program): every iteration embeds one token, runs the decoder with a static key-value cache
    updated in place by dynamic_update_slice, and takes the argmax of the tied-embedding logits. While the
    position is inside the prompt the next input is the prompt token, afterwards the argmax. Arguments: the
    weights (bf16), prompt i32[prompt_len]. Results: tokens i32[prompt_len + new_tokens] (prompt followed by the
    generated ids) and the last step's logits f32[vocab]. Norms, rotary embedding and softmax compute in f32."""
    spec = gemma_param_spec(vocab, dim, layers, heads, head_dim, hidden)
    total = prompt_len + new_tokens
    assert total <= cache_len
    b = Builder()
    W = {n: b.arg(s, dtype) for n, s in spec}
    prompt = b.arg((prompt_len,), "i32")
    half = head_dim // 2
    inv_freq = b.const_array((1.0 / (10000.0 ** (np.arange(half, dtype=np.float64) * 2 / head_dim))).astype(np.float32))
    pos_ids = b.iota((cache_len,), "i32", 0)

    def rms_norm(s, x, w):                           # x f32[dim]; weight stored as (1 + w)
        ms = s.mean(s.mul(x, x), (0,))
        inv = s.rsqrt(s.add(ms, s.const(1e-6, "f32")))
        scale = s.add(s.convert(w, "f32"), s.full((dim,), 1.0, "f32"))
        return s.mul(s.mul(x, s.bcast(inv, (dim,))), scale)

    def rope(s, x, cos, sin, n):                     # x f32[n, head_dim], rotate-half form
        x1, x2 = s.slice(x, (0, 0), (n, half)), s.slice(x, (0, half), (n, head_dim))
        c, sn = s.bcast(cos, (n, half), (1,)), s.bcast(sin, (n, half), (1,))
        return s.concatenate([s.sub(s.mul(x1, c), s.mul(x2, sn)), s.add(s.mul(x2, c), s.mul(x1, sn))], 1)

    def gelu(s, x):
        c = s.full(x.shape, math.sqrt(2.0 / math.pi), "f32")
        inner = s.mul(c, s.add(x, s.mul(s.full(x.shape, 0.044715, "f32"), s.mul(x, s.mul(x, x)))))
        return s.mul(s.mul(x, s.full(x.shape, 0.5, "f32")), s.add(s.full(x.shape, 1.0, "f32"), s.tanh(inner)))

    def lin(s, x, w):                                # f32[1, k] through a bf16 weight, bf16 product, f32 out
        return s.convert(s.matmul(s.convert(x, dtype), w), "f32")

    n_state = 3 + 2 * layers

    def cond(s, t, *rest):
        return s.compare(t, s.const(total, "i32"), "LT")

    def body(s, t, tok, toks, *caches):
        z = s.const(0, "i32")
        caches = list(caches)
        x = s.convert(s.take_rows(W["embed"], s.reshape(tok, (1,))), "f32")            # [1, dim]
        x = s.reshape(s.mul(x, s.full((1, dim), math.sqrt(dim), "f32")), (dim,))
        ang = s.mul(s.bcast(s.convert(t, "f32"), (half,)), inv_freq)
        cos, sin = s.cos(ang), s.sin(ang)
        for i in range(layers):
            p = f"layer{i}."
            h = s.reshape(rms_norm(s, x, W[p + "attn_norm"]), (1, dim))
            q = rope(s, s.reshape(lin(s, h, W[p + "wq"]), (heads, head_dim)), cos, sin, heads)
            k = rope(s, lin(s, h, W[p + "wk"]), cos, sin, 1)
            v = lin(s, h, W[p + "wv"])
            kc = s.dynamic_update_slice(caches[2 * i], s.convert(k, dtype), [t, z])       # [cache_len, head_dim]
            vc = s.dynamic_update_slice(caches[2 * i + 1], s.convert(v, dtype), [t, z])
            caches[2 * i], caches[2 * i + 1] = kc, vc
            sc = s.convert(s.dot_general(s.convert(q, dtype), kc, ((1,), (1,))), "f32")   # [heads, cache_len]
            sc = s.mul(sc, s.full(sc.shape, 1.0 / math.sqrt(head_dim), "f32"))
            visible = s.compare(s.bcast(pos_ids, sc.shape, (1,)), s.bcast(t, sc.shape), "LE")
            sc = s.select(visible, sc, s.full(sc.shape, -1e30, "f32"))
            m = s.reduce_max(sc, (1,))
            e = s.exp(s.sub(sc, s.bcast(m, sc.shape, (0,))))
            pr = s.div(e, s.bcast(s.reduce_sum(e, (1,)), sc.shape, (0,)))
            att = s.convert(s.matmul(s.convert(pr, dtype), vc), "f32")                    # [heads, head_dim]
            o = lin(s, s.reshape(att, (1, heads * head_dim)), W[p + "wo"])
            x = s.add(x, s.reshape(o, (dim,)))
            h2 = s.reshape(rms_norm(s, x, W[p + "mlp_norm"]), (1, dim))
            ff = s.mul(gelu(s, lin(s, h2, W[p + "w_gate"])), lin(s, h2, W[p + "w_up"]))
            x = s.add(x, s.reshape(lin(s, ff, W[p + "w_down"]), (dim,)))
        hf = s.convert(s.reshape(rms_norm(s, x, W["final_norm"]), (1, dim)), dtype)
        logits = s.reshape(s.convert(s.dot_general(hf, W["embed"], ((1,), (1,))), "f32"), (vocab,))
        best = s.reshape(s.argmax(logits, 0), (1,))
        t1 = s.add(t, s.const(1, "i32"))
        # next input: the prompt while inside it, the prediction afterwards
        idx = s.min(t1, s.const(prompt_len - 1, "i32"))
        from_prompt = s.dynamic_slice(prompt, [idx], (1,))
        nxt = s.select(s.reshape(s.compare(t1, s.const(prompt_len, "i32"), "LT"), (1,)), from_prompt, best)
        toks2 = s.dynamic_update_slice(toks, nxt, [s.min(t1, s.const(total - 1, "i32"))])
        return [t1, nxt, toks2, *caches, logits]

    tok0 = b.slice(prompt, (0,), (1,))
    toks0 = b.dynamic_update_slice(b.full((total,), 0, "i32"), tok0, [b.const(0, "i32")])
    caches0 = [b.full((cache_len, head_dim), 0.0, dtype) for _ in range(2 * layers)]
    logits0 = b.full((vocab,), 0.0, "f32")
    init = [b.const(0, "i32"), tok0, toks0, *caches0, logits0]
    outs = b.while_(init, lambda s, *a: cond(s, *a), lambda s, t, tok, toks, *r: body(s, t, tok, toks, *r[:-1]))
    text = b.module([outs[2], outs[-1]], name="jit_greedy_decode")
    args = [(n, s, dtype) for n, s in spec] + [("prompt", (prompt_len,), "i32")]
    res = [("tokens", (total,), "i32"), ("last_logits", (vocab,), "f32")]
    return Program("gemma_greedy_decode", text, args, res, 1,
                   {"vocab": vocab, "dim": dim, "layers": layers, "prompt_len": prompt_len, "new_tokens": new_tokens})


def _gemma_ops(dim: int, heads: int, head_dim: int, dtype: str):
    """Building blocks shared by the prefill and the decode-loop programs (examples/gemma/model.py:118-296 of the
    reference): RMSNorm with the weight stored as (1 + w), rotate-half rotary embedding, tanh GELU, and a linear
    layer that rounds its input to `dtype`, multiplies by a `dtype` weight and returns f32."""
    half = head_dim // 2

    def rms_norm(s, x, w):                           # x f32[rows, dim]
        rows = x.shape[0]
        ms = s.mean(s.mul(x, x), (1,))
        inv = s.rsqrt(s.add(ms, s.full((rows,), 1e-6, "f32")))
        scale = s.add(s.convert(w, "f32"), s.full((dim,), 1.0, "f32"))
        return s.mul(s.mul(x, s.bcast(inv, x.shape, (0,))), s.bcast(scale, x.shape, (1,)))

    def rope(s, x, cos, sin):                        # x f32[rows, n, head_dim]; cos, sin f32[rows, half]
        rows, n = x.shape[0], x.shape[1]
        x1, x2 = s.slice(x, (0, 0, 0), (rows, n, half)), s.slice(x, (0, 0, half), (rows, n, head_dim))
        c, sn = s.bcast(cos, (rows, n, half), (0, 2)), s.bcast(sin, (rows, n, half), (0, 2))
        return s.concatenate([s.sub(s.mul(x1, c), s.mul(x2, sn)), s.add(s.mul(x2, c), s.mul(x1, sn))], 2)

    def gelu(s, x):
        c = s.full(x.shape, math.sqrt(2.0 / math.pi), "f32")
        inner = s.mul(c, s.add(x, s.mul(s.full(x.shape, 0.044715, "f32"), s.mul(x, s.mul(x, x)))))
        return s.mul(s.mul(x, s.full(x.shape, 0.5, "f32")), s.add(s.full(x.shape, 1.0, "f32"), s.tanh(inner)))

    def lin(s, x, w):                                # f32[rows, k] through a `dtype` weight, `dtype` product, f32 out
        return s.convert(s.matmul(s.convert(x, dtype), w), "f32")

    return rms_norm, rope, gelu, lin


def gemma_prefill(vocab: int = 256000, dim: int = 2048, layers: int = 18, heads: int = 8, head_dim: int = 256,
                  hidden: int = 16384, prompt_len: int = 512, cache_len: int = 640, dtype: str = "bf16") -> Program:
    """The whole prompt in one pass (the `prefill` jit of examples/gemma/main.py:109-123 of the reference): every
    projection is a product with `prompt_len` rows, attention is causal over the prompt with the one key-value head
    shared by all query heads, and the keys (after the rotary embedding) and values are written into static caches
    of `cache_len` positions. Arguments: the weights, prompt i32[prompt_len]. Results: the first generated token
    i32[1], the logits f32[vocab] of the last prompt position, then for every layer the key and the value cache
    `dtype`[cache_len, head_dim]."""
    spec = gemma_param_spec(vocab, dim, layers, heads, head_dim, hidden)
    T, H, half = prompt_len, heads, head_dim // 2
    assert T <= cache_len
    b = Builder()
    W = {n: b.arg(s, dtype) for n, s in spec}
    prompt = b.arg((T,), "i32")
    rms_norm, rope, gelu, lin = _gemma_ops(dim, heads, head_dim, dtype)
    inv_freq = b.const_array((1.0 / (10000.0 ** (np.arange(half, dtype=np.float64) * 2 / head_dim))).astype(np.float32))
    pos = b.convert(b.iota((T,), "i32", 0), "f32")
    ang = b.mul(b.bcast(pos, (T, half), (0,)), b.bcast(inv_freq, (T, half), (1,)))
    cos, sin = b.cos(ang), b.sin(ang)
    x = b.convert(b.take_rows(W["embed"], prompt), "f32")                             # [T, dim]
    x = b.mul(x, b.full((T, dim), math.sqrt(dim), "f32"))
    qi, kj = b.iota((H, T, T), "i32", 1), b.iota((H, T, T), "i32", 2)
    visible = b.compare(kj, qi, "LE")
    zero = b.const(0.0, dtype)
    caches = []
    for i in range(layers):
        p = f"layer{i}."
        h = rms_norm(b, x, W[p + "attn_norm"])
        q = rope(b, b.reshape(lin(b, h, W[p + "wq"]), (T, H, head_dim)), cos, sin)       # [T, H, hd]
        k = b.reshape(rope(b, b.reshape(lin(b, h, W[p + "wk"]), (T, 1, head_dim)), cos, sin), (T, head_dim))
        v = lin(b, h, W[p + "wv"])
        kb, vb = b.convert(k, dtype), b.convert(v, dtype)
        caches += [b.pad(kb, zero, (0, 0), (cache_len - T, 0)), b.pad(vb, zero, (0, 0), (cache_len - T, 0))]
        qb = b.convert(b.reshape(b.transpose(q, (1, 0, 2)), (H * T, head_dim)), dtype)
        sc = b.convert(b.dot_general(qb, kb, ((1,), (1,))), "f32")                    # [H * T, T]
        sc = b.reshape(b.mul(sc, b.full(sc.shape, 1.0 / math.sqrt(head_dim), "f32")), (H, T, T))
        sc = b.select(visible, sc, b.full(sc.shape, -1e30, "f32"))
        m = b.reduce_max(sc, (2,))
        e = b.exp(b.sub(sc, b.bcast(m, sc.shape, (0, 1))))
        pr = b.div(e, b.bcast(b.reduce_sum(e, (2,)), sc.shape, (0, 1)))
        att = b.convert(b.matmul(b.convert(b.reshape(pr, (H * T, T)), dtype), vb), "f32")   # [H * T, hd]
        att = b.reshape(b.transpose(b.reshape(att, (H, T, head_dim)), (1, 0, 2)), (T, H * head_dim))
        x = b.add(x, lin(b, att, W[p + "wo"]))
        h2 = rms_norm(b, x, W[p + "mlp_norm"])
        ff = b.mul(gelu(b, lin(b, h2, W[p + "w_gate"])), lin(b, h2, W[p + "w_up"]))
        x = b.add(x, lin(b, ff, W[p + "w_down"]))
    last = b.slice(x, (T - 1, 0), (T, dim))
    hf = b.convert(rms_norm(b, last, W["final_norm"]), dtype)
    logits = b.reshape(b.convert(b.dot_general(hf, W["embed"], ((1,), (1,))), "f32"), (vocab,))
    best = b.reshape(b.argmax(logits, 0), (1,))
    text = b.module([best, logits, *caches], name="jit_prefill")
    args = [(n, s, dtype) for n, s in spec] + [("prompt", (T,), "i32")]
    res = [("token", (1,), "i32"), ("logits", (vocab,), "f32")]
    for i in range(layers):
        res += [(f"layer{i}.k_cache", (cache_len, head_dim), dtype), (f"layer{i}.v_cache", (cache_len, head_dim), dtype)]
    return Program("gemma_prefill", text, args, res, 1,
                   {"vocab": vocab, "dim": dim, "layers": layers, "prompt_len": T, "cache_len": cache_len})


def gemma_decode_loop(vocab: int = 256000, dim: int = 2048, layers: int = 18, heads: int = 8, head_dim: int = 256,
                      hidden: int = 16384, start: int = 512, new_tokens: int = 128, cache_len: int = 640,
                      dtype: str = "bf16") -> Program:
    """`new_tokens` greedy decode steps in one stablehlo.while (the decode loop of examples/gemma/main.py:125-134 of
    the reference moved inside the program): every iteration embeds the current token, runs the decoder at position
    `start + i` against the static key-value caches (updated in place by dynamic_update_slice) and takes the argmax
    of the tied-embedding logits as the next token. Arguments: the weights, the current token i32[1], the caches as
    `gemma_prefill` returns them. Results: the generated ids i32[new_tokens], the logits f32[vocab] of the last
    step, the caches."""
    spec = gemma_param_spec(vocab, dim, layers, heads, head_dim, hidden)
    assert start + new_tokens <= cache_len
    half = head_dim // 2
    b = Builder()
    W = {n: b.arg(s, dtype) for n, s in spec}
    tok_in = b.arg((1,), "i32")
    caches_in = [b.arg((cache_len, head_dim), dtype) for _ in range(2 * layers)]
    rms_norm, rope, gelu, lin = _gemma_ops(dim, heads, head_dim, dtype)
    inv_freq = b.const_array((1.0 / (10000.0 ** (np.arange(half, dtype=np.float64) * 2 / head_dim))).astype(np.float32))
    pos_ids = b.iota((cache_len,), "i32", 0)
    end = start + new_tokens

    def cond(s, t, *rest):
        return s.compare(t, s.const(end, "i32"), "LT")

    def body(s, t, tok, toks, *caches):
        z = s.const(0, "i32")
        caches = list(caches)
        x = s.convert(s.take_rows(W["embed"], tok), "f32")                              # [1, dim]
        x = s.mul(x, s.full((1, dim), math.sqrt(dim), "f32"))
        ang = s.reshape(s.mul(s.bcast(s.convert(t, "f32"), (half,)), inv_freq), (1, half))
        cos, sin = s.cos(ang), s.sin(ang)
        for i in range(layers):
            p = f"layer{i}."
            h = rms_norm(s, x, W[p + "attn_norm"])
            q = s.reshape(rope(s, s.reshape(lin(s, h, W[p + "wq"]), (1, heads, head_dim)), cos, sin), (heads, head_dim))
            k = s.reshape(rope(s, s.reshape(lin(s, h, W[p + "wk"]), (1, 1, head_dim)), cos, sin), (1, head_dim))
            v = lin(s, h, W[p + "wv"])
            kc = s.dynamic_update_slice(caches[2 * i], s.convert(k, dtype), [t, z])
            vc = s.dynamic_update_slice(caches[2 * i + 1], s.convert(v, dtype), [t, z])
            caches[2 * i], caches[2 * i + 1] = kc, vc
            sc = s.convert(s.dot_general(s.convert(q, dtype), kc, ((1,), (1,))), "f32")   # [heads, cache_len]
            sc = s.mul(sc, s.full(sc.shape, 1.0 / math.sqrt(head_dim), "f32"))
            visible = s.compare(s.bcast(pos_ids, sc.shape, (1,)), s.bcast(t, sc.shape), "LE")
            sc = s.select(visible, sc, s.full(sc.shape, -1e30, "f32"))
            m = s.reduce_max(sc, (1,))
            e = s.exp(s.sub(sc, s.bcast(m, sc.shape, (0,))))
            pr = s.div(e, s.bcast(s.reduce_sum(e, (1,)), sc.shape, (0,)))
            att = s.convert(s.matmul(s.convert(pr, dtype), vc), "f32")                    # [heads, head_dim]
            x = s.add(x, lin(s, s.reshape(att, (1, heads * head_dim)), W[p + "wo"]))
            h2 = rms_norm(s, x, W[p + "mlp_norm"])
            ff = s.mul(gelu(s, lin(s, h2, W[p + "w_gate"])), lin(s, h2, W[p + "w_up"]))
            x = s.add(x, lin(s, ff, W[p + "w_down"]))
        hf = s.convert(rms_norm(s, x, W["final_norm"]), dtype)
        logits = s.reshape(s.convert(s.dot_general(hf, W["embed"], ((1,), (1,))), "f32"), (vocab,))
        best = s.reshape(s.argmax(logits, 0), (1,))
        toks2 = s.dynamic_update_slice(toks, best, [s.sub(t, s.const(start, "i32"))])
        return [s.add(t, s.const(1, "i32")), best, toks2, *caches, logits]

    init = [b.const(start, "i32"), tok_in, b.full((new_tokens,), 0, "i32"), *caches_in, b.full((vocab,), 0.0, "f32")]
    outs = b.while_(init, lambda s, *a: cond(s, *a), lambda s, t, tok, toks, *r: body(s, t, tok, toks, *r[:-1]))
    text = b.module([outs[2], outs[-1], *outs[3:-1]], name="jit_decode_loop")
    args = [(n, s, dtype) for n, s in spec] + [("token", (1,), "i32")]
    res = [("tokens", (new_tokens,), "i32"), ("last_logits", (vocab,), "f32")]
    for i in range(layers):
        kv = [(f"layer{i}.k_cache", (cache_len, head_dim), dtype), (f"layer{i}.v_cache", (cache_len, head_dim), dtype)]
        args += kv
        res += kv
    return Program("gemma_decode_loop", text, args, res, 1,
                   {"vocab": vocab, "dim": dim, "layers": layers, "start": start, "new_tokens": new_tokens,
                    "cache_len": cache_len, "weight_bytes": sum(int(np.prod(s)) for n, s in spec) * 2})


def gemma_weights(spec, seed: int = 0, weight_std: float = 0.02, tile: int = 1 << 24, as_bits: bool = False) -> list:
    """Weights ~N(0, weight_std) rounded to bfloat16 (norm weights 0, i.e. scale 1), as float32 arrays or, with
    `as_bits`, as uint16 bit patterns. Tensors larger than `tile` elements are filled by repeating one block of `tile`
    normal samples from a per-tensor random offset: drawing 2.5 billion samples one by one takes minutes, and neither
    timing nor parity depends on independence across far-apart entries."""
    from .builder import f32_to_bf16_bits
    rng = np.random.default_rng(seed)
    def bits(a): return f32_to_bf16_bits(a.astype(np.float32)).reshape(a.shape)
    def back(b): return (b.astype(np.uint32) << 16).view(np.float32)
    block = bits(rng.standard_normal(tile) * weight_std)
    out = []
    for n, s in spec:
        size = int(np.prod(s))
        if n.endswith("norm"):
            w = np.zeros(s, np.uint16)
        elif size <= tile:
            w = bits(rng.standard_normal(s) * weight_std)
        else:
            off = int(rng.integers(0, tile))
            reps = (size + off + tile - 1) // tile
            w = np.tile(block, reps)[off:off + size].reshape(s)
        out.append(w if as_bits else back(w))
    return out


def gemma_inputs(prog: Program, seed: int = 0, weight_std: float = 0.02) -> list:
    """Synthetic arguments: weights ~N(0, weight_std) (norm weights 0, i.e. scale 1), prompt uniform over the
    vocabulary. Returned as float32 / int32 arrays; float arguments are converted to the program's dtype on upload."""
    rng = np.random.default_rng(seed)
    out = []
    for n, s, d in prog.args:
        if n == "prompt":
            out.append(rng.integers(0, prog.meta["vocab"], s).astype(np.int32))
        elif n.endswith("norm"):
            out.append(np.zeros(s, np.float32))
        else:
            out.append((rng.standard_normal(s) * weight_std).astype(np.float32))
    return out


# --------------------------------------------------------------------------
# LSTM by scan: one training step
# --------------------------------------------------------------------------

def lstm_param_spec(in_dim: int = 32, hidden: int = 256):
    """Two stacked LSTM layers in the concatenated form: gates = [x, h] @ W + b with gate order i, f, g, o."""
    return [("w1", (in_dim + hidden, 4 * hidden)), ("b1", (4 * hidden,)),
            ("w2", (2 * hidden, 4 * hidden)), ("b2", (4 * hidden,))]


def lstm_scan_train_step(steps: int = 100, batch: int = 64, in_dim: int = 32, hidden: int = 256, lr: float = 1e-3,
                         beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8) -> Program:
    """Forward `lax.scan` over `steps` time steps (a stablehlo.while reading xs[t] by dynamic_slice and stacking
    the carries by dynamic_update_slice), mean-squared error of the last hidden state against `targets`, the
    reverse scan of its gradient (a second while that recomputes each step from the stacked carries and
    accumulates the weight gradients), and one Adam update (the first step: bias corrections 1 - beta).
    The loop structure follows benchmarks/bench_rnn_training.py:63-90 of the reference with LSTM cells.
    Arguments: 4 parameters, 4 first moments, 4 second moments, xs f32[steps,batch,in_dim], targets
    f32[batch,hidden]. Results: loss, new parameters, new first moments, new second moments."""
    spec = lstm_param_spec(in_dim, hidden)
    H, T, B = hidden, steps, batch
    b = Builder()
    P = [b.arg(s, "f32") for _, s in spec]
    M = [b.arg(s, "f32") for _, s in spec]
    V = [b.arg(s, "f32") for _, s in spec]
    xs = b.arg((T, B, in_dim), "f32")
    targets = b.arg((B, H), "f32")

    def cell(s, x, h, c, w, bias):
        z = s.add(s.matmul(s.concatenate([x, h], 1), w), s.bcast(bias, (B, 4 * H)))
        i = s.logistic(s.slice(z, (0, 0), (B, H)))
        f = s.logistic(s.slice(z, (0, H), (B, 2 * H)))
        g = s.tanh(s.slice(z, (0, 2 * H), (B, 3 * H)))
        o = s.logistic(s.slice(z, (0, 3 * H), (B, 4 * H)))
        c2 = s.add(s.mul(f, c), s.mul(i, g))
        return s.mul(o, s.tanh(c2)), c2

    def step(s, x, h1, c1, h2, c2, params):
        w1, b1, w2, b2 = params
        h1n, c1n = cell(s, x, h1, c1, w1, b1)
        h2n, c2n = cell(s, h1n, h2, c2, w2, b2)
        return h1n, c1n, h2n, c2n

    def x_at(s, t):
        z = s.const(0, "i32")
        return s.reshape(s.dynamic_slice(xs, [t, z, z], (1, B, in_dim)), (B, in_dim))

    # forward scan: carries entering step t are stacked for the reverse pass
    def fcond(s, t, *r): return s.compare(t, s.const(T, "i32"), "LT")
    def fbody(s, t, h1, c1, h2, c2, *stacks):
        z = s.const(0, "i32")
        new_stacks = [s.dynamic_update_slice(st, s.reshape(v, (1, B, H)), [t, z, z]) for st, v in zip(stacks, (h1, c1, h2, c2))]
        out = step(s, x_at(s, t), h1, c1, h2, c2, P)
        return [s.add(t, s.const(1, "i32")), *out, *new_stacks]
    zeros = b.full((B, H), 0.0, "f32")
    stack0 = b.full((T, B, H), 0.0, "f32")
    fw = b.while_([b.const(0, "i32"), zeros, zeros, zeros, zeros, stack0, stack0, stack0, stack0], fcond, fbody)
    h2_last, stacks = fw[3], fw[5:9]
    diff = b.sub(h2_last, targets)
    loss = b.mean(b.mul(diff, diff), (0, 1))
    d_h2 = b.mul(diff, b.full((B, H), 2.0 / (B * H), "f32"))

    # reverse scan
    def bcond(s, k, *r): return s.compare(k, s.const(T, "i32"), "LT")
    def bbody(s, k, dh1, dc1, dh2, dc2, *gacc):
        z = s.const(0, "i32")
        t = s.sub(s.const(T - 1, "i32"), k)
        carry = [s.reshape(s.dynamic_slice(st, [t, z, z], (1, B, H)), (B, H)) for st in stacks]
        x = x_at(s, t)
        s.root.taping = True
        try:
            outs = step(s, x, *carry, P)
            total = None
            for o, d in zip(outs, (dh1, dc1, dh2, dc2)):
                term = s.reduce_sum(s.mul(o, d), (0, 1))
                total = term if total is None else s.add(total, term)
            grads = s.grad(total, [*carry, *P])
        finally:
            s.root.taping = False
        return [s.add(k, s.const(1, "i32")), *grads[:4], *[s.add(a, g) for a, g in zip(gacc, grads[4:])]]
    bw = b.while_([b.const(0, "i32"), zeros, zeros, d_h2, zeros, *[b.full(s_, 0.0, "f32") for _, s_ in spec]], bcond, bbody)
    grads = bw[5:9]
    b.root.taping = False
    new_p, new_m, new_v = [], [], []
    for (n, s_), p, m, v, g in zip(spec, P, M, V, grads):
        m2 = b.add(b.mul(m, b.full(s_, beta1, "f32")), b.mul(g, b.full(s_, 1.0 - beta1, "f32")))
        v2 = b.add(b.mul(v, b.full(s_, beta2, "f32")), b.mul(b.mul(g, g), b.full(s_, 1.0 - beta2, "f32")))
        mhat = b.div(m2, b.full(s_, 1.0 - beta1, "f32"))
        vhat = b.div(v2, b.full(s_, 1.0 - beta2, "f32"))
        new_p.append(b.sub(p, b.div(b.mul(mhat, b.full(s_, lr, "f32")), b.add(b.sqrt(vhat), b.full(s_, eps, "f32")))))
        new_m.append(m2)
        new_v.append(v2)
    text = b.module([loss, *new_p, *new_m, *new_v], name="jit_lstm_train_step")
    args = ([("p." + n, s_, "f32") for n, s_ in spec] + [("m." + n, s_, "f32") for n, s_ in spec] +
            [("v." + n, s_, "f32") for n, s_ in spec] + [("xs", (T, B, in_dim), "f32"), ("targets", (B, H), "f32")])
    res = ([("loss", (), "f32")] + [("p." + n, s_, "f32") for n, s_ in spec] + [("m." + n, s_, "f32") for n, s_ in spec] +
           [("v." + n, s_, "f32") for n, s_ in spec])
    return Program("lstm_scan_train_step", text, args, res, 1, {"steps": T, "batch": B, "in_dim": in_dim, "hidden": H})


def lstm_inputs(prog: Program, seed: int = 0) -> list:
    """Glorot-uniform weights, zero biases and moments, xs and targets ~N(0,1)."""
    rng = np.random.default_rng(seed)
    out = []
    for n, s, _ in prog.args:
        if n.startswith("p.w"):
            lim = math.sqrt(6.0 / (s[0] + s[1]))
            out.append(rng.uniform(-lim, lim, s).astype(np.float32))
        elif n in ("xs", "targets"):
            out.append(rng.standard_normal(s).astype(np.float32))
        else:
            out.append(np.zeros(s, np.float32))
    return out


def decode_attention(G, M, T, D, N, dt="bf16", masked=True, out_f32=True, scale=True, keepdims=False) -> str:
    """Attention of M query rows per group over T cached positions, the chain a decode step contains
    (examples/gemma/model.py:186-230 of the reference): q [G, M, D] (or [M, D] when G is None), k [.., T, D],
    v [.., T, N] and `upto` i32 (positions <= upto are visible); scores scaled by 1 / sqrt(D), softmax in f32,
    probabilities rounded to `dt` for the second product; `keepdims` writes the softmax's row statistics as [..., 1]
    tensors broadcast over all dimensions. Returns the module text."""
    b = Builder()
    lead = () if G is None else (G,)
    q, k, v = b.arg(lead + (M, D), dt), b.arg(lead + (T, D), dt), b.arg(lead + (T, N), dt)
    upto = b.arg((), "i32")
    r = len(lead)
    batch = ((0,), (0,)) if lead else ((), ())
    sc = b.convert(b.dot_general(q, k, ((r + 1,), (r + 1,)), batch), "f32")
    if scale:
        sc = b.mul(sc, b.full(sc.shape, 1.0 / math.sqrt(D), "f32"))
    if masked:
        pos = b.iota(sc.shape, "i32", r + 1)
        sc = b.select(b.compare(pos, b.bcast(upto, sc.shape), "LE"), sc, b.full(sc.shape, -1e30, "f32"))
    kept = tuple(range(r + 1))

    def along_rows(stat):                      # a per-row statistic against the rows; keepdims is how jax.nn.softmax spells it
        if keepdims:
            return b.broadcast_in_dim(b.reshape(stat, stat.shape + (1,)), sc.shape, tuple(range(r + 2)))
        return b.bcast(stat, sc.shape, kept)
    m = b.reduce_max(sc, (r + 1,))
    e = b.exp(b.sub(sc, along_rows(m)))
    pr = b.div(e, along_rows(b.reduce_sum(e, (r + 1,))))
    att = b.dot_general(b.convert(pr, dt), v, ((r + 1,), (r,)), batch)
    if out_f32:
        att = b.convert(att, "f32")
    return b.module([att])



# --------------------------------------------------------------------------
# DistilBERT-shaped masked-language-model step (forward + backward)
# --------------------------------------------------------------------------

def distilbert_param_spec(vocab: int, max_pos: int, dim: int, layers: int, ffn: int):
    """Leaves per examples/distilbert/model.py:11-94: word and position embeddings with their LayerNorm, per layer
    q/k/v/out projections, two LayerNorms and the two feed-forward matrices, then the MLM head (transform,
    LayerNorm, output bias; the projector is tied to the word embedding)."""
    spec = [("word_emb", (vocab, dim)), ("pos_emb", (max_pos, dim)), ("emb_ln.scale", (dim,)), ("emb_ln.bias", (dim,))]
    for i in range(layers):
        p = f"layer{i}."
        for n in ("q", "k", "v", "o"):
            spec += [(p + n + ".w", (dim, dim)), (p + n + ".b", (dim,))]
        spec += [(p + "attn_ln.scale", (dim,)), (p + "attn_ln.bias", (dim,)), (p + "ff1.w", (dim, ffn)), (p + "ff1.b", (ffn,)),
                 (p + "ff2.w", (ffn, dim)), (p + "ff2.b", (dim,)), (p + "out_ln.scale", (dim,)), (p + "out_ln.bias", (dim,))]
    spec += [("head.w", (dim, dim)), ("head.b", (dim,)), ("head_ln.scale", (dim,)), ("head_ln.bias", (dim,)), ("vocab_bias", (vocab,))]
    return spec


def distilbert_mlm_step(batch: int = 32, seq: int = 128, vocab: int = 30522, dim: int = 768, layers: int = 6, heads: int = 12,
                        ffn: int = 3072, dtype: str = "bf16") -> Program:
    """Loss and the gradient of every leaf for one masked-language-model batch. Weights and activations are
    `dtype`; LayerNorm, softmax and the log-softmax of the logits compute in f32. Arguments: the leaves, ids
    i32[batch,seq], weights f32[batch,seq] (1 at masked positions). Labels are the ids themselves. Results: loss f32
    and one gradient per leaf (in the leaf's dtype). The embedding gradient is a row scatter-add."""
    spec = distilbert_param_spec(vocab, seq, dim, layers, ffn)
    b = Builder()
    W = {n: b.arg(s, dtype) for n, s in spec}
    ids = b.arg((batch, seq), "i32")
    mask_w = b.arg((batch, seq), "f32")
    N, hd = batch * seq, dim // heads

    def layer_norm(x, scale, bias):                       # x dtype[N, dim] -> dtype[N, dim], f32 statistics
        xf = b.convert(x, "f32")
        mu = b.mean(xf, (1,))
        xc = b.sub(xf, b.bcast(mu, xf.shape, (0,)))
        var = b.mean(b.mul(xc, xc), (1,))
        inv = b.rsqrt(b.add(var, b.full(var.shape, 1e-12, "f32")))
        y = b.mul(xc, b.bcast(inv, xf.shape, (0,)))
        y = b.add(b.mul(y, b.bcast(b.convert(scale, "f32"), xf.shape, (1,))), b.bcast(b.convert(bias, "f32"), xf.shape, (1,)))
        return b.convert(y, dtype)

    def linear(x, w, bias):
        y = b.matmul(x, w)
        return b.add(y, b.bcast(bias, y.shape, (1,)))

    def gelu(x):
        xf = b.convert(x, "f32")
        c = b.full(xf.shape, math.sqrt(2.0 / math.pi), "f32")
        inner = b.mul(c, b.add(xf, b.mul(b.full(xf.shape, 0.044715, "f32"), b.mul(xf, b.mul(xf, xf)))))
        y = b.mul(b.mul(xf, b.full(xf.shape, 0.5, "f32")), b.add(b.full(xf.shape, 1.0, "f32"), b.tanh(inner)))
        return b.convert(y, dtype)

    x = b.take_rows(W["word_emb"], b.reshape(ids, (N,)))                                   # [N, dim]
    pos = b.reshape(b.bcast(W["pos_emb"], (batch, seq, dim), (1, 2)), (N, dim))
    x = layer_norm(b.add(x, pos), W["emb_ln.scale"], W["emb_ln.bias"])
    for i in range(layers):
        p = f"layer{i}."
        def split(t):                                     # [N, dim] -> [batch, heads, seq, hd]
            return b.transpose(b.reshape(t, (batch, seq, heads, hd)), (0, 2, 1, 3))
        q, k, v = (split(linear(x, W[p + n + ".w"], W[p + n + ".b"])) for n in ("q", "k", "v"))
        sc = b.convert(b.dot_general(q, k, ((3,), (3,)), ((0, 1), (0, 1))), "f32")          # [batch, heads, seq, seq]
        sc = b.mul(sc, b.full(sc.shape, 1.0 / math.sqrt(hd), "f32"))
        m = b.stop_gradient(b.reduce_max(sc, (3,)))
        e = b.exp(b.sub(sc, b.bcast(m, sc.shape, (0, 1, 2))))
        pr = b.convert(b.div(e, b.bcast(b.reduce_sum(e, (3,)), sc.shape, (0, 1, 2))), dtype)
        ctx = b.dot_general(pr, v, ((3,), (2,)), ((0, 1), (0, 1)))                            # [batch, heads, seq, hd]
        ctx = b.reshape(b.transpose(ctx, (0, 2, 1, 3)), (N, dim))
        x = layer_norm(b.add(x, linear(ctx, W[p + "o.w"], W[p + "o.b"])), W[p + "attn_ln.scale"], W[p + "attn_ln.bias"])
        ff = linear(gelu(linear(x, W[p + "ff1.w"], W[p + "ff1.b"])), W[p + "ff2.w"], W[p + "ff2.b"])
        x = layer_norm(b.add(x, ff), W[p + "out_ln.scale"], W[p + "out_ln.bias"])
    h = layer_norm(gelu(linear(x, W["head.w"], W["head.b"])), W["head_ln.scale"], W["head_ln.bias"])
    logits = b.convert(b.dot_general(h, W["word_emb"], ((1,), (1,))), "f32")                 # [N, vocab], tied projector
    logits = b.add(logits, b.bcast(b.convert(W["vocab_bias"], "f32"), logits.shape, (1,)))
    mx = b.stop_gradient(b.reduce_max(logits, (1,)))
    sh = b.sub(logits, b.bcast(mx, logits.shape, (0,)))
    lse = b.log(b.reduce_sum(b.exp(sh), (1,)))
    picked = b.take_along_last(sh, b.reshape(ids, (N,)))
    nll = b.sub(lse, picked)                                                                 # [N]
    wv = b.reshape(mask_w, (N,))
    denom = b.max(b.reduce_sum(wv, (0,)), b.const(1.0, "f32"))
    loss = b.div(b.reduce_sum(b.mul(nll, wv), (0,)), denom)
    grads = b.grad(loss, [W[n] for n, _ in spec])
    text = b.module([loss, *grads], name="jit_mlm_step")
    args = [(n, s, dtype) for n, s in spec] + [("ids", (batch, seq), "i32"), ("mask", (batch, seq), "f32")]
    res = [("loss", (), "f32")] + [("g." + n, s, dtype) for n, s in spec]
    return Program("distilbert_mlm_step", text, args, res, 1, {"vocab": vocab, "batch": batch, "seq": seq, "dim": dim})


def distilbert_inputs(prog: Program, seed: int = 0, weight_std: float = 0.02, mask_rate: float = 0.15) -> list:
    """Weights ~N(0, weight_std), LayerNorm scale 1 / bias 0, ids uniform over the vocabulary, mask Bernoulli."""
    rng = np.random.default_rng(seed)
    out = []
    for n, s, d in prog.args:
        if n == "ids":
            out.append(rng.integers(0, prog.meta["vocab"], s).astype(np.int32))
        elif n == "mask":
            out.append((rng.random(s) < mask_rate).astype(np.float32))
        elif n.endswith("ln.scale"):
            out.append(np.ones(s, np.float32))
        elif n.endswith(".bias") or n.endswith(".b") or n == "vocab_bias":
            out.append(np.zeros(s, np.float32))
        else:
            out.append((rng.standard_normal(s) * weight_std).astype(np.float32))
    return out


# ---------------------------------------------------------------------------
# Threefry-2x32 as elementwise integer operations (what jax.random lowers to where no fused kernel exists; the
# reference pins its fused Metal kernel bit for bit against the CPU backend: tests/configs/random.py:54-74)
# ---------------------------------------------------------------------------
def _threefry2x32(b: Builder, k0: Val, k1: Val, x0: Val, x1: Val):
    """Twenty rounds of Threefry-2x32 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3") on ui32 tensors of one
    shape; k0 and k1 are already broadcast to it."""
    shape = x0.shape
    u = lambda v: b.full(shape, int(v), "ui32")
    rotl = lambda v, r: b.or_(b.shl(v, u(r)), b.shr_logical(v, u(32 - r)))
    ks = [k0, k1, b.xor(b.xor(k0, k1), u(0x1BD11BDA))]
    rot = [(13, 15, 26, 6), (17, 29, 16, 24)]
    x0, x1 = b.add(x0, ks[0]), b.add(x1, ks[1])
    for i in range(5):
        for r in rot[i % 2]:
            x0 = b.add(x0, x1)
            x1 = b.xor(rotl(x1, r), x0)
        x0 = b.add(x0, ks[(i + 1) % 3])
        x1 = b.add(b.add(x1, ks[(i + 2) % 3]), u(i + 1))
    return x0, x1


def threefry_block(n: int) -> Program:
    """key ui32[2], x0 ui32[n], x1 ui32[n] -> the two output words per lane."""
    b = Builder()
    key, x0, x1 = b.arg((2,), "ui32"), b.arg((n,), "ui32"), b.arg((n,), "ui32")
    k0 = b.broadcast_in_dim(b.reshape(b.slice(key, (0,), (1,)), ()), (n,), ())
    k1 = b.broadcast_in_dim(b.reshape(b.slice(key, (1,), (2,)), ()), (n,), ())
    y0, y1 = _threefry2x32(b, k0, k1, x0, x1)
    return Program("threefry_block", b.module([y0, y1], name="jit_threefry"),
                   [("key", (2,), "ui32"), ("x0", (n,), "ui32"), ("x1", (n,), "ui32")],
                   [("y0", (n,), "ui32"), ("y1", (n,), "ui32")], 1, {"n": n})


def threefry_bits(n: int) -> Program:
    """key ui32[2] -> n random ui32 words the way jax.random.bits lays them out: the counters 0 .. n-1 (n even) split into
    a lower and an upper half, one Threefry block per pair, the two output halves concatenated."""
    assert n % 2 == 0
    b = Builder()
    key = b.arg((2,), "ui32")
    h = n // 2
    counts = b.iota((n,), "ui32", 0)
    k0 = b.broadcast_in_dim(b.reshape(b.slice(key, (0,), (1,)), ()), (h,), ())
    k1 = b.broadcast_in_dim(b.reshape(b.slice(key, (1,), (2,)), ()), (h,), ())
    y0, y1 = _threefry2x32(b, k0, k1, b.slice(counts, (0,), (h,)), b.slice(counts, (h,), (n,)))
    return Program("threefry_bits", b.module([b.concatenate([y0, y1], 0)], name="jit_random_bits"), [("key", (2,), "ui32")],
                   [("bits", (n,), "ui32")], 1, {"n": n})
