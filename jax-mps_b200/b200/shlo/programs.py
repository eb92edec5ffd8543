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
