"""TEST INFRASTRUCTURE — PyTorch-CPU twins of the benchmark models.

An implementation of the same mathematics that shares no code with the
StableHLO generators or the interpreter: torch modules + autograd. Used (1) to
pin the interpreter and the generated programs (loss, every gradient leaf,
updated parameters), and (2) as the timed CPU baseline (the jaxlib CPU backend
the reference's README compares against is not installable here; this is the
stand-in, labelled "PyTorch-CPU" wherever it is reported).

Architecture: examples/resnet/model.py:6-163 of the reference (CIFAR ResNet18,
NHWC data, HWIO kernels, SAME padding, training-mode BatchNorm eps 1e-5).
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F


def _same_pad(size, k, s):
    out = -(-size // s)
    tot = max((out - 1) * s + k - size, 0)
    return tot // 2, tot - tot // 2


def _conv_same(x, w_hwio, stride):
    """x NCHW, kernel stored HWIO. XLA's SAME padding puts the extra pixel at
    the high edge, so pad explicitly."""
    kh, kw = w_hwio.shape[0], w_hwio.shape[1]
    pt, pb = _same_pad(x.shape[2], kh, stride)
    pl, pr = _same_pad(x.shape[3], kw, stride)
    x = F.pad(x, (pl, pr, pt, pb))
    return F.conv2d(x, w_hwio.permute(3, 2, 0, 1), None, stride=stride)


def _bn(x, scale, bias, eps=1e-5):
    mean = x.mean((0, 2, 3))
    mean2 = (x * x).mean((0, 2, 3))
    var = torch.clamp_min(mean2 - mean * mean, 0.0)
    mul = torch.rsqrt(var + eps) * scale
    return (x - mean[None, :, None, None]) * mul[None, :, None, None] + bias[None, :, None, None]


def resnet18_logits(p: dict, x_nhwc: torch.Tensor) -> torch.Tensor:
    x = x_nhwc.permute(0, 3, 1, 2)
    y = F.relu(_bn(_conv_same(x, p["conv_init.kernel"], 1), p["bn_init.scale"], p["bn_init.bias"]))
    for stage in range(4):
        for blk in range(2):
            n = f"stage{stage + 1}_block{blk + 1}"
            stride = 2 if (stage > 0 and blk == 0) else 1
            res = y
            z = _conv_same(y, p[n + ".conv1.kernel"], stride)
            z = F.relu(_bn(z, p[n + ".bn1.scale"], p[n + ".bn1.bias"]))
            z = _conv_same(z, p[n + ".conv2.kernel"], 1)
            z = _bn(z, p[n + ".bn2.scale"], p[n + ".bn2.bias"])
            if (n + ".conv_proj.kernel") in p:
                res = _bn(_conv_same(res, p[n + ".conv_proj.kernel"], stride),
                          p[n + ".bn_proj.scale"], p[n + ".bn_proj.bias"])
            y = F.relu(res + z)
    y = y.mean((2, 3))
    return y @ p["dense.kernel"] + p["dense.bias"]


def resnet18_train_step(params: dict, moms: dict, x: np.ndarray, y: np.ndarray, lr=0.1, momentum=0.9,
                        dtype=torch.float32, grad_transform=None):
    """One SGD-momentum step. Returns (loss, new_params, new_moms, grads) as
    numpy. `grad_transform(list_of_grads, loss)` lets a data-parallel test
    average gradients across ranks before the update."""
    names = list(params)
    tp = {n: torch.tensor(np.asarray(params[n]), dtype=dtype, requires_grad=True) for n in names}
    xt = torch.tensor(x, dtype=dtype)
    yt = torch.tensor(y, dtype=torch.long)
    logits = resnet18_logits(tp, xt)
    loss = F.cross_entropy(logits, yt)
    grads = torch.autograd.grad(loss, [tp[n] for n in names])
    grads = [g.detach() for g in grads]
    loss = loss.detach()
    if grad_transform is not None:
        grads, loss = grad_transform(grads, loss)
    new_p, new_m = {}, {}
    with torch.no_grad():
        for n, g in zip(names, grads):
            m = torch.tensor(np.asarray(moms[n]), dtype=dtype) * momentum + g
            new_m[n] = m.numpy()
            new_p[n] = (tp[n] - lr * m).numpy()
    return float(loss), new_p, new_m, {n: g.numpy() for n, g in zip(names, grads)}


class ResNet18Stepper:
    """Stateful torch-CPU training loop used as the timed CPU baseline."""

    def __init__(self, params: dict, lr=0.1, momentum=0.9, threads: int | None = None):
        if threads:
            torch.set_num_threads(threads)
        self.names = list(params)
        self.p = {n: torch.tensor(np.asarray(params[n]), dtype=torch.float32, requires_grad=True) for n in self.names}
        self.m = {n: torch.zeros_like(self.p[n]) for n in self.names}
        self.lr, self.mu = lr, momentum

    def step(self, x: np.ndarray, y: np.ndarray) -> float:
        xt = torch.from_numpy(x)
        yt = torch.from_numpy(y.astype(np.int64))
        loss = F.cross_entropy(resnet18_logits(self.p, xt), yt)
        grads = torch.autograd.grad(loss, [self.p[n] for n in self.names])
        with torch.no_grad():
            for n, g in zip(self.names, grads):
                self.m[n].mul_(self.mu).add_(g)
                self.p[n].sub_(self.lr * self.m[n])
        return float(loss)


def lstm_train_step(params, xs, targets, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, dtype=None):
    """PyTorch twin of b200.shlo.programs.lstm_scan_train_step (two stacked LSTM layers in the concatenated
    form, gate order i, f, g, o; MSE of the last hidden state; first Adam step from zero moments) by autograd.
    `params` = [w1, b1, w2, b2] as numpy arrays. Returns loss, new params, first moments, second moments."""
    import numpy as np
    import torch
    dtype = dtype or torch.float64
    P = [torch.tensor(np.asarray(a), dtype=dtype, requires_grad=True) for a in params]
    xs = torch.tensor(np.asarray(xs), dtype=dtype)
    tg = torch.tensor(np.asarray(targets), dtype=dtype)
    B, H = tg.shape

    def cell(x, h, c, w, b):
        z = torch.cat([x, h], 1) @ w + b
        i, f, g, o = torch.sigmoid(z[:, :H]), torch.sigmoid(z[:, H:2 * H]), torch.tanh(z[:, 2 * H:3 * H]), torch.sigmoid(z[:, 3 * H:])
        c2 = f * c + i * g
        return o * torch.tanh(c2), c2

    h1 = c1 = h2 = c2 = torch.zeros(B, H, dtype=dtype)
    for t in range(xs.shape[0]):
        h1, c1 = cell(xs[t], h1, c1, P[0], P[1])
        h2, c2 = cell(h1, h2, c2, P[2], P[3])
    loss = ((h2 - tg) ** 2).mean()
    loss.backward()
    new_p, ms, vs = [], [], []
    for p in P:
        g = p.grad.numpy()
        m, v = (1 - beta1) * g, (1 - beta2) * g * g
        new_p.append(p.detach().numpy() - lr * (m / (1 - beta1)) / (np.sqrt(v / (1 - beta2)) + eps))
        ms.append(m)
        vs.append(v)
    return float(loss), new_p, ms, vs
