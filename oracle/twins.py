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


class GemmaTwin:
    """PyTorch-CPU twin of b200.shlo.programs.gemma_prefill / gemma_decode_loop (the decoder of
    examples/gemma/model.py:118-296 of the reference: RMSNorm with weight 1 + w, rotate-half rotary embedding, one
    shared key-value head, GeGLU feed-forward, tied embedding scaled by sqrt(dim)). Weights arrive as float32 arrays
    holding bfloat16 values. Every product takes operands rounded to bfloat16, accumulates in fp32 and rounds its
    result to bfloat16 once; norms, rotary embedding and softmax run in fp32: the rounding points of the program."""

    def __init__(self, weights: dict, heads: int, head_dim: int, cache_len: int):
        self.w = {k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in weights.items()}
        self.layers = sum(1 for k in self.w if k.endswith(".wq"))
        self.heads, self.hd, self.cache_len = heads, head_dim, cache_len
        self.dim = self.w["embed"].shape[1]
        half = head_dim // 2
        self.inv_freq = torch.from_numpy((1.0 / (10000.0 ** (np.arange(half, dtype=np.float64) * 2 / head_dim))).astype(np.float32))
        self.k = [torch.zeros(cache_len, head_dim) for _ in range(self.layers)]
        self.v = [torch.zeros(cache_len, head_dim) for _ in range(self.layers)]

    @staticmethod
    def bf(x):
        return x.to(torch.bfloat16).to(torch.float32)

    def lin(self, x, w):
        return self.bf(self.bf(x) @ w)

    def rms(self, x, w):
        inv = torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6)
        return x * inv * (w + 1.0)

    def rope(self, x, pos):                           # x [rows, n, hd], pos float32 [rows]
        ang = pos[:, None] * self.inv_freq[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        half = self.hd // 2
        x1, x2 = x[..., :half], x[..., half:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)

    @staticmethod
    def gelu(x):
        return 0.5 * x * (1.0 + torch.tanh(np.float32(np.sqrt(2.0 / np.pi)) * (x + np.float32(0.044715) * x * x * x)))

    def forward(self, tokens: np.ndarray, start: int) -> torch.Tensor:
        """Runs positions start .. start + len(tokens) - 1 (causal among themselves, attending to the caches before
        them), writes their keys and values into the caches and returns the fp32 logits of the last position."""
        with torch.no_grad():
            T, H, hd = len(tokens), self.heads, self.hd
            pos = torch.arange(start, start + T, dtype=torch.float32)
            x = self.w["embed"][torch.from_numpy(np.asarray(tokens, np.int64))] * np.float32(np.sqrt(self.dim))
            end = start + T
            visible = torch.arange(end)[None, :] <= torch.arange(start, end)[:, None]        # [T, end]
            for i in range(self.layers):
                p = f"layer{i}."
                h = self.rms(x, self.w[p + "attn_norm"])
                q = self.rope(self.lin(h, self.w[p + "wq"]).reshape(T, H, hd), pos)
                k = self.rope(self.lin(h, self.w[p + "wk"]).reshape(T, 1, hd), pos).reshape(T, hd)
                v = self.lin(h, self.w[p + "wv"])
                self.k[i][start:end] = self.bf(k)
                self.v[i][start:end] = self.bf(v)
                kc, vc = self.k[i][:end], self.v[i][:end]
                sc = self.bf(torch.einsum("thd,sd->hts", self.bf(q), kc)) * np.float32(1.0 / np.sqrt(hd))
                sc = torch.where(visible[None], sc, torch.tensor(-1e30))
                pr = torch.softmax(sc, -1)
                att = self.bf(torch.einsum("hts,sd->thd", self.bf(pr), vc)).reshape(T, H * hd)
                x = x + self.lin(att, self.w[p + "wo"])
                h2 = self.rms(x, self.w[p + "mlp_norm"])
                ff = self.gelu(self.lin(h2, self.w[p + "w_gate"])) * self.lin(h2, self.w[p + "w_up"])
                x = x + self.lin(ff, self.w[p + "w_down"])
            hf = self.bf(self.rms(x[-1:], self.w["final_norm"]))
            return self.bf(hf @ self.w["embed"].T)[0]


def distilbert_loss_and_grads(weights: dict, ids: np.ndarray, mask: np.ndarray, heads: int, dtype=torch.float32):
    """PyTorch autograd twin of b200.shlo.programs.distilbert_mlm_step (examples/distilbert/model.py:11-94 of the
    reference: post-LayerNorm encoder, tanh GELU, tied-projector masked-LM head, labels = ids, loss averaged over the
    masked positions) in `dtype` arithmetic without intermediate rounding: the reference value a bfloat16 execution is
    held against. Returns the loss and one gradient per weight, in the order of `weights`."""
    W = {k: torch.tensor(np.asarray(v), dtype=dtype, requires_grad=True) for k, v in weights.items()}
    B, S = ids.shape
    N, dim = B * S, W["word_emb"].shape[1]
    hd = dim // heads
    layers = sum(1 for k in W if k.endswith(".q.w"))
    idt = torch.from_numpy(ids.reshape(-1).astype(np.int64))

    def ln(x, s, b):
        mu = x.mean(-1, keepdim=True)
        xc = x - mu
        return xc * torch.rsqrt((xc * xc).mean(-1, keepdim=True) + 1e-12) * s + b

    def gelu(x):
        return 0.5 * x * (1.0 + torch.tanh(np.sqrt(2.0 / np.pi) * (x + 0.044715 * x * x * x)))

    x = W["word_emb"][idt] + W["pos_emb"][:S].repeat(B, 1)
    x = ln(x, W["emb_ln.scale"], W["emb_ln.bias"])
    for i in range(layers):
        p = f"layer{i}."
        def split(t): return t.reshape(B, S, heads, hd).permute(0, 2, 1, 3)
        q, k, v = (split(x @ W[p + n + ".w"] + W[p + n + ".b"]) for n in ("q", "k", "v"))
        pr = torch.softmax(q @ k.transpose(-1, -2) / np.sqrt(hd), -1)
        ctx = (pr @ v).permute(0, 2, 1, 3).reshape(N, dim)
        x = ln(x + ctx @ W[p + "o.w"] + W[p + "o.b"], W[p + "attn_ln.scale"], W[p + "attn_ln.bias"])
        ff = gelu(x @ W[p + "ff1.w"] + W[p + "ff1.b"]) @ W[p + "ff2.w"] + W[p + "ff2.b"]
        x = ln(x + ff, W[p + "out_ln.scale"], W[p + "out_ln.bias"])
    h = ln(gelu(x @ W["head.w"] + W["head.b"]), W["head_ln.scale"], W["head_ln.bias"])
    logits = h @ W["word_emb"].T + W["vocab_bias"]
    nll = F.cross_entropy(logits, idt, reduction="none")
    wv = torch.tensor(np.asarray(mask).reshape(-1), dtype=dtype)
    loss = (nll * wv).sum() / torch.clamp(wv.sum(), min=1.0)
    grads = torch.autograd.grad(loss, [W[k] for k in weights])
    return float(loss.detach()), [g.numpy() for g in grads]
