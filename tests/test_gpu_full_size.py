"""The transformer configurations at their full sizes on the GPU against the PyTorch twins (tests/test_twins.py pins
the twins against the interpreter at sizes the interpreter can reach):

  * Gemma-2B-shaped inference: 18 layers, width 2048, 8 query heads sharing one key-value head of 256, GeGLU 16384,
    vocabulary 256000, bf16; prefill of 512 prompt tokens in one pass, then 128 greedy decode steps inside one
    stablehlo.while (examples/gemma/main.py:109-134 of the reference).
  * DistilBERT-base-shaped masked-LM step: 6 layers, width 768, 12 heads, FFN 3072, vocabulary 30522, batch 32 x 128,
    bf16, loss and the gradient of every leaf (examples/distilbert/model.py:11-94 of the reference).
"""
import numpy as np
import pytest
import torch

from b200.shlo import programs
from oracle import twins

pytestmark = pytest.mark.gpu


def test_gemma_2b_prefill_and_decode_full_size(client):
    """Token ids: the twin is fed the GPU's own tokens position by position (so that both see one context) and must
    choose the same next token wherever its best logit leads the runner-up by more than the resolution of the bf16
    logits; inside that resolution the GPU's choice must be one of the tied leaders. Logits agree at bf16 tolerance."""
    pre = programs.gemma_prefill()
    dec = programs.gemma_decode_loop()
    spec = [(n, s) for n, s, _ in pre.args[:-1]]
    bits = programs.gemma_weights(spec, seed=0, as_bits=True)
    wb = [client.buffer_from_host(b, dtype="bf16") for b in bits]
    prompt = np.random.default_rng(1).integers(0, 256000, 512).astype(np.int32)
    e_pre, e_dec = client.compile(pre.text), client.compile(dec.text)
    assert "gemm16" in e_pre.plan_text() and "gemv16" in e_dec.plan_text() and "igemm" not in e_dec.plan_text()
    po = e_pre.execute(wb + [client.buffer_from_host(prompt)])
    do = e_dec.execute(wb + [po[0]] + po[2:])
    g0, logits_p = int(po[0].to_numpy()[0]), po[1].to_numpy()
    gen, logits_d = do[0].to_numpy(), do[1].to_numpy()
    assert gen.shape == (128,) and gen.min() >= 0 and gen.max() < 256000
    del wb

    tw = twins.GemmaTwin({n: (b.astype(np.uint32) << 16).view(np.float32) for (n, _), b in zip(spec, bits)},
                         heads=8, head_dim=256, cache_len=640)
    del bits
    torch.set_num_threads(torch.get_num_threads())

    def agrees(lg: np.ndarray, chosen: int) -> bool:
        tie = 2.0 ** -7 * float(np.abs(lg).max())           # two units in the last place of a bf16 logit
        return int(lg.argmax()) == chosen or lg[chosen] >= lg.max() - tie

    lg = tw.forward(prompt, 0).numpy()
    np.testing.assert_allclose(logits_p, lg, rtol=2e-2, atol=2e-2 * float(np.abs(lg).max()))
    assert agrees(lg, g0)
    exact = int(int(lg.argmax()) == g0)
    tok = g0
    for i in range(128):
        lg = tw.forward(np.array([tok]), 512 + i).numpy()
        assert agrees(lg, int(gen[i])), (i, int(lg.argmax()), int(gen[i]))
        exact += int(int(lg.argmax()) == int(gen[i]))
        tok = int(gen[i])
    np.testing.assert_allclose(logits_d, lg, rtol=2e-2, atol=2e-2 * float(np.abs(lg).max()))
    assert exact >= 120, exact            # ties inside bf16 resolution are rare
    # the caches the decode loop returns hold the twin's keys and values
    for layer in (0, 17):
        kc = do[2 + 2 * layer].to_numpy().astype(np.float32)
        np.testing.assert_allclose(kc[:640], tw.k[layer].numpy(), rtol=2e-2, atol=2e-2 * float(tw.k[layer].abs().max()))


def test_distilbert_base_step_full_size(client):
    """Loss and every gradient leaf of the bf16 step against the fp32 autograd twin on the same bf16-valued weights:
    rtol 2e-2, atol 2e-2 of the leaf's own scale (never below a hundredth of the largest gradient: the key biases
    have no gradient in exact arithmetic)."""
    prog = programs.distilbert_mlm_step()
    args = programs.distilbert_inputs(prog, seed=0)
    from b200.shlo.builder import f32_to_bf16_bits
    n_w = len(args) - 2
    bits = [f32_to_bf16_bits(a).reshape(a.shape) for a in args[:n_w]]
    vals = [(b.astype(np.uint32) << 16).view(np.float32) for b in bits]
    exe = client.compile(prog.text)
    plan = exe.plan_text()
    assert "gemm16" in plan and "igemm" not in plan and "scatter rows=30522" in plan
    outs = exe.execute([client.buffer_from_host(b, dtype="bf16") for b in bits] +
                       [client.buffer_from_host(args[-2]), client.buffer_from_host(args[-1])])
    got = [o.to_numpy() for o in outs]
    names = [n for n, _, _ in prog.args[:n_w]]
    loss, grads = twins.distilbert_loss_and_grads(dict(zip(names, vals)), args[-2], args[-1], heads=12)
    assert abs(float(got[0]) - loss) < 2e-2 * abs(loss), (float(got[0]), loss)
    top = max(float(np.abs(g).max()) for g in grads)
    for n, g, w in zip(names, got[1:], grads):
        scale = max(float(np.abs(w).max()), 1e-2 * top)
        np.testing.assert_allclose(np.asarray(g, np.float64), w, rtol=2e-2, atol=2e-2 * scale, err_msg=n)
