"""The PyTorch twins of the Gemma-shaped decoder and the DistilBERT-shaped step against the StableHLO interpreter on
the generated programs (CPU): two independent statements of the same mathematics must agree before either is used to
judge the GPU at sizes the interpreter cannot reach."""
import numpy as np
import torch

from b200.shlo import programs
from oracle import interp, twins

TINY = dict(vocab=384, dim=64, layers=2, heads=4, head_dim=16, hidden=128)


def test_gemma_twin_matches_interpreter_on_prefill_and_decode_loop():
    pre = programs.gemma_prefill(**TINY, prompt_len=8, cache_len=16)
    dec = programs.gemma_decode_loop(**TINY, start=8, new_tokens=6, cache_len=16)
    spec = [(n, s) for n, s, _ in pre.args[:-1]]
    for seed in (0, 1):
        w = programs.gemma_weights(spec, seed=seed, weight_std=0.3, tile=1 << 16)
        prompt = np.random.default_rng(seed + 10).integers(0, TINY["vocab"], 8).astype(np.int32)
        po = interp.run_text(pre.text, w + [prompt])
        do = interp.run_text(dec.text, w + [po[0]] + list(po[2:]))
        tw = twins.GemmaTwin({n: a for (n, _), a in zip(spec, w)}, heads=4, head_dim=16, cache_len=16)
        lg = tw.forward(prompt, 0).numpy()
        assert int(lg.argmax()) == int(po[0][0])
        # both round the logits to bfloat16: they may differ by one unit in the last place where accumulation order differs
        np.testing.assert_allclose(lg, po[1], rtol=2 ** -7, atol=2 ** -7 * np.abs(po[1]).max())
        tok, toks = int(lg.argmax()), []
        for i in range(6):
            lg = tw.forward(np.array([tok]), 8 + i).numpy()
            tok = int(lg.argmax())
            toks.append(tok)
        assert toks == list(do[0])
        np.testing.assert_allclose(lg, do[1], rtol=2 ** -7, atol=2 ** -7 * np.abs(do[1]).max())
        # the caches the twin holds are the ones the programs return
        np.testing.assert_allclose(tw.k[1].numpy(), do[2 + 2], rtol=2 ** -7, atol=1e-2)


def test_gemma_weights_are_bfloat16_values_and_bit_patterns_agree():
    spec = [("embed", (300, 64)), ("layer0.attn_norm", (64,)), ("big", (5000, 4096))]
    a = programs.gemma_weights(spec, seed=3, tile=1 << 20)
    b = programs.gemma_weights(spec, seed=3, tile=1 << 20, as_bits=True)
    for x, y in zip(a, b):
        assert x.dtype == np.float32 and y.dtype == np.uint16 and x.shape == y.shape
        np.testing.assert_array_equal((y.astype(np.uint32) << 16).view(np.float32), x)
    assert abs(float(a[2].std()) - 0.02) < 1e-3 and not a[1].any()


def test_distilbert_twin_matches_interpreter():
    shape = dict(batch=2, seq=16, vocab=160, dim=64, layers=2, heads=4, ffn=128)
    prog = programs.distilbert_mlm_step(**shape, dtype="f32")
    args = programs.distilbert_inputs(prog, seed=3, weight_std=0.1, mask_rate=0.3)
    want = interp.run_text(prog.text, args)
    names = [n for n, _, _ in prog.args[:-2]]
    loss, grads = twins.distilbert_loss_and_grads(dict(zip(names, args)), args[-2], args[-1], heads=4, dtype=torch.float64)
    assert abs(loss - float(want[0])) < 1e-5 * abs(loss)
    top = max(float(np.abs(w).max()) for w in want[1:])
    for n, g, w in zip(names, grads, want[1:]):
        scale = max(float(np.abs(w).max()), 1e-3 * top)      # key biases have no gradient in exact arithmetic
        np.testing.assert_allclose(g, w, rtol=2e-4, atol=2e-5 * scale, err_msg=n)
