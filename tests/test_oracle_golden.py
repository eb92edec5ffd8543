"""CPU: the oracle against the committed fixtures (tests/golden/), i.e. against
the literal expectations of the reference's own tests and against the PyTorch
float64 twin. This is what pins the oracle before the GPU tests trust it."""
import json
from pathlib import Path

import numpy as np
import pytest

from oracle import interp

GOLD = Path(__file__).resolve().parent / "golden"
LITERALS = json.loads((GOLD / "reference_literals.json").read_text())


def literal_inputs(case):
    from oracle.mlir_text import np_dtype
    return [np.array(v, dtype=np_dtype(dt)) for v, dt in zip(case["inputs"], case["input_dtypes"])]


@pytest.mark.parametrize("case", LITERALS, ids=[c["name"] for c in LITERALS])
def test_reference_literals(case):
    outs = interp.run_text(case["mlir"], literal_inputs(case))
    for i, (o, e) in enumerate(zip(outs, case["expected"])):
        if i in case["skip"]:
            continue
        np.testing.assert_allclose(o, np.array(e, np.float32), rtol=case["rtol"], atol=case["atol"])


def resnet_tiny_args():
    from b200.shlo import programs
    g = json.loads((GOLD / "resnet18_tiny.json").read_text())
    prog = programs.resnet18_train_step(**g["config"])
    args = programs.resnet18_inputs(prog, seed_w=0, seed_x=1)
    rng = np.random.default_rng(g["perturb_seed"])
    args = [a if n in ("x", "y") else (a + 0.1 * rng.standard_normal(a.shape)).astype(np.float32)
            for a, (n, _, _) in zip(args, prog.args)]
    return g, prog, args


def check_resnet_against_golden(g, prog, outs, rtol, atol_scale):
    assert abs(float(outs[0]) - g["loss"]) <= rtol * abs(g["loss"]) + 1e-5
    for (name, _, _), o in zip(prog.results[1:], outs[1:]):
        ref = g["leaves"][name]
        o = np.asarray(o, np.float64)
        scale = ref["abs_sum"] + 1e-3
        assert abs(o.sum() - ref["sum"]) <= atol_scale * scale, (name, o.sum(), ref["sum"])
        assert abs(np.abs(o).sum() - ref["abs_sum"]) <= atol_scale * scale, name
        np.testing.assert_allclose(o.reshape(-1)[:4], ref["first"], rtol=50 * rtol, atol=50 * atol_scale * scale / o.size + 1e-5,
                                   err_msg=name)


def test_resnet_step_oracle_float64_matches_torch_twin():
    g, prog, args = resnet_tiny_args()
    outs = interp.run_text(prog.text, args, wide=True)
    check_resnet_against_golden(g, prog, outs, rtol=1e-6, atol_scale=1e-7)   # f32 literals (lr, momentum, eps) vs doubles in the twin


def test_resnet_step_oracle_float32_within_plugin_tolerance():
    g, prog, args = resnet_tiny_args()
    outs = interp.run_text(prog.text, args)
    check_resnet_against_golden(g, prog, outs, rtol=1e-4, atol_scale=1e-5)
