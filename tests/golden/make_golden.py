"""Generates the committed fixtures in this directory. Run from the repo root:

    python tests/golden/make_golden.py

1. reference_literals.json — the literal expectations the reference's own
   tests hold for raw StableHLO programs (the reference needs an Apple GPU, so
   they are taken from its test sources, not from running it):
     tests/test_ops.py:216-281         composite decompositions vs numpy.arcsin / numpy.sinh
     tests/test_control_flow_compile.py:107-133   token threading (3 + 1 == 4), value_and_grad of x*x at 3 (9, 6)
2. resnet18_tiny.json — loss and per-leaf checksums of one ResNet18
   SGD-momentum step computed by the PyTorch float64 twin (oracle/twins.py),
   an implementation independent of the StableHLO generator and interpreter.
"""
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "jax-mps_b200"))
sys.path.insert(0, str(ROOT))
HERE = Path(__file__).resolve().parent

COMPOSITE = """
module @test {{
  func.func private @{impl}(%arg0: tensor<4xf32>) -> tensor<4xf32> {{
{body}
  }}
  func.func @main(%arg0: tensor<4xf32>) -> tensor<4xf32> {{
    %0 = stablehlo.composite "{name}" %arg0 {{decomposition = @{impl}}} : (tensor<4xf32>) -> tensor<4xf32>
    return %0 : tensor<4xf32>
  }}
}}
"""
ASIN_BODY = """    %cst = stablehlo.constant dense<1.000000e+00> : tensor<4xf32>
    %0 = stablehlo.multiply %arg0, %arg0 : tensor<4xf32>
    %1 = stablehlo.subtract %cst, %0 : tensor<4xf32>
    %2 = stablehlo.sqrt %1 : tensor<4xf32>
    %3 = stablehlo.atan2 %arg0, %2 : tensor<4xf32>
    return %3 : tensor<4xf32>"""
SINH_BODY = """    %0 = stablehlo.exponential %arg0 : tensor<4xf32>
    %1 = stablehlo.negate %arg0 : tensor<4xf32>
    %2 = stablehlo.exponential %1 : tensor<4xf32>
    %3 = stablehlo.subtract %0, %2 : tensor<4xf32>
    %cst = stablehlo.constant dense<2.000000e+00> : tensor<4xf32>
    %4 = stablehlo.divide %3, %cst : tensor<4xf32>
    return %4 : tensor<4xf32>"""
TOKEN_ADD = """
module @jit_f {
  func.func public @main(%arg0: tensor<f32>) -> (tensor<f32>, !stablehlo.token) {
    %cst = stablehlo.constant dense<1.000000e+00> : tensor<f32>
    %0 = stablehlo.add %arg0, %cst : tensor<f32>
    %1 = "stablehlo.create_token"() : () -> !stablehlo.token
    %2 = "stablehlo.after_all"(%1) : (!stablehlo.token) -> !stablehlo.token
    return %0, %2 : tensor<f32>, !stablehlo.token
  }
}
"""
SQUARE_GRAD = """
module @jit_value_and_grad {
  func.func public @main(%arg0: tensor<f32>) -> (tensor<f32>, !stablehlo.token, tensor<f32>) {
    %0 = stablehlo.multiply %arg0, %arg0 : tensor<f32>
    %1 = "stablehlo.create_token"() : () -> !stablehlo.token
    %2 = "stablehlo.after_all"(%1) : (!stablehlo.token) -> !stablehlo.token
    %cst = stablehlo.constant dense<1.000000e+00> : tensor<f32>
    %3 = stablehlo.multiply %cst, %arg0 : tensor<f32>
    %4 = stablehlo.multiply %arg0, %cst : tensor<f32>
    %5 = stablehlo.add %3, %4 : tensor<f32>
    return %0, %2, %5 : tensor<f32>, !stablehlo.token, tensor<f32>
  }
}
"""


def literals():
    x = [0.0, 0.5, -0.5, 0.9]
    xa = np.array(x, np.float32)
    return [
        {"name": "composite-arcsin", "source": "tests/test_ops.py:216-281", "mlir": COMPOSITE.format(impl="chlo.asin.impl", name="chlo.asin", body=ASIN_BODY),
         "inputs": [x], "input_dtypes": ["f32"], "expected": [np.arcsin(xa).tolist()], "skip": [], "atol": 1e-5, "rtol": 1e-5},
        {"name": "composite-sinh", "source": "tests/test_ops.py:216-281", "mlir": COMPOSITE.format(impl="chlo.sinh.impl", name="chlo.sinh", body=SINH_BODY),
         "inputs": [x], "input_dtypes": ["f32"], "expected": [np.sinh(xa).tolist()], "skip": [], "atol": 1e-5, "rtol": 1e-5},
        {"name": "token-threaded-add", "source": "tests/test_control_flow_compile.py:107-115", "mlir": TOKEN_ADD,
         "inputs": [3.0], "input_dtypes": ["f32"], "expected": [4.0, None], "skip": [1], "atol": 0, "rtol": 0},
        {"name": "grad-with-live-token", "source": "tests/test_control_flow_compile.py:118-133", "mlir": SQUARE_GRAD,
         "inputs": [3.0], "input_dtypes": ["f32"], "expected": [9.0, None, 6.0], "skip": [1], "atol": 0, "rtol": 0},
    ]


RESNET_TINY = dict(batch=8, image=16, width=8)


def resnet_tiny():
    import torch
    from b200.shlo import programs
    from oracle import twins
    prog = programs.resnet18_train_step(**RESNET_TINY)
    args = programs.resnet18_inputs(prog, seed_w=0, seed_x=1)
    # non-trivial momentum and BatchNorm parameters so every term of the update is exercised
    rng = np.random.default_rng(7)
    args = [a if n in ("x", "y") else (a + 0.1 * rng.standard_normal(a.shape)).astype(np.float32)
            for a, (n, _, _) in zip(args, prog.args)]
    names = [n for n, _, _ in prog.args]
    P = {n[2:]: a for n, a in zip(names, args) if n.startswith("p.")}
    M = {n[2:]: a for n, a in zip(names, args) if n.startswith("m.")}
    loss, new_p, new_m, grads = twins.resnet18_train_step(P, M, args[-2], args[-1], dtype=torch.float64)
    out = {"config": RESNET_TINY, "perturb_seed": 7, "loss": loss, "leaves": {}}
    for kind, d in (("p", new_p), ("m", new_m)):
        for n, a in d.items():
            a = np.asarray(a, np.float64)
            out["leaves"][f"{kind}.{n}"] = {"sum": float(a.sum()), "abs_sum": float(np.abs(a).sum()),
                                            "first": [float(v) for v in a.reshape(-1)[:4]]}
    return out


if __name__ == "__main__":
    (HERE / "reference_literals.json").write_text(json.dumps(literals(), indent=1))
    (HERE / "resnet18_tiny.json").write_text(json.dumps(resnet_tiny(), indent=1))
    print("wrote", [p.name for p in HERE.glob("*.json")])
