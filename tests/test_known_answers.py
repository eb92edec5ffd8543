"""Known-answer fixtures (tests/golden/known_answers.json, made by tests/golden/make_known_answers.py from brute-force
nested loops): the interpreter under oracle/ must reproduce them on the CPU, and the CUDA path on the GPU. They pin
the corner rules of convolution (dilate, then pad; batch groups), dot_general with several free dimensions, case with
an index outside the branches, a long counted loop, clamped dynamic_update_slice, scatter-add with repeated rows,
negative / interior padding and argmax ties independently of the interpreter's own convolution backend."""
import json
from pathlib import Path

import numpy as np
import pytest

from oracle import interp

CASES = json.loads((Path(__file__).parent / "golden" / "known_answers.json").read_text())["cases"]


def _arrays(items):
    return [np.array(i["data"], dtype=i["dtype"]).reshape(i["shape"]) for i in items]


def _check(outs, case):
    want = _arrays(case["expected"])
    assert len(outs) == len(want)
    for o, w in zip(outs, want):
        o = np.asarray(o)
        assert o.shape == w.shape, (case["name"], o.shape, w.shape)
        if w.dtype.kind in "iub":
            np.testing.assert_array_equal(o, w, err_msg=case["name"])
        else:
            np.testing.assert_allclose(o, w, rtol=case["rtol"], atol=case["atol"], err_msg=case["name"])


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_reproduces_known_answers(case):
    _check(interp.run_text(case["mlir"], _arrays(case["inputs"])), case)


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_gpu_reproduces_known_answers(client, case):
    from tests.util import run_gpu
    outs, _ = run_gpu(client, case["mlir"], _arrays(case["inputs"]))
    _check(outs, case)
