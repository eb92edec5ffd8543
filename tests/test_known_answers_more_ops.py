"""Known answers for the later operations (tests/golden/known_answers_more_ops.json, made by
tests/golden/make_known_answers_more_ops.py from plain-Python loops: an insertion sort, Cholesky-Banachiewicz,
substitution, Philox-4x32-10 on Python integers, a sequential scatter): the interpreter under oracle/ must reproduce
them. The CUDA path is held to the interpreter on the same operations in tests/test_sort.py, tests/test_rng_bits.py,
tests/test_linalg.py and tests/test_gpu_ops.py; the plans of all cases must compile, generated source included."""
import json
from pathlib import Path

import numpy as np
import pytest

import b200
from oracle import interp

CASES = json.loads((Path(__file__).parent / "golden" / "known_answers_more_ops.json").read_text())["cases"]


def _arrays(items):
    return [np.array(i["data"], dtype=i["dtype"]).reshape(i["shape"]) for i in items]


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_reproduces_known_answers(case):
    outs = interp.run_text(case["mlir"], _arrays(case["inputs"]))
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
def test_plans_compile(case):
    plan, _ = b200.compile_to_plan(case["mlir"], validate=True)
    assert "kernel" in plan
