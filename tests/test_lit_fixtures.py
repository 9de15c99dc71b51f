"""The reference's own textual PTIR fixtures (crates/gpt-rs/tests/fixtures/*.lit, the INPUT / EXPECTED pairs of its
canonicalisation passes) in the serde wire form, as written by tests/golden/make_lit_fixtures.py:

* host: the reader and the verifier of this backend accept every program, and the numpy interpreter evaluates INPUT and
  EXPECTED to the same values (the pass the fixture pins is semantics-preserving, so both forms pin the interpreter);
* GPU: run_program on either form equals the interpreter (moves, adds and maxima bit for bit; the one Rsqrt within
  2 ulp, rtol 2.4e-7)."""
import json
from pathlib import Path

import numpy as np
import pytest

from gptrs_b200 import check, lib
from oracle import ptir_ref as pr

CASES = json.loads((Path(__file__).parent / "golden" / "lit_programs.json").read_text())
DT = {"F32": np.float32, "Si32": np.int32, "I1": np.bool_}


def _inputs(program, seed):
    rng = np.random.default_rng(seed)
    out = []
    for ty in program["functions"][0]["parameters"]:
        t = ty["Tensor"]
        dims = [d["Static"] for d in t["shape"]["dims"]]
        if t["dtype"] == "F32":
            out.append(rng.uniform(0.25, 4.0, size=dims).astype(np.float32))   # positive: some fixtures take logs / roots
        else:
            out.append(rng.integers(0, 4, size=dims).astype(DT[t["dtype"]]))
    return out


def _same_signature(a, b):
    return a["functions"][0]["parameters"] == b["functions"][0]["parameters"]


def test_fixture_file_covers_the_reference_set():
    names = {c["name"].split(".")[0] for c in CASES}
    assert names == {"dedup", "elementwise", "param_only_fold_to_param", "reshape", "slice", "transpose"}
    assert len(CASES) == 9


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_verifier_accepts_and_interpreter_agrees(case):
    for side in ("input", "expected"):
        text = json.dumps(case[side]).encode()
        check(lib().gptrs_cuda_verify_program(text, len(text)))
    ins = _inputs(case["input"], 7)
    want = pr.run_program(case["input"], ins)
    assert len(want) == len(case["input"]["functions"][0]["results"])
    if _same_signature(case["input"], case["expected"]):
        got = pr.run_program(case["expected"], ins)
        for g, w in zip(got, want):
            assert g.shape == w.shape and np.array_equal(g, w, equal_nan=True)


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_run_program_matches_interpreter(cuda, case):
    from gptrs_b200.backend import CudaBackend
    be = CudaBackend()
    for side in ("input", "expected"):
        ins = _inputs(case[side], 11)
        want = pr.run_program(case[side], ins)
        for fusion in (True, False):
            be.set_fusion(fusion)
            got = [be.to_literal(h) for h in be.run_program(json.dumps(case[side]), [be.materialize(a) for a in ins])]
            assert len(got) == len(want)
            for g, w in zip(got, want):
                assert g.shape == w.shape and np.allclose(g, w, rtol=2.4e-7, atol=0), (case["name"], side, fusion)
    be.set_fusion(True)
