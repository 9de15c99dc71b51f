"""Host-only checks of the program verifier that run_program applies before its first launch
(gptrs_cuda_verify_program): a program whose declared types do not follow from its operands, whose
attributes are out of range or whose operand counts are wrong is a SpecViolation, the way the reference
interpreter refuses it (crates/gpt-rs-backend-ref-cpu/src/cpu.rs), never an out-of-bounds access."""
import copy
import json

import pytest

from gptrs_b200 import BackendError, check, lib
from gptrs_b200 import ptir


def _verify(program: dict):
    text = json.dumps(program).encode()
    check(lib().gptrs_cuda_verify_program(text, len(text)))


def _base():
    """x[4,6] -> transpose -> slice -> reduce -> binary with a broadcast scalar; concat and a dot on the side."""
    b = ptir.Builder()
    x = b.parameter(ptir.F32, [4, 6])
    w = b.parameter(ptir.F32, [6, 3])
    ids = b.parameter(ptir.SI32, [2])
    t = x.transpose([1, 0])
    s = t.slice([1, 0], [4, 4])
    r = s.reduce("Sum", 1)
    y = r * 0.5
    d = x.dot_general(w, [], [1], [0])
    c = b.concat(0, [d, d])
    g = b.take(x, ids)
    b.set_results([y, c, g])
    return b.program()


def _inst(program, name):
    for i in program["functions"][0]["body"]:
        op = i["op"]
        if (isinstance(op, str) and op == name) or (isinstance(op, dict) and name in op):
            return i
    raise KeyError(name)


def test_well_formed_program_passes():
    _verify(_base())


def _expect_violation(program, fragment=None):
    with pytest.raises(BackendError) as e:
        _verify(program)
    assert e.value.kind == "SpecViolation", str(e.value)
    if fragment:
        assert fragment in str(e.value), str(e.value)


def test_declared_output_must_follow_from_operands():
    p = _base()
    _inst(p, "ElementwiseBinary")["output"]["Tensor"]["shape"]["dims"][0] = {"Static": 400}
    _expect_violation(p, "ElementwiseBinary")
    p = _base()
    _inst(p, "Concat")["output"]["Tensor"]["shape"]["dims"][0] = {"Static": 9}
    _expect_violation(p, "Concat")
    p = _base()
    _inst(p, "DotGeneral")["output"]["Tensor"]["shape"]["dims"][1] = {"Static": 7}
    _expect_violation(p, "DotGeneral")
    p = _base()
    _inst(p, "Reduce")["output"]["Tensor"]["shape"]["dims"] = [{"Static": 4}, {"Static": 4}]
    _expect_violation(p, "Reduce")
    p = _base()
    _inst(p, "Take")["output"]["Tensor"]["shape"]["dims"][1] = {"Static": 60}
    _expect_violation(p, "Take")


def test_attribute_ranges():
    p = _base()
    _inst(p, "Transpose")["op"]["Transpose"]["perm"] = [1, 1]
    _expect_violation(p, "perm")
    p = _base()
    _inst(p, "Transpose")["op"]["Transpose"]["perm"] = [0, 5]
    _expect_violation(p, "perm")
    p = _base()
    _inst(p, "Slice")["op"]["Slice"]["starts"] = [-1, 0]
    _expect_violation(p, "slice")
    p = _base()
    _inst(p, "Slice")["op"]["Slice"]["sizes"] = [4]
    _expect_violation(p, "Slice")
    p = _base()
    _inst(p, "Reduce")["op"]["Reduce"]["axes"] = [2]
    _expect_violation(p, "axes")
    p = _base()
    _inst(p, "Concat")["op"]["Concat"]["axis"] = 3
    _expect_violation(p, "axis")
    p = _base()
    _inst(p, "DotGeneral")["op"]["DotGeneral"]["contract_rhs"] = [4]
    _expect_violation(p, "DotGeneral")


def test_operand_counts_and_missing_attributes():
    p = _base()
    _inst(p, "ElementwiseBinary")["operands"].pop()
    _expect_violation(p, "2 operands")
    p = _base()
    _inst(p, "Take")["operands"].pop()
    _expect_violation(p, "Take")
    p = _base()
    _inst(p, "Transpose")["op"] = "Transpose"          # an operation that needs attributes, written as a bare string
    _expect_violation(p, "without its attributes")
    p = _base()
    _inst(p, "ElementwiseBinary")["op"] = {"ElementwiseBinary": {"kind": "Add"}}
    _expect_violation(p, "must be a string")


def test_undefined_values_and_duplicate_ids():
    p = _base()
    _inst(p, "Reduce")["operands"][0] = {"Value": 9999}
    _expect_violation(p, "undefined value")
    p = _base()
    body = p["functions"][0]["body"]
    body[1]["id"] = body[0]["id"]
    _expect_violation(p)
    p = _base()
    p["functions"][0]["result_ids"][0] = 4242
    _expect_violation(p, "undefined")


def test_literal_byte_length_is_checked():
    p = _base()
    for inst in p["functions"][0]["body"]:
        for o in inst["operands"]:
            if "Literal" in o:
                o["Literal"]["bytes"] = o["Literal"]["bytes"][:-1]
                _expect_violation(copy.deepcopy(p), "literal")
                return
    raise AssertionError("the base program has a literal operand")


def test_fused_custom_calls_are_checked_too():
    b = ptir.Builder()
    x = b.parameter(ptir.F32, [3, 8])
    g = b.parameter(ptir.F32, [8])
    y = b.custom_call("gpt_rs.cuda.rms_norm.f32.v1", [x, g], ptir.F32, [3, 8], {"eps": {"kind": "F64", "value": 1e-5}})
    b.set_results([y])
    _verify(b.program())
    b = ptir.Builder()
    x = b.parameter(ptir.F32, [3, 8])
    g = b.parameter(ptir.F32, [7])   # gain of the wrong width
    y = b.custom_call("gpt_rs.cuda.rms_norm.f32.v1", [x, g], ptir.F32, [3, 8], {"eps": {"kind": "F64", "value": 1e-5}})
    b.set_results([y])
    _expect_violation(b.program(), "gain")
