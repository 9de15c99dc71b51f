"""Turns the reference's textual PTIR fixtures (crates/gpt-rs/tests/fixtures/*.lit: INPUT / EXPECTED program pairs of
its canonicalisation passes, written by `Display for Program`, crates/gpt-rs/src/backend/spec.rs:858-1075) into the
serde-JSON wire form a backend receives, and writes them to tests/golden/lit_programs.json.

    python tests/golden/make_lit_fixtures.py /path/to/gpt.rs

The text form prints every operation with Rust's `Debug` of its spec (`Slice(SliceSpec { starts: [1, 1], ... })`); serde's
derive writes a struct as a map of its fields, a unit variant as its name and a one-field tuple variant as
{"Variant": value}, so the conversion is mechanical: struct names are dropped, the rest keeps its shape. Run where the
reference tree is present; the tests read only the JSON it writes."""
from __future__ import annotations

import json
import re
import sys
from pathlib import Path


class DebugParser:
    """Rust `{:?}` of the spec structs -> JSON-shaped Python values."""

    def __init__(self, text):
        self.s, self.i = text, 0

    def ws(self):
        while self.i < len(self.s) and self.s[self.i].isspace():
            self.i += 1

    def peek(self):
        self.ws()
        return self.s[self.i] if self.i < len(self.s) else ""

    def expect(self, ch):
        self.ws()
        assert self.s[self.i] == ch, (self.s, self.i, ch)
        self.i += 1

    def value(self):
        c = self.peek()
        if c == "[":
            self.i += 1
            out = []
            while self.peek() != "]":
                out.append(self.value())
                if self.peek() == ",":
                    self.i += 1
            self.i += 1
            return out
        if c == '"':
            j = self.s.index('"', self.i + 1)
            v = self.s[self.i + 1:j]
            self.i = j + 1
            return v
        m = re.compile(r"-?\d+(\.\d+)?([eE][-+]?\d+)?").match(self.s, self.i)
        if m:
            self.i = m.end()
            t = m.group(0)
            return float(t) if ("." in t or "e" in t or "E" in t) else int(t)
        m = re.compile(r"[A-Za-z_][A-Za-z_0-9]*").match(self.s, self.i)
        assert m, (self.s, self.i)
        name = m.group(0)
        self.i = m.end()
        if name in ("true", "false"):
            return name == "true"
        if name == "None":
            return None
        nxt = self.peek()
        if nxt == "{":       # struct: the name is not part of the wire form
            self.i += 1
            out = {}
            while self.peek() != "}":
                k = re.compile(r"[A-Za-z_][A-Za-z_0-9]*").match(self.s, self.i)
                self.i = k.end()
                self.expect(":")
                out[k.group(0)] = self.value()
                if self.peek() == ",":
                    self.i += 1
            self.i += 1
            return out
        if nxt == "(":       # tuple variant / newtype
            self.i += 1
            inner = self.value()
            self.expect(")")
            if name == "Some":
                return inner
            return {name: inner}
        return name          # unit variant


def parse_type(text):
    m = re.fullmatch(r"tensor<(\w+) x (.*)>", text.strip())
    assert m, text
    dims = [] if m.group(2).strip() == "[]" else [int(d) for d in m.group(2).split("x")]
    return {"Tensor": {"dtype": m.group(1), "shape": {"dims": [{"Static": d} for d in dims]}}}


def split_op(line):
    """`%3 = Name(Debug...)(%0, %1) -> type`  ->  (id, op json, operand ids, type json)"""
    m = re.match(r"\s*%(\d+) = (.*) -> (tensor<.*>)\s*$", line)
    assert m, line
    vid, rest, ty = int(m.group(1)), m.group(2).strip(), m.group(3)
    operands = []
    om = re.search(r"\(((?:%\d+(?:,\s*)?)*)\)$", rest)   # the trailing operand list, when there is one
    if om and (om.group(1) or rest[:om.start()].rstrip().endswith(")")):
        operands = [int(x) for x in re.findall(r"%(\d+)", om.group(1))]
        rest = rest[:om.start()]
    op = DebugParser(rest).value()
    if isinstance(op, dict) and "Constant" in op:   # TensorLiteral: the bytes stay a list of numbers
        pass
    return vid, op, operands, parse_type(ty)


def parse_program(text):
    head = re.search(r"program @(\w+) \(spec_version = ([\w.]+)\)", text)
    fn_name = re.search(r"func @(\w+)", text).group(1)
    fn = {"name": fn_name, "parameters": [], "parameter_ids": [], "results": [], "body": [], "hints": [], "result_ids": []}
    section = None
    for line in text.splitlines():
        t = line.strip()
        if t in ("params:", "body:", "results:"):
            section = t[:-1]
            continue
        if not t.startswith("%"):
            continue
        if section in ("params", "results"):
            m = re.match(r"%(\d+) : (tensor<.*>)", t)
            vid, ty = int(m.group(1)), parse_type(m.group(2))
            if section == "params":
                fn["parameters"].append(ty)
                fn["parameter_ids"].append(vid)
            else:
                fn["results"].append(ty)
                fn["result_ids"].append(vid)
        elif section == "body":
            vid, op, operands, ty = split_op(line)
            fn["body"].append({"id": vid, "op": op, "operands": [{"Value": o} for o in operands], "output": ty})
    return {"spec_version": head.group(2), "entry": head.group(1), "functions": [fn], "regions": []}


def main(root):
    fixtures = sorted((Path(root) / "crates" / "gpt-rs" / "tests" / "fixtures").glob("*.lit"))
    cases = []
    for path in fixtures:
        text = path.read_text()
        for n, block in enumerate(b for b in text.split("run_test") if "INPUT:" in b):
            expected = block.split("EXPECTED:")[1].split("INPUT:")[0]
            given = block.split("INPUT:")[1]
            cases.append({"name": f"{path.stem}.{n}", "source": f"crates/gpt-rs/tests/fixtures/{path.name}",
                          "input": parse_program(given), "expected": parse_program(expected)})
    out = Path(__file__).resolve().parent / "lit_programs.json"
    out.write_text(json.dumps(cases, indent=1) + "\n")
    print(f"{len(cases)} program pairs from {len(fixtures)} files -> {out}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_lit_fixtures.py <root of a gpt.rs source tree>")
    main(sys.argv[1])
