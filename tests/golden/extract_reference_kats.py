#!/usr/bin/env python3
"""Extract the known-answer vectors held by the reference's own unit tests.

Reads the gtest sources under <reference>/test/cuBERT (as text; nothing is compiled
or run) and writes tests/golden/reference_kats.json:

    { "<file>::<test name>": {
          "arrays": {name: [numbers...]},          # every initialised array in the test
          "expect": [[array, index, value, tol|null]] # EXPECT_NEAR / EXPECT_FLOAT_EQ on array[index]
      }, ...,
      "<file>::<globals>": {"arrays": {...}}       # file-scope arrays (TransformerTest weights)
    }

The reference tree is only present in the build container, so the JSON is committed
and the tests read the JSON, never the reference.

Usage: python tests/golden/extract_reference_kats.py [<reference checkout>]
"""
import json
import math
import os
import re
import sys

FILES = [
    "op/EmbeddingTest.cpp",
    "op/LayerNormTest.cpp",
    "op/SoftmaxTest.cpp",
    "op/GELUTest.cpp",
    "op/DenseTest.cpp",
    "op_att/AttentionMaskTest.cpp",
    "op_att/BatchMatMulTest.cpp",
    "op_att/AttentionSelfTest.cpp",
    "op_att/TransformerTest.cpp",
    "op_bert/BertEmbeddingsTest.cpp",
    "op_bert/BertPoolerTest.cpp",
    "op_out/AdditionalOutputLayerTest.cpp",
]

ARRAY_RE = re.compile(
    r"\b(?:float|double|int|int8_t|size_t)\s+(\w+)\s*\[\s*\d*\s*\]\s*=\s*\{(.*?)\}\s*;", re.S)
EXPECT_RE = re.compile(
    r"EXPECT_(NEAR|FLOAT_EQ)\s*\(\s*(\w+)\[(\d+)\]\s*,\s*(.*?)\)\s*;")
TEST_RE = re.compile(r"TEST_F\s*\(\s*CommonTest\s*,\s*(\w+)\s*\)")


def _number(tok):
    tok = tok.strip()
    tok = re.sub(r"(?<=[0-9.])f$", "", tok)
    return float(tok)


def _eval_expr(expr):
    """Evaluate the small C++ expressions used as expected values."""
    e = expr.strip()
    e = e.replace("std::sqrt", "math.sqrt").replace("tanhf", "math.tanh")
    e = re.sub(r"(\d+\.?\d*)f\b", r"\1", e)
    return float(eval(e, {"math": math, "__builtins__": {}}))


def _split_top_level(args):
    """Split 'a, b' at the last top-level comma (value, tolerance)."""
    depth = 0
    for i in range(len(args) - 1, -1, -1):
        c = args[i]
        if c == ")":
            depth += 1
        elif c == "(":
            depth -= 1
        elif c == "," and depth == 0:
            return args[:i], args[i + 1:]
    return args, None


def parse_block(text):
    arrays = {}
    for m in ARRAY_RE.finditer(text):
        body = re.sub(r"//[^\n]*", "", m.group(2))
        toks = [t for t in body.replace("\n", " ").split(",") if t.strip()]
        try:
            arrays[m.group(1)] = [_number(t) for t in toks]
        except ValueError:
            continue
    expect = []
    for m in EXPECT_RE.finditer(text):
        kind, name, idx, rest = m.group(1), m.group(2), int(m.group(3)), m.group(4)
        try:
            if kind == "NEAR":
                val, tol = _split_top_level(rest)
                expect.append([name, idx, _eval_expr(val), _eval_expr(tol)])
            else:
                expect.append([name, idx, _eval_expr(rest), None])
        except NameError:
            # value computed at run time by the test (GELUTest): restated by the caller
            continue
    return arrays, expect


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.sep, "root", "reference")
    root = os.path.join(ref, "test", "cuBERT")
    out = {}
    for rel in FILES:
        with open(os.path.join(root, rel)) as f:
            src = f.read()
        marks = [(m.start(), m.group(1)) for m in TEST_RE.finditer(src)]
        head = src[:marks[0][0]] if marks else src
        g_arrays, _ = parse_block(head)
        if g_arrays:
            out[rel + "::<globals>"] = {"arrays": g_arrays}
        for i, (pos, name) in enumerate(marks):
            end = marks[i + 1][0] if i + 1 < len(marks) else len(src)
            arrays, expect = parse_block(src[pos:end])
            # GELUTest computes its expectation in a loop from double erf: restate it.
            if rel == "op/GELUTest.cpp":
                xs = arrays["inout"]
                expect = [["inout", j, x * 0.5 * (1.0 + math.erf(x / math.sqrt(2.0))), 1e-5]
                          for j, x in enumerate(xs)]
            out[rel + "::" + name] = {"arrays": arrays, "expect": expect}
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_kats.json")
    with open(dst, "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print("wrote", dst, "with", len(out), "entries")


if __name__ == "__main__":
    main()
