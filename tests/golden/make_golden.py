"""Regenerates the golden fixtures of this folder. Needs the NiuTensor sources
(their folder in the environment variable REF) and the compiled reference CPU library
(`make -C oracle ref`); the fixtures themselves are committed so the tests run
without either.

  ref_kat.json     the literal input/answer arrays of the reference's own unit tests
                   for this path, read as text from source/tensor/test/TMatrixMul.cpp,
                   TMatrixMul2D.cpp, TMatrixMul2DParallel.cpp, TMatrixMulBatched.cpp
                   (one entry per `bool TestXxxN()` function; both the `_Op` and the
                   user-level call of a case share the arrays).
  ref_seeded.npz   outputs of the reference library itself (built-in fp32 CPU path,
                   through oracle/ref_driver.cpp) on the seeded inputs that
                   tests/golden/cases.py regenerates: all four transposition
                   combinations x alpha/beta pairs x 2-D / batched / broadcast /
                   flatten forms, ragged sizes included. Only the outputs are stored.

  ref_mulandshift.npz  outputs of the reference's user-level MulAndShift (CPU) on the
                   seeded inputs of tests/golden/cases.py::mulandshift_cases.

  ref_attention.npz  outputs of the reference's CPU operator chain for inference-time
                   attention (scale, BMMul, Sum(mask), Softmax, BMMul) on the seeded inputs
                   of tests/golden/cases.py::attention_cases; ref_attention_wide.npz: the same
                   chain for head size 128, long key sequences and dropout with a given mask
                   (attention_cases_wide).

  ref_output_layer.npz  outputs of the reference's CPU MMul(h, w^T) + LogSoftmax on
                   tests/golden/cases.py::output_layer_cases.

Usage: python tests/golden/make_golden.py
"""
import json
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = os.environ.get("REF") or os.path.join(os.path.dirname(ROOT), "reference")

from oracle.oracle import Reference, ref_mulandshift, ref_attention, ref_output_layer, X_TRANS, X_NOTRANS  # noqa: E402
from tests.golden.cases import (seeded_cases, mulandshift_cases, attention_cases, attention_cases_wide,  # noqa: E402
                                output_layer_cases)

TEST_FILES = ["TMatrixMul.cpp", "TMatrixMul2D.cpp", "TMatrixMul2DParallel.cpp",
              "TMatrixMulBatched.cpp"]
FLAG = {"X_TRANS": X_TRANS, "X_NOTRANS": X_NOTRANS}


def parse_array(text, name):
    m = re.search(r"DTYPE\s+%s((?:\[\d+\])+)\s*=\s*(\{.*?\});" % name, text, re.S)
    dims = [int(x) for x in re.findall(r"\[(\d+)\]", m.group(1))]
    vals = [float(x.rstrip("Ff")) for x in
            re.findall(r"-?\d+\.?\d*(?:[eE][-+]?\d+)?[Ff]?", m.group(2))]
    assert len(vals) == int(np.prod(dims)), (name, dims, len(vals))
    return dims, vals


def parse_file(fn):
    text = open(os.path.join(REF, "source", "tensor", "test", fn)).read()
    # split into the bodies of the `bool TestXxxN()` case functions
    parts = re.split(r"\nbool (Test\w+\d+)\(\)\s*\n\{", text)
    cases = []
    for name, body in zip(parts[1::2], parts[2::2]):
        call = re.search(r"_(MatrixMul\w*)\(\s*s1\s*,\s*(X_\w+)\s*,\s*s2\s*,\s*(X_\w+)\s*,\s*t\s*\)",
                         body)
        ad, av = parse_array(body, "sData1")
        bd, bv = parse_array(body, "sData2")
        cd, cv = parse_array(body, "answer")
        line = text[:text.index("bool %s()" % name)].count("\n") + 1
        cases.append({"source": "source/tensor/test/%s:%d" % (fn, line), "name": name,
                      "op": "_" + call.group(1), "transA": FLAG[call.group(2)],
                      "transB": FLAG[call.group(3)], "alpha": 1.0, "beta": 0.0,
                      "a_shape": ad, "a": av, "b_shape": bd, "b": bv,
                      "c_shape": cd, "answer": cv, "tolerance": 1e-4})
    return cases


def main():
    kat = []
    for fn in TEST_FILES:
        kat += parse_file(fn)
    with open(os.path.join(HERE, "ref_kat.json"), "w") as f:
        json.dump({"generator": "tests/golden/make_golden.py", "cases": kat}, f, indent=1)
    print("ref_kat.json: %d cases" % len(kat))

    ref = Reference("builtin")
    arrays = {}
    meta = []
    for i, (key, form, a, tA, b, tB, alpha, beta, c0) in enumerate(seeded_cases()):
        c = ref.run(form, a, tA, b, tB, alpha, beta, c0)
        arrays["c%d" % i] = c
        meta.append({"kind": key, "form": form, "transA": tA, "transB": tB,
                     "alpha": alpha, "beta": beta})
    arrays["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "ref_seeded.npz"), **arrays)
    print("ref_seeded.npz: %d cases" % len(meta))

    arrays = {}
    for i, (x, w, b, alpha, tX, tW) in enumerate(mulandshift_cases()):
        arrays["y%d" % i] = ref_mulandshift(ref, x, w, b, alpha, tX, tW)
    np.savez_compressed(os.path.join(HERE, "ref_mulandshift.npz"), **arrays)
    print("ref_mulandshift.npz: %d cases" % len(arrays))

    arrays = {}
    for i, (q, k, v, mask, scale) in enumerate(attention_cases()):
        arrays["o%d" % i] = ref_attention(ref, q, k, v, mask, scale)
    np.savez_compressed(os.path.join(HERE, "ref_attention.npz"), **arrays)
    print("ref_attention.npz: %d cases" % len(arrays))

    arrays = {}
    for i, (q, k, v, mask, scale, keep, keep_scale) in enumerate(attention_cases_wide()):
        arrays["o%d" % i] = ref_attention(ref, q, k, v, mask, scale, keep, keep_scale)
    np.savez_compressed(os.path.join(HERE, "ref_attention_wide.npz"), **arrays)
    print("ref_attention_wide.npz: %d cases" % len(arrays))

    arrays = {}
    for i, (h, w) in enumerate(output_layer_cases()):
        arrays["y%d" % i] = ref_output_layer(ref, h, w)
    np.savez_compressed(os.path.join(HERE, "ref_output_layer.npz"), **arrays)
    print("ref_output_layer.npz: %d cases" % len(arrays))


if __name__ == "__main__":
    main()
