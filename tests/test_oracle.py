"""Pins the CPU oracle (oracle/matmul_oracle.c): against the known-answer vectors of
the reference's own unit tests, against outputs of the compiled reference stored under
tests/golden/, and -- where the compiled reference is present -- bit for bit against
the reference library on fresh seeded inputs."""
import json
import os

import numpy as np
import pytest

from oracle.oracle import (Oracle, Reference, ref_available, rel_fro, X_TRANS, X_NOTRANS)
from tests.golden.cases import (seeded_cases, mulandshift_cases, attention_cases, attention_cases_wide, output_layer_cases, FORM_GENERAL, FORM_BATCHED,
                                FORM_2D)

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def is_float_equal(a, b, tol):
    """The reference's comparator (source/tensor/core/utilities/CheckData.cpp:29-39):
    absolute error below tol, or relative error below tol."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    err = np.abs(a - b)
    rel = err / np.maximum(np.abs(b), 1e-300)
    return bool(np.all((err < tol) | (rel < tol)))


def run_form(o, op_or_form, a, tA, b, tB, alpha, beta, c0):
    if op_or_form in ("_MatrixMul", FORM_GENERAL):
        return o.matmul(a, tA, b, tB, alpha, beta, c0)
    if op_or_form in ("_MatrixMulBatched", FORM_BATCHED):
        return o.matmul_batched(a, tA, b, tB, alpha, beta, c0)
    return o.matmul2d(a, tA, b, tB, alpha, beta, c0)


def kat_cases():
    with open(os.path.join(GOLD, "ref_kat.json")) as f:
        return json.load(f)["cases"]


@pytest.mark.parametrize("case", kat_cases(), ids=lambda c: c["name"])
def test_oracle_matches_reference_unit_test_vectors(oracle, case):
    a = np.asarray(case["a"], np.float32).reshape(case["a_shape"])
    b = np.asarray(case["b"], np.float32).reshape(case["b_shape"])
    want = np.asarray(case["answer"], np.float32).reshape(case["c_shape"])
    got = run_form(oracle, case["op"], a, case["transA"], b, case["transB"],
                   case["alpha"], case["beta"], None)
    assert got.shape == want.shape
    assert is_float_equal(got, want, case["tolerance"])


def test_oracle_matches_stored_reference_outputs_bit_for_bit(oracle):
    z = np.load(os.path.join(GOLD, "ref_seeded.npz"))
    meta = json.loads(bytes(z["meta"]).decode())
    cases = seeded_cases()
    assert len(cases) == len(meta) == 80
    for i, (kind, form, a, tA, b, tB, alpha, beta, c0) in enumerate(cases):
        m = meta[i]
        assert (m["kind"], m["transA"], m["transB"]) == (kind, tA, tB)
        got = run_form(oracle, form, a, tA, b, tB, alpha, beta, c0)
        want = z["c%d" % i]
        assert got.shape == want.shape
        assert np.array_equal(got, want), "case %d %s" % (i, m)


def test_mulandshift_oracle_matches_stored_reference_outputs_bit_for_bit(oracle):
    z = np.load(os.path.join(GOLD, "ref_mulandshift.npz"))
    cases = mulandshift_cases()
    assert len(cases) == len(z.files) == 6
    for i, (x, w, b, alpha, tX, tW) in enumerate(cases):
        got = oracle.mulandshift(x, w, b, alpha, tX, tW)
        assert got.shape == z["y%d" % i].shape
        assert np.array_equal(got, z["y%d" % i]), i
    x, w, b = cases[1][:3]
    r = oracle.mulandshift(x, w, b, rectify=True)
    assert np.array_equal(r, np.maximum(oracle.mulandshift(x, w, b), 0))


def test_attention_oracle_matches_stored_reference_outputs(oracle):
    """Pinned at 1e-6: the reference's row sums run in vector lanes, the oracle's left to right."""
    z = np.load(os.path.join(GOLD, "ref_attention.npz"))
    cases = attention_cases()
    assert len(cases) == len(z.files) == 5
    for i, (q, k, v, mask, scale) in enumerate(cases):
        got = oracle.attention(q, k, v, mask, scale)
        assert got.shape == z["o%d" % i].shape
        assert rel_fro(got, z["o%d" % i]) <= 1e-6, i


def test_attention_oracle_head_128_long_keys_and_dropout(oracle):
    z = np.load(os.path.join(GOLD, "ref_attention_wide.npz"))
    cases = attention_cases_wide()
    assert len(cases) == len(z.files) == 6
    for i, (q, k, v, mask, scale, keep, keep_scale) in enumerate(cases):
        got = oracle.attention(q, k, v, mask, scale) if keep is None else \
            oracle.attention_dropout(q, k, v, keep, keep_scale, mask, scale)
        assert got.shape == z["o%d" % i].shape
        assert rel_fro(got, z["o%d" % i]) <= 1e-6, i


def test_output_layer_oracle_matches_stored_reference_outputs(oracle):
    z = np.load(os.path.join(GOLD, "ref_output_layer.npz"))
    cases = output_layer_cases()
    assert len(cases) == len(z.files) == 4
    for i, (h, w) in enumerate(cases):
        got = oracle.output_layer(h, w)
        want = z["y%d" % i]
        assert got.shape == want.shape
        assert rel_fro(got, want) <= 1e-6, i
        assert got.min() >= -20.0
    assert (z["y2"] == -20.0).any(), "the floor case must reach the floor"


def test_thread_count_does_not_change_bits():
    o = Oracle()
    rng = np.random.default_rng(5)
    a = rng.uniform(-1, 1, (70, 45)).astype(np.float32)
    b = rng.uniform(-1, 1, (45, 31)).astype(np.float32)
    o.set_threads(1)
    x = o.matmul2d(a, X_NOTRANS, b, X_NOTRANS, 0.3, 0.0)
    o.set_threads(7)
    y = o.matmul2d(a, X_NOTRANS, b, X_NOTRANS, 0.3, 0.0)
    assert np.array_equal(x, y)


@pytest.mark.skipif(not ref_available("builtin"), reason="compiled reference not present")
def test_oracle_equals_compiled_reference_on_fresh_inputs(oracle):
    ref = Reference("builtin")
    rng = np.random.default_rng(77)
    for tA in (X_TRANS, X_NOTRANS):
        for tB in (X_TRANS, X_NOTRANS):
            for alpha, beta in ((1.0, 0.0), (0.5, 0.0), (1.0, 1.0), (2.0, -0.5)):
                M, N, K = rng.integers(1, 90, 3)
                a = rng.uniform(-1, 1, (K, M) if tA == X_TRANS else (M, K)).astype(np.float32)
                b = rng.uniform(-1, 1, (N, K) if tB == X_TRANS else (K, N)).astype(np.float32)
                c0 = rng.normal(size=(M, N)).astype(np.float32)
                assert np.array_equal(oracle.matmul2d(a, tA, b, tB, alpha, beta, c0),
                                      ref.run(FORM_2D, a, tA, b, tB, alpha, beta, c0))


@pytest.mark.skipif(not ref_available("openblas"), reason="OpenBLAS build of the reference not present")
def test_reference_openblas_build_agrees_except_tt(oracle):
    ref = Reference("openblas")
    rng = np.random.default_rng(78)
    for tA, tB in ((X_NOTRANS, X_NOTRANS), (X_TRANS, X_NOTRANS), (X_NOTRANS, X_TRANS)):
        M, N, K = 96, 80, 112
        a = rng.uniform(-1, 1, (K, M) if tA == X_TRANS else (M, K)).astype(np.float32)
        b = rng.uniform(-1, 1, (N, K) if tB == X_TRANS else (K, N)).astype(np.float32)
        got = ref.run(FORM_2D, a, tA, b, tB, 1.0, 0.0)
        assert rel_fro(got, oracle.matmul2d(a, tA, b, tB)) < 1e-6
