"""NiuTensor's own samples, unchanged, on top of the replacement library. The sources of
sample/fnnlm, the transformer sample, source/network and source/train are linked twice
(`make -C oracle dropin_samples`): against the reference's matrix-multiplication units,
i.e. cuBLAS, and against the shim over libntb_gemm.so. Each test runs the same sample entry
in two child processes, one per library, on the same seeded synthetic data, and compares
what the sample computes. The feed-forward language model trains with its hand-written
backward pass and with automatic differentiation (MatrixMul N/N, T/N, N/T, beta = 1
accumulation, XBackwardMath's gradient products); the transformer step covers MulAndShift,
BMMul and the output layer's MMul with a transposed weight on tensors that live in the
sample's XMem pools. Synthetic word indices stand in for the corpora."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBS = {"ref": os.path.join(ROOT, "oracle", "_ref", "libnts_samples_ref.so"),
        "dropin": os.path.join(ROOT, "oracle", "_ref", "libnts_samples_dropin.so")}

CHILD = r"""
import ctypes, json, sys
job = json.loads(sys.argv[1])
lib = ctypes.CDLL(job["lib"])
argv = [a.encode() for a in job["argv"]]
arr = (ctypes.c_char_p * len(argv))(*argv)
out = {}
if job["what"] == "fnnlm":
    out["rc"] = lib.nts_samples_fnnlm(len(argv), arr, job["seed"])
else:
    res = (ctypes.c_double * 4)()
    out["rc"] = lib.nts_samples_transformer_step(len(argv), arr, job["batch"], job["len_src"], job["len_tgt"], job["seed"], res)
    out["res"] = list(res)
if job["lib"].endswith("dropin.so"):
    g = ctypes.CDLL(job["gemm"])
    g.ntb_route_count.restype = ctypes.c_longlong
    out["routes"] = [g.ntb_route_count(r) for r in range(6)]
    out["status"] = g.ntb_device_status(0)
print("RESULT " + json.dumps(out))
"""


def _have_libs():
    return all(os.path.exists(p) for p in LIBS.values())


def _child(job):
    job["gemm"] = os.path.join(ROOT, "niutensor_b200", "libntb_gemm.so")
    r = subprocess.run([sys.executable, "-c", CHILD, json.dumps(job)], capture_output=True, text=True, timeout=600)
    lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
    assert r.returncode == 0 and lines, (r.returncode, r.stdout[-2000:], r.stderr[-2000:])
    return json.loads(lines[-1][7:])


def _write_corpus(path, rng, sentences, vocab):
    with open(path, "w") as f:
        for _ in range(sentences):
            n = int(rng.integers(8, 28))
            # a skewed unigram distribution with some local structure, so that training has something to learn
            words = np.minimum(rng.zipf(1.3, size=n), vocab - 1)
            words[1:] = (words[1:] + words[:-1]) % vocab
            f.write(" ".join(str(int(w)) for w in words) + "\n")


def _floats_of(path):
    vals = []
    for line in open(path):
        parts = line.split("|||")
        if len(parts) == 3:
            vals.extend(float(x) for x in parts[1].split() if x != "<s>")
            vals.append(float(parts[2]))
    return np.array(vals)


@pytest.mark.skipif(not _have_libs(), reason="sample libraries not built (make -C oracle dropin_samples needs the NiuTensor sources)")
@pytest.mark.parametrize("autodiff", [False, True])
def test_fnnlm_trains_to_the_same_model(autodiff, tmp_path):
    rng = np.random.default_rng(11)
    vocab = 2000
    train, test = str(tmp_path / "train.txt"), str(tmp_path / "test.txt")
    _write_corpus(train, rng, 600, vocab)
    _write_corpus(test, rng, 40, vocab)
    outs = {}
    for name, lib in LIBS.items():
        out = str(tmp_path / ("probs_%s.txt" % name))
        argv = ["fnnlm", "-train", train, "-test", test, "-output", out, "-model", str(tmp_path / ("model_%s.txt" % name)),
                "-n", "4", "-esize", "96", "-vsize", str(vocab), "-hdepth", "2", "-hsize", "160",
                # the hand-written pass sums the loss over a batch, the automatic one averages it
                "-lrate", "0.05" if autodiff else "0.002",
                "-nstep", "80", "-nepoch", "1", "-wbatch", "192", "-dev", "0"] + (["-autodiff"] if autodiff else [])
        res = _child({"what": "fnnlm", "lib": lib, "argv": argv, "seed": 7})
        assert res["rc"] == 0
        outs[name] = (_floats_of(out), res)
    ref, got = outs["ref"][0], outs["dropin"][0]
    assert ref.size > 500 and ref.shape == got.shape
    assert np.all(np.isfinite(got))
    assert np.median(got) > -15.0                   # a trained model, not the -20 floor of a diverged one
    # word log-probabilities after the updates: the two builds went through the same arithmetic up to
    # the rounding of the products (fp32: cuBLAS FFMA vs three-pass TF32 / FFMA here)
    assert np.max(np.abs(got - ref) / np.maximum(1.0, np.abs(ref))) <= 2e-4
    routes = outs["dropin"][1]["routes"]
    assert outs["dropin"][1]["status"] == 0
    assert sum(routes[1:]) > 300                    # every product of the run went through this library
    print("fnnlm autodiff=%s routes (none, f16, 3xtf32, simt, pair, f16x2): %s" % (autodiff, routes))


@pytest.mark.skipif(not _have_libs(), reason="sample libraries not built (make -C oracle dropin_samples needs the NiuTensor sources)")
def test_transformer_training_step_matches(tmp_path):
    vocab = 640
    header = str(tmp_path / "train.bin")
    np.array([vocab, vocab, 1, 2, 2, 3], dtype=np.int32).tofile(header)      # vocabulary sizes, pad, sos, eos, unk
    argv = ["nmt", "-dev", "0", "-train", header, "-model", str(tmp_path / "no-such-model.bin"),
            "-enclayer", "2", "-declayer", "2", "-encemb", "128", "-decemb", "128", "-encffn", "256", "-decffn", "256",
            "-encheads", "4", "-decheads", "4", "-encdecheads", "4", "-dropout", "0", "-ffndropout", "0",
            "-attdropout", "0", "-labelsmoothing", "0.1"]
    res = {name: _child({"what": "nmt", "lib": lib, "argv": argv, "batch": 6, "len_src": 23, "len_tgt": 19, "seed": 5})
           for name, lib in LIBS.items()}
    ref, got = res["ref"]["res"], res["dropin"]["res"]
    assert res["ref"]["rc"] == 0 and res["dropin"]["rc"] == 0
    assert np.isfinite(got).all() and got[3] == ref[3] and got[3] > 20         # same number of parameters with gradients
    for i, what in enumerate(("loss", "sum of output probabilities", "gradient norm")):
        assert abs(got[i] - ref[i]) <= 1e-4 * max(1.0, abs(ref[i])), (what, got[i], ref[i])
    assert res["dropin"]["status"] == 0
    routes = res["dropin"]["routes"]
    assert sum(routes[1:]) > 50
    print("transformer step routes (none, f16, 3xtf32, simt, pair, f16x2): %s" % routes)
