"""The five benchmark configurations: seeded synthetic inputs with the stated shapes and
value distributions, CUDA path against the CPU oracle. The 8192^3 case is checked on a
row sample by the oracle and, over the whole output, through row and column checksums
and through agreement of column-sharded launches with the single launch."""
import os

import numpy as np
import pytest
import torch

from niutensor_b200 import capi, ops
from niutensor_b200.capi import X_TRANS, X_NOTRANS
from oracle.oracle import rel_fro, round_to_half

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(x, dtype):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV).to(dtype)


def test_config1_fp32_512(oracle):
    rng = np.random.default_rng(1001)
    a = rng.uniform(-1, 1, (512, 512)).astype(np.float32)
    b = rng.uniform(-1, 1, (512, 512)).astype(np.float32)
    c = ops.MatrixMul(dev(a, torch.float32), X_NOTRANS, dev(b, torch.float32), X_NOTRANS, 1.0)
    assert capi.lib().ntb_last_route() == capi.ROUTE_TC_3XTF32
    assert rel_fro(c.cpu().numpy(), oracle.matmul2d(a, X_NOTRANS, b, X_NOTRANS)) <= 1e-5


def test_config2_ffn_fp16(oracle):
    rng = np.random.default_rng(1002)
    x = round_to_half(rng.normal(size=(4096, 512)))
    w1 = round_to_half(rng.normal(size=(512, 2048)) / np.sqrt(512.0))
    w2 = round_to_half(rng.normal(size=(2048, 512)) / np.sqrt(2048.0))
    h = ops.MMul(dev(x, torch.float16), dev(w1, torch.float16))
    assert capi.lib().ntb_last_route() in (capi.ROUTE_TC_F16, capi.ROUTE_TC_F16_PAIR)
    assert rel_fro(h.float().cpu().numpy(), oracle.matmul2d(x, X_NOTRANS, w1, X_NOTRANS)) <= 2e-3
    hh = h.float().cpu().numpy()              # second GEMM on the first one's fp16 output
    y = ops.MMul(h, dev(w2, torch.float16))
    assert rel_fro(y.float().cpu().numpy(), oracle.matmul2d(hh, X_NOTRANS, w2, X_NOTRANS)) <= 2e-3


def test_config3_attention_bmmul_fp16(oracle):
    rng = np.random.default_rng(1003)
    q = round_to_half(rng.normal(size=(64, 256, 64)))
    k = round_to_half(rng.normal(size=(64, 256, 64)))
    v = round_to_half(rng.normal(size=(64, 256, 64)))
    s = ops.BMMul(dev(q, torch.float16), X_NOTRANS, dev(k, torch.float16), X_TRANS, 0.125)
    assert capi.lib().ntb_last_route() in (capi.ROUTE_TC_F16, capi.ROUTE_TC_F16_PAIR)
    assert rel_fro(s.float().cpu().numpy(), oracle.matmul_batched(q, X_NOTRANS, k, X_TRANS, 0.125)) <= 2e-3
    logits = rng.normal(size=(64, 256, 256)).astype(np.float32)
    e = np.exp(logits - logits.max(-1, keepdims=True))
    p = round_to_half(e / e.sum(-1, keepdims=True))
    o = ops.BMMul(dev(p, torch.float16), X_NOTRANS, dev(v, torch.float16), X_NOTRANS)
    assert rel_fro(o.float().cpu().numpy(), oracle.matmul_batched(p, X_NOTRANS, v, X_NOTRANS)) <= 2e-3
    # the same through the 4-D [batch, heads, len, d] view the transformer uses
    s4 = ops.BMMul(dev(q, torch.float16).view(8, 8, 256, 64), X_NOTRANS,
                   dev(k, torch.float16).view(8, 8, 256, 64), X_TRANS, 0.125)
    assert torch.equal(s4.view(64, 256, 256), s)


def test_config4_output_layer_fp16(oracle):
    rng = np.random.default_rng(1004)
    h = round_to_half(rng.normal(size=(256, 512)))
    w = round_to_half(rng.normal(size=(65536, 512)) * 0.02)
    y = ops.MatrixMul(dev(h, torch.float16), X_NOTRANS, dev(w, torch.float16), X_TRANS)
    assert capi.lib().ntb_last_route() in (capi.ROUTE_TC_F16, capi.ROUTE_TC_F16_PAIR)
    assert rel_fro(y.float().cpu().numpy(), oracle.matmul2d(h, X_NOTRANS, w, X_TRANS)) <= 2e-3
    # vocabulary shards: rows [v0, v1) of w give columns [v0, v1) of the logits
    wd = dev(w, torch.float16)
    for g in (2, 8):
        parts = [ops.MatrixMul(dev(h, torch.float16), X_NOTRANS, wd[i * 65536 // g:(i + 1) * 65536 // g], X_TRANS)
                 for i in range(g)]
        assert torch.equal(torch.cat(parts, dim=1), y)


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 2e-3), (torch.float32, 1e-5)])
def test_config5_large_square(dtype, tol, oracle):
    n = 8192
    g = torch.Generator(device=DEV)
    g.manual_seed(1005)
    a = (torch.rand(n, n, device=DEV, generator=g) * 2 - 1).to(dtype)
    b = (torch.rand(n, n, device=DEV, generator=g) * 2 - 1).to(dtype)
    c0 = torch.randn(n, n, device=DEV, generator=g).to(dtype)
    c = c0.clone()
    ops.MatrixMul(a, X_NOTRANS, b, X_NOTRANS, 1.0, 0.5, c=c)
    # (1) oracle on a sample of rows spread over every row block
    rows = np.arange(0, n, 257)[:32]
    a_s = a[rows].float().cpu().numpy()
    want = oracle.matmul2d(a_s, X_NOTRANS, b.float().cpu().numpy(), X_NOTRANS, 1.0, 0.5,
                           c0[rows].float().cpu().numpy())
    assert rel_fro(c[rows].float().cpu().numpy(), want) <= tol
    # (2) checksums in both directions, in float64: C 1 = A (B 1) + 0.5 C0 1 and
    #     1^T C = (1^T A) B + 0.5 1^T C0 -- every output tile enters one row sum and one
    #     column sum; the sums average the output rounding, hence the tighter bound
    ad, bd, c0d, cd = a.double(), b.double(), c0.double(), c.double()
    row_want = ad @ bd.sum(1) + 0.5 * c0d.sum(1)
    col_want = ad.sum(0) @ bd + 0.5 * c0d.sum(0)
    sum_tol = 5e-4 if dtype == torch.float16 else 1e-5
    assert float((cd.sum(1) - row_want).norm() / row_want.norm()) <= sum_tol
    assert float((cd.sum(0) - col_want).norm() / col_want.norm()) <= sum_tol
    del ad, bd, c0d, cd
    # (3) column shards with a pitched B and C reproduce the full result bit for bit
    L = capi.lib()
    code = capi.X_FLOAT16 if dtype == torch.float16 else capi.X_FLOAT
    es = a.element_size()
    c2 = c0.clone()
    for i in range(4):
        off = i * (n // 4)
        rc = L.ntb_gemm(0, None, a.data_ptr(), X_NOTRANS, b.data_ptr() + off * es, X_NOTRANS,
                        c2.data_ptr() + off * es, code, code, n, n, n, n // 4, n, n // 4, n, n, n, 1.0, 0.5)
        assert rc == capi.OK
    assert torch.equal(c2, c)
    assert L.ntb_device_status(0) == capi.OK
