"""Fused scaled-dot-product attention against the CPU oracle (the reference's fp32 operator
chain on fp16-valued inputs; tolerance 2e-3 as for every half-precision result) and against
the same computation composed from this library's own BMMul calls."""
import os

import numpy as np
import pytest
import torch

from niutensor_b200 import capi, ops
from niutensor_b200.capi import X_TRANS, X_NOTRANS
from oracle.oracle import rel_fro, round_to_half
from tests.golden.cases import attention_cases

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def dev(x, dtype):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV).to(dtype)


def test_against_reference_chain_fixtures(oracle):
    for i, (q, k, v, mask, scale) in enumerate(attention_cases()):
        q, k, v = round_to_half(q), round_to_half(k), round_to_half(v)
        want = oracle.attention(q, k, v, mask, scale)
        m = None if mask is None else dev(mask, torch.float32)
        out = ops.ScaledDotProductAttention(dev(q, torch.float16), dev(k, torch.float16), dev(v, torch.float16), m, scale)
        assert tuple(out.shape) == want.shape
        assert rel_fro(out.float().cpu().numpy(), want) <= 2e-3, i
    assert capi.lib().ntb_device_status(0) == capi.OK


def test_benchmark_attention_shapes_heads_by_batch(oracle):
    """8 heads x 8 sentences, length 256, head size 64; more blocks than SMs further down."""
    rng = np.random.default_rng(1003)
    for heads, batch, length in ((8, 8, 256), (8, 40, 96)):
        q = round_to_half(rng.normal(size=(heads, batch, length, 64)))
        k = round_to_half(rng.normal(size=(heads, batch, length, 64)))
        v = round_to_half(rng.normal(size=(heads, batch, length, 64)))
        out = ops.ScaledDotProductAttention(dev(q, torch.float16), dev(k, torch.float16), dev(v, torch.float16))
        want = oracle.attention(q.reshape(-1, length, 64), k.reshape(-1, length, 64), v.reshape(-1, length, 64),
                                None, 0.125).reshape(q.shape)
        assert rel_fro(out.float().cpu().numpy(), want) <= 2e-3
        # composed from the library's own products, softmax done by torch in fp32
        tq, tk, tv = dev(q, torch.float16), dev(k, torch.float16), dev(v, torch.float16)
        s = ops.BMMul(tq, X_NOTRANS, tk, X_TRANS, 0.125)
        p = torch.softmax(s.float(), dim=-1).half()
        o2 = ops.BMMul(p, X_NOTRANS, tv, X_NOTRANS)
        assert rel_fro(out.float().cpu().numpy(), o2.float().cpu().numpy()) <= 2e-3
    assert capi.lib().ntb_device_status(0) == capi.OK


def test_fully_masked_row_gives_zeros_and_limits_are_reported():
    q = torch.randn(1, 4, 64, device=DEV).half()
    k = torch.randn(1, 6, 64, device=DEV).half()
    v = torch.randn(1, 6, 64, device=DEV).half()
    mask = torch.zeros(4, 6, device=DEV)
    mask[2, :] = float("-inf")
    out = ops.ScaledDotProductAttention(q, k, v, mask)
    assert torch.equal(out[0, 2], torch.zeros(64, device=DEV, dtype=torch.float16))
    assert torch.isfinite(out).all()
    L = capi.lib()
    big = torch.zeros(1, 300, 64, device=DEV).half()
    rc = L.ntb_attention(0, None, q.data_ptr(), big.data_ptr(), big.data_ptr(), None, q.data_ptr(),
                         capi.X_FLOAT16, 1, 4, 300, 64, 0, 0.125)
    assert rc == capi.ERR_LIMIT
    rc = L.ntb_attention(0, None, q.data_ptr(), k.data_ptr(), v.data_ptr(), None, q.data_ptr(),
                         capi.X_FLOAT16, 1, 4, 6, 128, 0, 0.125)
    assert rc == capi.ERR_LIMIT
    rc = L.ntb_attention(0, None, q.data_ptr(), k.data_ptr(), v.data_ptr(), None, q.data_ptr(),
                         capi.X_FLOAT, 1, 4, 6, 64, 0, 0.125)
    assert rc == capi.ERR_DTYPE
