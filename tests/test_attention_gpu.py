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
from tests.golden.cases import attention_cases, attention_cases_wide

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
    rc = L.ntb_attention(0, None, q.data_ptr(), k.data_ptr(), v.data_ptr(), None, q.data_ptr(),
                         capi.X_FLOAT16, 1, 4, 6, 96, 0, 0.125)
    assert rc == capi.ERR_LIMIT                    # head sizes other than 64 and 128
    rc = L.ntb_attention(0, None, q.data_ptr(), k.data_ptr(), v.data_ptr(), None, q.data_ptr(),
                         capi.X_FLOAT, 1, 4, 6, 64, 0, 0.125)
    assert rc == capi.ERR_DTYPE


def test_head_128_long_keys_and_dropout_against_the_reference_chain(oracle):
    """The transformer sample's default head size (128), key sequences beyond one 256-key
    step (scores computed twice: maxima, then sums and the second product) and dropout with
    a given keep-mask, against the stored outputs of the reference's CPU operator chain."""
    z = np.load(os.path.join(GOLD, "ref_attention_wide.npz"))
    for i, (q, k, v, mask, scale, keep, keep_scale) in enumerate(attention_cases_wide()):
        q, k, v = round_to_half(q), round_to_half(k), round_to_half(v)
        want = oracle.attention(q, k, v, mask, scale) if keep is None else \
            oracle.attention_dropout(q, k, v, keep, keep_scale, mask, scale)
        m = None if mask is None else dev(mask, torch.float32)
        kp = None if keep is None else torch.from_numpy(keep).to(DEV)
        out = ops.ScaledDotProductAttention(dev(q, torch.float16), dev(k, torch.float16), dev(v, torch.float16), m, scale,
                                            kp, 0.0 if keep is None else 1.0 - 1.0 / keep_scale)
        got = out.float().cpu().numpy()
        assert rel_fro(got, want) <= 2e-3, (i, rel_fro(got, want))
        # the stored fixture was computed from the unrounded fp32 inputs: half inputs add their own rounding
        assert rel_fro(got, z["o%d" % i]) <= 5e-3, i
    assert capi.lib().ntb_device_status(0) == capi.OK


def test_long_keys_equal_the_composition_of_library_products():
    rng = np.random.default_rng(1009)
    heads, batch, lenq, lenk, d = 4, 3, 200, 777, 128
    q = dev(rng.normal(size=(heads, batch, lenq, d)), torch.float16)
    k = dev(rng.normal(size=(heads, batch, lenk, d)), torch.float16)
    v = dev(rng.normal(size=(heads, batch, lenk, d)), torch.float16)
    out = ops.ScaledDotProductAttention(q, k, v)
    s = ops.BMMul(q, X_NOTRANS, k, X_TRANS, 1.0 / d ** 0.5)
    p = torch.softmax(s.float(), dim=-1).half()
    o2 = ops.BMMul(p, X_NOTRANS, v, X_NOTRANS)
    assert rel_fro(out.float().cpu().numpy(), o2.float().cpu().numpy()) <= 2e-3
    assert capi.lib().ntb_device_status(0) == capi.OK
