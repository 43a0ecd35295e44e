"""Host-side mirror of NiuTensor's matrix-multiplication operators over torch CUDA
tensors. torch supplies device memory and streams only; every product is computed by the
library behind include/ntb_gemm.h.

Names, argument meaning and shape rules follow the reference:
  _MatrixMul         source/tensor/core/arithmetic/MatrixMul.cpp:52-208
  _MatrixMul2D       source/tensor/core/arithmetic/MatrixMul2D.cpp:46-181
  _MatrixMulBatched  source/tensor/core/arithmetic/MatrixMulBatched.cpp:49-138
  MatrixMul          source/tensor/core/arithmetic/MatrixMul.cpp:272-361
  MatrixMulBatched   source/tensor/core/arithmetic/MatrixMulBatched.cpp:291-390 (= BMMul)
  MulAndShift        source/tensor/core/arithmetic/MulAndShift.cpp:38-110, 120-188
Transposition flags are the reference's enum values: X_TRANS = 0, X_NOTRANS = 1.
Where the reference prints an error and terminates, these raise NtError.
"""
import ctypes

import torch

from . import capi
from .capi import X_TRANS, X_NOTRANS, X_FLOAT, X_FLOAT16


class NtError(RuntimeError):
    """The reference's CheckNTErrors / ShowNTErrors (source/tensor/XGlobal.h:78-102)."""


def _check(cond, msg):
    if not cond:
        raise NtError(msg)


def _dtype_code(t):
    if t.dtype == torch.float32:
        return X_FLOAT
    if t.dtype == torch.float16:
        return X_FLOAT16
    raise NtError("Unsupported data type!")


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _common_checks(a, b, c):
    _check(a is not None and b is not None and c is not None, "Empty input tensors!")
    _check(a.is_cuda and b.is_cuda and c.is_cuda,
           "this library has no CPU path: tensors must live on a CUDA device")
    _check(a.device == b.device == c.device, "The code must be run on the same GPU!")
    _check(a.is_contiguous() and b.is_contiguous() and c.is_contiguous(),
           "tensors must be dense and packed")
    _check(a.dtype == b.dtype, "Input tensors should have the same data type!")
    _dtype_code(a)
    _check(c.dtype == a.dtype or (a.dtype == torch.float16 and c.dtype == torch.float32),
           "Input tensors should have the same data type!")


def _raise_rc(rc, what):
    if rc != capi.OK:
        raise NtError("%s: %s" % (what, capi.strerror(rc)))


def _MatrixMul2D(a, transposedA, b, transposedB, c, alpha=1.0, beta=0.0):
    _common_checks(a, b, c)
    _check(a.dim() == 2 and b.dim() == 2 and c.dim() == 2, "Input tensors must have a order = 2!")
    an, am = (a.shape[1], a.shape[0]) if transposedA == X_TRANS else (a.shape[0], a.shape[1])
    bn, bm = (b.shape[1], b.shape[0]) if transposedB == X_TRANS else (b.shape[0], b.shape[1])
    _check(am == bn and an == c.shape[0] and bm == c.shape[1], "Unmatched tensors in multiplication!")
    rc = capi.lib().ntb_gemm(a.device.index, _stream(a), a.data_ptr(), transposedA, b.data_ptr(), transposedB,
                             c.data_ptr(), _dtype_code(a), _dtype_code(c),
                             a.shape[0], a.shape[1], b.shape[0], b.shape[1], c.shape[0], c.shape[1],
                             a.shape[1], b.shape[1], c.shape[1], alpha, beta)
    _raise_rc(rc, "_MatrixMul2D")


def _MatrixMul(a, transposedA, b, transposedB, c, alpha=1.0, beta=0.0):
    _common_checks(a, b, c)
    _check(a.dim() >= 2 and b.dim() >= 2 and c.dim() >= 2, "Input tensors must have a order >= 2!")
    _check(c.dim() == a.dim() + b.dim() - 2, "wrong tensor order")
    if transposedA == X_NOTRANS and a.dim() > 2 and b.dim() == 2:
        # the reference folds the leading extents of a and c into rows (MatrixMul.cpp:65-77)
        _MatrixMul2D(a.view(-1, a.shape[-1]), transposedA, b, transposedB,
                     c.view(-1, c.shape[-1]), alpha, beta)
        return
    na, ma = a.shape[-2], a.shape[-1]
    nb, mb = b.shape[-2], b.shape[-1]
    nc, mc = c.shape[-2], c.shape[-1]
    an, am = (ma, na) if transposedA == X_TRANS else (na, ma)
    bn, bm = (mb, nb) if transposedB == X_TRANS else (nb, mb)
    _check(am == bn and an == nc and bm == mc, "Unmatched tensors in multiplication!")
    a_lead, b_lead = tuple(a.shape[:-2]), tuple(b.shape[:-2])
    _check(tuple(c.shape[:len(a_lead)]) == a_lead, "Incorrect tensor sizes!")
    _check(tuple(c.shape[len(a_lead):-2]) == b_lead, "Incorrect tensor sizes!")
    P = 1
    for d in a_lead:
        P *= d
    Q = 1
    for d in b_lead:
        Q *= d
    rc = capi.lib().ntb_gemm_broadcast(a.device.index, _stream(a), a.data_ptr(), transposedA,
                                       b.data_ptr(), transposedB, c.data_ptr(),
                                       _dtype_code(a), _dtype_code(c), na, ma, nb, mb, nc, mc,
                                       P, Q, alpha, beta)
    _raise_rc(rc, "_MatrixMul")


def _MatrixMulBatched(a, transposedA, b, transposedB, c, alpha=1.0, beta=0.0):
    _common_checks(a, b, c)
    _check(a.dim() >= 2 and b.dim() >= 2 and c.dim() >= 2, "Input tensors must have a order >= 2!")
    _check(a.dim() == b.dim() and a.dim() == c.dim(), "Input tensor and output tensor must have same order!")
    na, ma = a.shape[-2], a.shape[-1]
    nb, mb = b.shape[-2], b.shape[-1]
    nc, mc = c.shape[-2], c.shape[-1]
    an, am = (ma, na) if transposedA == X_TRANS else (na, ma)
    bn, bm = (mb, nb) if transposedB == X_TRANS else (nb, mb)
    _check(am == bn and an == nc and bm == mc, "Unmatched tensors in multiplication!")
    _check(tuple(a.shape[:-2]) == tuple(b.shape[:-2]) == tuple(c.shape[:-2]), "Incorrect tensor sizes!")
    count = 1
    for d in a.shape[:-2]:
        count *= d
    rc = capi.lib().ntb_gemm_strided_batched(a.device.index, _stream(a), a.data_ptr(), transposedA,
                                             b.data_ptr(), transposedB, c.data_ptr(),
                                             _dtype_code(a), _dtype_code(c), na, ma, nb, mb, nc, mc,
                                             ma, mb, mc, na * ma, nb * mb, nc * mc, count, alpha, beta)
    _raise_rc(rc, "_MatrixMulBatched")


def MatrixMul(a, transposedA, b, transposedB, alpha=1.0, beta=0.0, c=None):
    """Allocating form (c is None: result on a's device, shape a.lead + b.lead + [an, bm],
    MatrixMul.cpp:279-298) or the form writing into the caller's c with alpha and beta
    (MatrixMul.cpp:317-361; a c of the wrong shape is re-made, CheckMMulShape :210-249)."""
    an = a.shape[-1] if transposedA == X_TRANS else a.shape[-2]
    bm = b.shape[-2] if transposedB == X_TRANS else b.shape[-1]
    shape = tuple(a.shape[:-2]) + tuple(b.shape[:-2]) + (an, bm)
    if c is None or tuple(c.shape) != shape:
        c = torch.zeros(shape, dtype=a.dtype, device=a.device)
    _MatrixMul(a, transposedA, b, transposedB, c, alpha, beta)
    return c


def MMul(a, b, alpha=1.0):
    """No-transposition shortcut (MatrixMul.cpp:371-459)."""
    return MatrixMul(a, X_NOTRANS, b, X_NOTRANS, alpha)


def MatrixMulBatched(a, transposedA, b, transposedB, alpha=1.0):
    an = a.shape[-1] if transposedA == X_TRANS else a.shape[-2]
    bm = b.shape[-2] if transposedB == X_TRANS else b.shape[-1]
    c = torch.empty(tuple(a.shape[:-2]) + (an, bm), dtype=a.dtype, device=a.device)
    _MatrixMulBatched(a, transposedA, b, transposedB, c, alpha, 0.0)
    return c


BMMul = MatrixMulBatched


def MulAndShift(x, w, b, alpha=1.0, transposedX=X_NOTRANS, transposedW=X_NOTRANS, act=capi.ACT_NONE):
    """alpha * op(x) * op(w) + b, b a vector added along the last dimension of the result
    (the linear layer of the transformer). One kernel: the bias -- and with
    act=capi.ACT_RECTIFY the feed-forward layer's Rectify -- is applied in the epilogue,
    where the reference writes the product to a scratch tensor and runs _SumDim over it
    (MulAndShift.cpp:66-88). Leading extents of an untransposed x fold into rows, as in
    _MatrixMul; other higher-order combinations are not supported here."""
    _check(x.dtype == w.dtype, "Input tensors should have the same data type!")
    _check(x.dim() >= 2 and w.dim() >= 2, "Input tensors must have a order >= 2!")
    _check(x.is_cuda and w.is_cuda and b.is_cuda, "this library has no CPU path: tensors must live on a CUDA device")
    _check(w.dim() == 2 and (x.dim() == 2 or transposedX == X_NOTRANS),
           "only a matrix w and an untransposed higher-order x are supported")
    _check(x.is_contiguous() and w.is_contiguous() and b.is_contiguous(), "tensors must be dense and packed")
    x2 = x.view(-1, x.shape[-1]) if x.dim() > 2 else x
    xn, xm = (x2.shape[1], x2.shape[0]) if transposedX == X_TRANS else (x2.shape[0], x2.shape[1])
    wn, wm = (w.shape[1], w.shape[0]) if transposedW == X_TRANS else (w.shape[0], w.shape[1])
    _check(xm == wn, "Unmatched tensors in multiplication!")
    _check(b.dim() == 1 and b.shape[0] == wm and b.dtype == x.dtype, "the bias must be a vector over the last dimension")
    out_shape = tuple(x.shape[:-2]) + ((x.shape[-1] if transposedX == X_TRANS else x.shape[-2]), wm)
    c = torch.empty(out_shape, dtype=x.dtype, device=x.device)
    rc = capi.lib().ntb_gemm_bias_act(x.device.index, _stream(x), x2.data_ptr(), transposedX, w.data_ptr(), transposedW,
                                      b.data_ptr(), c.data_ptr(), _dtype_code(x), _dtype_code(c),
                                      x2.shape[0], x2.shape[1], w.shape[0], w.shape[1], xn, wm,
                                      x2.shape[1], w.shape[1], wm, alpha, 0.0, act)
    _raise_rc(rc, "MulAndShift")
    return c


def ScaledDotProductAttention(q, k, v, mask=None, scale=None, keep=None, drop_prob=0.0):
    """softmax(scale * q k^T + mask) v over the last two dimensions, leading dimensions being
    (head, batch) blocks: the fused form of the chain in Attention::MakeAttention
    (source/sample/transformer/submodel/Attention.cpp:206-238). q [..., lenQ, d], k, v
    [..., lenK, d] half tensors, d = 64 or 128, any lenK; mask None or fp32 of shape
    [lenQ, lenK] (shared) or [..., lenQ, lenK]; scale defaults to 1 / sqrt(d). Training:
    keep is a uint8 tensor [..., lenQ, lenK] (1 = keep) applied to the probabilities with the
    factor 1 / (1 - drop_prob), the reference's Dropout with the caller's mask
    (Attention.cpp:229-230, source/tensor/function/Dropout.cpp:148-158)."""
    _check(q.is_cuda and k.is_cuda and v.is_cuda, "this library has no CPU path: tensors must live on a CUDA device")
    _check(q.dtype == torch.float16 and k.dtype == q.dtype and v.dtype == q.dtype, "Unsupported data type!")
    _check(q.dim() >= 2 and q.shape[:-2] == k.shape[:-2] == v.shape[:-2], "Incorrect tensor sizes!")
    _check(k.shape == v.shape and q.shape[-1] == k.shape[-1], "Unmatched tensors in multiplication!")
    _check(q.is_contiguous() and k.is_contiguous() and v.is_contiguous(), "tensors must be dense and packed")
    lenQ, d = q.shape[-2], q.shape[-1]
    lenK = k.shape[-2]
    blocks = 1
    for n in q.shape[:-2]:
        blocks *= n
    stride = 0
    mptr = None
    if mask is not None:
        _check(mask.is_cuda and mask.dtype == torch.float32 and mask.is_contiguous(), "the mask must be a packed fp32 CUDA tensor")
        if mask.dim() == 2:
            _check(tuple(mask.shape) == (lenQ, lenK), "Incorrect tensor sizes!")
        else:
            _check(tuple(mask.shape) == tuple(q.shape[:-2]) + (lenQ, lenK), "Incorrect tensor sizes!")
            stride = lenQ * lenK
        mptr = mask.data_ptr()
    kptr, keep_scale = None, 1.0
    if keep is not None:
        _check(keep.is_cuda and keep.dtype == torch.uint8 and keep.is_contiguous(), "the keep-mask must be a packed uint8 CUDA tensor")
        _check(tuple(keep.shape) == tuple(q.shape[:-2]) + (lenQ, lenK), "Incorrect tensor sizes!")
        _check(0.0 <= drop_prob < 1.0, "The probability must be 0-1!")
        kptr, keep_scale = keep.data_ptr(), 1.0 / (1.0 - drop_prob)
    out = torch.empty_like(q)
    if scale is None:
        scale = 1.0 / (d ** 0.5)
    rc = capi.lib().ntb_attention_dropout(q.device.index, _stream(q), q.data_ptr(), k.data_ptr(), v.data_ptr(), mptr, kptr,
                                          out.data_ptr(), X_FLOAT16, blocks, lenQ, lenK, d, stride, scale, keep_scale)
    _raise_rc(rc, "ScaledDotProductAttention")
    return out


def RowStats(x):
    """(row maximum, sum of exp(x - maximum)) over the last dimension of a 2-D tensor, fp32."""
    _check(x.is_cuda and x.dim() == 2 and x.stride(1) == 1, "a CUDA matrix with unit column stride is required")
    rows, cols = x.shape
    mx = torch.empty(rows, dtype=torch.float32, device=x.device)
    sm = torch.empty(rows, dtype=torch.float32, device=x.device)
    rc = capi.lib().ntb_row_stats(x.device.index, _stream(x), x.data_ptr(), _dtype_code(x), rows, cols, x.stride(0),
                                  mx.data_ptr(), sm.data_ptr())
    _raise_rc(rc, "RowStats")
    return mx, sm


def LogSoftmaxApply(x, row_max, row_sum, out=None):
    """log(exp(x - row_max) / row_sum) with the reference's floor of -20 (LogSoftmax.cpp:133-148)."""
    _check(x.is_cuda and x.dim() == 2 and x.stride(1) == 1, "a CUDA matrix with unit column stride is required")
    y = x if out is None else out
    rows, cols = x.shape
    rc = capi.lib().ntb_logsoftmax_apply(x.device.index, _stream(x), x.data_ptr(), y.data_ptr(), _dtype_code(x),
                                         rows, cols, x.stride(0), y.stride(0), row_max.data_ptr(), row_sum.data_ptr())
    _raise_rc(rc, "LogSoftmaxApply")
    return y


def LogSoftmax(x):
    """Log-softmax over the last dimension (source/tensor/function/LogSoftmax.cpp:40), in place
    on a copy: leading dimensions fold into rows."""
    x2 = x.reshape(-1, x.shape[-1]).clone()
    mx, sm = RowStats(x2)
    return LogSoftmaxApply(x2, mx, sm).view(x.shape)


def GradMatrixMul(a, transposedA, b, transposedB, dedc, deda, dedb, alpha=1.0):
    """Backward of c = alpha * op(a) * op(b) (2-D or batched with equal leading extents):
    deda and dedb are accumulated into (beta = 1) with the operand table of
    XMathGrad::GradMatrixMul / GradMatrixMulBatched (source/network/XBackwardMath.cpp:655-699,
    :714-786). Both products run in one launch. Either gradient may be None."""
    _check(a.is_cuda and b.is_cuda and dedc.is_cuda, "this library has no CPU path: tensors must live on a CUDA device")
    _check(a.dtype == b.dtype == dedc.dtype, "Input tensors should have the same data type!")
    _check(a.dim() == b.dim() and a.dim() >= 2 and tuple(a.shape[:-2]) == tuple(b.shape[:-2]), "Incorrect tensor sizes!")
    for t in (a, b, dedc, deda, dedb):
        _check(t is None or t.is_contiguous(), "tensors must be dense and packed")
    _check(deda is None or deda.shape == a.shape, "Incorrect tensor sizes!")
    _check(dedb is None or dedb.shape == b.shape, "Incorrect tensor sizes!")
    an = a.shape[-1] if transposedA == X_TRANS else a.shape[-2]
    bm = b.shape[-2] if transposedB == X_TRANS else b.shape[-1]
    _check(tuple(dedc.shape) == tuple(a.shape[:-2]) + (an, bm), "Unmatched tensors in multiplication!")
    count = 1
    for n in a.shape[:-2]:
        count *= n
    rc = capi.lib().ntb_gemm_grad(a.device.index, _stream(a), a.data_ptr(), transposedA, b.data_ptr(), transposedB,
                                  dedc.data_ptr(), None if deda is None else deda.data_ptr(),
                                  None if dedb is None else dedb.data_ptr(), _dtype_code(a),
                                  a.shape[-2], a.shape[-1], b.shape[-2], b.shape[-1], count, alpha)
    _raise_rc(rc, "GradMatrixMul")


def MatrixMul2DToPeers(a, transposedA, b, transposedB, c_full, col0, peer_bases, alpha=1.0, beta=0.0):
    """c_full[:, col0:col0+n] = alpha * op(a) * op(b) + beta * c_full[:, col0:col0+n], and the same
    block written to the same place of every buffer in peer_bases (device addresses of
    matrices with the shape and pitch of c_full: other GPUs' copies of C mapped into this
    process, or other buffers of this GPU). The stores to the peers are issued by the
    epilogue of the product (ntb_gemm_peers); no separate gather pass runs."""
    _common_checks(a, b, c_full)
    _check(a.dim() == 2 and b.dim() == 2 and c_full.dim() == 2, "Input tensors must have a order = 2!")
    an, am = (a.shape[1], a.shape[0]) if transposedA == X_TRANS else (a.shape[0], a.shape[1])
    bn, bm = (b.shape[1], b.shape[0]) if transposedB == X_TRANS else (b.shape[0], b.shape[1])
    _check(am == bn and an == c_full.shape[0] and 0 <= col0 and col0 + bm <= c_full.shape[1],
           "Unmatched tensors in multiplication!")
    _check(len(peer_bases) <= capi.MAX_PEERS, "too many peers")
    es = c_full.element_size()
    ptrs = (ctypes.c_void_p * max(1, len(peer_bases)))(*[int(x) + col0 * es for x in peer_bases])
    rc = capi.lib().ntb_gemm_peers(a.device.index, _stream(a), a.data_ptr(), transposedA, b.data_ptr(), transposedB,
                                   c_full.data_ptr() + col0 * es, ptrs, len(peer_bases),
                                   _dtype_code(a), _dtype_code(c_full),
                                   a.shape[0], a.shape[1], b.shape[0], b.shape[1], an, bm,
                                   a.shape[1], b.shape[1], c_full.shape[1], alpha, beta)
    _raise_rc(rc, "MatrixMul2DToPeers")


def MatrixMul2DToMulticast(a, transposedA, b, transposedB, c_full, col0, mc_base, alpha=1.0, beta=0.0):
    """As MatrixMul2DToPeers, with the NVLink switch replicating the block: mc_base is the
    multicast address of c_full (symmetric memory bound to every rank's copy); each finished
    line is written once with multimem.st and lands in every rank's C (ntb_gemm_multicast)."""
    _common_checks(a, b, c_full)
    _check(a.dim() == 2 and b.dim() == 2 and c_full.dim() == 2, "Input tensors must have a order = 2!")
    an, am = (a.shape[1], a.shape[0]) if transposedA == X_TRANS else (a.shape[0], a.shape[1])
    bn, bm = (b.shape[1], b.shape[0]) if transposedB == X_TRANS else (b.shape[0], b.shape[1])
    _check(am == bn and an == c_full.shape[0] and 0 <= col0 and col0 + bm <= c_full.shape[1],
           "Unmatched tensors in multiplication!")
    es = c_full.element_size()
    rc = capi.lib().ntb_gemm_multicast(a.device.index, _stream(a), a.data_ptr(), transposedA, b.data_ptr(), transposedB,
                                       c_full.data_ptr() + col0 * es, int(mc_base) + col0 * es,
                                       _dtype_code(a), _dtype_code(c_full),
                                       a.shape[0], a.shape[1], b.shape[0], b.shape[1], an, bm,
                                       a.shape[1], b.shape[1], c_full.shape[1], alpha, beta)
    _raise_rc(rc, "MatrixMul2DToMulticast")
