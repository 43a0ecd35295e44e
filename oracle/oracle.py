"""TEST INFRASTRUCTURE ONLY: Python face of the CPU oracle.

`Oracle` loads oracle/liboracle_matmul.so (the plain-C restatement of NiuTensor's
built-in fp32 CPU matrix multiplication, oracle/matmul_oracle.c). `Reference` loads
the unmodified NiuTensor CPU library built by `make -C oracle ref` into oracle/_ref/
(absent on machines where the reference sources are not available).

Only tests, the smoke check and the CPU-baseline legs of the benchmark may import this
module; the product package never does.

Transposition flags follow the reference enum (source/tensor/XDataType.h:36):
X_TRANS = 0, X_NOTRANS = 1.
"""
import ctypes
import os
import subprocess

import numpy as np

X_TRANS = 0
X_NOTRANS = 1

_HERE = os.path.dirname(os.path.abspath(__file__))
_F32P = ctypes.POINTER(ctypes.c_float)
_I32P = ctypes.POINTER(ctypes.c_int)


def _fp(x):
    return x.ctypes.data_as(_F32P)


def _as_f32(x):
    return np.ascontiguousarray(x, dtype=np.float32)


def build_oracle():
    """Compile the C restatement if it is missing or older than its source."""
    so = os.path.join(_HERE, "liboracle_matmul.so")
    src = os.path.join(_HERE, "matmul_oracle.c")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "oracle"])
    return so


def mm_dims(a_shape, tA, b_shape, tB):
    """(M, N, K) of op(a) * op(b) from the stored 2-D shapes."""
    na, ma = a_shape[-2], a_shape[-1]
    nb, mb = b_shape[-2], b_shape[-1]
    M, K = (ma, na) if tA == X_TRANS else (na, ma)
    K2, N = (mb, nb) if tB == X_TRANS else (nb, mb)
    if K != K2:
        raise ValueError("unmatched inner dimensions %r %r" % (a_shape, b_shape))
    return M, N, K


class Oracle:
    """ctypes binding of oracle/matmul_oracle.c."""

    def __init__(self):
        self.lib = ctypes.CDLL(build_oracle())
        self.lib.orc_matmul2d_f32.argtypes = [_F32P, ctypes.c_int, _F32P, ctypes.c_int, _F32P] + \
            [ctypes.c_int] * 6 + [ctypes.c_float] * 2
        self.lib.orc_matmul_batched_f32.argtypes = [_F32P, ctypes.c_int, _F32P, ctypes.c_int, _F32P] + \
            [ctypes.c_int] * 7 + [ctypes.c_float] * 2
        self.lib.orc_matmul_broadcast_f32.argtypes = [_F32P, ctypes.c_int, _F32P, ctypes.c_int, _F32P] + \
            [ctypes.c_int] * 8 + [ctypes.c_float] * 2
        self.lib.orc_set_threads.argtypes = [ctypes.c_int]
        self.lib.orc_logsoftmax_f32.argtypes = [_F32P, _F32P, ctypes.c_int, ctypes.c_int]
        self.lib.orc_attention_f32.argtypes = [_F32P, _F32P, _F32P, _F32P, _F32P] + [ctypes.c_int] * 4 + \
            [ctypes.c_longlong, ctypes.c_float]
        self.lib.orc_mulandshift_f32.argtypes = [_F32P, ctypes.c_int, _F32P, ctypes.c_int, _F32P, _F32P] + \
            [ctypes.c_int] * 6 + [ctypes.c_float, ctypes.c_int]

    def set_threads(self, n):
        self.lib.orc_set_threads(int(n))

    def matmul2d(self, a, tA, b, tB, alpha=1.0, beta=0.0, c=None):
        a, b = _as_f32(a), _as_f32(b)
        M, N, _ = mm_dims(a.shape, tA, b.shape, tB)
        c = np.zeros((M, N), np.float32) if c is None else _as_f32(c).copy()
        self.lib.orc_matmul2d_f32(_fp(a), tA, _fp(b), tB, _fp(c), a.shape[0], a.shape[1],
                                  b.shape[0], b.shape[1], M, N, alpha, beta)
        return c

    def mulandshift(self, x, w, b, alpha=1.0, tX=X_NOTRANS, tW=X_NOTRANS, rectify=False):
        """MulAndShift: alpha * op(x) * op(w) + b along the last dimension; leading extents
        of an untransposed x fold into rows."""
        x, w, b = _as_f32(x), _as_f32(w), _as_f32(b)
        lead = x.shape[:-2]
        if tX == X_NOTRANS and x.ndim > 2:
            x2 = x.reshape(-1, x.shape[-1])
        else:
            if x.ndim != 2:
                raise ValueError("a transposed x must be a matrix here")
            x2 = x
        M, N, _ = mm_dims(x2.shape, tX, w.shape, tW)
        c = np.zeros((M, N), np.float32)
        self.lib.orc_mulandshift_f32(_fp(x2), tX, _fp(w), tW, _fp(b), _fp(c), x2.shape[0], x2.shape[1],
                                     w.shape[0], w.shape[1], M, N, alpha, 1 if rectify else 0)
        return c.reshape(lead + (M // max(1, int(np.prod(lead, dtype=np.int64))), N)) if lead else c

    def logsoftmax(self, x):
        """LogSoftmax over the last dimension with the reference's floor of -20."""
        x = _as_f32(x)
        y = np.zeros_like(x)
        self.lib.orc_logsoftmax_f32(_fp(x), _fp(y), int(np.prod(x.shape[:-1], dtype=np.int64)), x.shape[-1])
        return y

    def output_layer(self, h, w):
        """log-probabilities of the output layer: LogSoftmax(h w^T), w stored [vocab, hidden]."""
        return self.logsoftmax(self.matmul2d(_as_f32(h), X_NOTRANS, _as_f32(w), X_TRANS))

    def attention_dropout(self, q, k, v, keep, keep_scale, mask=None, scale=1.0):
        """attention with Dropout on the probabilities: keep [blocks, lenQ, lenK] uint8 (1 = keep),
        kept probabilities times keep_scale = 1 / (1 - p)."""
        q, k, v = _as_f32(q), _as_f32(k), _as_f32(v)
        blocks, lenQ, d = q.shape
        lenK = k.shape[1]
        keep = np.ascontiguousarray(keep, dtype=np.uint8)
        assert keep.shape == (blocks, lenQ, lenK)
        out = np.zeros((blocks, lenQ, d), np.float32)
        mp, stride = None, 0
        if mask is not None:
            mask = _as_f32(mask)
            mp = _fp(mask)
            stride = lenQ * lenK if mask.ndim == 3 else 0
        fn = self.lib.orc_attention_dropout_f32
        fn.argtypes = [_F32P, _F32P, _F32P, _F32P, ctypes.c_void_p, ctypes.c_float, _F32P] + [ctypes.c_int] * 4 + \
            [ctypes.c_longlong, ctypes.c_float]
        fn.restype = None
        fn(_fp(q), _fp(k), _fp(v), mp, keep.ctypes.data, keep_scale, _fp(out), blocks, lenQ, lenK, d, stride, scale)
        return out

    def attention(self, q, k, v, mask=None, scale=1.0):
        """softmax(scale * q k^T + mask) v per block; q [blocks, lenQ, d], k, v [blocks, lenK, d],
        mask None, [lenQ, lenK] (shared) or [blocks, lenQ, lenK]."""
        q, k, v = _as_f32(q), _as_f32(k), _as_f32(v)
        blocks, lenQ, d = q.shape
        lenK = k.shape[1]
        out = np.zeros((blocks, lenQ, d), np.float32)
        mp, stride = None, 0
        if mask is not None:
            mask = _as_f32(mask)
            mp = _fp(mask)
            stride = lenQ * lenK if mask.ndim == 3 else 0
        self.lib.orc_attention_f32(_fp(q), _fp(k), _fp(v), mp, _fp(out), blocks, lenQ, lenK, d, stride, scale)
        return out

    def matmul_batched(self, a, tA, b, tB, alpha=1.0, beta=0.0, c=None):
        """_MatrixMulBatched: equal leading extents, block i of a meets block i of b."""
        a, b = _as_f32(a), _as_f32(b)
        if a.shape[:-2] != b.shape[:-2]:
            raise ValueError("leading extents differ")
        M, N, _ = mm_dims(a.shape, tA, b.shape, tB)
        count = int(np.prod(a.shape[:-2], dtype=np.int64))
        shape = a.shape[:-2] + (M, N)
        c = np.zeros(shape, np.float32) if c is None else _as_f32(c).copy().reshape(shape)
        self.lib.orc_matmul_batched_f32(_fp(a), tA, _fp(b), tB, _fp(c), count,
                                        a.shape[-2], a.shape[-1], b.shape[-2], b.shape[-1],
                                        M, N, alpha, beta)
        return c

    def matmul(self, a, tA, b, tB, alpha=1.0, beta=0.0, c=None):
        """_MatrixMul: general form; c has shape a.lead + b.lead + (M, N)."""
        a, b = _as_f32(a), _as_f32(b)
        M, N, _ = mm_dims(a.shape, tA, b.shape, tB)
        shape = a.shape[:-2] + b.shape[:-2] + (M, N)
        c = np.zeros(shape, np.float32) if c is None else _as_f32(c).copy().reshape(shape)
        P = int(np.prod(a.shape[:-2], dtype=np.int64))
        Q = int(np.prod(b.shape[:-2], dtype=np.int64))
        self.lib.orc_matmul_broadcast_f32(_fp(a), tA, _fp(b), tB, _fp(c), P, Q,
                                          a.shape[-2], a.shape[-1], b.shape[-2], b.shape[-1],
                                          M, N, alpha, beta)
        return c


def ref_path(kind):
    return os.path.join(_HERE, "_ref", "libnts_ref_%s.so" % kind)


def ref_available(kind="builtin"):
    return os.path.exists(ref_path(kind))


def _preload_openblas_deps():
    """The OpenBLAS the reference is linked to here ships inside the
    opencv_python_headless wheel; its libgfortran/libquadmath sit beside it and are not
    on the loader path, so they are opened first."""
    import glob
    import sys
    dirs = glob.glob(os.path.join(sys.prefix, "lib", "python3*", "site-packages",
                                  "opencv_python_headless.libs"))
    for d in dirs:
        for pat in ("libquadmath-*.so*", "libgfortran-*.so*"):
            for f in sorted(glob.glob(os.path.join(d, pat))):
                ctypes.CDLL(f, mode=ctypes.RTLD_GLOBAL)


class Reference:
    """The compiled NiuTensor CPU library behind oracle/ref_driver.cpp.

    kind "builtin": the reference's own scalar loops (correct for all four
    transposition combinations, single-threaded). kind "openblas": the reference built
    with USE_BLAS against OpenBLAS; its T/T branch is wrong in the reference itself
    (source/tensor/core/arithmetic/XTensorBLAS.cpp:64-65), so callers avoid T/T there.
    """
    FORM_GENERAL, FORM_BATCHED, FORM_2D = 0, 1, 2

    def __init__(self, kind="builtin"):
        self.kind = kind
        if kind == "openblas":
            _preload_openblas_deps()
        self.lib = ctypes.CDLL(ref_path(kind))
        self.lib.ref_matmul_f32.argtypes = [
            ctypes.c_int,
            _F32P, ctypes.c_int, _I32P, ctypes.c_int,
            _F32P, ctypes.c_int, _I32P, ctypes.c_int,
            _F32P, ctypes.c_int, _I32P,
            ctypes.c_float, ctypes.c_float]
        self.lib.ref_set_blas_threads.argtypes = [ctypes.c_int]
        self.lib.ref_mulandshift_f32.argtypes = [
            _F32P, ctypes.c_int, _I32P, ctypes.c_int, _F32P, ctypes.c_int, _I32P, ctypes.c_int,
            _F32P, ctypes.c_int, _F32P, ctypes.c_float]

    def set_threads(self, n):
        self.lib.ref_set_blas_threads(int(n))

    def run(self, form, a, tA, b, tB, alpha=1.0, beta=0.0, c=None, inplace=False):
        """c (if given) is copied unless inplace is set, in which case it must be a packed
        float32 array of the output shape and is overwritten."""
        a, b = _as_f32(a), _as_f32(b)
        M, N, _ = mm_dims(a.shape, tA, b.shape, tB)
        if form == self.FORM_GENERAL:
            shape = a.shape[:-2] + b.shape[:-2] + (M, N)
        else:
            shape = a.shape[:-2] + (M, N)
        if inplace:
            assert c is not None and c.dtype == np.float32 and c.flags.c_contiguous and c.shape == shape
        else:
            c = np.zeros(shape, np.float32) if c is None else _as_f32(c).copy().reshape(shape)
        ad = np.asarray(a.shape, np.int32)
        bd = np.asarray(b.shape, np.int32)
        cd = np.asarray(c.shape, np.int32)
        self.lib.ref_matmul_f32(form, _fp(a), a.ndim, ad.ctypes.data_as(_I32P), tA,
                                _fp(b), b.ndim, bd.ctypes.data_as(_I32P), tB,
                                _fp(c), c.ndim, cd.ctypes.data_as(_I32P), alpha, beta)
        return c


def ref_mulandshift(ref, x, w, b, alpha=1.0, tX=X_NOTRANS, tW=X_NOTRANS):
    """The reference's own user-level MulAndShift on CPU tensors."""
    x, w, b = _as_f32(x), _as_f32(w), _as_f32(b)
    M, N, _ = mm_dims(x.shape, tX, w.shape, tW)
    c = np.zeros(x.shape[:-2] + (M, N), np.float32)
    xd = np.asarray(x.shape, np.int32)
    wd = np.asarray(w.shape, np.int32)
    rc = ref.lib.ref_mulandshift_f32(_fp(x), x.ndim, xd.ctypes.data_as(_I32P), tX,
                                     _fp(w), w.ndim, wd.ctypes.data_as(_I32P), tW,
                                     _fp(b), b.shape[0], _fp(c), alpha)
    if rc != 0:
        raise RuntimeError("ref_mulandshift_f32 failed: %d" % rc)
    return c


def ref_attention(ref, q, k, v, mask=None, scale=1.0, keep=None, keep_scale=1.0):
    """The reference's own CPU operator chain for attention; with `keep`, the probabilities are
    multiplied by the dropout mask (zeros and keep_scale) as the reference's Dropout does."""
    q, k, v = _as_f32(q), _as_f32(k), _as_f32(v)
    blocks, lenQ, d = q.shape
    lenK = k.shape[1]
    out = np.zeros((blocks, lenQ, d), np.float32)
    fn = ref.lib.ref_attention_dropout_f32
    fn.argtypes = [_F32P, _F32P, _F32P, _F32P, _F32P, _F32P] + [ctypes.c_int] * 4 + [ctypes.c_float]
    mp = None
    if mask is not None:
        mask = _as_f32(np.broadcast_to(mask, (blocks, lenQ, lenK)))
        mp = _fp(mask)
    dp = None
    if keep is not None:
        drop = _as_f32(np.where(np.asarray(keep) != 0, np.float32(keep_scale), np.float32(0)))
        dp = _fp(drop)
    rc = fn(_fp(q), _fp(k), _fp(v), mp, dp, _fp(out), blocks, lenQ, lenK, d, scale)
    if rc != 0:
        raise RuntimeError("ref_attention_dropout_f32 failed")
    return out


def ref_output_layer(ref, h, w):
    """The reference's CPU MMul + LogSoftmax of the normalised output layer."""
    h, w = _as_f32(h), _as_f32(w)
    rows, hidden = h.shape
    vocab = w.shape[0]
    out = np.zeros((rows, vocab), np.float32)
    ref.lib.ref_output_layer_f32.argtypes = [_F32P, _F32P, _F32P, _F32P, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    rc = ref.lib.ref_output_layer_f32(_fp(h), _fp(w), None, _fp(out), rows, hidden, vocab)
    if rc != 0:
        raise RuntimeError("ref_output_layer_f32 failed")
    return out


def grad_matmul(oracle, a, tA, b, tB, dedc, deda, dedb, alpha=1.0):
    """The two accumulating products of XMathGrad::GradMatrixMul / GradMatrixMulBatched
    (source/network/XBackwardMath.cpp:655-699, :714-786) computed with the oracle's
    batched matmul (beta = 1). Returns the new (deda, dedb)."""
    N, T = X_NOTRANS, X_TRANS
    mm = oracle.matmul_batched
    if tA == N and tB == N:
        return mm(dedc, N, b, T, alpha, 1.0, deda), mm(a, T, dedc, N, alpha, 1.0, dedb)
    if tA == T and tB == N:
        return mm(b, N, dedc, T, alpha, 1.0, deda), mm(a, N, dedc, N, alpha, 1.0, dedb)
    if tA == N and tB == T:
        return mm(dedc, N, b, N, alpha, 1.0, deda), mm(dedc, T, a, N, alpha, 1.0, dedb)
    return mm(b, T, dedc, T, alpha, 1.0, deda), mm(dedc, T, a, T, alpha, 1.0, dedb)


def round_to_half(x):
    """IEEE round-to-nearest-even fp32 -> fp16 -> fp32: the values an X_FLOAT16 tensor
    holds. The reference has no CPU fp16 arithmetic (MatrixMul.cpp:181 "TODO!"), so the
    fp16 oracle is the fp32 CPU path run on fp16-valued inputs."""
    return np.asarray(x, np.float32).astype(np.float16).astype(np.float32)


def rel_fro(x, ref):
    """Relative Frobenius error, accumulated in float64."""
    x = np.asarray(x, np.float64)
    ref = np.asarray(ref, np.float64)
    den = np.linalg.norm(ref.ravel())
    return float(np.linalg.norm((x - ref).ravel()) / (den if den > 0 else 1.0))
