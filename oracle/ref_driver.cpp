/*
 * TEST INFRASTRUCTURE ONLY. Thin C driver around the unmodified NiuTensor CPU
 * matrix-multiplication operators, compiled together with the NiuTensor sources
 * (where they lie, never copied) into oracle/_ref/. It wraps caller-owned host
 * buffers in header-only XTensor objects and calls the reference's own
 *   nts::_MatrixMul          (source/tensor/core/arithmetic/MatrixMul.cpp:52)
 *   nts::_MatrixMulBatched   (source/tensor/core/arithmetic/MatrixMulBatched.cpp:49)
 *   nts::_MatrixMul2D        (source/tensor/core/arithmetic/MatrixMul2D.cpp:46)
 * Nothing on the product path may link or load this file's output.
 */
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include "tensor/XTensor.h"
#include "tensor/XCall.h"
#include "tensor/core/arithmetic/MatrixMul.h"
#include "tensor/core/arithmetic/MatrixMul2D.h"
#include "tensor/core/arithmetic/MatrixMulBatched.h"
#include "tensor/core/arithmetic/MulAndShift.h"
#include "tensor/core/arithmetic/Sum.h"
#include "tensor/core/math/ScaleAndShift.h"
#include "tensor/function/Softmax.h"
#include "tensor/function/LogSoftmax.h"
#ifdef USE_BLAS
#include "tensor/XBLAS.h"
#endif

using namespace nts;

namespace {
/* header without storage: negative leading extent (XTensor.cpp:1459-1462) */
XTensor * View(float * data, int order, const int * dims)
{
    int d[8];
    for (int i = 0; i < order; i++)
        d[i] = dims[i];
    d[0] = -d[0];
    XTensor * t = NewTensorV2(order, d, X_FLOAT, 1.0F, -1, NULL);
    t->data = data;
    return t;
}
void Drop(XTensor * t)
{
    t->data = NULL;
    delete t;
}
}

extern "C" {

/* form: 0 = _MatrixMul (general / broadcast / flatten), 1 = _MatrixMulBatched,
   2 = _MatrixMul2D. trans flags carry the reference enum: 0 = X_TRANS, 1 = X_NOTRANS. */
int ref_matmul_f32(int form,
                   const float * a, int aOrder, const int * aDims, int transA,
                   const float * b, int bOrder, const int * bDims, int transB,
                   float * c, int cOrder, const int * cDims,
                   float alpha, float beta)
{
    XTensor * ta = View((float*)a, aOrder, aDims);
    XTensor * tb = View((float*)b, bOrder, bDims);
    XTensor * tc = View(c, cOrder, cDims);
    MATRIX_TRANS_TYPE tA = transA == 0 ? X_TRANS : X_NOTRANS;
    MATRIX_TRANS_TYPE tB = transB == 0 ? X_TRANS : X_NOTRANS;
    if (form == 0)
        _MatrixMul(ta, tA, tb, tB, tc, alpha, beta);
    else if (form == 1)
        _MatrixMulBatched(ta, tA, tb, tB, tc, alpha, beta);
    else
        _MatrixMul2D(ta, tA, tb, tB, tc, alpha, beta);
    Drop(ta);
    Drop(tb);
    Drop(tc);
    return 0;
}

/* the reference's user-level MulAndShift (source/tensor/core/arithmetic/MulAndShift.cpp:38,
   120) on CPU tensors: y = alpha * op(x) * op(w) + bias along the last dimension */
int ref_mulandshift_f32(const float * x, int xOrder, const int * xDims, int transX,
                        const float * w, int wOrder, const int * wDims, int transW,
                        const float * bias, int biasLen, float * y, float alpha)
{
    XTensor * tx = View((float*)x, xOrder, xDims);
    XTensor * tw = View((float*)w, wOrder, wDims);
    int bd[1] = { biasLen };
    XTensor * tb = View((float*)bias, 1, bd);
    int rc = 0;
    {
        XTensor out = (transX == 1 && transW == 1)
            ? MulAndShift(*tx, *tw, *tb, alpha)
            : MulAndShift(*tx, transX == 0 ? X_TRANS : X_NOTRANS, *tw, transW == 0 ? X_TRANS : X_NOTRANS, *tb, alpha);
        if (out.data == NULL)
            rc = 1;
        else
            memcpy(y, out.data, sizeof(float) * (size_t)out.unitNum);
    }
    Drop(tx);
    Drop(tw);
    Drop(tb);
    return rc;
}

/* The inference-time attention chain of source/sample/transformer/submodel/Attention.cpp:
   206-238 with the reference's own CPU operators: scale q, BMMul(q, k^T), add the mask,
   Softmax over the last dimension, BMMul(att, v). mask may be NULL; otherwise it has the
   shape of the scores. */
int ref_attention_dropout_f32(const float * q, const float * k, const float * v, const float * mask,
                              const float * dropMask, float * out,
                              int blocks, int lenQ, int lenK, int dim, float scale)
{
    int dq[3] = { blocks, lenQ, dim }, dk[3] = { blocks, lenK, dim }, ds[3] = { blocks, lenQ, lenK };
    XTensor tq, att, att2;
    InitTensorV2(&tq, 3, dq, X_FLOAT, 1.0F, -1);
    InitTensorV2(&att, 3, ds, X_FLOAT, 1.0F, -1);
    InitTensorV2(&att2, 3, ds, X_FLOAT, 1.0F, -1);
    memcpy(tq.data, q, sizeof(float) * (size_t)tq.unitNum);
    XTensor * tk = View((float*)k, 3, dk);
    XTensor * tv = View((float*)v, 3, dk);
    XTensor * to = View(out, 3, dq);
    _ScaleAndShiftMe(&tq, scale, 0);
    _MatrixMulBatched(&tq, X_NOTRANS, tk, X_TRANS, &att);
    if (mask != NULL) {
        XTensor * tm = View((float*)mask, 3, ds);
        _Sum(&att, tm, &att);
        Drop(tm);
    }
    _Softmax(&att, &att2, 2);
    if (dropMask != NULL) {
        /* Dropout as source/tensor/function/Dropout.cpp:148-158 applies it: a product with a mask
           of zeros and 1 / (1 - p); the mask is the caller's instead of the operator's own draw */
        XTensor * td = View((float*)dropMask, 3, ds);
        _Multiply(&att2, td, &att2);
        Drop(td);
    }
    _MatrixMulBatched(&att2, X_NOTRANS, tv, X_NOTRANS, to);
    Drop(tk);
    Drop(tv);
    Drop(to);
    return 0;
}

int ref_attention_f32(const float * q, const float * k, const float * v, const float * mask, float * out,
                      int blocks, int lenQ, int lenK, int dim, float scale)
{
    return ref_attention_dropout_f32(q, k, v, mask, NULL, out, blocks, lenQ, lenK, dim, scale);
}

/* The normalised output layer of source/sample/transformer/submodel/Output.cpp:86-101 with
   the reference's CPU operators: logits = h * w^T (w stored [vocab, hidden]), then
   LogSoftmax over the vocabulary. logits may be NULL. */
int ref_output_layer_f32(const float * h, const float * w, float * logits, float * logprob,
                         int rows, int hidden, int vocab)
{
    int dh[2] = { rows, hidden }, dw[2] = { vocab, hidden }, dy[2] = { rows, vocab };
    XTensor * th = View((float*)h, 2, dh);
    XTensor * tw = View((float*)w, 2, dw);
    XTensor * ty = View(logprob, 2, dy);
    XTensor tmp;
    InitTensorV2(&tmp, 2, dy, X_FLOAT, 1.0F, -1);
    _MatrixMul(th, X_NOTRANS, tw, X_TRANS, &tmp);
    if (logits != NULL)
        memcpy(logits, tmp.data, sizeof(float) * (size_t)tmp.unitNum);
    _LogSoftmax(&tmp, ty, 1);
    Drop(th);
    Drop(tw);
    Drop(ty);
    return 0;
}

/* 1 when this build routes dense fp32 GEMMs to cblas_sgemm (XTensorBLAS.cpp:39) */
int ref_uses_blas(void)
{
#ifdef USE_BLAS
    return 1;
#else
    return 0;
#endif
}

void ref_set_blas_threads(int n)
{
#ifdef USE_BLAS
    openblas_set_num_threads(n);
#else
    (void)n;
#endif
}

}
