/*
 * TEST INFRASTRUCTURE ONLY. Entry points of the drop-in check library built by
 * `make -C oracle dropin`: the unmodified NiuTensor GPU build (USE_CUDA) in which the
 * reference's matrix-multiplication translation units are replaced by
 * niutensor_b200/host/nts_matmul_shim.cpp + libntb_gemm.so. The functions below run the
 * reference's OWN unit tests for this path (source/tensor/test/TMatrixMul.cpp,
 * TMatrixMul2D.cpp, TMatrixMul2DParallel.cpp, TMatrixMulBatched.cpp -- compiled from where
 * they lie), whose GPU halves now execute on the new kernels, a half-precision
 * user-level call the reference has no test for, and the two list forms of the cuBLAS
 * wrapper layer that none of the reference's tests reaches.
 */
#include <cstdio>
#include <cstring>
#include <vector>
#include <cuda_fp16.h>
#include "tensor/XTensor.h"
#include "tensor/XCall.h"
#include "tensor/core/arithmetic/MatrixMul.h"
#include "tensor/core/arithmetic/MatrixMulBatched.h"
#include "tensor/core/arithmetic/MulAndShift.h"
#include "tensor/core/arithmetic/XTensorBLAS.h"
#include "tensor/test/TMatrixMul.h"
#include "tensor/test/TMatrixMul2D.h"
#include "tensor/test/TMatrixMul2DParallel.h"
#include "tensor/test/TMatrixMulBatched.h"

using namespace nts;

extern "C" {

/* bit i set = test i passed: 0 TestMatrixMul, 1 TestMatrixMul2D, 2 TestMatrixMul2DParallel,
   3 TestMatrixMulBatched */
int dropin_run_reference_tests(void)
{
    int mask = 0;
    if (TestMatrixMul()) mask |= 1;
    if (TestMatrixMul2D()) mask |= 2;
    if (TestMatrixMul2DParallel()) mask |= 4;
    if (TestMatrixMulBatched()) mask |= 8;
    return mask;
}

/* user-level BMMul on X_FLOAT16 tensors living on GPU `dev` (pool-less, cudaMalloc'ed):
   scores = alpha * q * k^T for `batch` blocks of [len x dk]; inputs and output are host
   arrays of IEEE half bit patterns. Returns 0 on success. */
int dropin_bmmul_half(int dev, int batch, int len, int dk, const unsigned short * q, const unsigned short * k,
                      unsigned short * scores, float alpha)
{
    int dq[3] = { batch, len, dk };
    XTensor tq, tk;
    InitTensorV2(&tq, 3, dq, X_FLOAT16, 1.0F, dev);
    InitTensorV2(&tk, 3, dq, X_FLOAT16, 1.0F, dev);
    cudaMemcpy(tq.data, q, sizeof(unsigned short) * tq.unitNum, cudaMemcpyHostToDevice);
    cudaMemcpy(tk.data, k, sizeof(unsigned short) * tk.unitNum, cudaMemcpyHostToDevice);
    XTensor s = BMMul(tq, X_NOTRANS, tk, X_TRANS, alpha);
    if (s.order != 3 || s.dimSize[0] != batch || s.dimSize[1] != len || s.dimSize[2] != len)
        return 1;
    cudaMemcpy(scores, s.data, sizeof(unsigned short) * s.unitNum, cudaMemcpyDeviceToHost);
    return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

/* the transformer's linear layer x * w + b (MulAndShift.cpp:38) on fp32 GPU tensors: the
   reference's MulAndShift is unchanged and calls _MatrixMul of the shim */
int dropin_mulandshift_f32(int dev, int rows, int in, int out, const float * x, const float * w, const float * b, float * y)
{
    int dx[2] = { rows, in }, dw[2] = { in, out }, db[1] = { out };
    XTensor tx, tw, tb;
    InitTensorV2(&tx, 2, dx, X_FLOAT, 1.0F, dev);
    InitTensorV2(&tw, 2, dw, X_FLOAT, 1.0F, dev);
    InitTensorV2(&tb, 1, db, X_FLOAT, 1.0F, dev);
    tx.SetData(x, tx.unitNum);
    tw.SetData(w, tw.unitNum);
    tb.SetData(b, tb.unitNum);
    XTensor ty = MulAndShift(tx, tw, tb);
    if (ty.order != 2 || ty.dimSize[0] != rows || ty.dimSize[1] != out)
        return 1;
    cudaMemcpy(y, ty.data, sizeof(float) * ty.unitNum, cudaMemcpyDeviceToHost);
    return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

/* _CudaBLASMatrixMULList (XTensorBLAS.cu:252-387) on a list of fp32 GPU tensors whose shapes
   differ from item to item (m[i] x k[i] times k[i] x n[i]): the reference loops over single
   cuBLAS calls there, the shim hands the whole list to one grouped launch. Operands and
   results are packed one item after the other in the host arrays. */
int dropin_list_unequal_f32(int dev, int count, const int * m, const int * n, const int * k,
                            const float * a, const float * b, float * c, float alpha, float beta)
{
    std::vector<XTensor *> keep;
    TensorList la, lb, lc;
    size_t oa = 0, ob = 0, oc = 0;
    for (int i = 0; i < count; i++) {
        int da[2] = { m[i], k[i] }, db[2] = { k[i], n[i] }, dc[2] = { m[i], n[i] };
        XTensor * ta = new XTensor(), * tb = new XTensor(), * tc = new XTensor();
        InitTensorV2(ta, 2, da, X_FLOAT, 1.0F, dev);
        InitTensorV2(tb, 2, db, X_FLOAT, 1.0F, dev);
        InitTensorV2(tc, 2, dc, X_FLOAT, 1.0F, dev);
        ta->SetData(a + oa, ta->unitNum);
        tb->SetData(b + ob, tb->unitNum);
        tc->SetData(c + oc, tc->unitNum);
        oa += (size_t)ta->unitNum; ob += (size_t)tb->unitNum; oc += (size_t)tc->unitNum;
        la.Add(ta); lb.Add(tb); lc.Add(tc);
        keep.push_back(ta); keep.push_back(tb); keep.push_back(tc);
    }
    _CudaBLASMatrixMULList(NULL, &la, X_NOTRANS, &lb, X_NOTRANS, &lc, count, alpha, beta);
    oc = 0;
    for (int i = 0; i < count; i++) {
        XTensor * tc = keep[3 * i + 2];
        cudaMemcpy(c + oc, tc->data, sizeof(float) * tc->unitNum, cudaMemcpyDeviceToHost);
        oc += (size_t)tc->unitNum;
    }
    const int rc = cudaGetLastError() == cudaSuccess ? 0 : 2;
    for (size_t i = 0; i < keep.size(); i++)
        delete keep[i];
    return rc;
}

/* MatrixMul(a, tA, b, tB, c, alpha, beta) -- the overload with an existing c and beta != 0
   (MatrixMul.cpp:317) -- on fp32 tensors that live in an XMem pool of GPU `dev`. An int
   tensor of `pad` elements is allocated from the pool first, so the matrices that follow
   start wherever the pool's cursor stands (XMem.cpp:668-686), 16-byte aligned or not.
   Returns 0 on success; *aligned receives 1 when a's address is a multiple of 16. */
int dropin_matmul_beta_in_pool_f32(int dev, int pad, int m, int n, int k, const float * a, const float * b, float * c,
                                   float alpha, float beta, int * aligned)
{
    XMem * mem = new XMem(dev, UNI_FREE, (MTYPE)64 * 1024 * 1024, 1, 0);
    int rc = 0;
    {
        int dp[1] = { pad }, da[2] = { m, k }, db[2] = { k, n }, dc[2] = { m, n };
        XTensor tp, ta, tb, tc;
        InitTensorV2(&tp, 1, dp, X_INT, 1.0F, dev, mem);
        InitTensorV2(&ta, 2, da, X_FLOAT, 1.0F, dev, mem);
        InitTensorV2(&tb, 2, db, X_FLOAT, 1.0F, dev, mem);
        InitTensorV2(&tc, 2, dc, X_FLOAT, 1.0F, dev, mem);
        ta.SetData(a, ta.unitNum);
        tb.SetData(b, tb.unitNum);
        tc.SetData(c, tc.unitNum);
        *aligned = ((size_t)ta.data % 16) == 0 ? 1 : 0;
        MatrixMul(ta, X_NOTRANS, tb, X_NOTRANS, tc, alpha, beta);
        cudaMemcpy(c, tc.data, sizeof(float) * tc.unitNum, cudaMemcpyDeviceToHost);
        rc = cudaGetLastError() == cudaSuccess ? 0 : 2;
    }
    delete mem;
    return rc;
}

/* _CudaBLASMatrixMULBatched (XTensorBLAS.cu:109-178): DEVICE tables of device pointers to
   `count` fp32 matrices of one shape, as cublasGemmBatchedEx took them */
int dropin_batched_pointer_tables_f32(int dev, int count, int m, int n, int k,
                                      const float * a, const float * b, float * c, float alpha, float beta)
{
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(dev);
    float * da = NULL, * db = NULL, * dc = NULL;
    void ** tables = NULL;
    const size_t sa = (size_t)m * k, sb = (size_t)k * n, sc = (size_t)m * n;
    int rc = 2;
    if (cudaMalloc(&da, sizeof(float) * sa * count) == cudaSuccess && cudaMalloc(&db, sizeof(float) * sb * count) == cudaSuccess &&
        cudaMalloc(&dc, sizeof(float) * sc * count) == cudaSuccess && cudaMalloc(&tables, sizeof(void *) * 3 * count) == cudaSuccess) {
        cudaMemcpy(da, a, sizeof(float) * sa * count, cudaMemcpyHostToDevice);
        cudaMemcpy(db, b, sizeof(float) * sb * count, cudaMemcpyHostToDevice);
        cudaMemcpy(dc, c, sizeof(float) * sc * count, cudaMemcpyHostToDevice);
        std::vector<void *> host(3 * count);
        /* an irregular order of the items, so that no stride pattern describes the tables */
        for (int i = 0; i < count; i++) {
            const int j = (i * 5 + 3) % count;
            host[i] = da + sa * j;
            host[count + i] = db + sb * j;
            host[2 * count + i] = dc + sc * j;
        }
        cudaMemcpy(tables, host.data(), sizeof(void *) * 3 * count, cudaMemcpyHostToDevice);
        _CudaBLASMatrixMULBatched(NULL, (const void **)tables, X_NOTRANS, X_FLOAT, (const void **)(tables + count), X_NOTRANS, X_FLOAT,
                                  tables + 2 * count, X_FLOAT, count, m, k, k, n, m, n, alpha, beta);
        cudaMemcpy(c, dc, sizeof(float) * sc * count, cudaMemcpyDeviceToHost);
        rc = cudaGetLastError() == cudaSuccess ? 0 : 2;
    }
    cudaFree(da); cudaFree(db); cudaFree(dc); cudaFree(tables);
    cudaSetDevice(prev);
    return rc;
}

}
