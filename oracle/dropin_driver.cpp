/*
 * TEST INFRASTRUCTURE ONLY. Entry points of the drop-in check library built by
 * `make -C oracle dropin`: the unmodified NiuTensor GPU build (USE_CUDA) in which the
 * reference's matrix-multiplication translation units are replaced by
 * niutensor_b200/host/nts_matmul_shim.cpp + libntb_gemm.so. The functions below run the
 * reference's OWN unit tests for this path (source/tensor/test/TMatrixMul.cpp,
 * TMatrixMul2D.cpp, TMatrixMul2DParallel.cpp, TMatrixMulBatched.cpp -- compiled from where
 * they lie), whose GPU halves now execute on the new kernels, and a half-precision
 * user-level call the reference has no test for.
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

}
