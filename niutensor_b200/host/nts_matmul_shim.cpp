/*
 * Link-level drop-in for NiuTensor's matrix-multiplication translation units.
 *
 * Compile this file against the UNMODIFIED NiuTensor headers (-I<niutensor>/source,
 * -DUSE_CUDA) and link it, together with libntb_gemm.so, IN PLACE OF the reference's
 *     source/tensor/core/arithmetic/MatrixMul.cpp
 *     source/tensor/core/arithmetic/MatrixMul2D.cpp, MatrixMul2D.cu
 *     source/tensor/core/arithmetic/MatrixMulBatched.cpp
 *     source/tensor/core/arithmetic/XTensorBLAS.cpp, XTensorBLAS.cu
 *     source/tensor/core/arithmetic/MulAndShift.cpp
 * It defines every nts:: symbol those files define (declared in MatrixMul.h,
 * MatrixMul2D.h, MatrixMul2D.cuh, MatrixMulBatched.h, XTensorBLAS.h, MulAndShift.h), with the same
 * signatures and default arguments, so sample/fnnlm, sample/transformer, source/network
 * and the reference's own unit tests link and run unchanged. GPU tensors (devID >= 0) are
 * computed by the sm_100a kernels behind include/ntb_gemm.h; the cuBLAS handle arguments
 * are accepted and ignored. Tensors that live on the CPU (devID < 0) are handed to the
 * reference's own CPU routine _MatrixMul2DParallel, which stays in the build untouched
 * (MatrixMul2DParallel.cpp, MatrixMul2DMultiTheading.cpp): this library has no CPU
 * arithmetic of its own.
 *
 * Behaviour kept from the reference: shape checks and their messages; X_TRANS == 0;
 * result placement on a's device and memory pool; SetTMPFlag and the XLink bookkeeping of
 * the user-level calls (MatrixMul.cpp:297-309, MatrixMulBatched.cpp:314-326), without
 * which autograd breaks; errors are fatal through ShowNTErrors. Dropped on purpose: the
 * memset of c when beta == 0 (the kernels never read c then), the per-pair heap XTensor
 * headers of the general form (MatrixMul.cpp:112-146) and the pointer tables with their
 * three synchronous copies (XTensorBLAS.cu:315-347). Not supported on the GPU: sparse
 * operands (MatrixMul2D.cu:49-106) and X_DOUBLE -- both stop with an error.
 */
#include "tensor/XTensor.h"
#include "tensor/XDevice.h"
#include "tensor/XName.h"
#include "tensor/XLink.h"
#include "tensor/XCall.h"
#include "tensor/core/arithmetic/MatrixMul.h"
#include "tensor/core/arithmetic/MatrixMul2D.h"
#include "tensor/core/arithmetic/MatrixMul2D.cuh"
#include "tensor/core/arithmetic/MatrixMul2DParallel.h"
#include "tensor/core/arithmetic/MatrixMulBatched.h"
#include "tensor/core/arithmetic/XTensorBLAS.h"
#include "tensor/core/arithmetic/MulAndShift.h"
#include "tensor/core/arithmetic/Sum.h"
#include "tensor/core/arithmetic/SumDim.h"
#include "tensor/core/math/ScaleAndShift.h"
#include "ntb_gemm.h"

namespace nts {

namespace {

struct Dims2 {
    int rows, cols;         /* stored */
    int n, m;               /* after the transposition flag */
};

Dims2 LastTwo(const XTensor * t, MATRIX_TRANS_TYPE trans)
{
    Dims2 d;
    d.rows = t->dimSize[t->order - 2];
    d.cols = t->dimSize[t->order - 1];
    d.n = trans == X_TRANS ? d.cols : d.rows;
    d.m = trans == X_TRANS ? d.rows : d.cols;
    return d;
}

int LeadingCount(const XTensor * t)
{
    int n = 1;
    for (int i = 0; i < t->order - 2; i++)
        n *= t->dimSize[i];
    return n;
}

void Fatal(int rc, const char * where)
{
    if (rc != NTB_OK) {
        fprintf(stderr, "[ERROR] %s: %s\n", where, ntb_strerror(rc));
        ShowNTErrors("the B200 matrix-multiplication library reported an error");
    }
}

void CheckGpuOperands(const XTensor * a, const XTensor * b, const XTensor * c)
{
    CheckNTErrors(a->devID == b->devID && a->devID == c->devID, "The code must be run on the same GPU!");
    CheckNTErrors(!a->isSparse && !b->isSparse && !c->isSparse, "sparse operands are not supported on the GPU by this library");
}

/* shape of the result of the general form: a.lead + b.lead + [an, bm] */
int GeneralShape(const XTensor & a, MATRIX_TRANS_TYPE tA, const XTensor & b, MATRIX_TRANS_TYPE tB, int * dims)
{
    Dims2 da = LastTwo(&a, tA), db = LastTwo(&b, tB);
    CheckNTErrors(da.m == db.n, "Unmatched tensors in multiplication!");
    int k = 0;
    for (int i = 0; i < a.order - 2; i++)
        dims[k++] = a.dimSize[i];
    for (int i = 0; i < b.order - 2; i++)
        dims[k++] = b.dimSize[i];
    dims[k++] = da.n;
    dims[k++] = db.m;
    return k;
}

int BatchedShape(const XTensor & a, MATRIX_TRANS_TYPE tA, const XTensor & b, MATRIX_TRANS_TYPE tB, int * dims)
{
    Dims2 da = LastTwo(&a, tA), db = LastTwo(&b, tB);
    CheckNTErrors(da.m == db.n, "Unmatched tensors in multiplication!");
    int k = 0;
    for (int i = 0; i < a.order - 2; i++)
        dims[k++] = a.dimSize[i];
    dims[k++] = da.n;
    dims[k++] = db.m;
    return k;
}

/* autograd bookkeeping of the user-level calls: operands, operator id, then the two flags
   and alpha as head parameters (beta is not recorded by the reference either) */
void LinkResult(const XTensor & a, MATRIX_TRANS_TYPE tA, const XTensor & b, MATRIX_TRANS_TYPE tB,
                XTensor & c, DTYPE alpha, int opId)
{
    if (!(a.enableGrad && b.enableGrad))
        return;
    XLink::MakeLink(&a, &b, &c, opId);
    XLink::AddParamToHeadTrans(&c, tA);
    XLink::AddParamToHeadTrans(&c, tB);
    XLink::AddParamToHead(&c, alpha);
}

/* one 2-D product of CPU tensors through the reference's own routine */
void CpuProduct(const XTensor * a, MATRIX_TRANS_TYPE tA, const XTensor * b, MATRIX_TRANS_TYPE tB,
                XTensor * c, DTYPE alpha, DTYPE beta, XPRunner * runner)
{
    CheckNTErrors(a->dataType == DEFAULT_DTYPE && b->dataType == DEFAULT_DTYPE && c->dataType == DEFAULT_DTYPE, "TODO!");
    CheckNTErrors(!a->isSparse && !b->isSparse, "TODO!");
    _MatrixMul2DParallel(a, tA, b, tB, c, alpha, beta, runner);
}

/* `count` CPU products over blocks of three packed tensors; block i of x starts at
   x.data + i * stride_x bytes (stride 0 re-uses a block) */
void CpuBlocks(const XTensor * a, MATRIX_TRANS_TYPE tA, const XTensor * b, MATRIX_TRANS_TYPE tB, XTensor * c,
               int P, int Q, bool outer, DTYPE alpha, DTYPE beta, XPRunner * runner)
{
    Dims2 da = LastTwo(a, tA), db = LastTwo(b, tB), dc = LastTwo(c, X_NOTRANS);
    XTensor * a2 = NewTensor2DV2(da.rows, -da.cols, a->dataType, a->devID, a->mem);
    XTensor * b2 = NewTensor2DV2(db.rows, -db.cols, b->dataType, b->devID, b->mem);
    XTensor * c2 = NewTensor2DV2(dc.rows, -dc.cols, c->dataType, c->devID, c->mem);
    const size_t aBytes = (size_t)da.rows * da.cols * a->unitSize;
    const size_t bBytes = (size_t)db.rows * db.cols * b->unitSize;
    const size_t cBytes = (size_t)dc.rows * dc.cols * c->unitSize;
    for (int p = 0; p < P; p++) {
        for (int q = 0; q < Q; q++) {
            /* outer: every a block meets every b block; otherwise Q == 1 and block p meets block p */
            a2->data = (char *)a->data + aBytes * p;
            b2->data = (char *)b->data + bBytes * (outer ? q : p);
            c2->data = (char *)c->data + cBytes * ((size_t)p * Q + q);
            CpuProduct(a2, tA, b2, tB, c2, alpha, beta, runner);
        }
    }
    a2->data = NULL; b2->data = NULL; c2->data = NULL;
    delete a2; delete b2; delete c2;
}

}

/* ------------------------------------------------------------------ raw-pointer layer
   (declared in XTensorBLAS.h; the handle is not used) */

void _CudaBLASMatrixMUL(cublasHandle_t * handle,
                        const void * a, MATRIX_TRANS_TYPE transposedA, TENSOR_DATA_TYPE dataTypeA,
                        const void * b, MATRIX_TRANS_TYPE transposedB, TENSOR_DATA_TYPE dataTypeB,
                        void * c, TENSOR_DATA_TYPE dataTypeC,
                        int na, int ma, int nb, int mb, int nc, int mc, DTYPE alpha, DTYPE beta)
{
    (void)handle;
    CheckNTErrors(dataTypeA == dataTypeB, "Unsupported data type!");
    int dev = 0;
    cudaGetDevice(&dev);
    Fatal(ntb_gemm(dev, NULL, a, (int)transposedA, b, (int)transposedB, c, (int)dataTypeA, (int)dataTypeC,
                   na, ma, nb, mb, nc, mc, ma, mb, mc, alpha, beta), "_CudaBLASMatrixMUL");
}

void _CudaBLASMatrixMULBatchedStrided(cublasHandle_t * handle,
                                      const void * a, MATRIX_TRANS_TYPE transposedA, TENSOR_DATA_TYPE dataTypeA, long long int strideA,
                                      const void * b, MATRIX_TRANS_TYPE transposedB, TENSOR_DATA_TYPE dataTypeB, long long int strideB,
                                      void * c, TENSOR_DATA_TYPE dataTypeC, long long int strideC,
                                      int count, int na, int ma, int nb, int mb, int nc, int mc,
                                      DTYPE alpha, DTYPE beta)
{
    (void)handle;
    CheckNTErrors(dataTypeA == dataTypeB, "Unsupported data type!");
    int dev = 0;
    cudaGetDevice(&dev);
    /* a list of one problem carries MAX_INT placeholders as strides (XTensorBLAS.cu:266-268) */
    if (count == 1)
        strideA = strideB = strideC = 0;
    Fatal(ntb_gemm_strided_batched(dev, NULL, a, (int)transposedA, b, (int)transposedB, c,
                                   (int)dataTypeA, (int)dataTypeC, na, ma, nb, mb, nc, mc, ma, mb, mc,
                                   strideA, strideB, strideC, count, alpha, beta),
          "_CudaBLASMatrixMULBatchedStrided");
}

/* a, b, c are DEVICE arrays of device pointers here, as in the reference; they are read
   back once so that the planner can look for a stride pattern. The reference's own callers
   never reach this function once _CudaBLASMatrixMULList is replaced (it builds the tables
   itself); the symbol stays for code that linked to it. The tables must have been written by
   work the device has already finished or that was queued on the legacy default stream
   before this call, as cublasGemmBatchedEx on the handle's stream required. */
void _CudaBLASMatrixMULBatched(cublasHandle_t * handle,
                               const void ** a, MATRIX_TRANS_TYPE transposedA, TENSOR_DATA_TYPE dataTypeA,
                               const void ** b, MATRIX_TRANS_TYPE transposedB, TENSOR_DATA_TYPE dataTypeB,
                               void ** c, TENSOR_DATA_TYPE dataTypeC,
                               int count, int na, int ma, int nb, int mb, int nc, int mc,
                               DTYPE alpha, DTYPE beta)
{
    (void)handle;
    CheckNTErrors(dataTypeA == dataTypeB, "Unsupported data type!");
    if (count <= 0)
        return;
    int dev = 0;
    cudaGetDevice(&dev);
    const void ** ha = new const void *[count];
    const void ** hb = new const void *[count];
    void ** hc = new void *[count];
    /* three copies in flight on the calling thread's default stream, one wait for all */
    cudaMemcpyAsync(ha, a, sizeof(void *) * count, cudaMemcpyDeviceToHost, cudaStreamPerThread);
    cudaMemcpyAsync(hb, b, sizeof(void *) * count, cudaMemcpyDeviceToHost, cudaStreamPerThread);
    cudaMemcpyAsync(hc, c, sizeof(void *) * count, cudaMemcpyDeviceToHost, cudaStreamPerThread);
    cudaStreamSynchronize(cudaStreamPerThread);
    int rc = ntb_gemm_list(dev, NULL, ha, (int)transposedA, hb, (int)transposedB, hc,
                           (int)dataTypeA, (int)dataTypeC, count, na, ma, nb, mb, nc, mc, alpha, beta);
    delete[] ha; delete[] hb; delete[] hc;
    Fatal(rc, "_CudaBLASMatrixMULBatched");
}

void _CudaBLASMatrixMULList(cublasHandle_t * handle, const TensorList * a, MATRIX_TRANS_TYPE transposedA,
                            const TensorList * b, MATRIX_TRANS_TYPE transposedB, TensorList * c,
                            int count, DTYPE alpha, DTYPE beta)
{
    (void)handle;
    CheckNTErrors((a && b && c), "Empty input lists!");
    CheckNTErrors((a->count == b->count && a->count == c->count), "Input lists must be of the same size!");
    if (a->count == 0)
        return;
    count = a->count;
    XTensor * a0 = (XTensor *)a->GetItem(0);
    XTensor * b0 = (XTensor *)b->GetItem(0);
    XTensor * c0 = (XTensor *)c->GetItem(0);
    bool uniform = true;
    for (int i = 1; i < count && uniform; i++) {
        XTensor * ai = (XTensor *)a->GetItem(i);
        XTensor * bi = (XTensor *)b->GetItem(i);
        XTensor * ci = (XTensor *)c->GetItem(i);
        uniform = ai->dimSize[0] == a0->dimSize[0] && ai->dimSize[1] == a0->dimSize[1] &&
                  bi->dimSize[0] == b0->dimSize[0] && bi->dimSize[1] == b0->dimSize[1] &&
                  ci->dimSize[0] == c0->dimSize[0] && ci->dimSize[1] == c0->dimSize[1] &&
                  ai->dataType == a0->dataType && ci->dataType == c0->dataType;
    }
    if (uniform) {
        const void ** ha = new const void *[count];
        const void ** hb = new const void *[count];
        void ** hc = new void *[count];
        for (int i = 0; i < count; i++) {
            ha[i] = ((XTensor *)a->GetItem(i))->data;
            hb[i] = ((XTensor *)b->GetItem(i))->data;
            hc[i] = ((XTensor *)c->GetItem(i))->data;
        }
        int rc = ntb_gemm_list(a0->devID, NULL, ha, (int)transposedA, hb, (int)transposedB, hc,
                               (int)a0->dataType, (int)c0->dataType, count,
                               a0->dimSize[0], a0->dimSize[1], b0->dimSize[0], b0->dimSize[1],
                               c0->dimSize[0], c0->dimSize[1], alpha, beta);
        delete[] ha; delete[] hb; delete[] hc;
        Fatal(rc, "_CudaBLASMatrixMULList");
        return;
    }
    /* shapes differ: one grouped launch per eight items instead of the reference's loop of
       single calls (XTensorBLAS.cu:373-385); items of another data type or device go out alone */
    {
        const void ** ha = new const void *[count];
        const void ** hb = new const void *[count];
        void ** hc = new void *[count];
        int * dims = new int[6 * count];
        int n = 0;
        for (int i = 0; i < count; i++) {
            XTensor * ai = (XTensor *)a->GetItem(i);
            XTensor * bi = (XTensor *)b->GetItem(i);
            XTensor * ci = (XTensor *)c->GetItem(i);
            if (ai->dataType != a0->dataType || ci->dataType != c0->dataType || ai->devID != a0->devID) {
                Fatal(ntb_gemm(ai->devID, NULL, ai->data, (int)transposedA, bi->data, (int)transposedB, ci->data,
                               (int)ai->dataType, (int)ci->dataType, ai->dimSize[0], ai->dimSize[1],
                               bi->dimSize[0], bi->dimSize[1], ci->dimSize[0], ci->dimSize[1],
                               ai->dimSize[1], bi->dimSize[1], ci->dimSize[1], alpha, beta),
                      "_CudaBLASMatrixMULList");
                continue;
            }
            ha[n] = ai->data; hb[n] = bi->data; hc[n] = ci->data;
            dims[0 * count + n] = ai->dimSize[0]; dims[1 * count + n] = ai->dimSize[1];
            dims[2 * count + n] = bi->dimSize[0]; dims[3 * count + n] = bi->dimSize[1];
            dims[4 * count + n] = ci->dimSize[0]; dims[5 * count + n] = ci->dimSize[1];
            n++;
        }
        int rc = ntb_gemm_grouped(a0->devID, NULL, n, ha, (int)transposedA, hb, (int)transposedB, hc,
                                  (int)a0->dataType, (int)c0->dataType, dims, dims + count, dims + 2 * count,
                                  dims + 3 * count, dims + 4 * count, dims + 5 * count, alpha, beta);
        delete[] ha; delete[] hb; delete[] hc; delete[] dims;
        Fatal(rc, "_CudaBLASMatrixMULList");
    }
}

/* CPU BLAS entry of the reference (XTensorBLAS.cpp:39): kept as a name; routed to the
   reference's built-in CPU routine, which is right for all four transposition pairs */
void _MatrixMULCPU(const XTensor * a, MATRIX_TRANS_TYPE transposedA, const XTensor * b, MATRIX_TRANS_TYPE transposedB,
                   XTensor * c, DTYPE alpha, DTYPE beta)
{
    CpuProduct(a, transposedA, b, transposedB, c, alpha, beta, NULL);
}

/* ------------------------------------------------------------------ 2-D */

void _CudaMatrixMul2D(const XTensor * a, MATRIX_TRANS_TYPE transposedA, const XTensor * b, MATRIX_TRANS_TYPE transposedB,
                      XTensor * c, DTYPE alpha, DTYPE beta)
{
    CheckNTErrors((a && b && c), "Empty input tensors!");
    CheckNTErrors((a->order == 2 && b->order == 2 && c->order == 2), "Input tensors must have a order = 2!");
    CheckGpuOperands(a, b, c);
    Dims2 da = LastTwo(a, transposedA), db = LastTwo(b, transposedB);
    CheckNTErrors((da.m == db.n && da.n == c->dimSize[0] && db.m == c->dimSize[1]), "Unmatched tensors in multiplication!");
    Fatal(ntb_gemm(a->devID, NULL, a->data, (int)transposedA, b->data, (int)transposedB, c->data,
                   (int)a->dataType, (int)c->dataType, da.rows, da.cols, db.rows, db.cols,
                   c->dimSize[0], c->dimSize[1], da.cols, db.cols, c->dimSize[1], alpha, beta),
          "_CudaMatrixMul2D");
}

void _MatrixMul2D(const XTensor * a, MATRIX_TRANS_TYPE transposedA, const XTensor * b, MATRIX_TRANS_TYPE transposedB,
                  XTensor * c, DTYPE alpha, DTYPE beta, XPRunner * parallelRunner)
{
    CheckNTErrors((a && b && c), "Empty input tensors!");
    CheckNTErrors((a->dataType == b->dataType), "Input tensors should have the same data type!");
    CheckNTErrors((a->order == 2 && b->order == 2 && c->order == 2), "Input tensors must have a order = 2!");
    if (a->devID >= 0 || b->devID >= 0 || c->devID >= 0) {
        _CudaMatrixMul2D(a, transposedA, b, transposedB, c, alpha, beta);
        return;
    }
    Dims2 da = LastTwo(a, transposedA), db = LastTwo(b, transposedB);
    CheckNTErrors((da.m == db.n && da.n == c->dimSize[0] && db.m == c->dimSize[1]), "Unmatched tensors in multiplication!");
    CpuProduct(a, transposedA, b, transposedB, c, alpha, beta, parallelRunner);
}

/* ------------------------------------------------------------------ general form */

void _MatrixMul(const XTensor * a, MATRIX_TRANS_TYPE transposedA, const XTensor * b, MATRIX_TRANS_TYPE transposedB,
                XTensor * c, DTYPE alpha, DTYPE beta, XPRunner * parallelRunner)
{
    CheckNTErrors(a && b && c, "Empty input tensors!");
    CheckNTErrors(a->dataType == b->dataType && a->dataType == c->dataType, "Input tensors should have the same data type!");
    CheckNTErrors(a->order >= 2 && b->order >= 2 && c->order >= 2, "Input tensors must have a order >= 2!");
    CheckNTErrors(c->order == a->order + b->order - 2, "wrong tensor order");

    Dims2 da = LastTwo(a, transposedA), db = LastTwo(b, transposedB), dc = LastTwo(c, X_NOTRANS);
    const bool gpu = a->devID >= 0 && b->devID >= 0 && c->devID >= 0;

    /* higher-order a against a matrix: the leading extents of a and c fold into rows */
    if (transposedA == X_NOTRANS && a->order > 2 && b->order == 2) {
        const int rowsA = a->unitNum / da.cols, rowsC = c->unitNum / dc.cols;
        CheckNTErrors((da.m == db.n && rowsA == rowsC && db.m == dc.cols), "Unmatched tensors in multiplication!");
        if (gpu) {
            CheckGpuOperands(a, b, c);
            Fatal(ntb_gemm(a->devID, NULL, a->data, (int)transposedA, b->data, (int)transposedB, c->data,
                           (int)a->dataType, (int)c->dataType, rowsA, da.cols, db.rows, db.cols, rowsC, dc.cols,
                           da.cols, db.cols, dc.cols, alpha, beta), "_MatrixMul");
        }
        else {
            XTensor * a2 = NewTensor2DV2(rowsA, -da.cols, a->dataType, a->devID, a->mem);
            XTensor * c2 = NewTensor2DV2(rowsC, -dc.cols, c->dataType, c->devID, c->mem);
            a2->data = a->data;
            c2->data = c->data;
            CpuProduct(a2, transposedA, b, transposedB, c2, alpha, beta, parallelRunner);
            a2->data = NULL; c2->data = NULL;
            delete a2; delete c2;
        }
        return;
    }

    CheckNTErrors((da.m == db.n && da.n == dc.rows && db.m == dc.cols), "Unmatched tensors in multiplication!");
    for (int i = 0; i < a->order - 2; i++)
        CheckNTErrors(a->dimSize[i] == c->dimSize[i], "Incorrect tensor sizes!");
    for (int i = 0; i < b->order - 2; i++)
        CheckNTErrors(b->dimSize[i] == c->dimSize[i - 2 + a->order], "Incorrect tensor sizes!");
    const int P = LeadingCount(a), Q = LeadingCount(b);

    if (gpu) {
        CheckGpuOperands(a, b, c);
        Fatal(ntb_gemm_broadcast(a->devID, NULL, a->data, (int)transposedA, b->data, (int)transposedB, c->data,
                                 (int)a->dataType, (int)c->dataType, da.rows, da.cols, db.rows, db.cols,
                                 dc.rows, dc.cols, P, Q, alpha, beta), "_MatrixMul");
    }
    else {
        CheckNTErrors((a->devID < 0 && b->devID < 0 && c->devID < 0), "The code must be run on the same device!");
        CpuBlocks(a, transposedA, b, transposedB, c, P, Q, true, alpha, beta, parallelRunner);
    }
}

bool CheckMMulShape(const XTensor * a, MATRIX_TRANS_TYPE transposedA, const XTensor * b, MATRIX_TRANS_TYPE transposedB, XTensor * c)
{
    if (!(a && b && c))
        return false;
    if (!(a->dataType == b->dataType && a->dataType == c->dataType))
        return false;
    if (!(a->order >= 2 && b->order >= 2 && c->order >= 2))
        return false;
    int dims[2 * MAX_TENSOR_DIM_NUM];
    const int order = GeneralShape(*a, transposedA, *b, transposedB, dims);
    if (order != c->order)
        return false;
    for (int i = 0; i < order; i++)
        if (dims[i] != c->dimSize[i])
            return false;
    return true;
}

XTensor MatrixMul(const XTensor & a, MATRIX_TRANS_TYPE transposedA, const XTensor & b, MATRIX_TRANS_TYPE transposedB,
                  DTYPE alpha, XPRunner * parallelRunner)
{
    CheckNTErrors(a.dataType == b.dataType, "Input tensors should have the same data type!");
    CheckNTErrors(a.order >= 2 && b.order >= 2, "Input tensors must have a order >= 2!");
    int dims[2 * MAX_TENSOR_DIM_NUM];
    const int order = GeneralShape(a, transposedA, b, transposedB, dims);
    const float dr = (!a.isSparse || !b.isSparse) ? 1.0F : MAX(a.denseRatio, b.denseRatio);
    XTensor c(order, dims, a.dataType, dr, a.devID, a.mem);
    c.SetTMPFlag();
    _MatrixMul(&a, transposedA, &b, transposedB, &c, alpha, 0, parallelRunner);
    LinkResult(a, transposedA, b, transposedB, c, alpha, MATH_MATRIXMUL);
    return c;
}

void MatrixMul(const XTensor & a, MATRIX_TRANS_TYPE transposedA, const XTensor & b, MATRIX_TRANS_TYPE transposedB,
               XTensor & c, DTYPE alpha, DTYPE beta, XPRunner * parallelRunner)
{
    CheckNTErrors(a.dataType == b.dataType, "Input tensors should have the same data type!");
    CheckNTErrors(a.order >= 2 && b.order >= 2, "Input tensors must have a order >= 2!");
    if (!c.isInit || !CheckMMulShape(&a, transposedA, &b, transposedB, &c)) {
        int dims[2 * MAX_TENSOR_DIM_NUM];
        const int order = GeneralShape(a, transposedA, b, transposedB, dims);
        const float dr = (!a.isSparse || !b.isSparse) ? 1.0F : MAX(a.denseRatio, b.denseRatio);
        InitTensorV2(&c, order, dims, a.dataType, dr, a.devID, a.mem);
    }
    _MatrixMul(&a, transposedA, &b, transposedB, &c, alpha, beta, parallelRunner);
    LinkResult(a, transposedA, b, transposedB, c, alpha, MATH_MATRIXMUL);
}

XTensor MatrixMul(const XTensor & a, const XTensor & b, DTYPE alpha, XPRunner * parallelRunner)
{
    return MatrixMul(a, X_NOTRANS, b, X_NOTRANS, alpha, parallelRunner);
}

void MatrixMul(const XTensor & a, const XTensor & b, XTensor & c, DTYPE alpha, XPRunner * parallelRunner)
{
    MatrixMul(a, X_NOTRANS, b, X_NOTRANS, c, alpha, 0, parallelRunner);
}

/* ------------------------------------------------------------------ batched form */

void _MatrixMulBatchedGPU(const XTensor * a, MATRIX_TRANS_TYPE transposedA, const XTensor * b, MATRIX_TRANS_TYPE transposedB,
                          XTensor * c, DTYPE alpha, DTYPE beta)
{
    CheckNTErrors((a && b && c), "Empty input tensors!");
    CheckNTErrors((a->dataType == b->dataType && a->dataType == c->dataType), "Input tensors should have the same data type!");
    CheckNTErrors((a->order >= 2 && b->order >= 2 && c->order >= 2), "Input tensors must have a order >= 2!");
    CheckNTErrors((a->order == b->order && a->order == c->order), "Input tensor and output tensor must have same order!");
    CheckNTErrors(a->devID >= 0 && b->devID >= 0 && c->devID >= 0, "The tensors must be on GPUs");
    CheckGpuOperands(a, b, c);
    Dims2 da = LastTwo(a, transposedA), db = LastTwo(b, transposedB), dc = LastTwo(c, X_NOTRANS);
    CheckNTErrors((da.m == db.n && da.n == dc.rows && db.m == dc.cols), "Unmatched tensors in multiplication!");
    for (int i = 0; i < a->order - 2; i++) {
        CheckNTErrors((a->dimSize[i] == b->dimSize[i]), "Incorrect tensor sizes!");
        CheckNTErrors((a->dimSize[i] == c->dimSize[i]), "Incorrect tensor sizes!");
    }
    const int count = LeadingCount(a);
    Fatal(ntb_gemm_strided_batched(a->devID, NULL, a->data, (int)transposedA, b->data, (int)transposedB, c->data,
                                   (int)a->dataType, (int)c->dataType, da.rows, da.cols, db.rows, db.cols,
                                   dc.rows, dc.cols, da.cols, db.cols, dc.cols,
                                   (long long)da.rows * da.cols, (long long)db.rows * db.cols,
                                   (long long)dc.rows * dc.cols, count, alpha, beta), "_MatrixMulBatchedGPU");
}

void _MatrixMulBatchedCPU(const XTensor * a, MATRIX_TRANS_TYPE transposedA, const XTensor * b, MATRIX_TRANS_TYPE transposedB,
                          XTensor * c, DTYPE alpha, DTYPE beta)
{
    CheckNTErrors((a && b && c), "Empty input tensors!");
    CheckNTErrors((a->order == b->order && a->order == c->order), "Input tensor and output tensor must have same order!");
    Dims2 da = LastTwo(a, transposedA), db = LastTwo(b, transposedB), dc = LastTwo(c, X_NOTRANS);
    CheckNTErrors((da.m == db.n && da.n == dc.rows && db.m == dc.cols), "Unmatched tensors in multiplication!");
    for (int i = 0; i < a->order - 2; i++) {
        CheckNTErrors((a->dimSize[i] == b->dimSize[i]), "Incorrect tensor sizes!");
        CheckNTErrors((a->dimSize[i] == c->dimSize[i]), "Incorrect tensor sizes!");
    }
    CpuBlocks(a, transposedA, b, transposedB, c, LeadingCount(a), 1, false, alpha, beta, NULL);
}

void _MatrixMulBatchedCPU(const TensorList * a, MATRIX_TRANS_TYPE transposedA, const TensorList * b, MATRIX_TRANS_TYPE transposedB,
                          TensorList * c, DTYPE alpha, DTYPE beta)
{
    CheckNTErrors(a && b && c, "Empty input lists!");
    CheckNTErrors(a->count == b->count && a->count == c->count, "Input lists must be of the same size!");
    for (int i = 0; i < a->count; i++) {
        XTensor * ai = (XTensor *)a->GetItem(i);
        XTensor * bi = (XTensor *)b->GetItem(i);
        XTensor * ci = (XTensor *)c->GetItem(i);
        CheckNTErrors((ai->order == 2 && bi->order == 2 && ci->order == 2), "2d tensor (i.e., matrix) is required!");
        CpuProduct(ai, transposedA, bi, transposedB, ci, alpha, beta, NULL);
    }
}

void _MatrixMulBatched(const XTensor * a, MATRIX_TRANS_TYPE transposedA, const XTensor * b, MATRIX_TRANS_TYPE transposedB,
                       XTensor * c, DTYPE alpha, DTYPE beta, XPRunner * parallelRunner)
{
    (void)parallelRunner;
    CheckNTErrors((a && b && c), "Empty input tensors!");
    CheckNTErrors((a->dataType == b->dataType && a->dataType == c->dataType), "Input tensors should have the same data type!");
    CheckNTErrors((a->order >= 2 && b->order >= 2 && c->order >= 2), "Input tensors must have a order >= 2!");
    CheckNTErrors((a->order == b->order && a->order == c->order), "Input tensor and output tensor must have same order!");
    if (a->devID >= 0 || b->devID >= 0 || c->devID >= 0)
        _MatrixMulBatchedGPU(a, transposedA, b, transposedB, c, alpha, beta);
    else
        _MatrixMulBatchedCPU(a, transposedA, b, transposedB, c, alpha, beta);
}

XTensor MatrixMulBatched(const XTensor & a, MATRIX_TRANS_TYPE transposedA, const XTensor & b, MATRIX_TRANS_TYPE transposedB,
                         DTYPE alpha, XPRunner * parallelRunner)
{
    CheckNTErrors(a.dataType == b.dataType, "Input tensors should have the same data type!");
    CheckNTErrors(a.order >= 2 && b.order >= 2, "Input tensors must have a order >= 2!");
    CheckNTErrors(a.order == b.order, "Input tensor and output tensor must have same order!");
    int dims[MAX_TENSOR_DIM_NUM];
    const int order = BatchedShape(a, transposedA, b, transposedB, dims);
    const float dr = (!a.isSparse || !b.isSparse) ? 1.0F : MAX(a.denseRatio, b.denseRatio);
    XTensor c(order, dims, a.dataType, dr, a.devID, a.mem);
    c.SetTMPFlag();
    _MatrixMulBatched(&a, transposedA, &b, transposedB, &c, alpha, 0, parallelRunner);
    LinkResult(a, transposedA, b, transposedB, c, alpha, MATH_MATRIXMULBATCHED);
    return c;
}

XTensor MatrixMulBatched(const XTensor & a, const XTensor & b, DTYPE alpha, XPRunner * parallelRunner)
{
    return MatrixMulBatched(a, X_NOTRANS, b, X_NOTRANS, alpha, parallelRunner);
}

/* ------------------------------------------------------------------ MulAndShift
   x * w + b (MulAndShift.cpp:38-110, 120-188). On the GPU, with the usual bias vector over
   the last dimension, product and bias are one kernel (the reference writes the product to
   a scratch tensor, then _SumDim reads and rewrites it). Every other case -- CPU tensors, a
   scalar b, a bias along another dimension -- runs the product into c and lets the
   reference's own _SumDim / ScaleAndShift add b in place. */

namespace {

XTensor MulAndShiftImpl(const XTensor & x, MATRIX_TRANS_TYPE tX, const XTensor & w, MATRIX_TRANS_TYPE tW,
                        const XTensor & b, DTYPE alpha, XPRunner * runner)
{
    CheckNTErrors(x.dataType == w.dataType, "Input tensors should have the same data type!");
    CheckNTErrors(x.order >= 2 && w.order >= 2, "Input tensors must have a order >= 2!");
    int dims[2 * MAX_TENSOR_DIM_NUM];
    const int order = GeneralShape(x, tX, w, tW, dims);
    const float dr = (!x.isSparse || !w.isSparse) ? 1.0F : MAX(x.denseRatio, w.denseRatio);
    XTensor c(order, dims, x.dataType, dr, x.devID, x.mem);
    c.SetTMPFlag();

    int n = -2;
    if (b.order > 0) {
        n = GetBroadcastDimIndex(c, b);
        CheckNTErrors(n != -1, "TODO!");
        CheckNTErrors(n >= 0 && n < c.order, "Something is wrong!");
    }

    const bool gpu = x.devID >= 0 && w.devID >= 0 && b.devID >= 0;
    const bool fusable = gpu && b.order == 1 && n == c.order - 1 && b.dataType == c.dataType &&
                         w.order == 2 && (x.order == 2 || tX == X_NOTRANS) && !x.isSparse && !w.isSparse;
    if (fusable) {
        CheckNTErrors(x.devID == w.devID && x.devID == b.devID, "The code must be run on the same GPU!");
        const int xCols = x.dimSize[x.order - 1];
        const int xRows = x.unitNum / xCols;            /* leading extents fold into rows */
        const int cCols = c.dimSize[c.order - 1];
        const int cRows = c.unitNum / cCols;
        Fatal(ntb_gemm_bias_act(x.devID, NULL, x.data, (int)tX, w.data, (int)tW, b.data, c.data,
                                (int)x.dataType, (int)c.dataType, xRows, xCols, w.dimSize[0], w.dimSize[1],
                                cRows, cCols, xCols, w.dimSize[1], cCols, alpha, 0, NTB_ACT_NONE), "MulAndShift");
    }
    else {
        _MatrixMul(&x, tX, &w, tW, &c, alpha, 0, runner);
        if (b.order == 0)
            _ScaleAndShiftMe(&c, 1.0F, b.Get0D());
        else
            _SumDim(&c, &b, n);
    }

    if (b.order > 0 && w.enableGrad && b.enableGrad) {
        XLink::MakeLink(&x, &w, &b, &c, MATH_MULANDSHIFT);
        XLink::AddParamToHeadInt(&c, n);
        XLink::AddParamToHeadTrans(&c, tX);
        XLink::AddParamToHeadTrans(&c, tW);
        XLink::AddParamToHead(&c, alpha);
    }
    return c;
}

}

XTensor MulAndShift(const XTensor & x, const XTensor & w, const XTensor & b, DTYPE alpha, XPRunner * parallelRunner)
{
    return MulAndShiftImpl(x, X_NOTRANS, w, X_NOTRANS, b, alpha, parallelRunner);
}

XTensor MulAndShift(const XTensor & x, MATRIX_TRANS_TYPE transposedX, const XTensor & w, MATRIX_TRANS_TYPE transposedW,
                    const XTensor & b, DTYPE alpha, XPRunner * parallelRunner)
{
    return MulAndShiftImpl(x, transposedX, w, transposedW, b, alpha, parallelRunner);
}

}
