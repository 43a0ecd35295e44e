/*
 * TEST INFRASTRUCTURE ONLY -- never linked, loaded or called by the product path.
 *
 * Plain-C restatement of NiuTensor's built-in fp32 CPU matrix multiplication, the
 * path the reference takes for dense X_FLOAT tensors on devID < 0 when it is built
 * without USE_BLAS. Parity status: PINNED -- tests/test_oracle.py checks every
 * function here against the known-answer vectors of the reference's own unit tests
 * (source/tensor/test/TMatrixMul.cpp, TMatrixMul2D.cpp, TMatrixMul2DParallel.cpp,
 * TMatrixMulBatched.cpp) and, where the compiled reference is present under
 * oracle/_ref/, bit-for-bit against the reference library on seeded inputs.
 *
 * Accumulation order and the placement of alpha are kept exactly as the reference
 * has them, so fp32 results are bit-identical to it when compiled without FMA
 * contraction (-ffp-contract=off, the x86-64 default of the reference's g++ -O2).
 *
 * Transposition flags use the reference's enum values
 * (source/tensor/XDataType.h:36): 0 = X_TRANS, 1 = X_NOTRANS.
 */
#include <stddef.h>
#include <string.h>
#include <pthread.h>
#include <math.h>
#include <stdlib.h>

#define ORC_TRANS 0
#define ORC_NOTRANS 1

/* Rows of C are independent, so spreading the row loop over host threads leaves
   every element's accumulation order -- and therefore every bit -- unchanged
   (orc_matmul2d_f32 below hands row ranges to pthreads). The
   reference itself runs this loop on one thread (it never creates an XPRunner). */
static int orc_threads = 1;
void orc_set_threads(int n)
{
    orc_threads = n > 0 ? n : 1;
}

/*
 * One dense 2-D product  c = op(a) * op(b) * alpha + c * beta.
 * a is na x ma, b is nb x mb, c is nc x mc, all stored row-major and packed.
 *
 * N/N follows source/tensor/core/arithmetic/MatrixMul2DMultiTheading.cpp:66-145
 * (four variants by beta == 0 and alpha == 1: alpha multiplies every product inside
 * the k loop unless it is exactly 1; C is overwritten when beta == 0, otherwise
 * c*beta + r). The other three combinations follow
 * source/tensor/core/arithmetic/MatrixMul2DParallel.cpp:69-128: C is zeroed first
 * when beta == 0 (:56-57), alpha always multiplies inside the k loop, and the
 * result is c*beta + r.
 */
static void orc_rows_f32(int i0, int i1,
                         const float * a, int transA, const float * b, int transB, float * c,
                         int na, int ma, int nb, int mb, int nc, int mc,
                         float alpha, float beta)
{
    int i, j, k;
    (void)nb;
    (void)nc;
    if (transA == ORC_NOTRANS && transB == ORC_NOTRANS) {
        int num = ma;
        for (i = i0; i < i1; i++) {
            for (j = 0; j < mc; j++) {
                float r = 0;
                const float * p1 = a + (size_t)i * ma;
                const float * p2 = b + j;
                if (alpha == 1) {
                    for (k = 0; k < num; k++) {
                        r += (*p1) * (*p2);
                        p1 += 1;
                        p2 += mb;
                    }
                }
                else {
                    for (k = 0; k < num; k++) {
                        r += (*p1) * (*p2) * alpha;
                        p1 += 1;
                        p2 += mb;
                    }
                }
                if (beta == 0)
                    c[(size_t)i * mc + j] = r;
                else
                    c[(size_t)i * mc + j] = c[(size_t)i * mc + j] * beta + r;
            }
        }
        return;
    }

    if (beta == 0)
        memset(c + (size_t)i0 * mc, 0, sizeof(float) * (size_t)(i1 - i0) * mc);

    {
        /* k extent and the strides that walk k in a and b */
        int num = (transA == ORC_TRANS) ? na : ma;
        ptrdiff_t aStepK = (transA == ORC_TRANS) ? ma : 1;
        ptrdiff_t aStepI = (transA == ORC_TRANS) ? 1 : ma;
        ptrdiff_t bStepK = (transB == ORC_TRANS) ? 1 : mb;
        ptrdiff_t bStepJ = (transB == ORC_TRANS) ? mb : 1;
        for (i = i0; i < i1; i++) {
            for (j = 0; j < mc; j++) {
                float r = 0;
                const float * p1 = a + i * aStepI;
                const float * p2 = b + j * bStepJ;
                for (k = 0; k < num; k++) {
                    r += (*p1) * (*p2) * alpha;
                    p1 += aStepK;
                    p2 += bStepK;
                }
                c[(size_t)i * mc + j] = c[(size_t)i * mc + j] * beta + r;
            }
        }
    }
}

struct orc_job {
    int i0, i1;
    const float * a; int transA; const float * b; int transB; float * c;
    int na, ma, nb, mb, nc, mc;
    float alpha, beta;
};

static void * orc_job_main(void * arg)
{
    struct orc_job * j = (struct orc_job *)arg;
    orc_rows_f32(j->i0, j->i1, j->a, j->transA, j->b, j->transB, j->c,
                 j->na, j->ma, j->nb, j->mb, j->nc, j->mc, j->alpha, j->beta);
    return NULL;
}

void orc_matmul2d_f32(const float * a, int transA, const float * b, int transB, float * c,
                      int na, int ma, int nb, int mb, int nc, int mc,
                      float alpha, float beta)
{
    enum { MAXT = 256 };
    pthread_t tid[MAXT];
    struct orc_job job[MAXT];
    int nt = orc_threads < MAXT ? orc_threads : MAXT;
    int t, started = 0;
    if (nt > nc)
        nt = nc;
    if (nt <= 1) {
        orc_rows_f32(0, nc, a, transA, b, transB, c, na, ma, nb, mb, nc, mc, alpha, beta);
        return;
    }
    for (t = 0; t < nt; t++) {
        struct orc_job * j = &job[t];
        j->i0 = (int)((long long)nc * t / nt);
        j->i1 = (int)((long long)nc * (t + 1) / nt);
        j->a = a; j->transA = transA; j->b = b; j->transB = transB; j->c = c;
        j->na = na; j->ma = ma; j->nb = nb; j->mb = mb; j->nc = nc; j->mc = mc;
        j->alpha = alpha; j->beta = beta;
        if (pthread_create(&tid[t], NULL, orc_job_main, j) != 0)
            break;
        started++;
    }
    /* rows whose thread could not be created are done here */
    for (t = started; t < nt; t++)
        orc_job_main(&job[t]);
    for (t = 0; t < started; t++)
        pthread_join(tid[t], NULL);
}

/*
 * Batched form: c_i = op(a_i) * op(b_i) * alpha + c_i * beta for i < count, the
 * three tensors holding `count` packed matrices back to back
 * (source/tensor/core/arithmetic/MatrixMulBatched.cpp:157-218: blockNum is the
 * product of the leading extents, every block re-points three 2-D headers).
 */
void orc_matmul_batched_f32(const float * a, int transA, const float * b, int transB, float * c,
                            int count, int na, int ma, int nb, int mb, int nc, int mc,
                            float alpha, float beta)
{
    int i;
    for (i = 0; i < count; i++)
        orc_matmul2d_f32(a + (size_t)i * na * ma, transA, b + (size_t)i * nb * mb, transB,
                         c + (size_t)i * nc * mc, na, ma, nb, mb, nc, mc, alpha, beta);
}

/*
 * General form of _MatrixMul (source/tensor/core/arithmetic/MatrixMul.cpp:52-208):
 * every leading block p of a (aBlockNum of them) meets every leading block q of b
 * (bBlockNum); the product lands in block p * bBlockNum + q of c (:121-125).
 * The 2-D "flatten" shortcut (:65-77: transA == X_NOTRANS, a.order > 2, b.order == 2)
 * is the same arithmetic with aBlockNum folded into na, which callers express by
 * passing aBlockNum = 1 and na = rows * blocks.
 */
void orc_matmul_broadcast_f32(const float * a, int transA, const float * b, int transB, float * c,
                              int aBlockNum, int bBlockNum,
                              int na, int ma, int nb, int mb, int nc, int mc,
                              float alpha, float beta)
{
    int p, q;
    for (p = 0; p < aBlockNum; p++)
        for (q = 0; q < bBlockNum; q++)
            orc_matmul2d_f32(a + (size_t)p * na * ma, transA, b + (size_t)q * nb * mb, transB,
                             c + ((size_t)p * bBlockNum + q) * nc * mc,
                             na, ma, nb, mb, nc, mc, alpha, beta);
}

/*
 * MulAndShift (source/tensor/core/arithmetic/MulAndShift.cpp:38-110, 120-188): the product
 * alpha * op(x) * op(w) is written to a scratch tensor with beta = 0 (:69), then the bias
 * vector b is added along the last dimension by _SumDim with beta = 1 (:88;
 * source/tensor/core/arithmetic/SumDim.cpp: c = a + b * beta, one fp32 multiply-add per
 * element, b indexed by the column). x holds `blocks` stacked matrices that the flatten
 * rule of _MatrixMul folds into rows when x is not transposed; callers pass the folded
 * row count. rectify != 0 applies the reference's Rectify afterwards (max(x, 0),
 * source/tensor/function/Rectify.cpp), the next operator of the feed-forward layer.
 */
void orc_mulandshift_f32(const float * x, int transX, const float * w, int transW, const float * b,
                         float * c, int nx, int mx, int nw, int mw, int nc, int mc,
                         float alpha, int rectify)
{
    int i, j;
    orc_matmul2d_f32(x, transX, w, transW, c, nx, mx, nw, mw, nc, mc, alpha, 0.0f);
    for (i = 0; i < nc; i++) {
        for (j = 0; j < mc; j++) {
            float v = c[(size_t)i * mc + j] + b[j] * 1.0f;
            if (rectify && v < 0)
                v = 0;
            c[(size_t)i * mc + j] = v;
        }
    }
}

/*
 * Scaled-dot-product attention as the transformer sample composes it in inference
 * (source/sample/transformer/submodel/Attention.cpp:206-238): q is scaled in place (:206),
 * att = BMMul(q, k^T) (:212), the additive mask is summed in (:221-224), Softmax over the
 * last dimension (:227; source/tensor/function/Softmax.cpp:60-115: subtract the row
 * maximum, exp, divide by the row sum, clamp to [0, 1], an all-zero row when the sum is 0),
 * out = BMMul(att, v) (:236). All in fp32 here. The row sum is accumulated left to right;
 * the reference's _ReduceSum sums in vector lanes (source/tensor/core/reduce/
 * ReduceSum.cpp), so this function agrees with the compiled reference to rounding error,
 * not bit for bit -- the test pins it at 1e-6.
 * q: [blocks, lenQ, dim], k, v: [blocks, lenK, dim], mask: NULL or [.., lenQ, lenK] with
 * maskBlockStride elements between blocks (0 = one mask for all), out: [blocks, lenQ, dim].
 */
void orc_attention_dropout_f32(const float * q, const float * k, const float * v, const float * mask,
                               const unsigned char * keep, float keepScale, float * out,
                               int blocks, int lenQ, int lenK, int dim, long long maskBlockStride, float scale)
{
    int b, i, j;
    float * qs = (float *)malloc(sizeof(float) * (size_t)lenQ * dim);
    float * att = (float *)malloc(sizeof(float) * (size_t)lenQ * lenK);
    for (b = 0; b < blocks; b++) {
        const float * qb = q + (size_t)b * lenQ * dim;
        const float * kb = k + (size_t)b * lenK * dim;
        const float * vb = v + (size_t)b * lenK * dim;
        const float * mb = mask ? mask + (size_t)b * maskBlockStride : NULL;
        for (i = 0; i < lenQ * dim; i++)
            qs[i] = qb[i] * scale;
        orc_matmul2d_f32(qs, ORC_NOTRANS, kb, ORC_TRANS, att, lenQ, dim, lenK, dim, lenQ, lenK, 1.0f, 0.0f);
        for (i = 0; i < lenQ; i++) {
            float * row = att + (size_t)i * lenK;
            float mx, sum = 0;
            if (mb)
                for (j = 0; j < lenK; j++)
                    row[j] = row[j] + mb[(size_t)i * lenK + j];
            mx = row[0];
            for (j = 1; j < lenK; j++)
                if (row[j] > mx)
                    mx = row[j];
            for (j = 0; j < lenK; j++)
                sum += (float)exp(row[j] - mx);
            for (j = 0; j < lenK; j++) {
                float r = 0;
                if (sum != 0) {
                    r = (float)exp(row[j] - mx) / sum;
                    if (r > 1.0f)
                        r = 1.0f;
                    else if (r < 0)
                        r = 0;
                }
                /* training: Dropout on the probabilities (Attention.cpp:229-230), i.e. a product
                   with a mask of zeros and 1 / (1 - p) (source/tensor/function/Dropout.cpp:148-158) */
                if (keep)
                    r = r * (keep[((size_t)b * lenQ + i) * lenK + j] ? keepScale : 0.0f);
                row[j] = r;
            }
        }
        orc_matmul2d_f32(att, ORC_NOTRANS, vb, ORC_NOTRANS, out + (size_t)b * lenQ * dim,
                         lenQ, lenK, lenK, dim, lenQ, dim, 1.0f, 0.0f);
    }
    free(qs);
    free(att);
}

void orc_attention_f32(const float * q, const float * k, const float * v, const float * mask, float * out,
                       int blocks, int lenQ, int lenK, int dim, long long maskBlockStride, float scale)
{
    orc_attention_dropout_f32(q, k, v, mask, NULL, 1.0f, out, blocks, lenQ, lenK, dim, maskBlockStride, scale);
}

/*
 * LogSoftmax over the last dimension as the reference's CPU path computes it
 * (source/tensor/function/LogSoftmax.cpp:87-88, 123-148): row maximum, row sum of
 * exp(x - max), then r = log(exp(x - max) / sum); NaN and infinities become LOGPROB_MIN
 * (-20, source/tensor/XGlobal.h:69) and r is floored at LOGPROB_MIN; a row whose sum is 0
 * becomes zeros; a dimension of size 1 gives zeros (:50-53). The row sum is accumulated
 * left to right here (the reference sums in vector lanes): agreement to rounding error.
 */
void orc_logsoftmax_f32(const float * x, float * y, int rows, int cols)
{
    int i, j;
    for (i = 0; i < rows; i++) {
        const float * ip = x + (size_t)i * cols;
        float * op = y + (size_t)i * cols;
        float mx = ip[0], sum = 0;
        if (cols == 1) {
            op[0] = 0;
            continue;
        }
        for (j = 1; j < cols; j++)
            if (ip[j] > mx)
                mx = ip[j];
        for (j = 0; j < cols; j++)
            sum += (float)exp(ip[j] - mx);
        for (j = 0; j < cols; j++) {
            float r = 0;
            if (sum != 0) {
                r = (float)log(exp(ip[j] - mx) / sum);
                if (isnan(r) || isinf(r))
                    r = -20.0f;
                if (r < -20.0f)
                    r = -20.0f;
            }
            op[j] = r;
        }
    }
}
