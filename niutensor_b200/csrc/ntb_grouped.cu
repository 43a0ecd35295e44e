/*
 * Lists of products of UNEQUAL shapes in one launch. The reference issues one cuBLAS call per
 * item when the shapes of a list differ (source/tensor/core/arithmetic/XTensorBLAS.cu:373-385);
 * here up to GROUP_MAX problems share one persistent launch of the single-CTA kernel, whose
 * tile walk runs through the tiles of the first problem, then of the second, and so on, so
 * small products fill the SMs together instead of one after the other. Longer lists take
 * several launches; items TMA cannot address, and items with K = 0, go out on their own.
 */
#include "ntb_tc_single.cuh"
#include <cstring>

namespace ntb {

int LaunchWideGroup(const TcGroupWide & grp, int mode, int dtC, bool oldc, int smCount, cudaStream_t stream)
{
#define NTB_WIDE(MD, ST, GG, T) (oldc ? LaunchOne<MD, 128, ST, GG, T, true, false, GROUP_MAX>(grp, smCount, stream) \
                                      : LaunchOne<MD, 128, ST, GG, T, false, false, GROUP_MAX>(grp, smCount, stream))
    if (mode == 0)
        return dtC == NTB_X_FLOAT16 ? NTB_WIDE(0, 6, 2, __half) : NTB_WIDE(0, 6, 2, float);
    return NTB_WIDE(1, 3, 1, float);
#undef NTB_WIDE
}

}

using namespace ntb;

extern "C" int ntb_gemm_grouped(int devID, void * stream, int count,
                                const void * const * a, int transA, const void * const * b, int transB, void * const * c,
                                int dtypeAB, int dtypeC,
                                const int * na, const int * ma, const int * nb, const int * mb, const int * nc, const int * mc,
                                float alpha, float beta)
{
    if (count < 0)
        return NTB_ERR_ARG;
    if (count == 0)
        return NTB_OK;
    if (!a || !b || !c || !na || !ma || !nb || !mb || !nc || !mc)
        return NTB_ERR_ARG;
    if ((transA != NTB_X_TRANS && transA != NTB_X_NOTRANS) || (transB != NTB_X_TRANS && transB != NTB_X_NOTRANS))
        return NTB_ERR_ARG;
    if (!((dtypeAB == NTB_X_FLOAT16 && (dtypeC == NTB_X_FLOAT16 || dtypeC == NTB_X_FLOAT)) ||
          (dtypeAB == NTB_X_FLOAT && dtypeC == NTB_X_FLOAT)))
        return NTB_ERR_DTYPE;
    /* all shapes are checked before anything is launched */
    for (int i = 0; i < count; i++) {
        if (na[i] < 0 || ma[i] < 0 || nb[i] < 0 || mb[i] < 0 || nc[i] < 0 || mc[i] < 0)
            return NTB_ERR_ARG;
        const int an = transA == NTB_X_TRANS ? ma[i] : na[i], am = transA == NTB_X_TRANS ? na[i] : ma[i];
        const int bn = transB == NTB_X_TRANS ? mb[i] : nb[i], bm = transB == NTB_X_TRANS ? nb[i] : mb[i];
        if (am != bn || an != nc[i] || bm != mc[i])
            return NTB_ERR_SHAPE;
        if (nc[i] > 0 && mc[i] > 0 && (!c[i] || (am > 0 && (!a[i] || !b[i]))))
            return NTB_ERR_ARG;                     /* empty operands (K = 0) may be NULL */
    }
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess || (prev != devID && cudaSetDevice(devID) != cudaSuccess)) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    int rc = NTB_OK;
    DeviceCtx * ctx = CtxFor(devID);
    if (!ctx)
        rc = NTB_ERR_CUDA;
    const int mode = dtypeAB == NTB_X_FLOAT16 ? 0 : 1;
    const bool oldc = beta != 0.f;
    const bool grouping = ForcedRoute() == 0;
    TcGroupWide grp;
    grp.n = 0;
    grp.total = 0;
    grp.first[0] = 0;
    auto flush = [&]() -> int {
        if (grp.n == 0)
            return NTB_OK;
        for (int k = grp.n; k <= GROUP_MAX; k++)
            grp.first[k] = grp.total;
        for (int k = grp.n; k < GROUP_MAX; k++) {          /* unused slots: harmless copies */
            grp.p[k] = grp.p[0];
            for (int m = 0; m < 3; m++)
                grp.tm[k][m] = grp.tm[0][m];
        }
        const int r = LaunchWideGroup(grp, mode, dtypeC, oldc, ctx->smCount, (cudaStream_t)stream);
        if (r == NTB_OK)
            for (int k = 0; k < grp.n; k++)
                SetLastRoute(mode == 0 ? NTB_ROUTE_TC_F16 : NTB_ROUTE_TC_3XTF32);
        grp.n = 0;
        grp.total = 0;
        return r;
    };
    for (int i = 0; i < count && rc == NTB_OK; i++) {
        if (nc[i] == 0 || mc[i] == 0)
            continue;
        Problem p;
        memset(&p, 0, sizeof(p));
        p.a = a[i]; p.b = b[i]; p.c = c[i];
        p.dtAB = dtypeAB; p.dtC = dtypeC;
        p.aMN = transA == NTB_X_TRANS;
        p.bMN = transB == NTB_X_NOTRANS;
        p.M = nc[i]; p.N = mc[i]; p.K = transA == NTB_X_TRANS ? na[i] : ma[i];
        p.aRows = na[i]; p.aCols = ma[i]; p.bRows = nb[i]; p.bCols = mb[i];
        p.lda = ma[i]; p.ldb = mb[i]; p.ldc = mc[i];
        p.count = 1; p.Q = 1;
        p.alpha = alpha; p.beta = beta;
        const long long tiles = (long long)((p.M + BM - 1) / BM) * ((p.N + 127) / 128);
        if (!grouping || p.K == 0 || !TcEligible(p) || tiles > (1 << 24)) {
            /* not for the shared launch: on its own, through the usual routing */
            rc = ntb_gemm(devID, stream, a[i], transA, b[i], transB, c[i], dtypeAB, dtypeC,
                          na[i], ma[i], nb[i], mb[i], nc[i], mc[i], ma[i], mb[i], mc[i], alpha, beta);
            continue;
        }
        rc = PrepareSingle(*ctx, p, 128, grp.p[grp.n], grp.tm[grp.n]);
        if (rc != NTB_OK)
            break;
        grp.first[grp.n] = grp.total;
        grp.total += grp.p[grp.n].totalTiles;
        grp.n++;
        if (grp.n == GROUP_MAX)
            rc = flush();
    }
    if (rc == NTB_OK)
        rc = flush();
    if (rc == NTB_ERR_CUDA)
        cudaGetLastError();
    if (prev >= 0 && prev != devID)
        cudaSetDevice(prev);
    return rc;
}
