/*
 * extern "C" layer: argument checks with the reference's shape rules, per-device
 * contexts, routing between the tensor-core and the FFMA kernels, and the host-buffer
 * entry point. See include/ntb_gemm.h for the contract of every function.
 */
#include "ntb_internal.h"
#include <atomic>
#include <mutex>
#include <vector>
#include <cstdlib>
#include <cstring>

namespace ntb {

namespace {

constexpr int MAX_DEV = 64;
std::mutex gLock;
DeviceCtx * gCtx[MAX_DEV] = { nullptr };
std::atomic<long long> gLaunches(0);
std::atomic<int> gForcedRoute(0);
std::atomic<int> gSkipKBlock(-1);
std::atomic<long long> gRouteCount[8];
thread_local int tLastRoute = NTB_ROUTE_NONE;

/* save / restore the calling thread's current device around a call */
struct DeviceGuard {
    int prev;
    bool ok;
    explicit DeviceGuard(int dev) : prev(-1), ok(false)
    {
        if (cudaGetDevice(&prev) != cudaSuccess)
            return;
        ok = (prev == dev) || cudaSetDevice(dev) == cudaSuccess;
        if (!ok)
            prev = -1;
    }
    ~DeviceGuard()
    {
        if (prev >= 0) {
            int cur = -1;
            if (cudaGetDevice(&cur) == cudaSuccess && cur != prev)
                cudaSetDevice(prev);
        }
    }
};

/* caller holds the device current */
DeviceCtx * GetCtx(int dev)
{
    if (dev < 0 || dev >= MAX_DEV)
        return nullptr;
    std::lock_guard<std::mutex> g(gLock);
    if (gCtx[dev])
        return gCtx[dev];
    DeviceCtx * c = new DeviceCtx();
    memset(c, 0, sizeof(*c));
    c->devID = dev;
    c->mayAllocate = true;
    if (cudaDeviceGetAttribute(&c->smCount, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaMalloc((void **)&c->status, 2 * sizeof(int)) != cudaSuccess ||
        cudaMemset(c->status, 0, 2 * sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        delete c;
        return nullptr;
    }
    gCtx[dev] = c;
    return c;
}

int CheckDtypes(int dtAB, int dtC)
{
    if (dtAB == NTB_X_FLOAT16 && (dtC == NTB_X_FLOAT16 || dtC == NTB_X_FLOAT))
        return NTB_OK;
    if (dtAB == NTB_X_FLOAT && dtC == NTB_X_FLOAT)
        return NTB_OK;
    return NTB_ERR_DTYPE;
}

/* fills shape fields of a Problem from the stored extents, with the reference's checks
   (am == bn, an == cn, bm == cm: source/tensor/core/arithmetic/MatrixMul.cpp:79-87) */
int SetShape(Problem & p, int transA, int transB, int na, int ma, int nb, int mb, int nc, int mc)
{
    if ((transA != NTB_X_TRANS && transA != NTB_X_NOTRANS) || (transB != NTB_X_TRANS && transB != NTB_X_NOTRANS))
        return NTB_ERR_ARG;
    if (na < 0 || ma < 0 || nb < 0 || mb < 0 || nc < 0 || mc < 0)
        return NTB_ERR_ARG;
    const int an = transA == NTB_X_TRANS ? ma : na;
    const int am = transA == NTB_X_TRANS ? na : ma;
    const int bn = transB == NTB_X_TRANS ? mb : nb;
    const int bm = transB == NTB_X_TRANS ? nb : mb;
    if (am != bn || an != nc || bm != mc)
        return NTB_ERR_SHAPE;
    p.M = an; p.N = bm; p.K = am;
    p.aMN = transA == NTB_X_TRANS;       /* stored K x M: M contiguous */
    p.bMN = transB == NTB_X_NOTRANS;     /* stored K x N: N contiguous */
    p.aRows = na; p.aCols = ma; p.bRows = nb; p.bCols = mb;
    return NTB_OK;
}

int Dispatch(int devID, cudaStream_t stream, Problem & p)
{
    if (p.count == 0 || p.M == 0 || p.N == 0)
        return NTB_OK;
    /* with K = 0 the operands are empty and never read: frameworks hand out NULL for them */
    if (!p.c || (p.K > 0 && (!p.a || !p.b)))
        return NTB_ERR_ARG;
    DeviceGuard guard(devID);
    if (!guard.ok) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    DeviceCtx * ctx = GetCtx(devID);
    if (!ctx)
        return NTB_ERR_CUDA;
    const int forced = ForcedRoute();
    const bool tc = forced != NTB_ROUTE_SIMT && TcEligible(p);
    /* operands TMA cannot address still go to the tensor cores, through loader warps; the FFMA
       kernel remains for K == 0 and for a forced NTB_ROUTE_SIMT */
    const bool ldg = !tc && forced != NTB_ROUTE_SIMT && forced != NTB_ROUTE_TC_F16_PAIR && LdgEligible(p);
    if (p.nPeers > 0 && !tc && !ldg)
        return NTB_ERR_ARG;                         /* only the tensor-core kernels store to peers */
    int rc;
    if (tc || ldg) {
        int route = NTB_ROUTE_NONE;
        rc = tc ? LaunchTc(*ctx, p, stream, &route) : LaunchLdg(*ctx, p, stream, &route);
        if (rc == NTB_OK)
            SetLastRoute(route);
    }
    else {
        if (forced == NTB_ROUTE_TC_F16 || forced == NTB_ROUTE_TC_3XTF32 || forced == NTB_ROUTE_TC_F16_PAIR)
            return NTB_ERR_ARG;
        rc = LaunchSimt(*ctx, p, stream);
        if (rc == NTB_OK)
            SetLastRoute(NTB_ROUTE_SIMT);
    }
    return rc;
}

/* streams and events of the pipelined host-buffer path, created once per device */
bool EnsurePipe(DeviceCtx * ctx)
{
    std::lock_guard<std::mutex> g(gLock);
    if (ctx->pipeReady)
        return true;
    bool ok = cudaStreamCreateWithFlags(&ctx->copyIn, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&ctx->copyOut, cudaStreamNonBlocking) == cudaSuccess &&
              cudaEventCreateWithFlags(&ctx->evStart, cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; ok && i < 16; i++)
        ok = cudaEventCreateWithFlags(&ctx->evIn[i], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&ctx->evOut[i], cudaEventDisableTiming) == cudaSuccess;
    if (!ok)
        cudaGetLastError();
    ctx->pipeReady = ok;
    return ok;
}

int GrowStage(DeviceCtx * ctx, int slot, size_t bytes)
{
    if (ctx->stageBytes[slot] >= bytes)
        return NTB_OK;
    if (ctx->stage[slot])
        cudaFree(ctx->stage[slot]);
    ctx->stage[slot] = nullptr;
    ctx->stageBytes[slot] = 0;
    if (cudaMalloc(&ctx->stage[slot], bytes) != cudaSuccess) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    ctx->stageBytes[slot] = bytes;
    return NTB_OK;
}

}

DeviceCtx * CtxFor(int dev)
{
    return GetCtx(dev);
}

int EnsureScratch(const DeviceCtx & ctx, int slot, size_t bytes, void ** out)
{
    DeviceCtx * c = ctx.mayAllocate ? GetCtx(ctx.devID) : nullptr;
    if (!c || slot < 0 || slot >= 4)
        return NTB_ERR_CUDA;
    std::lock_guard<std::mutex> g(gLock);
    if (c->scratchBytes[slot] < bytes) {
        if (c->scratch[slot]) {
            /* queued work may still use the old buffer */
            if (cudaDeviceSynchronize() != cudaSuccess) {
                cudaGetLastError();
                return NTB_ERR_CUDA;
            }
            cudaFree(c->scratch[slot]);
        }
        c->scratch[slot] = nullptr;
        c->scratchBytes[slot] = 0;
        const size_t want = bytes + bytes / 8;              /* some room, so that slowly growing shapes do not reallocate each time */
        if (cudaMalloc(&c->scratch[slot], want) != cudaSuccess) {
            cudaGetLastError();
            return NTB_ERR_CUDA;
        }
        c->scratchBytes[slot] = want;
    }
    *out = c->scratch[slot];
    return NTB_OK;
}

int EnsureCounted(const DeviceCtx & ctx, size_t workBytes, size_t flagBytes, cudaStream_t stream, float ** work, int ** flags)
{
    /* the counter area has one fixed size, so that its end does not move with the problem */
    const size_t flagArea = 64 * 1024;
    if (flagBytes > flagArea)
        return NTB_ERR_LIMIT;
    void * base = nullptr;
    const int rc = EnsureScratch(ctx, 3, flagArea + workBytes, &base);
    if (rc != NTB_OK)
        return rc;
    DeviceCtx * c = GetCtx(ctx.devID);
    {
        std::lock_guard<std::mutex> g(gLock);
        if (c->countersCleared != base) {
            if (cudaMemsetAsync(base, 0, flagArea, stream) != cudaSuccess) {
                cudaGetLastError();
                return NTB_ERR_CUDA;
            }
            c->countersCleared = base;
        }
    }
    *flags = (int *)base;
    *work = (float *)((char *)base + flagArea);
    return NTB_OK;
}

int ScratchAcquire(const DeviceCtx & ctx, cudaStream_t stream)
{
    DeviceCtx * c = ctx.mayAllocate ? GetCtx(ctx.devID) : nullptr;
    if (!c)
        return NTB_ERR_CUDA;
    /* inside a stream capture the graph orders its own nodes; work outside it is the caller's to order */
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
        return NTB_OK;
    cudaGetLastError();
    std::lock_guard<std::mutex> g(gLock);
    if (c->haveScratchEvent && cudaStreamWaitEvent(stream, c->scratchEvent, 0) != cudaSuccess) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    return NTB_OK;
}

int ScratchRelease(const DeviceCtx & ctx, cudaStream_t stream)
{
    DeviceCtx * c = ctx.mayAllocate ? GetCtx(ctx.devID) : nullptr;
    if (!c)
        return NTB_ERR_CUDA;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
        return NTB_OK;
    cudaGetLastError();
    std::lock_guard<std::mutex> g(gLock);
    if (!c->haveScratchEvent) {
        if (cudaEventCreateWithFlags(&c->scratchEvent, cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            return NTB_ERR_CUDA;
        }
        c->haveScratchEvent = true;
    }
    if (cudaEventRecord(c->scratchEvent, stream) != cudaSuccess) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    return NTB_OK;
}

void CountLaunch()
{
    gLaunches.fetch_add(1);
}

void SetLastRoute(int route)
{
    tLastRoute = route;
    if (route >= 0 && route < 8)
        gRouteCount[route].fetch_add(1);
}

void CountVariant(int index)
{
    if (index >= 0 && index < 8)
        gRouteCount[index].fetch_add(1);
}

int InjectedSkipKBlock()
{
    return gSkipKBlock.load();
}

int ForcedRoute()
{
    const int r = gForcedRoute.load();
    if (r != 0)
        return r;
    /* NTB_ROUTE in the environment gives the default when ntb_set_route() was not used */
    const char * v = getenv("NTB_ROUTE");
    return v && *v ? atoi(v) : 0;
}

EncodeTiledFn GetEncodeTiled()
{
    static std::atomic<EncodeTiledFn> cached(nullptr);
    EncodeTiledFn f = cached.load();
    if (f)
        return f;
    void * sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess || !sym) {
        cudaGetLastError();
        return nullptr;
    }
    cached.store((EncodeTiledFn)sym);
    return (EncodeTiledFn)sym;
}

}

using namespace ntb;

extern "C" {

int ntb_gemm_strided_batched(int devID, void * stream,
                             const void * a, int transA, const void * b, int transB, void * c,
                             int dtypeAB, int dtypeC,
                             int na, int ma, int nb, int mb, int nc, int mc,
                             long long lda, long long ldb, long long ldc,
                             long long strideA, long long strideB, long long strideC,
                             int count, float alpha, float beta)
{
    Problem p;
    memset(&p, 0, sizeof(p));
    int rc = CheckDtypes(dtypeAB, dtypeC);
    if (rc != NTB_OK)
        return rc;
    rc = SetShape(p, transA, transB, na, ma, nb, mb, nc, mc);
    if (rc != NTB_OK)
        return rc;
    if (count < 0 || lda < ma || ldb < mb || ldc < mc || strideA < 0 || strideB < 0 || strideC < 0)
        return NTB_ERR_ARG;
    p.a = a; p.b = b; p.c = c;
    p.dtAB = dtypeAB; p.dtC = dtypeC;
    p.lda = lda; p.ldb = ldb; p.ldc = ldc;
    p.count = count; p.Q = 1;
    p.sAp = strideA; p.sBp = strideB; p.sCp = strideC;
    p.alpha = alpha; p.beta = beta;
    return Dispatch(devID, (cudaStream_t)stream, p);
}

int ntb_gemm_bias_act(int devID, void * stream,
                      const void * a, int transA, const void * b, int transB, const void * bias, void * c,
                      int dtypeAB, int dtypeC,
                      int na, int ma, int nb, int mb, int nc, int mc,
                      long long lda, long long ldb, long long ldc,
                      float alpha, float beta, int act)
{
    Problem p;
    memset(&p, 0, sizeof(p));
    int rc = CheckDtypes(dtypeAB, dtypeC);
    if (rc != NTB_OK)
        return rc;
    rc = SetShape(p, transA, transB, na, ma, nb, mb, nc, mc);
    if (rc != NTB_OK)
        return rc;
    if (lda < ma || ldb < mb || ldc < mc || (act != NTB_ACT_NONE && act != NTB_ACT_RECTIFY))
        return NTB_ERR_ARG;
    p.a = a; p.b = b; p.c = c;
    p.dtAB = dtypeAB; p.dtC = dtypeC;
    p.lda = lda; p.ldb = ldb; p.ldc = ldc;
    p.count = 1; p.Q = 1;
    p.alpha = alpha; p.beta = beta;
    p.bias = bias; p.act = act;
    return Dispatch(devID, (cudaStream_t)stream, p);
}

namespace {

/* one packed, batched product out (+)= alpha * op(x) * op(y) + beta * out as a Problem */
int FillPacked(Problem & p, const void * x, int tX, int xr, int xc, const void * y, int tY, int yr, int yc,
               void * out, int outr, int outc, int dtype, int count, float alpha, float beta)
{
    memset(&p, 0, sizeof(p));
    int rc = SetShape(p, tX, tY, xr, xc, yr, yc, outr, outc);
    if (rc != NTB_OK)
        return rc;
    p.a = x; p.b = y; p.c = out;
    p.dtAB = dtype; p.dtC = dtype;
    p.lda = xc; p.ldb = yc; p.ldc = outc;
    p.count = count; p.Q = 1;
    p.sAp = (long long)xr * xc; p.sBp = (long long)yr * yc; p.sCp = (long long)outr * outc;
    p.alpha = alpha; p.beta = beta;
    return NTB_OK;
}

}

int ntb_gemm_grad(int devID, void * stream,
                  const void * a, int transA, const void * b, int transB, const void * dedc,
                  void * deda, void * dedb, int dtype,
                  int na, int ma, int nb, int mb, int count, float alpha)
{
    if ((transA != NTB_X_TRANS && transA != NTB_X_NOTRANS) || (transB != NTB_X_TRANS && transB != NTB_X_NOTRANS))
        return NTB_ERR_ARG;
    if (na < 0 || ma < 0 || nb < 0 || mb < 0 || count < 0)
        return NTB_ERR_ARG;
    int rc = CheckDtypes(dtype, dtype);
    if (rc != NTB_OK)
        return rc;
    const bool tA = transA == NTB_X_TRANS, tB = transB == NTB_X_TRANS;
    const int an = tA ? ma : na, am = tA ? na : ma;
    const int bn = tB ? mb : nb, bm = tB ? nb : mb;
    if (am != bn)
        return NTB_ERR_SHAPE;
    const int cn = an, cm = bm;                       /* dedc is cn x cm */
    if (count == 0 || (!deda && !dedb))
        return NTB_OK;
    if (!a || !b || !dedc)
        return NTB_ERR_ARG;
    const int T = NTB_X_TRANS, N = NTB_X_NOTRANS;
    Problem pa, pb;
    int ra = NTB_OK, rb = NTB_OK;
    if (!tA && !tB) {
        ra = FillPacked(pa, dedc, N, cn, cm, b, T, nb, mb, deda, na, ma, dtype, count, alpha, 1.f);
        rb = FillPacked(pb, a, T, na, ma, dedc, N, cn, cm, dedb, nb, mb, dtype, count, alpha, 1.f);
    }
    else if (tA && !tB) {
        ra = FillPacked(pa, b, N, nb, mb, dedc, T, cn, cm, deda, na, ma, dtype, count, alpha, 1.f);
        rb = FillPacked(pb, a, N, na, ma, dedc, N, cn, cm, dedb, nb, mb, dtype, count, alpha, 1.f);
    }
    else if (!tA && tB) {
        ra = FillPacked(pa, dedc, N, cn, cm, b, N, nb, mb, deda, na, ma, dtype, count, alpha, 1.f);
        rb = FillPacked(pb, dedc, T, cn, cm, a, N, na, ma, dedb, nb, mb, dtype, count, alpha, 1.f);
    }
    else {
        ra = FillPacked(pa, b, T, nb, mb, dedc, T, cn, cm, deda, na, ma, dtype, count, alpha, 1.f);
        rb = FillPacked(pb, dedc, T, cn, cm, a, T, na, ma, dedb, nb, mb, dtype, count, alpha, 1.f);
    }
    if (ra != NTB_OK)
        return ra;
    if (rb != NTB_OK)
        return rb;
    cudaStream_t st = (cudaStream_t)stream;
    if (!deda)
        return Dispatch(devID, st, pb);
    if (!dedb)
        return Dispatch(devID, st, pa);
    const int forced = ForcedRoute();
    const bool empty = pa.M == 0 || pa.N == 0 || pb.M == 0 || pb.N == 0;
    if (!empty && forced != NTB_ROUTE_SIMT && TcEligible(pa) && TcEligible(pb)) {
        DeviceGuard guard(devID);
        if (!guard.ok) {
            cudaGetLastError();
            return NTB_ERR_CUDA;
        }
        DeviceCtx * ctx = GetCtx(devID);
        if (!ctx)
            return NTB_ERR_CUDA;
        /* one shared launch pays when both products are small enough for the single-CTA
           kernel; a product that wants CTA pairs or a split of K gets its own launch */
        if (TcTileChoice(*ctx, pa) > 0 && TcTileChoice(*ctx, pb) > 0) {
            rc = LaunchTcTwo(*ctx, pa, pb, st);
            if (rc == NTB_OK)
                SetLastRoute(dtype == NTB_X_FLOAT16 ? NTB_ROUTE_TC_F16 : NTB_ROUTE_TC_3XTF32);
            return rc;
        }
    }
    rc = Dispatch(devID, st, pa);
    return rc != NTB_OK ? rc : Dispatch(devID, st, pb);
}

int ntb_gemm(int devID, void * stream,
             const void * a, int transA, const void * b, int transB, void * c,
             int dtypeAB, int dtypeC,
             int na, int ma, int nb, int mb, int nc, int mc,
             long long lda, long long ldb, long long ldc,
             float alpha, float beta)
{
    return ntb_gemm_strided_batched(devID, stream, a, transA, b, transB, c, dtypeAB, dtypeC,
                                    na, ma, nb, mb, nc, mc, lda, ldb, ldc, 0, 0, 0, 1, alpha, beta);
}

int ntb_gemm_peers(int devID, void * stream,
                   const void * a, int transA, const void * b, int transB, void * c,
                   void * const * peers, int nPeers,
                   int dtypeAB, int dtypeC,
                   int na, int ma, int nb, int mb, int nc, int mc,
                   long long lda, long long ldb, long long ldc,
                   float alpha, float beta)
{
    Problem p;
    memset(&p, 0, sizeof(p));
    int rc = CheckDtypes(dtypeAB, dtypeC);
    if (rc != NTB_OK)
        return rc;
    rc = SetShape(p, transA, transB, na, ma, nb, mb, nc, mc);
    if (rc != NTB_OK)
        return rc;
    if (lda < ma || ldb < mb || ldc < mc || nPeers < 0 || (nPeers > 0 && !peers))
        return NTB_ERR_ARG;
    if (nPeers > NTB_MAX_PEERS)
        return NTB_ERR_LIMIT;
    const long long ces = ElemSize(dtypeC);
    for (int i = 0; i < nPeers; i++) {
        if (!peers[i] || ((uintptr_t)peers[i] & 15) || (ldc * ces) % 16)
            return NTB_ERR_ARG;
        p.peers[i] = peers[i];
    }
    p.nPeers = nPeers;
    p.a = a; p.b = b; p.c = c;
    p.dtAB = dtypeAB; p.dtC = dtypeC;
    p.lda = lda; p.ldb = ldb; p.ldc = ldc;
    p.count = 1; p.Q = 1;
    p.alpha = alpha; p.beta = beta;
    if (nPeers > 0 && p.K == 0)
        return NTB_ERR_ARG;                         /* K == 0 takes the FFMA kernel, which has no peer stores */
    if (nPeers > 0 && !TcEligible(p))
        return NTB_ERR_ARG;
    return Dispatch(devID, (cudaStream_t)stream, p);
}

int ntb_gemm_multicast(int devID, void * stream,
                       const void * a, int transA, const void * b, int transB, void * c, void * mc,
                       int dtypeAB, int dtypeC,
                       int na, int ma, int nb, int mb, int nc, int mc_cols,
                       long long lda, long long ldb, long long ldc,
                       float alpha, float beta)
{
    Problem p;
    memset(&p, 0, sizeof(p));
    int rc = CheckDtypes(dtypeAB, dtypeC);
    if (rc != NTB_OK)
        return rc;
    rc = SetShape(p, transA, transB, na, ma, nb, mb, nc, mc_cols);
    if (rc != NTB_OK)
        return rc;
    const long long ces = ElemSize(dtypeC);
    if (lda < ma || ldb < mb || ldc < mc_cols || !mc || ((uintptr_t)mc & 15) || (ldc * ces) % 16 || (mc_cols * ces) % 16)
        return NTB_ERR_ARG;
    p.peers[0] = mc;
    p.nPeers = 1;
    p.peerMcast = 1;
    p.a = a; p.b = b; p.c = c;
    p.dtAB = dtypeAB; p.dtC = dtypeC;
    p.lda = lda; p.ldb = ldb; p.ldc = ldc;
    p.count = 1; p.Q = 1;
    p.alpha = alpha; p.beta = beta;
    if (p.K == 0 || !TcEligible(p))
        return NTB_ERR_ARG;
    return Dispatch(devID, (cudaStream_t)stream, p);
}

int ntb_gemm_broadcast(int devID, void * stream,
                       const void * a, int transA, const void * b, int transB, void * c,
                       int dtypeAB, int dtypeC,
                       int na, int ma, int nb, int mb, int nc, int mc,
                       int aBlockNum, int bBlockNum,
                       float alpha, float beta)
{
    Problem p;
    memset(&p, 0, sizeof(p));
    int rc = CheckDtypes(dtypeAB, dtypeC);
    if (rc != NTB_OK)
        return rc;
    rc = SetShape(p, transA, transB, na, ma, nb, mb, nc, mc);
    if (rc != NTB_OK)
        return rc;
    if (aBlockNum < 0 || bBlockNum < 0)
        return NTB_ERR_ARG;
    if ((long long)aBlockNum * bBlockNum > 2147483647LL)
        return NTB_ERR_LIMIT;
    p.a = a; p.b = b; p.c = c;
    p.dtAB = dtypeAB; p.dtC = dtypeC;
    p.lda = ma; p.ldb = mb; p.ldc = mc;
    p.count = aBlockNum * bBlockNum;
    p.Q = bBlockNum > 0 ? bBlockNum : 1;
    p.sAp = (long long)na * ma; p.sAq = 0;
    p.sBp = 0;                  p.sBq = (long long)nb * mb;
    p.sCq = (long long)nc * mc; p.sCp = p.sCq * p.Q;
    p.alpha = alpha; p.beta = beta;
    return Dispatch(devID, (cudaStream_t)stream, p);
}

int ntb_gemm_list(int devID, void * stream,
                  const void * const * a, int transA, const void * const * b, int transB,
                  void * const * c, int dtypeAB, int dtypeC,
                  int count, int na, int ma, int nb, int mb, int nc, int mc,
                  float alpha, float beta)
{
    if (count < 0)
        return NTB_ERR_ARG;
    if (count == 0)
        return NTB_OK;
    if (!a || !b || !c)
        return NTB_ERR_ARG;
    int rc = CheckDtypes(dtypeAB, dtypeC);
    if (rc != NTB_OK)
        return rc;
    const long long esAB = (long long)ElemSize(dtypeAB), esC = (long long)ElemSize(dtypeC);
    auto gap = [](const void * x, const void * y) { return (long long)((const char *)x - (const char *)y); };

    if (count == 1)
        return ntb_gemm(devID, stream, a[0], transA, b[0], transB, c[0], dtypeAB, dtypeC,
                        na, ma, nb, mb, nc, mc, ma, mb, mc, alpha, beta);

    /* constant byte gaps -> one strided launch */
    {
        const long long gA = gap(a[1], a[0]), gB = gap(b[1], b[0]), gC = gap(c[1], c[0]);
        bool strided = gA >= 0 && gB >= 0 && gC >= 0 && gA % esAB == 0 && gB % esAB == 0 && gC % esC == 0;
        for (int i = 2; strided && i < count; i++)
            strided = gap(a[i], a[i - 1]) == gA && gap(b[i], b[i - 1]) == gB && gap(c[i], c[i - 1]) == gC;
        if (strided)
            return ntb_gemm_strided_batched(devID, stream, a[0], transA, b[0], transB, c[0], dtypeAB, dtypeC,
                                            na, ma, nb, mb, nc, mc, ma, mb, mc,
                                            gA / esAB, gB / esAB, gC / esC, count, alpha, beta);
    }
    /* the (p, q) pattern of the general form: a constant over runs of Q problems, b
       repeating with period Q, c packed */
    {
        int Q = 1;
        while (Q < count && a[Q] == a[0])
            Q++;
        if (Q > 1 && Q < count && count % Q == 0) {
            const int P = count / Q;
            const long long aBytes = (long long)na * ma * esAB, bBytes = (long long)nb * mb * esAB,
                            cBytes = (long long)nc * mc * esC;
            bool match = true;
            for (int i = 0; match && i < count; i++) {
                const int pIdx = i / Q, qIdx = i % Q;
                match = gap(a[i], a[0]) == pIdx * aBytes && gap(b[i], b[0]) == qIdx * bBytes &&
                        gap(c[i], c[0]) == i * cBytes;
            }
            if (match)
                return ntb_gemm_broadcast(devID, stream, a[0], transA, b[0], transB, c[0], dtypeAB, dtypeC,
                                          na, ma, nb, mb, nc, mc, P, Q, alpha, beta);
        }
    }
    for (int i = 0; i < count; i++) {
        rc = ntb_gemm(devID, stream, a[i], transA, b[i], transB, c[i], dtypeAB, dtypeC,
                      na, ma, nb, mb, nc, mc, ma, mb, mc, alpha, beta);
        if (rc != NTB_OK)
            return rc;
    }
    return NTB_OK;
}

}

namespace {

/* the host-buffer product; aResident: a is device memory already (only b and c are staged) */
int HostProduct(int devID, void * stream, bool aResident,
                const void * a, int transA, const void * b, int transB, void * c,
                int dtypeAB, int dtypeC,
                int na, int ma, int nb, int mb, int nc, int mc,
                long long strideA, long long strideB, long long strideC,
                int count, float alpha, float beta)
{
    if (!a || !b || !c || count < 0 || na < 0 || ma < 0 || nb < 0 || mb < 0 || nc < 0 || mc < 0)
        return NTB_ERR_ARG;
    int rc = CheckDtypes(dtypeAB, dtypeC);
    if (rc != NTB_OK)
        return rc;
    if (count == 0)
        return NTB_OK;
    DeviceGuard guard(devID);
    if (!guard.ok) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    DeviceCtx * ctx = GetCtx(devID);
    if (!ctx)
        return NTB_ERR_CUDA;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t esAB = ElemSize(dtypeAB), esC = ElemSize(dtypeC);
    /* A single product is staged with row pitches that are multiples of 16 bytes (the host
       buffers are packed), so that TMA can address the staged copies whatever the extents;
       batches keep the caller's packed layout and strides. */
    const bool pad = count == 1;
    const long long ldaS = pad && !aResident ? (long long)((((size_t)ma * esAB + 15) & ~(size_t)15) / esAB) : ma;
    const long long ldbS = pad ? (long long)((((size_t)mb * esAB + 15) & ~(size_t)15) / esAB) : mb;
    const long long ldcS = pad ? (long long)((((size_t)mc * esC + 15) & ~(size_t)15) / esC) : mc;
    /* a stride of 0 shares one matrix; otherwise `count` matrices at the given stride */
    const size_t aBytes = pad ? (size_t)na * ldaS * esAB : ((size_t)(strideA ? strideA * (count - 1) : 0) + (size_t)na * ma) * esAB;
    const size_t bBytes = pad ? (size_t)nb * ldbS * esAB : ((size_t)(strideB ? strideB * (count - 1) : 0) + (size_t)nb * mb) * esAB;
    const size_t cBytes = pad ? (size_t)nc * ldcS * esC : ((size_t)(strideC ? strideC * (count - 1) : 0) + (size_t)nc * mc) * esC;
    {
        std::lock_guard<std::mutex> g(gLock);
        if ((!aResident && GrowStage(ctx, 0, aBytes) != NTB_OK) || GrowStage(ctx, 1, bBytes) != NTB_OK ||
            GrowStage(ctx, 2, cBytes) != NTB_OK)
            return NTB_ERR_CUDA;
    }
    const void * aDev = aResident ? a : ctx->stage[0];
    /* One large 2-D product: cut C (and the matching part of B) into column chunks and
       overlap the copy-in of chunk j+1 and the copy-out of chunk j-1 with the product of
       chunk j. PCIe is full duplex, so the result rides back while operands still arrive.
       (Row chunks of a and c, whose copies are single contiguous blocks, measured 4-5 % slower
       on one and on two GPUs.) */
    const long long N = transB == NTB_X_TRANS ? nb : mb;
    /* tuning: fewest columns a chunk may have (a chunk of a row-major matrix is copied in pieces
       of that many elements) */
    const char * minColsKnob = getenv("NTB_HOST_CHUNK_COLS");
    const long long minCols = minColsKnob && atoi(minColsKnob) >= 64 ? atoi(minColsKnob) : 256;
    const int chunks = N >= 8 * minCols ? 8 : (int)(N / minCols);
    if (count == 1 && chunks >= 2 && (aResident ? 0 : aBytes) + bBytes + cBytes >= ((size_t)16 << 20) && EnsurePipe(ctx)) {
        const long long step = ((N + chunks - 1) / chunks + 63) / 64 * 64;      /* columns per chunk */
        rc = NTB_ERR_CUDA;
        do {
            if (cudaEventRecord(ctx->evStart, st) != cudaSuccess ||
                cudaStreamWaitEvent(ctx->copyIn, ctx->evStart, 0) != cudaSuccess ||
                cudaStreamWaitEvent(ctx->copyOut, ctx->evStart, 0) != cudaSuccess)
                break;
            if (!aResident && cudaMemcpy2DAsync(ctx->stage[0], (size_t)ldaS * esAB, a, (size_t)ma * esAB, (size_t)ma * esAB, (size_t)na,
                                                cudaMemcpyHostToDevice, ctx->copyIn) != cudaSuccess)
                break;
            bool fail = false;
            int used = 0;
            for (long long n0 = 0; n0 < N && !fail; n0 += step, used++) {
                const long long w = N - n0 < step ? N - n0 : step;
                /* B: columns [n0, n0+w) of a stored k x N matrix, or rows of a stored N x k one */
                if (transB == NTB_X_TRANS)
                    fail |= cudaMemcpy2DAsync((char *)ctx->stage[1] + (size_t)n0 * ldbS * esAB, (size_t)ldbS * esAB,
                                              (const char *)b + (size_t)n0 * mb * esAB, (size_t)mb * esAB, (size_t)mb * esAB, (size_t)w,
                                              cudaMemcpyHostToDevice, ctx->copyIn) != cudaSuccess;
                else
                    fail |= cudaMemcpy2DAsync((char *)ctx->stage[1] + n0 * esAB, (size_t)ldbS * esAB, (const char *)b + n0 * esAB,
                                              (size_t)mb * esAB, (size_t)w * esAB, nb, cudaMemcpyHostToDevice, ctx->copyIn) != cudaSuccess;
                if (beta != 0.f)
                    fail |= cudaMemcpy2DAsync((char *)ctx->stage[2] + n0 * esC, (size_t)ldcS * esC, (const char *)c + n0 * esC,
                                              (size_t)mc * esC, (size_t)w * esC, nc, cudaMemcpyHostToDevice, ctx->copyIn) != cudaSuccess;
                fail |= cudaEventRecord(ctx->evIn[used], ctx->copyIn) != cudaSuccess;
                fail |= cudaStreamWaitEvent(st, ctx->evIn[used], 0) != cudaSuccess;
                if (fail)
                    break;
                int r2;
                if (transB == NTB_X_TRANS)
                    r2 = ntb_gemm(devID, stream, aDev, transA, (char *)ctx->stage[1] + (size_t)n0 * ldbS * esAB, transB,
                                  (char *)ctx->stage[2] + n0 * esC, dtypeAB, dtypeC, na, ma, (int)w, mb, nc, (int)w,
                                  ldaS, ldbS, ldcS, alpha, beta);
                else
                    r2 = ntb_gemm(devID, stream, aDev, transA, (char *)ctx->stage[1] + n0 * esAB, transB,
                                  (char *)ctx->stage[2] + n0 * esC, dtypeAB, dtypeC, na, ma, nb, (int)w, nc, (int)w,
                                  ldaS, ldbS, ldcS, alpha, beta);
                if (r2 != NTB_OK) { rc = r2; fail = true; break; }
                fail |= cudaEventRecord(ctx->evOut[used], st) != cudaSuccess;
                fail |= cudaStreamWaitEvent(ctx->copyOut, ctx->evOut[used], 0) != cudaSuccess;
                fail |= cudaMemcpy2DAsync((char *)c + n0 * esC, (size_t)mc * esC, (char *)ctx->stage[2] + n0 * esC,
                                          (size_t)ldcS * esC, (size_t)w * esC, nc, cudaMemcpyDeviceToHost, ctx->copyOut) != cudaSuccess;
            }
            /* even after a failure, let everything issued so far drain before returning */
            const bool s1 = cudaStreamSynchronize(ctx->copyIn) == cudaSuccess;
            const bool s2 = cudaStreamSynchronize(st) == cudaSuccess;
            const bool s3 = cudaStreamSynchronize(ctx->copyOut) == cudaSuccess;
            if (!fail && s1 && s2 && s3)
                rc = NTB_OK;
        } while (0);
        if (rc == NTB_ERR_CUDA)
            cudaGetLastError();
        return rc;
    }

    if (pad) {
        /* packed host rows to padded device rows and back */
        if ((!aResident && na && ma &&
             cudaMemcpy2DAsync(ctx->stage[0], (size_t)ldaS * esAB, a, (size_t)ma * esAB, (size_t)ma * esAB, (size_t)na,
                               cudaMemcpyHostToDevice, st) != cudaSuccess) ||
            (nb && mb &&
             cudaMemcpy2DAsync(ctx->stage[1], (size_t)ldbS * esAB, b, (size_t)mb * esAB, (size_t)mb * esAB, (size_t)nb,
                               cudaMemcpyHostToDevice, st) != cudaSuccess))
            return NTB_ERR_CUDA;
        if (beta != 0.f && nc && mc &&
            cudaMemcpy2DAsync(ctx->stage[2], (size_t)ldcS * esC, c, (size_t)mc * esC, (size_t)mc * esC, (size_t)nc,
                              cudaMemcpyHostToDevice, st) != cudaSuccess)
            return NTB_ERR_CUDA;
        rc = ntb_gemm(devID, stream, aDev, transA, ctx->stage[1], transB, ctx->stage[2], dtypeAB, dtypeC,
                      na, ma, nb, mb, nc, mc, ldaS, ldbS, ldcS, alpha, beta);
        if (rc != NTB_OK)
            return rc;
        if ((nc && mc && cudaMemcpy2DAsync(c, (size_t)mc * esC, ctx->stage[2], (size_t)ldcS * esC, (size_t)mc * esC, (size_t)nc,
                                           cudaMemcpyDeviceToHost, st) != cudaSuccess) ||
            cudaStreamSynchronize(st) != cudaSuccess) {
            cudaGetLastError();
            return NTB_ERR_CUDA;
        }
        return NTB_OK;
    }
    if ((!aResident && cudaMemcpyAsync(ctx->stage[0], a, aBytes, cudaMemcpyHostToDevice, st) != cudaSuccess) ||
        cudaMemcpyAsync(ctx->stage[1], b, bBytes, cudaMemcpyHostToDevice, st) != cudaSuccess)
        return NTB_ERR_CUDA;
    if (beta != 0.f && cudaMemcpyAsync(ctx->stage[2], c, cBytes, cudaMemcpyHostToDevice, st) != cudaSuccess)
        return NTB_ERR_CUDA;
    rc = ntb_gemm_strided_batched(devID, stream, aDev, transA, ctx->stage[1], transB, ctx->stage[2],
                                  dtypeAB, dtypeC, na, ma, nb, mb, nc, mc, ma, mb, mc,
                                  strideA, strideB, strideC, count, alpha, beta);
    if (rc != NTB_OK)
        return rc;
    if (cudaMemcpyAsync(c, ctx->stage[2], cBytes, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    return NTB_OK;
}

}

extern "C" {

int ntb_gemm_host(int devID, void * stream,
                  const void * a, int transA, const void * b, int transB, void * c,
                  int dtypeAB, int dtypeC,
                  int na, int ma, int nb, int mb, int nc, int mc,
                  long long strideA, long long strideB, long long strideC,
                  int count, float alpha, float beta)
{
    return HostProduct(devID, stream, false, a, transA, b, transB, c, dtypeAB, dtypeC, na, ma, nb, mb, nc, mc,
                       strideA, strideB, strideC, count, alpha, beta);
}

int ntb_gemm_host_resident_a(int devID, void * stream,
                             const void * aDevice, int transA, const void * b, int transB, void * c,
                             int dtypeAB, int dtypeC,
                             int na, int ma, int nb, int mb, int nc, int mc,
                             long long strideA, long long strideB, long long strideC,
                             int count, float alpha, float beta)
{
    return HostProduct(devID, stream, true, aDevice, transA, b, transB, c, dtypeAB, dtypeC, na, ma, nb, mb, nc, mc,
                       strideA, strideB, strideC, count, alpha, beta);
}

int ntb_debug_inject(int devID, int skipKBlock, int waitLimitKiloCycles)
{
    if (waitLimitKiloCycles < 0)
        return NTB_ERR_ARG;
    DeviceGuard guard(devID);
    if (!guard.ok) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    DeviceCtx * ctx = GetCtx(devID);
    if (!ctx)
        return NTB_ERR_CUDA;
    if (cudaDeviceSynchronize() != cudaSuccess ||
        cudaMemcpy(ctx->status + 1, &waitLimitKiloCycles, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    gSkipKBlock.store(skipKBlock < 0 ? -1 : skipKBlock);
    return NTB_OK;
}

int ntb_last_route(void)
{
    return tLastRoute;
}

int ntb_set_route(int route)
{
    if (route != 0 && route != NTB_ROUTE_SIMT && route != NTB_ROUTE_TC_F16 && route != NTB_ROUTE_TC_3XTF32 &&
        route != NTB_ROUTE_TC_F16_PAIR)
        return NTB_ERR_ARG;
    gForcedRoute.store(route);
    return NTB_OK;
}

int ntb_device_status(int devID)
{
    DeviceGuard guard(devID);
    if (!guard.ok) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    DeviceCtx * ctx = GetCtx(devID);
    if (!ctx)
        return NTB_ERR_CUDA;
    int v = 0;
    if (cudaDeviceSynchronize() != cudaSuccess ||
        cudaMemcpy(&v, ctx->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    if (v != 0) {
        cudaMemset(ctx->status, 0, sizeof(int));
        std::lock_guard<std::mutex> g(gLock);
        ctx->countersCleared = nullptr;     /* counters of an abandoned launch may be left non-zero */
    }
    return v;
}

int ntb_plan(int dtypeAB, int M, int N, int K, int count, int smCount)
{
    if ((dtypeAB != NTB_X_FLOAT16 && dtypeAB != NTB_X_FLOAT) || M <= 0 || N <= 0 || K <= 0 || count <= 0 || smCount <= 0)
        return NTB_PLAN_PAIR_256X256 - 100;         /* no plan: bad argument */
    Problem p;
    memset(&p, 0, sizeof(p));
    p.dtAB = dtypeAB;
    p.dtC = dtypeAB;
    p.M = M; p.N = N; p.K = K;
    p.count = count; p.Q = 1;
    DeviceCtx ctx;
    memset(&ctx, 0, sizeof(ctx));
    ctx.smCount = smCount;
    return TcTileChoice(ctx, p);
}

long long ntb_route_count(int route)
{
    return route >= 0 && route < 8 ? gRouteCount[route].load() : 0;
}

long long ntb_launch_count(void)
{
    return gLaunches.load();
}

void ntb_release(void)
{
    std::lock_guard<std::mutex> g(gLock);
    for (int d = 0; d < MAX_DEV; d++) {
        DeviceCtx * c = gCtx[d];
        if (!c)
            continue;
        int prev = -1;
        cudaGetDevice(&prev);
        if (cudaSetDevice(d) == cudaSuccess) {
            for (int s = 0; s < 3; s++)
                if (c->stage[s])
                    cudaFree(c->stage[s]);
            if (c->pipeReady) {
                cudaStreamDestroy(c->copyIn);
                cudaStreamDestroy(c->copyOut);
                cudaEventDestroy(c->evStart);
                for (int i = 0; i < 16; i++) {
                    cudaEventDestroy(c->evIn[i]);
                    cudaEventDestroy(c->evOut[i]);
                }
            }
            for (int s = 0; s < 4; s++)
                if (c->scratch[s])
                    cudaFree(c->scratch[s]);
            if (c->haveScratchEvent)
                cudaEventDestroy(c->scratchEvent);
            cudaFree(c->status);
        }
        if (prev >= 0)
            cudaSetDevice(prev);
        delete c;
        gCtx[d] = nullptr;
    }
}

const char * ntb_strerror(int code)
{
    switch (code) {
    case NTB_OK: return "ok";
    case NTB_ERR_ARG: return "bad argument";
    case NTB_ERR_SHAPE: return "unmatched tensors in multiplication";
    case NTB_ERR_DTYPE: return "unsupported data type";
    case NTB_ERR_CUDA: return "CUDA call failed or no usable device";
    case NTB_ERR_DEVICE_WAIT: return "a bounded wait on the device ran out";
    case NTB_ERR_LIMIT: return "size beyond a fixed limit";
    default: return "unknown error";
    }
}

}
