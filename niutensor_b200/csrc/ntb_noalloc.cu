/*
 * ntb_gemm_host_noalloc: the host-buffer product for callers that must not allocate.
 *
 * Who needs it: a NiuTensor process normally hands all of a GPU's free memory to its XMem
 * pools at start-up, so a later cudaMalloc inside a library can simply fail; and trainer
 * worker threads that share a device cannot afford cudaMalloc / cudaFree either, because
 * both stall every stream of the device while they run. The regular host-buffer entry
 * point (ntb_gemm_host) grows its staging buffers with cudaMalloc, and every other entry
 * point creates its device context (a cudaMalloc'ed status word) on first use. This one
 * touches no allocator at all: its device-side scratch -- the status word the kernels
 * write when a bounded wait runs out, plus the staging space for a, b and c -- is the
 * fixed array below, which every GPU that loads this library holds until the process
 * exits.
 *
 * Limit: the staged a, b and c (each rounded up to 256 bytes) must fit in
 * NTB_NOALLOC_MAX_BYTES; larger problems are refused with NTB_ERR_LIMIT.
 *
 * Sharing: all calls on a device use the same array, and it keeps what the previous call
 * left in it. Each call clears the status word before it launches; nothing else needs to
 * start at zero, because the staging areas are fully overwritten by the copies (c only when
 * beta != 0, and it is never read otherwise). Two calls that overlap on one GPU -- from two
 * threads, or on two streams -- race on the array; callers serialise them.
 *
 * Set-up: the first call on a device resolves the array's device address (with that device
 * current) and caches it. With CUDA's default lazy module loading that look-up is also the
 * moment the runtime loads the module holding the array and reserves its 16 MiB on the
 * device, so the promise "no allocation" holds from the second call on: make the first call
 * (a tiny warm-up product will do) early -- before the host's memory pools take what is left
 * of the GPU, and before the process begins any stream capture -- or start the process with
 * CUDA_MODULE_LOADING=EAGER, which reserves the array when the library is loaded.
 *
 * Routing follows ntb_set_route() / NTB_ROUTE like every other entry point, and
 * ntb_last_route() reports the kernel family used.
 */
#include "ntb_internal.h"
#include <mutex>
#include <cstring>

namespace ntb {

namespace {

constexpr size_t HEADER_BYTES = 256;          /* status word, padded so staging stays 256-aligned */

/* In host code this name is only a handle for the runtime's symbol calls, not an address a
   kernel could use; the device address comes from cudaGetSymbolAddress in SetUp(). */
static __device__ __align__(256) unsigned char gNoAllocScratch[HEADER_BYTES + NTB_NOALLOC_MAX_BYTES];

constexpr int MAX_DEV = 64;
std::mutex gSetUpLock;
unsigned char * gScratchAddr[MAX_DEV] = { nullptr };
int gSmCount[MAX_DEV] = { 0 };

size_t RoundUp256(size_t n)
{
    return (n + 255) & ~(size_t)255;
}

/* once per device, with that device current */
int SetUp(int dev, unsigned char ** out, int * smCount)
{
    std::lock_guard<std::mutex> g(gSetUpLock);
    if (!gScratchAddr[dev]) {
        unsigned char * ptr = nullptr;
        if (cudaGetSymbolAddress((void **)&ptr, gNoAllocScratch) != cudaSuccess || !ptr ||
            cudaDeviceGetAttribute(&gSmCount[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
            cudaGetLastError();
            return NTB_ERR_CUDA;
        }
        gScratchAddr[dev] = ptr;
    }
    *out = gScratchAddr[dev];
    *smCount = gSmCount[dev];
    return NTB_OK;
}

}

}

using namespace ntb;

extern "C" int ntb_gemm_host_noalloc(int devID, void * stream,
                                     const void * a, int transA, const void * b, int transB, void * c,
                                     int dtypeAB, int dtypeC,
                                     int na, int ma, int nb, int mb, int nc, int mc,
                                     float alpha, float beta)
{
    if (!a || !b || !c || devID < 0 || devID >= MAX_DEV)
        return NTB_ERR_ARG;
    if ((transA != NTB_X_TRANS && transA != NTB_X_NOTRANS) || (transB != NTB_X_TRANS && transB != NTB_X_NOTRANS))
        return NTB_ERR_ARG;
    if (na < 0 || ma < 0 || nb < 0 || mb < 0 || nc < 0 || mc < 0)
        return NTB_ERR_ARG;
    const bool f16 = dtypeAB == NTB_X_FLOAT16 && (dtypeC == NTB_X_FLOAT16 || dtypeC == NTB_X_FLOAT);
    const bool f32 = dtypeAB == NTB_X_FLOAT && dtypeC == NTB_X_FLOAT;
    if (!f16 && !f32)
        return NTB_ERR_DTYPE;
    const int an = transA == NTB_X_TRANS ? ma : na, am = transA == NTB_X_TRANS ? na : ma;
    const int bn = transB == NTB_X_TRANS ? mb : nb, bm = transB == NTB_X_TRANS ? nb : mb;
    if (am != bn || an != nc || bm != mc)
        return NTB_ERR_SHAPE;
    if (nc == 0 || mc == 0)
        return NTB_OK;

    /* The staged copies get row pitches that are multiples of 16 bytes (the host buffers are
       packed), so that every staged operand can be described to TMA whatever its extents. */
    const size_t rowA = (size_t)ma * ElemSize(dtypeAB), rowB = (size_t)mb * ElemSize(dtypeAB), rowC = (size_t)mc * ElemSize(dtypeC);
    const size_t pitchA = (rowA + 15) & ~(size_t)15, pitchB = (rowB + 15) & ~(size_t)15, pitchC = (rowC + 15) & ~(size_t)15;
    const size_t aBytes = (size_t)na * pitchA;
    const size_t bBytes = (size_t)nb * pitchB;
    const size_t cBytes = (size_t)nc * pitchC;
    if (RoundUp256(aBytes) + RoundUp256(bBytes) + RoundUp256(cBytes) > (size_t)NTB_NOALLOC_MAX_BYTES)
        return NTB_ERR_LIMIT;      /* the fixed scratch array cannot hold this problem */

    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess || (prev != devID && cudaSetDevice(devID) != cudaSuccess)) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    int rc = NTB_OK;
    int hostStatus = 0;
    bool queued = false, drained = false;     /* work was put on the stream / the stream was synchronised */
    do {
        unsigned char * scratch = nullptr;
        DeviceCtx ctx;
        memset(&ctx, 0, sizeof(ctx));
        ctx.devID = devID;
        rc = SetUp(devID, &scratch, &ctx.smCount);
        if (rc != NTB_OK)
            break;
        ctx.status = (int *)scratch;
        unsigned char * dA = scratch + HEADER_BYTES;
        unsigned char * dB = dA + RoundUp256(aBytes);
        unsigned char * dC = dB + RoundUp256(bBytes);
        cudaStream_t st = (cudaStream_t)stream;

        rc = NTB_ERR_CUDA;
        /* the array still holds the previous call's status word: clear it */
        if (cudaMemsetAsync(scratch, 0, HEADER_BYTES, st) != cudaSuccess)
            break;
        queued = true;
        if (aBytes && cudaMemcpy2DAsync(dA, pitchA, a, rowA, rowA, (size_t)na, cudaMemcpyHostToDevice, st) != cudaSuccess)
            break;
        if (bBytes && cudaMemcpy2DAsync(dB, pitchB, b, rowB, rowB, (size_t)nb, cudaMemcpyHostToDevice, st) != cudaSuccess)
            break;
        if (beta != 0.f && cudaMemcpy2DAsync(dC, pitchC, c, rowC, rowC, (size_t)nc, cudaMemcpyHostToDevice, st) != cudaSuccess)
            break;

        Problem p;
        memset(&p, 0, sizeof(p));
        p.a = dA; p.b = dB; p.c = dC;
        p.dtAB = dtypeAB; p.dtC = dtypeC;
        p.aMN = transA == NTB_X_TRANS;
        p.bMN = transB == NTB_X_NOTRANS;
        p.M = an; p.N = bm; p.K = am;
        p.aRows = na; p.aCols = ma; p.bRows = nb; p.bCols = mb;
        p.lda = (long long)(pitchA / ElemSize(dtypeAB)); p.ldb = (long long)(pitchB / ElemSize(dtypeAB));
        p.ldc = (long long)(pitchC / ElemSize(dtypeC));
        p.count = 1; p.Q = 1;
        p.alpha = alpha; p.beta = beta;
        int route = NTB_ROUTE_NONE;
        const int forced = ForcedRoute();
        if (forced != NTB_ROUTE_SIMT && TcEligible(p)) {
            rc = LaunchTc(ctx, p, st, &route);
        }
        else if (forced != NTB_ROUTE_SIMT && forced != NTB_ROUTE_TC_F16_PAIR && LdgEligible(p)) {
            rc = LaunchLdg(ctx, p, st, &route);         /* not reached with the padded staging pitches; kept for safety */
        }
        else if (forced == NTB_ROUTE_TC_F16 || forced == NTB_ROUTE_TC_3XTF32 || forced == NTB_ROUTE_TC_F16_PAIR) {
            rc = NTB_ERR_ARG;                       /* a tensor-core route was demanded and cannot address this */
        }
        else {
            rc = LaunchSimt(ctx, p, st);
            route = NTB_ROUTE_SIMT;
        }
        if (rc != NTB_OK)
            break;
        SetLastRoute(route);
        rc = NTB_ERR_CUDA;
        if (cudaMemcpy2DAsync(c, rowC, dC, pitchC, rowC, (size_t)nc, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
            cudaMemcpyAsync(&hostStatus, scratch, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
            cudaStreamSynchronize(st) != cudaSuccess)
            break;
        drained = true;
        rc = hostStatus == 0 ? NTB_OK : NTB_ERR_DEVICE_WAIT;
    } while (0);
    /* After a failure part-way, copies already queued may still read a / b or write the
       shared array: let them finish, so that the caller's buffers are free on return and the
       next (serialised) call does not race with this one's leftovers. */
    if (queued && !drained)
        cudaStreamSynchronize((cudaStream_t)stream);
    if (rc == NTB_ERR_CUDA)
        cudaGetLastError();
    if (prev >= 0 && prev != devID)
        cudaSetDevice(prev);
    return rc;
}
