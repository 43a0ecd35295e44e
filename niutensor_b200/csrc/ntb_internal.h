/* Internal declarations shared by the API layer and the kernel launchers. */
#ifndef NTB_INTERNAL_H
#define NTB_INTERNAL_H

#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>
#include <stdlib.h>
#include <atomic>
#include <mutex>
#include "../../include/ntb_gemm.h"

namespace ntb {

/*
 * One launch: `count` problems of one shape. Problem i splits into (p, q) =
 * (i / Q, i % Q); operand x of problem i starts at x + p * sXp + q * sXq (elements).
 *   strided batched: Q = 1, sXp = strideX
 *   general form   : Q = bBlockNum, A walks p, B walks q, C walks p * Q + q
 */
struct Problem {
    const void * a;
    const void * b;
    void * c;
    int dtAB, dtC;          /* NTB_X_FLOAT / NTB_X_FLOAT16 */
    int aMN, bMN;           /* operand is MN-major (M resp. N contiguous) instead of K-major */
    int M, N, K;
    int aRows, aCols, bRows, bCols;   /* stored extents */
    long long lda, ldb, ldc;
    int count, Q;
    long long sAp, sAq, sBp, sBq, sCp, sCq;
    float alpha, beta;
    const void * bias;      /* optional row vector of N values (type of c) added to every row of every problem */
    int act;                /* NTB_ACT_NONE / NTB_ACT_RECTIFY, applied last */
    /* further destinations of the result, same shape and pitch as c (other GPUs' copies of C
       mapped into this process, or other buffers of this GPU) */
    void * peers[NTB_MAX_PEERS];
    int nPeers;
    int peerMcast;          /* peers[0] is an NVLink multicast address: one multimem store reaches every GPU bound to it */
};

struct DeviceCtx {
    int devID;
    int smCount;
    int * status;           /* two device words: [0] written by a kernel that gave up a wait, [1] test-only wait limit */
    void * stage[3];        /* host-buffer entry point: device staging for a, b, c */
    size_t stageBytes[3];
    /* host-buffer entry point, pipelined form: copy-in and copy-out streams, one event pair per chunk */
    cudaStream_t copyIn, copyOut;
    cudaEvent_t evIn[16], evOut[16], evStart;
    bool pipeReady;
    /* fp32-as-two-halves route: planes of a and b, scale vectors; shared by the calls on this
       device, which are ordered on the device through scratchEvent */
    bool mayAllocate;       /* false for the context of the entry point that must not allocate */
    void * scratch[4];         /* 0-2: operand planes and vectors of the pre-passes; 3: partial sums of the split on CTA pairs */
    size_t scratchBytes[4];
    void * countersCleared;    /* the slot-3 buffer whose counters have been zeroed */
    cudaEvent_t scratchEvent;
    bool haveScratchEvent;
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn GetEncodeTiled();

/* true when the tcgen05/TMA route can address this problem (alignment, strides) */
bool TcEligible(const Problem & p);
/* *route receives the NTB_ROUTE_* code of the kernel launched */
int LaunchTc(const DeviceCtx & ctx, const Problem & p, cudaStream_t stream, int * route);
int LaunchSimt(const DeviceCtx & ctx, const Problem & p, cudaStream_t stream);
/* tensor-core route for operands TMA cannot address (base or pitch not a multiple of 16 bytes):
   loader warps fetch them with ordinary loads */
bool LdgEligible(const Problem & p);
int LaunchLdg(const DeviceCtx & ctx, const Problem & p, cudaStream_t stream, int * route);
/* realigning pre-pass (ntb_repack.cu): operands TMA cannot address are copied into 16-byte
   aligned rows in scratch memory and the product runs on the TMA-fed kernels; LaunchRepacked
   returns NTB_ERR_ARG, with nothing launched, when that does not apply */
bool RepackWorthwhile(const DeviceCtx & ctx, const Problem & p);
int LaunchRepacked(const DeviceCtx & ctx, const Problem & p, cudaStream_t stream, int * route);
/* NTB_PDL=0 in the environment turns programmatic stream serialisation off */
inline bool PdlEnabled()
{
    const char * v = getenv("NTB_PDL");
    return !(v && *v && atoi(v) == 0);
}

/* Launch with programmatic stream serialisation: the next kernel of the stream that was
   launched the same way may start its set-up (barrier initialisation, TMEM allocation,
   descriptor fetch) while this one drains; it waits (griddepcontrol.wait) before its first
   access to global memory. Kernels launched any other way are ordered as always.
   NTB_PDL=0 turns it off. */
template <typename... Params, typename... Args>
cudaError_t LaunchPdl(void (*kern)(Params...), int grid, int block, int smem, cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)block, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = PdlEnabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

/* tile choice of the cost model for p alone: > 0 single-CTA width, <= 0 a cluster kernel (pair or split-K) */
int TcTileChoice(const DeviceCtx & ctx, const Problem & p);
/* two tensor-core-eligible problems of equal operand and output types in one launch */
int LaunchTcTwo(const DeviceCtx & ctx, const Problem & p0, const Problem & p1, cudaStream_t stream);

/* the device's context (created on first use); the caller has made `dev` current */
DeviceCtx * CtxFor(int dev);
/* scratch buffer `slot` of the device's context, at least `bytes` long (grown with cudaMalloc when
   needed, after the device has finished with the old one); the device is current */
int EnsureScratch(const DeviceCtx & ctx, int slot, size_t bytes, void ** out);
/* orders this stream behind the last use of the device's scratch / marks a new last use */
/* scratch slot 3 as flagBytes of zeroed counters followed by workBytes of workspace; the counters
   are cleared on the stream when the buffer is new or after a device wait ran out (kernels
   leave them at zero otherwise) */
int EnsureCounted(const DeviceCtx & ctx, size_t workBytes, size_t flagBytes, cudaStream_t stream, float ** work, int ** flags);
int ScratchAcquire(const DeviceCtx & ctx, cudaStream_t stream);
int ScratchRelease(const DeviceCtx & ctx, cudaStream_t stream);
/* tensor maps of an operand and of the output (ntb_tc.cu) */
int EncodeOperandMap(CUtensorMap * map, int mode, const void * base, int mnMajor, int rows, int cols,
                     long long ld, long long batchStride, int batchExtent, int tileRows);
int EncodeOutputMap(CUtensorMap * map, int dtC, void * base, int rows, int cols, long long ld,
                    long long batchStride, int batchExtent);
/* large 2-D fp32 products as three half-precision products of split operands (ntb_tc_f32pair.cu) */
bool F32SplitEligible(const DeviceCtx & ctx, const Problem & p);
int LaunchF32Split(const DeviceCtx & ctx, const Problem & p, cudaStream_t stream);

void CountLaunch();
int ForcedRoute();           /* value of the last ntb_set_route() */
int InjectedSkipKBlock();    /* test hook (ntb_debug_inject): k-block whose loads the producers leave out, or -1 */
void CountVariant(int index);  /* NTB_COUNT_*: variants of a route, read through ntb_route_count() */
void SetLastRoute(int route); /* what ntb_last_route() reports for the calling thread */

/* The opt-in to more than 48 KB of dynamic shared memory is per kernel and per device. One
   object per kernel instantiation; threads that share a device may launch concurrently, so
   the flag is only published after the attribute call has returned. */
struct SmemOptIn {
    std::atomic<int> done[64];
    std::mutex lock;
    SmemOptIn() { for (int i = 0; i < 64; i++) done[i].store(0); }
    bool Ensure(const void * kern, int smem)
    {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess)
            return false;
        const bool tracked = dev >= 0 && dev < 64;
        if (tracked && done[dev].load(std::memory_order_acquire))
            return true;
        std::lock_guard<std::mutex> g(lock);
        if (tracked && done[dev].load(std::memory_order_relaxed))
            return true;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return false;
        if (tracked)
            done[dev].store(1, std::memory_order_release);
        return true;
    }
};

static inline size_t ElemSize(int dt) { return dt == NTB_X_FLOAT16 ? 2 : 4; }

}

#endif
