/*
 * The split-K tensor-core kernel (clusters of 2 or 4 CTAs share one output tile and
 * exchange partial sums through distributed shared memory) and its launcher.
 */
#include "ntb_tc_common.cuh"

namespace ntb {

namespace {

/* barrier probe that also acquires what other CTAs of the cluster wrote before arriving */
__device__ __forceinline__ uint32_t MbarTryWaitCluster(uint32_t bar, uint32_t parity, uint32_t hintNs)
{
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar), "r"(parity), "r"(hintNs) : "memory");
    return done;
}

__device__ __forceinline__ bool MbarWaitClusterWarp(uint32_t bar, uint32_t parity, volatile int * abortFlag, int * status)
{
    uint32_t ok = 1;
    if ((threadIdx.x & 31) == 0) {
        const long long t0 = clock64();
        for (uint32_t it = 0; ; ++it) {
            if (MbarTryWaitCluster(bar, parity, 200))
                break;
            if ((it & 63u) == 63u) {
                if (*abortFlag) { ok = 0; break; }
                if (clock64() - t0 > WaitLimit(status)) {
                    *abortFlag = 1;
                    atomicExch(status, NTB_ERR_DEVICE_WAIT);
                    ok = 0;
                    break;
                }
            }
        }
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    /* every lane acquires at cluster scope before it reads what the peers wrote */
    asm volatile("fence.acq_rel.cluster;" ::: "memory");
    return ok != 0;
}

/*
 * fp16 GEMM for products with few output tiles and a long K (weight gradients: K is the
 * number of tokens): a cluster of S CTAs shares one 128 x 128 output tile, CTA r running the
 * main loop over the r-th part of the k-blocks with its own TMA pipeline and TMEM
 * accumulators. The partial sums are combined through distributed shared memory as a
 * reduce-scatter: CTA d owns columns [d*W, (d+1)*W) of the tile (W = 128 / S); every other
 * CTA writes its fp32 partial of that slice into CTA d's receive area (st.shared::cluster,
 * swizzled so that one-row-per-lane writes do not collide) and arrives on CTA d's barrier;
 * CTA d adds the S - 1 partials to its own in rank order -- a fixed order, so results do not
 * depend on timing -- and runs the usual epilogue on its slice. No global workspace, no
 * atomics. The receive area is double-buffered; a sender cannot be two tiles ahead of a
 * receiver, because its own wait for tile i+1 needs the receiver's partials of tile i+1,
 * which the receiver's warp sends only after it has consumed tile i.
 */
template <int S, int STAGES, int G, typename OutT, bool OLDC>
__global__ void __cluster_dims__(S, 1, 1) __launch_bounds__(192, 1)
GemmTcSplitKernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmC, TcParams p)
{
    constexpr int ES = 2;
    constexpr int EPR = ROW_BYTES / ES;
    constexpr int BN = 128;
    constexpr int W = BN / S;                           /* columns of the tile this CTA finishes */
    constexpr int B_TILE_BYTES = BN * ROW_BYTES;
    constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
    constexpr int TMEM_COLS = 256;
    constexpr int KSTEPS = ROW_BYTES / UMMA_K_BYTES;
    constexpr int SLOT_BYTES = BM * W * 4;              /* one sender's slice: 128 rows x W floats */
    constexpr int RECV_BYTES = 2 * (S - 1) * SLOT_BYTES;
    constexpr int NSTG = STAGES / G;                    /* barrier pairs: G k-blocks share a hand-shake */
    static_assert((S == 2 || S == 4) && STAGES % G == 0, "cluster size, k-blocks per hand-shake");

    extern __shared__ uint8_t smemRaw[];
    __shared__ __align__(8) uint64_t barFull[STAGES];
    __shared__ __align__(8) uint64_t barEmpty[STAGES];
    __shared__ __align__(8) uint64_t barTFull[2];
    __shared__ __align__(8) uint64_t barTEmpty[2];
    __shared__ __align__(8) uint64_t barOldC[8];    /* per epilogue warp and staging box: old C values have landed */
    __shared__ __align__(8) uint64_t barRecv[2];
    __shared__ uint32_t tmemBaseSlot;
    __shared__ int abortFlag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ClusterCtaRank();
    const uint32_t smemBase = (SmemAddr(smemRaw) + 1023u) & ~1023u;
    const uint32_t recvBase = smemBase + STAGES * STAGE_BYTES;
    volatile int * abortPtr = &abortFlag;
    /* a kernel launched behind this one with programmatic serialisation may start setting up */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (threadIdx.x == 128 || threadIdx.x == 160) {
        /* idle epilogue lanes in the scheduler partitions of the producer warp and of the
           MMA warp pull the kernel parameters (one of them also the tensor maps) towards
           their constant caches while the other warps set up */
        if (threadIdx.x == 128) {
            PrefetchTensorMap(&tmA);
            PrefetchTensorMap(&tmB);
            if (p.cTma)
                PrefetchTensorMap(&tmC);
        }
        int touch = 0;
        const int * words = (const int *)&p;
        for (int w = 0; w < (int)(sizeof(TcParams) / sizeof(int)); w += 8)
            touch += words[w];
        asm volatile("" :: "r"(touch));
    }
    if (warp == 0) {
        if (lane < STAGES) {
            MbarInit(SmemAddr(&barFull[lane]), 1);
            MbarInit(SmemAddr(&barEmpty[lane]), 1);
        }
        else if (lane >= 8 && lane < 10) {
            MbarInit(SmemAddr(&barTFull[lane - 8]), 1);
            MbarInit(SmemAddr(&barTEmpty[lane - 8]), 4);
            MbarInit(SmemAddr(&barRecv[lane - 8]), (S - 1) * 4);
        }
        else if (OLDC && lane >= 16 && lane < 24) {
            MbarInit(SmemAddr(&barOldC[lane - 16]), 1);
        }
        if (lane == 0)
            abortFlag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(SmemAddr(&tmemBaseSlot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    TcFenceBefore();
    ClusterSync();              /* every CTA's barriers exist before a peer signals them */
    TcFenceAfter();
    const uint32_t tmemBase = *(volatile uint32_t *)&tmemBaseSlot;

    const int kBlocks = (p.K + EPR - 1) / EPR;
    const int kbLo = (int)((long long)kBlocks * rank / S), kbHi = (int)((long long)kBlocks * (rank + 1) / S);
    /* set-up is done; nothing before this point touched global memory. A kernel launched
       with programmatic serialisation waits here for the kernels before it in the stream. */
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int firstTile = blockIdx.x / S;
    const int tileStep = gridDim.x / S;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = firstTile; ok && t < p.totalTiles; t += tileStep) {
                TileCoord tc = DecodeTile(t, p);
                const int m0 = tc.mBlk * BM, n0 = tc.nBlk * BN;
                const int ba = BatchCoord(p.aSel, tc.prob, p);
                const int bb = BatchCoord(p.bSel, tc.prob, p);
                const bool aMN = p.aMN != 0, bMN = p.bMN != 0;
                int * const status = p.status;
                for (int kb = kbLo; kb < kbHi; kb += G) {
                    ok = MbarWait(SmemAddr(&barEmpty[s]), ph ^ 1u, abortPtr, status);
                    if (!ok)
                        break;
                    const uint32_t full = SmemAddr(&barFull[s]);
                    const int nb = G == 1 ? 1 : (kbHi - kb < G ? kbHi - kb : G);
                    MbarExpectTx(full, (uint32_t)nb * STAGE_BYTES);
#pragma unroll
                    for (int j = 0; j < G; j++) {
                        if (j < nb) {
                            const uint32_t aDst = smemBase + (uint32_t)(s * G + j) * STAGE_BYTES;
                            const uint32_t bDst = aDst + A_TILE_BYTES;
                            const int k0 = (kb + j) * EPR;
                            if (!aMN) {
                                TmaLoad3D(aDst, &tmA, full, k0, m0, ba);
                            }
                            else {
#pragma unroll
                                for (int i = 0; i < BM / EPR; i++)
                                    TmaLoad3D(aDst + i * EPR * ROW_BYTES, &tmA, full, m0 + i * EPR, k0, ba);
                            }
                            if (!bMN) {
                                TmaLoad3D(bDst, &tmB, full, k0, n0, bb);
                            }
                            else {
#pragma unroll
                                for (int i = 0; i < BN / EPR; i++)
                                    TmaLoad3D(bDst + i * EPR * ROW_BYTES, &tmB, full, n0 + i * EPR, k0, bb);
                            }
                        }
                    }
                    if (++s == NSTG) { s = 0; ph ^= 1u; }
                }
            }
        }
    }
    else if (warp == 1) {
        if (lane == 0) {
            const uint32_t iDesc = InstrDesc(0, p.aMN, p.bMN, BN);
            const uint32_t aLbo = p.aMN ? EPR * ROW_BYTES : 16, bLbo = p.bMN ? EPR * ROW_BYTES : 16;
            const uint32_t mnStep = (UMMA_K_BYTES / ES) * ROW_BYTES;
            const uint32_t aStep = p.aMN ? mnStep : UMMA_K_BYTES;
            const uint32_t bStep = p.bMN ? mnStep : UMMA_K_BYTES;
            int s = 0;
            uint32_t ph = 0, it = 0;
            bool ok = true;
            int * const status = p.status;
            const uint64_t aD0 = SmemDesc(smemBase, aLbo, 1024, 2);
            const uint64_t bD0 = SmemDesc(smemBase + A_TILE_BYTES, bLbo, 1024, 2);
            const uint32_t aLo0 = (uint32_t)aD0, aHiW = (uint32_t)(aD0 >> 32);
            const uint32_t bLo0 = (uint32_t)bD0, bHiW = (uint32_t)(bD0 >> 32);
            const uint32_t aStep4 = aStep >> 4, bStep4 = bStep >> 4;
            const uint32_t barFull0 = SmemAddr(&barFull[0]), barEmpty0 = SmemAddr(&barEmpty[0]);
            uint32_t stageOff = 0;
            for (int t = firstTile; ok && t < p.totalTiles; t += tileStep, ++it) {
                const uint32_t buf = it & 1u;
                ok = MbarWait(SmemAddr(&barTEmpty[buf]), ((it >> 1) & 1u) ^ 1u, abortPtr, status);
                if (!ok)
                    break;
                TcFenceAfter();
                const uint32_t dTmem = tmemBase + buf * BN;
                uint32_t acc = 0u;
                for (int kb = kbLo; kb < kbHi; kb += G) {
                    ok = MbarWait(barFull0 + (uint32_t)s * 8u, ph, abortPtr, status);
                    if (!ok)
                        break;
                    TcFenceAfter();
                    const int nb = G == 1 ? 1 : (kbHi - kb < G ? kbHi - kb : G);
#pragma unroll
                    for (int j = 0; j < G; j++) {
                        if (j < nb) {
                            uint32_t aLo = aLo0 + stageOff + (uint32_t)j * (STAGE_BYTES >> 4);
                            uint32_t bLo = bLo0 + stageOff + (uint32_t)j * (STAGE_BYTES >> 4);
#pragma unroll
                            for (int k = 0; k < KSTEPS; k++) {
                                TcMmaLH<0>(dTmem, aLo, aHiW, bLo, bHiW, iDesc, acc);
                                acc = 1u;
                                aLo += aStep4;
                                bLo += bStep4;
                            }
                        }
                    }
                    TcCommit(barEmpty0 + (uint32_t)s * 8u);
                    stageOff += (uint32_t)G * (STAGE_BYTES >> 4);
                    if (++s == NSTG) { s = 0; ph ^= 1u; stageOff = 0; }
                }
                if (ok)
                    TcCommit(SmemAddr(&barTFull[buf]));
            }
        }
    }
    else {
        const int sub = warp & 3;
        const int rowInTile = sub * 32 + lane;
        uint32_t it = 0;
        bool ok = true;
        TileWriter<OutT, OLDC> writer;
        writer.Init(recvBase + RECV_BYTES, sub, &tmC, &barOldC[sub * 2], abortPtr, p.status);
        for (int t = firstTile; ok && t < p.totalTiles; t += tileStep, ++it) {
            TileCoord tc = DecodeTile(t, p);
            const uint32_t buf = it & 1u;
            const int row0 = tc.mBlk * BM + sub * 32, row = row0 + lane;
            const int n0 = tc.nBlk * BN;
            int pp, qq;
            SplitProb(p, tc.prob, pp, qq);
            const int bc = BatchCoord(p.cSel, tc.prob, p);
            OutT * cRow = (OutT *)p.c + pp * p.sCp + qq * p.sCq + (long long)row * p.ldc;
            const bool rowOk = row < p.M;
            writer.BeginTile(p, cRow + n0 + (int)rank * W, row0, 0, 1, n0 + (int)rank * W, W, bc, lane);
            ok = MbarWaitWarp(SmemAddr(&barTFull[buf]), (it >> 1) & 1u, abortPtr, p.status, (uint32_t)p.epiHint);
            if (!ok)
                break;
            TcFenceAfter();
            const uint32_t tRow = tmemBase + ((uint32_t)(sub * 32) << 16) + buf * BN;
            /* this CTA's partial sums of the other CTAs' column slices go to their receive areas */
#pragma unroll
            for (int dd = 1; dd < S; dd++) {
                const uint32_t d = (rank + dd) % S;
                const uint32_t slot = rank < d ? rank : rank - 1;          /* position among d's senders */
                const uint32_t dstRow = MapToCta(recvBase + (buf * (S - 1) + slot) * SLOT_BYTES
                                                 + rowInTile * (W * 4), d);
#pragma unroll
                for (int cc = 0; cc < W / 32; cc++) {
                    float v[32];
                    TmemLoad32(tRow + d * W + cc * 32, v);
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const uint32_t chunk = (uint32_t)((cc * 8 + j) ^ (lane & 7));
                        asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};"
                                     :: "r"(dstRow + (chunk << 4)), "f"(v[j * 4]), "f"(v[j * 4 + 1]), "f"(v[j * 4 + 2]),
                                        "f"(v[j * 4 + 3]) : "memory");
                    }
                }
            }
            asm volatile("fence.acq_rel.cluster;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
#pragma unroll
                for (int dd = 1; dd < S; dd++)
                    MbarArriveCluster(MapToCta(SmemAddr(&barRecv[buf]), (rank + dd) % S));
            }
            /* this CTA's slice: own partial plus the others', in rank order */
            ok = MbarWaitClusterWarp(SmemAddr(&barRecv[buf]), (it >> 1) & 1u, abortPtr, p.status);
            if (!ok)
                break;
#pragma unroll
            for (int cc = 0; cc < W / 32; cc++) {
                float v[32];
                TmemLoad32(tRow + rank * W + cc * 32, v);
#pragma unroll
                for (int sl = 0; sl < S - 1; sl++) {
                    const uint32_t srcRow = recvBase + (buf * (S - 1) + sl) * SLOT_BYTES + rowInTile * (W * 4);
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const uint32_t chunk = (uint32_t)((cc * 8 + j) ^ (lane & 7));
                        float4 r;
                        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                     : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "r"(srcRow + (chunk << 4)) : "memory");
                        v[j * 4] += r.x; v[j * 4 + 1] += r.y; v[j * 4 + 2] += r.z; v[j * 4 + 3] += r.w;
                    }
                }
                const int c0 = n0 + (int)rank * W + cc * 32;
                if (c0 < p.N)
                    writer.Put32(p, cRow, rowOk, row0, c0, bc, v, lane);
            }
            TcFenceBefore();
            __syncwarp();
            if (lane == 0)
                MbarArrive(SmemAddr(&barTEmpty[buf]));
        }
        writer.Finish(lane);
    }

    __syncwarp();
    if (*abortPtr) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
    }
    TcFenceBefore();
    ClusterSync();              /* no CTA's shared memory goes away while a peer may still write to it */
    TcFenceAfter();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     :: "r"(tmemBase), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

template <int S, int STAGES, int G, typename OutT, bool OLDC>
int LaunchSplit(const CUtensorMap & tmA, const CUtensorMap & tmB, const CUtensorMap & tmC, const TcParams & tp, int clusters,
                cudaStream_t stream)
{
    constexpr int smem = (A_TILE_BYTES + 128 * ROW_BYTES) * STAGES + 2 * (S - 1) * (BM * (128 / S) * 4) + EPI_BYTES + 1024;
    auto kern = GemmTcSplitKernel<S, STAGES, G, OutT, OLDC>;
    static SmemOptIn optIn;
    if (!optIn.Ensure((const void *)kern, smem))
        return NTB_ERR_CUDA;
    const cudaError_t err = LaunchPdl(kern, S * clusters, 192, smem, stream, tmA, tmB, tmC, tp);
    CountLaunch();
    return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? NTB_OK : NTB_ERR_CUDA;
}

}

int LaunchSplitKernel(int split, int g, bool half, bool oldc, const CUtensorMap * maps, const TcParams & tp,
                      int clusters, cudaStream_t stream)
{
#define NTB_SPLIT(SS, ST, GG, T) (oldc ? LaunchSplit<SS, ST, GG, T, true>(maps[0], maps[1], maps[2], tp, clusters, stream) \
                                       : LaunchSplit<SS, ST, GG, T, false>(maps[0], maps[1], maps[2], tp, clusters, stream))
    if (split == 2) {
        if (g == 1)
            return half ? NTB_SPLIT(2, 4, 1, __half) : NTB_SPLIT(2, 4, 1, float);
        return half ? NTB_SPLIT(2, 4, 2, __half) : NTB_SPLIT(2, 4, 2, float);
    }
    return half ? NTB_SPLIT(4, 3, 1, __half) : NTB_SPLIT(4, 3, 1, float);
#undef NTB_SPLIT
}

}
