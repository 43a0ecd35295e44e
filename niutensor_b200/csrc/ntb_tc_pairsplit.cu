/*
 * Split-K on CTA pairs: S pairs (S = 2 or 4) share ONE 256 x 256 output tile and exchange
 * partial sums through an L2-resident workspace, and its launcher.
 */
#include "ntb_tc_common.cuh"

namespace ntb {

namespace {

/* bounded wait of a warp until the counter in global memory, which warps of other CTAs
   increment with release semantics, has reached `want` (lane 0 polls) */
__device__ __forceinline__ bool CounterWaitWarp(const int * counter, int want, volatile int * abortFlag, int * status)
{
    uint32_t ok = 1;
    if ((threadIdx.x & 31) == 0) {
        const long long t0 = clock64();
        for (uint32_t it = 1; ; ++it) {
            int v;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
            if (v >= want)
                break;
            if ((it & 15u) == 0) {
                if (*abortFlag) { ok = 0; break; }
                if (clock64() - t0 > WaitLimit(status)) {
                    *abortFlag = 1;
                    atomicExch(status, NTB_ERR_DEVICE_WAIT);
                    ok = 0;
                    break;
                }
            }
            __nanosleep(40);
        }
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0;
}

/* untiled bulk copy global -> shared, completion counted in bytes on an mbarrier of this CTA */
__device__ __forceinline__ void BulkLoad(uint32_t dst, const void * src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

/*
 * fp16 GEMM for products with few 256 x 256 output tiles and a long K (second FFN product,
 * weight gradients): whole tiles would occupy a fraction of the SMs, smaller tiles move
 * twice the operand bytes per flop. Here S CTA pairs (ordinary clusters of two, so every SM
 * can take part; clusters of 2 S CTAs sharing the sums through distributed shared memory
 * were measured first and found room for only a third of the SMs) share one tile. Pair q of
 * a tile runs the main loop of the CTA-pair kernel (tcgen05 cta_group::2, 256 x 256 x 16
 * MMAs, each CTA loading its 128 rows of A and its half of the B tile) over the q-th part of
 * the k-blocks. Then the partial sums are combined as a reduce-scatter: pair d owns columns
 * [d W, (d + 1) W) of the tile, W = 256 / S. Every epilogue warp of every other pair writes
 * its 32 rows of that slice, as raw fp32, into the workspace (coalesced 512-byte stores),
 * fences and increments the counter of the owner's warp that holds the same rows; that warp
 * waits for S - 1 increments (bounded), clears the counter for the next launch, pulls the
 * S - 1 pieces into the idle operand ring with bulk copies (one request each, so the
 * latency of L2 is paid once, not per load instruction), adds them to its own in pair order --
 * a fixed order, so results do not depend on timing -- and runs the usual epilogue on
 * 32 rows x W columns. Every pair waits for every other pair of its tile: the launcher only
 * uses the kernel when all pairs of the grid are resident at once.
 *
 * Shared memory: STAGES x 32 KB operand ring. Once the accumulator is complete the ring is
 * idle (every load that was issued has been consumed): its first 32 KB become the epilogue's
 * staging boxes, the next 4 x (S - 1) x 32 x W x 4 bytes the landing area of the pieces.
 */
template <int S, int STAGES, int G, typename OutT, bool OLDC>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
GemmTcPairSplitKernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmC, TcParams p)
{
    constexpr int ES = 2;
    constexpr int EPR = ROW_BYTES / ES;                 /* 64 halves of K per stage */
    constexpr int BN = 256, BNH = 128, PM = 2 * BM;
    constexpr int W = BN / S;                           /* columns of the tile this pair finishes */
    constexpr int STAGE_BYTES = A_TILE_BYTES + BNH * ROW_BYTES;
    constexpr int TMEM_COLS = 256;
    constexpr int KSTEPS = ROW_BYTES / UMMA_K_BYTES;
    constexpr int PIECE_BYTES = 32 * W * 4;             /* one warp's rows of one sender's slice */
    constexpr int PIECE_V4 = PIECE_BYTES / 16;
    constexpr int NSTG = STAGES / G;                    /* barrier pairs: G k-blocks share a hand-shake */
    static_assert(S == 2 || S == 4, "pairs per tile");
    static_assert(STAGES % G == 0, "k-blocks per hand-shake");
    static_assert(STAGES * STAGE_BYTES >= EPI_BYTES + 4 * (S - 1) * PIECE_BYTES, "staging boxes and landing area live in the idle ring");

    extern __shared__ uint8_t smemRaw[];
    __shared__ __align__(8) uint64_t barFull[STAGES];
    __shared__ __align__(8) uint64_t barEmpty[STAGES];
    __shared__ __align__(8) uint64_t barTFull;
    __shared__ __align__(8) uint64_t barRecv[4];        /* per epilogue warp: the pieces have landed */
    __shared__ __align__(8) uint64_t barOldC[8];
    __shared__ uint32_t tmemBaseSlot;
    __shared__ int abortFlag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ClusterCtaRank();
    const int pairIdx = blockIdx.x >> 1;
    const int t = pairIdx / S;                          /* the tile this pair works on */
    const uint32_t q = (uint32_t)(pairIdx - t * S);     /* its part of K, and the column slice it finishes */
    const uint32_t smemBase = (SmemAddr(smemRaw) + 1023u) & ~1023u;
    const uint32_t recvBase = smemBase + EPI_BYTES;
    volatile int * abortPtr = &abortFlag;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (threadIdx.x == 128 || threadIdx.x == 160) {
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
        if (lane < NSTG) {
            MbarInit(SmemAddr(&barFull[lane]), 1);
            MbarInit(SmemAddr(&barEmpty[lane]), 1);
        }
        else if (lane == 8) {
            MbarInit(SmemAddr(&barTFull), 1);
        }
        else if (lane >= 10 && lane < 14) {
            MbarInit(SmemAddr(&barRecv[lane - 10]), 1);
        }
        else if (OLDC && lane >= 16 && lane < 24) {
            MbarInit(SmemAddr(&barOldC[lane - 16]), 1);
        }
        if (lane == 0)
            abortFlag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(SmemAddr(&tmemBaseSlot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    TcFenceBefore();
    ClusterSync();              /* barriers of both CTAs are initialised before any remote signal */
    TcFenceAfter();
    const uint32_t tmemBase = *(volatile uint32_t *)&tmemBaseSlot;

    const int kBlocks = (p.K + EPR - 1) / EPR;
    const int kbLo = (int)((long long)kBlocks * q / S), kbHi = (int)((long long)kBlocks * (q + 1) / S);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const TileCoord tc = DecodeTile(t, p);

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            const int m0 = tc.mBlk * PM + (int)rank * BM;
            const int n0 = tc.nBlk * BN + (int)rank * BNH;
            const int ba = BatchCoord(p.aSel, tc.prob, p);
            const int bb = BatchCoord(p.bSel, tc.prob, p);
            const bool aMN = p.aMN != 0, bMN = p.bMN != 0;
            for (int kb = kbLo; kb < kbHi; kb += G) {
                if (!MbarWait(SmemAddr(&barEmpty[s]), ph ^ 1u, abortPtr, p.status))
                    break;
                const uint32_t fullLeader = MapToCta(SmemAddr(&barFull[s]), 0);
                const int nb = kbHi - kb < G ? kbHi - kb : G;
                if (rank == 0)
                    MbarExpectTx(SmemAddr(&barFull[s]), (uint32_t)nb * 2u * STAGE_BYTES);
#pragma unroll
                for (int j = 0; j < G; j++) {
                    if (j < nb) {
                        const uint32_t aDst = smemBase + (uint32_t)(s * G + j) * STAGE_BYTES;
                        const uint32_t bDst = aDst + A_TILE_BYTES;
                        const int k0 = (kb + j) * EPR;
                        if (!aMN) {
                            TmaLoad3DPair(aDst, &tmA, fullLeader, k0, m0, ba);
                        }
                        else {
#pragma unroll
                            for (int i = 0; i < BM / EPR; i++)
                                TmaLoad3DPair(aDst + i * EPR * ROW_BYTES, &tmA, fullLeader, m0 + i * EPR, k0, ba);
                        }
                        if (!bMN) {
                            TmaLoad3DPair(bDst, &tmB, fullLeader, k0, n0, bb);
                        }
                        else {
#pragma unroll
                            for (int i = 0; i < BNH / EPR; i++)
                                TmaLoad3DPair(bDst + i * EPR * ROW_BYTES, &tmB, fullLeader, n0 + i * EPR, k0, bb);
                        }
                    }
                }
                if (++s == NSTG) { s = 0; ph ^= 1u; }
            }
        }
    }
    else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t iDesc = (1u << 4) | ((uint32_t)(p.aMN ? 1 : 0) << 15) | ((uint32_t)(p.bMN ? 1 : 0) << 16)
                                 | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            const uint32_t aLbo = p.aMN ? EPR * ROW_BYTES : 16, bLbo = p.bMN ? EPR * ROW_BYTES : 16;
            const uint32_t mnStep = (UMMA_K_BYTES / ES) * ROW_BYTES;
            const uint32_t aStep4 = (p.aMN ? mnStep : UMMA_K_BYTES) >> 4, bStep4 = (p.bMN ? mnStep : UMMA_K_BYTES) >> 4;
            const uint64_t aD0 = SmemDesc(smemBase, aLbo, 1024, 2);
            const uint64_t bD0 = SmemDesc(smemBase + A_TILE_BYTES, bLbo, 1024, 2);
            const uint32_t aLo0 = (uint32_t)aD0, aHiW = (uint32_t)(aD0 >> 32);
            const uint32_t bLo0 = (uint32_t)bD0, bHiW = (uint32_t)(bD0 >> 32);
            int s = 0;
            uint32_t ph = 0, acc = 0u;
            bool ok = true;
            for (int kb = kbLo; kb < kbHi; kb += G) {
                ok = MbarWait(SmemAddr(&barFull[s]), ph, abortPtr, p.status);
                if (!ok)
                    break;
                TcFenceAfter();
                const int nb = kbHi - kb < G ? kbHi - kb : G;
#pragma unroll
                for (int j = 0; j < G; j++) {
                    if (j < nb) {
                        uint32_t aLo = aLo0 + (uint32_t)(s * G + j) * (STAGE_BYTES >> 4);
                        uint32_t bLo = bLo0 + (uint32_t)(s * G + j) * (STAGE_BYTES >> 4);
#pragma unroll
                        for (int k = 0; k < KSTEPS; k++) {
                            TcMmaPairLH(tmemBase, aLo, aHiW, bLo, bHiW, iDesc, acc);
                            acc = 1u;
                            aLo += aStep4;
                            bLo += bStep4;
                        }
                    }
                }
                TcCommitPair(SmemAddr(&barEmpty[s]));
                if (++s == NSTG) { s = 0; ph ^= 1u; }
            }
            if (ok)
                TcCommitPair(SmemAddr(&barTFull));
        }
    }
    else {
        const int sub = warp & 3;                 /* TMEM sub-partition (lanes 32 * sub ..) this warp may read */
        const int row0 = tc.mBlk * PM + (int)rank * BM + sub * 32, row = row0 + lane;
        const int n0 = tc.nBlk * BN;
        int pp, qq;
        SplitProb(p, tc.prob, pp, qq);
        const int bc = BatchCoord(p.cSel, tc.prob, p);
        OutT * cRow = (OutT *)p.c + pp * p.sCp + qq * p.sCq + (long long)row * p.ldc;
        const bool rowOk = row < p.M;
        TileWriter<OutT, OLDC> writer;
        writer.Init(smemBase, sub, &tmC, &barOldC[sub * 2], abortPtr, p.status);
        bool ok = MbarWaitWarp(SmemAddr(&barTFull), 0u, abortPtr, p.status, (uint32_t)p.epiHint);
        if (ok) {
            TcFenceAfter();
            /* the ring is idle from here on: old C values may land in its first boxes */
            writer.BeginTile(p, cRow + n0 + (int)q * W, row0, 0, 1, n0 + (int)q * W, W, bc, lane);
            const uint32_t tRow = tmemBase + ((uint32_t)(sub * 32) << 16);
            /* this warp's rows of the other pairs' column slices go to the workspace. A piece is
               addressed by (tile, owner, sender's position among the owner's senders, CTA, warp) */
#pragma unroll
            for (int dd = 1; dd < S; dd++) {
                const uint32_t d = (q + dd) % S;
                const uint32_t slot = q < d ? q : q - 1;
                float4 * dst = (float4 *)p.psWork
                             + ((((size_t)(t * S + (int)d) * (S - 1) + slot) * 2 + rank) * 4 + sub) * PIECE_V4 + lane;
#pragma unroll
                for (int cc = 0; cc < W / 32; cc++) {
                    float v[32];
                    TmemLoad32(tRow + d * W + cc * 32, v);
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        __stcg(dst + (cc * 8 + j) * 32, make_float4(v[j * 4], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]));
                }
            }
            __threadfence();
            __syncwarp();
            if (lane == 0) {
#pragma unroll
                for (int dd = 1; dd < S; dd++) {
                    int * ctr = p.psFlags + ((t * S + (int)((q + dd) % S)) * 2 + (int)rank) * 4 + sub;
                    asm volatile("red.release.gpu.global.add.s32 [%0], %1;" :: "l"(ctr), "r"(1) : "memory");
                }
            }
            /* this pair's slice: wait for the S - 1 pieces of these rows, pull them in */
            int * myCtr = p.psFlags + ((t * S + (int)q) * 2 + (int)rank) * 4 + sub;
            ok = CounterWaitWarp(myCtr, S - 1, abortPtr, p.status);
            if (ok) {
                if (lane == 0) {
                    *myCtr = 0;                     /* every sender has arrived: clear for the next launch */
                    asm volatile("fence.proxy.async;" ::: "memory");
                    const uint32_t bar = SmemAddr(&barRecv[sub]);
                    MbarExpectTx(bar, (uint32_t)(S - 1) * PIECE_BYTES);
#pragma unroll
                    for (int sl = 0; sl < S - 1; sl++) {
                        const float4 * src = (const float4 *)p.psWork
                                           + ((((size_t)(t * S + (int)q) * (S - 1) + sl) * 2 + rank) * 4 + sub) * PIECE_V4;
                        BulkLoad(recvBase + (uint32_t)(sub * (S - 1) + sl) * PIECE_BYTES, src, PIECE_BYTES, bar);
                    }
                }
                ok = MbarWaitWarp(SmemAddr(&barRecv[sub]), 0u, abortPtr, p.status, 0u);
            }
        }
        if (ok) {
#pragma unroll
            for (int cc = 0; cc < W / 32; cc++) {
                float v[32];
                TmemLoad32(tmemBase + ((uint32_t)(sub * 32) << 16) + q * W + cc * 32, v);
#pragma unroll
                for (int sl = 0; sl < S - 1; sl++) {
                    const uint32_t src = recvBase + (uint32_t)(sub * (S - 1) + sl) * PIECE_BYTES + (uint32_t)lane * 16u;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        float4 r;
                        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                     : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "r"(src + (uint32_t)((cc * 8 + j) * 32) * 16u) : "memory");
                        v[j * 4] += r.x; v[j * 4 + 1] += r.y; v[j * 4 + 2] += r.z; v[j * 4 + 3] += r.w;
                    }
                }
                const int c0 = n0 + (int)q * W + cc * 32;
                if (c0 < p.N)
                    writer.Put32(p, cRow, rowOk, row0, c0, bc, v, lane);
            }
        }
        TcFenceBefore();
        writer.Finish(lane);
    }

    __syncwarp();
    if (*abortPtr) {
        /* give copies and MMAs in flight time to land before shared memory and TMEM go away */
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
    }
    TcFenceBefore();
    ClusterSync();              /* neither CTA's shared memory or TMEM goes away while the other may still use it */
    TcFenceAfter();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;"
                     :: "r"(tmemBase), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

template <int S, int STAGES, int G, typename OutT, bool OLDC>
int LaunchPairSplit(const CUtensorMap & tmA, const CUtensorMap & tmB, const CUtensorMap & tmC, const TcParams & tp, cudaStream_t stream)
{
    constexpr int smem = (A_TILE_BYTES + 128 * ROW_BYTES) * STAGES + 1024;
    auto kern = GemmTcPairSplitKernel<S, STAGES, G, OutT, OLDC>;
    static SmemOptIn optIn;
    if (!optIn.Ensure((const void *)kern, smem))
        return NTB_ERR_CUDA;
    const cudaError_t err = LaunchPdl(kern, 2 * S * tp.totalTiles, 192, smem, stream, tmA, tmB, tmC, tp);
    CountLaunch();
    return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? NTB_OK : NTB_ERR_CUDA;
}

}

/* tp and maps as for the CTA-pair kernel with a 256 x 256 tile (one 128-row sub-tile per CTA);
   tp.psWork / tp.psFlags: workspace of PairSplitWorkBytes / cleared counters of PairSplitFlagBytes */
int LaunchPairSplitKernel(int split, int g, bool half, bool oldc, const CUtensorMap * maps, const TcParams & tp, cudaStream_t stream)
{
    if (tp.totalTiles <= 0 || tp.totalTiles > (1 << 20))
        return NTB_ERR_LIMIT;
#define NTB_PSPLIT(SS, ST, T) (g == 1 ? (oldc ? LaunchPairSplit<SS, ST, 1, T, true>(maps[0], maps[1], maps[2], tp, stream)   \
                                             : LaunchPairSplit<SS, ST, 1, T, false>(maps[0], maps[1], maps[2], tp, stream)) \
                                     : (oldc ? LaunchPairSplit<SS, ST, 2, T, true>(maps[0], maps[1], maps[2], tp, stream)   \
                                             : LaunchPairSplit<SS, ST, 2, T, false>(maps[0], maps[1], maps[2], tp, stream)))
    if (!tp.psWork || !tp.psFlags)
        return NTB_ERR_ARG;
    if (split == 2)
        return half ? NTB_PSPLIT(2, 6, __half) : NTB_PSPLIT(2, 6, float);
    return half ? NTB_PSPLIT(4, 6, __half) : NTB_PSPLIT(4, 6, float);
#undef NTB_PSPLIT
}

}
