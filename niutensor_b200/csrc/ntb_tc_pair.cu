/*
 * The CTA-pair tensor-core kernel (tcgen05 cta_group::2) and its launcher.
 */
#include "ntb_tc_common.cuh"

namespace ntb {

namespace {

/*
 * fp16 GEMM on pairs of CTAs (a cluster of two SMs, tcgen05 cta_group::2). A pair owns a
 * (256 * MSUB) x BN output tile, BN = 256 or 128. CTA r of the pair loads, per k-block, MSUB
 * sub-tiles of 128 rows of A (rows j*256 + r*128.. of the tile) and columns r*BN/2.. of the
 * B tile into its own shared memory; the leader (rank 0) issues, per k-step, MSUB
 * 256 x BN x 16 MMAs that read both CTAs' shared memory, and each CTA's TMEM receives its
 * 128 rows of each accumulator. Every CTA fetches half as much of B per flop as a lone CTA
 * with the same accumulator, and with MSUB = 2 half as much again: the rate at which
 * operand tiles reach the SMs, not the tensor pipe, bounds the smaller tiles. The narrow
 * tile gives mid-size products (a few hundred 128 x 128 blocks of output) twice as many
 * CTAs at three quarters of the single-CTA kernel's traffic.
 *
 * MSUB = 1 keeps two accumulator sets, so the epilogue of a tile overlaps the main loop of
 * the next; MSUB = 2 with BN = 256 fills all 512 TMEM columns with one tile and the
 * epilogue runs between main loops while the producer already refills the pipeline.
 * G k-blocks share a barrier hand-shake as in the single-CTA kernel.
 *
 * Barriers: full[s] lives in the leader and counts the bytes of both CTAs' loads;
 * empty[s] and tfull[buf] exist in both CTAs and are signalled together by the leader's
 * tcgen05.commit; tempty[buf] lives in the leader and collects the eight epilogue warps
 * of the pair. All waits are local and bounded as in the single-CTA kernel.
 */
template <int MSUB, int BN, int STAGES, int G, int EPIW, typename OutT, bool OLDC>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(64 + 32 * EPIW, 1)
GemmTcPairKernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ PeerMaps peerMaps, TcParams p)
{
    constexpr int ES = 2;
    constexpr int EPR = ROW_BYTES / ES;                 /* 64 halves of K per stage */
    constexpr int NSTG = STAGES / G;                    /* barrier pairs: G k-blocks share a hand-shake */
    static_assert(STAGES % G == 0 && (BN == 256 || BN == 128), "pair tile");
    constexpr int BNH = BN / 2;                         /* columns of B this CTA loads */
    constexpr int PM = 2 * BM * MSUB;                   /* rows of the pair's tile */
    constexpr int NBUF = 2 / MSUB;                      /* accumulator sets that fit in TMEM */
    constexpr int B_TILE_BYTES = BNH * ROW_BYTES;
    constexpr int STAGE_BYTES = MSUB * A_TILE_BYTES + B_TILE_BYTES;
    constexpr int TMEM_COLS = 512;
    constexpr int KSTEPS = ROW_BYTES / UMMA_K_BYTES;
    static_assert(MSUB == 1 || MSUB == 2, "one or two A sub-tiles per CTA");
    /* EPIW epilogue warps: 4, or 8 -- two per TMEM sub-partition, each taking half of the
       tile's 64-column chunks, which halves the time the accumulators of a tile that fills
       tensor memory (no second set to overlap with) stay occupied after its last MMA. Eight
       warps share the staging space of four: one box each instead of two. */
    static_assert(EPIW == 4 || EPIW == 8, "epilogue warps");
    constexpr int NBOX = EPIW == 4 ? 2 : 1;
    constexpr int CH_PER_SUB = BN / 64;
    constexpr int CH_PER_WARP = MSUB * CH_PER_SUB / (EPIW / 4);
    static_assert(CH_PER_WARP >= 1, "chunks per epilogue warp");

    extern __shared__ uint8_t smemRaw[];
    __shared__ __align__(8) uint64_t barFull[STAGES];
    __shared__ __align__(8) uint64_t barEmpty[STAGES];
    __shared__ __align__(8) uint64_t barTFull[2];
    __shared__ __align__(8) uint64_t barTEmpty[2];
    __shared__ __align__(8) uint64_t barOldC[2 * EPIW];    /* per epilogue warp and staging box: old C values have landed */
    __shared__ uint32_t tmemBaseSlot;
    __shared__ int abortFlag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ClusterCtaRank();
    const uint32_t smemBase = (SmemAddr(smemRaw) + 1023u) & ~1023u;
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
            MbarInit(SmemAddr(&barTEmpty[lane - 8]), 2 * EPIW);
        }
        else if (OLDC && lane >= 16 && lane < 16 + 2 * EPIW) {
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

#ifdef NTB_WAIT_STATS
    long long wstat[4] = {0, 0, 0, 0};
    const long long kernelT0 = clock64();
#endif
    const int kBlocks = (p.K + EPR - 1) / EPR;
    /* set-up is done; nothing before this point touched global memory. A kernel launched
       with programmatic serialisation waits here for the kernels before it in the stream. */
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int firstTile = blockIdx.x >> 1;
    const int tileStep = gridDim.x >> 1;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = firstTile; ok && t < p.totalTiles; t += tileStep) {
                TileCoord tc = DecodeTile(t, p);
                const int m0 = tc.mBlk * PM + (int)rank * BM;
                const int n0 = tc.nBlk * BN + (int)rank * BNH;
                const int ba = BatchCoord(p.aSel, tc.prob, p);
                const int bb = BatchCoord(p.bSel, tc.prob, p);
                const bool aMN = p.aMN != 0, bMN = p.bMN != 0;
                int * const status = p.status;
                const int hint = p.l2Hint;
                const int skipKb = t == firstTile ? p.skipKBlock : -1;    /* test hook, -1 in normal use */
                const uint64_t polA = L2Policy(hint & 3), polB = L2Policy((hint >> 2) & 3);
                for (int kb = 0; kb < kBlocks; kb += G) {
                    NTB_TIMED(0, ok = MbarWait(SmemAddr(&barEmpty[s]), ph ^ 1u, abortPtr, status));
                    if (!ok)
                        break;
                    const uint32_t fullLeader = MapToCta(SmemAddr(&barFull[s]), 0);
                    const int nb = G == 1 ? 1 : (kBlocks - kb < G ? kBlocks - kb : G);
                    if (rank == 0)
                        MbarExpectTx(SmemAddr(&barFull[s]), (uint32_t)nb * 2u * STAGE_BYTES);
#pragma unroll
                    for (int j = 0; j < G; j++) {
                        if (j < nb && kb + j != skipKb) {
                            const uint32_t aDst = smemBase + (uint32_t)(s * G + j) * STAGE_BYTES;
                            const uint32_t bDst = aDst + MSUB * A_TILE_BYTES;
                            const int k0 = (kb + j) * EPR;
#pragma unroll
                            for (int sub = 0; sub < MSUB; sub++) {
                                const int ms = m0 + sub * 2 * BM;
                                const uint32_t dst = aDst + sub * A_TILE_BYTES;
                                if (!aMN) {
                                    if (hint & 3)
                                        TmaLoad3DPairHint(dst, &tmA, fullLeader, k0, ms, ba, polA);
                                    else
                                        TmaLoad3DPair(dst, &tmA, fullLeader, k0, ms, ba);
                                }
                                else {
#pragma unroll
                                    for (int i = 0; i < BM / EPR; i++)
                                        TmaLoad3DPair(dst + i * EPR * ROW_BYTES, &tmA, fullLeader, ms + i * EPR, k0, ba);
                                }
                            }
                            if (!bMN) {
                                if (hint >> 2)
                                    TmaLoad3DPairHint(bDst, &tmB, fullLeader, k0, n0, bb, polB);
                                else
                                    TmaLoad3DPair(bDst, &tmB, fullLeader, k0, n0, bb);
                            }
                            else {
#pragma unroll
                                for (int i = 0; i < BNH / EPR; i++) {
                                    if (hint >> 2)
                                        TmaLoad3DPairHint(bDst + i * EPR * ROW_BYTES, &tmB, fullLeader, n0 + i * EPR, k0, bb, polB);
                                    else
                                        TmaLoad3DPair(bDst + i * EPR * ROW_BYTES, &tmB, fullLeader, n0 + i * EPR, k0, bb);
                                }
                            }
                        }
                    }
                    if (++s == NSTG) { s = 0; ph ^= 1u; }
                }
            }
        }
    }
    else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t iDesc = (1u << 4) | ((uint32_t)(p.aMN ? 1 : 0) << 15) | ((uint32_t)(p.bMN ? 1 : 0) << 16)
                                 | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            const uint32_t aLbo = p.aMN ? EPR * ROW_BYTES : 16, bLbo = p.bMN ? EPR * ROW_BYTES : 16;
            const uint32_t mnStep = (UMMA_K_BYTES / ES) * ROW_BYTES;
            const uint32_t aStep = p.aMN ? mnStep : UMMA_K_BYTES;
            const uint32_t bStep = p.bMN ? mnStep : UMMA_K_BYTES;
            int s = 0;
            uint32_t ph = 0;
            uint32_t it = 0;
            bool ok = true;
            int * const status = p.status;
            /* descriptors of slot 0, k-step 0; in the loop only the start-address field moves */
            const uint64_t aD0 = SmemDesc(smemBase, aLbo, 1024, 2);
            const uint64_t bD0 = SmemDesc(smemBase + MSUB * A_TILE_BYTES, bLbo, 1024, 2);
            const uint32_t aLo0 = (uint32_t)aD0, aHiW = (uint32_t)(aD0 >> 32);
            const uint32_t bLo0 = (uint32_t)bD0, bHiW = (uint32_t)(bD0 >> 32);
            const uint32_t aStep4 = aStep >> 4, bStep4 = bStep >> 4;
            const uint32_t barFull0 = SmemAddr(&barFull[0]), barEmpty0 = SmemAddr(&barEmpty[0]);
            uint32_t stageOff = 0;                /* s * G * STAGE_BYTES in 16-byte units */
            for (int t = firstTile; ok && t < p.totalTiles; t += tileStep, ++it) {
                const uint32_t buf = it % NBUF;
                NTB_TIMED(2, ok = MbarWait(SmemAddr(&barTEmpty[buf]), ((it / NBUF) & 1u) ^ 1u, abortPtr, status));
                if (!ok)
                    break;
                TcFenceAfter();
                const uint32_t dTmem = tmemBase + buf * (MSUB * BN);
                uint32_t acc = 0u;
                for (int kb = 0; kb < kBlocks; kb += G) {
                    NTB_TIMED(1, ok = MbarWait(barFull0 + (uint32_t)s * 8u, ph, abortPtr, status));
                    if (!ok)
                        break;
                    TcFenceAfter();
                    const int nb = G == 1 ? 1 : (kBlocks - kb < G ? kBlocks - kb : G);
#pragma unroll
                    for (int j = 0; j < G; j++) {
                        if (j < nb) {
                            uint32_t aLo = aLo0 + stageOff + (uint32_t)j * (STAGE_BYTES >> 4);
                            uint32_t bLo = bLo0 + stageOff + (uint32_t)j * (STAGE_BYTES >> 4);
#pragma unroll
                            for (int k = 0; k < KSTEPS; k++) {
#pragma unroll
                                for (int sub = 0; sub < MSUB; sub++)
                                    TcMmaPairLH(dTmem + sub * BN, aLo + (uint32_t)sub * (A_TILE_BYTES >> 4), aHiW, bLo, bHiW, iDesc, acc);
                                acc = 1u;
                                aLo += aStep4;
                                bLo += bStep4;
                            }
                        }
                    }
                    TcCommitPair(barEmpty0 + (uint32_t)s * 8u);
                    stageOff += (uint32_t)G * (STAGE_BYTES >> 4);
                    if (++s == NSTG) { s = 0; ph ^= 1u; stageOff = 0; }
                }
                if (ok)
                    TcCommitPair(SmemAddr(&barTFull[buf]));
            }
        }
    }
    else {
        const int sub32 = warp & 3;               /* TMEM sub-partition (lanes 32 * sub32 ..) this warp may read */
        const int ew = warp - 2;                  /* 0 .. EPIW-1 */
        const int chBeg = (ew >> 2) * CH_PER_WARP;    /* first of this warp's chunks, counted sub-tile by sub-tile */
        uint32_t it = 0;
        bool ok = true;
        TileWriter<OutT, OLDC, NBOX> writer;
        writer.Init(smemBase + STAGES * STAGE_BYTES, ew, &tmC, &barOldC[ew * 2], abortPtr, p.status);
        if (OLDC && p.nPeers > 0 && p.peerTma)
            writer.peerMaps = peerMaps.m;
        for (int t = firstTile; ok && t < p.totalTiles; t += tileStep, ++it) {
            TileCoord tc = DecodeTile(t, p);
            const int n0 = tc.nBlk * BN;
            int pp, qq;
            SplitProb(p, tc.prob, pp, qq);
            const int bc = BatchCoord(p.cSel, tc.prob, p);
            OutT * cBase = (OutT *)p.c + pp * p.sCp + qq * p.sCq;
            const uint32_t buf = it % NBUF;
            const int tileRow0 = tc.mBlk * PM + (int)rank * BM + sub32 * 32;   /* this warp's rows of sub-tile 0 */
            {
                /* this warp's part of the tile: sub-tiles firstSub .. lastSub, columns from colBeg */
                const int firstSub = chBeg / CH_PER_SUB, lastSub = (chBeg + CH_PER_WARP - 1) / CH_PER_SUB;
                const int colBeg = n0 + (chBeg % CH_PER_SUB) * 64;
                const int cols = CH_PER_WARP >= CH_PER_SUB ? BN : CH_PER_WARP * 64;
                const int r0 = tileRow0 + firstSub * 2 * BM;
                writer.BeginTile(p, cBase + (long long)(r0 + lane) * p.ldc + colBeg, r0, 2 * BM, lastSub - firstSub + 1,
                                 colBeg, cols, bc, lane);
                writer.OldRequest(p, cBase + (long long)(r0 + lane) * p.ldc, colBeg, r0 + lane < p.M);
            }
            NTB_TIMED(3, ok = MbarWaitWarp(SmemAddr(&barTFull[buf]), (it / NBUF) & 1u, abortPtr, p.status, (uint32_t)p.epiHint));
            if (!ok)
                break;
            TcFenceAfter();
#pragma unroll 1
            for (int i = 0; i < CH_PER_WARP; i++) {
                const int idx = chBeg + i;
                const int sub = idx / CH_PER_SUB, ch = idx % CH_PER_SUB;
                const int row0 = tileRow0 + sub * 2 * BM;
                const int row = row0 + lane;
                OutT * cRow = cBase + (long long)row * p.ldc;
                const bool rowOk = row < p.M;
                const int c0 = n0 + ch * 64;
                if (c0 >= p.N)
                    continue;                      /* uniform across the warp */
                writer.OldAdvance();
                if (i + 1 < CH_PER_WARP) {
                    /* old values of the chunk after this one: further right, or the next sub-tile's first */
                    if (ch + 1 < CH_PER_SUB) {
                        if (c0 + 64 < p.N)
                            writer.OldRequest(p, cRow, c0 + 64, rowOk);
                    }
                    else {
                        writer.OldRequest(p, cRow + (long long)(2 * BM) * p.ldc, n0, row + 2 * BM < p.M);
                    }
                }
                const uint32_t tRow = tmemBase + ((uint32_t)(sub32 * 32) << 16) + buf * (MSUB * BN) + sub * BN;
                float v[64];
                TmemLoad64(tRow + ch * 64, v);
                writer.Put32(p, cRow, rowOk, row0, c0, bc, v, lane);
                if (c0 + 32 < p.N)
                    writer.Put32(p, cRow, rowOk, row0, c0 + 32, bc, v + 32, lane);
            }
            TcFenceBefore();
            __syncwarp();
            if (lane == 0)
                MbarArriveCluster(MapToCta(SmemAddr(&barTEmpty[buf]), 0));
        }
        writer.Finish(lane);
    }

#ifdef NTB_WAIT_STATS
    if (lane == 0 && (warp <= 2)) {
        if (warp == 0) { atomicAdd(&gWaitStats[0], (unsigned long long)wstat[0]); atomicAdd(&gWaitStats[5], 1ULL);
                         if (blockIdx.x == 0) atomicAdd(&gWaitStats[4], (unsigned long long)(clock64() - kernelT0)); }
        if (warp == 1) { atomicAdd(&gWaitStats[1], (unsigned long long)wstat[1]); atomicAdd(&gWaitStats[2], (unsigned long long)wstat[2]); }
        if (warp == 2) atomicAdd(&gWaitStats[3], (unsigned long long)wstat[3]);
    }
#endif
    __syncwarp();
    if (*abortPtr) {
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

template <int MSUB, int BN, int STAGES, int G, int EPIW, typename OutT, bool OLDC>
int LaunchPair(const CUtensorMap & tmA, const CUtensorMap & tmB, const CUtensorMap & tmC, const PeerMaps & pm, const TcParams & tp,
               int pairs, cudaStream_t stream)
{
    constexpr int smem = (MSUB * A_TILE_BYTES + (BN / 2) * ROW_BYTES) * STAGES + EPI_BYTES + 1024;
    auto kern = GemmTcPairKernel<MSUB, BN, STAGES, G, EPIW, OutT, OLDC>;
    static SmemOptIn optIn;
    if (!optIn.Ensure((const void *)kern, smem))
        return NTB_ERR_CUDA;
    const cudaError_t err = LaunchPdl(kern, 2 * pairs, 64 + 32 * EPIW, smem, stream, tmA, tmB, tmC, pm, tp);
    CountLaunch();
    return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? NTB_OK : NTB_ERR_CUDA;
}

}

int LaunchPairKernel(int msub, int bn, int g, int epiWarps, bool half, bool oldc, const CUtensorMap * maps, const TcParams & tp,
                     const PeerMaps * peerMaps, int pairs, cudaStream_t stream)
{
    static const PeerMaps noPeers = {};
    const PeerMaps & pm = peerMaps ? *peerMaps : noPeers;
#define NTB_PAIR2(MS, W, ST, GG, EW, T) (oldc ? LaunchPair<MS, W, ST, GG, EW, T, true>(maps[0], maps[1], maps[2], pm, tp, pairs, stream) \
                                              : LaunchPair<MS, W, ST, GG, EW, T, false>(maps[0], maps[1], maps[2], pm, tp, pairs, stream))
#define NTB_PAIR(MS, W, ST, GG, EW) (half ? NTB_PAIR2(MS, W, ST, GG, EW, __half) : NTB_PAIR2(MS, W, ST, GG, EW, float))
    if (bn == 256) {
        if (msub == 2)
            return epiWarps == 4 ? NTB_PAIR(2, 256, 4, 1, 4) : NTB_PAIR(2, 256, 4, 1, 8);
        return NTB_PAIR(1, 256, 6, 1, 4);
    }
    if (msub == 2)
        return NTB_PAIR(2, 128, 4, 2, 4);
    return g == 4 ? NTB_PAIR(1, 128, 8, 4, 4) : NTB_PAIR(1, 128, 8, 2, 4);
#undef NTB_PAIR2
#undef NTB_PAIR
}

#ifdef NTB_WAIT_STATS
extern "C" void ntb_debug_wait_stats(unsigned long long * out)
{
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, gWaitStats, sizeof(unsigned long long) * 8);
    unsigned long long zero[8] = {0};
    cudaMemcpyToSymbol(gWaitStats, zero, sizeof(zero));
}
#endif

}
