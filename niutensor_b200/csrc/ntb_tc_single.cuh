/*
 * The single-CTA tensor-core kernel (tcgen05 cta_group::1) as a template, with its launcher:
 * instantiated for operands that TMA brings in (ntb_tc.cu) and for operands that loader warps
 * fetch with ordinary loads because TMA cannot address them (ntb_tc_ldg.cu).
 */
#ifndef NTB_TC_SINGLE_CUH
#define NTB_TC_SINGLE_CUH

#include "ntb_tc_common.cuh"

namespace ntb {

/* Several problems of different shapes in one launch: tiles [first[i], first[i + 1]) belong to
   problem i. NP = 2 serves the two gradient products of a matrix multiplication (and every
   single product); NP = GROUP_MAX the grouped entry point for lists of unequal shapes. The
   whole group travels as kernel parameters, so NP is kept small where it is not needed. */
constexpr int GROUP_MAX = 8;
template <int NP>
struct TcGroupT {
    CUtensorMap tm[NP][3];     /* A, B, C maps of each problem */
    TcParams p[NP];
    int n, total;
    int first[NP + 1];
};
typedef TcGroupT<2> TcGroup;
typedef TcGroupT<GROUP_MAX> TcGroupWide;

/* launcher of the kernels whose operands are fetched by loader warps (ntb_tc_ldg.cu) */
int LaunchLdgKernel(const TcGroup & grp, int mode, int dtC, bool oldc, int smCount, cudaStream_t stream);
/* launcher of the kernels that walk up to GROUP_MAX problems of unequal shapes (ntb_grouped.cu) */
int LaunchWideGroup(const TcGroupWide & grp, int mode, int dtC, bool oldc, int smCount, cudaStream_t stream);
/* kernel parameters and tensor maps of one problem for the single-CTA kernel with tiles bn wide (ntb_tc.cu) */
int PrepareSingle(const DeviceCtx & ctx, const Problem & p, int bn, TcParams & tp, CUtensorMap * maps);

namespace {

/* ---------------------------------------------------------------- the kernel */

/* per-tile view of the problem a tile belongs to; names match the single-problem code */
#define NTB_SELECT_PROBLEM() \
    int gi = 0; \
    _Pragma("unroll") \
    for (int k_ = 1; k_ < NP; k_++) \
        gi += (k_ < grp.n && t >= grp.first[k_]) ? 1 : 0; \
    const TcParams & p = grp.p[gi]; \
    const CUtensorMap & tmA = grp.tm[gi][0]; \
    const CUtensorMap & tmB = grp.tm[gi][1]; \
    const CUtensorMap & tmC = grp.tm[gi][2]; \
    (void)tmA; (void)tmB; (void)tmC; \
    const int tl = t - grp.first[gi]; \
    const int kBlocks = (p.K + EPR - 1) / EPR; \
    /* k-blocks accumulated in TMEM before the partial sum is handed to the epilogue */ \
    const int chunkBlocks = MODE == 0 ? kBlocks : FP32_CHUNK_BLOCKS; \
    (void)chunkBlocks

/* loader warps of the kernels whose operands TMA cannot address (LDG) */
constexpr int LDG_THREADS = 256;

/*
 * One 16-byte chunk of a 128-byte row segment that starts at the byte address g (aligned to
 * the element size only): the bytes [16 c + s, 16 c + s + 16) of the stream of 16-byte
 * aligned vectors that begins at g rounded down, s = g mod 16. `own` is aligned vector c,
 * `next` vector c + 1; bytes at or beyond `valid` (counted from g) come out as zero.
 */
__device__ __forceinline__ uint4 RealignChunk(uint4 own, uint4 next, uint32_t s, int c, int valid)
{
    const uint32_t x[8] = { own.x, own.y, own.z, own.w, next.x, next.y, next.z, next.w };
    const uint32_t b = (s & 3u) * 8u;
    uint32_t o[4];
    /* word offset 0 .. 3: one branch, then constant register indices (lanes of a warp differ
       only when the row pitch is not a multiple of 16 bytes) */
    switch (s >> 2) {
    case 0:
#pragma unroll
        for (int i = 0; i < 4; i++) o[i] = __funnelshift_r(x[i], x[i + 1], b);
        break;
    case 1:
#pragma unroll
        for (int i = 0; i < 4; i++) o[i] = __funnelshift_r(x[i + 1], x[i + 2], b);
        break;
    case 2:
#pragma unroll
        for (int i = 0; i < 4; i++) o[i] = __funnelshift_r(x[i + 2], x[i + 3], b);
        break;
    default:
#pragma unroll
        for (int i = 0; i < 4; i++) o[i] = __funnelshift_r(x[i + 3], x[(i + 4) & 7], b);
        break;
    }
    if (16 * c + 16 > valid) {
        /* the matrix ends inside (or before) this chunk */
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int left = valid - (16 * c + 4 * i);          /* valid bytes from this word on */
            if (left <= 0)
                o[i] = 0u;
            else if (left < 4)
                o[i] &= (1u << (8 * left)) - 1u;
        }
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

template <int MODE, int BN, int STAGES, int G, typename OutT, bool OLDC, bool LDG = false, int NP = 2>
__global__ void __launch_bounds__((MODE == 0 ? 192 : 192 + CONV_THREADS) + (LDG ? LDG_THREADS : 0), 1)
GemmTcKernel(const __grid_constant__ TcGroupT<NP> grp)
{
    static_assert(!LDG || G == 1, "loader warps fill one k-block per hand-shake");
    /* G k-blocks share one full / empty barrier pair: the producer and the MMA thread each
       pay for a barrier hand-shake (a few hundred clocks of their own time, most of it the
       MMA thread's shared-memory probe waiting behind the tensor-core instructions it has
       just issued) once per G k-blocks instead of once per k-block */
    static_assert(STAGES % G == 0 && (MODE == 0 || G == 1), "k-blocks per hand-shake");
    constexpr int NSTG = STAGES / G;                    /* barrier pairs in the ring */
    constexpr int ES = MODE == 0 ? 2 : 4;               /* operand element size */
    constexpr int EPR = ROW_BYTES / ES;                 /* elements per 128-byte row = K per stage */
    constexpr int B_TILE_BYTES = BN * ROW_BYTES;
    constexpr int PLANE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
    constexpr int STAGE_BYTES = PLANE_BYTES * (MODE == 0 ? 1 : 2);   /* fp32: hi plane + lo plane */
    /* two accumulators, plus (fp32 route) one running sum; a power of two */
    constexpr int TMEM_NEED = (MODE == 0 ? 2 : 3) * BN;
    constexpr int TMEM_COLS = TMEM_NEED <= 128 ? 128 : TMEM_NEED <= 256 ? 256 : 512;
    constexpr int KSTEPS = ROW_BYTES / UMMA_K_BYTES;                 /* 4 */
    static_assert(BN == 64 || BN == 128 || BN == 256, "tile width");
    static_assert(STAGES <= 8, "barrier initialisation assigns lanes 0-7 to the stages");

#ifdef NTB_WAIT_STATS
    const long long kernelT0 = clock64();
    __shared__ unsigned long long tlShared[64];
    if (threadIdx.x < 64) tlShared[threadIdx.x] = 0;
    __syncthreads();
#endif
    extern __shared__ uint8_t smemRaw[];
    __shared__ __align__(8) uint64_t barFull[STAGES];
    __shared__ __align__(8) uint64_t barEmpty[STAGES];
    __shared__ __align__(8) uint64_t barConv[STAGES];
    __shared__ __align__(8) uint64_t barTFull[2];
    __shared__ __align__(8) uint64_t barTEmpty[2];
    __shared__ __align__(8) uint64_t barOldC[8];    /* per epilogue warp and staging box: old C values have landed */
    __shared__ uint32_t tmemBaseSlot;
    __shared__ int abortFlag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t smemBase = (SmemAddr(smemRaw) + 1023u) & ~1023u;
    volatile int * abortPtr = &abortFlag;
    /* a kernel launched behind this one with programmatic serialisation may start setting up */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (threadIdx.x == 128 || threadIdx.x == 160) {
        /* Idle epilogue lanes pull the kernel parameters (and one of them the tensor maps)
           towards the SM while the other warps set up. Warps 4 and 5 share their scheduler
           partition, and with it the first-level constant cache, with the producer warp and
           the MMA warp: a constant load that misses stalls its warp for the whole miss,
           one line after the other, and the producer reads half a dozen lines before its
           first copy. */
        int touch = grp.total + grp.first[1];
        for (int gi = 0; gi < grp.n; gi++) {
            const TcParams & p = grp.p[gi];
            if (threadIdx.x == 128) {
                if (!LDG) {
                    PrefetchTensorMap(&grp.tm[gi][0]);
                    PrefetchTensorMap(&grp.tm[gi][1]);
                }
                if (p.cTma)
                    PrefetchTensorMap(&grp.tm[gi][2]);
            }
            const int * words = (const int *)&p;
            for (int w = 0; w < (int)(sizeof(TcParams) / sizeof(int)); w += 8)
                touch += words[w];
        }
        asm volatile("" :: "r"(touch));
    }
    if (warp == 0) {
        /* one barrier per lane: thirty-odd initialisations one after the other cost the
           producer, which goes first, several hundred clocks */
        if (lane == 0) NTB_MARK(8);
        if (lane < STAGES) {
            MbarInit(SmemAddr(&barFull[lane]), LDG ? LDG_THREADS / 32 : 1);
            MbarInit(SmemAddr(&barEmpty[lane]), 1);
            MbarInit(SmemAddr(&barConv[lane]), CONV_THREADS);
        }
        else if (lane >= 8 && lane < 10) {
            MbarInit(SmemAddr(&barTFull[lane - 8]), 1);
            MbarInit(SmemAddr(&barTEmpty[lane - 8]), 4);
        }
        else if (OLDC && lane >= 16 && lane < 24) {
            MbarInit(SmemAddr(&barOldC[lane - 16]), 1);
        }
        if (lane == 0)
            abortFlag = 0;
        if (lane == 0) NTB_MARK(9);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (lane == 0) NTB_MARK(10);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(SmemAddr(&tmemBaseSlot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        if (lane == 0) NTB_MARK(11);
    }
    /* The producer warp initialised the barriers itself and needs no TMEM: it signals the
       CTA-wide barrier without waiting and starts loading, so the TMEM allocation and the
       hand-shake overlap the first copies. Everybody else waits for both. */
    uint32_t tmemBase = 0;
    if (warp == 0) {
        __syncwarp();
        asm volatile("bar.arrive 1, %0;" :: "r"((uint32_t)blockDim.x) : "memory");
    }
    else {
        TcFenceBefore();
        asm volatile("bar.sync 1, %0;" :: "r"((uint32_t)blockDim.x) : "memory");
        TcFenceAfter();
        tmemBase = *(volatile uint32_t *)&tmemBaseSlot;
    }

#ifdef NTB_WAIT_STATS
    long long wstat[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#endif
    if (threadIdx.x == 0) NTB_MARK(0);
    /* set-up is done; nothing before this point touched global memory. A kernel launched
       with programmatic serialisation waits here for the kernels before it in the stream. */
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int firstTile = blockIdx.x;
    const int tileStep = gridDim.x;

    if (warp == 0) {
        /* ------------------------------------------------------------ TMA producer */
        if (!LDG && lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = firstTile; ok && t < grp.total; t += tileStep) {
                NTB_SELECT_PROBLEM();
                TileCoord tc = DecodeTile(tl, p);
                const int m0 = tc.mBlk * BM, n0 = tc.nBlk * BN;
                const int ba = BatchCoord(p.aSel, tc.prob, p);
                const int bb = BatchCoord(p.bSel, tc.prob, p);
                NTB_MARK(12);
                /* everything the k-loop needs, in registers: the loop itself touches no
                   kernel parameter */
                const bool aMN = p.aMN != 0, bMN = p.bMN != 0;
                const int pfDist = p.pfDist, nkb = kBlocks;
                const int skipKb = t == firstTile ? p.skipKBlock : -1;    /* test hook, -1 in normal use */
                int * const status = p.status;
                const CUtensorMap * const mapA = &tmA;
                const CUtensorMap * const mapB = &tmB;
#ifdef NTB_WAIT_STATS
                const long long loopT0 = clock64();
#endif
                for (int kb = 0; kb < nkb; kb += G) {
                    NTB_TIMED(0, ok = MbarWait(SmemAddr(&barEmpty[s]), ph ^ 1u, abortPtr, status));
                    NTB_MARK(13);
                    if (!ok)
                        break;
                    const uint32_t full = SmemAddr(&barFull[s]);
                    const int nb = G == 1 ? 1 : (nkb - kb < G ? nkb - kb : G);
                    NTB_TIMED(6, MbarExpectTx(full, (uint32_t)nb * PLANE_BYTES));
                    NTB_MARK(14);
#pragma unroll
                    for (int j = 0; j < G; j++) {
                        if (j < nb && kb + j != skipKb) {
                            const uint32_t aDst = smemBase + (uint32_t)(s * G + j) * STAGE_BYTES;
                            const uint32_t bDst = aDst + A_TILE_BYTES;
                            const int k0 = (kb + j) * EPR;
                            if (!aMN) {
                                NTB_TIMED(7, TmaLoad3D(aDst, mapA, full, k0, m0, ba));
                            }
                            else {
#pragma unroll
                                for (int i = 0; i < BM / EPR; i++)
                                    TmaLoad3D(aDst + i * EPR * ROW_BYTES, mapA, full, m0 + i * EPR, k0, ba);
                            }
                            if (!bMN) {
                                NTB_TIMED(5, TmaLoad3D(bDst, mapB, full, k0, n0, bb));
                            }
                            else {
#pragma unroll
                                for (int i = 0; i < BN / EPR; i++)
                                    TmaLoad3D(bDst + i * EPR * ROW_BYTES, mapB, full, n0 + i * EPR, k0, bb);
                            }
                            if (pfDist > 0 && kb + j + pfDist < nkb) {
                                const int kp = k0 + pfDist * EPR;
                                if (!aMN) {
                                    TmaPrefetch3D(mapA, kp, m0, ba);
                                }
                                else {
#pragma unroll
                                    for (int i = 0; i < BM / EPR; i++)
                                        TmaPrefetch3D(mapA, m0 + i * EPR, kp, ba);
                                }
                                if (!bMN) {
                                    TmaPrefetch3D(mapB, kp, n0, bb);
                                }
                                else {
#pragma unroll
                                    for (int i = 0; i < BN / EPR; i++)
                                        TmaPrefetch3D(mapB, n0 + i * EPR, kp, bb);
                                }
                            }
                        }
                    }
                    NTB_MARK(1);
                    NTB_MARKK(0, kb);
                    if (++s == NSTG) { s = 0; ph ^= 1u; }
                }
#ifdef NTB_WAIT_STATS
                wstat[3] += clock64() - loopT0;
#endif
            }
        }
    }
    else if (warp == 1) {
        /* ------------------------------------------------------------ MMA issuer */
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            uint32_t stageOff = 0;                /* s * STAGE_BYTES in 16-byte units */
            uint32_t it = 0;                      /* accumulator hand-overs so far */
            bool ok = true;
            const uint32_t barFull0 = SmemAddr(MODE == 0 ? &barFull[0] : &barConv[0]);
            const uint32_t barEmpty0 = SmemAddr(&barEmpty[0]);
            for (int t = firstTile; ok && t < grp.total; t += tileStep) {
                NTB_SELECT_PROBLEM();
                (void)tl;
                const uint32_t iDesc = InstrDesc(MODE, p.aMN, p.bMN, BN);
                /* K-major: rows of 128 B, 8-row groups 1024 B apart, k-step = 32 B along the row.
                   MN-major: boxes of EPR k-rows x 128 B; 64- (or 32-) element MN chunks are
                   EPR*128 B apart (leading offset), 8-k-row groups 1024 B apart (stride offset),
                   k-step = UMMA_K k-rows. */
                const uint32_t aLbo = p.aMN ? EPR * ROW_BYTES : 16, bLbo = p.bMN ? EPR * ROW_BYTES : 16;
                const uint32_t mnStep = (UMMA_K_BYTES / ES) * ROW_BYTES;
                const uint32_t aStep = p.aMN ? mnStep : UMMA_K_BYTES;
                const uint32_t bStep = p.bMN ? mnStep : UMMA_K_BYTES;
                /* MN-major fp32 tiles are loaded with the 32-byte-chunk swizzle, whose pattern
                   repeats every 4 k-rows (512 B) instead of every 8 */
                const uint32_t aLay = (MODE != 0 && p.aMN) ? 1u : 2u, bLay = (MODE != 0 && p.bMN) ? 1u : 2u;
                const uint32_t aSbo = (MODE != 0 && p.aMN) ? 512u : 1024u, bSbo = (MODE != 0 && p.bMN) ? 512u : 1024u;
                int * const status = p.status;
                const int nkb = kBlocks, chunk = chunkBlocks;
                /* descriptors of stage 0, k-step 0; inside the loop only their start-address
                   field (bits 0-13 of the low word, in 16-byte units) moves */
                const uint64_t aD0 = SmemDesc(smemBase, aLbo, aSbo, aLay);
                const uint64_t bD0 = SmemDesc(smemBase + A_TILE_BYTES, bLbo, bSbo, bLay);
                const uint32_t aLo0 = (uint32_t)aD0, aHiW = (uint32_t)(aD0 >> 32);
                const uint32_t bLo0 = (uint32_t)bD0, bHiW = (uint32_t)(bD0 >> 32);
                const uint32_t aStep4 = aStep >> 4, bStep4 = bStep >> 4;
                for (int kb0 = 0; ok && kb0 < nkb; kb0 += chunk, ++it) {
                    const uint32_t buf = it & 1u;
                    NTB_TIMED(2, ok = MbarWait(SmemAddr(&barTEmpty[buf]), ((it >> 1) & 1u) ^ 1u, abortPtr, status));
                    if (!ok)
                        break;
                    TcFenceAfter();
                    const uint32_t dTmem = tmemBase + buf * BN;
                    const int kbEnd = min(nkb, kb0 + chunk);
                    uint32_t acc = 0u;                /* the first instruction of a chain overwrites */
                    for (int kb = kb0; kb < kbEnd; kb += G) {
                        NTB_TIMED(1, ok = MbarWait(barFull0 + (uint32_t)s * 8u, ph, abortPtr, status));
                        if (!ok)
                            break;
                        NTB_MARK(2);
                        NTB_MARKK(1, kb);
                        TcFenceAfter();
                        if (LDG)    /* the stage was written with ordinary stores: order them before the tensor core's reads */
                            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        const int nb = G == 1 ? 1 : (kbEnd - kb < G ? kbEnd - kb : G);
#pragma unroll
                        for (int j = 0; j < G; j++) {
                            if (j < nb) {
                                uint32_t aLo = aLo0 + stageOff + (uint32_t)j * (STAGE_BYTES >> 4);
                                uint32_t bLo = bLo0 + stageOff + (uint32_t)j * (STAGE_BYTES >> 4);
#pragma unroll
                                for (int k = 0; k < KSTEPS; k++) {
                                    if (MODE == 0) {
                                        TcMmaLH<MODE>(dTmem, aLo, aHiW, bLo, bHiW, iDesc, acc);
                                    }
                                    else {
                                        constexpr uint32_t PLANE4 = PLANE_BYTES >> 4;
                                        TcMmaLH<MODE>(dTmem, aLo + PLANE4, aHiW, bLo, bHiW, iDesc, acc);
                                        TcMmaLH<MODE>(dTmem, aLo, aHiW, bLo + PLANE4, bHiW, iDesc, 1u);
                                        TcMmaLH<MODE>(dTmem, aLo, aHiW, bLo, bHiW, iDesc, 1u);
                                    }
                                    acc = 1u;
                                    aLo += aStep4;
                                    bLo += bStep4;
                                }
                            }
                        }
                        TcCommit(barEmpty0 + (uint32_t)s * 8u);
                        NTB_MARKK(2, kb);
                        stageOff += (uint32_t)G * (STAGE_BYTES >> 4);
                        if (++s == NSTG) { s = 0; ph ^= 1u; stageOff = 0; }
                    }
                    if (ok)
                        TcCommit(SmemAddr(&barTFull[buf]));
                    NTB_MARK(3);
                }
            }
        }
    }
    else if (warp < 6) {
        /* ------------------------------------------------------------ epilogue */
        const int sub = warp & 3;                 /* TMEM sub-partition this warp may read */
        uint32_t it = 0;
        bool ok = true;
        TileWriter<OutT, OLDC> writer;
        writer.Init(smemBase + STAGES * STAGE_BYTES, sub, nullptr, &barOldC[sub * 2], abortPtr, nullptr);
        for (int t = firstTile; ok && t < grp.total; t += tileStep) {
            NTB_SELECT_PROBLEM();
            writer.map = &tmC;
            writer.status = p.status;
            TileCoord tc = DecodeTile(tl, p);
            const int row0 = tc.mBlk * BM + sub * 32;
            const int row = row0 + lane;
            const int n0 = tc.nBlk * BN;
            int pp, qq;
            SplitProb(p, tc.prob, pp, qq);
            const int bc = BatchCoord(p.cSel, tc.prob, p);
            OutT * cRow = (OutT *)p.c + pp * p.sCp + qq * p.sCq + (long long)row * p.ldc;
            const bool rowOk = row < p.M;
            writer.BeginTile(p, cRow + n0, row0, 0, 1, n0, BN, bc, lane);
            if (MODE == 0) {
                writer.OldRequest(p, cRow, n0, rowOk);
                /* one accumulator hand-over per tile: load 32 columns, scale, store */
                const uint32_t buf = it & 1u;
                ok = MbarWaitWarp(SmemAddr(&barTFull[buf]), (it >> 1) & 1u, abortPtr, p.status, (uint32_t)p.epiHint);
                if (!ok)
                    break;
                if (warp == 2 && lane == 0) NTB_MARK(4);
                TcFenceAfter();
                const uint32_t tRow = tmemBase + ((uint32_t)(sub * 32) << 16) + buf * BN;
#pragma unroll 1
                for (int ch = 0; ch < BN / 64; ch++) {
                    const int c0 = n0 + ch * 64;
                    if (c0 >= p.N)
                        break;                     /* uniform across the warp */
                    writer.OldAdvance();
                    if (ch + 1 < BN / 64 && c0 + 64 < p.N)
                        writer.OldRequest(p, cRow, c0 + 64, rowOk);
                    float v[64];
                    TmemLoad64(tRow + ch * 64, v);
                    writer.Put32(p, cRow, rowOk, row0, c0, bc, v, lane);
                    if (c0 + 32 < p.N)
                        writer.Put32(p, cRow, rowOk, row0, c0 + 32, bc, v + 32, lane);
                }
                TcFenceBefore();
                __syncwarp();
                if (lane == 0)
                    MbarArrive(SmemAddr(&barTEmpty[buf]));
                ++it;
            }
            else {
                /* fp32 inputs: the tensor core truncates its fp32 accumulator after every
                   instruction, an error that grows with the length of the accumulation
                   chain. K is therefore cut into chunks of chunkBlocks k-blocks; each
                   chunk's partial sum is handed over here and added, with round-to-nearest
                   FADDs, to a running sum kept in a third TMEM region (the sum of a
                   128-column row does not fit the registers a ten-warp CTA leaves a thread). */
                const uint32_t tRun = tmemBase + ((uint32_t)(sub * 32) << 16) + 2 * BN;   /* running sum */
                for (int kb0 = 0; ok && kb0 < kBlocks; kb0 += chunkBlocks, ++it) {
                    const uint32_t buf = it & 1u;
                    ok = MbarWaitWarp(SmemAddr(&barTFull[buf]), (it >> 1) & 1u, abortPtr, p.status, (uint32_t)p.epiHint);
                    if (!ok)
                        break;
                    TcFenceAfter();
                    const uint32_t tRow = tmemBase + ((uint32_t)(sub * 32) << 16) + buf * BN;
                    const bool first = kb0 == 0, last = kb0 + chunkBlocks >= kBlocks;
#pragma unroll 1
                    for (int ch = 0; ch < BN / 32; ch++) {
                        float v[32];
                        TmemLoad32(tRow + ch * 32, v);
                        if (!first) {
                            float r[32];
                            TmemLoad32(tRun + ch * 32, r);
#pragma unroll
                            for (int e = 0; e < 32; e++)
                                v[e] += r[e];
                        }
                        if (!last) {
                            TmemStore32(tRun + ch * 32, v);
                        }
                        else {
                            const int c0 = n0 + ch * 32;
                            if (c0 < p.N)
                                writer.Put32(p, cRow, rowOk, row0, c0, bc, v, lane);
                        }
                    }
                    TcFenceBefore();
                    __syncwarp();
                    if (lane == 0)
                        MbarArrive(SmemAddr(&barTEmpty[buf]));
                }
            }
        }
        if (warp == 2 && lane == 0) NTB_MARK(5);
        writer.Finish(lane);
        if (warp == 2 && lane == 0) NTB_MARK(6);
    }
    else if (MODE != 0 && warp < 6 + CONV_THREADS / 32) {
        /* ------------------------------------------------------------ fp32 hi/lo split */
        const int ct = threadIdx.x - 192;         /* 0 .. CONV_THREADS-1 */
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int t = firstTile; ok && t < grp.total; t += tileStep) {
            NTB_SELECT_PROBLEM();
            (void)tl;
            for (int kb = 0; kb < kBlocks; kb++) {
                ok = MbarWait(SmemAddr(&barFull[s]), ph, abortPtr, p.status);
                if (!ok)
                    break;
                uint8_t * hi = smemRaw + (smemBase - SmemAddr(smemRaw)) + s * STAGE_BYTES;
                uint8_t * lo = hi + PLANE_BYTES;
#pragma unroll 4
                for (int i = ct; i < PLANE_BYTES / 16; i += CONV_THREADS) {
                    /* The tensor core reads an fp32 word as tf32 by ignoring its 13 low mantissa
                       bits, so the loaded plane already is the hi operand (hi = x truncated);
                       only lo = x - hi, exact in fp32, has to be written. Rounding hi to
                       nearest instead halves |lo| but costs a second 32 KB store per stage on
                       a path bound by shared-memory traffic: 168 -> 188 TFLOP/s at 8192^3 for
                       a relative error of 2.2e-6 instead of 1.8e-6 (budget 1e-5). */
                    const float4 x = *(const float4 *)(hi + i * 16);
                    float4 l;
                    l.x = x.x - __uint_as_float(__float_as_uint(x.x) & 0xFFFFE000u);
                    l.y = x.y - __uint_as_float(__float_as_uint(x.y) & 0xFFFFE000u);
                    l.z = x.z - __uint_as_float(__float_as_uint(x.z) & 0xFFFFE000u);
                    l.w = x.w - __uint_as_float(__float_as_uint(x.w) & 0xFFFFE000u);
                    *(float4 *)(lo + i * 16) = l;
                }
                /* make the generic-proxy stores visible to the tensor core's async-proxy reads
                   (one arrival per warp instead of per thread was measured and is slower) */
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                MbarArrive(SmemAddr(&barConv[s]));
                if (++s == STAGES) { s = 0; ph ^= 1u; }
            }
        }
    }

    else if (LDG) {
        /* ------------------------------------------------------------ loader warps
           Operands whose base or pitch is not a multiple of 16 bytes (tensors carved out of a
           memory pool one after the other) cannot be described to TMA. Eight warps bring each
           stage in with ordinary loads instead: a 128-byte row segment is covered by the 16-byte
           ALIGNED vectors around it, one per lane (eight lanes per segment, the lane of the last
           chunk fetching a ninth), neighbours are exchanged by shuffle, and every lane funnel-
           shifts its 16 bytes into place and stores them where TMA would have put them
           (128-byte swizzle). An aligned vector that holds at least one wanted byte lies inside
           the tensor's allocation, so nothing is read that could fault; bytes outside the
           matrix are zeroed, as TMA's out-of-bounds fill does. */
        constexpr int LW0 = MODE == 0 ? 6 : 6 + CONV_THREADS / 32;
        static_assert(!LDG || (BM == 128 && BN == 128 && LDG_THREADS == 256), "four loader warps per operand, eight chunks per thread and stage");
        constexpr int TASKS = 8;                                    /* 128 segments x 8 chunks / 128 threads */
        constexpr int PER_BOX = EPR / 16;                           /* tasks of a thread inside one MN-major box */
        const int lt = (int)threadIdx.x - LW0 * 32;                /* 0 .. LDG_THREADS-1 */
        const bool opB = lt >= LDG_THREADS / 2;                     /* warps 0-3 of the group load A, 4-7 load B */
        const int l = lt & (LDG_THREADS / 2 - 1);
        const int c = l & 7;                                        /* 16-byte chunk of the segment */
        const int sg0 = l >> 3;                                     /* segment of task 0; task i: sg0 + 16 i */
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int t = firstTile; ok && t < grp.total; t += tileStep) {
            NTB_SELECT_PROBLEM();
            TileCoord tc = DecodeTile(tl, p);
            int pp, qq;
            SplitProb(p, tc.prob, pp, qq);
            const bool mn = (opB ? p.bMN : p.aMN) != 0;
            const long long ld = opB ? p.ldb : p.lda;
            const int ext0 = opB ? tc.nBlk * BN : tc.mBlk * BM;     /* first row / column of the tile */
            const int extN = opB ? p.N : p.M;
            const char * base = opB ? (const char *)p.b + (pp * p.sBp + qq * p.sBq) * ES
                                    : (const char *)p.a + (pp * p.sAp + qq * p.sAq) * ES;
            /* Task i of this thread, k-block kb: segment address = p0 + (i % perBox) * stepI +
               (i / perBox) * 128 + kb * stepK. K-major: a segment is EPR values of K of row
               ext0 + sg0 + 16 i (perBox = 8: no boxes). MN-major: boxes of EPR k-rows x 128 bytes
               of M (resp. N); task i is k-row sg0 + 16 (i % PER_BOX) of box i / PER_BOX. In both
               layouts the chunk lands at dst0 + 2048 i of the stage. */
            const long long stepI = 16 * ld * ES;
            const long long stepK = mn ? (long long)EPR * ld * ES : ROW_BYTES;
            const char * p0 = mn ? base + ((long long)sg0 * ld + ext0) * ES : base + (long long)(ext0 + sg0) * ld * ES;
            uint32_t chunk = (uint32_t)c;
            if (MODE != 0 && mn)
                chunk = (((chunk >> 1) ^ ((uint32_t)sg0 & 3u)) << 1) | (chunk & 1u);      /* 32-byte-chunk swizzle of MN-major fp32 */
            else
                chunk ^= (uint32_t)sg0 & 7u;
            const uint32_t dst0 = (opB ? (uint32_t)A_TILE_BYTES : 0u) + (uint32_t)sg0 * ROW_BYTES + (chunk << 4);

            /* bytes of task i's segment that lie inside the matrix at k-block kb */
            auto validOf = [&](int i, int kb) -> int {
                const int k0 = kb * EPR;
                int live;
                if (!mn)
                    live = ext0 + sg0 + 16 * i < extN ? p.K - k0 : 0;
                else
                    live = k0 + sg0 + 16 * (i % PER_BOX) < p.K ? extN - ext0 - (i / PER_BOX) * EPR : 0;
                live = live < 0 ? 0 : (live > EPR ? EPR : live);
                return live * ES;
            };
            /* i is a compile-time constant wherever this is called: no division is left */
            auto addrOf = [&](int i, int kb) -> uintptr_t {
                const int inBox = mn ? i % PER_BOX : i, box = mn ? i / PER_BOX : 0;
                return (uintptr_t)(p0 + inBox * stepI + box * ROW_BYTES + kb * stepK);
            };
            uint4 own[TASKS], ninth[TASKS];
            /* general form: anything outside the matrix is not read and comes out as zero */
            auto fetch = [&](int i, int kb) {
                const int valid = validOf(i, kb);
                const uintptr_t g = addrOf(i, kb);
                const int last = (int)(g & 15) + valid;             /* wanted bytes of the aligned stream: [g & 15, last) */
                const uint4 * vec = (const uint4 *)(g & ~(uintptr_t)15);
                own[i] = (valid > 0 && 16 * c < last) ? __ldg(vec + c) : make_uint4(0u, 0u, 0u, 0u);
                ninth[i] = (valid > 0 && c == 7 && 128 < last) ? __ldg(vec + 8) : make_uint4(0u, 0u, 0u, 0u);
            };
            /* a k-block whose segments all lie inside the matrix: no bounds to look at */
            auto fetchInside = [&](int i, int kb) {
                const uintptr_t g = addrOf(i, kb);
                const uint4 * vec = (const uint4 *)(g & ~(uintptr_t)15);
                own[i] = __ldg(vec + c);
                if (c == 7 && (g & 15) != 0)
                    ninth[i] = __ldg(vec + 8);
            };
            const bool rowsInside = ext0 + 128 <= extN;             /* the same for every thread of this operand's warps */
            if (rowsInside && EPR <= p.K) {
#pragma unroll
                for (int i = 0; i < TASKS; i++)
                    fetchInside(i, 0);
            }
            else {
#pragma unroll
                for (int i = 0; i < TASKS; i++)
                    fetch(i, 0);
            }
            for (int kb = 0; kb < kBlocks; kb++) {
                /* one decision for the whole warp: the shuffles below need every lane */
                ok = MbarWaitWarp(SmemAddr(&barEmpty[s]), ph ^ 1u, abortPtr, p.status, NTB_WAIT_HINT_NS);
                if (!ok)
                    break;
                const uint32_t stage = smemBase + (uint32_t)s * STAGE_BYTES + dst0;
                const bool inside = rowsInside && (kb + 1) * EPR <= p.K;
                const bool more = kb + 1 < kBlocks;
                const bool nextInside = rowsInside && (kb + 2) * EPR <= p.K;
#pragma unroll
                for (int i = 0; i < TASKS; i++) {
                    uint4 nxt;
                    nxt.x = __shfl_down_sync(0xffffffffu, own[i].x, 1);
                    nxt.y = __shfl_down_sync(0xffffffffu, own[i].y, 1);
                    nxt.z = __shfl_down_sync(0xffffffffu, own[i].z, 1);
                    nxt.w = __shfl_down_sync(0xffffffffu, own[i].w, 1);
                    if (c == 7)
                        nxt = ninth[i];
                    const uint4 o = RealignChunk(own[i], nxt, (uint32_t)(addrOf(i, kb) & 15), c, inside ? ROW_BYTES : validOf(i, kb));
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                 :: "r"(stage + (uint32_t)i * 2048u), "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w) : "memory");
                    /* the registers are free again: start on the next k-block, whose data then
                       arrives under the rest of this one and under the wait for its stage */
                    if (more) {
                        if (nextInside)
                            fetchInside(i, kb + 1);
                        else
                            fetch(i, kb + 1);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0)
                    MbarArrive(SmemAddr(&barFull[s]));
                if (++s == STAGES) { s = 0; ph ^= 1u; }
            }
        }
    }

    /* ---------------------------------------------------------------- teardown */
#ifdef NTB_WAIT_STATS
    if (lane == 0 && warp <= 1) {
        if (warp == 0) { atomicAdd(&gWaitStats[0], (unsigned long long)wstat[0]); atomicAdd(&gWaitStats[5], 1ULL); atomicAdd(&gWaitStats[6], (unsigned long long)wstat[6]); atomicAdd(&gWaitStats[7], (unsigned long long)wstat[7]); atomicAdd(&gWaitStats[3], (unsigned long long)wstat[3]); atomicAdd(&gWaitStats[2], (unsigned long long)wstat[5]);
                         if (blockIdx.x == 0) atomicAdd(&gWaitStats[4], (unsigned long long)(clock64() - kernelT0)); }
        if (warp == 1) { atomicAdd(&gWaitStats[1], (unsigned long long)wstat[1]); }
    }
#endif
    __syncwarp();
    if (*abortPtr) {
        /* give copies and MMAs in flight time to land before shared memory and TMEM go away */
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
    }
    TcFenceBefore();
    __syncthreads();
    TcFenceAfter();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     :: "r"(tmemBase), "r"((uint32_t)TMEM_COLS) : "memory");
    }
#ifdef NTB_WAIT_STATS
    if (threadIdx.x == 32) NTB_MARK(7);
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x < 64) gTimeline[threadIdx.x] = tlShared[threadIdx.x];
#endif
}

template <int MODE, int BN, int STAGES, int G, typename OutT, bool OLDC, bool LDG = false, int NP = 2>
int LaunchOne(const TcGroupT<NP> & grp, int smCount, cudaStream_t stream)
{
    constexpr int stage = (A_TILE_BYTES + BN * ROW_BYTES) * (MODE == 0 ? 1 : 2);
    constexpr int smem = stage * STAGES + EPI_BYTES + 1024;
    auto kern = GemmTcKernel<MODE, BN, STAGES, G, OutT, OLDC, LDG, NP>;
    static SmemOptIn optIn;
    if (!optIn.Ensure((const void *)kern, smem))
        return NTB_ERR_CUDA;
    const int grid = grp.total < smCount ? grp.total : smCount;
    const cudaError_t err = LaunchPdl(kern, grid, (MODE == 0 ? 192 : 192 + CONV_THREADS) + (LDG ? LDG_THREADS : 0), smem, stream, grp);
    CountLaunch();
    return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? NTB_OK : NTB_ERR_CUDA;
}




}

}

#endif
