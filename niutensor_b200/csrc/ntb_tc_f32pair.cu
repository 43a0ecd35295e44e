/*
 * fp32 products on the fp16 tensor pipe of CTA pairs: every fp32 operand value x is written,
 * by a pre-pass, as two half-precision pieces of a scaled copy,
 *
 *        s * x = h1 + h2 (+ a remainder below 2^-22 |s * x|),   h1 = half(s * x), h2 = half(s * x - h1),
 *
 * s a power of two chosen per row of op(a) and per column of op(b) so that the largest
 * scaled magnitude of that row / column lies in [2^14, 2^15): inside half's range with room
 * to spare, and exact to undo. The product is then three half-precision products with fp32
 * accumulation -- a2 * b1 + a1 * b2 + a1 * b1, small terms first -- at the full rate of
 * tcgen05.mma.kind::f16: half the cost of three kind::tf32 passes, whose instructions run at
 * half that rate. The dropped term a2 * b2 is 2^-22 of the result, like the lo * lo term a
 * 3xTF32 scheme drops. An element more than 2^17 below the largest of its row / column keeps
 * an absolute error of 2^-39 of that largest value instead of a relative one.
 *
 * Kernel: pair tile 256 x 256 (tcgen05 cta_group::2), one accumulator per chain of 8
 * k-blocks (512 of K), two of them alternating in tensor memory. A stage of the TMA ring
 * holds the four planes of one k-block -- a1, a2 (this CTA's 128 rows) and b1, b2 (its half
 * of the columns) -- so each plane is fetched once for the two or three products that read
 * it. The tensor core truncates its fp32 accumulator after every instruction, an error
 * that grows with the length of a chain: every chain's partial sum is handed to the epilogue
 * warps, which scale it by alpha and the inverse row and column scales and send it to c
 * while the next chain runs -- the first chain of a tile with a plain TMA store (folding in
 * beta * c and the bias), every later one with a TMA reduce-add, so the additions are
 * round-to-nearest fp32 additions made by the L2 and c is never read back. (A per-lane read
 * of c between chains was tried first: it alone took as long as all the MMAs.)
 *
 * The pre-pass needs scratch for the planes (the size of a and b together) and the scale
 * vectors; it belongs to the device context and grows on demand. Callers that must not
 * allocate, small products and batched ones take the kind::tf32 kernel instead.
 */
#include "ntb_tc_common.cuh"
#include <cmath>

namespace ntb {

namespace {

constexpr int F32_STAGES = 3;
constexpr int F32_BN = 256;
constexpr int F32_BNH = F32_BN / 2;
constexpr int F32_CHAIN = 8;                        /* k-blocks (of 64) per accumulation chain */
constexpr int F32_PLANE_A = A_TILE_BYTES;           /* 128 rows x 128 B */
constexpr int F32_PLANE_B = F32_BNH * ROW_BYTES;
constexpr int F32_STAGE_BYTES = 2 * F32_PLANE_A + 2 * F32_PLANE_B;     /* 64 KB */
constexpr int F32_EPIW = 8;
constexpr int F32_THREADS = 64 + 32 * F32_EPIW;
constexpr int F32_SMEM = F32_STAGES * F32_STAGE_BYTES + F32_EPIW * EPI_BOX_BYTES + 1024;

struct F32Params {
    float * c;
    long long ldc;
    int M, N, K;                 /* K: extent of the product, a multiple of nothing in particular */
    int aMN, bMN;
    int tilesM, tilesN, totalTiles, group;
    FastDiv fdBand, fdGroup, fdLast;
    const float * rowInv;        /* M inverse scales of op(a)'s rows */
    const float * colInv;        /* N inverse scales of op(b)'s columns */
    float alpha, beta;
    const float * bias;
    int act;
    int epiHint;
    int * status;
};

__device__ __forceinline__ void DecodeTile2D(int t, const F32Params & p, int & mBlk, int & nBlk)
{
    uint32_t band, inBand, q, rem;
    p.fdBand.DivMod((uint32_t)t, band, inBand);
    const int first = (int)band * p.group;
    if (p.tilesM - first >= p.group)
        p.fdGroup.DivMod(inBand, q, rem);
    else
        p.fdLast.DivMod(inBand, q, rem);
    mBlk = first + (int)rem;
    nBlk = (int)q;
}

/* 32 fp32 values of one row of c, read through L2 only: the same warp wrote them with a TMA
   store one chain earlier, which a line cached in L1 would not show */
__device__ __forceinline__ void LoadC32(const float * cRow, int c0, int N, bool rowOk, float4 * o)
{
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int c = c0 + j * 4;
        if (rowOk && c + 4 <= N) {
            o[j] = __ldcg((const float4 *)(cRow + c));
        }
        else {
            float t[4] = {0.f, 0.f, 0.f, 0.f};
            if (rowOk) {
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (c + e < N)
                        t[e] = __ldcg(cRow + c + e);
            }
            o[j] = make_float4(t[0], t[1], t[2], t[3]);
        }
    }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(F32_THREADS, 1)
GemmF32SplitPairKernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmC, F32Params p)
{
    constexpr int EPR = 64;                              /* halves of K per k-block */
    constexpr int KSTEPS = ROW_BYTES / UMMA_K_BYTES;     /* 4 */
    constexpr int STAGES = F32_STAGES;

    extern __shared__ uint8_t smemRaw[];
    __shared__ __align__(8) uint64_t barFull[STAGES];
    __shared__ __align__(8) uint64_t barEmpty[STAGES];
    __shared__ __align__(8) uint64_t barTFull[2];
    __shared__ __align__(8) uint64_t barTEmpty[2];
    __shared__ uint32_t tmemBaseSlot;
    __shared__ int abortFlag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ClusterCtaRank();
    const uint32_t smemBase = (SmemAddr(smemRaw) + 1023u) & ~1023u;
    volatile int * abortPtr = &abortFlag;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (threadIdx.x == 128) {
        PrefetchTensorMap(&tmA);
        PrefetchTensorMap(&tmB);
        PrefetchTensorMap(&tmC);
    }
    if (warp == 0) {
        if (lane < STAGES) {
            MbarInit(SmemAddr(&barFull[lane]), 1);
            MbarInit(SmemAddr(&barEmpty[lane]), 1);
        }
        else if (lane >= 8 && lane < 10) {
            MbarInit(SmemAddr(&barTFull[lane - 8]), 1);
            MbarInit(SmemAddr(&barTEmpty[lane - 8]), 2 * F32_EPIW);
        }
        if (lane == 0)
            abortFlag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(SmemAddr(&tmemBaseSlot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    TcFenceBefore();
    ClusterSync();
    TcFenceAfter();
    const uint32_t tmemBase = *(volatile uint32_t *)&tmemBaseSlot;

    const int kBlocks = (p.K + EPR - 1) / EPR;
#ifdef NTB_WAIT_STATS
    long long wstat[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const long long kernelT0 = clock64();
#endif
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int firstTile = blockIdx.x >> 1;
    const int tileStep = gridDim.x >> 1;

    if (warp == 0) {
        /* ------------------------------------------------------------ TMA producer */
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            const bool aMN = p.aMN != 0, bMN = p.bMN != 0;
            int * const status = p.status;
            for (int t = firstTile; ok && t < p.totalTiles; t += tileStep) {
                int mBlk, nBlk;
                DecodeTile2D(t, p, mBlk, nBlk);
                const int m0 = mBlk * 2 * BM + (int)rank * BM;
                const int n0 = nBlk * F32_BN + (int)rank * F32_BNH;
                for (int kb = 0; kb < kBlocks; kb++) {
                    NTB_TIMED(0, ok = MbarWait(SmemAddr(&barEmpty[s]), ph ^ 1u, abortPtr, status));
                    if (!ok)
                        break;
                    const uint32_t fullLeader = MapToCta(SmemAddr(&barFull[s]), 0);
                    if (rank == 0)
                        MbarExpectTx(SmemAddr(&barFull[s]), 2u * F32_STAGE_BYTES);
                    const uint32_t base = smemBase + (uint32_t)s * F32_STAGE_BYTES;
                    const int k0 = kb * EPR;
#pragma unroll
                    for (int pl = 0; pl < 2; pl++) {
                        const uint32_t aDst = base + pl * F32_PLANE_A;
                        const uint32_t bDst = base + 2 * F32_PLANE_A + pl * F32_PLANE_B;
                        if (!aMN) {
                            TmaLoad3DPair(aDst, &tmA, fullLeader, k0, m0, pl);
                        }
                        else {
#pragma unroll
                            for (int i = 0; i < BM / EPR; i++)
                                TmaLoad3DPair(aDst + i * EPR * ROW_BYTES, &tmA, fullLeader, m0 + i * EPR, k0, pl);
                        }
                        if (!bMN) {
                            TmaLoad3DPair(bDst, &tmB, fullLeader, k0, n0, pl);
                        }
                        else {
#pragma unroll
                            for (int i = 0; i < F32_BNH / EPR; i++)
                                TmaLoad3DPair(bDst + i * EPR * ROW_BYTES, &tmB, fullLeader, n0 + i * EPR, k0, pl);
                        }
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    }
    else if (warp == 1) {
        /* ------------------------------------------------------------ MMA issuer (leader CTA) */
        if (lane == 0 && rank == 0) {
            const uint32_t iDesc = (1u << 4) | ((uint32_t)(p.aMN ? 1 : 0) << 15) | ((uint32_t)(p.bMN ? 1 : 0) << 16)
                                 | ((uint32_t)(F32_BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            const uint32_t aLbo = p.aMN ? EPR * ROW_BYTES : 16, bLbo = p.bMN ? EPR * ROW_BYTES : 16;
            const uint32_t mnStep = (UMMA_K_BYTES / 2) * ROW_BYTES;
            const uint32_t aStep4 = (p.aMN ? mnStep : UMMA_K_BYTES) >> 4, bStep4 = (p.bMN ? mnStep : UMMA_K_BYTES) >> 4;
            const uint64_t aD0 = SmemDesc(smemBase, aLbo, 1024, 2);
            const uint64_t bD0 = SmemDesc(smemBase + 2 * F32_PLANE_A, bLbo, 1024, 2);
            const uint32_t aLo0 = (uint32_t)aD0, aHiW = (uint32_t)(aD0 >> 32);
            const uint32_t bLo0 = (uint32_t)bD0, bHiW = (uint32_t)(bD0 >> 32);
            constexpr uint32_t A2 = F32_PLANE_A >> 4, B2 = F32_PLANE_B >> 4;     /* second plane, in 16-byte units */
            const uint32_t barFull0 = SmemAddr(&barFull[0]), barEmpty0 = SmemAddr(&barEmpty[0]);
            int s = 0;
            uint32_t ph = 0, it = 0, stageOff = 0;
            bool ok = true;
            int * const status = p.status;
            for (int t = firstTile; ok && t < p.totalTiles; t += tileStep) {
                for (int kb0 = 0; ok && kb0 < kBlocks; kb0 += F32_CHAIN, ++it) {
                    const uint32_t buf = it & 1u;
                    NTB_TIMED(2, ok = MbarWait(SmemAddr(&barTEmpty[buf]), ((it >> 1) & 1u) ^ 1u, abortPtr, status));
                    if (!ok)
                        break;
                    TcFenceAfter();
                    const uint32_t dTmem = tmemBase + buf * F32_BN;
                    const int kbEnd = min(kBlocks, kb0 + F32_CHAIN);
                    uint32_t acc = 0u;
                    for (int kb = kb0; kb < kbEnd; kb++) {
                        NTB_TIMED(1, ok = MbarWait(barFull0 + (uint32_t)s * 8u, ph, abortPtr, status));
                        if (!ok)
                            break;
                        TcFenceAfter();
                        uint32_t aLo = aLo0 + stageOff, bLo = bLo0 + stageOff;
#pragma unroll
                        for (int k = 0; k < KSTEPS; k++) {
                            TcMmaPairLH(dTmem, aLo + A2, aHiW, bLo, bHiW, iDesc, acc);          /* a2 * b1 */
                            TcMmaPairLH(dTmem, aLo, aHiW, bLo + B2, bHiW, iDesc, 1u);           /* a1 * b2 */
                            TcMmaPairLH(dTmem, aLo, aHiW, bLo, bHiW, iDesc, 1u);                /* a1 * b1 */
                            acc = 1u;
                            aLo += aStep4;
                            bLo += bStep4;
                        }
                        TcCommitPair(barEmpty0 + (uint32_t)s * 8u);
                        stageOff += F32_STAGE_BYTES >> 4;
                        if (++s == STAGES) { s = 0; ph ^= 1u; stageOff = 0; }
                    }
                    if (ok)
                        TcCommitPair(SmemAddr(&barTFull[buf]));
                }
            }
        }
    }
    else {
        /* ------------------------------------------------------------ epilogue: eight warps, two per
           TMEM sub-partition, each owning 128 of the tile's 256 columns */
        const int sub32 = warp & 3;
        const int ew = warp - 2;
        const int colHalf = ew >> 2;
        const uint32_t box = smemBase + STAGES * F32_STAGE_BYTES + (uint32_t)ew * EPI_BOX_BYTES;
        const uint32_t rowAddr = box + lane * ROW_BYTES;
        uint32_t it = 0;
        bool ok = true;
        bool stored = false;
        for (int t = firstTile; ok && t < p.totalTiles; t += tileStep) {
            int mBlk, nBlk;
            DecodeTile2D(t, p, mBlk, nBlk);
            const int row0 = mBlk * 2 * BM + (int)rank * BM + sub32 * 32;
            const int row = row0 + lane;
            const bool rowOk = row < p.M;
            const int cBeg = nBlk * F32_BN + colHalf * 128;
            float * cRow = p.c + (long long)row * p.ldc;
            const float rs = rowOk ? p.alpha * __ldg(p.rowInv + row) : 0.f;
            int it1 = 0;                          /* chains of this tile handled so far */
            for (int kb0 = 0; ok && kb0 < kBlocks; kb0 += F32_CHAIN, ++it, ++it1) {
                const uint32_t buf = it & 1u;
                const bool first = kb0 == 0, last = kb0 + F32_CHAIN >= kBlocks;
                /* The first chain of a tile writes beta * c + its partial sum with a plain store;
                   later chains are added to c by the L2 itself (TMA reduce-add, a round-to-nearest
                   fp32 addition), so c is not read back. Only a rectifier, which needs the complete
                   sum, makes the last chain read c, add and store. */
                const bool finalRmw = last && !first && p.act == NTB_ACT_RECTIFY;
                const bool readC = first ? p.beta != 0.f : finalRmw;
                const bool reduce = !first && !finalRmw;
                const float cf = first ? p.beta : 1.f;
                if (stored && (it1 == 1 || finalRmw)) {
                    /* the plain stores of the first chain must have landed before anything is added
                       to them; every addition must have landed before the sum is read back */
                    if (lane == 0)
                        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                    __syncwarp();
                }
                float4 oldNxt[8];
                if (readC && cBeg < p.N)
                    LoadC32(cRow, cBeg, p.N, rowOk, oldNxt);
                NTB_TIMED(3, ok = MbarWaitWarp(SmemAddr(&barTFull[buf]), (it >> 1) & 1u, abortPtr, p.status, (uint32_t)p.epiHint));
                if (!ok)
                    break;
                TcFenceAfter();
                const uint32_t tRow = tmemBase + ((uint32_t)(sub32 * 32) << 16) + buf * F32_BN + colHalf * 128;
#pragma unroll 1
                for (int h = 0; h < 4; h++) {
                    const int c0 = cBeg + h * 32;
                    if (c0 >= p.N)
                        break;                     /* uniform across the warp */
                    float4 old[8];
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        old[j] = oldNxt[j];
                    if (readC && h + 1 < 4 && c0 + 32 < p.N)
                        LoadC32(cRow, c0 + 32, p.N, rowOk, oldNxt);
                    float v[32];
                    TmemLoad32(tRow + h * 32, v);
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const int c = c0 + j * 4;
                        float cs[4];
                        if (c + 4 <= p.N) {
                            const float4 q = __ldg((const float4 *)(p.colInv + c));
                            cs[0] = q.x; cs[1] = q.y; cs[2] = q.z; cs[3] = q.w;
                        }
                        else {
#pragma unroll
                            for (int e = 0; e < 4; e++)
                                cs[e] = c + e < p.N ? __ldg(p.colInv + c + e) : 0.f;
                        }
                        const float o4[4] = { old[j].x, old[j].y, old[j].z, old[j].w };
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            float x = rs * cs[e] * v[j * 4 + e];
                            if (readC)
                                x = fmaf(cf, o4[e], x);
                            v[j * 4 + e] = x;
                        }
                    }
                    /* the bias joins the first chain; the rectifier closes the last */
                    if (first && p.bias != nullptr) {
#pragma unroll
                        for (int e = 0; e < 32; e++)
                            if (c0 + e < p.N)
                                v[e] += __ldg(p.bias + c0 + e);
                    }
                    if (last && p.act == NTB_ACT_RECTIFY) {
#pragma unroll
                        for (int e = 0; e < 32; e++)
                            v[e] = fmaxf(v[e], 0.f);
                    }
                    /* the store that last used the box must have read it */
                    if (lane == 0 && stored)
                        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const uint32_t dst = rowAddr + (uint32_t)((j ^ (lane & 7)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                     :: "r"(dst), "r"(__float_as_uint(v[j * 4])), "r"(__float_as_uint(v[j * 4 + 1])),
                                        "r"(__float_as_uint(v[j * 4 + 2])), "r"(__float_as_uint(v[j * 4 + 3])) : "memory");
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0 && row0 < p.M) {
                        if (reduce)
                            asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
                                         :: "l"(&tmC), "r"(c0), "r"(row0), "r"(0), "r"(box) : "memory");
                        else
                            asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                                         :: "l"(&tmC), "r"(c0), "r"(row0), "r"(0), "r"(box) : "memory");
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                    stored = true;
                }
                TcFenceBefore();
                __syncwarp();
                if (lane == 0)
                    MbarArriveCluster(MapToCta(SmemAddr(&barTEmpty[buf]), 0));
            }
        }
        if (lane == 0)
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
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
    ClusterSync();
    TcFenceAfter();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;"
                     :: "r"(tmemBase), "r"(512u) : "memory");
    }
}

/* ---------------------------------------------------------------- the pre-pass */

/* power of two that brings a largest magnitude m into [2^14, 2^15); 1 for 0, inf and NaN */
__device__ __forceinline__ float ScaleFor(float m, float * inv)
{
    float s = 1.f, is = 1.f;
    if (m > 0.f && m <= 3.4028234e38f) {
        int e;
        frexpf(m, &e);                                  /* m = f * 2^e, f in [0.5, 1) */
        int k = 15 - e;
        k = k > 126 ? 126 : (k < -126 ? -126 : k);
        s = ldexpf(1.f, k);
        is = ldexpf(1.f, -k);
    }
    *inv = is;
    return s;
}

__device__ __forceinline__ void SplitOne(float x, float s, __half & h1, __half & h2)
{
    const float y = x * s;
    h1 = __float2half_rn(y);
    h2 = __float2half_rn(y - __half2float(h1));
}

/* operand whose scaled index is its stored row: one block per row. VEC: rows start on
   16-byte boundaries and hold a multiple of four values, so the row is read four values and
   written four halves at a time */
template <bool VEC>
__global__ void __launch_bounds__(256)
SplitRowsKernel(const float * __restrict__ x, long long ld, int rows, int cols, __half * __restrict__ p1,
                __half * __restrict__ p2, long long pitch, float * __restrict__ inv)
{
    __shared__ float red[8];
    __shared__ float scaleShared;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const float FMAX = 3.4028234e38f;
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const float * src = x + (long long)r * ld;
        float m = 0.f;
        bool bad = false;
        if (VEC) {
            for (int c = threadIdx.x * 4; c < cols; c += blockDim.x * 4) {
                const float4 q = *(const float4 *)(src + c);
                const float v = fmaxf(fmaxf(fabsf(q.x), fabsf(q.y)), fmaxf(fabsf(q.z), fabsf(q.w)));
                bad |= !(fabsf(q.x) <= FMAX) | !(fabsf(q.y) <= FMAX) | !(fabsf(q.z) <= FMAX) | !(fabsf(q.w) <= FMAX);
                m = fmaxf(m, v);
            }
        }
        else {
            for (int c = threadIdx.x; c < cols; c += blockDim.x) {
                const float v = fabsf(src[c]);
                bad |= !(v <= FMAX);
                m = fmaxf(m, v);
            }
        }
        if (bad)
            m = __int_as_float(0x7f800000);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, m, o);
            m = (other > m || !(other <= FMAX)) ? other : m;
        }
        if ((threadIdx.x & 31) == 0)
            red[threadIdx.x >> 5] = m;
        __syncthreads();
        if (threadIdx.x == 0) {
            float mm = red[0];
            for (int i = 1; i < 8; i++)
                mm = (red[i] > mm || !(red[i] <= FMAX)) ? red[i] : mm;
            float is;
            scaleShared = ScaleFor(mm, &is);
            inv[r] = is;
        }
        __syncthreads();
        const float s = scaleShared;
        __half * d1 = p1 + (long long)r * pitch;
        __half * d2 = p2 + (long long)r * pitch;
        if (VEC) {
            for (int c = threadIdx.x * 4; c < cols; c += blockDim.x * 4) {
                const float4 q = *(const float4 *)(src + c);
                __half a[4], b[4];
                SplitOne(q.x, s, a[0], b[0]);
                SplitOne(q.y, s, a[1], b[1]);
                SplitOne(q.z, s, a[2], b[2]);
                SplitOne(q.w, s, a[3], b[3]);
                *(uint2 *)(d1 + c) = *(const uint2 *)a;
                *(uint2 *)(d2 + c) = *(const uint2 *)b;
            }
        }
        else {
            for (int c = threadIdx.x; c < cols; c += blockDim.x) {
                __half h1, h2;
                SplitOne(src[c], s, h1, h2);
                d1[c] = h1;
                d2[c] = h2;
            }
        }
        __syncthreads();
    }
}

/* operand whose scaled index is its stored column: largest magnitude per column ... */
__global__ void __launch_bounds__(256)
ColAbsMaxKernel(const float * __restrict__ x, long long ld, int rows, int cols, int rowsPerBlock, unsigned * __restrict__ colMax)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols)
        return;
    const int r0 = blockIdx.y * rowsPerBlock;
    const int r1 = min(rows, r0 + rowsPerBlock);
    unsigned m = 0;
    for (int r = r0; r < r1; r++) {
        /* bit patterns of non-negative floats order like the floats; NaN sorts above infinity */
        const unsigned b = __float_as_uint(x[(long long)r * ld + c]) & 0x7fffffffu;
        m = b > m ? b : m;
    }
    if (m)
        atomicMax(colMax + c, m);
}

/* ... turned into scales (in place: the word becomes the scale, inv gets its inverse) ... */
__global__ void __launch_bounds__(256)
ColScaleKernel(unsigned * __restrict__ colMax, int cols, float * __restrict__ inv)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols)
        return;
    float is;
    const float s = ScaleFor(__uint_as_float(colMax[c]), &is);
    colMax[c] = __float_as_uint(s);
    inv[c] = is;
}

/* ... and the split itself */
__global__ void __launch_bounds__(256)
SplitColsKernel(const float * __restrict__ x, long long ld, int rows, int cols, int rowsPerBlock,
                const float * __restrict__ scale, __half * __restrict__ p1, __half * __restrict__ p2, long long pitch)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols)
        return;
    const float s = scale[c];
    const int r0 = blockIdx.y * rowsPerBlock;
    const int r1 = min(rows, r0 + rowsPerBlock);
    for (int r = r0; r < r1; r++) {
        __half h1, h2;
        SplitOne(x[(long long)r * ld + c], s, h1, h2);
        p1[(long long)r * pitch + c] = h1;
        p2[(long long)r * pitch + c] = h2;
    }
}

bool Ok(cudaError_t e)
{
    return e == cudaSuccess;
}

/* splits one stored operand (rows x cols, pitch ld) into planes; byRow: scale per stored row */
int SplitOperand(const DeviceCtx & ctx, const float * x, long long ld, int rows, int cols, bool byRow,
                 __half * planes, long long pitch, long long planeElems, float * inv, unsigned * colWork, cudaStream_t st)
{
    if (byRow) {
        const int grid = rows < ctx.smCount * 8 ? rows : ctx.smCount * 8;
        /* plain launches: the pre-pass must not start before the product ahead of it in the
           stream, which may still read the planes, has finished */
        const bool vec = ((uintptr_t)x & 15) == 0 && ld % 4 == 0 && cols % 4 == 0 && planeElems % 4 == 0;
        if (vec)
            SplitRowsKernel<true><<<grid, 256, 0, st>>>(x, ld, rows, cols, planes, planes + planeElems, pitch, inv);
        else
            SplitRowsKernel<false><<<grid, 256, 0, st>>>(x, ld, rows, cols, planes, planes + planeElems, pitch, inv);
        CountLaunch();
        return Ok(cudaGetLastError()) ? NTB_OK : NTB_ERR_CUDA;
    }
    if (!Ok(cudaMemsetAsync(colWork, 0, sizeof(unsigned) * (size_t)cols, st)))
        return NTB_ERR_CUDA;
    const int rowsPerBlock = 64;
    const dim3 grid((unsigned)((cols + 255) / 256), (unsigned)((rows + rowsPerBlock - 1) / rowsPerBlock), 1);
    ColAbsMaxKernel<<<grid, 256, 0, st>>>(x, ld, rows, cols, rowsPerBlock, colWork);
    ColScaleKernel<<<(cols + 255) / 256, 256, 0, st>>>(colWork, cols, inv);
    SplitColsKernel<<<grid, 256, 0, st>>>(x, ld, rows, cols, rowsPerBlock, (const float *)colWork, planes, planes + planeElems, pitch);
    CountLaunch();
    CountLaunch();
    CountLaunch();
    return Ok(cudaGetLastError()) ? NTB_OK : NTB_ERR_CUDA;
}

}

#ifdef NTB_WAIT_STATS
extern "C" void ntb_debug_wait_stats_f32(unsigned long long * out)
{
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, gWaitStats, sizeof(unsigned long long) * 8);
    unsigned long long zero[8] = {0};
    cudaMemcpyToSymbol(gWaitStats, zero, sizeof(zero));
}
#endif

bool F32SplitEligible(const DeviceCtx & ctx, const Problem & p)
{
    if (!ctx.mayAllocate || p.dtAB != NTB_X_FLOAT || p.dtC != NTB_X_FLOAT || p.count != 1 || p.nPeers > 0)
        return false;
    if (ctx.smCount < 2 || p.M <= 0 || p.N <= 0 || p.K <= 0)
        return false;
    /* the pre-pass and the start of a pair kernel only pay on large products */
    if ((double)p.M * p.N * p.K < 4.0e9 || p.M < 512 || p.N < 512)
        return false;
    /* c through TMA stores: 16-byte aligned base and pitch */
    if (((uintptr_t)p.c & 15) || (p.ldc * 4) % 16 || p.ldc < p.N)
        return false;
    if (p.bias && ((uintptr_t)p.bias & 3))
        return false;
    return true;
}

int LaunchF32Split(const DeviceCtx & ctx, const Problem & p, cudaStream_t stream)
{
    /* planes: [2][rows][pitch] halves per operand, pitch a multiple of 8 (16-byte rows) */
    const long long pitchA = ((long long)p.aCols + 7) / 8 * 8, pitchB = ((long long)p.bCols + 7) / 8 * 8;
    const long long planeA = pitchA * p.aRows, planeB = pitchB * p.bRows;
    const size_t bytesA = (size_t)(2 * planeA) * 2, bytesB = (size_t)(2 * planeB) * 2;
    /* scale vectors: inverse scales of M rows and N columns, and a work vector for column maxima */
    const size_t vecLen = (size_t)(p.M > p.N ? p.M : p.N);
    void * bufA = nullptr, * bufB = nullptr, * bufV = nullptr;
    /* the planes are shared by all calls on this device: start behind their last reader */
    int rc = ScratchAcquire(ctx, stream);
    if (rc != NTB_OK)
        return rc;
    rc = EnsureScratch(ctx, 0, bytesA, &bufA);
    if (rc == NTB_OK)
        rc = EnsureScratch(ctx, 1, bytesB, &bufB);
    if (rc == NTB_OK)
        rc = EnsureScratch(ctx, 2, 4 * vecLen * sizeof(float), &bufV);
    if (rc != NTB_OK)
        return rc;
    float * rowInv = (float *)bufV, * colInv = rowInv + vecLen;
    unsigned * workA = (unsigned *)(colInv + vecLen), * workB = workA + vecLen;

    /* op(a)'s rows are a's stored rows unless a is used transposed; op(b)'s columns are b's
       stored columns unless b is used transposed */
    rc = SplitOperand(ctx, (const float *)p.a, p.lda, p.aRows, p.aCols, !p.aMN, (__half *)bufA, pitchA, planeA, rowInv, workA, stream);
    if (rc != NTB_OK)
        return rc;
    rc = SplitOperand(ctx, (const float *)p.b, p.ldb, p.bRows, p.bCols, !p.bMN, (__half *)bufB, pitchB, planeB, colInv, workB, stream);
    if (rc != NTB_OK)
        return rc;

    CUtensorMap maps[3];
    rc = EncodeOperandMap(&maps[0], 0, bufA, p.aMN, p.aRows, p.aCols, pitchA, planeA, 2, BM);
    if (rc == NTB_OK)
        rc = EncodeOperandMap(&maps[1], 0, bufB, p.bMN, p.bRows, p.bCols, pitchB, planeB, 2, F32_BNH);
    if (rc == NTB_OK)
        rc = EncodeOutputMap(&maps[2], NTB_X_FLOAT, p.c, p.M, p.N, p.ldc, 0, 1);
    if (rc != NTB_OK)
        return rc;

    F32Params fp;
    fp.c = (float *)p.c; fp.ldc = p.ldc;
    fp.M = p.M; fp.N = p.N; fp.K = p.K;
    fp.aMN = p.aMN; fp.bMN = p.bMN;
    fp.tilesM = (p.M + 2 * BM - 1) / (2 * BM);
    fp.tilesN = (p.N + F32_BN - 1) / F32_BN;
    const long long tiles = (long long)fp.tilesM * fp.tilesN;
    if (tiles > 1073741823LL)
        return NTB_ERR_LIMIT;
    fp.totalTiles = (int)tiles;
    fp.group = 8;
    fp.fdBand.Set((uint32_t)(fp.group * fp.tilesN));
    fp.fdGroup.Set((uint32_t)fp.group);
    fp.fdLast.Set((uint32_t)(fp.tilesM % fp.group ? fp.tilesM % fp.group : fp.group));
    fp.rowInv = rowInv; fp.colInv = colInv;
    fp.alpha = p.alpha; fp.beta = p.beta;
    fp.bias = (const float *)p.bias; fp.act = p.act;
    fp.epiHint = 2000;
    fp.status = ctx.status;

    static SmemOptIn optIn;
    if (!optIn.Ensure((const void *)GemmF32SplitPairKernel, F32_SMEM))
        return NTB_ERR_CUDA;
    const int pairs = (int)(tiles < ctx.smCount / 2 ? tiles : ctx.smCount / 2);
    const cudaError_t err = LaunchPdl(GemmF32SplitPairKernel, 2 * pairs, F32_THREADS, F32_SMEM, stream, maps[0], maps[1], maps[2], fp);
    CountLaunch();
    if (err != cudaSuccess || cudaGetLastError() != cudaSuccess)
        return NTB_ERR_CUDA;
    return ScratchRelease(ctx, stream);
}

}
