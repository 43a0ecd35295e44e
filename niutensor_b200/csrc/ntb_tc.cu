/*
 * Tensor-core route for sm_100a: a persistent, warp-specialised GEMM built directly on
 * tcgen05.mma with accumulators in tensor memory (TMEM) and operands brought into
 * 128-byte-swizzled shared memory by TMA (cp.async.bulk.tensor, no cluster multicast).
 *
 *   warp 0      TMA producer: one lane arms full[s] with the byte count of a group of
 *               G k-blocks and issues their A and B boxes into the G slots of stage s.
 *   warp 1      owns TMEM (tcgen05.alloc / dealloc); one lane issues the tcgen05.mma
 *               instructions of the group and commits them to empty[s]; after the last
 *               k-block of a tile it commits to tfull[buf]. G > 1 because this lane
 *               waits about 200 clocks for the answer to a barrier probe issued behind
 *               tensor-core instructions: per hand-shake it spends 300-400 clocks that
 *               only enough MMAs between two hand-shakes can cover. Its loop touches no
 *               kernel parameter and moves each shared-memory descriptor with one add.
 *   warps 2-5   epilogue: tcgen05.ld of the finished accumulator (each warp reads the 32
 *               TMEM lanes of its sub-partition), alpha / beta / bias / rectifier in
 *               fp32, cast, staging in swizzled shared memory and TMA stores to C (direct
 *               stores when C is not 16-byte aligned), then release of the accumulator
 *               through tempty[buf]. Two accumulators alternate, so the epilogue of tile
 *               i overlaps the main loop of tile i+1. Old values of C (beta != 0) come by
 *               TMA load into the staging boxes (narrow tiles) or are requested one
 *               64-column chunk ahead into registers (wide tiles); kernels for
 *               beta == 0 are instantiated without any of that.
 *   warps 6-9   (fp32 inputs only) write, for every fp32 operand value x in shared memory,
 *               lo = x - hi into a second plane, hi being x with its 13 low mantissa bits
 *               dropped, which is how the tensor core reads the loaded plane itself; the
 *               MMA lane then issues three kind::tf32 products per k-step,
 *               lo*hi + hi*lo + hi*hi, small terms first.
 *               K is cut into chains of 256; the epilogue warps add the chains' partial
 *               sums into a running sum held in a third TMEM region.
 *
 * One CTA per SM walks output tiles tile = blockIdx.x + i * gridDim.x over
 * (problem, mBlock, nBlock); all problems of a batched / broadcast call are covered by
 * this one launch, base addresses coming from the problem index.
 *
 * Every wait on an mbarrier is bounded: when the limit passes, the waiter raises the
 * CTA's abort flag, records NTB_ERR_DEVICE_WAIT in the device status word, and every role
 * leaves its loop; the CTA then lets copies in flight land, frees its TMEM and returns.
 */
#include "ntb_internal.h"
#include <cstdio>
#include "ntb_ptx.cuh"
#include <cstdlib>
#include <cmath>

namespace ntb {

namespace {

/* fp32 route: threads that split operands into hi/lo planes (warps 6 and up) */
#ifndef NTB_CONV_THREADS
#define NTB_CONV_THREADS 128
#endif
constexpr int CONV_THREADS = NTB_CONV_THREADS;
constexpr int FP32_CHUNK_BLOCKS = 8;  /* fp32 route: 8 k-blocks = 256 of K per TMEM accumulation chain */

/* Division of a 31-bit unsigned number by a run-time constant as multiply-high, add and
   shift: the tile walk and the batch indices need several divisions per tile, and a
   hardware-emulated integer division costs about two hundred clocks of latency each. */
struct FastDiv {
    uint32_t d, m, s;
    __host__ void Set(uint32_t div)
    {
        d = div ? div : 1;
        s = 0;
        while ((1ull << s) < d)
            s++;
        m = (uint32_t)((((1ull << 32) * ((1ull << s) - d)) / d) + 1);
    }
    __device__ __forceinline__ uint32_t Div(uint32_t n) const { return (__umulhi(n, m) + n) >> s; }
    __device__ __forceinline__ void DivMod(uint32_t n, uint32_t & q, uint32_t & r) const { q = Div(n); r = n - q * d; }
};

struct TcParams {
    void * c;
    long long ldc, sCp, sCq;
    int M, N, K, count, Q;
    int aSel, bSel;         /* which index walks the operand's batch dimension: 0 none, 1 p, 2 q, 3 i */
    int aMN, bMN;
    int tilesM, tilesN;
    int totalTiles;
    int cVec;               /* C rows can be accessed with 16-byte vectors */
    int cTma;               /* C is written with TMA stores from swizzled staging boxes */
    int cSel;               /* index that walks C's batch dimension in its tensor map (as aSel) */
    int pfDist;             /* producer asks L2 for the boxes of k-block kb + pfDist while loading kb; 0 = off */
    int group;              /* m-blocks per band of the tile walk */
    FastDiv fdPerProb, fdBand, fdGroup, fdLast, fdQ;   /* tiles per problem, tiles per band, rows of a full / of the last band, Q */
    int epiHint;            /* suspend-time hint (ns) of the epilogue warps' barrier probes */
    void * peers[NTB_MAX_PEERS];   /* further destinations of every result tile (peer GPUs' C), or none */
    int nPeers;
    int l2Hint;             /* pair kernel: L2 eviction policy of the A loads (bits 0-1) and B loads (bits 2-3): 0 none, 1 keep, 2 stream */
    int cPrefetch;          /* wide tiles with beta != 0: 0 no L2 prefetch of old C, 1 boxes through TMA, 2 one request per line */
    float alpha, beta;
    const void * bias;      /* N values of C's type added to every output row, or NULL */
    int act;                /* 1: max(x, 0) applied last */
    int * status;
};

/* Optional wait accounting (compile with -DNTB_WAIT_STATS): cycles each role of the
   CTA-pair kernel spends blocked on its barriers, summed over CTAs.
   0 producer on empty, 1 MMA on full, 2 MMA on tempty, 3 epilogue warp 2 on tfull,
   4 kernel cycles of CTA 0's producer lane, 5 CTAs counted */
#ifdef NTB_WAIT_STATS
__device__ unsigned long long gWaitStats[8];
/* timeline of CTA 0 of the single-CTA kernel, in SM clocks since kernel entry:
   0 set-up done, 1 first TMA issued, 2 first stage landed, 3 first tile's MMAs committed,
   4 epilogue saw the accumulator, 5 epilogue stores issued, 6 stores complete, 7 kernel end */
__device__ unsigned long long gTimeline[64];
#define NTB_MARKK(row, kb) do { if (blockIdx.x == 0 && (kb) < 16 && tlShared[16 + (row) * 16 + (kb)] == 0) tlShared[16 + (row) * 16 + (kb)] = (unsigned long long)(clock64() - kernelT0) + 1; } while (0)
#define NTB_MARK(slot) do { if (blockIdx.x == 0 && tlShared[slot] == 0) tlShared[slot] = (unsigned long long)(clock64() - kernelT0) + 1; } while (0)
#ifdef NTB_CLOCKS
#define NTB_TIMED(slot, expr) do { long long t0_ = clock64(); expr; wstat[slot] += clock64() - t0_; } while (0)
#else
#undef NTB_MARK
#undef NTB_MARKK
#define NTB_MARK(slot) do { } while (0)
#define NTB_MARKK(row, kb) do { } while (0)
#define NTB_TIMED(slot, expr) do { expr; } while (0)
#endif
#else
#define NTB_MARK(slot) do { } while (0)
#define NTB_MARKK(row, kb) do { } while (0)
#define NTB_TIMED(slot, expr) do { expr; } while (0)
#endif

/* ---------------------------------------------------------------- epilogue helpers */

template <typename OutT> struct Vec16;
template <> struct Vec16<__half> { static constexpr int N = 8; };
template <> struct Vec16<float>  { static constexpr int N = 4; };

__device__ __forceinline__ void StoreVec(__half * dst, const float * v)
{
    uint4 u;
    __half2 h0 = __floats2half2_rn(v[0], v[1]);
    __half2 h1 = __floats2half2_rn(v[2], v[3]);
    __half2 h2 = __floats2half2_rn(v[4], v[5]);
    __half2 h3 = __floats2half2_rn(v[6], v[7]);
    u.x = *(uint32_t *)&h0; u.y = *(uint32_t *)&h1; u.z = *(uint32_t *)&h2; u.w = *(uint32_t *)&h3;
    *(uint4 *)dst = u;
}
__device__ __forceinline__ void StoreVec(float * dst, const float * v)
{
    *(float4 *)dst = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void LoadVec(const __half * src, float * v)
{
    uint4 u = *(const uint4 *)src;
    float2 f;
    f = __half22float2(*(__half2 *)&u.x); v[0] = f.x; v[1] = f.y;
    f = __half22float2(*(__half2 *)&u.y); v[2] = f.x; v[3] = f.y;
    f = __half22float2(*(__half2 *)&u.z); v[4] = f.x; v[5] = f.y;
    f = __half22float2(*(__half2 *)&u.w); v[6] = f.x; v[7] = f.y;
}
__device__ __forceinline__ void LoadVec(const float * src, float * v)
{
    float4 f = *(const float4 *)src;
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}
__device__ __forceinline__ float LoadOne(const __half * p) { return __half2float(*p); }
__device__ __forceinline__ float LoadOne(const float * p) { return *p; }
__device__ __forceinline__ void StoreOne(__half * p, float v) { *p = __float2half_rn(v); }
__device__ __forceinline__ void StoreOne(float * p, float v) { *p = v; }

/* v <- act(alpha * v (+ beta * old C) (+ bias)) for 32 consecutive columns of one output
   row starting at column c0; old values and the bias are read with 16-byte vectors where
   alignment allows it */
template <typename OutT>
__device__ __forceinline__ void ScaleRow32(const OutT * cRow, int c0, bool rowOk, float * v, const TcParams & p,
                                           bool scaled = false)
{
    constexpr int VN = Vec16<OutT>::N;
    if (scaled) {
        /* the caller has already formed alpha * v + beta * old C */
    }
    else if (p.beta == 0.f || !rowOk) {
#pragma unroll
        for (int e = 0; e < 32; e++)
            v[e] = p.alpha * v[e];
    }
    else {
#pragma unroll
        for (int g = 0; g < 32 / VN; g++) {
            const int c = c0 + g * VN;
            float * vv = v + g * VN;
            if (p.cVec && c + VN <= p.N) {
                float old[VN];
                LoadVec(cRow + c, old);
#pragma unroll
                for (int e = 0; e < VN; e++)
                    vv[e] = fmaf(p.beta, old[e], p.alpha * vv[e]);
            }
            else {
#pragma unroll
                for (int e = 0; e < VN; e++) {
                    float x = p.alpha * vv[e];
                    if (c + e < p.N)
                        x = fmaf(p.beta, LoadOne(cRow + c + e), x);
                    vv[e] = x;
                }
            }
        }
    }
    if (p.bias != nullptr) {
        const OutT * bias = (const OutT *)p.bias;
        const bool vec = (((uintptr_t)bias) & 15) == 0;
#pragma unroll
        for (int g = 0; g < 32 / VN; g++) {
            const int c = c0 + g * VN;
            float * vv = v + g * VN;
            if (vec && c + VN <= p.N) {
                float bv[VN];
                LoadVec(bias + c, bv);
#pragma unroll
                for (int e = 0; e < VN; e++)
                    vv[e] += bv[e];
            }
            else {
#pragma unroll
                for (int e = 0; e < VN; e++)
                    if (c + e < p.N)
                        vv[e] += LoadOne(bias + c + e);
            }
        }
    }
    if (p.act == NTB_ACT_RECTIFY) {
#pragma unroll
        for (int e = 0; e < 32; e++)
            v[e] = fmaxf(v[e], 0.f);
    }
}

/* final values of 32 consecutive columns of one row, straight from registers: 16-byte
   vectors where the row allows it, element by element at a ragged edge or for rows that
   are not 16-byte aligned */
template <typename OutT>
__device__ __forceinline__ void StoreRow32Direct(OutT * cRow, int c0, const float * v, const TcParams & p)
{
    constexpr int VN = Vec16<OutT>::N;
#pragma unroll
    for (int g = 0; g < 32 / VN; g++) {
        const int c = c0 + g * VN;
        const float * vv = v + g * VN;
        if (p.cVec && c + VN <= p.N) {
            StoreVec(cRow + c, vv);
        }
        else {
#pragma unroll
            for (int e = 0; e < VN; e++)
                if (c + e < p.N)
                    StoreOne(cRow + c + e, vv[e]);
        }
    }
}

/*
 * Per-warp writer of output tiles. When C allows it (16-byte aligned base and pitches)
 * the 32 rows x 128 bytes a warp produces are staged in shared memory in the 128-byte
 * swizzled layout (conflict-free for one-row-per-lane writes) and sent to HBM by one TMA
 * store per box: full 128-byte lines, asynchronous, clipped by TMA at the ragged edges of
 * C. Two boxes per warp alternate; before a box is refilled the warp waits until the store
 * that last used it has read it. Otherwise values go out with direct stores.
 *
 * With beta != 0 and tiles of at most two boxes per warp (128 half columns) the old values
 * of C come the same way in the other direction: a TMA load brings each box into the
 * staging buffer that will hold its result, requested when the tile is announced
 * (BeginTile), before the accumulator is waited for, so it arrives under the main loop.
 * One row per lane straight from global memory touches 32 lines per instruction and waits
 * for each 32-column piece in turn; that is what wider tiles still do, after BeginTile
 * has asked L2 to fetch the tile.
 */
constexpr int EPI_BOX_BYTES = 32 * ROW_BYTES;               /* 32 rows x 128 B */
constexpr int EPI_BYTES = 4 * 2 * EPI_BOX_BYTES;            /* four epilogue warps, two boxes each */

/* OLDC: the kernel was built for products that read the old C (beta != 0) or that also
   store their result to peer buffers; without it all of that support compiles away, which
   keeps the epilogue of the plain beta == 0 product short */
template <typename OutT, bool OLDC>
struct TileWriter {
    static constexpr int BOX_COLS = ROW_BYTES / (int)sizeof(OutT);   /* 64 halves / 32 floats */
    static constexpr int CHUNKS = 32 * (int)sizeof(OutT) / 16;      /* 16-byte chunks per 32 columns */
    uint32_t stage;          /* shared-memory address of this warp's two boxes */
    uint32_t boxes;          /* boxes handed to TMA so far */
    const CUtensorMap * map;
    uint32_t bars;           /* two mbarriers, one per box buffer, for the loads of old C values */
    uint32_t phase;          /* bit b: parity of the next wait on buffer b's barrier */
    volatile int * abortFlag;
    int * status;
    /* old-C fetch plan of the current tile: boxes 0 .. fTotal-1, fPerSub per 128-row sub-tile */
    bool fOn;
    int fRow0, fRowStep, fCol0, fPerSub, fTotal, fBatch;

    /* barPair: this warp's two mbarriers (initialised with count 1) */
    __device__ __forceinline__ void Init(uint32_t epiBase, int sub, const CUtensorMap * m, uint64_t * barPair,
                                         volatile int * abortPtr, int * statusPtr)
    {
        stage = epiBase + sub * 2 * EPI_BOX_BYTES;
        boxes = 0;
        map = m;
        bars = SmemAddr(barPair);
        phase = 0;
        abortFlag = abortPtr;
        status = statusPtr;
        fOn = false;
        fTotal = 0;
        oldCurOk = oldNxtOk = false;
    }

    /* Old C values of wide tiles (beta != 0, half output): every lane keeps the 64 columns
       of its row that the next chunk needs in registers, requested one chunk ahead (the
       first chunk of a tile before the accumulator is waited for), so the memory latency
       of one chunk runs under the work on the chunk before it. */
    static constexpr bool OLD_REGS = OLDC && sizeof(OutT) == 2;
    uint4 oldCur[OLD_REGS ? 8 : 1], oldNxt[OLD_REGS ? 8 : 1];
    bool oldCurOk, oldNxtOk;

    __device__ __forceinline__ void OldRequest(const TcParams & p, const OutT * cRow, int c0, bool rowOk)
    {
        oldNxtOk = false;
        if (!OLD_REGS)
            return;
        oldNxtOk = !fOn && p.beta != 0.f && p.cVec && rowOk && c0 + 64 <= p.N;
        if (oldNxtOk) {
#pragma unroll
            for (int j = 0; j < (OLD_REGS ? 8 : 1); j++)
                oldNxt[j] = *(const uint4 *)(cRow + c0 + j * 8);
        }
    }

    __device__ __forceinline__ void OldAdvance()
    {
#pragma unroll
        for (int j = 0; j < (OLD_REGS ? 8 : 1); j++)
            oldCur[j] = oldNxt[j];
        oldCurOk = oldNxtOk;
        oldNxtOk = false;
    }

    /* v <- alpha * v + beta * old for the 32 columns whose old values sit in o[0..3] */
    __device__ __forceinline__ void CombineOld32(const TcParams & p, const uint4 * o, float * v)
    {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float2 f;
            f = __half22float2(*(const __half2 *)&o[j].x);
            v[j * 8 + 0] = fmaf(p.beta, f.x, p.alpha * v[j * 8 + 0]); v[j * 8 + 1] = fmaf(p.beta, f.y, p.alpha * v[j * 8 + 1]);
            f = __half22float2(*(const __half2 *)&o[j].y);
            v[j * 8 + 2] = fmaf(p.beta, f.x, p.alpha * v[j * 8 + 2]); v[j * 8 + 3] = fmaf(p.beta, f.y, p.alpha * v[j * 8 + 3]);
            f = __half22float2(*(const __half2 *)&o[j].z);
            v[j * 8 + 4] = fmaf(p.beta, f.x, p.alpha * v[j * 8 + 4]); v[j * 8 + 5] = fmaf(p.beta, f.y, p.alpha * v[j * 8 + 5]);
            f = __half22float2(*(const __half2 *)&o[j].w);
            v[j * 8 + 6] = fmaf(p.beta, f.x, p.alpha * v[j * 8 + 6]); v[j * 8 + 7] = fmaf(p.beta, f.y, p.alpha * v[j * 8 + 7]);
        }
    }

    /* lane 0: request old C values of box k of the current tile into buffer bufIdx */
    __device__ __forceinline__ void FetchBox(const TcParams & p, int k, uint32_t bufIdx)
    {
        const int sub = k >= fPerSub ? 1 : 0;
        const int row0 = fRow0 + sub * fRowStep;
        const int col = fCol0 + (k - sub * fPerSub) * BOX_COLS;
        if (row0 < p.M) {
            const uint32_t bar = bars + bufIdx * 8;
            MbarExpectTx(bar, EPI_BOX_BYTES);
            TmaLoad3D(stage + bufIdx * EPI_BOX_BYTES, map, bar, col, row0, fBatch);
        }
    }

    /* Announces the next tile of this warp: nSub (1 or 2) sub-tiles of 32 rows starting at
       row0 and row0 + rowStep, columns col0 .. col0 + cols - 1 (col0 on a box boundary),
       visited sub-tile by sub-tile, left to right; cLane points at column col0 of row
       row0 + lane. Call it before waiting for the accumulator. */
    __device__ __forceinline__ void BeginTile(const TcParams & p, const OutT * cLane, int row0, int rowStep, int nSub,
                                              int col0, int cols, int batch, int lane)
    {
        fOn = false;
        if (!OLDC || !p.cTma || p.beta == 0.f)
            return;
        int live = p.N - col0 < cols ? p.N - col0 : cols;
        fPerSub = live > 0 ? (live + BOX_COLS - 1) / BOX_COLS : 0;
        fTotal = fPerSub * nSub;
        fRow0 = row0; fRowStep = rowStep; fCol0 = col0; fBatch = batch;
        if (fTotal > 2) {
            /* more boxes than staging buffers: a later box could only be requested after the
               store two boxes earlier has left its buffer, and that store queues in the TMA
               unit behind the next tile's operand loads. Such tiles read old C directly;
               here it is only pulled into L2. */
            if (p.cPrefetch == 1 && lane == 0) {
                for (int k = 0; k < fTotal; k++) {
                    const int sub = k >= fPerSub ? 1 : 0;
                    if (fRow0 + sub * fRowStep < p.M)
                        TmaPrefetch3D(map, fCol0 + (k - sub * fPerSub) * BOX_COLS, fRow0 + sub * fRowStep, fBatch);
                }
            }
            if (p.cPrefetch == 2) {
                /* every lane asks for the lines of its own rows */
                for (int sub = 0; sub < nSub; sub++) {
                    if (row0 + sub * rowStep + lane < p.M) {
                        const char * line = (const char *)(cLane + (long long)sub * rowStep * p.ldc);
                        for (int b = 0; b < live * (int)sizeof(OutT); b += 128)
                            asm volatile("prefetch.global.L2 [%0];" :: "l"(line + b));
                    }
                }
            }
            return;
        }
        fOn = true;
        if (lane == 0 && fTotal > 0) {
            /* every earlier store has read its buffer */
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            for (int k = 0; k < fTotal; k++)
                FetchBox(p, k, (boxes + (uint32_t)k) & 1u);
        }
    }

    /* v: raw accumulators of columns c0 .. c0+31 of this lane's row (row = row0 + lane) */
    __device__ __forceinline__ void Put32(const TcParams & p, OutT * cRow, bool rowOk, int row0, int c0,
                                          int batch, float * v, int lane)
    {
        const bool fromRegs = OLD_REGS && oldCurOk;       /* old values of this chunk are in oldCur */
        if (fromRegs) {
            if (c0 & 32)
                CombineOld32(p, oldCur + (OLD_REGS ? 4 : 0), v);
            else
                CombineOld32(p, oldCur, v);
        }
        if (!p.cTma) {
            ScaleRow32(cRow, c0, rowOk, v, p, fromRegs);
            if (rowOk)
                StoreRow32Direct(cRow, c0, v, p);
            return;
        }
        const int colInBox = c0 % BOX_COLS;
        const uint32_t bufIdx = boxes & 1u;
        const uint32_t box = stage + bufIdx * EPI_BOX_BYTES;
        const bool live = row0 < p.M;             /* uniform across the warp */
        if (colInBox == 0) {
            if (fOn) {
                /* the old values of this box were requested into this buffer */
                if (live) {
                    MbarWait(bars + bufIdx * 8, (phase >> bufIdx) & 1u, abortFlag, status, 20);
                    phase ^= 1u << bufIdx;
                }
                else {
                    __syncwarp();                 /* lane 0 has waited for the last reader of this buffer */
                }
            }
            else {
                /* the store that used this box two boxes ago must have read it */
                if (lane == 0 && boxes >= 2)
                    asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                __syncwarp();
            }
        }
        const uint32_t rowAddr = box + lane * ROW_BYTES;
        const int firstChunk = colInBox * (int)sizeof(OutT) / 16;
        if (fOn && live) {
            /* alpha * v + beta * old, the old values read from where the result will go */
#pragma unroll
            for (int j = 0; j < CHUNKS; j++) {
                const uint32_t src = rowAddr + (uint32_t)(((firstChunk + j) ^ (lane & 7)) << 4);
                uint32_t w0, w1, w2, w3;
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3) : "r"(src) : "memory");
                if (sizeof(OutT) == 2) {
                    float2 f;
                    f = __half22float2(*(__half2 *)&w0);
                    v[j * 8 + 0] = fmaf(p.beta, f.x, p.alpha * v[j * 8 + 0]); v[j * 8 + 1] = fmaf(p.beta, f.y, p.alpha * v[j * 8 + 1]);
                    f = __half22float2(*(__half2 *)&w1);
                    v[j * 8 + 2] = fmaf(p.beta, f.x, p.alpha * v[j * 8 + 2]); v[j * 8 + 3] = fmaf(p.beta, f.y, p.alpha * v[j * 8 + 3]);
                    f = __half22float2(*(__half2 *)&w2);
                    v[j * 8 + 4] = fmaf(p.beta, f.x, p.alpha * v[j * 8 + 4]); v[j * 8 + 5] = fmaf(p.beta, f.y, p.alpha * v[j * 8 + 5]);
                    f = __half22float2(*(__half2 *)&w3);
                    v[j * 8 + 6] = fmaf(p.beta, f.x, p.alpha * v[j * 8 + 6]); v[j * 8 + 7] = fmaf(p.beta, f.y, p.alpha * v[j * 8 + 7]);
                }
                else {
                    v[j * 4 + 0] = fmaf(p.beta, __uint_as_float(w0), p.alpha * v[j * 4 + 0]);
                    v[j * 4 + 1] = fmaf(p.beta, __uint_as_float(w1), p.alpha * v[j * 4 + 1]);
                    v[j * 4 + 2] = fmaf(p.beta, __uint_as_float(w2), p.alpha * v[j * 4 + 2]);
                    v[j * 4 + 3] = fmaf(p.beta, __uint_as_float(w3), p.alpha * v[j * 4 + 3]);
                }
            }
            ScaleRow32(cRow, c0, rowOk, v, p, true);
        }
        else {
            ScaleRow32(cRow, c0, rowOk, v, p, fromRegs);
        }
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) {
            const uint32_t dst = rowAddr + (uint32_t)(((firstChunk + j) ^ (lane & 7)) << 4);
            uint32_t w0, w1, w2, w3;
            if (sizeof(OutT) == 2) {
                __half2 h0 = __floats2half2_rn(v[j * 8 + 0], v[j * 8 + 1]);
                __half2 h1 = __floats2half2_rn(v[j * 8 + 2], v[j * 8 + 3]);
                __half2 h2 = __floats2half2_rn(v[j * 8 + 4], v[j * 8 + 5]);
                __half2 h3 = __floats2half2_rn(v[j * 8 + 6], v[j * 8 + 7]);
                w0 = *(uint32_t *)&h0; w1 = *(uint32_t *)&h1; w2 = *(uint32_t *)&h2; w3 = *(uint32_t *)&h3;
            }
            else {
                w0 = __float_as_uint(v[j * 4 + 0]); w1 = __float_as_uint(v[j * 4 + 1]);
                w2 = __float_as_uint(v[j * 4 + 2]); w3 = __float_as_uint(v[j * 4 + 3]);
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" :: "r"(dst), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
        }
        if (colInBox + 32 == BOX_COLS || c0 + 32 >= p.N) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0 && row0 < p.M) {
                asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                             :: "l"(map), "r"(c0 - colInBox), "r"(row0), "r"(batch), "r"(box) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            if (OLDC && p.nPeers > 0 && live)
                BoxToPeers(p, cRow - (long long)lane * p.ldc, box, row0, c0 - colInBox, lane);
            boxes++;
        }
    }

    /* The finished box (32 rows x 128 bytes, swizzled in shared memory) goes to the same
       place of every peer buffer with plain 16-byte stores: eight lanes cover the 128 bytes
       of one row, so a warp instruction writes four full lines. cBox0 points at row row0,
       column 0 of this problem's C. */
    __device__ __forceinline__ void BoxToPeers(const TcParams & p, const OutT * cBox0, uint32_t box, int row0, int col0,
                                               int lane)
    {
        constexpr int VN = Vec16<OutT>::N;
        const long long base = cBox0 - (const OutT *)p.c;          /* element offset of (row0, 0) in C */
        const int chunk = lane & 7;
        const int col = col0 + chunk * VN;
#pragma unroll
        for (int r = 0; r < 8; r++) {
            const int rr = r * 4 + (lane >> 3);
            uint32_t w0, w1, w2, w3;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3)
                         : "r"(box + (uint32_t)rr * ROW_BYTES + (uint32_t)((chunk ^ (rr & 7)) << 4)) : "memory");
            if (row0 + rr < p.M && col + VN <= p.N) {
                const long long off = base + (long long)rr * p.ldc + col;
                for (int k = 0; k < p.nPeers; k++)
                    *(uint4 *)((OutT *)p.peers[k] + off) = make_uint4(w0, w1, w2, w3);
            }
            else if (row0 + rr < p.M) {
                const uint32_t w[4] = { w0, w1, w2, w3 };          /* ragged right edge: element by element */
                const OutT * e = (const OutT *)w;
                for (int j = 0; j < VN; j++)
                    if (col + j < p.N) {
                        const long long off = base + (long long)rr * p.ldc + col + j;
                        for (int k = 0; k < p.nPeers; k++)
                            ((OutT *)p.peers[k])[off] = e[j];
                    }
            }
        }
    }

    /* all of this warp's stores have read their staging boxes, so shared memory may go
       away; the writes themselves complete before the grid does */
    __device__ __forceinline__ void Finish(int lane)
    {
        if (lane == 0)
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
    }
};

/* ---------------------------------------------------------------- tile walk */

struct TileCoord {
    int prob, mBlk, nBlk;
};

/* Tiles of one problem are visited in bands of `GROUP` m-blocks, n fastest inside a band's
   column, so the CTAs running at the same time share A row panels and B column panels
   in L2. */
__device__ __forceinline__ TileCoord DecodeTile(int t, const TcParams & p)
{
    TileCoord tc;
    uint32_t prob, r, band, inBand, q, rem;
    p.fdPerProb.DivMod((uint32_t)t, prob, r);
    p.fdBand.DivMod(r, band, inBand);
    const int first = (int)band * p.group;
    if (p.tilesM - first >= p.group)
        p.fdGroup.DivMod(inBand, q, rem);
    else
        p.fdLast.DivMod(inBand, q, rem);
    tc.prob = (int)prob;
    tc.mBlk = first + (int)rem;
    tc.nBlk = (int)q;
    return tc;
}

/* (p, q) = (prob / Q, prob % Q) */
__device__ __forceinline__ void SplitProb(const TcParams & p, int prob, int & pp, int & qq)
{
    uint32_t a, b;
    p.fdQ.DivMod((uint32_t)prob, a, b);
    pp = (int)a;
    qq = (int)b;
}

__device__ __forceinline__ int BatchCoord(int sel, int prob, const TcParams & p)
{
    if (sel == 0)
        return 0;
    if (sel == 3)
        return prob;
    int pp, qq;
    SplitProb(p, prob, pp, qq);
    return sel == 1 ? pp : qq;
}

/* ---------------------------------------------------------------- the kernel */

/* Up to two problems of different shapes in one launch (the two gradient products of a
   matrix multiplication): tiles [0, split) belong to problem 0, the rest to problem 1. */
struct TcGroup {
    CUtensorMap tm[2][3];      /* A, B, C maps of each problem */
    TcParams p[2];
    int n, split, total;
};

/* per-tile view of the problem a tile belongs to; names match the single-problem code */
#define NTB_SELECT_PROBLEM() \
    const int gi = t >= grp.split ? 1 : 0; \
    const TcParams & p = grp.p[gi]; \
    const CUtensorMap & tmA = grp.tm[gi][0]; \
    const CUtensorMap & tmB = grp.tm[gi][1]; \
    const CUtensorMap & tmC = grp.tm[gi][2]; \
    (void)tmA; (void)tmB; (void)tmC; \
    const int tl = t - gi * grp.split; \
    const int kBlocks = (p.K + EPR - 1) / EPR; \
    /* k-blocks accumulated in TMEM before the partial sum is handed to the epilogue */ \
    const int chunkBlocks = MODE == 0 ? kBlocks : FP32_CHUNK_BLOCKS; \
    (void)chunkBlocks

template <int MODE, int BN, int STAGES, int G, typename OutT, bool OLDC>
__global__ void __launch_bounds__(MODE == 0 ? 192 : 192 + CONV_THREADS, 1)
GemmTcKernel(const __grid_constant__ TcGroup grp)
{
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
        int touch = grp.total + grp.split;
        for (int gi = 0; gi < grp.n; gi++) {
            const TcParams & p = grp.p[gi];
            if (threadIdx.x == 128) {
                PrefetchTensorMap(&grp.tm[gi][0]);
                PrefetchTensorMap(&grp.tm[gi][1]);
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
            MbarInit(SmemAddr(&barFull[lane]), 1);
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
        if (lane == 0) {
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
                        if (j < nb) {
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
    else if (MODE != 0) {
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
                /* make the generic-proxy stores visible to the tensor core's async-proxy reads */
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                MbarArrive(SmemAddr(&barConv[s]));
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

/* ---------------------------------------------------------------- the CTA-pair kernel */

__device__ __forceinline__ uint32_t ClusterCtaRank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

/* address of the same shared-memory object in the CTA of rank `rank` of this cluster */
__device__ __forceinline__ uint32_t MapToCta(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}

__device__ __forceinline__ void MbarArriveCluster(uint32_t clusterAddr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(clusterAddr) : "memory");
}

__device__ __forceinline__ void ClusterSync()
{
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}

/* L2 eviction policy for a stream of loads: 1 keep (evict last), 2 stream (evict first) */
__device__ __forceinline__ uint64_t L2Policy(int kind)
{
    uint64_t pol = 0;
    if (kind == 1)
        asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    else if (kind == 2)
        asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

/* the pair load with an L2 eviction policy */
__device__ __forceinline__ void TmaLoad3DPairHint(uint32_t dst, const CUtensorMap * map, uint32_t barCluster, int c0, int c1,
                                                  int c2, uint64_t policy)
{
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
                 " [%0], [%1, {%3, %4, %5}], [%2], %6;"
                 :: "r"(dst), "l"(map), "r"(barCluster), "r"(c0), "r"(c1), "r"(c2), "l"(policy) : "memory");
}

/* TMA load whose completion bytes are counted on a barrier of the pair's leader CTA */
__device__ __forceinline__ void TmaLoad3DPair(uint32_t dst, const CUtensorMap * map, uint32_t barCluster, int c0, int c1, int c2)
{
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4, %5}], [%2];"
                 :: "r"(dst), "l"(map), "r"(barCluster), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

__device__ __forceinline__ void TcMmaPairLH(uint32_t dTmem, uint32_t aLo, uint32_t aHi, uint32_t bLo, uint32_t bHi,
                                            uint32_t iDesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\t"
                 "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}"
                 :: "r"(dTmem), "r"(aLo), "r"(aHi), "r"(bLo), "r"(bHi), "r"(iDesc), "r"(accumulate) : "memory");
}

/* arrive, once the MMAs issued so far have finished, on the barrier at this offset in
   both CTAs of the pair */
__device__ __forceinline__ void TcCommitPair(uint32_t bar)
{
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 :: "r"(bar), "h"(mask) : "memory");
}

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
template <int MSUB, int BN, int STAGES, int G, typename OutT, bool OLDC>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
GemmTcPairKernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, TcParams p)
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

    extern __shared__ uint8_t smemRaw[];
    __shared__ __align__(8) uint64_t barFull[STAGES];
    __shared__ __align__(8) uint64_t barEmpty[STAGES];
    __shared__ __align__(8) uint64_t barTFull[2];
    __shared__ __align__(8) uint64_t barTEmpty[2];
    __shared__ __align__(8) uint64_t barOldC[8];    /* per epilogue warp and staging box: old C values have landed */
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
            MbarInit(SmemAddr(&barTEmpty[lane - 8]), 8);
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
                        if (j < nb) {
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
        const int sub32 = warp & 3;
        uint32_t it = 0;
        bool ok = true;
        TileWriter<OutT, OLDC> writer;
        writer.Init(smemBase + STAGES * STAGE_BYTES, sub32, &tmC, &barOldC[sub32 * 2], abortPtr, p.status);
        for (int t = firstTile; ok && t < p.totalTiles; t += tileStep, ++it) {
            TileCoord tc = DecodeTile(t, p);
            const int n0 = tc.nBlk * BN;
            int pp, qq;
            SplitProb(p, tc.prob, pp, qq);
            const int bc = BatchCoord(p.cSel, tc.prob, p);
            OutT * cBase = (OutT *)p.c + pp * p.sCp + qq * p.sCq;
            const uint32_t buf = it % NBUF;
            writer.BeginTile(p, cBase + (long long)(tc.mBlk * PM + (int)rank * BM + sub32 * 32 + lane) * p.ldc + n0,
                             tc.mBlk * PM + (int)rank * BM + sub32 * 32, 2 * BM, MSUB, n0, BN, bc, lane);
            {
                const int r0 = tc.mBlk * PM + (int)rank * BM + sub32 * 32 + lane;
                writer.OldRequest(p, cBase + (long long)r0 * p.ldc, n0, r0 < p.M);
            }
            NTB_TIMED(3, ok = MbarWaitWarp(SmemAddr(&barTFull[buf]), (it / NBUF) & 1u, abortPtr, p.status, (uint32_t)p.epiHint));
            if (!ok)
                break;
            TcFenceAfter();
#pragma unroll 1
            for (int sub = 0; sub < MSUB; sub++) {
                const int row0 = tc.mBlk * PM + sub * 2 * BM + (int)rank * BM + sub32 * 32;
                const int row = row0 + lane;
                OutT * cRow = cBase + (long long)row * p.ldc;
                const bool rowOk = row < p.M;
                const uint32_t tRow = tmemBase + ((uint32_t)(sub32 * 32) << 16) + buf * (MSUB * BN) + sub * BN;
#pragma unroll 1
                for (int ch = 0; ch < BN / 64; ch++) {
                    const int c0 = n0 + ch * 64;
                    if (c0 >= p.N)
                        break;
                    writer.OldAdvance();
                    if (ch + 1 < BN / 64 && c0 + 64 < p.N)
                        writer.OldRequest(p, cRow, c0 + 64, rowOk);
                    else if (sub + 1 < MSUB)
                        writer.OldRequest(p, cRow + (long long)(2 * BM) * p.ldc, n0, row + 2 * BM < p.M);
                    float v[64];
                    TmemLoad64(tRow + ch * 64, v);
                    writer.Put32(p, cRow, rowOk, row0, c0, bc, v, lane);
                    if (c0 + 32 < p.N)
                        writer.Put32(p, cRow, rowOk, row0, c0 + 32, bc, v + 32, lane);
                }
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

/* ---------------------------------------------------------------- the split-K kernel */

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
                if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
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

/* ---------------------------------------------------------------- host side */

/* offset of operand x for problem i is idx * stride with idx in {p, q, i}; find which */
bool BatchSelector(long long sp, long long sq, int P, int Q, int * sel, long long * stride, int * extent)
{
    if (sp == 0 && sq == 0) { *sel = 0; *stride = 0; *extent = 1; return true; }
    if (sq == 0 || Q == 1)  { *sel = 1; *stride = sp; *extent = P; if (sp == 0) { *sel = 0; *extent = 1; } return true; }
    if (sp == 0 || P == 1)  { *sel = 2; *stride = sq; *extent = Q; return true; }
    if (sp == sq * Q)       { *sel = 3; *stride = sq; *extent = P * Q; return true; }
    return false;
}

/* integer tuning knob from the environment, read at every launch */
int Knob(const char * name, int dflt)
{
    const char * v = getenv(name);
    return v && *v ? atoi(v) : dflt;
}

template <int MODE, int BN, int STAGES, int G, typename OutT, bool OLDC>
int LaunchOne(const TcGroup & grp, int smCount, cudaStream_t stream)
{
    constexpr int stage = (A_TILE_BYTES + BN * ROW_BYTES) * (MODE == 0 ? 1 : 2);
    constexpr int smem = stage * STAGES + EPI_BYTES + 1024;
    auto kern = GemmTcKernel<MODE, BN, STAGES, G, OutT, OLDC>;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return NTB_ERR_CUDA;
        configured[dev] = true;
    }
    const int grid = grp.total < smCount ? grp.total : smCount;
    const cudaError_t err = LaunchPdl(kern, grid, MODE == 0 ? 192 : 192 + CONV_THREADS, smem, stream, grp);
    CountLaunch();
    return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? NTB_OK : NTB_ERR_CUDA;
}

template <int S, int STAGES, int G, typename OutT, bool OLDC>
int LaunchSplit(const CUtensorMap & tmA, const CUtensorMap & tmB, const CUtensorMap & tmC, const TcParams & tp, int clusters,
                cudaStream_t stream)
{
    constexpr int smem = (A_TILE_BYTES + 128 * ROW_BYTES) * STAGES + 2 * (S - 1) * (BM * (128 / S) * 4) + EPI_BYTES + 1024;
    auto kern = GemmTcSplitKernel<S, STAGES, G, OutT, OLDC>;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return NTB_ERR_CUDA;
        configured[dev] = true;
    }
    const cudaError_t err = LaunchPdl(kern, S * clusters, 192, smem, stream, tmA, tmB, tmC, tp);
    CountLaunch();
    return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? NTB_OK : NTB_ERR_CUDA;
}


/* single-CTA kernel for a group, chosen by operand mode, tile width and output type */
int LaunchGroup(const TcGroup & grp, int mode, int bn, int dtC, int smCount, cudaStream_t stream)
{
    /* kernels built with support for reading the old C only where a product asks for it */
    const bool oldc = grp.p[0].beta != 0.f || grp.p[0].nPeers > 0 || (grp.n > 1 && (grp.p[1].beta != 0.f || grp.p[1].nPeers > 0));
#define NTB_ONE(MD, W, ST, GG, T) (oldc ? LaunchOne<MD, W, ST, GG, T, true>(grp, smCount, stream) \
                                        : LaunchOne<MD, W, ST, GG, T, false>(grp, smCount, stream))
    if (mode == 0) {
        const bool half = dtC == NTB_X_FLOAT16;
        /* k-blocks per barrier hand-shake: two, except for the widest tile, whose four MMAs
           already cover a hand-shake (NTB_GROUP_K = 1 asks for one everywhere) */
        const int g = Knob("NTB_GROUP_K", 0);
        if (bn == 256)
            return half ? NTB_ONE(0, 256, 4, 1, __half) : NTB_ONE(0, 256, 4, 1, float);
        if (bn == 128) {
            if (g == 1)
                return half ? NTB_ONE(0, 128, 6, 1, __half) : NTB_ONE(0, 128, 6, 1, float);
            return half ? NTB_ONE(0, 128, 6, 2, __half) : NTB_ONE(0, 128, 6, 2, float);
        }
        if (g == 1)
            return half ? NTB_ONE(0, 64, 8, 1, __half) : NTB_ONE(0, 64, 8, 1, float);
        return half ? NTB_ONE(0, 64, 8, 2, __half) : NTB_ONE(0, 64, 8, 2, float);
    }
    if (bn == 128)
        return NTB_ONE(1, 128, 3, 1, float);
    return NTB_ONE(1, 64, 4, 1, float);
#undef NTB_ONE
}

template <int MSUB, int BN, int STAGES, int G, typename OutT, bool OLDC>
int LaunchPair(const CUtensorMap & tmA, const CUtensorMap & tmB, const CUtensorMap & tmC, const TcParams & tp, int pairs,
               cudaStream_t stream)
{
    constexpr int smem = (MSUB * A_TILE_BYTES + (BN / 2) * ROW_BYTES) * STAGES + EPI_BYTES + 1024;
    auto kern = GemmTcPairKernel<MSUB, BN, STAGES, G, OutT, OLDC>;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return NTB_ERR_CUDA;
        configured[dev] = true;
    }
    const cudaError_t err = LaunchPdl(kern, 2 * pairs, 192, smem, stream, tmA, tmB, tmC, tp);
    CountLaunch();
    return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? NTB_OK : NTB_ERR_CUDA;
}

int EncodeOperand(CUtensorMap * map, int mode, const void * base, int mnMajor, int rows, int cols,
                  long long ld, long long batchStride, int batchExtent, int tileRows)
{
    EncodeTiledFn enc = GetEncodeTiled();
    if (!enc)
        return NTB_ERR_CUDA;
    const int es = mode == 0 ? 2 : 4;
    const int epr = ROW_BYTES / es;
    cuuint64_t dims[3] = { (cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batchExtent };
    cuuint64_t strides[2] = { (cuuint64_t)ld * es,
                              (cuuint64_t)(batchExtent > 1 ? batchStride : (long long)rows * ld) * es };
    /* K-major: the stored row is K -> box = 128 bytes of K x tileRows rows.
       MN-major: the stored row is M (or N) -> box = 128 bytes of MN x one stage of K rows. */
    cuuint32_t box[3] = { (cuuint32_t)epr, (cuuint32_t)(mnMajor ? epr : tileRows), 1 };
    cuuint32_t estr[3] = { 1, 1, 1 };
    const int promo = Knob("NTB_L2_PROMOTION", 3);   /* tuning: L2 fetch granularity of operand loads */
    CUresult r = enc(map, mode == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                     3, (void *)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     (mode != 0 && mnMajor) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                     promo == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE : promo == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                     : promo == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? NTB_OK : NTB_ERR_CUDA;
}

/* tensor map of C for the epilogue's stores: boxes of 32 rows x 128 bytes, 128-byte swizzle */
int EncodeOutput(CUtensorMap * map, int dtC, void * base, int rows, int cols, long long ld,
                 long long batchStride, int batchExtent)
{
    EncodeTiledFn enc = GetEncodeTiled();
    if (!enc)
        return NTB_ERR_CUDA;
    const int es = dtC == NTB_X_FLOAT16 ? 2 : 4;
    cuuint64_t dims[3] = { (cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batchExtent };
    cuuint64_t strides[2] = { (cuuint64_t)ld * es,
                              (cuuint64_t)(batchExtent > 1 ? batchStride : (long long)rows * ld) * es };
    cuuint32_t box[3] = { (cuuint32_t)(ROW_BYTES / es), 32, 1 };
    cuuint32_t estr[3] = { 1, 1, 1 };
    CUresult r = enc(map, dtC == NTB_X_FLOAT16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                     3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? NTB_OK : NTB_ERR_CUDA;
}

/*
 * Cost model for the tile shape, in SM clocks: waves x (k-blocks x clocks per k-block +
 * cost of starting and finishing one tile). A k-block costs the largest of
 *   - its MMA time;
 *   - the time its operand bytes take to arrive: an SM takes in about 62 bytes per clock,
 *     and all SMs together about 5800 (what the L2-to-SM fabric delivered to TMA loads in
 *     every kernel timed here), so the more CTAs run, the less each one gets;
 *   - the time of the thread that issues the MMAs: about 47 clocks per instruction plus
 *     about 400 (500 in a CTA pair) per barrier hand-shake, shared by the k-blocks of a group;
 *   - its shared-memory traffic at 128 bytes per clock: the bytes TMA writes plus the operand
 *     bytes every MMA reads back (a 128 x 128 tile reads 8 KB per 64 clocks of math and is
 *     bound by this at half the MMA rate).
 * Returns the tile width of the single-CTA kernel; 0 / -1 for the CTA-pair kernel with
 * 256 x 256 / 512 x 256 tiles, -8 / -9 for pair tiles of 256 x 128 / 512 x 128; -2 / -4 for
 * the split-K kernel with clusters of 2 / 4 CTAs. Constants were fitted to timings of the
 * benchmark configurations and of mid-size products on a B200.
 */
struct KbCost {
    double math, bytes, reads, mmas, shake;   /* reads: operand bytes the MMAs fetch from shared memory */
    int g;
};

double PerKBlock(const KbCost & c, long long activeCtas)
{
    const double perSm = 62.0, fabric = 5800.0;
    const double ingest = fmin(perSm, fabric / (double)(activeCtas > 0 ? activeCtas : 1));
    const double thread = (c.shake + 47.0 * c.mmas * c.g) / c.g;
    const double smem = (c.bytes + c.reads) / 128.0;  /* TMA writes and operand reads share 128 bytes per clock */
    return fmax(fmax(c.math, smem), fmax(c.bytes / ingest, thread));
}

int PickBN(const Problem & p, int smCount, int mode)
{
    const int es = mode == 0 ? 2 : 4;
    const int kElems = ROW_BYTES / es;
    const double kBlocks = (double)((p.K + kElems - 1) / kElems);
    const double mmaPerCol = mode == 0 ? 2.0 : 6.0;   /* clocks per k-block per output column (3 passes at half rate for fp32) */
    int best = 128;
    double bestCost = 1e300;
    const int cand[3] = { 256, 128, 64 };
    for (int i = (mode == 0 ? 0 : 1); i < 3; i++) {
        const int bn = cand[i];
        const long long tiles = (long long)((p.M + BM - 1) / BM) * ((p.N + bn - 1) / bn) * p.count;
        const long long waves = (tiles + smCount - 1) / smCount;
        KbCost c;
        c.math = mmaPerCol * bn;
        c.bytes = (double)(BM + bn) * ROW_BYTES;
        /* fp32: three MMAs per k-step read both planes, and the splitter reads and writes a plane */
        c.reads = mode == 0 ? c.bytes : 5.0 * c.bytes;
        c.mmas = mode == 0 ? 4.0 : 12.0;
        c.shake = 400.0;
        c.g = (mode == 0 && bn != 256) ? 2 : 1;
        const double perK = PerKBlock(c, tiles < smCount ? tiles : smCount);
        const double cost = (double)waves * (kBlocks * perK + 1500.0 + 4.0 * bn);
        if (cost < bestCost) { bestCost = cost; best = bn; }
    }
    if (mode == 0 && smCount >= 2) {
        const long long pairs = smCount / 2;
        for (int w = 256; w >= 128; w -= 128) {
            for (int msub = 1; msub <= 2; msub++) {
                const int pm = 2 * BM * msub;
                const long long tiles = (long long)((p.M + pm - 1) / pm) * ((p.N + w - 1) / w) * p.count;
                const long long waves = (tiles + pairs - 1) / pairs;
                KbCost c;
                c.math = 2.0 * w * msub;
                c.bytes = (double)(msub * BM + w / 2) * ROW_BYTES;
                c.reads = (double)msub * (BM + w / 2) * ROW_BYTES;
                c.mmas = 4.0 * msub;
                c.shake = 500.0;
                c.g = w == 256 ? 1 : 2;
                const double perK = PerKBlock(c, 2 * (tiles < pairs ? tiles : pairs));
                /* the second accumulator set of the 512-row tile is not double-buffered: its
                   epilogue is exposed; pairs also pay for cluster start-up and hand-shakes */
                const double perTile = (w == 256 ? 2524.0 : 1700.0) * msub + (msub == 2 ? (w == 256 ? 6000.0 : 3000.0) : 0.0);
                const double cost = (double)waves * (kBlocks * perK + perTile) + 2000.0;
                if (cost < bestCost) { bestCost = cost; best = (msub == 1 ? 0 : -1) - (w == 128 ? 8 : 0); }
            }
        }
    }
    if (mode == 0) {
        /* split-K clusters: S CTAs share a 128 x 128 tile and a 1/S part of K each, then
           exchange partial sums through distributed shared memory */
        for (int sp = 2; sp <= 4; sp *= 2) {
            if (kBlocks < 4.0 * sp || smCount < sp)
                continue;
            const long long tiles = (long long)((p.M + BM - 1) / BM) * ((p.N + 127) / 128) * p.count;
            const long long clusters = smCount / sp;
            const long long waves = (tiles + clusters - 1) / clusters;
            KbCost c;
            c.math = 256.0;
            c.bytes = (double)(BM + 128) * ROW_BYTES;
            c.reads = c.bytes;
            c.mmas = 4.0;
            c.shake = 400.0;
            c.g = 1;
            const double perK = PerKBlock(c, sp * (tiles < clusters ? tiles : clusters));
            const double cost = (double)waves * (ceil(kBlocks / sp) * perK + 2012.0 + 2500.0) + 2000.0;
            if (cost < bestCost) { bestCost = cost; best = -sp; }
        }
    }
    return best;
}

}

bool TcEligible(const Problem & p)
{
    if (p.M <= 0 || p.N <= 0 || p.K <= 0 || p.count <= 0)
        return false;
    const bool f16 = p.dtAB == NTB_X_FLOAT16 && (p.dtC == NTB_X_FLOAT16 || p.dtC == NTB_X_FLOAT);
    const bool f32 = p.dtAB == NTB_X_FLOAT && p.dtC == NTB_X_FLOAT;
    if (!f16 && !f32)
        return false;
    const long long es = ElemSize(p.dtAB);
    if (((uintptr_t)p.a & 15) || ((uintptr_t)p.b & 15))
        return false;
    if ((p.lda * es) % 16 || (p.ldb * es) % 16)
        return false;
    if ((p.sAp * es) % 16 || (p.sAq * es) % 16 || (p.sBp * es) % 16 || (p.sBq * es) % 16)
        return false;
    if (p.lda < p.aCols || p.ldb < p.bCols)
        return false;
    int sel, ext;
    long long st;
    const int P = p.count / p.Q;
    if (!BatchSelector(p.sAp, p.sAq, P, p.Q, &sel, &st, &ext) || st < 0)
        return false;
    if (!BatchSelector(p.sBp, p.sBq, P, p.Q, &sel, &st, &ext) || st < 0)
        return false;
    return true;
}

namespace {

/* kernel parameters and tensor maps of one problem for tile width bn (pair: CTA-pair
   kernel with msub 128-row sub-tiles per CTA) */
int Prepare(const DeviceCtx & ctx, const Problem & p, int mode, int bn, bool pair, int msub,
            TcParams & tp, CUtensorMap * maps)
{
    const int P = p.count / p.Q;
    tp.c = p.c; tp.ldc = p.ldc; tp.sCp = p.sCp; tp.sCq = p.sCq;
    tp.M = p.M; tp.N = p.N; tp.K = p.K; tp.count = p.count; tp.Q = p.Q;
    tp.aMN = p.aMN; tp.bMN = p.bMN;
    tp.tilesM = pair ? (p.M + 2 * BM * msub - 1) / (2 * BM * msub) : (p.M + BM - 1) / BM;
    tp.tilesN = (p.N + bn - 1) / bn;
    const long long tiles64 = (long long)tp.tilesM * tp.tilesN * p.count;
    if (tiles64 > 1073741823LL)
        return NTB_ERR_LIMIT;
    tp.totalTiles = (int)tiles64;
    tp.alpha = p.alpha; tp.beta = p.beta;
    tp.bias = p.bias; tp.act = p.act;
    tp.nPeers = p.nPeers;
    for (int i = 0; i < NTB_MAX_PEERS; i++)
        tp.peers[i] = i < p.nPeers ? p.peers[i] : nullptr;
    tp.status = ctx.status;
    tp.pfDist = Knob("NTB_PREFETCH_DIST", 0);
    tp.group = Knob("NTB_TILE_GROUP", 8);
    if (tp.group < 1)
        tp.group = 1;
    tp.epiHint = Knob("NTB_EPI_HINT_NS", 2000);
    tp.cPrefetch = Knob("NTB_C_PREFETCH", 0);
    tp.l2Hint = Knob("NTB_L2_HINT", 0);
    tp.fdPerProb.Set((uint32_t)(tp.tilesM * tp.tilesN));
    tp.fdBand.Set((uint32_t)(tp.group * tp.tilesN));
    tp.fdGroup.Set((uint32_t)tp.group);
    tp.fdLast.Set((uint32_t)(tp.tilesM % tp.group ? tp.tilesM % tp.group : tp.group));
    tp.fdQ.Set((uint32_t)p.Q);
    const long long ces = ElemSize(p.dtC);
    tp.cVec = (((uintptr_t)p.c & 15) == 0) && ((p.ldc * ces) % 16 == 0) &&
              ((p.sCp * ces) % 16 == 0) && ((p.sCq * ces) % 16 == 0);

    long long stA = 0, stB = 0;
    int extA = 1, extB = 1;
    BatchSelector(p.sAp, p.sAq, P, p.Q, &tp.aSel, &stA, &extA);
    BatchSelector(p.sBp, p.sBq, P, p.Q, &tp.bSel, &stB, &extB);

    int rc = EncodeOperand(&maps[0], mode, p.a, p.aMN, p.aRows, p.aCols, p.lda, stA, extA, BM);
    if (rc != NTB_OK)
        return rc;
    rc = EncodeOperand(&maps[1], mode, p.b, p.bMN, p.bRows, p.bCols, p.ldb, stB, extB, pair ? bn / 2 : bn);
    if (rc != NTB_OK)
        return rc;

    /* C through TMA stores when its base, pitch and batch strides are 16-byte aligned and
       its batch offset is one index times one stride; otherwise direct stores */
    maps[2] = maps[0];
    long long stC = 0;
    int extC = 1;
    tp.cSel = 0;
    tp.cTma = tp.cVec && Knob("NTB_TMA_STORE", 1) != 0 && p.ldc >= p.N &&
              BatchSelector(p.sCp, p.sCq, P, p.Q, &tp.cSel, &stC, &extC) && stC >= 0;
    if (tp.cTma) {
        rc = EncodeOutput(&maps[2], p.dtC, p.c, p.M, p.N, p.ldc, stC, extC);
        if (rc != NTB_OK)
            return rc;
    }
    return NTB_OK;
}

}

int LaunchTc(const DeviceCtx & ctx, const Problem & p, cudaStream_t stream, int * route)
{
    const int mode = p.dtAB == NTB_X_FLOAT16 ? 0 : 1;
    int bn = PickBN(p, ctx.smCount, mode);
    const int forced = ForcedRoute();
    const int knobBN = Knob("NTB_BN", 0);           /* tuning: force the single-CTA tile width */
    if (knobBN == 64 || knobBN == 128 || (knobBN == 256 && mode == 0))
        bn = knobBN;
    const int knobSplit = Knob("NTB_SPLIT_K", -1);  /* tuning: 0 forbids, 2 / 4 force the split-K kernel */
    if (mode == 0 && (knobSplit == 2 || knobSplit == 4) && (p.K + 63) / 64 >= knobSplit && ctx.smCount >= knobSplit)
        bn = -knobSplit;
    const bool isSplit = bn == -2 || bn == -4;
    if (isSplit && (knobSplit == 0 || forced == NTB_ROUTE_TC_F16_PAIR)) {
        Problem q = p;
        q.K = 64;                                   /* too short to split: re-ask the model */
        bn = PickBN(q, ctx.smCount, mode);
    }
    if (mode == 0 && forced == NTB_ROUTE_TC_F16_PAIR && ctx.smCount >= 2 && bn > 0)
        bn = Knob("NTB_PAIR_MSUB", 2) == 1 ? 0 : -1;
    if ((bn == 0 || bn == -1 || bn == -8 || bn == -9) && forced == NTB_ROUTE_TC_F16)
        bn = 256;
    /* tuning: width of the pair tile (the model's choice otherwise) */
    const int knobPairBN = Knob("NTB_PAIR_BN", 0);
    if (knobPairBN == 128 && (bn == 0 || bn == -1))
        bn -= 8;
    if (knobPairBN == 256 && (bn == -8 || bn == -9))
        bn += 8;
    int split = (bn == -2 || bn == -4) ? -bn : 0;
    if (split == 4 && p.nPeers > 0 && p.dtC == NTB_X_FLOAT16)
        split = 2;                                  /* the 4-way split of a half tile stores directly */
    if (split)
        bn = 128;
    const bool pair = bn <= 0;
    const int msub = (bn == -1 || bn == -9) ? 2 : 1;
    if (pair)
        bn = bn <= -8 ? 128 : 256;
    *route = mode != 0 ? NTB_ROUTE_TC_3XTF32 : pair ? NTB_ROUTE_TC_F16_PAIR : NTB_ROUTE_TC_F16;
    if (Knob("NTB_DEBUG_CHOICE", 0))
        fprintf(stderr, "ntb: M %d N %d K %d count %d -> %s width %d msub %d split %d\n", p.M, p.N, p.K, p.count,
                pair ? "pair" : split ? "split-K" : "single", bn, msub, split);

    TcGroup grp;
    grp.n = 1;
    int rc = Prepare(ctx, p, mode, bn, pair, msub, grp.p[0], grp.tm[0]);
    if (rc != NTB_OK)
        return rc;
    grp.p[1] = grp.p[0];
    for (int i = 0; i < 3; i++)
        grp.tm[1][i] = grp.tm[0][i];
    grp.split = grp.total = grp.p[0].totalTiles;

    if (p.nPeers > 0 && !grp.p[0].cTma)
        return NTB_ERR_ARG;                         /* peer copies are made from the staged boxes */
    if (split) {
        /* a 32-column slice of half values is half a store box: direct stores instead */
        if (split == 4 && p.dtC == NTB_X_FLOAT16)
            grp.p[0].cTma = 0;
        const TcParams & tp = grp.p[0];
        const int clusters = (int)(tp.totalTiles < ctx.smCount / split ? tp.totalTiles : ctx.smCount / split);
        const bool half = p.dtC == NTB_X_FLOAT16;
        const bool oldc = tp.beta != 0.f || tp.nPeers > 0;
#define NTB_SPLIT(SS, ST, GG, T) (oldc ? LaunchSplit<SS, ST, GG, T, true>(grp.tm[0][0], grp.tm[0][1], grp.tm[0][2], tp, clusters, stream) \
                                       : LaunchSplit<SS, ST, GG, T, false>(grp.tm[0][0], grp.tm[0][1], grp.tm[0][2], tp, clusters, stream))
        const int sg = Knob("NTB_SPLIT_G", 2);
        if (split == 2) {
            if (sg == 1)
                return half ? NTB_SPLIT(2, 4, 1, __half) : NTB_SPLIT(2, 4, 1, float);
            return half ? NTB_SPLIT(2, 4, 2, __half) : NTB_SPLIT(2, 4, 2, float);
        }
        return half ? NTB_SPLIT(4, 3, 1, __half) : NTB_SPLIT(4, 3, 1, float);
#undef NTB_SPLIT
    }
    if (pair) {
        const TcParams & tp = grp.p[0];
        const int pairs = (int)(tp.totalTiles < ctx.smCount / 2 ? tp.totalTiles : ctx.smCount / 2);
        const bool half = p.dtC == NTB_X_FLOAT16;
        /* k-blocks per barrier hand-shake: enough MMAs between two hand-shakes to cover one */
        /* 256 x 128 tiles: two k-blocks per hand-shake keep four barrier stages in flight;
           four (NTB_PAIR_G = 4) gain a few per cent on short K and lose more on long K */
        const int g = Knob("NTB_PAIR_G", 2);
        const bool oldc = tp.beta != 0.f || tp.nPeers > 0;
#define NTB_PAIR2(MS, W, ST, GG, T) (oldc ? LaunchPair<MS, W, ST, GG, T, true>(grp.tm[0][0], grp.tm[0][1], grp.tm[0][2], tp, pairs, stream) \
                                          : LaunchPair<MS, W, ST, GG, T, false>(grp.tm[0][0], grp.tm[0][1], grp.tm[0][2], tp, pairs, stream))
#define NTB_PAIR(MS, W, ST, GG) (half ? NTB_PAIR2(MS, W, ST, GG, __half) : NTB_PAIR2(MS, W, ST, GG, float))
        if (bn == 256)
            return msub == 2 ? NTB_PAIR(2, 256, 4, 1) : NTB_PAIR(1, 256, 6, 1);
        if (msub == 2)
            return NTB_PAIR(2, 128, 4, 2);
        return g == 4 ? NTB_PAIR(1, 128, 8, 4) : NTB_PAIR(1, 128, 8, 2);
#undef NTB_PAIR2
#undef NTB_PAIR
    }
    return LaunchGroup(grp, mode, bn, p.dtC, ctx.smCount, stream);
}

/* what the cost model would launch for p alone: > 0 single-CTA tile width, <= 0 a cluster kernel */
int TcTileChoice(const DeviceCtx & ctx, const Problem & p)
{
    return PickBN(p, ctx.smCount, p.dtAB == NTB_X_FLOAT16 ? 0 : 1);
}

/*
 * Two problems of the same operand and output types in ONE launch of the single-CTA
 * kernel: the tile walk covers the tiles of the first, then of the second. Used for the
 * two gradient products of a matrix multiplication, which share dE/dc. The tile width is
 * the one the cost model prefers for the two problems taken together.
 */
int LaunchTcTwo(const DeviceCtx & ctx, const Problem & p0, const Problem & p1, cudaStream_t stream)
{
    const int mode = p0.dtAB == NTB_X_FLOAT16 ? 0 : 1;
    const int cand[3] = { 256, 128, 64 };
    int bn = 128;
    double bestCost = 1e300;
    for (int i = (mode == 0 ? 0 : 1); i < 3; i++) {
        const int w = cand[i];
        const long long t0 = (long long)((p0.M + BM - 1) / BM) * ((p0.N + w - 1) / w) * p0.count;
        const long long t1 = (long long)((p1.M + BM - 1) / BM) * ((p1.N + w - 1) / w) * p1.count;
        const long long waves = (t0 + t1 + ctx.smCount - 1) / ctx.smCount;
        const int kElems = ROW_BYTES / (mode == 0 ? 2 : 4);
        const double kb = 0.5 * ((p0.K + kElems - 1) / kElems + (p1.K + kElems - 1) / kElems);
        const double perK = fmax((mode == 0 ? 2.0 : 6.0) * w, (double)(BM + w) * ROW_BYTES / 62.0);
        const double cost = (double)waves * (kb * perK + 1500.0 + 4.0 * w);
        if (cost < bestCost) { bestCost = cost; bn = w; }
    }
    const int knobBN = Knob("NTB_BN", 0);
    if (knobBN == 64 || knobBN == 128 || (knobBN == 256 && mode == 0))
        bn = knobBN;
    TcGroup grp;
    grp.n = 2;
    int rc = Prepare(ctx, p0, mode, bn, false, 1, grp.p[0], grp.tm[0]);
    if (rc != NTB_OK)
        return rc;
    rc = Prepare(ctx, p1, mode, bn, false, 1, grp.p[1], grp.tm[1]);
    if (rc != NTB_OK)
        return rc;
    grp.split = grp.p[0].totalTiles;
    grp.total = grp.p[0].totalTiles + grp.p[1].totalTiles;
    return LaunchGroup(grp, mode, bn, p0.dtC, ctx.smCount, stream);
}


#ifdef NTB_WAIT_STATS
extern "C" void ntb_debug_wait_stats(unsigned long long * out)
{
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, gWaitStats, sizeof(unsigned long long) * 8);
    unsigned long long zero[8] = {0};
    cudaMemcpyToSymbol(gWaitStats, zero, sizeof(zero));
}

extern "C" void ntb_debug_timeline(unsigned long long * out)
{
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, gTimeline, sizeof(unsigned long long) * 64);
    unsigned long long zero[64] = {0};
    cudaMemcpyToSymbol(gTimeline, zero, sizeof(zero));
}
#endif

}
