/*
 * Pieces shared by the tensor-core kernels (single-CTA, CTA-pair, split-K): kernel
 * parameters, the per-warp writer of output tiles (staging in swizzled shared memory, TMA
 * stores, old values of C, copies to peer buffers), the tile walk, and the cluster helpers.
 * Each kernel family is its own translation unit so that they compile side by side.
 */
#ifndef NTB_TC_COMMON_CUH
#define NTB_TC_COMMON_CUH

#include "ntb_internal.h"
#include "ntb_ptx.cuh"

namespace ntb {

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
    int peerMcast;          /* peers[0] is a multicast address, written with multimem.st */
    int peerTma;            /* CTA-pair kernel: the peers are written with TMA stores through their own tensor maps */
    int l2Hint;             /* pair kernel: L2 eviction policy of the A loads (bits 0-1) and B loads (bits 2-3): 0 none, 1 keep, 2 stream */
    int cPrefetch;          /* wide tiles with beta != 0: 0 no L2 prefetch of old C, 1 boxes through TMA, 2 one request per line */
    float alpha, beta;
    const void * bias;      /* N values of C's type added to every output row, or NULL */
    int act;                /* 1: max(x, 0) applied last */
    int * status;
    /* operands as plain addresses, for the kernels whose loader warps fetch them with ordinary loads */
    const void * a;
    const void * b;
    long long lda, ldb, sAp, sAq, sBp, sBq;   /* elements */
    int skipKBlock;         /* test hook: the producer arms this k-block of its first tile but never loads it; -1 off */
    /* split-K on CTA pairs: workspace for the partial sums and its arrival counters */
    float * psWork;
    int * psFlags;
};


/* tensor maps of the peer copies of C (same shape and pitch as C): the CTA-pair kernel sends
   each finished box to them with TMA stores instead of per-lane stores */
struct PeerMaps {
    CUtensorMap m[NTB_MAX_PEERS];
};

/* launchers of the cluster kernels (ntb_tc_pair.cu, ntb_tc_split.cu); maps: A, B, C */
int LaunchPairKernel(int msub, int bn, int g, int epiWarps, bool half, bool oldc, const CUtensorMap * maps, const TcParams & tp,
                     const PeerMaps * peerMaps, int pairs, cudaStream_t stream);
int LaunchSplitKernel(int split, int g, bool half, bool oldc, const CUtensorMap * maps, const TcParams & tp,
                      int clusters, cudaStream_t stream);
/* split-K on CTA pairs (ntb_tc_pairsplit.cu): tp and maps as for the pair kernel's 256 x 256 tile */
int LaunchPairSplitKernel(int split, int g, bool half, bool oldc, const CUtensorMap * maps, const TcParams & tp, cudaStream_t stream);

namespace {

/* fp32 route: threads that split operands into hi/lo planes (warps 6 and up) */
#ifndef NTB_CONV_THREADS
#define NTB_CONV_THREADS 128
#endif
constexpr int CONV_THREADS = NTB_CONV_THREADS;
constexpr int FP32_CHUNK_BLOCKS = 8;  /* fp32 route: 8 k-blocks = 256 of K per TMEM accumulation chain */

/* Optional wait accounting (compile with -DNTB_WAIT_STATS): cycles each role of the
   CTA-pair kernel spends blocked on its barriers, summed over CTAs.
   0 producer on empty, 1 MMA on full, 2 MMA on tempty, 3 epilogue warp 2 on tfull,
   4 kernel cycles of CTA 0's producer lane, 5 CTAs counted */
#ifdef NTB_WAIT_STATS
static __device__ unsigned long long gWaitStats[8];
/* timeline of CTA 0 of the single-CTA kernel, in SM clocks since kernel entry:
   0 set-up done, 1 first TMA issued, 2 first stage landed, 3 first tile's MMAs committed,
   4 epilogue saw the accumulator, 5 epilogue stores issued, 6 stores complete, 7 kernel end */
static __device__ unsigned long long gTimeline[64];
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
/* NBOX: staging boxes this warp alternates between (2, or 1 where eight epilogue warps
   share the staging space of four) */
template <typename OutT, bool OLDC, int NBOX = 2>
struct TileWriter {
    static constexpr int BOX_COLS = ROW_BYTES / (int)sizeof(OutT);   /* 64 halves / 32 floats */
    static constexpr int CHUNKS = 32 * (int)sizeof(OutT) / 16;      /* 16-byte chunks per 32 columns */
    uint32_t stage;          /* shared-memory address of this warp's two boxes */
    uint32_t boxes;          /* boxes handed to TMA so far */
    const CUtensorMap * map;
    const CUtensorMap * peerMaps;   /* maps of the peer copies of C, or NULL: peers are then written with per-lane stores */
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
        stage = epiBase + sub * NBOX * EPI_BOX_BYTES;
        boxes = 0;
        map = m;
        peerMaps = nullptr;
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
        if (fTotal > NBOX) {
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
                FetchBox(p, k, (boxes + (uint32_t)k) & (uint32_t)(NBOX - 1));
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
        const uint32_t bufIdx = boxes & (uint32_t)(NBOX - 1);
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
                /* the store that last used this box (NBOX boxes ago) must have read it */
                if (lane == 0 && boxes >= (uint32_t)NBOX) {
                    if (NBOX == 2)
                        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    else
                        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                }
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
                if (OLDC && peerMaps != nullptr) {
                    /* the same box to the same place of every peer's C: more stores of the same
                       bulk group, so the wait before the box is refilled covers them too */
                    for (int k = 0; k < p.nPeers; k++)
                        asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                                     :: "l"(peerMaps + k), "r"(c0 - colInBox), "r"(row0), "r"(batch), "r"(box) : "memory");
                }
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            if (OLDC && p.nPeers > 0 && live && peerMaps == nullptr)
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
                if (p.peerMcast) {
                    /* one store, replicated by the NVLink switch into every GPU's copy of C */
                    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                                 :: "l"((OutT *)p.peers[0] + off), "f"(__uint_as_float(w0)), "f"(__uint_as_float(w1)),
                                    "f"(__uint_as_float(w2)), "f"(__uint_as_float(w3)) : "memory");
                }
                else {
                    for (int k = 0; k < p.nPeers; k++)
                        *(uint4 *)((OutT *)p.peers[k] + off) = make_uint4(w0, w1, w2, w3);
                }
            }
            else if (row0 + rr < p.M && !p.peerMcast) {
                const uint32_t w[4] = { w0, w1, w2, w3 };          /* ragged right edge: element by element (multicast destinations
                                                                      are only accepted with whole 16-byte columns) */
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

/* ---------------------------------------------------------------- cluster helpers */

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

}

}

#endif
