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
#include "ntb_tc_single.cuh"
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cmath>
#include <atomic>
#include <mutex>

namespace ntb {

namespace {

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

/* integer knob from the environment, read at every launch: the knobs that pick a kernel
   (tests and tuning runs change these between calls of one process) */
int Knob(const char * name, int dflt)
{
    const char * v = getenv(name);
    return v && *v ? atoi(v) : dflt;
}

/* knobs that only tune a kernel already chosen are read once per process */
struct TuneKnobs {
    int pfDist, group, epiHint, cPrefetch, l2Hint, l2Promotion, tmaStore, debugChoice;
};
const TuneKnobs & Tune()
{
    static const TuneKnobs k = { Knob("NTB_PREFETCH_DIST", 0), Knob("NTB_TILE_GROUP", 8), Knob("NTB_EPI_HINT_NS", 2000),
                                 Knob("NTB_C_PREFETCH", 0), Knob("NTB_L2_HINT", 0), Knob("NTB_L2_PROMOTION", 3),
                                 Knob("NTB_TMA_STORE", 1), Knob("NTB_DEBUG_CHOICE", 0) };
    return k;
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
    const int promo = Tune().l2Promotion;   /* tuning: L2 fetch granularity of operand loads */
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
 * the split-K kernel with clusters of 2 / 4 CTAs; -18 / -20 for split-K on CTA pairs (2 / 4
 * pairs per 256 x 256 tile). Constants were fitted to timings of the
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

int PickBN(const Problem & p, int smCount, int mode, bool allowPairSplit = true)
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
    if (mode == 0 && smCount >= 8 && allowPairSplit) {
        /* split-K on CTA pairs: S pairs share a 256 x 256 tile and a 1/S part of K each; the
           pair tile moves half the operand bytes per flop of the 128 x 128 split above */
        for (int sp = 2; sp <= 4; sp *= 2) {
            /* measured: the exchange of the partial sums costs 7 (two pairs) to 11 us (four),
               which pays from K = 4096 on (4096 x 512 x 8192: 44 -> 35 us, 1024 x 1024 x 8192:
               30 -> 26, 512 x 2048 x 4096: 19.4 -> 16.5) and not at K = 2048 (14.2 -> 15.3) */
            if (kBlocks < 64.0 || kBlocks < 8.0 * sp || smCount < 2 * sp)
                continue;
            const long long tiles = (long long)((p.M + 255) / 256) * ((p.N + 255) / 256) * p.count;
            /* the pairs of a tile wait for one another: one wave only */
            const long long clusters = (long long)(smCount / 2) / sp;
            if (clusters < 1 || tiles > clusters)
                continue;
            const long long waves = 1;
            KbCost c;
            c.math = 512.0;
            c.bytes = (double)(BM + 128) * ROW_BYTES;
            c.reads = c.bytes;
            c.mmas = 4.0;
            c.shake = 500.0;
            c.g = 1;
            const double perK = PerKBlock(c, 2 * sp * (tiles < clusters ? tiles : clusters));
            const double cost = (double)waves * (ceil(kBlocks / sp) * perK * 1.25 + (sp == 2 ? 5000.0 : 9000.0)) + 2500.0;
            if (cost < bestCost) { bestCost = cost; best = -16 - sp; }
        }
    }
    return best;
}

}

int EncodeOperandMap(CUtensorMap * map, int mode, const void * base, int mnMajor, int rows, int cols,
                     long long ld, long long batchStride, int batchExtent, int tileRows)
{
    return EncodeOperand(map, mode, base, mnMajor, rows, cols, ld, batchStride, batchExtent, tileRows);
}

int EncodeOutputMap(CUtensorMap * map, int dtC, void * base, int rows, int cols, long long ld,
                    long long batchStride, int batchExtent)
{
    return EncodeOutput(map, dtC, base, rows, cols, ld, batchStride, batchExtent);
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
            TcParams & tp, CUtensorMap * maps, bool ldg = false)
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
    tp.peerTma = 0;
    tp.peerMcast = p.peerMcast;
    for (int i = 0; i < NTB_MAX_PEERS; i++)
        tp.peers[i] = i < p.nPeers ? p.peers[i] : nullptr;
    tp.status = ctx.status;
    tp.skipKBlock = InjectedSkipKBlock();
    tp.psWork = nullptr;
    tp.psFlags = nullptr;
    tp.pfDist = Tune().pfDist;
    tp.group = Tune().group;
    if (tp.group < 1)
        tp.group = 1;
    tp.epiHint = Tune().epiHint;
    tp.cPrefetch = Tune().cPrefetch;
    tp.l2Hint = Tune().l2Hint;
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

    tp.a = p.a; tp.b = p.b;
    tp.lda = p.lda; tp.ldb = p.ldb;
    tp.sAp = p.sAp; tp.sAq = p.sAq; tp.sBp = p.sBp; tp.sBq = p.sBq;
    int rc = NTB_OK;
    if (ldg) {
        /* loader warps address the operands themselves; no tensor maps */
        memset(&maps[0], 0, sizeof(CUtensorMap));
        memset(&maps[1], 0, sizeof(CUtensorMap));
    }
    else {
        rc = EncodeOperand(&maps[0], mode, p.a, p.aMN, p.aRows, p.aCols, p.lda, stA, extA, BM);
        if (rc != NTB_OK)
            return rc;
        rc = EncodeOperand(&maps[1], mode, p.b, p.bMN, p.bRows, p.bCols, p.ldb, stB, extB, pair ? bn / 2 : bn);
        if (rc != NTB_OK)
            return rc;
    }

    /* C through TMA stores when its base, pitch and batch strides are 16-byte aligned and
       its batch offset is one index times one stride; otherwise direct stores */
    maps[2] = maps[0];
    long long stC = 0;
    int extC = 1;
    tp.cSel = 0;
    tp.cTma = tp.cVec && Tune().tmaStore != 0 && p.ldc >= p.N &&
              BatchSelector(p.sCp, p.sCq, P, p.Q, &tp.cSel, &stC, &extC) && stC >= 0;
    if (tp.cTma) {
        rc = EncodeOutput(&maps[2], p.dtC, p.c, p.M, p.N, p.ldc, stC, extC);
        if (rc != NTB_OK)
            return rc;
    }
    return NTB_OK;
}

}

int PrepareSingle(const DeviceCtx & ctx, const Problem & p, int bn, TcParams & tp, CUtensorMap * maps)
{
    return Prepare(ctx, p, p.dtAB == NTB_X_FLOAT16 ? 0 : 1, bn, false, 1, tp, maps, false);
}

bool LdgEligible(const Problem & p)
{
    if (p.M <= 0 || p.N <= 0 || p.K <= 0 || p.count <= 0)
        return false;
    const bool f16 = p.dtAB == NTB_X_FLOAT16 && (p.dtC == NTB_X_FLOAT16 || p.dtC == NTB_X_FLOAT);
    const bool f32 = p.dtAB == NTB_X_FLOAT && p.dtC == NTB_X_FLOAT;
    if (!f16 && !f32)
        return false;
    const long long es = ElemSize(p.dtAB);
    if (((uintptr_t)p.a % es) || ((uintptr_t)p.b % es) || p.lda < p.aCols || p.ldb < p.bCols)
        return false;
    return p.sAp >= 0 && p.sAq >= 0 && p.sBp >= 0 && p.sBq >= 0;
}

int LaunchLdg(const DeviceCtx & ctx, const Problem & p, cudaStream_t stream, int * route)
{
    const int mode = p.dtAB == NTB_X_FLOAT16 ? 0 : 1;
    /* a large fp32 product is split into half pieces by a pre-pass that reads the operands with
       ordinary loads anyway: alignment does not matter to it */
    if (mode == 1 && ForcedRoute() != NTB_ROUTE_TC_3XTF32 && Knob("NTB_F32_SPLIT", 1) != 0 && F32SplitEligible(ctx, p)) {
        const int rc = LaunchF32Split(ctx, p, stream);
        if (rc == NTB_OK)
            *route = NTB_ROUTE_TC_F16X2;
        return rc;
    }
    /* large enough to pay for one more pass over the operands: copy them into aligned rows
       once and use the TMA-fed kernels (NTB_REPACK=0 keeps the loader warps) */
    if (Knob("NTB_REPACK", 1) != 0 && RepackWorthwhile(ctx, p)) {
        const int rr = LaunchRepacked(ctx, p, stream, route);
        if (rr != NTB_ERR_ARG)
            return rr;
    }
    TcGroup grp;
    grp.n = 1;
    int rc = Prepare(ctx, p, mode, 128, false, 1, grp.p[0], grp.tm[0], true);
    if (rc != NTB_OK)
        return rc;
    grp.p[1] = grp.p[0];
    for (int i = 0; i < 3; i++)
        grp.tm[1][i] = grp.tm[0][i];
    grp.first[0] = 0;
    grp.first[1] = grp.first[2] = grp.total = grp.p[0].totalTiles;
    if (p.nPeers > 0 && !grp.p[0].cTma)
        return NTB_ERR_ARG;
    *route = mode == 0 ? NTB_ROUTE_TC_F16 : NTB_ROUTE_TC_3XTF32;
    if (Tune().debugChoice)
        fprintf(stderr, "ntb: M %d N %d K %d count %d -> single 128 wide, loader warps (operands not addressable by TMA)\n",
                p.M, p.N, p.K, p.count);
    const bool oldc = p.beta != 0.f || p.nPeers > 0;
    return LaunchLdgKernel(grp, mode, p.dtC, oldc, ctx.smCount, stream);
}

int LaunchTc(const DeviceCtx & ctx, const Problem & p, cudaStream_t stream, int * route)
{
    const int mode = p.dtAB == NTB_X_FLOAT16 ? 0 : 1;
    const int forced = ForcedRoute();
    /* large 2-D fp32 products: two half-precision pieces per value on the fp16 pipe of CTA
       pairs (NTB_F32_SPLIT=0, or a forced kind::tf32 route, keeps them on the tf32 kernel) */
    if (mode == 1 && forced != NTB_ROUTE_TC_3XTF32 && Knob("NTB_F32_SPLIT", 1) != 0 && F32SplitEligible(ctx, p)) {
        const int rc = LaunchF32Split(ctx, p, stream);
        if (rc == NTB_OK)
            *route = NTB_ROUTE_TC_F16X2;
        return rc;
    }
    /* split-K on CTA pairs is chosen by the model only when nothing restricts the choice
       (NTB_PAIR_SPLIT: 0 never, 2 / 4 force that many pairs per tile) */
    const int knobPS = Knob("NTB_PAIR_SPLIT", -1);
    const bool modelMayPairSplit = forced == 0 && knobPS != 0 && Knob("NTB_BN", 0) == 0 && Knob("NTB_SPLIT_K", -1) < 0 &&
                                   Knob("NTB_PAIR_BN", 0) == 0 && Knob("NTB_PAIR_MSUB", 0) == 0;
    int bn = PickBN(p, ctx.smCount, mode, modelMayPairSplit);
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
    {
        int pairSplit = bn == -18 ? 2 : bn == -20 ? 4 : 0;
        const long long tiles256 = (long long)((p.M + 255) / 256) * ((p.N + 255) / 256) * p.count;
        if (mode == 0 && (knobPS == 2 || knobPS == 4) && (p.K + 63) / 64 >= 2 * knobPS && tiles256 * knobPS <= ctx.smCount / 2 &&
            ctx.mayAllocate && (forced == 0 || forced == NTB_ROUTE_TC_F16_PAIR))
            pairSplit = knobPS;
        if (pairSplit) {
            TcParams tp;
            CUtensorMap maps[3];
            int rc = Prepare(ctx, p, mode, 256, true, 1, tp, maps);
            if (rc != NTB_OK)
                return rc;
            if (p.nPeers > 0 && !tp.cTma)
                return NTB_ERR_ARG;
            /* every pair of a tile waits for the others: all of them must be resident at once */
            if ((long long)tp.totalTiles * pairSplit > ctx.smCount / 2 || !ctx.mayAllocate)
                return NTB_ERR_ARG;
            const size_t workBytes = (size_t)tp.totalTiles * pairSplit * (pairSplit - 1) * 2 * 128 * (256 / pairSplit) * sizeof(float);
            const size_t flagBytes = (size_t)tp.totalTiles * pairSplit * 2 * 4 * sizeof(int);
            rc = ScratchAcquire(ctx, stream);
            if (rc == NTB_OK)
                rc = EnsureCounted(ctx, workBytes, flagBytes, stream, &tp.psWork, &tp.psFlags);
            if (rc != NTB_OK)
                return rc;
            *route = NTB_ROUTE_TC_F16_PAIR;
            if (Tune().debugChoice)
                fprintf(stderr, "ntb: M %d N %d K %d count %d -> %d pairs per 256 x 256 tile, split along K\n",
                        p.M, p.N, p.K, p.count, pairSplit);
            rc = LaunchPairSplitKernel(pairSplit, Knob("NTB_PAIR_SPLIT_G", 2) == 1 ? 1 : 2, p.dtC == NTB_X_FLOAT16, tp.beta != 0.f || tp.nPeers > 0, maps, tp,
                                       stream);
            const int rel = ScratchRelease(ctx, stream);
            return rc != NTB_OK ? rc : rel;
        }
    }
    int split = (bn == -2 || bn == -4) ? -bn : 0;
    if (split == 4 && p.nPeers > 0 && p.dtC == NTB_X_FLOAT16)
        split = 2;                                  /* the 4-way split of a half tile stores directly */
    if (split)
        bn = 128;
    const bool pair = bn <= 0;
    int msub = (bn == -1 || bn == -9) ? 2 : 1;
    /* tuning: height of the pair tile in 256-row units (the model's choice otherwise) */
    const int knobMsub = Knob("NTB_PAIR_MSUB", 0);
    if (pair && (knobMsub == 1 || knobMsub == 2))
        msub = knobMsub;
    /* The peers' copies of C are written as tiles finish. When the 512-row tiles fit one wave,
       every tile finishes at the very end and the links idle until then (8192 x 1024 x 8192 on
       8 GPUs: 0.106 ms of product, then 0.131 ms of stores); with 256-row tiles the first
       wave's stores run under the second wave's MMAs. */
    if (pair && msub == 2 && p.nPeers > 0 && knobMsub == 0 && Knob("NTB_PEER_WAVES", 1) != 0) {
        const int width = bn <= -8 ? 128 : 256;
        const long long tilesBig = (long long)((p.M + 4 * BM - 1) / (4 * BM)) * ((p.N + width - 1) / width) * p.count;
        if (tilesBig <= ctx.smCount / 2)
            msub = 1;
    }
    if (pair)
        bn = bn <= -8 ? 128 : 256;
    *route = mode != 0 ? NTB_ROUTE_TC_3XTF32 : pair ? NTB_ROUTE_TC_F16_PAIR : NTB_ROUTE_TC_F16;
    if (Tune().debugChoice)
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
    grp.first[0] = 0;
    grp.first[1] = grp.first[2] = grp.total = grp.p[0].totalTiles;

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
        return LaunchSplitKernel(split, Knob("NTB_SPLIT_G", 2), half, oldc, grp.tm[0], tp, clusters, stream);
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
        /* tuning: epilogue warps of the 512 x 256 tile (8: two per tensor-memory sub-partition) */
        const int epiWarps = Knob("NTB_PAIR_EPIW", 8) == 4 ? 4 : 8;
        /* peer copies of C through TMA stores (NTB_PEER_TMA=0: per-lane stores, as the other kernels do) */
        PeerMaps pm;
        const bool peerTma = tp.nPeers > 0 && tp.cTma && !p.peerMcast && Knob("NTB_PEER_TMA", 1) != 0;
        if (peerTma) {
            long long stC = 0;
            int extC = 1, sel = 0;
            BatchSelector(p.sCp, p.sCq, p.count / p.Q, p.Q, &sel, &stC, &extC);
            for (int k = 0; k < tp.nPeers; k++) {
                rc = EncodeOutput(&pm.m[k], p.dtC, p.peers[k], p.M, p.N, p.ldc, stC, extC);
                if (rc != NTB_OK)
                    return rc;
            }
            grp.p[0].peerTma = 1;
        }
        return LaunchPairKernel(msub, bn, g, epiWarps, half, oldc, grp.tm[0], grp.p[0], peerTma ? &pm : nullptr, pairs, stream);
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
    grp.first[0] = 0;
    grp.first[1] = grp.p[0].totalTiles;
    grp.first[2] = grp.total = grp.p[0].totalTiles + grp.p[1].totalTiles;
    return LaunchGroup(grp, mode, bn, p0.dtC, ctx.smCount, stream);
}


#ifdef NTB_WAIT_STATS
extern "C" void ntb_debug_timeline(unsigned long long * out)
{
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, gTimeline, sizeof(unsigned long long) * 64);
    unsigned long long zero[64] = {0};
    cudaMemcpyToSymbol(gTimeline, zero, sizeof(zero));
}
#endif

}
