/*
 * Fused scaled-dot-product attention for half tensors on sm_100a:
 *
 *        out = softmax(scale * q * k^T + mask) * v          per (batch x head) block
 *
 * One kernel replaces the reference's chain BMMul(q, k^T) -> ConvertDataType -> Sum(mask)
 * -> Softmax -> ConvertDataType -> BMMul(att, v)
 * (source/sample/transformer/submodel/Attention.cpp:206-238), which writes and re-reads the
 * [blocks, lenQ, lenK] score tensor four times. Here the scores of a 128-row query block
 * never leave the SM:
 *
 *   warp 0     TMA: q block, k and v of the (batch x head) block into shared memory
 *   warp 1     tcgen05.mma: S = q * k^T into TMEM (128 lanes x up to 256 columns, fp32);
 *              later O = P * v into a second TMEM region
 *   warps 2-5  one thread per query row (= TMEM lane): scale, mask, row maximum, exp, row
 *              sum -- the softmax of source/tensor/function/Softmax.cpp:60-115 in fp32 --
 *              then the un-normalised probabilities, rounded to half, go to shared memory
 *              in the swizzled K-major operand layout for the second product; after it the
 *              same thread scales its output row by 1 / sum and stores it through TMA.
 *
 * Half tensors, packed; head size 64 or 128 (the sample's default is 512 / 4 = 128,
 * source/sample/transformer/Config.cpp:126,137). Keys are taken 256 at a time: up to 256
 * (the sample caps sentences at 200, Config.cpp:128-129) everything happens in one step;
 * longer key sequences are walked twice, first for the row maxima, then for the sums and the
 * second product, so no partial result is ever rescaled. Attention dropout
 * (Attention.cpp:229-230) takes the caller's keep-mask, one byte per probability, so that a
 * test can apply the very same mask to the reference chain. Waits are bounded as in the GEMM
 * kernels.
 */
#include "ntb_internal.h"
#include "ntb_ptx.cuh"
#include <cstring>

namespace ntb {

namespace {

constexpr int KBLK = 256;                     /* keys per step: one score tile of 128 x 256 in tensor memory */
constexpr int V_BOX_BYTES = 64 * ROW_BYTES;           /* 64 k-rows x 64 halves */
constexpr int P_TILE_BYTES = BM * ROW_BYTES;          /* 128 rows x 64 halves of keys */
constexpr int OUT_BOX_BYTES = 32 * ROW_BYTES;         /* one warp's 32 rows x 64 halves */
constexpr int TMEM_S = 0, TMEM_O = 256, ATTN_TMEM_COLS = 512;

/* shared memory of the kernel for head size D: q, k (later the probabilities, which replace
   it once the scores are in tensor memory), v, and the output boxes of the four softmax warps */
template <int D> struct AttnSmem {
    static constexpr int Q_BYTES = (D / 64) * BM * ROW_BYTES;
    static constexpr int K_BYTES = (D / 64) * KBLK * ROW_BYTES;
    static constexpr int P_BYTES = (KBLK / 64) * P_TILE_BYTES;
    static constexpr int KP_BYTES = K_BYTES > P_BYTES ? K_BYTES : P_BYTES;
    static constexpr int V_BYTES = (KBLK / 64) * (D / 64) * V_BOX_BYTES;
    static constexpr int OUT_BYTES = 4 * (D / 64) * OUT_BOX_BYTES;
    static constexpr int TOTAL = Q_BYTES + KP_BYTES + V_BYTES + OUT_BYTES + 1024;
};

#ifdef NTB_WAIT_STATS
__device__ unsigned long long gAttnTimeline[8];
#define ATTN_MARK(slot) do { if (blockIdx.x == 0 && threadIdx.x == 64) gAttnTimeline[slot] = (unsigned long long)(clock64() - attnT0); } while (0)
#else
#define ATTN_MARK(slot) do { } while (0)
#endif

struct AttnParams {
    const float * mask;          /* additive, fp32, [.., lenQ, lenK] per block, or NULL */
    long long maskBlockStride;   /* elements between the masks of consecutive blocks; 0 = one mask for all */
    const unsigned char * keep;  /* dropout: 1 = keep, 0 = drop, [blocks, lenQ, lenK], or NULL */
    float keepScale;             /* what a kept probability is multiplied by, 1 / (1 - p) */
    int blocks, lenQ, lenK, qTiles, totalItems;
    int kSteps;                  /* key blocks of KBLK per item */
    float scale;
    int * status;
};

/*
 * One item = one 128-row query tile of one (batch x head) block. Its keys are walked in
 * steps of KBLK. With a single step the row maximum, the exponentials and the second
 * product all happen in it. With several, the walk is made twice: the first pass only takes
 * the row maxima of the scores (the second product of those steps is empty), the second
 * pass recomputes the scores and accumulates exp(s - max) * v over the key blocks into one
 * accumulator, so nothing ever has to be rescaled. Every step runs the same hand-shake:
 * producer (k, and v in the second pass; q with the item's first step) -> scores -> softmax
 * warps -> second product -> next step.
 */
template <int D>
__global__ void __launch_bounds__(192, 1)
AttentionKernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, AttnParams p)
{
    using SM = AttnSmem<D>;
    constexpr int DC = D / 64;                    /* 64-wide chunks of the head dimension */
#ifdef NTB_WAIT_STATS
    const long long attnT0 = clock64();
#endif
    extern __shared__ uint8_t smemRaw[];
    __shared__ __align__(8) uint64_t barQK, barV, barS, barP, barO, barOFree;
    __shared__ uint32_t tmemBaseSlot;
    __shared__ int abortFlag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t smemBase = (SmemAddr(smemRaw) + 1023u) & ~1023u;
    const uint32_t qS = smemBase, kS = qS + SM::Q_BYTES, pS = kS, vS = kS + SM::KP_BYTES, oS = vS + SM::V_BYTES;
    volatile int * abortPtr = &abortFlag;
    /* a kernel launched behind this one with programmatic serialisation may start setting up */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (threadIdx.x == 64) {
        PrefetchTensorMap(&tmQ);
        PrefetchTensorMap(&tmK);
        PrefetchTensorMap(&tmV);
        PrefetchTensorMap(&tmO);
    }
    if (threadIdx.x == 0) {
        MbarInit(SmemAddr(&barQK), 1);
        MbarInit(SmemAddr(&barV), 1);
        MbarInit(SmemAddr(&barS), 1);
        MbarInit(SmemAddr(&barP), 128);
        MbarInit(SmemAddr(&barO), 1);
        MbarInit(SmemAddr(&barOFree), 4);
        abortFlag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(SmemAddr(&tmemBaseSlot)), "r"((uint32_t)ATTN_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    TcFenceBefore();
    __syncthreads();
    TcFenceAfter();
    const uint32_t tmemBase = *(volatile uint32_t *)&tmemBaseSlot;
    const int passes = p.kSteps > 1 ? 2 : 1;
    /* set-up touched no global memory; wait here for the kernels before this one in the stream */
    asm volatile("griddepcontrol.wait;" ::: "memory");

    /* keys of step j: rows j * KBLK .., padded to a multiple of 64 */
    auto padOf = [&](int j) -> int {
        const int left = p.lenK - j * KBLK;
        return ((left < KBLK ? left : KBLK) + 63) / 64 * 64;
    };

    if (warp == 0) {
        if (lane == 0) {
            uint32_t st = 0;                      /* steps so far (all items) */
            uint32_t vLoads = 0;                  /* steps that loaded v */
            bool ok = true;
            for (int item = blockIdx.x; ok && item < p.totalItems; item += gridDim.x) {
                const int blk = item / p.qTiles, qt = item - blk * p.qTiles;
                for (int pass = 0; ok && pass < passes; pass++) {
                    const bool withV = pass == passes - 1;
                    for (int j = 0; j < p.kSteps; j++, ++st) {
                        /* the step before has finished with shared memory */
                        if (st > 0) {
                            ok = MbarWait(SmemAddr(&barO), (st - 1) & 1u, abortPtr, p.status);
                            if (!ok)
                                break;
                        }
                        const bool first = pass == 0 && j == 0;
                        MbarExpectTx(SmemAddr(&barQK), (first ? SM::Q_BYTES : 0) + SM::K_BYTES);
                        if (first) {
#pragma unroll
                            for (int dc = 0; dc < DC; dc++)
                                TmaLoad3D(qS + dc * BM * ROW_BYTES, &tmQ, SmemAddr(&barQK), dc * 64, qt * BM, blk);
                        }
#pragma unroll
                        for (int dc = 0; dc < DC; dc++)
                            TmaLoad3D(kS + dc * KBLK * ROW_BYTES, &tmK, SmemAddr(&barQK), dc * 64, j * KBLK, blk);
                        if (withV) {
                            const int kBoxes = padOf(j) / 64;
                            MbarExpectTx(SmemAddr(&barV), kBoxes * DC * V_BOX_BYTES);
                            for (int kb = 0; kb < kBoxes; kb++)
#pragma unroll
                                for (int dc = 0; dc < DC; dc++)
                                    TmaLoad3D(vS + (kb * DC + dc) * V_BOX_BYTES, &tmV, SmemAddr(&barV), dc * 64, j * KBLK + kb * 64, blk);
                            ++vLoads;
                        }
                    }
                }
            }
            (void)vLoads;
        }
    }
    else if (warp == 1) {
        if (lane == 0) {
            /* S: A = q (K-major), B = k (K-major), N = keys of the step; O: A = P (K-major), B = v (MN-major), N = D */
            const uint32_t iDescO = (1u << 4) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            uint32_t st = 0, vUses = 0, items = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < p.totalItems; item += gridDim.x, ++items) {
                for (int pass = 0; ok && pass < passes; pass++) {
                    const bool withV = pass == passes - 1;
                    for (int j = 0; j < p.kSteps; j++, ++st) {
                        const uint32_t ph = st & 1u;
                        const int kPad = padOf(j);
                        const uint32_t iDescS = (1u << 4) | ((uint32_t)(kPad >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
                        ok = MbarWait(SmemAddr(&barQK), ph, abortPtr, p.status);
                        if (!ok)
                            break;
                        TcFenceAfter();
#pragma unroll
                        for (int dc = 0; dc < DC; dc++)
#pragma unroll
                            for (int ks = 0; ks < 4; ks++)
                                TcMma<0>(tmemBase + TMEM_S, SmemDesc(qS + dc * BM * ROW_BYTES + ks * UMMA_K_BYTES, 16, 1024, 2),
                                         SmemDesc(kS + dc * KBLK * ROW_BYTES + ks * UMMA_K_BYTES, 16, 1024, 2), iDescS,
                                         (dc | ks) != 0 ? 1u : 0u);
                        TcCommit(SmemAddr(&barS));

                        ok = MbarWait(SmemAddr(&barP), ph, abortPtr, p.status);
                        if (ok && withV) {
                            ok = MbarWait(SmemAddr(&barV), vUses & 1u, abortPtr, p.status);
                            /* the accumulator of the item before has been read out */
                            if (ok && j == 0 && items > 0)
                                ok = MbarWait(SmemAddr(&barOFree), (items - 1) & 1u, abortPtr, p.status);
                        }
                        if (!ok)
                            break;
                        TcFenceAfter();
                        if (withV) {
                            const int kBoxes = kPad / 64;
                            for (int kb = 0; kb < kBoxes; kb++) {
#pragma unroll
                                for (int ks = 0; ks < 4; ks++)
                                    TcMma<0>(tmemBase + TMEM_O,
                                             SmemDesc(pS + kb * P_TILE_BYTES + ks * UMMA_K_BYTES, 16, 1024, 2),
                                             SmemDesc(vS + kb * DC * V_BOX_BYTES + ks * 16 * ROW_BYTES, V_BOX_BYTES, 1024, 2),
                                             iDescO, (j | kb | ks) != 0 ? 1u : 0u);
                            }
                            ++vUses;
                        }
                        /* first-pass steps have no second product: this only hands the step on */
                        TcCommit(SmemAddr(&barO));
                    }
                }
            }
        }
    }
    else {
        const int sub = warp & 3;
        const uint32_t laneBase = (uint32_t)(sub * 32) << 16;
        const uint32_t outBox = oS + sub * DC * OUT_BOX_BYTES;
        const uint32_t pRow = (uint32_t)(sub * 32 + lane) * ROW_BYTES;
        uint32_t st = 0, items = 0;
        bool ok = true;
        for (int item = blockIdx.x; ok && item < p.totalItems; item += gridDim.x, ++items) {
            const int blk = item / p.qTiles, qt = item - blk * p.qTiles;
            const int row0 = qt * BM + sub * 32, row = row0 + lane;
            const bool rowOk = row < p.lenQ;
            const float * maskRow = (p.mask != nullptr && rowOk)
                ? p.mask + (long long)blk * p.maskBlockStride + (long long)row * p.lenK : nullptr;
            const unsigned char * keepRow = (p.keep != nullptr && rowOk)
                ? p.keep + ((long long)blk * p.lenQ + row) * p.lenK : nullptr;
            /* Both scans are written without data-dependent branches and with four
               independent accumulators: a softmax warp has its SM sub-partition to itself,
               so nothing hides the latency of a dependent chain or of a branch. Full
               64-column chunks without a mask take the short path. */
            float m4[4] = { -INFINITY, -INFINITY, -INFINITY, -INFINITY };
            float s4[4] = { 0.f, 0.f, 0.f, 0.f };
            float mRef = 0.f, rowLive = 1.f;

            /* row maximum of scale * s + mask over the valid keys of step j */
            auto scanMax = [&](int j) {
                const int kPad = padOf(j), base = j * KBLK;
                for (int c0 = 0; c0 < kPad; c0 += 64) {
                    float v[64];
                    TmemLoad64(tmemBase + laneBase + TMEM_S + c0, v);
                    if (maskRow == nullptr && base + c0 + 64 <= p.lenK) {
#pragma unroll
                        for (int e = 0; e < 64; e++)
                            m4[e & 3] = fmaxf(m4[e & 3], v[e] * p.scale);
                    }
                    else {
#pragma unroll
                        for (int e = 0; e < 64; e++) {
                            const int c = base + c0 + e;
                            const bool valid = c < p.lenK;
                            float x = v[e] * p.scale;
                            if (maskRow != nullptr)
                                x += valid ? maskRow[c] : 0.f;
                            m4[e & 3] = fmaxf(m4[e & 3], valid ? x : -INFINITY);
                        }
                    }
                }
            };
            auto closeMax = [&]() {
                const float m = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
                rowLive = m == -INFINITY ? 0.f : 1.f;      /* a fully masked row gives zeros */
                mRef = m == -INFINITY ? 0.f : m;
            };
            /* e = exp(x - max) for the keys of step j; the halves (times the dropout factor, if
               any) go to shared memory as the K-major, 128-byte-swizzled A operand of P * v.
               Without dropout the row sum is taken over the rounded values, the ones the second
               product really uses; with it, over the unrounded probabilities before dropping. */
            auto expStore = [&](int j) {
                const int kPad = padOf(j), base = j * KBLK;
                for (int c0 = 0; c0 < kPad; c0 += 64) {
                    float v[64];
                    TmemLoad64(tmemBase + laneBase + TMEM_S + c0, v);
                    const bool plain = maskRow == nullptr && base + c0 + 64 <= p.lenK;
                    if (plain) {
#pragma unroll
                        for (int e = 0; e < 64; e++)
                            v[e] = __expf(v[e] * p.scale - mRef) * rowLive;
                    }
                    else {
#pragma unroll
                        for (int e = 0; e < 64; e++) {
                            const int c = base + c0 + e;
                            const bool valid = c < p.lenK;
                            float x = v[e] * p.scale;
                            if (maskRow != nullptr)
                                x += valid ? maskRow[c] : 0.f;
                            /* x == -inf (masked) gives exp(-inf) = 0 */
                            v[e] = valid ? __expf(x - mRef) * rowLive : 0.f;
                        }
                    }
                    if (p.keep != nullptr) {
#pragma unroll
                        for (int e = 0; e < 64; e++) {
                            const int c = base + c0 + e;
                            s4[e & 3] += v[e];
                            const bool kept = keepRow != nullptr && c < p.lenK && keepRow[c] != 0;
                            v[e] = kept ? v[e] * p.keepScale : 0.f;
                        }
                    }
                    const uint32_t tile = pS + (c0 / 64) * P_TILE_BYTES + pRow;
#pragma unroll
                    for (int jj = 0; jj < 8; jj++) {
                        uint32_t w[4];
#pragma unroll
                        for (int h = 0; h < 4; h++) {
                            __half2 hh = __floats2half2_rn(v[jj * 8 + h * 2], v[jj * 8 + h * 2 + 1]);
                            if (p.keep == nullptr) {
                                float2 back = __half22float2(hh);
                                s4[h] += back.x + back.y;
                            }
                            w[h] = *(uint32_t *)&hh;
                        }
                        const uint32_t dst = tile + (uint32_t)((jj ^ (lane & 7)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                     :: "r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
                    }
                }
            };

            for (int pass = 0; ok && pass < passes; pass++) {
                const bool last = pass == passes - 1;
                for (int j = 0; j < p.kSteps; j++, ++st) {
                    ok = MbarWaitWarp(SmemAddr(&barS), st & 1u, abortPtr, p.status, 200);
                    if (!ok)
                        break;
                    TcFenceAfter();
                    ATTN_MARK(0);
                    if (passes == 1 || !last)
                        scanMax(j);
                    if (passes == 1 || (last && j == 0))
                        closeMax();
                    ATTN_MARK(1);
                    if (last)
                        expStore(j);
                    ATTN_MARK(2);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    TcFenceBefore();
                    MbarArrive(SmemAddr(&barP));
                    ATTN_MARK(3);
                }
            }
            if (!ok)
                break;
            const float sum = (s4[0] + s4[1]) + (s4[2] + s4[3]);

            /* the output row: (P * v) / sum, after the last step's second product */
            ok = MbarWaitWarp(SmemAddr(&barO), (st - 1) & 1u, abortPtr, p.status, 200);
            if (!ok)
                break;
            TcFenceAfter();
            ATTN_MARK(4);
            const float inv = sum > 0.f ? 1.f / sum : 0.f;
            if (lane == 0 && items > 0)
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   /* the boxes are free again */
            __syncwarp();
#pragma unroll 1
            for (int dc = 0; dc < DC; dc++) {
                float o[64];
                TmemLoad64(tmemBase + laneBase + TMEM_O + dc * 64, o);
                if (dc == DC - 1) {
                    TcFenceBefore();
                    __syncwarp();
                    if (lane == 0)
                        MbarArrive(SmemAddr(&barOFree));
                }
#pragma unroll
                for (int jj = 0; jj < 8; jj++) {
                    __half2 h0 = __floats2half2_rn(o[jj * 8 + 0] * inv, o[jj * 8 + 1] * inv);
                    __half2 h1 = __floats2half2_rn(o[jj * 8 + 2] * inv, o[jj * 8 + 3] * inv);
                    __half2 h2 = __floats2half2_rn(o[jj * 8 + 4] * inv, o[jj * 8 + 5] * inv);
                    __half2 h3 = __floats2half2_rn(o[jj * 8 + 6] * inv, o[jj * 8 + 7] * inv);
                    const uint32_t dst = outBox + dc * OUT_BOX_BYTES + lane * ROW_BYTES + (uint32_t)((jj ^ (lane & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                 :: "r"(dst), "r"(*(uint32_t *)&h0), "r"(*(uint32_t *)&h1), "r"(*(uint32_t *)&h2),
                                    "r"(*(uint32_t *)&h3) : "memory");
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0 && row0 < p.lenQ) {
#pragma unroll
                for (int dc = 0; dc < DC; dc++)
                    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                                 :: "l"(&tmO), "r"(dc * 64), "r"(row0), "r"(blk), "r"(outBox + dc * OUT_BOX_BYTES) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        }
        ATTN_MARK(5);
        if (lane == 0)
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
        ATTN_MARK(6);
    }

    __syncwarp();
    if (*abortPtr) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
    }
    TcFenceBefore();
    __syncthreads();
    TcFenceAfter();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     :: "r"(tmemBase), "r"((uint32_t)ATTN_TMEM_COLS) : "memory");
    }
}

int Encode3D(CUtensorMap * map, const void * base, int cols, int rows, int blocks, int boxCols, int boxRows)
{
    EncodeTiledFn enc = GetEncodeTiled();
    if (!enc)
        return NTB_ERR_CUDA;
    cuuint64_t dims[3] = { (cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)blocks };
    cuuint64_t strides[2] = { (cuuint64_t)cols * 2, (cuuint64_t)rows * cols * 2 };       /* packed [blocks][rows][cols] halves */
    cuuint32_t box[3] = { (cuuint32_t)boxCols, (cuuint32_t)boxRows, 1 };
    cuuint32_t estr[3] = { 1, 1, 1 };
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, (void *)base, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? NTB_OK : NTB_ERR_CUDA;
}

}

}

using namespace ntb;

namespace {

template <int D>
int LaunchAttention(const DeviceCtx & ctx, const void * q, const void * k, const void * v, void * out, const AttnParams & p,
                    cudaStream_t stream)
{
    CUtensorMap tmQ, tmK, tmV, tmO;
    int rc;
    if ((rc = Encode3D(&tmQ, q, D, p.lenQ, p.blocks, 64, BM)) != NTB_OK ||
        (rc = Encode3D(&tmK, k, D, p.lenK, p.blocks, 64, KBLK)) != NTB_OK ||
        (rc = Encode3D(&tmV, v, D, p.lenK, p.blocks, 64, 64)) != NTB_OK ||
        (rc = Encode3D(&tmO, out, D, p.lenQ, p.blocks, 64, 32)) != NTB_OK)
        return rc;
    static SmemOptIn optIn;
    if (!optIn.Ensure((const void *)AttentionKernel<D>, AttnSmem<D>::TOTAL))
        return NTB_ERR_CUDA;
    const int grid = p.totalItems < ctx.smCount ? p.totalItems : ctx.smCount;
    const cudaError_t err = LaunchPdl(AttentionKernel<D>, grid, 192, AttnSmem<D>::TOTAL, stream, tmQ, tmK, tmV, tmO, p);
    CountLaunch();
    return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? NTB_OK : NTB_ERR_CUDA;
}

}

extern "C" int ntb_attention_dropout(int devID, void * stream,
                                     const void * q, const void * k, const void * v, const float * mask,
                                     const unsigned char * keep, void * out,
                                     int dtype, int blocks, int lenQ, int lenK, int dim,
                                     long long maskBlockStride, float scale, float keepScale)
{
    if (!q || !k || !v || !out || blocks < 0 || lenQ < 0 || lenK < 0 || maskBlockStride < 0)
        return NTB_ERR_ARG;
    if (dtype != NTB_X_FLOAT16)
        return NTB_ERR_DTYPE;
    if (blocks == 0 || lenQ == 0)
        return NTB_OK;
    if ((dim != 64 && dim != 128) || lenK < 1)
        return NTB_ERR_LIMIT;
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15)
        return NTB_ERR_ARG;

    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess || (prev != devID && cudaSetDevice(devID) != cudaSuccess)) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    int rc = NTB_ERR_CUDA;
    do {
        DeviceCtx * ctx = CtxFor(devID);
        if (!ctx)
            break;
        AttnParams p;
        memset(&p, 0, sizeof(p));
        p.mask = mask;
        p.maskBlockStride = maskBlockStride;
        p.keep = keep;
        p.keepScale = keepScale;
        p.blocks = blocks; p.lenQ = lenQ; p.lenK = lenK;
        p.qTiles = (lenQ + BM - 1) / BM;
        p.kSteps = (lenK + KBLK - 1) / KBLK;
        const long long items = (long long)blocks * p.qTiles;
        if (items > 2147483647LL - 1024) {
            rc = NTB_ERR_LIMIT;
            break;
        }
        p.totalItems = (int)items;
        p.scale = scale;
        p.status = ctx->status;
        rc = dim == 64 ? LaunchAttention<64>(*ctx, q, k, v, out, p, (cudaStream_t)stream)
                       : LaunchAttention<128>(*ctx, q, k, v, out, p, (cudaStream_t)stream);
    } while (0);
    if (rc == NTB_ERR_CUDA)
        cudaGetLastError();
    if (prev >= 0 && prev != devID)
        cudaSetDevice(prev);
    return rc;
}

extern "C" int ntb_attention(int devID, void * stream,
                             const void * q, const void * k, const void * v, const float * mask, void * out,
                             int dtype, int blocks, int lenQ, int lenK, int dim,
                             long long maskBlockStride, float scale)
{
    return ntb_attention_dropout(devID, stream, q, k, v, mask, nullptr, out, dtype, blocks, lenQ, lenK, dim,
                                 maskBlockStride, scale, 1.f);
}

#ifdef NTB_WAIT_STATS
extern "C" void ntb_debug_attn_timeline(unsigned long long * out)
{
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, ntb::gAttnTimeline, sizeof(unsigned long long) * 8);
}
#endif
