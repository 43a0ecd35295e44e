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
 * Limits of this version: half tensors, head size 64, lenK <= 256 (one score tile; the
 * transformer sample caps sentence length at 200, Config.cpp:128-129), packed operands.
 * Dropout (training) is not applied. Waits are bounded as in the GEMM kernels.
 */
#include "ntb_internal.h"
#include "ntb_ptx.cuh"
#include <cstring>

namespace ntb {

namespace {

constexpr int HD = 64;                        /* head size */
constexpr int MAX_LK = 256;
constexpr int Q_BYTES = BM * ROW_BYTES;               /* 128 rows x 64 halves */
constexpr int K_BYTES = MAX_LK * ROW_BYTES;           /* up to 256 rows x 64 halves */
constexpr int V_BOX_BYTES = 64 * ROW_BYTES;           /* 64 k-rows x 64 halves */
constexpr int V_BYTES = (MAX_LK / 64) * V_BOX_BYTES;
constexpr int P_TILE_BYTES = BM * ROW_BYTES;          /* 128 rows x 64 halves of lenK */
constexpr int P_BYTES = (MAX_LK / 64) * P_TILE_BYTES;
constexpr int OUT_BOX_BYTES = 32 * ROW_BYTES;         /* one warp's 32 rows x 64 halves */
constexpr int ATTN_SMEM = Q_BYTES + K_BYTES + V_BYTES + P_BYTES + 4 * OUT_BOX_BYTES + 1024;
constexpr int TMEM_S = 0, TMEM_O = 256, ATTN_TMEM_COLS = 512;

#ifdef NTB_WAIT_STATS
__device__ unsigned long long gAttnTimeline[8];
#define ATTN_MARK(slot) do { if (blockIdx.x == 0 && threadIdx.x == 64) gAttnTimeline[slot] = (unsigned long long)(clock64() - attnT0); } while (0)
#else
#define ATTN_MARK(slot) do { } while (0)
#endif

struct AttnParams {
    const float * mask;          /* additive, fp32, [.., lenQ, lenK] per block, or NULL */
    long long maskBlockStride;   /* elements between the masks of consecutive blocks; 0 = one mask for all */
    int blocks, lenQ, lenK, qTiles, totalItems;
    int kPad;                    /* lenK rounded up to a multiple of 64 */
    float scale;
    int * status;
};

__global__ void __launch_bounds__(192, 1)
AttentionKernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, AttnParams p)
{
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
    const uint32_t qS = smemBase, kS = qS + Q_BYTES, vS = kS + K_BYTES, pS = vS + V_BYTES, oS = pS + P_BYTES;
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
    const int kBoxes = p.kPad / 64;
    /* set-up touched no global memory; wait here for the kernels before this one in the stream */
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < p.totalItems; item += gridDim.x, ++it) {
                const int blk = item / p.qTiles, qt = item - blk * p.qTiles;
                /* the previous item's second product has finished reading shared memory */
                if (it > 0) {
                    ok = MbarWait(SmemAddr(&barO), (it - 1) & 1u, abortPtr, p.status);
                    if (!ok)
                        break;
                }
                MbarExpectTx(SmemAddr(&barQK), Q_BYTES + K_BYTES);
                TmaLoad3D(qS, &tmQ, SmemAddr(&barQK), 0, qt * BM, blk);
                TmaLoad3D(kS, &tmK, SmemAddr(&barQK), 0, 0, blk);
                MbarExpectTx(SmemAddr(&barV), kBoxes * V_BOX_BYTES);
                for (int kb = 0; kb < kBoxes; kb++)
                    TmaLoad3D(vS + kb * V_BOX_BYTES, &tmV, SmemAddr(&barV), 0, kb * 64, blk);
            }
        }
    }
    else if (warp == 1) {
        if (lane == 0) {
            /* S: A = q (K-major), B = k (K-major), N = kPad; O: A = P (K-major), B = v (MN-major), N = 64 */
            const uint32_t iDescS = (1u << 4) | ((uint32_t)(p.kPad >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            const uint32_t iDescO = (1u << 4) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            uint32_t it = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < p.totalItems; item += gridDim.x, ++it) {
                const uint32_t ph = it & 1u;
                ok = MbarWait(SmemAddr(&barQK), ph, abortPtr, p.status);
                if (!ok)
                    break;
                TcFenceAfter();
#pragma unroll
                for (int ks = 0; ks < 4; ks++)
                    TcMma<0>(tmemBase + TMEM_S, SmemDesc(qS + ks * UMMA_K_BYTES, 16, 1024, 2),
                             SmemDesc(kS + ks * UMMA_K_BYTES, 16, 1024, 2), iDescS, ks != 0 ? 1u : 0u);
                TcCommit(SmemAddr(&barS));

                ok = MbarWait(SmemAddr(&barP), ph, abortPtr, p.status) &&
                     MbarWait(SmemAddr(&barV), ph, abortPtr, p.status);
                if (ok && it > 0)
                    ok = MbarWait(SmemAddr(&barOFree), (it - 1) & 1u, abortPtr, p.status);
                if (!ok)
                    break;
                TcFenceAfter();
                for (int kb = 0; kb < kBoxes; kb++) {
#pragma unroll
                    for (int ks = 0; ks < 4; ks++)
                        TcMma<0>(tmemBase + TMEM_O,
                                 SmemDesc(pS + kb * P_TILE_BYTES + ks * UMMA_K_BYTES, 16, 1024, 2),
                                 SmemDesc(vS + kb * V_BOX_BYTES + ks * 16 * ROW_BYTES, V_BYTES, 1024, 2),
                                 iDescO, (kb | ks) != 0 ? 1u : 0u);
                }
                TcCommit(SmemAddr(&barO));
            }
        }
    }
    else {
        const int sub = warp & 3;
        const uint32_t laneBase = (uint32_t)(sub * 32) << 16;
        const uint32_t outBox = oS + sub * OUT_BOX_BYTES;
        const uint32_t pRow = (uint32_t)(sub * 32 + lane) * ROW_BYTES;
        uint32_t it = 0;
        bool ok = true;
        for (int item = blockIdx.x; ok && item < p.totalItems; item += gridDim.x, ++it) {
            const uint32_t ph = it & 1u;
            const int blk = item / p.qTiles, qt = item - blk * p.qTiles;
            const int row0 = qt * BM + sub * 32, row = row0 + lane;
            const bool rowOk = row < p.lenQ;
            const float * maskRow = (p.mask != nullptr && rowOk)
                ? p.mask + (long long)blk * p.maskBlockStride + (long long)row * p.lenK : nullptr;

            ok = MbarWaitWarp(SmemAddr(&barS), ph, abortPtr, p.status, 200);
            if (!ok)
                break;
            TcFenceAfter();
            ATTN_MARK(0);
            /* Both passes are written without data-dependent branches and with four
               independent accumulators: a softmax warp has its SM sub-partition to itself,
               so nothing hides the latency of a dependent chain or of a branch. Full
               64-column chunks without a mask take the short path. */
            /* pass 1: row maximum of scale * s + mask over the valid columns */
            float m4[4] = { -INFINITY, -INFINITY, -INFINITY, -INFINITY };
            for (int c0 = 0; c0 < p.kPad; c0 += 64) {
                float v[64];
                TmemLoad64(tmemBase + laneBase + TMEM_S + c0, v);
                if (maskRow == nullptr && c0 + 64 <= p.lenK) {
#pragma unroll
                    for (int e = 0; e < 64; e++)
                        m4[e & 3] = fmaxf(m4[e & 3], v[e] * p.scale);
                }
                else {
#pragma unroll
                    for (int e = 0; e < 64; e++) {
                        const int c = c0 + e;
                        const bool valid = c < p.lenK;
                        float x = v[e] * p.scale;
                        if (maskRow != nullptr)
                            x += valid ? maskRow[c] : 0.f;
                        m4[e & 3] = fmaxf(m4[e & 3], valid ? x : -INFINITY);
                    }
                }
            }
            const float m = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            const float rowLive = m == -INFINITY ? 0.f : 1.f;     /* a fully masked row gives zeros */
            const float mRef = m == -INFINITY ? 0.f : m;
            ATTN_MARK(1);
            /* pass 2: e = exp(x - m), rounded to half; row sum of the rounded values; the
               halves go to shared memory as the K-major, 128-byte-swizzled A operand of P * v */
            float s4[4] = { 0.f, 0.f, 0.f, 0.f };
            for (int c0 = 0; c0 < p.kPad; c0 += 64) {
                float v[64];
                TmemLoad64(tmemBase + laneBase + TMEM_S + c0, v);
                const bool plain = maskRow == nullptr && c0 + 64 <= p.lenK;
                if (plain) {
#pragma unroll
                    for (int e = 0; e < 64; e++)
                        v[e] = __expf(v[e] * p.scale - mRef) * rowLive;
                }
                else {
#pragma unroll
                    for (int e = 0; e < 64; e++) {
                        const int c = c0 + e;
                        const bool valid = c < p.lenK;
                        float x = v[e] * p.scale;
                        if (maskRow != nullptr)
                            x += valid ? maskRow[c] : 0.f;
                        /* x == -inf (masked) gives exp(-inf) = 0 */
                        v[e] = valid ? __expf(x - mRef) * rowLive : 0.f;
                    }
                }
                const uint32_t tile = pS + (c0 / 64) * P_TILE_BYTES + pRow;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    uint32_t w[4];
#pragma unroll
                    for (int h = 0; h < 4; h++) {
                        __half2 hh = __floats2half2_rn(v[j * 8 + h * 2], v[j * 8 + h * 2 + 1]);
                        float2 back = __half22float2(hh);
                        s4[h] += back.x + back.y;
                        w[h] = *(uint32_t *)&hh;
                    }
                    const uint32_t dst = tile + (uint32_t)((j ^ (lane & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                 :: "r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
                }
            }
            const float sum = (s4[0] + s4[1]) + (s4[2] + s4[3]);
            ATTN_MARK(2);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            TcFenceBefore();
            MbarArrive(SmemAddr(&barP));
            ATTN_MARK(3);

            /* the output row: (P * v) / sum */
            ok = MbarWaitWarp(SmemAddr(&barO), ph, abortPtr, p.status, 200);
            if (!ok)
                break;
            TcFenceAfter();
            ATTN_MARK(4);
            float o[64];
            TmemLoad64(tmemBase + laneBase + TMEM_O, o);
            TcFenceBefore();
            __syncwarp();
            if (lane == 0)
                MbarArrive(SmemAddr(&barOFree));
            const float inv = sum > 0.f ? 1.f / sum : 0.f;
            if (lane == 0 && it > 0)
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   /* the box is free again */
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 8; j++) {
                __half2 h0 = __floats2half2_rn(o[j * 8 + 0] * inv, o[j * 8 + 1] * inv);
                __half2 h1 = __floats2half2_rn(o[j * 8 + 2] * inv, o[j * 8 + 3] * inv);
                __half2 h2 = __floats2half2_rn(o[j * 8 + 4] * inv, o[j * 8 + 5] * inv);
                __half2 h3 = __floats2half2_rn(o[j * 8 + 6] * inv, o[j * 8 + 7] * inv);
                const uint32_t dst = outBox + lane * ROW_BYTES + (uint32_t)((j ^ (lane & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                             :: "r"(dst), "r"(*(uint32_t *)&h0), "r"(*(uint32_t *)&h1), "r"(*(uint32_t *)&h2),
                                "r"(*(uint32_t *)&h3) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0 && row0 < p.lenQ) {
                asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                             :: "l"(&tmO), "r"(0), "r"(row0), "r"(blk), "r"(outBox) : "memory");
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
    cuuint64_t strides[2] = { (cuuint64_t)cols * 2, (cuuint64_t)rows * cols * 2 };
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

extern "C" int ntb_attention(int devID, void * stream,
                             const void * q, const void * k, const void * v, const float * mask, void * out,
                             int dtype, int blocks, int lenQ, int lenK, int dim,
                             long long maskBlockStride, float scale)
{
    if (!q || !k || !v || !out || blocks < 0 || lenQ < 0 || lenK < 0 || maskBlockStride < 0)
        return NTB_ERR_ARG;
    if (dtype != NTB_X_FLOAT16)
        return NTB_ERR_DTYPE;
    if (blocks == 0 || lenQ == 0)
        return NTB_OK;
    if (dim != HD || lenK < 1 || lenK > MAX_LK)
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
        CUtensorMap tmQ, tmK, tmV, tmO;
        if ((rc = Encode3D(&tmQ, q, HD, lenQ, blocks, 64, BM)) != NTB_OK ||
            (rc = Encode3D(&tmK, k, HD, lenK, blocks, 64, MAX_LK)) != NTB_OK ||
            (rc = Encode3D(&tmV, v, HD, lenK, blocks, 64, 64)) != NTB_OK ||
            (rc = Encode3D(&tmO, out, HD, lenQ, blocks, 64, 32)) != NTB_OK)
            break;
        AttnParams p;
        memset(&p, 0, sizeof(p));
        p.mask = mask;
        p.maskBlockStride = maskBlockStride;
        p.blocks = blocks; p.lenQ = lenQ; p.lenK = lenK;
        p.qTiles = (lenQ + BM - 1) / BM;
        const long long items = (long long)blocks * p.qTiles;
        if (items > 2147483647LL - 1024) {
            rc = NTB_ERR_LIMIT;
            break;
        }
        p.totalItems = (int)items;
        p.kPad = (lenK + 63) / 64 * 64;
        p.scale = scale;
        p.status = ctx->status;
        static SmemOptIn optIn;
        if (!optIn.Ensure((const void *)AttentionKernel, ATTN_SMEM)) {
            rc = NTB_ERR_CUDA;
            break;
        }
        const int grid = p.totalItems < ctx->smCount ? p.totalItems : ctx->smCount;
        const cudaError_t err = LaunchPdl(AttentionKernel, grid, 192, ATTN_SMEM, (cudaStream_t)stream, tmQ, tmK, tmV, tmO, p);
        CountLaunch();
        rc = (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? NTB_OK : NTB_ERR_CUDA;
    } while (0);
    if (rc == NTB_ERR_CUDA)
        cudaGetLastError();
    if (prev >= 0 && prev != devID)
        cudaSetDevice(prev);
    return rc;
}

#ifdef NTB_WAIT_STATS
extern "C" void ntb_debug_attn_timeline(unsigned long long * out)
{
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, ntb::gAttnTimeline, sizeof(unsigned long long) * 8);
}
#endif
