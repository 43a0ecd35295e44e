/*
 * FFMA route: a tiled SIMT GEMM for operands the TMA-fed tensor-core route cannot
 * address -- base pointers that are not 16-byte aligned (NiuTensor's XMem pools carve
 * pieces back to back without padding, source/tensor/XMem.cpp:672-685), row pitches
 * that are not multiples of 16 bytes, or K == 0. It reads elements one by one through
 * generic (row, column) strides, so any layout the C ABI can describe works here.
 * Products are accumulated in fp32 with fused multiply-add.
 */
#include "ntb_internal.h"
#include <cuda_fp16.h>

namespace ntb {

namespace {

constexpr int TM = 64, TN = 64, TK = 16, NTHREADS = 256;

struct SimtParams {
    const void * a;
    const void * b;
    void * c;
    long long sAm, sAk, sBn, sBk, ldc;
    long long sAp, sAq, sBp, sBq, sCp, sCq;
    int M, N, K, count, Q, tilesM, tilesN;
    int aMN, bMN;
    float alpha, beta;
    const void * bias;
    int act;
};

template <typename T> __device__ __forceinline__ float ToF(T x);
template <> __device__ __forceinline__ float ToF<float>(float x) { return x; }
template <> __device__ __forceinline__ float ToF<__half>(__half x) { return __half2float(x); }
template <typename T> __device__ __forceinline__ T FromF(float x);
template <> __device__ __forceinline__ float FromF<float>(float x) { return x; }
template <> __device__ __forceinline__ __half FromF<__half>(float x) { return __float2half_rn(x); }

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(NTHREADS) GemmSimtKernel(SimtParams p)
{
    /* a product launched behind this kernel with programmatic serialisation may start setting up */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ float As[TK][TM + 4];
    __shared__ float Bs[TK][TN + 4];

    const int tid = threadIdx.x;
    long long tile = blockIdx.x;
    const int tn = (int)(tile % p.tilesN);
    tile /= p.tilesN;
    const int tm = (int)(tile % p.tilesM);
    const int prob = (int)(tile / p.tilesM);
    const int pp = prob / p.Q, qq = prob % p.Q;

    const TIn * A = (const TIn *)p.a + pp * p.sAp + qq * p.sAq;
    const TIn * B = (const TIn *)p.b + pp * p.sBp + qq * p.sBq;
    TOut * C = (TOut *)p.c + pp * p.sCp + qq * p.sCq;

    const int m0 = tm * TM, n0 = tn * TN;
    const int tx = tid % 16, ty = tid / 16;   /* 16 x 16 threads, 4 x 4 outputs each */

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
            acc[i][j] = 0.f;

    for (int k0 = 0; k0 < p.K; k0 += TK) {
        /* the contiguous direction of each operand goes across neighbouring threads */
#pragma unroll
        for (int r = 0; r < (TM * TK) / NTHREADS; r++) {
            int e = r * NTHREADS + tid;
            int mm, kk;
            if (p.aMN) { mm = e % TM; kk = e / TM; }
            else       { kk = e % TK; mm = e / TK; }
            int gm = m0 + mm, gk = k0 + kk;
            float v = 0.f;
            if (gm < p.M && gk < p.K)
                v = ToF<TIn>(A[gm * p.sAm + gk * p.sAk]);
            As[kk][mm] = v;
        }
#pragma unroll
        for (int r = 0; r < (TN * TK) / NTHREADS; r++) {
            int e = r * NTHREADS + tid;
            int nn, kk;
            if (p.bMN) { nn = e % TN; kk = e / TN; }
            else       { kk = e % TK; nn = e / TK; }
            int gn = n0 + nn, gk = k0 + kk;
            float v = 0.f;
            if (gn < p.N && gk < p.K)
                v = ToF<TIn>(B[gn * p.sBn + gk * p.sBk]);
            Bs[kk][nn] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; kk++) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; i++)
                av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++)
                bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++)
                    acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; i++) {
        int gm = m0 + ty * 4 + i;
        if (gm >= p.M)
            continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int gn = n0 + tx * 4 + j;
            if (gn >= p.N)
                continue;
            TOut * dst = C + gm * p.ldc + gn;
            float v = p.alpha * acc[i][j];
            if (p.beta != 0.f)
                v = fmaf(p.beta, ToF<TOut>(*dst), v);
            if (p.bias != nullptr)
                v += ToF<TOut>(((const TOut *)p.bias)[gn]);
            if (p.act == NTB_ACT_RECTIFY)
                v = fmaxf(v, 0.f);
            *dst = FromF<TOut>(v);
        }
    }
}

}

int LaunchSimt(const DeviceCtx & ctx, const Problem & pr, cudaStream_t stream)
{
    (void)ctx;
    SimtParams p;
    p.a = pr.a; p.b = pr.b; p.c = pr.c;
    p.sAm = pr.aMN ? 1 : pr.lda;  p.sAk = pr.aMN ? pr.lda : 1;
    p.sBn = pr.bMN ? 1 : pr.ldb;  p.sBk = pr.bMN ? pr.ldb : 1;
    p.ldc = pr.ldc;
    p.sAp = pr.sAp; p.sAq = pr.sAq; p.sBp = pr.sBp; p.sBq = pr.sBq; p.sCp = pr.sCp; p.sCq = pr.sCq;
    p.M = pr.M; p.N = pr.N; p.K = pr.K; p.count = pr.count; p.Q = pr.Q;
    p.tilesM = (pr.M + TM - 1) / TM;
    p.tilesN = (pr.N + TN - 1) / TN;
    p.aMN = pr.aMN; p.bMN = pr.bMN;
    p.alpha = pr.alpha; p.beta = pr.beta;
    p.bias = pr.bias; p.act = pr.act;
    long long tiles = (long long)p.tilesM * p.tilesN * pr.count;
    if (tiles <= 0)
        return NTB_OK;
    if (tiles > 2147483647LL)
        return NTB_ERR_LIMIT;
    dim3 grid((unsigned)tiles), block(NTHREADS);
    if (pr.dtAB == NTB_X_FLOAT16 && pr.dtC == NTB_X_FLOAT16)
        GemmSimtKernel<__half, __half><<<grid, block, 0, stream>>>(p);
    else if (pr.dtAB == NTB_X_FLOAT16 && pr.dtC == NTB_X_FLOAT)
        GemmSimtKernel<__half, float><<<grid, block, 0, stream>>>(p);
    else if (pr.dtAB == NTB_X_FLOAT && pr.dtC == NTB_X_FLOAT)
        GemmSimtKernel<float, float><<<grid, block, 0, stream>>>(p);
    else
        return NTB_ERR_DTYPE;
    CountLaunch();
    return cudaGetLastError() == cudaSuccess ? NTB_OK : NTB_ERR_CUDA;
}

}
