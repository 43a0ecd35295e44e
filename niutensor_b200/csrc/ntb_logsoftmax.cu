/*
 * Row-wise log-softmax in two halves, so that a row may be spread over several GPUs
 * (the vocabulary-sharded output layer): ntb_row_stats gives, per row of the local shard,
 * the maximum and the sum of exp(x - maximum); the caller combines these across shards
 * (an all-reduce of two floats per row instead of a gather of the logits) and
 * ntb_logsoftmax_apply writes log(exp(x - max) / sum) with the reference's clamps
 * (source/tensor/function/LogSoftmax.cpp:133-148: values below LOGPROB_MIN = -20, NaN and
 * infinities become -20; a row whose sum is 0 becomes zeros). On one GPU the two calls in
 * a row are the reference's LogSoftmax over the last dimension
 * (source/sample/transformer/submodel/Output.cpp:86-101 applies it to the output layer's
 * product). Both kernels stream the shard once with 16-byte loads: they are HBM-bound.
 */
#include "ntb_internal.h"
#include <cuda_fp16.h>
#include <cmath>

namespace ntb {

namespace {

constexpr int LS_THREADS = 256;
constexpr float LOGPROB_FLOOR = -20.0f;       /* LOGPROB_MIN, source/tensor/XGlobal.h:69 */

template <typename T> struct Pack;
template <> struct Pack<__half> { static constexpr int N = 8; };
template <> struct Pack<float>  { static constexpr int N = 4; };

__device__ __forceinline__ void Load16(const __half * p, float * v)
{
    uint4 u = *(const uint4 *)p;
    float2 f;
    f = __half22float2(*(__half2 *)&u.x); v[0] = f.x; v[1] = f.y;
    f = __half22float2(*(__half2 *)&u.y); v[2] = f.x; v[3] = f.y;
    f = __half22float2(*(__half2 *)&u.z); v[4] = f.x; v[5] = f.y;
    f = __half22float2(*(__half2 *)&u.w); v[6] = f.x; v[7] = f.y;
}
__device__ __forceinline__ void Load16(const float * p, float * v)
{
    float4 f = *(const float4 *)p;
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}
__device__ __forceinline__ void Store16(__half * p, const float * v)
{
    uint4 u;
    __half2 h0 = __floats2half2_rn(v[0], v[1]), h1 = __floats2half2_rn(v[2], v[3]);
    __half2 h2 = __floats2half2_rn(v[4], v[5]), h3 = __floats2half2_rn(v[6], v[7]);
    u.x = *(uint32_t *)&h0; u.y = *(uint32_t *)&h1; u.z = *(uint32_t *)&h2; u.w = *(uint32_t *)&h3;
    *(uint4 *)p = u;
}
__device__ __forceinline__ void Store16(float * p, const float * v)
{
    *(float4 *)p = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ float ToFloat(__half x) { return __half2float(x); }
__device__ __forceinline__ float ToFloat(float x) { return x; }
__device__ __forceinline__ void FromFloat(__half * p, float v) { *p = __float2half_rn(v); }
__device__ __forceinline__ void FromFloat(float * p, float v) { *p = v; }

/* running (max, sum of exp(x - max)) with one more value */
__device__ __forceinline__ void Online(float & m, float & s, float x)
{
    if (x > m) {
        s = s * __expf(m - x) + 1.f;
        m = x;
    }
    else if (x != -INFINITY) {
        s += __expf(x - m);
    }
}

__device__ __forceinline__ void Merge(float & m, float & s, float m2, float s2)
{
    const float mm = fmaxf(m, m2);
    if (mm == -INFINITY) {
        s = 0.f;
        return;
    }
    s = s * __expf(m - mm) + s2 * __expf(m2 - mm);
    m = mm;
}

/* one CTA per row */
template <typename T>
__global__ void __launch_bounds__(LS_THREADS) RowStatsKernel(const T * x, int cols, long long ld, bool vec,
                                                             float * rowMax, float * rowSum)
{
    /* a product launched behind this kernel with programmatic serialisation may start setting up */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int PN = Pack<T>::N;
    const T * row = x + (long long)blockIdx.x * ld;
    float m = -INFINITY, s = 0.f;
    const int packs = vec ? cols / PN : 0;
    for (int i = threadIdx.x; i < packs; i += LS_THREADS) {
        float v[PN];
        Load16(row + i * PN, v);
        float pm = v[0];
#pragma unroll
        for (int e = 1; e < PN; e++)
            pm = fmaxf(pm, v[e]);
        if (pm != -INFINITY) {
            float ps = 0.f;
#pragma unroll
            for (int e = 0; e < PN; e++)
                ps += __expf(v[e] - pm);
            Merge(m, s, pm, ps);
        }
    }
    for (int c = packs * PN + threadIdx.x; c < cols; c += LS_THREADS)
        Online(m, s, ToFloat(row[c]));

    __shared__ float sm[LS_THREADS / 32], ss[LS_THREADS / 32];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, off), s2 = __shfl_xor_sync(0xffffffffu, s, off);
        Merge(m, s, m2, s2);
    }
    if ((threadIdx.x & 31) == 0) {
        sm[threadIdx.x >> 5] = m;
        ss[threadIdx.x >> 5] = s;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < LS_THREADS / 32; w++)
            Merge(m, s, sm[w], ss[w]);
        rowMax[blockIdx.x] = m;
        rowSum[blockIdx.x] = s;
    }
}

template <typename T>
__global__ void __launch_bounds__(LS_THREADS) LogSoftmaxApplyKernel(const T * x, T * y, int cols, long long ldx, long long ldy,
                                                                   bool vec, const float * rowMax, const float * rowSum)
{
    /* a product launched behind this kernel with programmatic serialisation may start setting up */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int PN = Pack<T>::N;
    const T * in = x + (long long)blockIdx.y * ldx;
    T * out = y + (long long)blockIdx.y * ldy;
    const float m = rowMax[blockIdx.y], s = rowSum[blockIdx.y];
    const bool dead = !(s > 0.f);                       /* sum 0 (or NaN): the reference writes zeros */
    const float shift = dead ? 0.f : m + logf(s);
    auto value = [&](float xv) {
        if (dead)
            return 0.f;
        float r = xv - shift;
        if (isnan(r) || isinf(r))
            r = LOGPROB_FLOOR;
        return fmaxf(r, LOGPROB_FLOOR);
    };
    const int packs = vec ? cols / PN : 0;
    for (int i = blockIdx.x * LS_THREADS + threadIdx.x; i < packs; i += gridDim.x * LS_THREADS) {
        float v[PN];
        Load16(in + i * PN, v);
#pragma unroll
        for (int e = 0; e < PN; e++)
            v[e] = value(v[e]);
        Store16(out + i * PN, v);
    }
    for (int c = packs * PN + blockIdx.x * LS_THREADS + threadIdx.x; c < cols; c += gridDim.x * LS_THREADS)
        FromFloat(out + c, value(ToFloat(in[c])));
}

bool Aligned16(const void * p, long long ld, int es)
{
    return (((uintptr_t)p) & 15) == 0 && (ld * es) % 16 == 0;
}

struct Guard {
    int prev;
    bool ok;
    explicit Guard(int dev) : prev(-1), ok(false)
    {
        if (cudaGetDevice(&prev) != cudaSuccess)
            return;
        ok = prev == dev || cudaSetDevice(dev) == cudaSuccess;
        if (!ok)
            prev = -1;
    }
    ~Guard()
    {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev)
            cudaSetDevice(prev);
    }
};

}

}

using namespace ntb;

extern "C" int ntb_row_stats(int devID, void * stream, const void * x, int dtype, int rows, int cols, long long ld,
                             float * rowMax, float * rowSumExp)
{
    if (rows < 0 || cols < 0 || ld < cols)
        return NTB_ERR_ARG;
    if (dtype != NTB_X_FLOAT16 && dtype != NTB_X_FLOAT)
        return NTB_ERR_DTYPE;
    if (rows == 0)
        return NTB_OK;
    if (!x || !rowMax || !rowSumExp)
        return NTB_ERR_ARG;
    Guard g(devID);
    if (!g.ok) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == NTB_X_FLOAT16)
        RowStatsKernel<__half><<<rows, LS_THREADS, 0, st>>>((const __half *)x, cols, ld, Aligned16(x, ld, 2), rowMax, rowSumExp);
    else
        RowStatsKernel<float><<<rows, LS_THREADS, 0, st>>>((const float *)x, cols, ld, Aligned16(x, ld, 4), rowMax, rowSumExp);
    CountLaunch();
    return cudaGetLastError() == cudaSuccess ? NTB_OK : NTB_ERR_CUDA;
}

extern "C" int ntb_logsoftmax_apply(int devID, void * stream, const void * x, void * y, int dtype,
                                    int rows, int cols, long long ldx, long long ldy,
                                    const float * rowMax, const float * rowSumExp)
{
    if (rows < 0 || cols < 0 || ldx < cols || ldy < cols)
        return NTB_ERR_ARG;
    if (dtype != NTB_X_FLOAT16 && dtype != NTB_X_FLOAT)
        return NTB_ERR_DTYPE;
    if (rows == 0 || cols == 0)
        return NTB_OK;
    if (!x || !y || !rowMax || !rowSumExp)
        return NTB_ERR_ARG;
    if (rows > 65535)
        return NTB_ERR_LIMIT;
    Guard g(devID);
    if (!g.ok) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    cudaStream_t st = (cudaStream_t)stream;
    const int es = dtype == NTB_X_FLOAT16 ? 2 : 4;
    const bool vec = Aligned16(x, ldx, es) && Aligned16(y, ldy, es);
    const int perRow = (cols / (16 / es) + LS_THREADS - 1) / LS_THREADS;
    dim3 grid((unsigned)(perRow < 1 ? 1 : perRow > 64 ? 64 : perRow), (unsigned)rows);
    if (dtype == NTB_X_FLOAT16)
        LogSoftmaxApplyKernel<__half><<<grid, LS_THREADS, 0, st>>>((const __half *)x, (__half *)y, cols, ldx, ldy, vec, rowMax, rowSumExp);
    else
        LogSoftmaxApplyKernel<float><<<grid, LS_THREADS, 0, st>>>((const float *)x, (float *)y, cols, ldx, ldy, vec, rowMax, rowSumExp);
    CountLaunch();
    return cudaGetLastError() == cudaSuccess ? NTB_OK : NTB_ERR_CUDA;
}
