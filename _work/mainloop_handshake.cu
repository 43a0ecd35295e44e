/*
 * Micro-benchmarks of what one main-loop iteration costs the threads of a tcgen05 GEMM on
 * one SM: barrier probes, tcgen05.mma issue rate, and the hand-shake between a producer
 * thread and the MMA-issuing thread. One CTA, timed with clock64 by the thread under test.
 * Every wait is bounded by an iteration count, after which the kernel carries on and ends.
 *
 *   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o handshake mainloop_handshake.cu && ./handshake
 *
 * The constants of the tile cost model in ../csrc/ntb_tc.cu come from these numbers.
 */
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>

__device__ __forceinline__ uint32_t sa(const void * p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void init(uint32_t b, uint32_t c)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(b), "r"(c) : "memory");
}
__device__ __forceinline__ void arrive(uint32_t b)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(b) : "memory");
}
__device__ __forceinline__ uint32_t trywait(uint32_t b, uint32_t par)
{
    uint32_t d;
    asm volatile("{.reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0,1,0,p;}"
                 : "=r"(d) : "r"(b), "r"(par) : "memory");
    return d;
}
__device__ __forceinline__ void waitb(uint32_t b, uint32_t par)
{
    int g = 0;
    while (!trywait(b, par) && ++g < 1000000) { }
}
__device__ __forceinline__ void commit(uint32_t b)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(b) : "memory");
}
/* K-major operand tile of 128-byte rows, 128-byte swizzle */
__device__ __forceinline__ uint64_t desc(uint32_t addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)64 << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ uint32_t idesc(int n) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24); }
__device__ __forceinline__ void mma(uint32_t tm, uint64_t a, uint64_t b, uint32_t id)
{
    asm volatile("{.reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;}"
                 :: "r"(tm), "l"(a), "l"(b), "r"(id), "r"(1) : "memory");
}

/*
 * MODE 0: MMAs back to back.                      MODE 1: KS MMAs + commit, no wait.
 * MODE 2: try_wait (barrier completed by this thread's commit five stages ago), KS MMAs, commit.
 * MODE 3: as 2 with a plain ld.shared of a flag instead of the barrier probe.
 * MODE 4: as 2, result of the probe never branched on.
 * MODE 5: KS MMAs, commit, wait for that commit.
 * MODE 6: producer thread (warp 0: try_wait empty, arrive full) against this thread
 *         (try_wait full, KS MMAs, commit empty), ring of 6 stages.
 */
template <int N, int MODE, int KS>
__global__ void bench(int iters, long long * out)
{
    constexpr int ST = 6;
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t full[8], empty[8];
    __shared__ uint32_t slot;
    __shared__ volatile uint32_t flag[8];
    for (int i = threadIdx.x; i < (16384 + N * 128) / 4; i += blockDim.x)
        ((uint32_t *)smem)[i] = 0;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 8; i++) { init(sa(&full[i]), 1); init(sa(&empty[i]), 1); flag[i] = 1; }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t tm = 0;
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" :: "r"(sa(&slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        __syncwarp();
        tm = *(volatile uint32_t *)&slot;
    }
    const long long t0 = clock64();
    if (warp == 0 && lane == 0 && MODE == 6) {
        int s = 0; uint32_t ph = 0;
        for (int i = 0; i < iters; i++) {
            waitb(sa(&empty[s]), ph ^ 1);
            arrive(sa(&full[s]));
            if (++s == ST) { s = 0; ph ^= 1; }
        }
    }
    if (warp == 1 && lane == 0) {
        const uint32_t base = (sa(smem) + 1023) & ~1023u;
        const uint64_t aD = desc(base), bD = desc(base + 16384);
        const uint32_t id = idesc(N);
        int s = 0; uint32_t ph = 0, acc = 0;
        for (int i = 0; i < iters; i++) {
            int g = 0;
            if (MODE == 2) waitb(sa(&empty[s]), ph ^ 1);
            if (MODE == 3) { while (!flag[s] && ++g < 1000000) { } }
            if (MODE == 4) acc += trywait(sa(&empty[s]), ph ^ 1);
            if (MODE == 6) { waitb(sa(&full[s]), ph); asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
#pragma unroll
            for (int k = 0; k < KS; k++)
                mma(tm, aD + (k & 3) * 2, bD + (k & 3) * 2, id);
            if (MODE != 0)
                commit(sa(&empty[s]));
            if (MODE == 5) waitb(sa(&empty[s]), ph);
            if (++s == ST) { s = 0; ph ^= 1; }
        }
        out[0] = clock64() - t0;
        out[1] = acc;
        commit(sa(&full[7]));
        waitb(sa(&full[7]), 0);
    }
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" :: "r"(tm) : "memory");
}

/* latencies of single barrier operations, one thread, dependent chains */
__global__ void latency(int iters, long long * out)
{
    __shared__ __align__(8) uint64_t bar[4];
    if (threadIdx.x == 0) {
        for (int i = 0; i < 4; i++) init(sa(&bar[i]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        uint32_t acc = 0;
        long long t0 = clock64();
        for (int i = 0; i < iters; i++) acc += trywait(sa(&bar[0]), 1);
        out[0] = clock64() - t0;
        t0 = clock64();
        for (int i = 0; i < iters; i++) arrive(sa(&bar[1]));
        out[1] = clock64() - t0;
        out[7] = acc;
    }
}

static long long * d;
static long long h[8];
static const int ITERS = 4000;

template <int N, int MODE, int KS>
void run(const char * what)
{
    cudaFuncSetAttribute(bench<N, MODE, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 70000);
    bench<N, MODE, KS><<<1, 64, 70000>>>(ITERS, d);
    cudaDeviceSynchronize();
    bench<N, MODE, KS><<<1, 64, 70000>>>(ITERS, d);
    cudaMemcpy(h, d, 64, cudaMemcpyDeviceToHost);
    printf("N %3d, %d MMAs per iteration: %-58s %7.1f clk per iteration (math %d) [%s]\n", N, KS, what,
           (double)h[0] / ITERS, N / 2 * KS, cudaGetErrorString(cudaGetLastError()));
}

int main()
{
    cudaMalloc(&d, 64);
    latency<<<1, 32>>>(ITERS, d);
    cudaMemcpy(h, d, 64, cudaMemcpyDeviceToHost);
    printf("try_wait on a completed phase %.1f clk, arrive %.1f clk [%s]\n", (double)h[0] / ITERS, (double)h[1] / ITERS,
           cudaGetErrorString(cudaGetLastError()));
    run<64, 0, 4>("MMAs back to back");
    run<128, 0, 4>("MMAs back to back");
    run<256, 0, 4>("MMAs back to back");
    run<128, 1, 4>("MMAs + commit");
    run<128, 2, 4>("try_wait, MMAs, commit");
    run<64, 2, 4>("try_wait, MMAs, commit");
    run<128, 3, 4>("ld.shared flag, MMAs, commit");
    run<128, 4, 4>("try_wait (result unused), MMAs, commit");
    run<128, 5, 4>("MMAs, commit, wait for it");
    run<256, 5, 4>("MMAs, commit, wait for it");
    run<64, 6, 4>("producer thread against MMA thread, 6 stages");
    run<128, 6, 4>("producer thread against MMA thread, 6 stages");
    run<256, 6, 4>("producer thread against MMA thread, 6 stages");
    run<128, 6, 8>("producer thread against MMA thread, 6 stages");
    cudaFree(d);
    return 0;
}
