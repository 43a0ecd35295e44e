/*
 * Device-side building blocks shared by the sm_100a kernels: mbarrier operations with
 * bounded waits, TMA loads and prefetches, tcgen05 fences / commit / MMA, TMEM loads and
 * stores, and the shared-memory and instruction descriptors of tcgen05.mma.
 */
#ifndef NTB_PTX_CUH
#define NTB_PTX_CUH

#include <cuda.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "../../include/ntb_gemm.h"

namespace ntb {

namespace {

constexpr int BM = 128;             /* rows of an output tile = UMMA M = TMEM lanes */
constexpr int ROW_BYTES = 128;      /* one swizzle row: 64 halves or 32 floats of K (or MN) */
constexpr int A_TILE_BYTES = BM * ROW_BYTES;
constexpr int UMMA_K_BYTES = 32;    /* K extent of one tcgen05.mma: 16 halves / 8 tf32 */
constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;   /* about two seconds */

/* The status area of a device is two words: [0] the error code a kernel leaves, [1] a wait
   limit in units of 1024 clocks set by the host for tests of the give-up path (0, the
   normal state: WAIT_LIMIT_CYCLES). Only a wait that is already long reads it. */
__device__ __forceinline__ long long WaitLimit(const int * status)
{
    const int k = ((const volatile int *)status)[1];
    return k > 0 ? ((long long)k << 10) : WAIT_LIMIT_CYCLES;
}

/* ---------------------------------------------------------------- PTX wrappers */

#ifndef NTB_WAIT_HINT_NS
#define NTB_WAIT_HINT_NS 200
#endif

__device__ __forceinline__ uint32_t SmemAddr(const void * p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void MbarInit(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void MbarExpectTx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void MbarArrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}

/* One probe of the barrier. The hardware may park the thread for up to `hintNs`
   nanoseconds while the phase is incomplete (it is woken when the phase completes), which
   keeps waiting warps out of the issue slots. */
__device__ __forceinline__ uint32_t MbarTryWait(uint32_t bar, uint32_t parity, uint32_t hintNs)
{
    uint32_t done;
    if (hintNs == 0) {
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        return done;
    }
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar), "r"(parity), "r"(hintNs) : "memory");
    return done;
}

/* Bounded wait. Returns false when the CTA is aborting (this waiter ran out of time, or
   another one did). */
__device__ __forceinline__ bool MbarWait(uint32_t bar, uint32_t parity, volatile int * abortFlag, int * status,
                                         uint32_t hintNs = NTB_WAIT_HINT_NS)
{
    if (MbarTryWait(bar, parity, hintNs))
        return true;
    const long long t0 = clock64();
    for (uint32_t it = 1; ; ++it) {
        if (MbarTryWait(bar, parity, hintNs))
            return true;
        if ((it & 63u) == 0) {
            if (*abortFlag)
                return false;
            if (clock64() - t0 > WaitLimit(status)) {
                *abortFlag = 1;
                atomicExch(status, NTB_ERR_DEVICE_WAIT);
                return false;
            }
        }
    }
}

/* The same wait for a whole warp: lane 0 polls, the other lanes rest at the warp barrier. */
__device__ __forceinline__ bool MbarWaitWarp(uint32_t bar, uint32_t parity, volatile int * abortFlag, int * status,
                                             uint32_t hintNs)
{
    uint32_t ok = 1;
    if ((threadIdx.x & 31) == 0)
        ok = MbarWait(bar, parity, abortFlag, status, hintNs) ? 1u : 0u;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0;
}

__device__ __forceinline__ void TmaLoad3D(uint32_t dst, const CUtensorMap * map, uint32_t bar, int c0, int c1, int c2)
{
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4, %5}], [%2];"
                 :: "r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

/* asks L2 to fetch a box ahead of the load that will need it: by then the load finds its
   sectors in L2 and completes with L2 latency instead of DRAM latency */
__device__ __forceinline__ void TmaPrefetch3D(const CUtensorMap * map, int c0, int c1, int c2)
{
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global [%0, {%1, %2, %3}];"
                 :: "l"(map), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

/* starts the fetch of a tensor map into the descriptor cache, so that the first copy that
   uses it does not wait for it */
__device__ __forceinline__ void PrefetchTensorMap(const CUtensorMap * map)
{
    asm volatile("prefetch.tensormap [%0];" :: "l"(map) : "memory");
}

__device__ __forceinline__ void TcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcFenceAfter()  { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void TcCommit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}

template <int MODE>
__device__ __forceinline__ void TcMma(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t iDesc, uint32_t accumulate)
{
    if (MODE == 0) {
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                     :: "r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(iDesc), "r"(accumulate) : "memory");
    }
    else {
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                     :: "r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(iDesc), "r"(accumulate) : "memory");
    }
}

/* The same instruction with each shared-memory descriptor given as its two 32-bit halves:
   inside a main loop only the low word (the start address field) changes from one
   instruction to the next, a single 32-bit add. */
template <int MODE>
__device__ __forceinline__ void TcMmaLH(uint32_t dTmem, uint32_t aLo, uint32_t aHi, uint32_t bLo, uint32_t bHi,
                                        uint32_t iDesc, uint32_t accumulate)
{
    if (MODE == 0) {
        asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\t"
                     "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
                     "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
                     :: "r"(dTmem), "r"(aLo), "r"(aHi), "r"(bLo), "r"(bHi), "r"(iDesc), "r"(accumulate) : "memory");
    }
    else {
        asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\t"
                     "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
                     "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %5, p;\n\t}"
                     :: "r"(dTmem), "r"(aLo), "r"(aHi), "r"(bLo), "r"(bHi), "r"(iDesc), "r"(accumulate) : "memory");
    }
}

/* 32 consecutive fp32 columns of this thread's TMEM lane */
__device__ __forceinline__ void TmemLoad32(uint32_t taddr, float * v)
{
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++)
        v[i] = __uint_as_float(r[i]);
}

/* 64 consecutive fp32 columns of this thread's TMEM lane in one instruction */
__device__ __forceinline__ void TmemLoad64(uint32_t taddr, float * v)
{
    uint32_t r[64];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
                 "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
                 "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n\t"
                 "tcgen05.wait::ld.sync.aligned;"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]),
                   "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
                   "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]),
                   "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
                   "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
                 : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 64; i++)
        v[i] = __uint_as_float(r[i]);
}

/* the reverse: 32 values into 32 consecutive columns of this thread's TMEM lane */
__device__ __forceinline__ void TmemStore32(uint32_t taddr, const float * v)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 :: "r"(taddr),
                    "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
                    "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
                    "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
                    "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
                    "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
                    "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
                    "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
                    "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
                 : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

/*
 * Shared-memory matrix descriptor of tcgen05.mma: start address, leading and stride byte
 * offsets in 16-byte units, descriptor version 1, and the swizzle code: 2 = 128-byte
 * swizzle of 16-byte chunks, 1 = 128-byte swizzle of 32-byte chunks (the only swizzled
 * layout the tensor core accepts for MN-major 32-bit operands).
 */
__device__ __forceinline__ uint64_t SmemDesc(uint32_t addr, uint32_t lboBytes, uint32_t sboBytes, uint32_t layout)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lboBytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sboBytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)layout << 61;
    return d;
}

/* Instruction descriptor: fp32 accumulate, operand format, majors, N >> 3, M >> 4. */
__host__ __device__ constexpr uint32_t InstrDesc(int mode, int aMN, int bMN, int n)
{
    return (1u << 4)                                  /* D format: F32 */
         | ((mode == 0 ? 0u : 2u) << 7)               /* A format: F16 = 0, TF32 = 2 */
         | ((mode == 0 ? 0u : 2u) << 10)              /* B format */
         | ((uint32_t)(aMN ? 1 : 0) << 15)
         | ((uint32_t)(bMN ? 1 : 0) << 16)
         | ((uint32_t)(n >> 3) << 17)
         | ((uint32_t)(BM >> 4) << 24);
}

}

}

#endif
