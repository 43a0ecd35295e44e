/*
 * Realigning pre-pass for operands TMA cannot address.
 *
 * A tensor that NiuTensor's memory pool hands out may start at any element and have any row
 * pitch (tensor/XMem.cpp:668-686 packs pieces back to back; XMem.h:60 sets the pitch unit
 * to one byte), while a tensor map needs a 16-byte aligned base and pitches that are
 * multiples of 16 bytes. For every product but the tiniest (from 4e6 flop on: even at
 * 128 x 128 x 256 the copy plus the TMA-fed kernel take 8.5 us against 12.5 us for the
 * loader-warp kernel), each such operand is copied once into 16-byte aligned rows in scratch memory
 * (aligned 16-byte loads, funnel shifts, aligned 16-byte stores: an HBM-bound copy), and the
 * product then runs on the TMA-fed kernels like any other. The tiniest products, and contexts that
 * must not allocate, keep the loader-warp kernel (ntb_tc_ldg.cu), which needs no scratch.
 */
#include <cstdlib>
#include <cstring>

#include "ntb_internal.h"
#include "ntb_tc_common.cuh"
#include "ntb_tc_single.cuh"

namespace ntb {

namespace {

constexpr int REPACK_THREADS = 256;
constexpr int REPACK_PER_THREAD = 8;

struct RepackJob {
    const char * src;
    char * dst;
    int rows, cols;                 /* stored extent of one matrix, in elements */
    long long ld;                   /* source pitch in elements */
    int chunksPerRow;               /* 16-byte units of one destination row */
    int nP, nQ;                     /* matrices along the two batch axes (1 where the stride is 0) */
    long long sP, sQ;               /* source strides in elements */
    long long total;                /* destination chunks in all */
};

/* one or two operands in one launch: blocks 0 .. blocks0-1 copy job[0], the rest job[1] */
struct RepackJobs {
    RepackJob job[2];
    unsigned blocks0;
};

template <int ES>
__global__ void __launch_bounds__(REPACK_THREADS) RepackKernel(const RepackJobs jobs)
{
    constexpr int PER16 = 16 / ES;
    /* the product launched behind this copy may set up meanwhile; this copy itself must not
       read the operands before the kernels ahead of it in the stream, which may have written
       them, are done */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const bool second = blockIdx.x >= jobs.blocks0;
    const RepackJob & j = jobs.job[second ? 1 : 0];
    const long long base = ((long long)(blockIdx.x - (second ? jobs.blocks0 : 0u)) * REPACK_PER_THREAD) * REPACK_THREADS + threadIdx.x;
    /* one 64-bit division per thread; the chunks after the first are reached by stepping
       (column, row) with 32-bit arithmetic */
    const uint32_t cpr = (uint32_t)j.chunksPerRow;
    uint32_t col = (uint32_t)(base % cpr);
    uint32_t rowAll = (uint32_t)(base / cpr);           /* row counted through all matrices (< 2^31, checked by the host) */
    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint4 own[REPACK_PER_THREAD], nxt[REPACK_PER_THREAD];
    uint32_t shift[REPACK_PER_THREAD];
    int valid[REPACK_PER_THREAD];
    /* all loads first, so that each thread has up to 2 x REPACK_PER_THREAD 16-byte requests in flight */
#pragma unroll
    for (int i = 0; i < REPACK_PER_THREAD; i++) {
        const long long idx = base + (long long)i * REPACK_THREADS;
        own[i] = nxt[i] = make_uint4(0u, 0u, 0u, 0u);
        shift[i] = 0u;
        valid[i] = 0;
        if (idx < j.total) {
            const uint32_t row = rowAll % (uint32_t)j.rows, mat = rowAll / (uint32_t)j.rows;
            const uint32_t q = mat % (uint32_t)j.nQ, p = mat / (uint32_t)j.nQ;
            const int left = (j.cols - (int)col * PER16) * ES;     /* bytes of the row from this chunk on */
            valid[i] = left < 0 ? 0 : (left > 16 ? 16 : left);
            if (valid[i] != 0) {
                const uintptr_t g = (uintptr_t)j.src
                                  + (uintptr_t)(((long long)p * j.sP + (long long)q * j.sQ + (long long)row * j.ld + (long long)col * PER16) * ES);
                shift[i] = (uint32_t)(g & 15);
                const uint4 * v = reinterpret_cast<const uint4 *>(g - shift[i]);
                own[i] = __ldg(v);                                  /* holds the byte at g, which is inside the matrix */
                if ((int)shift[i] + valid[i] > 16)
                    nxt[i] = __ldg(v + 1);                          /* holds the byte at g + 16 - shift, inside as well */
            }
        }
        col += REPACK_THREADS;
        rowAll += col / cpr;
        col %= cpr;
    }
#pragma unroll
    for (int i = 0; i < REPACK_PER_THREAD; i++) {
        const long long idx = base + (long long)i * REPACK_THREADS;
        if (idx >= j.total)
            continue;
        const uint4 o = valid[i] ? RealignChunk(own[i], nxt[i], shift[i], 0, valid[i]) : make_uint4(0u, 0u, 0u, 0u);
        reinterpret_cast<uint4 *>(j.dst)[idx] = o;
    }
}

bool NeedsRepack(const void * base, long long ld, long long sP, long long sQ, long long es)
{
    return ((uintptr_t)base & 15) || (ld * es) % 16 || (sP * es) % 16 || (sQ * es) % 16;
}

/* fills job and the replacement pitch / strides of one operand; returns the scratch bytes */
size_t PlanOperand(const void * src, int rows, int cols, long long ld, long long sP, long long sQ, int P, int Q,
                   int es, RepackJob & job, long long * ldOut, long long * sPOut, long long * sQOut)
{
    const int per16 = 16 / es;
    job.src = (const char *)src;
    job.rows = rows; job.cols = cols; job.ld = ld;
    job.chunksPerRow = (cols + per16 - 1) / per16;
    job.nP = sP ? P : 1;
    job.nQ = sQ ? Q : 1;
    job.sP = sP; job.sQ = sQ;
    job.total = (long long)job.chunksPerRow * rows * job.nP * job.nQ;   /* LaunchRepacked refuses more than 2^31 rows in all */
    *ldOut = (long long)job.chunksPerRow * per16;
    const long long mat = *ldOut * rows;
    *sQOut = sQ ? mat : 0;
    *sPOut = sP ? mat * job.nQ : 0;
    return (size_t)job.total * 16;
}

unsigned BlocksOf(const RepackJob & job)
{
    const long long perBlock = (long long)REPACK_THREADS * REPACK_PER_THREAD;
    return (unsigned)((job.total + perBlock - 1) / perBlock);
}

int LaunchJobs(const RepackJob * a, const RepackJob * b, int es, cudaStream_t stream)
{
    RepackJobs jobs;
    memset(&jobs, 0, sizeof(jobs));
    const RepackJob * first = a ? a : b, * second = a && b ? b : nullptr;
    if (first->total + (second ? second->total : 0) > (1LL << 40))
        return NTB_ERR_LIMIT;
    jobs.job[0] = *first;
    jobs.blocks0 = BlocksOf(*first);
    unsigned blocks = jobs.blocks0;
    if (second) {
        jobs.job[1] = *second;
        blocks += BlocksOf(*second);
    }
    const cudaError_t err = es == 2 ? LaunchPdl(RepackKernel<2>, (int)blocks, REPACK_THREADS, 0, stream, jobs)
                                    : LaunchPdl(RepackKernel<4>, (int)blocks, REPACK_THREADS, 0, stream, jobs);
    CountLaunch();
    return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? NTB_OK : NTB_ERR_CUDA;
}

}

bool RepackWorthwhile(const DeviceCtx & ctx, const Problem & p)
{
    if (!ctx.mayAllocate || p.count <= 0 || p.Q <= 0)
        return false;
    const double flop = 2.0 * p.M * p.N * p.K * p.count;
    const char * knob = getenv("NTB_REPACK_MIN_MFLOP");         /* tuning: threshold in units of 1e6 flop */
    const double least = knob && *knob ? atof(knob) * 1.0e6 : 4.0e6;    /* measured: the copy wins from 128 x 128 x 256 (8.4e6 flop) on */
    return flop >= least;
}

/* NTB_ERR_ARG: not applicable after all (the caller keeps the loader-warp kernel) */
int LaunchRepacked(const DeviceCtx & ctx, const Problem & p, cudaStream_t stream, int * route)
{
    const int es = (int)ElemSize(p.dtAB);
    const int P = p.count / p.Q;
    Problem q = p;
    RepackJob jobA, jobB;
    const bool doA = NeedsRepack(p.a, p.lda, p.sAp, p.sAq, es);
    const bool doB = NeedsRepack(p.b, p.ldb, p.sBp, p.sBq, es);
    size_t bytesA = 0, bytesB = 0;
    if (doA)
        bytesA = PlanOperand(p.a, p.aRows, p.aCols, p.lda, p.sAp, p.sAq, P, p.Q, es, jobA, &q.lda, &q.sAp, &q.sAq);
    if (doB)
        bytesB = PlanOperand(p.b, p.bRows, p.bCols, p.ldb, p.sBp, p.sBq, P, p.Q, es, jobB, &q.ldb, &q.sBp, &q.sBq);
    if ((!doA && !doB) || bytesA + bytesB > ((size_t)4 << 30))
        return NTB_ERR_ARG;
    /* the copy kernel counts rows through all matrices of an operand in 32 bits */
    if ((doA && (long long)p.aRows * jobA.nP * jobA.nQ >= (1LL << 31)) || (doB && (long long)p.bRows * jobB.nP * jobB.nQ >= (1LL << 31)))
        return NTB_ERR_ARG;
    int rc = ScratchAcquire(ctx, stream);
    if (rc != NTB_OK)
        return rc;
    void * bufA = nullptr, * bufB = nullptr;
    if (doA && (rc = EnsureScratch(ctx, 0, bytesA, &bufA)) != NTB_OK)
        return rc;
    if (doB && (rc = EnsureScratch(ctx, 1, bytesB, &bufB)) != NTB_OK)
        return rc;
    if (doA) { jobA.dst = (char *)bufA; q.a = bufA; }
    if (doB) { jobB.dst = (char *)bufB; q.b = bufB; }
    if (!TcEligible(q))
        return NTB_ERR_ARG;                         /* nothing launched yet */
    if ((rc = LaunchJobs(doA ? &jobA : nullptr, doB ? &jobB : nullptr, es, stream)) != NTB_OK)
        return rc;
    CountVariant(NTB_COUNT_REPACK);
    rc = LaunchTc(ctx, q, stream, route);
    const int rel = ScratchRelease(ctx, stream);
    return rc != NTB_OK ? rc : rel;
}

}
