/*
 * One product sharded over several GPUs of ONE process (the process model of NiuTensor's
 * trainer: one process, one worker thread per device, source/train/XWorkerJob.cpp), and the
 * helper that puts column shards gathered by a collective back into row-major order.
 *
 * ntb_gemm_sharded: output tiles are independent, so the product shards with no exchange --
 * device d multiplies the replicated a by its own columns of op(b) (or its own part of the
 * batch) on its own stream. When the caller wants the whole c on every device, the
 * epilogues of the column-sharded products write their tiles straight into every device's
 * copy of c over NVLink (ntb_gemm_peers), so no separate gather pass exists; batch shards
 * are contiguous and go out as one peer copy per destination. The reference's only way to
 * bring tensors of several devices together is a whole-tensor device-to-device cudaMemcpy
 * after the operator (source/tensor/XUtility.cpp:196-201, source/train/XWorkerCollect.cpp:
 * 59-78).
 */
#include "ntb_internal.h"
#include <mutex>
#include <cstring>

namespace ntb {

namespace {

constexpr int MAX_SHARDS = NTB_MAX_PEERS + 1;
constexpr int MAX_DEV = 64;

std::mutex gEventLock;
cudaEvent_t gDone[MAX_SHARDS][MAX_DEV];       /* per shard slot and device, created on first use */
bool gHaveEvent[MAX_SHARDS][MAX_DEV];

/* the caller has made `dev` current */
int EventFor(int slot, int dev, cudaEvent_t * ev)
{
    std::lock_guard<std::mutex> g(gEventLock);
    if (!gHaveEvent[slot][dev]) {
        if (cudaEventCreateWithFlags(&gDone[slot][dev], cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            return NTB_ERR_CUDA;
        }
        gHaveEvent[slot][dev] = true;
    }
    *ev = gDone[slot][dev];
    return NTB_OK;
}

/* lets the current device `dev` address the memory of `peer` */
int EnablePeer(int dev, int peer)
{
    if (dev == peer)
        return NTB_OK;
    int can = 0;
    if (cudaDeviceCanAccessPeer(&can, dev, peer) != cudaSuccess || !can) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
    if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    cudaGetLastError();
    return NTB_OK;
}

/* dst[r][s * w + j] = src[s][r][j] for 16-byte units j: column shards stored one after the
   other (what an all-gather of packed shards leaves) become one row-major matrix */
__global__ void __launch_bounds__(256)
UnshardColumnsKernel(const uint4 * __restrict__ src, uint4 * __restrict__ dst, long long rows, int shards, int unitsPerShardRow,
                     long long dstPitchUnits)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const long long perShard = rows * unitsPerShardRow;
    const long long total = perShard * shards;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        /* walk the destination in order, so that stores are contiguous */
        const long long r = i / ((long long)unitsPerShardRow * shards);
        const int rest = (int)(i - r * (long long)unitsPerShardRow * shards);
        const int s = rest / unitsPerShardRow, j = rest - s * unitsPerShardRow;
        dst[r * dstPitchUnits + (long long)s * unitsPerShardRow + j] = src[(long long)s * perShard + r * unitsPerShardRow + j];
    }
}

}

}

using namespace ntb;

extern "C" {

void ntb_shard_range(int total, int shards, int shard, int multiple, int * lo, int * hi)
{
    int l = 0, h = 0;
    if (total > 0 && shards > 0 && shard >= 0 && shard < shards) {
        if (multiple < 1)
            multiple = 1;
        const long long blocks = ((long long)total + multiple - 1) / multiple;
        long long a = blocks * shard / shards * multiple, b = blocks * (shard + 1) / shards * multiple;
        l = (int)(a < total ? a : total);
        h = (int)(b < total ? b : total);
    }
    if (lo) *lo = l;
    if (hi) *hi = h;
}

int ntb_unshard_columns(int devID, void * stream, const void * src, void * dst, int dtype,
                        long long rows, int shards, int colsPerShard, long long ldDst)
{
    if (dtype != NTB_X_FLOAT16 && dtype != NTB_X_FLOAT)
        return NTB_ERR_DTYPE;
    if (rows < 0 || shards < 0 || colsPerShard < 0 || ldDst < (long long)shards * colsPerShard)
        return NTB_ERR_ARG;
    if (rows == 0 || shards == 0 || colsPerShard == 0)
        return NTB_OK;
    if (!src || !dst)
        return NTB_ERR_ARG;
    const long long es = (long long)ElemSize(dtype);
    if (((uintptr_t)src & 15) || ((uintptr_t)dst & 15) || (colsPerShard * es) % 16 || (ldDst * es) % 16)
        return NTB_ERR_ARG;                         /* shards are moved in 16-byte units */
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess || (prev != devID && cudaSetDevice(devID) != cudaSuccess)) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    int rc = NTB_ERR_CUDA;
    DeviceCtx * ctx = CtxFor(devID);
    if (ctx) {
        const int units = (int)(colsPerShard * es / 16);
        const long long total = rows * units * shards;
        long long blocks = (total + 255) / 256;
        const long long cap = (long long)ctx->smCount * 16;
        if (blocks > cap)
            blocks = cap;
        const cudaError_t e = LaunchPdl(UnshardColumnsKernel, (int)blocks, 256, 0, (cudaStream_t)stream,
                                        (const uint4 *)src, (uint4 *)dst, rows, shards, units, ldDst * es / 16);
        CountLaunch();
        rc = (e == cudaSuccess && cudaGetLastError() == cudaSuccess) ? NTB_OK : NTB_ERR_CUDA;
    }
    if (rc == NTB_ERR_CUDA)
        cudaGetLastError();
    if (prev >= 0 && prev != devID)
        cudaSetDevice(prev);
    return rc;
}

int ntb_gemm_sharded(const int * devIDs, int nDev, void * const * streams,
                     const void * const * a, int transA, const void * const * b, int transB, void * const * c,
                     int dtypeAB, int dtypeC,
                     int na, int ma, int nb, int mb, int nc, int mc,
                     int count, int shardAxis, int gather, float alpha, float beta)
{
    if (!devIDs || !a || !b || !c || nDev < 1 || count < 0)
        return NTB_ERR_ARG;
    if (nDev > MAX_SHARDS)
        return NTB_ERR_LIMIT;
    if (shardAxis != NTB_SHARD_COLUMNS && shardAxis != NTB_SHARD_BATCH)
        return NTB_ERR_ARG;
    if ((transA != NTB_X_TRANS && transA != NTB_X_NOTRANS) || (transB != NTB_X_TRANS && transB != NTB_X_NOTRANS))
        return NTB_ERR_ARG;
    if (na < 0 || ma < 0 || nb < 0 || mb < 0 || nc < 0 || mc < 0)
        return NTB_ERR_ARG;
    if (!((dtypeAB == NTB_X_FLOAT16 && (dtypeC == NTB_X_FLOAT16 || dtypeC == NTB_X_FLOAT)) ||
          (dtypeAB == NTB_X_FLOAT && dtypeC == NTB_X_FLOAT)))
        return NTB_ERR_DTYPE;
    for (int d = 0; d < nDev; d++)
        if (devIDs[d] < 0 || devIDs[d] >= MAX_DEV || !a[d] || !b[d] || !c[d])
            return NTB_ERR_ARG;
    const int am = transA == NTB_X_TRANS ? na : ma, an = transA == NTB_X_TRANS ? ma : na;
    const int bn = transB == NTB_X_TRANS ? mb : nb, bm = transB == NTB_X_TRANS ? nb : mb;
    if (am != bn || an != nc || bm != mc)
        return NTB_ERR_SHAPE;
    if (shardAxis == NTB_SHARD_COLUMNS && count != 1)
        return NTB_ERR_ARG;                         /* column shards are defined for the 2-D form */
    if (count == 0 || nc == 0 || mc == 0)
        return NTB_OK;

    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess) {
        cudaGetLastError();
        return NTB_ERR_CUDA;
    }
    const long long esC = (long long)ElemSize(dtypeC);
    int rc = NTB_OK;
    cudaEvent_t done[MAX_SHARDS];
    /* every device must be able to write every other device's copy of c */
    if (gather) {
        for (int d = 0; d < nDev && rc == NTB_OK; d++) {
            if (cudaSetDevice(devIDs[d]) != cudaSuccess) {
                rc = NTB_ERR_CUDA;
                break;
            }
            for (int e = 0; e < nDev && rc == NTB_OK; e++)
                rc = EnablePeer(devIDs[d], devIDs[e]);
        }
    }
    for (int d = 0; d < nDev && rc == NTB_OK; d++) {
        const int dev = devIDs[d];
        void * st = streams ? streams[d] : nullptr;
        if (shardAxis == NTB_SHARD_COLUMNS) {
            int lo, hi;
            ntb_shard_range(mc, nDev, d, 8, &lo, &hi);
            const int w = hi - lo;
            if (w == 0)
                continue;
            /* the shard of b is packed: w stored rows (transposed use) or w stored columns */
            const int sbn = transB == NTB_X_TRANS ? w : nb, sbm = transB == NTB_X_TRANS ? mb : w;
            if (!gather) {
                rc = ntb_gemm(dev, st, a[d], transA, b[d], transB, c[d], dtypeAB, dtypeC,
                              na, ma, sbn, sbm, nc, w, ma, sbm, w, alpha, beta);
            }
            else {
                void * peers[NTB_MAX_PEERS];
                int np = 0;
                for (int e = 0; e < nDev; e++)
                    if (e != d)
                        peers[np++] = (char *)c[e] + (long long)lo * esC;
                rc = ntb_gemm_peers(dev, st, a[d], transA, b[d], transB, (char *)c[d] + (long long)lo * esC,
                                    peers, np, dtypeAB, dtypeC, na, ma, sbn, sbm, nc, w, ma, sbm, mc, alpha, beta);
            }
        }
        else {
            int lo, hi;
            ntb_shard_range(count, nDev, d, 1, &lo, &hi);
            const int n = hi - lo;
            if (n == 0)
                continue;
            const long long sa = (long long)na * ma, sb = (long long)nb * mb, sc = (long long)nc * mc;
            /* without a gather every device holds only its own problems, packed; with it, c[d] has
               room for all `count` results and the device's own start at problem lo */
            char * cd = (char *)c[d] + (gather ? (long long)lo * sc * esC : 0);
            rc = ntb_gemm_strided_batched(dev, st, a[d], transA, b[d], transB, cd, dtypeAB, dtypeC,
                                          na, ma, nb, mb, nc, mc, ma, mb, mc, sa, sb, sc, n, alpha, beta);
            if (rc == NTB_OK && gather) {
                if (cudaSetDevice(dev) != cudaSuccess) {
                    rc = NTB_ERR_CUDA;
                    break;
                }
                for (int e = 0; e < nDev && rc == NTB_OK; e++) {
                    if (e == d)
                        continue;
                    char * ce = (char *)c[e] + (long long)lo * sc * esC;
                    const cudaError_t err = devIDs[e] == dev
                        ? cudaMemcpyAsync(ce, cd, (size_t)((long long)n * sc * esC), cudaMemcpyDeviceToDevice, (cudaStream_t)st)
                        : cudaMemcpyPeerAsync(ce, devIDs[e], cd, dev, (size_t)((long long)n * sc * esC), (cudaStream_t)st);
                    if (err != cudaSuccess)
                        rc = NTB_ERR_CUDA;
                }
            }
        }
    }
    /* Join: work queued later on any of the streams starts only after every shard has been
       written everywhere. (Without a gather each stream owns its shard and nothing is joined.) */
    if (rc == NTB_OK && gather && nDev > 1) {
        for (int d = 0; d < nDev && rc == NTB_OK; d++) {
            if (cudaSetDevice(devIDs[d]) != cudaSuccess || EventFor(d, devIDs[d], &done[d]) != NTB_OK ||
                cudaEventRecord(done[d], streams ? (cudaStream_t)streams[d] : nullptr) != cudaSuccess)
                rc = NTB_ERR_CUDA;
        }
        for (int d = 0; d < nDev && rc == NTB_OK; d++) {
            if (cudaSetDevice(devIDs[d]) != cudaSuccess) {
                rc = NTB_ERR_CUDA;
                break;
            }
            for (int e = 0; e < nDev && rc == NTB_OK; e++)
                if (e != d && cudaStreamWaitEvent(streams ? (cudaStream_t)streams[d] : nullptr, done[e], 0) != cudaSuccess)
                    rc = NTB_ERR_CUDA;
        }
    }
    if (rc == NTB_ERR_CUDA)
        cudaGetLastError();
    if (prev >= 0)
        cudaSetDevice(prev);
    return rc;
}

}
