/*
 * ntb_gemm.h -- C ABI of the B200 (sm_100a) dense matrix-multiplication library that
 * stands in for NiuTensor's cuBLAS wrapper layer.
 *
 * Every function computes, for row-major packed-or-strided matrices,
 *
 *        c = alpha * op(a) * op(b) + beta * c
 *
 * with the reference's conventions: `na x ma`, `nb x mb`, `nc x mc` are the STORED
 * (pre-transposition) rows x cols; transposition flags carry the reference's enum
 * values (source/tensor/XDataType.h:36: X_TRANS = 0, X_NOTRANS = 1 -- note that 0
 * means "transposed"); data types carry TENSOR_DATA_TYPE values
 * (source/tensor/XDataType.h:33). alpha and beta arrive as float even for half
 * tensors, as DTYPE does in the reference (source/tensor/XGlobal.h:54).
 *
 * Supported type triples (a, b, c): (X_FLOAT16, X_FLOAT16, X_FLOAT16),
 * (X_FLOAT16, X_FLOAT16, X_FLOAT) and (X_FLOAT, X_FLOAT, X_FLOAT). Products are
 * accumulated in fp32 and alpha/beta are applied in fp32 before the single final
 * rounding. X_DOUBLE, X_INT and X_INT8 return NTB_ERR_DTYPE.
 *
 * Ownership: all matrix pointers are caller-owned device memory on `devID`; the
 * library never allocates or frees tensor storage. `stream` is a cudaStream_t passed as
 * void*; NULL means the legacy default stream, which is where the reference issues all
 * of its work. When beta == 0 the output is never read, so the reference's memset of c
 * before the call (source/tensor/core/arithmetic/MatrixMul2D.cu:154-155) is not needed.
 * c must not overlap a or b.
 *
 * Errors: every function returns 0 on success or an NTB_ERR_* code; nothing throws or
 * exits. The C++ operator layer turns a nonzero code into the reference's fatal
 * ShowNTErrors behaviour. There is no CPU fallback: without a usable CUDA device every
 * compute entry point returns NTB_ERR_CUDA.
 *
 * Threading: re-entrant per device; a per-device context (tensor-map encoder, status
 * word, staging buffers of the host-buffer entry point) is created lazily under a lock.
 * The current device of the calling thread is saved and restored around each call
 * (the reference's ProtectCudaDev/BacktoCudaDev, source/tensor/XDevice.h:233-244).
 */
#ifndef NTB_GEMM_H
#define NTB_GEMM_H

#ifdef __cplusplus
extern "C" {
#endif

/* TENSOR_DATA_TYPE (source/tensor/XDataType.h:33) */
#define NTB_X_INT      0
#define NTB_X_INT8     1
#define NTB_X_FLOAT    2
#define NTB_X_FLOAT16  3
#define NTB_X_DOUBLE   4

/* MATRIX_TRANS_TYPE (source/tensor/XDataType.h:36) */
#define NTB_X_TRANS    0
#define NTB_X_NOTRANS  1

#define NTB_OK              0
#define NTB_ERR_ARG         1   /* NULL pointer, negative size, bad flag */
#define NTB_ERR_SHAPE       2   /* inner dimensions or output shape do not match */
#define NTB_ERR_DTYPE       3   /* unsupported data-type triple */
#define NTB_ERR_CUDA        4   /* CUDA runtime / driver call failed, or no device */
#define NTB_ERR_DEVICE_WAIT 5   /* a bounded on-device wait ran out (kernel gave up) */
#define NTB_ERR_LIMIT       6   /* a size exceeds a documented fixed limit */

/* kernel routes, as reported by ntb_last_route() */
#define NTB_ROUTE_NONE      0
#define NTB_ROUTE_TC_F16    1   /* tcgen05 kind::f16, TMEM accumulators; operands by TMA (after a realigning copy where
                                   TMA could not address them) or, for the tiniest such products, by loader warps */
#define NTB_ROUTE_TC_3XTF32 2   /* tcgen05 kind::tf32, three passes on hi/lo split fp32; operands as above */
#define NTB_ROUTE_SIMT      3   /* FFMA kernel: K = 0, operands not aligned to their element size, or forced */
#define NTB_ROUTE_TC_F16_PAIR 4 /* kind::f16 on CTA pairs (cta_group::2): 512 x 256 to 256 x 128 tiles, or several
                                   pairs sharing a 256 x 256 tile along K */
#define NTB_ROUTE_TC_F16X2  5   /* large fp32 products: every value as two scaled half pieces, three
                                   kind::f16 products on CTA pairs (needs scratch for the pieces) */

/*
 * Single GEMM. Replaces _CudaBLASMatrixMUL
 * (source/tensor/core/arithmetic/XTensorBLAS.cu:38-104) and the dense GPU branch of
 * _CudaMatrixMul2D (source/tensor/core/arithmetic/MatrixMul2D.cu:123-209).
 * lda/ldb/ldc are row pitches in elements (the reference always has lda = ma etc.;
 * explicit pitches allow a column shard of a resident matrix to be multiplied in place).
 */
int ntb_gemm(int devID, void * stream,
             const void * a, int transA, const void * b, int transB, void * c,
             int dtypeAB, int dtypeC,
             int na, int ma, int nb, int mb, int nc, int mc,
             long long lda, long long ldb, long long ldc,
             float alpha, float beta);

/*
 * Single GEMM with a fused row-vector bias and optional activation:
 *
 *        c = act(alpha * op(a) * op(b) + beta * c + bias)
 *
 * bias holds mc values of c's data type (NULL: none) and is added to every row; act is
 * NTB_ACT_NONE or NTB_ACT_RECTIFY (max(x, 0), source/tensor/function/Rectify.cpp).
 * Replaces the two-pass MulAndShift of the reference -- _MatrixMul into a scratch tensor,
 * then _SumDim re-reading and re-writing it (source/tensor/core/arithmetic/
 * MulAndShift.cpp:66-88, SumDim.cu:43-103) -- and, with NTB_ACT_RECTIFY, the Rectify pass
 * that follows it in the feed-forward layer (source/sample/transformer/submodel/FFN.cpp:
 * 90-101). The sum is formed in fp32 and rounded once. A leading-dimension fold of a
 * (rows = product of its leading extents) is the caller's business, as in ntb_gemm.
 */
#define NTB_ACT_NONE    0
#define NTB_ACT_RECTIFY 1
int ntb_gemm_bias_act(int devID, void * stream,
                      const void * a, int transA, const void * b, int transB, const void * bias, void * c,
                      int dtypeAB, int dtypeC,
                      int na, int ma, int nb, int mb, int nc, int mc,
                      long long lda, long long ldb, long long ldc,
                      float alpha, float beta, int act);

/*
 * Fused scaled-dot-product attention on half tensors:
 *
 *        out = softmax(scale * q * k^T + mask) * v        for each of `blocks` blocks
 *
 * q, out: [blocks, lenQ, dim]; k, v: [blocks, lenK, dim], packed, X_FLOAT16. mask is NULL or
 * fp32, additive, [lenQ, lenK] per block with maskBlockStride elements between blocks
 * (0 = one mask for all blocks). One kernel instead of the inference-time chain of the
 * transformer sample -- BMMul(q, k^T), ConvertDataType, Sum(mask), Softmax, ConvertDataType,
 * BMMul(att, v) (source/sample/transformer/submodel/Attention.cpp:206-238) -- whose score
 * tensor never reaches HBM here. Softmax as source/tensor/function/Softmax.cpp:60-115
 * (maximum subtracted, fp32, a row whose sum is 0 gives zeros). dim is 64 or 128 (the
 * sample's default head size, Config.cpp:126,137), else NTB_ERR_LIMIT; lenK is unlimited (keys
 * are taken 256 at a time; beyond 256 the scores are computed twice, once for the row maxima
 * and once for the sums and the second product).
 *
 * ntb_attention_dropout is the training form (Attention.cpp:229-230: Dropout on the
 * probabilities): keep holds one byte per probability, [blocks, lenQ, lenK], 1 = keep, 0 =
 * drop (NULL: no dropout), and kept probabilities are multiplied by keepScale = 1 / (1 - p).
 * The mask is the caller's, so that the same one can be given to any other implementation.
 */
int ntb_attention(int devID, void * stream,
                  const void * q, const void * k, const void * v, const float * mask, void * out,
                  int dtype, int blocks, int lenQ, int lenK, int dim,
                  long long maskBlockStride, float scale);
int ntb_attention_dropout(int devID, void * stream,
                          const void * q, const void * k, const void * v, const float * mask,
                          const unsigned char * keep, void * out,
                          int dtype, int blocks, int lenQ, int lenK, int dim,
                          long long maskBlockStride, float scale, float keepScale);

/*
 * Row-wise log-softmax over the last dimension in two halves, for logits whose rows are
 * spread over several GPUs (vocabulary shards of the output layer,
 * source/sample/transformer/submodel/Output.cpp:86-101, LogSoftmax.cpp:40-170).
 * ntb_row_stats: rowMax[r] = max_c x[r, c], rowSumExp[r] = sum_c exp(x[r, c] - rowMax[r])
 * over the local `cols` columns (fp32 device arrays of `rows` entries). The caller
 * combines shards: M = max of the maxima, S = sum of rowSumExp * exp(rowMax - M).
 * ntb_logsoftmax_apply: y[r, c] = log(exp(x[r, c] - M[r]) / S[r]), floored at -20, NaN and
 * infinities replaced by -20, zeros for a row with S == 0, as the reference does; y may be
 * x. x, y: X_FLOAT16 or X_FLOAT device matrices with row pitches ldx, ldy (elements).
 * With one shard, the two calls in sequence are the reference's LogSoftmax.
 */
int ntb_row_stats(int devID, void * stream, const void * x, int dtype, int rows, int cols, long long ld,
                  float * rowMax, float * rowSumExp);
int ntb_logsoftmax_apply(int devID, void * stream, const void * x, void * y, int dtype,
                         int rows, int cols, long long ldx, long long ldy,
                         const float * rowMax, const float * rowSumExp);

/*
 * Both gradient products of c = alpha * op(a) * op(b) in one launch:
 *
 *        deda += alpha * (...),   dedb += alpha * (...)        (beta = 1, accumulating)
 *
 * with the operand order and transposition flags of the reference's backward pass
 * (source/network/XBackwardMath.cpp:655-699 for MatrixMul, :714-786 for MatrixMulBatched):
 *   N/N: deda += dedc * b^T,    dedb += a^T * dedc
 *   T/N: deda += b * dedc^T,    dedb += a * dedc
 *   N/T: deda += dedc * b,      dedb += dedc^T * a
 *   T/T: deda += b^T * dedc^T,  dedb += dedc^T * a^T
 * a: na x ma, b: nb x mb (stored), dedc: the shape of c; deda, dedb: the shapes of a, b; all
 * packed, `count` matrices back to back (count = 1 for the 2-D form). Either gradient
 * pointer may be NULL (that product is skipped, the reference's isEfficient case). The
 * reference issues two GEMMs; here the tiles of both products are walked by one persistent
 * kernel, so the second product starts while the first one's last tiles finish and dedc is
 * read once into L2 for both. Operands the tensor-core route cannot address, and products
 * large enough for the CTA-pair or split-K kernels, are issued as two launches.
 */
int ntb_gemm_grad(int devID, void * stream,
                  const void * a, int transA, const void * b, int transB, const void * dedc,
                  void * deda, void * dedb, int dtype,
                  int na, int ma, int nb, int mb, int count, float alpha);

/*
 * `count` GEMMs of one shape whose matrices lie at constant element strides; a stride
 * of 0 reuses one matrix for every problem. One launch covers all problems.
 * Replaces _CudaBLASMatrixMULBatchedStrided
 * (source/tensor/core/arithmetic/XTensorBLAS.cu:181-247), the call behind
 * _MatrixMulBatchedGPU (source/tensor/core/arithmetic/MatrixMulBatched.cpp:84-138).
 */
int ntb_gemm_strided_batched(int devID, void * stream,
                             const void * a, int transA, const void * b, int transB, void * c,
                             int dtypeAB, int dtypeC,
                             int na, int ma, int nb, int mb, int nc, int mc,
                             long long lda, long long ldb, long long ldc,
                             long long strideA, long long strideB, long long strideC,
                             int count, float alpha, float beta);

/*
 * The general form of _MatrixMul
 * (source/tensor/core/arithmetic/MatrixMul.cpp:100-146): a holds aBlockNum packed
 * matrices, b holds bBlockNum; every pair (p, q) is multiplied and written to block
 * p * bBlockNum + q of c. One launch, base addresses computed on the device from
 * (p, q) -- there are no pointer tables and no host-to-device copies (the reference
 * builds three and copies them synchronously, XTensorBLAS.cu:315-347).
 */
int ntb_gemm_broadcast(int devID, void * stream,
                       const void * a, int transA, const void * b, int transB, void * c,
                       int dtypeAB, int dtypeC,
                       int na, int ma, int nb, int mb, int nc, int mc,
                       int aBlockNum, int bBlockNum,
                       float alpha, float beta);

/*
 * Uniform-shape list given as HOST arrays of device pointers. Replaces
 * _CudaBLASMatrixMULList + _CudaBLASMatrixMULBatched
 * (source/tensor/core/arithmetic/XTensorBLAS.cu:252-387, 109-178). The planner looks
 * for a constant stride or for the two-level (p, q) pattern of the general form and
 * issues one launch when it finds either; any other pointer pattern is issued as one
 * launch per problem on the same stream.
 */
int ntb_gemm_list(int devID, void * stream,
                  const void * const * a, int transA, const void * const * b, int transB,
                  void * const * c, int dtypeAB, int dtypeC,
                  int count, int na, int ma, int nb, int mb, int nc, int mc,
                  float alpha, float beta);

/*
 * A list of `count` products whose shapes may all differ (host arrays of device pointers and
 * of stored extents; packed matrices; one pair of transposition flags, one alpha and beta for
 * the whole list, as in _CudaBLASMatrixMULList). Replaces the fallback loop of single cuBLAS
 * calls the reference takes when the shapes of a list are not uniform
 * (source/tensor/core/arithmetic/XTensorBLAS.cu:373-385): up to eight problems share one
 * persistent launch whose tile walk covers them one after the other; longer lists take one
 * launch per eight. Items TMA cannot address and items with an empty inner dimension are
 * issued on their own on the same stream. Shapes are all checked before anything is launched.
 */
int ntb_gemm_grouped(int devID, void * stream, int count,
                     const void * const * a, int transA, const void * const * b, int transB, void * const * c,
                     int dtypeAB, int dtypeC,
                     const int * na, const int * ma, const int * nb, const int * mb, const int * nc, const int * mc,
                     float alpha, float beta);

/*
 * One 2-D product whose result is also written, tile by tile from the epilogue, to the
 * same rows and columns of up to NTB_MAX_PEERS further buffers of the shape and pitch of c:
 * the copies of C that other GPUs hold (their memory mapped into this process) or other
 * buffers of this GPU. With the columns of C sharded over GPUs, every rank passes its column
 * block of every other rank's full C and the all-gather of C is done by the products
 * themselves, with plain 16-byte stores of full 128-byte lines over NVLink; no rank reads
 * another's memory. The reference gathers tensors across devices with a device-to-device
 * cudaMemcpy of the whole tensor after the operator (source/tensor/XUtility.cpp:196-201,
 * source/train/XWorkerCollect.cpp:59-78); it has no fused form. c and the peers must allow
 * the staged store path (16-byte aligned bases and pitches), else NTB_ERR_ARG; old values
 * (beta != 0) are read from c only. The caller makes the writes visible to the other ranks
 * by synchronising its stream and then the ranks (a host barrier), as after any copy.
 */
#define NTB_MAX_PEERS 8
int ntb_gemm_peers(int devID, void * stream,
                   const void * a, int transA, const void * b, int transB, void * c,
                   void * const * peers, int nPeers,
                   int dtypeAB, int dtypeC,
                   int na, int ma, int nb, int mb, int nc, int mc,
                   long long lda, long long ldb, long long ldc,
                   float alpha, float beta);

/*
 * One product sharded over nDev GPUs driven by ONE process -- NiuTensor's own process model
 * (one process, a worker thread per device: source/train/XWorkerJob.cpp, XLeader.cpp). The
 * reference never shards an operator; the only cross-device movement it has is a
 * whole-tensor device-to-device cudaMemcpy after the operator (source/tensor/XUtility.cpp:
 * 196-201, source/train/XWorkerCollect.cpp:59-78), which is what `gather` replaces.
 *
 * devIDs[d] runs shard d on streams[d] (streams == NULL: each device's default stream).
 * All per-device arrays have nDev entries of device pointers on that device.
 *
 * NTB_SHARD_COLUMNS (2-D form, count == 1): a[d] is the whole stored a (replicated); device
 * d owns columns [lo_d, hi_d) = ntb_shard_range(mc, nDev, d, 8) of c; b[d] is the PACKED
 * part of the stored b that produces them -- rows lo_d..hi_d-1 of b when transB ==
 * NTB_X_TRANS (rows of a vocabulary matrix), columns otherwise -- and nb, mb, nc, mc are the
 * extents of the WHOLE b and c. gather == 0: c[d] is the packed nc x (hi_d - lo_d) block.
 * gather != 0: every c[d] is a whole nc x mc matrix; device d's epilogue writes its block
 * into its own c[d] and, over NVLink, into every other c[e] (peer access is enabled here;
 * old values for beta != 0 are read from c[d] only), and each stream is then made to wait for
 * all shards, so work queued afterwards on any of the streams sees the whole c.
 *
 * NTB_SHARD_BATCH: `count` products of one shape (MatrixMulBatched); device d owns problems
 * ntb_shard_range(count, nDev, d, 1); a[d], b[d] hold that device's problems, packed.
 * gather == 0: so does c[d]. gather != 0: every c[d] has room for all `count` results; each
 * device computes its own in place and copies them to the other devices.
 *
 * The call only queues work; it returns without waiting for the GPUs. More than
 * NTB_MAX_PEERS + 1 devices: NTB_ERR_LIMIT.
 */
#define NTB_SHARD_COLUMNS 0
#define NTB_SHARD_BATCH   1
int ntb_gemm_sharded(const int * devIDs, int nDev, void * const * streams,
                     const void * const * a, int transA, const void * const * b, int transB, void * const * c,
                     int dtypeAB, int dtypeC,
                     int na, int ma, int nb, int mb, int nc, int mc,
                     int count, int shardAxis, int gather, float alpha, float beta);

/*
 * [lo, hi) of `total` units owned by shard `shard` of `shards`: contiguous, balanced in
 * units of `multiple` (the last shard takes a ragged remainder). The split used by
 * ntb_gemm_sharded: multiple = 8 for columns, so that fp16 row segments stay 16-byte
 * aligned, 1 for the batch. No counterpart in the reference, which never shards an operator.
 */
void ntb_shard_range(int total, int shards, int shard, int multiple, int * lo, int * hi);

/*
 * Column shards that a collective left one after the other -- src holds `shards` packed
 * matrices of rows x colsPerShard, as an all-gather of packed shards writes them -- become
 * the row-major matrix dst (rows x shards * colsPerShard, row pitch ldDst elements) in one
 * pass. Used when the whole c is gathered with NCCL instead of by the products' own
 * epilogues. Addresses and row segments must be 16-byte aligned, else NTB_ERR_ARG. No
 * counterpart in the reference (it has no collectives).
 */
int ntb_unshard_columns(int devID, void * stream, const void * src, void * dst, int dtype,
                        long long rows, int shards, int colsPerShard, long long ldDst);

/*
 * ntb_gemm_peers with the NVLink switch doing the fan-out: mc is the MULTICAST address of the
 * place of this product's block in the copies of C that all GPUs of a group hold (a multicast
 * object bound to every GPU's buffer: cuMulticastCreate / cuMulticastBindMem, or the
 * multicast pointer of a symmetric-memory allocation). The epilogue writes every finished
 * 128-byte line once, with multimem.st; the switch delivers it to every GPU, this one included,
 * so each GPU sends its block once instead of once per peer. c is this GPU's ordinary address
 * of the same block (old values for beta != 0 are read there, and the block is also written
 * there directly). The column count of the block must be a whole number of 16-byte units.
 * Visibility on the other GPUs as for ntb_gemm_peers: synchronise the stream, then the ranks.
 * The reference has no counterpart (source/tensor/XUtility.cpp:196-201 copies whole tensors).
 */
int ntb_gemm_multicast(int devID, void * stream,
                       const void * a, int transA, const void * b, int transB, void * c, void * mc,
                       int dtypeAB, int dtypeC,
                       int na, int ma, int nb, int mb, int nc, int mc_cols,
                       long long lda, long long ldb, long long ldc,
                       float alpha, float beta);

/*
 * Host-buffer form: a, b and c are HOST memory (pinned or pageable). Copies the
 * operands (and c when beta != 0) to staging buffers owned by the device context (a single
 * product with rows padded to a multiple of 16 bytes, so that TMA can address any extents), runs
 * the strided-batched GEMM, copies c back and synchronises the stream. This is what a
 * caller holding CPU tensors does through the reference with SetDevice/FlushToDevice
 * (source/tensor/XTensor.cpp:533-539, 1992-1999) around MatrixMul. Staging buffers grow
 * on demand and are kept until ntb_release(). A single large 2-D product is cut into
 * column chunks whose copy-in, product and copy-out overlap on internal streams (this
 * needs pinned host memory to take effect). Calls on one device share the staging buffers:
 * do not overlap them.
 */
int ntb_gemm_host(int devID, void * stream,
                  const void * a, int transA, const void * b, int transB, void * c,
                  int dtypeAB, int dtypeC,
                  int na, int ma, int nb, int mb, int nc, int mc,
                  long long strideA, long long strideB, long long strideC,
                  int count, float alpha, float beta);

/*
 * The same with `aDevice` already in DEVICE memory (b and c are host buffers as above): for
 * a product sharded over several GPUs, where every rank needs the whole of a but the host's
 * copy should cross PCIe once, not once per GPU -- each rank copies a slice in, the ranks
 * all-gather it over NVLink, then each calls this with its shards of b and c. aDevice must be
 * ready on `stream`. The reference's counterpart is a tensor that SetDevice moved earlier
 * (source/tensor/XTensor.cpp:533-539) multiplied with ones that still live on the host.
 */
int ntb_gemm_host_resident_a(int devID, void * stream,
                             const void * aDevice, int transA, const void * b, int transB, void * c,
                             int dtypeAB, int dtypeC,
                             int na, int ma, int nb, int mb, int nc, int mc,
                             long long strideA, long long strideB, long long strideC,
                             int count, float alpha, float beta);

/*
 * Host-buffer form of one product that allocates nothing. It has no counterpart in the
 * reference, whose wrappers borrow scratch from XMem or cudaMalloc (XTensorBLAS.cu:
 * 329-343); it exists for callers that cannot allocate device memory at call time: a
 * process whose XMem pools already own the GPU's memory, where a library-side cudaMalloc
 * may fail, and worker threads sharing a device, which cudaMalloc / cudaFree would stall.
 * a, b and c are HOST buffers, packed (pitch = columns). All device scratch -- staging for
 * a, b, c and the status word -- is a fixed array inside the library, so the staged
 * operands (rows padded to a multiple of 16 bytes, so that TMA can address every shape; each
 * operand rounded up to 256 bytes) must fit in NTB_NOALLOC_MAX_BYTES; a larger problem
 * returns NTB_ERR_LIMIT. Calls on one device share that array: do not overlap
 * them. The first call on a device looks up the array's address, and with CUDA's default
 * lazy module loading that look-up is also when the runtime reserves the array's 16 MiB on
 * the device: make that first call (any tiny product) early -- before the host's pools take
 * the rest of the GPU's memory and before the process begins any stream capture -- or run
 * with CUDA_MODULE_LOADING=EAGER; from then on no call allocates anything. The call returns
 * after the result is back in c; after an error it still waits for copies it had queued.
 * ntb_set_route() applies as everywhere else.
 */
#define NTB_NOALLOC_MAX_BYTES (16u << 20)
int ntb_gemm_host_noalloc(int devID, void * stream,
                          const void * a, int transA, const void * b, int transB, void * c,
                          int dtypeAB, int dtypeC,
                          int na, int ma, int nb, int mb, int nc, int mc,
                          float alpha, float beta);

/* Route taken by the calling thread's most recent successful launch (NTB_ROUTE_*). */
int ntb_last_route(void);

/*
 * Restricts routing: 0 = automatic (default), NTB_ROUTE_SIMT = always the FFMA kernel,
 * NTB_ROUTE_TC_F16 / NTB_ROUTE_TC_3XTF32 = fail with NTB_ERR_ARG instead of using the
 * FFMA kernel when the tensor-core route cannot address the operands (and, for
 * NTB_ROUTE_TC_F16, never use CTA pairs), NTB_ROUTE_TC_F16_PAIR = likewise, but always
 * CTA pairs for half operands whatever the problem size. Process-wide.
 */
int ntb_set_route(int route);

/*
 * Synchronises `devID` and reads its status word: NTB_OK, or NTB_ERR_DEVICE_WAIT when a
 * kernel abandoned a bounded wait since the last call (the word is cleared on read).
 */
int ntb_device_status(int devID);

/*
 * Test hook for the give-up path of the kernels' bounded waits; it has no counterpart in the
 * reference, which has no device-side waits. skipKBlock >= 0: from now on the copy engine
 * producers of the tensor-core kernels (single-CTA and CTA-pair) announce that k-block of
 * their first tile but never load it, so the consumer's wait on it cannot complete;
 * waitLimitKiloCycles > 0: waits on `devID` give up after that many thousand SM clocks
 * instead of about two seconds. The kernel then records NTB_ERR_DEVICE_WAIT, lets copies in
 * flight land, frees its tensor memory and returns; nothing traps or faults. (-1, 0) restores
 * normal operation. Process-wide for the producers, per device for the limit; meant for
 * tests only. Synchronises the device.
 */
int ntb_debug_inject(int devID, int skipKBlock, int waitLimitKiloCycles);

/*
 * The kernel the tile cost model picks for `count` fp16 (NTB_X_FLOAT16) or fp32 products
 * of M x N x K on a device with smCount SMs, without launching anything (no CUDA call):
 * the tile width 64 / 128 / 256 of the single-CTA kernel, or NTB_PLAN_PAIR_* /
 * NTB_PLAN_SPLIT_* for the cluster kernels. An inspection aid for tuning and for tests of
 * the model; it has no counterpart in the reference, whose cuBLAS calls choose internally.
 * Environment knobs that override the model at launch are not applied here.
 */
#define NTB_PLAN_PAIR_256X256   0
#define NTB_PLAN_PAIR_512X256  (-1)
#define NTB_PLAN_SPLIT_K2      (-2)
#define NTB_PLAN_SPLIT_K4      (-4)
#define NTB_PLAN_PAIR_256X128  (-8)
#define NTB_PLAN_PAIR_512X128  (-9)
#define NTB_PLAN_PAIRSPLIT_K2 (-18)   /* two CTA pairs share a 256 x 256 tile, half of K each */
#define NTB_PLAN_PAIRSPLIT_K4 (-20)   /* four pairs per tile, a quarter of K each */
int ntb_plan(int dtypeAB, int M, int N, int K, int count, int smCount);

/* Products issued so far in this process through the kernel family `route` (NTB_ROUTE_*): shows,
   for a whole program, how many products alignment pushed off the tensor cores. */
long long ntb_route_count(int route);
/* one more counter read through the same call: products whose operands were first copied
   into 16-byte aligned rows because TMA could not address them where they lay */
#define NTB_COUNT_REPACK   7

/* Number of kernels this library has launched in the process so far. */
long long ntb_launch_count(void);

/* Frees the per-device contexts (staging buffers, status words). */
void ntb_release(void);

const char * ntb_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif
