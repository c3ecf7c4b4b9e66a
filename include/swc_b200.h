/*
 * swc_b200.h -- C-ABI kernel table: B200 (sm_100a) replacements for the operator
 * kernels SWCompiler's code generator emits calls to.
 *
 * The reference has no FFI; its boundary is textual.  Codegen prints
 * `#include "utils/kernels.h"` (src/codegen/Codegen.cpp:260) and, per op node,
 * one call `<kernel>_<dtype flag>(...)` (Codegen.cpp:1171-2494 for CPU,
 * :2602-2674 for its CUDA sketch).  Every entry point below keeps the name and
 * the argument order of the function it replaces, with two changes: a context
 * comes first and an int status comes back (0 = ok), because the reference's
 * void calls have no way to report an error.
 *
 * Conventions
 *   - every tensor pointer is a DEVICE pointer into memory the caller owns;
 *     shape/attribute arrays (`const size_t*`) are HOST arrays, read during the
 *     call, exactly as the emitted program passes them (Codegen.cpp:1761-1782);
 *   - calls are asynchronous on the context's stream; swcb200_sync waits;
 *   - a context belongs to one host thread at a time (the emitted main() is
 *     single-threaded, Codegen.cpp:1037-1058);
 *   - nothing here falls back to the CPU: without a usable device every call
 *     returns SWCB200_ERR_NO_DEVICE or SWCB200_ERR_CUDA.
 */
#ifndef SWC_B200_H_
#define SWC_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct swcb200_ctx swcb200_ctx;

enum swcb200_status {
    SWCB200_OK = 0,
    SWCB200_ERR_BAD_ARG = 1,     /* null pointer, negative size, unknown enum            */
    SWCB200_ERR_BAD_SHAPE = 2,   /* shapes inconsistent with each other                  */
    SWCB200_ERR_MISALIGNED = 3,  /* pointer / leading dimension breaks a stated alignment */
    SWCB200_ERR_UNSUPPORTED = 4, /* valid in the reference's signature, not built here   */
    SWCB200_ERR_CUDA = 5,        /* a CUDA runtime/driver call failed; see last_error    */
    SWCB200_ERR_NCCL = 6,        /* NCCL missing or a collective failed                  */
    SWCB200_ERR_TIMEOUT = 7,     /* a bounded device- or host-side wait gave up          */
    SWCB200_ERR_NO_DEVICE = 8,   /* no CUDA device / not an sm_100 device                */
    SWCB200_ERR_TOO_LARGE = 9    /* exceeds a documented size limit                      */
};

/* How the fp32 entry points matrixMatrixMul_f and conv2d_f compute. */
enum swcb200_precision {
    SWCB200_STRICT_F32 = 0, /* fp32 products and sums, one rounding each, in the reference's order:
                               results equal the reference's generated C bit for bit              */
    SWCB200_TC_BF16 = 1     /* operands rounded to bf16, tcgen05 tensor cores, fp32 accumulation  */
};

enum swcb200_dtype { SWCB200_F32 = 0, SWCB200_BF16 = 1, SWCB200_I32 = 2 };
enum swcb200_act { SWCB200_ACT_NONE = 0, SWCB200_ACT_RELU = 1, SWCB200_ACT_TANH = 2 };

/* ------------------------------------------------------------------ context */

/* Creates a context on `device` with its own stream.  Replaces the emitted
 * environment set-up (cublasCreate + cudaStreamCreate, Codegen.cpp:142-173). */
int swcb200_init(int device, int precision, swcb200_ctx **out);
/* Same, but work is issued on `cuda_stream` (a cudaStream_t; NULL = the legacy default stream),
 * which the caller keeps owning. */
int swcb200_init_on_stream(int device, int precision, void *cuda_stream, swcb200_ctx **out);
int swcb200_destroy(swcb200_ctx *ctx);
int swcb200_sync(swcb200_ctx *ctx);
int swcb200_set_precision(swcb200_ctx *ctx, int precision);
/* Every wait inside the tensor-core kernels (on an operand tile, a pipeline stage, an accumulator) is
 * bounded: when it runs out the kernel unwinds normally and the next swcb200_sync returns
 * SWCB200_ERR_TIMEOUT; the context stays usable.  The limit is counted in SM clock cycles, 4e9 by
 * default (2 to 3 seconds).  The reference has no counterpart (its kernels cannot wait). */
int swcb200_set_wait_limit(swcb200_ctx *ctx, long long cycles);
/* The persistent tensor-core kernels (swcb200_fc_bf16*, swcb200_conv2d_bf16) launched through this context take at
 * most `sms` SMs (0 = all, the default).  They hold nearly all of an SM's shared memory, so a kernel of another
 * stream -- a collective that should run BESIDE a GEMM -- only finds room on SMs left free this way. */
int swcb200_set_sm_limit(swcb200_ctx *ctx, int sms);
/* Self-test of that path: launches one thread that waits, with the same bounded wait, on a barrier
 * nothing arrives at.  After the context's limit the kernel returns and swcb200_sync reports
 * SWCB200_ERR_TIMEOUT.  Set a short limit first (a million cycles is half a millisecond). */
int swcb200_selftest_wait_timeout(swcb200_ctx *ctx);
void *swcb200_stream(swcb200_ctx *ctx);
const char *swcb200_status_string(int status);
const char *swcb200_last_error(swcb200_ctx *ctx);
/* Kernel launches issued through this context since it was created. */
uint64_t swcb200_launch_count(swcb200_ctx *ctx);
/* Library version, e.g. 100 = 0.1.0. */
int swcb200_version(void);

/* ----------------------------------------------- dense ops (row-major, 2-D) */

/* C[m,n] = A[m,k] . B[k,n].  Replaces matrixMatrixMul_f (kernels.h:41-56; call site
 * Codegen.cpp:1334-1337) and the cublasSgemm sketch (Codegen.cpp:2610-2632). */
int swcb200_matrixMatrixMul_f(swcb200_ctx *ctx, int m, int n, int k, const float *a, int lda,
                              const float *b, int ldb, float *c, int ldc);
/* dest[r,:] = batch[r,:] + slice[:].  Replaces batchedadd_f (kernels.h:542-552;
 * Codegen.cpp:1501-1516) and batchedadd_float (cuda_kernels.h:29-37). */
int swcb200_batchedadd_f(swcb200_ctx *ctx, float *dest, const float *batch, const float *slice,
                         size_t numSlice, size_t sliceSize);
/* b = 1 - 2/(exp(2a)+1).  Replaces matrixTanh_f (kernels.h:58-64; Codegen.cpp:2286-2296)
 * and matrixTanh_float (cuda_kernels.h:22-27). */
int swcb200_matrixTanh_f(swcb200_ctx *ctx, int m, int n, const float *a, int lda, float *b,
                         int ldb);
/* Row softmax.  Replaces matrixSoftmax_f (kernels.h:88-103; Codegen.cpp:2349-2354)
 * and matrixSoftmax_float (cuda_kernels.h:4-20). */
int swcb200_matrixSoftmax_f(swcb200_ctx *ctx, int m, int n, const float *a, int lda, float *b,
                            int ldb);
/* Top-k column indices per row, ties to the higher index.  Replaces argMax_i
 * (kernels.h:601-613; Codegen.cpp:2372-2386).  top_k <= n. */
int swcb200_argMax_i(swcb200_ctx *ctx, const float *input, int *idx, int m, int n, int top_k);
/* Running hit count of a streaming evaluation: accum_cnt[0] += number of rows i whose label[i] is among
 * the n predictions pred[i, :], accum_cnt[1] += m.  Replaces accuracy_i (kernels.h:617-627;
 * Codegen.cpp:2387-2398).  The caller zeroes accum_cnt before the first batch. */
int swcb200_accuracy_i(swcb200_ctx *ctx, const int *pred, const int *label, int *accum_cnt, int m,
                       int n);

/* The same product as swcb200_matrixMatrixMul_f in SWCB200_TC_BF16 mode, for callers that must not
 * allocate device memory (a generated program whose single arena already owns the GPU, a server with a
 * fixed memory budget, code running between the collectives of a multi-GPU job).  It has no counterpart
 * in the reference.  The bf16 operand copies live in a fixed 40 MiB array inside the library, held by every
 * GPU that loads the library until the process exits; sizes with 2*roundup(k,8)*(m+n) beyond 40 MiB return
 * SWCB200_ERR_TOO_LARGE.  No context is needed: kernels go on `cuda_stream` of `device`, and EVERY call waits
 * for that stream before it returns (C is complete on return, the host thread blocks).  So no call may be made
 * while the stream is being captured; the first call on a device, which also caches the array's device
 * address, least of all.  The calling thread's current device is left as it was.  All calls on a device
 * share the array (its old contents are overwritten where they matter; nothing needs clearing), so calls
 * that overlap on one GPU race: serialise them.  Calls no cudaMalloc / cudaFree or allocating library
 * routine, and prints nothing: the calling thread's last failure is described by
 * swcb200_matrixMatrixMul_f_noalloc_last_error(). */
int swcb200_matrixMatrixMul_f_noalloc(int device, void *cuda_stream, int m, int n, int k,
                                      const float *a, int lda, const float *b, int ldb, float *c,
                                      int ldc);
const char *swcb200_matrixMatrixMul_f_noalloc_last_error(void);

/* ------------------------------------------------------- flat elementwise */

/* dest = src > 0 ? src : 0.  Replaces relu_f (kernels.h:575-580; Codegen.cpp:2133-2135). */
int swcb200_relu_f(swcb200_ctx *ctx, const float *src, float *dest, size_t size);
/* c = a + b.  Replaces vecAdd_f (kernels.h:592-596; Codegen.cpp:1606-1610). */
int swcb200_vecAdd_f(swcb200_ctx *ctx, int size, const float *a, const float *b, float *c);

/* ------------------------------------------------------------- NHWC ops */

/* Replaces conv2d_f (kernels.h:177-243; Codegen.cpp:1761-1782).  dims arrays have 4 entries
 * (NHWC; filter [oC,kh,kw,iC]); kernels/strides 2; pads 4 of which [0]=top and [1]=left are
 * read, as in the reference.  group must be 1 (the reference's own group > 1 indexing reads
 * past its filter, kernels.h:208-209). */
int swcb200_conv2d_f(swcb200_ctx *ctx, float *output, const float *input, const float *filter,
                     const float *bias, const size_t *odims, const size_t *idims,
                     const size_t *fdims, const size_t *bdims, const size_t *kernels,
                     const size_t *strides, const size_t *pads, size_t group);
/* Replaces maxpool_f (kernels.h:323-377; Codegen.cpp:2020-2037). */
int swcb200_maxpool_f(swcb200_ctx *ctx, const float *input, float *output, const size_t *idims,
                      const size_t *odims, const size_t *kernels, const size_t *strides,
                      const size_t *pads);
/* Replaces avgpool_f (kernels.h:444-493): divides by the full window. */
int swcb200_avgpool_f(swcb200_ctx *ctx, const float *input, float *output, const size_t *idims,
                      const size_t *odims, const size_t *kernels, const size_t *strides,
                      const size_t *pads);
/* Replaces batchnormalization_f (kernels.h:496-517; Codegen.cpp:1907-1915). */
int swcb200_batchnormalization_f(swcb200_ctx *ctx, float *output, const float *input,
                                 const float *mean, const float *var, const float *scale,
                                 const float *bias, const size_t *idims, float epsilon);
/* Replace transpose2d_f / transpose4d_f (kernels.h:519-540): out[idx[shuffle]] = in[idx]. */
int swcb200_transpose2d_f(swcb200_ctx *ctx, const float *input, float *output,
                          const size_t *idims, const size_t *odims, const size_t *shuffle);
int swcb200_transpose4d_f(swcb200_ctx *ctx, const float *input, float *output,
                          const size_t *idims, const size_t *odims, const size_t *shuffle);

/* ------------------------------------- tensor-core path with bf16 storage
 * The graph IR has no 16-bit type (src/common.h:17), so bf16 is a storage mode of the backend:
 * the generator keeps activations and packed weights as bf16 in its arena and calls these
 * instead of the fp32 entry points.  One call covers the chain the lowering pass produces for
 * an FC layer, MatrixMatrixMul -> MatrixVectorAdd -> activation
 * (src/op/dlOp/dlOpEinsum.cpp:154-237). */

int swcb200_cast_f32_to_bf16(swcb200_ctx *ctx, const float *src, void *dst_bf16, size_t count);
int swcb200_cast_bf16_to_f32(swcb200_ctx *ctx, const void *src_bf16, float *dst, size_t count);
/* W[k,n] row-major fp32 (the reference's weight layout) -> Wp[n,k] row-major bf16, the K-major
 * operand layout the tensor-core kernel reads.  Done once per weight, at load time. */
int swcb200_pack_weight_bf16(swcb200_ctx *ctx, const float *w, int k, int n, int ldb,
                             void *wp_bf16);
/* C[m,n] = act(A[m,k] . Wp[n,k]^T + bias[n]).  A, Wp bf16; bias fp32 or NULL; C fp32 or bf16
 * (c_dtype).  lda, ldw multiples of 8 elements and A, Wp 16-byte aligned (TMA rule); C may have
 * any pitch (128-bit stores are used when C and ldc*elem are 16-byte aligned).  fp32 accumulation
 * in tensor memory. */
int swcb200_fc_bf16(swcb200_ctx *ctx, int m, int n, int k, const void *a_bf16, int lda,
                    const void *wp_bf16, int ldw, const float *bias, int act, void *c,
                    int c_dtype, int ldc);
/* The same layer with SPLIT activations, for networks whose decisions hang on less than a bf16
 * rounding of a hidden activation (the k-sequential fp32 sum of kernels.h:41-56 is the yardstick).
 * An activation is carried as two bf16 tensors of the same shape and pitch, hi = bf16(v) and
 * lo = bf16(v - hi); the layer computes act(A_hi . Wp^T + A_lo . Wp^T + bias) in one fp32
 * accumulator.  a_lo NULL: the input has one term (an input that is bf16 to begin with).  c_lo
 * non-NULL (bf16 output only): the output's second term is written there.  About twice the tensor
 * time of swcb200_fc_bf16 when a_lo is given. */
int swcb200_fc_bf16_split(swcb200_ctx *ctx, int m, int n, int k, const void *a_hi, const void *a_lo,
                          int lda, const void *wp_bf16, int ldw, const float *bias, int act,
                          void *c, void *c_lo, int c_dtype, int ldc);

/* filter fp32 [oC,kh,kw,iC] -> bf16, same index order (K-major for the implicit GEMM). */
int swcb200_pack_filter_bf16(swcb200_ctx *ctx, const float *filter, const size_t *fdims,
                             void *fp_bf16);

/* Epilogue applied to a convolution's accumulator, in this order, each step optional:
 * + conv bias; inference batch-norm as an affine map (computed in fp32); + residual;
 * ReLU.  Covers Conv->BN->ReLU and Conv->BN->ElementAdd->ReLU chains. */
typedef struct swcb200_conv_epilogue {
    const float *bn_scale, *bn_bias, *bn_mean, *bn_var; /* all four or none */
    float bn_eps;
    const void *residual; /* same shape and dtype as the convolution's result, or NULL */
    int relu;
    /* MaxPool 2x2, stride 2, no padding (maxpool_f, kernels.h:323-377) applied last, inside the same launch: the
     * output tensor is then [N, OH/2, OW/2, oC] while odims stay the convolution's.  Only where the
     * row-interleaved kernel runs (3x3 filter, 64 -> 64 channels, H, OH and OW even): other shapes return
     * SWCB200_ERR_UNSUPPORTED and the caller pools with swcb200_maxpool_bf16. */
    int pool2x2;
} swcb200_conv_epilogue;
/* NHWC implicit-GEMM convolution on tensor cores (replaces the chain conv2d_f -> batchnormalization_f ->
 * vecAdd_f -> relu_f, kernels.h:177-243, :496-517, :592-596, :575-580, in one launch).  input, filter
 * (swcb200_pack_filter_bf16), output and residual bf16; bias and batch-norm vectors fp32.  stride 1,
 * group 1, iC a multiple of 64, oC a multiple of 32 and <= 256, filter at most 96 KiB in bf16; other
 * shapes return SWCB200_ERR_UNSUPPORTED.  pads[0] (top) and pads[1] (left) are read, as in conv2d_f. */
int swcb200_conv2d_bf16(swcb200_ctx *ctx, void *output, const void *input, const void *fp_bf16,
                        const float *bias, const size_t *odims, const size_t *idims,
                        const size_t *fdims, const size_t *kernels, const size_t *strides,
                        const size_t *pads, const swcb200_conv_epilogue *ep);
/* MaxPool on bf16 NHWC storage (same semantics as maxpool_f). */
int swcb200_maxpool_bf16(swcb200_ctx *ctx, const void *input, void *output, const size_t *idims,
                         const size_t *odims, const size_t *kernels, const size_t *strides,
                         const size_t *pads);

/* ---------------------------------------------------- partitioned graphs
 * NCCL over NVLink in place of the MPI text ParallelCodegen prints
 * (src/codegen/ParallelCodegen.cpp:457-896).  One process per GPU.  `axis` follows the
 * reference's tiling labels (src/parallel/TilingLabel.h): >= 0 splits that axis evenly over
 * the ranks, -1 replicates.  Root is rank 0 in the reference (master/worker); it is a
 * parameter here. */

#define SWCB200_UNIQUE_ID_BYTES 128
#define SWCB200_MAX_PEERS 8 /* ranks whose memory one kernel addresses directly (one NVSwitch box) */
/* Path of libnccl.so.2 to dlopen (NULL: the loader's default search). Call before comm_init. */
int swcb200_comm_load(const char *libnccl_path);
int swcb200_comm_unique_id(void *id_out /* SWCB200_UNIQUE_ID_BYTES */);
/* Replaces MPI_Init/Comm_size/Comm_rank (ParallelCodegen.cpp:94-112). */
int swcb200_comm_init(swcb200_ctx *ctx, const void *unique_id, int nranks, int rank);
int swcb200_comm_destroy(swcb200_ctx *ctx);
int swcb200_comm_rank(swcb200_ctx *ctx, int *rank, int *nranks);
/* Bounded wait for the collectives queued on the context's stream.  Polls the stream and the communicator's
 * asynchronous error state; returns SWCB200_OK once the stream is idle, SWCB200_ERR_NCCL if NCCL reports an
 * error, SWCB200_ERR_TIMEOUT after timeout_ms of wall-clock time.  In both failure cases the communicator has
 * been aborted and removed from the context (a peer has died or hangs): the process does not hang with it.
 * The reference ignores MPI's return codes and has nothing of the kind. */
int swcb200_comm_watch(swcb200_ctx *ctx, int timeout_ms);
/* The same polling loop run against the NCCL library at `libnccl_path` and a stream that never becomes idle;
 * needs no GPU.  For testing the loop with a stand-in library. */
int swcb200_comm_watch_selftest(const char *libnccl_path, int timeout_ms);
/* The Reduce join of a model-parallel layer (ParallelCodegen.cpp:873-896: MPI_Reduce of the partial sums) done by
 * the producing GEMM itself, over peer memory instead of a collective kernel.  Every rank owns m/p rows of the output
 * and holds a slot array of p slots [m/p, ld_slot] fp32, slot r for rank r's partial block.
 *   swcb200_peer_slots_setup      collective, once: exchanges CUDA-IPC handles of the ranks' slot arrays (each must
 *                                 come from the CUDA allocator); all_slots_out[r] = rank r's array as this rank
 *                                 addresses it (SWCB200_MAX_PEERS entries at most).
 *   swcb200_fc_bf16_scatter_rows  C = A . Wp^T (bf16 in, fp32 out, no bias) whose epilogue stores row i into slot
 *                                 `rank` of the array of the rank that owns it, owner_slots[i / (m/p)]: plain 128-bit
 *                                 stores over NVLink, overlapped with the tensor-core work of the other tiles.
 *   swcb200_sum_slots             out[i] = ((s_0[i] + s_1[i]) + ...): the owner adds its p slots in rank order
 *                                 (a result that does not depend on timing), after the ranks have met (e.g. a
 *                                 one-word swcb200_allreduce_sum on the same streams).
 * No waiting on a peer happens inside any kernel. */
int swcb200_peer_slots_setup(swcb200_ctx *ctx, void *local_slots, void **all_slots_out);
int swcb200_peer_slots_release(swcb200_ctx *ctx);
int swcb200_fc_bf16_scatter_rows(swcb200_ctx *ctx, int m, int n, int k, const void *a_bf16, int lda,
                                 const void *wp_bf16, int ldw, void *const *owner_slots, int nranks,
                                 int rank, int ld_slot);
int swcb200_sum_slots(swcb200_ctx *ctx, const float *slots, size_t slot_stride, int nslots, float *out,
                      size_t count);
/* Scatter node (ParallelCodegen.cpp:457-575): axis -1 = MPI_Bcast; axis >= 0 = each rank gets
 * its slice of `src` (read on root only) packed contiguously into `dst`. */
int swcb200_scatter(swcb200_ctx *ctx, const void *src, void *dst, const size_t *dims, int ndim,
                    int axis, int dtype, int root);
/* Gather node (:576-682): inverse of scatter; `dst` is written on root only. */
int swcb200_gather(swcb200_ctx *ctx, const void *src, void *dst, const size_t *dims, int ndim,
                   int axis, int dtype, int root);
/* Gather along axis 0 without kernels: root exports `dst_on_root` once (CUDA IPC, exchanged through the
 * communicator), the other ranks map it, and each swcb200_gather_rows is one device-to-device copy of this
 * rank's `bytes_per_rank` block into its place in root's buffer, done by a copy engine over NVLink on the
 * context's stream.  No SM is used, so a persistent GEMM running beside it is not disturbed (an NCCL
 * send/recv kernel is).  Same result as swcb200_gather(axis 0).  The data is in root's buffer once the
 * SENDER's stream has passed the call: ranks must meet (stream sync, then a host barrier) before root reads
 * it or before the buffer is written again.  setup/release are collective; dst must come from cudaMalloc. */
int swcb200_gather_rows_setup(swcb200_ctx *ctx, void *dst_on_root, size_t bytes_per_rank, int root);
int swcb200_gather_rows(swcb200_ctx *ctx, const void *src);
int swcb200_gather_rows_release(swcb200_ctx *ctx);
/* Reduce node (:873-896): dst(root) = sum over ranks of src. */
int swcb200_reduce_sum(swcb200_ctx *ctx, const void *src, void *dst, size_t count, int dtype,
                       int root);
/* Same sum, result on every rank (what the row-split FC pair needs before its next layer). */
int swcb200_allreduce_sum(swcb200_ctx *ctx, const void *src, void *dst, size_t count, int dtype);
/* Gather along axis 0 with the result on every rank. */
int swcb200_allgather(swcb200_ctx *ctx, const void *src, void *dst, size_t count_per_rank,
                      int dtype);
/* Transform node (:685-871): re-tile a tensor of un-partitioned shape dims[ndim] from pre_axis to
 * post_axis.  Axes: a >= 0 = split along axis a (shards packed: dims[a] / p), -1 = whole tensor on every
 * rank, -2 (pre only) = a full-size partial sum on every rank.  i -> j is an all-to-all, -2 -> j a
 * reduce(-scatter), -1 -> j a local slice, j -> -1 an all-gather. */
int swcb200_transform(swcb200_ctx *ctx, const void *src, void *dst, const size_t *dims, int ndim,
                      int pre_axis, int post_axis, int dtype);

#ifdef __cplusplus
}
#endif
#endif /* SWC_B200_H_ */
