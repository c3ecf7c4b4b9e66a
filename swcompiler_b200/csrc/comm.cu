// Partitioned graphs: the reference's Scatter / Gather / Reduce / Transform nodes over NCCL.
//
// ParallelCodegen prints MPI text for these nodes (src/codegen/ParallelCodegen.cpp:457-896):
// MPI_Bcast or MPI_Type_vector + MPI_Send/Recv for Scatter, the mirror image for Gather, MPI_Reduce for
// Reduce, a ring of MPI_Sendrecv for Transform.  Here each becomes NCCL calls on the context's stream,
// one process per GPU.  NCCL is loaded with dlopen, so the library has no link-time dependency on it
// and a single-GPU user never needs it.
//
// Tiling convention (src/parallel/TilingLabel.h, src/codegen/ParallelCodegen.cpp:503-521): splitting a
// tensor of shape dims[] along `axis` over p ranks views it as `outer` rows of `inner` elements,
// outer = prod(dims[<axis]), inner = prod(dims[>=axis]); rank r owns, of every row, the block
// [r*inner/p, (r+1)*inner/p), and stores its shard packed ([outer, inner/p], leading dimension
// inner/p).  axis 0 shards are contiguous in the full tensor; other axes are strided and go through a
// staging block (the context's scratch) packed and unpacked with strided device copies.
#include <cuda.h>
#include <dlfcn.h>
#include <time.h>

#include <mutex>

#include "common.cuh"

namespace {

typedef void *ncclComm_t;
struct ncclUniqueId {
    char internal[SWCB200_UNIQUE_ID_BYTES];
};
enum { ncclSuccess = 0, ncclInProgress = 7 };
enum { ncclSum = 0 };
enum { ncclInt32 = 2, ncclFloat32 = 7, ncclBfloat16 = 9 };

struct NcclApi {
    void *handle = nullptr;
    int (*GetUniqueId)(ncclUniqueId *) = nullptr;
    int (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*CommAbort)(ncclComm_t) = nullptr;
    int (*CommGetAsyncError)(ncclComm_t, int *) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    int (*Broadcast)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*Reduce)(const void *, void *, size_t, int, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*ReduceScatter)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*Send)(const void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*Recv)(void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
};
NcclApi g_nccl;
std::mutex g_nccl_mutex;

int load_nccl(const char *path) {
    std::lock_guard<std::mutex> lock(g_nccl_mutex);
    if (g_nccl.handle) return SWCB200_OK;
    void *h = dlopen(path ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h && !path) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return SWCB200_ERR_NCCL;
#define SWC_SYM(field, name)                                        \
    *(void **)(&g_nccl.field) = dlsym(h, name);                     \
    if (!g_nccl.field) {                                            \
        dlclose(h);                                                 \
        return SWCB200_ERR_NCCL;                                    \
    }
    SWC_SYM(GetUniqueId, "ncclGetUniqueId")
    SWC_SYM(CommInitRank, "ncclCommInitRank")
    SWC_SYM(CommDestroy, "ncclCommDestroy")
    SWC_SYM(CommAbort, "ncclCommAbort")
    SWC_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
    SWC_SYM(GetErrorString, "ncclGetErrorString")
    SWC_SYM(Broadcast, "ncclBroadcast")
    SWC_SYM(AllReduce, "ncclAllReduce")
    SWC_SYM(Reduce, "ncclReduce")
    SWC_SYM(ReduceScatter, "ncclReduceScatter")
    SWC_SYM(AllGather, "ncclAllGather")
    SWC_SYM(Send, "ncclSend")
    SWC_SYM(Recv, "ncclRecv")
    SWC_SYM(GroupStart, "ncclGroupStart")
    SWC_SYM(GroupEnd, "ncclGroupEnd")
#undef SWC_SYM
    g_nccl.handle = h;
    return SWCB200_OK;
}

}  // namespace

struct swcb200_comm {
    ncclComm_t comm = nullptr;
    int rank = 0, nranks = 1;
    // peer-copy gather (swcb200_gather_rows_*): root's destination as this rank can address it
    void *rows_dst = nullptr;      // on root: the caller's buffer; elsewhere: the IPC mapping + offset
    void *rows_ipc_base = nullptr; // what cudaIpcOpenMemHandle returned (non-root), to close later
    size_t rows_bytes = 0;
    int rows_root = -1;
    // peer slots (swcb200_peer_slots_*): every rank's slot array as this rank can address it
    void *slots[SWCB200_MAX_PEERS] = {nullptr};      // [rank]: own array, or IPC mapping + offset
    void *slots_ipc_base[SWCB200_MAX_PEERS] = {nullptr};
    int slots_ready = 0;
};

namespace {

#define SWC_NCCL(ctx, call)                                                                              \
    do {                                                                                                 \
        int r__ = (call);                                                                                \
        if (r__ != ncclSuccess)                                                                          \
            return swc_fail((ctx), SWCB200_ERR_NCCL, "%s: %s", #call, g_nccl.GetErrorString(r__));       \
    } while (0)

// An NCCL group that is closed on every way out of the scope: a Send or Recv that fails returns from the
// middle of the group, and a group left open would swallow every later collective of the thread.
struct NcclGroup {
    bool open = false;
    int start() {
        int r = g_nccl.GroupStart();
        open = r == ncclSuccess;
        return r;
    }
    int end() {
        open = false;
        return g_nccl.GroupEnd();
    }
    ~NcclGroup() {
        if (open) g_nccl.GroupEnd();
    }
};

int nccl_type(int dtype, size_t *elem) {
    switch (dtype) {
        case SWCB200_F32: *elem = 4; return ncclFloat32;
        case SWCB200_BF16: *elem = 2; return ncclBfloat16;
        case SWCB200_I32: *elem = 4; return ncclInt32;
        default: *elem = 0; return -1;
    }
}

struct Tiling {
    size_t outer, inner, blk, elem;
    int type;
};

int make_tiling(swcb200_ctx *ctx, const char *what, const size_t *dims, int ndim, int axis, int dtype, Tiling *t) {
    SWC_REQUIRE(ctx, ctx->comm != nullptr, SWCB200_ERR_NCCL, "%s: no communicator (call swcb200_comm_init)", what);
    SWC_REQUIRE(ctx, dims && ndim >= 1 && ndim <= 8, SWCB200_ERR_BAD_ARG, "%s: bad dims", what);
    SWC_REQUIRE(ctx, axis >= -1 && axis < ndim, SWCB200_ERR_BAD_ARG, "%s: axis %d outside [-1, %d)", what, axis, ndim);
    t->type = nccl_type(dtype, &t->elem);
    SWC_REQUIRE(ctx, t->type >= 0, SWCB200_ERR_BAD_ARG, "%s: unknown dtype %d", what, dtype);
    t->outer = 1;
    t->inner = 1;
    for (int d = 0; d < ndim; d++) {
        if (axis >= 0 && d < axis)
            t->outer *= dims[d];
        else
            t->inner *= dims[d];
    }
    const size_t p = (size_t)ctx->comm->nranks;
    if (axis >= 0) {
        // the tiling pass only picks strategies with dim % p == 0 (src/pass/ParallelLabelingPass.h:95-135)
        SWC_REQUIRE(ctx, dims[axis] % p == 0, SWCB200_ERR_BAD_SHAPE, "%s: dims[%d] = %zu not divisible by %zu ranks", what,
                    axis, dims[axis], p);
        t->blk = t->inner / p;
    } else {
        t->blk = t->inner;
    }
    return SWCB200_OK;
}

// strided [outer x blk] window of a row-major [outer x inner] matrix <-> packed [outer x blk]
int copy_window(swcb200_ctx *ctx, void *dst, size_t dst_pitch_elems, const void *src, size_t src_pitch_elems, size_t blk,
                size_t outer, size_t elem) {
    SWC_CUDA(ctx, cudaMemcpy2DAsync(dst, dst_pitch_elems * elem, src, src_pitch_elems * elem, blk * elem, outer,
                                    cudaMemcpyDeviceToDevice, ctx->stream));
    return SWCB200_OK;
}

}  // namespace

SWC_EXPORT int swcb200_comm_load(const char *libnccl_path) { return load_nccl(libnccl_path); }

SWC_EXPORT int swcb200_comm_unique_id(void *id_out) {
    if (!id_out) return SWCB200_ERR_BAD_ARG;
    int rc = load_nccl(nullptr);
    if (rc) return rc;
    ncclUniqueId id;
    if (g_nccl.GetUniqueId(&id) != ncclSuccess) return SWCB200_ERR_NCCL;
    memcpy(id_out, &id, sizeof(id));
    return SWCB200_OK;
}

SWC_EXPORT int swcb200_comm_init(swcb200_ctx *ctx, const void *unique_id, int nranks, int rank) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, unique_id && nranks >= 1 && rank >= 0 && rank < nranks, SWCB200_ERR_BAD_ARG, "comm_init: bad argument");
    SWC_REQUIRE(ctx, ctx->comm == nullptr, SWCB200_ERR_BAD_ARG, "comm_init: context already has a communicator");
    int rc = load_nccl(nullptr);
    SWC_REQUIRE(ctx, rc == SWCB200_OK, SWCB200_ERR_NCCL, "comm_init: libnccl.so.2 could not be loaded (%s)", dlerror());
    ncclUniqueId id;
    memcpy(&id, unique_id, sizeof(id));
    swcb200_comm *c = new swcb200_comm();
    c->rank = rank;
    c->nranks = nranks;
    int r = g_nccl.CommInitRank(&c->comm, nranks, id, rank);
    if (r != ncclSuccess) {
        delete c;
        return swc_fail(ctx, SWCB200_ERR_NCCL, "ncclCommInitRank: %s", g_nccl.GetErrorString(r));
    }
    ctx->comm = c;
    return SWCB200_OK;
}

SWC_EXPORT int swcb200_comm_destroy(swcb200_ctx *ctx) {
    if (!ctx) return SWCB200_ERR_BAD_ARG;
    if (!ctx->comm) return SWCB200_OK;
    swcb200_gather_rows_release(ctx);
    swcb200_peer_slots_release(ctx);
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    int r = g_nccl.CommDestroy(ctx->comm->comm);
    delete ctx->comm;
    ctx->comm = nullptr;
    return r == ncclSuccess ? SWCB200_OK : SWCB200_ERR_NCCL;
}

// ---------------------------------------------------------------------------------------------------
// Failure detection on the host.  A collective whose peer has died never completes, and a host thread that
// synchronises its stream behind it waits for ever.  swcb200_comm_watch is the bounded form of that
// synchronisation: it polls the stream and the communicator's asynchronous error state until the stream is
// idle (OK), NCCL reports an error (ERR_NCCL) or the wall-clock limit has passed (ERR_TIMEOUT); in the two
// failure cases the communicator is aborted, which takes its kernels off the GPU, and dropped, so that the
// process can carry on (or exit) instead of hanging.  The reference has no counterpart: its MPI return
// codes are ignored (src/codegen/ParallelCodegen.cpp:457-896).
namespace {

struct WatchFns {
    int (*stream_idle)(void *stream);                 // 1 idle, 0 busy, < 0 error
    int (*async_error)(void *comm, int *state);       // NCCL's convention: returns ncclSuccess, state = ncclSuccess / ncclInProgress / error
    int (*abort)(void *comm);
};

int watch_loop(const WatchFns &f, void *comm, void *stream, int timeout_ms, char *err, size_t errlen) {
    timespec t0;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (unsigned spin = 0;; spin++) {
        const int idle = f.stream_idle(stream);
        if (idle > 0) return SWCB200_OK;
        if (idle < 0) {
            snprintf(err, errlen, "comm_watch: the stream reported an error");
            return SWCB200_ERR_CUDA;
        }
        int state = ncclSuccess;
        if (f.async_error(comm, &state) != ncclSuccess || (state != ncclSuccess && state != ncclInProgress)) {
            f.abort(comm);
            snprintf(err, errlen, "comm_watch: the communicator reported an asynchronous error (state %d); aborted", state);
            return SWCB200_ERR_NCCL;
        }
        timespec t1;
        clock_gettime(CLOCK_MONOTONIC, &t1);
        const long long ms = (t1.tv_sec - t0.tv_sec) * 1000ll + (t1.tv_nsec - t0.tv_nsec) / 1000000ll;
        if (ms > timeout_ms) {
            f.abort(comm);
            snprintf(err, errlen, "comm_watch: collectives still pending after %d ms; communicator aborted", timeout_ms);
            return SWCB200_ERR_TIMEOUT;
        }
        if (spin > 64) {  // a short sleep once the quick polls have not sufficed
            timespec nap = {0, 200000};
            nanosleep(&nap, nullptr);
        }
    }
}

int real_stream_idle(void *stream) {
    cudaError_t e = cudaStreamQuery((cudaStream_t)stream);
    if (e == cudaSuccess) return 1;
    if (e == cudaErrorNotReady) return 0;
    cudaGetLastError();
    return -1;
}
int real_async_error(void *comm, int *state) { return g_nccl.CommGetAsyncError((ncclComm_t)comm, state); }
int real_abort(void *comm) { return g_nccl.CommAbort((ncclComm_t)comm); }

}  // namespace

SWC_EXPORT int swcb200_comm_watch(swcb200_ctx *ctx, int timeout_ms) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, ctx->comm != nullptr, SWCB200_ERR_NCCL, "comm_watch: no communicator");
    SWC_REQUIRE(ctx, timeout_ms > 0, SWCB200_ERR_BAD_ARG, "comm_watch: the limit must be positive");
    const WatchFns f = {real_stream_idle, real_async_error, real_abort};
    int rc = watch_loop(f, ctx->comm->comm, ctx->stream, timeout_ms, ctx->last_error, sizeof(ctx->last_error));
    if (rc == SWCB200_ERR_NCCL || rc == SWCB200_ERR_TIMEOUT) {
        // the communicator is gone (ncclCommAbort frees it); peer mappings of the row gather go with it
        swcb200_gather_rows_release(ctx);
        swcb200_peer_slots_release(ctx);
        delete ctx->comm;
        ctx->comm = nullptr;
    }
    return rc;
}

// The watch loop against an NCCL library given by path and a stream that never becomes idle, without any GPU:
// for a stand-in library whose asynchronous error state stays "in progress" (expected: SWCB200_ERR_TIMEOUT after
// timeout_ms, one abort) or turns into an error (expected: SWCB200_ERR_NCCL, one abort).
SWC_EXPORT int swcb200_comm_watch_selftest(const char *libnccl_path, int timeout_ms) {
    int rc = load_nccl(libnccl_path);
    if (rc) return rc;
    ncclUniqueId id;
    if (g_nccl.GetUniqueId(&id) != ncclSuccess) return SWCB200_ERR_NCCL;
    ncclComm_t comm = nullptr;
    if (g_nccl.CommInitRank(&comm, 1, id, 0) != ncclSuccess) return SWCB200_ERR_NCCL;
    const WatchFns f = {[](void *) { return 0; }, real_async_error, real_abort};
    char err[256];
    return watch_loop(f, comm, nullptr, timeout_ms, err, sizeof(err));
}

SWC_EXPORT int swcb200_comm_rank(swcb200_ctx *ctx, int *rank, int *nranks) {
    if (!ctx || !ctx->comm) return SWCB200_ERR_BAD_ARG;
    if (rank) *rank = ctx->comm->rank;
    if (nranks) *nranks = ctx->comm->nranks;
    return SWCB200_OK;
}

SWC_EXPORT int swcb200_scatter(swcb200_ctx *ctx, const void *src, void *dst, const size_t *dims, int ndim, int axis,
                               int dtype, int root) {
    SWC_CTX(ctx);
    Tiling t;
    int rc = make_tiling(ctx, "scatter", dims, ndim, axis, dtype, &t);
    if (rc) return rc;
    swcb200_comm *c = ctx->comm;
    SWC_REQUIRE(ctx, root >= 0 && root < c->nranks, SWCB200_ERR_BAD_ARG, "scatter: bad root");
    SWC_REQUIRE(ctx, dst && (c->rank != root || src), SWCB200_ERR_BAD_ARG, "scatter: null tensor");
    const size_t shard = t.outer * t.blk;
    if (shard == 0) return SWCB200_OK;
    if (axis < 0) {  // replicate: MPI_Bcast in the reference (ParallelCodegen.cpp:488-495)
        SWC_NCCL(ctx, g_nccl.Broadcast(c->rank == root ? src : dst, dst, shard, t.type, root, c->comm, ctx->stream));
        return SWCB200_OK;
    }
    const uint8_t *send_base = (const uint8_t *)src;
    if (c->rank == root && t.outer > 1) {
        // strided shards: pack every peer's window into the staging block first
        void *stage = nullptr;
        rc = swc_scratch(ctx, shard * t.elem * c->nranks, &stage);
        if (rc) return rc;
        for (int r = 0; r < c->nranks; r++) {
            if (r == root) continue;
            rc = copy_window(ctx, (uint8_t *)stage + (size_t)r * shard * t.elem, t.blk,
                             (const uint8_t *)src + (size_t)r * t.blk * t.elem, t.inner, t.blk, t.outer, t.elem);
            if (rc) return rc;
        }
        send_base = (const uint8_t *)stage;
    }
    NcclGroup group;
    SWC_NCCL(ctx, group.start());
    if (c->rank == root) {
        for (int r = 0; r < c->nranks; r++)
            if (r != root)
                SWC_NCCL(ctx, g_nccl.Send(send_base + (size_t)r * shard * t.elem, shard, t.type, r, c->comm, ctx->stream));
    } else {
        SWC_NCCL(ctx, g_nccl.Recv(dst, shard, t.type, root, c->comm, ctx->stream));
    }
    SWC_NCCL(ctx, group.end());
    if (c->rank == root)  // root's own shard: a local copy
        return copy_window(ctx, dst, t.blk, (const uint8_t *)src + (size_t)root * t.blk * t.elem, t.inner, t.blk, t.outer,
                           t.elem);
    return SWCB200_OK;
}

SWC_EXPORT int swcb200_gather(swcb200_ctx *ctx, const void *src, void *dst, const size_t *dims, int ndim, int axis,
                              int dtype, int root) {
    SWC_CTX(ctx);
    Tiling t;
    int rc = make_tiling(ctx, "gather", dims, ndim, axis, dtype, &t);
    if (rc) return rc;
    swcb200_comm *c = ctx->comm;
    SWC_REQUIRE(ctx, root >= 0 && root < c->nranks, SWCB200_ERR_BAD_ARG, "gather: bad root");
    SWC_REQUIRE(ctx, src && (c->rank != root || dst), SWCB200_ERR_BAD_ARG, "gather: null tensor");
    const size_t shard = t.outer * t.blk;
    if (shard == 0) return SWCB200_OK;
    if (axis < 0) {  // a replicated tensor: root already has it
        if (c->rank == root && dst != src)
            SWC_CUDA(ctx, cudaMemcpyAsync(dst, src, shard * t.elem, cudaMemcpyDeviceToDevice, ctx->stream));
        return SWCB200_OK;
    }
    uint8_t *recv_base = (uint8_t *)dst;
    const bool staged = c->rank == root && t.outer > 1;
    if (staged) {
        void *stage = nullptr;
        rc = swc_scratch(ctx, shard * t.elem * c->nranks, &stage);
        if (rc) return rc;
        recv_base = (uint8_t *)stage;
    }
    NcclGroup group;
    SWC_NCCL(ctx, group.start());
    if (c->rank == root) {
        for (int r = 0; r < c->nranks; r++)
            if (r != root)
                SWC_NCCL(ctx, g_nccl.Recv(recv_base + (size_t)r * shard * t.elem, shard, t.type, r, c->comm, ctx->stream));
    } else {
        SWC_NCCL(ctx, g_nccl.Send(src, shard, t.type, root, c->comm, ctx->stream));
    }
    SWC_NCCL(ctx, group.end());
    if (c->rank == root) {
        rc = copy_window(ctx, (uint8_t *)dst + (size_t)root * t.blk * t.elem, t.inner, src, t.blk, t.blk, t.outer, t.elem);
        if (rc) return rc;
        if (staged)
            for (int r = 0; r < c->nranks; r++) {
                if (r == root) continue;
                rc = copy_window(ctx, (uint8_t *)dst + (size_t)r * t.blk * t.elem, t.inner,
                                 recv_base + (size_t)r * shard * t.elem, t.blk, t.blk, t.outer, t.elem);
                if (rc) return rc;
            }
    }
    return SWCB200_OK;
}

// ---- Gather along axis 0 by peer-to-peer copies.
// ncclSend/ncclRecv run as kernels and take SMs for the length of the transfer; a persistent GEMM that
// wants every SM then waits for them.  A Gather of contiguous row blocks needs no kernel at all: root
// exports its destination buffer once (CUDA IPC), every other rank maps it, and each Gather is one
// cudaMemcpyAsync on the sender's stream, carried out by a copy engine over NVLink.
namespace {
typedef CUresult (*GetRangeFn)(CUdeviceptr *, size_t *, CUdeviceptr);
GetRangeFn get_range_fn() {
    static GetRangeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (GetRangeFn)p;
    });
    return fn;
}
struct RowsExport {
    cudaIpcMemHandle_t handle;
    unsigned long long offset;
};
}  // namespace

SWC_EXPORT int swcb200_gather_rows_setup(swcb200_ctx *ctx, void *dst_on_root, size_t bytes_per_rank, int root) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, ctx->comm != nullptr, SWCB200_ERR_NCCL, "gather_rows_setup: no communicator");
    swcb200_comm *c = ctx->comm;
    SWC_REQUIRE(ctx, root >= 0 && root < c->nranks && bytes_per_rank > 0, SWCB200_ERR_BAD_ARG, "gather_rows_setup: bad argument");
    SWC_REQUIRE(ctx, c->rank != root || dst_on_root != nullptr, SWCB200_ERR_BAD_ARG, "gather_rows_setup: root needs a destination");
    SWC_REQUIRE(ctx, c->rows_root < 0, SWCB200_ERR_BAD_ARG, "gather_rows_setup: already set up (release first)");
    RowsExport ex;
    memset(&ex, 0, sizeof(ex));
    if (c->rank == root) {
        GetRangeFn range = get_range_fn();
        SWC_REQUIRE(ctx, range != nullptr, SWCB200_ERR_CUDA, "gather_rows_setup: cuMemGetAddressRange not found");
        CUdeviceptr base = 0;
        size_t size = 0;
        SWC_REQUIRE(ctx, range(&base, &size, (CUdeviceptr)dst_on_root) == CUDA_SUCCESS, SWCB200_ERR_CUDA,
                    "gather_rows_setup: destination is not a device allocation");
        SWC_CUDA(ctx, cudaIpcGetMemHandle(&ex.handle, (void *)base));
        ex.offset = (unsigned long long)((CUdeviceptr)dst_on_root - base);
    }
    // hand the export to every rank through the communicator (a small device-side broadcast)
    void *dev = nullptr;
    int rc = swc_scratch(ctx, sizeof(ex), &dev);
    if (rc) return rc;
    SWC_CUDA(ctx, cudaMemcpyAsync(dev, &ex, sizeof(ex), cudaMemcpyHostToDevice, ctx->stream));
    SWC_NCCL(ctx, g_nccl.Broadcast(dev, dev, sizeof(ex), /*ncclInt8*/ 0, root, c->comm, ctx->stream));
    SWC_CUDA(ctx, cudaMemcpyAsync(&ex, dev, sizeof(ex), cudaMemcpyDeviceToHost, ctx->stream));
    SWC_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (c->rank == root) {
        c->rows_dst = dst_on_root;
    } else {
        void *mapped = nullptr;
        SWC_CUDA(ctx, cudaIpcOpenMemHandle(&mapped, ex.handle, cudaIpcMemLazyEnablePeerAccess));
        c->rows_ipc_base = mapped;
        c->rows_dst = (uint8_t *)mapped + ex.offset;
    }
    c->rows_bytes = bytes_per_rank;
    c->rows_root = root;
    return SWCB200_OK;
}

SWC_EXPORT int swcb200_gather_rows(swcb200_ctx *ctx, const void *src) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, ctx->comm != nullptr && ctx->comm->rows_root >= 0, SWCB200_ERR_BAD_ARG,
                "gather_rows: call swcb200_gather_rows_setup first");
    SWC_REQUIRE(ctx, src != nullptr, SWCB200_ERR_BAD_ARG, "gather_rows: null source");
    swcb200_comm *c = ctx->comm;
    SWC_CUDA(ctx, cudaMemcpyAsync((uint8_t *)c->rows_dst + (size_t)c->rank * c->rows_bytes, src, c->rows_bytes,
                                  cudaMemcpyDeviceToDevice, ctx->stream));
    return SWCB200_OK;
}

SWC_EXPORT int swcb200_gather_rows_release(swcb200_ctx *ctx) {
    if (!ctx) return SWCB200_ERR_BAD_ARG;
    if (!ctx->comm || ctx->comm->rows_root < 0) return SWCB200_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->comm->rows_ipc_base) cudaIpcCloseMemHandle(ctx->comm->rows_ipc_base);
    ctx->comm->rows_ipc_base = ctx->comm->rows_dst = nullptr;
    ctx->comm->rows_root = -1;
    return SWCB200_OK;
}

// Peer slots: the join of a model-parallel layer without a collective kernel.  Every rank owns a block of the
// output rows and keeps, for each rank, a slot that rank's partial block is written into -- by the producing GEMM's
// own epilogue, straight over NVLink (swcb200_fc_bf16_scatter_rows).  Here the ranks exchange CUDA-IPC handles of
// their slot arrays once, so that each can address all of them.
SWC_EXPORT int swcb200_peer_slots_setup(swcb200_ctx *ctx, void *local_slots, void **all_slots_out) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, ctx->comm != nullptr, SWCB200_ERR_NCCL, "peer_slots_setup: no communicator");
    swcb200_comm *c = ctx->comm;
    SWC_REQUIRE(ctx, c->nranks <= SWCB200_MAX_PEERS, SWCB200_ERR_UNSUPPORTED, "peer_slots_setup: at most %d ranks", SWCB200_MAX_PEERS);
    SWC_REQUIRE(ctx, local_slots && all_slots_out, SWCB200_ERR_BAD_ARG, "peer_slots_setup: null argument");
    SWC_REQUIRE(ctx, !c->slots_ready, SWCB200_ERR_BAD_ARG, "peer_slots_setup: already set up (release first)");
    GetRangeFn range = get_range_fn();
    SWC_REQUIRE(ctx, range != nullptr, SWCB200_ERR_CUDA, "peer_slots_setup: cuMemGetAddressRange not found");
    RowsExport mine;
    memset(&mine, 0, sizeof(mine));
    CUdeviceptr base = 0;
    size_t size = 0;
    SWC_REQUIRE(ctx, range(&base, &size, (CUdeviceptr)local_slots) == CUDA_SUCCESS, SWCB200_ERR_CUDA,
                "peer_slots_setup: the slot array is not a device allocation");
    SWC_CUDA(ctx, cudaIpcGetMemHandle(&mine.handle, (void *)base));
    mine.offset = (unsigned long long)((CUdeviceptr)local_slots - base);
    // every rank's export to every rank: an all-gather of a few bytes through the communicator
    void *dev = nullptr;
    int rc = swc_scratch(ctx, sizeof(mine) * (size_t)(c->nranks + 1), &dev);
    if (rc) return rc;
    RowsExport all[SWCB200_MAX_PEERS];
    uint8_t *send = (uint8_t *)dev, *recv = send + sizeof(mine);
    SWC_CUDA(ctx, cudaMemcpyAsync(send, &mine, sizeof(mine), cudaMemcpyHostToDevice, ctx->stream));
    SWC_NCCL(ctx, g_nccl.AllGather(send, recv, sizeof(mine), /*ncclInt8*/ 0, c->comm, ctx->stream));
    SWC_CUDA(ctx, cudaMemcpyAsync(all, recv, sizeof(mine) * (size_t)c->nranks, cudaMemcpyDeviceToHost, ctx->stream));
    SWC_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (int r = 0; r < c->nranks; r++) {
        if (r == c->rank) {
            c->slots[r] = local_slots;
            continue;
        }
        void *mapped = nullptr;
        SWC_CUDA(ctx, cudaIpcOpenMemHandle(&mapped, all[r].handle, cudaIpcMemLazyEnablePeerAccess));
        c->slots_ipc_base[r] = mapped;
        c->slots[r] = (uint8_t *)mapped + all[r].offset;
    }
    c->slots_ready = 1;
    for (int r = 0; r < c->nranks; r++) all_slots_out[r] = c->slots[r];
    return SWCB200_OK;
}

SWC_EXPORT int swcb200_peer_slots_release(swcb200_ctx *ctx) {
    if (!ctx) return SWCB200_ERR_BAD_ARG;
    if (!ctx->comm || !ctx->comm->slots_ready) return SWCB200_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (int r = 0; r < SWCB200_MAX_PEERS; r++) {
        if (ctx->comm->slots_ipc_base[r]) cudaIpcCloseMemHandle(ctx->comm->slots_ipc_base[r]);
        ctx->comm->slots_ipc_base[r] = ctx->comm->slots[r] = nullptr;
    }
    ctx->comm->slots_ready = 0;
    return SWCB200_OK;
}

SWC_EXPORT int swcb200_reduce_sum(swcb200_ctx *ctx, const void *src, void *dst, size_t count, int dtype, int root) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, ctx->comm != nullptr, SWCB200_ERR_NCCL, "reduce_sum: no communicator");
    size_t elem;
    int type = nccl_type(dtype, &elem);
    SWC_REQUIRE(ctx, type >= 0, SWCB200_ERR_BAD_ARG, "reduce_sum: unknown dtype");
    SWC_REQUIRE(ctx, root >= 0 && root < ctx->comm->nranks, SWCB200_ERR_BAD_ARG, "reduce_sum: bad root");
    if (count == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, src && (ctx->comm->rank != root || dst), SWCB200_ERR_BAD_ARG, "reduce_sum: null tensor");
    SWC_NCCL(ctx, g_nccl.Reduce(src, dst, count, type, ncclSum, root, ctx->comm->comm, ctx->stream));
    return SWCB200_OK;
}

SWC_EXPORT int swcb200_allreduce_sum(swcb200_ctx *ctx, const void *src, void *dst, size_t count, int dtype) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, ctx->comm != nullptr, SWCB200_ERR_NCCL, "allreduce_sum: no communicator");
    size_t elem;
    int type = nccl_type(dtype, &elem);
    SWC_REQUIRE(ctx, type >= 0, SWCB200_ERR_BAD_ARG, "allreduce_sum: unknown dtype");
    if (count == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, src && dst, SWCB200_ERR_BAD_ARG, "allreduce_sum: null tensor");
    SWC_NCCL(ctx, g_nccl.AllReduce(src, dst, count, type, ncclSum, ctx->comm->comm, ctx->stream));
    return SWCB200_OK;
}

SWC_EXPORT int swcb200_allgather(swcb200_ctx *ctx, const void *src, void *dst, size_t count_per_rank, int dtype) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, ctx->comm != nullptr, SWCB200_ERR_NCCL, "allgather: no communicator");
    size_t elem;
    int type = nccl_type(dtype, &elem);
    SWC_REQUIRE(ctx, type >= 0, SWCB200_ERR_BAD_ARG, "allgather: unknown dtype");
    if (count_per_rank == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, src && dst, SWCB200_ERR_BAD_ARG, "allgather: null tensor");
    SWC_NCCL(ctx, g_nccl.AllGather(src, dst, count_per_rank, type, ctx->comm->comm, ctx->stream));
    return SWCB200_OK;
}

namespace {

// Re-tiling of a tensor with any number of dimensions.  A tile split along axis a, seen as `outer` rows of
// `inner` elements (outer = product of the tile's dims before a, inner = of those from a on), holds for every
// rank q one window of inner/p columns; the reference builds MPI vector types of exactly this shape
// (src/codegen/ParallelCodegen.cpp:723-797).  split i -> split j: the window for q along j of the local tile is
// packed, exchanged, and unpacked as the window from q along i of the result tile; both sides enumerate the same
// sub-box (i in the sender's range, j in the receiver's) in row-major order.
int transform_nd(swcb200_ctx *ctx, const void *src, void *dst, const size_t *dims, int ndim, int pre, int post, int dtype) {
    size_t elem;
    int type = nccl_type(dtype, &elem);
    SWC_REQUIRE(ctx, type >= 0, SWCB200_ERR_BAD_ARG, "transform: unknown dtype");
    swcb200_comm *c = ctx->comm;
    const size_t p = (size_t)c->nranks;
    size_t total = 1;
    for (int d = 0; d < ndim; d++) total *= dims[d];
    if (total == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, src && dst, SWCB200_ERR_BAD_ARG, "transform: null tensor");
    SWC_REQUIRE(ctx, pre < 0 || dims[pre] % p == 0, SWCB200_ERR_BAD_SHAPE, "transform: dims[%d] not divisible by the ranks", pre);
    SWC_REQUIRE(ctx, post < 0 || dims[post] % p == 0, SWCB200_ERR_BAD_SHAPE, "transform: dims[%d] not divisible by the ranks", post);
    // (outer, inner) of a tensor whose dims are `dims` with dims[split] divided by p (split < 0: undivided), seen along `axis`
    auto view = [&](int split, int axis, size_t *outer, size_t *inner) {
        *outer = 1;
        *inner = 1;
        for (int d = 0; d < ndim; d++) {
            const size_t e = d == split ? dims[d] / p : dims[d];
            if (d < axis)
                *outer *= e;
            else
                *inner *= e;
        }
    };
    const uint8_t *s = (const uint8_t *)src;
    uint8_t *d = (uint8_t *)dst;
    const size_t tile = total / p;
    int rc;
    if (pre == post) {
        const size_t n = pre >= 0 ? tile : total;
        if (dst != src) SWC_CUDA(ctx, cudaMemcpyAsync(dst, src, n * elem, cudaMemcpyDeviceToDevice, ctx->stream));
        return SWCB200_OK;
    }
    if (pre == -1 || pre == -2) {
        const uint8_t *full = s;
        if (pre == -2) {  // partial sums: reduce first (MPI_Reduce + master scatter in the reference, :798-862)
            if (post == -1) {
                SWC_NCCL(ctx, g_nccl.AllReduce(src, dst, total, type, ncclSum, c->comm, ctx->stream));
                return SWCB200_OK;
            }
            void *stage = nullptr;
            rc = swc_scratch(ctx, total * elem, &stage);
            if (rc) return rc;
            SWC_NCCL(ctx, g_nccl.AllReduce(src, stage, total, type, ncclSum, c->comm, ctx->stream));
            full = (const uint8_t *)stage;
        }
        size_t outer, inner;  // replicated -> split: the local window, no communication (:864-867)
        view(-1, post, &outer, &inner);
        const size_t blk = inner / p;
        return copy_window(ctx, d, blk, full + (size_t)c->rank * blk * elem, inner, blk, outer, elem);
    }
    if (post == -1) {  // split -> replicated: all-gather the tiles, then place each as its window along `pre`
        void *stage = nullptr;
        rc = swc_scratch(ctx, total * elem, &stage);
        if (rc) return rc;
        SWC_NCCL(ctx, g_nccl.AllGather(src, stage, tile, type, c->comm, ctx->stream));
        size_t outer, inner;
        view(-1, pre, &outer, &inner);
        const size_t blk = inner / p;
        for (size_t q = 0; q < p; q++) {
            rc = copy_window(ctx, d + q * blk * elem, inner, (const uint8_t *)stage + q * tile * elem, blk, blk, outer, elem);
            if (rc) return rc;
        }
        return SWCB200_OK;
    }
    // split pre -> split post
    size_t so, si, ro, ri;
    view(pre, post, &so, &si);   // the local tile, seen along `post`
    view(post, pre, &ro, &ri);   // the result tile, seen along `pre`
    const size_t sblk = si / p, rblk = ri / p, box = tile / p;
    void *stage = nullptr;
    rc = swc_scratch(ctx, 2 * tile * elem, &stage);
    if (rc) return rc;
    uint8_t *st_send = (uint8_t *)stage, *st_recv = st_send + tile * elem;
    for (size_t q = 0; q < p; q++) {
        rc = copy_window(ctx, st_send + q * box * elem, sblk, s + q * sblk * elem, si, sblk, so, elem);
        if (rc) return rc;
    }
    NcclGroup group;
    SWC_NCCL(ctx, group.start());
    for (size_t q = 0; q < p; q++) {
        SWC_NCCL(ctx, g_nccl.Send(st_send + q * box * elem, box, type, (int)q, c->comm, ctx->stream));
        SWC_NCCL(ctx, g_nccl.Recv(st_recv + q * box * elem, box, type, (int)q, c->comm, ctx->stream));
    }
    SWC_NCCL(ctx, group.end());
    for (size_t q = 0; q < p; q++) {
        rc = copy_window(ctx, d + q * rblk * elem, ri, st_recv + q * box * elem, rblk, rblk, ro, elem);
        if (rc) return rc;
    }
    return SWCB200_OK;
}

}  // namespace

// Re-tiling.  Shards are packed: split along axis a -> the tensor with dims[a] / p; -1 -> the whole tensor on every
// rank; -2 -> a full-size partial sum on every rank.  2-D tensors [R, C] take the paths below (contiguous blocks are
// exchanged in place); other ranks of tensor go through transform_nd.
SWC_EXPORT int swcb200_transform(swcb200_ctx *ctx, const void *src, void *dst, const size_t *dims, int ndim, int pre_axis,
                                 int post_axis, int dtype) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, ctx->comm != nullptr, SWCB200_ERR_NCCL, "transform: no communicator");
    SWC_REQUIRE(ctx, dims && ndim >= 1 && ndim <= 8, SWCB200_ERR_BAD_ARG, "transform: bad dims");
    SWC_REQUIRE(ctx, pre_axis >= -2 && pre_axis < ndim && post_axis >= -1 && post_axis < ndim, SWCB200_ERR_BAD_ARG,
                "transform: axes must be in {-2,-1,0..%d} -> {-1,0..%d}", ndim - 1, ndim - 1);
    if (ndim != 2) return transform_nd(ctx, src, dst, dims, ndim, pre_axis, post_axis, dtype);
    size_t elem;
    int type = nccl_type(dtype, &elem);
    SWC_REQUIRE(ctx, type >= 0, SWCB200_ERR_BAD_ARG, "transform: unknown dtype");
    swcb200_comm *c = ctx->comm;
    const size_t p = (size_t)c->nranks, R = dims[0], C = dims[1];
    if (R * C == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, src && dst, SWCB200_ERR_BAD_ARG, "transform: null tensor");
    SWC_REQUIRE(ctx, (pre_axis != 0 && post_axis != 0) || R % p == 0, SWCB200_ERR_BAD_SHAPE, "transform: rows not divisible");
    SWC_REQUIRE(ctx, (pre_axis != 1 && post_axis != 1) || C % p == 0, SWCB200_ERR_BAD_SHAPE, "transform: columns not divisible");
    const size_t Rp = R / p, Cp = C / p;
    const uint8_t *s = (const uint8_t *)src;
    uint8_t *d = (uint8_t *)dst;
    int rc;
    if (pre_axis == post_axis) {
        size_t n = pre_axis == 0 ? Rp * C : pre_axis == 1 ? R * Cp : R * C;
        if (dst != src) SWC_CUDA(ctx, cudaMemcpyAsync(dst, src, n * elem, cudaMemcpyDeviceToDevice, ctx->stream));
        return SWCB200_OK;
    }
    if (pre_axis == -1) {  // replicated -> split: take the local slice, no communication (ParallelCodegen.cpp:864-867)
        if (post_axis == 0) return copy_window(ctx, d, C, s + (size_t)c->rank * Rp * C * elem, C, C, Rp, elem);
        return copy_window(ctx, d, Cp, s + (size_t)c->rank * Cp * elem, C, Cp, R, elem);
    }
    if (pre_axis == -2) {  // partial sums -> reduce (+ scatter): MPI_Reduce + master scatter in the reference (:798-862)
        if (post_axis == 0) {
            SWC_NCCL(ctx, g_nccl.ReduceScatter(src, dst, Rp * C, type, ncclSum, c->comm, ctx->stream));
            return SWCB200_OK;
        }
        void *stage = nullptr;
        if (post_axis == -1) {
            SWC_NCCL(ctx, g_nccl.AllReduce(src, dst, R * C, type, ncclSum, c->comm, ctx->stream));
            return SWCB200_OK;
        }
        rc = swc_scratch(ctx, R * C * elem, &stage);
        if (rc) return rc;
        SWC_NCCL(ctx, g_nccl.AllReduce(src, stage, R * C, type, ncclSum, c->comm, ctx->stream));
        return copy_window(ctx, d, Cp, (uint8_t *)stage + (size_t)c->rank * Cp * elem, C, Cp, R, elem);
    }
    if (post_axis == -1) {  // split -> replicated: all-gather
        if (pre_axis == 0) {
            SWC_NCCL(ctx, g_nccl.AllGather(src, dst, Rp * C, type, c->comm, ctx->stream));
            return SWCB200_OK;
        }
        void *stage = nullptr;
        rc = swc_scratch(ctx, R * C * elem, &stage);
        if (rc) return rc;
        SWC_NCCL(ctx, g_nccl.AllGather(src, stage, R * Cp, type, c->comm, ctx->stream));
        for (size_t q = 0; q < p; q++) {
            rc = copy_window(ctx, d + q * Cp * elem, C, (uint8_t *)stage + q * R * Cp * elem, Cp, Cp, R, elem);
            if (rc) return rc;
        }
        return SWCB200_OK;
    }
    // split i -> split j: all-to-all of [R/p, C/p] blocks (ring of MPI_Sendrecv in the reference, :714-797)
    const size_t blk = Rp * Cp;
    void *stage = nullptr;
    rc = swc_scratch(ctx, blk * p * elem, &stage);
    if (rc) return rc;
    uint8_t *st = (uint8_t *)stage;
    if (pre_axis == 0) {
        // local [R/p, C]: block for rank q is columns [q*Cp, (q+1)*Cp) -> pack; received block from q is rows
        // [q*Rp, (q+1)*Rp) of the result [R, C/p], which is contiguous
        for (size_t q = 0; q < p; q++) {
            rc = copy_window(ctx, st + q * blk * elem, Cp, s + q * Cp * elem, C, Cp, Rp, elem);
            if (rc) return rc;
        }
        NcclGroup group;
        SWC_NCCL(ctx, group.start());
        for (size_t q = 0; q < p; q++) {
            SWC_NCCL(ctx, g_nccl.Send(st + q * blk * elem, blk, type, (int)q, c->comm, ctx->stream));
            SWC_NCCL(ctx, g_nccl.Recv(d + q * blk * elem, blk, type, (int)q, c->comm, ctx->stream));
        }
        SWC_NCCL(ctx, group.end());
        return SWCB200_OK;
    }
    // pre 1 -> post 0: local [R, C/p]: block for rank q is rows [q*Rp, (q+1)*Rp), contiguous; the block received
    // from q becomes columns [q*Cp, (q+1)*Cp) of the result [R/p, C] -> unpack
    NcclGroup group;
    SWC_NCCL(ctx, group.start());
    for (size_t q = 0; q < p; q++) {
        SWC_NCCL(ctx, g_nccl.Send(s + q * blk * elem, blk, type, (int)q, c->comm, ctx->stream));
        SWC_NCCL(ctx, g_nccl.Recv(st + q * blk * elem, blk, type, (int)q, c->comm, ctx->stream));
    }
    SWC_NCCL(ctx, group.end());
    for (size_t q = 0; q < p; q++) {
        rc = copy_window(ctx, d + q * Cp * elem, C, st + q * blk * elem, Cp, Cp, Rp, elem);
        if (rc) return rc;
    }
    return SWCB200_OK;
}
