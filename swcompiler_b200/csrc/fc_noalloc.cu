// swcb200_matrixMatrixMul_f_noalloc -- the tensor-core matrix multiply for callers that must not
// allocate device memory.
//
// Who cannot allocate: a program the code generator emits sizes ONE arena per device up front and
// hands every tensor an offset into it; once that arena has taken most of the GPU, a cudaMalloc made
// behind the program's back by a library call in the middle of the forward pass can fail, and even when
// it succeeds it stalls the whole device while the driver maps memory.  The same holds for a serving
// process that has promised its memory budget to someone else, and for code running between the
// collectives of a multi-GPU job, where an allocation's implicit device-wide synchronisation can stall
// peers.  swcb200_matrixMatrixMul_f in tensor-core mode does allocate: it keeps bf16 copies of its two
// fp32 operands in a scratch block that the context grows with cudaMalloc on demand.  This entry point
// does the same arithmetic with that scratch placed in a fixed array that is part of the library image.
//
// What it costs: every GPU on which this library is used holds kScratchBytes (40 MiB) from the moment
// the library's device code is loaded until the process exits, whether or not this function is ever
// called.  Operands whose bf16 copies do not fit are refused with SWCB200_ERR_TOO_LARGE:
//     2 * roundup(k, 8) * (m + n)  [+ up to 255 bytes of padding]  <=  40 MiB
// e.g. a 4096 x 4096 weight together with up to 1024 rows of activations.
//
// Rules for callers
//   * The first call on each device looks up the device address of the array (and of the status word)
//     and caches it.
//   * The function needs no context.  It issues its kernels on the stream it is given, then waits for
//     that stream before it returns, so on return C is complete and a device-side timeout has been
//     turned into a status.  Because EVERY call ends with that wait (and a small blocking read-back of
//     the status word), no call -- not only the first -- may be made while the stream is being
//     captured, and the call blocks the host thread.
//   * The calling thread's current device is the same after the call as before it.
//   * Nothing is printed.  What went wrong with the calling thread's last failed call can be read with
//     swcb200_matrixMatrixMul_f_noalloc_last_error().
//   * All calls on one device share the one array, and it keeps whatever the previous call left there.
//     Nothing in it has to start at zero: each call overwrites exactly the part it later reads (the
//     padding columns k..roundup(k,8) are outside the tensor maps and are never read), and the status
//     word is cleared at the start of every call.  Two calls that overlap on the same GPU -- from two
//     host threads, or on two streams -- race on the array; run them one after the other.
//   * It calls no cudaMalloc, cudaFree, or any library routine that allocates device memory.
#include <mutex>

#include "common.cuh"

int swc_fc_tc(swcb200_ctx *ctx, int m, int n, int k, const void *a, const void *a_lo, int lda, const void *wp, int ldw,
              const float *bias, int act, void *c, void *c_lo, int c_dtype, int ldc);

namespace {

constexpr size_t kScratchBytes = (size_t)40 << 20;
constexpr int kMaxDevices = 64;

// The scratch itself.  In host code these names are only handles for the runtime; the addresses the
// kernels use are obtained with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];
// the status block of the bounded waits: {code, pad} and the wait limit in SM cycles (see tc_common.cuh)
static __device__ __align__(16) long long g_noalloc_status[2] = {0, 4000000000ll};

struct DeviceSlot {
    bool ready = false;
    void *scratch = nullptr;
    int *status = nullptr;
    int sm_count = 0;
};
DeviceSlot g_slots[kMaxDevices];
std::mutex g_slots_mutex;
thread_local char t_last_error[512] = {0};

// puts the caller's current device back on every way out
struct DeviceGuard {
    int prev = -1;
    DeviceGuard() {
        if (cudaGetDevice(&prev) != cudaSuccess) {
            prev = -1;
            cudaGetLastError();
        }
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// once per device, with that device current
int setup_device(int device, DeviceSlot **out, char *err, size_t errlen) {
    std::lock_guard<std::mutex> lock(g_slots_mutex);
    DeviceSlot &s = g_slots[device];
    if (!s.ready) {
        int major = 0, sms = 0;
        cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess) {
            snprintf(err, errlen, "device query: %s", cudaGetErrorString(e));
            return SWCB200_ERR_CUDA;
        }
        if (major != 10) return SWCB200_ERR_NO_DEVICE;
        void *scratch = nullptr, *status = nullptr;
        e = cudaGetSymbolAddress(&scratch, g_noalloc_scratch);
        if (e != cudaSuccess) {
            snprintf(err, errlen, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
            return SWCB200_ERR_CUDA;
        }
        e = cudaGetSymbolAddress(&status, g_noalloc_status);
        if (e != cudaSuccess) {
            snprintf(err, errlen, "cudaGetSymbolAddress(status): %s", cudaGetErrorString(e));
            return SWCB200_ERR_CUDA;
        }
        s.scratch = scratch;
        s.status = (int *)status;
        s.sm_count = sms;
        s.ready = true;
    }
    *out = &s;
    return SWCB200_OK;
}

}  // namespace

SWC_EXPORT int swcb200_matrixMatrixMul_f_noalloc(int device, void *cuda_stream, int m, int n, int k, const float *a,
                                                 int lda, const float *b, int ldb, float *c, int ldc) {
    if (device < 0 || device >= kMaxDevices) return SWCB200_ERR_BAD_ARG;
    if (m < 0 || n < 0 || k <= 0) return SWCB200_ERR_BAD_ARG;
    if (lda < k || ldb < n || ldc < n) return SWCB200_ERR_BAD_SHAPE;
    if (m == 0 || n == 0) return SWCB200_OK;
    if (!a || !b || !c) return SWCB200_ERR_BAD_ARG;
    const size_t kp = ((size_t)k + 7) & ~(size_t)7;
    const size_t a_bytes = ((size_t)m * kp * 2 + 255) & ~(size_t)255, b_bytes = (size_t)n * kp * 2;
    t_last_error[0] = 0;
    if (a_bytes + b_bytes > kScratchBytes) {
        snprintf(t_last_error, sizeof(t_last_error),
                 "%d x %d x %d needs %zu bytes of bf16 operand copies; the fixed scratch holds %zu (limit: "
                 "2*roundup(k,8)*(m+n) <= 40 MiB)", m, n, k, a_bytes + b_bytes, kScratchBytes);
        return SWCB200_ERR_TOO_LARGE;
    }
    DeviceGuard guard;
    if (cudaSetDevice(device) != cudaSuccess) {
        snprintf(t_last_error, sizeof(t_last_error), "cudaSetDevice(%d) failed", device);
        cudaGetLastError();
        return SWCB200_ERR_CUDA;
    }
    DeviceSlot *slot = nullptr;
    int rc = setup_device(device, &slot, t_last_error, sizeof(t_last_error));
    if (rc) return rc;
    // A context object on the host stack: plain data describing where to launch, owning nothing.
    swcb200_ctx ctx;
    ctx.device = device;
    ctx.precision = SWCB200_TC_BF16;
    ctx.stream = (cudaStream_t)cuda_stream;
    ctx.own_stream = false;
    ctx.sm_count = slot->sm_count;
    ctx.dev_status = slot->status;
    cudaError_t e = cudaMemsetAsync(slot->status, 0, sizeof(int), ctx.stream);
    if (e != cudaSuccess) {
        snprintf(t_last_error, sizeof(t_last_error), "clearing the status word: %s", cudaGetErrorString(e));
        return SWCB200_ERR_CUDA;
    }
    void *a16 = slot->scratch, *b16 = (unsigned char *)slot->scratch + a_bytes;
    rc = swc_cast_pad_rows(&ctx, a, m, k, lda, a16, (int)kp);
    if (!rc) rc = swc_pack_weight_padded(&ctx, b, k, n, ldb, b16, (int)kp);
    if (!rc) rc = swc_fc_tc(&ctx, m, n, k, a16, nullptr, (int)kp, b16, (int)kp, nullptr, SWCB200_ACT_NONE, c, nullptr, SWCB200_F32, ldc);
    if (rc) {
        snprintf(t_last_error, sizeof(t_last_error), "%s", ctx.last_error);
        return rc;
    }
    e = cudaStreamSynchronize(ctx.stream);
    int code = 0;
    if (e == cudaSuccess) e = cudaMemcpy(&code, slot->status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
        snprintf(t_last_error, sizeof(t_last_error), "%s", cudaGetErrorString(e));
        return SWCB200_ERR_CUDA;
    }
    if (code != 0) snprintf(t_last_error, sizeof(t_last_error), "a device-side wait ran out (code %d)", code);
    return code == 0 ? SWCB200_OK : SWCB200_ERR_TIMEOUT;
}

SWC_EXPORT const char *swcb200_matrixMatrixMul_f_noalloc_last_error(void) { return t_last_error; }
