// Context life-cycle and status strings.
#include <stdarg.h>

#include "tc_common.cuh"

int swc_fail(swcb200_ctx *ctx, int status, const char *fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->last_error, sizeof(ctx->last_error), fmt, ap);
        va_end(ap);
    }
    return status;
}

int swc_check_launch(swcb200_ctx *ctx, const char *what) {
    ctx->launches++;
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        cudaGetLastError();
        return swc_fail(ctx, SWCB200_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    }
    return SWCB200_OK;
}

int swc_scratch(swcb200_ctx *ctx, size_t bytes, void **out) {
    if (bytes > ctx->scratch_bytes) {
        if (ctx->scratch) {
            // earlier work on the stream may still read the old block
            SWC_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            SWC_CUDA(ctx, cudaFree(ctx->scratch));
            ctx->scratch = nullptr;
            ctx->scratch_bytes = 0;
        }
        size_t want = (bytes + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
        SWC_CUDA(ctx, cudaMalloc(&ctx->scratch, want));
        ctx->scratch_bytes = want;
    }
    *out = ctx->scratch;
    return SWCB200_OK;
}

static int init_common(int device, int precision, void *stream, bool own, swcb200_ctx **out) {
    if (!out) return SWCB200_ERR_BAD_ARG;
    *out = nullptr;
    if (precision != SWCB200_STRICT_F32 && precision != SWCB200_TC_BF16) return SWCB200_ERR_BAD_ARG;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        cudaGetLastError();
        return SWCB200_ERR_NO_DEVICE;
    }
    if (device < 0 || device >= count) return SWCB200_ERR_BAD_ARG;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return SWCB200_ERR_CUDA;
    // the library holds sm_100a code only
    if (prop.major != 10) return SWCB200_ERR_NO_DEVICE;
    if (cudaSetDevice(device) != cudaSuccess) return SWCB200_ERR_CUDA;
    swcb200_ctx *ctx = new swcb200_ctx();
    ctx->device = device;
    ctx->precision = precision;
    ctx->sm_count = prop.multiProcessorCount;
    if (own) {
        if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
            delete ctx;
            return SWCB200_ERR_CUDA;
        }
        ctx->own_stream = true;
    } else {
        ctx->stream = (cudaStream_t)stream;
    }
    const long long block[2] = {0, 4000000000ll};  // code 0; the default limit of the device-side waits, in SM cycles
    if (cudaMalloc(&ctx->dev_status, sizeof(block)) != cudaSuccess ||
        cudaMemcpy(ctx->dev_status, block, sizeof(block), cudaMemcpyHostToDevice) != cudaSuccess) {
        if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
        delete ctx;
        return SWCB200_ERR_CUDA;
    }
    *out = ctx;
    return SWCB200_OK;
}

SWC_EXPORT int swcb200_init(int device, int precision, swcb200_ctx **out) {
    return init_common(device, precision, nullptr, true, out);
}

SWC_EXPORT int swcb200_init_on_stream(int device, int precision, void *cuda_stream, swcb200_ctx **out) {
    return init_common(device, precision, cuda_stream, false, out);
}

SWC_EXPORT int swcb200_destroy(swcb200_ctx *ctx) {
    if (!ctx) return SWCB200_ERR_BAD_ARG;
    int rc = SWCB200_OK;
    if (ctx->comm) swcb200_comm_destroy(ctx);
    cudaSetDevice(ctx->device);
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) rc = SWCB200_ERR_CUDA;
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->dev_status) cudaFree(ctx->dev_status);
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return rc;
}

SWC_EXPORT int swcb200_sync(swcb200_ctx *ctx) {
    SWC_CTX(ctx);
    SWC_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    int code = 0;
    SWC_CUDA(ctx, cudaMemcpy(&code, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (code != 0) {
        cudaMemset(ctx->dev_status, 0, sizeof(int));
        static const char *where[] = {"", "operand tile to arrive (TMA)", "a pipeline stage to be released",
                                      "an accumulator to be published", "an accumulator to be drained",
                                      "outstanding copies at kernel exit"};
        return swc_fail(ctx, SWCB200_ERR_TIMEOUT, "a tensor-core kernel gave up waiting for %s (code %d)",
                        (code >= 1 && code <= 5) ? where[code] : "?", code);
    }
    return SWCB200_OK;
}

SWC_EXPORT int swcb200_set_wait_limit(swcb200_ctx *ctx, long long cycles) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, cycles > 0, SWCB200_ERR_BAD_ARG, "set_wait_limit: the limit must be positive");
    // ordered with the kernels of the stream: launches made before this call keep the old limit
    SWC_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    SWC_CUDA(ctx, cudaMemcpy((long long *)ctx->dev_status + 1, &cycles, sizeof(cycles), cudaMemcpyHostToDevice));
    return SWCB200_OK;
}

namespace {
// One thread waits, with the library's bounded wait, on a barrier nobody will ever arrive at: the wait runs out
// after the context's limit, records its code and the kernel returns normally.
__global__ void selftest_wait_kernel(int *status) {
    __shared__ uint64_t bar;
    tc::mbar_init(&bar, 1);
    tc::fence_barrier_init();
    tc::mbar_wait(&bar, 0, status, tc::kWaitFull);
}
}  // namespace

SWC_EXPORT int swcb200_selftest_wait_timeout(swcb200_ctx *ctx) {
    SWC_CTX(ctx);
    selftest_wait_kernel<<<1, 1, 0, ctx->stream>>>(ctx->dev_status);
    return swc_check_launch(ctx, "selftest_wait_timeout");
}

SWC_EXPORT int swcb200_set_sm_limit(swcb200_ctx *ctx, int sms) {
    if (!ctx) return SWCB200_ERR_BAD_ARG;
    SWC_REQUIRE(ctx, sms >= 0, SWCB200_ERR_BAD_ARG, "set_sm_limit: negative count");
    ctx->tc_sm_limit = sms;
    return SWCB200_OK;
}

SWC_EXPORT int swcb200_set_precision(swcb200_ctx *ctx, int precision) {
    if (!ctx) return SWCB200_ERR_BAD_ARG;
    SWC_REQUIRE(ctx, precision == SWCB200_STRICT_F32 || precision == SWCB200_TC_BF16, SWCB200_ERR_BAD_ARG,
                "unknown precision %d", precision);
    ctx->precision = precision;
    return SWCB200_OK;
}

SWC_EXPORT void *swcb200_stream(swcb200_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

SWC_EXPORT const char *swcb200_last_error(swcb200_ctx *ctx) { return ctx ? ctx->last_error : "null context"; }

SWC_EXPORT uint64_t swcb200_launch_count(swcb200_ctx *ctx) { return ctx ? ctx->launches : 0; }

SWC_EXPORT int swcb200_version(void) { return 100; }

SWC_EXPORT const char *swcb200_status_string(int s) {
    switch (s) {
        case SWCB200_OK: return "ok";
        case SWCB200_ERR_BAD_ARG: return "bad argument";
        case SWCB200_ERR_BAD_SHAPE: return "inconsistent shapes";
        case SWCB200_ERR_MISALIGNED: return "misaligned pointer or leading dimension";
        case SWCB200_ERR_UNSUPPORTED: return "unsupported attribute";
        case SWCB200_ERR_CUDA: return "CUDA error";
        case SWCB200_ERR_NCCL: return "NCCL error";
        case SWCB200_ERR_TIMEOUT: return "timed out";
        case SWCB200_ERR_NO_DEVICE: return "no sm_100 CUDA device";
        case SWCB200_ERR_TOO_LARGE: return "size beyond a documented limit";
        default: return "unknown status";
    }
}
