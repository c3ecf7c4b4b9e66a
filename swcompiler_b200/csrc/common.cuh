// Shared pieces of the kernel library: the context, status plumbing, launch geometry.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "swc_b200.h"

#define SWC_EXPORT extern "C" __attribute__((visibility("default")))

struct swcb200_comm;  // comm.cu

struct swcb200_ctx {
    int device = 0;
    int precision = SWCB200_STRICT_F32;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    int sm_count = 148;
    int tc_sm_limit = 0;  // persistent tensor-core kernels take at most this many SMs (0 = all of them)
    uint64_t launches = 0;
    char last_error[512] = {0};
    // private scratch for the fp32 entry points in tensor-core mode (bf16 copies of operands);
    // grown on demand, released in destroy
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    swcb200_comm *comm = nullptr;
    // the status block in device memory, {int code; int pad; long long wait_limit_cycles}: kernels with
    // bounded waits read the limit from it and write a code into it when a wait runs out; the code is
    // read (and cleared) by swcb200_sync
    int *dev_status = nullptr;
};

int swc_fail(swcb200_ctx *ctx, int status, const char *fmt, ...);
int swc_check_launch(swcb200_ctx *ctx, const char *what);
int swc_scratch(swcb200_ctx *ctx, size_t bytes, void **out);
// fp32 [m, k] with pitch lda -> bf16 [m, k] with pitch ldo (pad columns are left untouched)
int swc_cast_pad_rows(swcb200_ctx *ctx, const float *a, int m, int k, int lda, void *out_bf16, int ldo);
// fp32 W[k, n] with pitch ldb -> bf16 Wp[n, k] with pitch ldo
int swc_pack_weight_padded(swcb200_ctx *ctx, const float *w, int k, int n, int ldb, void *wp_bf16, int ldo);

#define SWC_REQUIRE(ctx, cond, status, ...)                         \
    do {                                                            \
        if (!(cond)) return swc_fail((ctx), (status), __VA_ARGS__); \
    } while (0)

#define SWC_CTX(ctx)                                       \
    do {                                                   \
        if ((ctx) == nullptr) return SWCB200_ERR_BAD_ARG;  \
        cudaError_t e__ = cudaSetDevice((ctx)->device);    \
        if (e__ != cudaSuccess)                            \
            return swc_fail((ctx), SWCB200_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e__)); \
    } while (0)

#define SWC_CUDA(ctx, call)                                                                    \
    do {                                                                                       \
        cudaError_t e__ = (call);                                                              \
        if (e__ != cudaSuccess)                                                                \
            return swc_fail((ctx), SWCB200_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e__)); \
    } while (0)

// SMs a persistent tensor-core kernel of this context may occupy
static inline int swc_tc_sms(const swcb200_ctx *ctx) {
    return (ctx->tc_sm_limit > 0 && ctx->tc_sm_limit < ctx->sm_count) ? ctx->tc_sm_limit : ctx->sm_count;
}

static inline bool swc_aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Grid for a grid-stride kernel: enough CTAs to cover `work_items` at `per_cta`, capped at a
// whole number of waves over the SMs.
static inline unsigned swc_grid(const swcb200_ctx *ctx, size_t work_items, size_t per_cta, int ctas_per_sm) {
    size_t need = (work_items + per_cta - 1) / per_cta;
    size_t cap = (size_t)ctx->sm_count * (size_t)ctas_per_sm;
    if (need < 1) need = 1;
    return (unsigned)(need < cap ? need : cap);
}
