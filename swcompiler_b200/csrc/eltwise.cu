// Bandwidth-bound elementwise kernels: ReLU, add, bias-add, tanh, fp32<->bf16 casts, weight packing.
//
// All of them move each byte once.  The geometry is the same everywhere: 256-thread CTAs,
// a grid that is a whole number of waves over the SMs, 128-bit loads and stores, four independent
// loads in flight per thread before the first use, grid-stride for the rest.  Unaligned bases or
// ragged tails take a scalar path inside the same launch.
#include <cuda_bf16.h>

#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;
constexpr int kCtasPerSm = 8;

__device__ __forceinline__ float4 ld4(const float *p) { return __ldcs(reinterpret_cast<const float4 *>(p)); }
__device__ __forceinline__ void st4(float *p, float4 v) { __stcs(reinterpret_cast<float4 *>(p), v); }

struct ReluOp {
    // (x > 0) ? x : +0 -- NaN and -0 give +0, as relu_f does (kernels.h:578)
    __device__ __forceinline__ float operator()(float x) const { return (x > 0.f) ? x : 0.f; }
};

template <bool kStrict>
struct TanhOp {
    // 1 - 2/(exp(2x)+1) in float, the reference's formula (kernels.h:61), not tanhf.  kStrict takes
    // the exponential in double and rounds it once, which lands on the correctly rounded float
    // that glibc's expf also returns for all but a fraction of a percent of arguments.
    __device__ __forceinline__ float operator()(float x) const {
        float t = __fmul_rn(x, 2.0f);
        float e = kStrict ? (float)exp((double)t) : expf(t);
        return __fsub_rn(1.0f, __fdiv_rn(2.0f, __fadd_rn(e, 1.0f)));
    }
};

template <class Op>
__global__ void __launch_bounds__(kThreads) map1_kernel(const float *__restrict__ in, float *__restrict__ out,
                                                        size_t n, bool vec, Op op) {
    const size_t tid = (size_t)blockIdx.x * kThreads + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * kThreads;
    if (vec) {
        const size_t n4 = n >> 2;
        for (size_t base = tid; base < n4; base += nthreads * kUnroll) {
            float4 v[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; u++) {
                size_t i = base + (size_t)u * nthreads;
                if (i < n4) v[u] = ld4(in + 4 * i);
            }
#pragma unroll
            for (int u = 0; u < kUnroll; u++) {
                size_t i = base + (size_t)u * nthreads;
                if (i < n4) st4(out + 4 * i, make_float4(op(v[u].x), op(v[u].y), op(v[u].z), op(v[u].w)));
            }
        }
        const size_t tail = (n4 << 2) + tid;
        if (tail < n) out[tail] = op(in[tail]);
    } else {
        for (size_t i = tid; i < n; i += nthreads) out[i] = op(in[i]);
    }
}

// rows x cols with leading dimensions (tanh keeps the reference's lda/ldb arguments)
template <class Op>
__global__ void __launch_bounds__(kThreads) map1_strided_kernel(const float *__restrict__ in, int lda,
                                                                float *__restrict__ out, int ldb, int m, int n,
                                                                Op op) {
    const size_t total = (size_t)m * n;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += (size_t)gridDim.x * kThreads) {
        size_t r = i / n, c = i - r * n;
        out[r * ldb + c] = op(in[r * lda + c]);
    }
}

__global__ void __launch_bounds__(kThreads) add_kernel(const float *__restrict__ a, const float *__restrict__ b,
                                                       float *__restrict__ c, size_t n, bool vec) {
    const size_t tid = (size_t)blockIdx.x * kThreads + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * kThreads;
    if (vec) {
        const size_t n4 = n >> 2;
        constexpr int U = 2;  // two streams in: 2 x 2 loads in flight
        for (size_t base = tid; base < n4; base += nthreads * U) {
            float4 x[U], y[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                size_t i = base + (size_t)u * nthreads;
                if (i < n4) {
                    x[u] = ld4(a + 4 * i);
                    y[u] = ld4(b + 4 * i);
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                size_t i = base + (size_t)u * nthreads;
                if (i < n4)
                    st4(c + 4 * i, make_float4(__fadd_rn(x[u].x, y[u].x), __fadd_rn(x[u].y, y[u].y),
                                               __fadd_rn(x[u].z, y[u].z), __fadd_rn(x[u].w, y[u].w)));
            }
        }
        const size_t tail = (n4 << 2) + tid;
        if (tail < n) c[tail] = __fadd_rn(a[tail], b[tail]);
    } else {
        for (size_t i = tid; i < n; i += nthreads) c[i] = __fadd_rn(a[i], b[i]);
    }
}

// dest[r, :] = batch[r, :] + slice[:]; vec path needs cols % 4 == 0 so a float4 never straddles rows
__global__ void __launch_bounds__(kThreads) bias_add_kernel(float *__restrict__ dest, const float *__restrict__ batch,
                                                            const float *__restrict__ slice, size_t rows, size_t cols,
                                                            bool vec) {
    const size_t tid = (size_t)blockIdx.x * kThreads + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * kThreads;
    const size_t n = rows * cols;
    if (vec) {
        const size_t n4 = n >> 2, c4 = cols >> 2;
        for (size_t base = tid; base < n4; base += nthreads * kUnroll) {
            float4 v[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; u++) {
                size_t i = base + (size_t)u * nthreads;
                if (i < n4) v[u] = ld4(batch + 4 * i);
            }
#pragma unroll
            for (int u = 0; u < kUnroll; u++) {
                size_t i = base + (size_t)u * nthreads;
                if (i < n4) {
                    float4 s = __ldg(reinterpret_cast<const float4 *>(slice) + (i % c4));
                    st4(dest + 4 * i, make_float4(__fadd_rn(v[u].x, s.x), __fadd_rn(v[u].y, s.y),
                                                  __fadd_rn(v[u].z, s.z), __fadd_rn(v[u].w, s.w)));
                }
            }
        }
    } else {
        for (size_t i = tid; i < n; i += nthreads) dest[i] = __fadd_rn(batch[i], slice[i % cols]);
    }
}

__global__ void __launch_bounds__(kThreads) f32_to_bf16_kernel(const float *__restrict__ in,
                                                               __nv_bfloat16 *__restrict__ out, size_t n, bool vec) {
    const size_t tid = (size_t)blockIdx.x * kThreads + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * kThreads;
    if (vec) {
        const size_t n8 = n >> 3;
        for (size_t i = tid; i < n8; i += nthreads) {
            float4 a = ld4(in + 8 * i), b = ld4(in + 8 * i + 4);
            __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
            uint4 o;
            o.x = *reinterpret_cast<uint32_t *>(&p0);
            o.y = *reinterpret_cast<uint32_t *>(&p1);
            o.z = *reinterpret_cast<uint32_t *>(&p2);
            o.w = *reinterpret_cast<uint32_t *>(&p3);
            __stcs(reinterpret_cast<uint4 *>(out + 8 * i), o);
        }
        const size_t tail = (n8 << 3) + tid;
        if (tail < n) out[tail] = __float2bfloat16_rn(in[tail]);
    } else {
        for (size_t i = tid; i < n; i += nthreads) out[i] = __float2bfloat16_rn(in[i]);
    }
}

__global__ void __launch_bounds__(kThreads) bf16_to_f32_kernel(const __nv_bfloat16 *__restrict__ in,
                                                               float *__restrict__ out, size_t n, bool vec) {
    const size_t tid = (size_t)blockIdx.x * kThreads + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * kThreads;
    if (vec) {
        const size_t n8 = n >> 3;
        for (size_t i = tid; i < n8; i += nthreads) {
            uint4 v = __ldcs(reinterpret_cast<const uint4 *>(in + 8 * i));
            const __nv_bfloat162 *p = reinterpret_cast<const __nv_bfloat162 *>(&v);
            float2 f0 = __bfloat1622float2(p[0]), f1 = __bfloat1622float2(p[1]);
            float2 f2 = __bfloat1622float2(p[2]), f3 = __bfloat1622float2(p[3]);
            st4(out + 8 * i, make_float4(f0.x, f0.y, f1.x, f1.y));
            st4(out + 8 * i + 4, make_float4(f2.x, f2.y, f3.x, f3.y));
        }
        const size_t tail = (n8 << 3) + tid;
        if (tail < n) out[tail] = __bfloat162float(in[tail]);
    } else {
        for (size_t i = tid; i < n; i += nthreads) out[i] = __bfloat162float(in[i]);
    }
}

// W[k, n] fp32 (ldb) -> Wp[n, k] bf16: 32x32 tiles through shared memory, both sides coalesced
__global__ void __launch_bounds__(256) pack_weight_kernel(const float *__restrict__ w, int k, int n, int ldb,
                                                          __nv_bfloat16 *__restrict__ wp, int ldo) {
    __shared__ float tile[32][33];
    const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
#pragma unroll
    for (int r = ty; r < 32; r += 8) {
        int kk = k0 + r, nn = n0 + tx;
        tile[r][tx] = (kk < k && nn < n) ? w[(size_t)kk * ldb + nn] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int r = ty; r < 32; r += 8) {
        int nn = n0 + r, kk = k0 + tx;
        if (nn < n && kk < k) wp[(size_t)nn * ldo + kk] = __float2bfloat16_rn(tile[tx][r]);
    }
}

__global__ void __launch_bounds__(kThreads) cast_rows_kernel(const float *__restrict__ a, int m, int k, int lda,
                                                             __nv_bfloat16 *__restrict__ out, int ldo) {
    const size_t total = (size_t)m * k;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += (size_t)gridDim.x * kThreads) {
        size_t r = i / k, c = i - r * k;
        out[r * ldo + c] = __float2bfloat16_rn(a[r * lda + c]);
    }
}

template <class Op>
int launch_map1(swcb200_ctx *ctx, const float *in, float *out, size_t n, Op op, const char *what) {
    if (n == 0) return SWCB200_OK;
    bool vec = swc_aligned16(in) && swc_aligned16(out);
    unsigned grid = swc_grid(ctx, n, (size_t)kThreads * 4 * kUnroll, kCtasPerSm);
    map1_kernel<<<grid, kThreads, 0, ctx->stream>>>(in, out, n, vec, op);
    return swc_check_launch(ctx, what);
}

// out[i] = ((s_0[i] + s_1[i]) + s_2[i]) + ... over `nslots` arrays of `n` floats lying `stride` floats apart: the join
// of the partial sums of a model-parallel layer, always in rank order so that the result does not depend on timing.
__global__ void __launch_bounds__(kThreads) sum_slots_kernel(const float *__restrict__ slots, size_t stride, int nslots,
                                                             float *__restrict__ out, size_t n, bool vec) {
    const size_t tid = (size_t)blockIdx.x * kThreads + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * kThreads;
    if (vec) {
        const size_t n4 = n >> 2;
        for (size_t i = tid; i < n4; i += nthreads) {
            float4 acc = ld4(slots + 4 * i);
            for (int r = 1; r < nslots; r++) {
                const float4 v = ld4(slots + (size_t)r * stride + 4 * i);
                acc = make_float4(__fadd_rn(acc.x, v.x), __fadd_rn(acc.y, v.y), __fadd_rn(acc.z, v.z), __fadd_rn(acc.w, v.w));
            }
            st4(out + 4 * i, acc);
        }
        for (size_t i = (n4 << 2) + tid; i < n; i += nthreads) {
            float acc = slots[i];
            for (int r = 1; r < nslots; r++) acc = __fadd_rn(acc, slots[(size_t)r * stride + i]);
            out[i] = acc;
        }
    } else {
        for (size_t i = tid; i < n; i += nthreads) {
            float acc = slots[i];
            for (int r = 1; r < nslots; r++) acc = __fadd_rn(acc, slots[(size_t)r * stride + i]);
            out[i] = acc;
        }
    }
}

}  // namespace

SWC_EXPORT int swcb200_relu_f(swcb200_ctx *ctx, const float *src, float *dest, size_t size) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, size == 0 || (src && dest), SWCB200_ERR_BAD_ARG, "relu_f: null tensor");
    return launch_map1(ctx, src, dest, size, ReluOp(), "relu_f");
}

SWC_EXPORT int swcb200_sum_slots(swcb200_ctx *ctx, const float *slots, size_t slot_stride, int nslots, float *out, size_t count) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, nslots >= 1 && slot_stride >= count, SWCB200_ERR_BAD_ARG, "sum_slots: bad slot count or stride");
    if (count == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, slots && out, SWCB200_ERR_BAD_ARG, "sum_slots: null tensor");
    const bool vec = swc_aligned16(slots) && swc_aligned16(out) && slot_stride % 4 == 0;
    unsigned grid = swc_grid(ctx, count, (size_t)kThreads * 4, kCtasPerSm);
    sum_slots_kernel<<<grid, kThreads, 0, ctx->stream>>>(slots, slot_stride, nslots, out, count, vec);
    return swc_check_launch(ctx, "sum_slots");
}

SWC_EXPORT int swcb200_vecAdd_f(swcb200_ctx *ctx, int size, const float *a, const float *b, float *c) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, size >= 0, SWCB200_ERR_BAD_ARG, "vecAdd_f: negative size %d", size);
    SWC_REQUIRE(ctx, size == 0 || (a && b && c), SWCB200_ERR_BAD_ARG, "vecAdd_f: null tensor");
    if (size == 0) return SWCB200_OK;
    bool vec = swc_aligned16(a) && swc_aligned16(b) && swc_aligned16(c);
    unsigned grid = swc_grid(ctx, (size_t)size, (size_t)kThreads * 4 * 2, kCtasPerSm);
    add_kernel<<<grid, kThreads, 0, ctx->stream>>>(a, b, c, (size_t)size, vec);
    return swc_check_launch(ctx, "vecAdd_f");
}

SWC_EXPORT int swcb200_batchedadd_f(swcb200_ctx *ctx, float *dest, const float *batch, const float *slice,
                                    size_t numSlice, size_t sliceSize) {
    SWC_CTX(ctx);
    size_t n = numSlice * sliceSize;
    SWC_REQUIRE(ctx, n == 0 || (dest && batch && slice), SWCB200_ERR_BAD_ARG, "batchedadd_f: null tensor");
    if (n == 0) return SWCB200_OK;
    bool vec = (sliceSize % 4 == 0) && swc_aligned16(dest) && swc_aligned16(batch) && swc_aligned16(slice);
    unsigned grid = swc_grid(ctx, n, (size_t)kThreads * 4 * kUnroll, kCtasPerSm);
    bias_add_kernel<<<grid, kThreads, 0, ctx->stream>>>(dest, batch, slice, numSlice, sliceSize, vec);
    return swc_check_launch(ctx, "batchedadd_f");
}

SWC_EXPORT int swcb200_matrixTanh_f(swcb200_ctx *ctx, int m, int n, const float *a, int lda, float *b, int ldb) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, m >= 0 && n >= 0, SWCB200_ERR_BAD_ARG, "matrixTanh_f: negative shape");
    SWC_REQUIRE(ctx, lda >= n && ldb >= n, SWCB200_ERR_BAD_SHAPE, "matrixTanh_f: leading dimension below n");
    size_t total = (size_t)m * n;
    SWC_REQUIRE(ctx, total == 0 || (a && b), SWCB200_ERR_BAD_ARG, "matrixTanh_f: null tensor");
    if (total == 0) return SWCB200_OK;
    const bool strict = ctx->precision == SWCB200_STRICT_F32;
    if (lda == n && ldb == n) {
        return strict ? launch_map1(ctx, a, b, total, TanhOp<true>(), "matrixTanh_f")
                      : launch_map1(ctx, a, b, total, TanhOp<false>(), "matrixTanh_f");
    }
    unsigned grid = swc_grid(ctx, total, kThreads, kCtasPerSm);
    if (strict)
        map1_strided_kernel<<<grid, kThreads, 0, ctx->stream>>>(a, lda, b, ldb, m, n, TanhOp<true>());
    else
        map1_strided_kernel<<<grid, kThreads, 0, ctx->stream>>>(a, lda, b, ldb, m, n, TanhOp<false>());
    return swc_check_launch(ctx, "matrixTanh_f");
}

SWC_EXPORT int swcb200_cast_f32_to_bf16(swcb200_ctx *ctx, const float *src, void *dst, size_t count) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, count == 0 || (src && dst), SWCB200_ERR_BAD_ARG, "cast_f32_to_bf16: null tensor");
    if (count == 0) return SWCB200_OK;
    bool vec = swc_aligned16(src) && swc_aligned16(dst);
    unsigned grid = swc_grid(ctx, count, (size_t)kThreads * 8, kCtasPerSm);
    f32_to_bf16_kernel<<<grid, kThreads, 0, ctx->stream>>>(src, (__nv_bfloat16 *)dst, count, vec);
    return swc_check_launch(ctx, "cast_f32_to_bf16");
}

SWC_EXPORT int swcb200_cast_bf16_to_f32(swcb200_ctx *ctx, const void *src, float *dst, size_t count) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, count == 0 || (src && dst), SWCB200_ERR_BAD_ARG, "cast_bf16_to_f32: null tensor");
    if (count == 0) return SWCB200_OK;
    bool vec = swc_aligned16(src) && swc_aligned16(dst);
    unsigned grid = swc_grid(ctx, count, (size_t)kThreads * 8, kCtasPerSm);
    bf16_to_f32_kernel<<<grid, kThreads, 0, ctx->stream>>>((const __nv_bfloat16 *)src, dst, count, vec);
    return swc_check_launch(ctx, "cast_bf16_to_f32");
}

int swc_cast_pad_rows(swcb200_ctx *ctx, const float *a, int m, int k, int lda, void *out, int ldo) {
    if (lda == k && ldo == k) return swcb200_cast_f32_to_bf16(ctx, a, out, (size_t)m * k);
    unsigned grid = swc_grid(ctx, (size_t)m * k, kThreads, kCtasPerSm);
    cast_rows_kernel<<<grid, kThreads, 0, ctx->stream>>>(a, m, k, lda, (__nv_bfloat16 *)out, ldo);
    return swc_check_launch(ctx, "cast rows to bf16");
}

int swc_pack_weight_padded(swcb200_ctx *ctx, const float *w, int k, int n, int ldb, void *wp, int ldo) {
    dim3 grid((n + 31) / 32, (k + 31) / 32);
    SWC_REQUIRE(ctx, grid.y <= 65535, SWCB200_ERR_TOO_LARGE, "pack_weight_bf16: k beyond 2M rows");
    pack_weight_kernel<<<grid, 256, 0, ctx->stream>>>(w, k, n, ldb, (__nv_bfloat16 *)wp, ldo);
    return swc_check_launch(ctx, "pack_weight_bf16");
}

SWC_EXPORT int swcb200_pack_weight_bf16(swcb200_ctx *ctx, const float *w, int k, int n, int ldb, void *wp) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, k > 0 && n > 0 && w && wp, SWCB200_ERR_BAD_ARG, "pack_weight_bf16: bad argument");
    SWC_REQUIRE(ctx, ldb >= n, SWCB200_ERR_BAD_SHAPE, "pack_weight_bf16: ldb below n");
    return swc_pack_weight_padded(ctx, w, k, n, ldb, wp, k);
}

SWC_EXPORT int swcb200_pack_filter_bf16(swcb200_ctx *ctx, const float *filter, const size_t *fdims, void *fp) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, filter && fdims && fp, SWCB200_ERR_BAD_ARG, "pack_filter_bf16: null argument");
    return swcb200_cast_f32_to_bf16(ctx, filter, fp, fdims[0] * fdims[1] * fdims[2] * fdims[3]);
}
