// Row-wise kernels: softmax and top-k argmax over [m, n] fp32.
#include <float.h>

#include "common.cuh"

namespace {

constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(kFull, v, o));
    return v;
}

template <bool kStrict>
__device__ __forceinline__ float exp_of(float x) {
    // kStrict: exponential in double, rounded once (see TanhOp in eltwise.cu).  Otherwise the hardware
    // exp2 approximation: relative error about 2^-22 plus |x| * 2^-24 from the scaling, far inside 1e-5
    // for every x whose exponential is not already negligible against the row maximum's 1.0.
    return kStrict ? (float)exp((double)x) : __expf(x);
}

// 128-bit variant of softmax_warp_kernel: lane l owns float4 groups l, l+32, ...; needs n % 4 == 0 and
// 16-byte aligned rows.  In the fast mode each element is multiplied by the reciprocal of the row sum
// (one division per row) instead of being divided by it.
template <int kVecPerLane, bool kStrict>
__global__ void __launch_bounds__(256) softmax_warp_vec_kernel(const float *__restrict__ a, int lda,
                                                               float *__restrict__ b, int ldb, int m, int n) {
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const int n4 = n >> 2;
    for (long long row = (long long)blockIdx.x * warps_per_cta + (threadIdx.x >> 5); row < m;
         row += (long long)gridDim.x * warps_per_cta) {
        const float4 *ar = reinterpret_cast<const float4 *>(a + (size_t)row * lda);
        float4 *br = reinterpret_cast<float4 *>(b + (size_t)row * ldb);
        float4 v[kVecPerLane];
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < kVecPerLane; i++) {
            int j = lane + 32 * i;
            v[i] = (j < n4) ? __ldcs(ar + j) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            mx = fmaxf(fmaxf(mx, fmaxf(v[i].x, v[i].y)), fmaxf(v[i].z, v[i].w));
        }
        mx = warp_max(mx);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < kVecPerLane; i++) {
            int j = lane + 32 * i;
            if (j < n4) {
                v[i].x = exp_of<kStrict>(__fsub_rn(v[i].x, mx));
                v[i].y = exp_of<kStrict>(__fsub_rn(v[i].y, mx));
                v[i].z = exp_of<kStrict>(__fsub_rn(v[i].z, mx));
                v[i].w = exp_of<kStrict>(__fsub_rn(v[i].w, mx));
                s = __fadd_rn(s, __fadd_rn(__fadd_rn(v[i].x, v[i].y), __fadd_rn(v[i].z, v[i].w)));
            }
        }
        s = warp_sum(s);
        const float inv = __fdiv_rn(1.0f, s);
#pragma unroll
        for (int i = 0; i < kVecPerLane; i++) {
            int j = lane + 32 * i;
            if (j < n4) {
                float4 o;
                if (kStrict) {
                    o = make_float4(__fdiv_rn(v[i].x, s), __fdiv_rn(v[i].y, s), __fdiv_rn(v[i].z, s), __fdiv_rn(v[i].w, s));
                } else {
                    o = make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv);
                }
                __stcs(br + j, o);
            }
        }
    }
}

// One warp per row, the row held in registers: lane l owns columns l, l+32, ...  Each load
// instruction of a warp reads 128 contiguous bytes.  kPerLane*32 >= n.  The row is read once and
// written once: 8 bytes per element of traffic.
template <int kPerLane, bool kStrict>
__global__ void __launch_bounds__(256) softmax_warp_kernel(const float *__restrict__ a, int lda,
                                                           float *__restrict__ b, int ldb, int m, int n) {
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    for (long long row = (long long)blockIdx.x * warps_per_cta + (threadIdx.x >> 5); row < m;
         row += (long long)gridDim.x * warps_per_cta) {
        const float *ar = a + (size_t)row * lda;
        float *br = b + (size_t)row * ldb;
        float v[kPerLane];
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < kPerLane; i++) {
            int j = lane + 32 * i;
            v[i] = (j < n) ? __ldcs(ar + j) : -INFINITY;
            mx = fmaxf(mx, v[i]);
        }
        mx = warp_max(mx);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < kPerLane; i++) {
            int j = lane + 32 * i;
            v[i] = (j < n) ? exp_of<kStrict>(__fsub_rn(v[i], mx)) : 0.f;
            s = __fadd_rn(s, v[i]);
        }
        s = warp_sum(s);
#pragma unroll
        for (int i = 0; i < kPerLane; i++) {
            int j = lane + 32 * i;
            if (j < n) __stcs(br + j, __fdiv_rn(v[i], s));
        }
    }
}

// One CTA per row for rows too long for registers; three passes over the row (the second and third
// hit L2 for any row that fits there).
template <bool kStrict>
__global__ void __launch_bounds__(256) softmax_cta_kernel(const float *__restrict__ a, int lda,
                                                          float *__restrict__ b, int ldb, int m, int n) {
    __shared__ float red[8];
    __shared__ float bcast;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int row = blockIdx.x; row < m; row += gridDim.x) {
        const float *ar = a + (size_t)row * lda;
        float *br = b + (size_t)row * ldb;
        float mx = -INFINITY;
        for (int j = threadIdx.x; j < n; j += blockDim.x) mx = fmaxf(mx, ar[j]);
        mx = warp_max(mx);
        if (lane == 0) red[warp] = mx;
        __syncthreads();
        if (warp == 0) {
            float t = (lane < 8) ? red[lane] : -INFINITY;
            t = warp_max(t);
            if (lane == 0) bcast = t;
        }
        __syncthreads();
        mx = bcast;
        float s = 0.f;
        for (int j = threadIdx.x; j < n; j += blockDim.x) {
            float e = exp_of<kStrict>(__fsub_rn(ar[j], mx));
            br[j] = e;
            s = __fadd_rn(s, e);
        }
        s = warp_sum(s);
        __syncthreads();
        if (lane == 0) red[warp] = s;
        __syncthreads();
        if (warp == 0) {
            float t = (lane < 8) ? red[lane] : 0.f;
            t = warp_sum(t);
            if (lane == 0) bcast = t;
        }
        __syncthreads();
        s = bcast;
        for (int j = threadIdx.x; j < n; j += blockDim.x) br[j] = __fdiv_rn(br[j], s);
        __syncthreads();
    }
}

// (value, index) ordering of std::greater<std::pair<float,int>>: a beats b if a.v > b.v, or the
// values compare equal and a.i > b.i.
__device__ __forceinline__ bool beats(float av, int ai, float bv, int bi) {
    return av > bv || (av == bv && ai > bi);
}

// One warp per row, top_k rounds; round t picks the best pair that still sorts after round t-1's.
__global__ void __launch_bounds__(256) argmax_kernel(const float *__restrict__ in, int *__restrict__ idx, int m, int n,
                                                     int top_k) {
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    for (long long row = (long long)blockIdx.x * warps_per_cta + (threadIdx.x >> 5); row < m;
         row += (long long)gridDim.x * warps_per_cta) {
        const float *r = in + (size_t)row * n;
        float pv = 0.f;
        int pi = -1;
        for (int t = 0; t < top_k; t++) {
            float bv = 0.f;
            int bi = -1;
            // eight independent loads in flight per lane, then the comparisons in index order
            for (int j0 = lane; j0 < n; j0 += 32 * 8) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    int j = j0 + 32 * u;
                    v[u] = (j < n) ? __ldg(r + j) : 0.f;
                }
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    int j = j0 + 32 * u;
                    if (j >= n) continue;
                    if (pi >= 0 && !beats(pv, pi, v[u], j)) continue;  // emitted already, or not below the last winner
                    if (bi < 0 || beats(v[u], j, bv, bi)) {
                        bv = v[u];
                        bi = j;
                    }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                float ov = __shfl_xor_sync(kFull, bv, o);
                int oi = __shfl_xor_sync(kFull, bi, o);
                if (oi >= 0 && (bi < 0 || beats(ov, oi, bv, bi))) {
                    bv = ov;
                    bi = oi;
                }
            }
            if (lane == 0) idx[(size_t)row * top_k + t] = bi;
            pv = bv;
            pi = bi;
        }
    }
}

// top_k = 1 on rows of 16-byte aligned float4: the whole row of a warp's lanes is requested before the first
// comparison (P float4 per lane, n <= 128 * P), scanned in index order so that `>=` leaves the HIGHEST index among
// equal maxima, the same winner as the pair ordering above.
template <int P>
__global__ void __launch_bounds__(256) argmax_top1_vec_kernel(const float *__restrict__ in, int *__restrict__ idx, int m, int n) {
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const int n4 = n >> 2;
    for (long long row = (long long)blockIdx.x * warps_per_cta + (threadIdx.x >> 5); row < m;
         row += (long long)gridDim.x * warps_per_cta) {
        const float4 *r = reinterpret_cast<const float4 *>(in + (size_t)row * n);
        float4 v[P];
#pragma unroll
        for (int u = 0; u < P; u++) {
            const int j4 = lane + 32 * u;
            v[u] = j4 < n4 ? __ldcs(r + j4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float bv = 0.f;
        int bi = -1;
#pragma unroll
        for (int u = 0; u < P; u++) {
            const int j4 = lane + 32 * u;
            if (j4 >= n4) continue;
            const float e[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
            for (int k = 0; k < 4; k++)
                if (bi < 0 || e[k] >= bv) {
                    bv = e[k];
                    bi = 4 * j4 + k;
                }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(kFull, bv, o);
            int oi = __shfl_xor_sync(kFull, bi, o);
            if (oi >= 0 && (bi < 0 || beats(ov, oi, bv, bi))) {
                bv = ov;
                bi = oi;
            }
        }
        if (lane == 0) idx[row] = bi;
    }
}

// accum[0] += rows whose label is among their n predictions, accum[1] += rows; integer counters, so the result does
// not depend on the order of the atomic additions
__global__ void __launch_bounds__(256) accuracy_kernel(const int *__restrict__ pred, const int *__restrict__ label,
                                                       int *__restrict__ accum, int m, int n) {
    int hits = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)m; i += (size_t)gridDim.x * blockDim.x) {
        const int want = label[i];
        const int *row = pred + i * (size_t)n;
        for (int j = 0; j < n; j++)
            if (row[j] == want) {
                hits++;
                break;
            }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) hits += __shfl_xor_sync(kFull, hits, o);
    if ((threadIdx.x & 31) == 0 && hits) atomicAdd(accum, hits);
    if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(accum + 1, m);
}

template <bool kStrict>
int launch_softmax(swcb200_ctx *ctx, int m, int n, const float *a, int lda, float *b, int ldb) {
    const int warps = 8;
    unsigned grid = swc_grid(ctx, (size_t)m, warps, 8);
    if (n % 4 == 0 && lda % 4 == 0 && ldb % 4 == 0 && swc_aligned16(a) && swc_aligned16(b) && n >= 128) {
#define SWC_SMV_CASE(P)                                                                                     \
    if (n <= 128 * (P)) {                                                                                   \
        softmax_warp_vec_kernel<P, kStrict><<<grid, 32 * warps, 0, ctx->stream>>>(a, lda, b, ldb, m, n);    \
        return swc_check_launch(ctx, "matrixSoftmax_f");                                                   \
    }
        SWC_SMV_CASE(1)
        SWC_SMV_CASE(2)
        SWC_SMV_CASE(4)
        SWC_SMV_CASE(8)
#undef SWC_SMV_CASE
    }
#define SWC_SM_CASE(P)                                                                                   \
    if (n <= 32 * (P)) {                                                                                 \
        softmax_warp_kernel<P, kStrict><<<grid, 32 * warps, 0, ctx->stream>>>(a, lda, b, ldb, m, n);    \
        return swc_check_launch(ctx, "matrixSoftmax_f");                                                \
    }
    SWC_SM_CASE(1)
    SWC_SM_CASE(2)
    SWC_SM_CASE(4)
    SWC_SM_CASE(8)
    SWC_SM_CASE(16)
    SWC_SM_CASE(32)
#undef SWC_SM_CASE
    unsigned g2 = swc_grid(ctx, (size_t)m, 1, 8);
    softmax_cta_kernel<kStrict><<<g2, 256, 0, ctx->stream>>>(a, lda, b, ldb, m, n);
    return swc_check_launch(ctx, "matrixSoftmax_f");
}

}  // namespace

SWC_EXPORT int swcb200_matrixSoftmax_f(swcb200_ctx *ctx, int m, int n, const float *a, int lda, float *b, int ldb) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, m >= 0 && n >= 0, SWCB200_ERR_BAD_ARG, "matrixSoftmax_f: negative shape");
    SWC_REQUIRE(ctx, lda >= n && ldb >= n, SWCB200_ERR_BAD_SHAPE, "matrixSoftmax_f: leading dimension below n");
    if (m == 0 || n == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, a && b, SWCB200_ERR_BAD_ARG, "matrixSoftmax_f: null tensor");
    return ctx->precision == SWCB200_STRICT_F32 ? launch_softmax<true>(ctx, m, n, a, lda, b, ldb)
                                                : launch_softmax<false>(ctx, m, n, a, lda, b, ldb);
}

SWC_EXPORT int swcb200_argMax_i(swcb200_ctx *ctx, const float *input, int *idx, int m, int n, int top_k) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, m >= 0 && n >= 0 && top_k >= 0, SWCB200_ERR_BAD_ARG, "argMax_i: negative shape");
    SWC_REQUIRE(ctx, top_k <= n, SWCB200_ERR_BAD_SHAPE, "argMax_i: top_k %d exceeds n %d", top_k, n);
    if (m == 0 || top_k == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, input && idx, SWCB200_ERR_BAD_ARG, "argMax_i: null tensor");
    unsigned grid = swc_grid(ctx, (size_t)m, 8, 8);
    if (top_k == 1 && n % 4 == 0 && n >= 128 && n <= 128 * 8 && swc_aligned16(input)) {
        if (n <= 128 * 2)
            argmax_top1_vec_kernel<2><<<grid, 256, 0, ctx->stream>>>(input, idx, m, n);
        else if (n <= 128 * 4)
            argmax_top1_vec_kernel<4><<<grid, 256, 0, ctx->stream>>>(input, idx, m, n);
        else
            argmax_top1_vec_kernel<8><<<grid, 256, 0, ctx->stream>>>(input, idx, m, n);
        return swc_check_launch(ctx, "argMax_i");
    }
    argmax_kernel<<<grid, 256, 0, ctx->stream>>>(input, idx, m, n, top_k);
    return swc_check_launch(ctx, "argMax_i");
}

SWC_EXPORT int swcb200_accuracy_i(swcb200_ctx *ctx, const int *pred, const int *label, int *accum_cnt, int m, int n) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, m >= 0 && n >= 0, SWCB200_ERR_BAD_ARG, "accuracy_i: negative shape");
    if (m == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, label && accum_cnt && (n == 0 || pred), SWCB200_ERR_BAD_ARG, "accuracy_i: null tensor");
    unsigned grid = swc_grid(ctx, (size_t)m, 256, 4);
    accuracy_kernel<<<grid, 256, 0, ctx->stream>>>(pred, label, accum_cnt, m, n);
    return swc_check_launch(ctx, "accuracy_i");
}
