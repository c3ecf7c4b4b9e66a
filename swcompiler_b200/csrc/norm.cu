// Inference batch normalisation (NHWC) and the two transposes.
#include "common.cuh"

namespace {

// batchnormalization_f (kernels.h:509-512) evaluates
//     (x - mean[c]) * pow(var[c] + eps, -0.5) * scale[c] + bias[c]
// with the two float operations (x - mean, var + eps) in float and everything after the call to
// pow in double, rounding to float once at the end.  This kernel does the same: the per-channel
// factor 1/sqrt(double(var+eps)) is formed in double (two correctly rounded operations), the two
// products and the sum are IEEE double operations in the reference's order.  Per-channel vectors
// sit in shared memory; x is read once and y written once with 128-bit accesses.
template <int kVec>
__global__ void __launch_bounds__(256) batchnorm_kernel(float *__restrict__ out, const float *__restrict__ in,
                                                        const float *__restrict__ mean, const float *__restrict__ var,
                                                        const float *__restrict__ scale, const float *__restrict__ bias,
                                                        size_t pixels, int C, float eps) {
    extern __shared__ double smem_d[];
    double *rstd = smem_d;                                // [C]
    float *s_mean = reinterpret_cast<float *>(rstd + C);  // [C]
    float *s_scale = s_mean + C;
    float *s_bias = s_scale + C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float veps = __fadd_rn(var[c], eps);
        rstd[c] = __ddiv_rn(1.0, __dsqrt_rn((double)veps));
        s_mean[c] = mean[c];
        s_scale[c] = scale[c];
        s_bias[c] = bias[c];
    }
    __syncthreads();
    const int cg = C / kVec;
    const size_t total = pixels * cg;
    const size_t nthreads = (size_t)gridDim.x * blockDim.x;
    // When the thread stride is a multiple of the channel-group count (always for power-of-two channel
    // counts up to 1024), a thread meets the same channels at every step: their parameters move into
    // registers and the loop has no division.
    const bool fixed_c = (nthreads % cg) == 0;
    size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    int c = (int)(t % cg) * kVec;
    // scale and bias are widened to double once per thread, not once per element: float<->double
    // conversions run at a fraction of the FP64 rate and would otherwise set the pace of the kernel
    double r_[kVec], s_[kVec], b_[kVec];
    float m_[kVec];
#pragma unroll
    for (int i = 0; i < kVec; i++) {
        r_[i] = rstd[c + i];
        m_[i] = s_mean[c + i];
        s_[i] = (double)s_scale[c + i];
        b_[i] = (double)s_bias[c + i];
    }
    if (fixed_c && kVec == 4) {
        // main path: kU independent 128-bit loads in flight per thread
        constexpr int kU = 4;
        for (size_t base = t; base < total; base += nthreads * kU) {
            float4 v[kU];
#pragma unroll
            for (int u = 0; u < kU; u++) {
                size_t tt = base + (size_t)u * nthreads;
                if (tt < total) v[u] = __ldcs(reinterpret_cast<const float4 *>(in + tt * 4));
            }
#pragma unroll
            for (int u = 0; u < kU; u++) {
                size_t tt = base + (size_t)u * nthreads;
                if (tt >= total) continue;
                const float x[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
                float y[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    double d = (double)__fsub_rn(x[i], m_[i % kVec]);
                    d = __dmul_rn(d, r_[i % kVec]);
                    d = __dmul_rn(d, s_[i % kVec]);
                    d = __dadd_rn(d, b_[i % kVec]);
                    y[i] = (float)d;
                }
                __stcs(reinterpret_cast<float4 *>(out + tt * 4), make_float4(y[0], y[1], y[2], y[3]));
            }
        }
        return;
    }
    for (; t < total; t += nthreads) {
        if (!fixed_c) {
            c = (int)(t % cg) * kVec;
#pragma unroll
            for (int i = 0; i < kVec; i++) {
                r_[i] = rstd[c + i];
                m_[i] = s_mean[c + i];
                s_[i] = (double)s_scale[c + i];
                b_[i] = (double)s_bias[c + i];
            }
        }
        const size_t off = t * kVec;  // (t / cg) * C + c, since C = cg * kVec
        float x[kVec], y[kVec];
        if (kVec == 4) {
            float4 v = __ldcs(reinterpret_cast<const float4 *>(in + off));
            x[0] = v.x;
            x[1 % kVec] = v.y;
            x[2 % kVec] = v.z;
            x[3 % kVec] = v.w;
        } else {
            x[0] = in[off];
        }
#pragma unroll
        for (int i = 0; i < kVec; i++) {
            double d = (double)__fsub_rn(x[i], m_[i]);
            d = __dmul_rn(d, r_[i]);
            d = __dmul_rn(d, s_[i]);
            d = __dadd_rn(d, b_[i]);
            y[i] = (float)d;
        }
        if (kVec == 4)
            __stcs(reinterpret_cast<float4 *>(out + off), make_float4(y[0], y[1 % kVec], y[2 % kVec], y[3 % kVec]));
        else
            out[off] = y[0];
    }
}

// out[idx[shuffle]] = in[idx]: one thread per OUTPUT element (coalesced writes), gathering its input
__global__ void __launch_bounds__(256) transpose4d_kernel(const float *__restrict__ in, float *__restrict__ out,
                                                          size_t i0, size_t i1, size_t i2, size_t i3, size_t o1,
                                                          size_t o2, size_t o3, int s0, int s1, int s2, int s3) {
    const size_t total = i0 * i1 * i2 * i3;
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
        size_t o[4];
        size_t r = t;
        o[3] = r % o3;
        r /= o3;
        o[2] = r % o2;
        r /= o2;
        o[1] = r % o1;
        o[0] = r / o1;
        size_t id[4];
        id[s0] = o[0];
        id[s1] = o[1];
        id[s2] = o[2];
        id[s3] = o[3];
        out[t] = in[((id[0] * i1 + id[1]) * i2 + id[2]) * i3 + id[3]];
    }
}

}  // namespace

SWC_EXPORT int swcb200_batchnormalization_f(swcb200_ctx *ctx, float *output, const float *input, const float *mean,
                                            const float *var, const float *scale, const float *bias,
                                            const size_t *idims, float epsilon) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, idims, SWCB200_ERR_BAD_ARG, "batchnormalization_f: null idims");
    const size_t pixels = idims[0] * idims[1] * idims[2], C = idims[3];
    if (pixels * C == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, output && input && mean && var && scale && bias, SWCB200_ERR_BAD_ARG,
                "batchnormalization_f: null tensor");
    SWC_REQUIRE(ctx, C <= 8192, SWCB200_ERR_TOO_LARGE, "batchnormalization_f: %zu channels beyond 8192", C);
    size_t smem = C * (sizeof(double) + 3 * sizeof(float));
    bool vec = (C % 4 == 0) && swc_aligned16(input) && swc_aligned16(output);
    if (vec) {
        auto k = batchnorm_kernel<4>;
        if (smem > 48 * 1024) SWC_CUDA(ctx, cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        unsigned grid = swc_grid(ctx, pixels * C / 4, 256 * 4, 8);
        k<<<grid, 256, smem, ctx->stream>>>(output, input, mean, var, scale, bias, pixels, (int)C, epsilon);
    } else {
        auto k = batchnorm_kernel<1>;
        if (smem > 48 * 1024) SWC_CUDA(ctx, cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        unsigned grid = swc_grid(ctx, pixels * C, 256 * 4, 8);
        k<<<grid, 256, smem, ctx->stream>>>(output, input, mean, var, scale, bias, pixels, (int)C, epsilon);
    }
    return swc_check_launch(ctx, "batchnormalization_f");
}

static int transpose_common(swcb200_ctx *ctx, const float *input, float *output, const size_t *id, const size_t *od,
                            const size_t *sh, int nd) {
    size_t i[4] = {1, 1, 1, 1}, o[4] = {1, 1, 1, 1};
    int s[4] = {0, 1, 2, 3};
    // right-align an nd-dimensional problem into 4-D
    const int pad = 4 - nd;
    bool seen[4] = {false, false, false, false};
    for (int d = 0; d < nd; d++) {
        SWC_REQUIRE(ctx, sh[d] < (size_t)nd && !seen[sh[d]], SWCB200_ERR_BAD_ARG, "transpose: shuffle is not a permutation");
        seen[sh[d]] = true;
        i[pad + d] = id[d];
        o[pad + d] = od[d];
        s[pad + d] = pad + (int)sh[d];
    }
    for (int d = 0; d < nd; d++)
        SWC_REQUIRE(ctx, od[d] == id[sh[d]], SWCB200_ERR_BAD_SHAPE, "transpose: odims[%d] is not idims[shuffle[%d]]", d, d);
    size_t total = i[0] * i[1] * i[2] * i[3];
    if (total == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, input && output, SWCB200_ERR_BAD_ARG, "transpose: null tensor");
    unsigned grid = swc_grid(ctx, total, 256, 8);
    transpose4d_kernel<<<grid, 256, 0, ctx->stream>>>(input, output, i[0], i[1], i[2], i[3], o[1], o[2], o[3], s[0], s[1],
                                                      s[2], s[3]);
    return swc_check_launch(ctx, "transpose");
}

SWC_EXPORT int swcb200_transpose2d_f(swcb200_ctx *ctx, const float *input, float *output, const size_t *idims,
                                     const size_t *odims, const size_t *shuffle) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, idims && odims && shuffle, SWCB200_ERR_BAD_ARG, "transpose2d_f: null attribute array");
    return transpose_common(ctx, input, output, idims, odims, shuffle, 2);
}

SWC_EXPORT int swcb200_transpose4d_f(swcb200_ctx *ctx, const float *input, float *output, const size_t *idims,
                                     const size_t *odims, const size_t *shuffle) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, idims && odims && shuffle, SWCB200_ERR_BAD_ARG, "transpose4d_f: null attribute array");
    return transpose_common(ctx, input, output, idims, odims, shuffle, 4);
}
