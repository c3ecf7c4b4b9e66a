// Strict fp32 NHWC convolution: bit-for-bit the result of conv2d_f (kernels.h:177-243).
//
// Per output element the reference starts from bias[co] and adds one product at a time in the order
// filter row kx, filter column ky, input channel ci, skipping taps outside the image; product and
// sum are rounded separately.  This kernel keeps that order.  A CTA owns 8 output pixels x 32
// output channels: one warp per pixel, one lane per output channel, so the tap-in-range test is
// uniform within a warp and the input value is a broadcast load.  Filter slices [32 co][32 ci] of
// the current tap are staged through shared memory, transposed so lanes read consecutive words.
#include "common.cuh"

namespace {

struct ConvGeom {
    int N, H, W, C, OH, OW, OC, kh, kw, sh, sw, pt, pl;
};

constexpr int kPix = 8, kCo = 32, kCi = 32;

__global__ void __launch_bounds__(256) conv_strict_kernel(float *__restrict__ out, const float *__restrict__ in,
                                                          const float *__restrict__ filt, const float *__restrict__ bias,
                                                          ConvGeom g) {
    __shared__ float fs[kCi][kCo + 1];  // fs[ci][co]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t npix = (size_t)g.N * g.OH * g.OW;
    const size_t pix = (size_t)blockIdx.x * kPix + warp;
    const int co = blockIdx.y * kCo + lane;
    const bool pix_ok = pix < npix, co_ok = co < g.OC;
    int n = 0, oh = 0, ow = 0;
    if (pix_ok) {
        size_t p = pix;
        ow = (int)(p % g.OW);
        p /= g.OW;
        oh = (int)(p % g.OH);
        n = (int)(p / g.OH);
    }
    float acc = co_ok ? bias[co] : 0.f;
    for (int kx = 0; kx < g.kh; kx++) {
        const int ih = oh * g.sh - g.pt + kx;
        for (int ky = 0; ky < g.kw; ky++) {
            const int iw = ow * g.sw - g.pl + ky;
            const bool tap_ok = pix_ok && ih >= 0 && ih < g.H && iw >= 0 && iw < g.W;
            const float *ip = tap_ok ? in + (((size_t)n * g.H + ih) * g.W + iw) * g.C : in;
            for (int c0 = 0; c0 < g.C; c0 += kCi) {
                // stage filter[co_tile][kx][ky][c0 .. c0+31]: warp w loads rows co = w, w+8, ...; lane = ci
                __syncthreads();
#pragma unroll
                for (int r = warp; r < kCo; r += 8) {
                    const int fco = blockIdx.y * kCo + r, ci = c0 + lane;
                    fs[lane][r] = (fco < g.OC && ci < g.C)
                                      ? filt[(((size_t)fco * g.kh + kx) * g.kw + ky) * g.C + ci]
                                      : 0.f;
                }
                __syncthreads();
                if (tap_ok) {
                    const int cmax = min(kCi, g.C - c0);
                    for (int ci = 0; ci < cmax; ci++)
                        acc = __fadd_rn(acc, __fmul_rn(__ldg(ip + c0 + ci), fs[ci][lane]));
                }
            }
        }
    }
    if (pix_ok && co_ok) out[pix * g.OC + co] = acc;
}

// The same arithmetic with the CTA's whole filter slice (32 output channels x kh*kw*C) resident in shared memory:
// staged once per CTA, then no barrier inside the tap loops, and a CTA walks many groups of 8 pixels.  For the
// filters that fit (kh*kw*C <= kMaxResidentK); the kernel above takes the rest.
constexpr int kMaxResidentK = 1536;  // 1536 x 33 floats = 198 KiB

__global__ void __launch_bounds__(256) conv_strict_resident_kernel(float *__restrict__ out, const float *__restrict__ in,
                                                                   const float *__restrict__ filt,
                                                                   const float *__restrict__ bias, ConvGeom g) {
    extern __shared__ float fr[];  // fr[q][co], pitch kCo + 1, q = (kx * kw + ky) * C + ci
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = g.kh * g.kw * g.C;
    const int co0 = blockIdx.y * kCo, co = co0 + lane;
    for (int idx = threadIdx.x; idx < K * kCo; idx += blockDim.x) {
        const int r = idx / K, q = idx - r * K;  // consecutive threads read consecutive words of one filter row
        fr[q * (kCo + 1) + r] = (co0 + r < g.OC) ? filt[(size_t)(co0 + r) * K + q] : 0.f;
    }
    __syncthreads();
    const bool co_ok = co < g.OC;
    const float b = co_ok ? bias[co] : 0.f;
    const size_t npix = (size_t)g.N * g.OH * g.OW;
    for (size_t pix = (size_t)blockIdx.x * kPix + warp; pix < npix; pix += (size_t)gridDim.x * kPix) {
        size_t p = pix;
        const int ow = (int)(p % g.OW);
        p /= g.OW;
        const int oh = (int)(p % g.OH), n = (int)(p / g.OH);
        float acc = b;
        for (int kx = 0; kx < g.kh; kx++) {
            const int ih = oh * g.sh - g.pt + kx;
            if (ih < 0 || ih >= g.H) continue;  // uniform within the warp: one pixel per warp
            for (int ky = 0; ky < g.kw; ky++) {
                const int iw = ow * g.sw - g.pl + ky;
                if (iw < 0 || iw >= g.W) continue;
                const float *ip = in + (((size_t)n * g.H + ih) * g.W + iw) * g.C;
                const float *fq = fr + (size_t)((kx * g.kw + ky) * g.C) * (kCo + 1) + lane;
                for (int ci = 0; ci < g.C; ci++) acc = __fadd_rn(acc, __fmul_rn(__ldg(ip + ci), fq[ci * (kCo + 1)]));
            }
        }
        if (co_ok) out[pix * g.OC + co] = acc;
    }
}

}  // namespace

int swc_conv_tc_from_f32(swcb200_ctx *ctx, float *output, const float *input, const float *filter, const float *bias,
                         const size_t *odims, const size_t *idims, const size_t *fdims, const size_t *kernels,
                         const size_t *strides, const size_t *pads);

SWC_EXPORT int swcb200_conv2d_f(swcb200_ctx *ctx, float *output, const float *input, const float *filter,
                                const float *bias, const size_t *odims, const size_t *idims, const size_t *fdims,
                                const size_t *bdims, const size_t *kernels, const size_t *strides, const size_t *pads,
                                size_t group) {
    SWC_CTX(ctx);
    (void)bdims;
    SWC_REQUIRE(ctx, odims && idims && fdims && kernels && strides && pads, SWCB200_ERR_BAD_ARG,
                "conv2d_f: null attribute array");
    SWC_REQUIRE(ctx, group == 1, SWCB200_ERR_UNSUPPORTED,
                "conv2d_f: group %zu (the reference's own group > 1 indexing reads past its filter)", group);
    for (int i = 0; i < 4; i++)
        SWC_REQUIRE(ctx, idims[i] <= 0x7fffffff && odims[i] <= 0x7fffffff && fdims[i] <= 0x7fffffff,
                    SWCB200_ERR_TOO_LARGE, "conv2d_f: dimension beyond 2^31");
    SWC_REQUIRE(ctx, strides[0] > 0 && strides[1] > 0, SWCB200_ERR_BAD_ARG, "conv2d_f: zero stride");
    SWC_REQUIRE(ctx, odims[0] == idims[0] && odims[3] == fdims[0] && fdims[3] == idims[3] && fdims[1] == kernels[0] &&
                         fdims[2] == kernels[1],
                SWCB200_ERR_BAD_SHAPE, "conv2d_f: input/filter/output dims disagree");
    ConvGeom g{(int)idims[0], (int)idims[1], (int)idims[2], (int)idims[3], (int)odims[1], (int)odims[2], (int)odims[3],
               (int)kernels[0], (int)kernels[1], (int)strides[0], (int)strides[1], (int)pads[0], (int)pads[1]};
    const size_t npix = (size_t)g.N * g.OH * g.OW;
    if (npix * g.OC == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, output && input && filter && bias, SWCB200_ERR_BAD_ARG, "conv2d_f: null tensor");
    if (ctx->precision == SWCB200_TC_BF16) {
        int rc = swc_conv_tc_from_f32(ctx, output, input, filter, bias, odims, idims, fdims, kernels, strides, pads);
        if (rc != SWCB200_ERR_UNSUPPORTED) return rc;  // shapes the tensor-core kernel does not take run strict
    }
    dim3 grid((unsigned)((npix + kPix - 1) / kPix), (g.OC + kCo - 1) / kCo);
    SWC_REQUIRE(ctx, grid.y <= 65535, SWCB200_ERR_TOO_LARGE, "conv2d_f: too many output channels");
    const long long K = (long long)g.kh * g.kw * g.C;
    if (K <= kMaxResidentK) {
        static bool attr_set[64] = {false};  // per device: the opt-in to large dynamic shared memory
        if (!attr_set[ctx->device & 63]) {
            SWC_CUDA(ctx, cudaFuncSetAttribute(conv_strict_resident_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               kMaxResidentK * (kCo + 1) * (int)sizeof(float)));
            attr_set[ctx->device & 63] = true;
        }
        const size_t smem = (size_t)K * (kCo + 1) * sizeof(float);
        // as many CTAs as keep every SM busy for this filter's shared-memory footprint; each walks its share of the pixels
        const unsigned per_sm = (unsigned)(smem > 100 * 1024 ? 1 : (smem > 48 * 1024 ? 2 : 4));
        unsigned cap = (unsigned)ctx->sm_count * per_sm / grid.y;
        if (cap < 1) cap = 1;
        dim3 gr(grid.x < cap ? grid.x : cap, grid.y);
        conv_strict_resident_kernel<<<gr, 256, smem, ctx->stream>>>(output, input, filter, bias, g);
        return swc_check_launch(ctx, "conv2d_f(strict)");
    }
    conv_strict_kernel<<<grid, 256, 0, ctx->stream>>>(output, input, filter, bias, g);
    return swc_check_launch(ctx, "conv2d_f(strict)");
}
