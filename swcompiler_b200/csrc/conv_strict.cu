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
    conv_strict_kernel<<<grid, 256, 0, ctx->stream>>>(output, input, filter, bias, g);
    return swc_check_launch(ctx, "conv2d_f(strict)");
}
