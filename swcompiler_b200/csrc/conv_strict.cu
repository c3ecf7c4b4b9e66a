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
// staged once per CTA, then no barrier inside the tap loops, and a CTA walks many groups of pixels.  For the
// filters that fit (kh*kw*C <= kMaxResidentK); the kernel above takes the rest.
//
// A warp works on P consecutive pixels at once, one accumulator each: the sum of one output element is a chain of
// dependent additions (the reference's order), so P pixels are P independent chains, and one filter word read from
// shared memory serves all of them.  The host picks P (4, 2 or 1) so that a small layer still spreads over enough
// warps to hide its load latency.  With VEC4 (iC a multiple of 4, 16-byte aligned input) a pixel's channels are
// fetched four at a time.  Row and column offsets are advanced by additions; on the small layers of a
// latency-bound network the address arithmetic of a tap used to cost more instructions than its multiply-adds.
constexpr int kMaxResidentK = 1536;  // 1536 x 33 floats = 198 KiB

template <int P, bool VEC4>
__global__ void __launch_bounds__(256) conv_strict_resident_kernel(float *__restrict__ out, const float *__restrict__ in,
                                                                   const float *__restrict__ filt,
                                                                   const float *__restrict__ bias, ConvGeom g) {
    extern __shared__ float fr[];  // fr[q][co], pitch kCo + 1, q = (kx * kw + ky) * C + ci
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = g.kh * g.kw * g.C;
    const int co0 = blockIdx.y * kCo, co = co0 + lane;
    for (int r = warp; r < kCo; r += kPix) {  // a warp reads consecutive words of one filter row
        const bool row_ok = co0 + r < g.OC;
        const float *src = filt + (size_t)(co0 + r) * K;
        for (int q = lane; q < K; q += 32) fr[q * (kCo + 1) + r] = row_ok ? src[q] : 0.f;
    }
    __syncthreads();
    const bool co_ok = co < g.OC;
    const float b = co_ok ? bias[co] : 0.f;
    const size_t npix = (size_t)g.N * g.OH * g.OW;
    const size_t stride = (size_t)gridDim.x * kPix * P;
    const int row_words = g.W * g.C;
    for (size_t base = ((size_t)blockIdx.x * kPix + warp) * P; base < npix; base += stride) {
        // the warp's pixels base .. base+P-1 (consecutive in n, oh, ow order; they may straddle a row or an image)
        int ih0[P], iw0[P];
        const float *img[P];
        bool live[P];
        float acc[P];
        {
            size_t p = base;
            int ow = (int)(p % g.OW);
            p /= g.OW;
            int oh = (int)(p % g.OH), n = (int)(p / g.OH);
#pragma unroll
            for (int u = 0; u < P; u++) {
                live[u] = base + u < npix;
                ih0[u] = oh * g.sh - g.pt;
                iw0[u] = ow * g.sw - g.pl;
                img[u] = in + (size_t)n * g.H * row_words;
                acc[u] = b;
                if (++ow == g.OW) {
                    ow = 0;
                    if (++oh == g.OH) {
                        oh = 0;
                        n++;
                    }
                }
            }
        }
        const float *fq = fr + lane;  // walks the resident filter in q order
        for (int kx = 0; kx < g.kh; kx++) {
            const float *rowp[P];
            bool row_ok[P];
#pragma unroll
            for (int u = 0; u < P; u++) {
                const int ih = ih0[u] + kx;
                row_ok[u] = live[u] && ih >= 0 && ih < g.H;
                rowp[u] = img[u] + (size_t)(row_ok[u] ? ih : 0) * row_words;
            }
            for (int ky = 0; ky < g.kw; ky++, fq += g.C * (kCo + 1)) {
                // a tap outside the image is skipped for that pixel (uniform within the warp: every lane has the same pixels)
                const float *ip[P];
                bool ok[P];
                bool any = false;
#pragma unroll
                for (int u = 0; u < P; u++) {
                    const int iw = iw0[u] + ky;
                    ok[u] = row_ok[u] && iw >= 0 && iw < g.W;
                    ip[u] = ok[u] ? rowp[u] + iw * g.C : in;
                    any = any || ok[u];
                }
                if (!any) continue;
                if (VEC4) {
                    for (int ci = 0; ci < g.C; ci += 4) {
                        const float *f = fq + ci * (kCo + 1);
                        const float w0 = f[0], w1 = f[kCo + 1], w2 = f[2 * (kCo + 1)], w3 = f[3 * (kCo + 1)];
#pragma unroll
                        for (int u = 0; u < P; u++) {
                            const float4 v = __ldg(reinterpret_cast<const float4 *>(ip[u] + ci));
                            if (ok[u]) {
                                acc[u] = __fadd_rn(acc[u], __fmul_rn(v.x, w0));
                                acc[u] = __fadd_rn(acc[u], __fmul_rn(v.y, w1));
                                acc[u] = __fadd_rn(acc[u], __fmul_rn(v.z, w2));
                                acc[u] = __fadd_rn(acc[u], __fmul_rn(v.w, w3));
                            }
                        }
                    }
                } else {
                    for (int ci = 0; ci < g.C; ci++) {
                        const float w = fq[ci * (kCo + 1)];
#pragma unroll
                        for (int u = 0; u < P; u++) {
                            const float v = __ldg(ip[u] + ci);
                            if (ok[u]) acc[u] = __fadd_rn(acc[u], __fmul_rn(v, w));
                        }
                    }
                }
            }
        }
        if (co_ok) {
#pragma unroll
            for (int u = 0; u < P; u++)
                if (live[u]) out[(base + u) * g.OC + co] = acc[u];
        }
    }
}

// Small layers (a few input channels, the whole filter of every output channel resident): one output element per
// thread, output channel fastest, so a warp is one or two pixels, its input values are broadcast loads and its
// store is one line.  No per-warp bookkeeping for groups of pixels: on a [32,28,28,1] -> 16 channel 5x5 layer the
// kernel above spends 200 instructions per tap on it, this one about 20.  Same order of additions per element.
constexpr int kPointMaxC = 32;

// KH, KW and CI, where not 0, are the filter's rows, columns and input channels as compile-time constants (loops
// unrolled, offsets folded).
template <bool VEC4, int KH, int KW, int CI>
__global__ void __launch_bounds__(256, 4) conv_strict_point_kernel(float *__restrict__ out, const float *__restrict__ in,
                                                                const float *__restrict__ filt, const float *__restrict__ bias,
                                                                ConvGeom gg, int ocp, unsigned total) {
    extern __shared__ float fr[];  // fr[q][co], pitch ocp, q = (kx * kw + ky) * C + ci
    ConvGeom g = gg;
    if (KH) {
        g.kh = KH;
        g.kw = KW;
    }
    if (CI) g.C = CI;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = g.kh * g.kw * g.C;
    for (int r = warp; r < g.OC; r += 8) {  // a warp reads consecutive words of one filter row
        const float *src = filt + (size_t)r * K;
        for (int q = lane; q < K; q += 32) fr[q * ocp + r] = src[q];
    }
    __syncthreads();
    const int row_words = g.W * g.C, tap_words = g.C * ocp;
    for (unsigned idx = blockIdx.x * 256u + threadIdx.x; idx < total; idx += gridDim.x * 256u) {
        const unsigned pix = idx / (unsigned)g.OC;
        const int co = (int)(idx - pix * (unsigned)g.OC);
        const unsigned t = pix / (unsigned)g.OW;
        const int ow = (int)(pix - t * (unsigned)g.OW);
        const unsigned n = t / (unsigned)g.OH;
        const int oh = (int)(t - n * (unsigned)g.OH);
        const float *img = in + (size_t)n * g.H * row_words;
        const int ih0 = oh * g.sh - g.pt, iw0 = ow * g.sw - g.pl;
        float acc = bias[co];
        const float *fk = fr + co;
#pragma unroll
        for (int kx = 0; kx < g.kh; kx++, fk += g.kw * tap_words) {
            const int ih = ih0 + kx;
            if (ih < 0 || ih >= g.H) continue;
            const float *rowp = img + ih * row_words;
            const float *fq = fk;
#pragma unroll
            for (int ky = 0; ky < g.kw; ky++, fq += tap_words) {
                const int iw = iw0 + ky;
                if (iw < 0 || iw >= g.W) continue;
                const float *ip = rowp + iw * g.C;
                if (VEC4) {
#pragma unroll
                    for (int ci = 0; ci < g.C; ci += 4) {
                        const float4 v = __ldg(reinterpret_cast<const float4 *>(ip + ci));
                        const float *f = fq + ci * ocp;
                        acc = __fadd_rn(acc, __fmul_rn(v.x, f[0]));
                        acc = __fadd_rn(acc, __fmul_rn(v.y, f[ocp]));
                        acc = __fadd_rn(acc, __fmul_rn(v.z, f[2 * ocp]));
                        acc = __fadd_rn(acc, __fmul_rn(v.w, f[3 * ocp]));
                    }
                } else {
#pragma unroll
                    for (int ci = 0; ci < g.C; ci++) acc = __fadd_rn(acc, __fmul_rn(__ldg(ip + ci), fq[ci * ocp]));
                }
            }
        }
        out[idx] = acc;
    }
}

// The same with TWO horizontally adjacent output pixels per thread (iC a multiple of 4): every filter word read from
// shared memory serves both, which halves the reads that bound the kernel above once a layer has 16 or more input
// channels (one shared-memory read per multiply-add there).  Output columns are paired inside a row: OW must be even.
template <int CI>
__global__ void __launch_bounds__(256, 4) conv_strict_point2_kernel(float *__restrict__ out, const float *__restrict__ in,
                                                                 const float *__restrict__ filt, const float *__restrict__ bias,
                                                                 ConvGeom gg, int ocp, unsigned total_pairs) {
    extern __shared__ float fr[];  // fr[q][co], pitch ocp, q = (kx * kw + ky) * C + ci
    ConvGeom g = gg;
    if (CI) g.C = CI;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = g.kh * g.kw * g.C;
    for (int r = warp; r < g.OC; r += 8) {
        const float *src = filt + (size_t)r * K;
        for (int q = lane; q < K; q += 32) fr[q * ocp + r] = src[q];
    }
    __syncthreads();
    const int row_words = g.W * g.C, tap_words = g.C * ocp, half_ow = g.OW >> 1;
    for (unsigned idx = blockIdx.x * 256u + threadIdx.x; idx < total_pairs; idx += gridDim.x * 256u) {
        const unsigned pp = idx / (unsigned)g.OC;          // pixel pair
        const int co = (int)(idx - pp * (unsigned)g.OC);
        const unsigned t = pp / (unsigned)half_ow;
        const int ow = 2 * (int)(pp - t * (unsigned)half_ow);
        const unsigned n = t / (unsigned)g.OH;
        const int oh = (int)(t - n * (unsigned)g.OH);
        const float *img = in + (size_t)n * g.H * row_words;
        const int ih0 = oh * g.sh - g.pt, iwa = ow * g.sw - g.pl, iwb = iwa + g.sw;
        float acc0 = bias[co], acc1 = acc0;
        const float *fk = fr + co;
        for (int kx = 0; kx < g.kh; kx++, fk += g.kw * tap_words) {
            const int ih = ih0 + kx;
            if (ih < 0 || ih >= g.H) continue;
            const float *rowp = img + ih * row_words;
            const float *fq = fk;
            for (int ky = 0; ky < g.kw; ky++, fq += tap_words) {
                const int ia = iwa + ky, ib = iwb + ky;
                const bool oka = ia >= 0 && ia < g.W, okb = ib >= 0 && ib < g.W;
                if (!oka && !okb) continue;
                const float *pa = oka ? rowp + ia * g.C : in, *pb = okb ? rowp + ib * g.C : in;
#pragma unroll
                for (int ci = 0; ci < g.C; ci += 4) {
                    const float4 va = __ldg(reinterpret_cast<const float4 *>(pa + ci));
                    const float4 vb = __ldg(reinterpret_cast<const float4 *>(pb + ci));
                    const float *f = fq + ci * ocp;
                    const float w0 = f[0], w1 = f[ocp], w2 = f[2 * ocp], w3 = f[3 * ocp];
                    if (oka) {
                        acc0 = __fadd_rn(acc0, __fmul_rn(va.x, w0));
                        acc0 = __fadd_rn(acc0, __fmul_rn(va.y, w1));
                        acc0 = __fadd_rn(acc0, __fmul_rn(va.z, w2));
                        acc0 = __fadd_rn(acc0, __fmul_rn(va.w, w3));
                    }
                    if (okb) {
                        acc1 = __fadd_rn(acc1, __fmul_rn(vb.x, w0));
                        acc1 = __fadd_rn(acc1, __fmul_rn(vb.y, w1));
                        acc1 = __fadd_rn(acc1, __fmul_rn(vb.z, w2));
                        acc1 = __fadd_rn(acc1, __fmul_rn(vb.w, w3));
                    }
                }
            }
        }
        const size_t o = ((size_t)(t * (unsigned)g.OW) + (unsigned)ow) * (unsigned)g.OC + (unsigned)co;
        out[o] = acc0;
        out[o + g.OC] = acc1;
    }
}

template <int P, bool VEC4>
int launch_resident(swcb200_ctx *ctx, float *out, const float *in, const float *filt, const float *bias, const ConvGeom &g,
                    unsigned cap, unsigned grid_y, size_t smem) {
    static bool attr_set[64] = {false};  // per device: the opt-in to large dynamic shared memory
    if (!attr_set[ctx->device & 63]) {
        SWC_CUDA(ctx, cudaFuncSetAttribute(conv_strict_resident_kernel<P, VEC4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kMaxResidentK * (kCo + 1) * (int)sizeof(float)));
        attr_set[ctx->device & 63] = true;
    }
    const size_t npix = (size_t)g.N * g.OH * g.OW;
    const unsigned want = (unsigned)((npix + (size_t)kPix * P - 1) / ((size_t)kPix * P));
    dim3 gr(want < cap ? want : cap, grid_y);
    conv_strict_resident_kernel<P, VEC4><<<gr, 256, smem, ctx->stream>>>(out, in, filt, bias, g);
    return swc_check_launch(ctx, "conv2d_f(strict)");
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
    if (g.C <= kPointMaxC && K * g.OC * 4 <= 96 * 1024 && npix * g.OC < 0x7fffffffu &&
        (size_t)g.H * g.W * g.C < 0x7fffffffu) {
        // odd pitch in words (or 1 mod 32 for 32 channels and more): a warp's lanes read different banks
        const int ocp = g.OC | 1;
        const size_t smem = (size_t)K * ocp * sizeof(float);
        const unsigned total = (unsigned)(npix * g.OC);
        const bool vec = g.C % 4 == 0 && swc_aligned16(input);
        unsigned per_sm = (unsigned)((227 * 1024) / (smem + 1024));  // CTAs of this filter size that share an SM
        per_sm = per_sm > 8 ? 8 : per_sm;
        const unsigned want = (total + 255) / 256, cap = (unsigned)ctx->sm_count * per_sm;
        const unsigned gx = want < cap ? want : cap;
        // the filter shapes of the small networks this path exists for get kernels with their tap loops unrolled
#define SWC_POINT(VEC, KH_, KW_, CI_)                                                                                          \
    do {                                                                                                                       \
        static bool set_[64] = {false};                                                                                        \
        if (!set_[ctx->device & 63]) {                                                                                         \
            SWC_CUDA(ctx, cudaFuncSetAttribute(conv_strict_point_kernel<VEC, KH_, KW_, CI_>,                                   \
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));                      \
            set_[ctx->device & 63] = true;                                                                                     \
        }                                                                                                                      \
        conv_strict_point_kernel<VEC, KH_, KW_, CI_><<<gx, 256, smem, ctx->stream>>>(output, input, filter, bias, g, ocp, total); \
    } while (0)
        if (vec && g.C >= 16 && g.OW % 2 == 0) {
            // two pixels per thread: half the shared-memory reads per multiply-add
            const unsigned pairs = total / 2, want2 = (pairs + 255) / 256, gx2 = want2 < cap ? want2 : cap;
            static bool set2[64] = {false};
            if (!set2[ctx->device & 63]) {
                SWC_CUDA(ctx, cudaFuncSetAttribute(conv_strict_point2_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
                SWC_CUDA(ctx, cudaFuncSetAttribute(conv_strict_point2_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
                set2[ctx->device & 63] = true;
            }
            if (g.C == 16)
                conv_strict_point2_kernel<16><<<gx2, 256, smem, ctx->stream>>>(output, input, filter, bias, g, ocp, pairs);
            else
                conv_strict_point2_kernel<0><<<gx2, 256, smem, ctx->stream>>>(output, input, filter, bias, g, ocp, pairs);
            return swc_check_launch(ctx, "conv2d_f(strict)");
        }
        if (g.kh == 5 && g.kw == 5 && g.C == 1) SWC_POINT(false, 5, 5, 1);
        else if (g.kh == 3 && g.kw == 3 && g.C == 1) SWC_POINT(false, 3, 3, 1);
        else if (g.C == 16 && vec) SWC_POINT(true, 0, 0, 16);
        else if (g.C == 32 && vec) SWC_POINT(true, 0, 0, 32);
        else if (vec) SWC_POINT(true, 0, 0, 0);
        else SWC_POINT(false, 0, 0, 0);
#undef SWC_POINT
        return swc_check_launch(ctx, "conv2d_f(strict)");
    }
    if (K <= kMaxResidentK) {
        const size_t smem = (size_t)K * (kCo + 1) * sizeof(float);
        // as many CTAs as keep every SM busy for this filter's shared-memory footprint; each walks its share of the pixels
        const unsigned per_sm = (unsigned)(smem > 100 * 1024 ? 1 : (smem > 48 * 1024 ? 2 : 4));
        unsigned cap = (unsigned)ctx->sm_count * per_sm / grid.y;
        if (cap < 1) cap = 1;
        // pixels per warp: as many as still leave about 24 warps per SM
        const size_t enough = (size_t)24 * ctx->sm_count;
        const int P = (npix / 4) * grid.y >= enough ? 4 : ((npix / 2) * grid.y >= enough ? 2 : 1);
        const bool vec = g.C % 4 == 0 && swc_aligned16(input);
#define SWC_RESIDENT(PP, VV) launch_resident<PP, VV>(ctx, output, input, filter, bias, g, cap, grid.y, smem)
        if (vec) return P == 4 ? SWC_RESIDENT(4, true) : (P == 2 ? SWC_RESIDENT(2, true) : SWC_RESIDENT(1, true));
        return P == 4 ? SWC_RESIDENT(4, false) : (P == 2 ? SWC_RESIDENT(2, false) : SWC_RESIDENT(1, false));
#undef SWC_RESIDENT
    }
    conv_strict_kernel<<<grid, 256, 0, ctx->stream>>>(output, input, filter, bias, g);
    return swc_check_launch(ctx, "conv2d_f(strict)");
}
