// NHWC pooling: MaxPool (fp32 and bf16 storage) and AvgPool.
//
// One thread produces one output pixel x one group of channels (4 fp32 or 8 bf16 = 16 bytes when the
// channel count allows, else one channel).  Channels are the fastest thread index, so a warp reads
// whole 128-byte lines of every tap; with a 2x2/2 window every input byte is read exactly once.
#include <cuda_bf16.h>

#include "common.cuh"

namespace {

struct PoolGeom {
    int N, H, W, C, OH, OW, kh, kw, sh, sw, pt, pl;
};

// maxpool_f semantics (kernels.h:347-371): first in-range tap initialises, later taps replace only
// when strictly greater, out-of-range taps are ignored, no in-range tap -> 0.
struct MaxAcc {
    float v = 0.f;
    bool init = false;
    __device__ __forceinline__ void tap(float x) {
        if (!init || x > v) {
            v = x;
            init = true;
        }
    }
};

// Thread mapping shared by the pooling kernels: blockIdx.x walks output rows (n, oh), the threads of
// a CTA (and blockIdx.y) walk the ow x channel-group positions of that row, channel group fastest.
// All index arithmetic is 32-bit; the only divisions are by the channel-group count.
#define SWC_POOL_COORDS(kVec)                                                   \
    const int cg = g.C / (kVec);                                                \
    const int rowlen = g.OW * cg;                                               \
    const int pos = blockIdx.y * blockDim.x + threadIdx.x;                      \
    if (pos >= rowlen) return;                                                  \
    const int ow = pos / cg, c = (pos - ow * cg) * (kVec);

template <int kVec>  // 4: float4 over channels, 1: scalar
__global__ void __launch_bounds__(256) maxpool_f32_kernel(const float *__restrict__ in, float *__restrict__ out,
                                                          PoolGeom g) {
    SWC_POOL_COORDS(kVec)
    for (int row = blockIdx.x; row < g.N * g.OH; row += gridDim.x) {
        const int n = row / g.OH, oh = row - n * g.OH;
        MaxAcc acc[kVec];
        for (int kx = 0; kx < g.kh; kx++) {
            int ih = oh * g.sh - g.pt + kx;
            if (ih < 0 || ih >= g.H) continue;
            for (int ky = 0; ky < g.kw; ky++) {
                int iw = ow * g.sw - g.pl + ky;
                if (iw < 0 || iw >= g.W) continue;
                const float *src = in + (((size_t)n * g.H + ih) * g.W + iw) * g.C + c;
                if (kVec == 4) {
                    float4 x = __ldcs(reinterpret_cast<const float4 *>(src));
                    acc[0].tap(x.x);
                    acc[1 % kVec].tap(x.y);
                    acc[2 % kVec].tap(x.z);
                    acc[3 % kVec].tap(x.w);
                } else {
                    acc[0].tap(__ldcs(src));
                }
            }
        }
        float *dst = out + (((size_t)n * g.OH + oh) * g.OW + ow) * g.C + c;
        if (kVec == 4)
            __stcs(reinterpret_cast<float4 *>(dst), make_float4(acc[0].v, acc[1 % kVec].v, acc[2 % kVec].v, acc[3 % kVec].v));
        else
            *dst = acc[0].v;
    }
}

template <int kVec>  // 8: uint4 (8 bf16) over channels, 1: scalar
__global__ void __launch_bounds__(256) maxpool_bf16_kernel(const __nv_bfloat16 *__restrict__ in,
                                                           __nv_bfloat16 *__restrict__ out, PoolGeom g) {
    SWC_POOL_COORDS(kVec)
    for (int row = blockIdx.x; row < g.N * g.OH; row += gridDim.x) {
        const int n = row / g.OH, oh = row - n * g.OH;
        MaxAcc acc[kVec];
        for (int kx = 0; kx < g.kh; kx++) {
            int ih = oh * g.sh - g.pt + kx;
            if (ih < 0 || ih >= g.H) continue;
            for (int ky = 0; ky < g.kw; ky++) {
                int iw = ow * g.sw - g.pl + ky;
                if (iw < 0 || iw >= g.W) continue;
                const __nv_bfloat16 *src = in + (((size_t)n * g.H + ih) * g.W + iw) * g.C + c;
                if (kVec == 8) {
                    uint4 x = __ldcs(reinterpret_cast<const uint4 *>(src));
                    const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                    for (int i = 0; i < 4; i++) {  // bf16 -> fp32 is a 16-bit shift
                        acc[(2 * i) % kVec].tap(__uint_as_float(w[i] << 16));
                        acc[(2 * i + 1) % kVec].tap(__uint_as_float(w[i] & 0xffff0000u));
                    }
                } else {
                    acc[0].tap(__bfloat162float(*src));
                }
            }
        }
        __nv_bfloat16 *dst = out + (((size_t)n * g.OH + oh) * g.OW + ow) * g.C + c;
        if (kVec == 8) {
            uint4 o;  // the maxima are bf16 values already: the upper halves are the exact results
            o.x = (__float_as_uint(acc[0].v) >> 16) | (__float_as_uint(acc[1 % kVec].v) & 0xffff0000u);
            o.y = (__float_as_uint(acc[2 % kVec].v) >> 16) | (__float_as_uint(acc[3 % kVec].v) & 0xffff0000u);
            o.z = (__float_as_uint(acc[4 % kVec].v) >> 16) | (__float_as_uint(acc[5 % kVec].v) & 0xffff0000u);
            o.w = (__float_as_uint(acc[6 % kVec].v) >> 16) | (__float_as_uint(acc[7 % kVec].v) & 0xffff0000u);
            __stcs(reinterpret_cast<uint4 *>(dst), o);
        } else {
            *dst = __float2bfloat16_rn(acc[0].v);
        }
    }
}

// The common window, 2x2 stride 2 without padding and with every tap inside the image, on bf16 storage: the four
// 16-byte loads of a thread are issued back to back (the general kernel's bounds checks keep them apart), two
// output pixels per thread, and the comparisons then run in the reference's tap order (kx, then ky; a later
// tap replaces only when strictly greater).  128 bytes in flight per thread.
__global__ void __launch_bounds__(256) maxpool_bf16_2x2_kernel(const uint4 *__restrict__ in, uint4 *__restrict__ out,
                                                               int rows, int H, int W, int OH, int OW, int cg) {
    const int rowlen = OW * cg;           // uint4 per output row
    const int half = (rowlen + 1) >> 1;   // a thread takes positions pos and pos + half of the row
    const int pos = blockIdx.y * blockDim.x + threadIdx.x;
    if (pos >= half) return;
    const bool two = pos + half < rowlen;
    const int p0 = pos, p1 = two ? pos + half : pos;
    const int ow0 = p0 / cg, c0 = p0 - ow0 * cg, ow1 = p1 / cg, c1 = p1 - ow1 * cg;
    const size_t in_row = (size_t)W * cg;
    auto pick = [](uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
        // per 16-bit half: first tap, then strictly-greater replacements, compared as the fp32 values they stand for
        uint32_t r = 0;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t sh = h ? 0u : 16u, mask = h ? 0xffff0000u : 0xffffu;
            float v = __uint_as_float(h ? (a & mask) : (a << 16));
            const float tb = __uint_as_float(h ? (b & mask) : (b << 16)), tc = __uint_as_float(h ? (c & mask) : (c << 16)),
                        td = __uint_as_float(h ? (d & mask) : (d << 16));
            v = tb > v ? tb : v;
            v = tc > v ? tc : v;
            v = td > v ? td : v;
            r |= h ? (__float_as_uint(v) & mask) : (__float_as_uint(v) >> sh);
        }
        return r;
    };
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const int n = row / OH, oh = row - n * OH;
        const uint4 *top = in + ((size_t)n * H + 2 * oh) * in_row, *bot = top + in_row;
        const size_t i0 = (size_t)(2 * ow0) * cg + c0, i1 = (size_t)(2 * ow1) * cg + c1;
        const uint4 a0 = __ldcs(top + i0), b0 = __ldcs(top + i0 + cg), c0v = __ldcs(bot + i0), d0 = __ldcs(bot + i0 + cg);
        const uint4 a1 = __ldcs(top + i1), b1 = __ldcs(top + i1 + cg), c1v = __ldcs(bot + i1), d1 = __ldcs(bot + i1 + cg);
        uint4 *dst = out + (size_t)row * rowlen;
        __stcs(dst + p0, make_uint4(pick(a0.x, b0.x, c0v.x, d0.x), pick(a0.y, b0.y, c0v.y, d0.y), pick(a0.z, b0.z, c0v.z, d0.z),
                                    pick(a0.w, b0.w, c0v.w, d0.w)));
        if (two)
            __stcs(dst + p1, make_uint4(pick(a1.x, b1.x, c1v.x, d1.x), pick(a1.y, b1.y, c1v.y, d1.y),
                                        pick(a1.z, b1.z, c1v.z, d1.z), pick(a1.w, b1.w, c1v.w, d1.w)));
    }
}

// avgpool_f (kernels.h:444-493): in-range taps summed kx then ky, divided by kh*kw regardless of padding
__global__ void __launch_bounds__(256) avgpool_f32_kernel(const float *__restrict__ in, float *__restrict__ out,
                                                          PoolGeom g) {
    const size_t total = (size_t)g.N * g.OH * g.OW * g.C;
    const float cnt = (float)((size_t)g.kh * g.kw);
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
        int c = (int)(t % g.C);
        size_t p = t / g.C;
        int ow = (int)(p % g.OW);
        p /= g.OW;
        int oh = (int)(p % g.OH);
        int n = (int)(p / g.OH);
        float sum = 0.f;
        for (int kx = 0; kx < g.kh; kx++) {
            int ih = oh * g.sh - g.pt + kx;
            if (ih < 0 || ih >= g.H) continue;
            for (int ky = 0; ky < g.kw; ky++) {
                int iw = ow * g.sw - g.pl + ky;
                if (iw < 0 || iw >= g.W) continue;
                sum = __fadd_rn(sum, in[(((size_t)n * g.H + ih) * g.W + iw) * g.C + c]);
            }
        }
        out[t] = __fdiv_rn(sum, cnt);
    }
}

int make_geom(swcb200_ctx *ctx, const char *what, const size_t *idims, const size_t *odims, const size_t *kernels,
              const size_t *strides, const size_t *pads, PoolGeom *g) {
    SWC_REQUIRE(ctx, idims && odims && kernels && strides && pads, SWCB200_ERR_BAD_ARG, "%s: null attribute array", what);
    for (int i = 0; i < 4; i++)
        SWC_REQUIRE(ctx, idims[i] <= 0x7fffffff && odims[i] <= 0x7fffffff, SWCB200_ERR_TOO_LARGE,
                    "%s: dimension beyond 2^31", what);
    SWC_REQUIRE(ctx, strides[0] > 0 && strides[1] > 0, SWCB200_ERR_BAD_ARG, "%s: zero stride", what);
    SWC_REQUIRE(ctx, odims[0] == idims[0] && odims[3] == idims[3], SWCB200_ERR_BAD_SHAPE,
                "%s: batch/channel of output differ from input", what);
    *g = PoolGeom{(int)idims[0], (int)idims[1], (int)idims[2], (int)idims[3], (int)odims[1], (int)odims[2],
                  (int)kernels[0], (int)kernels[1], (int)strides[0], (int)strides[1], (int)pads[0], (int)pads[1]};
    return SWCB200_OK;
}

// rows of the output on grid.x (capped at a few waves), positions within a row on threads x grid.y
int pool_launch_geom(swcb200_ctx *ctx, const PoolGeom &g, int vec, dim3 *grid, dim3 *block) {
    const long long rowlen = (long long)g.OW * (g.C / vec);
    SWC_REQUIRE(ctx, rowlen <= 0x7fffffffLL && (long long)g.N * g.OH <= 0x7fffffffLL, SWCB200_ERR_TOO_LARGE,
                "pooling: output row or row count beyond 2^31");
    int threads = rowlen >= 256 ? 256 : (int)((rowlen + 31) / 32 * 32);
    const long long by = (rowlen + threads - 1) / threads;
    SWC_REQUIRE(ctx, by <= 65535, SWCB200_ERR_TOO_LARGE, "pooling: output row too long");
    const long long rows = (long long)g.N * g.OH;
    const long long cap = (long long)ctx->sm_count * 16;
    long long gx = rows < cap ? rows : cap;
    *grid = dim3((unsigned)gx, (unsigned)by);
    *block = dim3((unsigned)threads);
    return SWCB200_OK;
}

}  // namespace

SWC_EXPORT int swcb200_maxpool_f(swcb200_ctx *ctx, const float *input, float *output, const size_t *idims,
                                 const size_t *odims, const size_t *kernels, const size_t *strides,
                                 const size_t *pads) {
    SWC_CTX(ctx);
    PoolGeom g;
    int rc = make_geom(ctx, "maxpool_f", idims, odims, kernels, strides, pads, &g);
    if (rc) return rc;
    size_t total = (size_t)g.N * g.OH * g.OW * g.C;
    if (total == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, input && output, SWCB200_ERR_BAD_ARG, "maxpool_f: null tensor");
    bool vec = (g.C % 4 == 0) && swc_aligned16(input) && swc_aligned16(output);
    dim3 grid, block;
    rc = pool_launch_geom(ctx, g, vec ? 4 : 1, &grid, &block);
    if (rc) return rc;
    if (vec)
        maxpool_f32_kernel<4><<<grid, block, 0, ctx->stream>>>(input, output, g);
    else
        maxpool_f32_kernel<1><<<grid, block, 0, ctx->stream>>>(input, output, g);
    return swc_check_launch(ctx, "maxpool_f");
}

SWC_EXPORT int swcb200_maxpool_bf16(swcb200_ctx *ctx, const void *input, void *output, const size_t *idims,
                                    const size_t *odims, const size_t *kernels, const size_t *strides,
                                    const size_t *pads) {
    SWC_CTX(ctx);
    PoolGeom g;
    int rc = make_geom(ctx, "maxpool_bf16", idims, odims, kernels, strides, pads, &g);
    if (rc) return rc;
    size_t total = (size_t)g.N * g.OH * g.OW * g.C;
    if (total == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, input && output, SWCB200_ERR_BAD_ARG, "maxpool_bf16: null tensor");
    bool vec = (g.C % 8 == 0) && swc_aligned16(input) && swc_aligned16(output);
    dim3 grid, block;
    if (vec && g.kh == 2 && g.kw == 2 && g.sh == 2 && g.sw == 2 && g.pt == 0 && g.pl == 0 && 2 * g.OH <= g.H && 2 * g.OW <= g.W) {
        const int cg = g.C / 8;
        const long long rowlen = (long long)g.OW * cg, half = (rowlen + 1) / 2, rows = (long long)g.N * g.OH;
        SWC_REQUIRE(ctx, rowlen <= 0x7fffffffLL && rows <= 0x7fffffffLL, SWCB200_ERR_TOO_LARGE,
                    "maxpool_bf16: output row or row count beyond 2^31");
        const int threads = half >= 256 ? 256 : (int)((half + 31) / 32 * 32);
        const long long by = (half + threads - 1) / threads, cap = (long long)ctx->sm_count * 16;
        SWC_REQUIRE(ctx, by <= 65535, SWCB200_ERR_TOO_LARGE, "maxpool_bf16: output row too long");
        maxpool_bf16_2x2_kernel<<<dim3((unsigned)(rows < cap ? rows : cap), (unsigned)by), threads, 0, ctx->stream>>>(
            (const uint4 *)input, (uint4 *)output, (int)rows, g.H, g.W, g.OH, g.OW, cg);
        return swc_check_launch(ctx, "maxpool_bf16");
    }
    rc = pool_launch_geom(ctx, g, vec ? 8 : 1, &grid, &block);
    if (rc) return rc;
    if (vec)
        maxpool_bf16_kernel<8><<<grid, block, 0, ctx->stream>>>((const __nv_bfloat16 *)input, (__nv_bfloat16 *)output, g);
    else
        maxpool_bf16_kernel<1><<<grid, block, 0, ctx->stream>>>((const __nv_bfloat16 *)input, (__nv_bfloat16 *)output, g);
    return swc_check_launch(ctx, "maxpool_bf16");
}

SWC_EXPORT int swcb200_avgpool_f(swcb200_ctx *ctx, const float *input, float *output, const size_t *idims,
                                 const size_t *odims, const size_t *kernels, const size_t *strides,
                                 const size_t *pads) {
    SWC_CTX(ctx);
    PoolGeom g;
    int rc = make_geom(ctx, "avgpool_f", idims, odims, kernels, strides, pads, &g);
    if (rc) return rc;
    SWC_REQUIRE(ctx, g.kh > 0 && g.kw > 0, SWCB200_ERR_BAD_ARG, "avgpool_f: empty window");
    size_t total = (size_t)g.N * g.OH * g.OW * g.C;
    if (total == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, input && output, SWCB200_ERR_BAD_ARG, "avgpool_f: null tensor");
    unsigned grid = swc_grid(ctx, total, 256, 8);
    avgpool_f32_kernel<<<grid, 256, 0, ctx->stream>>>(input, output, g);
    return swc_check_launch(ctx, "avgpool_f");
}
