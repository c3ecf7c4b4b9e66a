// NHWC convolution as an implicit GEMM on the 5th-generation tensor cores, with the reference's
// Conv2d -> BatchNormalization -> [ElementAdd] -> [Relu] chain folded into the epilogue
// (arithmetic of kernels.h:177-243, :496-517, :592-596, :575-580).
//
//   out[n, oh, ow, :] = epi( sum over taps (kx, ky) and channels of  in[n, oh+kx-pt, ow+ky-pl, :] . filt[:, kx, ky, :] )
//
// GEMM view: M = output pixels, N = oC, K = kh*kw*iC, bf16 operands, fp32 accumulation in tensor memory.
//   * A tile of 128 output pixels is two 8x8 pixel blocks (so 56x56 images tile with no waste, and a tile
//     may straddle images).  For one filter tap its A operand is the same two blocks shifted by the tap:
//     two 4-D TMA boxes {64 ch, 8, 8, 1} of the input; pixels outside the image (the padding) arrive as
//     zeros from TMA's out-of-bounds fill, so there is no im2col buffer and no halo logic.  A pixel's 64
//     channels are exactly one 128-byte swizzle row, which makes the box a K-major UMMA operand as is.
//   * The whole filter stays resident in shared memory for the life of the (persistent) CTA:
//     kh*kw*(iC/64) slices of [oC x 64] loaded once by TMA.
//   * Shared-memory barrier operations cost on the order of 100 cycles each on this part, and one MMA of
//     this shape (N = oC = 64) lasts well under that, so the pipeline hands over a whole filter ROW at a
//     time: a stage holds the A operands of the kw taps of one filter row (kw * iC/64 slots of 16 KiB),
//     filled by two producer warps (warp 0: the first 8x8 block of every slot, warp 6: the second), one
//     barrier wait and one expect-tx per producer per row.  Warp 1 waits once per row, issues all of its
//     tcgen05.mma (4 per slot, M128 x N=oC x K16) back to back and releases the row with one commit.
//     Warps 2-5 run the epilogue out of up to four tensor-memory accumulators while the next tiles compute.
//   Restrictions: stride 1, group 1, iC a multiple of 64, oC a multiple of 32 and <= 256, filter at most
//   96 KiB in bf16.  Other shapes return SWCB200_ERR_UNSUPPORTED (the strict kernel takes them).
#include "tc_common.cuh"

namespace {

using namespace tc;

constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int BLOCK_PIX = 64;            // 8 x 8 pixels
constexpr int A_STAGE_BYTES = BM * 128;  // 16 KiB
constexpr int kThreads = 224;  // producer A, MMA issuer, 4 epilogue warps, producer B
constexpr int kMaxFilterBytes = 96 * 1024;
constexpr int kMaxSmem = 227 * 1024;

struct ConvParams {
    int N, H, W, C, OH, OW, OC, kh, kw, pt, pl;
    int kchunks;            // C / 64
    int blocks_h, blocks_w; // 8x8 blocks per image
    long long num_blocks, num_tiles;
    int stages, slots, acc_stride, num_acc, tmem_cols;  // stages = row stages in the ring, slots = 16 KiB slots per row
    int filter_bytes;
    const float *bias;
    const float *bn_scale, *bn_bias, *bn_mean, *bn_var;
    float bn_eps;
    const void *residual;
    int relu;
    void *out;
    int out_is_f32, res_is_f32;
    int *status;
};

__global__ void __launch_bounds__(kThreads, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap tmIn, const __grid_constant__ CUtensorMap tmF, const ConvParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *s_filter = smem;                                   // [taps*kchunks][OC x 128 B]
    uint8_t *s_a = smem + p.filter_bytes;                       // stages x slots x 16 KiB
    const int row_bytes = p.slots * A_STAGE_BYTES;
    float *s_alpha = reinterpret_cast<float *>(s_a + (size_t)p.stages * row_bytes);  // [OC]
    float *s_beta = s_alpha + p.OC;                             // [OC]
    uint64_t *full = reinterpret_cast<uint64_t *>(s_beta + p.OC);
    uint64_t *empty = full + 8;
    uint64_t *tmem_full = empty + 8;
    uint64_t *tmem_empty = tmem_full + 4;
    uint64_t *filter_bar = tmem_empty + 4;
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(filter_bar + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int taps = p.kh * p.kw;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmIn);
        tma_prefetch_desc(&tmF);
        for (int s = 0; s < p.stages; s++) {
            mbar_init(&full[s], 2);   // one arrive(+expect-tx) from each producer warp
            mbar_init(&empty[s], 1);  // one tcgen05.commit
        }
        for (int b = 0; b < p.num_acc; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], 4);  // one arrival per epilogue warp
        }
        mbar_init(filter_bar, 1);
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        tmem_alloc(tmem_holder, (uint32_t)p.tmem_cols);
        tmem_relinquish();
    }
    // per-channel epilogue coefficients: y = acc * alpha[c] + beta[c]
    //   no batch-norm: alpha = 1, beta = bias;  batch-norm: alpha = scale / sqrt(var + eps),
    //   beta = (bias - mean) * alpha + bn_bias
    for (int c = threadIdx.x; c < p.OC; c += kThreads) {
        float a = 1.f, b = p.bias ? p.bias[c] : 0.f;
        if (p.bn_scale) {
            a = p.bn_scale[c] * rsqrtf(p.bn_var[c] + p.bn_eps);
            b = (b - p.bn_mean[c]) * a + p.bn_bias[c];
        }
        s_alpha[c] = a;
        s_beta[c] = b;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0 || warp == 6) {
        // ------------------------------------------------------------ TMA producers
        // Lane 0 of each producer warp does the work; the other lanes wait at the __syncwarp of each round
        // (a lone lane looping while its siblings sit at the CTA barrier runs several times slower).
        const int half = warp == 0 ? 0 : 1;  // which 8x8 block of every slot this warp fills
        if (warp == 0 && lane == 0) {
            // the filter, once: one box [OC x 64] per (tap, channel chunk)
            mbar_expect_tx(filter_bar, (uint32_t)p.filter_bytes);
            for (int t = 0; t < taps; t++)
                for (int kc = 0; kc < p.kchunks; kc++)
                    tma_load_3d(s_filter + (size_t)(t * p.kchunks + kc) * p.OC * 128, &tmF, filter_bar, kc * BK, t, 0);
        }
        __syncwarp();
        uint32_t issued = 0, ph = 0;
        int st = 0;
        bool ok = true;
        const int bpi = p.blocks_h * p.blocks_w;
        const uint32_t tx_bytes = (uint32_t)p.slots * (BLOCK_PIX * 128);
        for (long long tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
            const long long b = tile * 2 + half;
            const int bn = (int)(b / bpi), r = (int)(b - (long long)bn * bpi);  // bn >= N past the end: all zeros
            const int bh0 = (r / p.blocks_w) * 8 - p.pt, bw0 = (r % p.blocks_w) * 8 - p.pl;
            for (int kx = 0; kx < p.kh; kx++) {
                if (lane == 0) {
                    ok = mbar_wait(&empty[st], ph ^ 1, p.status, kWaitEmpty);
                    if (ok) {
                        mbar_expect_tx(&full[st], tx_bytes);
                        uint8_t *dst = s_a + (size_t)st * row_bytes + half * (BLOCK_PIX * 128);
                        for (int ky = 0; ky < p.kw; ky++)
                            for (int kc = 0; kc < p.kchunks; kc++, dst += A_STAGE_BYTES)
                                tma_load_4d(dst, &tmIn, &full[st], kc * BK, bw0 + ky, bh0 + kx, bn);
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                issued++;
                if (++st == p.stages) {
                    st = 0;
                    ph ^= 1;
                }
            }
        }
        // Drain: do not leave while copies may still be landing in this CTA's shared memory.  Walk back
        // over the last fill of every stage and wait for it to complete.
        if (lane == 0) {
            int s2 = st;
            uint32_t ph2 = ph;
            for (uint32_t back = 0; back < (uint32_t)p.stages && back < issued; back++) {
                if (s2 == 0) {
                    s2 = p.stages;
                    ph2 ^= 1;
                }
                s2--;
                if (!mbar_wait(&full[s2], ph2, p.status, kWaitDrain)) break;
            }
            if (warp == 0) mbar_wait(filter_bar, 0, p.status, kWaitDrain);
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (lane 0 works, the warp re-converges each round)
        const uint32_t idesc = idesc_bf16_f32(BM, p.OC);
        bool ok = true;
        if (lane == 0) ok = mbar_wait(filter_bar, 0, p.status, kWaitFull);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        tc_fence_after();
        uint32_t it = 0, ph = 0;
        int st = 0;
        // descriptors differ from slot to slot and from tap to tap only in the 14-bit address field
        const uint64_t da0 = smem_desc_sw128(smem_u32(s_a)), db0 = smem_desc_sw128(smem_u32(s_filter));
        const uint64_t b_step = (uint64_t)((p.OC * 128) >> 4);
        for (long long tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, it++) {
            const uint32_t buf = it % p.num_acc, aph = (it / p.num_acc) & 1;
            if (lane == 0) {
                ok = mbar_wait(&tmem_empty[buf], aph ^ 1, p.status, kWaitTmemEmpty);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * p.acc_stride;
                uint64_t db = db0;
                for (int kx = 0; kx < p.kh && ok; kx++) {
                    ok = mbar_wait(&full[st], ph, p.status, kWaitFull);
                    if (!ok) break;
                    tc_fence_after();
                    uint64_t da = da0 + (uint64_t)st * (uint64_t)(row_bytes >> 4);
                    for (int i = 0; i < p.slots; i++) {
                        // advancing K by 16 elements = 32 bytes inside the swizzle row: +2 in the >>4 address field
                        umma_bf16(d_tmem, da, db, idesc, (uint32_t)((kx | i) != 0));
                        umma_bf16(d_tmem, da + 2, db + 2, idesc, 1u);
                        umma_bf16(d_tmem, da + 4, db + 4, idesc, 1u);
                        umma_bf16(d_tmem, da + 6, db + 6, idesc, 1u);
                        da += A_STAGE_BYTES >> 4;
                        db += b_step;
                    }
                    umma_commit(&empty[st]);  // the row's slots are reusable once these MMAs have read them
                    if (++st == p.stages) {
                        st = 0;
                        ph ^= 1;
                    }
                }
                if (ok) umma_commit(&tmem_full[buf]);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            st = __shfl_sync(0xffffffffu, st, 0);
            ph = __shfl_sync(0xffffffffu, ph, 0);
        }
    } else {
        // ------------------------------------------------------------ epilogue: one thread per output pixel
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;          // row of the tile = TMEM lane
        const int half = row >> 6, r64 = row & 63;    // which 8x8 block, position inside it
        const int bpi = p.blocks_h * p.blocks_w;
        uint32_t it = 0;
        for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, it++) {
            const uint32_t buf = it % p.num_acc, aph = (it / p.num_acc) & 1;
            bool ok = true;
            if (lane == 0) ok = mbar_wait(&tmem_full[buf], aph, p.status, kWaitTmemFull);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            tc_fence_after();
            const long long b = tile * 2 + half;
            const int n = (int)(b / bpi), r = (int)(b - (long long)n * bpi);
            const int oh = (r / p.blocks_w) * 8 + (r64 >> 3), ow = (r % p.blocks_w) * 8 + (r64 & 7);
            const bool valid = n < p.N && oh < p.OH && ow < p.OW;
            const size_t pix = ((size_t)n * p.OH + oh) * p.OW + ow;
            for (int c0 = 0; c0 < p.OC; c0 += 32) {
                uint32_t acc[32];
                __syncwarp();
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * p.acc_stride + c0, acc);
                tmem_ld_wait();
                if (!valid) continue;
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; j++) v[j] = fmaf(__uint_as_float(acc[j]), s_alpha[c0 + j], s_beta[c0 + j]);
                if (p.residual) {
                    if (p.res_is_f32) {
                        const float4 *rp = reinterpret_cast<const float4 *>(
                            reinterpret_cast<const float *>(p.residual) + pix * p.OC + c0);
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            float4 q = __ldg(rp + j);
                            v[4 * j] += q.x;
                            v[4 * j + 1] += q.y;
                            v[4 * j + 2] += q.z;
                            v[4 * j + 3] += q.w;
                        }
                    } else {
                        const uint4 *rp = reinterpret_cast<const uint4 *>(
                            reinterpret_cast<const __nv_bfloat16 *>(p.residual) + pix * p.OC + c0);
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            uint4 q = __ldg(rp + j);
                            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                v[8 * j + 2 * e] += __uint_as_float(w[e] << 16);
                                v[8 * j + 2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
                            }
                        }
                    }
                }
                if (p.relu) {
#pragma unroll
                    for (int j = 0; j < 32; j++) v[j] = (v[j] > 0.f) ? v[j] : 0.f;
                }
                if (p.out_is_f32) {
                    float4 *op = reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.out) + pix * p.OC + c0);
#pragma unroll
                    for (int j = 0; j < 8; j++) op[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                } else {
                    uint4 *op = reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(p.out) + pix * p.OC + c0);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        uint4 o;
                        __nv_bfloat162 *h2 = reinterpret_cast<__nv_bfloat162 *>(&o);
                        h2[0] = __floats2bfloat162_rn(v[8 * j], v[8 * j + 1]);
                        h2[1] = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
                        h2[2] = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]);
                        h2[3] = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
                        op[j] = o;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[buf]);
        }
    }

    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
    }
}

}  // namespace

// input/filter bf16; output and residual bf16 or fp32
int swc_conv_tc(swcb200_ctx *ctx, void *output, int out_dtype, const void *input, const void *filt, const float *bias,
                const size_t *odims, const size_t *idims, const size_t *fdims, const size_t *kernels, const size_t *strides,
                const size_t *pads, const swcb200_conv_epilogue *ep, int res_dtype) {
    ConvParams p;
    memset(&p, 0, sizeof(p));
    p.N = (int)idims[0]; p.H = (int)idims[1]; p.W = (int)idims[2]; p.C = (int)idims[3];
    p.OH = (int)odims[1]; p.OW = (int)odims[2]; p.OC = (int)odims[3];
    p.kh = (int)kernels[0]; p.kw = (int)kernels[1]; p.pt = (int)pads[0]; p.pl = (int)pads[1];
    if (strides[0] != 1 || strides[1] != 1) return swc_fail(ctx, SWCB200_ERR_UNSUPPORTED, "conv2d_bf16: stride must be 1");
    if (p.C % 64 != 0 || p.OC % 32 != 0 || p.OC > 256 || p.OC < 32)
        return swc_fail(ctx, SWCB200_ERR_UNSUPPORTED, "conv2d_bf16: needs iC %% 64 == 0 and oC in {32, 64, ..., 256}");
    p.kchunks = p.C / 64;
    p.filter_bytes = p.kh * p.kw * p.kchunks * p.OC * 128;
    if (p.filter_bytes > kMaxFilterBytes)
        return swc_fail(ctx, SWCB200_ERR_UNSUPPORTED, "conv2d_bf16: filter (%d bytes in bf16) beyond the 96 KiB kept resident",
                        p.filter_bytes);
    SWC_REQUIRE(ctx, swc_aligned16(input) && swc_aligned16(filt) && swc_aligned16(output) &&
                         (!ep || !ep->residual || swc_aligned16(ep->residual)),
                SWCB200_ERR_MISALIGNED, "conv2d_bf16: tensors must be 16-byte aligned");
    // the output a stride-1 convolution of this input can have; rows/columns beyond it would read outside the padding
    SWC_REQUIRE(ctx, p.OH <= p.H + 2 * p.kh && p.OW <= p.W + 2 * p.kw, SWCB200_ERR_BAD_SHAPE, "conv2d_bf16: odims too large");
    p.blocks_h = (p.OH + 7) / 8;
    p.blocks_w = (p.OW + 7) / 8;
    p.num_blocks = (long long)p.N * p.blocks_h * p.blocks_w;
    p.num_tiles = (p.num_blocks + 1) / 2;
    p.acc_stride = p.OC <= 64 ? 64 : (p.OC <= 128 ? 128 : 256);
    p.num_acc = 512 / p.acc_stride < 4 ? 512 / p.acc_stride : 4;
    p.tmem_cols = p.acc_stride * p.num_acc;
    const int fixed = p.filter_bytes + 2 * p.OC * 4 + 256 + 1024;
    p.slots = p.kw * p.kchunks;
    p.stages = (kMaxSmem - fixed) / (p.slots * A_STAGE_BYTES);
    if (p.stages > 8) p.stages = 8;
    if (p.stages < 2)
        return swc_fail(ctx, SWCB200_ERR_UNSUPPORTED, "conv2d_bf16: two filter rows of operands (2 x %d KiB) do not fit beside the filter",
                        p.slots * A_STAGE_BYTES / 1024);
    p.bias = bias;
    if (ep) {
        const int nbn = (ep->bn_scale != nullptr) + (ep->bn_bias != nullptr) + (ep->bn_mean != nullptr) + (ep->bn_var != nullptr);
        SWC_REQUIRE(ctx, nbn == 0 || nbn == 4, SWCB200_ERR_BAD_ARG, "conv2d_bf16: give all four batch-norm vectors or none");
        p.bn_scale = ep->bn_scale; p.bn_bias = ep->bn_bias; p.bn_mean = ep->bn_mean; p.bn_var = ep->bn_var;
        p.bn_eps = ep->bn_eps;
        p.residual = ep->residual;
        p.relu = ep->relu;
    }
    p.out = output;
    p.out_is_f32 = out_dtype == SWCB200_F32;
    p.res_is_f32 = res_dtype == SWCB200_F32;
    p.status = ctx->dev_status;

    CUtensorMap tmIn, tmF;
    {
        uint64_t dims[4] = {(uint64_t)p.C, (uint64_t)p.W, (uint64_t)p.H, (uint64_t)p.N};
        uint64_t str[4] = {2, (uint64_t)p.C * 2, (uint64_t)p.W * p.C * 2, (uint64_t)p.H * p.W * p.C * 2};
        uint32_t box[4] = {64, 8, 8, 1};
        int rc = tc::make_tmap_bf16(ctx, &tmIn, input, 4, dims, str, box);
        if (rc) return rc;
    }
    {
        // filter [oC, kh, kw, iC] seen as {iC, tap, oC}: one box = all output channels of one tap and channel chunk
        uint64_t dims[3] = {(uint64_t)p.C, (uint64_t)(p.kh * p.kw), (uint64_t)p.OC};
        uint64_t str[3] = {2, (uint64_t)p.C * 2, (uint64_t)p.kh * p.kw * p.C * 2};
        uint32_t box[3] = {64, 1, (uint32_t)p.OC};
        int rc = tc::make_tmap_bf16(ctx, &tmF, filt, 3, dims, str, box);
        if (rc) return rc;
    }
    const size_t smem = (size_t)p.filter_bytes + (size_t)p.stages * p.slots * A_STAGE_BYTES + 2 * p.OC * 4 + 256 + 1024;
    if (!ctx->conv_attr_set) {
        SWC_CUDA(ctx, cudaFuncSetAttribute(conv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem));
        ctx->conv_attr_set = true;
    }
    unsigned grid = (unsigned)(p.num_tiles < ctx->sm_count ? p.num_tiles : ctx->sm_count);
    conv_tc_kernel<<<grid, kThreads, smem, ctx->stream>>>(tmIn, tmF, p);
    return swc_check_launch(ctx, "conv2d_bf16");
}

static int check_conv_args(swcb200_ctx *ctx, const size_t *odims, const size_t *idims, const size_t *fdims,
                           const size_t *kernels, const size_t *strides, const size_t *pads) {
    SWC_REQUIRE(ctx, odims && idims && fdims && kernels && strides && pads, SWCB200_ERR_BAD_ARG,
                "conv2d_bf16: null attribute array");
    for (int i = 0; i < 4; i++)
        SWC_REQUIRE(ctx, idims[i] <= 0x7fffffff && odims[i] <= 0x7fffffff && fdims[i] <= 0x7fffffff, SWCB200_ERR_TOO_LARGE,
                    "conv2d_bf16: dimension beyond 2^31");
    SWC_REQUIRE(ctx, odims[0] == idims[0] && odims[3] == fdims[0] && fdims[3] == idims[3] && fdims[1] == kernels[0] &&
                         fdims[2] == kernels[1],
                SWCB200_ERR_BAD_SHAPE, "conv2d_bf16: input/filter/output dims disagree");
    return SWCB200_OK;
}

SWC_EXPORT int swcb200_conv2d_bf16(swcb200_ctx *ctx, void *output, const void *input, const void *fp_bf16,
                                   const float *bias, const size_t *odims, const size_t *idims, const size_t *fdims,
                                   const size_t *kernels, const size_t *strides, const size_t *pads,
                                   const swcb200_conv_epilogue *ep) {
    SWC_CTX(ctx);
    int rc = check_conv_args(ctx, odims, idims, fdims, kernels, strides, pads);
    if (rc) return rc;
    if (odims[0] * odims[1] * odims[2] * odims[3] == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, output && input && fp_bf16, SWCB200_ERR_BAD_ARG, "conv2d_bf16: null tensor");
    return swc_conv_tc(ctx, output, SWCB200_BF16, input, fp_bf16, bias, odims, idims, fdims, kernels, strides, pads, ep,
                       SWCB200_BF16);
}

// conv2d_f with the context in tensor-core mode: input and filter are rounded to bf16 into the context's
// scratch, the result is written as fp32.  Shapes the tensor-core kernel does not take are reported as
// SWCB200_ERR_UNSUPPORTED and the caller runs the strict kernel instead.
int swc_conv_tc_from_f32(swcb200_ctx *ctx, float *output, const float *input, const float *filter, const float *bias,
                         const size_t *odims, const size_t *idims, const size_t *fdims, const size_t *kernels,
                         const size_t *strides, const size_t *pads) {
    if (strides[0] != 1 || strides[1] != 1 || idims[3] % 64 != 0 || odims[3] % 32 != 0 || odims[3] > 256 ||
        kernels[0] * kernels[1] * idims[3] * odims[3] * 2 > (size_t)kMaxFilterBytes)
        return SWCB200_ERR_UNSUPPORTED;
    const size_t n_in = idims[0] * idims[1] * idims[2] * idims[3], n_f = fdims[0] * fdims[1] * fdims[2] * fdims[3];
    const size_t in_bytes = (n_in * 2 + 255) & ~(size_t)255;
    void *scratch = nullptr;
    int rc = swc_scratch(ctx, in_bytes + n_f * 2, &scratch);
    if (rc) return rc;
    void *in16 = scratch, *f16 = (uint8_t *)scratch + in_bytes;
    rc = swcb200_cast_f32_to_bf16(ctx, input, in16, n_in);
    if (!rc) rc = swcb200_cast_f32_to_bf16(ctx, filter, f16, n_f);
    if (rc) return rc;
    return swc_conv_tc(ctx, output, SWCB200_F32, in16, f16, bias, odims, idims, fdims, kernels, strides, pads, nullptr,
                       SWCB200_F32);
}
