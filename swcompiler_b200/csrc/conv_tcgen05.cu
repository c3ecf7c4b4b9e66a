// NHWC convolution as an implicit GEMM on the 5th-generation tensor cores, with the reference's
// Conv2d -> BatchNormalization -> [ElementAdd] -> [Relu] chain folded into the epilogue
// (arithmetic of kernels.h:177-243, :496-517, :592-596, :575-580).
//
//   out[n, oh, ow, :] = epi( sum over taps (kx, ky) and channels of  in[n, oh+kx-pt, ow+ky-pl, :] . filt[:, kx, ky, :] )
//
// GEMM view: M = output pixels, N = oC, K = kh*kw*iC, bf16 operands, fp32 accumulation in tensor memory.
// A pixel's 64 channels are exactly one 128-byte swizzle row, so a TMA box of pixels is a K-major UMMA
// operand as it lands; pixels outside the image (the padding) arrive as zeros from TMA's out-of-bounds
// fill, so there is no im2col buffer.  The whole filter stays resident in shared memory for the life of
// the (persistent) CTA: kh*kw*(iC/64) slices of [oC x 64] loaded once by TMA.
//
// What bounds this kernel.  With N = oC = 64 one tcgen05.mma (128 x 64 x 16) is 32 cycles of math but
// reads 6 KiB of operands from shared memory, 48 cycles of the SM's 128 B/clk L1/shared data pipe -- and
// that pipe also carries TMA's writes, the epilogue's shared-memory traffic and every global load/store
// wavefront (one per 128-byte line touched).  The design therefore minimises data-pipe wavefronts:
//   * Halo window.  A tile is 2 output rows x 64 columns (kw-1 of the columns are scrap); its input window,
//     (kh+1) rows x 64 pixels, is loaded ONCE by one 4-D TMA box per 64-channel chunk, dense in shared
//     memory at 128 bytes per pixel.  The A operand of tap (kx, ky) is the same buffer read from a start
//     address (kx*64 + ky) pixels further on: the 128-byte swizzle is a function of the absolute
//     shared-memory address for TMA and for the MMA alike, so a descriptor whose start is shifted by whole
//     128-byte rows reads rows r+shift of the buffer (checked on the hardware with an identity-matrix
//     product for shifts 0..17).  Columns whose window runs into the next row compute scrap that is not
//     stored.  Per tile 32 KiB of TMA writes instead of one 16 KiB operand per tap, and one barrier
//     hand-over per tile.
//   * Staged epilogue (bf16 output, oC a multiple of 64).  An epilogue thread owns one pixel, and pixels
//     are 128 bytes apart in global memory, so direct 16-byte stores touch 32 lines per instruction.
//     Instead the tile is written to shared memory in the swizzled layout of a TMA box {64 ch, cw, 2, 1}
//     (4 wavefronts per instruction) and leaves with one TMA store per 64 channels; TMA clips rows and
//     columns outside the image.  A bf16 residual arrives the same way, by a TMA load issued by the producer.
//     Other outputs (fp32, oC not a multiple of 64) are stored directly.
//   * Per-channel epilogue coefficients are read from shared memory as 128-bit broadcasts.
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 epilogue (two warps per tensor-memory
// lane quarter, 32 channels each per pass).  The producer and issuer loops run warp-uniform with one
// elected lane executing the asynchronous instructions: a loop run by a lone lane under a divergent
// branch issues tcgen05.mma at 75 cycles apiece on this part, the uniform form at the 48 cycles the
// shared-memory reads allow.
//
// A CTA-pair form (cta_group::2, M = 256, half the filter per CTA: 5 KiB of operand reads per MMA instead of 6) was
// built and measured: correct, but a cta_group::2 MMA does not issue faster than about every 155 cycles whatever its
// N, so at N = 64 the pair ran the layer in 91 us against 65 us for this kernel.  It pays from N = 256 up, which is
// where the FC kernel uses it.
//
// A fused-row form was built and measured too: the three taps of a filter row share their window rows, so one MMA
// with N = 3 * oC = 192 over the row's three (contiguous) filter slices replaces three N = 64 MMAs -- 12 MMAs of 96
// cycles per tile instead of 36 of 48 -- and the epilogue adds the three column blocks shifted by one and two pixels
// with warp shuffles (tiles of 4 rows x 32 window columns, so that a warp is one row).  Correct, but 69.5 us against
// 62.6 us on the same run: the epilogue then reads three times the tensor memory and shuffles 128 values per thread
// and tile, and even with its arithmetic switched off the kernel took 53.7 us (58 us for this kernel in that state).
//
// The 3 x 3 convolution over 64 -> 64 channels with an even number of rows -- the shape where the operand reads
// bind hardest -- has a form of its own that halves the pixel reads of two thirds of its MMAs (row-interleaved
// tiles, conv_rows_tcgen05.cu); swc_conv_tc tries it first.
//
// Restrictions: stride 1, group 1, iC a multiple of 64, oC a multiple of 32 and <= 256, kw <= 9, filter at
// most 96 KiB in bf16, two windows fitting beside it.  Other shapes return SWCB200_ERR_UNSUPPORTED (the
// strict kernel takes them).

#include "conv_common.cuh"

namespace {

using namespace tc;

constexpr int BM = 128, BK = 64;
constexpr int kThreads = 384;            // window producer, two MMA issuers, residual producer, 8 epilogue warps
constexpr int kIssuers = 2;
constexpr int kResidualWarp = 3;
constexpr int kFirstEpilogueWarp = 4;
constexpr int kEpilogueGroups = 2;        // each of four warps (one per tensor-memory lane quarter)
constexpr int kEpilogueGroupThreads = 128;
constexpr int kMaxFilterBytes = 96 * 1024;
constexpr int kMaxGroups = kMaxFilterBytes / (32 * 128);  // filter slices of [oC x 64] bf16 at the smallest oC (32)
constexpr int kMaxSmem = 227 * 1024;

struct ConvParams {
    int N, H, W, C, OH, OW, OC, kh, kw, pt, pl;
    int kchunks;            // C / 64
    long long num_tiles;
    int stages, acc_stride, num_acc, tmem_cols;
    int filter_bytes;
    // tile = 2 output rows x 64 columns of which `cw` are stored; window = `hr` input rows x 64 pixels
    int hr, cw, col_blocks, row_blocks, chunk_bytes, stage_bytes;
    int out_tma, res_tma;   // staged epilogue / residual brought in by TMA
    int bw;                 // columns of a staged tile: min(cw, OW)
    int out_chunk_bytes;    // staging slot of one 64-channel chunk of a tile: 2 x bw pixels x 128 B, rounded up to 1 KiB
    int out_tile_bytes;     // (OC / 64) * out_chunk_bytes
    // MMA groups of a tile (one per filter tap and 64-channel chunk, 4 MMAs each), in filter-slice order:
    // a_off[g] = offset of the group's A operand inside a window, in 16-byte descriptor address units
    int groups;
    uint32_t a_off[kMaxGroups];
    const float *bias;
    const float *bn_scale, *bn_bias, *bn_mean, *bn_var;
    float bn_eps;
    const void *residual;
    int relu;
    void *out;
    int out_is_f32, res_is_f32;
    int *status;
};

// v[j] = acc[j] * alpha[c0+j] + beta[c0+j], coefficients read as 128-bit broadcasts
__device__ __forceinline__ void apply_affine(const uint32_t (&acc)[32], const float *s_alpha, const float *s_beta, int c0,
                                             float (&v)[32]) {
    const float4 *a4 = reinterpret_cast<const float4 *>(s_alpha + c0), *b4 = reinterpret_cast<const float4 *>(s_beta + c0);
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const float4 a = a4[j], b = b4[j];
        v[4 * j] = fmaf(__uint_as_float(acc[4 * j]), a.x, b.x);
        v[4 * j + 1] = fmaf(__uint_as_float(acc[4 * j + 1]), a.y, b.y);
        v[4 * j + 2] = fmaf(__uint_as_float(acc[4 * j + 2]), a.z, b.z);
        v[4 * j + 3] = fmaf(__uint_as_float(acc[4 * j + 3]), a.w, b.w);
    }
}
// residual of channels [c0, c0+32) of pixel `pix`, read from global memory
__device__ __forceinline__ void add_residual_global(const ConvParams &p, float (&v)[32], size_t pix, int c0) {
    if (p.res_is_f32) {
        const float4 *rp = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.residual) + pix * p.OC + c0);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float4 q = __ldg(rp + j);
            v[4 * j] += q.x;
            v[4 * j + 1] += q.y;
            v[4 * j + 2] += q.z;
            v[4 * j + 3] += q.w;
        }
    } else {
        const uint4 *rp = reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(p.residual) + pix * p.OC + c0);
#pragma unroll
        for (int j = 0; j < 4; j++) add_bf16x8(v + 8 * j, __ldg(rp + j));
    }
}
__device__ __forceinline__ void store_global(const ConvParams &p, const float (&v)[32], size_t pix, int c0) {
    if (p.out_is_f32) {
        float4 *op = reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.out) + pix * p.OC + c0);
#pragma unroll
        for (int j = 0; j < 8; j++) op[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
        uint4 *op = reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(p.out) + pix * p.OC + c0);
#pragma unroll
        for (int j = 0; j < 4; j++) op[j] = pack_bf16x8(v + 8 * j);
    }
}

// The MMA sequence of one tile with every descriptor offset a compile-time constant: tap (kx, ky), channel chunk kc
// and the four K = 16 steps of a 64-channel chunk.  The tensor pipe takes a new N = 64 MMA every 48 cycles and runs
// at most about one instruction ahead of the issuing thread, so anything that thread computes between two
// tcgen05.mma (a table look-up, a division) lengthens the tile.
template <int KH, int KW, int KC>
__device__ __forceinline__ void issue_tile_unrolled(uint32_t d_tmem, uint32_t a_win, uint32_t b0, uint32_t b_step, uint32_t desc_hi,
                                                    uint32_t idesc, bool leader) {
    constexpr uint32_t chunk_step = (uint32_t)((KH + 1) * ROW_PIX * 128) >> 4;
    if (leader) {
#pragma unroll
        for (int kx = 0; kx < KH; kx++)
#pragma unroll
            for (int ky = 0; ky < KW; ky++)
#pragma unroll
                for (int kc = 0; kc < KC; kc++) {
                    const uint32_t g = (uint32_t)((kx * KW + ky) * KC + kc);
                    const uint32_t a = a_win + (uint32_t)((kx * ROW_PIX + ky) * 8) + (uint32_t)kc * chunk_step;
                    const uint32_t b = b0 + g * b_step;
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        umma_bf16(d_tmem, ((uint64_t)desc_hi << 32) | (a + 2 * k), ((uint64_t)desc_hi << 32) | (b + 2 * k), idesc,
                                  (uint32_t)((g | (uint32_t)k) != 0));
                }
    }
    __syncwarp();
}

__global__ void __launch_bounds__(kThreads, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap tmIn, const __grid_constant__ CUtensorMap tmF,
               const __grid_constant__ CUtensorMap tmOut, const __grid_constant__ CUtensorMap tmRes, const ConvParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *s_filter = smem;                                   // [taps*kchunks][OC x 128 B]
    uint8_t *s_a = smem + p.filter_bytes;                       // stages x kchunks x (hr x 64 pixels x 128 B)
    // 1 KiB of slack after the last window: the scrap columns of the last tap read kw-1 pixels past it
    // windows, then (staged epilogue) 2 x out_tile_bytes, or 1 KiB of slack where there is no staging
    uint8_t *s_out = s_a + (size_t)p.stages * p.stage_bytes + (p.out_tma ? 0 : 1024);
    uint8_t *s_res = s_out + (p.out_tma ? 2 * p.out_tile_bytes : 0);            // 2 x out_tile_bytes (TMA residual)
    float *s_alpha = reinterpret_cast<float *>(s_res + (p.res_tma ? 2 * p.out_tile_bytes : 0));  // [OC]
    float *s_beta = s_alpha + p.OC;                             // [OC]
    uint64_t *full = reinterpret_cast<uint64_t *>(s_beta + p.OC);
    uint64_t *empty = full + 8;
    uint64_t *tmem_full = empty + 8;
    uint64_t *tmem_empty = tmem_full + 4;
    uint64_t *filter_bar = tmem_empty + 4;
    uint64_t *res_full = filter_bar + 1;
    uint64_t *res_empty = res_full + 2;
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(res_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int taps = p.kh * p.kw;
    const int ochunks = p.OC >> 6;  // 64-channel chunks of the output (staged epilogue only)

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmIn);
        tma_prefetch_desc(&tmF);
        if (p.out_tma) tma_prefetch_desc(&tmOut);
        if (p.res_tma) tma_prefetch_desc(&tmRes);
        for (int s = 0; s < p.stages; s++) {
            mbar_init(&full[s], 1);   // the producer's arrive(+expect-tx)
            mbar_init(&empty[s], 1);  // one tcgen05.commit
        }
        for (int b = 0; b < p.num_acc; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], 4);  // one arrival per warp of the epilogue group that reads it
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&res_full[b], 1);   // the residual tile has landed in residual buffer b
            mbar_init(&res_empty[b], 4);  // one arrival per warp of the epilogue group that read it
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

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (warp-uniform loop, one elected lane issues)
        const bool leader = elect_one();
        if (leader) {
            // the filter, once: one box [OC x 64] per (tap, channel chunk)
            mbar_expect_tx(filter_bar, (uint32_t)p.filter_bytes);
            for (int t = 0; t < taps; t++)
                for (int kc = 0; kc < p.kchunks; kc++)
                    tma_load_3d(s_filter + (size_t)(t * p.kchunks + kc) * p.OC * 128, &tmF, filter_bar, kc * BK, t, 0);
        }
        __syncwarp();
        uint32_t issued = 0, ph = 0;
        int st = 0;
        TileWalk tw(blockIdx.x, gridDim.x, p.row_blocks, p.col_blocks);
        for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, tw.advance()) {
            const int n = tw.n, oh0 = tw.rb * 2, ow0 = tw.cb * p.cw;
            bool ok = mbar_wait(&empty[st], ph ^ 1, p.status, kWaitEmpty);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (leader) {
                mbar_expect_tx(&full[st], (uint32_t)p.stage_bytes);
                uint8_t *dst = s_a + (size_t)st * p.stage_bytes;
                for (int kc = 0; kc < p.kchunks; kc++, dst += p.chunk_bytes)
                    tma_load_4d(dst, &tmIn, &full[st], kc * BK, ow0 - p.pl, oh0 - p.pt, n);  // outside the image: zeros
            }
            __syncwarp();
            issued++;
            if (++st == p.stages) {
                st = 0;
                ph ^= 1;
            }
        }
        // Drain: do not leave while copies may still be landing in this CTA's shared memory.  Walk back
        // over the last fill of every stage (and of both residual buffers) and wait for it to complete.
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
            mbar_wait(filter_bar, 0, p.status, kWaitDrain);
        }
        __syncwarp();
    } else if (warp == kResidualWarp) {
        // ------------------------------------------------------------ residual producer (only with a bf16 residual)
        // A warp of its own, so that the input windows can run ahead of the epilogue by every free stage while the
        // residual of a tile waits for its staging buffer (the one the epilogue of two tiles back is still reading).
        if (p.res_tma) {
            const bool leader = elect_one();
            const uint32_t res_box_bytes = (uint32_t)(p.bw * 2 * 128);
            uint32_t issued = 0;
            TileWalk tw(blockIdx.x, gridDim.x, p.row_blocks, p.col_blocks);
            for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, tw.advance()) {
                const int n = tw.n, oh0 = tw.rb * 2, ow0 = tw.cb * p.cw;
                const uint32_t b = issued & 1, rph = (issued >> 1) & 1;
                bool ok = mbar_wait(&res_empty[b], rph ^ 1, p.status, kWaitEmpty);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (leader) {
                    // in the layout the epilogue stages its output in
                    mbar_expect_tx(&res_full[b], res_box_bytes * (uint32_t)ochunks);
                    for (int oc = 0; oc < ochunks; oc++)
                        tma_load_4d(s_res + (size_t)b * p.out_tile_bytes + (size_t)oc * p.out_chunk_bytes, &tmRes, &res_full[b],
                                    oc * 64, ow0, oh0, n);
                }
                __syncwarp();
                issued++;
            }
            // drain: the last fill of both buffers must have landed before the CTA may leave
            if (lane == 0)
                for (uint32_t back = 0; back < 2 && back < issued; back++) {
                    const uint32_t i = issued - 1 - back;
                    if (!mbar_wait(&res_full[i & 1], (i >> 1) & 1, p.status, kWaitDrain)) break;
                }
            __syncwarp();
        }
    } else if (warp <= kIssuers) {
        // ------------------------------------------------------------ MMA issuers (warp-uniform loops, one elected lane issues)
        // Two warps, each issuing the MMAs of every other tile into its own accumulators.  A tcgen05.mma holds
        // the issuing thread while the pipe takes its operands, and what that thread executes between two of
        // them (descriptor arithmetic, the moves into uniform registers) is not overlapped: a single issuer
        // runs the pipe at 67 cycles per N = 64 MMA against the 48 its shared-memory reads take.  With a second
        // warp the pipe takes one warp's MMA while the other prepares its next.
        const uint32_t iw = (uint32_t)(warp - 1);
        const bool leader = elect_one();
        const uint32_t idesc = idesc_bf16_f32(BM, p.OC);
        bool ok = mbar_wait(filter_bar, 0, p.status, kWaitFull);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        uint32_t it = iw, ph = (iw / (uint32_t)p.stages) & 1;
        int st = (int)(iw % (uint32_t)p.stages);
        uint32_t buf = iw % (uint32_t)p.num_acc, aph = (iw / (uint32_t)p.num_acc) & 1;
        // Descriptors differ from window to window and from tap to tap only in the 14-bit address field, the low
        // bits of the low word (no carry leaves the field: shared-memory addresses stay below 256 KiB).
        const uint64_t da0 = smem_desc_sw128(smem_u32(s_a)), db0 = smem_desc_sw128(smem_u32(s_filter));
        const uint32_t desc_hi = (uint32_t)(da0 >> 32);  // same for A and B: stride 1024 B, version, 128-byte swizzle
        const uint32_t a_lo0 = (uint32_t)da0, b_lo0 = (uint32_t)db0;
        const uint32_t b_step = (uint32_t)((p.OC * 128) >> 4), stage_step = (uint32_t)(p.stage_bytes >> 4);
        auto desc = [desc_hi](uint32_t lo) { return ((uint64_t)desc_hi << 32) | lo; };
        for (long long tile = blockIdx.x + (long long)iw * gridDim.x; tile < p.num_tiles && ok;
             tile += (long long)kIssuers * gridDim.x, it += kIssuers) {
            ok = mbar_wait(&tmem_empty[buf], aph ^ 1, p.status, kWaitTmemEmpty);
            if (ok) ok = mbar_wait(&full[st], ph, p.status, kWaitFull);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * p.acc_stride;
            if (p.kh == 3 && p.kw == 3 && p.kchunks == 1) {
                issue_tile_unrolled<3, 3, 1>(d_tmem, a_lo0 + (uint32_t)st * stage_step, b_lo0, b_step, desc_hi, idesc, leader);
            } else {
                const uint32_t a_win = a_lo0 + (uint32_t)st * stage_step;
                uint32_t b = b_lo0, a = a_win + p.a_off[0];
                for (int g = 0; g < p.groups; g++, b += b_step) {
                    // group g: tap (kx, ky) and channel chunk kc; its A operand is the window read from (kx*64 + ky)
                    // pixels further on.  Advancing K by 16 elements = 32 bytes inside the swizzle row: +2 in the field.
                    // The next group's offset is fetched before this group's MMAs are issued.
                    const uint32_t a_next = a_win + p.a_off[g + 1 < p.groups ? g + 1 : g];
                    if (leader) {
                        umma_bf16(d_tmem, desc(a), desc(b), idesc, (uint32_t)(g != 0));
                        umma_bf16(d_tmem, desc(a + 2), desc(b + 2), idesc, 1u);
                        umma_bf16(d_tmem, desc(a + 4), desc(b + 4), idesc, 1u);
                        umma_bf16(d_tmem, desc(a + 6), desc(b + 6), idesc, 1u);
                    }
                    a = a_next;
                }
            }
            if (leader) {
                umma_commit(&empty[st]);       // the window is reusable once these MMAs have read it
                umma_commit(&tmem_full[buf]);  // and the accumulator is complete
            }
            __syncwarp();
            // this warp's next tile is kIssuers further on (stages >= 2 and num_acc >= 2, so one wrap at most)
            st += kIssuers;
            if (st >= p.stages) {
                st -= p.stages;
                ph ^= 1;
            }
            buf += kIssuers;
            if (buf >= (uint32_t)p.num_acc) {
                buf -= (uint32_t)p.num_acc;
                aph ^= 1;
            }
        }
    } else if (warp >= kFirstEpilogueWarp) {
        // ------------------------------------------------------------ epilogue: two groups of four warps, alternate tiles
        // A thread owns one output pixel (one tensor-memory lane) and walks its channels 64 at a time.  One tile's
        // epilogue is a chain of latencies (accumulator ready -> tcgen05.ld -> arithmetic -> staging -> TMA store)
        // about as long as the tile's MMAs, so two tiles are kept in flight: group g takes every other tile, with
        // its own staging buffer, named barrier and bulk-store queue.  The accumulator is handed back as soon as
        // the last tcgen05.ld has returned, before the arithmetic.
        const int group = (warp - kFirstEpilogueWarp) >> 2;
        const int quarter = warp & 3;                 // the tensor-memory lane quarter this warp may read
        const int row = quarter * 32 + lane;          // row of the tile = TMEM lane
        const int trow = row >> 6, tcol = row & 63;   // position inside the 2 x 64 tile
        const int q = trow * p.bw + tcol;             // pixel's row in the staged tile (box {64 ch, bw, 2, 1})
        const uint32_t swz = (uint32_t)(q & 7);       // 128-byte swizzle: 16-byte chunk index ^ (row & 7)
        const bool issuer = ((warp - kFirstEpilogueWarp) & 3) == 0 && lane == 0;  // issues the group's TMA stores
        const int bar_id = 1 + group;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        uint8_t *const so_tile = s_out + (size_t)group * p.out_tile_bytes;
        const uint8_t *const sr_tile = s_res + (size_t)group * p.out_tile_bytes;
        uint32_t buf = (uint32_t)group % (uint32_t)p.num_acc, aph = ((uint32_t)group / (uint32_t)p.num_acc) & 1, sph = 0;
        TileWalk tw(blockIdx.x + (long long)group * gridDim.x, (long long)kEpilogueGroups * gridDim.x, p.row_blocks, p.col_blocks);
        for (long long tile = blockIdx.x + (long long)group * gridDim.x; tile < p.num_tiles;
             tile += (long long)kEpilogueGroups * gridDim.x, tw.advance()) {
            const int n = tw.n, oh0 = tw.rb * 2, ow0 = tw.cb * p.cw;
            const int oh = oh0 + trow, ow = ow0 + tcol;
            const bool valid = tcol < p.cw && oh < p.OH && ow < p.OW;
            const bool skip = p.out_tma ? tcol >= p.bw : !valid;  // staged tiles are clipped by the TMA store
            const size_t pix = ((size_t)n * p.OH + oh) * p.OW + ow;
            bool ok = true;
            if (p.out_tma) {
                // the group's previous store must have finished reading the staging buffer before anyone refills it
                if (issuer) bulk_wait_read_all();
                named_barrier(bar_id, kEpilogueGroupThreads);
            }
            if (lane == 0) {
                ok = mbar_wait(&tmem_full[buf], aph, p.status, kWaitTmemFull);
                if (ok && p.res_tma) ok = mbar_wait(&res_full[group], sph, p.status, kWaitFull);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            tc_fence_after();

            // one 32-channel pass: affine, residual, ReLU, then staging (or a direct store)
            auto pass = [&](const uint32_t (&acc)[32], int c0) {
                if (skip) return;
                float v[32];
                apply_affine(acc, s_alpha, s_beta, c0, v);
                // this pass's 64 bytes of the pixel's 128-byte row in a staged 64-channel chunk: 16-byte chunks ch16 .. ch16+3
                const uint32_t row_off = (uint32_t)(c0 >> 6) * p.out_chunk_bytes + (uint32_t)q * 128u;
                const uint32_t ch16 = (uint32_t)(c0 & 63) >> 3;
                if (p.residual) {
                    if (p.res_tma) {
                        const uint8_t *rr = sr_tile + row_off;
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            add_bf16x8(v + 8 * j, *reinterpret_cast<const uint4 *>(rr + (((ch16 + j) ^ swz) << 4)));
                    } else if (valid) {
                        add_residual_global(p, v, pix, c0);
                    }
                }
                if (p.relu) {
#pragma unroll
                    for (int j = 0; j < 32; j++) v[j] = fmaxf(v[j], 0.f);
                }
                if (p.out_tma) {
                    uint8_t *so = so_tile + row_off;
#pragma unroll
                    for (int j = 0; j < 4; j++) *reinterpret_cast<uint4 *>(so + (((ch16 + j) ^ swz) << 4)) = pack_bf16x8(v + 8 * j);
                } else {
                    store_global(p, v, pix, c0);
                }
            };
            const uint32_t acc_base = lane_base + buf * p.acc_stride;
            for (int c0 = 0; c0 < p.OC; c0 += 64) {
                uint32_t acc0[32], acc1[32];
                const bool two = c0 + 32 < p.OC;  // warp-uniform
                __syncwarp();
                tmem_ld_32x32(acc_base + c0, acc0);
                if (two) tmem_ld_32x32(acc_base + c0 + 32, acc1);
                tmem_ld_wait();
                if (c0 + 64 >= p.OC) {
                    // every column of the accumulator is in registers: the MMA issuer may have it back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&tmem_empty[buf]);
                }
                pass(acc0, c0);
                if (two) pass(acc1, c0 + 32);
            }
            __syncwarp();
            if (p.res_tma && lane == 0) mbar_arrive(&res_empty[group]);
            if (p.out_tma) {
                // the staged tile leaves by TMA once the whole group has written its part
                fence_proxy_async();
                named_barrier(bar_id, kEpilogueGroupThreads);
                if (issuer) {
                    for (int oc = 0; oc < ochunks; oc++) tma_store_4d(&tmOut, so_tile + (size_t)oc * p.out_chunk_bytes, oc * 64, ow0, oh0, n);
                    bulk_commit_group();
                }
            }
            buf += kEpilogueGroups;
            if (buf >= (uint32_t)p.num_acc) {
                buf -= (uint32_t)p.num_acc;
                aph ^= 1;
            }
            sph ^= 1;
        }
        if (p.out_tma && issuer) bulk_wait_all();  // shared memory stays valid until the last store has read it
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
int swc_conv_tc_rows(swcb200_ctx *ctx, void *output, const void *input, const void *filt, const float *bias, const size_t *odims,
                     const size_t *idims, const size_t *kernels, const size_t *pads, const swcb200_conv_epilogue *ep);

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
    if (p.kw > 9) return swc_fail(ctx, SWCB200_ERR_UNSUPPORTED, "conv2d_bf16: filter wider than 9");
    SWC_REQUIRE(ctx, swc_aligned16(input) && swc_aligned16(filt) && swc_aligned16(output) &&
                         (!ep || !ep->residual || swc_aligned16(ep->residual)),
                SWCB200_ERR_MISALIGNED, "conv2d_bf16: tensors must be 16-byte aligned");
    SWC_REQUIRE(ctx, p.OH <= p.H + 2 * p.kh && p.OW <= p.W + 2 * p.kw, SWCB200_ERR_BAD_SHAPE, "conv2d_bf16: odims too large");
    if (out_dtype == SWCB200_BF16 && (!ep || !ep->residual || res_dtype == SWCB200_BF16)) {
        // the row-interleaved form of the 3 x 3, 64 -> 64 channel convolution (conv_rows_tcgen05.cu)
        const int rc = swc_conv_tc_rows(ctx, output, input, filt, bias, odims, idims, kernels, pads, ep);
        if (rc != SWCB200_ERR_UNSUPPORTED) return rc;
    }
    if (ep && ep->pool2x2)
        return swc_fail(ctx, SWCB200_ERR_UNSUPPORTED,
                        "conv2d_bf16: the fused 2x2 max-pool needs a 3x3 filter over 64 -> 64 channels, bf16 tensors and even H, OH, OW");
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
    p.acc_stride = p.OC <= 64 ? 64 : (p.OC <= 128 ? 128 : 256);
    p.num_acc = 512 / p.acc_stride < 4 ? 512 / p.acc_stride : 4;
    p.tmem_cols = p.acc_stride * p.num_acc;
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

    // shared-memory plan: filter | windows | output staging, residual staging (or 1 KiB slack) | coefficients | barriers
    p.hr = p.kh + 1;
    p.cw = ROW_PIX - (p.kw - 1);
    p.chunk_bytes = p.hr * ROW_PIX * 128;
    p.stage_bytes = p.chunk_bytes * p.kchunks;
    p.bw = p.OW < p.cw ? p.OW : p.cw;
    p.out_chunk_bytes = (2 * p.bw * 128 + 1023) & ~1023;  // 1 KiB granules keep every chunk on a swizzle-pattern boundary
    p.out_tile_bytes = (p.OC / 64) * p.out_chunk_bytes;
    const int fixed = p.filter_bytes + 2 * p.OC * 4 + 256 + 1024;  // filter, coefficients, barriers, alignment of the base
    p.out_tma = !p.out_is_f32 && p.OC % 64 == 0;
    p.res_tma = p.out_tma && p.residual != nullptr && !p.res_is_f32;
    // the 1 KiB of slack after the windows (scrap columns of the last tap read up to kw-1 pixels past them) is only
    // needed where no staging buffer follows
    auto smem_for = [&](int stages, int out_tma, int res_tma) {
        return fixed + stages * p.stage_bytes + (out_tma ? 2 * p.out_tile_bytes : 1024) + (res_tma ? 2 * p.out_tile_bytes : 0);
    };
    auto stages_for = [&](int out_tma, int res_tma) { return (kMaxSmem - smem_for(0, out_tma, res_tma)) / p.stage_bytes; };
    if (stages_for(p.out_tma, p.res_tma) < 2) p.res_tma = 0;
    if (stages_for(p.out_tma, p.res_tma) < 2) p.out_tma = 0;
    p.stages = stages_for(p.out_tma, p.res_tma);
    if (p.stages > 8) p.stages = 8;
    if (p.stages < 2)
        return swc_fail(ctx, SWCB200_ERR_UNSUPPORTED, "conv2d_bf16: two input windows (2 x %d KiB) do not fit beside the filter",
                        p.stage_bytes / 1024);
    p.row_blocks = (p.OH + 1) / 2;
    p.col_blocks = (p.OW + p.cw - 1) / p.cw;
    p.num_tiles = (long long)p.N * p.row_blocks * p.col_blocks;
    p.groups = p.kh * p.kw * p.kchunks;  // <= kMaxGroups: the filter fits in kMaxFilterBytes and oC >= 32
    SWC_REQUIRE(ctx, p.groups <= kMaxGroups, SWCB200_ERR_UNSUPPORTED, "conv2d_bf16: %d filter slices", p.groups);
    for (int kx = 0, g = 0; kx < p.kh; kx++)
        for (int ky = 0; ky < p.kw; ky++)
            for (int kc = 0; kc < p.kchunks; kc++, g++)
                p.a_off[g] = (uint32_t)(((kx * ROW_PIX + ky) * 128 + kc * p.chunk_bytes) >> 4);

    CUtensorMap tmIn, tmF, tmOut, tmRes;
    {
        uint64_t dims[4] = {(uint64_t)p.C, (uint64_t)p.W, (uint64_t)p.H, (uint64_t)p.N};
        uint64_t str[4] = {2, (uint64_t)p.C * 2, (uint64_t)p.W * p.C * 2, (uint64_t)p.H * p.W * p.C * 2};
        uint32_t box[4] = {64, (uint32_t)ROW_PIX, (uint32_t)p.hr, 1};
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
    tmOut = tmIn;
    tmRes = tmIn;
    if (p.out_tma) {
        // output (and residual) seen tile by tile: 64 channels x cw columns x 2 rows
        uint64_t dims[4] = {(uint64_t)p.OC, (uint64_t)p.OW, (uint64_t)p.OH, (uint64_t)p.N};
        uint64_t str[4] = {2, (uint64_t)p.OC * 2, (uint64_t)p.OW * p.OC * 2, (uint64_t)p.OH * p.OW * p.OC * 2};
        uint32_t box[4] = {64, (uint32_t)p.bw, 2, 1};
        int rc = tc::make_tmap_bf16(ctx, &tmOut, output, 4, dims, str, box);
        if (rc) return rc;
        if (p.res_tma) {
            rc = tc::make_tmap_bf16(ctx, &tmRes, p.residual, 4, dims, str, box);
            if (rc) return rc;
        }
    }
    static bool attr_set[64] = {false};  // per device: the opt-in to large dynamic shared memory
    if (!attr_set[ctx->device & 63]) {
        SWC_CUDA(ctx, cudaFuncSetAttribute(conv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem));
        attr_set[ctx->device & 63] = true;
    }
    const size_t smem = (size_t)smem_for(p.stages, p.out_tma, p.res_tma);
    unsigned grid = (unsigned)(p.num_tiles < swc_tc_sms(ctx) ? p.num_tiles : swc_tc_sms(ctx));
    conv_tc_kernel<<<grid, kThreads, smem, ctx->stream>>>(tmIn, tmF, tmOut, tmRes, p);
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
