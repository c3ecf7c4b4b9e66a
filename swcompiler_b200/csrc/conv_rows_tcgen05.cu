// 3 x 3 convolution over 64 -> 64 channels (NHWC, stride 1, bf16 in and out) on the 5th-generation tensor
// cores: the row-interleaved form of the implicit GEMM in conv_tcgen05.cu, for the one shape where that
// kernel is bound by shared-memory operand reads (a ResNet-style stage at 56 x 56).
//
// Why a second form.  With N = oC = 64 one tcgen05.mma (128 pixels x 64 channels x K 16) is 32 cycles of math
// but reads 4 KiB of pixels and 2 KiB of filter from shared memory, 48 cycles of the 128 B/clk operand path.
// Here a tile is FOUR output rows held in two accumulators: D0 = rows {0, 2} (tensor-memory columns 0..63)
// and D1 = rows {1, 3} (columns 64..127).  Count input rows i from the tile's first one.  The window rows
// {i, i+2} are what D0 needs for filter row i and what D1 needs for filter row i-1.  For i = 1 and i = 2 ONE
// MMA with N = 128 serves both accumulators: its A operand is the window rows {i, i+2} (shifted by the filter
// column ky), its B operand the two filter slices [W(i, ky); W(i-1, ky)], which lie next to each other
// because the producer stores a filter column's slices in descending row order.  Such an MMA reads 8 KiB for
// 64 cycles of math, so the operand path no longer limits it.  The rows {0, 2} and {3, 5} serve one
// accumulator each (N = 64).  Per tile and filter column: 2 x 64 + 2 x 48 cycles for work that is 6 x 32
// cycles of math (0.86), against 6 x 48 (0.67) with one accumulator per tile.
//
// Shared memory (227 KiB): the filter (72 KiB, resident) | four half-windows of 24 KiB | four output half
// buffers of 14 KiB | epilogue coefficients | barriers.
//   * A half-window is three input rows of one parity (rows 1, 3, 5 or 0, 2, 4 of the tile's six), 64 pixels
//     each, so that the rows {i, i+2} are adjacent in shared memory: 128 consecutive 128-byte swizzle rows, a
//     K-major UMMA operand as TMA writes them.  The input's rows are split into (row / 2, row % 2) in a 5-D
//     tensor map, so three rows of one parity are one box; rows outside the image arrive as zeros.
//     The filter column shift ky is a descriptor start address ky pixels further on (the 128-byte swizzle is a
//     function of the absolute shared-memory address for TMA and MMA alike); the columns whose window runs
//     into the next row compute scrap that is never stored.
//   * The odd half-window is multiplied first, so that one MMA (i = 1) starts both accumulators, and is
//     handed back to the producer as soon as its MMAs are queued.
//   * An output half buffer takes the two rows of one accumulator ({64 ch, bw, parity, 2 rows} of the
//     parity-split output map).  It goes round a ring of four: ready -> the epilogue adds the residual that is
//     already there, applies batch-norm and ReLU and writes the result in place -> staged -> stored by TMA ->
//     once the store has read it, the residual of the step four further on is loaded into it.
// Warp roles (640 threads): warp 0 window producer, warps 1-2 MMA issuers (alternate tiles, own
// accumulators: a tcgen05.mma holds its issuing thread while the pipe takes the operands), warp 3 output
// staging (TMA stores, residual loads), warps 4-19 epilogue.  An epilogue warp owns one tensor-memory lane
// quarter (32 pixels) and 16 of the 64 channels, with its batch-norm coefficients in registers: sixteen
// short instruction streams per tile instead of four long ones, because a lone warp issues its (dependent)
// epilogue arithmetic at one instruction every five cycles or so and four of them could not keep up with
// the tensor pipe.
//
// Taken by swc_conv_tc for kh = kw = 3, iC = oC = 64, bf16 output, H and OH even, OH >= 4, and a residual
// that is absent or bf16.
#include "conv_common.cuh"

namespace {

using namespace tc;

constexpr int kRowsThreads = 640;
constexpr int kEpilogueWarps = 16, kFirstEpilogueWarp = 4, kStagingWarp = 3;
constexpr int kSlots = 4;                              // half-windows in flight (two tiles, one per issuing warp)
constexpr int kSlotBytes = 3 * ROW_PIX * 128;          // three rows of 64 pixels
constexpr int kFilterBytes = 9 * 64 * 128;             // nine [64 x 64] slices
constexpr int kHalves = 4, kAccs = 4, kAccCols = 128;  // output half buffers; accumulator pairs in tensor memory
constexpr int kTileCols = 56;                          // output columns of a tile (a window row holds 64 pixels)
constexpr int kMaxSmem = 227 * 1024;

struct RowsParams {
    int N, H, W, OH, OW, pt, pl;
    int bw;                  // columns of a staged tile: min(kTileCols, OW)
    int half_bytes;          // 2 x bw pixels x 128 B, in 1 KiB granules (a swizzle-pattern boundary)
    int row_blocks, col_blocks;
    long long num_tiles;
    const float *bias;
    const float *bn_scale, *bn_bias, *bn_mean, *bn_var;
    float bn_eps;
    int has_res, relu;
    int pool;                // the 2x2 / 2 max-pool of the result is what is stored, straight from registers
    void *pool_out;          // [N, OH/2, OW/2, 64] bf16
    int *status;
};

// The MMAs of one half-window, every descriptor offset a compile-time constant.  HALF 0 is the odd half-window
// (tile input rows 1, 3, 5), HALF 1 the even one (rows 0, 2, 4).
template <int HALF>
__device__ __forceinline__ void issue_half(uint32_t d_tmem, uint32_t a_half, uint32_t b0, uint32_t desc_hi, uint32_t idesc128,
                                           uint32_t idesc64, bool leader) {
    constexpr uint32_t slice = (64 * 128) >> 4;     // one [64 x 64] filter slice, in descriptor address units (16 B)
    constexpr uint32_t row = (ROW_PIX * 128) >> 4;  // one window row
    auto desc = [desc_hi](uint32_t lo) { return ((uint64_t)desc_hi << 32) | lo; };
    if (leader) {
        // both accumulators: window rows {1, 3} against filter rows (1 | 0), or {2, 4} against (2 | 1);
        // the filter slices of column ky lie at 3 * ky + (2 - row)
#pragma unroll
        for (int ky = 0; ky < 3; ky++) {
            const uint32_t a = a_half + (HALF == 0 ? 0u : row) + (uint32_t)ky * 8u;
            const uint32_t b = b0 + (uint32_t)(ky * 3 + (HALF == 0 ? 1 : 0)) * slice;
#pragma unroll
            for (int k = 0; k < 4; k++)  // K = 16 channels = 32 bytes inside the swizzle row: +2 in the address field
                umma_bf16(d_tmem, desc(a + 2 * k), desc(b + 2 * k), idesc128, (uint32_t)(HALF != 0 || (ky | k) != 0));
        }
        // one accumulator: window rows {3, 5} against filter row 2 into D1, or {0, 2} against filter row 0 into D0
#pragma unroll
        for (int ky = 0; ky < 3; ky++) {
            const uint32_t a = a_half + (HALF == 0 ? row : 0u) + (uint32_t)ky * 8u;
            const uint32_t b = b0 + (uint32_t)(ky * 3 + (HALF == 0 ? 0 : 2)) * slice;
#pragma unroll
            for (int k = 0; k < 4; k++) umma_bf16(d_tmem + (HALF == 0 ? 64u : 0u), desc(a + 2 * k), desc(b + 2 * k), idesc64, 1u);
        }
    }
    __syncwarp();
}

// POOL: the 2x2 / 2 max-pool of the result is what is stored (RowsParams::pool), fixed at compile time so that the
// plain form carries none of its registers.
template <bool POOL>
__global__ void __launch_bounds__(kRowsThreads, 1)
conv_rows_kernel(const __grid_constant__ CUtensorMap tmIn, const __grid_constant__ CUtensorMap tmF,
                 const __grid_constant__ CUtensorMap tmOut, const __grid_constant__ CUtensorMap tmRes, const RowsParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *s_filter = smem;                        // 9 slices [64 oC x 128 B], column by column, rows descending
    uint8_t *s_win = s_filter + kFilterBytes;        // kSlots half-windows; the scrap columns of the last one read
                                                     // two pixels past it, into the half buffers that follow
    uint8_t *s_out = s_win + kSlots * kSlotBytes;    // kHalves output half buffers
    float *s_alpha = reinterpret_cast<float *>(s_out + kHalves * p.half_bytes);  // [64]
    float *s_beta = s_alpha + 64;                                                // [64]
    uint64_t *full = reinterpret_cast<uint64_t *>(s_beta + 64);  // [kSlots]  half-window landed
    uint64_t *empty = full + kSlots;                             // [kSlots]  its MMAs have read it
    uint64_t *tmem_full = empty + kSlots;                        // [kAccs]   accumulator pair complete
    uint64_t *tmem_empty = tmem_full + kAccs;                    // [kAccs]   read out by all sixteen epilogue warps
    uint64_t *half_ready = tmem_empty + kAccs;                   // [kHalves] free, and holding the residual if there is one
    uint64_t *staged = half_ready + kHalves;                     // [kHalves] written by all sixteen epilogue warps
    uint64_t *filter_bar = staged + kHalves;
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(filter_bar + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmIn);
        tma_prefetch_desc(&tmF);
        tma_prefetch_desc(&tmOut);
        if (p.has_res) tma_prefetch_desc(&tmRes);
        for (int s = 0; s < kSlots; s++) {
            mbar_init(&full[s], 1);   // the producer's arrive(+expect-tx)
            mbar_init(&empty[s], 1);  // one tcgen05.commit
        }
        for (int b = 0; b < kAccs; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], kEpilogueWarps);
        }
        for (int h = 0; h < kHalves; h++) {
            mbar_init(&half_ready[h], 1);
            mbar_init(&staged[h], kEpilogueWarps);
        }
        mbar_init(filter_bar, 1);
        fence_barrier_init();
        fence_proxy_async();
        // The filter is asked for at once, by the thread that has just initialised its barrier: the 72 KiB arrive
        // while the other warps allocate tensor memory and compute the epilogue coefficients.
        mbar_expect_tx(filter_bar, (uint32_t)kFilterBytes);
        for (int t = 0; t < 9; t++)  // tap t = (row t / 3, column t % 3) -> slice 3 * column + (2 - row)
            tma_load_3d(s_filter + (size_t)((t % 3) * 3 + (2 - t / 3)) * 64 * 128, &tmF, filter_bar, 0, t, 0);
    }
    if (warp == 1) {
        tmem_alloc(tmem_holder, (uint32_t)(kAccs * kAccCols));
        tmem_relinquish();
    }
    // per-channel epilogue coefficients: y = acc * alpha[c] + beta[c]
    //   no batch-norm: alpha = 1, beta = bias;  batch-norm: alpha = scale / sqrt(var + eps),
    //   beta = (bias - mean) * alpha + bn_bias
    if (threadIdx.x < 64) {
        const int c = threadIdx.x;
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
        // ------------------------------------------------------------ window producer (warp-uniform loop, one elected lane issues)
        const bool leader = elect_one();
        uint32_t issued = 0, ph = 0;
        int st = 0;
        bool ok = true;
        TileWalk tw(blockIdx.x, gridDim.x, p.row_blocks, p.col_blocks);
        for (long long tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, tw.advance()) {
            const int n = tw.n, oh0 = tw.rb * 4, ow0 = tw.cb * kTileCols;
            for (int half = 0; half < 2; half++) {
                ok = mbar_wait(&empty[st], ph ^ 1, p.status, kWaitEmpty);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (leader) {
                    const int r = oh0 - p.pt + 1 - half;  // first input row of the half-window; negative rows are zeros
                    mbar_expect_tx(&full[st], (uint32_t)kSlotBytes);
                    tma_load_5d(s_win + (size_t)st * kSlotBytes, &tmIn, &full[st], 0, ow0 - p.pl, r & 1, r >> 1, n);
                }
                __syncwarp();
                issued++;
                if (++st == kSlots) {
                    st = 0;
                    ph ^= 1;
                }
            }
        }
        // Drain: do not leave while copies may still be landing in this CTA's shared memory.
        if (lane == 0) {
            int s2 = st;
            uint32_t ph2 = ph;
            for (uint32_t back = 0; back < (uint32_t)kSlots && back < issued; back++) {
                if (s2 == 0) {
                    s2 = kSlots;
                    ph2 ^= 1;
                }
                s2--;
                if (!mbar_wait(&full[s2], ph2, p.status, kWaitDrain)) break;
            }
            mbar_wait(filter_bar, 0, p.status, kWaitDrain);
        }
        __syncwarp();
    } else if (warp <= 2) {
        // ------------------------------------------------------------ MMA issuers: warp 1 the even tiles of this CTA, warp 2 the odd ones
        const uint32_t iw = (uint32_t)(warp - 1);
        const bool leader = elect_one();
        const uint32_t idesc128 = idesc_bf16_f32(128, 128), idesc64 = idesc_bf16_f32(128, 64);
        bool ok = mbar_wait(filter_bar, 0, p.status, kWaitFull);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        const uint64_t da0 = smem_desc_sw128(smem_u32(s_win)), db0 = smem_desc_sw128(smem_u32(s_filter));
        const uint32_t desc_hi = (uint32_t)(da0 >> 32);  // same for A and B: stride 1024 B, version, 128-byte swizzle
        const uint32_t a_lo0 = (uint32_t)da0, b_lo0 = (uint32_t)db0;
        constexpr uint32_t slot_step = (uint32_t)kSlotBytes >> 4;
        // four slots, two issuers: this warp's tiles always use the slots 2 * iw and 2 * iw + 1, and every other accumulator
        const uint32_t st = 2 * iw;
        uint32_t ph = 0, buf = iw, aph = 0;
        for (long long tile = blockIdx.x + (long long)iw * gridDim.x; tile < p.num_tiles && ok; tile += 2ll * gridDim.x) {
            ok = mbar_wait(&tmem_empty[buf], aph ^ 1, p.status, kWaitTmemEmpty);
            if (ok) ok = mbar_wait(&full[st], ph, p.status, kWaitFull);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * kAccCols;
            issue_half<0>(d_tmem, a_lo0 + st * slot_step, b_lo0, desc_hi, idesc128, idesc64, leader);
            if (leader) umma_commit(&empty[st]);  // the half-window is reusable once these MMAs have read it
            __syncwarp();
            ok = mbar_wait(&full[st + 1], ph, p.status, kWaitFull);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            issue_half<1>(d_tmem, a_lo0 + (st + 1) * slot_step, b_lo0, desc_hi, idesc128, idesc64, leader);
            if (leader) {
                umma_commit(&empty[st + 1]);
                umma_commit(&tmem_full[buf]);  // both accumulators are complete
            }
            __syncwarp();
            ph ^= 1;
            buf += 2;
            if (buf >= (uint32_t)kAccs) {
                buf -= (uint32_t)kAccs;
                aph ^= 1;
            }
        }
    } else if (warp == kStagingWarp) {
        // ------------------------------------------------------------ output staging: TMA stores, residual loads
        // Step s = 2 * (tile number in this CTA) + accumulator uses half buffer s % 4.  After the store of step s
        // has read its buffer, the buffer is made ready for step s + 4 (same accumulator, two tiles further on):
        // with a residual by loading it (the barrier completes when it has landed), without one by a plain arrive.
        // With the pool fused, nothing is staged for a store: a half buffer only ever carries a residual (or nothing).
        if (lane == 0 && !(POOL && !p.has_res)) {
            const uint32_t half_tx = (uint32_t)(p.bw * 2 * 128);
            auto make_ready = [&](int h, int n, int oh0, int ow0) {
                if (p.has_res) {
                    mbar_expect_tx(&half_ready[h], half_tx);
                    tma_load_5d(s_out + (size_t)h * p.half_bytes, &tmRes, &half_ready[h], 0, ow0, h & 1, oh0 >> 1, n);
                } else {
                    mbar_arrive(&half_ready[h]);
                }
            };
            TileWalk tw(blockIdx.x, gridDim.x, p.row_blocks, p.col_blocks);     // the tile being stored
            TileWalk ahead(blockIdx.x, gridDim.x, p.row_blocks, p.col_blocks);  // two tiles further on
            long long tile_ahead = blockIdx.x;
            for (int i = 0; i < 2 && tile_ahead < p.num_tiles; i++, tile_ahead += gridDim.x, ahead.advance())
                for (int j = 0; j < 2; j++) make_ready(2 * i + j, ahead.n, ahead.rb * 4, ahead.cb * kTileCols);
            uint32_t i = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, tw.advance(), i++) {
                for (int j = 0; j < 2; j++) {
                    const int h = (int)((2 * i + j) & 3);
                    ok = mbar_wait(&staged[h], (i >> 1) & 1, p.status, kWaitFull);
                    if (!ok) break;
                    if (!POOL) {
                        // rows {j, j + 2} of the tile: parity j, row pairs oh0 / 2 and oh0 / 2 + 1; TMA clips what lies outside
                        tma_store_5d(&tmOut, s_out + (size_t)h * p.half_bytes, 0, tw.cb * kTileCols, j, (tw.rb * 4) >> 1, tw.n);
                        bulk_commit_group();
                        bulk_wait_read_all();
                    }
                    if (tile_ahead < p.num_tiles) make_ready(h, ahead.n, ahead.rb * 4, ahead.cb * kTileCols);
                }
                if (tile_ahead < p.num_tiles) {
                    tile_ahead += gridDim.x;
                    ahead.advance();
                }
            }
            bulk_wait_all();  // the stores are complete before the CTA leaves
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue: 16 warps = 4 lane quarters x 4 channel slices
        const int quarter = warp & 3;                          // the tensor-memory lane quarter this warp may read
        const int slice = (warp - kFirstEpilogueWarp) >> 2;    // channels [16 * slice, 16 * slice + 16)
        const int row = quarter * 32 + lane;                   // tensor-memory lane = pixel of the accumulator's two rows
        const int trow = row >> 6, tcol = row & 63;
        const int q = trow * p.bw + tcol;                      // the pixel's 128-byte row in a half buffer (box {64 ch, bw, 1, 2, 1})
        const bool skip = tcol >= p.bw;                        // scrap columns
        // this thread's two 16-byte chunks of the pixel's row, under the 128-byte swizzle (chunk index ^ (row & 7))
        const uint32_t off0 = (uint32_t)q * 128u + (((uint32_t)(2 * slice) ^ (uint32_t)(q & 7)) << 4);
        const uint32_t off1 = (uint32_t)q * 128u + (((uint32_t)(2 * slice + 1) ^ (uint32_t)(q & 7)) << 4);
        float alpha[16], beta[16];
#pragma unroll
        for (int c = 0; c < 16; c++) {
            alpha[c] = s_alpha[16 * slice + c];
            beta[c] = s_beta[16 * slice + c];
        }
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(16 * slice);
        uint32_t buf = 0, aph = 0, step = 0;
        bool ok = true;
        const bool use_halves = !(POOL && !p.has_res);  // half buffers carry the output, the residual, or both
        TileWalk tw(blockIdx.x, gridDim.x, p.row_blocks, p.col_blocks);
        for (long long tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, tw.advance()) {
            if (lane == 0) ok = mbar_wait(&tmem_full[buf], aph, p.status, kWaitTmemFull);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            tc_fence_after();
            float vmax[16];  // pool: the running maximum over the tile's two accumulators (rows 2r and 2r + 1)
#pragma unroll 1
            for (int j = 0; j < 2; j++, step++) {
                const uint32_t h = step & 3;
                if (use_halves) {
                    if (lane == 0) ok = mbar_wait(&half_ready[h], (step >> 2) & 1, p.status, kWaitFull);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                }
                uint32_t acc[16];
                tmem_ld_32x16(lane_base + buf * kAccCols + (uint32_t)(j * 64), acc);
                tmem_ld_wait();
                if (j == 1) {
                    // both accumulators are in registers (of this warp): the MMA issuer may have them back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&tmem_empty[buf]);
                }
                {
                    uint8_t *half = s_out + (size_t)h * p.half_bytes;
                    float v[16];
#pragma unroll
                    for (int c = 0; c < 16; c++) v[c] = fmaf(__uint_as_float(acc[c]), alpha[c], beta[c]);
                    if (p.has_res && !skip) {  // the residual is already in the buffer, in the output's layout
                        add_bf16x8(v, *reinterpret_cast<const uint4 *>(half + off0));
                        add_bf16x8(v + 8, *reinterpret_cast<const uint4 *>(half + off1));
                    }
                    if (p.relu) {
#pragma unroll
                        for (int c = 0; c < 16; c++) v[c] = fmaxf(v[c], 0.f);
                    }
                    if (POOL) {
#pragma unroll
                        for (int c = 0; c < 16; c++) vmax[c] = j == 0 ? v[c] : fmaxf(vmax[c], v[c]);
                    } else if (!skip) {
                        *reinterpret_cast<uint4 *>(half + off0) = pack_bf16x8(v);
                        *reinterpret_cast<uint4 *>(half + off1) = pack_bf16x8(v + 8);
                    }
                }
                if (use_halves) {
                    // staged (or, with the pool fused, its residual consumed): the staging warp takes the half over
                    // once all sixteen warps have said so
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&staged[h]);
                }
            }
            if (!ok) break;
            if (POOL) {
                // A thread holds column tcol of rows 2 * trow and 2 * trow + 1 of the tile: the vertical half of the
                // 2 x 2 window is the maximum it already took, the horizontal half its neighbour lane's.  Rounding
                // to bf16 is monotonic, so pooling before the rounding gives the same bits as pooling after it.
#pragma unroll
                for (int c = 0; c < 16; c++) vmax[c] = fmaxf(vmax[c], __shfl_xor_sync(0xffffffffu, vmax[c], 1));
                // both lanes of a pair now hold the window's maximum: the even one stores channels 0..7 of the slice,
                // the odd one channels 8..15, so that a pair writes one whole 32-byte sector
                const int oh = tw.rb * 4 + 2 * trow, pcol = tcol & ~1, ow = tw.cb * kTileCols + pcol;
                if (pcol < p.bw && oh < p.OH && ow < p.OW) {
                    const size_t pix = ((size_t)tw.n * (p.OH >> 1) + (oh >> 1)) * (p.OW >> 1) + (ow >> 1);
                    uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(p.pool_out) + pix * 64 + 16 * slice);
                    const uint4 lo = pack_bf16x8(vmax), hi = pack_bf16x8(vmax + 8);
                    dst[lane & 1] = (lane & 1) ? hi : lo;
                }
            }
            if (++buf == (uint32_t)kAccs) {
                buf = 0;
                aph ^= 1;
            }
        }
    }

    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, (uint32_t)(kAccs * kAccCols));
    }
}

}  // namespace

// Returns SWCB200_ERR_UNSUPPORTED (without setting the context's error text) for shapes this form does not take.
int swc_conv_tc_rows(swcb200_ctx *ctx, void *output, const void *input, const void *filt, const float *bias, const size_t *odims,
                     const size_t *idims, const size_t *kernels, const size_t *pads, const swcb200_conv_epilogue *ep) {
    RowsParams p;
    memset(&p, 0, sizeof(p));
    p.N = (int)idims[0]; p.H = (int)idims[1]; p.W = (int)idims[2];
    p.OH = (int)odims[1]; p.OW = (int)odims[2];
    p.pt = (int)pads[0]; p.pl = (int)pads[1];
    if (kernels[0] != 3 || kernels[1] != 3 || idims[3] != 64 || odims[3] != 64) return SWCB200_ERR_UNSUPPORTED;
    if (p.H % 2 != 0 || p.OH % 2 != 0 || p.OH < 4) return SWCB200_ERR_UNSUPPORTED;
    p.bw = p.OW < kTileCols ? p.OW : kTileCols;
    p.half_bytes = (2 * p.bw * 128 + 1023) & ~1023;
    p.row_blocks = (p.OH + 3) / 4;
    p.col_blocks = (p.OW + kTileCols - 1) / kTileCols;
    p.num_tiles = (long long)p.N * p.row_blocks * p.col_blocks;
    p.bias = bias;
    if (ep) {
        p.bn_scale = ep->bn_scale; p.bn_bias = ep->bn_bias; p.bn_mean = ep->bn_mean; p.bn_var = ep->bn_var;
        p.bn_eps = ep->bn_eps;
        p.has_res = ep->residual != nullptr;
        p.relu = ep->relu;
        p.pool = ep->pool2x2 != 0;
    }
    if (p.pool && p.OW % 2 != 0) return SWCB200_ERR_UNSUPPORTED;
    p.pool_out = output;
    p.status = ctx->dev_status;
    const size_t smem = 1024 /*alignment of the base*/ + kFilterBytes + kSlots * kSlotBytes + kHalves * (size_t)p.half_bytes + 2 * 64 * 4 +
                        (2 * kSlots + 2 * kAccs + 2 * kHalves + 1) * 8 + 16;
    if (smem > (size_t)kMaxSmem) return SWCB200_ERR_UNSUPPORTED;

    CUtensorMap tmIn, tmF, tmOut, tmRes;
    {
        // rows split by parity, {iC, W, row % 2, row / 2, N}: a box of three rows of one parity is a half-window
        uint64_t dims[5] = {64, (uint64_t)p.W, 2, (uint64_t)(p.H / 2), (uint64_t)p.N};
        uint64_t str[5] = {2, 128, (uint64_t)p.W * 128, (uint64_t)p.W * 256, (uint64_t)p.H * p.W * 128};
        uint32_t box[5] = {64, (uint32_t)ROW_PIX, 1, 3, 1};
        int rc = tc::make_tmap_bf16(ctx, &tmIn, input, 5, dims, str, box);
        if (rc) return rc;
    }
    {
        // filter [oC, 3, 3, iC] seen as {iC, tap, oC}: one box = all output channels of one tap
        uint64_t dims[3] = {64, 9, 64};
        uint64_t str[3] = {2, 128, 9 * 128};
        uint32_t box[3] = {64, 1, 64};
        int rc = tc::make_tmap_bf16(ctx, &tmF, filt, 3, dims, str, box);
        if (rc) return rc;
    }
    {
        // output (and residual) with the rows split the same way: one box = the two rows of one accumulator
        uint64_t dims[5] = {64, (uint64_t)p.OW, 2, (uint64_t)(p.OH / 2), (uint64_t)p.N};
        uint64_t str[5] = {2, 128, (uint64_t)p.OW * 128, (uint64_t)p.OW * 256, (uint64_t)p.OH * p.OW * 128};
        uint32_t box[5] = {64, (uint32_t)p.bw, 1, 2, 1};
        int rc = tc::make_tmap_bf16(ctx, &tmOut, output, 5, dims, str, box);
        if (rc) return rc;
        tmRes = tmOut;
        if (p.has_res) {
            rc = tc::make_tmap_bf16(ctx, &tmRes, ep->residual, 5, dims, str, box);
            if (rc) return rc;
        }
    }
    static bool attr_set[64] = {false};  // per device: the opt-in to large dynamic shared memory
    if (!attr_set[ctx->device & 63]) {
        SWC_CUDA(ctx, cudaFuncSetAttribute(conv_rows_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem));
        SWC_CUDA(ctx, cudaFuncSetAttribute(conv_rows_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem));
        attr_set[ctx->device & 63] = true;
    }
    unsigned grid = (unsigned)(p.num_tiles < swc_tc_sms(ctx) ? p.num_tiles : swc_tc_sms(ctx));
    if (p.pool)
        conv_rows_kernel<true><<<grid, kRowsThreads, smem, ctx->stream>>>(tmIn, tmF, tmOut, tmRes, p);
    else
        conv_rows_kernel<false><<<grid, kRowsThreads, smem, ctx->stream>>>(tmIn, tmF, tmOut, tmRes, p);
    return swc_check_launch(ctx, "conv2d_bf16");
}
