// Fully-connected layer on the 5th-generation tensor cores:
//     C[m,n] = act( A[m,k] . Wp[n,k]^T + bias[n] )       A, Wp bf16 (K-major), fp32 accumulate
// One launch covers the MatrixMatrixMul -> MatrixVectorAdd -> ReLU/Tanh chain the reference's
// lowering produces for an FC layer (src/op/dlOp/dlOpEinsum.cpp:154-237; arithmetic of
// kernels.h:41-56, :542-552, :575-580, :58-64).
//
// Shape of the kernel
//   * persistent: one CTA per SM, tiles of 128 x BN outputs (BN <= 256) taken round-robin, the n
//     index fastest so the CTAs running together share a few A row panels and keep Wp in L2;
//   * warp 0: TMA producer -- per 64-deep k block one 128x64 box of A and one BNx64 box of Wp into a
//     4-stage shared-memory ring (128-byte swizzle), completion counted on an mbarrier per stage;
//   * warp 1: MMA issuer -- one elected thread issues 4 tcgen05.mma (K = 16 each) per stage into a
//     128-lane x BN-column fp32 accumulator in tensor memory; tcgen05.commit releases the stage back
//     to the producer and, after the last k block, publishes the accumulator;
//   * warps 2-5: epilogue -- tcgen05.ld 32 lanes x 32 columns at a time, + bias, activation, convert,
//     128-bit global stores.  Two accumulators (2 x 256 columns = all 512 of the SM) alternate, so the
//     epilogue of tile i overlaps the main loop of tile i+1.
//   Out-of-range rows/columns/k are zero-filled by TMA on the way in and masked on the way out.
//
// Split activations (the SPLIT instantiations).  A bf16 activation keeps 8 bits of mantissa; on a network whose
// top-two logits are often closer than that rounding, the stored hidden activations -- not the arithmetic --
// decide the argmax.  In split mode a layer writes its output as TWO bf16 terms, hi = bf16(v) and
// lo = bf16(v - hi) (together 16 bits of mantissa), and the next layer multiplies both by the same weight tile
// into the same fp32 accumulator: C = A_hi . Wp^T + A_lo . Wp^T.  Twice the MMAs and twice the A traffic per
// layer, the weights (bf16 by definition of the workload) unchanged.
#include <mutex>
#include <unordered_map>

#include "tc_common.cuh"

namespace tc {

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

int make_tmap_bf16(swcb200_ctx *ctx, CUtensorMap *out, const void *base, int rank, const uint64_t *dims,
                   const uint64_t *strides_bytes, const uint32_t *box) {
    EncodeTiledFn fn = encode_tiled_fn();
    SWC_REQUIRE(ctx, fn != nullptr, SWCB200_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
    cuuint64_t gdim[5], gstr[5];
    cuuint32_t bx[5], es[5];
    for (int i = 0; i < rank; i++) {
        gdim[i] = dims[i];
        bx[i] = box[i];
        es[i] = 1;
        if (i > 0) gstr[i - 1] = strides_bytes[i];
    }
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void *>(base), gdim, gstr, bx, es,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    SWC_REQUIRE(ctx, r == CUDA_SUCCESS, SWCB200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return SWCB200_OK;
}

}  // namespace tc

namespace {

using namespace tc;

constexpr int BM = 128;        // UMMA M
constexpr int BN_MAX = 256;    // UMMA N upper bound
constexpr int BK = 64;         // one 128-byte swizzle row of bf16
constexpr int UMMA_K = 16;     // K per tcgen05.mma for 16-bit inputs
// scattered-rows epilogue: a 32 x 32 fp32 chunk per epilogue warp, rows 36 floats apart (16-byte aligned rows)
constexpr int kXposePitch = 36;
constexpr int kXposeBytes = 4 * 32 * kXposePitch * 4;
constexpr int A_BYTES = BM * BK * 2;                 // 16 KiB
constexpr int B_BYTES = BN_MAX * BK * 2;             // 32 KiB
// one stage of the single-CTA kernel: A [, A_lo], Wp tile; 4 stages of 48 KiB, or 3 of 64 KiB with split activations
template <bool SPLIT> struct Single {
    static constexpr int kStages = SPLIT ? 3 : 4;
    static constexpr int A_TOTAL = SPLIT ? 2 * A_BYTES : A_BYTES;
    static constexpr int STAGE_BYTES = A_TOTAL + B_BYTES;
    static constexpr size_t kSmemBytes = (size_t)kStages * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + kXposeBytes;
};
constexpr int kTmemCols = 512;                       // two 256-column accumulators
constexpr int kThreads = 192;                        // TMA warp, MMA warp, 4 epilogue warps
constexpr int kEpilogueThreads = 128;

struct FcParams {
    int m, n, k;
    int bn;  // tile width actually used: 32, 64, 128 or 256
    int tiles_m, tiles_n;
    int band;  // n tiles per band of the tile order (see tile_coords)
    const float *bias;
    int act;
    void *c;
    int c_is_bf16;
    int ldc;
    int c_vec;  // C base and row pitch are 16-byte aligned: 128-bit stores allowed
    void *c_lo;  // bf16 outputs only: where the rounding remainder bf16(v - bf16(v)) goes (same pitch), or null
    // Rows scattered to their owners (fp32 output only, owners > 0): row i belongs to rank o = i / owner_rows and is
    // written to that rank's memory, owner_base[o] + ((owner_rank * owner_rows) + i % owner_rows) * ldc -- slot
    // `owner_rank` of the owner's slot array.  owner_base[] are peer mappings (plain stores over NVLink).
    float *owner_base[SWCB200_MAX_PEERS];
    int owners, owner_rows, owner_rank;
    int *status;
};

// Tile order.  Tiles are taken band by band: a band is `band` consecutive n tiles wide and is walked m
// panel by m panel, n fastest inside the band.  The CTAs running at the same moment therefore share a few A
// panels and at most `band` Wp tiles, which keeps both in L2 even when Wp as a whole does not fit.  With
// band = tiles_n this is the plain n-fastest order (each A panel read once, Wp resident).
__device__ __forceinline__ void tile_coords(const FcParams &p, int t, int &tm, int &tn) {
    const int per_band = p.band * p.tiles_m;
    const int b = t / per_band, i = t - b * per_band;
    const int n0 = b * p.band;
    const int gw = min(p.band, p.tiles_n - n0);
    tm = i / gw;
    tn = n0 + (i - tm * gw);
}

__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == SWCB200_ACT_RELU) return (v > 0.f) ? v : 0.f;
    if (act == SWCB200_ACT_TANH) return 1.0f - __fdividef(2.0f, __expf(2.0f * v) + 1.0f);
    return v;
}

// bias + activation + conversion + store of 32 consecutive columns of one output row
__device__ __forceinline__ void store_row_chunk(const FcParams &p, const uint32_t (&r)[32], int row, int col) {
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; j++) {
        float x = __uint_as_float(r[j]);
        if (p.bias != nullptr && col + j < p.n) x += __ldg(p.bias + col + j);
        v[j] = apply_act(x, p.act);
    }
    if (p.c_is_bf16) {
        __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(p.c) + (size_t)row * p.ldc + col;
        __nv_bfloat16 *dst_lo = p.c_lo ? reinterpret_cast<__nv_bfloat16 *>(p.c_lo) + (size_t)row * p.ldc + col : nullptr;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            if (p.c_vec && col + j + 8 <= p.n) {
                uint4 o;
                __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&o);
                h[0] = __floats2bfloat162_rn(v[j], v[j + 1]);
                h[1] = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                h[2] = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
                h[3] = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4 *>(dst + j) = o;
                if (dst_lo != nullptr) {
                    uint4 l;
                    __nv_bfloat162 *g = reinterpret_cast<__nv_bfloat162 *>(&l);
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float2 hi = __bfloat1622float2(h[e]);
                        g[e] = __floats2bfloat162_rn(v[j + 2 * e] - hi.x, v[j + 2 * e + 1] - hi.y);
                    }
                    *reinterpret_cast<uint4 *>(dst_lo + j) = l;
                }
            } else {
                for (int e = 0; e < 8; e++)
                    if (col + j + e < p.n) {
                        const __nv_bfloat16 hi = __float2bfloat16_rn(v[j + e]);
                        dst[j + e] = hi;
                        if (dst_lo != nullptr) dst_lo[j + e] = __float2bfloat16_rn(v[j + e] - __bfloat162float(hi));
                    }
            }
        }
    } else {
        float *dst = reinterpret_cast<float *>(p.c) + (size_t)row * p.ldc + col;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            if (p.c_vec && col + j + 4 <= p.n) {
                *reinterpret_cast<float4 *>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
                for (int e = 0; e < 4; e++)
                    if (col + j + e < p.n) dst[j + e] = v[j + e];
            }
        }
    }
}

// Scattered rows (FcParams::owners > 0): the warp's 32 x 32 chunk goes to other GPUs' memory.  A thread holds 32
// columns of ONE row, so storing straight from registers would send 16-byte pieces of 32 different lines per
// instruction, which NVLink carries badly (measured: 130 GB/s).  The chunk is turned through shared memory instead and
// leaves as whole 128-byte lines, four rows per instruction.
__device__ __forceinline__ void store_chunk_to_owners(const FcParams &p, const uint32_t (&r)[32], int row_base, int lane, int col,
                                                      float *sx) {
    float4 *mine = reinterpret_cast<float4 *>(sx + lane * kXposePitch);
#pragma unroll
    for (int j = 0; j < 8; j++)
        mine[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                              __uint_as_float(r[4 * j + 3]));
    __syncwarp();
    const int sub = lane >> 3, c4 = (lane & 7) * 4;
#pragma unroll
    for (int r0 = 0; r0 < 32; r0 += 4) {
        const int rr = r0 + sub, row = row_base + rr;
        const float4 v = *reinterpret_cast<const float4 *>(sx + rr * kXposePitch + c4);
        if (row < p.m && col + c4 < p.n) {  // n is a multiple of 4 in this mode
            const int o = row / p.owner_rows;
            float *dst = p.owner_base[o] + ((size_t)p.owner_rank * p.owner_rows + (size_t)(row - o * p.owner_rows)) * p.ldc + col + c4;
            *reinterpret_cast<float4 *>(dst) = v;
        }
    }
    __syncwarp();
}

template <bool SPLIT>
__global__ void __launch_bounds__(kThreads, 1)
fc_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmAlo,
             const __grid_constant__ CUtensorMap tmB, const FcParams p) {
    constexpr int kStages = Single<SPLIT>::kStages, STAGE_BYTES = Single<SPLIT>::STAGE_BYTES, A_TOTAL = Single<SPLIT>::A_TOTAL;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + (size_t)kStages * STAGE_BYTES);
    uint64_t *empty = full + kStages;
    uint64_t *tmem_full = empty + kStages;
    uint64_t *tmem_empty = tmem_full + 2;
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(tmem_empty + 2);
    float *s_xpose = reinterpret_cast<float *>(smem + (size_t)kStages * STAGE_BYTES + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_tiles = p.tiles_m * p.tiles_n;
    const int kblocks = (p.k + BK - 1) / BK;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmA);
        if (SPLIT) tma_prefetch_desc(&tmAlo);
        tma_prefetch_desc(&tmB);
        for (int s = 0; s < kStages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], kEpilogueThreads);
        }
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        tmem_alloc(tmem_holder, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            const uint32_t tx_bytes = (uint32_t)(A_TOTAL + p.bn * BK * 2);
            uint32_t g = 0;  // k blocks issued so far (ring position)
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                int tm, tn;
                tile_coords(p, t, tm, tn);
                for (int kb = 0; kb < kblocks; kb++, g++) {
                    const int s = g % kStages;
                    const uint32_t ph = (g / kStages) & 1;
                    if (!mbar_wait(&empty[s], ph ^ 1, p.status, kWaitEmpty)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&full[s], tx_bytes);
                    uint8_t *sa = smem + (size_t)s * STAGE_BYTES;
                    tma_load_2d(sa, &tmA, &full[s], kb * BK, tm * BM);
                    if (SPLIT) tma_load_2d(sa + A_BYTES, &tmAlo, &full[s], kb * BK, tm * BM);
                    tma_load_2d(sa + A_TOTAL, &tmB, &full[s], kb * BK, tn * p.bn);
                }
            }
            // Drain: do not leave the CTA while copies may still be landing in its shared memory.
            // Every issued stage either was consumed (its empty barrier completes) or still has to
            // complete its full barrier; waiting for the last kStages fills covers both.
            const uint32_t issued = g;
            for (uint32_t back = 0; back < (uint32_t)kStages && back < issued; back++) {
                const uint32_t gi = issued - 1 - back;
                if (!mbar_wait(&full[gi % kStages], (gi / kStages) & 1, p.status, kWaitDrain)) break;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = idesc_bf16_f32(BM, p.bn);
            uint32_t g = 0, it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, it++) {
                const uint32_t buf = it & 1, aph = (it >> 1) & 1;
                if (!mbar_wait(&tmem_empty[buf], aph ^ 1, p.status, kWaitTmemEmpty)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN_MAX;
                for (int kb = 0; kb < kblocks; kb++, g++) {
                    const int s = g % kStages;
                    const uint32_t ph = (g / kStages) & 1;
                    if (!mbar_wait(&full[s], ph, p.status, kWaitFull)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + (size_t)s * STAGE_BYTES);
                    const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sa + A_TOTAL);
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; j++) {
                        // advancing K by 16 elements = 32 bytes inside the swizzle row: +2 in the >>4 address field
                        umma_bf16(d_tmem, da + 2 * j, db + 2 * j, idesc, (uint32_t)((kb | j) != 0));
                        if (SPLIT) umma_bf16(d_tmem, da + (A_BYTES >> 4) + 2 * j, db + 2 * j, idesc, 1u);  // the lo term, same weights
                    }
                    umma_commit(&empty[s]);  // stage reusable once these MMAs have read it
                }
                if (ok) umma_commit(&tmem_full[buf]);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;  // the TMEM lane quarter this warp may read
        uint32_t it = 0;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, it++) {
            const uint32_t buf = it & 1, aph = (it >> 1) & 1;
            int tm, tn;
            tile_coords(p, t, tm, tn);
            bool ok = mbar_wait(&tmem_full[buf], aph, p.status, kWaitTmemFull);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row = tm * BM + quarter * 32 + lane;
            const bool row_ok = row < p.m;
            const int col_base = tn * p.bn;
            for (int c0 = 0; c0 < p.bn; c0 += 32) {
                uint32_t r[32];
                __syncwarp();  // tcgen05.ld is warp-collective
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN_MAX + c0, r);
                tmem_ld_wait();
                const int col = col_base + c0;
                if (p.owners > 0) {  // warp-uniform
                    if (col < p.n) store_chunk_to_owners(p, r, tm * BM + quarter * 32, lane, col, s_xpose + (warp - 2) * 32 * kXposePitch);
                    continue;
                }
                if (!row_ok || col >= p.n) continue;
                store_row_chunk(p, r, row, col);
            }
            tc_fence_before();
            mbar_arrive(&tmem_empty[buf]);
        }
    }

    // tear-down: everyone meets, then the allocating warp frees tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------------
// CTA-pair variant (cta_group::2): two CTAs of a cluster compute one 256 x BN tile.  Each CTA loads its own
// 128 rows of A and HALF of the BN rows of Wp per k block (32 KiB instead of 48 KiB), the leader's one
// thread issues tcgen05.mma with M = 256 that reads both CTAs' shared memory, and each CTA's tensor memory
// receives its 128 rows of the accumulator.  Per SM that is a third less operand traffic from L2 and a
// third less shared memory per stage, which buys a 6-deep ring: the 128 x 256 single-CTA kernel is bound
// by how many bytes it can keep in flight, not by the tensor pipe.
//   barriers: full[s] lives in the leader and counts the bytes of BOTH CTAs' loads; empty[s] and
//   tmem_full[b] exist in both CTAs and are signalled together by one tcgen05.commit; tmem_empty[b] lives in
//   the leader and collects the epilogue warps of both CTAs.
constexpr int B2_BYTES = (BN_MAX / 2) * BK * 2;       // 16 KiB: this CTA's half of the Wp tile
// one stage of the pair kernel: A [, A_lo], half Wp tile; 6 stages of 32 KiB, or 4 of 48 KiB with split activations
template <bool SPLIT> struct Pair {
    static constexpr int kStages = SPLIT ? 4 : 6;
    static constexpr int A_TOTAL = SPLIT ? 2 * A_BYTES : A_BYTES;
    static constexpr int STAGE_BYTES = A_TOTAL + B2_BYTES;
    static constexpr size_t kSmemBytes = (size_t)kStages * STAGE_BYTES + 1024 + 256 + kXposeBytes;
};

template <bool SPLIT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
fc_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmAlo,
                  const __grid_constant__ CUtensorMap tmB, const FcParams p) {
    constexpr int kStages2 = Pair<SPLIT>::kStages, STAGE2_BYTES = Pair<SPLIT>::STAGE_BYTES, A_TOTAL = Pair<SPLIT>::A_TOTAL;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + (size_t)kStages2 * STAGE2_BYTES);
    uint64_t *empty = full + kStages2;
    uint64_t *tmem_full = empty + kStages2;
    uint64_t *tmem_empty = tmem_full + 2;
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(tmem_empty + 2);
    float *s_xpose = reinterpret_cast<float *>(smem + (size_t)kStages2 * STAGE2_BYTES + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int num_tiles = p.tiles_m * p.tiles_n;
    const int kblocks = (p.k + BK - 1) / BK;
    const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
    const int half_bn = p.bn >> 1;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmA);
        if (SPLIT) tma_prefetch_desc(&tmAlo);
        tma_prefetch_desc(&tmB);
        for (int s = 0; s < kStages2; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], 8);  // 4 epilogue warps in each of the two CTAs
        }
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_holder, kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // the peer's barriers exist before anything is signalled across the pair
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    bool failed = false;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (one per CTA)
        if (lane == 0) {
            const uint32_t tx_bytes = 2u * (uint32_t)(A_TOTAL + half_bn * BK * 2);  // both CTAs' boxes
            int st = 0;
            uint32_t ph = 0;
            for (int t = cluster_id; t < num_tiles && !failed; t += num_clusters) {
                int tm, tn;
                tile_coords(p, t, tm, tn);
                const int row_a = tm * (2 * BM) + (int)rank * BM, row_b = tn * p.bn + (int)rank * half_bn;
                for (int kb = 0; kb < kblocks; kb++) {
                    if (!mbar_wait(&empty[st], ph ^ 1, p.status, kWaitEmpty)) {
                        failed = true;
                        break;
                    }
                    const uint32_t full_leader = map_to_cta(smem_u32(&full[st]), 0);
                    if (leader) mbar_expect_tx(&full[st], tx_bytes);
                    uint8_t *sa = smem + (size_t)st * STAGE2_BYTES;
                    tma_load_2d_pair(sa, &tmA, full_leader, kb * BK, row_a);
                    if (SPLIT) tma_load_2d_pair(sa + A_BYTES, &tmAlo, full_leader, kb * BK, row_a);
                    tma_load_2d_pair(sa + A_TOTAL, &tmB, full_leader, kb * BK, row_b);
                    if (++st == kStages2) {
                        st = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (leader && lane == 0) {
            const uint32_t idesc = idesc_bf16_f32(2 * BM, p.bn);
            const uint64_t da0 = smem_desc_sw128(smem_u32(smem)), db0 = smem_desc_sw128(smem_u32(smem + A_TOTAL));
            int st = 0;
            uint32_t ph = 0, it = 0;
            for (int t = cluster_id; t < num_tiles && !failed; t += num_clusters, it++) {
                const uint32_t buf = it & 1, aph = (it >> 1) & 1;
                if (!mbar_wait(&tmem_empty[buf], aph ^ 1, p.status, kWaitTmemEmpty)) {
                    failed = true;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN_MAX;
                for (int kb = 0; kb < kblocks; kb++) {
                    if (!mbar_wait(&full[st], ph, p.status, kWaitFull)) {
                        failed = true;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t off = (uint64_t)st * (STAGE2_BYTES >> 4);
                    const uint64_t da = da0 + off, db = db0 + off;
                    umma_bf16_pair(d_tmem, da, db, idesc, (uint32_t)(kb != 0));
                    if (SPLIT) umma_bf16_pair(d_tmem, da + (A_BYTES >> 4), db, idesc, 1u);  // the lo term, same weights
                    umma_bf16_pair(d_tmem, da + 2, db + 2, idesc, 1u);
                    if (SPLIT) umma_bf16_pair(d_tmem, da + (A_BYTES >> 4) + 2, db + 2, idesc, 1u);
                    umma_bf16_pair(d_tmem, da + 4, db + 4, idesc, 1u);
                    if (SPLIT) umma_bf16_pair(d_tmem, da + (A_BYTES >> 4) + 4, db + 4, idesc, 1u);
                    umma_bf16_pair(d_tmem, da + 6, db + 6, idesc, 1u);
                    if (SPLIT) umma_bf16_pair(d_tmem, da + (A_BYTES >> 4) + 6, db + 6, idesc, 1u);
                    umma_commit_pair(&empty[st], 3);  // both CTAs' stage `st` may be refilled once these have read it
                    if (++st == kStages2) {
                        st = 0;
                        ph ^= 1;
                    }
                }
                if (!failed) umma_commit_pair(&tmem_full[buf], 3);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
        const int quarter = warp & 3;
        uint32_t it = 0;
        for (int t = cluster_id; t < num_tiles; t += num_clusters, it++) {
            const uint32_t buf = it & 1, aph = (it >> 1) & 1;
            int tm, tn;
            tile_coords(p, t, tm, tn);
            bool ok = true;
            if (lane == 0) ok = mbar_wait(&tmem_full[buf], aph, p.status, kWaitTmemFull);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                failed = true;
                break;
            }
            tc_fence_after();
            const int row = tm * (2 * BM) + (int)rank * BM + quarter * 32 + lane;
            const bool row_ok = row < p.m;
            const int col_base = tn * p.bn;
            for (int c0 = 0; c0 < p.bn; c0 += 32) {
                uint32_t r[32];
                __syncwarp();
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN_MAX + c0, r);
                tmem_ld_wait();
                const int col = col_base + c0;
                if (p.owners > 0) {  // warp-uniform
                    if (col < p.n)
                        store_chunk_to_owners(p, r, tm * (2 * BM) + (int)rank * BM + quarter * 32, lane, col,
                                              s_xpose + (warp - 2) * 32 * kXposePitch);
                    continue;
                }
                if (!row_ok || col >= p.n) continue;
                store_row_chunk(p, r, row, col);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[buf]), 0));
        }
    }

    // A wait that gave up leaves copies possibly still in flight towards this CTA's shared memory: give them
    // a bounded time to land before anyone tears down (the clean path needs none: every load was consumed).
    if (failed) {
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000ll) {
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // neither CTA leaves while the other's MMAs may read its shared memory or signal its barriers
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

struct TmapKey {
    const void *base;
    uint64_t rows, cols, ld;
    uint32_t box_rows;
    bool operator==(const TmapKey &o) const {
        return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
struct TmapKeyHash {
    size_t operator()(const TmapKey &k) const {
        size_t h = (size_t)k.base;
        h = h * 1000003u ^ k.rows;
        h = h * 1000003u ^ k.cols;
        h = h * 1000003u ^ k.ld;
        h = h * 1000003u ^ k.box_rows;
        return h;
    }
};

// row-major [rows, cols] bf16 with leading dimension ld; box = box_rows x 64
int tmap_2d(swcb200_ctx *ctx, const void *base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
            CUtensorMap *out) {
    // Encoding costs a few microseconds of host time; the same few operands recur every forward pass.
    static thread_local std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
    TmapKey key{base, rows, cols, ld, box_rows};
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return SWCB200_OK;
    }
    uint64_t dims[2] = {cols, rows};
    uint64_t strides[2] = {2, ld * 2};
    uint32_t box[2] = {(uint32_t)BK, box_rows};
    int rc = make_tmap_bf16(ctx, out, base, 2, dims, strides, box);
    if (rc) return rc;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
    return SWCB200_OK;
}

}  // namespace

template <bool SPLIT>
static int launch_fc(swcb200_ctx *ctx, bool pair, const CUtensorMap &tmA, const CUtensorMap &tmAlo, const CUtensorMap &tmB,
                     FcParams &p, int m) {
    static bool attr_single[64] = {false}, attr_pair[64] = {false};  // per device: the opt-in to large dynamic shared memory
    const int dev = ctx->device & 63;
    if (pair) {
        p.tiles_m = (m + 2 * BM - 1) / (2 * BM);
        if (!attr_pair[dev]) {
            SWC_CUDA(ctx, cudaFuncSetAttribute(fc_tc_pair_kernel<SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)Pair<SPLIT>::kSmemBytes));
            attr_pair[dev] = true;
        }
        const long long tiles2 = (long long)p.tiles_m * p.tiles_n;
        const long long max_clusters = swc_tc_sms(ctx) / 2;
        unsigned grid2 = 2u * (unsigned)(tiles2 < max_clusters ? tiles2 : max_clusters);
        fc_tc_pair_kernel<SPLIT><<<grid2, kThreads, Pair<SPLIT>::kSmemBytes, ctx->stream>>>(tmA, tmAlo, tmB, p);
        return swc_check_launch(ctx, "fc_bf16");
    }
    if (!attr_single[dev]) {
        SWC_CUDA(ctx, cudaFuncSetAttribute(fc_tc_kernel<SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)Single<SPLIT>::kSmemBytes));
        attr_single[dev] = true;
    }
    const long long tiles = (long long)p.tiles_m * p.tiles_n;
    unsigned grid = (unsigned)(tiles < swc_tc_sms(ctx) ? tiles : swc_tc_sms(ctx));
    fc_tc_kernel<SPLIT><<<grid, kThreads, Single<SPLIT>::kSmemBytes, ctx->stream>>>(tmA, tmAlo, tmB, p);
    return swc_check_launch(ctx, "fc_bf16");
}

// rows of an fp32 output scattered over the ranks that own them (see FcParams); null: one local output
struct FcOwners {
    void *const *base;
    int owners, owner_rows, owner_rank;
};

int swc_fc_tc_owners(swcb200_ctx *ctx, int m, int n, int k, const void *a, const void *a_lo, int lda, const void *wp, int ldw,
                     const float *bias, int act, void *c, void *c_lo, int c_dtype, int ldc, const FcOwners *own);

// a_lo / c_lo: the second term of a split activation (see the top of the file), or null
int swc_fc_tc(swcb200_ctx *ctx, int m, int n, int k, const void *a, const void *a_lo, int lda, const void *wp, int ldw,
              const float *bias, int act, void *c, void *c_lo, int c_dtype, int ldc) {
    return swc_fc_tc_owners(ctx, m, n, k, a, a_lo, lda, wp, ldw, bias, act, c, c_lo, c_dtype, ldc, nullptr);
}

int swc_fc_tc_owners(swcb200_ctx *ctx, int m, int n, int k, const void *a, const void *a_lo, int lda, const void *wp, int ldw,
                     const float *bias, int act, void *c, void *c_lo, int c_dtype, int ldc, const FcOwners *own) {
    SWC_REQUIRE(ctx, swc_aligned16(a) && swc_aligned16(wp) && swc_aligned16(a_lo), SWCB200_ERR_MISALIGNED,
                "fc_bf16: A and Wp must be 16-byte aligned");
    SWC_REQUIRE(ctx, c_lo == nullptr || c_dtype == SWCB200_BF16, SWCB200_ERR_BAD_ARG,
                "fc_bf16: a remainder output only goes with a bf16 output");
    SWC_REQUIRE(ctx, lda % 8 == 0 && ldw % 8 == 0, SWCB200_ERR_MISALIGNED,
                "fc_bf16: lda (%d) and ldw (%d) must be multiples of 8 elements", lda, ldw);
    SWC_REQUIRE(ctx, lda >= k && ldw >= k && ldc >= n, SWCB200_ERR_BAD_SHAPE, "fc_bf16: leading dimension too small");
    const size_t celem = c_dtype == SWCB200_BF16 ? 2 : 4;
    int bn = 32;  // smallest tile width: the epilogue reads tensor memory 32 columns at a time
    while (bn < n && bn < BN_MAX) bn <<= 1;
    FcParams p;
    p.m = m;
    p.n = n;
    p.k = k;
    p.bn = bn;
    p.tiles_m = (m + BM - 1) / BM;
    p.tiles_n = (n + bn - 1) / bn;
    // keep the plain order while the packed weight is small enough to live in L2 next to the streams
    p.band = ((size_t)n * k * 2 <= ((size_t)48 << 20) || p.tiles_n <= 8) ? p.tiles_n : 8;
    p.bias = bias;
    p.act = act;
    p.c = c;
    p.c_is_bf16 = c_dtype == SWCB200_BF16;
    p.ldc = ldc;
    p.c_vec = swc_aligned16(c) && swc_aligned16(c_lo) && ((size_t)ldc * celem) % 16 == 0;
    p.c_lo = c_lo;
    p.owners = 0;
    p.owner_rows = p.owner_rank = 0;
    if (own != nullptr) {
        p.owners = own->owners;
        p.owner_rows = own->owner_rows;
        p.owner_rank = own->owner_rank;
        for (int o = 0; o < own->owners; o++) {
            p.owner_base[o] = (float *)own->base[o];
            p.c_vec = p.c_vec && swc_aligned16(own->base[o]);
        }
    }
    p.status = ctx->dev_status;
    // CTA pairs whenever there is more than one 128-row panel and the tile is wide enough to halve
    const bool pair = m > BM && bn >= 64 && ctx->sm_count >= 2;
    CUtensorMap tmA, tmAlo, tmB;
    int rc = tmap_2d(ctx, a, (uint64_t)m, (uint64_t)k, (uint64_t)lda, BM, &tmA);
    if (rc) return rc;
    tmAlo = tmA;
    if (a_lo != nullptr) {
        rc = tmap_2d(ctx, a_lo, (uint64_t)m, (uint64_t)k, (uint64_t)lda, BM, &tmAlo);
        if (rc) return rc;
    }
    rc = tmap_2d(ctx, wp, (uint64_t)n, (uint64_t)k, (uint64_t)ldw, (uint32_t)(pair ? bn / 2 : bn), &tmB);
    if (rc) return rc;
    return a_lo != nullptr ? launch_fc<true>(ctx, pair, tmA, tmAlo, tmB, p, m) : launch_fc<false>(ctx, pair, tmA, tmAlo, tmB, p, m);
}

SWC_EXPORT int swcb200_fc_bf16(swcb200_ctx *ctx, int m, int n, int k, const void *a_bf16, int lda, const void *wp_bf16,
                               int ldw, const float *bias, int act, void *c, int c_dtype, int ldc) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, m >= 0 && n >= 0 && k > 0, SWCB200_ERR_BAD_ARG, "fc_bf16: bad shape %d x %d x %d", m, n, k);
    SWC_REQUIRE(ctx, act >= SWCB200_ACT_NONE && act <= SWCB200_ACT_TANH, SWCB200_ERR_BAD_ARG, "fc_bf16: unknown activation");
    SWC_REQUIRE(ctx, c_dtype == SWCB200_F32 || c_dtype == SWCB200_BF16, SWCB200_ERR_BAD_ARG, "fc_bf16: unknown output dtype");
    if (m == 0 || n == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, a_bf16 && wp_bf16 && c, SWCB200_ERR_BAD_ARG, "fc_bf16: null tensor");
    return swc_fc_tc(ctx, m, n, k, a_bf16, nullptr, lda, wp_bf16, ldw, bias, act, c, nullptr, c_dtype, ldc);
}

SWC_EXPORT int swcb200_fc_bf16_scatter_rows(swcb200_ctx *ctx, int m, int n, int k, const void *a_bf16, int lda,
                                            const void *wp_bf16, int ldw, void *const *owner_slots, int nranks, int rank,
                                            int ld_slot) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, m >= 0 && n >= 0 && k > 0, SWCB200_ERR_BAD_ARG, "fc_bf16_scatter_rows: bad shape %d x %d x %d", m, n, k);
    SWC_REQUIRE(ctx, owner_slots && nranks >= 1 && nranks <= SWCB200_MAX_PEERS && rank >= 0 && rank < nranks, SWCB200_ERR_BAD_ARG,
                "fc_bf16_scatter_rows: bad rank / count (at most %d ranks)", SWCB200_MAX_PEERS);
    SWC_REQUIRE(ctx, m % nranks == 0 && ld_slot >= n, SWCB200_ERR_BAD_SHAPE,
                "fc_bf16_scatter_rows: %d rows do not split over %d ranks, or the slot pitch is below n", m, nranks);
    SWC_REQUIRE(ctx, n % 4 == 0 && ld_slot % 4 == 0, SWCB200_ERR_UNSUPPORTED,
                "fc_bf16_scatter_rows: n (%d) and the slot pitch (%d) must be multiples of 4", n, ld_slot);
    if (m == 0 || n == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, a_bf16 && wp_bf16, SWCB200_ERR_BAD_ARG, "fc_bf16_scatter_rows: null tensor");
    for (int o = 0; o < nranks; o++)
        SWC_REQUIRE(ctx, owner_slots[o] != nullptr, SWCB200_ERR_BAD_ARG, "fc_bf16_scatter_rows: null slot pointer for rank %d", o);
    const FcOwners own = {owner_slots, nranks, m / nranks, rank};
    return swc_fc_tc_owners(ctx, m, n, k, a_bf16, nullptr, lda, wp_bf16, ldw, nullptr, SWCB200_ACT_NONE, owner_slots[rank], nullptr,
                            SWCB200_F32, ld_slot, &own);
}

SWC_EXPORT int swcb200_fc_bf16_split(swcb200_ctx *ctx, int m, int n, int k, const void *a_hi, const void *a_lo, int lda,
                                     const void *wp_bf16, int ldw, const float *bias, int act, void *c, void *c_lo,
                                     int c_dtype, int ldc) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, m >= 0 && n >= 0 && k > 0, SWCB200_ERR_BAD_ARG, "fc_bf16_split: bad shape %d x %d x %d", m, n, k);
    SWC_REQUIRE(ctx, act >= SWCB200_ACT_NONE && act <= SWCB200_ACT_TANH, SWCB200_ERR_BAD_ARG, "fc_bf16_split: unknown activation");
    SWC_REQUIRE(ctx, c_dtype == SWCB200_F32 || c_dtype == SWCB200_BF16, SWCB200_ERR_BAD_ARG, "fc_bf16_split: unknown output dtype");
    if (m == 0 || n == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, a_hi && wp_bf16 && c, SWCB200_ERR_BAD_ARG, "fc_bf16_split: null tensor");
    return swc_fc_tc(ctx, m, n, k, a_hi, a_lo, lda, wp_bf16, ldw, bias, act, c, c_lo, c_dtype, ldc);
}

int swc_fc_strict(swcb200_ctx *ctx, int m, int n, int k, const float *a, int lda, const float *b, int ldb, float *c,
                  int ldc);

// fp32 entry point.  Strict mode: the bit-exact FFMA-pipe kernel.  Tensor-core mode: A and B are
// rounded to bf16 into the context's private scratch (B transposed to K-major on the way) and the
// tcgen05 kernel writes fp32 C.
SWC_EXPORT int swcb200_matrixMatrixMul_f(swcb200_ctx *ctx, int m, int n, int k, const float *a, int lda, const float *b,
                                         int ldb, float *c, int ldc) {
    SWC_CTX(ctx);
    SWC_REQUIRE(ctx, m >= 0 && n >= 0 && k >= 0, SWCB200_ERR_BAD_ARG, "matrixMatrixMul_f: negative shape");
    SWC_REQUIRE(ctx, lda >= k && ldb >= n && ldc >= n, SWCB200_ERR_BAD_SHAPE,
                "matrixMatrixMul_f: leading dimension too small");
    if (m == 0 || n == 0) return SWCB200_OK;
    SWC_REQUIRE(ctx, c && (k == 0 || (a && b)), SWCB200_ERR_BAD_ARG, "matrixMatrixMul_f: null tensor");
    const bool tc_ok = ctx->precision == SWCB200_TC_BF16 && k > 0;
    if (!tc_ok) return swc_fc_strict(ctx, m, n, k, a, lda, b, ldb, c, ldc);
    const size_t kp = ((size_t)k + 7) & ~(size_t)7;  // padded K so that row pitches are 16-byte multiples
    const size_t a_bytes = ((size_t)m * kp * 2 + 255) & ~(size_t)255, b_bytes = (size_t)n * kp * 2;
    void *scratch = nullptr;
    int rc = swc_scratch(ctx, a_bytes + b_bytes, &scratch);
    if (rc) return rc;
    void *a16 = scratch, *b16 = (uint8_t *)scratch + a_bytes;
    rc = swc_cast_pad_rows(ctx, a, m, k, lda, a16, (int)kp);
    if (rc) return rc;
    rc = swc_pack_weight_padded(ctx, b, k, n, ldb, b16, (int)kp);
    if (rc) return rc;
    return swc_fc_tc(ctx, m, n, k, a16, nullptr, (int)kp, b16, (int)kp, nullptr, SWCB200_ACT_NONE, c, nullptr, SWCB200_F32, ldc);
}
