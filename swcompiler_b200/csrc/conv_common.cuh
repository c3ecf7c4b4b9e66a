// Pieces shared by the tensor-core convolution kernels (conv_tcgen05.cu, conv_rows_tcgen05.cu).
#pragma once
#include "tc_common.cuh"

namespace {

constexpr int ROW_PIX = 64;  // pixels per window row in shared memory (8 KiB)

__device__ __forceinline__ void add_bf16x8(float *v, const uint4 q) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int e = 0; e < 4; e++) {
        v[2 * e] += __uint_as_float(w[e] << 16);
        v[2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
    }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float *v) {
    uint4 o;
    __nv_bfloat162 *h2 = reinterpret_cast<__nv_bfloat162 *>(&o);
    h2[0] = __floats2bfloat162_rn(v[0], v[1]);
    h2[1] = __floats2bfloat162_rn(v[2], v[3]);
    h2[2] = __floats2bfloat162_rn(v[4], v[5]);
    h2[3] = __floats2bfloat162_rn(v[6], v[7]);
    return o;
}

// Position of a CTA's successive tiles, kept without divisions: the tile index advances by a fixed step, so
// image / row block / column block advance by fixed amounts with one carry each.
struct TileWalk {
    int n, rb, cb;
    int sn, srb, scb, row_blocks, col_blocks;
    __device__ __forceinline__ TileWalk(long long first, long long step, int row_blocks_, int col_blocks_)
        : row_blocks(row_blocks_), col_blocks(col_blocks_) {
        const long long per_image = (long long)row_blocks * col_blocks;
        n = (int)(first / per_image);
        int r = (int)(first - (long long)n * per_image);
        rb = r / col_blocks;
        cb = r - rb * col_blocks;
        sn = (int)(step / per_image);
        r = (int)(step - (long long)sn * per_image);
        srb = r / col_blocks;
        scb = r - srb * col_blocks;
    }
    __device__ __forceinline__ void advance() {
        cb += scb;
        rb += srb;
        n += sn;
        if (cb >= col_blocks) {
            cb -= col_blocks;
            rb++;
        }
        if (rb >= row_blocks) {
            rb -= row_blocks;
            n++;
        }
    }
};

}  // namespace
