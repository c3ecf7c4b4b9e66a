// Strict fp32 matrix multiply: bit-for-bit the result of matrixMatrixMul_f (kernels.h:41-56).
//
// The reference adds the products of row i of A and column j of B into C(i,j) one at a time, p
// ascending, rounding the product and the sum separately (its generated Makefile gives g++ no FMA
// to contract into).  This kernel keeps that order per output element -- the k tiles are visited in
// ascending order and the products inside a tile too -- and uses __fmul_rn / __fadd_rn so the
// compiler cannot fuse them.  64x64 output tile per CTA, 16-deep k slices through shared memory,
// a 4x4 register block per thread.  It is the checking path, not the fast one: two instructions per
// multiply-add on the FP32 pipe.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256) fc_strict_kernel(int m, int n, int k, const float *__restrict__ a, int lda,
                                                        const float *__restrict__ b, int ldb, float *__restrict__ c,
                                                        int ldc) {
    __shared__ __align__(16) float As[BK][BM];  // As[p][i]
    __shared__ __align__(16) float Bs[BK][BN];  // Bs[p][j]
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < k; k0 += BK) {
        // A tile: 64 rows x 16 k; thread t loads row t/4, k (t%4)*4 .. +3
        {
            const int r = threadIdx.x >> 2, kk = (threadIdx.x & 3) * 4;
            const int gr = row0 + r;
#pragma unroll
            for (int u = 0; u < 4; u++) {
                int gk = k0 + kk + u;
                As[kk + u][r] = (gr < m && gk < k) ? a[(size_t)gr * lda + gk] : 0.f;
            }
        }
        // B tile: 16 k x 64 cols; thread t loads k t/16, cols (t%16)*4 .. +3
        {
            const int kk = threadIdx.x >> 4, cc = (threadIdx.x & 15) * 4;
            const int gk = k0 + kk;
#pragma unroll
            for (int u = 0; u < 4; u++) {
                int gc = col0 + cc + u;
                Bs[kk][cc + u] = (gk < k && gc < n) ? b[(size_t)gk * ldb + gc] : 0.f;
            }
        }
        __syncthreads();
        const int kmax = min(BK, k - k0);
        for (int p = 0; p < kmax; p++) {
            const float4 av = *reinterpret_cast<const float4 *>(&As[p][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4 *>(&Bs[p][tx * 4]);
            const float ar[4] = {av.x, av.y, av.z, av.w};
            const float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(ar[i], br[j]));
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int gr = row0 + ty * 4 + i;
        if (gr >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int gc = col0 + tx * 4 + j;
            if (gc < n) c[(size_t)gr * ldc + gc] = acc[i][j];
        }
    }
}

// The same arithmetic for shapes whose 64 x 64 tiles would occupy only a few SMs (a batch of 64 rows, a 10-column
// classifier): 8 x 32 output tiles, one output element per thread, 128-deep k slices.  The order of the additions
// per element is unchanged (k ascending), so the result is the same bit for bit.  These shapes are bound by
// latency -- a chain of k dependent additions per element -- so the next slice is fetched into registers while
// the current one is being added up: the global loads never stand between two slices.
constexpr int SM_ROWS = 8, SM_COLS = 32, SM_K = 128;

__global__ void __launch_bounds__(256) fc_strict_small_kernel(int m, int n, int k, const float *__restrict__ a, int lda,
                                                              const float *__restrict__ b, int ldb, float *__restrict__ c,
                                                              int ldc) {
    __shared__ float As[SM_ROWS][SM_K];       // As[i][p]: read as a broadcast by the 32 threads of a row
    __shared__ float Bs[SM_K][SM_COLS + 1];   // Bs[p][j]
    const int tid = threadIdx.x, tx = tid & 31, ty = tid >> 5;
    const int row0 = blockIdx.y * SM_ROWS, col0 = blockIdx.x * SM_COLS;
    const int row = row0 + ty, col = col0 + tx;
    constexpr int A_PER = SM_ROWS * SM_K / 256, B_PER = SM_K * SM_COLS / 256;  // 4 and 16 elements per thread and slice
    float ra[A_PER], rb[B_PER];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int u = 0; u < A_PER; u++) {
            const int idx = tid + 256 * u, r = idx / SM_K, kk = idx % SM_K;
            ra[u] = (row0 + r < m && k0 + kk < k) ? a[(size_t)(row0 + r) * lda + k0 + kk] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < B_PER; u++) {
            const int idx = tid + 256 * u, kk = idx / SM_COLS, cc = idx % SM_COLS;
            rb[u] = (k0 + kk < k && col0 + cc < n) ? b[(size_t)(k0 + kk) * ldb + col0 + cc] : 0.f;
        }
    };
    float acc = 0.f;
    fetch(0);
    for (int k0 = 0; k0 < k; k0 += SM_K) {
#pragma unroll
        for (int u = 0; u < A_PER; u++) {
            const int idx = tid + 256 * u;
            As[idx / SM_K][idx % SM_K] = ra[u];
        }
#pragma unroll
        for (int u = 0; u < B_PER; u++) {
            const int idx = tid + 256 * u;
            Bs[idx / SM_COLS][idx % SM_COLS] = rb[u];
        }
        __syncthreads();
        if (k0 + SM_K < k) fetch(k0 + SM_K);  // in flight while this slice is added up
        const int kmax = min(SM_K, k - k0);
        if (kmax == SM_K) {
#pragma unroll
            for (int p = 0; p < SM_K; p++) acc = __fadd_rn(acc, __fmul_rn(As[ty][p], Bs[p][tx]));
        } else {
            for (int p = 0; p < kmax; p++) acc = __fadd_rn(acc, __fmul_rn(As[ty][p], Bs[p][tx]));
        }
        __syncthreads();
    }
    if (row < m && col < n) c[(size_t)row * ldc + col] = acc;
}

}  // namespace

int swc_fc_strict(swcb200_ctx *ctx, int m, int n, int k, const float *a, int lda, const float *b, int ldb, float *c,
                  int ldc) {
    dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM);
    if ((long long)grid.x * grid.y < ctx->sm_count / 2) {  // too few 64 x 64 tiles to fill the GPU: small tiles
        dim3 gs((n + SM_COLS - 1) / SM_COLS, (m + SM_ROWS - 1) / SM_ROWS);
        fc_strict_small_kernel<<<gs, 256, 0, ctx->stream>>>(m, n, k, a, lda, b, ldb, c, ldc);
        return swc_check_launch(ctx, "matrixMatrixMul_f(strict)");
    }
    SWC_REQUIRE(ctx, grid.y <= 65535, SWCB200_ERR_TOO_LARGE, "matrixMatrixMul_f: m beyond 4M rows in strict mode");
    fc_strict_kernel<<<grid, 256, 0, ctx->stream>>>(m, n, k, a, lda, b, ldb, c, ldc);
    return swc_check_launch(ctx, "matrixMatrixMul_f(strict)");
}
