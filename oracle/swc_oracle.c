/*
 * swc_oracle.c -- CPU restatement of the arithmetic SWCompiler's emitted
 * inference program performs (its scalar kernel header
 * src/codegen/utils/kernels.h).
 *
 * THIS IS TEST INFRASTRUCTURE.  It is the checker the CUDA kernels are
 * compared against; nothing in the shipped library links or calls it.
 *
 * Parity status: PINNED.  Every function here is checked bit-for-bit against
 * the reference's own header compiled in place (oracle/ref_shim.cpp ->
 * oracle/_ref/libswc_ref.so) on seeded inputs, and the MLP chain reproduces the
 * reference's only known-answer fixture (top-1 labels 5 0 4 1 9 2 1 3 for
 * test/input/mnist_images_8.bin through mlp_weight{0,1}.bin, expected labels in
 * test/input/mnist_images_8.meta.txt).
 *
 * The loop nests are NOT the reference's (they are re-ordered so that rows are
 * independent and OpenMP can split them), but for every output element the
 * sequence of floating-point operations -- which products are formed, in which
 * order they are added, at which precision, where a value is rounded to float --
 * is the reference's.  Build with -ffp-contract=off so no multiply-add is fused:
 * the reference's generated Makefile uses plain `g++ -O3` on x86-64, which has no
 * FMA instructions available and therefore rounds the product and the sum
 * separately.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#if defined(_OPENMP)
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* Number of worker threads the row-parallel loops will use. */
ORC_API int orc_num_threads(void) {
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ORC_API void orc_set_num_threads(int n) {
#if defined(_OPENMP)
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/*
 * C = A.B, row-major, fp32.  Follows matrixMatrixMul_f (kernels.h:41-56):
 * C is zero-filled, then for p = 0..k-1 every C(i,j) receives
 * fl(fl(A(i,p)*B(p,j)) + C(i,j)).  The reference iterates p outermost; per
 * element that is a left-to-right sum over p starting from +0, which is what
 * the (i, p, j) nest below produces.
 */
ORC_API void orc_matmul_f32(int m, int n, int k, const float *a, int lda,
                            const float *b, int ldb, float *c, int ldc) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < m; i++) {
        float *crow = c + (size_t)i * ldc;
        for (int j = 0; j < n; j++) crow[j] = 0.f;
        for (int p = 0; p < k; p++) {
            const float aip = a[(size_t)i * lda + p];
            const float *brow = b + (size_t)p * ldb;
            for (int j = 0; j < n; j++) {
                float prod = aip * brow[j];
                crow[j] = crow[j] + prod;
            }
        }
    }
}

/* dest[r,:] = batch[r,:] + slice[:].  batchedadd_f, kernels.h:542-552. */
ORC_API void orc_bias_add_f32(float *dest, const float *batch, const float *slice,
                              size_t num_slice, size_t slice_size) {
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < num_slice; r++) {
        const size_t base = r * slice_size;
        for (size_t i = 0; i < slice_size; i++) dest[base + i] = batch[base + i] + slice[i];
    }
}

/* b = 1 - 2/(expf(2a)+1), all in float.  matrixTanh_f, kernels.h:58-64. */
ORC_API void orc_tanh_f32(int m, int n, const float *a, int lda, float *b, int ldb) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < m; i++)
        for (int j = 0; j < n; j++) {
            float x = a[(size_t)i * lda + j];
            float e = expf(x * 2.0f);
            b[(size_t)i * ldb + j] = 1.0f - 2.0f / (e + 1.0f);
        }
}

/* dest = src > 0 ? src : +0 (NaN and -0 map to +0).  relu_f, kernels.h:575-580. */
ORC_API void orc_relu_f32(const float *src, float *dest, size_t size) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < size; i++) dest[i] = (src[i] > 0) ? src[i] : 0.0f;
}

/* c = a + b.  vecAdd_f, kernels.h:592-596 (count is an int there). */
ORC_API void orc_add_f32(int size, const float *a, const float *b, float *c) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < size; i++) c[i] = a[i] + b[i];
}

/*
 * Row softmax.  matrixSoftmax_f, kernels.h:88-103: the running maximum starts
 * at A(i,0); exponentials of (x - max) are summed left to right in float; each
 * exponential is then divided by the sum.
 */
ORC_API void orc_softmax_f32(int m, int n, const float *a, int lda, float *b, int ldb) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < m; i++) {
        const float *arow = a + (size_t)i * lda;
        float *brow = b + (size_t)i * ldb;
        float mx = arow[0];
        for (int j = 0; j < n; j++) mx = (mx < arow[j]) ? arow[j] : mx;
        float sum = 0;
        for (int j = 0; j < n; j++) {
            brow[j] = expf(arow[j] - mx);
            sum += brow[j];
        }
        for (int j = 0; j < n; j++) brow[j] = brow[j] / sum;
    }
}

/*
 * Running accuracy counters.  accuracy_i, kernels.h:617-627: for every row, cnt (accum[1]) goes up by one, and
 * right_cnt (accum[0]) by one if the row's label equals any of its n predictions.
 */
ORC_API void orc_accuracy_i32(const int *pred, const int *label, int *accum, int m, int n) {
    for (int i = 0; i < m; i++) {
        accum[1] += 1;
        for (int j = 0; j < n; j++) {
            if (pred[(size_t)i * n + j] == label[i]) {
                accum[0] += 1;
                break;
            }
        }
    }
}

/*
 * Top-k column indices per row, best first.  argMax_i, kernels.h:601-613 sorts
 * (value, index) pairs with std::greater, i.e. descending by value and, among
 * equal values, descending by index: a tie goes to the HIGHER index.  Restated
 * as k rounds of selection of the lexicographically greatest pair that is
 * still below the previous winner.
 */
ORC_API void orc_argmax_i32(const float *in, int *idx, int m, int n, int top_k) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < m; i++) {
        const float *row = in + (size_t)i * n;
        float pv = 0.f;
        int pi = -1;
        for (int t = 0; t < top_k; t++) {
            int best = -1;
            float bv = 0.f;
            for (int j = 0; j < n; j++) {
                float v = row[j];
                /* candidate must sort strictly after the previous winner */
                if (pi >= 0 && !(v < pv || (v == pv && j < pi))) continue;
                if (best < 0 || v > bv || (v == bv && j > best)) {
                    best = j;
                    bv = v;
                }
            }
            idx[(size_t)i * top_k + t] = best;
            pv = bv;
            pi = best;
        }
    }
}

static inline size_t idx4(const size_t *d, size_t x, size_t y, size_t z, size_t w) {
    return ((x * d[1] + y) * d[2] + z) * d[3] + w;
}

/*
 * NHWC convolution.  conv2d_f, kernels.h:177-243 (+ conv2d_set_bias :163-175).
 * Every output element starts at bias[co]; contributions are then added one
 * product at a time in the order kx (filter row), ky (filter column), ci (input
 * channel within the group).  Taps that fall outside the image are skipped.
 * Only pads[0] (top) and pads[1] (left) are read.  Filter layout
 * [oC, kh, kw, iC/group].  The reference offsets the filter's channel index by
 * g*iC/group as well (kernels.h:208-209), which for group > 1 walks past the
 * tap's iC/group channels and, for the last taps, past the end of the filter:
 * group > 1 is undefined behaviour there.  The expression is restated as it
 * stands; only group == 1 is ever exercised.  The reference walks co, kx, ky outside the spatial
 * loops; per output element the order of additions is the same as here.
 */
ORC_API void orc_conv2d_f32(float *output, const float *input, const float *filter,
                            const float *bias, const size_t *odims, const size_t *idims,
                            const size_t *fdims, const size_t *bdims, const size_t *kernels,
                            const size_t *strides, const size_t *pads, size_t group) {
    (void)bdims;
    const size_t batch = idims[0], inC = idims[3], oC = odims[3];
    const size_t inCG = inC / group, oCG = oC / group;
    const size_t kh = kernels[0], kw = kernels[1];
    const size_t sh = strides[0], sw = strides[1];
    const size_t pt = pads[0], pl = pads[1];
    const long long rows = (long long)(batch * odims[1]);
#pragma omp parallel for schedule(static)
    for (long long row = 0; row < rows; row++) {
        const size_t n = (size_t)row / odims[1], ox = (size_t)row % odims[1];
        for (size_t oy = 0; oy < odims[2]; oy++) {
            for (size_t co = 0; co < oC; co++) {
                const size_t g = co / oCG;
                float acc = bias[co];
                for (size_t kx = 0; kx < kh; kx++) {
                    const long long ix = (long long)(ox * sh) - (long long)pt + (long long)kx;
                    if (ix < 0 || ix >= (long long)idims[1]) continue;
                    for (size_t ky = 0; ky < kw; ky++) {
                        const long long iy = (long long)(oy * sw) - (long long)pl + (long long)ky;
                        if (iy < 0 || iy >= (long long)idims[2]) continue;
                        const float *ip = input + idx4(idims, n, (size_t)ix, (size_t)iy, g * inCG);
                        const float *fp = filter + idx4(fdims, co, kx, ky, g * inCG);
                        for (size_t ci = 0; ci < inCG; ci++) {
                            float prod = ip[ci] * fp[ci];
                            acc = acc + prod;
                        }
                    }
                }
                output[idx4(odims, n, ox, oy, co)] = acc;
            }
        }
    }
}

/*
 * NHWC max pooling, values only.  maxpool_f, kernels.h:323-377: the window is
 * scanned kx then ky, the first in-range tap initialises the maximum, later
 * taps replace it only when strictly greater (so NaN never wins after the
 * first tap and the earliest of equal maxima is kept), out-of-range taps are
 * ignored, and a window with no in-range tap yields 0.
 */
ORC_API void orc_maxpool_f32(const float *input, float *output, const size_t *idims,
                             const size_t *odims, const size_t *kernels,
                             const size_t *strides, const size_t *pads) {
    const size_t kh = kernels[0], kw = kernels[1], sh = strides[0], sw = strides[1];
    const long long pt = (long long)pads[0], pl = (long long)pads[1];
    const long long rows = (long long)(idims[0] * odims[1]);
#pragma omp parallel for schedule(static)
    for (long long row = 0; row < rows; row++) {
        const size_t n = (size_t)row / odims[1], ox = (size_t)row % odims[1];
        for (size_t oy = 0; oy < odims[2]; oy++)
            for (size_t c = 0; c < idims[3]; c++) {
                int uninit = 1;
                float mx = 0;
                for (size_t kx = 0; kx < kh; kx++)
                    for (size_t ky = 0; ky < kw; ky++) {
                        long long ix = (long long)(ox * sh) - pt + (long long)kx;
                        long long iy = (long long)(oy * sw) - pl + (long long)ky;
                        if (ix < 0 || ix >= (long long)idims[1] || iy < 0 ||
                            iy >= (long long)idims[2])
                            continue;
                        float v = input[idx4(idims, n, (size_t)ix, (size_t)iy, c)];
                        if (uninit || v > mx) {
                            mx = v;
                            uninit = 0;
                        }
                    }
                output[idx4(odims, n, ox, oy, c)] = mx;
            }
    }
}

/*
 * NHWC average pooling.  avgpool_f, kernels.h:444-493: in-range taps are summed
 * kx then ky in float and the sum is divided by kh*kw, the FULL window size,
 * whether or not some taps fell in the padding.
 */
ORC_API void orc_avgpool_f32(const float *input, float *output, const size_t *idims,
                             const size_t *odims, const size_t *kernels,
                             const size_t *strides, const size_t *pads) {
    const size_t kh = kernels[0], kw = kernels[1], sh = strides[0], sw = strides[1];
    const float cnt = (float)(kh * kw);
    const long long pt = (long long)pads[0], pl = (long long)pads[1];
    const long long rows = (long long)(idims[0] * odims[1]);
#pragma omp parallel for schedule(static)
    for (long long row = 0; row < rows; row++) {
        const size_t n = (size_t)row / odims[1], ox = (size_t)row % odims[1];
        for (size_t oy = 0; oy < odims[2]; oy++)
            for (size_t c = 0; c < idims[3]; c++) {
                float sum = 0;
                for (size_t kx = 0; kx < kh; kx++)
                    for (size_t ky = 0; ky < kw; ky++) {
                        long long ix = (long long)(ox * sh) - pt + (long long)kx;
                        long long iy = (long long)(oy * sw) - pl + (long long)ky;
                        if (ix < 0 || ix >= (long long)idims[1] || iy < 0 ||
                            iy >= (long long)idims[2])
                            continue;
                        sum += input[idx4(idims, n, (size_t)ix, (size_t)iy, c)];
                    }
                output[idx4(odims, n, ox, oy, c)] = sum / cnt;
            }
    }
}

/*
 * Inference batch normalisation, NHWC.  batchnormalization_f,
 * kernels.h:496-517: (x - mean[c]) and (var[c] + eps) are float operations;
 * std::pow(float, double) promotes, so the inverse standard deviation, both
 * multiplications and the final addition are evaluated in double and the result
 * is rounded to float once.
 */
ORC_API void orc_batchnorm_f32(float *output, const float *input, const float *mean,
                               const float *var, const float *scale, const float *bias,
                               const size_t *idims, float epsilon) {
    const size_t C = idims[3];
    const long long pixels = (long long)(idims[0] * idims[1] * idims[2]);
#pragma omp parallel for schedule(static)
    for (long long p = 0; p < pixels; p++)
        for (size_t c = 0; c < C; c++) {
            const size_t i = (size_t)p * C + c;
            float centred = input[i] - mean[c];
            float veps = var[c] + epsilon;
            double r = (double)centred * pow((double)veps, -0.5) * (double)scale[c] +
                       (double)bias[c];
            output[i] = (float)r;
        }
}

/* 2-D transpose with an axis permutation.  transpose2d_f, kernels.h:533-540. */
ORC_API void orc_transpose2d_f32(const float *input, float *output, const size_t *idims,
                                 const size_t *odims, const size_t *shuffle) {
    size_t id[2];
    for (id[0] = 0; id[0] < idims[0]; id[0]++)
        for (id[1] = 0; id[1] < idims[1]; id[1]++)
            output[id[shuffle[0]] * odims[1] + id[shuffle[1]]] = input[id[0] * idims[1] + id[1]];
}

/* 4-D transpose: out[idx[shuffle]] = in[idx].  transpose4d_f, kernels.h:519-531. */
ORC_API void orc_transpose4d_f32(const float *input, float *output, const size_t *idims,
                                 const size_t *odims, const size_t *shuffle) {
    size_t id[4];
    for (id[0] = 0; id[0] < idims[0]; id[0]++)
        for (id[1] = 0; id[1] < idims[1]; id[1]++)
            for (id[2] = 0; id[2] < idims[2]; id[2]++)
                for (id[3] = 0; id[3] < idims[3]; id[3]++)
                    output[idx4(odims, id[shuffle[0]], id[shuffle[1]], id[shuffle[2]],
                                id[shuffle[3]])] = input[idx4(idims, id[0], id[1], id[2], id[3])];
}
