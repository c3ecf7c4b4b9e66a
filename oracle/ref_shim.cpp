// ref_shim.cpp -- C-linkage doorway onto the UNMODIFIED reference kernel header.
//
// TEST INFRASTRUCTURE ONLY.  This file contains no arithmetic of its own: it
// includes SWCompiler's src/codegen/utils/kernels.h from the reference checkout
// where it lies (the include path is given on the compiler command line by
// oracle/Makefile; no reference source is copied into this repository) and
// forwards each forward-pass function through an extern "C" symbol so that the
// tests can call the real reference from Python, and the benchmark's reference
// arm can time it.  The built library goes to oracle/_ref/ and is not tracked.
#include <sys/types.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <iostream>
#include <random>
#include <vector>

#include "kernels.h"  // the reference's header, found via -I

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API void ref_matrixMatrixMul_f(int m, int n, int k, const float *a, int lda, const float *b,
                                   int ldb, float *c, int ldc) {
    matrixMatrixMul_f(m, n, k, a, lda, b, ldb, c, ldc);
}
REF_API void ref_batchedadd_f(float *dest, const float *batch, const float *slice,
                              size_t numSlice, size_t sliceSize) {
    batchedadd_f(dest, batch, slice, numSlice, sliceSize);
}
REF_API void ref_matrixTanh_f(int m, int n, const float *a, int lda, float *b, int ldb) {
    matrixTanh_f(m, n, a, lda, b, ldb);
}
REF_API void ref_relu_f(const float *src, float *dest, size_t size) { relu_f(src, dest, size); }
REF_API void ref_vecAdd_f(int size, float *a, float *b, float *c) { vecAdd_f(size, a, b, c); }
REF_API void ref_matrixSoftmax_f(int m, int n, const float *a, int lda, float *b, int ldb) {
    matrixSoftmax_f(m, n, a, lda, b, ldb);
}
REF_API void ref_argMax_i(const float *in, int *idx, int m, int n, int top_k) {
    argMax_i(in, idx, m, n, top_k);
}
REF_API void ref_accuracy_i(const int *pred, const int *label, int *accum, int m, int n) {
    accuracy_i(pred, label, accum, m, n);
}
REF_API void ref_conv2d_f(float *output, const float *input, const float *filter,
                          const float *bias, const size_t *odims, const size_t *idims,
                          const size_t *fdims, const size_t *bdims, const size_t *kernels,
                          const size_t *strides, const size_t *pads, size_t group) {
    conv2d_f(output, input, filter, bias, odims, idims, fdims, bdims, kernels, strides, pads,
             group);
}
REF_API void ref_maxpool_f(const float *input, float *output, const size_t *idims,
                           const size_t *odims, const size_t *kernels, const size_t *strides,
                           const size_t *pads) {
    maxpool_f(input, output, idims, odims, kernels, strides, pads);
}
REF_API void ref_avgpool_f(const float *input, float *output, const size_t *idims,
                           const size_t *odims, const size_t *kernels, const size_t *strides,
                           const size_t *pads) {
    avgpool_f(input, output, idims, odims, kernels, strides, pads);
}
REF_API void ref_batchnormalization_f(float *output, const float *input, const float *mean,
                                      const float *var, const float *scale, const float *bias,
                                      const size_t *idims, float epsilon) {
    batchnormalization_f(output, input, mean, var, scale, bias, idims, epsilon);
}
REF_API void ref_transpose2d_f(const float *input, float *output, const size_t *idims,
                               const size_t *odims, const size_t *shuffle) {
    transpose2d_f(input, output, idims, odims, shuffle);
}
REF_API void ref_transpose4d_f(const float *input, float *output, const size_t *idims,
                               const size_t *odims, const size_t *shuffle) {
    transpose4d_f(input, output, idims, odims, shuffle);
}
