/*
 * CPU oracle for the quantized integer inference path of N2D2.
 *
 * TEST INFRASTRUCTURE ONLY: a from-scratch restatement of the reference's CPU ("Frame") cells and
 * Scaling kernels, used by the test-suite, by the smoke check and as the timed CPU baseline of the
 * benchmark.  The product never links or calls it.
 *
 * Parity status: the reference ships no golden integer vectors or known-answer tests for this path
 * (its tests pin it at accuracy level on MNIST only).  The restatement is pinned instead against the
 * reference's own kernel translation units compiled where they lie (see refshim/), and against the
 * hand-derived known-answer vectors under tests/golden/.
 *
 * Sources followed (paths inside the reference project):
 *   src/Cell/ConvCell_Frame_Kernels.cpp:26-174   convolution + bias
 *   src/Cell/FcCell_Frame.cpp:306-333            fully connected
 *   src/Cell/PoolCell_Frame_Kernels.cpp:26-197   max / average pooling
 *   src/Cell/ElemWiseCell_Frame.cpp:116-136      element-wise sum
 *   src/Scaling_Kernels.cpp:29-199               saturate, Clip, the four scaling modes
 *   include/Activation/{Rectifier,Linear,Saturation}Activation_Frame.hpp   activation order
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include "n2d2_oracle.h"

static inline int imax(int a, int b) { return a > b ? a : b; }
static inline int iclamp(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* Output extent of a convolution: ConvCell_Frame_Kernels.cpp:37-45 */
int n2d2o_conv_out_dim(int in, int k, int stride, int pad0, int pad1, int dil)
{
    return (int)((in + pad0 + pad1 - dil * (k - 1) - 1 + stride) / (double)stride);
}

/* Output extent of a pooling cell: src/Cell/PoolCell.cpp:233-239 (symmetric padding) */
int n2d2o_pool_out_dim(int in, int pool, int stride, int pad)
{
    return (int)((in + 2 * pad - pool + stride) / (double)stride);
}

/* Clip (src/Scaling_Kernels.cpp:41-53): clip > 0 clamps to [0, clip]; clip <= 0 clamps to [clip, 0] */
static inline float n2d2o_clipf(float v, float clip)
{
    float res = 0.0f;
    if (clip > 0.0f) res = (v < 0.0f) ? 0.0f : ((v > clip) ? clip : v);
    if (clip <= 0.0f) res = (v > 0.0f) ? 0.0f : ((v < clip) ? clip : v);
    return res;
}

#define T float
#define FN(name) name##_f32
#define IS_FLOAT 1
#include "n2d2_oracle_impl.inc"
#undef T
#undef FN
#undef IS_FLOAT

#define T int64_t
#define FN(name) name##_i64
#define IS_FLOAT 0
#include "n2d2_oracle_impl.inc"
#undef T
#undef FN
#undef IS_FLOAT

/* Launchers such as torchrun export OMP_NUM_THREADS=1; the CPU baseline wants every host core. */
void n2d2o_set_num_threads(int n)
{
#ifdef _OPENMP
    extern void omp_set_num_threads(int);
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int n2d2o_num_threads(void)
{
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* src/Target/Target_CUDA_kernels.cu:44-86 (cudaGetEstimatedTarget_kernel, topN > 1): the scores of a pixel and their
 * class indices go through an exchange sort, "for x: for y: if (v[y] < v[x]) swap(x, y)", which orders the values
 * descending; among equal scores the order is whatever those exchanges leave, neither by class nor stable, so the
 * loops are restated literally.  topN == 1 (:88-104): the first maximum. */
void n2d2o_estimated_labels_topn(const int64_t* scores, size_t pixels, int nbClass, int topN, int32_t* labels, int64_t* values)
{
#pragma omp parallel for schedule(dynamic)
    for (long long p = 0; p < (long long)pixels; ++p) {
        const int64_t* in = scores + (size_t)p * nbClass;
        if (topN == 1) {
            int best = 0;
            for (int c = 1; c < nbClass; ++c)
                if (in[c] > in[best]) best = c;
            labels[p] = best;
            values[p] = in[best];
            continue;
        }
        int64_t* v = (int64_t*)malloc(sizeof(int64_t) * (size_t)nbClass);
        int32_t* idx = (int32_t*)malloc(sizeof(int32_t) * (size_t)nbClass);
        for (int c = 0; c < nbClass; ++c) { v[c] = in[c]; idx[c] = c; }
        for (int x = 0; x < nbClass; ++x)
            for (int y = 0; y < nbClass; ++y)
                if (v[y] < v[x]) {
                    const int64_t tv = v[x]; v[x] = v[y]; v[y] = tv;
                    const int32_t ti = idx[x]; idx[x] = idx[y]; idx[y] = ti;
                }
        for (int k = 0; k < topN; ++k) {
            labels[(size_t)p * topN + k] = idx[k];
            values[(size_t)p * topN + k] = v[k];
        }
        free(v);
        free(idx);
    }
}
