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
