/* CPU oracle of N2D2's quantized inference path: test infrastructure, never part of the product. */
#ifndef N2D2_ORACLE_H
#define N2D2_ORACLE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

int n2d2o_conv_out_dim(int in, int k, int stride, int pad0, int pad1, int dil);
int n2d2o_pool_out_dim(int in, int pool, int stride, int pad);
/* Target top-N of one score vector per pixel (src/Target/Target_CUDA_kernels.cu:44-86): scores [pixels][nbClass]
 * (class fastest), labels / values [pixels][topN].  topN == 1 takes the first maximum (:88-104). */
void n2d2o_estimated_labels_topn(const int64_t* scores, size_t pixels, int nbClass, int topN, int32_t* labels, int64_t* values);
int n2d2o_num_threads(void);
void n2d2o_set_num_threads(int n);

#define N2D2O_DECLARE(T, S)                                                                        \
    void n2d2o_conv_##S(const T* in, int inW, int inH, int inC, int B, const T* w, int kW, int kH, \
                        int wC, int O, const uint8_t* maps, int nbGroups, int strideX, int strideY, \
                        int padL, int padT, int padR, int padB, int dilX, int dilY, int accumulate, \
                        int refQuirks, T* out);                                                                   \
    void n2d2o_add_bias_##S(T* out, int oW, int oH, int O, int B, const T* bias);                  \
    void n2d2o_fc_##S(const T* in, int K, int B, const T* w, const T* bias, int O, T* out);        \
    void n2d2o_pool_max_##S(const T* in, int inW, int inH, int C, int B, int pW, int pH,           \
                            int strideX, int strideY, int padX, int padY, T* out);                 \
    void n2d2o_pool_avg_##S(const T* in, int inW, int inH, int C, int B, int pW, int pH,           \
                            int strideX, int strideY, int padX, int padY, int isQuantized, T* out); \
    void n2d2o_elemwise_sum_##S(const T* const* ins, int nbInputs, const T* weights,               \
                                const T* shifts, size_t n, T* out);                                \
    int n2d2o_scaling_##S(const T* in, T* out, int B, int C, int HW, int mode, const float* fscale, \
                          const int32_t* mult, int fracBits, const uint8_t* fracBitsPerCh,         \
                          const uint8_t* shift0, const uint8_t* shift1, int isClipped,             \
                          const float* clip, int nbBits, int isUnsigned);                          \
    void n2d2o_activation_##S(T* data, size_t n, int kind, float leak, float threshold);

N2D2O_DECLARE(float, f32)
N2D2O_DECLARE(int64_t, i64)

#ifdef __cplusplus
}
#endif
#endif
