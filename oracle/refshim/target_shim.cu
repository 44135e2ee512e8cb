// C entry point over the reference's own Target top-N kernel (src/Target/Target_CUDA_kernels.cu), compiled from the
// reference tree where it lies by the Makefile beside this file.  TEST INFRASTRUCTURE ONLY: the GPU tests compare
// n2d2b_net_estimated_labels_topn with it.  Scores are floats holding the integer logits, [batch][class][y][x] like the
// reference's tensors; labels / values come back as [batch][topN][y][x].
#include <cuda_runtime.h>
#include "Target/Target_CUDA_kernels.hpp"

extern "C" int refshim_estimated_target(unsigned topN, unsigned nbClass, unsigned height, unsigned width, unsigned batch,
                                        const float* h_scores, float* h_values, int* h_labels)
{
    const size_t in_bytes = sizeof(float) * nbClass * height * width * batch;
    const size_t out_elems = (size_t)topN * height * width * batch;
    float *d_in = nullptr, *d_val = nullptr;
    int* d_lab = nullptr;
    int rc = 0;
    if (cudaMalloc(&d_in, in_bytes) != cudaSuccess || cudaMalloc(&d_val, out_elems * sizeof(float)) != cudaSuccess
        || cudaMalloc(&d_lab, out_elems * sizeof(int)) != cudaSuccess)
        rc = -1;
    if (!rc && cudaMemcpy(d_in, h_scores, in_bytes, cudaMemcpyHostToDevice) != cudaSuccess) rc = -2;
    if (!rc) {
        try {
            N2D2::cudaGetEstimatedTarget(topN, nbClass, height, width, batch, 0.0f, d_in, d_val, d_lab);
        } catch (...) {
            rc = -3;
        }
    }
    if (!rc && cudaDeviceSynchronize() != cudaSuccess) rc = -4;
    if (!rc && (cudaMemcpy(h_values, d_val, out_elems * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess
                || cudaMemcpy(h_labels, d_lab, out_elems * sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess))
        rc = -5;
    cudaFree(d_in);
    cudaFree(d_val);
    cudaFree(d_lab);
    return rc;
}
