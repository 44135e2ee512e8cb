// Host-side launch interface of the CUDA kernels (internal to the library).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "common.cuh"

namespace n2d2b {

struct ConvGeom {
    int B, H, W, C;      // input, NHWC
    int oH, oW, O;       // output, NHWC
    int kH, kW, sY, sX, pT, pL, dY, dX;
    int groups, Cg, Og;  // channels / outputs per group
};

struct PoolGeom {
    int B, H, W, C, oH, oW;
    int pH, pW, sY, sX, padY, padX;
    int is_max;
};

struct SumInputs {
    const void* ptr[4];
    int dtype[4];
    int is_unsigned[4];
    int n;
};

// Fused residual: after the cell's own requantisation t, out = requant2(t + res)
struct Residual {
    const void* ptr;   // int8 NHWC, same shape as the output; nullptr = none
    int is_unsigned;
    QuantDev q2;
};

// CUDA-core direct convolution (any geometry, groups, dilation); weights OHWI int8.
cudaError_t launch_conv_direct(const void* in, int in_unsigned, const int8_t* w, const ConvGeom& g,
                               const QuantDev& q, const Residual& r, void* out, int out_dtype,
                               cudaStream_t s);
// Depthwise convolution, C % 16 == 0; weights re-laid as [kH][kW][C].
struct FastQuant;
// `fast` (when enabled): the proved 32-bit rescale; 3x3 filters then take the dot-product kernel
cudaError_t launch_conv_depthwise(const void* in, int in_unsigned, const int8_t* w_hwc, const ConvGeom& g,
                                  const QuantDev& q, const FastQuant& fast, void* out, cudaStream_t s);
cudaError_t launch_pool(const void* in, int in_unsigned, const PoolGeom& g, void* out, cudaStream_t s);
cudaError_t launch_pool_i32(const void* in, const PoolGeom& g, void* out, cudaStream_t s);
cudaError_t launch_elemwise_sum(const SumInputs& ins, size_t pixels, int C, const QuantDev& q,
                                void* out, int out_dtype, cudaStream_t s);
// Top-1 class per pixel (first maximum wins) of [pixels][C] scores; values may be nullptr.
// [rows][ld] bytes -> [rows][C] bytes (C <= ld): drops the zero columns a padded cell computed
cudaError_t launch_drop_padded_columns(const uint8_t* src, int ld, uint8_t* dst, int C, size_t rows, cudaStream_t s);
// labels / values: [images][topN][hw]; pixels = images * hw score vectors of C entries; C <= 16384
cudaError_t launch_topn(const void* scores, int dtype, int is_unsigned, size_t pixels, size_t hw, int C, int topN, int32_t* labels,
                        int32_t* values, cudaStream_t s);
cudaError_t launch_argmax(const void* scores, int dtype, int is_unsigned, size_t pixels, int C, int32_t* labels, int32_t* values,
                          cudaStream_t s);
// Float stimuli NCHW -> trunc(x * factor) clamped to [lo, hi], 8-bit NHWC.
cudaError_t launch_quantize_stimuli(const float* in, int B, int C, int H, int W, float factor, int lo, int hi, void* out, cudaStream_t s);
// Fully connected on CUDA cores: in [B][K], w [O][K] int8.
cudaError_t launch_fc_direct(const void* in, int in_unsigned, const int8_t* w, int B, int K, int O,
                             const QuantDev& q, void* out, int out_dtype, cudaStream_t s);

// Per-channel constants of the 32-bit epilogue y = (clamp(acc, lo, hi) * mult + add) >> shift, which is
// exact whenever the host could bound every intermediate to 32 bits (see build_fast_quant in net.cu).
struct FastQuant {
    const int* fq = nullptr;    // [5][cpad]: lo, hi, mult, add, shift of the cell
    const int* fq2 = nullptr;   // the same for a fused residual sum
    int cpad = 0;
    int t_lo = 0, t_hi = 0;     // range the cell's own output saturates to
    int out_unsigned = 0;       // final 8-bit range
    bool need_clamp = true;     // false: no product can leave 32 bits and saturation is the final pack's
    bool wide = false;          // first rescale in 64 bits: row 0 of fq holds the upper words of the addends (no clamps)
    bool dp4a = false;          // residual stage as a byte dot product (multipliers <= 255, native 8-bit ranges)
    bool dp_t_unsigned = false; //   the cell's own output is packed as unsigned bytes (natively, or shifted by +128)
    unsigned dp_xor = 0;        //   bytes to flip from unsigned to signed (0x80 per byte)
    int dp_a_signed = 1;        //   signedness of the (t, r) byte vector
    bool enabled = false;
};

// ---- stride-2 first layer through space-to-depth (tcgen05 kind::i8, no gather) ----
struct StemS2dPlan {
    CUtensorMap tmA;      // re-laid image [B][Hs][Ws][16] as (8-byte words, rows, images); box = one band
    const int8_t* w;      // weights in the canonical unswizzled K-major layout (device)
    int BN, KH, KWp, Wp;
    int R, bands;
    int row_stride;       // convolution rows between bands
    int pool_k, pool_s, P, pool_oH, pool_oW;   // fused max pooling (P = pooled rows per band; 0 = none)
    int cbuf_alloc;       // bytes of one band-sized output buffer of the fused pooling
    int band_bytes, band_alloc, w_bytes;
    int in_unsigned;
    int num_sms;
    size_t smem_bytes;
};
bool stem_s2d_eligible(const ConvGeom& g);
bool stem_s2d_pool_eligible(const ConvGeom& g, const PoolGeom& p);
void stem_s2d_dims(const ConvGeom& g, int* Hs, int* Ws);
size_t stem_s2d_weight_bytes(const ConvGeom& g);
void stem_s2d_arrange_weights(const ConvGeom& g, const int8_t* w_ohwi, int8_t* dst);
cudaError_t launch_s2d_image(const void* in, const ConvGeom& g, int batch, void* out, cudaStream_t s);
// pool: a max pooling folded into the kernel (stem_s2d_pool_eligible); `out` of the launch is then the pooled tensor
int stem_s2d_make_plan(StemS2dPlan* plan, const void* d_s2d, const int8_t* d_w_arranged, const ConvGeom& g, int max_batch,
                       int in_unsigned, int num_sms, const char** why, const PoolGeom* pool = nullptr);
cudaError_t launch_stem_s2d(const StemS2dPlan& plan, const ConvGeom& g, int n_base, const FastQuant& fast, void* out,
                            int* status_word, cudaStream_t s);

// ---- stride-1 convolution from a shared-memory input patch (tcgen05 kind::i8) ----
struct PatchPlan {
    CUtensorMap tmA;      // NHWC activations, box = one patch: C x Wp x (R + halo rows) x 1 image
    CUtensorMap tmB;      // weights [O][taps*C], box = one tap of all outputs
    int BN;               // accumulator columns: 64 or 128
    int Wp;               // patch width in pixels: oW + (kW-1)*dX
    int R, bands;         // output rows per band, bands per image
    int patch_bytes;      // bytes of one patch load
    int patch_alloc;      // bytes reserved per patch buffer
    int b_stream;         // weights stream through a ring (too large to stay resident)
    int bring;            // slots of that ring (one filter tap each)
    int stage_cols;       // columns an epilogue warp stages per pass
    int in_unsigned;
    int num_sms;
    int G;                // channel groups: 1, or the block-diagonal groups of a depthwise layer
    size_t smem_bytes;
};
// dense stride-1 layers with 32 / 64 / 128 input channels, and depthwise stride-1 layers whose channels are a
// multiple of 32 (run as block-diagonal groups of 64 or 32 channels)
bool patch_eligible(const ConvGeom& g);
int patch_groups(const ConvGeom& g);
size_t patch_dw_weight_bytes(const ConvGeom& g);
void patch_dw_arrange_weights(const ConvGeom& g, const int8_t* w_ct, int8_t* dst);
void patch_permute_weights(const int8_t* w, int8_t* dst, int O, size_t row_bytes);
int patch_make_plan(PatchPlan* plan, const void* in, const int8_t* w, const ConvGeom& g, int in_unsigned, int num_sms,
                    const char** why);
// n_base: first image of this call within the tensors the plan was encoded for (`out` = the tensor's base)
cudaError_t launch_patch(const PatchPlan& plan, const ConvGeom& g, int n_base, const FastQuant& fast, void* out,
                         int* status_word, cudaStream_t s);

// ---- tensor-core implicit GEMM (tcgen05 kind::i8) ----
struct IgemmPlan {
    CUtensorMap tmA;      // activations: 2-D tiled [M][K] or 4-D im2col NHWC
    CUtensorMap tmB;      // weights [N][Ktot], K-major
    CUtensorMap tmO;      // output [M][N] bytes, box = 32 rows x BN/2 (TMA store of the epilogue)
    CUtensorMap tmR;      // residual operand, same geometry (TMA load of the epilogue)
    int has_out_maps;
    int a_im2col;         // 0: 2-D tiled, 1: im2col
    int M, N;             // GEMM extents (output pixels, output channels)
    int Cin, taps;        // K = taps * Cin, walked tap by tap
    int BK;               // bytes of K per pipeline stage: 32, 64 or 128 (also the swizzle width)
    int BN;               // tile N: 64, 128 or 256
    int stages;
    int grouped;          // depthwise layer as block-diagonal groups: column block n reads input channels [n * BN, (n + 1) * BN)
    int b_resident;       // weights of the CTA's column block stay in shared memory for the whole launch
    int res_slots;        // fused residual: staging regions per epilogue warp (2 or 4), 0 without a residual
    int w4;               // weights are packed 4-bit values in HBM ([N][Ktot / 2] bytes, even element in the high nibble)
    int perm;             // weight rows stored permuted inside blocks of this many output channels (32 or 16; 0 = not)
    int pair;             // large-K layer with 256-column tiles: CTAs take two 128-row tiles per weight slab
    CUtensorMap tmO32;    // output [M][N] bytes, box = 32 rows x 32 columns (the pair kernel's two-pass store)
    size_t pair_smem_bytes;
    int a_unsigned;
    // im2col geometry
    int oW, oH, kW, sX, sY, pL, pT, dX, dY;
    int grid;             // CTAs to launch
    size_t smem_bytes;
};
// depthwise layers the kernel takes as block-diagonal groups (channels a multiple of 64, or 32): channels per group,
// bytes and layout of the block-diagonal weight matrix [C][taps][group]
int igemm_dw_group(const ConvGeom& g);
size_t igemm_dw_weight_bytes(const ConvGeom& g);
void igemm_dw_arrange_weights(const ConvGeom& g, const int8_t* w_ct, int8_t* dst);
// Encodes the tensor maps for `in`/`w` and fills the tiling. Returns 0, or -1 with `why` set.
// force_pair: take the 256-row variant wherever its structure allows, whatever the layer's size (tests)
int igemm_make_plan(IgemmPlan* plan, const void* in, const int8_t* w, const void* out, const void* res,
                    const ConvGeom& g, int in_unsigned, int force_im2col, int force_bn, int num_sms, const char** why,
                    int force_pair = 0, int w4 = 0);
// Whether a launch of this plan takes the 32-bit epilogue; such a cell's weight rows must be stored in the
// permuted order (igemm_permute_weights with igemm_perm_block(plan)) and plan.perm set to that block size.
bool igemm_uses_fast_epilogue(const IgemmPlan& plan, const FastQuant& fast, bool has_residual, int out_dtype);
int igemm_perm_block(const IgemmPlan& plan);
void igemm_permute_weights(const int8_t* w, int8_t* dst, int N, size_t row_bytes, int perm_block);
// m_base: first output row (pixel) of this call within the tensors the plan was encoded for; `out` and the
// residual stay the tensors' base pointers
cudaError_t launch_igemm(const IgemmPlan& plan, const QuantDev& q, const Residual& r, const FastQuant& fast,
                         void* out, int out_dtype, int m_base, int* status_word, cudaStream_t s);

// ---- first-layer convolution (<= 4 input channels) on the tensor cores ----
struct StemPlan {
    CUtensorMap tmB;      // arranged weights [O][nkb*128]
    void* encode;         // cuTensorMapEncodeTiled (the output map is encoded per launch)
    int nkb;
    int BN;
    int stages;
    int in_unsigned;
    int num_sms;
    size_t smem_bytes;
};
bool stem_eligible(const ConvGeom& g);
size_t stem_weight_bytes(const ConvGeom& g);
void stem_arrange_weights(const ConvGeom& g, const int8_t* w_ohwi, int8_t* dst);
int stem_make_plan(StemPlan* plan, const int8_t* d_w_arranged, const ConvGeom& g, int in_unsigned, int num_sms,
                   const char** why);
// Re-lays [pixels][C] (C <= 4) as [pixels][4] with zero fill.
// [batch][H][W][C] -> [batch][Hp][Wp][4] with the zero padding written out (dimensions from stem_padded_dims)
void stem_padded_dims(const ConvGeom& g, int* Hp, int* Wp);
cudaError_t launch_pad_image(const void* in, const ConvGeom& g, int batch, void* out, cudaStream_t s);
cudaError_t launch_stem(const StemPlan& plan, const void* in4, const ConvGeom& g, const FastQuant& fast, void* out,
                        int* status_word, cudaStream_t s);

}  // namespace n2d2b
