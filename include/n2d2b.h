/*
 * n2d2b.h - C ABI of the B200-native quantized integer inference path of N2D2.
 *
 * This is the whole boundary between host code (the C++ classes that keep N2D2's Cell / Scaling /
 * DeepNet names, a test harness, another language's FFI) and the CUDA kernels.  Plain pointers and
 * sizes only; every function returns 0 on success or a negative n2d2b_status, and
 * n2d2b_last_error() gives the message for the calling thread.  Nothing here throws, resets the
 * device or falls back to the CPU: without a usable GPU the calls fail.
 *
 * Citations give the interface of the reference project (CEA-LIST/N2D2) each entry point replaces.
 *
 * Data layouts
 *   activations  NHWC, int8 (signed or unsigned per tensor) or int32 (cells whose Scaling is NONE)
 *   conv weights [Cout][kH][kW][Cin/groups] int8, or packed int4 (two per byte, even element in the
 *                high nibble, each output channel's row padded to a whole byte)
 *   fc weights   [Cout][K], K running over the input tensor in NHWC order
 *   biases       int32 per output channel
 */
#ifndef N2D2B_H
#define N2D2B_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct n2d2b_net n2d2b_net;
typedef void* n2d2b_stream; /* a cudaStream_t; NULL = the legacy default stream the reference uses */

typedef enum n2d2b_status {
    N2D2B_OK = 0,
    N2D2B_ERR_INVALID = -1,     /* bad argument or unsupported configuration (std::runtime_error / domain_error in N2D2) */
    N2D2B_ERR_CUDA = -2,        /* a CUDA call failed (CHECK_CUDA_STATUS in N2D2, include/CudaUtils.hpp:52-66, minus the device reset) */
    N2D2B_ERR_STATE = -3,       /* call made in the wrong state (e.g. forward before finalize) */
    N2D2B_ERR_TIMEOUT = -4,     /* a device-side bounded wait gave up; the context stays usable */
    N2D2B_ERR_TOO_LARGE = -5    /* a size exceeds a documented maximum */
} n2d2b_status;

/* include/ScalingMode.hpp:27-34 */
typedef enum n2d2b_scaling_mode {
    N2D2B_SCALING_NONE = 0,
    N2D2B_SCALING_FLOAT_MULT = 1,
    N2D2B_SCALING_FIXED_MULT16 = 2,
    N2D2B_SCALING_FIXED_MULT32 = 3,
    N2D2B_SCALING_SINGLE_SHIFT = 4,
    N2D2B_SCALING_DOUBLE_SHIFT = 5
} n2d2b_scaling_mode;

/* include/Activation/{Linear,Rectifier,Saturation}Activation_Frame.hpp */
typedef enum n2d2b_activation {
    N2D2B_ACT_LINEAR = 0,
    N2D2B_ACT_RECTIFIER = 1,
    N2D2B_ACT_SATURATION = 2
} n2d2b_activation;

typedef enum n2d2b_pooling { N2D2B_POOL_MAX = 0, N2D2B_POOL_AVERAGE = 1 } n2d2b_pooling;
typedef enum n2d2b_dtype { N2D2B_I8 = 0, N2D2B_I32 = 1 } n2d2b_dtype;

/*
 * Per-output-channel rescale: the payload of N2D2's Scaling value type (include/Scaling.hpp:45-427;
 * factories :339-373).  All arrays have nb_channels entries and are host pointers, copied by the call.
 *   FLOAT_MULT    fscale                      y = round(Clip?(x) * fscale[c])
 *   FIXED_MULT*   mult, frac_bits             y = (round(Clip?(x)) * mult[c] + 2^(f-1)) >> f
 *   SINGLE_SHIFT  shift0                      y = (x + 2^(s-1)) >> s[c]
 *   DOUBLE_SHIFT  shift0 (a), shift1 (b)      y = (x + (x << a[c]) + 2^(b-1)) >> b[c]
 * frac_bits_per_channel (optional) overrides frac_bits channel by channel; the reference API has one
 * nbFractionalBits per Scaling object (include/Scaling.hpp:129-193), so this is an extension.
 * Clipping happens before the rescale and, as on the reference's CPU path, only in the FLOAT and FIXED
 * modes (src/Scaling_Kernels.cpp:41-53,135-136).
 */
typedef struct n2d2b_scaling {
    int32_t mode; /* n2d2b_scaling_mode */
    int32_t nb_channels;
    const float* fscale;
    const int32_t* mult;
    int32_t frac_bits;
    const uint8_t* frac_bits_per_channel;
    const uint8_t* shift0;
    const uint8_t* shift1;
    int32_t is_clipped;
    const float* clip;
} n2d2b_scaling;

/*
 * What a cell does to its accumulators on the way out: Activation::propagate =
 * Scaling (with saturation to out_bits, signed or unsigned) then the activation
 * (include/Activation/RectifierActivation_Frame.hpp:54-87).  out_unsigned is what
 * DeepNetExport::isCellOutputUnsigned (src/Export/DeepNetExport.cpp:370-388) derives from the graph;
 * here it is explicit.
 */
typedef struct n2d2b_quant {
    n2d2b_scaling scaling;
    int32_t activation;   /* n2d2b_activation */
    int32_t out_bits;     /* 1..8; ignored when scaling.mode is NONE (the output stays int32) */
    int32_t out_unsigned;
    int32_t saturation_threshold; /* N2D2B_ACT_SATURATION only */
} n2d2b_quant;

/* ConvCell creation arguments (include/Cell/ConvCell.hpp:45-55) + input wiring */
typedef struct n2d2b_conv_desc {
    int32_t input;        /* tensor id */
    int32_t nb_outputs;
    int32_t kernel_h, kernel_w;
    int32_t stride_y, stride_x;
    int32_t pad_top, pad_left, pad_bottom, pad_right;
    int32_t dilation_y, dilation_x;
    int32_t groups;       /* 1 = dense, nb_channels = depthwise */
    int32_t weight_bits;  /* 8; or 4, 2, 1 for packed weights as the export's data<N> stores them: 8 / N values per byte,
                           * the first in the highest bits, rows starting on a byte, two's complement (1 bit: 0 = -1,
                           * 1 = +1).  3-bit weights come in 4-bit containers and 5- to 7-bit ones in bytes, as the export
                           * writes them.  4-bit weights stay packed in HBM where the implicit-GEMM kernel runs the cell;
                           * 2- and 1-bit ones are widened to bytes */
} n2d2b_conv_desc;

/* PoolCell creation arguments (include/Cell/PoolCell.hpp) */
typedef struct n2d2b_pool_desc {
    int32_t input;
    int32_t pooling;      /* n2d2b_pooling */
    int32_t pool_h, pool_w;
    int32_t stride_y, stride_x;
    int32_t pad_y, pad_x;
} n2d2b_pool_desc;

typedef struct n2d2b_tensor_info {
    int32_t channels, height, width;
    int32_t dtype;        /* n2d2b_dtype */
    int32_t is_unsigned;
    int32_t producer;     /* index of the producing cell, -1 for the network input */
    int32_t readable;     /* 1 when n2d2b_net_read_tensor can return it after a forward */
} n2d2b_tensor_info;

/* n2d2b_net_finalize flags */
#define N2D2B_KEEP_ALL_OUTPUTS 1u /* every cell keeps its own output buffer (layer-by-layer parity; DeepNet::logOutputs, src/DeepNet.cpp:1729-1759) */
#define N2D2B_NO_FUSION 2u        /* do not fold ElemWise sums into the producing convolution's epilogue */
#define N2D2B_FORCE_SIMT 4u       /* CUDA-core kernels everywhere (cross-check of the tensor-core path) */
#define N2D2B_FORCE_IM2COL 8u     /* tensor-core convolutions always load activations through the im2col map */
#define N2D2B_EXACT64_EPILOGUE 16u /* tensor-core cells always use the 64-bit requantisation (cross-check of the 32-bit form) */
#define N2D2B_FORCE_PAIR 32u      /* 256-row tiles wherever their structure allows, whatever the layer's size (tests) */
#define N2D2B_FUSE_FIRST_POOL 64u /* a stride-2 first layer whose only reader is an unpadded max pooling writes the pooled tensor itself (its own output never reaches HBM); off by default: measured slower than the two kernels on one GPU */

const char* n2d2b_last_error(void);
int n2d2b_version(void);
/* Number of CUDA devices, or a negative status. Replaces CudaContext device enumeration. */
int n2d2b_device_count(void);

/* A quantized network on one GPU: the cells DeepNetQuantization::quantizeNetwork leaves behind
 * (src/DeepNetQuantization.cpp:285-388), executed in insertion order like DeepNet::propagate
 * (src/DeepNet.cpp:2660-2743).  One net per GPU; a net is not thread-safe, different nets are. */
int n2d2b_net_create(int device, n2d2b_net** net);
void n2d2b_net_destroy(n2d2b_net* net);

/* The stimuli tensor (StimuliProvider batch after the x255 / x127 range transform,
 * src/DeepNetQuantization.cpp:359-370): channels x height x width of 8-bit values. Returns tensor id 0. */
int n2d2b_net_set_input(n2d2b_net* net, int channels, int height, int width, int is_unsigned, int* tensor_id);

/* ConvCell_Frame_CUDA (src/Cell/ConvCell_Frame_CUDA.cpp:1169-1270). bias may be NULL (NoBias). */
int n2d2b_net_add_conv(n2d2b_net* net, const n2d2b_conv_desc* desc, const void* weights, const int32_t* bias,
                       const n2d2b_quant* quant, int* tensor_id);
/* FcCell_Frame_CUDA (src/Cell/FcCell_Frame_CUDA.cpp:308-427) */
int n2d2b_net_add_fc(n2d2b_net* net, int input, int nb_outputs, int weight_bits, const void* weights,
                     const int32_t* bias, const n2d2b_quant* quant, int* tensor_id);
/* PoolCell_Frame_CUDA (src/Cell/PoolCell_Frame_CUDA.cpp:234-272); average pooling truncates like the
 * quantized CPU cell (src/Cell/PoolCell_Frame_Kernels.cpp:93-95) */
int n2d2b_net_add_pool(n2d2b_net* net, const n2d2b_pool_desc* desc, int* tensor_id);
/* ElemWiseCell_Frame_CUDA, Sum with unit weights (src/Cell/ElemWiseCell_Frame_CUDA.cpp:135-228) */
int n2d2b_net_add_elemwise_sum(n2d2b_net* net, const int* inputs, int nb_inputs, const n2d2b_quant* quant,
                               int* tensor_id);
/* ScalingCell_Frame_CUDA (src/Cell/ScalingCell_Frame_CUDA.cpp:67-76) */
int n2d2b_net_add_scaling(n2d2b_net* net, int input, const n2d2b_quant* quant, int* tensor_id);

/* Allocates activations for up to max_batch images, lays weights out for the kernels, builds the TMA
 * descriptors.  Replaces Cell::initialize() + the cuDNN descriptor/algorithm set-up
 * (src/Cell/ConvCell_Frame_CUDA.cpp:153-330,786-1094). */
int n2d2b_net_finalize(n2d2b_net* net, int max_batch, unsigned flags);

/* DeepNet::propagate(inference = true) on device buffers: d_input is batch x H x W x C 8-bit values,
 * d_output receives the last cell's output (batch x its size).  Asynchronous on `stream`: the call only
 * enqueues the kernels, so a device-side wait that gave up (N2D2B_ERR_TIMEOUT) is not known when it returns;
 * n2d2b_net_check reports it. */
int n2d2b_net_forward(n2d2b_net* net, const void* d_input, int batch, void* d_output, n2d2b_stream stream);
/* Waits for the work queued on `stream` and returns N2D2B_ERR_TIMEOUT if a kernel of this network gave up on a
 * bounded wait since the last check (its outputs are then incomplete), N2D2B_ERR_CUDA if the stream failed,
 * else 0.  The reference's counterpart is the cudaDeviceSynchronize + CHECK_CUDA_STATUS after each cell when
 * timings are on (src/DeepNet.cpp:2705-2717).  n2d2b_net_forward_host, _wait, _profile and _read_tensor make
 * the same check themselves. */
int n2d2b_net_check(n2d2b_net* net, n2d2b_stream stream);
/* The same with host buffers (the reference's mInputs.synchronizeHToD / mOutputs.synchronizeDToH):
 * copies in, runs, copies out and synchronises the stream.  From 256 images on the upload is cut into
 * slices (about 128 images each, at most 8, the last one half as large) on a second stream and the leading cells run per slice while
 * later slices arrive; pinned host memory lets the copies overlap. */
int n2d2b_net_forward_host(n2d2b_net* net, const void* h_input, int batch, void* h_output, n2d2b_stream stream);
/* Number of upload slices n2d2b_net_forward_host uses: 1..8, or 0 for the automatic choice above.  Fewer are
 * used when the batch has fewer than 2 * nb_slices - 1 images (every slice holds at least one image). */
int n2d2b_net_set_slices(n2d2b_net* net, int nb_slices);
/* Streaming form of n2d2b_net_forward_host, for a caller that feeds batch after batch: the reference prepares
 * the next batch on a second host thread while the current one is inferred (src/utils/Helper.cpp:428-454,
 * StimuliProvider::future).  n2d2b_net_submit_host enqueues upload, forward pass and download of one batch and
 * returns at once; the upload goes to one of two staging buffers on a copy stream, so it runs under the forward
 * pass of the batch submitted before.  h_input must stay valid and h_output is complete only after
 * n2d2b_net_wait, which waits for everything submitted and returns the status n2d2b_net_check would.  More than
 * two batches may be submitted back to back: the third upload waits on the device for the first batch to finish.
 * Use pinned host memory (pageable memory makes the copies synchronous) and one `stream` per network. */
int n2d2b_net_submit_host(n2d2b_net* net, const void* h_input, int batch, void* h_output, n2d2b_stream stream);
int n2d2b_net_wait(n2d2b_net* net);
/* Test hook for the bounded device-side waits (no counterpart in the reference): enqueues on `stream` a one-CTA
 * kernel that waits at most limit_us microseconds (1..100000) on a barrier nobody arrives at, gives up and
 * raises this network's status word exactly as a pipeline wait of the tensor-core kernels would.  Nothing
 * faults or traps; the next n2d2b_net_check returns N2D2B_ERR_TIMEOUT and the network stays usable. */
int n2d2b_net_selftest_wait_timeout(n2d2b_net* net, unsigned limit_us, n2d2b_stream stream);

/* Output edge, Target top-1 (src/Target/Target_CUDA_kernels.cu:88-104; TargetScore): the class with the highest
 * score of the last forward pass's final tensor, per image (and per pixel when the tensor is a map); among
 * equal scores the lowest class index wins, as in the reference.  d_labels (and d_values, optional: the winning
 * scores) are device buffers of batch x height x width int32.  Asynchronous on `stream`, which must be the stream
 * of that forward pass (or ordered after it). */
int n2d2b_net_estimated_labels(n2d2b_net* net, int batch, int32_t* d_labels, int32_t* d_values, n2d2b_stream stream);
/* Target top-N (src/Target/Target_CUDA_kernels.cu:44-86): the top_n classes per image (and pixel) by descending
 * score, d_labels / d_values = batch x top_n x height x width int32 like the reference's estimatedLabels.  Among
 * equal scores the reference's exchange sort leaves the classes in an order that is neither by index nor stable;
 * this entry point returns exactly that order (evaluated in closed form, not by the quadratic sort).  top_n = 1 is
 * n2d2b_net_estimated_labels.  Up to 16384 classes. */
int n2d2b_net_estimated_labels_topn(n2d2b_net* net, int batch, int top_n, int32_t* d_labels, int32_t* d_values,
                                    n2d2b_stream stream);
/* The same into host buffers, blocking (for a caller without device memory of its own, after
 * n2d2b_net_forward_host or n2d2b_net_wait); h_values may be NULL. */
int n2d2b_net_estimated_labels_topn_host(n2d2b_net* net, int batch, int top_n, int32_t* h_labels, int32_t* h_values);
/* Input edge: the transformation quantizeNetwork puts in front of the network (src/DeepNetQuantization.cpp:359-370:
 * multiply by 2^nb_bits - 1 for unsigned stimuli, 2^(nb_bits-1) - 1 for signed ones, then truncate).  d_in holds
 * float stimuli in the reference's layout [batch][channel][y][x]; d_out receives 8-bit [batch][y][x][channel], the
 * layout n2d2b_net_forward takes.  Values outside the 8-bit range of the signedness saturate. */
int n2d2b_quantize_stimuli(int device, const float* d_in, int batch, int channels, int height, int width, int nb_bits,
                           int env_unsigned, void* d_out, n2d2b_stream stream);

int n2d2b_net_num_tensors(const n2d2b_net* net);
int n2d2b_net_tensor_info(const n2d2b_net* net, int tensor_id, n2d2b_tensor_info* info);
/* Copies a tensor of the last forward (first `batch` images) to the host. */
int n2d2b_net_read_tensor(n2d2b_net* net, int tensor_id, int batch, void* host_dst, size_t bytes);
/* Bytes of weights the network keeps in HBM (*total_bytes), and how many of them are packed 4-bit weights
 * (*packed4_bytes: cells given weight_bits = 4 that run on the implicit-GEMM kernel, which expands them tile by
 * tile in shared memory; other cells hold int8).  Either pointer may be NULL. */
int n2d2b_net_weight_bytes(const n2d2b_net* net, size_t* total_bytes, size_t* packed4_bytes);
/* Number of kernel launches one forward of `batch` images issues. */
int n2d2b_net_launches_per_forward(const n2d2b_net* net);
/* Name of the kernel family cell `cell` runs on ("tcgen05", "tcgen05-pair", "tcgen05-w4", "patch-tcgen05",
 * "stem-tcgen05", "simt", "depthwise", "pool", "sum", "fused"). */
const char* n2d2b_net_cell_engine(const n2d2b_net* net, int cell);
/* Device time of every cell of one forward, in milliseconds (CUDA events on `stream`), like the
 * per-cell timings of DeepNet::propagate (src/DeepNet.cpp:2705-2717). ms has one entry per cell. */
int n2d2b_net_profile(n2d2b_net* net, const void* d_input, int batch, void* d_output, float* ms, int nb_cells,
                      n2d2b_stream stream);

/* Stand-alone Scaling::propagate on device buffers (cuda*Scaling_propagate,
 * src/Scaling_CUDA_Kernels.cu:209-430): d_in is int32 NHWC (nb_pixels x channels), d_out int8. */
int n2d2b_scaling_propagate(int device, const int32_t* d_in, void* d_out, size_t nb_pixels,
                            const n2d2b_quant* quant, n2d2b_stream stream);

/* Issue-rate probe of the int8 tensor pipe (no counterpart in the reference; it gives the roofline denominator
 * for the convolution kernels): one CTA per multiprocessor issues `reps` tcgen05.mma kind::i8 instructions of
 * shape 128 x n x 32 back to back from shared-memory operands, no memory traffic.  *tops = dense int8 TOP/s the
 * whole GPU sustained over the launch (CUDA events), *cycles_per_mma = SM cycles per instruction on one
 * multiprocessor.  n: multiple of 16 in 16..256; reps: 64..1000000.  Allocates and frees 128 bytes. */
int n2d2b_probe_i8_mma_rate(int device, int n, int reps, double* tops, double* cycles_per_mma);

/*
 * First-layer convolution that allocates no device memory.  It has no counterpart in the reference.
 *
 * For callers that cannot call cudaMalloc where they need the result: plugins inside a host
 * framework that owns the device heap, latency-bound loops that cannot afford an allocation's
 * device-wide synchronisation, processes at their memory budget.  The scratch the kernel needs
 * (the input re-laid with 4 bytes per pixel and its zero padding written out, the re-ordered weights,
 * the per-channel constants)
 * lives in a fixed array inside the library's device image instead of in allocated memory.
 *
 *   d_input / d_output  device buffers: batch x height x width x channels 8-bit values in, batch x
 *                       oH x oW x nb_outputs 8-bit values out (same layout and arithmetic as a conv
 *                       cell added with n2d2b_net_add_conv)
 *   desc, weights, bias, quant   host data, as for n2d2b_net_add_conv (desc->input is ignored);
 *                       8-bit weights; <= 4 channels, kernel <= 8x8, no dilation or groups, nb_outputs
 *                       a multiple of 32 and <= 128, output at least 2 wide; a shift or fixed-point scaling whose products
 *                       fit 32 bits, 8-bit output
 *
 * Limits and sharing
 *   - batch x padded height x padded width must not exceed N2D2B_NOALLOC_MAX_PIXELS (else
 *     N2D2B_ERR_TOO_LARGE); the padded image is the input plus its top / left padding, extended to the
 *     last pixel any output reads and to a multiple of four pixels per row.
 *   - Every GPU that loads the library holds N2D2B_NOALLOC_SCRATCH_BYTES for this array until the
 *     process exits, whether or not this function is ever called.
 *   - All calls on a device share the one array: calls whose GPU work overlaps (different streams,
 *     different threads) race on it.  Issue them on one stream, or order them yourself.
 *   - The first call on a device looks up the array's device address; make that call before any
 *     stream capture begins.  The call copies the small layer constants and waits for that copy
 *     (a stream synchronisation), then enqueues the kernels asynchronously.
 *   - It calls no cudaMalloc, cudaFree or other allocating CUDA routine.
 *   - The kernels are enqueued asynchronously, so a device-side wait that gave up is not known when the call
 *     returns.  The status word sits in the same array; the NEXT call on that device reads it during the wait
 *     it makes anyway and returns N2D2B_ERR_TIMEOUT ("the previous call's kernel gave up...") without
 *     launching; the call after that runs normally.  The caller's current device is restored on return.
 */
#define N2D2B_NOALLOC_MAX_PIXELS (8u * 1024u * 1024u)
#define N2D2B_NOALLOC_SCRATCH_BYTES (128u * 1024u + 4u * N2D2B_NOALLOC_MAX_PIXELS)
int n2d2b_first_conv_noalloc(int device, const void* d_input, int batch, int height, int width, int channels,
                             int in_unsigned, const n2d2b_conv_desc* desc, const int8_t* weights, const int32_t* bias,
                             const n2d2b_quant* quant, void* d_output, n2d2b_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* N2D2B_H */
