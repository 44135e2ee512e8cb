// First-layer ("stem") convolution on the tensor cores: few input channels (<= 4), kernel up to 8
// wide, any stride / padding - the 7x7/2 stem of the ResNets and the 3x3/2 stem of MobileNet.
//
// With 3 channels a pixel is 3 bytes, far below the 16-byte granule of a TMA load, so this layer
// cannot use the tensor-map path of the main kernel.  Instead the input is first re-laid with 4
// bytes per pixel (pad_channels_kernel, one pass over ~150 KB per image), and four producer warps
// gather, for every output pixel and kernel row ky, the 32 contiguous bytes
// [kx = 0..7][c = 0..3] starting at input pixel (oy*s - pad + ky, ox*s - pad) straight into the
// 128-byte-swizzled K-major layout the MMA expects (one 32-byte K step per kernel row, four kernel
// rows per 128-byte row).  The weights (Cout x K, a few KB) are loaded once per CTA by TMA and stay
// resident.  One thread issues tcgen05.mma kind::i8 into a double-buffered TMEM accumulator; four
// epilogue warps run the fused 32-bit requantisation.  Every wait is bounded.
#include <cstring>
#include "kernels.h"
#include "tc_common.cuh"
#include "host_internal.h"

namespace n2d2b {

static constexpr int SBM = 128;
static constexpr int S_PROD_WARPS = 4;
static constexpr int S_EPI_WARPS = 4;
static constexpr int S_THREADS = 32 * (1 + S_PROD_WARPS + S_EPI_WARPS);   // warp 0: weights + MMA

struct StemArgs {
    const uint8_t* in4;   // [B][H][W][4]
    int B, H, W, oH, oW, N, M;
    int kH, kW, sY, sX, pT, pL;
    int nkb;              // 128-byte K blocks = ceil(kH / 4)
    int stages;
    unsigned idesc, tmem_cols;
    void* out;
    int* status;
    const int* fq;
    int cpad;
    int out_unsigned;
    int need_clamp;
};

__global__ void pad_channels_kernel(const uint8_t* __restrict__ in, int C, size_t pixels, uint32_t* __restrict__ out)
{
    for (size_t p = blockIdx.x * (size_t)blockDim.x + threadIdx.x; p < pixels; p += (size_t)gridDim.x * blockDim.x) {
        uint32_t v = 0;
        for (int c = 0; c < C; ++c) v |= (uint32_t)in[p * C + c] << (8 * c);
        out[p] = v;
    }
}

cudaError_t launch_pad_channels(const void* in, int C, size_t pixels, void* out, cudaStream_t s)
{
    if (pixels == 0) return cudaSuccess;
    size_t g = (pixels + 255) / 256;
    if (g > 148u * 64u) g = 148u * 64u;
    pad_channels_kernel<<<(unsigned)g, 256, 0, s>>>((const uint8_t*)in, C, pixels, (uint32_t*)out);
    return cudaGetLastError();
}

template <bool CLAMP>
__global__ void __launch_bounds__(S_THREADS, 1)
stem_conv_tcgen05_kernel(const __grid_constant__ CUtensorMap tmB, const StemArgs a)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int b_bytes = a.nkb * a.N * 128;                 // resident weights: [nkb][N][128]
    const int a_stage_bytes = a.nkb * SBM * 128;           // one tile of gathered activations
    unsigned char* smB = smem;
    unsigned char* smA = smem + ((b_bytes + 1023) & ~1023);
    unsigned long long* bars = (unsigned long long*)(smA + (size_t)a.stages * a_stage_bytes);
    // bars: full[stages], empty[stages], tmem_full[2], tmem_empty[2], weights
    const unsigned full0 = smem_u32(bars);
    const unsigned empty0 = full0 + 8u * a.stages;
    const unsigned tfull0 = empty0 + 8u * a.stages;
    const unsigned tempty0 = tfull0 + 16u;
    const unsigned wbar = tempty0 + 16u;
    unsigned* tmem_slot = (unsigned*)(bars + 2 * a.stages + 5);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    int* par = (int*)(((uintptr_t)(tmem_slot + 4) + 15) & ~(uintptr_t)15);   // [FAST_NP][256], 16-byte aligned for vector loads

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(full0 + 8u * s, 32 * S_PROD_WARPS);
            mbar_init(empty0 + 8u * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(tfull0 + 8u * s, 1);
            mbar_init(tempty0 + 8u * s, S_EPI_WARPS);
        }
        mbar_init(wbar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // per-channel epilogue constants: the layer has a single column block
    for (int i = threadIdx.x; i < FAST_NP * 256; i += S_THREADS) {
        const int prm = i >> 8, c = i & 255;
        par[i] = (c < a.cpad) ? __ldg(a.fq + (size_t)prm * a.cpad + c) : 0;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    const int num_tiles = (a.M + SBM - 1) / SBM;

    if (warp == 0) {
        // ------------------------------------------------------------------ weights + MMA issuer
        if (lane == 0) {
            mbar_expect_tx(wbar, (unsigned)b_bytes);
            for (int kb = 0; kb < a.nkb; ++kb)
                tma_load_2d(smem_u32(smB + (size_t)kb * a.N * 128), &tmB, wbar, kb * 128, 0);
            bool ok = mbar_wait(wbar, 0, abort_flag, a.status, 6);
            unsigned it = 0, acc_it = 0;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it, ++acc_it) {
                const unsigned as = acc_it & 1u, aph = (acc_it >> 1) & 1u;
                const int s = it % a.stages;
                const unsigned ph = (it / a.stages) & 1u;
                if (!mbar_wait(tempty0 + 8u * as, aph ^ 1u, abort_flag, a.status, 2)) { ok = false; break; }
                if (!mbar_wait(full0 + 8u * s, ph, abort_flag, a.status, 3)) { ok = false; break; }
                tc_fence_after();
                const unsigned d_tmem = tmem_base + as * (unsigned)a.N;
                for (int kb = 0; kb < a.nkb; ++kb) {
                    const unsigned long long adesc =
                        make_smem_desc(smem_u32(smA + (size_t)s * a_stage_bytes + (size_t)kb * SBM * 128), 128);
                    const unsigned long long bdesc = make_smem_desc(smem_u32(smB + (size_t)kb * a.N * 128), 128);
                    for (int k = 0; k < 4; ++k)
                        tc_mma_i8(d_tmem, adesc + (unsigned long long)(2 * k), bdesc + (unsigned long long)(2 * k), a.idesc,
                                  (kb | k) ? 1u : 0u);
                }
                tc_commit(empty0 + 8u * s);
                tc_commit(tfull0 + 8u * as);
            }
        }
    } else if (warp <= S_PROD_WARPS) {
        // ------------------------------------------------------------------ gather producers
        const int r = (warp - 1) * 32 + lane;   // tile row = output pixel
        unsigned it = 0;
        bool ok = true;
        const uint32_t* in4 = (const uint32_t*)a.in4;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
            const int s = it % a.stages;
            const unsigned ph = (it / a.stages) & 1u;
            if (!mbar_wait(empty0 + 8u * s, ph ^ 1u, abort_flag, a.status, 1)) { ok = false; break; }
            const int m = tile * SBM + r;
            const bool m_ok = m < a.M;
            int ox = 0, oy = 0, n = 0;
            if (m_ok) {
                ox = m % a.oW;
                const int t = m / a.oW;
                oy = t % a.oH;
                n = t / a.oH;
            }
            const int ix0 = ox * a.sX - a.pL, iy0 = oy * a.sY - a.pT;
            unsigned char* stage = smA + (size_t)s * a_stage_bytes;
            // one 128-byte K block (four kernel rows) at a time: all 32 loads are issued before the first
            // store so that a tile costs one memory latency per K block, not one per kernel row
            for (int kb = 0; kb < a.nkb; ++kb) {
                uint32_t w[4][8];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int ky = kb * 4 + q;
                    const int iy = iy0 + ky;
                    const bool row_ok = m_ok && ky < a.kH && iy >= 0 && iy < a.H;
                    const uint32_t* rowp = in4 + ((size_t)n * a.H + (row_ok ? iy : 0)) * a.W;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int ix = ix0 + j;
                        w[q][j] = (row_ok && j < a.kW && ix >= 0 && ix < a.W) ? __ldg(rowp + ix) : 0u;
                    }
                }
                unsigned char* rowbase = stage + (size_t)kb * SBM * 128 + (size_t)r * 128;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    // kernel row q of the block occupies 16-byte chunks 2q and 2q+1 of the 128-byte row
                    *(uint4*)(rowbase + (((2 * q + 0) ^ (r & 7)) << 4)) = make_uint4(w[q][0], w[q][1], w[q][2], w[q][3]);
                    *(uint4*)(rowbase + (((2 * q + 1) ^ (r & 7)) << 4)) = make_uint4(w[q][4], w[q][5], w[q][6], w[q][7]);
                }
            }
            // make the generic-proxy stores visible to the tensor core (async proxy), then signal
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(full0 + 8u * s);
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        unsigned acc_it = 0;
        bool ok = true;
        const bool out_unsigned = a.out_unsigned != 0;
        const uint4 zero4 = make_uint4(0, 0, 0, 0);
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++acc_it) {
            const unsigned as = acc_it & 1u, aph = (acc_it >> 1) & 1u;
            if (!mbar_wait(tfull0 + 8u * as, aph, abort_flag, a.status, 4)) { ok = false; break; }
            tc_fence_after();
            const int m = tile * SBM + row;
            const bool m_ok = m < a.M;
            const unsigned tbase = tmem_base + ((unsigned)(quad * 32) << 16) + as * (unsigned)a.N;
            uint8_t* orow = (uint8_t*)a.out + (size_t)m * a.N;
            for (int c0 = 0; c0 < a.N; c0 += 32) {
                unsigned v[32];
                tc_ld32(tbase + (unsigned)c0, v);
                tc_wait_ld_into(v);
                if (m_ok) fast_chunk<false, CLAMP>(v, par, c0, zero4, zero4, false, out_unsigned, 0, 0, orow + c0);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8u * as);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(a.tmem_cols) : "memory");
    }
}

// ----------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool stem_eligible(const ConvGeom& g)
{
    return g.groups == 1 && g.C <= 4 && g.kW <= 8 && g.kH <= 8 && g.dX == 1 && g.dY == 1 && g.O % 32 == 0 && g.O <= 256;
}

size_t stem_weight_bytes(const ConvGeom& g)
{
    const int nkb = (g.kH + 3) / 4;
    return (size_t)g.O * nkb * 128;
}

// OHWI int8 weights -> [O][nkb*128] rows whose K order matches the gather: ky*32 + kx*4 + c
void stem_arrange_weights(const ConvGeom& g, const int8_t* w_ohwi, int8_t* dst)
{
    const int nkb = (g.kH + 3) / 4;
    memset(dst, 0, stem_weight_bytes(g));
    for (int o = 0; o < g.O; ++o)
        for (int ky = 0; ky < g.kH; ++ky)
            for (int kx = 0; kx < g.kW; ++kx)
                for (int c = 0; c < g.C; ++c)
                    dst[(size_t)o * nkb * 128 + ky * 32 + kx * 4 + c] = w_ohwi[(((size_t)o * g.kH + ky) * g.kW + kx) * g.C + c];
}

int stem_make_plan(StemPlan* plan, const int8_t* d_w_arranged, const ConvGeom& g, int in_unsigned, int num_sms,
                   const char** why)
{
    static const char* kWhy = "";
    *why = kWhy;
    if (!stem_eligible(g)) { *why = "geometry outside the stem kernel"; return -1; }
    cudaDriverEntryPointQueryResult qr;
    void* fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) != cudaSuccess || !fn) {
        *why = "cuTensorMapEncodeTiled is not available from the CUDA driver";
        return -1;
    }
    memset(plan, 0, sizeof(*plan));
    plan->nkb = (g.kH + 3) / 4;
    plan->in_unsigned = in_unsigned;
    const cuuint64_t dims[2] = {(cuuint64_t)plan->nkb * 128, (cuuint64_t)g.O};
    const cuuint64_t strides[1] = {(cuuint64_t)plan->nkb * 128};
    const cuuint32_t box[2] = {128, (cuuint32_t)g.O};
    const cuuint32_t estr[2] = {1, 1};
    CUresult rc = ((EncodeTiledFn)fn)(&plan->tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)d_w_arranged, dims, strides, box,
                                      estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) { *why = "cuTensorMapEncodeTiled failed for the stem weights"; return -1; }
    const size_t b_bytes = (((size_t)plan->nkb * g.O * 128) + 1023) & ~(size_t)1023;
    const size_t a_stage = (size_t)plan->nkb * SBM * 128;
    int stages = 4;
    auto smem_for = [&](int st) { return 1024 + b_bytes + st * a_stage + (2 * st + 5) * 8 + 32 + FAST_NP * 256 * 4 + 64; };
    while (stages > 2 && smem_for(stages) > 200 * 1024) --stages;
    plan->stages = stages;
    plan->smem_bytes = smem_for(stages);
    plan->num_sms = num_sms;
    return 0;
}

cudaError_t launch_stem(const StemPlan& plan, const void* in4, const ConvGeom& g, const FastQuant& fast, void* out,
                        int* status_word, cudaStream_t s)
{
    StemArgs a;
    memset(&a, 0, sizeof(a));
    a.in4 = (const uint8_t*)in4;
    a.B = g.B; a.H = g.H; a.W = g.W; a.oH = g.oH; a.oW = g.oW; a.N = g.O;
    a.M = g.B * g.oH * g.oW;
    if (a.M == 0) return cudaSuccess;
    a.kH = g.kH; a.kW = g.kW; a.sY = g.sY; a.sX = g.sX; a.pT = g.pT; a.pL = g.pL;
    a.nkb = plan.nkb;
    a.stages = plan.stages;
    a.idesc = (2u << 4) | ((plan.in_unsigned ? 0u : 1u) << 7) | (1u << 10) | ((unsigned)(g.O >> 3) << 17)
            | ((unsigned)(SBM >> 4) << 24);
    unsigned cols = 2u * g.O, p2 = 32;
    while (p2 < cols) p2 <<= 1;
    a.tmem_cols = p2;
    a.out = out;
    a.status = status_word;
    a.fq = fast.fq;
    a.cpad = fast.cpad;
    a.out_unsigned = fast.out_unsigned;
    a.need_clamp = fast.need_clamp ? 1 : 0;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(stem_conv_tcgen05_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             227 * 1024);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(stem_conv_tcgen05_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    const int tiles = (a.M + SBM - 1) / SBM;
    const int grid = tiles < plan.num_sms ? tiles : plan.num_sms;
    if (fast.need_clamp)
        stem_conv_tcgen05_kernel<true><<<grid, S_THREADS, plan.smem_bytes, s>>>(plan.tmB, a);
    else
        stem_conv_tcgen05_kernel<false><<<grid, S_THREADS, plan.smem_bytes, s>>>(plan.tmB, a);
    return cudaGetLastError();
}

}  // namespace n2d2b

// ------------------------------------------------------------------------------------------------
// First-layer convolution for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a result: a plugin
// running inside a framework that owns the whole device heap and forbids foreign allocations, a
// real-time inference loop where an allocation's unbounded latency (and its implicit device-wide
// synchronisation) is not acceptable, or a process near its memory budget.  The normal path
// (n2d2b_net_finalize) allocates the scratch the first-layer kernel needs - the input re-laid with
// four bytes per pixel, the weights in the kernel's K order, the per-channel epilogue constants.
// This entry point keeps all three in one fixed array that lives in the library's device image:
// every GPU that loads the library holds N2D2B_NOALLOC_SCRATCH_BYTES of it until the process exits,
// which is why the size is modest and the batch it can take is bounded.
// ------------------------------------------------------------------------------------------------
static constexpr size_t NA_WEIGHT_BYTES = 256 * 256;                 // 256 outputs x 2 K blocks of 128 bytes
static constexpr size_t NA_CONST_OFFSET = NA_WEIGHT_BYTES;           // [5][256] words
static constexpr size_t NA_PAD_OFFSET = 128 * 1024;                  // re-laid input starts here
static constexpr size_t NA_SCRATCH_BYTES = NA_PAD_OFFSET + (size_t)N2D2B_NOALLOC_MAX_PIXELS * 4;
static_assert(NA_SCRATCH_BYTES == N2D2B_NOALLOC_SCRATCH_BYTES, "header and implementation disagree on the scratch size");

static __device__ __align__(256) unsigned char g_noalloc_scratch[NA_SCRATCH_BYTES];

// In host code the array's name is only a handle; its device address comes from the runtime, once per
// device, with that device current.
static unsigned char* g_noalloc_ptr[64] = {nullptr};

static int noalloc_scratch_for(int device, unsigned char** ptr)
{
    if (device < 0 || device >= 64) return n2d2b::set_error(N2D2B_ERR_INVALID, "device %d out of range", device);
    if (!g_noalloc_ptr[device]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p)
            return n2d2b::set_error(N2D2B_ERR_CUDA, "cudaGetSymbolAddress(scratch) failed: %s", cudaGetErrorString(e));
        g_noalloc_ptr[device] = (unsigned char*)p;
    }
    *ptr = g_noalloc_ptr[device];
    return 0;
}

extern "C" int n2d2b_first_conv_noalloc(int device, const void* d_input, int batch, int height, int width, int channels,
                                        int in_unsigned, const n2d2b_conv_desc* desc, const int8_t* weights,
                                        const int32_t* bias, const n2d2b_quant* quant, void* d_output,
                                        n2d2b_stream stream)
{
    using namespace n2d2b;
    if (!d_input || !d_output || !desc || !weights || !quant)
        return set_error(N2D2B_ERR_INVALID, "input, output, desc, weights and quant must not be NULL");
    if (batch < 0 || height < 1 || width < 1 || channels < 1)
        return set_error(N2D2B_ERR_INVALID, "invalid input dimensions");
    if (batch == 0) return 0;
    if (desc->weight_bits != 8) return set_error(N2D2B_ERR_INVALID, "this entry point takes 8-bit weights");
    if (desc->nb_outputs < 1 || desc->kernel_h < 1 || desc->kernel_w < 1 || desc->stride_y < 1 || desc->stride_x < 1
        || desc->pad_top < 0 || desc->pad_left < 0 || desc->pad_bottom < 0 || desc->pad_right < 0)
        return set_error(N2D2B_ERR_INVALID, "invalid convolution geometry");
    ConvGeom g;
    memset(&g, 0, sizeof(g));
    g.B = batch; g.H = height; g.W = width; g.C = channels;
    g.O = desc->nb_outputs; g.kH = desc->kernel_h; g.kW = desc->kernel_w;
    g.sY = desc->stride_y; g.sX = desc->stride_x; g.pT = desc->pad_top; g.pL = desc->pad_left;
    g.dY = desc->dilation_y; g.dX = desc->dilation_x;
    g.groups = desc->groups; g.Cg = channels; g.Og = g.O;
    g.oH = (int)((height + desc->pad_top + desc->pad_bottom - (g.kH - 1) - 1 + g.sY) / (double)g.sY);
    g.oW = (int)((width + desc->pad_left + desc->pad_right - (g.kW - 1) - 1 + g.sX) / (double)g.sX);
    if (g.oH < 1 || g.oW < 1) return set_error(N2D2B_ERR_INVALID, "convolution output would be empty");
    if (!stem_eligible(g))
        return set_error(N2D2B_ERR_INVALID,
                         "outside the first-layer kernel: needs <= 4 channels, kernel <= 8x8, no dilation or groups, "
                         "outputs a multiple of 32 and <= 256");
    const size_t pixels = (size_t)batch * height * width;
    if (pixels > (size_t)N2D2B_NOALLOC_MAX_PIXELS)
        return set_error(N2D2B_ERR_TOO_LARGE, "batch x height x width = %zu input pixels exceeds the fixed scratch of %u pixels",
                         pixels, (unsigned)N2D2B_NOALLOC_MAX_PIXELS);
    if (stem_weight_bytes(g) > NA_WEIGHT_BYTES)
        return set_error(N2D2B_ERR_TOO_LARGE, "arranged weights exceed the fixed scratch");
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return set_error(N2D2B_ERR_CUDA, "cudaSetDevice(%d) failed: %s", device, cudaGetErrorString(e));
    int sms = 148;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) sms = 148;
    unsigned char* scratch = nullptr;
    if (int rc = noalloc_scratch_for(device, &scratch)) return rc;

    // host-side preparation: epilogue constants and weights in the kernel's K order
    std::vector<int32_t> consts;
    int cpad = 0, out_unsigned = 0;
    bool need_clamp = false;
    const long long acc_bound = (long long)g.kH * g.kW * g.C * 255ll * 128ll;
    const int prc = prepare_fast_constants(quant, g.O, bias, acc_bound, consts, &cpad, &out_unsigned, &need_clamp);
    if (prc < 0) return prc;
    if (prc > 0 || cpad != 256)
        return set_error(N2D2B_ERR_INVALID,
                         "this entry point takes shift or fixed-point scalings whose products fit 32 bits and 8-bit outputs");
    std::vector<int8_t> arranged(stem_weight_bytes(g));
    stem_arrange_weights(g, weights, arranged.data());

    cudaStream_t s = (cudaStream_t)stream;
    // both copies are ordered on the caller's stream behind any earlier call that still reads the scratch;
    // the host buffers are released when this function returns, hence the synchronisation
    e = cudaMemcpyAsync(scratch, arranged.data(), arranged.size(), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(scratch + NA_CONST_OFFSET, consts.data(), consts.size() * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return set_error(N2D2B_ERR_CUDA, "copy of the layer constants failed: %s", cudaGetErrorString(e));

    StemPlan plan;
    const char* why = "";
    if (stem_make_plan(&plan, (const int8_t*)scratch, g, in_unsigned ? 1 : 0, sms, &why))
        return set_error(N2D2B_ERR_INVALID, "first-layer plan failed: %s", why);
    const void* in4 = d_input;
    if (channels != 4) {
        // every pixel of the region is rewritten in full, so nothing of an earlier call survives
        e = launch_pad_channels(d_input, channels, pixels, scratch + NA_PAD_OFFSET, s);
        if (e != cudaSuccess) return set_error(N2D2B_ERR_CUDA, "re-layout launch failed: %s", cudaGetErrorString(e));
        in4 = scratch + NA_PAD_OFFSET;
    }
    FastQuant fq;
    fq.fq = (const int*)(scratch + NA_CONST_OFFSET);
    fq.cpad = cpad;
    fq.out_unsigned = out_unsigned;
    fq.need_clamp = need_clamp;
    fq.enabled = true;
    // the status word of the bounded waits also lives in the scratch (last 16 bytes of the constants area)
    int* status = (int*)(scratch + NA_PAD_OFFSET - 16);
    e = cudaMemsetAsync(status, 0, sizeof(int), s);
    if (e == cudaSuccess) e = launch_stem(plan, in4, g, fq, d_output, status, s);
    if (e != cudaSuccess) return set_error(N2D2B_ERR_CUDA, "first-layer launch failed: %s", cudaGetErrorString(e));
    return 0;
}

