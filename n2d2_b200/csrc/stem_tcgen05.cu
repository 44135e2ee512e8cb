// First-layer ("stem") convolution on the tensor cores: few input channels (<= 4), kernel up to 8
// wide, any stride / padding - the 7x7/2 stem of the ResNets and the 3x3/2 stem of MobileNet.
//
// With 3 channels a pixel is 3 bytes, far below the 16-byte granule of a TMA load, so this layer
// cannot use the tensor-map path of the main kernel.  Instead the input is first re-laid with 4
// bytes per pixel and its zero padding written out (pad_image_kernel, one pass over ~200 KB per
// image), so that the gather needs no bounds checks: eight producer warps (two threads per output
// pixel) read, for every kernel row ky, the 32 contiguous bytes [kx = 0..7][c = 0..3] starting at
// padded pixel (oy*s + ky, ox*s) and store them straight into the 128-byte-swizzled K-major layout
// the MMA expects (one 32-byte K step per kernel row, four kernel rows per 128-byte row).  Taps beyond
// the kernel width meet zero weights.  The weights (Cout x K, a few KB) are loaded once per CTA by TMA
// and stay resident.  One thread issues tcgen05.mma kind::i8 into a double-buffered TMEM accumulator;
// eight epilogue warps run the fused 32-bit requantisation and store through TMA.  Every wait is
// bounded.  A producer is a long chain of dependent instructions on few warps, so its instruction
// count per tile, not memory, sets the pace: hence the padded image, 8-byte loads where the stride
// allows, and multiplications by reciprocals instead of divisions.
#include <cstring>
#include <atomic>
#include <mutex>
#include "kernels.h"
#include "tc_common.cuh"
#include "host_internal.h"

namespace n2d2b {

static constexpr int SBM = 128;
static constexpr int S_PROD_WARPS = 8;     // two threads per tile row
static constexpr int S_EPI_WARPS = 8;      // 4 TMEM lane quadrants x 2 row halves
static constexpr int S_THREADS = 32 * (1 + S_PROD_WARPS + S_EPI_WARPS);   // warp 0: weights + MMA

struct StemArgs {
    const uint8_t* in4;   // zero-padded input [B][Hp][Wp][4]
    int B, Hp, Wp, oH, oW, N, M, BN;
    unsigned rcp_oW;            // ceil(2^32 / oW): exact quotients for the image sizes accepted
    unsigned step_n, step_rem;  // (gridDim.x * 128) / (oH*oW) and the remainder: a tile step in (image, pixel) terms
    int kH, sY, sX;
    int nkb;              // 128-byte K blocks = ceil(kH / 4)
    int stages;
    unsigned idesc, tmem_cols;
    int* status;
    const int* fq;
    int cpad;
    int out_unsigned;
    int wide;
};

// [B][H][W][C] (C <= 4) -> [B][Hp][Wp][4] with the image at (pT, pL) and zeros elsewhere.
// A block takes PAD_ROWS padded rows at a time, every thread one pixel column of each: the loads of the
// rows are independent, so several are in flight per thread.
static constexpr int PAD_ROWS = 4;
__global__ void pad_image_kernel(const uint8_t* __restrict__ in, int C, int H, int W, int Hp, int Wp, int pT, int pL,
                                 int rows, uint32_t* __restrict__ out)
{
    for (int row0 = blockIdx.x * PAD_ROWS; row0 < rows; row0 += gridDim.x * PAD_ROWS) {
        const uint8_t* irow[PAD_ROWS];
#pragma unroll
        for (int j = 0; j < PAD_ROWS; ++j) {
            const int row = row0 + j;
            const int n = row / Hp, y = row - n * Hp - pT;
            irow[j] = (row < rows && y >= 0 && y < H) ? in + ((size_t)n * H + y) * (size_t)W * C : nullptr;
        }
        for (int xp = threadIdx.x; xp < Wp; xp += blockDim.x) {
            const int x = xp - pL;
            const bool inside = x >= 0 && x < W;
            uint32_t v[PAD_ROWS];
#pragma unroll
            for (int j = 0; j < PAD_ROWS; ++j) {
                v[j] = 0u;
                if (inside && irow[j]) {
                    const uint8_t* p = irow[j] + (size_t)x * C;
                    if (C == 4) v[j] = __ldg((const uint32_t*)p);
                    else if (C == 3) v[j] = __ldg(p) | ((uint32_t)__ldg(p + 1) << 8) | ((uint32_t)__ldg(p + 2) << 16);
                    else if (C == 2) v[j] = __ldg(p) | ((uint32_t)__ldg(p + 1) << 8);
                    else v[j] = __ldg(p);
                }
            }
#pragma unroll
            for (int j = 0; j < PAD_ROWS; ++j)
                if (row0 + j < rows) out[(size_t)(row0 + j) * Wp + xp] = v[j];
        }
    }
}

void stem_padded_dims(const ConvGeom& g, int* Hp, int* Wp)
{
    *Hp = (g.oH - 1) * g.sY + ((g.kH + 3) / 4) * 4;   // every K block reads four kernel rows
    if (*Hp < g.H + g.pT) *Hp = g.H + g.pT;
    int w = (g.oW - 1) * g.sX + 8;                    // every kernel row reads eight pixels
    if (w < g.W + g.pL) w = g.W + g.pL;
    *Wp = (w + 3) & ~3;                               // rows stay 16-byte multiples
}

cudaError_t launch_pad_image(const void* in, const ConvGeom& g, int batch, void* out, cudaStream_t s)
{
    int Hp, Wp;
    stem_padded_dims(g, &Hp, &Wp);
    const long long rows = (long long)batch * Hp;
    if (rows == 0) return cudaSuccess;
    const long long blocks = (rows + PAD_ROWS - 1) / PAD_ROWS;
    const unsigned grid = (unsigned)(blocks < (1ll << 20) ? blocks : (1ll << 20));
    const int threads = Wp >= 256 ? 256 : ((Wp + 31) / 32) * 32;
    pad_image_kernel<<<grid, threads, 0, s>>>((const uint8_t*)in, g.C, g.H, g.W, Hp, Wp, g.pT, g.pL, (int)rows,
                                             (uint32_t*)out);
    return cudaGetLastError();
}

// VEC8: the first pixel of every row read is 8-byte aligned (even stride), so a row is four 8-byte loads
template <bool CLAMP, bool VEC8>
__global__ void __launch_bounds__(S_THREADS, 1)
stem_conv_tcgen05_kernel(const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmO, const StemArgs a)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int b_bytes = a.nkb * a.BN * 128;                // resident weights: [nkb][BN][128]
    const int a_stage_bytes = a.nkb * SBM * 128;           // one tile of gathered activations
    unsigned char* smB = smem;
    unsigned char* smA = smem + ((b_bytes + 1023) & ~1023);
    unsigned char* stage_out = smA + (size_t)a.stages * a_stage_bytes;
    const int region_bytes = 16 * a.BN;                    // staging of one epilogue warp: 32 rows x BN/2 bytes
    unsigned long long* bars = (unsigned long long*)(stage_out + S_EPI_WARPS * region_bytes);
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
            mbar_init(full0 + 8u * s, S_PROD_WARPS);
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
                tma_load_2d(smem_u32(smB + (size_t)kb * a.BN * 128), &tmB, wbar, kb * 128, 0);
            bool ok = mbar_wait(wbar, 0, abort_flag, a.status, 6);
            const unsigned desc_hi = (unsigned)(make_smem_desc(0u, 128) >> 32);
            const unsigned a_lo0 = (smem_u32(smA) & 0x3ffffu) >> 4, b_lo = (smem_u32(smB) & 0x3ffffu) >> 4;
            const unsigned stage16 = (unsigned)(a_stage_bytes >> 4), kb16 = (unsigned)((SBM * 128) >> 4);
            const unsigned bkb16 = (unsigned)((a.BN * 128) >> 4);
            const int k1 = a.nkb > 1 ? a.kH - 4 : 0;   // kernel rows (32-byte K steps) in the second K block
            const int k0 = a.nkb > 1 ? 4 : a.kH;       // and in the first
            int s = 0;
            unsigned ph = 0, acc_it = 0, a_lo = a_lo0;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++acc_it) {
                const unsigned as = acc_it & 1u, aph = (acc_it >> 1) & 1u;
                if (!mbar_wait(tempty0 + 8u * as, aph ^ 1u, abort_flag, a.status, 2)) { ok = false; break; }
                if (!mbar_wait(full0 + 8u * s, ph, abort_flag, a.status, 3)) { ok = false; break; }

                tc_fence_after();
                const unsigned d_tmem = tmem_base + as * (unsigned)a.BN;
                // one 32-byte K step per kernel row; unrolled with compile-time offsets and a bound check
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (k < k0) tc_mma_i8_lohi(d_tmem, a_lo + 2u * k, b_lo + 2u * k, desc_hi, a.idesc, k ? 1u : 0u);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (k < k1) tc_mma_i8_lohi(d_tmem, a_lo + kb16 + 2u * k, b_lo + bkb16 + 2u * k, desc_hi, a.idesc, 1u);
                tc_commit(empty0 + 8u * s);
                tc_commit(tfull0 + 8u * as);
                a_lo += stage16;
                if (++s == a.stages) { s = 0; ph ^= 1u; a_lo = a_lo0; }
            }
        }
    } else if (warp <= S_PROD_WARPS) {
        // ------------------------------------------------------------------ gather producers
        const int pt = (warp - 1) * 32 + lane;  // 0..255
        const int r = pt & 127;                 // tile row = output pixel
        const int h = pt >> 7;                  // kernel rows 2h and 2h+1 of every K block
        int s = 0;
        unsigned ph = 0;
        const size_t row_bytes = (size_t)a.Wp * 4;
        // this thread's part of a stage: 16-byte chunks 4h .. 4h+3 of row r in every K block
        const unsigned sw = (unsigned)(r & 7);
        unsigned char* const my_row = smA + (size_t)r * 128;
        // (image, pixel within the image) of this thread's row, advanced tile by tile without a division
        const unsigned oHW = (unsigned)(a.oH * a.oW);
        unsigned m = blockIdx.x * SBM + r;
        unsigned n = m / oHW;
        unsigned rem = m - n * oHW;
        // The loads of a tile are issued one tile ahead of its stores (two register sets, ping-pong), so the
        // global-memory latency of tile t+1 overlaps the stores of tile t instead of adding to them.
        auto issue = [&](uint32_t (&w)[2][2][8]) {
            // rows past the end repeat the last pixel; they are never stored
            const unsigned nn = m < (unsigned)a.M ? n : (unsigned)a.B - 1u;
            const unsigned rr = m < (unsigned)a.M ? rem : oHW - 1u;
            const unsigned oy = __umulhi(rr, a.rcp_oW);
            const unsigned ox = rr - oy * (unsigned)a.oW;
            const unsigned char* src = a.in4 + ((size_t)nn * a.Hp + (size_t)oy * a.sY + 2 * h) * row_bytes + (size_t)ox * a.sX * 4;
#pragma unroll
            for (int kb = 0; kb < 2; ++kb) {
                if (kb < a.nkb) {
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const unsigned char* rp = src + (size_t)(kb * 4 + q) * row_bytes;
                        if (VEC8) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const uint2 v = __ldg((const uint2*)rp + j);
                                w[kb][q][2 * j] = v.x;
                                w[kb][q][2 * j + 1] = v.y;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j) w[kb][q][j] = __ldg((const uint32_t*)rp + j);
                        }
                    }
                }
            }
            // next tile of this CTA
            m += gridDim.x * SBM;
            n += a.step_n;
            rem += a.step_rem;
            if (rem >= oHW) { rem -= oHW; ++n; }
        };
        auto flush = [&](const uint32_t (&w)[2][2][8]) -> bool {
            if (!mbar_wait_warp(empty0 + 8u * s, ph ^ 1u, abort_flag, a.status, 1, lane)) return false;
            unsigned char* dst = my_row + (size_t)s * a_stage_bytes;
#pragma unroll
            for (int kb = 0; kb < 2; ++kb) {
                if (kb < a.nkb) {
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        // kernel row c of the block occupies 16-byte chunks 2c and 2c+1 of the 128-byte row
                        const unsigned c = (unsigned)(2 * h + q);
                        unsigned char* rowbase = dst + (size_t)kb * SBM * 128;
                        *(uint4*)(rowbase + (((2 * c + 0) ^ sw) << 4)) =
                            make_uint4(w[kb][q][0], w[kb][q][1], w[kb][q][2], w[kb][q][3]);
                        *(uint4*)(rowbase + (((2 * c + 1) ^ sw) << 4)) =
                            make_uint4(w[kb][q][4], w[kb][q][5], w[kb][q][6], w[kb][q][7]);
                    }
                }
            }
            // make the generic-proxy stores visible to the tensor core (async proxy), then signal
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(full0 + 8u * s);
            if (++s == a.stages) { s = 0; ph ^= 1u; }
            return true;
        };
        uint32_t wa[2][2][8], wb[2][2][8];
        int tile = blockIdx.x;
        if (tile < num_tiles) issue(wa);
        while (tile < num_tiles) {
            if (tile + (int)gridDim.x < num_tiles) issue(wb);
            if (!flush(wa)) break;
            tile += gridDim.x;
            if (tile >= num_tiles) break;
            if (tile + (int)gridDim.x < num_tiles) issue(wa);
            if (!flush(wb)) break;
            tile += gridDim.x;
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        const int ew = warp - (1 + S_PROD_WARPS);
        const int quad = warp & 3;
        const int cp = (ew >> 2) & 1;           // column half of the tile
        unsigned acc_it = 0;
        EpiState est;
        frag_rowbase(est.rb, a.BN >> 1, lane);
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++acc_it) {
            const unsigned as = acc_it & 1u, aph = (acc_it >> 1) & 1u;
            EpiTile e;
            e.tmem_acc = tmem_base + as * (unsigned)a.BN;
            e.BN = a.BN; e.N = a.N; e.M = a.M; e.m0 = tile * SBM; e.n0 = 0;
            e.wp = a.BN >> 1;
            e.par_off = (unsigned)((unsigned char*)par - smem_raw);
            e.region_off = (unsigned)(stage_out - smem_raw) + (unsigned)(ew * region_bytes);
            e.region_stride = 0;
            e.slot_shift = 0;
            e.rbar = 0;
            e.tfull = tfull0 + 8u * as; e.tfull_parity = aph; e.tempty = tempty0 + 8u * as;
            e.abort_flag = abort_flag; e.status = a.status;
            e.ef = (a.out_unsigned ? EF_OUT_UNSIGNED : 0) | (a.wide ? EF_WIDE : 0);
            e.t_lo = 0; e.t_hi = 0; e.dp_xor = 0;
            if (!fast_epilogue_tile<false, CLAMP, false>(&tmO, &tmO, e, quad, cp, lane, est)) break;
        }
        if (lane == 0) bulk_wait_all();
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
    // the pixel decomposition multiplies by ceil(2^32 / oW): exact while oH * oW * oW < 2^32
    return g.groups == 1 && g.C <= 4 && g.kW <= 8 && g.kH <= 8 && g.dX == 1 && g.dY == 1 && g.O % 32 == 0 && g.O <= 128
           && g.oW >= 2 && (long long)g.oH * g.oW * g.oW < (1ll << 32);
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
    plan->BN = g.O <= 64 ? 64 : 128;
    const cuuint32_t box[2] = {128, (cuuint32_t)plan->BN};   // rows beyond the outputs read as zero
    const cuuint32_t estr[2] = {1, 1};
    CUresult rc = ((EncodeTiledFn)fn)(&plan->tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)d_w_arranged, dims, strides, box,
                                      estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) { *why = "cuTensorMapEncodeTiled failed for the stem weights"; return -1; }
    plan->encode = fn;
    const size_t b_bytes = (((size_t)plan->nkb * plan->BN * 128) + 1023) & ~(size_t)1023;
    const size_t a_stage = (size_t)plan->nkb * SBM * 128;
    int stages = 4;
    auto smem_for = [&](int st) {
        return 1024 + b_bytes + st * a_stage + S_EPI_WARPS * 16 * plan->BN + (2 * st + 5) * 8 + 32 + FAST_NP * 256 * 4 + 64;
    };
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
    a.B = g.B; a.oH = g.oH; a.oW = g.oW; a.N = g.O;
    stem_padded_dims(g, &a.Hp, &a.Wp);
    a.M = g.B * g.oH * g.oW;
    if (a.M == 0) return cudaSuccess;
    // The output map is encoded per launch (a host-side fill of 128 bytes): its row extent is this call's
    // pixel count, so the stores of a partial last tile are clipped exactly at the end of the batch slice.
    CUtensorMap tmO;
    {
        const cuuint64_t odims[2] = {(cuuint64_t)g.O, (cuuint64_t)a.M};
        const cuuint64_t ostrides[1] = {(cuuint64_t)g.O};
        const cuuint32_t obox[2] = {(cuuint32_t)(plan.BN / 2), 32};   // an epilogue warp's 32 rows x BN/2 columns (clipped to N)
        const cuuint32_t estr[2] = {1, 1};
        const CUresult rc = ((EncodeTiledFn)plan.encode)(
            &tmO, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, out, odims, ostrides, obox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            plan.BN == 128 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rc != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    a.kH = g.kH; a.sY = g.sY; a.sX = g.sX;
    a.rcp_oW = (unsigned)(((1ull << 32) + (unsigned)g.oW - 1) / (unsigned)g.oW);
    a.nkb = plan.nkb;
    a.stages = plan.stages;
    a.BN = plan.BN;
    a.idesc = (2u << 4) | ((plan.in_unsigned ? 0u : 1u) << 7) | (1u << 10) | ((unsigned)(plan.BN >> 3) << 17)
            | ((unsigned)(SBM >> 4) << 24);
    unsigned cols = 2u * plan.BN, p2 = 32;
    while (p2 < cols) p2 <<= 1;
    a.tmem_cols = p2;
    a.status = status_word;
    a.fq = fast.fq;
    a.cpad = fast.cpad;
    a.out_unsigned = fast.out_unsigned;
    a.wide = fast.wide ? 1 : 0;
    typedef void (*StemKernel)(const CUtensorMap, const CUtensorMap, const StemArgs);
    static const StemKernel variants[4] = {stem_conv_tcgen05_kernel<false, false>, stem_conv_tcgen05_kernel<false, true>,
                                           stem_conv_tcgen05_kernel<true, false>, stem_conv_tcgen05_kernel<true, true>};
    static std::atomic<bool> attr_set[64];   // set twice by racing first calls at worst: harmless
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        for (StemKernel k : variants) {
            cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e != cudaSuccess) return e;
        }
        attr_set[dev] = true;
    }
    const int tiles = (a.M + SBM - 1) / SBM;
    const int grid = tiles < plan.num_sms ? tiles : plan.num_sms;
    const unsigned step = (unsigned)grid * SBM, oHW = (unsigned)(g.oH * g.oW);
    a.step_n = step / oHW;
    a.step_rem = step % oHW;
    const bool vec8 = (g.sX % 2 == 0) && ((uintptr_t)in4 % 8 == 0);
    variants[(fast.need_clamp ? 2 : 0) + (vec8 ? 1 : 0)]<<<grid, S_THREADS, plan.smem_bytes, s>>>(plan.tmB, tmO, a);
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
static bool g_noalloc_used[64] = {false};   // the status word of a device means something only after a first call
static std::mutex g_noalloc_mutex;   // first calls from several host threads look the address up one at a time

static int noalloc_scratch_for(int device, unsigned char** ptr)
{
    if (device < 0 || device >= 64) return n2d2b::set_error(N2D2B_ERR_INVALID, "device %d out of range", device);
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
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
                         "outputs a multiple of 32 and <= 128, output at least 2 wide");
    int Hp = 0, Wp = 0;
    stem_padded_dims(g, &Hp, &Wp);
    const size_t pixels = (size_t)batch * Hp * Wp;
    if (pixels > (size_t)N2D2B_NOALLOC_MAX_PIXELS)
        return set_error(N2D2B_ERR_TOO_LARGE,
                         "batch x padded height x padded width = %zu pixels exceeds the fixed scratch of %u pixels", pixels,
                         (unsigned)N2D2B_NOALLOC_MAX_PIXELS);
    if (stem_weight_bytes(g) > NA_WEIGHT_BYTES)
        return set_error(N2D2B_ERR_TOO_LARGE, "arranged weights exceed the fixed scratch");
    // the caller's current device is put back on every way out
    struct DeviceGuard {
        int prev = -1;
        ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
    } guard;
    if (cudaGetDevice(&guard.prev) != cudaSuccess) guard.prev = -1;
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
    // The status word of the bounded waits lives in the scratch too (last 16 bytes of the constants area).  It
    // still holds what the previous call's kernel left: read it behind that kernel, during the wait this call
    // makes anyway, so a time-out of call k is reported by call k + 1.
    int* status = (int*)(scratch + NA_PAD_OFFSET - 16);
    int prev_status = 0;
    if (e == cudaSuccess) e = cudaMemcpyAsync(&prev_status, status, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return set_error(N2D2B_ERR_CUDA, "copy of the layer constants failed: %s", cudaGetErrorString(e));
    bool first_call_here;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        first_call_here = !g_noalloc_used[device];
        g_noalloc_used[device] = true;
    }
    if (!first_call_here && prev_status != 0) {
        cudaMemsetAsync(status, 0, sizeof(int), s);
        return set_error(N2D2B_ERR_TIMEOUT,
                         "the previous call's kernel gave up waiting on a pipeline barrier (role %d); its output is incomplete",
                         prev_status);
    }

    StemPlan plan;
    const char* why = "";
    if (stem_make_plan(&plan, (const int8_t*)scratch, g, in_unsigned ? 1 : 0, sms, &why))
        return set_error(N2D2B_ERR_INVALID, "first-layer plan failed: %s", why);
    // every pixel of the padded image is rewritten in full, so nothing of an earlier call survives
    e = launch_pad_image(d_input, g, batch, scratch + NA_PAD_OFFSET, s);
    if (e != cudaSuccess) return set_error(N2D2B_ERR_CUDA, "re-layout launch failed: %s", cudaGetErrorString(e));
    const void* in4 = scratch + NA_PAD_OFFSET;
    FastQuant fq;
    fq.fq = (const int*)(scratch + NA_CONST_OFFSET);
    fq.cpad = cpad;
    fq.out_unsigned = out_unsigned;
    fq.need_clamp = need_clamp;
    fq.enabled = true;
    e = cudaMemsetAsync(status, 0, sizeof(int), s);
    if (e == cudaSuccess) e = launch_stem(plan, in4, g, fq, d_output, status, s);
    if (e != cudaSuccess) return set_error(N2D2B_ERR_CUDA, "first-layer launch failed: %s", cudaGetErrorString(e));
    return 0;
}

