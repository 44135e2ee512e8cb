// Stride-1 convolution with a small channel count (32, 64 or 128) on the tensor cores, fed from an input
// patch that is loaded once: the 3x3 layers of the first ResNet stage, where the implicit-GEMM kernel
// would fetch every input pixel nine times through im2col loads and wait on a barrier per filter tap.
//
// A CTA works on a band of R output rows of one image.  One TMA load brings the (R + halo) x (oW + halo)
// x C input patch, zero-filled outside the image, into shared memory as rows of one pixel each (C bytes,
// swizzled by C).  Seen as a list of pixels p = y * Wp + x, the patch is its own im2col matrix: the operand
// of filter tap (ky, kx) for the 128 consecutive positions p0 .. p0+127 is the 128 patch rows that start
// at p0 + ky*dY*Wp + kx*dX.  So every tap is one shared-memory descriptor with a different start row,
// no data moves, and the MMAs of a tile (taps x C/32 of them) are issued back to back.  Positions in the
// halo columns (x >= oW) compute values nobody stores.  The weights of all taps stay resident.
//
// Depthwise 3x3 layers take the same route as block-diagonal groups: the channels are cut into groups of 64 (32), a
// CTA works on one group for its whole life (CTA b on group b mod G, so the group's weight block - its own taps on
// the diagonal, zeros elsewhere - stays resident), the patch load takes the group's channel slice of the NHWC tensor
// and the output rows are written into that slice.  The tensor core multiplies 64 times more than the layer needs,
// and still outruns the CUDA cores, where a byte dot product issues at a quarter of the integer rate.
//
// Warp 0 loads (weights once, patches double-buffered), warps 1-2 issue tcgen05.mma kind::i8 for alternate
// tiles into a ring of four TMEM accumulators, and four groups of four epilogue warps (one warp per TMEM lane quadrant) each
// drain every fourth tile: 32-bit requantisation in the fragment layout, the bytes going from the registers straight to
// the NHWC output (eight consecutive channels per lane).  Every wait is bounded.
#include <cstring>
#include <atomic>
#include "kernels.h"
#include "tc_common.cuh"

namespace n2d2b {

static constexpr int PBM = 128;
static constexpr int P_EPI_WARPS = 16;
static constexpr int P_SLOTS = 4;            // TMEM accumulators = epilogue groups
static constexpr int P_ISSUERS = 4;           // MMA-issuing warps: tiles alternate between them
static constexpr int P_EPI_WARP0 = 1 + P_ISSUERS;
static constexpr int P_THREADS = 32 * (P_EPI_WARP0 + P_EPI_WARPS);
static constexpr int P_BRING_MIN = 4;         // weight ring slots (one filter tap each) when the weights stream:
static constexpr int P_BRING_MAX = 8;         // as many as shared memory holds between these two

struct PatchArgs {
    int B, oH, oW, N, BN, C;   // N, C: output and input channels of one group (= of the layer when G == 1)
    int G;                  // channel groups (block-diagonal layers); CTA b works on group b % G
    int ldo;                // output channels per pixel of the whole tensor
    int taps_y, taps_x, dY, dX, pT, pL;
    int Wp;                 // patch width in pixels: oW + (kW-1)*dX
    int R;                  // output rows per band
    int bands;              // bands per image
    int n_base;             // first image of this call within the tensors (batch slices)
    int patch_bytes;        // bytes one patch load delivers (the full TMA box)
    int patch_alloc;        // bytes reserved per patch buffer (box + the rows a last tile may read past it)
    int b_stream;           // weights too large to stay resident: their tap blocks stream through a ring
    int bring;              // slots of that ring
    int stage_cols;         // columns an epilogue warp stages per pass (BN, or 32 to leave room for the ring)
    unsigned rcp_Wp;        // ceil(2^32 / Wp)
    unsigned idesc, tmem_cols;
    void* out;
    int* status;
    const int* fq;
    int cpad;
    int out_unsigned;
    int wide;               // 64-bit first rescale (see EF_WIDE)
};

// The MMAs of one tile with compile-time tap counts: a straight run of address adds and MMAs.  The issuing
// thread pays the latency of every instruction it executes, so loop control and address arithmetic around a
// short MMA (one of 128 x 64 x 32 takes about 60 cycles of the tensor pipe) would cost more than the MMA.
template <int KH, int KW, int KS>
__device__ __forceinline__ void issue_tile(unsigned d_tmem, unsigned a_lo, unsigned b_lo, unsigned desc_hi, unsigned idesc,
                                           unsigned row_step, unsigned col_step, unsigned btap, unsigned issue)
{
#pragma unroll
    for (int ky = 0; ky < KH; ++ky)
#pragma unroll
        for (int kx = 0; kx < KW; ++kx)
#pragma unroll
            for (int k = 0; k < KS; ++k)
                tc_mma_i8_lohi_p(d_tmem, a_lo + ky * row_step + kx * col_step + 2u * k, b_lo + (ky * KW + kx) * btap + 2u * k,
                                 desc_hi, idesc, (ky | kx | k) ? 1u : 0u, issue);
}

// The MMAs of one filter tap of one tile (C / 32 K steps), unrolled for the channel counts the kernel takes
template <int KS>
__device__ __forceinline__ void issue_tap_n(unsigned d_tmem, unsigned a_lo, unsigned b_lo, unsigned desc_hi, unsigned idesc, unsigned first,
                                            unsigned issue)
{
    tc_mma_i8_lohi_p(d_tmem, a_lo, b_lo, desc_hi, idesc, first, issue);
#pragma unroll
    for (int k = 1; k < KS; ++k) tc_mma_i8_lohi_p(d_tmem, a_lo + 2u * k, b_lo + 2u * k, desc_hi, idesc, 1u, issue);
}
__device__ __forceinline__ void issue_tap(int ksteps, unsigned d_tmem, unsigned a_lo, unsigned b_lo, unsigned desc_hi, unsigned idesc,
                                          unsigned first, unsigned issue)
{
    if (ksteps == 4) issue_tap_n<4>(d_tmem, a_lo, b_lo, desc_hi, idesc, first, issue);
    else if (ksteps == 2) issue_tap_n<2>(d_tmem, a_lo, b_lo, desc_hi, idesc, first, issue);
    else issue_tap_n<1>(d_tmem, a_lo, b_lo, desc_hi, idesc, first, issue);
}

// SHAPE: 0 = any filter (loops), 1 / 2 / 3 = 3x3 filter with 32 / 64 / 128 channels (unrolled issue)
template <bool CLAMP, int SHAPE>
__global__ void __launch_bounds__(P_THREADS, 1)
patch_conv_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const PatchArgs a)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int taps = a.taps_y * a.taps_x;
    const int b_tap_bytes = a.BN * a.C;
    unsigned char* res_b = smem;                                              // [taps][BN][C], or a ring of a.bring taps
    unsigned char* patch0 = smem + (((size_t)(a.b_stream ? a.bring : taps) * b_tap_bytes + 1023) & ~(size_t)1023);
    unsigned char* stage_out = patch0 + 2 * (size_t)a.patch_alloc;             // [16 warps][32 rows][stage_cols]
    const int region_bytes = 32 * a.stage_cols;
    unsigned long long* bars = (unsigned long long*)(stage_out + (size_t)P_EPI_WARPS * region_bytes);
    // bars: patch_full[2], patch_empty[2], tmem_full[4], tmem_empty[4], weights, (spare), ring_full[8], ring_empty[8]
    const unsigned pfull0 = smem_u32(bars);
    const unsigned pempty0 = pfull0 + 16u;
    const unsigned tfull0 = pempty0 + 16u;
    const unsigned tempty0 = tfull0 + 8u * P_SLOTS;
    const unsigned bfull = tempty0 + 8u * P_SLOTS;
    const unsigned rfull0 = bfull + 16u;
    const unsigned rempty0 = rfull0 + 8u * P_BRING_MAX;
    unsigned* tmem_slot = (unsigned*)(bars + 4 + 2 * P_SLOTS + 2 + 2 * P_BRING_MAX);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    int* par = (int*)(((uintptr_t)(tmem_slot + 4) + 15) & ~(uintptr_t)15);   // [FAST_NP][256]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(pfull0 + 8u * s, 1);
            mbar_init(pempty0 + 8u * s, P_ISSUERS);
        }
        for (int s = 0; s < P_SLOTS; ++s) {
            mbar_init(tfull0 + 8u * s, 1);
            mbar_init(tempty0 + 8u * s, 4);
        }
        mbar_init(bfull, 1);
        for (int r = 0; r < P_BRING_MAX; ++r) {
            mbar_init(rfull0 + 8u * r, 1);
            mbar_init(rempty0 + 8u * r, P_ISSUERS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // this CTA's channel group, and its place among the CTAs of that group
    const int grp = (int)blockIdx.x % a.G, cta = (int)blockIdx.x / a.G, nctas = (int)gridDim.x / a.G;
    const int ch0 = grp * a.N;                       // first output channel (= first input channel) of the group
    for (int i = threadIdx.x; i < FAST_NP * 256; i += P_THREADS) {
        const int prm = i >> 8, c = i & 255;
        par[i] = (ch0 + c < a.cpad) ? __ldg(a.fq + (size_t)prm * a.cpad + ch0 + c) : 0;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    const int items = a.B * a.bands;
    // rows and 128-position tiles of band `band` (the last band of an image may be shorter)
    auto band_rows = [&](int band) { const int r = a.oH - band * a.R; return r < a.R ? r : a.R; };
    auto band_tiles = [&](int band) { return (band_rows(band) * a.Wp + PBM - 1) / PBM; };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0 && cta < items) {
            if (!a.b_stream) {
                mbar_expect_tx(bfull, (unsigned)(taps * b_tap_bytes));
                for (int t = 0; t < taps; ++t)
                    tma_load_2d(smem_u32(res_b + (size_t)t * b_tap_bytes), &tmB, bfull, t * a.C, ch0);
            }
            pdl_wait();   // weights are constants; the activations are the previous kernel's output
            unsigned it = 0;
            int rs = 0;              // weight ring slot and its phase
            unsigned rph = 0;
            bool ok = true;
            int n = cta / a.bands, band = cta % a.bands;
            const int step_n = nctas / a.bands, step_b = nctas % a.bands;
            for (int item = cta; item < items; item += nctas, ++it) {
                const unsigned pb = it & 1u, ph = (it >> 1) & 1u;
                if (!mbar_wait(pempty0 + 8u * pb, ph ^ 1u, abort_flag, a.status, 1)) break;
                mbar_expect_tx(pfull0 + 8u * pb, (unsigned)a.patch_bytes);
                tma_load_4d(smem_u32(patch0 + (size_t)pb * a.patch_alloc), &tmA, pfull0 + 8u * pb, grp * a.C, -a.pL,
                            band * a.R - a.pT, a.n_base + n);
                if (a.b_stream) {
                    // every item walks all taps once: its weights follow the patch through the ring
                    for (int t = 0; t < taps && ok; ++t) {
                        if (!mbar_wait(rempty0 + 8u * rs, rph ^ 1u, abort_flag, a.status, 5)) { ok = false; break; }
                        mbar_expect_tx(rfull0 + 8u * rs, (unsigned)b_tap_bytes);
                        tma_load_2d(smem_u32(res_b + (size_t)rs * b_tap_bytes), &tmB, rfull0 + 8u * rs, t * a.C, ch0);
                        if (++rs == a.bring) { rs = 0; rph ^= 1u; }
                    }
                    if (!ok) break;
                }
                n += step_n;
                band += step_b;
                if (band >= a.bands) { band -= a.bands; ++n; }
            }
        }
    } else if (warp < P_EPI_WARP0) {
        // ------------------------------------------------------------------ MMA issuers
        // Issuing a tile costs one thread about 100 cycles per MMA, the tensor pipe about 60: two threads take
        // alternate tiles (each tile has its own accumulator, so their MMAs are independent).
        // every lane of the warp runs the loop; `issue` selects the lane whose MMAs and commits take effect
        const unsigned me = (unsigned)__shfl_sync(0xffffffffu, warp - 1, 0);
        const unsigned issue = lane == 0 ? 1u : 0u;
        if (cta < items) {
            bool ok = a.b_stream ? true : mbar_wait_uniform(bfull, 0, abort_flag, a.status, 8);
            const unsigned desc_hi = (unsigned)(make_smem_desc(0u, a.C) >> 32);
            const unsigned res_b_lo = (smem_u32(res_b) & 0x3ffffu) >> 4, patch_lo = (smem_u32(patch0) & 0x3ffffu) >> 4;
            const int ksteps = a.C / 32;
            const unsigned row_step = (unsigned)((a.dY * a.Wp * a.C) >> 4), col_step = (unsigned)((a.dX * a.C) >> 4);
            const unsigned btap = (unsigned)(b_tap_bytes >> 4);
            unsigned it = 0, seq = 0;
            int band = cta % a.bands;
            const int step_b = nctas % a.bands;
            const unsigned tile_step = (unsigned)((PBM * a.C) >> 4);
            int rs = 0;              // weight ring slot and its phase (streamed weights)
            unsigned rph = 0;
            for (int item = cta; item < items && ok; item += nctas, ++it) {
                const unsigned pb = it & 1u, ph = (it >> 1) & 1u;
                const int T = band_tiles(band);
                if (!mbar_wait_uniform(pfull0 + 8u * pb, ph, abort_flag, a.status, 3)) { ok = false; break; }
                tc_fence_after();
                unsigned a_lo = patch_lo + pb * (unsigned)(a.patch_alloc >> 4);
                if (a.b_stream) {
                    // At most P_SLOTS tiles per item, each with its own accumulator: this thread owns tiles `me` and
                    // `me + P_ISSUERS` and walks the taps as their weights arrive, so one pass of the weights serves
                    // the whole band; a thread without a tile still releases every ring slot.
                    const bool mine0 = (int)me < T, mine1 = (int)me + P_ISSUERS < T;
                    const unsigned seq0 = seq + me, seq1 = seq0 + P_ISSUERS;
                    const unsigned slot0 = seq0 & (P_SLOTS - 1), slot1 = seq1 & (P_SLOTS - 1);
                    if (mine0 && !mbar_wait_uniform(tempty0 + 8u * slot0, ((seq0 / P_SLOTS) & 1u) ^ 1u, abort_flag, a.status, 2)) { ok = false; break; }
                    if (mine1 && !mbar_wait_uniform(tempty0 + 8u * slot1, ((seq1 / P_SLOTS) & 1u) ^ 1u, abort_flag, a.status, 2)) { ok = false; break; }
                    tc_fence_after();
                    const unsigned d0 = tmem_base + slot0 * (unsigned)a.BN, d1 = tmem_base + slot1 * (unsigned)a.BN;
                    const unsigned tile2 = (unsigned)P_ISSUERS * tile_step;
                    unsigned ar = a_lo + me * tile_step, first = 0;
                    for (int ky = 0; ky < a.taps_y && ok; ++ky, ar += row_step) {
                        unsigned ac = ar;
                        for (int kx = 0; kx < a.taps_x; ++kx, ac += col_step) {
                            if (!mbar_wait_uniform(rfull0 + 8u * rs, rph, abort_flag, a.status, 6)) { ok = false; break; }
                            tc_fence_after();
                            const unsigned bt = res_b_lo + (unsigned)rs * btap;
                            if (mine0) issue_tap(ksteps, d0, ac, bt, desc_hi, a.idesc, first, issue);
                            if (mine1) issue_tap(ksteps, d1, ac + tile2, bt, desc_hi, a.idesc, first, issue);
                            first = 1u;
                            tc_commit_p(rempty0 + 8u * rs, issue);
                            if (++rs == a.bring) { rs = 0; rph ^= 1u; }
                        }
                    }
                    if (!ok) break;
                    if (mine0) tc_commit_p(tfull0 + 8u * slot0, issue);
                    if (mine1) tc_commit_p(tfull0 + 8u * slot1, issue);
                    seq += (unsigned)T;
                    tc_commit_p(pempty0 + 8u * pb, issue);
                    band += step_b;
                    if (band >= a.bands) band -= a.bands;
                    continue;
                }
                for (int t = 0; t < T; ++t, ++seq, a_lo += tile_step) {
                    if ((seq & (P_ISSUERS - 1)) != me) continue;
                    const unsigned slot = seq & (P_SLOTS - 1), sph = (seq / P_SLOTS) & 1u;
                    if (!mbar_wait_uniform(tempty0 + 8u * slot, sph ^ 1u, abort_flag, a.status, 2)) { ok = false; break; }
                    tc_fence_after();
                    const unsigned d_tmem = tmem_base + slot * (unsigned)a.BN;
                    // The operand of a tap starts at an arbitrary pixel row.  The swizzle is a function of the
                    // absolute shared-memory address, so the descriptor needs nothing but that address
                    // (measured: with the base-offset field left 0 every start row gives exact results).
                    if (SHAPE == 1) issue_tile<3, 3, 1>(d_tmem, a_lo, res_b_lo, desc_hi, a.idesc, row_step, col_step, btap, issue);
                    else if (SHAPE == 2) issue_tile<3, 3, 2>(d_tmem, a_lo, res_b_lo, desc_hi, a.idesc, row_step, col_step, btap, issue);
                    else if (SHAPE == 3) issue_tile<3, 3, 4>(d_tmem, a_lo, res_b_lo, desc_hi, a.idesc, row_step, col_step, btap, issue);
                    else {
                        unsigned ar = a_lo, bt = res_b_lo, first = 0;
                        for (int ky = 0; ky < a.taps_y; ++ky, ar += row_step) {
                            unsigned ac = ar;
                            for (int kx = 0; kx < a.taps_x; ++kx, ac += col_step, bt += btap)
                                for (int k = 0; k < ksteps; ++k) {
                                    tc_mma_i8_lohi_p(d_tmem, ac + 2u * k, bt + 2u * k, desc_hi, a.idesc, first, issue);
                                    first = 1u;
                                }
                        }
                    }
                    tc_commit_p(tfull0 + 8u * slot, issue);
                }
                if (ok) tc_commit_p(pempty0 + 8u * pb, issue);   // the patch is free once both issuers' MMAs have read it
                band += step_b;
                if (band >= a.bands) band -= a.bands;
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        pdl_wait();   // the output buffer may still be read by the previous kernel
        const int ew = warp - P_EPI_WARP0;
        const int quad = warp & 3;          // TMEM lane quadrant this warp may read
        const int group = ew >> 2;          // drains the tiles whose sequence number is `group` modulo 4
        const unsigned par_off = (unsigned)((unsigned char*)par - smem_raw);
        unsigned seq = 0;
        int n = cta / a.bands, band = cta % a.bands;
        const int step_n = nctas / a.bands, step_b = nctas % a.bands;
        bool ok = true;
        for (int item = cta; item < items && ok; item += nctas) {
            const int rows = band_rows(band);
            const int T = band_tiles(band);
            uint8_t* const band_out = (uint8_t*)a.out + ((size_t)(a.n_base + n) * a.oH + (size_t)(band * a.R)) * a.oW * a.ldo + ch0;
            for (int t = 0; t < T; ++t, ++seq) {
                if ((int)(seq & (P_SLOTS - 1)) != group) continue;
                const unsigned sph = (seq / P_SLOTS) & 1u;
                if (!mbar_wait_warp(tfull0 + 8u * group, sph, abort_flag, a.status, 4, lane)) { ok = false; break; }
                tc_fence_after();
                const unsigned tbase = tmem_base + ((unsigned)(quad * 32) << 16) + (unsigned)(group * a.BN);
                // This lane's four rows of the fragment (positions of the band's raster) and where they go: the bytes leave
                // the registers for global memory directly, eight channels per lane, a 32-byte sector per four lanes
                unsigned rowoff[4];   // byte offsets within the band: below 2^32
                unsigned rowok = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const unsigned p = (unsigned)(t * PBM + quad * 32 + (lane >> 2) + 8 * k);
                    const unsigned yy = __umulhi(p, a.rcp_Wp);
                    const unsigned x = p - yy * (unsigned)a.Wp;
                    if (x < (unsigned)a.oW && yy < (unsigned)rows) rowok |= 1u << k;
                    rowoff[k] = (yy * (unsigned)a.oW + x) * (unsigned)a.ldo;
                }
#pragma unroll 1
                for (int cb = 0; cb < a.N; cb += 32) {
                    unsigned va[16], vb[16];
                    tc_ld_2x16x256b_x4_wait(tbase + (unsigned)cb, va, vb);
                    if (a.wide) {
                        if (a.out_unsigned) perm_block_global<false, EF_WIDE | EF_OUT_UNSIGNED>(va, vb, par_off, cb, band_out + cb, rowoff, rowok, lane);
                        else perm_block_global<false, EF_WIDE>(va, vb, par_off, cb, band_out + cb, rowoff, rowok, lane);
                    } else if (a.out_unsigned) perm_block_global<CLAMP, EF_OUT_UNSIGNED>(va, vb, par_off, cb, band_out + cb, rowoff, rowok, lane);
                    else perm_block_global<CLAMP, 0>(va, vb, par_off, cb, band_out + cb, rowoff, rowok, lane);
                }
                // the accumulator is drained: hand it back
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty0 + 8u * group);
            }
            n += step_n;
            band += step_b;
            if (band >= a.bands) { band -= a.bands; ++n; }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(a.tmem_cols) : "memory");
    }
}

// ----------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// weights of up to this size stay resident; larger ones stream tap by tap through a ring of `bring` blocks, and
// the epilogue then stages 32 columns per pass so that the ring can be deep: its loads cross the L2 with a
// latency of thousands of cycles, and what is in flight bounds what arrives
static constexpr size_t P_RESIDENT_MAX = 96 * 1024;
static bool patch_streams(int taps, int C, int BN) { return (size_t)taps * BN * C > P_RESIDENT_MAX; }

static int patch_stage_cols(int taps, int C, int BN) { return patch_streams(taps, C, BN) ? 32 : BN; }

// (The term with patch_stage_cols is a staging area the epilogue no longer uses since it stores from its registers.  It
// stays in the budget because it caps the band height: with that area given to the patches, the 64-channel 55 x 55
// layers went from five bands of 11 rows to 22 + 22 + 11 and ran 18 % slower.)
static size_t patch_smem_bytes(int taps, int C, int BN, int patch_alloc, int bring = P_BRING_MIN)
{
    const int blocks = patch_streams(taps, C, BN) ? bring : taps;
    const size_t b = (((size_t)blocks * BN * C) + 1023) & ~(size_t)1023;
    return 1024 + b + 2 * (size_t)patch_alloc + (size_t)P_EPI_WARPS * 32 * patch_stage_cols(taps, C, BN)
         + (4 + 2 * P_SLOTS + 2 + 2 * P_BRING_MAX) * 8 + 32 + FAST_NP * 256 * 4 + 64;
}

// bytes a patch buffer must hold for bands of R rows: the tiles of a band read 128-row operands that start
// up to (kH-1)*dY*Wp + (kW-1)*dX rows after the tile's first position
static int patch_alloc_bytes(const ConvGeom& g, int Wp, int R)
{
    const int tiles = (R * Wp + PBM - 1) / PBM;
    const int reach = tiles * PBM + (g.kH - 1) * g.dY * Wp + (g.kW - 1) * g.dX;
    const int box = (R + (g.kH - 1) * g.dY) * Wp;
    const int rows = reach > box ? reach : box;
    return (rows * g.C + 1023) & ~1023;
}

// Channels per block-diagonal group of a depthwise layer (0: not a layer this kernel takes as groups)
static int patch_dw_group(const ConvGeom& g)
{
    if (g.groups <= 1 || g.groups != g.C || g.O != g.C || g.Cg != 1 || g.Og != 1) return 0;
    if (g.C % 64 == 0) return 64;
    if (g.C % 32 == 0) return 32;
    return 0;
}

// The geometry of one group of a depthwise layer as the dense layer the kernel sees
static ConvGeom patch_group_geom(const ConvGeom& g)
{
    ConvGeom e = g;
    const int cg = patch_dw_group(g);
    if (cg) { e.C = cg; e.O = cg; e.groups = 1; e.Cg = cg; e.Og = cg; }
    return e;
}

int patch_groups(const ConvGeom& g) { const int cg = patch_dw_group(g); return cg ? g.C / cg : 1; }

bool patch_eligible(const ConvGeom& g0)
{
    if (g0.groups != 1 && (!patch_dw_group(g0) || patch_groups(g0) > 64)) return false;
    const ConvGeom g = patch_group_geom(g0);
    if (g.groups != 1 || g.sX != 1 || g.sY != 1) return false;
    if (g.C != 32 && g.C != 64 && g.C != 128) return false;
    if (g.O % 32 != 0 || g.O > 128) return false;
    if (g.kH * g.kW < 2) return false;   // a 1x1 layer gains nothing from a patch
    const int BN = g.O <= 64 ? 64 : 128;
    const int Wp = g.oW + (g.kW - 1) * g.dX;
    if (Wp > 256 || Wp < 2 || g.oH < 1) return false;
    if ((g.kH - 1) * g.dY + 1 > 256) return false;
    // at least one output row per band must fit
    return patch_smem_bytes(g.kH * g.kW, g.C, BN, patch_alloc_bytes(g, Wp, 1)) <= 226 * 1024;
}

// Weight rows ([O][taps * C] bytes) in the order the kernel's epilogue expects
void patch_permute_weights(const int8_t* w, int8_t* dst, int O, size_t row_bytes)
{
    for (int n = 0; n < O; ++n) memcpy(dst + (size_t)n * row_bytes, w + (size_t)perm_real_channel(n, 4) * row_bytes, row_bytes);
}

// Depthwise weights [C][taps] as the block-diagonal matrix of the grouped form: row o = [taps][group channels] with
// the tap's weight at column o % group and zeros elsewhere; rows in the epilogue's order.
size_t patch_dw_weight_bytes(const ConvGeom& g) { return (size_t)g.C * g.kH * g.kW * patch_dw_group(g); }
void patch_dw_arrange_weights(const ConvGeom& g, const int8_t* w_ct, int8_t* dst)
{
    const int cg = patch_dw_group(g), taps = g.kH * g.kW;
    const size_t row_bytes = (size_t)taps * cg;
    memset(dst, 0, (size_t)g.C * row_bytes);
    for (int n = 0; n < g.C; ++n) {
        const int o = perm_real_channel(n, 4);
        for (int t = 0; t < taps; ++t) dst[(size_t)n * row_bytes + (size_t)t * cg + (o % cg)] = w_ct[(size_t)o * taps + t];
    }
}

int patch_make_plan(PatchPlan* plan, const void* in, const int8_t* w, const ConvGeom& g0, int in_unsigned, int num_sms,
                    const char** why)
{
    static const char* kWhy = "";
    *why = kWhy;
    if (!patch_eligible(g0)) { *why = "geometry outside the patch kernel"; return -1; }
    const ConvGeom g = patch_group_geom(g0);   // one group (the layer itself when it is dense)
    const int Ct = g0.C;                       // channels per pixel of the input tensor, rows of the weight matrix
    if (((uintptr_t)in & 15) || ((uintptr_t)w & 15)) { *why = "operands must be 16-byte aligned"; return -1; }
    cudaDriverEntryPointQueryResult qr;
    void* fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) != cudaSuccess || !fn) {
        *why = "cuTensorMapEncodeTiled is not available from the CUDA driver";
        return -1;
    }
    memset(plan, 0, sizeof(*plan));
    const int taps = g.kH * g.kW;
    plan->BN = g.O <= 64 ? 64 : 128;
    plan->Wp = g.oW + (g.kW - 1) * g.dX;
    plan->in_unsigned = in_unsigned;
    plan->num_sms = num_sms;
    plan->G = patch_groups(g0);
    // rows per band: among the heights that fit shared memory (and the 256-row TMA box), the one that
    // wastes the fewest 128-position tiles per image; ties go to the taller band (fewer halo rows re-read)
    int best_R = 0;
    long long best_tiles = 0;
    plan->b_stream = patch_streams(taps, g.C, plan->BN) ? 1 : 0;
    for (int R = 1; R <= g.oH; ++R) {
        if (R + (g.kH - 1) * g.dY > 256) break;
        if (patch_smem_bytes(taps, g.C, plan->BN, patch_alloc_bytes(g, plan->Wp, R)) > 226 * 1024) break;
        // streamed weights: every tile of a band accumulates while the taps pass, so a band has at most as many
        // tiles as there are accumulators
        if (plan->b_stream && (R * plan->Wp + PBM - 1) / PBM > P_SLOTS) break;
        const int full = g.oH / R, rest = g.oH % R;
        const long long tiles = (long long)full * ((R * plan->Wp + PBM - 1) / PBM)
                              + (rest ? (rest * plan->Wp + PBM - 1) / PBM : 0);
        if (best_R == 0 || tiles <= best_tiles) { best_R = R; best_tiles = tiles; }
    }
    if (best_R == 0) { *why = "no band height fits shared memory"; return -1; }
    plan->R = best_R;
    plan->bands = (g.oH + best_R - 1) / best_R;
    const int box_rows = best_R + (g.kH - 1) * g.dY;
    plan->patch_bytes = box_rows * plan->Wp * g.C;
    plan->patch_alloc = patch_alloc_bytes(g, plan->Wp, best_R);
    plan->stage_cols = patch_stage_cols(taps, g.C, plan->BN);
    plan->bring = P_BRING_MIN;
    while (plan->b_stream && plan->bring < P_BRING_MAX
           && patch_smem_bytes(taps, g.C, plan->BN, plan->patch_alloc, plan->bring + 1) <= 226 * 1024)
        ++plan->bring;
    plan->smem_bytes = patch_smem_bytes(taps, g.C, plan->BN, plan->patch_alloc, plan->bring);
    const CUtensorMapSwizzle swz = g.C == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                              : (g.C == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    CUresult rc;
    {   // weights [O][taps*C], one box = one tap of all outputs (rows beyond O read as zero)
        const cuuint64_t dims[2] = {(cuuint64_t)taps * g.C, (cuuint64_t)g0.O};
        const cuuint64_t strides[1] = {(cuuint64_t)taps * g.C};
        const cuuint32_t box[2] = {(cuuint32_t)g.C, (cuuint32_t)plan->BN};
        const cuuint32_t estr[2] = {1, 1};
        rc = ((EncodeTiledFn)fn)(&plan->tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)w, dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rc != CUDA_SUCCESS) { *why = "cuTensorMapEncodeTiled failed for the weights"; return -1; }
    }
    {   // NHWC activations as (C, W, H, B); one box = a whole patch, zero-filled outside the image
        const cuuint64_t dims[4] = {(cuuint64_t)Ct, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.B};
        const cuuint64_t strides[3] = {(cuuint64_t)Ct, (cuuint64_t)Ct * g.W, (cuuint64_t)Ct * g.W * g.H};
        const cuuint32_t box[4] = {(cuuint32_t)g.C, (cuuint32_t)plan->Wp, (cuuint32_t)box_rows, 1};
        const cuuint32_t estr[4] = {1, 1, 1, 1};
        rc = ((EncodeTiledFn)fn)(&plan->tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)in, dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rc != CUDA_SUCCESS) { *why = "cuTensorMapEncodeTiled failed for the activation patch"; return -1; }
    }
    return 0;
}

cudaError_t launch_patch(const PatchPlan& plan, const ConvGeom& g0, int n_base, const FastQuant& fast, void* out,
                         int* status_word, cudaStream_t s)
{
    const ConvGeom g = patch_group_geom(g0);
    PatchArgs a;
    memset(&a, 0, sizeof(a));
    a.B = g.B; a.oH = g.oH; a.oW = g.oW; a.N = g.O; a.BN = plan.BN; a.C = g.C;
    a.G = plan.G; a.ldo = g0.O;
    if (a.B == 0) return cudaSuccess;
    a.taps_y = g.kH; a.taps_x = g.kW; a.dY = g.dY; a.dX = g.dX; a.pT = g.pT; a.pL = g.pL;
    a.Wp = plan.Wp; a.R = plan.R; a.bands = plan.bands;
    a.n_base = n_base;
    a.patch_bytes = plan.patch_bytes; a.patch_alloc = plan.patch_alloc;
    a.b_stream = plan.b_stream;
    a.bring = plan.bring;
    a.stage_cols = plan.stage_cols;
    a.rcp_Wp = (unsigned)(((1ull << 32) + (unsigned)plan.Wp - 1) / (unsigned)plan.Wp);
    a.idesc = (2u << 4) | ((plan.in_unsigned ? 0u : 1u) << 7) | (1u << 10) | ((unsigned)(plan.BN >> 3) << 17)
            | ((unsigned)(PBM >> 4) << 24);
    a.tmem_cols = (unsigned)(P_SLOTS * plan.BN);   // 256 or 512: a power of two
    a.out = out;
    a.status = status_word;
    a.fq = fast.fq;
    a.cpad = fast.cpad;
    a.out_unsigned = fast.out_unsigned;
    a.wide = fast.wide ? 1 : 0;
    typedef void (*PatchKernel)(const CUtensorMap, const CUtensorMap, const PatchArgs);
    static const PatchKernel variants[8] = {
        patch_conv_tcgen05_kernel<false, 0>, patch_conv_tcgen05_kernel<false, 1>, patch_conv_tcgen05_kernel<false, 2>,
        patch_conv_tcgen05_kernel<false, 3>, patch_conv_tcgen05_kernel<true, 0>,  patch_conv_tcgen05_kernel<true, 1>,
        patch_conv_tcgen05_kernel<true, 2>,  patch_conv_tcgen05_kernel<true, 3>};
    static std::atomic<bool> attr_set[64];   // set twice by racing first calls at worst: harmless
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        for (PatchKernel k : variants) {
            cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e != cudaSuccess) return e;
        }
        attr_set[dev] = true;
    }
    // a multiple of the group count: CTA b works on group b % G
    const long long items = (long long)a.B * a.bands;
    const long long per_group = plan.num_sms / plan.G > 0 ? plan.num_sms / plan.G : 1;
    const int grid = (int)((items < per_group ? items : per_group) * plan.G);
    const int shape = (g.kH == 3 && g.kW == 3 && !plan.b_stream) ? (g.C == 32 ? 1 : (g.C == 64 ? 2 : 3)) : 0;
    return launch_pdl(variants[(fast.need_clamp ? 4 : 0) + shape], grid, P_THREADS, plan.smem_bytes, s, plan.tmA, plan.tmB, a);
}

}  // namespace n2d2b
