// First-layer convolution with stride 2 (the 7x7/2 stem of the ResNets, the 3x3/2 stem of MobileNet) on the
// tensor cores without a gather.
//
// Space-to-depth turns the stride-2 layer into a stride-1 one: the input (<= 4 channels) is re-laid as
// [B][Hs][Ws][16] where pixel (Y, X) holds the 2 x 2 block of padded input pixels (2Y + dy, 2X + dx), four
// bytes each.  A k x k / 2 filter becomes a KH x KW filter (KH = ceil((k + o) / 2), o = 0 or 1 from the
// padding's parity) over 16 channels, with zero weights where the original filter has no tap.
// A band of the re-laid image is loaded into shared memory by one TMA copy, pixels one after the other,
// 16 bytes each, no swizzle.  Seen as a K-major MMA operand this plain byte string already is the im2col
// matrix: row r (output position p0 + r) starts at byte 16 r and is 32 bytes long (two adjacent pixels = two
// filter taps), i.e. rows overlap.  The shared-memory descriptor expresses exactly that: 8-row core matrices
// of 16-byte rows (128 contiguous bytes), the next core matrix along K 16 bytes further (the same bytes, one
// pixel on), the next 8 rows 128 bytes further.  So no thread touches the activations between the TMA copy
// and the tensor core; the weights sit resident in the canonical unswizzled layout.
//
// Roles as in the patch kernel: warp 0 loads (weights once, bands double-buffered), warps 1-2 issue
// tcgen05.mma kind::i8 for alternate tiles into a ring of four TMEM accumulators, four groups of four
// epilogue warps each drain every fourth 128-position tile (32-bit requantisation in the fragment layout, the bytes going
// from the registers straight to the NHWC output, eight consecutive channels per lane).  Positions in the halo columns (x >= oW) compute
// values nobody stores.  Every wait is bounded.
//
// POOL variant: the layer is followed by a max pooling (k x k window, stride s, no padding) and nothing else reads
// its output.  A band then is the (P - 1) s + k convolution rows that P pooling rows need (bands advance by P s
// rows, so k - s rows are computed twice); the epilogue warps requantise every tile straight into a band-sized
// buffer in shared memory (one 64- or 128-byte row per position, 16-byte units swizzled like the staging regions),
// meet on a barrier once the band is complete, and then take the maxima from that buffer and write only the
// pooled rows.  Two such buffers alternate, so the pooling of one band overlaps the MMAs of the next.  The
// convolution's own output (the largest tensor of a ResNet) never exists in HBM.
#include <cstring>
#include <vector>
#include <atomic>
#include "kernels.h"
#include "tc_common.cuh"

namespace n2d2b {

static constexpr int ZBM = 128;
static constexpr int Z_EPI_WARPS = 16;
static constexpr int Z_SLOTS = 4;
static constexpr int Z_ISSUERS = 2;           // MMA-issuing warps: tiles alternate between them
static constexpr int Z_EPI_WARP0 = 1 + Z_ISSUERS;
static constexpr int Z_THREADS = 32 * (Z_EPI_WARP0 + Z_EPI_WARPS);

struct S2dArgs {
    int B, oH, oW, N, BN;
    int KH, KWp;            // filter rows and (even) filter columns after space-to-depth
    int Wp;                 // pixels per row of the re-laid image = oW + KWp - 1
    int R, bands;           // output rows per band, bands per image
    int row_stride;         // convolution rows from one band to the next (R, or P * pool_s with a fused pooling)
    int pool_k, pool_s, P;  // fused max pooling: window, stride, pooled rows per band
    int pool_oH, pool_oW;
    int cbuf_alloc;         // bytes of one band-sized output buffer (fused pooling)
    int n_base;             // first image of this call within the re-laid buffer (batch slices)
    int band_bytes;         // bytes one band load delivers (the full TMA box)
    int band_alloc;         // bytes reserved per band buffer
    int w_bytes;            // resident weights: KH blocks of BN x (KWp * 16) bytes
    unsigned rcp_Wp;        // ceil(2^32 / Wp)
    unsigned idesc, tmem_cols;
    const int8_t* w;        // weights in the canonical unswizzled K-major layout
    void* out;
    int* status;
    const int* fq;
    int cpad;
    int out_unsigned;
    int wide;               // 64-bit first rescale (see EF_WIDE)
};

// [B][H][W][C] (C <= 4) -> [B][Hs][Ws][2][2][4]: block (dy, dx) of pixel (Y, X) = input pixel
// (2Y + dy - P, 2X + dx - P), zero outside the image and in the unused channels.  One block per output row.
__global__ void s2d_image_kernel(const uint8_t* __restrict__ in, int C, int H, int W, int Hs, int Ws, int P, int rows,
                                 uint4* __restrict__ out)
{
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const int n = row / Hs, Y = row - n * Hs;
        const uint8_t* img = in + (size_t)n * H * W * C;
        uint4* orow = out + (size_t)row * Ws;
        for (int X = threadIdx.x; X < Ws; X += blockDim.x) {
            uint32_t v[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int y = 2 * Y + (q >> 1) - P, x = 2 * X + (q & 1) - P;
                uint32_t px = 0;
                if (y >= 0 && y < H && x >= 0 && x < W) {
                    const uint8_t* p = img + ((size_t)y * W + x) * C;
                    if (C == 4) px = __ldg((const uint32_t*)p);
                    else if (C == 3) px = __ldg(p) | ((uint32_t)__ldg(p + 1) << 8) | ((uint32_t)__ldg(p + 2) << 16);
                    else if (C == 2) px = __ldg(p) | ((uint32_t)__ldg(p + 1) << 8);
                    else px = __ldg(p);
                }
                v[q] = px;
            }
            orow[X] = make_uint4(v[0], v[1], v[2], v[3]);
        }
    }
}

// Unswizzled K-major descriptor words: low = address / 16 | (offset between core matrices along K) / 16 << 16,
// high = (offset between 8-row groups) / 16 | descriptor version
__device__ __forceinline__ unsigned noswz_lo(unsigned addr, unsigned k_step) { return ((addr & 0x3ffffu) >> 4) | ((k_step >> 4) << 16); }
__device__ __forceinline__ unsigned noswz_hi(unsigned row_group_step) { return (row_group_step >> 4) | (1u << 14); }

__device__ __forceinline__ void tc_mma_i8_words(unsigned d_tmem, unsigned a_lo, unsigned a_hi, unsigned b_lo, unsigned b_hi,
                                                unsigned idesc, unsigned accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void bulk_load(unsigned dst, const void* src, unsigned bytes, unsigned bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// The MMAs of one tile with compile-time filter extents (KH rows, KP column pairs)
template <int KH, int KP>
__device__ __forceinline__ void s2d_issue_tile(unsigned d_tmem, unsigned a_lo, unsigned a_hi, unsigned b_lo, unsigned b_hi,
                                               unsigned idesc, unsigned row_step, unsigned b_row_step)
{
#pragma unroll
    for (int ky = 0; ky < KH; ++ky)
#pragma unroll
        for (int j = 0; j < KP; ++j)
            // two pixels (32 bytes) on in the band, two 128-byte core matrices on in the weights
            tc_mma_i8_words(d_tmem, a_lo + ky * row_step + 2u * j, a_hi, b_lo + ky * b_row_step + 16u * j, b_hi, idesc,
                            (ky | j) ? 1u : 0u);
}

template <bool CLAMP, int EF>
__device__ __forceinline__ void s2d_drain(unsigned tbase, unsigned par_off, unsigned region_off, int BN, int lane)
{
    // the weight rows are stored permuted inside blocks of 32 channels (stem_s2d_arrange_weights): a thread's
    // columns of the fragment are eight consecutive channels
    unsigned rb[4];
    perm_rowbase(rb, BN, lane, 4);
#pragma unroll 1
    for (int cb = 0; cb < BN; cb += 32) {
        unsigned va[16], vb[16];
        tc_ld_2x16x256b_x4_wait(tbase + (unsigned)cb, va, vb);
        perm_block<4, false, CLAMP, false, EF | EF_PERM>(va, vb, par_off, cb, region_off, rb, cb, lane, 0, 0, 0u);
    }
}

// SHAPE: 0 = any filter (loops), 1 = 4 x 4 (a 7x7/2 or 8x8/2 filter), 2 = 2 x 2 (a 3x3/2 filter)
template <bool CLAMP, int SHAPE, bool POOL>
__global__ void __launch_bounds__(Z_THREADS, 1)
stem_s2d_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const S2dArgs a)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* res_b = smem;
    unsigned char* band0 = smem + (((size_t)a.w_bytes + 1023) & ~(size_t)1023);
    unsigned char* stage_out = band0 + 2 * (size_t)a.band_alloc;               // [16 warps][32 rows][BN], or two band-sized buffers
    const int region_bytes = 32 * a.BN;
    unsigned long long* bars = (unsigned long long*)(stage_out + (POOL ? 2 * (size_t)a.cbuf_alloc : (size_t)Z_EPI_WARPS * region_bytes));
    // bars: band_full[2], band_empty[2], tmem_full[4], tmem_empty[4], weights, (spare), band_complete[2]
    const unsigned pfull0 = smem_u32(bars);
    const unsigned pempty0 = pfull0 + 16u;
    const unsigned tfull0 = pempty0 + 16u;
    const unsigned tempty0 = tfull0 + 8u * Z_SLOTS;
    const unsigned bfull = tempty0 + 8u * Z_SLOTS;
    const unsigned cdone0 = bfull + 16u;
    unsigned* tmem_slot = (unsigned*)(bars + 4 + 2 * Z_SLOTS + 2 + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    int* par = (int*)(((uintptr_t)(tmem_slot + 4) + 15) & ~(uintptr_t)15);   // [FAST_NP][256]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(pfull0 + 8u * s, 1);
            mbar_init(pempty0 + 8u * s, Z_ISSUERS);
        }
        for (int s = 0; s < Z_SLOTS; ++s) {
            mbar_init(tfull0 + 8u * s, 1);
            mbar_init(tempty0 + 8u * s, 4);
        }
        mbar_init(bfull, 1);
        mbar_init(cdone0, Z_EPI_WARPS);
        mbar_init(cdone0 + 8u, Z_EPI_WARPS);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int i = threadIdx.x; i < FAST_NP * 256; i += Z_THREADS) {
        const int prm = i >> 8, c = i & 255;
        par[i] = (c < a.cpad) ? __ldg(a.fq + (size_t)prm * a.cpad + c) : 0;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    const int items = a.B * a.bands;
    auto band_rows = [&](int band) { const int r = a.oH - band * a.row_stride; return r < a.R ? r : a.R; };
    auto band_tiles = [&](int band) { return (band_rows(band) * a.Wp + ZBM - 1) / ZBM; };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0 && (int)blockIdx.x < items) {
            mbar_expect_tx(bfull, (unsigned)a.w_bytes);
            bulk_load(smem_u32(res_b), a.w, (unsigned)a.w_bytes, bfull);
            pdl_wait();   // weights are constants; the re-laid image is the previous kernel's output
            unsigned it = 0;
            int n = (int)blockIdx.x / a.bands, band = (int)blockIdx.x % a.bands;
            const int step_n = (int)gridDim.x / a.bands, step_b = (int)gridDim.x % a.bands;
            for (int item = blockIdx.x; item < items; item += gridDim.x, ++it) {
                const unsigned pb = it & 1u, ph = (it >> 1) & 1u;
                if (!mbar_wait(pempty0 + 8u * pb, ph ^ 1u, abort_flag, a.status, 1)) break;
                mbar_expect_tx(pfull0 + 8u * pb, (unsigned)a.band_bytes);
                tma_load_3d(smem_u32(band0 + (size_t)pb * a.band_alloc), &tmA, pfull0 + 8u * pb, 0, band * a.row_stride, a.n_base + n);
                n += step_n;
                band += step_b;
                if (band >= a.bands) { band -= a.bands; ++n; }
            }
        }
    } else if (warp < Z_EPI_WARP0) {
        // ------------------------------------------------------------------ MMA issuers (alternate tiles)
        const unsigned me = (unsigned)(warp - 1);
        if (lane == 0 && (int)blockIdx.x < items) {
            bool ok = mbar_wait(bfull, 0, abort_flag, a.status, 8);
            // activations: rows of 16 bytes, next K chunk = next pixel (16 bytes), next 8 rows 128 bytes on
            const unsigned a_hi = noswz_hi(128u);
            const unsigned band_lo = noswz_lo(smem_u32(band0), 16u);
            // weights per filter row: [n / 8][k / 16][n % 8][16 bytes], k < KWp * 16
            const unsigned b_hi = noswz_hi((unsigned)(a.KWp * 128));
            const unsigned b_lo0 = noswz_lo(smem_u32(res_b), 128u);
            const unsigned row_step = (unsigned)a.Wp;                        // one band row on, in 16-byte units
            const unsigned b_row_step = (unsigned)((a.BN * a.KWp * 16) >> 4);
            const unsigned tile_step = (unsigned)ZBM;
            unsigned it = 0, seq = 0;
            int band = (int)blockIdx.x % a.bands;
            const int step_b = (int)gridDim.x % a.bands;
            for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ++it) {
                const unsigned pb = it & 1u, ph = (it >> 1) & 1u;
                const int T = band_tiles(band);
                if (!mbar_wait(pfull0 + 8u * pb, ph, abort_flag, a.status, 3)) { ok = false; break; }
                tc_fence_after();
                unsigned a_lo = band_lo + pb * (unsigned)(a.band_alloc >> 4);
                for (int t = 0; t < T; ++t, ++seq, a_lo += tile_step) {
                    if ((seq & (Z_ISSUERS - 1)) != me) continue;
                    const unsigned slot = seq & (Z_SLOTS - 1), sph = (seq / Z_SLOTS) & 1u;
                    if (!mbar_wait(tempty0 + 8u * slot, sph ^ 1u, abort_flag, a.status, 2)) { ok = false; break; }
                    tc_fence_after();
                    const unsigned d_tmem = tmem_base + slot * (unsigned)a.BN;
                    if (SHAPE == 1) s2d_issue_tile<4, 2>(d_tmem, a_lo, a_hi, b_lo0, b_hi, a.idesc, row_step, b_row_step);
                    else if (SHAPE == 2) s2d_issue_tile<2, 1>(d_tmem, a_lo, a_hi, b_lo0, b_hi, a.idesc, row_step, b_row_step);
                    else {
                        unsigned ar = a_lo, br = b_lo0, first = 0;
                        for (int ky = 0; ky < a.KH; ++ky, ar += row_step, br += b_row_step)
                            for (int j = 0; 2 * j < a.KWp; ++j) {
                                tc_mma_i8_words(d_tmem, ar + 2u * j, a_hi, br + 16u * j, b_hi, a.idesc, first);
                                first = 1u;
                            }
                    }
                    tc_commit(tfull0 + 8u * slot);
                }
                if (ok) tc_commit(pempty0 + 8u * pb);   // the band is free once the item's MMAs have read it
                band += step_b;
                if (band >= a.bands) band -= a.bands;
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        pdl_wait();   // the output buffer may still be read by the previous kernel
        const int ew = warp - Z_EPI_WARP0;
        const int quad = warp & 3;          // TMEM lane quadrant this warp may read
        const int group = ew >> 2;          // drains the tiles whose sequence number is `group` modulo 4
        const unsigned par_off = (unsigned)((unsigned char*)par - smem_raw);
        const unsigned swz_mask = (unsigned)(a.BN / 16 - 1);
        unsigned seq = 0;
        int n = (int)blockIdx.x / a.bands, band = (int)blockIdx.x % a.bands;
        const int step_n = (int)gridDim.x / a.bands, step_b = (int)gridDim.x % a.bands;
        bool ok = true;
        if (POOL) {
            const unsigned cbuf0_off = (unsigned)(stage_out - smem_raw);
            const int epi_tid = ew * 32 + lane;
            const int nvec = a.N >> 4;                       // 16-byte units per pixel
            unsigned bandit = 0;
            for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ++bandit) {
                const int T = band_tiles(band);
                const unsigned cb = bandit & 1u;
                const unsigned cbuf_off = cbuf0_off + cb * (unsigned)a.cbuf_alloc;
                for (int t = 0; t < T; ++t, ++seq) {
                    if ((int)(seq & (Z_SLOTS - 1)) != group) continue;
                    const unsigned sph = (seq / Z_SLOTS) & 1u;
                    if (!mbar_wait_warp(tfull0 + 8u * group, sph, abort_flag, a.status, 4, lane)) { ok = false; break; }
                    tc_fence_after();
                    const unsigned tbase = tmem_base + ((unsigned)(quad * 32) << 16) + (unsigned)(group * a.BN);
                    // this warp's 32 positions of the tile, at their place in the band buffer (a multiple of 32 rows
                    // from its start, so the swizzle term of a row is the one the staging regions use)
                    const unsigned dst_off = cbuf_off + (unsigned)((t * ZBM + quad * 32) * a.BN);
                    if (a.wide) {
                        if (a.out_unsigned) s2d_drain<false, EF_WIDE | EF_OUT_UNSIGNED>(tbase, par_off, dst_off, a.BN, lane);
                        else s2d_drain<false, EF_WIDE>(tbase, par_off, dst_off, a.BN, lane);
                    } else if (a.out_unsigned) s2d_drain<CLAMP, EF_OUT_UNSIGNED>(tbase, par_off, dst_off, a.BN, lane);
                    else s2d_drain<CLAMP, 0>(tbase, par_off, dst_off, a.BN, lane);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tempty0 + 8u * group);
                }
                if (!ok) break;
                // every warp has written its tiles of the band: meet, then pool from the complete band
                __syncwarp();
                if (lane == 0) mbar_arrive(cdone0 + 8u * cb);
                if (!mbar_wait_warp(cdone0 + 8u * cb, (bandit >> 1) & 1u, abort_flag, a.status, 13, lane)) { ok = false; break; }
                const int prow0 = band * a.P;
                const int np = a.pool_oH - prow0 < a.P ? a.pool_oH - prow0 : a.P;
                const int units = np * a.pool_oW * nvec;
                const unsigned char* cbuf = dyn_smem() + cbuf_off;
                for (int u = epi_tid; u < units; u += 32 * Z_EPI_WARPS) {
                    const int v = u % nvec;
                    const int pq = u / nvec;
                    const int q = pq % a.pool_oW, pr = pq / a.pool_oW;
                    uint4 m = make_uint4(0, 0, 0, 0);
                    for (int dy = 0; dy < a.pool_k; ++dy)
                        for (int dx = 0; dx < a.pool_k; ++dx) {
                            const unsigned pos = (unsigned)((pr * a.pool_s + dy) * a.Wp + q * a.pool_s + dx);
                            const unsigned ro = pos * (unsigned)a.BN;
                            const uint4 x = *(const uint4*)(cbuf + ro + ((((unsigned)v) ^ ((ro >> 7) & swz_mask)) << 4));
                            if ((dy | dx) == 0) m = x;
                            else if (a.out_unsigned) {
                                m.x = __vmaxu4(m.x, x.x); m.y = __vmaxu4(m.y, x.y); m.z = __vmaxu4(m.z, x.z); m.w = __vmaxu4(m.w, x.w);
                            } else {
                                m.x = __vmaxs4(m.x, x.x); m.y = __vmaxs4(m.y, x.y); m.z = __vmaxs4(m.z, x.z); m.w = __vmaxs4(m.w, x.w);
                            }
                        }
                    uint8_t* dst = (uint8_t*)a.out + ((((size_t)n * a.pool_oH + (size_t)(prow0 + pr)) * a.pool_oW + q) * a.N);
                    *(uint4*)(dst + v * 16) = m;
                }
                n += step_n;
                band += step_b;
                if (band >= a.bands) { band -= a.bands; ++n; }
            }
        } else {
        for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
            const int rows = band_rows(band);
            const int T = band_tiles(band);
            uint8_t* const band_out = (uint8_t*)a.out + ((size_t)n * a.oH + (size_t)(band * a.R)) * a.oW * a.N;
            for (int t = 0; t < T; ++t, ++seq) {
                if ((int)(seq & (Z_SLOTS - 1)) != group) continue;
                const unsigned sph = (seq / Z_SLOTS) & 1u;
                if (!mbar_wait_warp(tfull0 + 8u * group, sph, abort_flag, a.status, 4, lane)) { ok = false; break; }
                tc_fence_after();
                const unsigned tbase = tmem_base + ((unsigned)(quad * 32) << 16) + (unsigned)(group * a.BN);
                // This lane's four rows of the fragment (positions of the band's raster) and where they go: the bytes leave
                // the registers for global memory directly, eight channels per lane, a 32-byte sector per four lanes
                unsigned rowoff[4];   // byte offsets within the band: below 2^32
                unsigned rowok = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const unsigned p = (unsigned)(t * ZBM + quad * 32 + (lane >> 2) + 8 * k);
                    const unsigned yy = __umulhi(p, a.rcp_Wp);
                    const unsigned x = p - yy * (unsigned)a.Wp;
                    if (x < (unsigned)a.oW && yy < (unsigned)rows) rowok |= 1u << k;
                    rowoff[k] = (yy * (unsigned)a.oW + x) * (unsigned)a.N;
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

// filter extents after space-to-depth; `off` = 1 when the padding is odd (the image is shifted by one more
// pixel so that every output's window starts on an even pixel)
static void s2d_filter(const ConvGeom& g, int* P, int* KH, int* KWp)
{
    const int offy = g.pT & 1, offx = g.pL & 1;
    *P = g.pT + offy;
    *KH = (g.kH + offy + 1) / 2;
    const int kw = (g.kW + offx + 1) / 2;
    *KWp = (kw + 1) & ~1;   // an MMA covers two pixels
}

// cbuf_alloc: bytes of one band-sized output buffer of the fused-pooling variant (0: per-warp staging regions)
static size_t s2d_smem_bytes(int w_bytes, int BN, int band_alloc, int cbuf_alloc = 0)
{
    const size_t b = ((size_t)w_bytes + 1023) & ~(size_t)1023;
    return 1024 + b + 2 * (size_t)band_alloc + (cbuf_alloc ? 2 * (size_t)cbuf_alloc : (size_t)Z_EPI_WARPS * 32 * BN)
         + (4 + 2 * Z_SLOTS + 2 + 2) * 8 + 32 + FAST_NP * 256 * 4 + 64;
}

static int s2d_band_alloc(int Wp, int KH, int KWp, int R)
{
    const int tiles = (R * Wp + ZBM - 1) / ZBM;
    const int reach = tiles * ZBM + (KH - 1) * Wp + KWp;   // last tile's rows, the filter's extent and the overlap
    const int box = (R + KH - 1) * Wp;
    const int px = reach > box ? reach : box;
    return (px * 16 + 1023) & ~1023;
}

bool stem_s2d_eligible(const ConvGeom& g)
{
    if (g.groups != 1 || g.C > 4 || g.sX != 2 || g.sY != 2 || g.dX != 1 || g.dY != 1) return false;
    if (g.pT != g.pL || g.kH > 16 || g.kW > 16) return false;
    if (g.O % 32 != 0 || g.O > 128 || g.oW < 2 || g.oH < 1) return false;
    int P, KH, KWp;
    s2d_filter(g, &P, &KH, &KWp);
    const int Wp = g.oW + KWp - 1;
    if (Wp * 2 > 256) return false;   // one row of the band is one row of the TMA box (8-byte elements)
    const int BN = g.O <= 64 ? 64 : 128;
    const int w_bytes = KH * BN * KWp * 16;
    if (w_bytes > 64 * 1024) return false;
    return s2d_smem_bytes(w_bytes, BN, s2d_band_alloc(Wp, KH, KWp, 1)) <= 226 * 1024;
}

void stem_s2d_dims(const ConvGeom& g, int* Hs, int* Ws)
{
    int P, KH, KWp;
    s2d_filter(g, &P, &KH, &KWp);
    *Hs = g.oH + KH - 1;
    *Ws = g.oW + KWp - 1;
}

size_t stem_s2d_weight_bytes(const ConvGeom& g)
{
    int P, KH, KWp;
    s2d_filter(g, &P, &KH, &KWp);
    const int BN = g.O <= 64 ? 64 : 128;
    return (size_t)KH * BN * KWp * 16;
}

// OHWI int8 weights -> per filter row of the re-laid problem a BN x (KWp*16) block in the canonical
// unswizzled K-major order [n / 8][k / 16][n % 8][k % 16], k = X * 16 + (dy * 2 + dx) * 4 + c.  Row n of a block holds
// output channel perm_real_channel(n, 4): the order the epilogue's fragment layout wants (see perm_block).
void stem_s2d_arrange_weights(const ConvGeom& g, const int8_t* w_ohwi, int8_t* dst)
{
    int P, KH, KWp;
    s2d_filter(g, &P, &KH, &KWp);
    const int BN = g.O <= 64 ? 64 : 128;
    const int offy = P - g.pT, offx = P - g.pL;
    const size_t row_block = (size_t)BN * KWp * 16;
    memset(dst, 0, (size_t)KH * row_block);
    for (int n = 0; n < BN; ++n) {
        const int o = perm_real_channel(n, 4);
        if (o >= g.O) continue;
        for (int ky = 0; ky < g.kH; ++ky)
            for (int kx = 0; kx < g.kW; ++kx)
                for (int c = 0; c < g.C; ++c) {
                    const int yy = ky + offy, xx = kx + offx;       // tap position in the shifted image
                    const int Y = yy >> 1, dy = yy & 1, X = xx >> 1, dx = xx & 1;
                    const int k = X * 16 + (dy * 2 + dx) * 4 + c;
                    const size_t off = (size_t)Y * row_block + (size_t)(n / 8) * (KWp * 128) + (size_t)(k / 16) * 128
                                     + (size_t)(n % 8) * 16 + (size_t)(k % 16);
                    dst[off] = w_ohwi[(((size_t)o * g.kH + ky) * g.kW + kx) * g.C + c];
                }
    }
}

cudaError_t launch_s2d_image(const void* in, const ConvGeom& g, int batch, void* out, cudaStream_t s)
{
    int P, KH, KWp, Hs, Ws;
    s2d_filter(g, &P, &KH, &KWp);
    stem_s2d_dims(g, &Hs, &Ws);
    const long long rows = (long long)batch * Hs;
    if (rows == 0) return cudaSuccess;
    const unsigned grid = (unsigned)(rows < (1ll << 20) ? rows : (1ll << 20));
    const int threads = Ws >= 128 ? 128 : ((Ws + 31) / 32) * 32;
    s2d_image_kernel<<<grid, threads, 0, s>>>((const uint8_t*)in, g.C, g.H, g.W, Hs, Ws, P, (int)rows, (uint4*)out);
    return cudaGetLastError();
}

// A max pooling this kernel can fold in: square window, same stride both ways, no padding, 8-bit channels in whole
// 16-byte units.
bool stem_s2d_pool_eligible(const ConvGeom& g, const PoolGeom& p)
{
    if (!(stem_s2d_eligible(g) && p.is_max && p.pH == p.pW && p.sY == p.sX && p.padY == 0 && p.padX == 0 && p.pH >= 1 && p.pH <= 4
          && p.sY >= 1 && p.sY <= p.pH && p.H == g.oH && p.W == g.oW && p.C == g.O && g.O % 16 == 0 && p.oH >= 1 && p.oW >= 1))
        return false;
    // one pooled row per band must fit shared memory
    int P0, KH, KWp;
    s2d_filter(g, &P0, &KH, &KWp);
    const int Wp = g.oW + KWp - 1, BN = g.O <= 64 ? 64 : 128, R = p.pH;
    const int cbuf = ((R * Wp + ZBM - 1) / ZBM) * ZBM * BN;
    return s2d_smem_bytes(KH * BN * KWp * 16, BN, s2d_band_alloc(Wp, KH, KWp, R), cbuf) <= 226 * 1024;
}

int stem_s2d_make_plan(StemS2dPlan* plan, const void* d_s2d, const int8_t* d_w_arranged, const ConvGeom& g, int max_batch,
                       int in_unsigned, int num_sms, const char** why, const PoolGeom* pool)
{
    static const char* kWhy = "";
    *why = kWhy;
    if (!stem_s2d_eligible(g)) { *why = "geometry outside the space-to-depth first-layer kernel"; return -1; }
    cudaDriverEntryPointQueryResult qr;
    void* fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) != cudaSuccess || !fn) {
        *why = "cuTensorMapEncodeTiled is not available from the CUDA driver";
        return -1;
    }
    memset(plan, 0, sizeof(*plan));
    int P;
    s2d_filter(g, &P, &plan->KH, &plan->KWp);
    plan->BN = g.O <= 64 ? 64 : 128;
    plan->Wp = g.oW + plan->KWp - 1;
    plan->w_bytes = plan->KH * plan->BN * plan->KWp * 16;
    plan->w = d_w_arranged;
    plan->in_unsigned = in_unsigned;
    plan->num_sms = num_sms;
    int best_R = 0;
    long long best_tiles = 0;
    if (pool) {
        // the most pooled rows per band that fit: fewer bands recompute fewer overlapping convolution rows
        if (!stem_s2d_pool_eligible(g, *pool)) { *why = "pooling outside the fused first-layer kernel"; return -1; }
        for (int P = 1; P <= pool->oH; ++P) {
            const int R = (P - 1) * pool->sY + pool->pH;
            if (R + plan->KH - 1 > 256) break;
            const int cbuf = ((R * plan->Wp + ZBM - 1) / ZBM) * ZBM * plan->BN;
            if (s2d_smem_bytes(plan->w_bytes, plan->BN, s2d_band_alloc(plan->Wp, plan->KH, plan->KWp, R), cbuf) > 226 * 1024) break;
            best_R = R;
            plan->P = P;
            plan->cbuf_alloc = cbuf;
        }
        if (best_R == 0) { *why = "no band of the fused pooling fits shared memory"; return -1; }
        plan->pool_k = pool->pH; plan->pool_s = pool->sY; plan->pool_oH = pool->oH; plan->pool_oW = pool->oW;
        plan->R = best_R;
        plan->row_stride = plan->P * pool->sY;
        plan->bands = (pool->oH + plan->P - 1) / plan->P;
    } else {
    for (int R = 1; R <= g.oH; ++R) {
        if (R + plan->KH - 1 > 256) break;
        if (s2d_smem_bytes(plan->w_bytes, plan->BN, s2d_band_alloc(plan->Wp, plan->KH, plan->KWp, R)) > 226 * 1024) break;
        const int full = g.oH / R, rest = g.oH % R;
        const long long tiles = (long long)full * ((R * plan->Wp + ZBM - 1) / ZBM)
                              + (rest ? (rest * plan->Wp + ZBM - 1) / ZBM : 0);
        if (best_R == 0 || tiles <= best_tiles) { best_R = R; best_tiles = tiles; }
    }
    if (best_R == 0) { *why = "no band height fits shared memory"; return -1; }
    plan->R = best_R;
    plan->row_stride = best_R;
    plan->bands = (g.oH + best_R - 1) / best_R;
    }
    const int box_rows = best_R + plan->KH - 1;
    plan->band_bytes = box_rows * plan->Wp * 16;
    plan->band_alloc = s2d_band_alloc(plan->Wp, plan->KH, plan->KWp, best_R);
    plan->smem_bytes = s2d_smem_bytes(plan->w_bytes, plan->BN, plan->band_alloc, plan->cbuf_alloc);
    int Hs, Ws;
    stem_s2d_dims(g, &Hs, &Ws);
    // the re-laid image as (8-byte words of a row, rows, images): one box = one band, rows below the image read as zero
    const cuuint64_t dims[3] = {(cuuint64_t)Ws * 2, (cuuint64_t)Hs, (cuuint64_t)max_batch};
    const cuuint64_t strides[2] = {(cuuint64_t)Ws * 16, (cuuint64_t)Ws * 16 * Hs};
    const cuuint32_t box[3] = {(cuuint32_t)plan->Wp * 2, (cuuint32_t)box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult rc = ((EncodeTiledFn)fn)(&plan->tmA, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, (void*)d_s2d, dims, strides, box, estr,
                                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) { *why = "cuTensorMapEncodeTiled failed for the re-laid image"; return -1; }
    return 0;
}

cudaError_t launch_stem_s2d(const StemS2dPlan& plan, const ConvGeom& g, int n_base, const FastQuant& fast, void* out,
                            int* status_word, cudaStream_t s)
{
    S2dArgs a;
    memset(&a, 0, sizeof(a));
    a.B = g.B; a.oH = g.oH; a.oW = g.oW; a.N = g.O; a.BN = plan.BN;
    if (a.B == 0) return cudaSuccess;
    a.KH = plan.KH; a.KWp = plan.KWp; a.Wp = plan.Wp; a.R = plan.R; a.bands = plan.bands;
    a.row_stride = plan.row_stride;
    a.pool_k = plan.pool_k; a.pool_s = plan.pool_s; a.P = plan.P; a.pool_oH = plan.pool_oH; a.pool_oW = plan.pool_oW;
    a.cbuf_alloc = plan.cbuf_alloc;
    a.n_base = n_base;
    a.band_bytes = plan.band_bytes; a.band_alloc = plan.band_alloc; a.w_bytes = plan.w_bytes;
    a.rcp_Wp = (unsigned)(((1ull << 32) + (unsigned)plan.Wp - 1) / (unsigned)plan.Wp);
    a.idesc = (2u << 4) | ((plan.in_unsigned ? 0u : 1u) << 7) | (1u << 10) | ((unsigned)(plan.BN >> 3) << 17)
            | ((unsigned)(ZBM >> 4) << 24);
    a.tmem_cols = (unsigned)(Z_SLOTS * plan.BN);
    a.w = plan.w;
    a.out = out;
    a.status = status_word;
    a.fq = fast.fq;
    a.cpad = fast.cpad;
    a.out_unsigned = fast.out_unsigned;
    a.wide = fast.wide ? 1 : 0;
    typedef void (*Kernel)(const CUtensorMap, const S2dArgs);
    static const Kernel variants[12] = {stem_s2d_tcgen05_kernel<false, 0, false>, stem_s2d_tcgen05_kernel<false, 1, false>,
                                        stem_s2d_tcgen05_kernel<false, 2, false>, stem_s2d_tcgen05_kernel<true, 0, false>,
                                        stem_s2d_tcgen05_kernel<true, 1, false>,  stem_s2d_tcgen05_kernel<true, 2, false>,
                                        stem_s2d_tcgen05_kernel<false, 0, true>,  stem_s2d_tcgen05_kernel<false, 1, true>,
                                        stem_s2d_tcgen05_kernel<false, 2, true>,  stem_s2d_tcgen05_kernel<true, 0, true>,
                                        stem_s2d_tcgen05_kernel<true, 1, true>,   stem_s2d_tcgen05_kernel<true, 2, true>};
    static std::atomic<bool> attr_set[64];   // set twice by racing first calls at worst: harmless
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        for (Kernel k : variants) {
            cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e != cudaSuccess) return e;
        }
        attr_set[dev] = true;
    }
    const long long items = (long long)a.B * a.bands;
    const int grid = (int)(items < plan.num_sms ? items : plan.num_sms);
    const int shape = (plan.KH == 4 && plan.KWp == 4) ? 1 : ((plan.KH == 2 && plan.KWp == 2) ? 2 : 0);
    return launch_pdl(variants[(plan.P ? 6 : 0) + (fast.need_clamp ? 3 : 0) + shape], grid, Z_THREADS, plan.smem_bytes, s, plan.tmA, a);
}

}  // namespace n2d2b
