// Implicit-GEMM convolution / fully-connected kernel on the Blackwell tensor cores.
//
//   D[M x N] (int32, in TMEM) = A[M x K] (u8 or s8 activations, NHWC) * B[N x K]^T (s8 weights, OHWI)
//   M = output pixels (batch * oH * oW), N = output channels, K = taps * Cin walked tap by tap.
//
// One persistent CTA per SM loops over 128 x BN output tiles.  Warp 0 issues TMA loads into a
// multi-stage shared-memory ring (A tile through a 2-D tiled map for a plain GEMM, or through an
// im2col map that applies stride / padding / dilation and zero-fills the halo; B tile through a 2-D
// map, or once into a resident block when the layer's weights are small), warp 1 issues
// tcgen05.mma kind::i8 into one of two TMEM accumulators, warps 2-17 drain the other accumulator with
// tcgen05.ld and run the fused epilogue (bias, per-channel rescale, rounding, saturation, ReLU,
// optional residual add + second rescale) straight to int8 NHWC: every warp owns the 32 rows of its
// TMEM lane quadrant and a quarter of the tile's columns.  Cells on the 32-bit epilogue store their weight
// rows permuted inside blocks of 32 (16) output channels, so that the column pairs a TMEM load hands a
// thread are 8 (4) consecutive channels: constants, residual and output move as 128- and 64-bit accesses.  This replaces the reference's
// cudnnConvolutionForward + cudnnAddTensor + Scaling kernel + cudnnActivationForward sequence
// (src/Cell/ConvCell_Frame_CUDA.cpp:1169-1270) and its cublasGemm FC
// (src/Cell/FcCell_Frame_CUDA.cpp:308-427).
//
// The kernel is launched with programmatic stream serialization: barriers, TMEM, constants and
// resident weights are set up while the previous kernel drains; activations are touched only after
// griddepcontrol.wait.
//
// Every wait on an mbarrier is bounded: a wait that does not complete within about a second sets
// *status_word and makes the whole CTA drain and exit, so a wrong descriptor cannot hang the GPU.
#include <cstdio>
#include <cstring>
#include <atomic>
#include "kernels.h"
#include "tc_common.cuh"

namespace n2d2b {

static constexpr int BM = 128;
static constexpr int EPI_WARP0 = 2;
static constexpr int NUM_EPI_WARPS = 16;      // four per TMEM lane quadrant, a quarter of the columns each
static constexpr int REGION_BYTES = 2048;     // staging per epilogue warp: 32 rows x up to 64 bytes
static constexpr int NUM_THREADS = 32 * (EPI_WARP0 + NUM_EPI_WARPS);
static constexpr int W4_UNPACK_WARPS = 4;     // extra warps of the packed-int4 variant

struct IgemmArgs {
    int M, N, Cin, taps, BK, BN, stages, a_im2col;
    int grouped;        // block-diagonal layer (depthwise as groups of BN channels): a column block reads its own input channels
    int res_slots;          // staging regions per epilogue warp of a residual cell (2 or 4)
    int m_base;         // first output row of this call within the tensors (a batch slice starts at image img0)
    int b_resident;     // the CTA's whole weight block stays in shared memory (its column block never changes)
    int oW, oH, kW, sX, sY, pL, pT, dX, dY;
    int num_m_tiles, num_n_tiles;
    int step_m, step_n;   // gridDim.x / num_n_tiles and gridDim.x % num_n_tiles: one persistent-loop step in tile coordinates
    int ef;               // EF_* switches of the 32-bit epilogue
    unsigned idesc;
    unsigned tmem_cols;
    int out_dtype;
    void* out;
    int* status;
    QuantDev q;
    Residual r;
    // fast 32-bit epilogue: y = (clamp(acc, lo, hi) * mult + add) >> shift, rows of cpad entries
    const int* fq;      // [FAST_NP][cpad] of the cell
    const int* fq2;     // [FAST_NP][cpad] of the fused residual sum (nullptr without one)
    int cpad;
    int t_lo, t_hi;     // saturation range of the cell's own output (before the residual add)
    int out_unsigned;   // final 8-bit range: 1 = [0,255], 0 = [-128,127]
    unsigned dp_xor;    // dot-product form of the residual stage: byte flips and operand signedness
    int dp_a_signed;
};

// ----------------------------------------------------------------------------- the kernel
// Eight packed 4-bit weights (one 32-bit word: byte i = elements 2i in the high and 2i + 1 in the low nibble) as
// eight signed bytes holding 16 x the weight: the nibble moves to the top of its byte, which is the value times 16
// with the right sign and needs no sign extension.  The accumulator then holds 16 x the sum, a multiple of 16: the
// epilogue shifts it right by four first, which is exact.
__device__ __forceinline__ void expand_int4_x16(unsigned x, unsigned& w0, unsigned& w1)
{
    const unsigned hi = x & 0xF0F0F0F0u, lo = (x << 4) & 0xF0F0F0F0u;
    w0 = __byte_perm(hi, lo, 0x5140);   // hi.b0, lo.b0, hi.b1, lo.b1
    w1 = __byte_perm(hi, lo, 0x7362);   // hi.b2, lo.b2, hi.b3, lo.b3
}

// W4: the weights sit in HBM as packed 4-bit values.  The producer's TMA load brings a BN x BK/2-byte packed block
// into the stage beside the operand tiles; four extra warps expand it into the swizzled int8 B tile the MMA reads
// (as 16 x the weight, see expand_int4_x16) and signal the issuing thread through one more barrier per stage.
template <int MODE, bool W4>
__global__ void __launch_bounds__(W4 ? NUM_THREADS + 32 * W4_UNPACK_WARPS : NUM_THREADS, 1)
igemm_i8_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmO, const __grid_constant__ CUtensorMap tmR,
                        const IgemmArgs a)
{
    constexpr bool FAST = MODE != 0;
    constexpr bool RES = (MODE == 2 || MODE == 4 || MODE == 5);
    constexpr bool CLAMP = (MODE == 1 || MODE == 2);
    constexpr bool DP = (MODE == 5);
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment of the tile ring (required by the 128-byte swizzle)
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int a_stage_bytes = BM * a.BK;
    const int b_stage_bytes = a.BN * a.BK;
    const int p_stage_bytes = W4 ? b_stage_bytes / 2 : 0;                       // packed weights of the stage
    const int stage_bytes = a_stage_bytes + (a.b_resident ? 0 : b_stage_bytes) + p_stage_bytes;
    const int tx_bytes = a_stage_bytes + (W4 ? p_stage_bytes : (a.b_resident ? 0 : b_stage_bytes));   // what TMA delivers per stage
    const int kchunks = (a.Cin + a.BK - 1) / a.BK;
    const int num_kb = a.taps * kchunks;
    // resident weights first (one BN x BK block per K block), then the ring of activation (and weight) stages
    unsigned char* res_b = smem;
    unsigned char* tiles = smem + (a.b_resident ? (size_t)num_kb * b_stage_bytes : 0);
    unsigned char* stage_out = tiles + (size_t)a.stages * stage_bytes;
    // output staging: one region per epilogue warp (32 rows x up to 64 bytes, swizzled for TMA)
    // cells with a fused residual keep two or four regions per warp so that the residual of the next tiles arrives early
    const int regions_per_warp = RES ? a.res_slots : 1;
    unsigned long long* bars = (unsigned long long*)(stage_out + NUM_EPI_WARPS * REGION_BYTES * regions_per_warp);
    // bars: full[stages], empty[stages], tmem_full[2], tmem_empty[2], params_ready[2], residual[4 * NUM_EPI_WARPS],
    //       resident weights
    const unsigned full0 = smem_u32(bars);
    const unsigned empty0 = full0 + 8u * a.stages;
    const unsigned tfull0 = empty0 + 8u * a.stages;
    const unsigned tempty0 = tfull0 + 16u;
    const unsigned pready0 = tempty0 + 16u;
    const unsigned rbar0 = pready0 + 16u;
    const unsigned bfull = rbar0 + 8u * (4 * NUM_EPI_WARPS);
    const unsigned bready0 = bfull + 16u;                                       // W4: expanded weights of a stage are in place
    unsigned* tmem_slot = (unsigned*)(bars + 2 * a.stages + 6 + 4 * NUM_EPI_WARPS + 2 + (W4 ? a.stages : 0));
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    // [2 buffers][2 quant sets][FAST_NP][256], 16-byte aligned for vector loads
    int* epi_params = (int*)(((uintptr_t)(tmem_slot + 4) + 15) & ~(uintptr_t)15);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(full0 + 8u * s, 1);
            mbar_init(empty0 + 8u * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(tfull0 + 8u * s, 1);
            mbar_init(tempty0 + 8u * s, NUM_EPI_WARPS);
            mbar_init(pready0 + 8u * s, NUM_EPI_WARPS);
        }
        for (int w = 0; w < 4 * NUM_EPI_WARPS; ++w) mbar_init(rbar0 + 8u * w, 1);
        mbar_init(bfull, 1);
        if (W4)
            for (int s = 0; s < a.stages; ++s) mbar_init(bready0 + 8u * s, W4_UNPACK_WARPS);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    const unsigned tiles_s = smem_u32(tiles), res_b_s = smem_u32(res_b);

    const int num_tiles = a.num_m_tiles * a.num_n_tiles;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            unsigned it = 0;
            bool ok = true;
            if (a.b_resident && (int)blockIdx.x < num_tiles) {
                // the launch keeps every CTA on one column block: its weights are fetched once
                const int n0 = ((int)blockIdx.x % a.num_n_tiles) * a.BN;
                mbar_expect_tx(bfull, (unsigned)(num_kb * b_stage_bytes));
                for (int kb = 0; kb < num_kb; ++kb) {
                    const int tap = kb / kchunks;
                    const int kc = kb - tap * kchunks;
                    tma_load_2d(smem_u32(res_b + (size_t)kb * b_stage_bytes), &tmB, bfull, tap * a.Cin + kc * a.BK, n0);
                }
            }
            pdl_wait();   // weights are constants; the activations are the previous kernel's output
            // The loops below keep ring slot, phase, tap and channel-chunk as running counters: a single
            // thread pays the full latency of every dependent instruction, so an integer division per K
            // block costs more than the load it prepares.
            int s = 0;
            unsigned ph = 0;
            int m_tile = (int)blockIdx.x / a.num_n_tiles, n_tile = (int)blockIdx.x % a.num_n_tiles;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m0 = a.m_base + m_tile * BM, n0 = n_tile * a.BN;
                m_tile += a.step_m;
                n_tile += a.step_n;
                if (n_tile >= a.num_n_tiles) { n_tile -= a.num_n_tiles; ++m_tile; }
                int iw0 = 0, ih0 = 0, in0 = 0;
                if (a.a_im2col) {
                    const int ox = m0 % a.oW;
                    const int t = m0 / a.oW;
                    const int oy = t % a.oH;
                    in0 = t / a.oH;
                    iw0 = ox * a.sX - a.pL;
                    ih0 = oy * a.sY - a.pT;
                }
                int kx = 0, ky = 0, kc = 0, kcoord = 0;   // kcoord = tap * Cin + kc * BK
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    if (!mbar_wait(empty0 + 8u * s, ph ^ 1u, abort_flag, a.status, 1)) { ok = false; break; }
                    const unsigned bar = full0 + 8u * s;
                    const unsigned dstA = tiles_s + (unsigned)(s * stage_bytes);
                    mbar_expect_tx(bar, (unsigned)tx_bytes);
                    if (a.a_im2col) {
                        tma_load_im2col_4d(dstA, &tmA, bar, kc * a.BK + (a.grouped ? n0 : 0), iw0, ih0, in0,
                                           (unsigned short)(kx * a.dX), (unsigned short)(ky * a.dY));
                    } else {
                        tma_load_2d(dstA, &tmA, bar, kcoord, m0);
                    }
                    if (W4) tma_load_2d(dstA + a_stage_bytes + b_stage_bytes, &tmB, bar, kcoord >> 1, n0);   // packed: two per byte
                    else if (!a.b_resident) tma_load_2d(dstA + a_stage_bytes, &tmB, bar, kcoord, n0);
                    if (++s == a.stages) { s = 0; ph ^= 1u; }
                    if (++kc == kchunks) {
                        kc = 0;
                        kcoord += a.Cin - (kchunks - 1) * a.BK;
                        if (++kx == a.kW) { kx = 0; ++ky; }
                    } else {
                        kcoord += a.BK;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        // The issuing thread pays the latency of every instruction it executes, so what surrounds a short
        // MMA is kept to 32-bit adds on running descriptor words and an unrolled K loop.
        if (lane == 0) {
            unsigned acc_it = 0;
            bool ok = true;
            if (a.b_resident && (int)blockIdx.x < num_tiles) ok = mbar_wait(bfull, 0, abort_flag, a.status, 8);
            int s = 0;
            unsigned ph = 0;
            // upper descriptor word: stride between 8-row groups, version, swizzle; lower word: address / 16
            const unsigned desc_hi = (unsigned)(make_smem_desc(0u, a.BK) >> 32);
            const unsigned a_lo0 = (tiles_s & 0x3ffffu) >> 4, b_res0 = (res_b_s & 0x3ffffu) >> 4;
            const unsigned stage16 = (unsigned)(stage_bytes >> 4), a16 = (unsigned)(a_stage_bytes >> 4);
            const unsigned b16 = (unsigned)(b_stage_bytes >> 4);
            unsigned a_lo = a_lo0;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++acc_it) {
                const unsigned as = acc_it & 1u;
                const unsigned aph = (acc_it >> 1) & 1u;
                if (!mbar_wait(tempty0 + 8u * as, aph ^ 1u, abort_flag, a.status, 2)) { ok = false; break; }
                tc_fence_after();
                const unsigned d_tmem = tmem_base + as * (unsigned)a.BN;
                unsigned b_res = b_res0;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(full0 + 8u * s, ph, abort_flag, a.status, 3)) { ok = false; break; }
                    if (W4 && !mbar_wait(bready0 + 8u * s, ph, abort_flag, a.status, 11)) { ok = false; break; }
                    tc_fence_after();
                    const unsigned b_lo = a.b_resident ? b_res : a_lo + a16;
                    const unsigned acc = kb ? 1u : 0u;
                    // advancing K by 32 bytes inside the swizzle span = +2 in the 16-byte address field
                    if (a.BK == 128) {
                        tc_mma_i8_lohi(d_tmem, a_lo, b_lo, desc_hi, a.idesc, acc);
                        tc_mma_i8_lohi(d_tmem, a_lo + 2u, b_lo + 2u, desc_hi, a.idesc, 1u);
                        tc_mma_i8_lohi(d_tmem, a_lo + 4u, b_lo + 4u, desc_hi, a.idesc, 1u);
                        tc_mma_i8_lohi(d_tmem, a_lo + 6u, b_lo + 6u, desc_hi, a.idesc, 1u);
                    } else if (a.BK == 64) {
                        tc_mma_i8_lohi(d_tmem, a_lo, b_lo, desc_hi, a.idesc, acc);
                        tc_mma_i8_lohi(d_tmem, a_lo + 2u, b_lo + 2u, desc_hi, a.idesc, 1u);
                    } else {
                        tc_mma_i8_lohi(d_tmem, a_lo, b_lo, desc_hi, a.idesc, acc);
                    }
                    tc_commit(empty0 + 8u * s);  // frees the stage once these MMAs have read it
                    a_lo += stage16;
                    b_res += b16;
                    if (++s == a.stages) { s = 0; ph ^= 1u; a_lo = a_lo0; }
                }
                if (ok) tc_commit(tfull0 + 8u * as);
            }
        }
    } else if (W4 && warp >= EPI_WARP0 + NUM_EPI_WARPS) {
        // ------------------------------------------------------------------ int4 expansion warps
        // Stage s may be rewritten once full[s] has completed for the new fill: the producer only refills a stage
        // after the MMAs that read its previous contents have committed (empty[s]).
        const int ut = (warp - (EPI_WARP0 + NUM_EPI_WARPS)) * 32 + lane;
        const int cpr_shift = a.BK == 128 ? 3 : (a.BK == 64 ? 2 : 1);   // 16-byte chunks per B row: BK / 16
        const int total_chunks = a.BN << cpr_shift;
        const int half_bk = a.BK >> 1;
        int s = 0;
        unsigned ph = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            for (int kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait_warp(full0 + 8u * s, ph, abort_flag, a.status, 12, lane)) { ok = false; break; }
                unsigned char* bt = tiles + (size_t)s * stage_bytes + a_stage_bytes;
                const unsigned char* pk = bt + b_stage_bytes;
#pragma unroll 2
                for (int id = ut; id < total_chunks; id += 32 * W4_UNPACK_WARPS) {
                    const int row = id >> cpr_shift, ch = id & ((1 << cpr_shift) - 1);
                    const uint2 p = *(const uint2*)(pk + row * half_bk + ch * 8);
                    uint4 o;
                    expand_int4_x16(p.x, o.x, o.y);
                    expand_int4_x16(p.y, o.z, o.w);
                    *(uint4*)(bt + swz_off(row, ch * 16, a.BK)) = o;
                }
                fence_async_smem();   // generic-proxy stores, read by the tensor core through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(bready0 + 8u * s);
                if (++s == a.stages) { s = 0; ph ^= 1u; }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        pdl_wait();   // residual loads and output stores touch tensors the previous kernel reads or writes
        const int quad = warp & 3;                       // TMEM lane quadrant this warp may read
        const int part = (warp - EPI_WARP0) >> 2;        // 0..3 within the quadrant: a quarter of the columns (32-bit epilogue)
        const int row = quad * 32 + lane;
        const int epi_tid = (warp - EPI_WARP0) * 32 + lane;
        // the exact 64-bit epilogue works in 32-column chunks on the first two warps of each quadrant
        const int cols_per_warp = a.BN / 2;
        unsigned acc_it = 0;
        unsigned stage_it = 0;
        EpiState est;
        perm_rowbase(est.rb, a.BN >> 2, lane, (a.BN >> 2) >= 32 ? 4 : 2);
        int staged_n_tile = -1;
        int* par = epi_params;
        bool ok = true;
        int m_next = (int)blockIdx.x / a.num_n_tiles, n_next = (int)blockIdx.x % a.num_n_tiles;
        // residual loads run ahead of the tiles: pf_* walk the same tile sequence, res_slots - 1 tiles in front
        int pf_tile = blockIdx.x, pf_m = m_next, pf_n = n_next;
        unsigned pf_it = 0;
        const unsigned slot_shift = a.res_slots == 4 ? 2u : 1u;
        const unsigned lookahead = a.res_slots == 4 ? 3u : 2u;
        const unsigned my_regions = (unsigned)(stage_out - smem_raw) + (unsigned)((warp - EPI_WARP0) * REGION_BYTES * regions_per_warp);
        const unsigned my_rbar = rbar0 + 32u * (unsigned)(warp - EPI_WARP0);
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++acc_it) {
            const int n_tile = n_next, m_tile = m_next;
            m_next += a.step_m;
            n_next += a.step_n;
            if (n_next >= a.num_n_tiles) { n_next -= a.num_n_tiles; ++m_next; }
            const int m0 = a.m_base + m_tile * BM, n0 = n_tile * a.BN;
            const unsigned as = acc_it & 1u;
            const unsigned aph = (acc_it >> 1) & 1u;
            if (FAST && n_tile != staged_n_tile) {
                // stage this column block's per-channel constants (once per CTA when the grid is a
                // multiple of the number of column blocks).  Two buffers: the other one may still be
                // read by slower warps, this one is free once everybody passed the previous barrier.
                par = epi_params + (size_t)(stage_it & 1u) * (2 * FAST_NP * 256);
                const int nq = a.fq2 ? 2 : 1;
                for (int i = epi_tid; i < nq * FAST_NP * a.BN; i += 32 * NUM_EPI_WARPS) {
                    const int set = i / (FAST_NP * a.BN);
                    const int rem = i - set * FAST_NP * a.BN;
                    const int prm = rem / a.BN, c = rem - prm * a.BN;
                    const int* src = set ? a.fq2 : a.fq;
                    par[(set * FAST_NP + prm) * 256 + c] = __ldg(src + (size_t)prm * a.cpad + n0 + c);
                }
                const unsigned pb = pready0 + 8u * (stage_it & 1u);
                __syncwarp();
                if (lane == 0) mbar_arrive(pb);
                if (!mbar_wait_warp(pb, (stage_it >> 1) & 1u, abort_flag, a.status, 5, lane)) { ok = false; break; }
                staged_n_tile = n_tile;
                ++stage_it;
            }
            const int m = m0 + row;
            const bool m_ok = m < a.m_base + a.M;
            const int nchunks = cols_per_warp / 32;
            const int cbase = part * cols_per_warp;
            if (FAST) {
                // fragment-layout epilogue with swizzled staging, TMA store and TMA residual load
                EpiTile e;
                e.tmem_acc = tmem_base + as * (unsigned)a.BN;
                e.BN = a.BN; e.N = a.N; e.M = a.m_base + a.M; e.m0 = m0; e.n0 = n0;
                e.wp = a.BN >> 2;
                e.par_off = (unsigned)((unsigned char*)par - smem_raw);
                e.region_off = my_regions;
                e.region_stride = RES ? REGION_BYTES : 0;
                e.slot_shift = slot_shift;
                e.rbar = my_rbar;
                if (RES) {
                    if (lane == 0) {
                        // two regions: the previous tile's store has finished reading, its region takes the next
                        // tile.  Four regions: the store before that one has, its region takes the tile two ahead,
                        // and nobody waits on a store that has only just been issued.
                        if (a.res_slots == 4) bulk_wait_read_1(); else bulk_wait_read_all();
                        while (pf_it < acc_it + lookahead && pf_tile < num_tiles) {
                            epi_issue_residual(&tmR, my_regions, REGION_BYTES, my_rbar, pf_it & ((1u << slot_shift) - 1u),
                                               pf_n * a.BN + part * e.wp, a.m_base + pf_m * BM + quad * 32, a.N, e.M, e.wp);
                            ++pf_it;
                            pf_tile += (int)gridDim.x;
                            pf_m += a.step_m;
                            pf_n += a.step_n;
                            if (pf_n >= a.num_n_tiles) { pf_n -= a.num_n_tiles; ++pf_m; }
                        }
                    }
                    __syncwarp();
                }
                e.tfull = tfull0 + 8u * as; e.tfull_parity = aph; e.tempty = tempty0 + 8u * as;
                e.abort_flag = abort_flag; e.status = a.status;
                e.ef = a.ef;
                e.t_lo = a.t_lo; e.t_hi = a.t_hi; e.dp_xor = a.dp_xor;
                if (!fast_epilogue_tile<RES, CLAMP, DP, true, W4>(&tmO, &tmR, e, quad, part, lane, est)) { ok = false; break; }
                continue;
            } else {
                if (!mbar_wait_warp(tfull0 + 8u * as, aph, abort_flag, a.status, 4, lane)) { ok = false; break; }
                tc_fence_after();
                for (int cc = 0; cc < cols_per_warp && part < 2; cc += 32) {
                    const int c0 = cbase + cc;
                    unsigned v[32];
                    const unsigned taddr = tmem_base + ((unsigned)(quad * 32) << 16) + as * (unsigned)a.BN + (unsigned)c0;
                    const int nbase = n0 + c0;
                    tc_ld32(taddr, v);
                    tc_wait_ld_into(v);
                    if (!m_ok || nbase >= a.N) continue;
                    int y[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int n = nbase + j;
                        if (n < a.N) {
                            // W4: the accumulator holds 16 x the sum (a multiple of 16: the shift is exact)
                            const long long x = (long long)(W4 ? ((int)v[j] >> 4) : (int)v[j]) + (a.q.bias ? (long long)a.q.bias[n] : 0ll);
                            int t = requant64(x, n, a.q);
                            if (a.r.ptr) {
                                const long long u = (long long)t
                                    + (long long)load_i8(a.r.ptr, (size_t)m * a.N + n, a.r.is_unsigned != 0);
                                t = requant64(u, n, a.r.q2);
                            }
                            y[j] = t;
                        } else {
                            y[j] = 0;
                        }
                    }
                    if (a.out_dtype == DT_I8) {
                        uint8_t* op = (uint8_t*)a.out + (size_t)m * a.N + nbase;
                        if ((a.N % 16 == 0) && nbase + 32 <= a.N) {
                            unsigned wds[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                wds[i] = ((unsigned)y[4 * i] & 0xffu) | (((unsigned)y[4 * i + 1] & 0xffu) << 8)
                                       | (((unsigned)y[4 * i + 2] & 0xffu) << 16) | (((unsigned)y[4 * i + 3] & 0xffu) << 24);
                            ((uint4*)op)[0] = make_uint4(wds[0], wds[1], wds[2], wds[3]);
                            ((uint4*)op)[1] = make_uint4(wds[4], wds[5], wds[6], wds[7]);
                        } else {
                            for (int j = 0; j < 32 && nbase + j < a.N; ++j) op[j] = (uint8_t)y[j];
                        }
                    } else {
                        int32_t* op = (int32_t*)a.out + (size_t)m * a.N + nbase;
                        for (int j = 0; j < 32 && nbase + j < a.N; ++j) op[j] = y[j];
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8u * as);
        }
        // no bulk store may still be reading this CTA's shared memory when it exits
        if (FAST && lane == 0) bulk_wait_all();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(a.tmem_cols) : "memory");
    }
}

// ----------------------------------------------------------------------------- 256-row tiles
// Large-K layers with 256 output channels per tile are bound by L2-to-shared bandwidth at 128 x 256 tiles
// (48 KB per K slab for 512 cycles of MMA).  This variant gives a CTA two 128-row tiles that share every
// weight slab: 64 KB per slab for 1024 cycles of MMA.  Both TMEM accumulators belong to the pair, so the
// epilogue of a pair does not overlap the MMAs of the next one - affordable when K is large.  No residual, the
// 32-bit epilogue only; the staging regions are 1 KB (32 rows x 32 columns, two passes per warp) to make
// room for three 64 KB stages.
static constexpr int PAIR_STAGES = 3;
static constexpr int PAIR_REGION = 1024;

template <bool CLAMP>
__global__ void __launch_bounds__(NUM_THREADS, 1)
igemm_pair_i8_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                             const __grid_constant__ CUtensorMap tmO32, const IgemmArgs a)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int A_BYTES = BM * 128, B_BYTES = 256 * 128, STAGE_BYTES = 2 * A_BYTES + B_BYTES;
    unsigned char* tiles = smem;
    unsigned char* stage_out = tiles + (size_t)PAIR_STAGES * STAGE_BYTES;
    unsigned long long* bars = (unsigned long long*)(stage_out + NUM_EPI_WARPS * PAIR_REGION);
    // bars: full[3], empty[3], tmem_full[2], tmem_empty[2], params_ready
    const unsigned full0 = smem_u32(bars);
    const unsigned empty0 = full0 + 8u * PAIR_STAGES;
    const unsigned tfull0 = empty0 + 8u * PAIR_STAGES;
    const unsigned tempty0 = tfull0 + 16u;
    const unsigned pready = tempty0 + 16u;
    unsigned* tmem_slot = (unsigned*)(bars + 2 * PAIR_STAGES + 6);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    int* par = (int*)(((uintptr_t)(tmem_slot + 4) + 15) & ~(uintptr_t)15);   // [FAST_NP][256]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) {
            mbar_init(full0 + 8u * s, 1);
            mbar_init(empty0 + 8u * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(tfull0 + 8u * s, 1);
            mbar_init(tempty0 + 8u * s, NUM_EPI_WARPS);
        }
        mbar_init(pready, NUM_EPI_WARPS);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    const int num_pairs = (a.num_m_tiles + 1) / 2;
    const int num_pt = num_pairs * a.num_n_tiles;          // pair tiles, column block fastest
    const int kchunks = a.Cin / 128;
    const int num_kb = a.taps * kchunks;
    const int m_end = a.m_base + a.M;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            pdl_wait();
            int s = 0;
            unsigned ph = 0;
            bool ok = true;
            int m_pair = (int)blockIdx.x / a.num_n_tiles, n_tile = (int)blockIdx.x % a.num_n_tiles;
            for (int pt = blockIdx.x; pt < num_pt && ok; pt += gridDim.x) {
                const int n0 = n_tile * 256;
                int m0[2], iw0[2] = {0, 0}, ih0[2] = {0, 0}, in0[2] = {0, 0};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    m0[h] = a.m_base + (2 * m_pair + h) * BM;
                    if (a.a_im2col) {
                        const int ox = m0[h] % a.oW;
                        const int t = m0[h] / a.oW;
                        const int oy = t % a.oH;
                        in0[h] = t / a.oH;
                        iw0[h] = ox * a.sX - a.pL;
                        ih0[h] = oy * a.sY - a.pT;
                    }
                }
                m_pair += a.step_m;
                n_tile += a.step_n;
                if (n_tile >= a.num_n_tiles) { n_tile -= a.num_n_tiles; ++m_pair; }
                int kx = 0, ky = 0, kc = 0, kcoord = 0;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(empty0 + 8u * s, ph ^ 1u, abort_flag, a.status, 1)) { ok = false; break; }
                    const unsigned bar = full0 + 8u * s;
                    const unsigned dst = smem_u32(tiles) + (unsigned)(s * STAGE_BYTES);
                    mbar_expect_tx(bar, (unsigned)STAGE_BYTES);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (a.a_im2col)
                            tma_load_im2col_4d(dst + h * A_BYTES, &tmA, bar, kc * 128, iw0[h], ih0[h], in0[h],
                                               (unsigned short)(kx * a.dX), (unsigned short)(ky * a.dY));
                        else
                            tma_load_2d(dst + h * A_BYTES, &tmA, bar, kcoord, m0[h]);
                    }
                    tma_load_2d(dst + 2 * A_BYTES, &tmB, bar, kcoord, n0);
                    if (++s == PAIR_STAGES) { s = 0; ph ^= 1u; }
                    if (++kc == kchunks) {
                        kc = 0;
                        kcoord += a.Cin - (kchunks - 1) * 128;
                        if (++kx == a.kW) { kx = 0; ++ky; }
                    } else {
                        kcoord += 128;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const unsigned desc_hi = (unsigned)(make_smem_desc(0u, 128) >> 32);
            const unsigned t_lo0 = (smem_u32(tiles) & 0x3ffffu) >> 4;
            const unsigned stage16 = (unsigned)(STAGE_BYTES >> 4), a16 = (unsigned)(A_BYTES >> 4);
            int s = 0;
            unsigned ph = 0, pit = 0, a_lo = t_lo0;
            bool ok = true;
            for (int pt = blockIdx.x; pt < num_pt && ok; pt += gridDim.x, ++pit) {
                const unsigned aph = pit & 1u;
                if (!mbar_wait(tempty0, aph ^ 1u, abort_flag, a.status, 2)) { ok = false; break; }
                if (!mbar_wait(tempty0 + 8u, aph ^ 1u, abort_flag, a.status, 2)) { ok = false; break; }
                tc_fence_after();
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(full0 + 8u * s, ph, abort_flag, a.status, 3)) { ok = false; break; }
                    tc_fence_after();
                    const unsigned b_lo = a_lo + 2u * a16;
                    const unsigned acc = kb ? 1u : 0u;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const unsigned d_tmem = tmem_base + (unsigned)(h * 256);
                        const unsigned al = a_lo + (unsigned)h * a16;
                        tc_mma_i8_lohi(d_tmem, al, b_lo, desc_hi, a.idesc, acc);
                        tc_mma_i8_lohi(d_tmem, al + 2u, b_lo + 2u, desc_hi, a.idesc, 1u);
                        tc_mma_i8_lohi(d_tmem, al + 4u, b_lo + 4u, desc_hi, a.idesc, 1u);
                        tc_mma_i8_lohi(d_tmem, al + 6u, b_lo + 6u, desc_hi, a.idesc, 1u);
                    }
                    tc_commit(empty0 + 8u * s);
                    a_lo += stage16;
                    if (++s == PAIR_STAGES) { s = 0; ph ^= 1u; a_lo = t_lo0; }
                }
                if (ok) {
                    tc_commit(tfull0);
                    tc_commit(tfull0 + 8u);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        pdl_wait();
        const int ew = warp - EPI_WARP0;
        const int quad = warp & 3;
        const int part = ew >> 2;                        // a quarter of the 256 columns
        const int cbase = part * 64;
        const unsigned par_off = (unsigned)((unsigned char*)par - smem_raw);
        const unsigned region_off = (unsigned)(stage_out - smem_raw) + (unsigned)(ew * PAIR_REGION);
        const unsigned region = smem_u32(stage_out + (size_t)ew * PAIR_REGION);
        unsigned rb[4];
        perm_rowbase(rb, 32, lane, 4);
        // the launch keeps every CTA on one column block: its constants are staged once
        const int n0 = ((int)blockIdx.x % a.num_n_tiles) * 256;
        for (int i = ew * 32 + lane; i < FAST_NP * 256; i += 32 * NUM_EPI_WARPS) {
            const int prm = i >> 8, c = i & 255;
            par[i] = (n0 + c < a.cpad) ? __ldg(a.fq + (size_t)prm * a.cpad + n0 + c) : 0;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(pready);
        bool ok = mbar_wait_warp(pready, 0, abort_flag, a.status, 5, lane);
        unsigned pit = 0;
        int m_pair = (int)blockIdx.x / a.num_n_tiles;
        const int gx = n0 + cbase;
        for (int pt = blockIdx.x; pt < num_pt && ok; pt += gridDim.x, ++pit) {
            const int pair_now = m_pair;
            {
                // same stepping as the producer; the column block stays
                const int n_tile = (int)blockIdx.x % a.num_n_tiles;
                m_pair += a.step_m + ((n_tile + a.step_n >= a.num_n_tiles) ? 1 : 0);
            }
#pragma unroll 1
            for (int h = 0; h < 2 && ok; ++h) {
                const int gy = a.m_base + (2 * pair_now + h) * BM + quad * 32;
                const bool active = gx < a.N && gy < m_end;
                if (!mbar_wait_warp(tfull0 + 8u * h, pit & 1u, abort_flag, a.status, 4, lane)) { ok = false; break; }
                tc_fence_after();
                const unsigned tbase = tmem_base + ((unsigned)(quad * 32) << 16) + (unsigned)(h * 256 + cbase);
#pragma unroll 1
                for (int pass = 0; pass < 2; ++pass) {
                    if (lane == 0) bulk_wait_read_all();   // the previous store has finished reading the region
                    __syncwarp();
                    if (active) {
                        unsigned va[16], vb[16];
                        tc_ld_2x16x256b_x4_wait(tbase + (unsigned)(32 * pass), va, vb);
                        if (a.out_unsigned)
                            perm_block<4, false, CLAMP, false, EF_OUT_UNSIGNED | EF_PERM>(va, vb, par_off, cbase + 32 * pass, region_off, rb,
                                                                                          0, lane, 0, 0, 0u);
                        else
                            perm_block<4, false, CLAMP, false, EF_PERM>(va, vb, par_off, cbase + 32 * pass, region_off, rb, 0, lane,
                                                                        0, 0, 0u);
                    }
                    if (pass == 1) {
                        // the accumulator is drained: hand it back before the store goes out
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tempty0 + 8u * h);
                    }
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0 && active) {
                        tma_store_2d(&tmO32, region, gx + 32 * pass, gy);
                        bulk_commit();
                    }
                }
            }
        }
        if (lane == 0) bulk_wait_all();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ----------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const int*, const int*, cuuint32_t, cuuint32_t,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn g_encode_tiled = nullptr;
static EncodeIm2colFn g_encode_im2col = nullptr;

static int load_driver_entry_points(const char** why)
{
    if (g_encode_tiled && g_encode_im2col) return 0;
    cudaDriverEntryPointQueryResult qr;
    void* fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) != cudaSuccess || !fn) {
        *why = "cuTensorMapEncodeTiled is not available from the CUDA driver";
        return -1;
    }
    g_encode_tiled = (EncodeTiledFn)fn;
    fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &qr) != cudaSuccess || !fn) {
        *why = "cuTensorMapEncodeIm2col is not available from the CUDA driver";
        return -1;
    }
    g_encode_im2col = (EncodeIm2colFn)fn;
    return 0;
}

static CUtensorMapSwizzle swizzle_for(int bk)
{
    return bk == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
         : (bk == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : (bk == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE));
}

// resident_b = bytes of the weight block kept in shared memory for the whole launch (0: weights ride the ring)
// regions = staging regions per epilogue warp (1; 2 or 4 with a fused residual)
// w4: a stage also holds the packed form of its weight block, and one more barrier
static size_t igemm_smem_bytes(int stages, int BK, int BN, int regions, size_t resident_b, int w4 = 0)
{
    return 1024 /*alignment slack*/ + resident_b + (size_t)stages * ((BM + (resident_b ? 0 : BN)) * BK + (w4 ? BN * BK / 2 : 0))
         + NUM_EPI_WARPS * REGION_BYTES * regions
         + (2 * stages + 8 + 4 * NUM_EPI_WARPS + (w4 ? stages : 0)) * 8 + 32 + 2 * 2 * FAST_NP * 256 * 4 + 64;
}

// Channels per block-diagonal group of a depthwise layer this kernel takes (0: not such a layer): groups of 64
// channels = one 64-column tile each, or a single group of 32
int igemm_dw_group(const ConvGeom& g)
{
    if (g.groups <= 1 || g.groups != g.C || g.O != g.C || g.Cg != 1 || g.Og != 1) return 0;
    if (g.C % 64 == 0) return 64;
    if (g.C == 32) return 32;
    return 0;
}

size_t igemm_dw_weight_bytes(const ConvGeom& g) { return (size_t)g.C * g.kH * g.kW * igemm_dw_group(g); }

// Depthwise weights [C][taps] as the block-diagonal matrix [C][taps][group channels] (real channel order)
void igemm_dw_arrange_weights(const ConvGeom& g, const int8_t* w_ct, int8_t* dst)
{
    const int cg = igemm_dw_group(g), taps = g.kH * g.kW;
    const size_t row_bytes = (size_t)taps * cg;
    memset(dst, 0, (size_t)g.C * row_bytes);
    for (int o = 0; o < g.C; ++o)
        for (int t = 0; t < taps; ++t) dst[(size_t)o * row_bytes + (size_t)t * cg + (o % cg)] = w_ct[(size_t)o * taps + t];
}

int igemm_make_plan(IgemmPlan* plan, const void* in, const int8_t* w, const void* out, const void* res,
                    const ConvGeom& g0, int in_unsigned, int force_im2col, int force_bn, int num_sms, const char** why,
                    int force_pair, int w4)
{
    static const char* kWhy = "";
    *why = kWhy;
    if (load_driver_entry_points(why)) return -1;
    // A depthwise layer runs as block-diagonal groups: per 64-column tile a dense layer over the tile's own 64 input
    // channels (weights [C][taps * 64], zeros off the diagonal); the activation loads take the group's channel slice.
    ConvGeom g = g0;
    const int Ct = g0.C;          // channels per pixel of the input tensor
    int grouped = 0;
    if (const int cg = igemm_dw_group(g0)) {
        if (w4 || res) { *why = "block-diagonal groups take neither packed weights nor a residual"; return -1; }
        g.C = cg; g.groups = 1; g.Cg = cg; g.Og = g0.O;
        grouped = Ct > cg ? 1 : 0;
        force_im2col = 1;
        force_bn = 64;
        force_pair = 0;
    }
    if (g.groups != 1) { *why = "grouped convolution is not a dense contraction"; return -1; }
    if (g.C % 16 != 0) { *why = "input channels must be a multiple of 16 for the TMA path"; return -1; }
    if (((uintptr_t)in & 15) || ((uintptr_t)w & 15)) { *why = "operands must be 16-byte aligned"; return -1; }
    memset(plan, 0, sizeof(*plan));
    const bool plain = (g.kH == 1 && g.kW == 1 && g.sY == 1 && g.sX == 1 && g.pT == 0 && g.pL == 0
                        && g.oH == g.H && g.oW == g.W);
    plan->a_im2col = (plain && !force_im2col) ? 0 : 1;
    plan->M = g.B * g.oH * g.oW;
    plan->N = g.O;
    plan->Cin = g.C;
    plan->taps = g.kH * g.kW;
    // widest K slab (= swizzle span) that divides the channel count; a channel count that is only a
    // multiple of 16 uses 32-byte slabs whose tail the TMA unit zero-fills
    plan->BK = (g.C % 128 == 0) ? 128 : (g.C % 64 == 0 ? 64 : 32);
    int bn = force_bn;
    if (bn == 0) {
        bn = (g.O >= 256) ? 256 : (g.O > 64 ? 128 : 64);
        // a layer with few output pixels (the classifier, late stages at small batch) would leave most
        // SMs without a tile: narrower column blocks give more tiles
        const long long m_tiles = ((long long)g.B * g.oH * g.oW + BM - 1) / BM;
        while (!force_pair && bn > 64 && m_tiles * ((g.O + bn - 1) / bn) < num_sms) bn >>= 1;
    }
    plan->BN = bn;
    plan->grouped = grouped;
    plan->w4 = w4 ? 1 : 0;
    plan->a_unsigned = in_unsigned;
    plan->oW = g.oW; plan->oH = g.oH; plan->kW = g.kW;
    plan->sX = g.sX; plan->sY = g.sY; plan->pL = g.pL; plan->pT = g.pT; plan->dX = g.dX; plan->dY = g.dY;
    // pipeline depth: fill up to ~200 KB of shared memory, at most 8 stages
    const int with_res = res ? 1 : 0;
    const int num_m_tiles = (plan->M + BM - 1) / BM;
    const int num_n_tiles = (plan->N + plan->BN - 1) / plan->BN;
    const long long tiles = (long long)num_m_tiles * num_n_tiles;
    plan->grid = (int)(tiles < num_sms ? tiles : num_sms);
    if (plan->grid < 1) plan->grid = 1;
    // A CTA whose column block never changes keeps that block's weights in shared memory: the loads of
    // a small-K layer are then activations only.
    const size_t wblock = (size_t)plan->taps * ((g.C + plan->BK - 1) / plan->BK) * plan->BK * plan->BN;
    plan->b_resident = (!w4 && wblock <= 96 * 1024 && (num_n_tiles == 1 || num_sms > num_n_tiles)) ? 1 : 0;
    const int num_kb = plan->taps * ((g.C + plan->BK - 1) / plan->BK);
    auto depth = [&](int regions, size_t resident) {
        int st = 8;
        while (st > 2 && igemm_smem_bytes(st, plan->BK, plan->BN, regions, resident, w4) > 226 * 1024) --st;
        return st;
    };
    auto fits = [&](int st, int regions, size_t resident) {
        return igemm_smem_bytes(st, plan->BK, plan->BN, regions, resident, w4) <= 226 * 1024;
    };
    // A residual cell stages the residual of up to three tiles ahead when that leaves the ring deep enough
    // (four regions per epilogue warp instead of two): its loads then have two tile times to arrive.
    int regions = with_res ? 4 : 1;
    size_t resident = plan->b_resident ? wblock : 0;
    int stages = depth(regions, resident);
    const int want = num_kb + 1 < 4 ? num_kb + 1 : 4;
    if (with_res && (!fits(stages, regions, resident) || stages < want)) {
        regions = 2;
        stages = depth(regions, resident);
    }
    if (plan->b_resident && !fits(stages, regions, resident)) {
        plan->b_resident = 0;
        resident = 0;
        stages = depth(regions, 0);
    }
    plan->stages = stages;
    plan->res_slots = with_res ? regions : 0;
    plan->smem_bytes = igemm_smem_bytes(stages, plan->BK, plan->BN, regions, resident, w4);
    if (!fits(stages, regions, resident)) { *why = "the tile ring does not fit shared memory"; return -1; }

    const CUtensorMapSwizzle swz = swizzle_for(plan->BK);
    CUresult rc;
    // B: weights [N][Ktot], K fastest; packed 4-bit weights: [N][Ktot / 2] bytes, loaded unswizzled (the expansion
    // warps write the swizzled tile)
    {
        const cuuint64_t kbytes = (cuuint64_t)plan->taps * g.C / (w4 ? 2 : 1);
        const cuuint64_t dims[2] = {kbytes, (cuuint64_t)g.O};
        const cuuint64_t strides[1] = {kbytes};
        const cuuint32_t box[2] = {(cuuint32_t)(plan->BK / (w4 ? 2 : 1)), (cuuint32_t)plan->BN};
        const cuuint32_t estr[2] = {1, 1};
        rc = g_encode_tiled(&plan->tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)w, dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, w4 ? CU_TENSOR_MAP_SWIZZLE_NONE : swz,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rc != CUDA_SUCCESS) { *why = "cuTensorMapEncodeTiled failed for the weight matrix"; return -1; }
    }
    if (!plan->a_im2col) {
        const cuuint64_t dims[2] = {(cuuint64_t)g.C, (cuuint64_t)plan->M};
        const cuuint64_t strides[1] = {(cuuint64_t)g.C};
        const cuuint32_t box[2] = {(cuuint32_t)plan->BK, (cuuint32_t)BM};
        const cuuint32_t estr[2] = {1, 1};
        rc = g_encode_tiled(&plan->tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)in, dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rc != CUDA_SUCCESS) { *why = "cuTensorMapEncodeTiled failed for the activation matrix"; return -1; }
    } else {
        // NHWC activations as a (C, W, H, N) tensor; the base pixel of output (ox, oy) is
        // (ox*sX - pL, oy*sY - pT) and the filter tap is passed as an offset per load.
        const cuuint64_t dims[4] = {(cuuint64_t)Ct, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.B};
        const cuuint64_t strides[3] = {(cuuint64_t)Ct, (cuuint64_t)Ct * g.W, (cuuint64_t)Ct * g.W * g.H};
        const int lower[2] = {-g.pL, -g.pT};
        // last base pixel = (oW-1)*sX - pL  ->  upper corner relative to the tensor edge
        const int upper[2] = {(g.oW - 1) * g.sX - g.pL - (g.W - 1), (g.oH - 1) * g.sY - g.pT - (g.H - 1)};
        const cuuint32_t estr[4] = {1, (cuuint32_t)g.sX, (cuuint32_t)g.sY, 1};
        rc = g_encode_im2col(&plan->tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)in, dims, strides, lower, upper,
                             (cuuint32_t)plan->BK, (cuuint32_t)BM, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rc != CUDA_SUCCESS) { *why = "cuTensorMapEncodeIm2col failed for the activation tensor"; return -1; }
        // Drivers up to CUDA 13.1 encode im2col maps of tensors smaller than 128 KiB with a flag
        // (bit 21 of the second 64-bit word) that makes the load misbehave; clearing it is the
        // documented remedy used by NVIDIA's own open-source templates.
        int drv = 0;
        if (cudaDriverGetVersion(&drv) == cudaSuccess && drv <= 13010) {
            const size_t bytes = (size_t)Ct * g.W * g.H * g.B;
            if (bytes < 131072) reinterpret_cast<unsigned long long*>(&plan->tmA)[1] &= ~(1ull << 21);
        }
    }
    // output (and residual) as [M][N] bytes, one box = an epilogue warp's 32 rows x BN/4 columns
    plan->has_out_maps = 0;
    if (out && g.O % 16 == 0 && !((uintptr_t)out & 15) && !((uintptr_t)res & 15)) {
        const int wb = plan->BN / 4;   // an epilogue warp's columns: 64, 32 or 16
        const cuuint64_t dims[2] = {(cuuint64_t)g.O, (cuuint64_t)plan->M};
        const cuuint64_t strides[1] = {(cuuint64_t)g.O};
        const cuuint32_t box[2] = {(cuuint32_t)wb, 32};
        const cuuint32_t estr[2] = {1, 1};
        rc = g_encode_tiled(&plan->tmO, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)out, dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(wb), CU_TENSOR_MAP_L2_PROMOTION_NONE,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rc != CUDA_SUCCESS) { *why = "cuTensorMapEncodeTiled failed for the output matrix"; return -1; }
        plan->tmR = plan->tmO;
        if (res) {
            rc = g_encode_tiled(&plan->tmR, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)res, dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(wb), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (rc != CUDA_SUCCESS) { *why = "cuTensorMapEncodeTiled failed for the residual matrix"; return -1; }
        }
        plan->has_out_maps = 1;
        // 256-row variant: 256-column tiles, 128-byte K slabs, no residual, weights not resident, and enough
        // work per CTA that halving the weight traffic pays for the un-overlapped epilogue
        const int num_kb = plan->taps * (g.C / 128);
        if (plan->BN == 256 && plan->BK == 128 && !res && !plan->b_resident && !w4 && g.O % 32 == 0
            && (force_pair || (num_kb >= 8 && (long long)num_m_tiles * num_n_tiles >= 4ll * num_sms))) {
            const cuuint32_t box32[2] = {32, 32};
            rc = g_encode_tiled(&plan->tmO32, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)out, dims, strides, box32, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (rc == CUDA_SUCCESS) {
                plan->pair = 1;
                plan->pair_smem_bytes = 1024 + (size_t)PAIR_STAGES * (2 * BM * 128 + 256 * 128) + NUM_EPI_WARPS * PAIR_REGION
                                      + (2 * PAIR_STAGES + 6) * 8 + 32 + FAST_NP * 256 * 4 + 64;
            }
        }
    }
    return 0;
}

bool igemm_uses_fast_epilogue(const IgemmPlan& plan, const FastQuant& fast, bool has_residual, int out_dtype)
{
    return fast.enabled && out_dtype == DT_I8 && (plan.N % 32 == 0) && (!has_residual || fast.fq2) && plan.has_out_maps;
}

int igemm_perm_block(const IgemmPlan& plan) { return (plan.BN >> 2) >= 32 ? 32 : 16; }

void igemm_permute_weights(const int8_t* w, int8_t* dst, int N, size_t row_bytes, int perm_block)
{
    const int ng = perm_block / 8;
    for (int n = 0; n < N; ++n) memcpy(dst + (size_t)n * row_bytes, w + (size_t)perm_real_channel(n, ng) * row_bytes, row_bytes);
}

cudaError_t launch_igemm(const IgemmPlan& plan, const QuantDev& q, const Residual& r, const FastQuant& fast, void* out,
                         int out_dtype, int m_base, int* status_word, cudaStream_t s)
{
    if (plan.M == 0 || plan.N == 0) return cudaSuccess;
    IgemmArgs a;
    memset(&a, 0, sizeof(a));
    a.m_base = m_base;
    a.M = plan.M; a.N = plan.N; a.Cin = plan.Cin; a.taps = plan.taps; a.BK = plan.BK; a.BN = plan.BN;
    a.b_resident = plan.b_resident;
    a.stages = plan.stages; a.a_im2col = plan.a_im2col;
    a.grouped = plan.grouped;
    a.res_slots = plan.res_slots ? plan.res_slots : 2;
    a.oW = plan.oW; a.oH = plan.oH; a.kW = plan.kW; a.sX = plan.sX; a.sY = plan.sY;
    a.pL = plan.pL; a.pT = plan.pT; a.dX = plan.dX; a.dY = plan.dY;
    a.num_m_tiles = (plan.M + BM - 1) / BM;
    a.num_n_tiles = (plan.N + plan.BN - 1) / plan.BN;
    // instruction descriptor: D = s32, A = u8/s8, B = s8, both K-major, N and M extents
    a.idesc = (2u << 4) | ((plan.a_unsigned ? 0u : 1u) << 7) | (1u << 10) | ((unsigned)(plan.BN >> 3) << 17)
            | ((unsigned)(BM >> 4) << 24);
    unsigned cols = 2u * plan.BN;
    unsigned p2 = 32;
    while (p2 < cols) p2 <<= 1;
    a.tmem_cols = p2;
    a.out_dtype = out_dtype;
    a.out = out;
    a.status = status_word;
    a.q = q;
    a.r = r;
    a.fq = fast.fq; a.fq2 = fast.fq2; a.cpad = fast.cpad; a.t_lo = fast.t_lo; a.t_hi = fast.t_hi;
    a.out_unsigned = fast.out_unsigned;
    a.dp_xor = fast.dp_xor;
    a.dp_a_signed = fast.dp_a_signed;
    const bool t_unsigned = fast.dp4a ? fast.dp_t_unsigned : (fast.t_lo == 0);
    a.ef = (fast.out_unsigned ? EF_OUT_UNSIGNED : 0) | (r.is_unsigned ? EF_RES_UNSIGNED : 0)
         | (t_unsigned ? EF_T_UNSIGNED : 0) | (fast.dp_a_signed ? EF_DP_A_SIGNED : 0) | (fast.wide ? EF_WIDE : 0);
    const bool use_fast = igemm_uses_fast_epilogue(plan, fast, r.ptr != nullptr, out_dtype);
    // the weights of a cell on the 32-bit epilogue are stored permuted (and only those)
    if (use_fast != (plan.perm != 0)) return cudaErrorInvalidConfiguration;
    const int mode = !use_fast ? 0 : (r.ptr ? (fast.need_clamp ? 2 : (fast.dp4a ? 5 : 4)) : (fast.need_clamp ? 1 : 3));
    static std::atomic<bool> attr_set[64];   // set twice by racing first calls at worst: harmless
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        const void* variants[12] = {(const void*)igemm_i8_tcgen05_kernel<0, false>, (const void*)igemm_i8_tcgen05_kernel<1, false>,
                                    (const void*)igemm_i8_tcgen05_kernel<2, false>, (const void*)igemm_i8_tcgen05_kernel<3, false>,
                                    (const void*)igemm_i8_tcgen05_kernel<4, false>, (const void*)igemm_i8_tcgen05_kernel<5, false>,
                                    (const void*)igemm_i8_tcgen05_kernel<0, true>, (const void*)igemm_i8_tcgen05_kernel<1, true>,
                                    (const void*)igemm_i8_tcgen05_kernel<2, true>, (const void*)igemm_i8_tcgen05_kernel<3, true>,
                                    (const void*)igemm_i8_tcgen05_kernel<4, true>, (const void*)igemm_i8_tcgen05_kernel<5, true>};
        for (const void* fn : variants) {
            cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e != cudaSuccess) return e;
        }
        attr_set[dev] = true;
    }
    int tiles = a.num_m_tiles * a.num_n_tiles;
    int grid = plan.grid < tiles ? plan.grid : tiles;
    // a grid that is a multiple of the number of column blocks keeps every CTA on one column block,
    // so its per-channel constants are staged once
    if (tiles > grid && a.num_n_tiles > 1 && grid > a.num_n_tiles) grid -= grid % a.num_n_tiles;
    // resident weights rely on exactly that (or on one tile per CTA)
    if (a.b_resident && tiles > grid && a.num_n_tiles > 1 && grid % a.num_n_tiles != 0) return cudaErrorInvalidConfiguration;
    a.step_m = grid / a.num_n_tiles;
    a.step_n = grid % a.num_n_tiles;
    if (plan.pair && use_fast && !r.ptr && !fast.wide) {
        typedef void (*PairKernel)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const IgemmArgs);
        static const PairKernel pair_kernels[2] = {igemm_pair_i8_tcgen05_kernel<false>, igemm_pair_i8_tcgen05_kernel<true>};
        static std::atomic<bool> pair_attr_set[64];
        if (dev >= 0 && dev < 64 && !pair_attr_set[dev]) {
            for (PairKernel k : pair_kernels) {
                cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
                if (e != cudaSuccess) return e;
            }
            pair_attr_set[dev] = true;
        }
        const int pair_tiles = ((a.num_m_tiles + 1) / 2) * a.num_n_tiles;
        int pgrid = plan.grid < pair_tiles ? plan.grid : pair_tiles;
        if (pair_tiles > pgrid && a.num_n_tiles > 1 && pgrid > a.num_n_tiles) pgrid -= pgrid % a.num_n_tiles;
        if (pair_tiles <= pgrid || a.num_n_tiles == 1 || pgrid % a.num_n_tiles == 0) {
            a.step_m = pgrid / a.num_n_tiles;
            a.step_n = pgrid % a.num_n_tiles;
            return launch_pdl(pair_kernels[fast.need_clamp ? 1 : 0], pgrid, NUM_THREADS, plan.pair_smem_bytes, s, plan.tmA,
                              plan.tmB, plan.tmO32, a);
        }
    }
    typedef void (*Kernel)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const IgemmArgs);
    static const Kernel kernels[2][6] = {
        {igemm_i8_tcgen05_kernel<0, false>, igemm_i8_tcgen05_kernel<1, false>, igemm_i8_tcgen05_kernel<2, false>,
         igemm_i8_tcgen05_kernel<3, false>, igemm_i8_tcgen05_kernel<4, false>, igemm_i8_tcgen05_kernel<5, false>},
        {igemm_i8_tcgen05_kernel<0, true>, igemm_i8_tcgen05_kernel<1, true>, igemm_i8_tcgen05_kernel<2, true>,
         igemm_i8_tcgen05_kernel<3, true>, igemm_i8_tcgen05_kernel<4, true>, igemm_i8_tcgen05_kernel<5, true>}};
    return launch_pdl(kernels[plan.w4 ? 1 : 0][mode], grid, NUM_THREADS + (plan.w4 ? 32 * W4_UNPACK_WARPS : 0), plan.smem_bytes, s,
                      plan.tmA, plan.tmB, plan.tmO, plan.tmR, a);
}

}  // namespace n2d2b
