// PTX wrappers shared by the tensor-core kernels: mbarriers with bounded waits, TMA loads, tcgen05
// allocation / MMA / commit / TMEM loads, shared-memory matrix descriptors, and the 32-bit epilogue.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "common.cuh"

namespace n2d2b {

static constexpr unsigned long long WAIT_LIMIT_NS = 1500ull * 1000ull * 1000ull;
static constexpr int FAST_NP = 5;             // words per channel of a fast requantisation: lo, hi, mult, add, shift

// ----------------------------------------------------------------------------- programmatic dependent launch
// A kernel launched with launch_pdl may start while the kernel before it on the stream still runs: its CTAs
// take the SMs the earlier kernel's CTAs leave, set up barriers, TMEM, constants and weights, and only then
// wait (pdl_wait) for the earlier kernel to complete and its memory to be visible.  Everything that reads
// activations or writes outputs sits behind that wait, directly or through the kernel's own barriers.
// pdl_launch_dependents, at the start of a kernel, lets the next one begin that early.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... P, typename... A>
static inline cudaError_t launch_pdl(void (*kernel)(P...), int grid, int threads, size_t smem, cudaStream_t s, A... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, P(args)...);
}

// ----------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity)
{
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long globaltimer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait. Returns false (and raises the CTA-wide abort flag) on time-out or when another
// role already aborted.
__device__ __forceinline__ bool mbar_wait_for(unsigned bar, unsigned parity, volatile int* abort_flag,
                                              int* status, int code, unsigned long long limit_ns)
{
    if (mbar_try_wait(bar, parity)) return true;
    // try_wait suspends the thread in hardware until the phase completes or a time limit passes, so a
    // waiting warp leaves the issue slots to the warps that work
    const unsigned long long t0 = globaltimer_ns();
    unsigned rounds = 0;
    while (true) {
        // a few polls per look at the abort flag and the clock
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        // A failed try_wait comes back within tens of cycles, so a long wait (an issuer whose accumulators the
        // epilogue still holds, an epilogue warp whose residual is still on its way from DRAM) would fill the issue
        // slots of the warps that work: after a short tight phase the waiter sleeps between polls.
        if (++rounds > 8) __nanosleep(128);
        if (*abort_flag) return false;
        if (globaltimer_ns() - t0 > limit_ns) {
            *abort_flag = 1;
            atomicCAS(status, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag,
                                          int* status, int code)
{
    return mbar_wait_for(bar, parity, abort_flag, status, code, WAIT_LIMIT_NS);
}

// Bounded wait of a whole warp with a warp-uniform result (votes), for loops that every lane runs
__device__ __forceinline__ bool mbar_wait_uniform(unsigned bar, unsigned parity, volatile int* abort_flag, int* status, int code)
{
    if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
    const unsigned long long t0 = globaltimer_ns();
    while (true) {
        if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
        if (__any_sync(0xffffffffu, *abort_flag != 0)) return false;
        if (__any_sync(0xffffffffu, globaltimer_ns() - t0 > WAIT_LIMIT_NS)) {
            *abort_flag = 1;
            atomicCAS(status, 0, code);
            return false;
        }
    }
}

// Warp-wide bounded wait: one lane polls (32 lanes polling one word, times many warps, crowd out the
// arrivals and the shared-memory traffic of the working warps), then every lane observes the completed
// phase itself, which costs one successful try_wait and gives each lane its own acquire.
__device__ __forceinline__ bool mbar_wait_warp(unsigned bar, unsigned parity, volatile int* abort_flag,
                                               int* status, int code, int lane)
{
    // the common case, a phase that completed long ago, costs one poll of the whole warp
    if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
    unsigned ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity, abort_flag, status, code) ? 1u : 0u;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ok) return false;
    return mbar_wait(bar, parity, abort_flag, status, code);
}

__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* tm, unsigned bar, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_3d(unsigned dst, const CUtensorMap* tm, unsigned bar, int c0, int c1, int c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_load_4d(unsigned dst, const CUtensorMap* tm, unsigned bar, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_im2col_4d(unsigned dst, const CUtensorMap* tm, unsigned bar, int c,
                                                   int w, int h, int n, unsigned short off_w,
                                                   unsigned short off_h)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
        ::"r"(dst), "l"(tm), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_mma_i8(unsigned d_tmem, unsigned long long adesc, unsigned long long bdesc,
                                          unsigned idesc, unsigned accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Descriptors as halves: both operands of a K-major int8 MMA share the upper word (stride between 8-row
// groups, version, swizzle mode), and the lower word is the 16-byte-granular shared-memory address, so a
// loop over filter taps or K steps advances a 32-bit integer.  The issuing thread pays the latency of every
// instruction it executes, which makes this arithmetic the cost of a short MMA, not the MMA.
__device__ __forceinline__ void tc_mma_i8_lohi(unsigned d_tmem, unsigned a_lo, unsigned b_lo, unsigned desc_hi, unsigned idesc,
                                               unsigned accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate) : "memory");
}
// Forms for an issuing WARP: every lane runs the loop (uniform control flow lets the compiler keep descriptor
// words, counters and barrier addresses in uniform registers, where the MMA wants them; a loop under
// `if (lane == 0)` computes them in vector registers and pays a move per operand per MMA), and `issue`
// (true on one lane) predicates the instruction itself.
__device__ __forceinline__ void tc_mma_i8_lohi_p(unsigned d_tmem, unsigned a_lo, unsigned b_lo, unsigned desc_hi, unsigned idesc,
                                                 unsigned accumulate, unsigned issue)
{
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "setp.ne.b32 q, %6, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate), "r"(issue) : "memory");
}
__device__ __forceinline__ void tc_commit_p(unsigned bar, unsigned issue)
{
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(bar), "r"(issue) : "memory");
}
__device__ __forceinline__ void tc_commit(unsigned bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld32(unsigned taddr, unsigned* v)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// tcgen05.ld fills its destination registers asynchronously; the compiler only sees them as outputs of
// the load statement and is free to schedule their consumers ahead of the wait.  Passing the
// registers through an empty volatile statement placed after the wait ties every later use to it.
__device__ __forceinline__ void tc_wait_ld_into(unsigned* v)
{
    tc_wait_ld();
    asm volatile("" : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
                      "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
                 :: "memory");
    asm volatile("" : "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]),
                      "+r"(v[23]), "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]),
                      "+r"(v[30]), "+r"(v[31])
                 :: "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are `swz` bytes wide (swz = 32, 64 or
// 128, equal to the TMA swizzle span): 8-row groups are swz*8 bytes apart.
__device__ __forceinline__ unsigned long long make_smem_desc(unsigned smem_addr, int swz)
{
    const unsigned long long layout = (swz == 128) ? 2ull : (swz == 64 ? 4ull : 6ull);
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)(((unsigned)(swz * 8)) >> 4) << 32;  // stride byte offset
    d |= 1ull << 46;                                               // descriptor version (sm_100)
    d |= layout << 61;
    return d;
}

// Byte j of w, zero- or sign-extended, in one permute: a selector nibble with its top bit set
// replicates the sign of the selected byte (the __byte_perm intrinsic only honours 3 bits per nibble,
// hence the PTX form).
__device__ __forceinline__ int byte_extend(unsigned w, int j, bool is_unsigned)
{
    unsigned d;
    const unsigned sel = is_unsigned ? (0x4440u + j) : (0x8880u + 0x1110u * j + j);
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(w), "r"(0u), "r"(sel));
    return (int)d;
}
// ---- TMA store / bulk-group helpers ----
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, unsigned src, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(tm), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until the bulk stores of this thread have finished *reading* shared memory
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// tcgen05.ld 16 lanes x 256 bits, repeated over 4 (x4: 32 columns) or 2 (x2: 16 columns) column groups.
// Thread t receives, for group i: regs 4i+{0,1} = row (lane0 + t/4), columns 8i + 2(t%4) + {0,1};
// regs 4i+{2,3} = the same columns of row (lane0 + t/4 + 8).
// The load and its wait form one statement, so every use of the registers follows the wait.
__device__ __forceinline__ void tc_ld_16x256b_x4_wait(unsigned taddr, unsigned* v)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr) : "memory");
}
// Two 16-lane halves of a warp's 32 TMEM lanes, one wait for both
__device__ __forceinline__ void tc_ld_2x16x256b_x4_wait(unsigned taddr, unsigned* va, unsigned* vb)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%32];\n\t"
        "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
        "{%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%33];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(va[0]), "=r"(va[1]), "=r"(va[2]), "=r"(va[3]), "=r"(va[4]), "=r"(va[5]), "=r"(va[6]), "=r"(va[7]),
          "=r"(va[8]), "=r"(va[9]), "=r"(va[10]), "=r"(va[11]), "=r"(va[12]), "=r"(va[13]), "=r"(va[14]), "=r"(va[15]),
          "=r"(vb[0]), "=r"(vb[1]), "=r"(vb[2]), "=r"(vb[3]), "=r"(vb[4]), "=r"(vb[5]), "=r"(vb[6]), "=r"(vb[7]),
          "=r"(vb[8]), "=r"(vb[9]), "=r"(vb[10]), "=r"(vb[11]), "=r"(vb[12]), "=r"(vb[13]), "=r"(vb[14]), "=r"(vb[15])
        : "r"(taddr), "r"(taddr + (16u << 16)) : "memory");
}
__device__ __forceinline__ void tc_ld_2x16x256b_x2_wait(unsigned taddr, unsigned* va, unsigned* vb)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%16];\n\t"
        "tcgen05.ld.sync.aligned.16x256b.x2.b32 {%8, %9, %10, %11, %12, %13, %14, %15}, [%17];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(va[0]), "=r"(va[1]), "=r"(va[2]), "=r"(va[3]), "=r"(va[4]), "=r"(va[5]), "=r"(va[6]), "=r"(va[7]),
          "=r"(vb[0]), "=r"(vb[1]), "=r"(vb[2]), "=r"(vb[3]), "=r"(vb[4]), "=r"(vb[5]), "=r"(vb[6]), "=r"(vb[7])
        : "r"(taddr), "r"(taddr + (16u << 16)) : "memory");
}
// Byte offset of (row r, byte column c) inside a staging region whose rows are `wb` bytes (32, 64 or
// 128) and which TMA reads / writes with the swizzle of that width: address bits [4,7) are XORed with
// bits [7,10) (masked to the swizzle width).  The region base must be 1024-byte aligned.
__device__ __forceinline__ unsigned swz_off(int r, int c, int wb)
{
    const unsigned a = (unsigned)(r * wb + c);
    return a ^ (((a >> 7) & (unsigned)(wb / 16 - 1)) << 4);
}

__device__ __forceinline__ void sts_u16(unsigned addr, unsigned v)
{
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"((unsigned short)v) : "memory");
}
__device__ __forceinline__ unsigned lds_u16(unsigned addr)
{
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr) : "memory");
    return (unsigned)v;
}

// The kernel's dynamic shared memory, named so that the compiler sees shared-space accesses (32-bit
// addresses, LDS/STS) in the epilogue instead of generic ones with 64-bit address arithmetic.
__device__ __forceinline__ unsigned char* dyn_smem()
{
    extern __shared__ unsigned char smem_raw[];
    return smem_raw;
}

// Compile-time switches of the epilogue arithmetic (a bit mask, so that no per-value branch remains)
static constexpr int EF_OUT_UNSIGNED = 1;   // final range [0,255] instead of [-128,127]
static constexpr int EF_RES_UNSIGNED = 2;   // residual operand is unsigned
static constexpr int EF_T_UNSIGNED = 4;     // DP: the cell's own output saturates to [0,255]
static constexpr int EF_DP_A_SIGNED = 8;    // DP: the packed (t, r) bytes are read as signed
static constexpr int EF_WIDE = 16;          // first rescale in 64 bits: x * mult + (row 0 : row 3 as a 64-bit addend) >> shift
static constexpr int EF_DP_XOR = 32;        // DP: some of the packed (t, r) bytes are flipped between unsigned and signed (dp_xor)
static constexpr int EF_PERM = 64;          // weights stored with permuted output channels (perm_block)
static constexpr int EF_W4 = 128;           // the accumulator holds 16 x the sum (packed 4-bit weights, see expand_int4_x16)

// NG 8-column groups (NG = 4: 32 columns, NG = 2: 16) of a warp's 32 accumulator rows in the fragment layout
// of the 16x256b TMEM load (thread t: rows t/4 + {0, 8, 16, 24}, column pair 8i + 2(t%4) of group i), through the
// 32-bit epilogue, into (and, for the residual, out of) the warp's swizzled staging region.  One load of
// the per-channel constants serves the thread's four rows: shared-memory bandwidth, not arithmetic, is
// what this epilogue runs out of first, and a 64-bit load costs two wavefronts however many lanes share it.  `region_off` / `par_off` = byte offsets of the
// region (1024-byte aligned in shared memory) and of the staged constants from the start of the dynamic
// shared memory; `col0` = first column of the block within the warp's columns (a multiple of 8*NG),
// `pcol0` = the same within the tile.
//
// Addressing: the byte at (row r, column c) of a region with wb-byte rows sits at
// r*wb + (c ^ x(r)), x(r) = the swizzle term of row r (address bits [7,10) folded into bits [4,7)).
// c = col0 | 8i | 2(t%4) has disjoint bit fields, so the address of group i is base(r) ^ 8i.
// DP (with RES, without CLAMP): the second requantisation of a shift scaling, (t + r) * m2 + add2, is one
// four-way byte dot product per value: the saturating pack that clamps t also places the two residual
// bytes beside it, a = [t0, t1, r0, r1], and b = [m2, 0, m2, 0] (resp. [0, m2, 0, m2]) selects one
// column.  When t and r differ in signedness the unsigned pair is flipped to signed by xor 0x80 and the
// host adds 128 * m2 to add2.
// Row terms of the staging addresses of one lane: rb[k] = (tr + 8k) * wb + (tc ^ x(row)), without the region and
// the column block.  They depend on the lane and the row width only, so a kernel computes them once.
__device__ __forceinline__ void frag_rowbase(unsigned* rb, int wb, int lane)
{
    const int tr = lane >> 2, tc = (lane & 3) * 2;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const unsigned ro = (unsigned)((tr + 8 * k) * wb);
        const unsigned xm = ((ro >> 7) & (unsigned)(wb / 16 - 1)) << 4;
        rb[k] = ro + ((unsigned)tc ^ xm);
    }
}

template <int NG, bool RES, bool CLAMP, bool DP, int EF>
__device__ __forceinline__ void frag_block(const unsigned* vA, const unsigned* vB, unsigned par_off, int pcol0, unsigned region_off,
                                           const unsigned* rb, int col0, int lane, int t_lo, int t_hi, unsigned dp_xor)
{
    unsigned char* const sm = dyn_smem();
    constexpr int NK = 4;   // rows tr + 8k: k = 0, 1 from vA (TMEM lanes 0-15), k = 2, 3 from vB (lanes 16-31)
    const int tc = (lane & 3) * 2;
    unsigned base[NK], base16[NK];
#pragma unroll
    for (int k = 0; k < NK; ++k) {
        // col0 (a multiple of 16 below the row width) occupies bits the row offset leaves clear, and the
        // region is 1024-byte aligned: the column block enters the address as an xor
        base[k] = (region_off + rb[k]) ^ (unsigned)col0;
        // group i sits at base ^ 8i: bit 3 of base is clear (tc <= 6, col0 a multiple of 16, the swizzle term
        // touches bits 4-6 only), so odd groups are +8 (an immediate offset) and groups 2-3 one xor away
        base16[k] = base[k] ^ 16u;
    }
    // the residual bytes of the whole block first: loads the compiler can keep in flight together
    unsigned rres[NG][NK];
    if (RES) {
#pragma unroll
        for (int i = 0; i < NG; ++i)
#pragma unroll
            for (int k = 0; k < NK; ++k) rres[i][k] = *(const unsigned short*)(sm + ((i & 2) ? base16[k] : base[k]) + 8 * (i & 1));
    }
    const unsigned pbase = par_off + (unsigned)(pcol0 + tc) * 4u;
#pragma unroll
    for (int i = 0; i < NG; ++i) {
        const unsigned pp = pbase + 32u * i;   // column pair 8i + tc within the tile
        const int2 mu = *(const int2*)(sm + pp + 2 * 1024);
        const int2 ad = *(const int2*)(sm + pp + 3 * 1024);
        const int2 sh = *(const int2*)(sm + pp + 4 * 1024);
        int2 lo = make_int2(0, 0), hi = make_int2(0, 0);
        if (CLAMP) {
            lo = *(const int2*)(sm + pp + 0 * 1024);
            hi = *(const int2*)(sm + pp + 1 * 1024);
        } else if (EF & EF_WIDE) {
            lo = *(const int2*)(sm + pp + 0 * 1024);   // upper words of the 64-bit addends
        }
        int2 mu2 = make_int2(0, 0), ad2 = mu2, sh2 = mu2, lo2 = mu2, hi2 = mu2;
        if (RES) {
            mu2 = *(const int2*)(sm + pp + (FAST_NP + 2) * 1024);
            ad2 = *(const int2*)(sm + pp + (FAST_NP + 3) * 1024);
            sh2 = *(const int2*)(sm + pp + (FAST_NP + 4) * 1024);
            if (CLAMP) {
                lo2 = *(const int2*)(sm + pp + (FAST_NP + 0) * 1024);
                hi2 = *(const int2*)(sm + pp + (FAST_NP + 1) * 1024);
            }
            if (DP) lo2 = *(const int2*)(sm + pp + (FAST_NP + 0) * 1024);
        }
#pragma unroll
        for (int k = 0; k < NK; ++k) {   // rows tr + 8k
            const unsigned* v = (k < 2) ? vA : vB;
            int x0 = (int)v[4 * i + 2 * (k & 1)], x1 = (int)v[4 * i + 2 * (k & 1) + 1];
            if (CLAMP) {
                x0 = min(max(x0, lo.x), hi.x);
                x1 = min(max(x1, lo.y), hi.y);
            }
            int y0, y1;
            if (EF & EF_WIDE) {
                // fixed-point scalings with many fractional bits: the product needs more than 32 bits, the
                // shifted result does not (proved on the host); no clamps in this form, the pack saturates
                const long long p0 = (long long)x0 * mu.x + (long long)(((unsigned long long)(unsigned)lo.x << 32) | (unsigned)ad.x);
                const long long p1 = (long long)x1 * mu.y + (long long)(((unsigned long long)(unsigned)lo.y << 32) | (unsigned)ad.y);
                y0 = (int)(p0 >> sh.x);
                y1 = (int)(p1 >> sh.y);
            } else {
                y0 = (x0 * mu.x + ad.x) >> sh.x;
                y1 = (x1 * mu.y + ad.y) >> sh.y;
            }
            if (RES && DP) {
                const unsigned rw = rres[i][k];   // two residual bytes, replaced below
                unsigned a4;
                if (EF & EF_T_UNSIGNED) asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(a4) : "r"(y1), "r"(y0), "r"(rw));
                else asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(a4) : "r"(y1), "r"(y0), "r"(rw));
                a4 ^= dp_xor;
                // lo2 row holds the column-selecting multiplier words, ad2 the (compensated) addends
                int d0, d1;
                if (EF & EF_DP_A_SIGNED) {
                    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d0) : "r"(a4), "r"(lo2.x), "r"(ad2.x));
                    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d1) : "r"(a4), "r"(lo2.y), "r"(ad2.y));
                } else {
                    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d0) : "r"(a4), "r"(lo2.x), "r"(ad2.x));
                    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d1) : "r"(a4), "r"(lo2.y), "r"(ad2.y));
                }
                y0 = d0 >> sh2.x;
                y1 = d1 >> sh2.y;
            } else if (RES) {
                const unsigned rw = rres[i][k];   // two residual bytes, replaced below
                int r0, r1;
                if (EF & EF_RES_UNSIGNED) {
                    r0 = (int)(rw & 0xffu);
                    r1 = (int)(rw >> 8);
                } else {
                    r0 = byte_extend(rw, 0, false);
                    r1 = byte_extend(rw, 1, false);
                }
                int u0 = min(max(y0, t_lo), t_hi) + r0;
                int u1 = min(max(y1, t_lo), t_hi) + r1;
                if (CLAMP) {
                    u0 = min(max(u0, lo2.x), hi2.x);
                    u1 = min(max(u1, lo2.y), hi2.y);
                }
                y0 = (u0 * mu2.x + ad2.x) >> sh2.x;
                y1 = (u1 * mu2.y + ad2.y) >> sh2.y;
            }
            unsigned d;
            // the third operand fills the upper half of d, which the 16-bit store drops: any live register will do
            // (a literal 0 would cost a register move per pack)
            if (EF & EF_OUT_UNSIGNED) asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(y1), "r"(y0), "r"(y0));
            else asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(y1), "r"(y0), "r"(y0));
            *(unsigned short*)(sm + ((i & 2) ? base16[k] : base[k]) + 8 * (i & 1)) = (unsigned short)d;
        }
    }
}

// ---- the same epilogue on weights whose output channels are permuted inside every block of 8 * NG channels -----------
// The 16x256b TMEM load hands a thread column pairs that are eight columns apart (8i + 2q + e, q = lane % 4).  When the
// weight rows of a block are stored in the order
//     stored row 8i + 2q + e  =  real channel 2 NG q + 2i + e        (i < NG, q < 4, e < 2)
// those columns are the thread's 2 NG CONSECUTIVE real channels: per row it reads its per-channel constants with
// 128-bit loads, the residual with one 64-bit (NG = 4) or 32-bit (NG = 2) load, and writes its bytes with one
// store, instead of one 16-bit access per column pair.  The staging region keeps the real channel order, so the
// TMA store and the residual load are unchanged.
__host__ __device__ inline int perm_real_channel(int stored, int ng)
{
    const int blk = 8 * ng, j = stored % blk;
    const int i = j >> 3, q = (j >> 1) & 3, e = j & 1;
    return stored - j + 2 * ng * q + 2 * i + e;
}

// Row terms of a lane's staging addresses for the permuted layout: the lane's first byte column is 2 NG q.
__device__ __forceinline__ void perm_rowbase(unsigned* rb, int wb, int lane, int ng)
{
    const int tr = lane >> 2, tc = (lane & 3) * 2 * ng;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const unsigned ro = (unsigned)((tr + 8 * k) * wb);
        const unsigned xm = ((ro >> 7) & (unsigned)(wb / 16 - 1)) << 4;
        rb[k] = ro + ((unsigned)tc ^ xm);
    }
}

__device__ __forceinline__ unsigned pack4_sat(int y0, int y1, int y2, int y3, bool out_unsigned)
{
    unsigned p, w;
    if (out_unsigned) {
        asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(p) : "r"(y3), "r"(y2), "r"(y2));
        asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(y1), "r"(y0), "r"(p));
    } else {
        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(p) : "r"(y3), "r"(y2), "r"(y2));
        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(y1), "r"(y0), "r"(p));
    }
    return w;   // bytes y0, y1, y2, y3 from the low end
}

template <int NG, bool RES, bool CLAMP, bool DP, int EF>
__device__ __forceinline__ void perm_block(const unsigned* vA, const unsigned* vB, unsigned par_off, int pcol0, unsigned region_off,
                                           const unsigned* rb, int col0, int lane, int t_lo, int t_hi, unsigned dp_xor)
{
    unsigned char* const sm = dyn_smem();
    constexpr int NK = 4;          // rows tr + 8k: k = 0, 1 from vA (TMEM lanes 0-15), k = 2, 3 from vB (lanes 16-31)
    constexpr int NH = NG / 2;     // the thread's channels in halves of four
    unsigned base[NK];
#pragma unroll
    for (int k = 0; k < NK; ++k) base[k] = (region_off + rb[k]) ^ (unsigned)col0;
    unsigned rres[NK][NH];
    if (RES) {
#pragma unroll
        for (int k = 0; k < NK; ++k) {
            if (NH == 2) {
                const uint2 r = *(const uint2*)(sm + base[k]);
                rres[k][0] = r.x;
                rres[k][NH - 1] = r.y;
            } else {
                rres[k][0] = *(const unsigned*)(sm + base[k]);
            }
        }
    }
    unsigned outw[NK][NH];
    const unsigned pbase = par_off + (unsigned)(pcol0 + 2 * NG * (lane & 3)) * 4u;
#pragma unroll
    for (int h = 0; h < NH; ++h) {
        const unsigned pp = pbase + 16u * h;   // channels 4h .. 4h + 3 of this thread
        const int4 mu = *(const int4*)(sm + pp + 2 * 1024);
        const int4 ad = *(const int4*)(sm + pp + 3 * 1024);
        const int4 sh = *(const int4*)(sm + pp + 4 * 1024);
        int4 lo = make_int4(0, 0, 0, 0), hi = lo;
        if (CLAMP) {
            lo = *(const int4*)(sm + pp + 0 * 1024);
            hi = *(const int4*)(sm + pp + 1 * 1024);
        } else if (EF & EF_WIDE) {
            lo = *(const int4*)(sm + pp + 0 * 1024);   // upper words of the 64-bit addends
        }
        int4 mu2 = make_int4(0, 0, 0, 0), ad2 = mu2, sh2 = mu2, lo2 = mu2, hi2 = mu2;
        if (RES) {
            ad2 = *(const int4*)(sm + pp + (FAST_NP + 3) * 1024);
            sh2 = *(const int4*)(sm + pp + (FAST_NP + 4) * 1024);
            if (!DP) mu2 = *(const int4*)(sm + pp + (FAST_NP + 2) * 1024);
            if (CLAMP) hi2 = *(const int4*)(sm + pp + (FAST_NP + 1) * 1024);
            if (CLAMP || DP) lo2 = *(const int4*)(sm + pp + (FAST_NP + 0) * 1024);   // DP: byte-lane multiplier words
        }
        const int muv[4] = {mu.x, mu.y, mu.z, mu.w}, adv[4] = {ad.x, ad.y, ad.z, ad.w}, shv[4] = {sh.x, sh.y, sh.z, sh.w};
        const int lov[4] = {lo.x, lo.y, lo.z, lo.w}, hiv[4] = {hi.x, hi.y, hi.z, hi.w};
        const int mu2v[4] = {mu2.x, mu2.y, mu2.z, mu2.w}, ad2v[4] = {ad2.x, ad2.y, ad2.z, ad2.w};
        const int sh2v[4] = {sh2.x, sh2.y, sh2.z, sh2.w}, lo2v[4] = {lo2.x, lo2.y, lo2.z, lo2.w}, hi2v[4] = {hi2.x, hi2.y, hi2.z, hi2.w};
#pragma unroll
        for (int k = 0; k < NK; ++k) {
            const unsigned* v = (k < 2) ? vA : vB;
            int y[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                // thread channel 4h + c = 2i + e  ->  group i = 2h + c / 2, element e = c % 2
                int x = (int)v[4 * (2 * h + (c >> 1)) + 2 * (k & 1) + (c & 1)];
                if (EF & EF_W4) x >>= 4;   // a multiple of 16: exact
                if (CLAMP) x = min(max(x, lov[c]), hiv[c]);
                if (EF & EF_WIDE) {
                    const long long p = (long long)x * muv[c] + (long long)(((unsigned long long)(unsigned)lov[c] << 32) | (unsigned)adv[c]);
                    y[c] = (int)(p >> shv[c]);
                } else {
                    y[c] = (x * muv[c] + adv[c]) >> shv[c];
                }
            }
            if (RES && DP) {
                // [t, t', r, r'] per column pair: the saturating pack of the cell's own output also places the two
                // residual bytes beside it; one byte dot product per value then gives (t + r) * m2 + add2
                const unsigned rw = rres[k][h];
                unsigned a01, a23;
                if (EF & EF_T_UNSIGNED) {
                    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(a01) : "r"(y[1]), "r"(y[0]), "r"(rw));
                    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(a23) : "r"(y[3]), "r"(y[2]), "r"(rw >> 16));
                } else {
                    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(a01) : "r"(y[1]), "r"(y[0]), "r"(rw));
                    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(a23) : "r"(y[3]), "r"(y[2]), "r"(rw >> 16));
                }
                if (EF & EF_DP_XOR) {
                    a01 ^= dp_xor;
                    a23 ^= dp_xor;
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const unsigned a4 = (c < 2) ? a01 : a23;
                    int d;
                    if (EF & EF_DP_A_SIGNED) asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a4), "r"(lo2v[c]), "r"(ad2v[c]));
                    else asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a4), "r"(lo2v[c]), "r"(ad2v[c]));
                    y[c] = d >> sh2v[c];
                }
            } else if (RES) {
                const unsigned rw = rres[k][h];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int r = byte_extend(rw, c, (EF & EF_RES_UNSIGNED) != 0);
                    int u = min(max(y[c], t_lo), t_hi) + r;
                    if (CLAMP) u = min(max(u, lo2v[c]), hi2v[c]);
                    y[c] = (u * mu2v[c] + ad2v[c]) >> sh2v[c];
                }
            }
            outw[k][h] = pack4_sat(y[0], y[1], y[2], y[3], (EF & EF_OUT_UNSIGNED) != 0);
        }
    }
#pragma unroll
    for (int k = 0; k < NK; ++k) {
        if (NH == 2) *(uint2*)(sm + base[k]) = make_uint2(outw[k][0], outw[k][NH - 1]);
        else *(unsigned*)(sm + base[k]) = outw[k][0];
    }
}

// The same block (no residual) written straight to global memory: with the permuted layout a thread holds eight
// consecutive channels of a row, four neighbouring lanes a whole 32-byte sector of it, so the bytes need no detour
// through a staging region when the rows' addresses have no regular pattern a TMA store could follow (the band
// kernels, whose rows are pixels of a padded raster).  out + rowoff[k] = address of channel pcol0's byte of row tr + 8k
// in the output, rowok bit k = that row exists.
template <bool CLAMP, int EF>
__device__ __forceinline__ void perm_block_global(const unsigned* vA, const unsigned* vB, unsigned par_off, int pcol0,
                                                  uint8_t* out, const unsigned (&rowoff)[4], unsigned rowok, int lane)
{
    unsigned char* const sm = dyn_smem();
    constexpr int NK = 4, NH = 2;
    unsigned outw[NK][NH];
    const unsigned pbase = par_off + (unsigned)(pcol0 + 8 * (lane & 3)) * 4u;
#pragma unroll
    for (int h = 0; h < NH; ++h) {
        const unsigned pp = pbase + 16u * h;
        const int4 mu = *(const int4*)(sm + pp + 2 * 1024);
        const int4 ad = *(const int4*)(sm + pp + 3 * 1024);
        const int4 sh = *(const int4*)(sm + pp + 4 * 1024);
        int4 lo = make_int4(0, 0, 0, 0), hi = lo;
        if (CLAMP) {
            lo = *(const int4*)(sm + pp + 0 * 1024);
            hi = *(const int4*)(sm + pp + 1 * 1024);
        } else if (EF & EF_WIDE) {
            lo = *(const int4*)(sm + pp + 0 * 1024);
        }
        const int muv[4] = {mu.x, mu.y, mu.z, mu.w}, adv[4] = {ad.x, ad.y, ad.z, ad.w}, shv[4] = {sh.x, sh.y, sh.z, sh.w};
        const int lov[4] = {lo.x, lo.y, lo.z, lo.w}, hiv[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int k = 0; k < NK; ++k) {
            const unsigned* v = (k < 2) ? vA : vB;
            int y[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                int x = (int)v[4 * (2 * h + (c >> 1)) + 2 * (k & 1) + (c & 1)];
                if (CLAMP) x = min(max(x, lov[c]), hiv[c]);
                if (EF & EF_WIDE) {
                    const long long p = (long long)x * muv[c] + (long long)(((unsigned long long)(unsigned)lov[c] << 32) | (unsigned)adv[c]);
                    y[c] = (int)(p >> shv[c]);
                } else {
                    y[c] = (x * muv[c] + adv[c]) >> shv[c];
                }
            }
            outw[k][h] = pack4_sat(y[0], y[1], y[2], y[3], (EF & EF_OUT_UNSIGNED) != 0);
        }
    }
#pragma unroll
    for (int k = 0; k < NK; ++k)
        if (rowok & (1u << k)) *(uint2*)(out + rowoff[k] + 8 * (lane & 3)) = make_uint2(outw[k][0], outw[k][1]);
}

// One accumulator tile through the fragment-layout epilogue: residual slice in by TMA (issued one tile
// ahead when the warp has two staging regions), accumulator slice out of TMEM, requantisation into the
// swizzled staging region, TMA store.  A warp owns the 32 rows of its TMEM quadrant `quad` and the column
// part `cp` (wp columns) of the tile.
struct EpiTile {
    unsigned tmem_acc;      // TMEM address of the accumulator stage (lane 0, first column)
    int BN, N, M, m0, n0;
    int wp;                 // columns per warp: BN / (epilogue warps per TMEM quadrant); 64, 32 or 16
    unsigned par_off;       // staged per-channel constants of this column block (byte offset in dynamic shared memory)
    unsigned region_off;    // this warp's staging region(s) (1024-byte aligned; byte offset in dynamic shared memory)
    unsigned region_stride; // distance between the regions of a residual cell, 0 = one region
    unsigned slot_shift;    // residual cells: log2 of the number of regions (1 or 2)
    unsigned rbar;          // this warp's residual-arrival mbarriers (one per region, 8 bytes apart)
    unsigned tfull, tfull_parity, tempty;
    volatile int* abort_flag;
    int* status;
    int ef;                 // EF_* switches of this cell
    int t_lo, t_hi;
    unsigned dp_xor;
};

// Per-warp state carried from tile to tile.
struct EpiState {
    unsigned t = 0;          // tiles handled so far (selects the staging region and barrier phase of a residual cell)
    unsigned rb[4] = {0, 0, 0, 0};   // frag_rowbase of this lane for the warp's row width (set once by the kernel)
};

// The accumulator slice of one warp: 32 rows, wp columns in blocks of 32 (or one block of 16)
template <bool RES, bool CLAMP, bool DP, int EF>
__device__ __forceinline__ void epi_drain(const EpiTile& e, unsigned tbase, int cbase, unsigned region_off, const unsigned* rb,
                                          int lane)
{
    constexpr bool PERM = (EF & EF_PERM) != 0;
    if (e.wp >= 32) {
#pragma unroll 1
        for (int cb = 0; cb < e.wp; cb += 32) {
            unsigned va[16], vb[16];
            tc_ld_2x16x256b_x4_wait(tbase + (unsigned)cb, va, vb);
            if (PERM)
                perm_block<4, RES, CLAMP, DP, EF>(va, vb, e.par_off, cbase + cb, region_off, rb, cb, lane, e.t_lo, e.t_hi, e.dp_xor);
            else
                frag_block<4, RES, CLAMP, DP, EF>(va, vb, e.par_off, cbase + cb, region_off, rb, cb, lane, e.t_lo, e.t_hi,
                                                  e.dp_xor);
        }
    } else {
        unsigned va[8], vb[8];
        tc_ld_2x16x256b_x2_wait(tbase, va, vb);
        if (PERM) perm_block<2, RES, CLAMP, DP, EF>(va, vb, e.par_off, cbase, region_off, rb, 0, lane, e.t_lo, e.t_hi, e.dp_xor);
        else frag_block<2, RES, CLAMP, DP, EF>(va, vb, e.par_off, cbase, region_off, rb, 0, lane, e.t_lo, e.t_hi, e.dp_xor);
    }
}

// One lane starts the residual load of the warp's slice (32 rows at gy, wp columns at gx) of some tile into
// region `slot`.  A slice outside the tensor arrives on the barrier without a load, so that every tile completes
// one phase per region and the waits need no bookkeeping.
__device__ __forceinline__ void epi_issue_residual(const CUtensorMap* tmR, unsigned region_off0, unsigned region_stride,
                                                   unsigned rbar, unsigned slot, int gx, int gy, int N, int M, int wp)
{
    const unsigned bar = rbar + 8u * slot;
    if (gx < N && gy < M) {
        mbar_expect_tx(bar, (unsigned)(32 * wp));
        tma_load_2d(smem_u32(dyn_smem() + region_off0 + slot * region_stride), tmR, bar, gx, gy);
    } else {
        mbar_arrive(bar);
    }
}

template <bool RES, bool CLAMP, bool DP, bool PERM = false, bool W4 = false>
__device__ __forceinline__ bool fast_epilogue_tile(const CUtensorMap* tmO, const CUtensorMap* tmR, const EpiTile& e, int quad,
                                                   int cp, int lane, EpiState& st)
{
    static_assert(PERM || !W4, "the packed-weight variant uses the permuted epilogue");
    constexpr int P = (PERM ? EF_PERM : 0) | (W4 ? EF_W4 : 0);
    const int wp = e.wp;
    const int cbase = cp * wp;
    const int gx = e.n0 + cbase, gy = e.m0 + quad * 32;
    const bool active = gx < e.N && gy < e.M;
    // a residual cell cycles through its staging regions; the caller issued this tile's residual load
    // (epi_issue_residual) into region t mod slots, after the store that last used the region had drained
    const unsigned b = RES ? (st.t & ((1u << e.slot_shift) - 1u)) : 0u;
    const unsigned region_off = e.region_off + b * e.region_stride;
    const unsigned region = smem_u32(dyn_smem() + region_off);
    if (!RES) {
        if (lane == 0) bulk_wait_read_all();   // the earlier store has finished reading the region
        __syncwarp();
    }
    if (!mbar_wait_warp(e.tfull, e.tfull_parity, e.abort_flag, e.status, 4, lane)) return false;
    if (RES) {
        if (!mbar_wait_warp(e.rbar + 8u * b, (st.t >> e.slot_shift) & 1u, e.abort_flag, e.status, 7, lane)) return false;
    }
    tc_fence_after();
    if (active) {
        const unsigned tbase = e.tmem_acc + ((unsigned)(quad * 32) << 16) + (unsigned)cbase;
        // one branch per tile selects the arithmetic variant; inside, nothing depends on a run-time flag
        if (!RES) {
            switch (e.ef & (EF_OUT_UNSIGNED | EF_WIDE)) {
            case 0: epi_drain<RES, CLAMP, DP, (0) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            case EF_OUT_UNSIGNED: epi_drain<RES, CLAMP, DP, (EF_OUT_UNSIGNED) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            case EF_WIDE: epi_drain<RES, false, DP, (EF_WIDE) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            default: epi_drain<RES, false, DP, (EF_WIDE | EF_OUT_UNSIGNED) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            }
        } else if (!DP) {
            switch (e.ef & (EF_OUT_UNSIGNED | EF_RES_UNSIGNED | EF_WIDE)) {
            case 0: epi_drain<RES, CLAMP, DP, (0) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            case 1: epi_drain<RES, CLAMP, DP, (1) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            case 2: epi_drain<RES, CLAMP, DP, (2) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            case 3: epi_drain<RES, CLAMP, DP, (3) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            case EF_WIDE | 0: epi_drain<RES, false, DP, (EF_WIDE | 0) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            case EF_WIDE | 1: epi_drain<RES, false, DP, (EF_WIDE | 1) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            case EF_WIDE | 2: epi_drain<RES, false, DP, (EF_WIDE | 2) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            default: epi_drain<RES, false, DP, (EF_WIDE | 3) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            }
        } else {
            switch (e.ef & (EF_OUT_UNSIGNED | EF_T_UNSIGNED | EF_DP_A_SIGNED)) {
            case 0: epi_drain<RES, CLAMP, DP, (0) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            case 1: epi_drain<RES, CLAMP, DP, (1) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            case 4: epi_drain<RES, CLAMP, DP, (4) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            case 5: epi_drain<RES, CLAMP, DP, (5) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            case 8: epi_drain<RES, CLAMP, DP, (8) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            case 9: epi_drain<RES, CLAMP, DP, (9) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            case 12: epi_drain<RES, CLAMP, DP, (12) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            default: epi_drain<RES, CLAMP, DP, (13) | P>(e, tbase, cbase, region_off, st.rb, lane); break;
            }
        }
    }
    // the accumulator is drained: hand it back before the store goes out
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(e.tempty);
    fence_async_smem();
    __syncwarp();
    if (lane == 0 && active) {
        tma_store_2d(tmO, region, gx, gy);
        bulk_commit();
    }
    ++st.t;
    return true;
}

}  // namespace n2d2b
