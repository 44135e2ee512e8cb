// CUDA-core kernels of the quantized integer path: the layers that are not dense contractions
// (depthwise convolution, pooling, element-wise sum, stand-alone rescale) plus a direct convolution
// and a direct fully-connected kernel that accept any geometry.  Every kernel ends in the same
// requantisation epilogue (common.cuh), so no float tensor or separate Scaling pass exists between
// layers.  Activations are NHWC int8 (signed or unsigned per tensor) or int32.
#include <algorithm>
#include "kernels.h"

namespace n2d2b {

static inline unsigned grid_for(size_t n, int block)
{
    size_t g = (n + block - 1) / block;
    const size_t cap = 148u * 32u * 64u;
    return (unsigned)(g < cap ? (g ? g : 1) : cap);
}

template <typename T>
__device__ __forceinline__ void store_out(void* out, size_t i, int v);
template <>
__device__ __forceinline__ void store_out<int8_t>(void* out, size_t i, int v)
{
    ((int8_t*)out)[i] = (int8_t)v;  // the low byte is the value for both u8 and s8 tensors
}
template <>
__device__ __forceinline__ void store_out<int32_t>(void* out, size_t i, int v)
{
    ((int32_t*)out)[i] = v;
}

// ---------------------------------------------------------------------------------------------
// Direct convolution: one thread per output value, output channel fastest (NHWC).  Replaces the
// reference's ConvCell_Frame_Kernels::forward + forwardBias + Scaling + activation for geometries
// the tensor-core kernel does not take (few input channels, groups, dilation).
// ---------------------------------------------------------------------------------------------
template <typename OutT>
__global__ void conv_direct_kernel(const uint8_t* __restrict__ in, int in_unsigned,
                                   const int8_t* __restrict__ w, ConvGeom g, QuantDev q,
                                   Residual r, void* __restrict__ out, size_t total)
{
    const bool vec4 = (g.Cg % 4 == 0);
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int o = (int)(idx % g.O);
        size_t p = idx / g.O;
        const int ox = (int)(p % g.oW); p /= g.oW;
        const int oy = (int)(p % g.oH);
        const int b = (int)(p / g.oH);
        const int grp = o / g.Og;
        const int iy0 = oy * g.sY - g.pT, ix0 = ox * g.sX - g.pL;
        const int8_t* wo = w + (size_t)o * g.kH * g.kW * g.Cg;
        int acc = 0;
        for (int ky = 0; ky < g.kH; ++ky) {
            const int iy = iy0 + ky * g.dY;
            if (iy < 0 || iy >= g.H) continue;
            for (int kx = 0; kx < g.kW; ++kx) {
                const int ix = ix0 + kx * g.dX;
                if (ix < 0 || ix >= g.W) continue;
                const uint8_t* ip = in + (((size_t)b * g.H + iy) * g.W + ix) * g.C + (size_t)grp * g.Cg;
                const int8_t* wp = wo + (size_t)(ky * g.kW + kx) * g.Cg;
                if (vec4 && ((((uintptr_t)ip) | ((uintptr_t)wp)) & 3) == 0) {
                    const unsigned* ip4 = (const unsigned*)ip;
                    const int* wp4 = (const int*)wp;
                    if (in_unsigned)
                        for (int c = 0; c < g.Cg / 4; ++c) acc = dp4a_us(ip4[c], wp4[c], acc);
                    else
                        for (int c = 0; c < g.Cg / 4; ++c) acc = dp4a_ss((int)ip4[c], wp4[c], acc);
                } else {
                    for (int c = 0; c < g.Cg; ++c)
                        acc += load_i8(ip, c, in_unsigned) * (int)wp[c];
                }
            }
        }
        long long x = (long long)acc + (q.bias ? (long long)q.bias[o] : 0ll);
        int y = requant64(x, o, q);
        if (r.ptr) {
            const long long u = (long long)y + (long long)load_i8(r.ptr, idx, r.is_unsigned);
            y = requant64(u, o, r.q2);
        }
        store_out<OutT>(out, idx, y);
    }
}

cudaError_t launch_conv_direct(const void* in, int in_unsigned, const int8_t* w, const ConvGeom& g,
                               const QuantDev& q, const Residual& r, void* out, int out_dtype,
                               cudaStream_t s)
{
    const size_t total = (size_t)g.B * g.oH * g.oW * g.O;
    if (total == 0) return cudaSuccess;
    const int block = 256;
    const unsigned grid = grid_for(total, block);
    if (out_dtype == DT_I8)
        conv_direct_kernel<int8_t><<<grid, block, 0, s>>>((const uint8_t*)in, in_unsigned, w, g, q, r, out, total);
    else
        conv_direct_kernel<int32_t><<<grid, block, 0, s>>>((const uint8_t*)in, in_unsigned, w, g, q, r, out, total);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Depthwise convolution: HBM-bound (one multiply-add per loaded byte and tap), so it stays on the
// CUDA cores.  One thread owns 16 consecutive channels of one output pixel: every tap is one
// 128-bit load of the input and one of the weights, the result one 128-bit store.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void unpack16(const uint4& v, bool is_unsigned, int* x)
{
    const unsigned wds[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const unsigned byte = (wds[i] >> (8 * j)) & 0xffu;
            x[i * 4 + j] = is_unsigned ? (int)byte : (int)(int8_t)byte;
        }
}

__device__ __forceinline__ uint4 pack16(const int* y)
{
    unsigned wds[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
        wds[i] = ((unsigned)y[i * 4] & 0xffu) | (((unsigned)y[i * 4 + 1] & 0xffu) << 8)
               | (((unsigned)y[i * 4 + 2] & 0xffu) << 16) | (((unsigned)y[i * 4 + 3] & 0xffu) << 24);
    return make_uint4(wds[0], wds[1], wds[2], wds[3]);
}

__global__ void conv_depthwise_kernel(const uint8_t* __restrict__ in, int in_unsigned,
                                      const int8_t* __restrict__ w_hwc, ConvGeom g, QuantDev q,
                                      uint8_t* __restrict__ out, size_t total_vec)
{
    const int cv = g.C / 16;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total_vec;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int c16 = (int)(idx % cv);
        size_t p = idx / cv;
        const int ox = (int)(p % g.oW); p /= g.oW;
        const int oy = (int)(p % g.oH);
        const int b = (int)(p / g.oH);
        const int c0 = c16 * 16;
        int acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0;
        const int iy0 = oy * g.sY - g.pT, ix0 = ox * g.sX - g.pL;
        for (int ky = 0; ky < g.kH; ++ky) {
            const int iy = iy0 + ky * g.dY;
            if (iy < 0 || iy >= g.H) continue;
            for (int kx = 0; kx < g.kW; ++kx) {
                const int ix = ix0 + kx * g.dX;
                if (ix < 0 || ix >= g.W) continue;
                const uint4 xv = *(const uint4*)(in + (((size_t)b * g.H + iy) * g.W + ix) * g.C + c0);
                const uint4 wv = __ldg((const uint4*)(w_hwc + (size_t)(ky * g.kW + kx) * g.C + c0));
                int xs[16], ws[16];
                unpack16(xv, in_unsigned != 0, xs);
                unpack16(wv, false, ws);
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[i] += xs[i] * ws[i];
            }
        }
        int y[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const long long x = (long long)acc[i] + (q.bias ? (long long)q.bias[c0 + i] : 0ll);
            y[i] = requant64(x, c0 + i, q);
        }
        *(uint4*)(out + idx * 16) = pack16(y);
    }
}

// Depthwise 3x3 convolution with the 32-bit epilogue.  A thread owns four channels (one 32-bit word per pixel) of
// four horizontally adjacent output pixels.  Its weights are kept as one word per (tap, channel) with the other three
// bytes cleared, so a channel's product is a single four-way byte dot product on the packed input word, without
// unpacking anything: 144 dp4a for 16 outputs.  One block per output row, no 64-bit index arithmetic.
// fq = [5][cpad] constants of the 32-bit rescale (lo, hi, mult, add, shift), proved exact on the host.
template <bool IN_UNSIGNED>
__device__ __forceinline__ void dw_mac4(int (&acc)[4], unsigned xv, const unsigned (&w)[4])
{
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (IN_UNSIGNED) asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(acc[j]) : "r"(xv), "r"(w[j]), "r"(acc[j]));
        else asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(acc[j]) : "r"(xv), "r"(w[j]), "r"(acc[j]));
    }
}

// S1: stride 1 and dilation 1 - the four pixels of a thread read six input columns per row instead of twelve
template <bool IN_UNSIGNED, bool CLAMP, bool OUT_UNSIGNED, bool S1>
__global__ void __launch_bounds__(256)
conv_depthwise3x3_dp4a_kernel(const uint8_t* __restrict__ in, const int8_t* __restrict__ w_hwc, ConvGeom g,
                              const int* __restrict__ fq, int cpad, uint8_t* __restrict__ out)
{
    const int cw = g.C / 4;                        // channel words per pixel
    // blockDim.x is a multiple of cw: a thread keeps its channel word over the whole launch.  A thread's four
    // pixels are adjacent, so most of its input words are shared between them (spreading a thread's pixels for
    // fully coalesced warp loads measured slower).  All offsets are 32-bit word indices (checked by the host).
    const int c4 = threadIdx.x % cw;
    const int xi = threadIdx.x / cw;
    const int xthreads = blockDim.x / cw;
    unsigned wm[9][4];
#pragma unroll
    for (int t = 0; t < 9; ++t) {
        const unsigned wv = __ldg((const unsigned*)(w_hwc + (size_t)t * g.C) + c4);
#pragma unroll
        for (int j = 0; j < 4; ++j) wm[t][j] = wv & (0xffu << (8 * j));
    }
    int lo[4], hi[4], mu[4], ad[4], sh[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int ch = c4 * 4 + j;
        lo[j] = __ldg(fq + 0 * cpad + ch); hi[j] = __ldg(fq + 1 * cpad + ch);
        mu[j] = __ldg(fq + 2 * cpad + ch); ad[j] = __ldg(fq + 3 * cpad + ch); sh[j] = __ldg(fq + 4 * cpad + ch);
    }
    const unsigned* in_w = (const unsigned*)in + c4;
    unsigned* out_w = (unsigned*)out + c4;
    for (int row = blockIdx.x; row < g.B * g.oH; row += gridDim.x) {
        const int b = row / g.oH, oy = row - b * g.oH;
        const int iy0 = oy * g.sY - g.pT;
        unsigned rbase[3];
        bool rok[3];
#pragma unroll
        for (int ky = 0; ky < 3; ++ky) {
            const int iy = iy0 + ky * g.dY;
            rok[ky] = iy >= 0 && iy < g.H;
            rbase[ky] = (unsigned)((b * g.H + (rok[ky] ? iy : 0)) * g.W * cw);
        }
        const unsigned obase = (unsigned)(row * g.oW * cw);
        for (int chunk0 = 0; chunk0 < g.oW; chunk0 += 4 * xthreads) {
            const int ox0 = chunk0 + 4 * xi;       // pixels ox0 .. ox0 + 3
            int acc[4][4];
#pragma unroll
            for (int p = 0; p < 4; ++p)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[p][j] = 0;
            if (S1) {
                // columns ox0 - pL .. ox0 - pL + 5; pixel p, tap kx reads column p + kx
                unsigned coff[6];
                bool cok[6];
#pragma unroll
                for (int q = 0; q < 6; ++q) {
                    const int ix = ox0 - g.pL + q;
                    cok[q] = ix >= 0 && ix < g.W;
                    coff[q] = (unsigned)((cok[q] ? ix : 0) * cw);
                }
#pragma unroll
                for (int ky = 0; ky < 3; ++ky) {
                    unsigned xv[6];
#pragma unroll
                    for (int q = 0; q < 6; ++q) xv[q] = (rok[ky] && cok[q]) ? __ldg(in_w + rbase[ky] + coff[q]) : 0u;
#pragma unroll
                    for (int p = 0; p < 4; ++p)
#pragma unroll
                        for (int kx = 0; kx < 3; ++kx) dw_mac4<IN_UNSIGNED>(acc[p], xv[p + kx], wm[ky * 3 + kx]);
                }
            } else {
                unsigned coff[4][3];
                bool cok[4][3];
#pragma unroll
                for (int p = 0; p < 4; ++p)
#pragma unroll
                    for (int kx = 0; kx < 3; ++kx) {
                        const int ix = (ox0 + p) * g.sX - g.pL + kx * g.dX;
                        cok[p][kx] = ix >= 0 && ix < g.W;
                        coff[p][kx] = (unsigned)((cok[p][kx] ? ix : 0) * cw);
                    }
#pragma unroll
                for (int ky = 0; ky < 3; ++ky)
#pragma unroll
                    for (int p = 0; p < 4; ++p)
#pragma unroll
                        for (int kx = 0; kx < 3; ++kx) {
                            const unsigned xv = (rok[ky] && cok[p][kx]) ? __ldg(in_w + rbase[ky] + coff[p][kx]) : 0u;
                            dw_mac4<IN_UNSIGNED>(acc[p], xv, wm[ky * 3 + kx]);
                        }
            }
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                if (ox0 + p >= g.oW) break;
                int y[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    int x = acc[p][j];
                    if (CLAMP) x = min(max(x, lo[j]), hi[j]);
                    y[j] = (x * mu[j] + ad[j]) >> sh[j];
                }
                unsigned tmp, d;
                if (OUT_UNSIGNED) {
                    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(tmp) : "r"(y[3]), "r"(y[2]), "r"(y[2]));   // upper half shifted out below
                    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(y[1]), "r"(y[0]), "r"(tmp));
                } else {
                    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(tmp) : "r"(y[3]), "r"(y[2]), "r"(y[2]));   // upper half shifted out below
                    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(y[1]), "r"(y[0]), "r"(tmp));
                }
                out_w[obase + (unsigned)((ox0 + p) * cw)] = d;
            }
        }
    }
}

cudaError_t launch_conv_depthwise(const void* in, int in_unsigned, const int8_t* w_hwc,
                                  const ConvGeom& g, const QuantDev& q, const FastQuant& fast, void* out, cudaStream_t s)
{
    // 3x3 filters whose rescale has the proved 32-bit form take the dot-product kernel
    const int cw = g.C / 4;
    const bool idx32 = (long long)g.B * g.H * g.W * cw < (1ll << 31) && (long long)g.B * g.oH * g.oW * cw < (1ll << 31);
    if (fast.enabled && !fast.wide && g.kH == 3 && g.kW == 3 && 256 % cw == 0 && idx32) {
        const long long rows = (long long)g.B * g.oH;
        if (rows == 0 || g.oW == 0) return cudaSuccess;
        // few, long-lived blocks: a thread's weights and constants (29 loads) are fetched once and serve many rows
        const long long max_blocks = 148ll * 6;
        const unsigned grid = (unsigned)(rows < max_blocks ? rows : max_blocks);
        // a block's threads cover 4 * (threads / cw) pixels of a row per pass
        int threads = 256;
        while (threads > 32 && (threads / 2) % cw == 0 && 4 * (threads / 2 / cw) >= g.oW) threads /= 2;
        const uint8_t* ip = (const uint8_t*)in;
        uint8_t* op = (uint8_t*)out;
        const bool s1 = g.sX == 1 && g.dX == 1;
#define N2D2B_DW(U, C, O)                                                                                         \
    do {                                                                                                          \
        if (s1) conv_depthwise3x3_dp4a_kernel<U, C, O, true><<<grid, threads, 0, s>>>(ip, w_hwc, g, fast.fq, fast.cpad, op); \
        else conv_depthwise3x3_dp4a_kernel<U, C, O, false><<<grid, threads, 0, s>>>(ip, w_hwc, g, fast.fq, fast.cpad, op);   \
    } while (0)
        const int v = (in_unsigned ? 4 : 0) | (fast.need_clamp ? 2 : 0) | (fast.out_unsigned ? 1 : 0);
        switch (v) {
        case 0: N2D2B_DW(false, false, false); break;
        case 1: N2D2B_DW(false, false, true); break;
        case 2: N2D2B_DW(false, true, false); break;
        case 3: N2D2B_DW(false, true, true); break;
        case 4: N2D2B_DW(true, false, false); break;
        case 5: N2D2B_DW(true, false, true); break;
        case 6: N2D2B_DW(true, true, false); break;
        default: N2D2B_DW(true, true, true); break;
        }
#undef N2D2B_DW
        return cudaGetLastError();
    }

    const size_t total = (size_t)g.B * g.oH * g.oW * (g.C / 16);
    if (total == 0) return cudaSuccess;
    const int block = 256;
    conv_depthwise_kernel<<<grid_for(total, block), block, 0, s>>>((const uint8_t*)in, in_unsigned, w_hwc, g, q,
                                                                   (uint8_t*)out, total);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Pooling (PoolCell): max over the in-image taps (0 for an all-padding window); average with the
// full window as divisor and truncation toward zero, as the reference's quantized PoolCell does.
// Vector path: 16 channels per thread when C % 16 == 0 and the tensor is int8.
// ---------------------------------------------------------------------------------------------
__global__ void pool_vec_kernel(const uint8_t* __restrict__ in, int in_unsigned, PoolGeom g,
                                uint8_t* __restrict__ out, size_t total_vec)
{
    const int cv = g.C / 16;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total_vec;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int c16 = (int)(idx % cv);
        size_t p = idx / cv;
        const int ox = (int)(p % g.oW); p /= g.oW;
        const int oy = (int)(p % g.oH);
        const int b = (int)(p / g.oH);
        const int iy0 = oy * g.sY - g.padY, ix0 = ox * g.sX - g.padX;
        int v[16];
        bool valid = false;
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0;
        for (int ky = 0; ky < g.pH; ++ky) {
            const int iy = iy0 + ky;
            if (iy < 0 || iy >= g.H) continue;
            for (int kx = 0; kx < g.pW; ++kx) {
                const int ix = ix0 + kx;
                if (ix < 0 || ix >= g.W) continue;
                const uint4 xv = *(const uint4*)(in + (((size_t)b * g.H + iy) * g.W + ix) * g.C + c16 * 16);
                int xs[16];
                unpack16(xv, in_unsigned != 0, xs);
                if (g.is_max) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = (!valid || xs[i] > v[i]) ? xs[i] : v[i];
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] += xs[i];
                }
                valid = true;
            }
        }
        if (!g.is_max) {
            const int count = g.pH * g.pW;
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = v[i] / count;  // C division truncates toward zero
        }
        *(uint4*)(out + idx * 16) = pack16(v);
    }
}

// Max pooling, 16 channels per thread, one block per output row: the window bounds of the row are
// computed once, the maximum runs on four bytes at a time, and no thread divides 64-bit indices.
template <bool UNSIGNED>
__global__ void pool_max_row_kernel(const uint8_t* __restrict__ in, PoolGeom g, uint8_t* __restrict__ out)
{
    const int cv = g.C / 16;
    for (int row = blockIdx.x; row < g.B * g.oH; row += gridDim.x) {
        const int b = row / g.oH, oy = row - b * g.oH;
        const int iy0 = oy * g.sY - g.padY;
        const int ky_lo = iy0 < 0 ? -iy0 : 0;
        const int ky_hi = (g.H - iy0) < g.pH ? (g.H - iy0) : g.pH;
        const uint8_t* img = in + (size_t)b * g.H * g.W * g.C;
        uint8_t* orow = out + (size_t)row * g.oW * g.C;
        for (int t = threadIdx.x; t < g.oW * cv; t += blockDim.x) {
            const int ox = t / cv, c16 = t - ox * cv;
            const int ix0 = ox * g.sX - g.padX;
            const int kx_lo = ix0 < 0 ? -ix0 : 0;
            const int kx_hi = (g.W - ix0) < g.pW ? (g.W - ix0) : g.pW;
            uint4 m = make_uint4(0u, 0u, 0u, 0u);
            if (g.pH == 3 && g.pW == 3 && ky_lo == 0 && ky_hi == 3 && kx_lo == 0 && kx_hi == 3) {
                // a whole 3x3 window: nine independent loads in flight, then the maxima (the general loop below
                // would wait for each load in turn)
                const uint8_t* p = img + ((size_t)iy0 * g.W + ix0) * g.C + c16 * 16;
                const size_t rs = (size_t)g.W * g.C;
                uint4 x[9];
#pragma unroll
                for (int ky = 0; ky < 3; ++ky)
#pragma unroll
                    for (int kx = 0; kx < 3; ++kx) x[ky * 3 + kx] = __ldg((const uint4*)(p + ky * rs + (size_t)kx * g.C));
                m = x[0];
#pragma unroll
                for (int i = 1; i < 9; ++i) {
                    if (UNSIGNED) {
                        m.x = __vmaxu4(m.x, x[i].x); m.y = __vmaxu4(m.y, x[i].y);
                        m.z = __vmaxu4(m.z, x[i].z); m.w = __vmaxu4(m.w, x[i].w);
                    } else {
                        m.x = __vmaxs4(m.x, x[i].x); m.y = __vmaxs4(m.y, x[i].y);
                        m.z = __vmaxs4(m.z, x[i].z); m.w = __vmaxs4(m.w, x[i].w);
                    }
                }
                *(uint4*)(orow + (size_t)t * 16) = m;
                continue;
            }
            bool first = true;
            for (int ky = ky_lo; ky < ky_hi; ++ky) {
                const uint8_t* p = img + ((size_t)(iy0 + ky) * g.W + ix0) * g.C + c16 * 16;
                for (int kx = kx_lo; kx < kx_hi; ++kx) {
                    const uint4 xv = __ldg((const uint4*)(p + (size_t)kx * g.C));
                    if (first) {
                        m = xv;
                        first = false;
                    } else if (UNSIGNED) {
                        m.x = __vmaxu4(m.x, xv.x); m.y = __vmaxu4(m.y, xv.y);
                        m.z = __vmaxu4(m.z, xv.z); m.w = __vmaxu4(m.w, xv.w);
                    } else {
                        m.x = __vmaxs4(m.x, xv.x); m.y = __vmaxs4(m.y, xv.y);
                        m.z = __vmaxs4(m.z, xv.z); m.w = __vmaxs4(m.w, xv.w);
                    }
                }
            }
            *(uint4*)(orow + (size_t)t * 16) = m;   // an all-padding window stays 0
        }
    }
}

template <typename ElemT>
__global__ void pool_scalar_kernel(const void* __restrict__ in, int in_unsigned, PoolGeom g,
                                   void* __restrict__ out, size_t total)
{
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(idx % g.C);
        size_t p = idx / g.C;
        const int ox = (int)(p % g.oW); p /= g.oW;
        const int oy = (int)(p % g.oH);
        const int b = (int)(p / g.oH);
        const int iy0 = oy * g.sY - g.padY, ix0 = ox * g.sX - g.padX;
        long long v = 0;
        bool valid = false;
        for (int ky = 0; ky < g.pH; ++ky) {
            const int iy = iy0 + ky;
            if (iy < 0 || iy >= g.H) continue;
            for (int kx = 0; kx < g.pW; ++kx) {
                const int ix = ix0 + kx;
                if (ix < 0 || ix >= g.W) continue;
                const size_t ii = (((size_t)b * g.H + iy) * g.W + ix) * g.C + c;
                long long x;
                if (sizeof(ElemT) == 4) x = ((const int32_t*)in)[ii];
                else x = load_i8(in, ii, in_unsigned != 0);
                if (g.is_max) v = (!valid || x > v) ? x : v;
                else v += x;
                valid = true;
            }
        }
        if (!g.is_max) v = v / (long long)(g.pH * g.pW);
        if (sizeof(ElemT) == 4) ((int32_t*)out)[idx] = (int32_t)v;
        else ((int8_t*)out)[idx] = (int8_t)v;
    }
}

// Average over the whole feature map (the pooling cell before the classifier): one thread per four channels of
// an image, so a warp reads 128 consecutive bytes per pixel and every load of the pixel loop is independent of
// the others.  Bytes are summed as two pairs of 16-bit lanes (signed inputs are biased to unsigned by flipping
// the top bit and un-biased at the end; up to 257 pixels fit a lane).  Divides by the window size and truncates
// toward zero like the reference's quantized cell.
template <bool UNSIGNED>
__global__ void pool_global_avg_kernel(const uint8_t* __restrict__ in, int pixels, int C, size_t total_words,
                                       uint8_t* __restrict__ out)
{
    const int cw = C / 4;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total_words; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t b = idx / cw;
        const int w = (int)(idx - b * cw);
        const unsigned* p = (const unsigned*)(in + b * (size_t)pixels * C) + w;
        unsigned even = 0, odd = 0;   // bytes 0, 2 and bytes 1, 3 as 16-bit lanes
#pragma unroll 7
        for (int i = 0; i < pixels; ++i) {
            unsigned x = __ldg(p + (size_t)i * cw);
            if (!UNSIGNED) x ^= 0x80808080u;
            even += x & 0x00ff00ffu;
            odd += (x >> 8) & 0x00ff00ffu;
        }
        int v[4] = {(int)(even & 0xffffu), (int)(odd & 0xffffu), (int)(even >> 16), (int)(odd >> 16)};
        unsigned o = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (!UNSIGNED) v[j] -= 128 * pixels;
            o |= ((unsigned)(v[j] / pixels) & 0xffu) << (8 * j);   // C division truncates toward zero
        }
        ((unsigned*)out)[idx] = o;
    }
}

cudaError_t launch_pool(const void* in, int in_unsigned, const PoolGeom& g, void* out, cudaStream_t s)
{
    // int8 tensors; int32 tensors go through launch_pool_i32
    const int block = 256;
    if (g.C % 16 == 0 && g.is_max) {
        const long long rows = (long long)g.B * g.oH;
        if (rows == 0 || g.oW == 0) return cudaSuccess;
        const int items = g.oW * (g.C / 16);
        const int threads = items >= 256 ? 256 : ((items + 31) / 32) * 32;
        const unsigned grid = (unsigned)(rows < (1ll << 20) ? rows : (1ll << 20));
        if (in_unsigned) pool_max_row_kernel<true><<<grid, threads, 0, s>>>((const uint8_t*)in, g, (uint8_t*)out);
        else pool_max_row_kernel<false><<<grid, threads, 0, s>>>((const uint8_t*)in, g, (uint8_t*)out);
    } else if (!g.is_max && g.C % 4 == 0 && g.pH == g.H && g.pW == g.W && g.padY == 0 && g.padX == 0 && g.oH == 1 && g.oW == 1
               && g.H * g.W <= 257 && ((uintptr_t)in & 3) == 0 && ((uintptr_t)out & 3) == 0) {
        const size_t total = (size_t)g.B * (g.C / 4);
        if (total == 0) return cudaSuccess;
        if (in_unsigned)
            pool_global_avg_kernel<true><<<grid_for(total, block), block, 0, s>>>((const uint8_t*)in, g.H * g.W, g.C, total, (uint8_t*)out);
        else
            pool_global_avg_kernel<false><<<grid_for(total, block), block, 0, s>>>((const uint8_t*)in, g.H * g.W, g.C, total, (uint8_t*)out);
    } else if (g.C % 16 == 0) {
        const size_t total = (size_t)g.B * g.oH * g.oW * (g.C / 16);
        if (total == 0) return cudaSuccess;
        pool_vec_kernel<<<grid_for(total, block), block, 0, s>>>((const uint8_t*)in, in_unsigned, g, (uint8_t*)out, total);
    } else {
        const size_t total = (size_t)g.B * g.oH * g.oW * g.C;
        if (total == 0) return cudaSuccess;
        pool_scalar_kernel<int8_t><<<grid_for(total, block), block, 0, s>>>(in, in_unsigned, g, out, total);
    }
    return cudaGetLastError();
}

cudaError_t launch_pool_i32(const void* in, const PoolGeom& g, void* out, cudaStream_t s)
{
    const size_t total = (size_t)g.B * g.oH * g.oW * g.C;
    if (total == 0) return cudaSuccess;
    pool_scalar_kernel<int32_t><<<grid_for(total, 256), 256, 0, s>>>(in, 0, g, out, total);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Element-wise sum of up to four tensors (ElemWiseCell, Sum, unit weights) followed by the cell's
// own requantisation; with a single input it is the stand-alone ScalingCell.
// ---------------------------------------------------------------------------------------------
template <typename OutT>
__global__ void elemwise_sum_kernel(SumInputs ins, size_t total, int C, QuantDev q, void* __restrict__ out)
{
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(idx % C);
        long long x = 0;
        for (int k = 0; k < ins.n; ++k) {
            if (ins.dtype[k] == DT_I32) x += ((const int32_t*)ins.ptr[k])[idx];
            else x += load_i8(ins.ptr[k], idx, ins.is_unsigned[k] != 0);
        }
        if (q.bias) x += q.bias[c];
        store_out<OutT>(out, idx, requant64(x, c, q));
    }
}

// Fast path: two int8 inputs, int8 output, 16 values per thread.
__global__ void elemwise_sum2_vec_kernel(const uint8_t* __restrict__ a, int a_unsigned,
                                         const uint8_t* __restrict__ b, int b_unsigned, size_t total_vec,
                                         int C, QuantDev q, uint8_t* __restrict__ out)
{
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total_vec;
         idx += (size_t)gridDim.x * blockDim.x) {
        const uint4 av = *(const uint4*)(a + idx * 16);
        const uint4 bv = *(const uint4*)(b + idx * 16);
        int xa[16], xb[16], y[16];
        unpack16(av, a_unsigned != 0, xa);
        unpack16(bv, b_unsigned != 0, xb);
        const int c0 = (int)((idx * 16) % C);
#pragma unroll
        for (int i = 0; i < 16; ++i) y[i] = requant64((long long)xa[i] + xb[i], c0 + i, q);
        *(uint4*)(out + idx * 16) = pack16(y);
    }
}

cudaError_t launch_elemwise_sum(const SumInputs& ins, size_t pixels, int C, const QuantDev& q,
                                void* out, int out_dtype, cudaStream_t s)
{
    const size_t total = pixels * (size_t)C;
    if (total == 0) return cudaSuccess;
    const int block = 256;
    if (ins.n == 2 && out_dtype == DT_I8 && ins.dtype[0] == DT_I8 && ins.dtype[1] == DT_I8 && C % 16 == 0
        && !q.bias) {
        elemwise_sum2_vec_kernel<<<grid_for(total / 16, block), block, 0, s>>>(
            (const uint8_t*)ins.ptr[0], ins.is_unsigned[0], (const uint8_t*)ins.ptr[1], ins.is_unsigned[1],
            total / 16, C, q, (uint8_t*)out);
    } else if (out_dtype == DT_I8) {
        elemwise_sum_kernel<int8_t><<<grid_for(total, block), block, 0, s>>>(ins, total, C, q, out);
    } else {
        elemwise_sum_kernel<int32_t><<<grid_for(total, block), block, 0, s>>>(ins, total, C, q, out);
    }
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Fully connected on CUDA cores: one warp per (image, output), lanes stride over K, shuffle-reduce.
// ---------------------------------------------------------------------------------------------
template <typename OutT>
__global__ void fc_direct_kernel(const uint8_t* __restrict__ in, int in_unsigned,
                                 const int8_t* __restrict__ w, int B, int K, int O, QuantDev q,
                                 void* __restrict__ out)
{
    const int lane = threadIdx.x & 31;
    const size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
    const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t idx = warp; idx < (size_t)B * O; idx += nwarps) {
        const int o = (int)(idx % O);
        const int b = (int)(idx / O);
        const uint8_t* ip = in + (size_t)b * K;
        const int8_t* wp = w + (size_t)o * K;
        int acc = 0;
        for (int k = lane; k < K; k += 32) acc += load_i8(ip, k, in_unsigned != 0) * (int)wp[k];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (lane == 0) {
            const long long x = (long long)acc + (q.bias ? (long long)q.bias[o] : 0ll);
            store_out<OutT>(out, idx, requant64(x, o, q));
        }
    }
}

cudaError_t launch_fc_direct(const void* in, int in_unsigned, const int8_t* w, int B, int K, int O,
                             const QuantDev& q, void* out, int out_dtype, cudaStream_t s)
{
    const size_t total = (size_t)B * O;
    if (total == 0) return cudaSuccess;
    const int block = 256;
    const unsigned grid = grid_for(total * 32, block);
    if (out_dtype == DT_I8)
        fc_direct_kernel<int8_t><<<grid, block, 0, s>>>((const uint8_t*)in, in_unsigned, w, B, K, O, q, out);
    else
        fc_direct_kernel<int32_t><<<grid, block, 0, s>>>((const uint8_t*)in, in_unsigned, w, B, K, O, q, out);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Output edge: estimated label = the class with the highest score, the first one among equals
// (Target top-1, src/Target/Target_CUDA_kernels.cu:88-104 of the reference: `if (tmp > maxVal)`).
// One warp per (image, pixel); scores are [pixels][C] int8 or int32.
// ---------------------------------------------------------------------------------------------
// 8 bytes per thread when both row lengths allow it, bytes otherwise
template <typename V>
__global__ void drop_padded_columns_kernel(const V* __restrict__ src, int ld, V* __restrict__ dst, int C, size_t rows)
{
    const size_t total = rows * (size_t)C;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / (size_t)C;
        dst[i] = src[r * (size_t)ld + (i - r * (size_t)C)];
    }
}

cudaError_t launch_drop_padded_columns(const uint8_t* src, int ld, uint8_t* dst, int C, size_t rows, cudaStream_t s)
{
    if (rows == 0) return cudaSuccess;
    const bool vec = (C % 8 == 0) && (ld % 8 == 0) && !((uintptr_t)src & 7) && !((uintptr_t)dst & 7);
    const size_t total = vec ? rows * (size_t)(C / 8) : rows * (size_t)C;
    const int threads = 256;
    const int blocks = (int)std::min<size_t>((total + threads - 1) / threads, 148 * 8);
    if (vec)
        drop_padded_columns_kernel<uint2><<<blocks, threads, 0, s>>>((const uint2*)src, ld / 8, (uint2*)dst, C / 8, rows);
    else
        drop_padded_columns_kernel<uint8_t><<<blocks, threads, 0, s>>>(src, ld, dst, C, rows);
    return cudaGetLastError();
}

template <typename T>
__global__ void argmax_kernel(const T* __restrict__ scores, size_t pixels, int C, int32_t* __restrict__ labels,
                              int32_t* __restrict__ values)
{
    const int lane = threadIdx.x & 31;
    const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
    for (size_t p = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); p < pixels; p += warps) {
        const T* row = scores + p * (size_t)C;
        int best = INT32_MIN, idx = 0x7fffffff;
        for (int c = lane; c < C; c += 32) {
            const int v = (int)row[c];
            if (v > best || idx == 0x7fffffff) { best = v; idx = c; }   // ascending c within a lane: the first of equals stays
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const int ob = __shfl_xor_sync(0xffffffffu, best, off), oi = __shfl_xor_sync(0xffffffffu, idx, off);
            if (oi != 0x7fffffff && (idx == 0x7fffffff || ob > best || (ob == best && oi < idx))) { best = ob; idx = oi; }
        }
        if (lane == 0) {
            labels[p] = idx;
            if (values) values[p] = best;
        }
    }
}

cudaError_t launch_argmax(const void* scores, int dtype, int is_unsigned, size_t pixels, int C, int32_t* labels, int32_t* values,
                          cudaStream_t s)
{
    if (pixels == 0 || C == 0) return cudaSuccess;
    const int block = 256;
    const unsigned grid = grid_for(pixels * 32, block);
    if (dtype == DT_I32) argmax_kernel<int32_t><<<grid, block, 0, s>>>((const int32_t*)scores, pixels, C, labels, values);
    else if (is_unsigned) argmax_kernel<uint8_t><<<grid, block, 0, s>>>((const uint8_t*)scores, pixels, C, labels, values);
    else argmax_kernel<int8_t><<<grid, block, 0, s>>>((const int8_t*)scores, pixels, C, labels, values);
    return cudaGetLastError();
}

// Target top-N (src/Target/Target_CUDA_kernels.cu:44-86).  The reference orders a pixel's scores with an exchange
// sort, "for x: for y: if (v[y] < v[x]) swap(x, y)", quadratic in the number of classes; among equal scores (int8
// logits tie all the time) the classes end in the order those exchanges leave.  That order has a closed form, which
// this kernel evaluates in O(topN x classes) per pixel:
//   * pass x = 0 leaves the minimum at position 0; every position where the running minimum dropped receives the
//     element the minimum displaced;
//   * every later pass x inserts element x into the descending prefix behind its equals, and each group of equal,
//     smaller scores gives its first element to the group below and takes the element coming from above, i.e. the
//     group is rotated by one.
// So a group of equal scores r, read in position order after pass 0, is a queue that appends on a score == r and
// moves its head to its tail on a score > r (when it holds more than one element).  The groups are emitted from the
// highest score down until topN entries are out.  One warp per pixel; the sequential parts run on lane 0.
// Shared memory: three int arrays of C entries.  Output [image][k][pixel of the image], like the reference.
template <typename T>
__global__ void topn_kernel(const T* __restrict__ scores, size_t pixels, size_t hw, int C, int topN, int32_t* __restrict__ labels,
                            int32_t* __restrict__ values)
{
    extern __shared__ int topn_smem[];
    int* val = topn_smem;
    int* ids = val + C;
    int* buf = ids + C;
    const int lane = threadIdx.x;
    for (size_t p = blockIdx.x; p < pixels; p += gridDim.x) {
        const T* row = scores + p * (size_t)C;
        for (int c = lane; c < C; c += 32) { val[c] = (int)row[c]; ids[c] = c; }
        __syncwarp();
        if (lane == 0) {
            int cur = val[0], curid = 0;
            for (int y = 1; y < C; ++y) {
                const int v = val[y];
                if (v < cur) { val[y] = cur; ids[y] = curid; cur = v; curid = y; }
            }
            val[0] = cur;
            ids[0] = curid;
        }
        __syncwarp();
        const size_t img = p / hw, pix = p - img * hw;
        int32_t* lab = labels + img * (size_t)topN * hw + pix;
        int32_t* vout = values ? values + img * (size_t)topN * hw + pix : nullptr;
        int emitted = 0;
        long long prev = (long long)INT32_MAX + 1;
        while (emitted < topN) {
            // next group: the highest score below the previous group's, and its size
            int r = INT32_MIN, found = 0;
            for (int c = lane; c < C; c += 32) {
                const int v = val[c];
                if ((long long)v < prev && (!found || v > r)) { r = v; found = 1; }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const int orr = __shfl_xor_sync(0xffffffffu, r, off), of = __shfl_xor_sync(0xffffffffu, found, off);
                if (of && (!found || orr > r)) { r = orr; found = 1; }
            }
            if (!found) break;   // fewer than topN classes
            int cnt = 0;
            for (int c = lane; c < C; c += 32) cnt += (val[c] == r);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, off);
            if (lane == 0) {
                int h = 0, L = 0;   // head and length of the queue in buf[0, cnt)
                for (int x = 0; x < C; ++x) {
                    const int v = val[x];
                    if (v == r) {
                        int t = h + L; if (t >= cnt) t -= cnt;
                        buf[t] = ids[x];
                        ++L;
                    } else if (v > r && L > 1) {
                        int t = h + L; if (t >= cnt) t -= cnt;
                        buf[t] = buf[h];
                        if (++h == cnt) h = 0;
                    }
                }
                for (int k = 0; k < cnt && emitted + k < topN; ++k) {
                    int t = h + k; if (t >= cnt) t -= cnt;
                    lab[(size_t)(emitted + k) * hw] = buf[t];
                    if (vout) vout[(size_t)(emitted + k) * hw] = r;
                }
            }
            emitted += cnt;
            prev = r;
            __syncwarp();
        }
        __syncwarp();
    }
}

cudaError_t launch_topn(const void* scores, int dtype, int is_unsigned, size_t pixels, size_t hw, int C, int topN, int32_t* labels,
                        int32_t* values, cudaStream_t s)
{
    if (pixels == 0 || C == 0 || topN == 0) return cudaSuccess;
    const size_t smem = (size_t)3 * C * sizeof(int);
    const unsigned grid = (unsigned)std::min<size_t>(pixels, 148 * 16);
#define N2D2B_TOPN(T)                                                                                                   \
    do {                                                                                                                \
        cudaError_t e = cudaFuncSetAttribute(topn_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        if (e != cudaSuccess) return e;                                                                                 \
        topn_kernel<T><<<grid, 32, smem, s>>>((const T*)scores, pixels, hw, C, topN, labels, values);                   \
    } while (0)
    if (dtype == DT_I32) N2D2B_TOPN(int32_t);
    else if (is_unsigned) N2D2B_TOPN(uint8_t);
    else N2D2B_TOPN(int8_t);
#undef N2D2B_TOPN
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Input edge: what the post-training quantization puts in front of the network
// (src/DeepNetQuantization.cpp:359-370: RangeAffineTransformation(Multiplies, 2^n - 1 or 2^(n-1) - 1) with
// Truncate): float stimuli [batch][channel][y][x] -> trunc(x * factor) as 8-bit [batch][y][x][channel].
// The product is a float32 multiply rounded to nearest, as on the reference's float tensors.
// ---------------------------------------------------------------------------------------------
__global__ void quantize_stimuli_kernel(const float* __restrict__ in, int C, int H, int W, size_t total, float factor, int lo, int hi,
                                        uint8_t* __restrict__ out)
{
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(idx % C);
        size_t p = idx / C;
        const int x = (int)(p % W); p /= W;
        const int y = (int)(p % H);
        const size_t b = p / H;
        float v = truncf(__fmul_rn(in[((b * C + c) * H + y) * W + x], factor));
        v = fminf(fmaxf(v, (float)lo), (float)hi);
        out[idx] = (uint8_t)(int)v;
    }
}

cudaError_t launch_quantize_stimuli(const float* in, int B, int C, int H, int W, float factor, int lo, int hi, void* out, cudaStream_t s)
{
    const size_t total = (size_t)B * C * H * W;
    if (total == 0) return cudaSuccess;
    quantize_stimuli_kernel<<<grid_for(total, 256), 256, 0, s>>>(in, C, H, W, total, factor, lo, hi, (uint8_t*)out);
    return cudaGetLastError();
}

}  // namespace n2d2b
