// Shared device-side definitions of the quantized integer path: the per-output-channel rescale
// ("Scaling" in N2D2), saturation and activation that every kernel's epilogue applies.
//
// Arithmetic follows the reference CPU kernels (src/Scaling_Kernels.cpp:29-199 in N2D2):
//   clip (optional, float/fixed modes only) -> rescale -> round -> saturate to nbBits -> activation.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace n2d2b {

enum ScalingMode : int {
    SC_NONE = 0, SC_FLOAT_MULT = 1, SC_FIXED_MULT16 = 2, SC_FIXED_MULT32 = 3,
    SC_SINGLE_SHIFT = 4, SC_DOUBLE_SHIFT = 5
};
enum ActKind : int { ACT_LINEAR = 0, ACT_RECTIFIER = 1, ACT_SATURATION = 2 };
enum DType : int { DT_I8 = 0, DT_I32 = 1 };

// Device view of one cell's output quantisation. All per-channel arrays have nb_channels entries.
struct QuantDev {
    int mode;            // ScalingMode
    int act;             // ActKind
    int saturate;        // 1 when the scaling saturates (every mode but NONE)
    int out_lo, out_hi;  // saturation bounds from (nbBits, signedness)
    int is_clipped;      // clip before rescale (FLOAT / FIXED modes)
    int sat_thr;         // threshold of a Saturation activation
    const int32_t* bias;      // nullable; added to the accumulator before anything else
    const int32_t* p0;        // FIXED: multiplier; SINGLE: shift; DOUBLE: first shift (a)
    const int32_t* p1;        // FIXED: fractional bits; DOUBLE: second shift (b)
    const float* fscale;      // FLOAT: factor
    const int32_t* clip_thr;  // clip > 0: floor(clip); clip <= 0: ceil(clip)
    const int32_t* clip_val;  // round(clip): what a clipped value becomes in FIXED mode
    const float* clip_f;      // clip itself: what a clipped value becomes in FLOAT mode
};

// Exact 64-bit requantisation of one value x (accumulator + bias already summed) of channel c.
// Integer-valued restatement of Scaling::propagate followed by the activation.
__device__ __forceinline__ int requant64(long long x, int c, const QuantDev& q)
{
    long long y;
    switch (q.mode) {
    default:
    case SC_NONE:
        y = x;
        break;
    case SC_FLOAT_MULT: {
        float v;
        bool clipped = false;
        if (q.is_clipped) {
            const int thr = q.clip_thr[c];
            const float cf = q.clip_f[c];
            if (cf > 0.0f) {
                if (x < 0) { v = 0.0f; clipped = true; }
                else if (x > (long long)thr) { v = cf; clipped = true; }
            } else {
                if (x > 0) { v = 0.0f; clipped = true; }
                else if (x < (long long)thr) { v = cf; clipped = true; }
            }
        }
        if (!clipped) v = __ll2float_rn(x);
        v = __fmul_rn(v, q.fscale[c]);
        v = roundf(v);
        v = fminf(fmaxf(v, (float)q.out_lo), (float)q.out_hi);
        y = (long long)v;
        break;
    }
    case SC_FIXED_MULT16:
    case SC_FIXED_MULT32: {
        long long r = x;
        if (q.is_clipped) {
            const int thr = q.clip_thr[c];
            const int cv = q.clip_val[c];
            if (q.clip_f[c] > 0.0f) r = (x < 0) ? 0 : ((x > (long long)thr) ? (long long)cv : x);
            else r = (x > 0) ? 0 : ((x < (long long)thr) ? (long long)cv : x);
        }
        const int f = q.p1[c];
        const long long half = (f > 0) ? (1ll << (f - 1)) : 0ll;
        y = (r * (long long)q.p0[c] + half) >> f;
        break;
    }
    case SC_SINGLE_SHIFT: {
        const int s = q.p0[c];
        const long long half = (s > 0) ? (1ll << (s - 1)) : 0ll;
        y = (x + half) >> s;
        break;
    }
    case SC_DOUBLE_SHIFT: {
        const int a = q.p0[c], s = q.p1[c];
        const long long half = (s > 0) ? (1ll << (s - 1)) : 0ll;
        y = (x + (x << a) + half) >> s;
        break;
    }
    }
    if (q.saturate) y = y < q.out_lo ? q.out_lo : (y > q.out_hi ? q.out_hi : y);
    if (q.act == ACT_RECTIFIER) y = y > 0 ? y : 0;
    else if (q.act == ACT_SATURATION) y = y < -q.sat_thr ? -q.sat_thr : (y > q.sat_thr ? q.sat_thr : y);
    // a NONE-mode value leaves the path as int32
    y = y < (long long)INT32_MIN ? (long long)INT32_MIN : (y > (long long)INT32_MAX ? (long long)INT32_MAX : y);
    return (int)y;
}

// u8 x s8 four-way dot product with 32-bit accumulate (the mixed-sign form has no intrinsic)
__device__ __forceinline__ int dp4a_us(unsigned a, int b, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_ss(int a, int b, int c)
{
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ int load_i8(const void* p, size_t i, bool is_unsigned)
{
    return is_unsigned ? (int)((const uint8_t*)p)[i] : (int)((const int8_t*)p)[i];
}

}  // namespace n2d2b
