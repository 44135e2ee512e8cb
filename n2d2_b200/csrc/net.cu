// C ABI (include/n2d2b.h) and the static executor behind it: a quantized network is a list of cells
// in execution order, every tensor an NHWC buffer in HBM, every cell one kernel launch (a residual
// sum is folded into the producing convolution's epilogue when the graph allows it).
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "../../include/n2d2b.h"
#include "kernels.h"
#include "host_internal.h"
#include "tc_common.cuh"

using namespace n2d2b;

// ------------------------------------------------------------------------------------ errors
static thread_local char g_err[512] = "";

static int fail(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

#define CUDA_TRY(expr)                                                                        \
    do {                                                                                      \
        cudaError_t e_ = (expr);                                                              \
        if (e_ != cudaSuccess)                                                                \
            return fail(N2D2B_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), \
                        __FILE__, __LINE__);                                                  \
    } while (0)

// ------------------------------------------------------------------------------------ model
enum CellType { CELL_CONV, CELL_FC, CELL_POOL, CELL_SUM, CELL_SCALING };
enum Engine { ENG_TCGEN05, ENG_SIMT, ENG_DEPTHWISE, ENG_POOL, ENG_SUM, ENG_FUSED, ENG_STEM, ENG_PATCH, ENG_STEM_S2D };

struct TensorRec {
    int C = 0, H = 0, W = 0;
    int dtype = DT_I8;
    int is_unsigned = 0;
    int producer = -1;
    int buffer = -1;      // index into Net::buffers, -1 for the network input
    bool readable = true;
    size_t elems() const { return (size_t)C * H * W; }
    size_t bytes_per_image() const { return elems() * (dtype == DT_I32 ? 4 : 1); }
};

struct QuantHost {
    int mode = SC_NONE, act = ACT_LINEAR, out_bits = 8, out_unsigned = 0, sat_thr = 0;
    int is_clipped = 0;
    int nb_channels = 0;
    std::vector<int32_t> bias, p0, p1, clip_thr, clip_val;
    std::vector<float> fscale, clip_f;
    bool has_bias = false;
    // device copy
    void* d_blob = nullptr;
    QuantDev dev{};
};

struct CellRec {
    CellType type;
    std::vector<int> inputs;
    int output = -1;
    n2d2b_conv_desc conv{};
    n2d2b_pool_desc pool{};
    ConvGeom geom{};
    PoolGeom pgeom{};
    QuantHost q;
    std::vector<int8_t> weights;  // host copy, OHWI int8 (int4 already widened)
    int wbits = 8;                // storage width the caller gave the weights in (8 or 4)
    int8_t* d_weights = nullptr;
    size_t d_weight_bytes = 0;    // bytes of weights this cell keeps in HBM
    Engine engine = ENG_SIMT;
    // fused residual sum
    int residual = -1;
    QuantHost q2;
    bool has_q2 = false;
    bool skipped = false;  // folded into another cell
    // 32-bit epilogue constants (tensor-core cells)
    FastQuant fast{};
    int* d_fast = nullptr;
    // a max pooling folded into the first-layer kernel (the cell's output then is the pooled tensor)
    bool pool_fused = false;
    PoolGeom fused_pool{};
    // first-layer tensor-core kernels
    StemPlan stem{};
    StemS2dPlan stem2{};
    void* d_pad4 = nullptr;   // input re-laid with 4 bytes per pixel and its zero padding written out
    // A cell whose output channels are not a multiple of 32 (a 1000-class classifier) cannot leave through the TMA
    // store of the 32-bit epilogue (rows of its output are not 16-byte multiples).  It runs with zero weight rows
    // appended up to pad_O channels into d_colpad ([pixels][pad_O]); a copy kernel then drops the padding.
    int pad_O = 0;
    void* d_colpad = nullptr;
    // stride-1 convolution from a shared-memory patch
    PatchPlan patch{};
    // tensor-core plan
    IgemmPlan plan{};
    bool has_plan = false;
    const void* plan_input = nullptr;
};

struct n2d2b_net {
    int device = 0;
    int num_sms = 148;
    bool finalized = false;
    int max_batch = 0;
    unsigned flags = 0;
    std::vector<TensorRec> tensors;
    std::vector<CellRec> cells;
    std::vector<void*> buffers;
    std::vector<size_t> buffer_bytes;
    int* d_status = nullptr;
    int launches = 0;
    const void* last_input = nullptr;
    void* d_labels_scratch = nullptr;   // device labels / scores of the host-buffer top-N entry point
    size_t labels_scratch_bytes = 0;
    void* d_stage_in = nullptr;   // device staging of the host-buffer entry point
    void* d_stage_out = nullptr;
    // host-buffer entry point: the upload is cut into slices on its own stream so that the leading
    // cells (which need no tensor map and work slice by slice) run while later slices still arrive
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t slice_ready[8] = {nullptr};
    cudaEvent_t stage_free = nullptr;
    int head_cells = 0;
    int head_limit = 0;      // cells [0, head_limit) may run slice by slice: the buffer planner keeps their tensors apart
    int forced_slices = 0;   // n2d2b_net_set_slices: 0 = automatic
    // streaming host-buffer entry points (submit / wait): two staging sets, so that the upload of one batch runs
    // under the forward pass of the batch before it
    void* d_pipe_in[2] = {nullptr, nullptr};
    void* d_pipe_out[2] = {nullptr, nullptr};
    cudaEvent_t pipe_uploaded[2] = {nullptr, nullptr};
    cudaEvent_t pipe_computed[2] = {nullptr, nullptr};
    cudaEvent_t pipe_done[2] = {nullptr, nullptr};
    cudaStream_t download_stream = nullptr;
    bool pipe_busy[2] = {false, false};
    cudaStream_t pipe_stream[2] = {nullptr, nullptr};   // the stream each slot's work was queued on
    unsigned pipe_next = 0;
};

static int validate_quant(const n2d2b_quant* qu, int channels, bool accumulators_have_bias, QuantHost& q,
                          const int32_t* bias)
{
    if (!qu) return fail(N2D2B_ERR_INVALID, "quant must not be NULL");
    const n2d2b_scaling& s = qu->scaling;
    q.mode = s.mode;
    q.act = qu->activation;
    q.out_bits = qu->out_bits;
    q.out_unsigned = qu->out_unsigned ? 1 : 0;
    q.sat_thr = qu->saturation_threshold;
    q.is_clipped = s.is_clipped ? 1 : 0;
    q.nb_channels = channels;
    if (q.mode < SC_NONE || q.mode > SC_DOUBLE_SHIFT) return fail(N2D2B_ERR_INVALID, "unknown scaling mode %d", q.mode);
    if (q.act < ACT_LINEAR || q.act > ACT_SATURATION) return fail(N2D2B_ERR_INVALID, "unknown activation %d", q.act);
    if (q.act == ACT_SATURATION && q.sat_thr < 0)
        return fail(N2D2B_ERR_INVALID, "saturation_threshold must not be negative (got %d)", q.sat_thr);
    if (q.mode != SC_NONE) {
        if (s.nb_channels != channels)
            return fail(N2D2B_ERR_INVALID, "scaling has %d channels, the cell has %d outputs", s.nb_channels, channels);
        // the integer modes throw on a non-quantized cell in the reference; a float-mode cell with
        // nbBits == 0 would produce fractional values, which this integer path cannot carry
        if (q.out_bits < 1 || q.out_bits > 8)
            return fail(N2D2B_ERR_INVALID, "out_bits must be in 1..8 (got %d)", q.out_bits);
    }
    q.p0.assign(channels, 0);
    q.p1.assign(channels, 0);
    q.fscale.assign(channels, 1.0f);
    q.clip_thr.assign(channels, 0);
    q.clip_val.assign(channels, 0);
    q.clip_f.assign(channels, 0.0f);
    switch (q.mode) {
    case SC_FLOAT_MULT:
        if (!s.fscale) return fail(N2D2B_ERR_INVALID, "FLOAT_MULT scaling needs fscale");
        for (int c = 0; c < channels; ++c) q.fscale[c] = s.fscale[c];
        break;
    case SC_FIXED_MULT16:
    case SC_FIXED_MULT32:
        if (!s.mult) return fail(N2D2B_ERR_INVALID, "FIXED_MULT scaling needs mult");
        for (int c = 0; c < channels; ++c) {
            const int f = s.frac_bits_per_channel ? s.frac_bits_per_channel[c] : s.frac_bits;
            if (f < 0 || f > 62) return fail(N2D2B_ERR_INVALID, "fractional bits %d out of range", f);
            q.p0[c] = s.mult[c];
            q.p1[c] = f;
        }
        break;
    case SC_SINGLE_SHIFT:
        if (!s.shift0) return fail(N2D2B_ERR_INVALID, "SINGLE_SHIFT scaling needs shift0");
        for (int c = 0; c < channels; ++c) {
            if (s.shift0[c] > 62) return fail(N2D2B_ERR_INVALID, "shift %d out of range", s.shift0[c]);
            q.p0[c] = s.shift0[c];
        }
        break;
    case SC_DOUBLE_SHIFT:
        if (!s.shift0 || !s.shift1) return fail(N2D2B_ERR_INVALID, "DOUBLE_SHIFT scaling needs shift0 and shift1");
        for (int c = 0; c < channels; ++c) {
            if (s.shift0[c] > 30 || s.shift1[c] > 62) return fail(N2D2B_ERR_INVALID, "shift pair out of range");
            q.p0[c] = s.shift0[c];
            q.p1[c] = s.shift1[c];
        }
        break;
    default:
        break;
    }
    // clipping only acts in the FLOAT and FIXED modes (CPU path of the reference)
    if (q.is_clipped && (q.mode == SC_FLOAT_MULT || q.mode == SC_FIXED_MULT16 || q.mode == SC_FIXED_MULT32)) {
        if (!s.clip) return fail(N2D2B_ERR_INVALID, "is_clipped needs clip values");
        for (int c = 0; c < channels; ++c) {
            const float cl = s.clip[c];
            if (!std::isfinite(cl)) return fail(N2D2B_ERR_INVALID, "clip[%d] is not finite", c);
            q.clip_f[c] = cl;
            q.clip_thr[c] = (int32_t)(cl > 0.0f ? std::floor(cl) : std::ceil(cl));
            q.clip_val[c] = (int32_t)std::round(cl);
        }
    } else {
        q.is_clipped = 0;
    }
    q.has_bias = accumulators_have_bias && bias != nullptr;
    q.bias.assign(channels, 0);
    if (q.has_bias)
        for (int c = 0; c < channels; ++c) q.bias[c] = bias[c];
    return 0;
}

static void quant_output_type(const QuantHost& q, int* dtype, int* is_unsigned)
{
    if (q.mode == SC_NONE) {
        *dtype = DT_I32;
        *is_unsigned = 0;
    } else {
        *dtype = DT_I8;
        *is_unsigned = q.out_unsigned;
    }
}

static int upload_quant(QuantHost& q)
{
    const int C = q.nb_channels;
    const size_t words = (size_t)C * 7;
    std::vector<int32_t> blob(words);
    memcpy(&blob[0 * C], q.bias.data(), C * 4);
    memcpy(&blob[1 * C], q.p0.data(), C * 4);
    memcpy(&blob[2 * C], q.p1.data(), C * 4);
    memcpy(&blob[3 * C], q.fscale.data(), C * 4);
    memcpy(&blob[4 * C], q.clip_thr.data(), C * 4);
    memcpy(&blob[5 * C], q.clip_val.data(), C * 4);
    memcpy(&blob[6 * C], q.clip_f.data(), C * 4);
    CUDA_TRY(cudaMalloc(&q.d_blob, words * 4 + 16));
    CUDA_TRY(cudaMemcpy(q.d_blob, blob.data(), words * 4, cudaMemcpyHostToDevice));
    int32_t* d = (int32_t*)q.d_blob;
    QuantDev& v = q.dev;
    v.mode = q.mode;
    v.act = q.act;
    v.saturate = (q.mode != SC_NONE) ? 1 : 0;
    if (q.out_unsigned) { v.out_lo = 0; v.out_hi = (1 << q.out_bits) - 1; }
    else { v.out_lo = -(1 << (q.out_bits - 1)); v.out_hi = (1 << (q.out_bits - 1)) - 1; }
    v.is_clipped = q.is_clipped;
    v.sat_thr = q.sat_thr;
    v.bias = q.has_bias ? d + 0 * C : nullptr;
    v.p0 = d + 1 * C;
    v.p1 = d + 2 * C;
    v.fscale = (const float*)(d + 3 * C);
    v.clip_thr = d + 4 * C;
    v.clip_val = d + 5 * C;
    v.clip_f = (const float*)(d + 6 * C);
    return 0;
}

// ---- 32-bit epilogue constants ----------------------------------------------------------------
// For the shift and fixed-point modes the rescale of channel c is f(x) = (x * m + half) >> s with
// m >= 0, a non-decreasing function of x.  Saturating f(x) to [out_lo, out_hi] (and a ReLU) equals
// evaluating f on x clamped to [L, H], where H is the smallest x with f(x) >= out_hi and L the
// largest x with f(x) <= out_lo: the clamp bounds every product, so 32-bit arithmetic is exact.
// Clipping to [0, clip] before the rescale tightens the same clamp, and the bias is folded in:
//   y = (clamp(acc, L - b, H - b) * m + (b * m + half)) >> s.
// Returns false when some intermediate could leave 32 bits or the configuration is outside this
// form (float mode, negative multipliers, clip <= 0, out_bits != 8); the
// exact 64-bit epilogue is used then.
static long long ceil_div(long long a, long long b)  // b > 0
{
    return (a >= 0) ? (a + b - 1) / b : -((-a) / b);
}

// 64-bit form of the same rescale, for fixed-point scalings whose products leave 32 bits: no clamps (the final
// pack saturates), so it applies when none is needed for other reasons; the shifted result must fit 32 bits.
static bool build_wide_quant(const QuantHost& q, int cpad, long long x_bound, std::vector<int32_t>& out)
{
    if (q.is_clipped || (q.act == ACT_RECTIFIER && !q.out_unsigned) || q.act == ACT_SATURATION) return false;
    const int C = q.nb_channels;
    out.assign((size_t)5 * cpad, 0);
    for (int c = 0; c < C; ++c) {
        long long m, s;
        if (q.mode == SC_SINGLE_SHIFT) { m = 1; s = q.p0[c]; }
        else if (q.mode == SC_DOUBLE_SHIFT) { m = 1 + (1ll << q.p0[c]); s = q.p1[c]; }
        else { m = q.p0[c]; s = q.p1[c]; }
        if (m < 0 || m > (1ll << 30) || s > 31) return false;
        const long long half = s > 0 ? (1ll << (s - 1)) : 0;
        const long long b = q.has_bias ? q.bias[c] : 0;
        if (std::llabs(b) > (1ll << 30)) return false;   // keeps every 64-bit intermediate below 2^61
        const long long add = b * m + half;                                   // < 2^62
        const long long worst = x_bound * m + std::llabs(add);               // < 2^62 for x_bound < 2^30
        if ((worst >> s) > (1ll << 31) - 2) return false;
        out[(size_t)0 * cpad + c] = (int32_t)(add >> 32);
        out[(size_t)2 * cpad + c] = (int32_t)m;
        out[(size_t)3 * cpad + c] = (int32_t)(uint32_t)(add & 0xffffffffll);
        out[(size_t)4 * cpad + c] = (int32_t)s;
    }
    return true;
}

static bool build_fast_quant(const QuantHost& q, int cpad, long long x_bound, std::vector<int32_t>& out, int* eff_lo,
                             int* eff_hi, bool* need_clamp)
{
    if (q.mode != SC_SINGLE_SHIFT && q.mode != SC_DOUBLE_SHIFT && q.mode != SC_FIXED_MULT16 && q.mode != SC_FIXED_MULT32)
        return false;
    if (q.out_bits != 8) return false;
    const int C = q.nb_channels;
    long long out_hi = q.out_unsigned ? 255 : 127;
    long long out_lo = q.out_unsigned ? 0 : -128;
    if (q.act == ACT_RECTIFIER && out_lo < 0) out_lo = 0;
    if (q.act == ACT_SATURATION) {
        // saturate to the output range, then clamp to +-threshold: one clamp to the intersection
        out_hi = std::min(out_hi, (long long)q.sat_thr);
        out_lo = std::max(out_lo, -(long long)q.sat_thr);
        *need_clamp = true;
    }
    *eff_lo = (int)out_lo;
    *eff_hi = (int)out_hi;
    out.assign((size_t)5 * cpad, 0);
    const long long LIM = (1ll << 31) - 1;
    // without the clamps the final 8-bit pack does the saturation (and, for unsigned outputs, the ReLU)
    if (q.is_clipped || (q.act == ACT_RECTIFIER && !q.out_unsigned)) *need_clamp = true;
    for (int c = 0; c < C; ++c) {
        long long m, s;
        if (q.mode == SC_SINGLE_SHIFT) { m = 1; s = q.p0[c]; }
        else if (q.mode == SC_DOUBLE_SHIFT) { m = 1 + (1ll << q.p0[c]); s = q.p1[c]; }
        else { m = q.p0[c]; s = q.p1[c]; }
        if (m < 0 || s > 30) return false;
        const long long half = s > 0 ? (1ll << (s - 1)) : 0;
        long long L = 0, H = 0;
        if (m > 0) {
            H = ceil_div((out_hi << s) - half, m);
            L = ceil_div(((out_lo + 1) << s) - half, m) - 1;
        }
        if (q.is_clipped) {
            if (!(q.clip_f[c] > 0.0f)) return false;
            L = std::max(L, 0ll);
            H = std::min(H, (long long)q.clip_val[c]);
        }
        if (H < L) L = H;   // everything saturates to the same value
        const long long b = q.has_bias ? q.bias[c] : 0;
        long long lo = L - b, hi = H - b;
        const long long add = b * m + half;
        // |x| never exceeds x_bound, so clamp bounds beyond it are equivalent to it (min(max(x, lo), hi)
        // with lo > hi yields hi, which is then on the saturating side as well)
        lo = std::max(lo, -x_bound);
        hi = std::min(hi, x_bound);
        const long long p0 = lo * m + add, p1 = hi * m + add;
        if (std::llabs(add) > LIM || std::llabs(p0) > LIM || std::llabs(p1) > LIM) return false;
        if (x_bound * m + std::llabs(add) > LIM) *need_clamp = true;   // an unclamped product could overflow
        out[(size_t)0 * cpad + c] = (int32_t)lo;
        out[(size_t)1 * cpad + c] = (int32_t)hi;
        out[(size_t)2 * cpad + c] = (int32_t)m;
        out[(size_t)3 * cpad + c] = (int32_t)add;
        out[(size_t)4 * cpad + c] = (int32_t)s;
    }
    return true;
}

// w4: the cell's weights are 4-bit values (|w| <= 8), which tightens the accumulator bound
static int upload_fast(CellRec& c, const TensorRec& tout, bool residual_dtype_i8 = false, int residual_unsigned = 0,
                       bool w4 = false)
{
    c.fast = FastQuant{};
    if (tout.dtype != DT_I8) return 0;
    const int C = c.q.nb_channels;
    const int cpad = ((C + 255) / 256) * 256;
    std::vector<int32_t> f1, f2;
    int lo1, hi1, lo2 = 0, hi2 = 0;
    // |accumulator| <= K * 255 * 128 (4-bit weights: K * 255 * 8; they enter the tensor core times 16 and the
    // epilogue divides the sum by 16 again before anything else); the residual stage adds two 8-bit values
    const long long acc_bound = (long long)c.geom.kH * c.geom.kW * c.geom.Cg * 255ll * (w4 ? 8ll : 128ll);
    if (acc_bound * (w4 ? 16 : 1) > (1ll << 30)) return 0;
    bool need_clamp = false, wide = false;
    if (!build_fast_quant(c.q, cpad, acc_bound, f1, &lo1, &hi1, &need_clamp)) {
        // eff range etc. were set before the failing channel; retry in 64 bits
        need_clamp = false;
        if (c.q.out_bits != 8 || c.q.act == ACT_SATURATION
            || (c.q.mode != SC_SINGLE_SHIFT && c.q.mode != SC_DOUBLE_SHIFT && c.q.mode != SC_FIXED_MULT16
                && c.q.mode != SC_FIXED_MULT32)
            || !build_wide_quant(c.q, cpad, acc_bound, f1))
            return 0;
        wide = true;
        lo1 = c.q.out_unsigned ? 0 : -128;
        hi1 = c.q.out_unsigned ? 255 : 127;
        if (c.q.act == ACT_RECTIFIER && lo1 < 0) lo1 = 0;
    }
    bool with_res = c.residual >= 0;
    if (with_res && !build_fast_quant(c.q2, cpad, 512, f2, &lo2, &hi2, &need_clamp)) return 0;
    if (wide && need_clamp) return 0;   // the 64-bit form has no clamps
    // Dot-product form of the residual stage (see perm_block): every multiplier of the sum's scaling fits a byte,
    // both operands have a native 8-bit range and no clamp is needed.  The four bytes [t, t', r, r'] of a dot
    // product share one signedness: when the cell's own output is signed and the residual unsigned, the first
    // rescale produces t + 128 instead (its addend grows by 128 << shift, a multiple of 2^shift, so the shifted
    // value is exactly 128 larger and the unsigned saturating pack clamps at the same places) and the second
    // addend drops 128 * m2.
    bool dp4a = false, dp_t_unsigned = false;
    unsigned dp_xor = 0;
    int dp_a_signed = 1;
    if (with_res && !need_clamp && !wide && residual_dtype_i8) {
        const bool t_uns = (lo1 == 0 && hi1 == 255), t_sig = (lo1 == -128 && hi1 == 127);
        const bool r_uns = residual_unsigned != 0;
        bool ok = t_uns || t_sig;
        for (int ch = 0; ch < C; ++ch) ok = ok && f2[(size_t)2 * cpad + ch] >= 0 && f2[(size_t)2 * cpad + ch] <= 255;
        if (ok && t_uns && !r_uns) ok = false;   // unsigned output with a signed residual: the exact two-step form
        const bool shift_t = ok && t_sig && r_uns;
        if (shift_t) {
            const long long LIM = (1ll << 31) - 1;
            for (int ch = 0; ch < C && ok; ++ch) {
                const long long m = f1[(size_t)2 * cpad + ch], add = f1[(size_t)3 * cpad + ch], sh = f1[(size_t)4 * cpad + ch];
                const long long nadd = add + (128ll << sh);
                if (acc_bound * m + std::llabs(nadd) > LIM) ok = false;
            }
        }
        if (ok) {
            dp4a = true;
            dp_t_unsigned = t_uns || shift_t;
            dp_a_signed = dp_t_unsigned ? 0 : 1;
            for (int ch = 0; ch < cpad; ++ch) {
                const long long m2 = f2[(size_t)2 * cpad + ch];
                // row 0 of the residual set: the multiplier in the byte lanes of this column (even column:
                // lanes 0 and 2 = t and r; odd column: lanes 1 and 3)
                f2[(size_t)0 * cpad + ch] = (int32_t)((ch & 1) ? (m2 << 8 | m2 << 24) : (m2 | m2 << 16));
                if (shift_t) {
                    f1[(size_t)3 * cpad + ch] += (int32_t)(128ll << f1[(size_t)4 * cpad + ch]);
                    f2[(size_t)3 * cpad + ch] -= (int32_t)(128 * m2);
                }
            }
        }
    }
    const size_t words = f1.size() + f2.size();
    CUDA_TRY(cudaMalloc((void**)&c.d_fast, words * 4 + 16));
    CUDA_TRY(cudaMemcpy(c.d_fast, f1.data(), f1.size() * 4, cudaMemcpyHostToDevice));
    if (with_res) CUDA_TRY(cudaMemcpy(c.d_fast + f1.size(), f2.data(), f2.size() * 4, cudaMemcpyHostToDevice));
    c.fast.fq = c.d_fast;
    c.fast.fq2 = with_res ? c.d_fast + f1.size() : nullptr;
    c.fast.cpad = cpad;
    c.fast.t_lo = lo1;
    c.fast.t_hi = hi1;
    c.fast.out_unsigned = with_res ? c.q2.out_unsigned : c.q.out_unsigned;
    c.fast.need_clamp = need_clamp;
    c.fast.wide = wide;
    c.fast.dp4a = dp4a;
    c.fast.dp_t_unsigned = dp_t_unsigned;
    c.fast.dp_xor = dp_xor;
    c.fast.dp_a_signed = dp_a_signed;
    c.fast.enabled = true;
    return 0;
}

static void unpack_weights(const void* src, int weight_bits, size_t rows, size_t row_elems, std::vector<int8_t>& dst)
{
    dst.resize(rows * row_elems);
    if (weight_bits == 8) {
        memcpy(dst.data(), src, rows * row_elems);
        return;
    }
    // Packed sub-byte weights as the reference's export stores them (data<N>, export/CPP_Quantization/include/
    // typedefs.hpp:359-517): 8 / N values per byte, the first one in the highest bits, every row starting on a byte;
    // two's complement in N bits, except N = 1 where the bit 0 stands for -1 and 1 for +1.
    const size_t per_byte = 8 / (size_t)weight_bits;
    const size_t row_bytes = (row_elems + per_byte - 1) / per_byte;
    const int mask = (1 << weight_bits) - 1, sign = 1 << (weight_bits - 1);
    const uint8_t* p = (const uint8_t*)src;
    for (size_t r = 0; r < rows; ++r)
        for (size_t i = 0; i < row_elems; ++i) {
            const uint8_t byte = p[r * row_bytes + i / per_byte];
            const int shift = 8 - weight_bits * (int)(i % per_byte + 1);
            int v = (byte >> shift) & mask;
            if (weight_bits == 1) v = v ? 1 : -1;
            else if (v & sign) v -= 1 << weight_bits;
            dst[r * row_elems + i] = (int8_t)v;
        }
}

// ---- helpers exported to the other translation units (host_internal.h) -------------------------
namespace n2d2b {
int set_error(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int prepare_fast_constants(const n2d2b_quant* quant, int channels, const int32_t* bias, long long acc_bound,
                           std::vector<int32_t>& consts, int* cpad, int* out_unsigned, bool* need_clamp)
{
    QuantHost q;
    if (int rc = validate_quant(quant, channels, true, q, bias)) return rc;
    *cpad = ((channels + 255) / 256) * 256;
    int lo = 0, hi = 0;
    *need_clamp = false;
    if (q.mode == SC_NONE || !build_fast_quant(q, *cpad, acc_bound, consts, &lo, &hi, need_clamp)) return 1;
    *out_unsigned = q.out_unsigned;
    return 0;
}
}  // namespace n2d2b

// One CTA waits, with the given limit, on a barrier that nobody ever arrives at: the bounded wait of the
// tensor-core kernels running out, on purpose and harmlessly (no fault, no trap; the kernel returns).
__global__ void wait_timeout_selftest_kernel(int* status, unsigned long long limit_ns)
{
    __shared__ unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) mbar_wait_for(smem_u32(&bar), 0, &abort_flag, status, 9, limit_ns);
    __syncthreads();
}

// ------------------------------------------------------------------------------------ C ABI
extern "C" {

const char* n2d2b_last_error(void) { return g_err; }
int n2d2b_version(void) { return 100; }

int n2d2b_device_count(void)
{
    int n = 0;
    CUDA_TRY(cudaGetDeviceCount(&n));
    return n;
}

int n2d2b_net_create(int device, n2d2b_net** net)
{
    if (!net) return fail(N2D2B_ERR_INVALID, "net must not be NULL");
    *net = nullptr;
    int n = 0;
    CUDA_TRY(cudaGetDeviceCount(&n));
    if (device < 0 || device >= n) return fail(N2D2B_ERR_INVALID, "device %d out of range (%d devices)", device, n);
    CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(N2D2B_ERR_INVALID, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major,
                    prop.minor);
    n2d2b_net* p = new n2d2b_net();
    p->device = device;
    p->num_sms = prop.multiProcessorCount;
    *net = p;
    return 0;
}

void n2d2b_net_destroy(n2d2b_net* net)
{
    if (!net) return;
    cudaSetDevice(net->device);
    for (void* b : net->buffers) cudaFree(b);
    for (CellRec& c : net->cells) {
        cudaFree(c.d_weights);
        cudaFree(c.q.d_blob);
        cudaFree(c.q2.d_blob);
        cudaFree(c.d_fast);
        cudaFree(c.d_pad4);
        cudaFree(c.d_colpad);
    }
    cudaFree(net->d_status);
    cudaFree(net->d_labels_scratch);
    cudaFree(net->d_stage_in);
    cudaFree(net->d_stage_out);
    if (net->copy_stream) cudaStreamDestroy(net->copy_stream);
    for (cudaEvent_t e : net->slice_ready)
        if (e) cudaEventDestroy(e);
    if (net->stage_free) cudaEventDestroy(net->stage_free);
    for (int k = 0; k < 2; ++k) {
        cudaFree(net->d_pipe_in[k]);
        cudaFree(net->d_pipe_out[k]);
        if (net->pipe_uploaded[k]) cudaEventDestroy(net->pipe_uploaded[k]);
        if (net->pipe_computed[k]) cudaEventDestroy(net->pipe_computed[k]);
        if (net->pipe_done[k]) cudaEventDestroy(net->pipe_done[k]);
    }
    if (net->download_stream) cudaStreamDestroy(net->download_stream);
    delete net;
}

int n2d2b_net_set_input(n2d2b_net* net, int channels, int height, int width, int is_unsigned, int* tensor_id)
{
    if (!net) return fail(N2D2B_ERR_INVALID, "net must not be NULL");
    if (net->finalized || !net->tensors.empty()) return fail(N2D2B_ERR_STATE, "input already set");
    if (channels < 1 || height < 1 || width < 1) return fail(N2D2B_ERR_INVALID, "input dimensions must be positive");
    TensorRec t;
    t.C = channels; t.H = height; t.W = width; t.dtype = DT_I8; t.is_unsigned = is_unsigned ? 1 : 0;
    net->tensors.push_back(t);
    if (tensor_id) *tensor_id = 0;
    return 0;
}

static int check_tensor(const n2d2b_net* net, int id)
{
    if (!net) return fail(N2D2B_ERR_INVALID, "net must not be NULL");
    if (net->finalized) return fail(N2D2B_ERR_STATE, "the network is already finalized");
    if (id < 0 || id >= (int)net->tensors.size()) return fail(N2D2B_ERR_INVALID, "unknown tensor id %d", id);
    return 0;
}

static int conv_out(int in, int k, int stride, int pad0, int pad1, int dil)
{
    // ConvCell_Frame_Kernels.cpp:37-45
    return (int)((in + pad0 + pad1 - dil * (k - 1) - 1 + stride) / (double)stride);
}

int n2d2b_net_add_conv(n2d2b_net* net, const n2d2b_conv_desc* d, const void* weights, const int32_t* bias,
                       const n2d2b_quant* quant, int* tensor_id)
{
    if (!d || !weights) return fail(N2D2B_ERR_INVALID, "desc and weights must not be NULL");
    if (int rc = check_tensor(net, d->input)) return rc;
    const TensorRec in = net->tensors[d->input];
    if (in.dtype != DT_I8) return fail(N2D2B_ERR_INVALID, "a convolution needs an 8-bit input tensor");
    if (d->nb_outputs < 1 || d->kernel_h < 1 || d->kernel_w < 1 || d->stride_y < 1 || d->stride_x < 1
        || d->dilation_y < 1 || d->dilation_x < 1 || d->groups < 1 || d->pad_top < 0 || d->pad_left < 0
        || d->pad_bottom < 0 || d->pad_right < 0)
        return fail(N2D2B_ERR_INVALID, "invalid convolution geometry");
    if (in.C % d->groups || d->nb_outputs % d->groups)
        return fail(N2D2B_ERR_INVALID, "groups (%d) must divide channels (%d) and outputs (%d)", d->groups, in.C,
                    d->nb_outputs);
    if (d->weight_bits != 8 && d->weight_bits != 4 && d->weight_bits != 2 && d->weight_bits != 1)
        return fail(N2D2B_ERR_INVALID, "weight_bits must be 8, 4, 2 or 1");
    CellRec c;
    c.type = CELL_CONV;
    c.inputs = {d->input};
    c.conv = *d;
    ConvGeom& g = c.geom;
    g.H = in.H; g.W = in.W; g.C = in.C;
    g.O = d->nb_outputs;
    g.kH = d->kernel_h; g.kW = d->kernel_w; g.sY = d->stride_y; g.sX = d->stride_x;
    g.pT = d->pad_top; g.pL = d->pad_left; g.dY = d->dilation_y; g.dX = d->dilation_x;
    g.groups = d->groups; g.Cg = in.C / d->groups; g.Og = d->nb_outputs / d->groups;
    g.oH = conv_out(in.H, g.kH, g.sY, d->pad_top, d->pad_bottom, g.dY);
    g.oW = conv_out(in.W, g.kW, g.sX, d->pad_left, d->pad_right, g.dX);
    if (g.oH < 1 || g.oW < 1) return fail(N2D2B_ERR_INVALID, "convolution output would be empty");
    if (int rc = validate_quant(quant, g.O, true, c.q, bias)) return rc;
    unpack_weights(weights, d->weight_bits, (size_t)g.O, (size_t)g.kH * g.kW * g.Cg, c.weights);
    c.wbits = d->weight_bits;
    TensorRec t;
    t.C = g.O; t.H = g.oH; t.W = g.oW;
    quant_output_type(c.q, &t.dtype, &t.is_unsigned);
    t.producer = (int)net->cells.size();
    c.output = (int)net->tensors.size();
    net->tensors.push_back(t);
    net->cells.push_back(std::move(c));
    if (tensor_id) *tensor_id = net->cells.back().output;
    return 0;
}

int n2d2b_net_add_fc(n2d2b_net* net, int input, int nb_outputs, int weight_bits, const void* weights,
                     const int32_t* bias, const n2d2b_quant* quant, int* tensor_id)
{
    if (!weights) return fail(N2D2B_ERR_INVALID, "weights must not be NULL");
    if (int rc = check_tensor(net, input)) return rc;
    const TensorRec in = net->tensors[input];
    if (in.dtype != DT_I8) return fail(N2D2B_ERR_INVALID, "a fully-connected cell needs an 8-bit input tensor");
    if (nb_outputs < 1) return fail(N2D2B_ERR_INVALID, "nb_outputs must be positive");
    if (weight_bits != 8 && weight_bits != 4 && weight_bits != 2 && weight_bits != 1)
        return fail(N2D2B_ERR_INVALID, "weight_bits must be 8, 4, 2 or 1");
    CellRec c;
    c.type = CELL_FC;
    c.inputs = {input};
    // a fully-connected cell is a 1x1 convolution over the flattened input
    ConvGeom& g = c.geom;
    g.H = 1; g.W = 1; g.C = (int)in.elems();
    g.O = nb_outputs; g.kH = g.kW = 1; g.sY = g.sX = 1; g.pT = g.pL = 0; g.dY = g.dX = 1;
    g.groups = 1; g.Cg = g.C; g.Og = g.O; g.oH = g.oW = 1;
    if (int rc = validate_quant(quant, g.O, true, c.q, bias)) return rc;
    unpack_weights(weights, weight_bits, (size_t)g.O, (size_t)g.C, c.weights);
    c.wbits = weight_bits;
    TensorRec t;
    t.C = g.O; t.H = 1; t.W = 1;
    quant_output_type(c.q, &t.dtype, &t.is_unsigned);
    t.producer = (int)net->cells.size();
    c.output = (int)net->tensors.size();
    net->tensors.push_back(t);
    net->cells.push_back(std::move(c));
    if (tensor_id) *tensor_id = net->cells.back().output;
    return 0;
}

int n2d2b_net_add_pool(n2d2b_net* net, const n2d2b_pool_desc* d, int* tensor_id)
{
    if (!d) return fail(N2D2B_ERR_INVALID, "desc must not be NULL");
    if (int rc = check_tensor(net, d->input)) return rc;
    const TensorRec in = net->tensors[d->input];
    if (d->pool_h < 1 || d->pool_w < 1 || d->stride_y < 1 || d->stride_x < 1 || d->pad_y < 0 || d->pad_x < 0
        || (d->pooling != N2D2B_POOL_MAX && d->pooling != N2D2B_POOL_AVERAGE))
        return fail(N2D2B_ERR_INVALID, "invalid pooling geometry");
    CellRec c;
    c.type = CELL_POOL;
    c.inputs = {d->input};
    c.pool = *d;
    PoolGeom& g = c.pgeom;
    g.H = in.H; g.W = in.W; g.C = in.C;
    g.pH = d->pool_h; g.pW = d->pool_w; g.sY = d->stride_y; g.sX = d->stride_x; g.padY = d->pad_y; g.padX = d->pad_x;
    g.is_max = (d->pooling == N2D2B_POOL_MAX);
    // PoolCell.cpp:233-239
    g.oH = (int)((in.H + 2 * d->pad_y - d->pool_h + d->stride_y) / (double)d->stride_y);
    g.oW = (int)((in.W + 2 * d->pad_x - d->pool_w + d->stride_x) / (double)d->stride_x);
    if (g.oH < 1 || g.oW < 1) return fail(N2D2B_ERR_INVALID, "pooling output would be empty");
    TensorRec t;
    t.C = in.C; t.H = g.oH; t.W = g.oW; t.dtype = in.dtype; t.is_unsigned = in.is_unsigned;
    t.producer = (int)net->cells.size();
    c.output = (int)net->tensors.size();
    net->tensors.push_back(t);
    net->cells.push_back(std::move(c));
    if (tensor_id) *tensor_id = net->cells.back().output;
    return 0;
}

int n2d2b_net_add_elemwise_sum(n2d2b_net* net, const int* inputs, int nb_inputs, const n2d2b_quant* quant,
                               int* tensor_id)
{
    if (!inputs || nb_inputs < 1 || nb_inputs > 4)
        return fail(N2D2B_ERR_INVALID, "an element-wise sum takes 1 to 4 inputs");
    for (int k = 0; k < nb_inputs; ++k)
        if (int rc = check_tensor(net, inputs[k])) return rc;
    const TensorRec a = net->tensors[inputs[0]];
    for (int k = 1; k < nb_inputs; ++k) {
        const TensorRec& b = net->tensors[inputs[k]];
        if (b.C != a.C || b.H != a.H || b.W != a.W)
            return fail(N2D2B_ERR_INVALID, "element-wise inputs differ in shape");
    }
    CellRec c;
    c.type = CELL_SUM;
    c.inputs.assign(inputs, inputs + nb_inputs);
    if (int rc = validate_quant(quant, a.C, false, c.q, nullptr)) return rc;
    TensorRec t;
    t.C = a.C; t.H = a.H; t.W = a.W;
    quant_output_type(c.q, &t.dtype, &t.is_unsigned);
    t.producer = (int)net->cells.size();
    c.output = (int)net->tensors.size();
    net->tensors.push_back(t);
    net->cells.push_back(std::move(c));
    if (tensor_id) *tensor_id = net->cells.back().output;
    return 0;
}

int n2d2b_net_add_scaling(n2d2b_net* net, int input, const n2d2b_quant* quant, int* tensor_id)
{
    const int ids[1] = {input};
    int rc = n2d2b_net_add_elemwise_sum(net, ids, 1, quant, tensor_id);
    if (rc == 0) net->cells.back().type = CELL_SCALING;
    return rc;
}

// ---- finalize -------------------------------------------------------------------------------
static void fuse_residuals(n2d2b_net* net)
{
    const int nc = (int)net->cells.size();
    std::vector<int> consumers(net->tensors.size(), 0);
    for (const CellRec& c : net->cells)
        for (int i : c.inputs) consumers[i]++;
    for (int si = 0; si < nc; ++si) {
        CellRec& s = net->cells[si];
        if (s.type != CELL_SUM || s.inputs.size() != 2) continue;
        if (s.q.mode == SC_NONE) continue;
        int best = -1;
        for (int k = 0; k < 2; ++k) {
            const int t = s.inputs[k], other = s.inputs[1 - k];
            const TensorRec& tt = net->tensors[t];
            const TensorRec& ot = net->tensors[other];
            if (tt.producer < 0 || consumers[t] != 1) continue;
            CellRec& p = net->cells[tt.producer];
            if (p.type != CELL_CONV || p.geom.groups != 1 || p.residual >= 0 || p.skipped) continue;
            if (tt.dtype != DT_I8 || ot.dtype != DT_I8) continue;
            if (ot.producer >= tt.producer) continue;  // the other operand must exist when p runs
            if (best < 0 || tt.producer > net->tensors[s.inputs[best]].producer) best = k;
        }
        if (best < 0) continue;
        const int t = s.inputs[best], other = s.inputs[1 - best];
        CellRec& p = net->cells[net->tensors[t].producer];
        p.residual = other;
        p.q2 = s.q;
        p.has_q2 = true;
        p.inputs.push_back(other);  // keeps the operand alive for the buffer planner
        net->tensors[t].readable = false;
        net->tensors[t].buffer = -2;  // never materialised
        p.output = s.output;
        net->tensors[s.output].producer = net->tensors[t].producer;
        s.skipped = true;
        s.engine = ENG_FUSED;
    }
}

// Cells [0, n) that the host-buffer entry point may run slice by slice (a structural rule, applied before the
// kernels are chosen; the engine-based rule in finalize can only shorten it): image-wise cells with large
// per-image tensors, up to the first fully-connected cell or stand-alone sum.
static int head_candidate_prefix(const n2d2b_net* net)
{
    int n = 0;
    for (size_t ci = 0; ci < net->cells.size(); ++ci) {
        const CellRec& c = net->cells[ci];
        if (!c.skipped) {
            if (c.type == CELL_FC || c.type == CELL_SUM || c.type == CELL_SCALING) break;
            const TensorRec& t = net->tensors[c.output];
            if ((long long)t.H * t.W < 2048) break;
        }
        n = (int)ci + 1;
    }
    return n;
}

// Buffers are shared by lifetime.  Cells of the head run once per batch slice at an image offset, so slice k of
// a head tensor may be written while slices < k of every other head tensor are complete and still needed: two
// head tensors share a buffer only when they have the same bytes per image (slice k of one then lies exactly
// over slice k of the other, which the per-slice order of the cells has already retired).
// A stride-2 first layer whose only reader is a max pooling writes the pooled tensor directly (the POOL variant of
// the space-to-depth kernel): the convolution's output, the largest tensor of such a network, is never stored.
static int fuse_stem_pool(n2d2b_net* net);

static int plan_buffers(n2d2b_net* net)
{
    const bool keep_all = (net->flags & N2D2B_KEEP_ALL_OUTPUTS) != 0;
    std::vector<size_t> head_bpi;   // per buffer: bytes per image of the head tensors it has held (0 = none)
    const int nt = (int)net->tensors.size();
    std::vector<int> last_use(nt, -1);
    for (int ci = 0; ci < (int)net->cells.size(); ++ci) {
        const CellRec& c = net->cells[ci];
        if (c.skipped) continue;
        for (int i : c.inputs) last_use[i] = std::max(last_use[i], ci);
    }
    int final_tensor = -1;
    for (int ci = (int)net->cells.size() - 1; ci >= 0; --ci)
        if (!net->cells[ci].skipped) { final_tensor = net->cells[ci].output; break; }
    std::vector<size_t> sizes;
    std::vector<int> free_list;
    for (int ci = 0; ci < (int)net->cells.size(); ++ci) {
        CellRec& c = net->cells[ci];
        if (c.skipped) continue;
        TensorRec& t = net->tensors[c.output];
        const size_t need = ((t.bytes_per_image() * (size_t)net->max_batch + 255) / 256) * 256 + 256;
        const bool in_head = ci < net->head_limit;
        int pick = -1;
        if (!keep_all) {
            for (size_t f = 0; f < free_list.size(); ++f) {
                const int b = free_list[f];
                if (in_head && head_bpi[b] != t.bytes_per_image()) continue;
                if (sizes[b] >= need && (pick < 0 || sizes[b] < sizes[free_list[pick]])) pick = (int)f;
            }
        }
        if (pick >= 0) {
            t.buffer = free_list[pick];
            free_list.erase(free_list.begin() + pick);
        } else {
            t.buffer = (int)sizes.size();
            sizes.push_back(need);
            head_bpi.push_back(in_head ? t.bytes_per_image() : 0);
        }
        if (!keep_all) {
            // release the inputs that die with this cell (never the network input or the final output)
            for (int i : c.inputs) {
                if (i == 0 || i == final_tensor) continue;
                if (last_use[i] == ci && net->tensors[i].buffer >= 0) {
                    if (std::find(free_list.begin(), free_list.end(), net->tensors[i].buffer) == free_list.end())
                        free_list.push_back(net->tensors[i].buffer);
                }
            }
            // a tensor nobody reads (other than the final one) can be reused at once
            if (last_use[c.output] < 0 && c.output != final_tensor) free_list.push_back(t.buffer);
        }
    }
    if (!keep_all)
        for (int i = 1; i < nt; ++i)
            if (net->tensors[i].buffer >= 0 && i != final_tensor) net->tensors[i].readable = false;
    net->buffers.assign(sizes.size(), nullptr);
    net->buffer_bytes = sizes;
    for (size_t b = 0; b < sizes.size(); ++b) {
        CUDA_TRY(cudaMalloc(&net->buffers[b], sizes[b]));
        CUDA_TRY(cudaMemset(net->buffers[b], 0, sizes[b]));
    }
    return 0;
}

static void* tensor_ptr(const n2d2b_net* net, int id, const void* d_input)
{
    if (id == 0) return (void*)d_input;
    const TensorRec& t = net->tensors[id];
    return t.buffer >= 0 ? net->buffers[t.buffer] : nullptr;
}

static int final_tensor_of(const n2d2b_net* net)
{
    for (int ci = (int)net->cells.size() - 1; ci >= 0; --ci)
        if (!net->cells[ci].skipped) return net->cells[ci].output;
    return -1;
}

int n2d2b_net_finalize(n2d2b_net* net, int max_batch, unsigned flags)
{
    if (!net) return fail(N2D2B_ERR_INVALID, "net must not be NULL");
    if (net->finalized) return fail(N2D2B_ERR_STATE, "the network is already finalized");
    if (net->cells.empty()) return fail(N2D2B_ERR_STATE, "the network has no cells");
    if (max_batch < 1) return fail(N2D2B_ERR_INVALID, "max_batch must be positive");
    CUDA_TRY(cudaSetDevice(net->device));
    net->max_batch = max_batch;
    net->flags = flags;
    if (!(flags & N2D2B_NO_FUSION)) fuse_residuals(net);
    if ((flags & N2D2B_FUSE_FIRST_POOL)
        && !(flags & (N2D2B_NO_FUSION | N2D2B_KEEP_ALL_OUTPUTS | N2D2B_FORCE_SIMT | N2D2B_EXACT64_EPILOGUE)))
        if (int rc = fuse_stem_pool(net)) return rc;
    net->head_limit = head_candidate_prefix(net);
    if (int rc = plan_buffers(net)) return rc;
    CUDA_TRY(cudaMalloc(&net->d_status, 64));
    CUDA_TRY(cudaMemset(net->d_status, 0, 64));
    net->launches = 0;
    for (CellRec& c : net->cells) {
        if (c.skipped) continue;
        net->launches++;
        if (c.type == CELL_POOL) { c.engine = ENG_POOL; continue; }
        if (int rc = upload_quant(c.q)) return rc;
        if (c.has_q2)
            if (int rc = upload_quant(c.q2)) return rc;
        if (c.type == CELL_SUM || c.type == CELL_SCALING) { c.engine = ENG_SUM; continue; }
        // conv / fc: choose the kernel family and lay the weights out for it
        const ConvGeom& g = c.geom;
        const bool depthwise = (c.type == CELL_CONV && g.groups == g.C && g.Cg == 1 && g.Og == 1 && g.C % 16 == 0
                                && g.groups > 1 && c.residual < 0
                                && net->tensors[c.output].dtype == DT_I8);
        std::vector<int8_t> laid = c.weights;
        const bool stem = !depthwise && c.type == CELL_CONV && !(flags & N2D2B_FORCE_SIMT) && c.residual < 0
                          && stem_eligible(g) && net->tensors[c.output].dtype == DT_I8 && !(flags & N2D2B_EXACT64_EPILOGUE);
        if (stem) {
            if (!c.d_fast)
                if (int rc = upload_fast(c, net->tensors[c.output])) return rc;
            if (c.fast.enabled && stem_s2d_eligible(g)) {
                // stride 2: space-to-depth image, no gather
                std::vector<int8_t> arranged(stem_s2d_weight_bytes(g));
                stem_s2d_arrange_weights(g, c.weights.data(), arranged.data());
                CUDA_TRY(cudaMalloc((void**)&c.d_weights, arranged.size() + 256));
                CUDA_TRY(cudaMemcpy(c.d_weights, arranged.data(), arranged.size(), cudaMemcpyHostToDevice));
                c.d_weight_bytes = arranged.size();
                int Hs = 0, Ws = 0;
                stem_s2d_dims(g, &Hs, &Ws);
                CUDA_TRY(cudaMalloc(&c.d_pad4, (size_t)max_batch * Hs * Ws * 16 + 256));
                const char* why = "";
                if (stem_s2d_make_plan(&c.stem2, c.d_pad4, c.d_weights, g, max_batch, net->tensors[c.inputs[0]].is_unsigned,
                                       net->num_sms, &why, c.pool_fused ? &c.fused_pool : nullptr) == 0) {
                    net->launches++;
                    c.engine = ENG_STEM_S2D;
                    continue;
                }
                if (c.pool_fused) return fail(N2D2B_ERR_STATE, "internal: the fused first layer has no plan (%s)", why);
                cudaFree(c.d_weights);
                c.d_weights = nullptr;
                cudaFree(c.d_pad4);
                c.d_pad4 = nullptr;
            }
            if (c.fast.enabled) {
                std::vector<int8_t> arranged(stem_weight_bytes(g));
                stem_arrange_weights(g, c.weights.data(), arranged.data());
                CUDA_TRY(cudaMalloc((void**)&c.d_weights, arranged.size() + 256));
                CUDA_TRY(cudaMemcpy(c.d_weights, arranged.data(), arranged.size(), cudaMemcpyHostToDevice));
                c.d_weight_bytes = arranged.size();
                const char* why = "";
                if (stem_make_plan(&c.stem, c.d_weights, g, net->tensors[c.inputs[0]].is_unsigned, net->num_sms, &why) == 0) {
                    int Hp = 0, Wp = 0;
                    stem_padded_dims(g, &Hp, &Wp);
                    CUDA_TRY(cudaMalloc(&c.d_pad4, (size_t)max_batch * Hp * Wp * 4 + 256));
                    net->launches++;
                    c.engine = ENG_STEM;
                    continue;
                }
                cudaFree(c.d_weights);
                c.d_weights = nullptr;
            }
            cudaFree(c.d_fast);
            c.d_fast = nullptr;
            c.fast = FastQuant{};
        }
        if (depthwise) {
            c.engine = ENG_DEPTHWISE;
            if (!(flags & N2D2B_EXACT64_EPILOGUE))
                if (int rc = upload_fast(c, net->tensors[c.output])) return rc;
            // Stride-1 layers whose channels come in whole groups of 32 run on the tensor cores as block-diagonal
            // groups (patch kernel); it needs the 32-bit epilogue
            ConvGeom gb = g;
            gb.B = max_batch;
            if (c.fast.enabled && !(flags & N2D2B_FORCE_SIMT) && patch_eligible(gb)) {
                std::vector<int8_t> arranged(patch_dw_weight_bytes(g));
                patch_dw_arrange_weights(g, c.weights.data(), arranged.data());
                CUDA_TRY(cudaMalloc((void**)&c.d_weights, arranged.size() + 256));
                CUDA_TRY(cudaMemcpy(c.d_weights, arranged.data(), arranged.size(), cudaMemcpyHostToDevice));
                c.d_weight_bytes = arranged.size();
                const char* why = "";
                const void* in_ptr = tensor_ptr(net, c.inputs[0], nullptr);
                static char dw_placeholder[16] __attribute__((aligned(16)));
                if (patch_make_plan(&c.patch, in_ptr ? in_ptr : (const void*)dw_placeholder, c.d_weights, gb,
                                    net->tensors[c.inputs[0]].is_unsigned, net->num_sms, &why) == 0) {
                    c.engine = ENG_PATCH;
                    c.plan_input = in_ptr;   // nullptr = re-encoded with the real input at the first forward pass
                    continue;
                }
                cudaFree(c.d_weights);
                c.d_weights = nullptr;
            }
            // Strided ones (and whatever else the patch kernel leaves) take the implicit-GEMM kernel the same way: one
            // 64-column tile per group of 64 channels, im2col loads of the group's channel slice
            if (c.fast.enabled && !(flags & (N2D2B_FORCE_SIMT | N2D2B_EXACT64_EPILOGUE)) && igemm_dw_group(gb)) {
                std::vector<int8_t> arranged(igemm_dw_weight_bytes(g));
                igemm_dw_arrange_weights(g, c.weights.data(), arranged.data());
                CUDA_TRY(cudaMalloc((void**)&c.d_weights, arranged.size() + 256));
                c.d_weight_bytes = arranged.size();
                const char* why = "";
                const void* in_ptr = tensor_ptr(net, c.inputs[0], nullptr);
                static char dwg_placeholder[16] __attribute__((aligned(16)));
                if (igemm_make_plan(&c.plan, in_ptr ? in_ptr : (const void*)dwg_placeholder, c.d_weights,
                                    tensor_ptr(net, c.output, nullptr), nullptr, gb, net->tensors[c.inputs[0]].is_unsigned, 1, 0,
                                    net->num_sms, &why, 0, 0) == 0
                    && igemm_uses_fast_epilogue(c.plan, c.fast, false, DT_I8)) {
                    const int pb = igemm_perm_block(c.plan);
                    std::vector<int8_t> rows(arranged.size());
                    igemm_permute_weights(arranged.data(), rows.data(), g.C, arranged.size() / (size_t)g.C, pb);
                    c.plan.perm = pb;
                    CUDA_TRY(cudaMemcpy(c.d_weights, rows.data(), rows.size(), cudaMemcpyHostToDevice));
                    c.engine = ENG_TCGEN05;
                    c.has_plan = true;
                    c.plan_input = in_ptr;
                    continue;
                }
                cudaFree(c.d_weights);
                c.d_weights = nullptr;
            }
            // [C][kH][kW] -> [kH][kW][C] so that 16 channels of a tap are one 128-bit load
            const int taps = g.kH * g.kW;
            for (int ch = 0; ch < g.C; ++ch)
                for (int t = 0; t < taps; ++t) laid[(size_t)t * g.C + ch] = c.weights[(size_t)ch * taps + t];
        } else {
            c.engine = ENG_SIMT;
        }
        // Packed 4-bit weights stay packed in HBM when the cell runs on the implicit-GEMM kernel, whose expansion
        // warps unpack them tile by tile; every other kernel takes them widened to int8.
        const bool igemm_shape = !depthwise && !(flags & N2D2B_FORCE_SIMT) && g.groups == 1 && g.C % 16 == 0;
        bool w4 = c.wbits == 4 && igemm_shape;
        auto pack4 = [](const std::vector<int8_t>& w) {
            std::vector<int8_t> p(w.size() / 2);
            for (size_t i = 0; i < p.size(); ++i) p[i] = (int8_t)(((w[2 * i] & 0xF) << 4) | (w[2 * i + 1] & 0xF));
            return p;
        };
        // Output channels that are not a multiple of 32: take the 32-bit epilogue on a padded copy (see pad_O)
        ConvGeom gplan = g;
        if (igemm_shape && !w4 && g.O % 32 != 0 && c.residual < 0 && net->tensors[c.output].dtype == DT_I8
            && !(flags & N2D2B_EXACT64_EPILOGUE)) {
            if (int rc = upload_fast(c, net->tensors[c.output])) return rc;
            if (c.fast.enabled) {
                c.pad_O = (g.O + 63) & ~63;
                gplan.O = c.pad_O;
                laid.resize((size_t)c.pad_O * g.kH * g.kW * g.Cg, 0);
                CUDA_TRY(cudaMalloc(&c.d_colpad, (size_t)max_batch * g.oH * g.oW * c.pad_O + 256));
                net->launches++;
            }
        }
        c.d_weight_bytes = w4 ? laid.size() / 2 : laid.size();
        CUDA_TRY(cudaMalloc((void**)&c.d_weights, c.d_weight_bytes + 256));
        CUDA_TRY(cudaMemset(c.d_weights, 0, c.d_weight_bytes + 256));
        if (!w4) CUDA_TRY(cudaMemcpy(c.d_weights, laid.data(), laid.size(), cudaMemcpyHostToDevice));
        if (igemm_shape) {
            ConvGeom gb = gplan;
            gb.B = max_batch;
            const char* why = "";
            const void* in_ptr = tensor_ptr(net, c.inputs[0], nullptr);
            // the network input pointer is only known at forward time; plan against a placeholder
            // that is re-encoded on first use
            static char placeholder[16] __attribute__((aligned(16)));
            const void* enc_ptr = in_ptr ? in_ptr : (const void*)placeholder;
            const void* out_ptr = c.pad_O ? c.d_colpad
                                : net->tensors[c.output].dtype == DT_I8 ? tensor_ptr(net, c.output, nullptr) : nullptr;
            const void* res_ptr = c.residual >= 0 ? tensor_ptr(net, c.residual, nullptr) : nullptr;
            int planned = igemm_make_plan(&c.plan, enc_ptr, c.d_weights, out_ptr, res_ptr, gb, net->tensors[c.inputs[0]].is_unsigned,
                                          (flags & N2D2B_FORCE_IM2COL) ? 1 : 0, 0, net->num_sms, &why,
                                          (flags & N2D2B_FORCE_PAIR) ? 1 : 0, w4 ? 1 : 0);
            if (planned != 0 && w4) {
                // no room for the packed variant: widen the weights after all
                w4 = false;
                cudaFree(c.d_weights);
                c.d_weights = nullptr;
                c.d_weight_bytes = laid.size();
                CUDA_TRY(cudaMalloc((void**)&c.d_weights, laid.size() + 256));
                CUDA_TRY(cudaMemset(c.d_weights, 0, laid.size() + 256));
                CUDA_TRY(cudaMemcpy(c.d_weights, laid.data(), laid.size(), cudaMemcpyHostToDevice));
                planned = igemm_make_plan(&c.plan, enc_ptr, c.d_weights, out_ptr, res_ptr, gb, net->tensors[c.inputs[0]].is_unsigned,
                                          (flags & N2D2B_FORCE_IM2COL) ? 1 : 0, 0, net->num_sms, &why,
                                          (flags & N2D2B_FORCE_PAIR) ? 1 : 0, 0);
            }
            if (planned == 0) {
                c.engine = ENG_TCGEN05;
                c.has_plan = true;
                c.plan_input = in_ptr;  // nullptr = must be re-encoded with the real input
                if (!(flags & N2D2B_EXACT64_EPILOGUE) && !c.pad_O) {
                    const bool res_i8 = c.residual >= 0 && net->tensors[c.residual].dtype == DT_I8;
                    if (int rc = upload_fast(c, net->tensors[c.output], res_i8,
                                             c.residual >= 0 ? net->tensors[c.residual].is_unsigned : 0, w4))
                        return rc;
                }
                // small-channel stride-1 layers read their input once, from a shared-memory patch
                if (!w4 && !c.pad_O && c.fast.enabled && c.residual < 0 && net->tensors[c.output].dtype == DT_I8
                    && !(flags & (N2D2B_FORCE_IM2COL | N2D2B_EXACT64_EPILOGUE)) && patch_eligible(gb)
                    && patch_make_plan(&c.patch, enc_ptr, c.d_weights, gb, net->tensors[c.inputs[0]].is_unsigned,
                                       net->num_sms, &why) == 0)
                    c.engine = ENG_PATCH;
                // a cell that stays on the implicit-GEMM kernel with the 32-bit epilogue stores its weight rows in
                // the permuted order that epilogue reads (see perm_block)
                const bool permute = c.engine == ENG_TCGEN05
                                     && igemm_uses_fast_epilogue(c.plan, c.fast, c.residual >= 0, net->tensors[c.output].dtype);
                if (c.engine == ENG_PATCH) {
                    std::vector<int8_t> rows(laid.size());
                    patch_permute_weights(laid.data(), rows.data(), g.O, (size_t)g.kH * g.kW * g.Cg);
                    CUDA_TRY(cudaMemcpy(c.d_weights, rows.data(), rows.size(), cudaMemcpyHostToDevice));
                } else if (permute || w4) {
                    std::vector<int8_t> rows = laid;
                    if (permute) {
                        const int pb = igemm_perm_block(c.plan);
                        igemm_permute_weights(laid.data(), rows.data(), gplan.O, (size_t)g.kH * g.kW * g.Cg, pb);
                        c.plan.perm = pb;
                    }
                    if (w4) rows = pack4(rows);
                    CUDA_TRY(cudaMemcpy(c.d_weights, rows.data(), rows.size(), cudaMemcpyHostToDevice));
                }
            } else if (w4 || c.pad_O) {
                return fail(N2D2B_ERR_STATE, "internal: a packed or padded cell without a plan (%s)", why);
            }
        }
    }
    CUDA_TRY(cudaMalloc(&net->d_stage_in, net->tensors[0].bytes_per_image() * (size_t)max_batch + 256));
    CUDA_TRY(cudaMalloc(&net->d_stage_out,
                        net->tensors[final_tensor_of(net)].bytes_per_image() * (size_t)max_batch + 256));
    CUDA_TRY(cudaStreamCreateWithFlags(&net->copy_stream, cudaStreamNonBlocking));
    for (cudaEvent_t& e : net->slice_ready) CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    CUDA_TRY(cudaEventCreateWithFlags(&net->stage_free, cudaEventDisableTiming));
    // Leading cells that the host-buffer entry point runs slice by slice while later slices of the batch
    // are still being uploaded: every cell works image by image, so a slice is an offset (in images for the
    // pointer-based kernels, in rows of the tensor maps for the tensor-core ones).  The head ends where the
    // per-image tensors get small (after the first stage of a ResNet): from there on a launch per slice would
    // cost more in fixed launch time than the overlap gains.
    net->head_cells = 0;
    for (size_t ci = 0; ci < net->cells.size(); ++ci) {
        const CellRec& c = net->cells[ci];
        bool sliceable = true;
        if (!c.skipped) {
            const bool mapped = c.engine == ENG_TCGEN05 || c.engine == ENG_PATCH;
            const bool pointer_based = (c.engine == ENG_STEM || c.engine == ENG_STEM_S2D || c.engine == ENG_POOL
                                        || c.engine == ENG_DEPTHWISE || c.engine == ENG_SIMT)
                                       && c.residual < 0 && c.inputs.size() == 1;
            sliceable = c.type != CELL_FC && (mapped || pointer_based);
            const TensorRec& t = net->tensors[c.output];
            if ((long long)t.H * t.W < 2048) sliceable = false;
        }
        if (!sliceable || (int)ci >= net->head_limit) break;
        net->head_cells = (int)ci + 1;
    }
    for (int k = 0; k < 2; ++k) {
        CUDA_TRY(cudaEventCreateWithFlags(&net->pipe_uploaded[k], cudaEventDisableTiming));
        CUDA_TRY(cudaEventCreateWithFlags(&net->pipe_computed[k], cudaEventDisableTiming));
        CUDA_TRY(cudaEventCreateWithFlags(&net->pipe_done[k], cudaEventDisableTiming));
    }
    CUDA_TRY(cudaStreamCreateWithFlags(&net->download_stream, cudaStreamNonBlocking));
    net->finalized = true;
    return 0;
}

static int fuse_stem_pool(n2d2b_net* net)
{
    std::vector<int> consumers(net->tensors.size(), 0);
    for (const CellRec& c : net->cells)
        if (!c.skipped)
            for (int i : c.inputs) consumers[i]++;
    for (size_t ci = 0; ci < net->cells.size(); ++ci) {
        CellRec& c = net->cells[ci];
        if (c.skipped || c.type != CELL_CONV || c.residual >= 0 || c.inputs[0] != 0) continue;
        if (!stem_eligible(c.geom) || !stem_s2d_eligible(c.geom)) continue;
        const int t = c.output;
        if (consumers[t] != 1 || net->tensors[t].dtype != DT_I8) continue;
        int pj = -1;
        for (size_t cj = ci + 1; cj < net->cells.size(); ++cj)
            if (!net->cells[cj].skipped && net->cells[cj].inputs.size() == 1 && net->cells[cj].inputs[0] == t) { pj = (int)cj; break; }
        if (pj < 0 || net->cells[pj].type != CELL_POOL) continue;
        CellRec& p = net->cells[pj];
        if (!stem_s2d_pool_eligible(c.geom, p.pgeom)) continue;
        // the first-layer kernel needs the 32-bit epilogue
        if (int rc = upload_fast(c, net->tensors[t])) return rc;
        if (!c.fast.enabled) continue;
        c.pool_fused = true;
        c.fused_pool = p.pgeom;
        net->tensors[t].readable = false;
        net->tensors[t].buffer = -2;   // never materialised
        c.output = p.output;
        net->tensors[p.output].producer = (int)ci;
        p.skipped = true;
        p.engine = ENG_FUSED;
    }
    return 0;
}

// ---- forward --------------------------------------------------------------------------------
// Runs one cell on images [img0, img0 + batch) of the batch (img0 != 0 only for cells without tensor maps).
static int run_cell(n2d2b_net* net, CellRec& c, const void* d_input, int batch, cudaStream_t s, int img0 = 0)
{
    const void* in0 = tensor_ptr(net, c.inputs[0], d_input);
    void* out = tensor_ptr(net, c.output, d_input);
    const TensorRec& tin = net->tensors[c.inputs[0]];
    const TensorRec& tout = net->tensors[c.output];
    if (!in0 || !out) return fail(N2D2B_ERR_STATE, "internal: tensor without a buffer");
    // the tensor-core cells address their tensors through maps encoded over the whole buffers: a batch slice
    // is an offset in rows / images there; every other cell takes offset pointers
    const bool mapped = c.engine == ENG_TCGEN05 || c.engine == ENG_PATCH;
    if (img0 && !mapped) {
        if (c.engine == ENG_SUM || c.residual >= 0)
            return fail(N2D2B_ERR_STATE, "internal: this cell cannot run on a slice");
        in0 = (const uint8_t*)in0 + (size_t)img0 * tin.bytes_per_image();
        out = (uint8_t*)out + (size_t)img0 * tout.bytes_per_image();
    }
    Residual r{};
    if (c.residual >= 0) {
        r.ptr = tensor_ptr(net, c.residual, d_input);
        r.is_unsigned = net->tensors[c.residual].is_unsigned;
        r.q2 = c.q2.dev;
    }
    switch (c.engine) {
    case ENG_TCGEN05: {
        void* const gemm_out = c.pad_O ? c.d_colpad : out;
        if (c.plan_input != in0) {
            ConvGeom gb = c.geom;
            gb.B = net->max_batch;
            if (c.pad_O) gb.O = c.pad_O;
            const char* why = "";
            const int perm = c.plan.perm, w4 = c.plan.w4;   // properties of the stored weights, not of the tensor maps
            if (igemm_make_plan(&c.plan, in0, c.d_weights, tout.dtype == DT_I8 ? gemm_out : nullptr, r.ptr, gb, tin.is_unsigned,
                                (net->flags & N2D2B_FORCE_IM2COL) ? 1 : 0, 0, net->num_sms, &why,
                                (net->flags & N2D2B_FORCE_PAIR) ? 1 : 0, w4))
                return fail(N2D2B_ERR_INVALID, "tensor-core plan failed: %s", why);
            c.plan.perm = perm;
            c.plan_input = in0;
        }
        IgemmPlan p = c.plan;
        p.M = batch * c.geom.oH * c.geom.oW;
        CUDA_TRY(launch_igemm(p, c.q.dev, r, c.fast, gemm_out, tout.dtype, img0 * c.geom.oH * c.geom.oW, net->d_status, s));
        if (c.pad_O) {
            const size_t row0 = (size_t)img0 * c.geom.oH * c.geom.oW;
            CUDA_TRY(launch_drop_padded_columns((const uint8_t*)c.d_colpad + row0 * c.pad_O, c.pad_O,
                                                (uint8_t*)out + row0 * c.geom.O, c.geom.O, (size_t)p.M, s));
        }
        break;
    }
    case ENG_PATCH: {
        if (c.plan_input != in0) {
            ConvGeom gb = c.geom;
            gb.B = net->max_batch;
            const char* why = "";
            if (patch_make_plan(&c.patch, in0, c.d_weights, gb, tin.is_unsigned, net->num_sms, &why))
                return fail(N2D2B_ERR_INVALID, "patch plan failed: %s", why);
            c.plan_input = in0;
        }
        ConvGeom g = c.geom;
        g.B = batch;
        CUDA_TRY(launch_patch(c.patch, g, img0, c.fast, out, net->d_status, s));
        break;
    }
    case ENG_STEM_S2D: {
        ConvGeom g = c.geom;
        g.B = batch;
        int Hs = 0, Ws = 0;
        stem_s2d_dims(g, &Hs, &Ws);
        CUDA_TRY(launch_s2d_image(in0, g, batch, (uint8_t*)c.d_pad4 + (size_t)img0 * Hs * Ws * 16, s));
        CUDA_TRY(launch_stem_s2d(c.stem2, g, img0, c.fast, out, net->d_status, s));
        break;
    }
    case ENG_STEM: {
        ConvGeom g = c.geom;
        g.B = batch;
        int Hp = 0, Wp = 0;
        stem_padded_dims(g, &Hp, &Wp);
        void* in4 = (uint8_t*)c.d_pad4 + (size_t)img0 * Hp * Wp * 4;
        CUDA_TRY(launch_pad_image(in0, g, batch, in4, s));
        CUDA_TRY(launch_stem(c.stem, in4, g, c.fast, out, net->d_status, s));
        break;
    }
    case ENG_SIMT: {
        ConvGeom g = c.geom;
        g.B = batch;
        if (c.type == CELL_FC && c.residual < 0)
            CUDA_TRY(launch_fc_direct(in0, tin.is_unsigned, c.d_weights, batch, g.C, g.O, c.q.dev, out, tout.dtype, s));
        else
            CUDA_TRY(launch_conv_direct(in0, tin.is_unsigned, c.d_weights, g, c.q.dev, r, out, tout.dtype, s));
        break;
    }
    case ENG_DEPTHWISE: {
        ConvGeom g = c.geom;
        g.B = batch;
        CUDA_TRY(launch_conv_depthwise(in0, tin.is_unsigned, c.d_weights, g, c.q.dev, c.fast, out, s));
        break;
    }
    case ENG_POOL: {
        PoolGeom g = c.pgeom;
        g.B = batch;
        if (tin.dtype == DT_I32) CUDA_TRY(launch_pool_i32(in0, g, out, s));
        else CUDA_TRY(launch_pool(in0, tin.is_unsigned, g, out, s));
        break;
    }
    case ENG_SUM: {
        SumInputs ins{};
        ins.n = (int)c.inputs.size();
        for (int k = 0; k < ins.n; ++k) {
            ins.ptr[k] = tensor_ptr(net, c.inputs[k], d_input);
            ins.dtype[k] = net->tensors[c.inputs[k]].dtype;
            ins.is_unsigned[k] = net->tensors[c.inputs[k]].is_unsigned;
        }
        CUDA_TRY(launch_elemwise_sum(ins, (size_t)batch * tout.H * tout.W, tout.C, c.q.dev, out, tout.dtype, s));
        break;
    }
    case ENG_FUSED:
        break;
    }
    return 0;
}

static int forward_impl(n2d2b_net* net, const void* d_input, int batch, void* d_output, cudaStream_t s, float* ms,
                        int nb_cells, int first_cell = 0)
{
    if (!net) return fail(N2D2B_ERR_INVALID, "net must not be NULL");
    if (!net->finalized) return fail(N2D2B_ERR_STATE, "forward before finalize");
    if (batch < 0 || batch > net->max_batch)
        return fail(N2D2B_ERR_TOO_LARGE, "batch %d exceeds the finalized maximum %d", batch, net->max_batch);
    if (batch == 0) return 0;
    if (!d_input) return fail(N2D2B_ERR_INVALID, "d_input must not be NULL");
    CUDA_TRY(cudaSetDevice(net->device));
    std::vector<cudaEvent_t> ev;
    if (ms) {
        if (nb_cells != (int)net->cells.size())
            return fail(N2D2B_ERR_INVALID, "ms must have one entry per cell (%d)", (int)net->cells.size());
        ev.resize(net->cells.size() + 1);
        for (auto& e : ev) CUDA_TRY(cudaEventCreate(&e));
        CUDA_TRY(cudaEventRecord(ev[0], s));
    }
    for (size_t ci = (size_t)first_cell; ci < net->cells.size(); ++ci) {
        CellRec& c = net->cells[ci];
        if (!c.skipped)
            if (int rc = run_cell(net, c, d_input, batch, s)) return rc;
        if (ms) CUDA_TRY(cudaEventRecord(ev[ci + 1], s));
    }
    const int ft = final_tensor_of(net);
    if (d_output) {
        const TensorRec& t = net->tensors[ft];
        CUDA_TRY(cudaMemcpyAsync(d_output, tensor_ptr(net, ft, d_input), t.bytes_per_image() * (size_t)batch,
                                 cudaMemcpyDeviceToDevice, s));
    }
    net->last_input = d_input;
    if (ms) {
        CUDA_TRY(cudaStreamSynchronize(s));
        for (size_t ci = 0; ci < net->cells.size(); ++ci) CUDA_TRY(cudaEventElapsedTime(&ms[ci], ev[ci], ev[ci + 1]));
        for (auto& e : ev) cudaEventDestroy(e);
    }
    return 0;
}

static int check_status(n2d2b_net* net)
{
    int st = 0;
    CUDA_TRY(cudaMemcpy(&st, net->d_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (st != 0) {
        cudaMemset(net->d_status, 0, sizeof(int));
        return fail(N2D2B_ERR_TIMEOUT, "a tensor-core kernel gave up waiting on a pipeline barrier (role %d)", st);
    }
    return 0;
}

int n2d2b_net_forward(n2d2b_net* net, const void* d_input, int batch, void* d_output, n2d2b_stream stream)
{
    return forward_impl(net, d_input, batch, d_output, (cudaStream_t)stream, nullptr, 0);
}

int n2d2b_net_check(n2d2b_net* net, n2d2b_stream stream)
{
    if (!net) return fail(N2D2B_ERR_INVALID, "net must not be NULL");
    if (!net->finalized) return fail(N2D2B_ERR_STATE, "check before finalize");
    CUDA_TRY(cudaSetDevice(net->device));
    CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    return check_status(net);
}

int n2d2b_net_selftest_wait_timeout(n2d2b_net* net, unsigned limit_us, n2d2b_stream stream)
{
    if (!net) return fail(N2D2B_ERR_INVALID, "net must not be NULL");
    if (!net->finalized) return fail(N2D2B_ERR_STATE, "selftest before finalize");
    if (limit_us < 1 || limit_us > 100000) return fail(N2D2B_ERR_INVALID, "limit_us must be in 1..100000");
    CUDA_TRY(cudaSetDevice(net->device));
    wait_timeout_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(net->d_status, (unsigned long long)limit_us * 1000ull);
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int n2d2b_net_profile(n2d2b_net* net, const void* d_input, int batch, void* d_output, float* ms, int nb_cells,
                      n2d2b_stream stream)
{
    if (!ms) return fail(N2D2B_ERR_INVALID, "ms must not be NULL");
    if (int rc = forward_impl(net, d_input, batch, d_output, (cudaStream_t)stream, ms, nb_cells)) return rc;
    return check_status(net);
}

int n2d2b_net_set_slices(n2d2b_net* net, int nb_slices)
{
    if (!net) return fail(N2D2B_ERR_INVALID, "net must not be NULL");
    if (nb_slices < 0 || nb_slices > 8) return fail(N2D2B_ERR_INVALID, "nb_slices must be in 0..8 (0 = automatic)");
    net->forced_slices = nb_slices;
    return 0;
}

static int host_call_checks(n2d2b_net* net, const void* h_input, int batch, void* h_output)
{
    if (!net) return fail(N2D2B_ERR_INVALID, "net must not be NULL");
    if (!net->finalized) return fail(N2D2B_ERR_STATE, "forward before finalize");
    if (batch < 0 || batch > net->max_batch)
        return fail(N2D2B_ERR_TOO_LARGE, "batch %d exceeds the finalized maximum %d", batch, net->max_batch);
    if (batch > 0 && (!h_input || !h_output)) return fail(N2D2B_ERR_INVALID, "host buffers must not be NULL");
    return 0;
}

int n2d2b_net_forward_host(n2d2b_net* net, const void* h_input, int batch, void* h_output, n2d2b_stream stream)
{
    if (int rc = host_call_checks(net, h_input, batch, h_output)) return rc;
    if (batch == 0) return 0;
    CUDA_TRY(cudaSetDevice(net->device));
    cudaStream_t s = (cudaStream_t)stream;
    const size_t in_bytes = net->tensors[0].bytes_per_image() * (size_t)batch;
    const int ft = final_tensor_of(net);
    const size_t out_bytes = net->tensors[ft].bytes_per_image() * (size_t)batch;
    void* d_in = net->d_stage_in;
    void* d_out = net->d_stage_out;
    // Slices of about 128 images, at most 8.  The upload is slower than the leading cells, so what the caller
    // waits for is the upload, then the leading cells of the LAST slice, then the rest of the network: the last
    // slice is half as large as the others.
    int nslices = (net->head_cells > 0 && batch >= 256) ? (batch / 128 > 8 ? 8 : batch / 128) : 1;
    if (net->forced_slices > 0 && net->head_cells > 0) nslices = net->forced_slices;
    while (nslices > 1 && batch < 2 * nslices - 1) --nslices;   // every slice holds at least one image
    const int wsum = 2 * nslices - 1;   // weights 2, 2, ..., 2, 1
    if (nslices == 1) {
        CUDA_TRY(cudaMemcpyAsync(d_in, h_input, in_bytes, cudaMemcpyHostToDevice, s));
        if (int rc = forward_impl(net, d_in, batch, d_out, s, nullptr, 0)) return rc;
    } else {
        // the staging buffer may still be read by work queued on `s` by an earlier call
        CUDA_TRY(cudaEventRecord(net->stage_free, s));
        CUDA_TRY(cudaStreamWaitEvent(net->copy_stream, net->stage_free, 0));
        const size_t img_bytes = net->tensors[0].bytes_per_image();
        for (int k = 0; k < nslices; ++k) {
            const int b0 = (int)((long long)batch * (2 * k) / wsum);
            const int b1 = k + 1 == nslices ? batch : (int)((long long)batch * (2 * k + 2) / wsum);
            if (b1 <= b0) continue;
            CUDA_TRY(cudaMemcpyAsync((uint8_t*)d_in + (size_t)b0 * img_bytes, (const uint8_t*)h_input + (size_t)b0 * img_bytes,
                                     (size_t)(b1 - b0) * img_bytes, cudaMemcpyHostToDevice, net->copy_stream));
            CUDA_TRY(cudaEventRecord(net->slice_ready[k], net->copy_stream));
            CUDA_TRY(cudaStreamWaitEvent(s, net->slice_ready[k], 0));
            for (int ci = 0; ci < net->head_cells; ++ci)
                if (!net->cells[ci].skipped)
                    if (int rc = run_cell(net, net->cells[ci], d_in, b1 - b0, s, b0)) return rc;
        }
        if (int rc = forward_impl(net, d_in, batch, d_out, s, nullptr, 0, net->head_cells)) return rc;
    }
    CUDA_TRY(cudaMemcpyAsync(h_output, d_out, out_bytes, cudaMemcpyDeviceToHost, s));
    CUDA_TRY(cudaStreamSynchronize(s));
    return check_status(net);
}

// Streaming form of the host-buffer entry point.  The reference overlaps the preparation of the next batch with
// the inference of the current one on a second host thread (src/utils/Helper.cpp:428-454); here the overlap is on
// the device: the upload of batch k + 1 runs on the copy stream, into the second staging buffer, under the
// forward pass of batch k.
int n2d2b_net_submit_host(n2d2b_net* net, const void* h_input, int batch, void* h_output, n2d2b_stream stream)
{
    if (int rc = host_call_checks(net, h_input, batch, h_output)) return rc;
    if (batch == 0) return 0;
    CUDA_TRY(cudaSetDevice(net->device));
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned slot = net->pipe_next & 1u;
    const size_t in_cap = net->tensors[0].bytes_per_image() * (size_t)net->max_batch + 256;
    const int ft = final_tensor_of(net);
    const size_t out_cap = net->tensors[ft].bytes_per_image() * (size_t)net->max_batch + 256;
    if (!net->d_pipe_in[slot]) {
        // the staging sets of this entry point are allocated on first use (callers of the blocking form never pay for them)
        CUDA_TRY(cudaMalloc(&net->d_pipe_in[slot], in_cap));
        CUDA_TRY(cudaMalloc(&net->d_pipe_out[slot], out_cap));
    }
    // the slot's previous batch (two submissions ago) must have left its staging buffers: its forward pass has
    // read the input (the upload waits for that) and its download has read the output (the forward pass, which
    // writes the output buffer last, waits for that)
    if (net->pipe_busy[slot]) {
        CUDA_TRY(cudaStreamWaitEvent(net->copy_stream, net->pipe_computed[slot], 0));
        CUDA_TRY(cudaStreamWaitEvent(s, net->pipe_done[slot], 0));
    }
    const size_t in_bytes = net->tensors[0].bytes_per_image() * (size_t)batch;
    const size_t out_bytes = net->tensors[ft].bytes_per_image() * (size_t)batch;
    CUDA_TRY(cudaMemcpyAsync(net->d_pipe_in[slot], h_input, in_bytes, cudaMemcpyHostToDevice, net->copy_stream));
    CUDA_TRY(cudaEventRecord(net->pipe_uploaded[slot], net->copy_stream));
    CUDA_TRY(cudaStreamWaitEvent(s, net->pipe_uploaded[slot], 0));
    if (int rc = forward_impl(net, net->d_pipe_in[slot], batch, net->d_pipe_out[slot], s, nullptr, 0)) return rc;
    // the download leaves on a stream of its own, so that `s` holds nothing but forward passes back to back
    CUDA_TRY(cudaEventRecord(net->pipe_computed[slot], s));
    CUDA_TRY(cudaStreamWaitEvent(net->download_stream, net->pipe_computed[slot], 0));
    CUDA_TRY(cudaMemcpyAsync(h_output, net->d_pipe_out[slot], out_bytes, cudaMemcpyDeviceToHost, net->download_stream));
    CUDA_TRY(cudaEventRecord(net->pipe_done[slot], net->download_stream));
    net->pipe_busy[slot] = true;
    net->pipe_stream[slot] = s;
    net->pipe_next++;
    return 0;
}

int n2d2b_net_wait(n2d2b_net* net)
{
    if (!net) return fail(N2D2B_ERR_INVALID, "net must not be NULL");
    if (!net->finalized) return fail(N2D2B_ERR_STATE, "wait before finalize");
    CUDA_TRY(cudaSetDevice(net->device));
    for (int k = 0; k < 2; ++k)
        if (net->pipe_busy[k]) {
            CUDA_TRY(cudaEventSynchronize(net->pipe_done[k]));
            net->pipe_busy[k] = false;
        }
    return check_status(net);
}

int n2d2b_net_estimated_labels(n2d2b_net* net, int batch, int32_t* d_labels, int32_t* d_values, n2d2b_stream stream)
{
    if (!net || !d_labels) return fail(N2D2B_ERR_INVALID, "net and d_labels must not be NULL");
    if (!net->finalized) return fail(N2D2B_ERR_STATE, "estimated labels before finalize");
    if (!net->last_input) return fail(N2D2B_ERR_STATE, "estimated labels before a forward pass");
    if (batch < 0 || batch > net->max_batch) return fail(N2D2B_ERR_TOO_LARGE, "batch out of range");
    CUDA_TRY(cudaSetDevice(net->device));
    const int ft = final_tensor_of(net);
    const TensorRec& t = net->tensors[ft];
    CUDA_TRY(launch_argmax(tensor_ptr(net, ft, net->last_input), t.dtype, t.is_unsigned, (size_t)batch * t.H * t.W, t.C, d_labels,
                           d_values, (cudaStream_t)stream));
    return 0;
}

int n2d2b_net_estimated_labels_topn(n2d2b_net* net, int batch, int top_n, int32_t* d_labels, int32_t* d_values, n2d2b_stream stream)
{
    if (!net || !d_labels) return fail(N2D2B_ERR_INVALID, "net and d_labels must not be NULL");
    if (!net->finalized) return fail(N2D2B_ERR_STATE, "estimated labels before finalize");
    if (!net->last_input) return fail(N2D2B_ERR_STATE, "estimated labels before a forward pass");
    if (batch < 0 || batch > net->max_batch) return fail(N2D2B_ERR_TOO_LARGE, "batch out of range");
    const int ft = final_tensor_of(net);
    const TensorRec& t = net->tensors[ft];
    if (top_n < 1 || top_n > t.C) return fail(N2D2B_ERR_INVALID, "top_n must be in 1..%d (the number of classes)", t.C);
    if (t.C > 16384) return fail(N2D2B_ERR_TOO_LARGE, "top-N handles up to 16384 classes");
    CUDA_TRY(cudaSetDevice(net->device));
    const void* scores = tensor_ptr(net, ft, net->last_input);
    if (top_n == 1)   // the reference's top-1 branch: first maximum; the layouts coincide
        CUDA_TRY(launch_argmax(scores, t.dtype, t.is_unsigned, (size_t)batch * t.H * t.W, t.C, d_labels, d_values, (cudaStream_t)stream));
    else
        CUDA_TRY(launch_topn(scores, t.dtype, t.is_unsigned, (size_t)batch * t.H * t.W, (size_t)t.H * t.W, t.C, top_n, d_labels,
                             d_values, (cudaStream_t)stream));
    return 0;
}

int n2d2b_net_estimated_labels_topn_host(n2d2b_net* net, int batch, int top_n, int32_t* h_labels, int32_t* h_values)
{
    if (!net || !h_labels) return fail(N2D2B_ERR_INVALID, "net and h_labels must not be NULL");
    if (!net->finalized) return fail(N2D2B_ERR_STATE, "estimated labels before finalize");
    if (batch < 0 || batch > net->max_batch) return fail(N2D2B_ERR_TOO_LARGE, "batch out of range");
    const TensorRec& t = net->tensors[final_tensor_of(net)];
    if (top_n < 1 || top_n > t.C) return fail(N2D2B_ERR_INVALID, "top_n must be in 1..%d (the number of classes)", t.C);
    CUDA_TRY(cudaSetDevice(net->device));
    const size_t n = (size_t)batch * top_n * t.H * t.W;
    if (n == 0) return 0;
    if (net->labels_scratch_bytes < 2 * n * sizeof(int32_t)) {
        cudaFree(net->d_labels_scratch);
        net->d_labels_scratch = nullptr;
        net->labels_scratch_bytes = 0;
        CUDA_TRY(cudaMalloc(&net->d_labels_scratch, 2 * n * sizeof(int32_t)));
        net->labels_scratch_bytes = 2 * n * sizeof(int32_t);
    }
    int32_t* d_labels = (int32_t*)net->d_labels_scratch;
    int32_t* d_values = d_labels + n;
    // the legacy stream orders this after the forward pass on any blocking stream
    if (int rc = n2d2b_net_estimated_labels_topn(net, batch, top_n, d_labels, d_values, nullptr)) return rc;
    CUDA_TRY(cudaMemcpy(h_labels, d_labels, n * sizeof(int32_t), cudaMemcpyDeviceToHost));
    if (h_values) CUDA_TRY(cudaMemcpy(h_values, d_values, n * sizeof(int32_t), cudaMemcpyDeviceToHost));
    return 0;
}

int n2d2b_quantize_stimuli(int device, const float* d_in, int batch, int channels, int height, int width, int nb_bits,
                           int env_unsigned, void* d_out, n2d2b_stream stream)
{
    if (!d_in || !d_out) return fail(N2D2B_ERR_INVALID, "device buffers must not be NULL");
    if (batch < 0 || channels < 1 || height < 1 || width < 1) return fail(N2D2B_ERR_INVALID, "invalid stimuli dimensions");
    if (nb_bits < 2 || nb_bits > 8) return fail(N2D2B_ERR_INVALID, "nb_bits must be in 2..8 (the path carries 8-bit stimuli)");
    CUDA_TRY(cudaSetDevice(device));
    const int hi = env_unsigned ? (1 << nb_bits) - 1 : (1 << (nb_bits - 1)) - 1;
    const int lo = env_unsigned ? 0 : -(1 << (nb_bits - 1));
    CUDA_TRY(launch_quantize_stimuli(d_in, batch, channels, height, width, (float)hi, lo, hi, d_out, (cudaStream_t)stream));
    return 0;
}

int n2d2b_net_num_tensors(const n2d2b_net* net) { return net ? (int)net->tensors.size() : fail(N2D2B_ERR_INVALID, "net must not be NULL"); }

int n2d2b_net_tensor_info(const n2d2b_net* net, int id, n2d2b_tensor_info* info)
{
    if (!net || !info) return fail(N2D2B_ERR_INVALID, "net and info must not be NULL");
    if (id < 0 || id >= (int)net->tensors.size()) return fail(N2D2B_ERR_INVALID, "unknown tensor id %d", id);
    const TensorRec& t = net->tensors[id];
    info->channels = t.C; info->height = t.H; info->width = t.W;
    info->dtype = t.dtype; info->is_unsigned = t.is_unsigned; info->producer = t.producer;
    info->readable = (t.readable && (id == 0 || t.buffer >= 0 || !net->finalized)) ? 1 : 0;
    return 0;
}

int n2d2b_net_read_tensor(n2d2b_net* net, int id, int batch, void* host_dst, size_t bytes)
{
    if (!net || !host_dst) return fail(N2D2B_ERR_INVALID, "net and host_dst must not be NULL");
    if (!net->finalized) return fail(N2D2B_ERR_STATE, "read before finalize");
    if (id < 0 || id >= (int)net->tensors.size()) return fail(N2D2B_ERR_INVALID, "unknown tensor id %d", id);
    const TensorRec& t = net->tensors[id];
    if (batch < 0 || batch > net->max_batch) return fail(N2D2B_ERR_TOO_LARGE, "batch out of range");
    const size_t need = t.bytes_per_image() * (size_t)batch;
    if (bytes < need) return fail(N2D2B_ERR_INVALID, "destination holds %zu bytes, the tensor needs %zu", bytes, need);
    const void* src = tensor_ptr(net, id, net->last_input);
    if (!src || !t.readable) return fail(N2D2B_ERR_STATE, "tensor %d is not kept (finalize with N2D2B_KEEP_ALL_OUTPUTS)", id);
    CUDA_TRY(cudaSetDevice(net->device));
    CUDA_TRY(cudaDeviceSynchronize());
    CUDA_TRY(cudaMemcpy(host_dst, src, need, cudaMemcpyDeviceToHost));
    return check_status(net);
}

int n2d2b_net_weight_bytes(const n2d2b_net* net, size_t* total_bytes, size_t* packed4_bytes)
{
    if (!net || !net->finalized) return fail(N2D2B_ERR_STATE, "the network is not finalized");
    size_t total = 0, packed = 0;
    for (const CellRec& c : net->cells) {
        total += c.d_weight_bytes;
        if (c.engine == ENG_TCGEN05 && c.plan.w4) packed += c.d_weight_bytes;
    }
    if (total_bytes) *total_bytes = total;
    if (packed4_bytes) *packed4_bytes = packed;
    return 0;
}

int n2d2b_net_launches_per_forward(const n2d2b_net* net)
{
    if (!net || !net->finalized) return fail(N2D2B_ERR_STATE, "the network is not finalized");
    return net->launches;
}

const char* n2d2b_net_cell_engine(const n2d2b_net* net, int cell)
{
    if (!net || cell < 0 || cell >= (int)net->cells.size()) return "";
    switch (net->cells[cell].engine) {
    case ENG_TCGEN05: {
        const CellRec& c = net->cells[cell];
        const bool pair = c.plan.pair && c.fast.enabled && !c.fast.wide && c.residual < 0
                          && net->tensors[c.output].dtype == DT_I8 && c.geom.O % 32 == 0;
        if (c.geom.groups > 1) return "depthwise-tcgen05";
        return pair ? "tcgen05-pair" : (c.plan.w4 ? "tcgen05-w4" : "tcgen05");
    }
    case ENG_SIMT: return "simt";
    case ENG_DEPTHWISE: return "depthwise";
    case ENG_POOL: return "pool";
    case ENG_SUM: return "sum";
    case ENG_FUSED: return "fused";
    case ENG_STEM: return "stem-tcgen05";
    case ENG_STEM_S2D: return net->cells[cell].pool_fused ? "stem-pool-tcgen05" : "stem-tcgen05";
    case ENG_PATCH: return net->cells[cell].geom.groups > 1 ? "depthwise-tcgen05" : "patch-tcgen05";
    }
    return "";
}

int n2d2b_scaling_propagate(int device, const int32_t* d_in, void* d_out, size_t nb_pixels, const n2d2b_quant* quant,
                            n2d2b_stream stream)
{
    if (!quant) return fail(N2D2B_ERR_INVALID, "quant must not be NULL");
    if (!d_in || !d_out) return fail(N2D2B_ERR_INVALID, "device buffers must not be NULL");
    if (quant->scaling.mode == SC_NONE) return fail(N2D2B_ERR_INVALID, "a NONE scaling has nothing to do");
    CUDA_TRY(cudaSetDevice(device));
    QuantHost q;
    if (int rc = validate_quant(quant, quant->scaling.nb_channels, false, q, nullptr)) return rc;
    if (int rc = upload_quant(q)) return rc;
    SumInputs ins{};
    ins.n = 1;
    ins.ptr[0] = d_in;
    ins.dtype[0] = DT_I32;
    cudaError_t e = launch_elemwise_sum(ins, nb_pixels, q.nb_channels, q.dev, d_out, DT_I8, (cudaStream_t)stream);
    cudaError_t e2 = cudaStreamSynchronize((cudaStream_t)stream);
    cudaFree(q.d_blob);
    if (e != cudaSuccess) return fail(N2D2B_ERR_CUDA, "scaling kernel launch failed: %s", cudaGetErrorString(e));
    if (e2 != cudaSuccess) return fail(N2D2B_ERR_CUDA, "scaling kernel failed: %s", cudaGetErrorString(e2));
    return 0;
}

}  // extern "C"
