// Post-training quantization front-end (n2d2_b200/host/DeepNetQuantization.hpp).
//
//   test_quantization --kat                known answers of the two scaling approximations and the graph rewrite of a
//                                          residual network (no GPU needed)
//   test_quantization --run <mode> <perch> quantizes two small float networks (mode: fixed | single | double; perch: 0 | 1)
//                                          from value-range calibration, runs the integer networks on cuda:0 and compares
//                                          them with the float networks computed by the CPU oracle, the way the reference
//                                          tests its quantization: by how well the quantized network tracks the float one
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <random>

#include "../../n2d2_b200/host/DeepNetQuantization.hpp"
#include "../../oracle/n2d2_oracle.h"

using namespace N2D2;

#define CHECK(cond)                                                                      \
    do {                                                                                 \
        if (!(cond)) { fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); return 1; } \
    } while (0)

static bool near(double a, double b, double tol = 1e-6) { return std::fabs(a - b) <= tol * std::max(1.0, std::fabs(b)); }

static int known_answers()
{
    typedef DeepNetQuantization Q;
    // ---- fixed point: the largest scaling decides the fractional bits
    {
        ScalingMode m = ScalingMode::FIXED_MULT16;
        auto r = Q::approximateScalingWithFixedPoint(m, {0.5f, 0.25f});
        CHECK(m == ScalingMode::FIXED_MULT16 && r.first == 15 && r.second[0] == 16384 && r.second[1] == 8192);
        m = ScalingMode::FIXED_MULT16;
        r = Q::approximateScalingWithFixedPoint(m, {40000.0f});                 // does not fit 16 bits: falls back to 32
        CHECK(m == ScalingMode::FIXED_MULT32 && r.first == 15 && r.second[0] == 1310720000);
        m = ScalingMode::FIXED_MULT32;
        r = Q::approximateScalingWithFixedPoint(m, {0.001953125f});              // 2^-9: 2^31-1 over it is just under 2^40
        CHECK(r.first == 39 && r.second[0] == (1 << 30));
        m = ScalingMode::FIXED_MULT16;
        r = Q::approximateScalingWithFixedPoint(m, {1e-13f});                    // capped at 50 fractional bits
        CHECK(r.first == 50 && r.second[0] == (std::int32_t)std::round(1e-13f * (float)(1ull << 50)));
        bool threw = false;
        m = ScalingMode::FIXED_MULT32;
        try { Q::approximateScalingWithFixedPoint(m, {3e9f}); } catch (const std::runtime_error&) { threw = true; }
        CHECK(threw);
    }
    // ---- powers of two
    {
        auto r = Q::approximateScalingWithPowerOf2Divs(0.3f, 1);     // 2^-2 covers 0.83 of it: below the threshold, so 2^-1 with p = 1.67
        CHECK(r.first.size() == 1 && r.first[0] == 1 && near(r.second, 0.5 / 0.3f));
        r = Q::approximateScalingWithPowerOf2Divs(0.3f, 2);          // 2^-2 + 2^-5 = 0.94 of it -> 2^-2 + 2^-4 = 0.3125
        CHECK(r.first[0] == 2 && r.first[1] == 4 && near(r.second, 0.3125 / 0.3f));
        r = Q::approximateScalingWithPowerOf2Divs(0.5f, 1);
        CHECK(r.first[0] == 1 && r.second == 1.0);
        r = Q::approximateScalingWithPowerOf2Divs(0.5f, 2);          // exact after one term: split into two halves
        CHECK(r.first[0] == 2 && r.first[1] == 2 && r.second == 1.0);
        r = Q::approximateScalingWithPowerOf2Divs(1.0f, 1);
        CHECK(r.first[0] == 0 && r.second == 1.0);
        r = Q::approximateScalingWithPowerOf2Divs(0.2525f, 1);       // 2^-2 covers 0.99 of it: counts as exact
        CHECK(r.first[0] == 2 && r.second == 1.0);
        r = Q::approximateScalingWithPowerOf2Divs(0.01f, 2);         // 2^-7 + 2^-9 = 0.977 of it -> 2^-7 + 2^-8
        CHECK(r.first[0] == 7 && r.first[1] == 8 && near(r.second, (1.0 / 128 + 1.0 / 256) / 0.01f));
        bool threw = false;
        try { Q::approximateScalingWithPowerOf2Divs(1.5f, 1); } catch (const std::runtime_error&) { threw = true; }
        CHECK(threw);
    }
    return 0;
}

// ------------------------------------------------------------------------------------------------------------
struct FloatNet {
    // a residual block or a plain chain, NCHW float parameters in the reference's order
    bool residual;
    int C = 3, H = 16, W = 16, F = 16, classes = 10;
    std::vector<float> w1, b1, w2, b2, wf, bf;
};

static FloatNet draw_net(bool residual, unsigned seed)
{
    FloatNet n;
    n.residual = residual;
    std::mt19937 g(seed);
    std::normal_distribution<float> nd(0.0f, 1.0f);
    auto fill = [&](std::vector<float>& v, size_t count, float sigma) { v.resize(count); for (auto& x : v) x = sigma * nd(g); };
    fill(n.w1, (size_t)n.F * n.C * 9, 0.25f); fill(n.b1, n.F, 0.1f);
    fill(n.w2, (size_t)n.F * n.F * 9, 0.09f); fill(n.b2, n.F, 0.1f);
    fill(n.wf, (size_t)n.classes * n.F * 8 * 8, 0.05f); fill(n.bf, n.classes, 0.1f);
    // uneven output channels, so that per-channel rescaling has something to do
    for (int o = 0; o < n.F; ++o)
        for (int i = 0; i < n.F * 9; ++i) n.w2[(size_t)o * n.F * 9 + i] *= (0.3f + 0.1f * o);
    return n;
}

// float forward with the oracle's float cells; returns every tensor (NCHW)
struct FloatOutputs { std::vector<float> c1, c2, sum, pool, fc; };
static FloatOutputs float_forward(const FloatNet& n, const std::vector<float>& x, int B)
{
    FloatOutputs o;
    const int H = n.H, W = n.W, F = n.F;
    o.c1.resize((size_t)B * F * H * W); o.c2.resize(o.c1.size()); o.sum.resize(o.c1.size());
    o.pool.resize((size_t)B * F * (H / 2) * (W / 2)); o.fc.resize((size_t)B * n.classes);
    n2d2o_conv_f32(x.data(), W, H, n.C, B, n.w1.data(), 3, 3, n.C, F, nullptr, 1, 1, 1, 1, 1, 1, 1, 1, 1, 0, 0, o.c1.data());
    n2d2o_add_bias_f32(o.c1.data(), W, H, F, B, n.b1.data());
    n2d2o_activation_f32(o.c1.data(), o.c1.size(), 1, 0.0f, 0.0f);
    n2d2o_conv_f32(o.c1.data(), W, H, F, B, n.w2.data(), 3, 3, F, F, nullptr, 1, 1, 1, 1, 1, 1, 1, 1, 1, 0, 0, o.c2.data());
    n2d2o_add_bias_f32(o.c2.data(), W, H, F, B, n.b2.data());
    const std::vector<float>* tail = &o.c2;
    if (n.residual) {
        for (size_t i = 0; i < o.sum.size(); ++i) o.sum[i] = o.c2[i] + o.c1[i];
        n2d2o_activation_f32(o.sum.data(), o.sum.size(), 1, 0.0f, 0.0f);
        tail = &o.sum;
    } else {
        n2d2o_activation_f32(o.c2.data(), o.c2.size(), 1, 0.0f, 0.0f);
    }
    n2d2o_pool_max_f32(tail->data(), W, H, F, B, 2, 2, 2, 2, 0, 0, o.pool.data());
    n2d2o_fc_f32(o.pool.data(), F * (H / 2) * (W / 2), B, n.wf.data(), n.bf.data(), n.classes, o.fc.data());
    return o;
}

static double max_abs(const std::vector<float>& v) { double m = 0; for (float x : v) m = std::max(m, (double)std::fabs(x)); return m; }

// the float network as host cells (float parameters, no scalings yet)
static void build_graph(DeepNet& dn, const FloatNet& n)
{
    auto conv1 = std::make_shared<ConvCell>("conv1", std::vector<unsigned>{3, 3}, n.F, std::vector<unsigned>{1, 1}, std::vector<unsigned>{1, 1},
                                            std::vector<int>{1, 1}, std::vector<unsigned>{1, 1}, std::make_shared<RectifierActivation>());
    conv1->setFloatWeights(n.w1); conv1->setFloatBiases(n.b1);
    std::shared_ptr<Activation> act2;
    if (n.residual) act2 = std::make_shared<LinearActivation>(); else act2 = std::make_shared<RectifierActivation>();
    auto conv2 = std::make_shared<ConvCell>("conv2", std::vector<unsigned>{3, 3}, n.F, std::vector<unsigned>{1, 1}, std::vector<unsigned>{1, 1},
                                            std::vector<int>{1, 1}, std::vector<unsigned>{1, 1}, act2);
    conv2->setFloatWeights(n.w2); conv2->setFloatBiases(n.b2);
    dn.addCell(conv1, {});
    dn.addCell(conv2, {conv1});
    std::shared_ptr<Cell> tail = conv2;
    if (n.residual) {
        auto sum = std::make_shared<ElemWiseCell>("sum", n.F, ElemWiseCell::Sum, std::make_shared<RectifierActivation>());
        dn.addCell(sum, {conv2, conv1});
        tail = sum;
    }
    auto pool = std::make_shared<PoolCell>("pool", std::vector<unsigned>{2, 2}, n.F, std::vector<unsigned>{2, 2}, std::vector<unsigned>{0, 0}, PoolCell::Max);
    dn.addCell(pool, {tail});
    auto fc = std::make_shared<FcCell>("fc", n.classes, std::make_shared<LinearActivation>());
    fc->setFloatWeights(n.wf); fc->setFloatBiases(n.bf);
    dn.addCell(fc, {pool});
}

static int graph_rewrite()
{
    // a residual block forces all-signed data in the reference (its analysis throws on mixed signedness otherwise)
    DeepNetExport::mUnsignedData() = false;
    DeepNetExport::mEnvDataUnsigned() = false;
    const FloatNet n = draw_net(true, 5);
    DeepNet dn(n.C, n.H, n.W);
    build_graph(dn, n);
    DeepNetExport::mUnsignedData() = true;
    bool threw = false;
    try { DeepNetQuantization(dn).quantizeFreeParemeters(8); } catch (const std::runtime_error& e) { threw = strstr(e.what(), "mixes signed and unsigned") != nullptr; }
    CHECK(threw);   // conv2 (Linear, signed) + conv1 (Rectifier, unsigned) into one sum
    DeepNetExport::mUnsignedData() = false;
    DeepNet dn2(n.C, n.H, n.W);
    build_graph(dn2, n);
    std::unordered_map<std::string, double> thr = {{"conv1", 3.0}, {"conv2", 2.0}, {"sum", 4.0}, {"fc", 5.0}};
    DeepNetQuantization q(dn2);
    q.quantizeNetwork(thr, 8, ScalingMode::SINGLE_SHIFT, false);
    // every `_rescale_act` cell went into its cell's activation; the sum's two inputs sit at different scales, so
    // one branch keeps a `_rescale_branch` ScalingCell (fixed point, as the shift modes prescribe for ScalingCells)
    size_t scalingCells = 0;
    for (const auto& kv : dn2.getCells()) {
        if (auto* sc = dynamic_cast<ScalingCell*>(kv.second.get())) {
            ++scalingCells;
            CHECK(sc->getScaling().getMode() == ScalingMode::FIXED_MULT16);
            CHECK(kv.first.find("_rescale_branch") != std::string::npos);
        } else if (kv.second->getActivation()) {
            // one shift, or fixed point where the scaling exceeds 1 (no shift form exists for that)
            const ScalingMode m = kv.second->getActivation()->getActivationScaling().getMode();
            CHECK(m == ScalingMode::SINGLE_SHIFT || m == ScalingMode::FIXED_MULT16);
        }
        // (a `_rescale_branch` cell inserted next to a `_rescale_act` one keeps that cell's name as its prefix)
        CHECK(kv.first.size() < 12 || kv.first.compare(kv.first.size() - 12, 12, "_rescale_act") != 0);
        CHECK(kv.second->getQuantizedNbBits() == 8);
    }
    CHECK(scalingCells >= 1);
    auto conv1 = dn2.getCell<ConvCell>("conv1");
    CHECK(conv1->getActivation()->getActivationScaling().getMode() == ScalingMode::SINGLE_SHIFT);
    int wmax = 0;
    for (std::int8_t w : conv1->getWeights()) wmax = std::max(wmax, std::abs((int)w));
    printf("conv1: max |weight| %d\n", wmax);
    CHECK(wmax <= 127 && wmax >= 63);   // scaled to +-127, then divided by the single-shift precision (< 2)
    CHECK(dn2.getParentCells("sum").size() == 2);
    printf("graph rewrite: %zu layers, %zu ScalingCell(s) left\n", dn2.getLayers().size() - 1, scalingCells);
    return 0;
}

// The committed vectors of the reference's own approximateScalingWithPowerOf2Divs / approximateScalingWithFixedPoint
// (tests/golden/quantization_golden.txt, written by tests/golden/make_quantization_golden.py): every value must be equal
static int golden(const char* path)
{
    typedef DeepNetQuantization Q;
    FILE* f = fopen(path, "r");
    if (!f) { fprintf(stderr, "cannot open %s\n", path); return 2; }
    char line[8192];
    int cases = 0;
    while (fgets(line, sizeof line, f)) {
        if (line[0] == '#' || line[0] == '\n') continue;
        char* bar = strchr(line, '|');
        if (!bar) { fclose(f); return 2; }
        *bar = 0;
        std::vector<std::string> in, out;
        for (char* t = strtok(line, " \n"); t; t = strtok(nullptr, " \n")) in.push_back(t);
        for (char* t = strtok(bar + 1, " \n"); t; t = strtok(nullptr, " \n")) out.push_back(t);
        if (in[0] == "p2") {
            const float scaling = (float)strtod(in[1].c_str(), nullptr);
            const std::size_t nb = (std::size_t)atoi(in[2].c_str());
            const auto r = Q::approximateScalingWithPowerOf2Divs(scaling, nb);
            bool ok = r.second == strtod(out[0].c_str(), nullptr) && r.first.size() == nb && out.size() == nb + 1;
            for (std::size_t i = 0; ok && i < nb; ++i) ok = r.first[i] == (unsigned char)atoi(out[1 + i].c_str());
            if (!ok) { fprintf(stderr, "power-of-two case %s x%zu differs: precision %a\n", in[1].c_str(), nb, r.second); fclose(f); return 1; }
        } else if (in[0] == "fx") {
            ScalingMode mode = atoi(in[1].c_str()) == 2 ? ScalingMode::FIXED_MULT16 : ScalingMode::FIXED_MULT32;
            std::vector<Float_T> sc;
            for (std::size_t i = 2; i < in.size(); ++i) sc.push_back((Float_T)strtod(in[i].c_str(), nullptr));
            const int wantFrac = atoi(out[0].c_str());
            bool threw = false;
            std::pair<std::size_t, std::vector<std::int32_t> > r;
            try { r = Q::approximateScalingWithFixedPoint(mode, sc); } catch (const std::runtime_error&) { threw = true; }
            bool ok = threw == (wantFrac < 0);
            if (ok && !threw) {
                ok = (int)r.first == wantFrac && (int)(mode == ScalingMode::FIXED_MULT16 ? 2 : 3) == atoi(out[1].c_str())
                     && r.second.size() == sc.size() && out.size() == sc.size() + 2;
                for (std::size_t i = 0; ok && i < sc.size(); ++i) ok = r.second[i] == (std::int32_t)atoll(out[2 + i].c_str());
            }
            if (!ok) { fprintf(stderr, "fixed-point case differs (mode %s, first scaling %s)\n", in[1].c_str(), in[2].c_str()); fclose(f); return 1; }
        } else {
            fclose(f);
            return 2;
        }
        ++cases;
    }
    fclose(f);
    printf("%d golden cases ok\n", cases);
    return cases > 0 ? 0 : 2;
}

// Calibration statistics of one float run, fed the way a caller's float framework would (two passes: ranges, then
// histograms over those ranges)
struct Stats {
    std::unordered_map<std::string, RangeStats> range;
    std::unordered_map<std::string, Histogram> hist;
};
static Stats collect_stats(DeepNet& dn, const FloatNet& n, const std::vector<float>& x, const FloatOutputs& o, ClippingMode mode,
                           bool envUnsigned)
{
    Stats st;
    DeepNetQuantization q(dn);
    std::vector<std::pair<std::string, const std::vector<float>*> > outs
        = {{"env", &x}, {"conv1", &o.c1}, {"conv2", &o.c2}, {"pool", &o.pool}, {"fc", &o.fc}};
    if (n.residual) outs.push_back({"sum", &o.sum});
    // two halves, as two calibration batches (the second one may enlarge the histograms)
    for (int half = 0; half < 2; ++half)
        for (auto& kv : outs) {
            const size_t h = kv.second->size() / 2;
            q.reportOutputsRange(st.range, kv.first, kv.second->data() + half * h, half ? kv.second->size() - h : h);
        }
    for (int half = 0; half < 2; ++half)
        for (auto& kv : outs) {
            const size_t h = kv.second->size() / 2;
            q.reportOutputsHistogram(st.hist, st.range, kv.first, kv.second->data() + half * h, half ? kv.second->size() - h : h, 8,
                                     mode, envUnsigned);
        }
    return st;
}

// CPU checks of the statistics-driven front-end
static int stats_frontend(const std::string& dir)
{
    for (int variant = 0; variant < 2; ++variant) {
        const bool residual = variant == 1;
        DeepNetExport::mUnsignedData() = !residual;
        DeepNetExport::mEnvDataUnsigned() = !residual;
        const FloatNet n = draw_net(residual, 21 + variant);
        const int B = 8;
        std::mt19937 g(5);
        std::vector<float> x((size_t)B * n.C * n.H * n.W);
        for (auto& v : x) v = (float)(g() & 0xff) / 255.0f;
        const FloatOutputs ref = float_forward(n, x, B);
        DeepNet dn(n.C, n.H, n.W);
        build_graph(dn, n);
        Stats st = collect_stats(dn, n, x, ref, ClippingMode::MSE, !residual);
        // ranges are the extreme values, histograms hold every value, unsigned cells start at 0
        CHECK(near(st.range.at("conv2").maxVal(), *std::max_element(ref.c2.begin(), ref.c2.end())));
        CHECK(near(st.range.at("conv2").minVal(), *std::min_element(ref.c2.begin(), ref.c2.end())));
        CHECK(st.hist.at("conv1").getNbValues() == ref.c1.size());
        CHECK(st.hist.at("conv1").getNbBins() >= 16384);   // min(2^8 * 64, 65536), possibly enlarged
        CHECK((st.hist.at("conv1").getMinVal() == 0.0) == !residual);
        CHECK(st.hist.at("conv2").getMinVal() < 0.0 || !residual);   // a Linear activation in a signed network
        CHECK(near(DeepNetQuantization::getCellThreshold("fc", st.hist, st.range, 8, ClippingMode::NONE), max_abs(ref.fc)));
        const double mse = DeepNetQuantization::getCellThreshold("conv1", st.hist, st.range, 8, ClippingMode::MSE);
        const double kl = DeepNetQuantization::getCellThreshold("conv1", st.hist, st.range, 8, ClippingMode::KL_DIVERGENCE);
        const double qt = DeepNetQuantization::getCellThreshold("conv1", st.hist, st.range, 8, ClippingMode::QUANTILE, 0.999);
        CHECK(mse > 0 && mse <= st.hist.at("conv1").getMaxVal() && kl > 0 && kl <= st.hist.at("conv1").getMaxVal());
        CHECK(qt > 0 && qt < max_abs(ref.c1));
        // which statistics quantizeActivations asks for: the max pooling's for the cell above it, with clipping on
        // cells of more than two outputs only
        std::vector<std::string> asked;
        DeepNetQuantization(dn).quantizeNetwork([&](const Cell& cell, const std::string& statsName, bool clip) {
            asked.push_back(cell.getName() + ":" + statsName + ":" + (clip ? "1" : "0"));
            return DeepNetQuantization::getCellThreshold(statsName, st.hist, st.range, 8, ClippingMode::NONE);
        }, 8, ScalingMode::FIXED_MULT32, false);
        const std::string tail = residual ? "sum:sum:0" : "conv2:pool:1";
        CHECK(std::find(asked.begin(), asked.end(), tail) != asked.end());
        CHECK(std::find(asked.begin(), asked.end(), "conv1:conv1:1") != asked.end());
        CHECK(std::find(asked.begin(), asked.end(), "fc:fc:1") != asked.end());
        // clipWeights: no weight beyond the threshold of its cell's histogram, and some weights did move
        DeepNet dn2(n.C, n.H, n.W);
        build_graph(dn2, n);
        const auto before = dn2.getCell<Cell>("conv2")->getFreeParametersRange(Cell::Multiplicative);
        DeepNetQuantization(dn2).clipWeights(8, ClippingMode::MSE);
        const auto after = dn2.getCell<Cell>("conv2")->getFreeParametersRange(Cell::Multiplicative);
        CHECK(after.second <= before.second && after.first >= before.first);
        CHECK(after.second < before.second || after.first > before.first);
        // state files round-trip
        RangeStats::saveOutputsRange(dir + "/n2d2b_test_range.bin", st.range);
        Histogram::saveOutputsHistogram(dir + "/n2d2b_test_hist.bin", st.hist);
        std::unordered_map<std::string, RangeStats> r2;
        std::unordered_map<std::string, Histogram> h2;
        RangeStats::loadOutputsRange(dir + "/n2d2b_test_range.bin", r2);
        Histogram::loadOutputsHistogram(dir + "/n2d2b_test_hist.bin", h2);
        CHECK(r2.size() == st.range.size() && h2.size() == st.hist.size());
        CHECK(r2.at("fc").maxVal() == st.range.at("fc").maxVal() && r2.at("fc").moments() == st.range.at("fc").moments());
        CHECK(h2.at("conv2").getBins() == st.hist.at("conv2").getBins() && h2.at("conv2").getMaxVal() == st.hist.at("conv2").getMaxVal());
        remove((dir + "/n2d2b_test_range.bin").c_str());
        remove((dir + "/n2d2b_test_hist.bin").c_str());
    }
    return 0;
}

// clip: 0 = thresholds given as a map of value ranges; 1 / 2 / 3 = calibration statistics with no clipping, MSE,
// KL divergence
static int run(const char* mode_name, bool per_channel, int clip = 0)
{
    const ScalingMode mode = !strcmp(mode_name, "fixed") ? ScalingMode::FIXED_MULT32
                             : (!strcmp(mode_name, "single") ? ScalingMode::SINGLE_SHIFT : ScalingMode::DOUBLE_SHIFT);
    const int B = 64;
    int failures = 0;
    for (int variant = 0; variant < 2; ++variant) {
        const bool residual = variant == 1;
        // plain chain: unsigned data allowed (ReLU outputs and the stimuli are unsigned); residual: all signed
        DeepNetExport::mUnsignedData() = !residual;
        DeepNetExport::mEnvDataUnsigned() = !residual;
        const FloatNet n = draw_net(residual, 11 + variant);
        std::mt19937 g(3);
        std::vector<std::uint8_t> pixels((size_t)B * n.H * n.W * n.C);   // NHWC 8-bit images
        for (auto& p : pixels) p = (std::uint8_t)(g() & 0xff);
        // float stimuli in [0, 1] (NCHW), and what the quantized network is fed: trunc(x * 255) or trunc(x * 127)
        std::vector<float> x((size_t)B * n.C * n.H * n.W);
        std::vector<std::uint8_t> stimuli(pixels.size());
        const float inQuant = residual ? 127.0f : 255.0f;
        for (int b = 0; b < B; ++b)
            for (int y = 0; y < n.H; ++y)
                for (int xx = 0; xx < n.W; ++xx)
                    for (int c = 0; c < n.C; ++c) {
                        const std::uint8_t p = pixels[(((size_t)b * n.H + y) * n.W + xx) * n.C + c];
                        const float f = (float)p / 255.0f;
                        x[(((size_t)b * n.C + c) * n.H + y) * n.W + xx] = f;
                        stimuli[(((size_t)b * n.H + y) * n.W + xx) * n.C + c] = (std::uint8_t)(int)std::trunc(f * inQuant);
                    }
        const FloatOutputs ref = float_forward(n, x, B);
        std::unordered_map<std::string, double> thr = {{"conv1", max_abs(ref.c1)}, {"conv2", max_abs(ref.c2)}, {"fc", max_abs(ref.fc)}};
        if (residual) thr["sum"] = max_abs(ref.sum);
        DeepNet dn(n.C, n.H, n.W);
        build_graph(dn, n);
        double out_threshold = max_abs(ref.fc);
        if (clip == 0) {
            DeepNetQuantization(dn).quantizeNetwork(thr, 8, mode, per_channel);
        } else {
            const ClippingMode cm = clip == 1 ? ClippingMode::NONE : (clip == 2 ? ClippingMode::MSE : ClippingMode::KL_DIVERGENCE);
            Stats st = collect_stats(dn, n, x, ref, cm == ClippingMode::NONE ? ClippingMode::MSE : cm, !residual);
            out_threshold = DeepNetQuantization::getCellThreshold("fc", st.hist, st.range, 8, cm);
            DeepNetQuantization(dn).quantizeNetwork(st.hist, st.range, 8, cm, mode, per_channel);
        }
        dn.initialize(B);
        const std::vector<int> logits = dn.test(stimuli, B);
        {   // Target top-1 / top-3 of the host classes: first maximum, descending scores that are the labels' logits
            const std::vector<int> top1 = dn.getEstimatedLabels(B, 1);
            std::vector<int> scores3;
            const std::vector<int> top3 = dn.getEstimatedLabels(B, 3, &scores3);
            for (int b = 0; b < B; ++b) {
                int am = 0;
                for (int c = 1; c < n.classes; ++c)
                    if (logits[(size_t)b * n.classes + c] > logits[(size_t)b * n.classes + am]) am = c;
                if (top1[b] != am) { fprintf(stderr, "top-1 of image %d: %d, expected %d\n", b, top1[b], am); return 1; }
                for (int k = 0; k < 3; ++k) {
                    if (scores3[(size_t)b * 3 + k] != logits[(size_t)b * n.classes + top3[(size_t)b * 3 + k]]) return 1;
                    if (k && scores3[(size_t)b * 3 + k] > scores3[(size_t)b * 3 + k - 1]) return 1;
                }
            }
        }
        // the integer logits track the float ones: y_int ~ y_float / threshold * 127 (signed 8-bit output)
        const double scale = out_threshold / 127.0;
        double err = 0, norm = 0;
        int agree = 0;
        for (int b = 0; b < B; ++b) {
            int am_i = 0, am_f = 0;
            for (int c = 0; c < n.classes; ++c) {
                const double yi = logits[(size_t)b * n.classes + c] * scale, yf = ref.fc[(size_t)b * n.classes + c];
                err += (yi - yf) * (yi - yf);
                norm += yf * yf;
                if (logits[(size_t)b * n.classes + c] > logits[(size_t)b * n.classes + am_i]) am_i = c;
                if (ref.fc[(size_t)b * n.classes + c] > ref.fc[(size_t)b * n.classes + am_f]) am_f = c;
            }
            agree += (am_i == am_f);
        }
        const double rel = std::sqrt(err / norm);
        printf("%s per_channel=%d clip=%d %s: relative error %.4f, top-1 agreement %d / %d, %zu layers\n", mode_name, (int)per_channel, clip,
               residual ? "residual" : "chain", rel, agree, B, dn.getLayers().size() - 1);
        // 8 bits leave a few percent of noise; shift scalings are as exact as fixed-point ones because the parameters
        // absorb the approximation
        // (clipped thresholds saturate the largest logits: compare top-1 only there)
        if ((clip < 2 && !(rel < 0.08)) || agree < B * 85 / 100) ++failures;
    }
    return failures;
}

int main(int argc, char** argv)
{
    try {
        if (argc >= 2 && !strcmp(argv[1], "--kat")) {
            if (int rc = known_answers()) return rc;
            if (int rc = graph_rewrite()) return rc;
            printf("known answers ok\n");
            return 0;
        }
        if (argc >= 3 && !strcmp(argv[1], "--golden")) return golden(argv[2]);
        if (argc >= 2 && !strcmp(argv[1], "--stats")) {
            if (argc < 3) { fprintf(stderr, "--stats needs a scratch directory\n"); return 2; }
            if (int rc = stats_frontend(argv[2])) return rc;
            printf("statistics front-end ok\n");
            return 0;
        }
        if (argc >= 4 && !strcmp(argv[1], "--run")) return run(argv[2], atoi(argv[3]) != 0, argc >= 5 ? atoi(argv[4]) : 0);
    } catch (const std::exception& e) {
        fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
    fprintf(stderr, "usage: see the top of the source file\n");
    return 2;
}
