// Exercises the C++ host classes (n2d2_b200/host/N2D2.hpp) the way the reference's own cell tests do:
// build cells with the reference's constructors, run DeepNet::test, compare every value with a CPU
// computation - here the oracle (test infrastructure), which follows the reference's CPU cells.
//
//   test_host_api            runs the mnist24 topology (8-bit, SingleShift) on cuda:0, exit 0 = equal
//   test_host_api --no-gpu   checks that DeepNet::initialize fails loudly without a device
#include <cstdio>
#include <cstring>
#include <numeric>

#include "../../n2d2_b200/host/N2D2.hpp"
#include "../../oracle/n2d2_oracle.h"

using namespace N2D2;

struct Lcg {
    uint64_t s;
    explicit Lcg(uint64_t seed) : s(seed) {}
    uint32_t next() { s = s * 6364136223846793005ull + 1442695040888963407ull; return (uint32_t)(s >> 33); }
    int range(int lo, int hi) { return lo + (int)(next() % (uint32_t)(hi - lo + 1)); }
};

struct Layer {
    std::vector<int8_t> w;        // reference order: OIHW
    std::vector<int32_t> b;
    std::vector<unsigned char> shift;
};

static Layer draw(Lcg& g, int O, int K)
{
    Layer l;
    l.w.resize((size_t)O * K);
    for (auto& v : l.w) v = (int8_t)g.range(-127, 127);
    l.b.resize(O);
    for (auto& v : l.b) v = g.range(-4096, 4096);
    l.shift.resize(O);
    for (auto& v : l.shift) v = (unsigned char)g.range(6, 12);
    return l;
}

static std::vector<float> to_f(const std::vector<int8_t>& v) { return std::vector<float>(v.begin(), v.end()); }
static std::vector<float> to_f(const std::vector<int32_t>& v) { return std::vector<float>(v.begin(), v.end()); }

int main(int argc, char** argv)
{
    const bool no_gpu = argc > 1 && !strcmp(argv[1], "--no-gpu");
    const int B = 64, C = 1, H = 24, W = 24;
    if (no_gpu) {
        try {
            DeepNet dn(C, H, W);
            auto lin = std::make_shared<LinearActivation>();
            lin->setActivationScaling(Scaling::singleShiftScaling(std::vector<unsigned char>(4, 3), false, {}));
            auto fc = std::make_shared<FcCell>("fc", 4, lin);
            fc->setWeights(std::vector<int8_t>((size_t)4 * C * H * W, 1));
            dn.addCell(fc, {});
            dn.initialize(1);     // device resources are created here: no GPU, no network
        } catch (const std::runtime_error& e) {
            printf("failed loudly as expected: %s\n", e.what());
            return 0;
        }
        fprintf(stderr, "DeepNet::initialize succeeded without a GPU\n");
        return 1;
    }

    // twice: dense, and with a sparse connection map on the second convolution (the reference's mnist24 model wires
    // conv2 to conv1 through a Mapping table; this one connects output o to 3-7 consecutive channels starting at o)
    for (int sparse = 0; sparse < 2; ++sparse) {
    std::vector<bool> mapping((size_t)24 * 16, false);
    std::vector<uint8_t> maps((size_t)24 * 16, 0);
    for (int o = 0; o < 24; ++o)
        for (int c = 0; c < 16; ++c) {
            const bool on = ((c - o) % 16 + 16) % 16 < 3 + (o % 5);
            mapping[(size_t)o * 16 + c] = on;
            maps[(size_t)o * 16 + c] = on ? 1 : 0;
        }
    Lcg g(12345 + sparse);
    Layer l1 = draw(g, 16, 1 * 4 * 4), l2 = draw(g, 24, 16 * 5 * 5), l3 = draw(g, 150, 24 * 4 * 4), l4 = draw(g, 10, 150);
    std::vector<uint8_t> stimuli((size_t)B * H * W * C);
    for (auto& v : stimuli) v = (uint8_t)g.range(0, 255);

    // ---- the network, written like reference code ----
    DeepNet deepNet(C, H, W);
    auto relu = [](const Layer& l) {
        auto a = std::make_shared<RectifierActivation>();
        a->setActivationScaling(Scaling::singleShiftScaling(l.shift, false, {}));
        return a;
    };
    auto conv1 = std::make_shared<ConvCell>("conv1", std::vector<unsigned>{4, 4}, 16, std::vector<unsigned>{1, 1},
                                            std::vector<unsigned>{2, 2}, std::vector<int>{0, 0}, std::vector<unsigned>{1, 1}, relu(l1));
    conv1->setWeights(l1.w); conv1->setBiases(l1.b); conv1->setQuantized(8);
    auto conv2 = std::make_shared<ConvCell>("conv2", std::vector<unsigned>{5, 5}, 24, std::vector<unsigned>{1, 1},
                                            std::vector<unsigned>{2, 2}, std::vector<int>{0, 0}, std::vector<unsigned>{1, 1}, relu(l2));
    conv2->setWeights(l2.w); conv2->setBiases(l2.b); conv2->setQuantized(8);
    if (sparse) conv2->setMapping(mapping);
    auto fc1 = std::make_shared<FcCell>("fc1", 150, relu(l3));
    fc1->setWeights(l3.w); fc1->setBiases(l3.b); fc1->setQuantized(8);
    auto lin = std::make_shared<LinearActivation>();
    lin->setActivationScaling(Scaling::singleShiftScaling(l4.shift, false, {}));
    auto fc2 = std::make_shared<FcCell>("fc2", 10, lin);
    fc2->setWeights(l4.w); fc2->setBiases(l4.b); fc2->setQuantized(8);
    deepNet.addCell(conv1, {});
    deepNet.addCell(conv2, {conv1});
    deepNet.addCell(fc1, {conv2});
    deepNet.addCell(fc2, {fc1});
    if (conv1->getOutputsWidth() != 11 || conv2->getOutputsWidth() != 4) { fprintf(stderr, "wrong output dims\n"); return 1; }
    if (!conv1->isOutputUnsigned() || fc2->isOutputUnsigned()) { fprintf(stderr, "wrong signedness\n"); return 1; }
    deepNet.initialize(B, true);
    const std::vector<int> logits = deepNet.test(stimuli, B);

    // ---- the same on the CPU, NCHW float like the reference ----
    std::vector<float> x((size_t)B * C * H * W);
    for (int b = 0; b < B; ++b)
        for (int y = 0; y < H; ++y)
            for (int xx = 0; xx < W; ++xx) x[((size_t)b * H + y) * W + xx] = stimuli[((size_t)b * H + y) * W + xx];
    auto scale = [&](std::vector<float>& t, int Cn, int HW, const Layer& l, int act, int uns) {
        n2d2o_scaling_f32(t.data(), t.data(), B, Cn, HW, 4, nullptr, nullptr, 0, nullptr, l.shift.data(), nullptr, 0, nullptr, 8, uns);
        n2d2o_activation_f32(t.data(), t.size(), act, 0.0f, 0.0f);
    };
    std::vector<float> t1((size_t)B * 16 * 11 * 11), t2((size_t)B * 24 * 4 * 4), t3((size_t)B * 150), t4((size_t)B * 10);
    { auto w = to_f(l1.w), bb = to_f(l1.b);
      n2d2o_conv_f32(x.data(), W, H, C, B, w.data(), 4, 4, 1, 16, nullptr, 1, 2, 2, 0, 0, 0, 0, 1, 1, 0, 0, t1.data());
      n2d2o_add_bias_f32(t1.data(), 11, 11, 16, B, bb.data()); scale(t1, 16, 121, l1, 1, 1); }
    { auto w = to_f(l2.w), bb = to_f(l2.b);
      n2d2o_conv_f32(t1.data(), 11, 11, 16, B, w.data(), 5, 5, 16, 24, sparse ? maps.data() : nullptr, 1, 2, 2, 0, 0, 0, 0, 1, 1, 0, 0, t2.data());
      n2d2o_add_bias_f32(t2.data(), 4, 4, 24, B, bb.data()); scale(t2, 24, 16, l2, 1, 1); }
    { auto w = to_f(l3.w), bb = to_f(l3.b); n2d2o_fc_f32(t2.data(), 384, B, w.data(), bb.data(), 150, t3.data()); scale(t3, 150, 1, l3, 1, 1); }
    { auto w = to_f(l4.w), bb = to_f(l4.b); n2d2o_fc_f32(t3.data(), 150, B, w.data(), bb.data(), 10, t4.data()); scale(t4, 10, 1, l4, 0, 0); }

    size_t bad = 0;
    for (size_t i = 0; i < t4.size(); ++i) bad += (logits[i] != (int)t4[i]);
    // an inner cell too (NHWC on the device, NCHW in the oracle)
    const std::vector<int> c2 = deepNet.getOutputs("conv2", B);
    for (int b = 0; b < B; ++b)
        for (int c = 0; c < 24; ++c)
            for (int p = 0; p < 16; ++p) bad += (c2[((size_t)b * 16 + p) * 24 + c] != (int)t2[((size_t)b * 24 + c) * 16 + p]);
    // error convention: exceptions, as in the reference
    bool threw = false;
    try { deepNet.getCell<ConvCell>("nope"); } catch (const std::runtime_error&) { threw = true; }
    if (!threw) { fprintf(stderr, "getCell on a missing cell did not throw\n"); return 1; }
    threw = false;
    try { deepNet.test(std::vector<uint8_t>((size_t)(B + 1) * H * W), B + 1); } catch (const std::runtime_error&) { threw = true; }
    if (!threw) { fprintf(stderr, "oversize batch did not throw\n"); return 1; }
    if (sparse && (conv2->isConnection(5, 0) || !conv2->isConnection(2, 0))) { fprintf(stderr, "isConnection disagrees with the map\n"); return 1; }
    printf("host api (%s): %zu mismatches over %zu logits + %zu inner values\n", sparse ? "sparse conv2" : "dense", bad, t4.size(), t2.size());
    if (bad) return 1;
    }
    return 0;
}
