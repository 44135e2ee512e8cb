// Command-line front of n2d2_b200/host/Calibration.hpp for tests/test_calibration.py.
//   test_calibration case <kind> <seed> <n> <scale> <bits> <mode>   one calibration case, results as hex doubles
//   test_calibration state <dir>                                     writes <dir>/hist.bin and <dir>/range.bin
// The values of a case come from a 64-bit linear congruential generator and a fixed sequence of IEEE double
// operations, which the Python test repeats bit for bit.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "../../n2d2_b200/host/Calibration.hpp"

using namespace N2D2;

struct Lcg {
    unsigned long long x;
    double next()
    {
        x = x * 6364136223846793005ull + 1442695040888963407ull;
        return (double)(x >> 11) * (1.0 / 9007199254740992.0);
    }
};

// kind: bell = sum of four uniforms around 0; relu = its positive part; tail = bell with rare large values
static std::vector<double> draw(const std::string& kind, unsigned long long seed, std::size_t n, double scale)
{
    Lcg g{seed};
    std::vector<double> v(n);
    for (std::size_t i = 0; i < n; ++i) {
        const double u1 = g.next(), u2 = g.next(), u3 = g.next(), u4 = g.next(), u5 = g.next();
        double b = (((u1 + u2) + (u3 + u4)) - 2.0) * scale;
        if (kind == "relu") b = b > 0.0 ? b : 0.0;
        if (kind == "tail") b = b * (1.0 + 8.0 * ((u5 * u5) * (u5 * u5)));
        v[i] = (double)(float)b;   // the reference's tensors hold floats
    }
    return v;
}

static int run_case(int argc, char** argv)
{
    if (argc < 8) return 2;
    const std::string kind = argv[2];
    const unsigned long long seed = strtoull(argv[3], nullptr, 10);
    const std::size_t n = strtoull(argv[4], nullptr, 10);
    const double scale = strtod(argv[5], nullptr);
    const std::size_t bits = strtoull(argv[6], nullptr, 10);
    const ClippingMode mode = parseClippingMode(argv[7]);
    const std::vector<double> v = draw(kind, seed, n, scale);
    // two batches, like DeepNetQuantization::reportOutputsRange / reportOutputsHistogram: the histogram is created
    // over the range of the first one and enlarged for the second
    const std::size_t h = n / 2;
    RangeStats r1, r;
    for (std::size_t i = 0; i < h; ++i) { r1(v[i]); r(v[i]); }
    for (std::size_t i = h; i < n; ++i) r(v[i]);
    const bool isUnsigned = kind == "relu";
    double val = std::max(std::fabs(r1.minVal()), std::fabs(r1.maxVal()));
    val = std::max(val, 0.1);
    Histogram hist(isUnsigned ? 0 : -val, val, getNbBinsForClippingMode(bits, mode));
    for (std::size_t i = 0; i < h; ++i) hist(v[i]);
    hist.enlarge(std::max(std::fabs(r.minVal()), std::fabs(r.maxVal())), hist.getMinVal() < 0.0);
    for (std::size_t i = h; i < n; ++i) hist(v[i]);
    unsigned long long check = 0;
    for (std::size_t i = 0; i < hist.getBins().size(); ++i) check += (unsigned long long)(i + 1) * hist.getBins()[i];
    printf("%a %a %a %a %a %zu %a %a %llu %a %a %a %a %a\n", r.minVal(), r.maxVal(), r.moments()[0], r.moments()[1], r.moments()[2],
           hist.getNbBins(), hist.getMinVal(), hist.getMaxVal(), check, hist.calibrateMSE(bits), hist.calibrateKLDivergence(bits),
           hist.getQuantileValue(0.9999), hist.getQuantileValue(0.5), hist.getBinValue(hist.getBinIdx(v[0])));
    return 0;
}

static int write_state(const char* dir)
{
    const std::vector<double> v = draw("bell", 42, 4000, 3.0);
    RangeStats r;
    for (double x : v) r(x);
    const double val = std::max(std::fabs(r.minVal()), std::fabs(r.maxVal()));
    Histogram hist(-val, val, 64);
    for (double x : v) hist(x);
    std::unordered_map<std::string, Histogram> hm;
    hm.insert(std::make_pair(std::string("conv1"), hist));
    std::unordered_map<std::string, RangeStats> rm;
    rm.insert(std::make_pair(std::string("conv1"), r));
    Histogram::saveOutputsHistogram(std::string(dir) + "/hist.bin", hm);
    RangeStats::saveOutputsRange(std::string(dir) + "/range.bin", rm);
    // and back
    std::unordered_map<std::string, Histogram> h2;
    std::unordered_map<std::string, RangeStats> r2;
    Histogram::loadOutputsHistogram(std::string(dir) + "/hist.bin", h2);
    RangeStats::loadOutputsRange(std::string(dir) + "/range.bin", r2);
    if (h2.at("conv1").getBins() != hist.getBins() || r2.at("conv1").moments() != r.moments()) return 1;
    return 0;
}

int main(int argc, char** argv)
{
    try {
        if (argc >= 2 && !strcmp(argv[1], "case")) return run_case(argc, argv);
        if (argc >= 3 && !strcmp(argv[1], "state")) return write_state(argv[2]);
    } catch (const std::exception& e) {
        fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
    fprintf(stderr, "usage: see the top of the source file\n");
    return 2;
}
