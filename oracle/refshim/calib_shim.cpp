// C entry points over the reference's own calibration statistics (Histogram, RangeStats), compiled from the
// reference tree where it lies by the Makefile beside this file.  TEST INFRASTRUCTURE ONLY: used to pin the host-side
// restatement (n2d2_b200/host/Calibration.hpp) and to generate the golden thresholds under tests/golden/.
#include <cstddef>
#include <cstring>
#include <fstream>
#include <string>
#include <unordered_map>
#include "Histogram.hpp"
#include "RangeStats.hpp"
#include "utils/Utils.hpp"

// The file helpers the reference's plotting members call; nothing here plots.
namespace N2D2 {
namespace Utils {
bool createDirectories(const std::string&) { return true; }
std::string dirName(const std::string&, bool) { return std::string(); }
std::string fileBaseName(const std::string& filePath, const std::string&) { return filePath; }
std::string fileExtension(const std::string&, const std::string&) { return std::string(); }
std::string filePath(const std::string& str) { return str; }
}
}

using N2D2::Histogram;
using N2D2::RangeStats;

extern "C" {

void* calib_hist_new(double minVal, double maxVal, std::size_t nbBins)
{
    try { return new Histogram(minVal, maxVal, nbBins); } catch (...) { return nullptr; }
}
void calib_hist_free(void* h) { delete (Histogram*)h; }
int calib_hist_add(void* h, const double* v, std::size_t n)
{
    try {
        for (std::size_t i = 0; i < n; ++i) (*(Histogram*)h)(v[i]);
        return 0;
    } catch (...) { return -1; }
}
void calib_hist_enlarge(void* h, double value, int symetric) { ((Histogram*)h)->enlarge(value, symetric != 0); }
double calib_hist_mse(void* h, std::size_t nbBits) { return ((Histogram*)h)->calibrateMSE(nbBits); }
double calib_hist_kl(void* h, std::size_t nbBits) { return ((Histogram*)h)->calibrateKLDivergence(nbBits); }
double calib_hist_quantile(void* h, double q) { return ((Histogram*)h)->getQuantileValue(q); }
std::size_t calib_hist_nb_bins(void* h) { return ((Histogram*)h)->getNbBins(); }
double calib_hist_min(void* h) { return ((Histogram*)h)->getMinVal(); }
double calib_hist_max(void* h) { return ((Histogram*)h)->getMaxVal(); }
void calib_hist_bins(void* h, unsigned long long* out)
{
    const std::vector<std::size_t>& b = ((Histogram*)h)->getBins();
    for (std::size_t i = 0; i < b.size(); ++i) out[i] = b[i];
}
// state file with one entry
int calib_hist_save(void* h, const char* name, const char* fileName)
{
    try {
        std::unordered_map<std::string, Histogram> m;
        m.insert(std::make_pair(std::string(name), *(Histogram*)h));
        Histogram::saveOutputsHistogram(fileName, m);
        return 0;
    } catch (...) { return -1; }
}

// out = min, max, moments 0..2
void calib_range(const double* v, std::size_t n, double* out)
{
    RangeStats r;
    for (std::size_t i = 0; i < n; ++i) r(v[i]);
    out[0] = r.minVal(); out[1] = r.maxVal();
    out[2] = r.moments()[0]; out[3] = r.moments()[1]; out[4] = r.moments()[2];
}
int calib_range_save(const double* v, std::size_t n, const char* name, const char* fileName)
{
    try {
        std::unordered_map<std::string, RangeStats> m;
        RangeStats r;
        for (std::size_t i = 0; i < n; ++i) r(v[i]);
        m.insert(std::make_pair(std::string(name), r));
        RangeStats::saveOutputsRange(fileName, m);
        return 0;
    } catch (...) { return -1; }
}

}  // extern "C"
