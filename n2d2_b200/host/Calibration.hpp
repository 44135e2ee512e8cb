// Calibration statistics of the post-training quantization: value ranges and histograms of every cell's
// float outputs, and the clipping thresholds found on them (mean-square error, Kullback-Leibler divergence,
// quantile).  Host-side C++, no GPU: the float network runs in the caller's framework, the values are fed in here.
//
// Restates, with the reference's names and on-disk state format:
//   RangeStats                 src/RangeStats.cpp:28-128 (running min / max and the first three moments)
//   ClippingMode and the bins  include/Histogram.hpp:36-77
//   Histogram                  src/Histogram.cpp:28-132,184-327 (bins, enlarge, calibrateMSE, calibrateKLDivergence,
//                              getQuantileValue, quantize, KLDivergence) and :329-395 (state files)
// The plots the reference draws from these (Histogram::log, RangeStats::logOutputsRange) are not part of the path.
#ifndef N2D2B_HOST_CALIBRATION_HPP
#define N2D2B_HOST_CALIBRATION_HPP

#include <algorithm>
#include <cassert>
#include <cmath>
#include <cstddef>
#include <fstream>
#include <limits>
#include <stdexcept>
#include <string>
#include <tuple>
#include <unordered_map>
#include <vector>

namespace N2D2 {

enum class ClippingMode { NONE, MSE, KL_DIVERGENCE, QUANTILE };

// include/Histogram.hpp:43-60
inline ClippingMode parseClippingMode(const std::string& str)
{
    if (str == "None") return ClippingMode::NONE;
    if (str == "MSE") return ClippingMode::MSE;
    if (str == "KL-Divergence") return ClippingMode::KL_DIVERGENCE;
    if (str == "Quantile") return ClippingMode::QUANTILE;
    throw std::runtime_error("Unknown clipping mode '" + str + "'.");
}

// include/Histogram.hpp:62-77
inline std::size_t getNbBinsForClippingMode(std::size_t nbBits, ClippingMode clippingMode)
{
    switch (clippingMode) {
    case ClippingMode::MSE:
    case ClippingMode::KL_DIVERGENCE: return (std::size_t)std::min((1 << nbBits) * 64, 65536);
    case ClippingMode::QUANTILE: return 65536;
    default: return 0;
    }
}

class RangeStats {
public:
    RangeStats() : mMinVal(0.0), mMaxVal(0.0), mMoments(3, 0.0) {}
    double minVal() const { return mMinVal; }
    double maxVal() const { return mMaxVal; }
    const std::vector<double>& moments() const { return mMoments; }
    double mean() const { return mMoments[1] / mMoments[0]; }
    double stdDev() const
    {
        const double m = mMoments[1] / mMoments[0];
        const double meanSquare = mMoments[2] / mMoments[0];
        return std::sqrt(meanSquare - m * m);
    }
    // src/RangeStats.cpp:50-70
    void operator()(double value)
    {
        if (mMoments[0] > 0) {
            mMinVal = std::min(mMinVal, value);
            mMaxVal = std::max(mMaxVal, value);
        } else {
            mMinVal = value;
            mMaxVal = value;
        }
        double inc = 1.0;
        for (double& m : mMoments) {
            m += inc;
            inc *= value;
        }
    }
    void save(std::ostream& state) const
    {
        state.write(reinterpret_cast<const char*>(&mMinVal), sizeof(mMinVal));
        state.write(reinterpret_cast<const char*>(&mMaxVal), sizeof(mMaxVal));
        const std::size_t momentsSize = mMoments.size();
        state.write(reinterpret_cast<const char*>(&momentsSize), sizeof(momentsSize));
        state.write(reinterpret_cast<const char*>(&mMoments[0]), momentsSize * sizeof(mMoments[0]));
    }
    void load(std::istream& state)
    {
        state.read(reinterpret_cast<char*>(&mMinVal), sizeof(mMinVal));
        state.read(reinterpret_cast<char*>(&mMaxVal), sizeof(mMaxVal));
        std::size_t momentsSize = 0;
        state.read(reinterpret_cast<char*>(&momentsSize), sizeof(momentsSize));
        if (!state.good() || momentsSize > 64) throw std::runtime_error("RangeStats: damaged state");
        mMoments.resize(momentsSize);
        state.read(reinterpret_cast<char*>(&mMoments[0]), momentsSize * sizeof(mMoments[0]));
    }
    static void saveOutputsRange(const std::string& fileName, const std::unordered_map<std::string, RangeStats>& outputsRange);
    static void loadOutputsRange(const std::string& fileName, std::unordered_map<std::string, RangeStats>& outputsRange);

private:
    double mMinVal, mMaxVal;
    std::vector<double> mMoments;
};

class Histogram {
public:
    Histogram(double minVal, double maxVal, std::size_t nbBins)
        : mMinVal(minVal), mMaxVal(maxVal), mNbBins(nbBins), mValues(nbBins, 0), mNbValues(0)
    {
        if (mNbBins <= 0) throw std::runtime_error("Number of bins must be > 0.");
        if (mMaxVal <= mMinVal) throw std::runtime_error("mMinVal must be strictly smaller than mMaxVal.");
    }
    std::size_t getNbBins() const { return mNbBins; }
    double getBinWidth() const { return (mMaxVal - mMinVal) / mNbBins; }
    double getBinValue(std::size_t binIdx) const
    {
        if (binIdx >= mNbBins) throw std::out_of_range("binIdx must be < mNbBins");
        return mMinVal + (binIdx + 0.5) * getBinWidth();
    }
    // src/Histogram.cpp:58-69: values are clamped into the range; the upper edge belongs to the last bin
    std::size_t getBinIdx(double value) const
    {
        const double clampedValue = std::min(std::max(value, mMinVal), mMaxVal);
        std::size_t binIdx = static_cast<std::size_t>((clampedValue - mMinVal) / getBinWidth() + 1e-6);
        if (binIdx == mNbBins) binIdx--;
        return binIdx;
    }
    double getMinVal() const { return mMinVal; }
    double getMaxVal() const { return mMaxVal; }
    const std::vector<std::size_t>& getBins() const { return mValues; }
    std::size_t getNbValues() const { return mNbValues; }

    void operator()(double value, std::size_t count = 1)
    {
        if (value > mMaxVal || value < mMinVal)
            throw std::out_of_range(std::to_string(value) + " not between [" + std::to_string(mMinVal) + ";"
                                    + std::to_string(mMaxVal) + "]");
        mValues[getBinIdx(value)] += count;
        mNbValues += count;
    }

    // src/Histogram.cpp:95-124: whole bins of the current width are added until `value` is inside (on both sides when
    // symetric)
    void enlarge(double value, bool symetric)
    {
        const double currBinWidth = getBinWidth();
        std::size_t newNbBins;
        if (value < mMinVal) newNbBins = static_cast<std::size_t>(std::ceil((mMinVal - value) / getBinWidth()));
        else if (value > mMaxVal) newNbBins = static_cast<std::size_t>(std::ceil((value - mMaxVal) / getBinWidth()));
        else return;
        if (symetric || value < mMinVal) {
            mValues.insert(mValues.begin(), newNbBins, 0);
            mMinVal = mMinVal - newNbBins * currBinWidth;
        }
        if (symetric || value > mMaxVal) {
            mValues.insert(mValues.end(), newNbBins, 0);
            mMaxVal = mMaxVal + newNbBins * currBinWidth;
        }
        mNbBins = mValues.size();
    }

    // src/Histogram.cpp:184-206: 1000 thresholds from max |range| downwards, the one with the smallest error wins
    // (the first one on ties, i.e. the largest)
    double calibrateMSE(std::size_t nbBits) const
    {
        if (mNbValues == 0) return 0.0;
        double threshold = std::max(std::fabs(mMinVal), std::fabs(mMaxVal));
        double bestThreshold = threshold;
        double bestMSE = std::numeric_limits<double>::max();
        const double threshold_decr_step = threshold / 1000.0;
        while (threshold > 0.0) {
            const double mse = MSE(threshold, nbBits);
            if (mse < bestMSE) {
                bestMSE = mse;
                bestThreshold = threshold;
            }
            threshold -= threshold_decr_step;
        }
        return bestThreshold;
    }

    // src/Histogram.cpp:232-257
    double calibrateKLDivergence(std::size_t nbBits) const
    {
        if (mNbValues == 0) return 0.0;
        const bool isUnsigned = mMinVal >= 0.0;
        const std::size_t nbQuantizedBins = static_cast<std::size_t>(1) << nbBits;
        double threshold = std::max(std::fabs(mMinVal), std::fabs(mMaxVal));
        double bestThreshold = threshold;
        double bestDivergence = std::numeric_limits<double>::max();
        const double threshold_decr_step = threshold / 1000.0;
        while (threshold > 0.0) {
            const double divergence = KLDivergence(*this, quantize(isUnsigned ? 0 : -threshold, threshold, nbQuantizedBins));
            if (divergence < bestDivergence) {
                bestDivergence = divergence;
                bestThreshold = threshold;
            }
            threshold -= threshold_decr_step;
        }
        return bestThreshold;
    }

    // src/Histogram.cpp:259-271
    double getQuantileValue(double quantile) const
    {
        const std::size_t quantileNbValues = (std::size_t)(quantile * mNbValues);
        std::size_t nbValues = 0;
        for (std::size_t bin = 0; bin < mNbBins; ++bin) {
            nbValues += mValues[bin];
            if (nbValues >= quantileNbValues) return getBinValue(bin);
        }
        return getBinValue(mNbBins - 1);
    }

    // src/Histogram.cpp:208-229: error of rounding the bin centres to nbBits integers over [-threshold, threshold]
    // (or [0, threshold] for a histogram without negative values), weighted by the bin counts
    double MSE(double threshold, std::size_t nbBits) const
    {
        assert(nbBits > 1);
        const bool isUnsigned = mMinVal >= 0.0;
        const double minVal = isUnsigned ? 0 : -(double)(1LL << (nbBits - 1));
        const double maxVal = isUnsigned ? (double)((1ULL << nbBits) - 1) : (double)((1ULL << (nbBits - 1)) - 1);
        const double scaling = maxVal / threshold;
        double mse = 0.0;
        for (std::size_t bin = 0; bin < mNbBins; bin++) {
            const double approx = std::min(std::max(std::round(getBinValue(bin) * scaling), minVal), maxVal) / scaling;
            const double normalizedValue = 1.0 * mValues[bin] / mNbValues;
            mse += std::pow(getBinValue(bin) - approx, 2) * normalizedValue;
        }
        return mse;
    }

    // src/Histogram.cpp:273-285: the same counts in newNbBins bins over [newMinVal, newMaxVal], outliers into the edge bins
    Histogram quantize(double newMinVal, double newMaxVal, std::size_t newNbBins) const
    {
        Histogram hist(newMinVal, newMaxVal, newNbBins);
        for (std::size_t bin = 0; bin < mNbBins; ++bin) {
            const double value = std::min(std::max(getBinValue(bin), hist.mMinVal), hist.mMaxVal);
            hist(value, mValues[bin]);
        }
        return hist;
    }

    // src/Histogram.cpp:287-314: divergence between the reference distribution and the quantized one spread back
    // over the reference's bins
    static double KLDivergence(const Histogram& ref, const Histogram& quant)
    {
        double qNorm = 0.0;
        for (std::size_t bin = 0; bin < ref.mNbBins; ++bin) {
            const std::size_t quantIdx = quant.getBinIdx(ref.getBinValue(bin));
            qNorm += quant.mValues[quantIdx];
        }
        double divergence = 0.0;
        for (std::size_t bin = 0; bin < ref.mNbBins; ++bin) {
            const std::size_t quantIdx = quant.getBinIdx(ref.getBinValue(bin));
            const double p = (ref.mValues[bin] / (double)ref.mNbValues);
            const double q = (quant.mValues[quantIdx] / qNorm);
            if (p != 0) divergence += p * std::log(p / q);
        }
        return divergence;
    }

    void save(std::ostream& state) const
    {
        state.write(reinterpret_cast<const char*>(&mMinVal), sizeof(mMinVal));
        state.write(reinterpret_cast<const char*>(&mMaxVal), sizeof(mMaxVal));
        state.write(reinterpret_cast<const char*>(&mNbBins), sizeof(mNbBins));
        const std::size_t valuesSize = mValues.size();
        state.write(reinterpret_cast<const char*>(&valuesSize), sizeof(valuesSize));
        state.write(reinterpret_cast<const char*>(&mValues[0]), valuesSize * sizeof(mValues[0]));
        state.write(reinterpret_cast<const char*>(&mNbValues), sizeof(mNbValues));
    }
    void load(std::istream& state)
    {
        state.read(reinterpret_cast<char*>(&mMinVal), sizeof(mMinVal));
        state.read(reinterpret_cast<char*>(&mMaxVal), sizeof(mMaxVal));
        state.read(reinterpret_cast<char*>(&mNbBins), sizeof(mNbBins));
        std::size_t valuesSize = 0;
        state.read(reinterpret_cast<char*>(&valuesSize), sizeof(valuesSize));
        if (!state.good() || valuesSize > (std::size_t)1 << 28) throw std::runtime_error("Histogram: damaged state");
        mValues.resize(valuesSize);
        state.read(reinterpret_cast<char*>(&mValues[0]), valuesSize * sizeof(mValues[0]));
        state.read(reinterpret_cast<char*>(&mNbValues), sizeof(mNbValues));
    }
    static void saveOutputsHistogram(const std::string& fileName, const std::unordered_map<std::string, Histogram>& outputsHistogram);
    static void loadOutputsHistogram(const std::string& fileName, std::unordered_map<std::string, Histogram>& outputsHistogram);

private:
    double mMinVal, mMaxVal;
    std::size_t mNbBins;
    std::vector<std::size_t> mValues;
    std::size_t mNbValues;
};

// ---- state files: count, then per entry the name's length, the name and the object (src/RangeStats.cpp:92-151,
// src/Histogram.cpp:354-395)
namespace calibration_detail {
template <class T, class Make>
void saveMap(const std::string& fileName, const std::unordered_map<std::string, T>& m, Make)
{
    std::ofstream state(fileName.c_str(), std::fstream::binary);
    if (!state.good()) throw std::runtime_error("Could not create state file: " + fileName);
    const std::size_t mapSize = m.size();
    state.write(reinterpret_cast<const char*>(&mapSize), sizeof(mapSize));
    for (const auto& kv : m) {
        const std::size_t nameSize = kv.first.size();
        state.write(reinterpret_cast<const char*>(&nameSize), sizeof(nameSize));
        state.write(kv.first.data(), nameSize);
        kv.second.save(state);
    }
    if (!state.good()) throw std::runtime_error("Error writing state file: " + fileName);
}
template <class T, class Make>
void loadMap(const std::string& fileName, std::unordered_map<std::string, T>& m, Make make)
{
    std::ifstream state(fileName.c_str(), std::fstream::binary);
    if (!state.good()) throw std::runtime_error("Could not open state file: " + fileName);
    std::size_t mapSize = 0;
    state.read(reinterpret_cast<char*>(&mapSize), sizeof(mapSize));
    for (std::size_t n = 0; n < mapSize && state.good(); ++n) {
        std::size_t nameSize = 0;
        state.read(reinterpret_cast<char*>(&nameSize), sizeof(nameSize));
        if (!state.good() || nameSize > 65536) throw std::runtime_error("Error while reading state file: " + fileName);
        std::string nameStr(nameSize, ' ');
        state.read(&nameStr[0], nameSize);
        typename std::unordered_map<std::string, T>::iterator it;
        std::tie(it, std::ignore) = m.insert(std::make_pair(nameStr, make()));
        it->second.load(state);
    }
    if (state.eof()) throw std::runtime_error("End-of-file reached prematurely in state file: " + fileName);
    if (!state.good()) throw std::runtime_error("Error while reading state file: " + fileName);
    if (state.get() != std::fstream::traits_type::eof()) throw std::runtime_error("State file size larger than expected: " + fileName);
}
}  // namespace calibration_detail

inline void RangeStats::saveOutputsRange(const std::string& fileName, const std::unordered_map<std::string, RangeStats>& outputsRange)
{
    calibration_detail::saveMap(fileName, outputsRange, [] { return RangeStats(); });
}
inline void RangeStats::loadOutputsRange(const std::string& fileName, std::unordered_map<std::string, RangeStats>& outputsRange)
{
    calibration_detail::loadMap(fileName, outputsRange, [] { return RangeStats(); });
}
inline void Histogram::saveOutputsHistogram(const std::string& fileName, const std::unordered_map<std::string, Histogram>& outputsHistogram)
{
    calibration_detail::saveMap(fileName, outputsHistogram, [] { return Histogram(0, 1, 1); });
}
inline void Histogram::loadOutputsHistogram(const std::string& fileName, std::unordered_map<std::string, Histogram>& outputsHistogram)
{
    calibration_detail::loadMap(fileName, outputsHistogram, [] { return Histogram(0, 1, 1); });
}

}  // namespace N2D2

#endif
