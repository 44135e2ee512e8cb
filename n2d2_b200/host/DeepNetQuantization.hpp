// Post-training quantization front-end: turns a floating-point network held by the host classes of
// N2D2.hpp into the integer path the device library runs.  It restates, step by step, the reference's
// DeepNetQuantization::quantizeNetwork (src/DeepNetQuantization.cpp:285-388):
//
//   quantizeFreeParemeters[PerOutputCh]   :538-671   weights to +-(2^(n-1) - 1), biases to the accumulator scale,
//                                                    `_rescale_branch` / `_rescale_params` ScalingCells
//   quantizeActivations                   :673-794   one `_rescale_act` ScalingCell per activation
//   fuseScalingCells and its three rules  :828-1002  into the parent's activation, into a parent ScalingCell, or
//                                                    above a parent element-wise sum
//   approximateScalingCell                :1004-1041 remaining ScalingCells to fixed point
//   approximateScalingWithFixedPoint      :1043-1093
//   approximateScalingWithPowerOf2Divs    :1095-1134
//   approximateActivationScaling          :1200-1283 fixed point, one shift or two shifts (the shift forms
//                                                    re-scale the cell's parameters to absorb their error)
//   rounding of the parameters, setQuantized :347-349
//
//   clipWeights                           :63-107    weights clamped to the MSE / KL threshold of their histogram
//   reportOutputsRange / reportOutputsHistogram :150-281 calibration statistics of every cell's float outputs
//   getCellThreshold                      :1181-1198 threshold of a cell from those statistics
//
// The float network itself runs in the caller's framework: its outputs are fed, cell by cell and batch by batch,
// to reportOutputsRange / reportOutputsHistogram (Calibration.hpp holds RangeStats and Histogram), and
// quantizeNetwork takes the statistics like the reference's.  A second form takes a map from cell name to threshold,
// however it was obtained.  Arithmetic on the scalings is done in long double / double / float exactly where the
// reference does.
#pragma once

#include <cassert>
#include <cmath>
#include <functional>
#include <limits>
#include <unordered_map>

#include "Calibration.hpp"
#include "N2D2.hpp"

namespace N2D2 {

class DeepNetQuantization {
public:
    explicit DeepNetQuantization(DeepNet& deepNet) : mDeepNet(deepNet) {}

    // The statistics name of a cell and whether its clipping mode applies -> its activation threshold
    typedef std::function<double(const Cell& cell, const std::string& cellStatsName, bool clip)> ThresholdFn;

    // src/DeepNetQuantization.cpp:285-388, with the reference's arguments
    void quantizeNetwork(const std::unordered_map<std::string, Histogram>& outputsHistogram,
                         const std::unordered_map<std::string, RangeStats>& outputsRange, std::size_t nbBits,
                         ClippingMode actClippingMode, ScalingMode actScalingMode, bool rescalePerOutputChannel,
                         double quantileValue = 0.9999)
    {
        quantizeNetwork([&](const Cell&, const std::string& cellStatsName, bool clip) {
            return getCellThreshold(cellStatsName, outputsHistogram, outputsRange, nbBits,
                                    clip ? actClippingMode : ClippingMode::NONE, quantileValue);
        }, nbBits, actScalingMode, rescalePerOutputChannel);
    }

    // outputsThreshold: for every cell with an activation (and every element-wise cell) the value
    // getCellThreshold would return: max |output| for ClippingMode::NONE, or the calibrated clipping threshold.
    // (With a clipping mode and a max pooling as the only child the reference takes the pooling cell's statistics,
    // :724-737; a map expresses that by the value it holds for the cell.)
    void quantizeNetwork(const std::unordered_map<std::string, double>& outputsThreshold, std::size_t nbBits,
                         ScalingMode actScalingMode, bool rescalePerOutputChannel)
    {
        quantizeNetwork([&](const Cell& cell, const std::string&, bool) {
            auto it = outputsThreshold.find(cell.getName());
            if (it == outputsThreshold.end())
                throw std::runtime_error("quantizeActivations(): no calibration threshold for cell '" + cell.getName() + "'");
            return it->second;
        }, nbBits, actScalingMode, rescalePerOutputChannel);
    }

    void quantizeNetwork(const ThresholdFn& threshold, std::size_t nbBits, ScalingMode actScalingMode, bool rescalePerOutputChannel)
    {
        std::unordered_map<std::string, long double> biasScalings
            = rescalePerOutputChannel ? quantizeFreeParemetersPerOutputCh(nbBits) : quantizeFreeParemeters(nbBits);
        quantizeActivations(threshold, biasScalings, nbBits);

        const std::vector<std::vector<std::string> > layers = mDeepNet.getLayers();
        for (std::size_t l = 1; l < layers.size(); ++l)
            for (const std::string& name : layers[l]) {
                std::shared_ptr<Cell> cell = mDeepNet.getCell<Cell>(name);
                if (auto* sc = dynamic_cast<ScalingCell*>(cell.get())) {
                    const ScalingMode scalingCellMode = (actScalingMode == ScalingMode::SINGLE_SHIFT || actScalingMode == ScalingMode::DOUBLE_SHIFT)
                                                            ? ScalingMode::FIXED_MULT16 : actScalingMode;
                    approximateScalingCell(*sc, scalingCellMode);
                } else if (cell->getActivation()) {
                    approximateActivationScaling(*cell, *cell->getActivation(), actScalingMode);
                }
                // after the approximation, which may have re-scaled the parameters (shift modes)
                cell->processFreeParameters([](Float_T p) { return std::round(p); });
                cell->roundFreeParameters(nbBits);
                cell->setQuantized(nbBits);
            }
    }

    // ---- the two approximations, usable on their own ---------------------------------------------------------
    // Highest number of fractional bits for which round(sc * 2^bits) of the largest scaling still fits an int16
    // (FIXED_MULT16) or int32 (FIXED_MULT32); a scaling too large for 16 bits falls back to 32 (mode is updated).
    static std::pair<std::size_t, std::vector<std::int32_t> > approximateScalingWithFixedPoint(ScalingMode& mode,
                                                                                            const std::vector<Float_T>& scalingPerOutput)
    {
        const std::uint64_t limit = (mode == ScalingMode::FIXED_MULT16) ? (std::uint64_t)std::numeric_limits<std::int16_t>::max()
                                                                        : (std::uint64_t)std::numeric_limits<std::int32_t>::max();
        const double maxScaling = *std::max_element(scalingPerOutput.begin(), scalingPerOutput.end());
        if (maxScaling >= limit) {
            if (mode == ScalingMode::FIXED_MULT16) {
                mode = ScalingMode::FIXED_MULT32;
                return approximateScalingWithFixedPoint(mode, scalingPerOutput);
            }
            throw std::runtime_error("Max scaling (" + std::to_string(maxScaling) + ") doesn't fit in FIXED_MULT32.");
        }
        const std::size_t maxNbFractionalBits = 50;
        const std::size_t nbFractionalBits = std::min((std::size_t)std::floor(std::log(limit / maxScaling) / std::log(2.0)), maxNbFractionalBits);
        std::vector<std::int32_t> scalingFixedPoint;
        for (Float_T sc : scalingPerOutput) scalingFixedPoint.push_back((std::int32_t)std::round(sc * (1ull << nbFractionalBits)));
        return std::make_pair(nbFractionalBits, scalingFixedPoint);
    }

    // scaling <= 1 as a sum of nbDivisions powers of two, 2^-e0 (+ 2^-e1): returns the exponents and the
    // "precision" p >= 1 with scaling * p = sum of the powers, i.e. what the outputs must be divided by to
    // compensate (a precision of at least 0.98 counts as exact).
    static std::pair<std::vector<unsigned char>, double> approximateScalingWithPowerOf2Divs(Float_T scaling, std::size_t nbDivisions)
    {
        static const double ROUNDING_THRESHOLD = 0.98;
        if (nbDivisions == 0 || !(scaling <= 1.0f) || !(scaling > 0.0f))
            throw std::runtime_error("approximateScalingWithPowerOf2Divs(): needs 0 < scaling <= 1 and at least one division");
        double precision = 0.0;
        std::vector<unsigned char> powerOf2Divs(nbDivisions);
        for (std::size_t iDiv = 0; iDiv < nbDivisions; iDiv++) {
            if (precision == 1.0) {
                powerOf2Divs[iDiv - 1]++;
                powerOf2Divs[iDiv] = powerOf2Divs[iDiv - 1];
            } else {
                const std::size_t exponent = (std::size_t)std::ceil(std::log2(1.0 / (scaling * (1.0 - precision))));
                precision += 1.0 / (scaling * std::pow(2, exponent));
                powerOf2Divs[iDiv] = static_cast<unsigned char>(exponent);
            }
        }
        if (precision >= ROUNDING_THRESHOLD) {
            precision = 1.0;
        } else if (precision < 1.0) {
            precision += 1.0 / (scaling * std::pow(2, powerOf2Divs.back()));
            powerOf2Divs.back() = powerOf2Divs.back() - 1;
        }
        return std::make_pair(powerOf2Divs, precision);
    }

    // ---- steps of quantizeNetwork -------------------------------------------------------------------------------
    std::unordered_map<std::string, long double> quantizeFreeParemeters(std::size_t nbBits)
    {
        std::unordered_map<std::string, long double> biasScalings;
        const std::vector<std::vector<std::string> > layers = mDeepNet.getLayers();
        for (std::size_t l = 1; l < layers.size(); ++l)
            for (const std::string& name : layers[l]) {
                std::shared_ptr<Cell> cell = mDeepNet.getCell<Cell>(name);
                long double biasScaling = getMaxParentsScaling(cell, biasScalings);
                rescaleParentsToScaling(cell, biasScalings, biasScaling);
                const long double wQuantScaling = std::pow(2, nbBits - 1) - 1;
                const long double bQuantScaling = mDeepNet.isCellInputsUnsigned(*cell) ? wQuantScaling * (std::pow(2, nbBits) - 1)
                                                                                      : wQuantScaling * (std::pow(2, nbBits - 1) - 1);
                const std::pair<Float_T, Float_T> wMinMax = cell->getFreeParametersRange(Cell::Multiplicative);
                const Float_T wScalingCell = maxAbs(wMinMax.first, wMinMax.second);
                if (wScalingCell != 0.0) {
                    cell->processFreeParameters([&](Float_T w) { return (Float_T)(w * (wQuantScaling / wScalingCell)); }, Cell::Multiplicative);
                    biasScaling *= wScalingCell;
                }
                cell->processFreeParameters([&](Float_T b) { return (Float_T)(b * (bQuantScaling / biasScaling)); }, Cell::Additive);
                biasScalings[cell->getName()] = biasScaling;
            }
        fuseScalingCells();
        return biasScalings;
    }

    std::unordered_map<std::string, long double> quantizeFreeParemetersPerOutputCh(std::size_t nbBits)
    {
        std::unordered_map<std::string, long double> biasScalings;
        const std::vector<std::vector<std::string> > layers = mDeepNet.getLayers();
        for (std::size_t l = 1; l < layers.size(); ++l)
            for (const std::string& name : layers[l]) {
                std::shared_ptr<Cell> cell = mDeepNet.getCell<Cell>(name);
                long double biasScaling = getMaxParentsScaling(cell, biasScalings);
                rescaleParentsToScaling(cell, biasScalings, biasScaling);
                const long double wQuantScaling = std::pow(2, nbBits - 1) - 1;
                const long double bQuantScaling = mDeepNet.isCellInputsUnsigned(*cell) ? wQuantScaling * (std::pow(2, nbBits) - 1)
                                                                                      : wQuantScaling * (std::pow(2, nbBits - 1) - 1);
                const std::pair<Float_T, Float_T> wMinMax = cell->getFreeParametersRange(Cell::Multiplicative);
                const Float_T wScalingCell = maxAbs(wMinMax.first, wMinMax.second);
                if (wScalingCell != 0.0) {
                    std::vector<Float_T> scalingPerOutput(cell->getNbOutputs());
                    for (std::size_t output = 0; output < cell->getNbOutputs(); output++) {
                        const auto woMinMax = cell->getFreeParametersRangePerOutput(output, Cell::Multiplicative);
                        const Float_T wScalingCellOutput = std::max(std::min(wScalingCell, 0.1f), maxAbs(woMinMax.first, woMinMax.second));
                        cell->processFreeParametersPerOutput([&](Float_T w) { return (Float_T)(w * (wQuantScaling / wScalingCellOutput)); }, output,
                                                             Cell::Multiplicative);
                        cell->processFreeParametersPerOutput(
                            [&](Float_T b) { return (Float_T)(b * (bQuantScaling / (biasScaling * wScalingCellOutput))); }, output, Cell::Additive);
                        scalingPerOutput[output] = wScalingCellOutput / wScalingCell;
                    }
                    auto scalingCell = std::make_shared<ScalingCell>(mDeepNet.generateNewCellName(cell->getName() + "_rescale_params"),
                                                                     cell->getNbOutputs(),
                                                                     Scaling::floatingPointScaling(std::move(scalingPerOutput), false, {}));
                    mDeepNet.addCellAfter(scalingCell, cell);
                    biasScaling *= wScalingCell;
                    biasScalings[scalingCell->getName()] = biasScaling;
                }
                biasScalings[cell->getName()] = biasScaling;
            }
        fuseScalingCells();
        return biasScalings;
    }

    // ---- calibration (src/DeepNetQuantization.cpp:63-107,150-281,1181-1198) -----------------------------------------
    // Weights beyond the MSE / KL threshold of their own histogram are clamped to it, cell by cell.
    void clipWeights(std::size_t nbBits, ClippingMode wtClippingMode)
    {
        if (wtClippingMode == ClippingMode::NONE) return;
        const std::size_t nbBins = getNbBinsForClippingMode(nbBits, wtClippingMode);
        const std::vector<std::vector<std::string> > layers = mDeepNet.getLayers();
        for (std::size_t l = 1; l < layers.size(); ++l)
            for (const std::string& name : layers[l]) {
                std::shared_ptr<Cell> cell = mDeepNet.getCell<Cell>(name);
                const std::pair<Float_T, Float_T> range = cell->getFreeParametersRange(Cell::Multiplicative);
                const Float_T maxWeight = std::max(std::abs(range.first), std::abs(range.second));
                if (maxWeight == 0) continue;
                Histogram hist(-maxWeight, maxWeight, nbBins);
                cell->processFreeParameters([&](Float_T wt) { hist(wt); return wt; }, Cell::Multiplicative);
                Float_T threshold;
                switch (wtClippingMode) {
                case ClippingMode::KL_DIVERGENCE: threshold = (Float_T)hist.calibrateKLDivergence(nbBits); break;
                case ClippingMode::MSE: threshold = (Float_T)hist.calibrateMSE(nbBits); break;
                default: throw std::runtime_error("Unsupported clipping mode.");
                }
                cell->processFreeParameters([&](Float_T wt) { return std::min(std::max(wt, -threshold), threshold); },
                                            Cell::Multiplicative);
            }
    }

    // One batch of float outputs of a cell (or of the stimuli, cellName "env") into its range statistics
    void reportOutputsRange(std::unordered_map<std::string, RangeStats>& outputsRange, const std::string& cellName,
                            const Float_T* outputs, std::size_t count) const
    {
        if (outputsRange.empty()) {
            const std::vector<std::vector<std::string> > layers = mDeepNet.getLayers();
            for (const std::vector<std::string>& layer : layers)
                for (const std::string& name : layer) outputsRange.insert(std::make_pair(name, RangeStats()));
        }
        RangeStats& rangeStats = outputsRange.at(cellName);
        for (std::size_t i = 0; i < count; ++i) rangeStats(outputs[i]);
    }

    // The same batch into the cell's histogram (second calibration pass: the ranges are complete).  On first use every
    // histogram is created over [-max|range|, max|range|], or [0, max|range|] for a cell with unsigned outputs, at
    // least 0.1 wide; later batches enlarge it by whole bins if the range has grown.
    void reportOutputsHistogram(std::unordered_map<std::string, Histogram>& outputsHistogram,
                                const std::unordered_map<std::string, RangeStats>& outputsRange, const std::string& cellName,
                                const Float_T* outputs, std::size_t count, std::size_t nbBits, ClippingMode actClippingMode,
                                bool envDataUnsigned = DeepNetExport::mEnvDataUnsigned()) const
    {
        if (actClippingMode == ClippingMode::NONE) return;
        if (outputsHistogram.empty()) {
            const std::size_t nbBins = getNbBinsForClippingMode(nbBits, actClippingMode);
            const std::vector<std::vector<std::string> > layers = mDeepNet.getLayers();
            for (std::size_t l = 0; l < layers.size(); ++l)
                for (const std::string& name : layers[l]) {
                    const RangeStats& range = outputsRange.at(name);
                    const bool isCellOutputUnsigned
                        = (l == 0) ? envDataUnsigned : mDeepNet.isCellOutputUnsigned(*mDeepNet.getCell<Cell>(name));
                    double val = std::max(std::fabs(range.minVal()), std::fabs(range.maxVal()));
                    val = std::max(val, 0.1);
                    outputsHistogram.insert(std::make_pair(name, Histogram(isCellOutputUnsigned ? 0 : -val, val, nbBins)));
                }
        }
        Histogram& hist = outputsHistogram.at(cellName);
        const RangeStats& range = outputsRange.at(cellName);
        const bool enlargeSymetric = hist.getMinVal() < 0.0;
        hist.enlarge(std::max(std::fabs(range.minVal()), std::fabs(range.maxVal())), enlargeSymetric);
        for (std::size_t i = 0; i < count; ++i) hist(outputs[i]);
    }

    static double getCellThreshold(const std::string& cellName, const std::unordered_map<std::string, Histogram>& outputsHistogram,
                                   const std::unordered_map<std::string, RangeStats>& outputsRange, std::size_t nbBits,
                                   ClippingMode actClippingMode, double quantileValue = 0.9999)
    {
        switch (actClippingMode) {
        case ClippingMode::KL_DIVERGENCE: return outputsHistogram.at(cellName).calibrateKLDivergence(nbBits);
        case ClippingMode::MSE: return outputsHistogram.at(cellName).calibrateMSE(nbBits);
        case ClippingMode::QUANTILE: return outputsHistogram.at(cellName).getQuantileValue(quantileValue);
        default: {
            const RangeStats& range = outputsRange.at(cellName);
            return std::max(std::fabs(range.minVal()), std::fabs(range.maxVal()));
        }
        }
    }

    void quantizeActivations(const ThresholdFn& threshold, std::unordered_map<std::string, long double>& biasScalings,
                             std::size_t nbBits)
    {
        std::unordered_map<std::string, long double> activationScalings;
        const std::vector<std::vector<std::string> > layers = mDeepNet.getLayers();
        for (std::size_t l = 1; l < layers.size(); ++l)
            for (const std::string& name : layers[l]) {
                std::shared_ptr<Cell> cell = mDeepNet.getCell<Cell>(name);
                const long double prevActivationScaling = getMaxParentsScaling(cell, activationScalings);
                rescaleParentsToScaling(cell, activationScalings, prevActivationScaling);
                long double activationScaling;
                const bool isElemWise = dynamic_cast<ElemWiseCell*>(cell.get()) != nullptr;
                if (dynamic_cast<PoolCell*>(cell.get()) || dynamic_cast<ScalingCell*>(cell.get())) {
                    activationScalings[cell->getName()] = prevActivationScaling;
                    continue;
                } else if (isElemWise) {
                    activationScaling = threshold(*cell, cell->getName(), false);
                } else if (cell->getActivation()) {
                    // clipping modes apply to cells with more than two outputs; when the only child is a max pooling,
                    // its statistics stand for the cell's (:716-737)
                    const bool clip = cell->getNbOutputs() > 2;
                    const std::vector<std::shared_ptr<Cell> > childrenCells = mDeepNet.getChildCells(cell->getName());
                    const PoolCell* childPool = childrenCells.size() == 1 ? dynamic_cast<const PoolCell*>(childrenCells[0].get()) : nullptr;
                    const bool isNextCellMaxPool = childPool && childPool->getPooling() == PoolCell::Max;
                    activationScaling = threshold(*cell, clip && isNextCellMaxPool ? childrenCells[0]->getName() : cell->getName(), clip);
                } else {
                    throw std::runtime_error("Quantization of cell '" + cell->getName() + "' of type '" + cell->getType() + "' is not supported yet.");
                }
                const long double biasScaling = biasScalings.at(cell->getName());
                activationScaling /= biasScaling;
                activationScaling = (activationScaling == 0.0) ? 1.0 : activationScaling;
                activationScalings[cell->getName()] = activationScaling;
                cell->processFreeParameters([&](Float_T d) { return (Float_T)(d / prevActivationScaling); }, Cell::Additive);
                const long double actQuantScaling = getActivationQuantizationScaling(*cell, nbBits);
                auto scalingCell = std::make_shared<ScalingCell>(
                    mDeepNet.generateNewCellName(cell->getName() + "_rescale_act"), cell->getNbOutputs(),
                    Scaling::floatingPointScaling(std::vector<Float_T>(cell->getNbOutputs(), (Float_T)((prevActivationScaling / activationScaling) / actQuantScaling)),
                                                  false, {}));
                mDeepNet.addCellAfter(scalingCell, cell);
                activationScalings[scalingCell->getName()] = activationScalings[cell->getName()];
                biasScalings[scalingCell->getName()] = biasScaling;
            }
        fuseScalingCells();
    }

    double getActivationQuantizationScaling(const Cell& cell, std::size_t nbBits) const
    {
        const double unsignedMax = std::pow(2, nbBits) - 1;
        const double signedMax = std::pow(2, nbBits - 1) - 1;
        if (!cell.getActivation() || dynamic_cast<const ElemWiseCell*>(&cell)) return 1.0;
        if (mDeepNet.isCellOutputUnsigned(cell))
            return mDeepNet.isCellInputsUnsigned(cell) ? signedMax * unsignedMax / unsignedMax : signedMax * signedMax / unsignedMax;
        return mDeepNet.isCellInputsUnsigned(cell) ? signedMax * unsignedMax / signedMax : signedMax * signedMax / signedMax;
    }

    void fuseScalingCells()
    {
        const std::vector<std::vector<std::string> > layers = mDeepNet.getLayers();   // a copy: the loop edits the graph
        for (std::size_t l = 1; l < layers.size(); ++l)
            for (const std::string& name : layers[l]) {
                if (!mDeepNet.hasCell(name)) continue;
                std::shared_ptr<Cell> cell = mDeepNet.getCell<Cell>(name);
                auto scalingCell = std::dynamic_pointer_cast<ScalingCell>(cell);
                if (!scalingCell) continue;
                auto parentsCells = mDeepNet.getParentCells(cell->getName());
                if (parentsCells.size() != 1 || !parentsCells.front() || mDeepNet.getChildCells(parentsCells.front()->getName()).size() != 1) continue;
                auto parentCell = parentsCells.front();
                auto parentScalingCell = std::dynamic_pointer_cast<ScalingCell>(parentCell);
                auto parentElemWiseCell = std::dynamic_pointer_cast<ElemWiseCell>(parentCell);
                if (parentScalingCell) {
                    // (a ScalingCell of this library carries its Scaling in a private Linear activation: test the type first)
                    fuseScalingCellWithParentScalingCell(scalingCell, parentScalingCell);
                } else if (parentCell->getActivation()) {
                    fuseScalingCellWithParentActivation(scalingCell, *parentCell->getActivation());
                } else if (parentElemWiseCell) {
                    if (moveScalingCellAboveParentElemWiseCell(scalingCell, parentElemWiseCell)) {
                        // the ScalingCell now sits on the sum's inputs: try to merge it with its new parents
                        fuseScalingCells();
                        return;
                    }
                }
            }
    }

    void approximateScalingCell(ScalingCell& cell, ScalingMode scalingCellMode)
    {
        if (cell.getScaling().getMode() != ScalingMode::FLOAT_MULT) throw std::runtime_error("approximateScalingCell(): the cell's scaling is not floating-point");
        if (scalingCellMode == ScalingMode::FLOAT_MULT) return;
        if (scalingCellMode != ScalingMode::FIXED_MULT16 && scalingCellMode != ScalingMode::FIXED_MULT32)
            throw std::runtime_error("The scaling cell can only be approximated by a fixed-point approximation.");
        auto scalingFixedPoint = approximateScalingWithFixedPoint(scalingCellMode, cell.getScaling().getFloatingPointScalingPerOutput());
        cell.setScaling(Scaling::fixedPointScaling(scalingCellMode, scalingFixedPoint.first, scalingFixedPoint.second, false, {}));
    }

    void approximateActivationScaling(Cell& cell, Activation& activation, ScalingMode actScalingMode)
    {
        if (activation.getActivationScaling().getMode() != ScalingMode::FLOAT_MULT)
            throw std::runtime_error("approximateActivationScaling(): the activation of " + cell.getName() + " has no floating-point scaling");
        const std::vector<Float_T> scalingPerOutput = activation.getActivationScaling().getFloatingPointScalingPerOutput();
        if ((actScalingMode == ScalingMode::SINGLE_SHIFT || actScalingMode == ScalingMode::DOUBLE_SHIFT)
            && std::any_of(scalingPerOutput.begin(), scalingPerOutput.end(), [](Float_T s) { return s > 1.0; }))
            actScalingMode = ScalingMode::FIXED_MULT16;   // scalings above 1 have no shift form
        if (actScalingMode == ScalingMode::FLOAT_MULT) return;
        if (actScalingMode == ScalingMode::FIXED_MULT32 || actScalingMode == ScalingMode::FIXED_MULT16) {
            auto scalingFixedPoint = approximateScalingWithFixedPoint(actScalingMode, scalingPerOutput);
            activation.setActivationScaling(Scaling::fixedPointScaling(actScalingMode, scalingFixedPoint.first, scalingFixedPoint.second, false, {}));
        } else if (actScalingMode == ScalingMode::SINGLE_SHIFT) {
            std::vector<unsigned char> shifts;
            for (const auto& exps : approximateActivationScalingWithPowerOf2Divs(cell, scalingPerOutput, 1)) shifts.push_back(exps[0]);
            activation.setActivationScaling(Scaling::singleShiftScaling(shifts, false, {}));
        } else if (actScalingMode == ScalingMode::DOUBLE_SHIFT) {
            std::vector<std::pair<unsigned char, unsigned char> > shifts;
            for (const auto& exps : approximateActivationScalingWithPowerOf2Divs(cell, scalingPerOutput, 2)) {
                assert(exps[0] <= exps[1]);
                shifts.push_back(std::make_pair((unsigned char)(exps[1] - exps[0]), exps[1]));
            }
            activation.setActivationScaling(Scaling::doubleShiftScaling(shifts, false, {std::make_pair((unsigned char)0, (unsigned char)0)}));
        } else {
            throw std::runtime_error("Unsupported scaling mode.");
        }
    }

private:
    static Float_T maxAbs(Float_T a, Float_T b) { return std::max(std::abs(a), std::abs(b)); }

    std::vector<std::vector<unsigned char> > approximateActivationScalingWithPowerOf2Divs(Cell& cell, const std::vector<Float_T>& scalingPerOutput,
                                                                                        std::size_t nbDivisions)
    {
        std::vector<std::vector<unsigned char> > exponentsPerOutput(cell.getNbOutputs());
        for (std::size_t output = 0; output < cell.getNbOutputs(); output++) {
            const auto approx = approximateScalingWithPowerOf2Divs(scalingPerOutput[output], nbDivisions);
            exponentsPerOutput[output] = approx.first;
            const Float_T rescaleOutputsBy = (Float_T)(1 / approx.second);
            // the weights and biases of the output absorb what the approximation lost
            cell.processFreeParametersPerOutput([&](Float_T d) { return rescaleOutputsBy * d; }, output);
        }
        return exponentsPerOutput;
    }

    long double getMaxParentsScaling(const std::shared_ptr<Cell>& cell, const std::unordered_map<std::string, long double>& scalingForCells) const
    {
        long double maxParentsScaling = 0.0;
        for (const auto& parentCell : mDeepNet.getParentCells(cell->getName())) {
            const long double parentScaling = parentCell ? scalingForCells.at(parentCell->getName()) : 1.0;
            maxParentsScaling = std::max(maxParentsScaling, parentScaling);
        }
        return maxParentsScaling;
    }

    void rescaleParentsToScaling(const std::shared_ptr<Cell>& cell, const std::unordered_map<std::string, long double>& scalingForCells,
                                 long double scaling)
    {
        const std::vector<std::shared_ptr<Cell> > parentsCells = mDeepNet.getParentCells(cell->getName());   // a copy: the loop edits the graph
        for (const std::shared_ptr<Cell>& parentCell : parentsCells) {
            const long double parentScaling = parentCell ? scalingForCells.at(parentCell->getName()) : 1.0;
            if (parentScaling == scaling) continue;
            if (!parentCell) throw std::runtime_error("rescaleParentsToScaling(): the stimuli cannot be re-scaled (cell " + cell->getName() + ")");
            auto scalingCell = std::make_shared<ScalingCell>(
                mDeepNet.generateNewCellName(parentCell->getName() + "_rescale_branch"), parentCell->getNbOutputs(),
                Scaling::floatingPointScaling(std::vector<Float_T>(parentCell->getNbOutputs(), (Float_T)(parentScaling / scaling)), false, {}));
            mDeepNet.addCellBetween(scalingCell, parentCell, cell);
        }
    }

    void fuseScalingCellWithParentActivation(const std::shared_ptr<ScalingCell>& scalingCell, Activation& parentCellActivation)
    {
        const std::vector<Float_T>& scalingPerOutput = scalingCell->getScaling().getFloatingPointScalingPerOutput();
        const ScalingMode parentScalingMode = parentCellActivation.getActivationScaling().getMode();
        if (parentScalingMode == ScalingMode::NONE) {
            parentCellActivation.setActivationScaling(scalingCell->getScaling());
            mDeepNet.removeCell(scalingCell);
        } else if (parentScalingMode == ScalingMode::FLOAT_MULT) {
            std::vector<Float_T> parentScalingPerOutput = parentCellActivation.getActivationScaling().getFloatingPointScalingPerOutput();
            for (std::size_t o = 0; o < parentScalingPerOutput.size(); o++) parentScalingPerOutput[o] *= scalingPerOutput[o];
            parentCellActivation.setActivationScaling(Scaling::floatingPointScaling(std::move(parentScalingPerOutput), false, {}));
            mDeepNet.removeCell(scalingCell);
        }
    }

    void fuseScalingCellWithParentScalingCell(const std::shared_ptr<ScalingCell>& scalingCell, const std::shared_ptr<ScalingCell>& parentScalingCell)
    {
        const std::vector<Float_T>& scalingPerOutput = scalingCell->getScaling().getFloatingPointScalingPerOutput();
        std::vector<Float_T> parentScalingPerOutput = parentScalingCell->getScaling().getFloatingPointScalingPerOutput();
        for (std::size_t o = 0; o < parentScalingPerOutput.size(); o++) parentScalingPerOutput[o] *= scalingPerOutput[o];
        parentScalingCell->setScaling(Scaling::floatingPointScaling(std::move(parentScalingPerOutput), false, {}));
        mDeepNet.removeCell(scalingCell);
    }

    // A sum with unit weights and no shifts commutes with a per-channel scaling: the ScalingCell is replaced by one
    // `_rescale_elemwise` ScalingCell on every input of the sum.
    bool moveScalingCellAboveParentElemWiseCell(const std::shared_ptr<ScalingCell>& scalingCell, const std::shared_ptr<ElemWiseCell>& parentElemWiseCell)
    {
        const std::vector<Float_T> scalingPerOutput = scalingCell->getScaling().getFloatingPointScalingPerOutput();
        auto grandParentsCells = mDeepNet.getParentCells(parentElemWiseCell->getName());
        for (auto grandParentCell : grandParentsCells) {
            if (!grandParentCell) return false;   // the stimuli themselves cannot carry a ScalingCell
        }
        for (auto grandParentCell : grandParentsCells) {
            auto grandParentScalingCell = std::make_shared<ScalingCell>(
                mDeepNet.generateNewCellName(grandParentCell->getName() + "_rescale_elemwise"), grandParentCell->getNbOutputs(),
                Scaling::floatingPointScaling(scalingPerOutput, false, {}));
            mDeepNet.addCellBetween(grandParentScalingCell, grandParentCell, parentElemWiseCell);
        }
        mDeepNet.removeCell(scalingCell);
        return true;
    }

    DeepNet& mDeepNet;
};

}  // namespace N2D2
