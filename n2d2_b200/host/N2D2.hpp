// Host-side C++ mirror of the part of N2D2's API that the quantized inference path uses, on top of
// the C ABI (include/n2d2b.h).  Class, factory and method names follow the reference so that code
// written against its Cell / Scaling / DeepNet interface reads the same here:
//
//   Scaling, ScalingMode               include/Scaling.hpp:339-373, include/ScalingMode.hpp:27-34
//   Activation and its three kinds     include/Activation/Activation.hpp:36-110
//   Cell::setQuantized & co            include/Cell/Cell.hpp:75-85
//   ConvCell creation arguments        include/Cell/ConvCell.hpp:45-55
//   DeepNet::addCell / getCell /
//     getLayers / test                 src/DeepNet.cpp:74-290,2622-2768
//   DeepNetExport::isCellOutputUnsigned src/Export/DeepNetExport.cpp:370-388
//
// Differences that follow from the integer representation: weights and stimuli are 8-bit integers
// (the reference holds the same integers in float tensors), activations live on the GPU as NHWC,
// and errors of the C ABI surface as std::runtime_error like the reference's own.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/n2d2b.h"

namespace N2D2 {

typedef float Float_T;

enum class ScalingMode { NONE, FLOAT_MULT, FIXED_MULT16, FIXED_MULT32, SINGLE_SHIFT, DOUBLE_SHIFT };

// Value type holding the per-output rescale of an activation (include/Scaling.hpp:45-427).
class Scaling {
public:
    Scaling() : mMode(ScalingMode::NONE), mNbFractionalBits(0), mIsClipped(false) {}

    static Scaling floatingPointScaling(std::vector<Float_T> scalingPerOutput, bool isClipped,
                                        std::vector<Float_T> clippingPerOutput)
    {
        Scaling s;
        s.mMode = ScalingMode::FLOAT_MULT;
        s.mFloat = std::move(scalingPerOutput);
        s.mIsClipped = isClipped;
        s.mClipping = std::move(clippingPerOutput);
        return s;
    }
    static Scaling fixedPointScaling(ScalingMode mode, std::size_t nbFractionalBits,
                                     std::vector<std::int32_t> scalingPerOutput, bool isClipped,
                                     std::vector<Float_T> clippingPerOutput)
    {
        if (mode != ScalingMode::FIXED_MULT16 && mode != ScalingMode::FIXED_MULT32)
            throw std::runtime_error("Scaling::fixedPointScaling(): mode must be FIXED_MULT16 or FIXED_MULT32");
        Scaling s;
        s.mMode = mode;
        s.mNbFractionalBits = nbFractionalBits;
        s.mFixed = std::move(scalingPerOutput);
        s.mIsClipped = isClipped;
        s.mClipping = std::move(clippingPerOutput);
        return s;
    }
    static Scaling singleShiftScaling(std::vector<unsigned char> scalingPerOutput, bool isClipped,
                                      std::vector<Float_T> clippingPerOutput)
    {
        Scaling s;
        s.mMode = ScalingMode::SINGLE_SHIFT;
        s.mShift0 = std::move(scalingPerOutput);
        s.mIsClipped = isClipped;
        s.mClipping = std::move(clippingPerOutput);
        return s;
    }
    static Scaling doubleShiftScaling(std::vector<std::pair<unsigned char, unsigned char> > scalingPerOutput,
                                      bool isClipped,
                                      std::vector<std::pair<unsigned char, unsigned char> > /*clippingPerOutput*/)
    {
        Scaling s;
        s.mMode = ScalingMode::DOUBLE_SHIFT;
        for (const auto& p : scalingPerOutput) {
            s.mShift0.push_back(p.first);
            s.mShift1.push_back(p.second);
        }
        s.mIsClipped = isClipped;  // ignored by the shift modes, as on the reference's CPU path
        return s;
    }

    ScalingMode getMode() const { return mMode; }
    std::size_t getFractionalBits() const { return mNbFractionalBits; }
    bool getIsClipped() const { return mIsClipped; }
    // payloads (getFloatingPointScaling().getScalingPerOutput() etc. in the reference)
    const std::vector<Float_T>& getFloatingPointScalingPerOutput() const { return mFloat; }
    const std::vector<std::int32_t>& getFixedPointScalingPerOutput() const { return mFixed; }
    const std::vector<unsigned char>& getSingleShiftScalingPerOutput() const { return mShift0; }
    std::vector<std::pair<unsigned char, unsigned char> > getDoubleShiftScalingPerOutput() const
    {
        std::vector<std::pair<unsigned char, unsigned char> > v;
        for (std::size_t i = 0; i < mShift0.size(); ++i) v.emplace_back(mShift0[i], mShift1[i]);
        return v;
    }
    const std::vector<Float_T>& getClippingPerOutput() const { return mClipping; }

    // Fills the C-ABI view (pointers stay valid as long as this object lives).
    void describe(n2d2b_scaling& d, int nbOutputs) const
    {
        d = n2d2b_scaling();
        d.mode = (int32_t)mMode;
        d.nb_channels = nbOutputs;
        d.fscale = mFloat.empty() ? nullptr : mFloat.data();
        d.mult = mFixed.empty() ? nullptr : mFixed.data();
        d.frac_bits = (int32_t)mNbFractionalBits;
        d.shift0 = mShift0.empty() ? nullptr : mShift0.data();
        d.shift1 = mShift1.empty() ? nullptr : mShift1.data();
        d.is_clipped = (mIsClipped && !mClipping.empty()) ? 1 : 0;
        d.clip = mClipping.empty() ? nullptr : mClipping.data();
    }

private:
    ScalingMode mMode;
    std::size_t mNbFractionalBits;
    bool mIsClipped;
    std::vector<Float_T> mFloat, mClipping;
    std::vector<std::int32_t> mFixed;
    std::vector<unsigned char> mShift0, mShift1;
};

// Activation: owns the Scaling (include/Activation/Activation.hpp:70-99).
class Activation {
public:
    virtual ~Activation() {}
    virtual const char* getType() const = 0;
    virtual int kind() const = 0;
    void setActivationScaling(Scaling scaling) { mScaling = std::move(scaling); }
    const Scaling& getActivationScaling() const { return mScaling; }
    void setQuantized(std::size_t nbBits) { mQuantizedNbBits = nbBits; }
    std::size_t getQuantizedNbBits() const { return mQuantizedNbBits; }

protected:
    Scaling mScaling;
    std::size_t mQuantizedNbBits = 0;
};
class LinearActivation : public Activation {
public:
    const char* getType() const override { return "Linear"; }
    int kind() const override { return N2D2B_ACT_LINEAR; }
};
class RectifierActivation : public Activation {
public:
    const char* getType() const override { return "Rectifier"; }
    int kind() const override { return N2D2B_ACT_RECTIFIER; }
};
class SaturationActivation : public Activation {
public:
    explicit SaturationActivation(int threshold = 0) : mThreshold(threshold) {}
    const char* getType() const override { return "Saturation"; }
    int kind() const override { return N2D2B_ACT_SATURATION; }
    int mThreshold;
};

// Process-wide export switches the reference keeps as statics (src/Export/DeepNetExport.cpp:33-34)
struct DeepNetExport {
    static bool& mUnsignedData() { static bool v = true; return v; }
    static bool& mEnvDataUnsigned() { static bool v = true; return v; }
};

class DeepNet;
struct Network {};   // the reference's event-simulation context, first argument of its cell factories; empty here

class Cell {
public:
    Cell(const std::string& name, unsigned int nbOutputs) : mName(name), mNbOutputs(nbOutputs) {}
    virtual ~Cell() {}
    virtual const char* getType() const = 0;
    const std::string& getName() const { return mName; }
    unsigned int getNbOutputs() const { return mNbOutputs; }
    bool isQuantized() const { return mQuantizedNbBits > 0; }
    void setQuantized(std::size_t nbBits) { mQuantizedNbBits = nbBits; }
    std::size_t getQuantizedNbBits() const { return mQuantizedNbBits; }
    const std::shared_ptr<Activation>& getActivation() const { return mActivation; }
    void setActivation(const std::shared_ptr<Activation>& activation) { mActivation = activation; }
    unsigned int getOutputsWidth() const { return mOutputsWidth; }
    unsigned int getOutputsHeight() const { return mOutputsHeight; }
    // known once the cell is wired into a DeepNet
    unsigned int getNbChannels() const { return mNbChannels; }
    unsigned int getChannelsWidth() const { return mChannelsWidth; }
    unsigned int getChannelsHeight() const { return mChannelsHeight; }

    // Free parameters while the network is still in floating point (before and during post-training
    // quantization): Multiplicative = weights, Additive = biases (include/Cell/Cell.hpp FreeParametersType).
    enum FreeParametersType { Additive, Multiplicative, All };
    virtual void processFreeParameters(const std::function<Float_T(Float_T)>& /*func*/, FreeParametersType /*type*/ = All) {}
    virtual void processFreeParametersPerOutput(const std::function<Float_T(Float_T)>& /*func*/, std::size_t /*output*/,
                                                FreeParametersType /*type*/ = All) {}
    virtual std::pair<Float_T, Float_T> getFreeParametersRange(FreeParametersType /*type*/ = All) const { return std::make_pair(0.0f, 0.0f); }
    virtual std::pair<Float_T, Float_T> getFreeParametersRangePerOutput(std::size_t /*output*/, FreeParametersType /*type*/ = All) const
    {
        return std::make_pair(0.0f, 0.0f);
    }
    // Rounds the floating-point parameters and stores them as the integers the device takes; throws when a value
    // does not fit (weights: nbBits signed; biases: 32 bits).
    virtual void roundFreeParameters(std::size_t /*nbBits*/) {}

    // Signedness of the cell's output as DeepNetExport::isCellOutputUnsigned derives it: unsigned only
    // when unsigned data is allowed and the output range starts at 0 (a Rectifier); may be overridden.
    bool isOutputUnsigned() const
    {
        if (mForcedSign >= 0) return mForcedSign != 0;
        return DeepNetExport::mUnsignedData() && mActivation && mActivation->kind() == N2D2B_ACT_RECTIFIER;
    }
    void setOutputUnsigned(bool u) { mForcedSign = u ? 1 : 0; }

protected:
    friend class DeepNet;
    // what the activation does on the way out, as the C ABI wants it
    void describeQuant(n2d2b_quant& q) const
    {
        q = n2d2b_quant();
        static const Scaling none;
        const Scaling& s = mActivation ? mActivation->getActivationScaling() : none;
        s.describe(q.scaling, (int)mNbOutputs);
        q.activation = mActivation ? mActivation->kind() : N2D2B_ACT_LINEAR;
        const std::size_t actBits = mActivation ? mActivation->getQuantizedNbBits() : 0;
        q.out_bits = (int32_t)(actBits > 0 ? actBits : (mQuantizedNbBits > 0 ? mQuantizedNbBits : 8));
        q.out_unsigned = isOutputUnsigned() ? 1 : 0;
        if (auto* sat = dynamic_cast<const SaturationActivation*>(mActivation.get())) q.saturation_threshold = sat->mThreshold;
    }
    std::string mName;
    unsigned int mNbOutputs;
    std::size_t mQuantizedNbBits = 0;
    std::shared_ptr<Activation> mActivation;
    unsigned int mOutputsWidth = 0, mOutputsHeight = 0;
    unsigned int mNbChannels = 0, mChannelsWidth = 0, mChannelsHeight = 0;
    int mForcedSign = -1;
    int mTensorId = -1;
};

// Floating-point weights [output][...] and biases [output] with the reference's processing hooks; shared by the
// convolution and the fully-connected cell.
class FreeParametersCell : public Cell {
public:
    using Cell::Cell;
    // weights in the reference's memory order, one contiguous run per output; biases may be empty (NoBias)
    void setFloatWeights(const std::vector<Float_T>& w) { mFloatWeights = w; }
    void setFloatBiases(const std::vector<Float_T>& b) { mFloatBiases = b; }
    const std::vector<Float_T>& getFloatWeights() const { return mFloatWeights; }
    const std::vector<Float_T>& getFloatBiases() const { return mFloatBiases; }

    void processFreeParameters(const std::function<Float_T(Float_T)>& func, FreeParametersType type = All) override
    {
        if (type != Additive) for (Float_T& w : mFloatWeights) w = func(w);
        if (type != Multiplicative) for (Float_T& b : mFloatBiases) b = func(b);
    }
    void processFreeParametersPerOutput(const std::function<Float_T(Float_T)>& func, std::size_t output, FreeParametersType type = All) override
    {
        const std::size_t per = mFloatWeights.size() / mNbOutputs;
        if (type != Additive) for (std::size_t i = output * per; i < (output + 1) * per; ++i) mFloatWeights[i] = func(mFloatWeights[i]);
        if (type != Multiplicative && !mFloatBiases.empty()) mFloatBiases[output] = func(mFloatBiases[output]);
    }
    std::pair<Float_T, Float_T> getFreeParametersRange(FreeParametersType type = All) const override
    {
        Float_T lo = 0.0f, hi = 0.0f;
        bool first = true;
        auto take = [&](Float_T v) { if (first) { lo = hi = v; first = false; } else { lo = std::min(lo, v); hi = std::max(hi, v); } };
        if (type != Additive) for (Float_T w : mFloatWeights) take(w);
        if (type != Multiplicative) for (Float_T b : mFloatBiases) take(b);
        return std::make_pair(lo, hi);
    }
    std::pair<Float_T, Float_T> getFreeParametersRangePerOutput(std::size_t output, FreeParametersType type = All) const override
    {
        Float_T lo = 0.0f, hi = 0.0f;
        bool first = true;
        auto take = [&](Float_T v) { if (first) { lo = hi = v; first = false; } else { lo = std::min(lo, v); hi = std::max(hi, v); } };
        const std::size_t per = mFloatWeights.size() / mNbOutputs;
        if (type != Additive) for (std::size_t i = output * per; i < (output + 1) * per; ++i) take(mFloatWeights[i]);
        if (type != Multiplicative && !mFloatBiases.empty()) take(mFloatBiases[output]);
        return std::make_pair(lo, hi);
    }

protected:
    void roundInto(std::size_t nbBits, std::vector<std::int8_t>& weights, std::vector<std::int32_t>& biases)
    {
        if (mFloatWeights.empty()) return;
        const long long wMax = (1ll << (nbBits - 1)) - 1, wMin = -(1ll << (nbBits - 1));
        weights.resize(mFloatWeights.size());
        for (std::size_t i = 0; i < mFloatWeights.size(); ++i) {
            const long long r = std::llround((double)mFloatWeights[i]);
            if (r < wMin || r > wMax) throw std::runtime_error("Cell " + mName + ": a rounded weight does not fit " + std::to_string(nbBits) + " bits");
            weights[i] = (std::int8_t)r;
        }
        biases.resize(mFloatBiases.size());
        for (std::size_t i = 0; i < mFloatBiases.size(); ++i) {
            const long long r = std::llround((double)mFloatBiases[i]);
            if (r < INT32_MIN || r > INT32_MAX) throw std::runtime_error("Cell " + mName + ": a rounded bias does not fit 32 bits");
            biases[i] = (std::int32_t)r;
        }
    }
    std::vector<Float_T> mFloatWeights, mFloatBiases;
};

class ConvCell : public FreeParametersCell {
public:
    // kernelDims / strideDims / dilationDims are {x, y}; paddingDims {x, y} or {left, top, right, bottom}
    ConvCell(const std::string& name, const std::vector<unsigned int>& kernelDims, unsigned int nbOutputs,
             const std::vector<unsigned int>& subSampleDims = {1, 1}, const std::vector<unsigned int>& strideDims = {1, 1},
             const std::vector<int>& paddingDims = {0, 0}, const std::vector<unsigned int>& dilationDims = {1, 1},
             const std::shared_ptr<Activation>& activation = std::shared_ptr<Activation>())
        : FreeParametersCell(name, nbOutputs), mKernelDims(kernelDims), mStrideDims(strideDims), mPaddingDims(paddingDims),
          mDilationDims(dilationDims)
    {
        for (unsigned int s : subSampleDims)
            if (s != 1) throw std::domain_error("ConvCell: sub-sampling is not supported (the reference's CUDA cell rejects it too)");
        if (mPaddingDims.size() == 2) { mPaddingDims.push_back(mPaddingDims[0]); mPaddingDims.push_back(mPaddingDims[1]); }
        mActivation = activation;
    }
    // The reference's creation signature (include/Cell/ConvCell.hpp:45-55): the event-simulation Network and the
    // DeepNet arguments carry nothing on this path.
    ConvCell(Network& /*net*/, const DeepNet& /*deepNet*/, const std::string& name, const std::vector<unsigned int>& kernelDims,
             unsigned int nbOutputs, const std::vector<unsigned int>& subSampleDims = {1, 1},
             const std::vector<unsigned int>& strideDims = {1, 1}, const std::vector<int>& paddingDims = {0, 0},
             const std::vector<unsigned int>& dilationDims = {1, 1},
             const std::shared_ptr<Activation>& activation = std::shared_ptr<Activation>())
        : ConvCell(name, kernelDims, nbOutputs, subSampleDims, strideDims, paddingDims, dilationDims, activation)
    {
    }
    const char* getType() const override { return "Conv"; }
    void setNbGroups(unsigned int groups) { mGroups = groups; }
    unsigned int getNbGroups() const { return mGroups; }
    // One kernel, as ConvCell::setWeight(output, channel, kernel) (include/Cell/ConvCell_Frame_CUDA.hpp:109-198):
    // kernel = kernelHeight x kernelWidth values, x fastest; channel counts within the output's group.  Valid once
    // the cell is wired into a DeepNet (the number of channels is known then).
    void setWeight(unsigned int output, unsigned int channel, const std::vector<std::int8_t>& kernel)
    {
        const std::size_t cg = mNbChannels / mGroups, ks = (std::size_t)mKernelDims[0] * mKernelDims[1];
        if (cg == 0) throw std::runtime_error("ConvCell::setWeight(): add the cell to a DeepNet first");
        if (output >= mNbOutputs || channel >= cg || kernel.size() != ks) throw std::runtime_error("ConvCell::setWeight(): out of range");
        if (mWeights.size() != (std::size_t)mNbOutputs * cg * ks) mWeights.assign((std::size_t)mNbOutputs * cg * ks, 0);
        std::copy(kernel.begin(), kernel.end(), mWeights.begin() + ((std::size_t)output * cg + channel) * ks);
    }
    void setBias(unsigned int output, std::int32_t value)
    {
        if (output >= mNbOutputs) throw std::runtime_error("ConvCell::setBias(): out of range");
        if (mBiases.size() != mNbOutputs) mBiases.assign(mNbOutputs, 0);
        mBiases[output] = value;
    }
    // Sparse connection map of the cell (the `mapping` argument of Cell::addInput and Cell::isConnection,
    // include/Cell/Cell.hpp; the reference's ini files write it as Mapping(...)): mapping[output * nbChannels + channel]
    // says whether the channel feeds the output.  The reference's kernels skip unconnected channels
    // (src/Cell/ConvCell_Frame_Kernels.cpp:93-96); here their weights are zero in the dense layer the device runs,
    // which gives the same integers.  Only without groups.
    void setMapping(const std::vector<bool>& mapping) { mMapping = mapping; }
    bool isConnection(unsigned int channel, unsigned int output) const
    {
        return mMapping.empty() || mMapping[(std::size_t)output * mNbChannels + channel];
    }
    const std::vector<std::int8_t>& getWeights() const { return mWeights; }
    const std::vector<std::int32_t>& getBiases() const { return mBiases; }
    void roundFreeParameters(std::size_t nbBits) override { roundInto(nbBits, mWeights, mBiases); }
    // weights in the reference's memory order: [output][channel][ky][kx] (kx fastest)
    void setWeights(const std::vector<std::int8_t>& oihw) { mWeights = oihw; }
    void setBiases(const std::vector<std::int32_t>& biases) { mBiases = biases; }
    std::int8_t getWeight(unsigned int output, unsigned int channel, unsigned int sx, unsigned int sy) const
    {
        const std::size_t cg = mWeights.size() / ((std::size_t)mNbOutputs * mKernelDims[0] * mKernelDims[1]);
        return mWeights[(((std::size_t)output * cg + channel) * mKernelDims[1] + sy) * mKernelDims[0] + sx];
    }

private:
    friend class DeepNet;
    std::vector<unsigned int> mKernelDims, mStrideDims;
    std::vector<int> mPaddingDims;
    std::vector<unsigned int> mDilationDims;
    unsigned int mGroups = 1;
    std::vector<bool> mMapping;
    std::vector<std::int8_t> mWeights;
    std::vector<std::int32_t> mBiases;
};

class FcCell : public FreeParametersCell {
public:
    FcCell(const std::string& name, unsigned int nbOutputs,
           const std::shared_ptr<Activation>& activation = std::shared_ptr<Activation>())
        : FreeParametersCell(name, nbOutputs)
    {
        mActivation = activation;
    }
    const char* getType() const override { return "Fc"; }
    // weights in the reference's order: [output][channel][y][x] over the input tensor
    void setWeights(const std::vector<std::int8_t>& w) { mWeights = w; }
    void setBiases(const std::vector<std::int32_t>& biases) { mBiases = biases; }
    const std::vector<std::int8_t>& getWeights() const { return mWeights; }
    const std::vector<std::int32_t>& getBiases() const { return mBiases; }
    void roundFreeParameters(std::size_t nbBits) override { roundInto(nbBits, mWeights, mBiases); }

private:
    friend class DeepNet;
    std::vector<std::int8_t> mWeights;
    std::vector<std::int32_t> mBiases;
};

class PoolCell : public Cell {
public:
    enum Pooling { Max, Average };
    PoolCell(const std::string& name, const std::vector<unsigned int>& poolDims, unsigned int nbOutputs,
             const std::vector<unsigned int>& strideDims = {1, 1}, const std::vector<unsigned int>& paddingDims = {0, 0},
             Pooling pooling = Max)
        : Cell(name, nbOutputs), mPoolDims(poolDims), mStrideDims(strideDims), mPaddingDims(paddingDims), mPooling(pooling)
    {
    }
    const char* getType() const override { return "Pool"; }
    Pooling getPooling() const { return mPooling; }

private:
    friend class DeepNet;
    std::vector<unsigned int> mPoolDims, mStrideDims, mPaddingDims;
    Pooling mPooling;
};

class ElemWiseCell : public Cell {
public:
    enum Operation { Sum };
    ElemWiseCell(const std::string& name, unsigned int nbOutputs, Operation operation = Sum,
                 const std::shared_ptr<Activation>& activation = std::shared_ptr<Activation>())
        : Cell(name, nbOutputs)
    {
        if (operation != Sum) throw std::runtime_error("ElemWiseCell: only Sum exists on the quantized path");
        mActivation = activation;
    }
    const char* getType() const override { return "ElemWise"; }
};

class ScalingCell : public Cell {
public:
    ScalingCell(const std::string& name, unsigned int nbOutputs, Scaling scaling) : Cell(name, nbOutputs)
    {
        // a ScalingCell applies its Scaling with its own quantized bit count and no non-linearity
        mActivation = std::make_shared<LinearActivation>();
        mActivation->setActivationScaling(std::move(scaling));
    }
    const char* getType() const override { return "Scaling"; }
    const Scaling& getScaling() const { return mActivation->getActivationScaling(); }
    void setScaling(Scaling scaling) { mActivation->setActivationScaling(std::move(scaling)); }
};

// Graph container + executor (src/DeepNet.cpp:74-415,826-854,2622-2768).  The graph lives on the host as in
// the reference: mLayers (layer 0 is the environment) gives the execution order, mParentLayers the wiring.
// It can be edited (addCellAfter / Before / Between, removeCell: what the post-training quantization does when
// it inserts and fuses ScalingCells) until initialize() hands the cells, layer by layer, to the C ABI.
class DeepNet {
public:
    DeepNet(unsigned int stimuliChannels, unsigned int stimuliHeight, unsigned int stimuliWidth, int device = 0)
        : mDevice(device), mStimuli{stimuliChannels, stimuliHeight, stimuliWidth}
    {
        mLayers.push_back(std::vector<std::string>(1, "env"));
    }
    ~DeepNet() { if (mNet) n2d2b_net_destroy(mNet); }
    DeepNet(const DeepNet&) = delete;
    DeepNet& operator=(const DeepNet&) = delete;

    // parents: empty or a null pointer = the stimuli (the reference passes a null parent for the environment)
    void addCell(const std::shared_ptr<Cell>& cell, const std::vector<std::shared_ptr<Cell> >& parents)
    {
        editable();
        if (mCells.count(cell->getName())) throw std::runtime_error("DeepNet::addCell(): cell " + cell->getName() + " already exists");
        std::vector<std::shared_ptr<Cell> > ps = parents;
        if (ps.empty()) ps.push_back(std::shared_ptr<Cell>());
        std::size_t order = 0;
        for (const auto& p : ps)
            if (p) order = std::max(order, layerOf(p->getName()));
        if (order + 1 >= mLayers.size()) mLayers.resize(order + 2);
        mLayers[order + 1].push_back(cell->getName());
        for (const auto& p : ps) mParentLayers.emplace_back(cell->getName(), p ? p->getName() : std::string("env"));
        mCells[cell->getName()] = cell;
        inferShapes();
    }

    // newCell takes `parent` as its input and every child of `parent` is re-wired to newCell
    void addCellAfter(const std::shared_ptr<Cell>& newCell, const std::shared_ptr<Cell>& parent)
    {
        editable();
        insertNew(newCell);
        for (auto& link : mParentLayers)
            if (link.second == parent->getName()) link.second = newCell->getName();
        mParentLayers.emplace_back(newCell->getName(), parent->getName());
        mLayers.insert(mLayers.begin() + layerOf(parent->getName()) + 1, std::vector<std::string>(1, newCell->getName()));
        inferShapes();
    }

    // newCell takes all the parents of `child`, and `child` takes newCell as its only input
    void addCellBefore(const std::shared_ptr<Cell>& newCell, const std::shared_ptr<Cell>& child)
    {
        editable();
        insertNew(newCell);
        std::vector<std::pair<std::string, std::string> > links;
        bool placed = false;
        for (const auto& link : mParentLayers) {
            if (link.first != child->getName()) { links.push_back(link); continue; }
            links.emplace_back(newCell->getName(), link.second);
            placed = true;
        }
        if (!placed) throw std::runtime_error("The cell '" + child->getName() + "' was not found in the graph.");
        links.emplace_back(child->getName(), newCell->getName());
        mParentLayers.swap(links);
        mLayers.insert(mLayers.begin() + layerOf(child->getName()), std::vector<std::string>(1, newCell->getName()));
        inferShapes();
    }

    void addCellBetween(const std::shared_ptr<Cell>& newCell, const std::shared_ptr<Cell>& parent, const std::shared_ptr<Cell>& child)
    {
        editable();
        bool found = false;
        for (const auto& link : mParentLayers) found = found || (link.first == child->getName() && link.second == parent->getName());
        if (!found) throw std::runtime_error("The cell '" + parent->getName() + "' isn't a parent of the cell '" + child->getName() + "'.");
        insertNew(newCell);
        for (auto& link : mParentLayers)
            if (link.first == child->getName() && link.second == parent->getName()) { link.second = newCell->getName(); break; }
        mParentLayers.emplace_back(newCell->getName(), parent->getName());
        mLayers.insert(mLayers.begin() + layerOf(parent->getName()) + 1, std::vector<std::string>(1, newCell->getName()));
        inferShapes();
    }

    // reconnect: the children of `cell` take its parents, in the position `cell` had among their inputs
    void removeCell(const std::shared_ptr<Cell>& cell, bool reconnect = true)
    {
        editable();
        const std::string name = cell->getName();
        if (!mCells.count(name)) throw std::runtime_error("DeepNet::removeCell(): layer " + name + " does not exist");
        std::vector<std::string> parents;
        for (const auto& link : mParentLayers)
            if (link.first == name) parents.push_back(link.second);
        std::vector<std::pair<std::string, std::string> > links;
        for (const auto& link : mParentLayers) {
            if (link.first == name) continue;
            if (link.second != name) { links.push_back(link); continue; }
            if (reconnect)
                for (const auto& p : parents) links.emplace_back(link.first, p);
        }
        mParentLayers.swap(links);
        mCells.erase(name);
        for (std::size_t l = 1; l < mLayers.size();) {
            auto& layer = mLayers[l];
            layer.erase(std::remove(layer.begin(), layer.end(), name), layer.end());
            if (layer.empty()) mLayers.erase(mLayers.begin() + l);
            else ++l;
        }
        inferShapes();
    }

    std::vector<std::shared_ptr<Cell> > getChildCells(const std::string& name) const
    {
        std::vector<std::shared_ptr<Cell> > out;
        for (const auto& link : mParentLayers)
            if (link.second == name) out.push_back(mCells.at(link.first));
        return out;
    }
    // a null pointer stands for the environment, as in the reference
    std::vector<std::shared_ptr<Cell> > getParentCells(const std::string& name) const
    {
        std::vector<std::shared_ptr<Cell> > out;
        for (const auto& link : mParentLayers)
            if (link.first == name) out.push_back(link.second == "env" ? std::shared_ptr<Cell>() : mCells.at(link.second));
        return out;
    }
    // DeepNetExport::isCellOutputUnsigned / isCellInputsUnsigned (src/Export/DeepNetExport.cpp:298-388) on this
    // graph: a Rectifier's output range starts at 0; pooling and ScalingCells (non-negative factors) hand their
    // parents' range on (src/Cell/PoolCell.cpp:242-244, src/Cell/ScalingCell.cpp:68-104); everything else is signed.
    bool isCellOutputUnsigned(const Cell& cell) const
    {
        if (!DeepNetExport::mUnsignedData()) return false;
        if (cell.mForcedSign >= 0) return cell.mForcedSign != 0;
        const bool passThrough = dynamic_cast<const PoolCell*>(&cell) || dynamic_cast<const ScalingCell*>(&cell);
        if (!passThrough) return cell.getActivation() && cell.getActivation()->kind() == N2D2B_ACT_RECTIFIER;
        if (auto* sc = dynamic_cast<const ScalingCell*>(&cell)) {
            const Scaling& s = sc->getScaling();
            for (Float_T v : s.getFloatingPointScalingPerOutput()) if (v < 0.0f) return false;
            for (std::int32_t v : s.getFixedPointScalingPerOutput()) if (v < 0) return false;
        }
        bool any = false;
        for (const auto& link : mParentLayers) {
            if (link.first != cell.getName()) continue;
            any = true;
            if (!(link.second == "env" ? DeepNetExport::mEnvDataUnsigned() : isCellOutputUnsigned(*mCells.at(link.second)))) return false;
        }
        return any;
    }
    bool isCellInputsUnsigned(const Cell& cell) const
    {
        if (!DeepNetExport::mUnsignedData()) return false;
        bool first = true, uns = false;
        for (const auto& link : mParentLayers) {
            if (link.first != cell.getName()) continue;
            const bool u = link.second == "env" ? DeepNetExport::mEnvDataUnsigned() : isCellOutputUnsigned(*mCells.at(link.second));
            if (first) { uns = u; first = false; }
            else if (u != uns)
                throw std::runtime_error("Unsupported: cell " + cell.getName() + " mixes signed and unsigned inputs. "
                                         "Try setting DeepNetExport::mUnsignedData to false");
        }
        return uns;
    }
    // a name nobody has yet: baseName, or baseName_1, baseName_2 ... (DeepNet::generateNewCellName)
    std::string generateNewCellName(const std::string& baseName) const
    {
        if (!mCells.count(baseName)) return baseName;
        for (std::size_t i = 1;; ++i) {
            const std::string n = baseName + "_" + std::to_string(i);
            if (!mCells.count(n)) return n;
        }
    }
    bool hasCell(const std::string& name) const { return mCells.count(name) != 0; }
    const std::map<std::string, std::shared_ptr<Cell> >& getCells() const { return mCells; }

    template <class T> std::shared_ptr<T> getCell(const std::string& name) const
    {
        auto it = mCells.find(name);
        if (it == mCells.end()) throw std::runtime_error("DeepNet::getCell(): layer " + name + " does not exist");
        auto p = std::dynamic_pointer_cast<T>(it->second);
        if (!p) throw std::runtime_error("DeepNet::getCell(): wrong type for layer " + name);
        return p;
    }
    const std::vector<std::vector<std::string> >& getLayers() const { return mLayers; }

    // Cell::initialize() of every cell: hands the graph to the device library in layer order, allocates
    // activations for up to maxBatch stimuli.  The graph is frozen afterwards.
    void initialize(unsigned int maxBatch, bool keepAllOutputs = false)
    {
        editable();
        // device resources appear here, as in the reference (Cell::initialize()); without a usable GPU this throws
        check(n2d2b_net_create(mDevice, &mNet));
        int id = 0;
        check(n2d2b_net_set_input(mNet, (int)mStimuli.c, (int)mStimuli.h, (int)mStimuli.w,
                                  DeepNetExport::mEnvDataUnsigned() ? 1 : 0, &id));
        for (std::size_t l = 1; l < mLayers.size(); ++l)
            for (const std::string& name : mLayers[l]) {
                lower(mCells.at(name));
                mLast = mCells.at(name);
            }
        if (!mLast) throw std::runtime_error("DeepNet::initialize(): the network has no cells");
        check(n2d2b_net_finalize(mNet, (int)maxBatch, keepAllOutputs ? (N2D2B_KEEP_ALL_OUTPUTS | N2D2B_NO_FUSION) : 0u));
        mInitialized = true;
    }

    // DeepNet::test on a batch of stimuli (8-bit, [batch][height][width][channels]); returns the last
    // cell's outputs as integers, [batch][outputs].
    // Target top-N of the last test() call (Target::process / TargetScore with the reference's getEstimatedLabels
    // kernel, src/Target/Target_CUDA_kernels.cu:24-104): labels (and scores) [batch][topN][height][width]; equal
    // scores come in the order the reference's sort leaves them, topN = 1 takes the first maximum.
    std::vector<int> getEstimatedLabels(unsigned int batch, unsigned int topN = 1, std::vector<int>* scores = nullptr)
    {
        if (!mInitialized) throw std::runtime_error("DeepNet::getEstimatedLabels(): initialize() and test() first");
        n2d2b_tensor_info info;
        check(n2d2b_net_tensor_info(mNet, mLast->mTensorId, &info));
        const std::size_t n = (std::size_t)batch * topN * info.height * info.width;
        std::vector<int> labels(n);
        if (scores) scores->resize(n);
        check(n2d2b_net_estimated_labels_topn_host(mNet, (int)batch, (int)topN, labels.data(), scores ? scores->data() : nullptr));
        return labels;
    }

    std::vector<int> test(const std::vector<std::uint8_t>& stimuli, unsigned int batch)
    {
        if (!mInitialized) throw std::runtime_error("DeepNet::test(): initialize() first");
        n2d2b_tensor_info info;
        check(n2d2b_net_tensor_info(mNet, mLast->mTensorId, &info));
        const std::size_t n = (std::size_t)info.channels * info.height * info.width * batch;
        std::vector<int> out(n);
        if (info.dtype == N2D2B_I32) {
            check(n2d2b_net_forward_host(mNet, stimuli.data(), (int)batch, out.data(), nullptr));
        } else {
            std::vector<std::uint8_t> raw(n);
            check(n2d2b_net_forward_host(mNet, stimuli.data(), (int)batch, raw.data(), nullptr));
            for (std::size_t i = 0; i < n; ++i) out[i] = info.is_unsigned ? (int)raw[i] : (int)(std::int8_t)raw[i];
        }
        return out;
    }

    // Outputs of one cell after test() (needs initialize(..., keepAllOutputs = true)), NHWC.
    std::vector<int> getOutputs(const std::string& name, unsigned int batch)
    {
        const auto cell = getCell<Cell>(name);
        n2d2b_tensor_info info;
        check(n2d2b_net_tensor_info(mNet, cell->mTensorId, &info));
        const std::size_t n = (std::size_t)info.channels * info.height * info.width * batch;
        std::vector<int> out(n);
        if (info.dtype == N2D2B_I32) {
            check(n2d2b_net_read_tensor(mNet, cell->mTensorId, (int)batch, out.data(), n * 4));
        } else {
            std::vector<std::uint8_t> raw(n);
            check(n2d2b_net_read_tensor(mNet, cell->mTensorId, (int)batch, raw.data(), n));
            for (std::size_t i = 0; i < n; ++i) out[i] = info.is_unsigned ? (int)raw[i] : (int)(std::int8_t)raw[i];
        }
        return out;
    }

private:
    struct Shape { unsigned int c, h, w; };
    static void check(int rc)
    {
        if (rc < 0) throw std::runtime_error(n2d2b_last_error());
    }
    void editable() const
    {
        if (mInitialized) throw std::runtime_error("DeepNet: the graph cannot change after initialize()");
    }
    void insertNew(const std::shared_ptr<Cell>& cell)
    {
        if (mCells.count(cell->getName())) throw std::runtime_error("DeepNet: cell " + cell->getName() + " already exists");
        mCells[cell->getName()] = cell;
    }
    std::size_t layerOf(const std::string& name) const
    {
        for (std::size_t l = 0; l < mLayers.size(); ++l)
            if (std::find(mLayers[l].begin(), mLayers[l].end(), name) != mLayers[l].end()) return l;
        throw std::runtime_error("The cell '" + name + "' was not found in the graph.");
    }
    Shape shapeOf(const std::string& name) const
    {
        if (name == "env") return mStimuli;
        const auto& c = mCells.at(name);
        return Shape{c->mNbOutputs, c->mOutputsHeight, c->mOutputsWidth};
    }
    // Output dimensions of every cell from its parents' (ConvCell_Frame_Kernels.cpp:37-45, PoolCell.cpp:233-239),
    // so that getOutputsWidth() / getNbChannels() answer before initialize() as they do in the reference.
    void inferShapes()
    {
        for (std::size_t l = 1; l < mLayers.size(); ++l)
            for (const std::string& name : mLayers[l]) {
                Cell& cell = *mCells.at(name);
                Shape in{0, 0, 0};
                bool first = true;
                for (const auto& link : mParentLayers) {
                    if (link.first != name) continue;
                    if (first) in = shapeOf(link.second);
                    first = false;
                }
                if (first) continue;   // not wired yet
                cell.mNbChannels = in.c;
                cell.mChannelsHeight = in.h;
                cell.mChannelsWidth = in.w;
                if (auto* conv = dynamic_cast<ConvCell*>(&cell)) {
                    auto dim = [](int n, int k, int s, int p0, int p1, int d) { return (unsigned)((n + p0 + p1 - d * (k - 1) - 1 + s) / (double)s); };
                    cell.mOutputsWidth = dim((int)in.w, (int)conv->mKernelDims[0], (int)conv->mStrideDims[0], conv->mPaddingDims[0], conv->mPaddingDims[2], (int)conv->mDilationDims[0]);
                    cell.mOutputsHeight = dim((int)in.h, (int)conv->mKernelDims[1], (int)conv->mStrideDims[1], conv->mPaddingDims[1], conv->mPaddingDims[3], (int)conv->mDilationDims[1]);
                } else if (auto* pool = dynamic_cast<PoolCell*>(&cell)) {
                    auto dim = [](int n, int k, int s, int p) { return (unsigned)((n + 2 * p - k + s) / (double)s); };
                    cell.mOutputsWidth = dim((int)in.w, (int)pool->mPoolDims[0], (int)pool->mStrideDims[0], (int)pool->mPaddingDims[0]);
                    cell.mOutputsHeight = dim((int)in.h, (int)pool->mPoolDims[1], (int)pool->mStrideDims[1], (int)pool->mPaddingDims[1]);
                } else if (dynamic_cast<FcCell*>(&cell)) {
                    cell.mOutputsWidth = cell.mOutputsHeight = 1;
                } else {
                    cell.mOutputsWidth = in.w;
                    cell.mOutputsHeight = in.h;
                }
            }
    }
    void lower(const std::shared_ptr<Cell>& cell)
    {
        std::vector<int> ins;
        Shape in{0, 0, 0};
        for (const auto& link : mParentLayers) {
            if (link.first != cell->getName()) continue;
            if (link.second != "env" && mCells.at(link.second)->mTensorId < 0)
                throw std::runtime_error("DeepNet::initialize(): cell " + cell->getName() + " runs before its parent " + link.second);
            if (ins.empty()) in = shapeOf(link.second);
            ins.push_back(link.second == "env" ? 0 : mCells.at(link.second)->mTensorId);
        }
        if (ins.empty()) throw std::runtime_error("DeepNet::initialize(): cell " + cell->getName() + " has no input");
        n2d2b_quant q;
        cell->describeQuant(q);
        q.out_unsigned = isCellOutputUnsigned(*cell) ? 1 : 0;
        int id = -1;
        if (auto* conv = dynamic_cast<ConvCell*>(cell.get())) {
            n2d2b_conv_desc d = n2d2b_conv_desc();
            d.input = ins[0];
            d.nb_outputs = (int)conv->getNbOutputs();
            d.kernel_w = (int)conv->mKernelDims[0]; d.kernel_h = (int)conv->mKernelDims[1];
            d.stride_x = (int)conv->mStrideDims[0]; d.stride_y = (int)conv->mStrideDims[1];
            d.pad_left = conv->mPaddingDims[0]; d.pad_top = conv->mPaddingDims[1];
            d.pad_right = conv->mPaddingDims[2]; d.pad_bottom = conv->mPaddingDims[3];
            d.dilation_x = (int)conv->mDilationDims[0]; d.dilation_y = (int)conv->mDilationDims[1];
            d.groups = (int)conv->mGroups;
            d.weight_bits = 8;
            // OIHW (reference memory order) -> OHWI (kernel order)
            const std::size_t cg = in.c / conv->mGroups, kh = d.kernel_h, kw = d.kernel_w, O = d.nb_outputs;
            if (conv->mWeights.size() != O * cg * kh * kw) throw std::runtime_error("ConvCell " + cell->getName() + ": wrong number of weights");
            if (!conv->mMapping.empty() && (conv->mGroups != 1 || conv->mMapping.size() != O * cg))
                throw std::runtime_error("ConvCell " + cell->getName() + ": a connection map needs nbOutputs x nbChannels entries and no groups");
            std::vector<std::int8_t> ohwi(conv->mWeights.size());
            for (std::size_t o = 0; o < O; ++o)
                for (std::size_t c = 0; c < cg; ++c) {
                    const bool connected = conv->mMapping.empty() || conv->mMapping[o * cg + c];
                    for (std::size_t y = 0; y < kh; ++y)
                        for (std::size_t x = 0; x < kw; ++x)
                            ohwi[((o * kh + y) * kw + x) * cg + c] = connected ? conv->mWeights[((o * cg + c) * kh + y) * kw + x] : 0;
                }
            check(n2d2b_net_add_conv(mNet, &d, ohwi.data(), conv->mBiases.empty() ? nullptr : conv->mBiases.data(), &q, &id));
        } else if (auto* fc = dynamic_cast<FcCell*>(cell.get())) {
            const std::size_t K = (std::size_t)in.c * in.h * in.w, O = fc->getNbOutputs();
            if (fc->mWeights.size() != O * K) throw std::runtime_error("FcCell " + cell->getName() + ": wrong number of weights");
            // the reference flattens the input as (channel, y, x); the device tensor is (y, x, channel)
            std::vector<std::int8_t> w(fc->mWeights.size());
            for (std::size_t o = 0; o < O; ++o)
                for (std::size_t c = 0; c < in.c; ++c)
                    for (std::size_t y = 0; y < in.h; ++y)
                        for (std::size_t x = 0; x < in.w; ++x)
                            w[o * K + (y * in.w + x) * in.c + c] = fc->mWeights[o * K + (c * in.h + y) * in.w + x];
            check(n2d2b_net_add_fc(mNet, ins[0], (int)O, 8, w.data(), fc->mBiases.empty() ? nullptr : fc->mBiases.data(), &q, &id));
        } else if (auto* pool = dynamic_cast<PoolCell*>(cell.get())) {
            n2d2b_pool_desc d = n2d2b_pool_desc();
            d.input = ins[0];
            d.pooling = pool->mPooling == PoolCell::Max ? N2D2B_POOL_MAX : N2D2B_POOL_AVERAGE;
            d.pool_w = (int)pool->mPoolDims[0]; d.pool_h = (int)pool->mPoolDims[1];
            d.stride_x = (int)pool->mStrideDims[0]; d.stride_y = (int)pool->mStrideDims[1];
            d.pad_x = (int)pool->mPaddingDims[0]; d.pad_y = (int)pool->mPaddingDims[1];
            check(n2d2b_net_add_pool(mNet, &d, &id));
        } else if (dynamic_cast<ElemWiseCell*>(cell.get())) {
            check(n2d2b_net_add_elemwise_sum(mNet, ins.data(), (int)ins.size(), &q, &id));
        } else if (dynamic_cast<ScalingCell*>(cell.get())) {
            check(n2d2b_net_add_scaling(mNet, ins[0], &q, &id));
        } else {
            throw std::runtime_error("DeepNet::initialize(): cell type " + std::string(cell->getType()) + " is not on the quantized path");
        }
        n2d2b_tensor_info info;
        check(n2d2b_net_tensor_info(mNet, id, &info));
        if ((unsigned)info.width != cell->mOutputsWidth || (unsigned)info.height != cell->mOutputsHeight)
            throw std::runtime_error("DeepNet::initialize(): output dimensions of " + cell->getName() + " disagree with the device library");
        cell->mTensorId = id;
    }

    n2d2b_net* mNet = nullptr;
    int mDevice;
    Shape mStimuli;
    bool mInitialized = false;
    std::map<std::string, std::shared_ptr<Cell> > mCells;
    std::vector<std::pair<std::string, std::string> > mParentLayers;   // (cell, parent) in input order; "env" = stimuli
    std::vector<std::vector<std::string> > mLayers;
    std::shared_ptr<Cell> mLast;
};

}  // namespace N2D2
