// C entry points around the reference's own CPU kernels, compiled from the reference tree where it
// lies (see Makefile).  TEST INFRASTRUCTURE: used to pin the CPU oracle against the real reference
// code and, optionally, as the timed CPU baseline.  No reference source is copied here; this file
// only builds Tensor<float> views of the caller's buffers and calls the reference functions.
#include <cstdint>
#include <cstring>
#include <utility>
#include <vector>

#include "Cell/Cell.hpp"
#include "Cell/ConvCell_Frame_Kernels.hpp"
#include "Cell/PoolCell_Frame_Kernels.hpp"
#include "Scaling_Kernels.hpp"
#include "containers/Tensor.hpp"

using N2D2::Tensor;

// Cell::getNbGroups / getNbGroupsHandMade (how a connection map is read as groups) come from the reference's own
// src/Cell/Cell.cpp; the link step keeps those two functions of that file and drops the rest (see the Makefile).

static Tensor<float> make_tensor(const float* src, std::vector<size_t> dims)
{
    Tensor<float> t(dims);
    if (src) std::memcpy(&t(0), src, t.size() * sizeof(float));
    return t;
}

extern "C" {

// The tensor container's explicit instantiations mention the spiking-network Node class in a
// dynamic_cast that this path never executes; its type_info object is the one unresolved *data*
// symbol of the library, so a placeholder of that name lets the library load.
const void* _ZTIN4N2D24NodeE[4] = {nullptr, nullptr, nullptr, nullptr};

// in: [B][C][H][W]; w: [O][wC][kH][kW]; maps: [O][C] or NULL; out: [B][O][oH][oW]
void refshim_conv(const float* in, int W, int H, int Cn, int B, const float* w, int kW, int kH, int wC, int O,
                  const uint8_t* maps, int strideX, int strideY, int padL, int padT, int padR, int padB, int dilX,
                  int dilY, const float* bias, int oW, int oH, float* out)
{
    Tensor<float> tin = make_tensor(in, {(size_t)W, (size_t)H, (size_t)Cn, (size_t)B});
    Tensor<float> tw = make_tensor(w, {(size_t)kW, (size_t)kH, (size_t)wC, (size_t)O});
    Tensor<float> tout = make_tensor(nullptr, {(size_t)oW, (size_t)oH, (size_t)O, (size_t)B});
    Tensor<bool> tmaps;
    if (maps) {
        tmaps.resize({(size_t)O, (size_t)Cn});
        for (int o = 0; o < O; ++o)
            for (int c = 0; c < Cn; ++c) tmaps(o, c) = maps[(size_t)o * Cn + c] != 0;
    }
    const N2D2::ConvCell_Frame_Kernels::Descriptor desc({1u, 1u}, {(unsigned)strideX, (unsigned)strideY},
                                                        {padL, padT, padR, padB}, {(unsigned)dilX, (unsigned)dilY});
    const float alpha = 1.0f, beta = 0.0f;
    N2D2::ConvCell_Frame_Kernels::forward<float>(&alpha, tin, tw, desc, &beta, tout, tmaps);
    if (bias) {
        Tensor<float> tb = make_tensor(bias, {1, 1, (size_t)O, 1});
        N2D2::ConvCell_Frame_Kernels::forwardBias<float>(&alpha, tb, &alpha, tout);
    }
    std::memcpy(out, &tout(0), tout.size() * sizeof(float));
}

void refshim_pool(const float* in, int W, int H, int Cn, int B, int pW, int pH, int strideX, int strideY, int padX,
                  int padY, int isMax, int isQuantized, int oW, int oH, float* out)
{
    Tensor<float> tin = make_tensor(in, {(size_t)W, (size_t)H, (size_t)Cn, (size_t)B});
    Tensor<float> tout = make_tensor(nullptr, {(size_t)oW, (size_t)oH, (size_t)Cn, (size_t)B});
    const unsigned pool[2] = {(unsigned)pW, (unsigned)pH};
    const unsigned stride[2] = {(unsigned)strideX, (unsigned)strideY};
    const unsigned pad[2] = {(unsigned)padX, (unsigned)padY};
    const N2D2::PoolCell_Frame_Kernels::Descriptor desc(2, pool, stride, pad);
    // one-to-one channel map, as Mapping.Size=1 / ChannelsPerGroup=1 gives
    Tensor<bool> tmaps({(size_t)Cn, (size_t)Cn}, false);
    for (int c = 0; c < Cn; ++c) tmaps(c, c) = true;
    const float alpha = 1.0f, beta = 0.0f;
    if (isMax) {
        Tensor<N2D2::PoolCell_Frame_Kernels::ArgMax> argMax({(size_t)oW, (size_t)oH, (size_t)Cn, (size_t)B});
        N2D2::PoolCell_Frame_Kernels::forwardMax<float>(&alpha, tin, desc, &beta, tout, argMax, false, tmaps);
    } else {
        N2D2::PoolCell_Frame_Kernels::forwardAverage<float>(&alpha, tin, desc, &beta, tout, isQuantized != 0, true,
                                                            tmaps);
    }
    std::memcpy(out, &tout(0), tout.size() * sizeof(float));
}

// mode: 1 float, 2 fixed, 4 single shift, 5 double shift. in/out: [B][C][H][W]
void refshim_scaling(const float* in, float* out, int B, int Cn, int H, int W, int mode, const float* fscale,
                     const int32_t* mult, int fracBits, const uint8_t* shift0, const uint8_t* shift1, int isClipped,
                     const float* clip, int nbBits, int isUnsigned)
{
    Tensor<float> tin = make_tensor(in, {(size_t)W, (size_t)H, (size_t)Cn, (size_t)B});
    Tensor<float> tout = make_tensor(nullptr, {(size_t)W, (size_t)H, (size_t)Cn, (size_t)B});
    std::vector<N2D2::Float_T> vclip(Cn, 0.0f);
    if (clip) vclip.assign(clip, clip + Cn);
    if (mode == 1) {
        std::vector<N2D2::Float_T> v(fscale, fscale + Cn);
        N2D2::floatingPointScaling_propagate<float>(tin, tout, B, Cn, H, W, isClipped != 0, vclip, v, nbBits,
                                                    isUnsigned != 0);
    } else if (mode == 2) {
        std::vector<std::int32_t> v(mult, mult + Cn);
        N2D2::fixedPointScaling_propagate<float>(tin, tout, B, Cn, H, W, isClipped != 0, vclip, v, fracBits, nbBits,
                                                 isUnsigned != 0);
    } else if (mode == 4) {
        std::vector<unsigned char> v(shift0, shift0 + Cn);
        N2D2::singleShiftScaling_propagate<float>(tin, tout, B, Cn, H, W, isClipped != 0, vclip, v, nbBits,
                                                  isUnsigned != 0);
    } else {
        std::vector<std::pair<unsigned char, unsigned char>> v(Cn), vc(Cn);
        for (int c = 0; c < Cn; ++c) v[c] = std::make_pair(shift0[c], shift1[c]);
        N2D2::doubleShiftScaling_propagate<float>(tin, tout, B, Cn, H, W, isClipped != 0, vc, v, nbBits,
                                                  isUnsigned != 0);
    }
    std::memcpy(out, &tout(0), tout.size() * sizeof(float));
}

}  // extern "C"
