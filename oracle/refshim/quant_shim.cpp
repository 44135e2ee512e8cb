// C entry points over two self-contained steps of the reference's DeepNetQuantization (src/DeepNetQuantization.cpp:
// approximateScalingWithFixedPoint :1043-1093, approximateScalingWithPowerOf2Divs :1095-1134), compiled from the
// reference tree where it lies; the rest of that file needs the whole library and is discarded at link time.
// TEST INFRASTRUCTURE ONLY: pins n2d2_b200/host/DeepNetQuantization.hpp.
#include <cstddef>
#include <cstdint>
#include <ostream>
#include <vector>
#include "DeepNet.hpp"
#define private public      // approximateScalingWithFixedPoint is a private static member
#define protected public
#include "DeepNetQuantization.hpp"
#undef private
#undef protected
using namespace N2D2;

// the two stream manipulators the fall-back warning of approximateScalingWithFixedPoint prints through
namespace N2D2 {
namespace Utils {
std::ostream& cwarning(std::ostream& s) { return s; }
std::ostream& cdef(std::ostream& s) { return s; }
}
}

extern "C" {

// mode: 2 = FIXED_MULT16, 3 = FIXED_MULT32 as in the reference's ScalingMode; returns the fractional bits (or -1 when
// the reference throws), writes the mode it ended with and the fixed-point scalings
int quantshim_fixed_point(int* mode, const float* scalings, std::size_t n, std::int32_t* out)
{
    try {
        ScalingMode m = (ScalingMode)*mode;
        const std::vector<Float_T> v(scalings, scalings + n);
        const auto r = N2D2::DeepNetQuantization::approximateScalingWithFixedPoint(m, v);
        *mode = (int)m;
        for (std::size_t i = 0; i < n; ++i) out[i] = r.second[i];
        return (int)r.first;
    } catch (...) {
        return -1;
    }
}

double quantshim_power_of_2_divs(float scaling, std::size_t nbDivisions, unsigned char* exponents)
{
    const auto r = N2D2::DeepNetQuantization::approximateScalingWithPowerOf2Divs(scaling, nbDivisions);
    for (std::size_t i = 0; i < nbDivisions; ++i) exponents[i] = r.first[i];
    return r.second;
}

}  // extern "C"
