// Definitions behind stub/opencv2/core.hpp: the image-conversion members of the reference's tensor
// container reference these, nothing on the oracle path calls them, and they abort if reached.
#include <cstdlib>
#include "opencv2/core.hpp"

namespace cv {
static void unreachable() { std::abort(); }
Mat::Mat() : rows(0), cols(0), data(nullptr), datastart(nullptr), dataend(nullptr) {}
Mat::Mat(int, int, int) : rows(0), cols(0), data(nullptr), datastart(nullptr), dataend(nullptr) { unreachable(); }
Mat::Mat(int, int, int, void*, std::size_t) : rows(0), cols(0), data(nullptr), datastart(nullptr), dataend(nullptr) { unreachable(); }
Mat::Mat(const Mat&) : rows(0), cols(0), data(nullptr), datastart(nullptr), dataend(nullptr) {}
Mat::~Mat() {}
Mat& Mat::operator=(const Mat&) { return *this; }
Mat Mat::clone() const { unreachable(); return Mat(); }
int Mat::channels() const { unreachable(); return 0; }
int Mat::depth() const { unreachable(); return 0; }
int Mat::type() const { unreachable(); return 0; }
bool Mat::isContinuous() const { unreachable(); return false; }
bool Mat::empty() const { return true; }
template <class T> T* Mat::ptr(int) { unreachable(); return nullptr; }
template <class T> const T* Mat::ptr(int) const { unreachable(); return nullptr; }
template const char* Mat::ptr<char>(int) const;
template const unsigned char* Mat::ptr<unsigned char>(int) const;
template const short* Mat::ptr<short>(int) const;
template const unsigned short* Mat::ptr<unsigned short>(int) const;
template const int* Mat::ptr<int>(int) const;
template const float* Mat::ptr<float>(int) const;
template const double* Mat::ptr<double>(int) const;
void split(const Mat&, std::vector<Mat>&) { unreachable(); }
void merge(const std::vector<Mat>&, Mat&) { unreachable(); }
}
