// Declaration-only stand-in for the few OpenCV names the reference's tensor container mentions.
// None of these functions is ever called by the oracle shim; they exist so the sources compile.
#pragma once
#include <vector>
#include <cstddef>
#define CV_8U 0
#define CV_8S 1
#define CV_16U 2
#define CV_16S 3
#define CV_32S 4
#define CV_32F 5
#define CV_64F 6
#define CV_MAKETYPE(depth, cn) ((depth) + (((cn)-1) << 3))
#define CV_8UC1 CV_MAKETYPE(CV_8U, 1)
#define CV_8SC1 CV_MAKETYPE(CV_8S, 1)
#define CV_16UC1 CV_MAKETYPE(CV_16U, 1)
#define CV_16SC1 CV_MAKETYPE(CV_16S, 1)
#define CV_32SC1 CV_MAKETYPE(CV_32S, 1)
#define CV_32FC1 CV_MAKETYPE(CV_32F, 1)
#define CV_64FC1 CV_MAKETYPE(CV_64F, 1)
namespace cv {
struct Point { int x, y; };
struct Rect {
    Rect();
    Rect(int x, int y, int width, int height);
    Point tl() const;
    Point br() const;
    int x, y, width, height;
};
struct Scalar {
    Scalar();
    Scalar(double v0, double v1 = 0, double v2 = 0, double v3 = 0);
    double val[4];
};
class Mat {
public:
    Mat();
    Mat operator()(const Rect& roi) const;
    Mat(int rows, int cols, int type);
    Mat(int rows, int cols, int type, void* data, std::size_t step = 0);
    Mat(const Mat&);
    ~Mat();
    Mat& operator=(const Mat&);
    Mat clone() const;
    int channels() const;
    int depth() const;
    int type() const;
    bool isContinuous() const;
    bool empty() const;
    template <class T> T* ptr(int i = 0);
    template <class T> const T* ptr(int i = 0) const;
    template <class T> T& at(int i, int j);
    template <class T> const T& at(int i, int j) const;
    int rows, cols;
    unsigned char* data;
    const unsigned char* datastart;
    const unsigned char* dataend;
};
void split(const Mat& m, std::vector<Mat>& mv);
void merge(const std::vector<Mat>& mv, Mat& dst);
}
