// Minimal stand-in for the one image container the reference's term builders are instantiated on
// (test infrastructure; lets MPLayers/aux/aux.cpp compile unmodified where OpenCV's C++ headers are
// not installed).  Only what aux.cpp touches: rows, cols, channels(), ptr(row, col) on an
// interleaved 8-bit image.  No arithmetic lives here.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdlib>
namespace cv {
class Mat {
 public:
  int rows, cols;
  Mat() : rows(0), cols(0), data_(nullptr), nch_(0), own_(false) {}
  Mat(int r, int c, int type) : rows(r), cols(c), nch_(type), own_(true) { data_ = new unsigned char[(long)r * c * type]; }
  Mat(int r, int c, int nch, unsigned char* borrowed) : rows(r), cols(c), data_(borrowed), nch_(nch), own_(false) {}
  Mat(const Mat& o) : rows(o.rows), cols(o.cols), data_(o.data_), nch_(o.nch_), own_(false) {}
  ~Mat() { if (own_) delete[] data_; }
  int channels() const { return nch_; }
  unsigned char* ptr(int y, int x) { return data_ + ((long)y * cols + x) * nch_; }
 private:
  Mat& operator=(const Mat&);
  unsigned char* data_;
  int nch_;
  bool own_;
};
}  // namespace cv
#define CV_8UC1 1
