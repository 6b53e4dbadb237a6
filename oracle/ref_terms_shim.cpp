// C entry points around the reference's own term builders (MPLayers/aux/aux.cpp, compiled
// unmodified with USE_OPENCV and USE_FLOAT as MPLayers/setup.py:39-56 does), with the image
// container replaced by the stand-in under mat_standin/.  Test infrastructure only.
#include "aux.h"

extern "C" {

void ref_compute_dsi(unsigned char* left, unsigned char* right, int height, int width, int channels,
                     int n_labels, int birchfield, int squared, int trunc, float* dsi) {
  cv::Mat im1(height, width, channels, left), im2(height, width, channels, right);
  computeDSI<cv::Mat>(im1, im2, dsi, n_labels, birchfield, squared, trunc);
}

void ref_compute_cues(unsigned char* img, int height, int width, int channels, int grad_thresh,
                      int grad_penalty, float* h_cue, float* v_cue) {
  cv::Mat im1(height, width, channels, img);
  computeCues<cv::Mat>(im1, h_cue, v_cue, grad_thresh, grad_penalty);
}

void ref_smoothness_context(int n_labels, const char* method, float smoothness_max, float* out) {
  float** rows = new float*[n_labels];
  for (int i = 0; i < n_labels; ++i) rows[i] = out + (long)i * n_labels;
  computeSmoothnessContext(n_labels, std::string(method), smoothness_max, rows);
  delete[] rows;
}

}  // extern "C"
