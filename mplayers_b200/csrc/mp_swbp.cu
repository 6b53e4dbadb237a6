// Stand-alone soft-weighted message ops on a stack of L x L edge-value tables
// (MPLayers/TRWP_hard_soft/TRWP_swbp.cu:135-245; exported by TRWP.cpp:382-419 and exercised by
// pytorch/unittest_mp.py).  message [T, L(front), L(current)]:
//   soft[t,c] = sum_f softmax_f(-message[t,:,c])[f] * message[t,f,c]
//   n[t]      = argmin_c soft[t,c]  (highest index among equal minima)
//   norm[t,c] = soft[t,c] - soft[t,n[t]]
// and the backward of norm with respect to message.  One CTA per table, one thread per current
// label; the three passes over the front labels read a column that the CTA's other threads read
// beside it, so every load instruction is one contiguous row of the table.
#include "mp_common.cuh"

namespace mpl {

namespace {

struct ColumnStats {
  float lo, sum, soft;
};

__device__ __forceinline__ ColumnStats column_stats(const float* __restrict__ col, int L) {
  ColumnStats s;
  s.lo = INFINITY;
  for (int f = 0; f < L; ++f) s.lo = fminf(s.lo, col[f * L]);
  s.sum = 0.f;
  for (int f = 0; f < L; ++f) s.sum += expf(-(col[f * L] - s.lo));
  s.soft = 0.f;
  for (int f = 0; f < L; ++f) {
    const float m = col[f * L];
    s.soft += m * (expf(-(m - s.lo)) / s.sum);
  }
  return s;
}

__global__ void soft_weighted_message_kernel(const float* __restrict__ msg, int L, float* __restrict__ norm,
                                             uint8_t* __restrict__ min_ind) {
  __shared__ float best_v[8];
  __shared__ int best_i[8];
  const long long t = blockIdx.x;
  const int c = threadIdx.x;
  float soft = INFINITY;
  if (c < L) soft = column_stats(msg + t * L * L + c, L).soft;
  // argmin over c, highest index among equal values
  float v = soft;
  int idx = c < L ? c : -1;
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov < v || (ov == v && oi > idx)) { v = ov; idx = oi; }
  }
  if ((c & 31) == 0) { best_v[c >> 5] = v; best_i[c >> 5] = idx; }
  __syncthreads();
  v = best_v[0];
  idx = best_i[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
    if (best_v[w] < v || (best_v[w] == v && best_i[w] > idx)) { v = best_v[w]; idx = best_i[w]; }
  if (c < L) norm[t * L + c] = soft - v;
  if (c == 0) min_ind[t] = (uint8_t)idx;
}

__global__ void soft_weighted_message_back_kernel(const float* __restrict__ dnorm, const float* __restrict__ msg,
                                                  const uint8_t* __restrict__ min_ind, int L,
                                                  float* __restrict__ dmsg) {
  __shared__ float part[8];
  const long long t = blockIdx.x;
  const int c = threadIdx.x;
  float g = c < L ? dnorm[t * L + c] : 0.f;
  float total = g;
  for (int o = 16; o; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
  if ((c & 31) == 0) part[c >> 5] = total;
  __syncthreads();
  total = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += part[w];
  if (c >= L) return;
  if (c == min_ind[t]) g -= total;
  const float* col = msg + t * L * L + c;
  const ColumnStats s = column_stats(col, L);
  float* out = dmsg + t * L * L + c;
  for (int f = 0; f < L; ++f) {
    const float m = col[f * L];
    const float prob = expf(-(m - s.lo)) / s.sum;
    out[f * L] = g * prob * (1.f - m + s.soft);
  }
}

}  // namespace

cudaError_t launch_soft_weighted_message(const float* msg, long long n_tables, int L, float* norm,
                                         uint8_t* min_ind, cudaStream_t st) {
  const int threads = (L + 31) / 32 * 32;
  soft_weighted_message_kernel<<<(unsigned)n_tables, threads, 0, st>>>(msg, L, norm, min_ind);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_soft_weighted_message_back(const float* dnorm, const float* msg, const uint8_t* min_ind,
                                              long long n_tables, int L, float* dmsg, cudaStream_t st) {
  const int threads = (L + 31) / 32 * 32;
  soft_weighted_message_back_kernel<<<(unsigned)n_tables, threads, 0, st>>>(dnorm, msg, min_ind, L, dmsg);
  count_launch();
  return cudaGetLastError();
}

}  // namespace mpl
