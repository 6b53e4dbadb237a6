// Builders of the layers' inputs on the GPU: the stereo matching cost volume and gradient cues
// (MPLayers/aux/aux.cpp:6-158), the pairwise label-context tables (aux.cpp:160-214) and the
// per-direction edge weights from an image or edge map (utils/edge_weights.py:45-111,
// MPLayers/extra_exp_edge_weights.py:64-128).  All of them are one pass over their output, which
// is written in the layout the message-passing kernels read ([H,W,L] costs, [D,B,1,H,W] weights),
// so nothing is permuted afterwards.  Integer arithmetic is reproduced exactly.
#include "mp_common.cuh"

namespace mpl {

namespace {

constexpr int kDsiTX = 32;        // pixels of one row per block
constexpr int kDsiThreads = 256;

// c | min(c, left, right) << 8 | max(...) << 16 of one channel of pixel x, the half-sample
// neighbours being (c + neighbour) / 2 in integers (aux.cpp:57-66).
__device__ __forceinline__ uint32_t bt_pack(const uint8_t* row, int x, int W, int nB, int b) {
  const int c = row[x * nB + b];
  const int l = x == 0 ? c : (c + row[(x - 1) * nB + b]) / 2;
  const int r = x == W - 1 ? c : (c + row[(x + 1) * nB + b]) / 2;
  const int lo = min(c, min(l, r)), hi = max(c, max(l, r));
  return (uint32_t)c | ((uint32_t)lo << 8) | ((uint32_t)hi << 16);
}

__device__ __forceinline__ int dsi_value(const uint32_t* s1, const uint32_t* s2, int nc, int birchfield,
                                         int squared, int maxsum) {
  int sum = 0;
#pragma unroll 3
  for (int b = 0; b < nc; ++b) {
    const uint32_t p1 = s1[b], p2 = s2[b];
    const int c1 = p1 & 255, c2 = p2 & 255;
    int diff;
    if (birchfield) {
      const int lo1 = (p1 >> 8) & 255, hi1 = (p1 >> 16) & 255, lo2 = (p2 >> 8) & 255, hi2 = (p2 >> 16) & 255;
      const int di1 = max(0, max(c1 - hi2, lo2 - c1));
      const int di2 = max(0, max(c2 - hi1, lo1 - c2));
      diff = min(di1, di2);
    } else {
      diff = abs(c1 - c2);
    }
    sum += squared ? diff * diff : diff;
  }
  return min(sum, maxsum);
}

// One block: kDsiTX pixels of one row, all labels.  The tile of the output is contiguous
// (kDsiTX * L floats), so consecutive threads write consecutive addresses.
template <bool VEC4>
__global__ void __launch_bounds__(kDsiThreads)
stereo_data_cost_kernel(const uint8_t* __restrict__ left, const uint8_t* __restrict__ right, int H, int W,
                        int nB, int L, int birchfield, int squared, int maxsum, int badcost,
                        float* __restrict__ out) {
  extern __shared__ uint32_t sm[];
  const int nc = min(3, nB);
  const int y = blockIdx.y, x0 = blockIdx.x * kDsiTX;
  const int tx = min(kDsiTX, W - x0);
  uint32_t* s1 = sm;                     // [kDsiTX][3]
  uint32_t* s2 = sm + kDsiTX * 3;        // [kDsiTX + L - 1][3], entry j <-> pixel x0 - (L - 1) + j
  const uint8_t* lrow = left + (long long)y * W * nB;
  const uint8_t* rrow = right + (long long)y * W * nB;
  for (int i = threadIdx.x; i < tx * nc; i += kDsiThreads) {
    const int px = i / nc, b = i - px * nc;
    s1[px * 3 + b] = bt_pack(lrow, x0 + px, W, nB, b);
  }
  const int n2 = tx + L - 1;
  for (int i = threadIdx.x; i < n2 * nc; i += kDsiThreads) {
    const int j = i / nc, b = i - j * nc;
    const int x = x0 - (L - 1) + j;
    if (x >= 0) s2[j * 3 + b] = bt_pack(rrow, x, W, nB, b);
  }
  __syncthreads();
  float* tile = out + ((long long)y * W + x0) * L;
  const int n = tx * L;
  if (VEC4) {
    for (int i = threadIdx.x * 4; i < n; i += kDsiThreads * 4) {
      const int px = i / L, d0 = i - px * L;
      float v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int d = d0 + k;
        v[k] = (x0 + px - d >= 0)
                   ? (float)dsi_value(s1 + px * 3, s2 + (px - d + L - 1) * 3, nc, birchfield, squared, maxsum)
                   : (float)badcost;
      }
      *reinterpret_cast<float4*>(tile + i) = make_float4(v[0], v[1], v[2], v[3]);
    }
  } else {
    for (int i = threadIdx.x; i < n; i += kDsiThreads) {
      const int px = i / L, d = i - px * L;
      tile[i] = (x0 + px - d >= 0)
                    ? (float)dsi_value(s1 + px * 3, s2 + (px - d + L - 1) * 3, nc, birchfield, squared, maxsum)
                    : (float)badcost;
    }
  }
}

// aux.cpp:93-158: squared colour difference to the right / lower neighbour (the pixel itself on the
// last column / row) against nColors * thresh^2.  compact != 0 writes what ComputerAllTerms hands
// to Python (auxPy.cpp:86-99): h_cue[h * (W-1) + w] for w < W-1, v_cue[w * (H-1) + h] for h < H-1.
__global__ void gradient_cues_kernel(const uint8_t* __restrict__ img, int H, int W, int nB, int thresh,
                                     float penalty, int compact, float* __restrict__ hcue,
                                     float* __restrict__ vcue) {
  const int n = H * W;   // below 2^31, checked by the caller
  const int nc = min(3, nB);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int y = i / W, x = i - y * W;
    const uint8_t* p = img + (long long)i * nB;
    const uint8_t* px = p + (x < W - 1 ? nB : 0);
    const uint8_t* py = p + (y < H - 1 ? (long long)W * nB : 0);
    int sx = 0, sy = 0;
    for (int b = 0; b < nc; ++b) {
      const int dx = (int)p[b] - (int)px[b], dy = (int)p[b] - (int)py[b];
      sx += dx * dx;
      sy += dy * dy;
    }
    const float hv = sx < thresh ? penalty : 1.f, vv = sy < thresh ? penalty : 1.f;
    if (!compact) {
      hcue[i] = hv;
      vcue[i] = vv;
    } else {
      if (x < W - 1) hcue[(long long)y * (W - 1) + x] = hv;
      if (y < H - 1) vcue[(long long)x * (H - 1) + y] = vv;
    }
  }
}

// aux.cpp:160-214.  method: 0 "L", 1 "Q", 2 "TL", 3 "TQ", 4 "Cauchy", 5 "Huber".
__global__ void smoothness_context_kernel(int L, int method, float smax, float* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= L * L) return;
  const int xj = i / L, xi = i - xj * L;
  const float value = (float)(xj - xi);
  float r;
  switch (method) {
    case 0: r = fabsf(value); break;
    case 1: r = value * value; break;
    case 2: r = fminf(fabsf(value), smax); break;
    case 3: r = fminf(value * value, smax * smax); break;
    case 4: {
      const float t = (float)((double)value / (double)smax);
      const float lg = logf(1.f + t * t);
      r = (float)(0.5 * (double)smax * (double)smax * (double)lg);
      break;
    }
    default:
      r = fabsf(value) <= smax ? value * value : 2.f * smax * fabsf(value) - smax * smax;
  }
  out[i] = r;
}

// Edge weights of all directions from an image or edge map (utils/edge_weights.py:45-111).
// For direction d the weight of the edge (front -> cur), front = cur - step_d, is stored at cur; a
// pixel whose front lies outside the image gets 0.  diff = |img[cur] - img[front]| per channel.
// Modes that keep the channels write [D,B,C,H,W]; modes that reduce over them write [D,B,1,H,W].
enum EdgeMode {
  kGtEdge = 0,           // diff = 1 where img[cur] == 255; weight = (diff == 0)
  kSuperpixelEdge = 1,   // weight = (sum_c diff == 0)                              (reduced)
  kCanny = 2,            // diff = 1 where img[cur] == 1; weight = 1 - diff
  kSobel = 3,            // weight = 1 - diff      (also "edge_net_sigmoid")
  kEdgeNet = 4,          // weight = exp(-diff)
  kKernelCueReal = 5,    // weight = exp(mean_c diff^2 / (-2 sigma^2))              (reduced)
  kKernelCueBinary = 6,  // the former, then (weight >= 0.8 * mean over the direction's patch)
  kThreshold = 7,        // weight = (mean_c diff^2 < threshold) * penalty          (reduced)
  kShifted = 8,          // weight = img[front]
  kCuePenalty = 9,       // weight = mean_c diff^2 < threshold ? penalty : 1        (reduced;
                         //   MPLayers/extra_exp_edge_weights.py:115-121)
};

__host__ __device__ inline bool edge_mode_reduces(int mode) {
  return mode == kSuperpixelEdge || mode == kKernelCueReal || mode == kKernelCueBinary ||
         mode == kThreshold || mode == kCuePenalty;
}

// Grid (pixel blocks, D, B); one thread per pixel, the channel loop is inside.  `sums` [D] (double) receives the sum of
// the weights of each direction's patch (kKernelCueBinary only).
__global__ void __launch_bounds__(256)
edge_weights_kernel(const float* __restrict__ img, int B, int C, int H, int W, int D, int mode,
                    float div, float threshold, float penalty, float* __restrict__ out,
                    double* __restrict__ sums) {
  const int hw = H * W;   // below 2^31, checked by the caller
  const bool reduced = edge_mode_reduces(mode);
  const int d = blockIdx.y, b = blockIdx.z;
  int hs, ws;
  dir_step(d, hs, ws);
  double local = 0.0;
  for (int pix = blockIdx.x * blockDim.x + threadIdx.x; pix < hw; pix += gridDim.x * blockDim.x) {
    const int h = pix / W, w = pix - h * W;
    const int fh = h - hs, fw = w - ws;
    const bool inside = fh >= 0 && fh < H && fw >= 0 && fw < W;
    const float* cur = img + (long long)b * C * hw + pix;
    const float* front = cur - (hs * W + ws);
    if (reduced) {
      float r = 0.f;
      if (inside) {
        float acc = 0.f;
        for (int c = 0; c < C; ++c) {
          const float df = fabsf(cur[(long long)c * hw] - front[(long long)c * hw]);
          acc += mode == kSuperpixelEdge ? df : df * df;
        }
        if (mode == kSuperpixelEdge) {
          r = acc == 0.f ? 1.f : 0.f;
        } else {
          const float mean = acc / (float)C;
          if (mode == kThreshold) r = mean < threshold ? penalty : 0.f;
          else if (mode == kCuePenalty) r = mean < threshold ? penalty : 1.f;
          else r = expf(mean / div);
        }
        local += (double)r;
      }
      out[((long long)d * B + b) * hw + pix] = r;
    } else {
      for (int c = 0; c < C; ++c) {
        float r = 0.f;
        if (inside) {
          const float a = cur[(long long)c * hw], f = front[(long long)c * hw];
          float df = fabsf(a - f);
          switch (mode) {
            case kGtEdge: if (a == 255.f) df = 1.f; r = df == 0.f ? 1.f : 0.f; break;
            case kCanny: if (a == 1.f) df = 1.f; r = 1.f - df; break;
            case kSobel: r = 1.f - df; break;
            case kEdgeNet: r = expf(-df); break;
            default: r = f;
          }
        }
        out[(((long long)d * B + b) * C + c) * hw + pix] = r;
      }
    }
  }
  if (mode == kKernelCueBinary) {
    __shared__ double part[8];
    for (int o = 16; o; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
      double t = 0.0;
      for (int k = 0; k < (int)(blockDim.x >> 5); ++k) t += part[k];
      atomicAdd(sums + d, t);
    }
  }
}

// Second pass of kKernelCueBinary: inside the patch, weight = (weight >= 0.8 * mean).
__global__ void __launch_bounds__(256)
edge_binarise_kernel(float* __restrict__ out, const double* __restrict__ sums, int B, int H, int W) {
  const int hw = H * W;
  const int d = blockIdx.y, b = blockIdx.z;
  int hs, ws;
  dir_step(d, hs, ws);
  const long long count = (long long)B * max(H - abs(hs), 0) * max(W - abs(ws), 0);
  if (count == 0) return;
  const float cut = 0.8f * (float)(sums[d] / (double)count);
  for (int pix = blockIdx.x * blockDim.x + threadIdx.x; pix < hw; pix += gridDim.x * blockDim.x) {
    const int h = pix / W, w = pix - h * W;
    const int fh = h - hs, fw = w - ws;
    if (fh >= 0 && fh < H && fw >= 0 && fw < W) {
      float* o = out + ((long long)d * B + b) * hw + pix;
      *o = *o >= cut ? 1.f : 0.f;
    }
  }
}

}  // namespace

cudaError_t launch_stereo_data_cost(const uint8_t* left, const uint8_t* right, int H, int W, int nB, int L,
                                    int birchfield, int squared, int trunc, float* out, cudaStream_t st) {
  const int nc = nB < 3 ? nB : 3;
  const int worst = nc * (squared ? 255 * 255 : 255);
  const int maxsum = squared ? trunc * trunc : nc * abs(trunc);
  const int bad = worst < maxsum ? worst : maxsum;
  dim3 grid((W + kDsiTX - 1) / kDsiTX, H);
  const size_t smem = (size_t)(kDsiTX * 3 + (kDsiTX + L - 1) * 3) * sizeof(uint32_t);
  if (L % 4 == 0)
    stereo_data_cost_kernel<true><<<grid, kDsiThreads, smem, st>>>(left, right, H, W, nB, L, birchfield, squared,
                                                                  maxsum, bad, out);
  else
    stereo_data_cost_kernel<false><<<grid, kDsiThreads, smem, st>>>(left, right, H, W, nB, L, birchfield,
                                                                   squared, maxsum, bad, out);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_gradient_cues(const uint8_t* img, int H, int W, int nB, int grad_thresh, int grad_penalty,
                                 int compact, float* hcue, float* vcue, cudaStream_t st) {
  const int nc = nB < 3 ? nB : 3;
  long long blocks = ((long long)H * W + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  gradient_cues_kernel<<<(int)blocks, 256, 0, st>>>(img, H, W, nB, grad_thresh * nc * grad_thresh,
                                                   (float)grad_penalty, compact, hcue, vcue);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_smoothness_context(int L, int method, float smax, float* out, cudaStream_t st) {
  smoothness_context_kernel<<<(L * L + 255) / 256, 256, 0, st>>>(L, method, smax, out);
  count_launch();
  return cudaGetLastError();
}

bool edge_weights_reduces(int mode) { return edge_mode_reduces(mode); }

cudaError_t launch_edge_weights(const float* img, int B, int C, int H, int W, int D, int mode, float sigma,
                                float threshold, float penalty, float* out, double* sums, cudaStream_t st) {
  long long bx = ((long long)H * W + 255) / 256;
  const long long cap = (148 * 16 + (long long)D * B - 1) / ((long long)D * B);
  if (bx > cap) bx = cap;
  if (bx < 1) bx = 1;
  dim3 grid((unsigned)bx, D, B);
  const float div = (float)(-2.0 * (double)sigma * (double)sigma);
  if (mode == kKernelCueBinary) {
    cudaError_t e = cudaMemsetAsync(sums, 0, sizeof(double) * D, st);
    if (e != cudaSuccess) return e;
  }
  edge_weights_kernel<<<grid, 256, 0, st>>>(img, B, C, H, W, D, mode, div, threshold, penalty, out, sums);
  count_launch();
  if (mode == kKernelCueBinary) {
    edge_binarise_kernel<<<grid, 256, 0, st>>>(out, sums, B, H, W);
    count_launch();
  }
  return cudaGetLastError();
}

}  // namespace mpl
