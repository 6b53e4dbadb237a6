// Builders of the layers' inputs on the GPU: the stereo matching cost volume and gradient cues
// (MPLayers/aux/aux.cpp:6-158), the pairwise label-context tables (aux.cpp:160-214) and the
// per-direction edge weights from an image or edge map (utils/edge_weights.py:45-111,
// MPLayers/extra_exp_edge_weights.py:64-128).  All of them are one pass over their output, which
// is written in the layout the message-passing kernels read ([H,W,L] costs, [D,B,1,H,W] weights),
// so nothing is permuted afterwards.  Integer arithmetic is reproduced exactly.
#include "mp_common.cuh"

namespace mpl {

namespace {

constexpr int kDsiTX = 64;        // pixels of one row per block
constexpr int kDsiThreads = 512;  // 8 per pixel

// Per pixel and pair of colours (two 16-bit halves per word): c, c + 256, lo + 256 and hi, where
// [lo, hi] spans the pixel's value and its two integer half-sample neighbours (c + neighbour) / 2
// (aux.cpp:57-66); lo = hi = c when the plain absolute difference is asked for.  With these, the
// one-sided distances of the Birchfield-Tomasi cost,
//   max(0, c1 - hi2, lo2 - c1) + 256 = max(256, (c1 + 256) - hi2, (lo2 + 256) - c1),
// are two 32-bit subtractions (every half stays in [1, 511]: no borrow crosses the halves) and one
// packed 3-input maximum for two colours at once.
struct __align__(16) BtWord {
  uint32_t c, cb, lob, hi;
};

__device__ __forceinline__ void bt_half(const uint8_t* row, int x, int W, int nB, int b, int birchfield,
                                        uint32_t& c, uint32_t& lo, uint32_t& hi) {
  const int v = row[x * nB + b];
  int l = v, r = v;
  if (birchfield) {
    l = x == 0 ? v : (v + row[(x - 1) * nB + b]) / 2;
    r = x == W - 1 ? v : (v + row[(x + 1) * nB + b]) / 2;
  }
  c = v;
  lo = min(v, min(l, r));
  hi = max(v, max(l, r));
}

// Words of pixel x for colours (b0, b0 + 1); a colour beyond nc counts as 0 in both images.
__device__ __forceinline__ BtWord bt_pack(const uint8_t* row, int x, int W, int nB, int nc, int b0,
                                          int birchfield) {
  uint32_t c[2] = {0, 0}, lo[2] = {0, 0}, hi[2] = {0, 0};
  for (int k = 0; k < 2; ++k)
    if (b0 + k < nc) bt_half(row, x, W, nB, b0 + k, birchfield, c[k], lo[k], hi[k]);
  BtWord w;
  w.c = c[0] | (c[1] << 16);
  w.cb = w.c + 0x01000100u;
  w.lob = (lo[0] + 256u) | ((lo[1] + 256u) << 16);
  w.hi = hi[0] | (hi[1] << 16);
  return w;
}

// min(di1, di2) + 256 of two colours, one per 16-bit half.
__device__ __forceinline__ uint32_t bt_pair(const BtWord& l, const BtWord& r) {
  const uint32_t k = 0x01000100u;
  const uint32_t d1 = __vimax3_u16x2(l.cb - r.hi, r.lob - l.c, k);
  const uint32_t d2 = __vimax3_u16x2(r.cb - l.hi, l.lob - r.c, k);
  return __vimin3_u16x2(d1, d2, d2);
}

// Third colour: the same left pixel against TWO neighbouring right pixels at once (one per half).
__device__ __forceinline__ BtWord bt_pack_third(const uint8_t* row, int x, int W, int nB, int nc, int birchfield) {
  uint32_t c[2] = {0, 0}, lo[2] = {0, 0}, hi[2] = {0, 0};
  if (nc > 2) {
    if (x >= 0) bt_half(row, x, W, nB, 2, birchfield, c[0], lo[0], hi[0]);
    if (x >= 1) bt_half(row, x - 1, W, nB, 2, birchfield, c[1], lo[1], hi[1]);
  }
  BtWord w;
  w.c = c[0] | (c[1] << 16);
  w.cb = w.c + 0x01000100u;
  w.lob = (lo[0] + 256u) | ((lo[1] + 256u) << 16);
  w.hi = hi[0] | (hi[1] << 16);
  return w;
}

// Sum over colours of one label's differences: the two halves of m01 and half `odd` of `third`,
// each biased by 256.  Not squared: two 2-way dot products with ones do the unpacking and the adds.
template <bool SQUARED>
__device__ __forceinline__ int dsi_sum(uint32_t m01, uint32_t third, int odd, int maxsum) {
  int sum;
  if (SQUARED) {
    const int d0 = (int)(m01 & 0xffffu) - 256, d1 = (int)(m01 >> 16) - 256;
    const int d2 = (int)(odd ? (third >> 16) : (third & 0xffffu)) - 256;
    sum = d0 * d0 + d1 * d1 + d2 * d2;
  } else {
    sum = (int)__dp2a_lo(m01, 0x0101u, __dp2a_lo(third, odd ? 0x0100u : 0x0001u, (unsigned)-768));
  }
  return min(sum, maxsum);
}

// Right pixels of a block live in shared memory de-interleaved by (index mod 4): entry j (pixel
// x0 - (L - 1) + j) sits at row j & 3, column j >> 2.  Plane 0: colours (0, 1) of the pixel; plane 1:
// colour 2 of the pixel (low half) and of its left neighbour (high half), so that one packed
// operation against the left pixel's colour 2 (duplicated in both halves) serves two labels.
constexpr int kDsiQ = (kDsiTX + 256 - 1 + 3) / 4 + 1;   // columns per row for up to 256 labels
__device__ __forceinline__ int dsi_slot(int j) { return (j & 3) * kDsiQ + (j >> 2); }

// One block: kDsiTX pixels of one row, all labels; its output tile is one contiguous run of
// kDsiTX * L floats.  VEC4 (L a multiple of 4): thread = (pixel, one of 8 lanes); a lane computes
// labels 4*lane .. 4*lane+3, then 32 further on, and stores them as one 16-byte word, so 8 lanes
// write 128 contiguous bytes.  Consecutive lanes read right pixels 4 apart, which the
// de-interleaved layout turns into consecutive 16-byte shared-memory words; the left pixel's words
// stay in registers and the four read pointers only step by a constant.
template <bool VEC4, bool THREE, bool SQUARED>
__global__ void __launch_bounds__(kDsiThreads)
stereo_data_cost_kernel(const uint8_t* __restrict__ left, const uint8_t* __restrict__ right, int H, int W,
                        int nB, int L, int birchfield, int maxsum, int badcost, float* __restrict__ out) {
  __shared__ BtWord s1[kDsiTX * 2];        // left pixels: colours (0,1), colour 2
  __shared__ BtWord s2[2 * 4 * kDsiQ];     // right pixels: plane of colours (0,1), plane of colour 2
  const int nc = min(3, nB);
  const int y = blockIdx.y, x0 = blockIdx.x * kDsiTX;
  const int tx = min(kDsiTX, W - x0);
  const uint8_t* lrow = left + (long long)y * W * nB;
  const uint8_t* rrow = right + (long long)y * W * nB;
  for (int i = threadIdx.x; i < tx * 2; i += kDsiThreads) {
    BtWord w = bt_pack(lrow, x0 + (i >> 1), W, nB, nc, (i & 1) * 2, birchfield);
    if (i & 1) {   // colour 2 in both halves
      w.c *= 0x00010001u, w.cb = w.c + 0x01000100u, w.lob = (w.lob & 0xffffu) * 0x00010001u, w.hi *= 0x00010001u;
    }
    s1[i] = w;
  }
  const int n2 = tx + L - 1;
  for (int i = threadIdx.x; i < n2 * 2; i += kDsiThreads) {
    const int j = i >> 1, x = x0 - (L - 1) + j;
    if (x >= 0)
      s2[(i & 1) * 4 * kDsiQ + dsi_slot(j)] =
          (i & 1) ? bt_pack_third(rrow, x, W, nB, nc, birchfield) : bt_pack(rrow, x, W, nB, nc, 0, birchfield);
  }
  __syncthreads();
  float* tile = out + ((long long)y * W + x0) * L;
  if (VEC4) {
    const int px = threadIdx.x >> 3, l8 = threadIdx.x & 7;
    if (px >= tx) return;
    const BtWord l[2] = {s1[px * 2], s1[px * 2 + 1]};
    const int xl = x0 + px;                       // labels d <= xl have a right pixel
    const int j0 = px + L - 1 - 4 * l8;           // entry matched by label 4 * l8
    const BtWord* r[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) r[k] = s2 + dsi_slot(j0 - k);
    float* o = tile + px * L + 4 * l8;
    for (int d0 = 4 * l8; d0 < L; d0 += 32) {
      float v[4];
      uint32_t third[2] = {0x01000100u, 0x01000100u};
      if (THREE) {   // labels (d0, d0+1) and (d0+2, d0+3): right pixels (j, j-1) and (j-2, j-3)
        third[0] = bt_pair(l[1], r[0][4 * kDsiQ]);
        third[1] = bt_pair(l[1], r[2][4 * kDsiQ]);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = dsi_sum<SQUARED>(bt_pair(l[0], r[k][0]), third[k >> 1], k & 1, maxsum);
        v[k] = (float)(d0 + k <= xl ? c : badcost);
        r[k] -= 8;                                // 32 labels further: 8 columns back
      }
      *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
      o += 32;
    }
  } else {
    const int n = tx * L;
    for (int i = threadIdx.x; i < n; i += kDsiThreads) {
      const int px = i / L, d = i - px * L;
      const BtWord l[2] = {s1[px * 2], s1[px * 2 + 1]};
      const BtWord* r = s2 + dsi_slot(px - d + L - 1);
      const uint32_t third = THREE ? bt_pair(l[1], r[4 * kDsiQ]) : 0x01000100u;
      const int c = dsi_sum<SQUARED>(bt_pair(l[0], r[0]), third, 0, maxsum);
      tile[i] = (float)(x0 + px - d >= 0 ? c : badcost);
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
  using Kern = void (*)(const uint8_t*, const uint8_t*, int, int, int, int, int, int, int, float*);
  static const Kern table[8] = {
      stereo_data_cost_kernel<false, false, false>, stereo_data_cost_kernel<false, false, true>,
      stereo_data_cost_kernel<false, true, false>,  stereo_data_cost_kernel<false, true, true>,
      stereo_data_cost_kernel<true, false, false>,  stereo_data_cost_kernel<true, false, true>,
      stereo_data_cost_kernel<true, true, false>,   stereo_data_cost_kernel<true, true, true>};
  const Kern kern = table[(L % 4 == 0 ? 4 : 0) + (nc == 3 ? 2 : 0) + (squared ? 1 : 0)];
  kern<<<grid, kDsiThreads, 0, st>>>(left, right, H, W, nB, L, birchfield, maxsum, bad, out);
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
