// Forward kernels of the TRWP / ISGMR layers for sm_100a.
//
// One sweep = one direction over every chain of every image.  The reference runs it as two
// launches (UpdateUnaryKernel, MPLayers/TRWP/TRWP_forward.cu:60-80, then one of the chain kernels
// :82-376) with L block barriers and L dependent global loads per chain step; here the unary update
// is fused into the chain walk, inputs are staged through a cp.async ring in shared memory several
// pixels ahead, labels live in registers, and min / argmin use warp-wide redux + ballot.
//
//   fwd_warp_kernel : L <= 32, one warp per chain, lane = label, context row in registers.
//   fwd_cta_kernel  : L  > 32, one CTA per chain, thread = label;
//                     MODE 1 rank-1 context: windowed O(L*R) evaluation when the context is
//                            non-decreasing and saturates at offset R, else dense;
//                     MODE 2 rank-2 context, L <= 64: context row in registers;
//                     MODE 0 rank-2 context, L > 64: context read through L1.
//
// Arithmetic follows the reference order (see Appendix of the oracle header): UU = ((U + M_0 + ...
// + M_{D-1}) - M_d) * rho - M_inv, candidate = fma(E, ctx, fma(rho, r, UU)); ties -> highest index.
#include "mp_common.cuh"

namespace mpl {

namespace {

constexpr int kPF = 8;  // pixels staged ahead per chain (power of two)

struct ChainCtx {
  int dir, inv, img, h0, w0, len, pstep;
};

__device__ __forceinline__ bool decode_chain(const FwdParams& p, int g, ChainCtx& c) {
  if (g >= p.chain_off[p.ndirs]) return false;
  int di = 0;
  while (g >= p.chain_off[di + 1]) ++di;
  c.dir = p.dir0 + di;
  c.inv = c.dir ^ 1;
  const DirGeom geo = make_geom(c.dir, p.H, p.W);
  const int local = g - p.chain_off[di];
  c.img = local / geo.n_chains;
  chain_start(geo, p.H, p.W, local - c.img * geo.n_chains, c.h0, c.w0, c.len);
  c.pstep = geo.hs * p.W + geo.ws;
  return c.len >= 2;
}

// UU of one pixel from its ring slot (rows: 0 = U, 1+k = M_k), column `col`, row stride `rs`.
__device__ __forceinline__ float uu_from_ring(const float* slot, int rs, int col, int D, int dir,
                                              int inv, float rho) {
  float s = slot[col];
  for (int k = 0; k < D; ++k) s += slot[(1 + k) * rs + col];
  s -= slot[(1 + dir) * rs + col];
  return fmaf(s, rho, -slot[(1 + inv) * rs + col]);
}

__device__ __forceinline__ float min3f(float a, float b, float c) {
  float d;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));  // 3-input min (sm_100)
  return d;
}

// Minimum of N registers with 3-input min instructions: depth ceil(log3 N) instead of the
// reference's serial scan.
template <int N>
__device__ __forceinline__ float min_tree(const float (&v)[N]) {
  if constexpr (N == 1) {
    return v[0];
  } else if constexpr (N == 2) {
    return fminf(v[0], v[1]);
  } else if constexpr (N == 3) {
    return min3f(v[0], v[1], v[2]);
  } else {
    constexpr int M = (N + 2) / 3;
    float t[M];
#pragma unroll
    for (int i = 0; i < M; ++i) {
      if (3 * i + 2 < N) {
        t[i] = min3f(v[3 * i], v[3 * i + 1], v[3 * i + 2]);
      } else if (3 * i + 1 < N) {
        t[i] = fminf(v[3 * i], v[3 * i + 1]);
      } else {
        t[i] = v[3 * i];
      }
    }
    return min_tree<M>(t);
  }
}

__device__ __forceinline__ float eq_flag(float a, float b) {
  float d;
  asm("set.eq.f32.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));  // 1.0f if a == b else 0.0f
  return d;
}

__device__ __forceinline__ constexpr float pow2f(int k) {
  float r = 1.f;
  for (int i = 0; i < k; ++i) r *= 2.f;
  return r;
}

// Candidates val[f] = e*ctx(c,f) + h[f] for the label c of this thread, their minimum and -- when
// TRAIN -- the HIGHEST f attaining it (what the reference's high-to-low strict-< scan returns,
// MPLayers/TRWP/TRWP_forward.cu:126-152).
//
// Compare / select / min instructions run at half the rate of fused multiply-adds, so the index is
// not tracked with a compare-and-select chain.  The exact minimum is taken first (3-input min
// tree); then every candidate contributes (val[f] == min) * 2^f to a float accumulator with one
// set + one fma (groups of 24 labels per accumulator, exact in a 24-bit mantissa), and the wanted
// index is the exponent of the accumulator.
template <int LMAX, bool TRAIN>
__device__ __forceinline__ void minplus_regrow(const float* hb, const float (&cr)[LMAX], float e,
                                               float& best, int& bi) {
  constexpr int NV = (LMAX + 3) / 4;
  float hv[NV * 4];
#pragma unroll
  for (int q = 0; q < NV; ++q) {
    const float4 t = reinterpret_cast<const float4*>(hb)[q];
    hv[4 * q] = t.x;
    hv[4 * q + 1] = t.y;
    hv[4 * q + 2] = t.z;
    hv[4 * q + 3] = t.w;
  }
  float val[LMAX];
#pragma unroll
  for (int f = 0; f < LMAX; ++f) val[f] = fmaf(e, cr[f], hv[f]);
  best = min_tree<LMAX>(val);
  bi = 0;
  if (TRAIN) {
    constexpr int NA = (LMAX + 23) / 24;
    float acc[NA];
#pragma unroll
    for (int a = 0; a < NA; ++a) acc[a] = 0.f;
#pragma unroll
    for (int f = 0; f < LMAX; ++f) acc[f / 24] = fmaf(eq_flag(val[f], best), pow2f(f % 24), acc[f / 24]);
#pragma unroll
    for (int a = 0; a < NA; ++a) {
      const int ex = ((__float_as_int(acc[a]) >> 23) & 0xff) - 127 + 24 * a;
      if (a == 0) {
        bi = ex;
      } else {
        bi = acc[a] != 0.f ? ex : bi;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// L <= 32: one warp per chain.  DT = compile-time direction count (0: read it from the params).
// ------------------------------------------------------------------------------------------------
// Generic kernel: any direction, any alignment.  Inputs are staged through a ring of 4-byte
// cp.async copies kPF pixels ahead (a register ring of plain loads was measured slower: waiting on
// a register load drains every younger load too, whereas cp.async groups retire in order).
// DT = compile-time direction count (0: read it from the params).
template <int LMAX, int DT, bool TRAIN>
__global__ void __launch_bounds__(128, 1) fwd_warp_kernel(const __grid_constant__ FwdParams p) {
  extern __shared__ __align__(16) float smem[];
  const int wpb = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  ChainCtx ch;
  if (!decode_chain(p, blockIdx.x * wpb + warp, ch)) return;
  const int L = p.L, D = DT ? DT : p.D, rows = D + 2;
  const int slot_floats = rows * 32;
  float* ring = smem + warp * (kPF * slot_floats + 64);
  float* hbuf = ring + kPF * slot_floats;
  float* ring_lane = ring + lane;
  const bool act = lane < L;
  const int lc = act ? lane : L - 1;  // idle lanes shadow the last label: no divergent code below
  const float rho = p.rho;

  float cr[LMAX];
#pragma unroll
  for (int f = 0; f < LMAX; ++f) cr[f] = (act && f < L) ? ctx_value(p.ctx, p.ctx_rank, L, lane, f) : 0.f;

  const long long ibase = (long long)ch.img * p.H * p.W;
  // per-lane base pointers; everything below addresses them with 32-bit element offsets
  const float* Ul = p.unary + ibase * L + lc;
  const float* Ml = p.msg_read + ibase * L + lc;
  float* Mwl = p.msg_write + (long long)ch.dir * p.slice + ibase * L + lc;
  const bool has_e = p.ew != nullptr;
  const float* E = has_e ? p.ew + (long long)ch.dir * p.pslice + ibase : p.unary;
  uint8_t* MIl = TRAIN ? p.min_idx + (long long)ch.dir * p.slice + ibase * L + lc : nullptr;
  uint8_t* NI = TRAIN ? p.norm_idx + (long long)ch.dir * p.pslice + ibase : nullptr;
  const int len = ch.len;
  const int ostep = ch.pstep * L;
  const int dir_row = (1 + ch.dir) * 32, inv_row = (1 + ch.inv) * 32;

  // Staging of chain pixel j (its unary and D messages, used when it is the predecessor, and its
  // edge weight, used when it is the current pixel).  Pixels past the chain end are replaced by
  // the last pixel (the copies land in slots nobody reads), which keeps the loop branch-free.
  const int px_last = ch.h0 * p.W + ch.w0 + (len - 1) * ch.pstep;
  int px_pf = ch.h0 * p.W + ch.w0;
  auto issue = [&](int j) {
    float* dst = ring_lane + (j & (kPF - 1)) * slot_floats;
    const int pxc = j < len ? px_pf : px_last;
    const int o = pxc * L;
    cp_async4(dst, Ul + o);
#pragma unroll
    for (int k = 0; k < (DT ? DT : 16); ++k)
      if (k < D) cp_async4(dst + (1 + k) * 32, Ml + k * p.slice + o);
    cp_async4(dst + (D + 1) * 32, E + pxc);
    cp_async_commit();
    px_pf += ch.pstep;
  };
  auto uu_of = [&](const float* sl) {  // sl: this lane's column of a ring slot
    float s = sl[0];
#pragma unroll
    for (int k = 0; k < (DT ? DT : 16); ++k)
      if (k < D) s += sl[(1 + k) * 32];
    s -= sl[dir_row];
    return fmaf(s, rho, -sl[inv_row]);
  };

#pragma unroll
  for (int j = 0; j < kPF; ++j) issue(j);
  cp_async_wait<kPF - 1>();
  float uu = uu_of(ring_lane);
  issue(kPF);
  float r = 0.f;
  int px = ch.h0 * p.W + ch.w0 + ch.pstep;  // pixel i = 1
  int of = px * L;

  for (int i = 1; i < len; ++i) {
    cp_async_wait<kPF - 1>();  // everything staged for chain pixel i has landed
    const float* sl = ring_lane + (i & (kPF - 1)) * slot_floats;
    const float e = has_e ? sl[(D + 1) * 32] : 1.f;
    // Old values at pixel i are consumed BEFORE the new message of pixel i is stored (TRWP updates
    // the message slice in place).
    const float uu_next = uu_of(sl);
    float* hb = hbuf + (i & 1) * 32;
    hb[lane] = act ? fmaf(rho, r, uu) : kInf;
    __syncwarp();
    float best;
    int bi;
    minplus_regrow<LMAX, TRAIN>(hb, cr, e, best, bi);
    const float m = warp_min(act ? best : kInf);
    r = best - m;
    if (act) Mwl[of] = r;
    if (TRAIN) {
      const unsigned bal = __ballot_sync(0xffffffffu, act && best == m);
      if (act) MIl[of] = (uint8_t)bi;
      if (lane == 0) NI[px] = (uint8_t)(31 - __clz(bal));
    }
    issue(i + kPF);
    uu = uu_next;
    px += ch.pstep;
    of += ostep;
  }
  cp_async_wait<0>();
}

// ------------------------------------------------------------------------------------------------
// L > 32: one CTA per chain, thread = label.
// ------------------------------------------------------------------------------------------------
// Block-wide min with the index of the HIGHEST thread attaining it.  One __syncthreads inside.
__device__ __forceinline__ void block_min_hi(float v, bool act, int tid, float* red_v, int* red_i,
                                             int nw, float& m, int& n) {
  const float x = act ? v : kInf;
  const float wm = warp_min(x);
  const unsigned bal = __ballot_sync(0xffffffffu, act && x == wm);
  if ((tid & 31) == 0) {
    red_v[tid >> 5] = wm;
    red_i[tid >> 5] = bal ? (tid & ~31) + 31 - __clz(bal) : -1;
  }
  __syncthreads();
  m = kInf;
  n = 0;
  for (int w = 0; w < nw; ++w) {
    const float y = red_v[w];
    const int yi = red_i[w];
    if (yi >= 0 && y <= m) {
      m = y;
      n = yi;
    }
  }
}

template <int MODE, bool TRAIN>
__global__ void __launch_bounds__(256) fwd_cta_kernel(const __grid_constant__ FwdParams p) {
  extern __shared__ __align__(16) float smem[];
  ChainCtx ch;
  if (!decode_chain(p, blockIdx.x, ch)) return;  // uniform for the CTA
  const int L = p.L, D = p.D, rows = D + 2, NT = blockDim.x, c = threadIdx.x, nw = NT >> 5;
  float* ring = smem;                  // [kPF][rows][NT]
  float* hbuf = ring + kPF * rows * NT;  // [NT]
  float* ctx1 = hbuf + NT;             // [NT]   (MODE 1)
  float* redA_v = ctx1 + NT;           // [8]
  int* redA_i = reinterpret_cast<int*>(redA_v + 8);
  float* redB_v = redA_v + 16;
  int* redB_i = reinterpret_cast<int*>(redB_v + 8);
  const bool act = c < L;

  bool windowed = false;
  int R = 0;
  float cmax = 0.f;
  if (MODE == 1) {
    ctx1[c] = act ? __ldg(p.ctx + c) : 0.f;
    const CtxInfo inf = *p.info;
    windowed = inf.windowed && (p.ew == nullptr || float_from_order_bits(inf.ew_min_bits) >= 0.f);
    R = inf.R;
    cmax = inf.cmax;
  }
  float cr[MODE == 2 ? 64 : 1];
  if constexpr (MODE == 2) {
#pragma unroll
    for (int f = 0; f < 64; ++f) cr[f] = (act && f < L) ? ctx_value(p.ctx, 2, L, c, f) : 0.f;
  }
  hbuf[c] = kInf;  // entries >= L stay +inf
  __syncthreads();

  const long long ibase = (long long)ch.img * p.H * p.W;
  const float* U = p.unary + ibase * L;
  const float* Mr = p.msg_read + ibase * L;
  float* Mw = p.msg_write + (long long)ch.dir * p.slice + ibase * L;
  const float* E = p.ew ? p.ew + (long long)ch.dir * p.pslice + ibase : nullptr;
  uint8_t* MI = TRAIN ? p.min_idx + (long long)ch.dir * p.slice + ibase * L : nullptr;
  uint8_t* NI = TRAIN ? p.norm_idx + (long long)ch.dir * p.pslice + ibase : nullptr;
  const int pix0 = ch.h0 * p.W + ch.w0;
  const int len = ch.len;

  auto issue = [&](int j) {
    if (j < len) {
      float* dst = ring + (j & (kPF - 1)) * rows * NT + c;
      const int px = pix0 + j * ch.pstep;
      if (act && j < len - 1) {
        cp_async4(dst, U + (long long)px * L + c);
        for (int k = 0; k < D; ++k) cp_async4(dst + (1 + k) * NT, Mr + k * p.slice + (long long)px * L + c);
      }
      if (E && j >= 1) cp_async4(dst + (D + 1) * NT, E + px);
    }
    cp_async_commit();
  };

#pragma unroll
  for (int j = 0; j < kPF; ++j) issue(j);
  cp_async_wait<kPF - 1>();
  float uu = act ? uu_from_ring(ring, NT, c, D, ch.dir, ch.inv, p.rho) : 0.f;
  issue(kPF);
  float r = 0.f;

  for (int i = 1; i < len; ++i) {
    cp_async_wait<kPF - 1>();
    const float* slot = ring + (i & (kPF - 1)) * rows * NT;
    const float e = E ? slot[(D + 1) * NT + c] : 1.f;
    const float uu_next = (act && i < len - 1) ? uu_from_ring(slot, NT, c, D, ch.dir, ch.inv, p.rho) : 0.f;
    const float h = act ? fmaf(p.rho, r, uu) : kInf;
    if (act) hbuf[c] = h;

    float best = kInf;
    int bi = 0;
    if (MODE == 1 && windowed) {
      float hmin;
      int fstar;
      block_min_hi(h, act, c, redA_v, redA_i, nw, hmin, fstar);  // also publishes hbuf
      const float gv = fmaf(e, cmax, hmin);
      if (fstar >= c + R) {  // scanned before the window in the reference's high-to-low order
        best = gv;
        bi = fstar;
      }
      int fhi = c + R - 1;
      if (fhi > L - 1) fhi = L - 1;
      int flo = c - R + 1;
      if (flo < 0) flo = 0;
      for (int f = fhi; f >= flo; --f) {
        const int k = f > c ? f - c : c - f;
        const float v = fmaf(e, ctx1[k], hbuf[f]);
        if (v < best) {
          best = v;
          bi = f;
        }
      }
      if (fstar <= c - R && gv < best) {
        best = gv;
        bi = fstar;
      }
    } else {
      __syncthreads();
      if constexpr (MODE == 2) {
        minplus_regrow<64, TRAIN>(hbuf, cr, e, best, bi);
      } else {
        for (int f = L - 1; f >= 0; --f) {
          float cv;
          if (MODE == 1) {
            cv = ctx1[f > c ? f - c : c - f];
          } else {
            cv = ctx_value(p.ctx, 2, L, c, f);
          }
          const float v = fmaf(e, cv, hbuf[f]);
          if (f == L - 1 || v < best) {
            best = v;
            bi = f;
          }
        }
      }
    }
    float m;
    int n;
    block_min_hi(best, act, c, redB_v, redB_i, nw, m, n);
    r = best - m;
    const int px = pix0 + i * ch.pstep;
    if (act) Mw[(long long)px * L + c] = r;
    if (TRAIN) {
      if (act) MI[(long long)px * L + c] = (uint8_t)bi;
      if (c == 0) NI[px] = (uint8_t)n;
    }
    issue(i + kPF);
    uu = uu_next;
  }
  cp_async_wait<0>();
}

// ------------------------------------------------------------------------------------------------
// Context / edge-weight analysis (rank-1 contexts with L > 32 only).
// ------------------------------------------------------------------------------------------------
__global__ void analyze_ctx_kernel(const float* ctx, int L, CtxInfo* info) {
  // Single thread: L <= 256 values.
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const float cmax = ctx[L - 1];
  int R = L - 1;
  while (R > 0 && ctx[R - 1] == cmax) --R;
  // Exactness of the windowed evaluation needs only ctx[k] <= cmax for every k < R (and weights
  // >= 0): candidates outside the window then cost at least h_min + w * cmax.
  bool mono = true;
  for (int k = 0; k < R; ++k) mono = mono && (ctx[k] <= cmax);
  info->windowed = (mono && 2 * R - 1 < L) ? 1 : 0;
  info->R = R;
  info->cmax = cmax;
  info->ew_min_bits = 0x7fffffff;
}

__global__ void analyze_ew_kernel(const float* ew, long long n, CtxInfo* info) {
  float m = kInf;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    m = fminf(m, ew[i]);
  m = warp_min(m);
  if ((threadIdx.x & 31) == 0) atomicMin(&info->ew_min_bits, float_order_bits(m));
}

// ------------------------------------------------------------------------------------------------
// Cost aggregation (+ optional labels).  MPLayers/TRWP/TRWP_forward.cu:8-58 and
// MPLayers/ISGMR/ISGMR_forward.cu:69-99, without the device-to-device copy of the unaries.
// ------------------------------------------------------------------------------------------------
__global__ void aggregate_kernel(const float* __restrict__ unary, const float* __restrict__ msg,
                                 float* __restrict__ cost, long long n, int D, long long slice,
                                 float factor, int min_a_dir) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float v = unary[i] * factor;
    if (min_a_dir) {
      float mm = msg[i];
      for (int k = 1; k < D; ++k) {
        const float x = msg[k * slice + i];
        if (x < mm) mm = x;
      }
      v += mm;
    } else {
      for (int k = 0; k < D; ++k) v += msg[k * slice + i];
    }
    cost[i] = v;
  }
}

__global__ void label_kernel(const float* __restrict__ cost, uint8_t* __restrict__ label,
                             long long npix, int L) {
  const long long px = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (px >= npix) return;
  const float* c = cost + px * L;
  float mv = c[0];
  int ml = 0;
  for (int l = 1; l < L; ++l) {
    const float v = c[l];
    if (v < mv) {
      mv = v;
      ml = l;
    }
  }
  label[px] = (uint8_t)ml;
}

template <typename K>
cudaError_t ensure_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024)
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  return cudaSuccess;
}

template <int LMAX, int DT, bool TRAIN>
cudaError_t launch_warp_d(const FwdParams& p, cudaStream_t st) {
  const int total = p.chain_off[p.ndirs];
  const int wpb = total >= 148 * 32 ? 4 : 1;
  const size_t smem = (size_t)wpb * (kPF * (p.D + 2) * 32 + 64) * sizeof(float);
  cudaError_t e = ensure_smem(fwd_warp_kernel<LMAX, DT, TRAIN>, smem);
  if (e != cudaSuccess) return e;
  ProfScope prof(kProfFwdSweep, st);
  fwd_warp_kernel<LMAX, DT, TRAIN><<<(total + wpb - 1) / wpb, wpb * 32, smem, st>>>(p);
  count_launch();
  return cudaGetLastError();
}

template <int LMAX, bool TRAIN>
cudaError_t launch_warp(const FwdParams& p, cudaStream_t st) {
  if (p.D == 4) return launch_warp_d<LMAX, 4, TRAIN>(p, st);
  if (p.D == 8) return launch_warp_d<LMAX, 8, TRAIN>(p, st);
  return launch_warp_d<LMAX, 0, TRAIN>(p, st);
}

template <int MODE, bool TRAIN>
cudaError_t launch_cta(const FwdParams& p, cudaStream_t st) {
  const int total = p.chain_off[p.ndirs];
  const int NT = MODE == 2 ? 64 : ((p.L + 31) / 32) * 32;
  const size_t smem = ((size_t)kPF * (p.D + 2) * NT + 2 * NT + 32) * sizeof(float);
  cudaError_t e = ensure_smem(fwd_cta_kernel<MODE, TRAIN>, smem);
  if (e != cudaSuccess) return e;
  ProfScope prof(kProfFwdSweep, st);
  fwd_cta_kernel<MODE, TRAIN><<<total, NT, smem, st>>>(p);
  count_launch();
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_analyze(const float* ctx, int L, int rank, const float* ew, long long n_ew,
                           CtxInfo* info, cudaStream_t st) {
  if (!(rank == 1 && L > 32)) return cudaSuccess;
  analyze_ctx_kernel<<<1, 32, 0, st>>>(ctx, L, info);
  count_launch();
  if (ew) {
    const int blocks = (int)((n_ew + 1023) / 1024 < 1184 ? (n_ew + 1023) / 1024 : 1184);
    analyze_ew_kernel<<<blocks, 256, 0, st>>>(ew, n_ew, info);
    count_launch();
  }
  return cudaGetLastError();
}

cudaError_t launch_forward_sweep(const FwdParams& p, bool train, cudaStream_t st) {
  if (p.chain_off[p.ndirs] == 0) return cudaSuccess;
  if (p.L <= 32) {
    if (p.L == 21) return train ? launch_warp<21, true>(p, st) : launch_warp<21, false>(p, st);
    return train ? launch_warp<32, true>(p, st) : launch_warp<32, false>(p, st);
  }
  if (p.ctx_rank == 1) return train ? launch_cta<1, true>(p, st) : launch_cta<1, false>(p, st);
  if (p.L <= 64) return train ? launch_cta<2, true>(p, st) : launch_cta<2, false>(p, st);
  return train ? launch_cta<0, true>(p, st) : launch_cta<0, false>(p, st);
}

cudaError_t launch_aggregate(const float* unary, const float* msg, float* cost, uint8_t* label,
                             long long npix, int L, int D, long long slice, float factor,
                             int min_a_dir, cudaStream_t st) {
  const long long n = npix * L;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  ProfScope prof(kProfElementwise, st);
  aggregate_kernel<<<(int)blocks, 256, 0, st>>>(unary, msg, cost, n, D, slice, factor, min_a_dir);
  count_launch();
  if (label) {
    label_kernel<<<(int)((npix + 127) / 128), 128, 0, st>>>(cost, label, npix, L);
    count_launch();
  }
  return cudaGetLastError();
}

}  // namespace mpl
