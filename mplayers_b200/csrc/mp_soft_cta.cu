// Soft (expected-value) TRWP for 32 < L <= 64: one CTA of 64 threads per chain, thread = label c.
//
// The message of label c is the expectation of its edge values v[f] = e*ctx(c,f) + h[f] under
// softmin weights (MPLayers/TRWP_hard_soft/TRWP_forward_soft.cu:55-92); in training the L x L edge
// values of every visited pixel are saved (entry [f][c] for even directions, [c][f] for odd ones)
// together with the normalisation index, and the backward pass recomputes the weights from them
// (MPLayers/TRWP_hard_soft/TRWP_backward_soft.cu:100-127).  With one thread per label a thread owns
// its whole row of L candidates, so every row reduction (minimum, sum of exponentials, expectation)
// is thread-local; the CTA meets twice per step: to publish the predecessor's vector h and to
// normalise.  Row sums are taken in the order of the reference's reduction -- a shuffle-down tree
// per block of 32 candidates, blocks added left to right (MPLayers/TRWP_hard_soft/TRWP_soft.cuh:45-71)
// -- which is the order the CPU oracle uses for rows longer than 32.
// The one-warp kernels of mp_forward.cu / mp_backward.cu serve L <= 32; this pair widens the soft
// variant to the label counts of the two-labels-per-lane hard kernels.  It is written for
// coverage, not for speed: inputs come straight from global memory (the next pixel's a step ahead).
#include <cstdlib>

#include "mp_common.cuh"
#include "mp_minplus.cuh"

namespace mpl {

namespace {

constexpr int kSL = 64;   // threads per CTA = most labels
constexpr int kSLS = 65;  // row stride of the shared context table (conflict-free column walks)

// Sum of 32 values in the order of a shuffle-down tree over a warp (x[i] += x[i + 16], then 8, 4,
// 2, 1; element 0 holds the total).
__device__ __forceinline__ float tree32(float (&x)[32]) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1)
#pragma unroll
    for (int i = 0; i < off; ++i) x[i] = __fadd_rn(x[i], x[i + off]);
  return x[0];
}

// Row sum of 64 values (entries >= L are zero) in the reference's order.
__device__ __forceinline__ float row_sum64(const float (&v)[kSL]) {
  float a[32], b[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) a[i] = v[i], b[i] = v[32 + i];
  return __fadd_rn(tree32(a), tree32(b));
}

// Minimum / sum over the two warps of the CTA.  `slot` alternates between steps so that a fast warp
// cannot overwrite what the slow one still reads.
__device__ __forceinline__ void cta_min_hi(float v, bool act, int tid, float* red, int slot, float& m, int& n) {
  const float x = act ? v : kInf;
  const float wm = warp_min(x);
  const unsigned bal = __ballot_sync(0xffffffffu, act && x == wm);
  float* rv = red + slot * 4;
  if ((tid & 31) == 0) {
    rv[tid >> 5] = wm;
    rv[2 + (tid >> 5)] = __int_as_float(bal ? (tid & ~31) + 31 - __clz(bal) : -1);
  }
  __syncthreads();
  m = fminf(rv[0], rv[1]);
  const int i0 = __float_as_int(rv[2]), i1 = __float_as_int(rv[3]);
  n = (rv[1] == m && i1 >= 0) ? i1 : i0;   // ties -> highest index (MPLayers/TRWP_hard_soft/TRWP_soft.cuh:74-140)
}

template <bool TRAIN>
__global__ void __launch_bounds__(kSL, 2) fwd_soft_cta_kernel(const __grid_constant__ FwdParams p) {
  extern __shared__ __align__(16) float smem[];
  float* ctab = smem;                 // [L][kSLS]
  float* hs = ctab + kSL * kSLS;      // [2][64]
  float* red = hs + 2 * kSL;          // [2][4]
  const int c = threadIdx.x, L = p.L, D = p.D;
  ChainCtx ch;
  if (!decode_chain(p, blockIdx.x, ch)) return;  // uniform for the CTA
  for (int i = c; i < L * L; i += kSL) ctab[(i / L) * kSLS + (i % L)] = ctx_value(p.ctx, p.ctx_rank, L, i / L, i % L);
  __syncthreads();
  const bool act = c < L;
  const int lc = act ? c : L - 1;   // idle threads shadow the last label; their stores are masked
  const float rho = p.rho;
  const float* crow = ctab + lc * kSLS;
  const long long ibase = (long long)ch.img * p.H * p.W;
  const float* U = p.unary + ibase * L + lc;
  const float* M = p.msg_read + ibase * L + lc;
  float* Mw = p.msg_write + (long long)ch.dir * p.slice + ibase * L + lc;
  const float* E = p.ew ? p.ew + (long long)ch.dir * p.pslice + ibase : nullptr;
  uint8_t* NI = TRAIN ? p.norm_idx + (long long)ch.dir * p.pslice + ibase : nullptr;
  float* EL = TRAIN ? p.edge_label + ((long long)ch.dir * p.pslice + ibase) * L * L : nullptr;
  const bool l2r = (ch.dir & 1) == 0;
  auto uu_of = [&](int px) {  // reference order of the additions
    const int o = px * L;
    float s = U[o];
    for (int k = 0; k < D; ++k) s += M[(long long)k * p.slice + o];
    s -= M[(long long)ch.dir * p.slice + o];
    return fmaf(s, rho, -M[(long long)ch.inv * p.slice + o]);
  };
  int px = ch.h0 * p.W + ch.w0;
  float uu = uu_of(px), r = 0.f;
  for (int i = 1; i < ch.len; ++i) {
    px += ch.pstep;
    const float e = E ? E[px] : 1.f;
    // Old values at pixel i are read BEFORE its new message is stored (the slice is updated in place).
    const float uu_next = uu_of(px);
    float* h = hs + (i & 1) * kSL;
    h[c] = act ? fmaf(rho, r, uu) : kInf;
    __syncthreads();
    float val[kSL], ex[kSL];
    float m = kInf;
#pragma unroll
    for (int f = 0; f < kSL; ++f) {
      val[f] = f < L ? fmaf(e, crow[f], h[f]) : kInf;
      m = fminf(m, val[f]);
    }
    if (TRAIN && act) {
      float* el = EL + (long long)px * L * L;
#pragma unroll
      for (int f = 0; f < kSL; ++f)
        if (f < L) el[l2r ? f * L + c : c * L + f] = val[f];
    }
#pragma unroll
    for (int f = 0; f < kSL; ++f) ex[f] = f < L ? __expf(-val[f] + m) : 0.f;
    const float se = row_sum64(ex);
#pragma unroll
    for (int f = 0; f < kSL; ++f) ex[f] = f < L ? __fdiv_rn(__fmul_rn(ex[f], val[f]), se) : 0.f;
    const float msg = row_sum64(ex);
    float mn;
    int n;
    cta_min_hi(msg, act, c, red, i & 1, mn, n);
    r = msg - mn;
    if (act) Mw[px * L] = r;
    if (TRAIN && c == 0) NI[px] = (uint8_t)n;
    uu = uu_next;
  }
}

// Backward, C + P bookkeeping (BwdParams::cp_scheme == 1): C in `dunary`, P_k in `dm_read`.
__global__ void __launch_bounds__(kSL, 2) bwd_soft_cta_kernel(const __grid_constant__ BwdParams p) {
  extern __shared__ __align__(16) float smem[];
  float* ctab = smem;                 // [L][kSLS]
  float* tile = ctab + kSL * kSLS;    // [64][kSLS]  d(value[c][f])
  float* red = tile + kSL * kSLS;     // [2][4]
  const int c = threadIdx.x, L = p.L;
  BChain ch;
  if (!decode_bchain(p, blockIdx.x, ch)) return;  // uniform for the CTA
  for (int i = c; i < L * L; i += kSL) ctab[(i / L) * kSLS + (i % L)] = ctx_value(p.ctx, p.ctx_rank, L, i / L, i % L);
  __syncthreads();
  const bool act = c < L;
  const int lc = act ? c : L - 1;
  const int dir = ch.dir, inv = dir ^ 1;
  const float rho = p.rho;
  const float* crow = ctab + lc * kSLS;
  const long long ibase = (long long)ch.img * p.H * p.W;
  float* C = p.dunary + ibase * L + lc;
  float* Pd = p.dm_read + (long long)dir * p.slice + ibase * L + lc;
  float* Pi = p.dm_read + (long long)inv * p.slice + ibase * L + lc;
  const float* E = p.ew ? p.ew + (long long)dir * p.pslice + ibase : nullptr;
  float* DE = p.dew ? p.dew + (long long)dir * p.pslice + ibase : nullptr;
  const uint8_t* NI = p.norm_idx + (long long)dir * p.pslice + ibase;
  const float* EL = p.edge_label + ((long long)dir * p.pslice + ibase) * L * L;
  const bool l2r = (dir & 1) == 0;
  float acc[kSL];  // label-context gradient of row c (diagonal included)
#pragma unroll
  for (int f = 0; f < kSL; ++f) acc[f] = 0.f;
  float q = 0.f;
  int px = ch.h0 * p.W + ch.w0 + (ch.len - 1) * ch.pstep;  // last pixel of the chain
  for (int s = 0; s < ch.len; ++s) {
    const int of = px * L;
    const float c_old = C[of];
    const float x0 = c_old + Pd[of];   // gradient of this pixel's message: C + P_dir
    const float rq = rho * q;
    float qn = 0.f;
    if (s < ch.len - 1) {
      const float e = E ? E[px] : 1.f;
      const int n = NI[px];
      const float* ev = EL + (long long)px * L * L;
      float d[kSL];
#pragma unroll
      for (int f = 0; f < kSL; ++f) d[f] = (f < L) ? (l2r ? ev[f * L + lc] : ev[lc * L + f]) : kInf;
      // normalisation backward (MPLayers/commonCUDA.cuh:131-145): t[n] -= sum_c t[c]
      float t = act ? x0 + rq : 0.f;
      const float ws = warp_sum(t);
      float* rs = red + (s & 1) * 4;
      if ((c & 31) == 0) rs[c >> 5] = ws;
      __syncthreads();
      const float S = rs[0] + rs[1];
      t = (c == n) ? t - S : t;
      // softmin weights of row c from the saved edge values
      float m = kInf;
#pragma unroll
      for (int f = 0; f < kSL; ++f) m = fminf(m, d[f]);
      float ex[kSL], se = 0.f, ms = 0.f;
#pragma unroll
      for (int f = 0; f < kSL; ++f) {
        ex[f] = (f < L) ? __expf(m - d[f]) : 0.f;
        se += ex[f];
      }
      const float inv_se = 1.f / se;
#pragma unroll
      for (int f = 0; f < kSL; ++f) {
        ex[f] *= inv_se;
        ms = (f < L) ? fmaf(ex[f], d[f], ms) : ms;
      }
      float de = 0.f;
#pragma unroll
      for (int f = 0; f < kSL; ++f) {
        const float dd = (f < L && act) ? t * ex[f] * (1.f - d[f] + ms) : 0.f;
        if (f < L) tile[c * kSLS + f] = dd;
        de = fmaf(crow[f < L ? f : 0], dd, de);
        acc[f] = fmaf(e, dd, acc[f]);
      }
      const float wde = warp_sum(de);
      if ((c & 31) == 0) rs[2 + (c >> 5)] = wde;
      __syncthreads();
      if (DE && c == 0) atomicAdd(DE + px, rs[2] + rs[3]);
      if (act) {  // scatter to the predecessor: column sums in a fixed order
        float qa = 0.f, qb = 0.f;
        int k = 0;
        for (; k + 1 < L; k += 2) {
          qa += tile[k * kSLS + c];
          qb += tile[(k + 1) * kSLS + c];
        }
        if (k < L) qa += tile[k * kSLS + c];
        qn = qa + qb;
      }
    }
    if (act) {
      const float cnew = c_old + rq;  // dU and every dM_k (k != dir, inv) receive rho*q
      C[of] = cnew;
      Pd[of] = -cnew;                 // dM_dir = C + P_dir = 0 after its sweep
      atomicAdd(Pi + of, -q);
    }
    q = qn;
    px -= ch.pstep;
  }
  float* part = p.dctx_part + (long long)(blockIdx.x % p.n_slots) * (p.ctx_rank == 2 ? L * L : L);
  if (act) {
#pragma unroll
    for (int f = 0; f < kSL; ++f) {
      if (f < L && acc[f] != 0.f) {
        if (p.ctx_rank == 2) {
          atomicAdd(part + c * L + f, acc[f]);
        } else {
          atomicAdd(part + (c > f ? c - f : f - c), acc[f]);
        }
      }
    }
  }
}

}  // namespace

cudaError_t launch_forward_soft_cta(const FwdParams& p, bool train, cudaStream_t st) {
  const int total = p.chain_off[p.ndirs];
  if (total == 0) return cudaSuccess;
  if (p.L <= 32 || p.L > kSL) return cudaErrorNotSupported;
  const size_t smem = ((size_t)kSL * kSLS + 2 * kSL + 8) * sizeof(float);
  ProfScope prof(kProfFwdSweep, st);
  if (train) {
    fwd_soft_cta_kernel<true><<<total, kSL, smem, st>>>(p);
  } else {
    fwd_soft_cta_kernel<false><<<total, kSL, smem, st>>>(p);
  }
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_backward_soft_cta(const BwdParams& p, int total, cudaStream_t st) {
  if (total == 0) return cudaSuccess;
  if (p.L <= 32 || p.L > kSL || p.cp_scheme != 1) return cudaErrorNotSupported;
  const size_t smem = ((size_t)2 * kSL * kSLS + 8) * sizeof(float);
  ProfScope prof(kProfBwdSweep, st);
  bwd_soft_cta_kernel<<<total, kSL, smem, st>>>(p);
  count_launch();
  return cudaGetLastError();
}

}  // namespace mpl
