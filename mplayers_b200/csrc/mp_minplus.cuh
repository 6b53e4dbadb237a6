// Device helpers shared by the chain kernels: exact minimum + highest argmin of a register row
// (forward), and the gather that replays saved argmin indices (backward).
#pragma once
#include "mp_common.cuh"

namespace mpl {

// A chain of a forward launch: direction, image, start pixel, length and pixel step.
struct ChainCtx {
  int dir, inv, img, h0, w0, len, pstep;
};

__device__ __forceinline__ bool decode_chain(const FwdParams& p, int g, ChainCtx& c) {
  if (g >= p.chain_off[p.ndirs]) return false;
  int di = 0;
  while (g >= p.chain_off[di + 1]) ++di;
  c.dir = p.dir0 + di;
  c.inv = c.dir ^ 1;
  // When a launch covers only a part of the chains, both directions of a pair must cover the same
  // lines (each reads the other's messages): the odd direction then enumerates the even one's
  // chains and walks each from its far end.
  const bool mirrored = p.parts > 1 && (c.dir & 1);
  DirGeom geo = make_geom(mirrored ? c.inv : c.dir, p.H, p.W);
  const int local = g - p.chain_off[di] + p.chain_begin[di];
  c.img = local / geo.n_chains;
  chain_start(geo, p.H, p.W, local - c.img * geo.n_chains, c.h0, c.w0, c.len);
  if (mirrored) {
    c.h0 += (c.len - 1) * geo.hs;
    c.w0 += (c.len - 1) * geo.ws;
    geo.hs = -geo.hs;
    geo.ws = -geo.ws;
  }
  c.pstep = geo.hs * p.W + geo.ws;
  return c.len >= 2;
}

// A chain of a backward launch.
struct BChain {
  int dir, img, h0, w0, len, pstep;
};

__device__ __forceinline__ bool decode_bchain(const BwdParams& p, int g, BChain& c) {
  if (g >= p.chain_off[p.ndirs]) return false;
  int di = 0;
  while (g >= p.chain_off[di + 1]) ++di;
  c.dir = p.dir + di;
  // partial launches: the odd direction of a pair covers the even one's lines (see decode_chain)
  const bool mirrored = p.parts > 1 && (c.dir & 1);
  DirGeom geo = make_geom(mirrored ? (c.dir ^ 1) : c.dir, p.H, p.W);
  const int local = g - p.chain_off[di] + p.chain_begin[di];
  c.img = local / geo.n_chains;
  chain_start(geo, p.H, p.W, local - c.img * geo.n_chains, c.h0, c.w0, c.len);
  if (mirrored) {
    c.h0 += (c.len - 1) * geo.hs;
    c.w0 += (c.len - 1) * geo.ws;
    geo.hs = -geo.hs;
    geo.ws = -geo.ws;
  }
  c.pstep = geo.hs * p.W + geo.ws;
  return true;
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
// CN / OFF: `cr` has CN entries of which LMAX starting at OFF are used (hb points at candidate OFF).
template <int LMAX, int CN = LMAX, int OFF = 0>
__device__ __forceinline__ void minplus_vals(const float* hb, const float (&cr)[CN], float e, float (&val)[LMAX]) {
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
#pragma unroll
  for (int f = 0; f + 1 < LMAX; f += 2) ffma2(val[f], val[f + 1], e, e, cr[OFF + f], cr[OFF + f + 1], hv[f], hv[f + 1]);
  if (LMAX & 1) val[LMAX - 1] = fmaf(e, cr[OFF + LMAX - 1], hv[LMAX - 1]);
}

// Highest f with val[f] == best (best must be the exact minimum of val, so at least one matches).
template <int LMAX>
__device__ __forceinline__ int highest_equal(const float (&val)[LMAX], float best) {
  // Sums of distinct powers of two are exact in any order, so each group of 24 labels is
  // accumulated in four interleaved partial sums (short dependency chains), two per packed fma.
  constexpr int NA = (LMAX + 23) / 24;
  float acc[NA][4];
#pragma unroll
  for (int a = 0; a < NA; ++a) acc[a][0] = acc[a][1] = acc[a][2] = acc[a][3] = 0.f;
  if constexpr (LMAX <= 24) {
    // one group: scalar fmas (measured on the 21-label sweeps: 102.1 against 104.1 us; with 32
    // candidates the packed form below is the faster one, 7.4 against 8.1 ms on the 64-label sweeps)
#pragma unroll
    for (int f = 0; f < LMAX; ++f) acc[0][f & 3] = fmaf(eq_flag(val[f], best), pow2f(f), acc[0][f & 3]);
  } else {
#pragma unroll
    for (int f = 0; f + 1 < LMAX; f += 2) {  // 24 is even: a pair never straddles two groups
      const int a = f / 24, j = f & 2;
      ffma2(acc[a][j], acc[a][j + 1], eq_flag(val[f], best), eq_flag(val[f + 1], best), pow2f(f % 24),
            pow2f((f + 1) % 24), acc[a][j], acc[a][j + 1]);
    }
    if (LMAX & 1) {
      constexpr int f = LMAX - 1;
      acc[f / 24][0] = fmaf(eq_flag(val[f], best), pow2f(f % 24), acc[f / 24][0]);
    }
  }
  int bi = 0;
#pragma unroll
  for (int a = 0; a < NA; ++a) {
    const float sum = (acc[a][0] + acc[a][1]) + (acc[a][2] + acc[a][3]);
    const int ex = ((__float_as_int(sum) >> 23) & 0xff) - 127 + 24 * a;
    if (a == 0) {
      bi = ex;
    } else {
      bi = sum != 0.f ? ex : bi;
    }
  }
  return bi;
}

// The same for a value that need not be among val: -1 if no val[f] equals it.
template <int LMAX>
__device__ __forceinline__ int highest_equal_or_none(const float (&val)[LMAX], float best) {
  constexpr int NA = (LMAX + 23) / 24;
  float acc[NA][4];
#pragma unroll
  for (int a = 0; a < NA; ++a) acc[a][0] = acc[a][1] = acc[a][2] = acc[a][3] = 0.f;
#pragma unroll
  for (int f = 0; f + 1 < LMAX; f += 2) {
    const int a = f / 24, j = f & 2;
    ffma2(acc[a][j], acc[a][j + 1], eq_flag(val[f], best), eq_flag(val[f + 1], best), pow2f(f % 24),
          pow2f((f + 1) % 24), acc[a][j], acc[a][j + 1]);
  }
  if (LMAX & 1) {
    constexpr int f = LMAX - 1;
    acc[f / 24][0] = fmaf(eq_flag(val[f], best), pow2f(f % 24), acc[f / 24][0]);
  }
  int bi = -1;
#pragma unroll
  for (int a = 0; a < NA; ++a) {
    const float sum = (acc[a][0] + acc[a][1]) + (acc[a][2] + acc[a][3]);
    const int ex = ((__float_as_int(sum) >> 23) & 0xff) - 127 + 24 * a;
    bi = sum != 0.f ? ex : bi;
  }
  return bi;
}

template <int LMAX, bool TRAIN, int CN = LMAX, int OFF = 0>
__device__ __forceinline__ void minplus_regrow(const float* hb, const float (&cr)[CN], float e,
                                               float& best, int& bi) {
  float val[LMAX];
  minplus_vals<LMAX, CN, OFF>(hb, cr, e, val);
  best = min_tree<LMAX>(val);
  bi = 0;
  if (TRAIN) bi = highest_equal<LMAX>(val, best);
}

// The argmin index alone, for a minimum that is already known (recomputes the candidates).
template <int LMAX>
__device__ __forceinline__ int minplus_index(const float* hb, const float (&cr)[LMAX], float e, float best) {
  float val[LMAX];
  minplus_vals<LMAX>(hb, cr, e, val);
  return highest_equal<LMAX>(val, best);
}

// q[f] = sum over labels c whose saved argmin is f of t[c], for f = `me`; fixed summation order
// (interleaved partial sums).  tb / ib: the t values and argmin indices (stored as floats)
// of all labels of this pixel in shared memory.  One compare-to-flag plus one fused multiply-add
// per label: compare/select instructions issue at half the rate of multiply-adds.
template <int LT>
__device__ __forceinline__ float gather_q(const float* tb, const float* ib, int L, float me) {
  float q0 = 0.f, q1 = 0.f, q2 = 0.f, q3 = 0.f;
  if constexpr (LT > 0) {
    constexpr int NV = (LT + 3) / 4;
    float tv[NV * 4], iv[NV * 4];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const float4 a = reinterpret_cast<const float4*>(tb)[v];
      const float4 b = reinterpret_cast<const float4*>(ib)[v];
      tv[4 * v] = a.x, tv[4 * v + 1] = a.y, tv[4 * v + 2] = a.z, tv[4 * v + 3] = a.w;
      iv[4 * v] = b.x, iv[4 * v + 1] = b.y, iv[4 * v + 2] = b.z, iv[4 * v + 3] = b.w;
    }
    // two labels per packed fma, two alternating accumulator pairs (scalar fmas in the same order
    // were measured slower here: 137 against 131 us per 21-label backward sweep)
#pragma unroll
    for (int c = 0; c + 1 < LT; c += 2) {
      if (c & 2) {
        ffma2(q2, q3, eq_flag(iv[c], me), eq_flag(iv[c + 1], me), tv[c], tv[c + 1], q2, q3);
      } else {
        ffma2(q0, q1, eq_flag(iv[c], me), eq_flag(iv[c + 1], me), tv[c], tv[c + 1], q0, q1);
      }
    }
    if (LT & 1) q0 = fmaf(eq_flag(iv[LT - 1], me), tv[LT - 1], q0);
  } else {
    int c = 0;
    for (; c + 2 < L; c += 3) {
      q0 = fmaf(eq_flag(ib[c], me), tb[c], q0);
      q1 = fmaf(eq_flag(ib[c + 1], me), tb[c + 1], q1);
      q2 = fmaf(eq_flag(ib[c + 2], me), tb[c + 2], q2);
    }
    for (; c < L; ++c) q0 = fmaf(eq_flag(ib[c], me), tb[c], q0);
  }
  return (q0 + q1) + (q2 + q3);
}

// Sum of n consecutive floats (n = LT when known at compile time).
template <int LT>
__device__ __forceinline__ float row_sum(const float* row, int L) {
  float s = 0.f;
  if constexpr (LT > 0) {
#pragma unroll
    for (int c = 0; c < LT; ++c) s += row[c];
  } else {
    for (int c = 0; c < L; ++c) s += row[c];
  }
  return s;
}

}  // namespace mpl
