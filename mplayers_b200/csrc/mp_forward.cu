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
#include <cstdlib>

#include "mp_common.cuh"
#include "mp_minplus.cuh"

namespace mpl {

namespace {

constexpr int kPF = 8;  // pixels staged ahead per chain (power of two)

// UU of one pixel from its ring slot (rows: 0 = U, 1+k = M_k), column `col`, row stride `rs`.
__device__ __forceinline__ float uu_from_ring(const float* slot, int rs, int col, int D, int dir,
                                              int inv, float rho, int agg = 0) {
  if (agg) return fmaf(slot[col] - slot[rs + col], rho, -slot[2 * rs + col]);  // rows: A, M_dir, M_inv
  float s = slot[col];
  for (int k = 0; k < D; ++k) s += slot[(1 + k) * rs + col];
  s -= slot[(1 + dir) * rs + col];
  return fmaf(s, rho, -slot[(1 + inv) * rs + col]);
}

// Sum of 32 values in the order of a shuffle-down tree over a warp (x[i] += x[i + 16], then 8, 4,
// 2, 1; lane 0 holds the total): the order in which the reference's soft kernels reduce a row
// (MPLayers/TRWP_hard_soft/TRWP_soft.cuh:45-71), so sums agree with them bit for bit.
__device__ __forceinline__ float tree32_sum(float (&x)[32]) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1)
#pragma unroll
    for (int i = 0; i < off; ++i) x[i] = __fadd_rn(x[i], x[i + off]);
  return x[0];
}

// Soft (expected-value) step of label c = this thread: val[f] = e*ctx(c,f) + h[f], weights
// softmin_f(val), message = sum_f weight * val (MPLayers/TRWP_hard_soft/TRWP_forward_soft.cu:55-92).
// Same intrinsics and operation order as the reference: __expf(-val + min), (w * val) / sum.
template <int LMAX>
__device__ __forceinline__ float soft_regrow(const float* hb, const float (&cr)[LMAX], float e, int L,
                                             float (&val)[LMAX]) {
  constexpr int NV = (LMAX + 3) / 4;
  float hv[NV * 4];
#pragma unroll
  for (int q = 0; q < NV; ++q) {
    const float4 t = reinterpret_cast<const float4*>(hb)[q];
    hv[4 * q] = t.x, hv[4 * q + 1] = t.y, hv[4 * q + 2] = t.z, hv[4 * q + 3] = t.w;
  }
#pragma unroll
  for (int f = 0; f < LMAX; ++f) val[f] = fmaf(e, cr[f], hv[f]);   // +inf beyond L
  const float m = min_tree<LMAX>(val);
  float ex[32], sf[32];
#pragma unroll
  for (int f = 0; f < 32; ++f) ex[f] = (f < LMAX && f < L) ? __expf(-val[f < LMAX ? f : 0] + m) : 0.f;
#pragma unroll
  for (int f = 0; f < 32; ++f) sf[f] = ex[f];
  const float se = tree32_sum(sf);
  // (w * val) / se for every f with ONE correctly rounded reciprocal: q0 = a*r, q = q0 + (a - se*q0)*r
  // is the correctly rounded quotient (Markstein), i.e. the same bits as the IEEE division the
  // reference performs per element; checked against __fdiv_rn on 3e10 random operand pairs.
  const float rs = __frcp_rn(se);
#pragma unroll
  for (int f = 0; f < 32; ++f) {
    const float a = __fmul_rn(ex[f], val[f < LMAX ? f : 0]);
    const float q0 = __fmul_rn(a, rs);
    sf[f] = (f < LMAX && f < L) ? __fmaf_rn(__fmaf_rn(-se, q0, a), rs, q0) : 0.f;
  }
  return tree32_sum(sf);
}

// ------------------------------------------------------------------------------------------------
// L <= 32: one warp per chain.  DT = compile-time direction count (0: read it from the params).
// ------------------------------------------------------------------------------------------------
// Generic kernel: any direction, any alignment.  Inputs are staged through a ring of 4-byte
// cp.async copies kPF pixels ahead (a register ring of plain loads was measured slower: waiting on
// a register load drains every younger load too, whereas cp.async groups retire in order).
// DT = compile-time direction count (0: read it from the params).
// SOFT: the soft (expected-value) message instead of the minimum; in training it saves the L x L
// edge values of every pixel (entry [f][c] for even directions, [c][f] for odd ones, as the
// reference does, MPLayers/TRWP_hard_soft/TRWP_forward_soft.cu:50-59) and no argmin indices.
// EXACT: the label count equals LMAX (lets the compiler drop every "f < L" test; used by the soft path).
template <int LMAX, int DT, bool TRAIN, bool SOFT = false, bool EXACT = false>
__global__ void __launch_bounds__(128, 1) fwd_warp_kernel(const __grid_constant__ FwdParams p) {
  extern __shared__ __align__(16) float smem[];
  const int wpb = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  ChainCtx ch;
  if (!decode_chain(p, blockIdx.x * wpb + warp, ch)) return;
  const int L = EXACT ? LMAX : p.L, D = p.agg ? 2 : (DT ? DT : p.D), rows = D + 2;  // D = staged message slices
  const int slot_floats = rows * 32;
  float* ring = smem + warp * (kPF * slot_floats + 64 + (SOFT ? 32 * 33 : 0));
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
  uint8_t* MIl = (TRAIN && !SOFT) ? p.min_idx + (long long)ch.dir * p.slice + ibase * L + lc : nullptr;
  uint8_t* NI = TRAIN ? p.norm_idx + (long long)ch.dir * p.pslice + ibase : nullptr;
  float* EL = (TRAIN && SOFT) ? p.edge_label + ((long long)ch.dir * p.pslice + ibase) * L * L : nullptr;
  const bool l2r = (ch.dir & 1) == 0;  // layout of the saved edge values
  // flat element lane + 32k of a pixel's [c][f] table -> its place in the padded shared tile
  constexpr int kFlat = SOFT ? (LMAX * LMAX + 31) / 32 : 1;
  int toff[kFlat];
#pragma unroll
  for (int k = 0; k < kFlat; ++k) {
    const int i = lane + 32 * k, c = i / L;
    toff[k] = c * 33 + (i - c * L);
  }
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
      if (k < D) cp_async4(dst + (1 + k) * 32, Ml + (p.agg ? (k == 0 ? ch.dir : ch.inv) : k) * p.slice + o);
    cp_async4(dst + (D + 1) * 32, E + pxc);
    cp_async_commit();
    px_pf += ch.pstep;
  };
  auto uu_of = [&](const float* sl) {  // sl: this lane's column of a ring slot
    if (p.agg) return fmaf(sl[0] - sl[32], rho, -sl[64]);  // rows: A, M_dir, M_inv
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
    int bi = 0;
    if constexpr (SOFT) {
      float val[LMAX];
      best = soft_regrow<LMAX>(hb, cr, e, L, val);
      if (TRAIN) {
        float* el = EL + (long long)px * L * L;
        if (l2r) {   // entry [f][c]: lanes are consecutive in memory for every f
          if (act) {
#pragma unroll
            for (int f = 0; f < LMAX; ++f)
              if (f < L) el[f * L + lane] = val[f];
          }
        } else {     // entry [c][f]: through a shared-memory tile so that the stores are coalesced
          float* tile = hbuf + 64;   // [L][33], private to the warp
          __syncwarp();
          if (act) {
#pragma unroll
            for (int f = 0; f < LMAX; ++f)
              if (f < L) tile[lane * 33 + f] = val[f];
          }
          __syncwarp();
          const int n2 = L * L;
#pragma unroll
          for (int k = 0; k < kFlat; ++k)
            if (lane + 32 * k < n2) el[lane + 32 * k] = tile[toff[k]];
        }
      }
    } else {
      minplus_regrow<LMAX, TRAIN>(hb, cr, e, best, bi);
    }
    const float m = warp_min(act ? best : kInf);
    r = best - m;
    if (act) Mwl[of] = r;
    if (TRAIN) {
      const unsigned bal = __ballot_sync(0xffffffffu, act && best == m);
      if (!SOFT && act) MIl[of] = (uint8_t)bi;
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
// L <= 32, directions 0..3, 16-byte-aligned rows: bulk-copy (TMA) staged kernel.
//
// A CTA walks four neighbouring chains (four image rows for the horizontal directions, four
// adjacent columns for the vertical ones) with one consumer warp each; a fifth warp is the
// producer.  Per stage of kTK chain pixels the producer issues plain (non-multicast)
// cp.async.bulk copies of whole row segments -- kTK*L floats per array and chain horizontally,
// 4*L floats per array and image row vertically -- into a ring of shared-memory tiles; completion
// is counted in bytes on one mbarrier per stage, and consumers hand a tile back through a second
// mbarrier.  The consumers therefore spend no instruction on global loads or their addresses.
// Every wait is bounded: after about a second it records a code in *status and the warp leaves.
// ------------------------------------------------------------------------------------------------
constexpr int kTK = 16;

// LT = compile-time label count (0: runtime, up to LMAX = 32); FWD = the chain walks towards
// increasing coordinates (directions 0 and 2).
template <int LMAX, int LT, int DT, bool TRAIN, bool VERT, bool FWD>
__global__ void __launch_bounds__(160, 1) fwd_tma_kernel(const __grid_constant__ FwdParams p,
                                                         const __grid_constant__ TmaMaps maps) {
  // No static shared memory in this kernel: the dynamic region starts at the CTA's shared window
  // base, which satisfies the 128-byte alignment the tiled TMA destination needs.  (Rounding the
  // pointer up by hand would hide its address space from the compiler and turn every shared
  // access into a slower generic one.)
  extern __shared__ __align__(128) float smem[];
  constexpr bool AGG = DT == 2;  // aggregate mode (see FwdParams::agg): arrays A, M_dir, M_inv
  constexpr int A = DT + 1;      // staged arrays: unary (or aggregate) + DT message slices
  constexpr int AE = A + 1;   // ... + edge weights
  const int L = LT ? LT : p.L, H = p.H, W = p.W, NS = p.tma_stages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int dir = p.dir0, inv = dir ^ 1;
  const bool has_e = p.ew != nullptr;
  const int len = VERT ? H : W;
  const int nstages = (len + kTK - 1) / kTK;
  const int tile_floats = A * kTK * 4 * L;

  float* tiles = smem;                                   // [NS][tile_floats]
  float* etiles = tiles + NS * tile_floats;              // [NS][64]
  float* hbufs = etiles + NS * 64;                       // [4][64]
  unsigned long long* full = reinterpret_cast<unsigned long long*>(hbufs + 4 * 64);  // [NS]
  unsigned long long* empty = full + NS;                 // [NS]

  // the four chains of this CTA
  int nact, img0 = 0, w0 = 0, chain0 = 0;
  if (VERT) {
    const int gpi = W >> 2;
    img0 = blockIdx.x / gpi;
    w0 = (blockIdx.x - img0 * gpi) << 2;
    nact = 4;
  } else {
    chain0 = blockIdx.x << 2;  // flattened (image, row)
    const int total = p.nimg * H;
    nact = total - chain0 < 4 ? total - chain0 : 4;
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < NS; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], nact);
    }
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == 4) {
    // ---------------------------------- producer ----------------------------------
    const unsigned row_bytes = VERT ? 16u * L : 0u;
    for (int s = 0; s < nstages; ++s) {
      const int slot = s % NS;
      if (s >= NS && !mbar_wait(&empty[slot], ((s / NS) - 1) & 1)) {
        if (lane == 0) atomicExch(p.status, 101);
        break;
      }
      const int npix = len - s * kTK < kTK ? len - s * kTK : kTK;
      float* T = tiles + slot * tile_floats;
      float* ET = etiles + slot * 64;
      if (VERT) {
        // 2-D tiled TMA: one copy per staged array brings kTK image rows of the 4-pixel column
        // group (box 4L x kTK).  Rows outside the tensor read as zero, rows of a neighbouring image
        // are never used; the full box is always transferred.
        if (lane == 0) {
          mbar_arrive_expect_tx(&full[slot], (unsigned)(A * kTK * row_bytes + (has_e ? kTK * 16u : 0u)));
          const int y0 = img0 * H + (FWD ? s * kTK : H - (s + 1) * kTK);
          tma_load_2d(T, &maps.a, w0 * L, y0, &full[slot]);
#pragma unroll
          for (int a = 1; a < A; ++a)
            tma_load_2d(T + a * kTK * 4 * L, &maps.b, w0 * L,
                        (AGG ? (a == 1 ? dir : inv) : a - 1) * p.nimg * H + y0, &full[slot]);
          if (has_e) tma_load_2d(ET, &maps.c, w0, dir * p.nimg * H + y0, &full[slot]);
        }
      } else {
        if (lane == 0)
          mbar_arrive_expect_tx(&full[slot], (unsigned)nact * (unsigned)npix * (A * 4u * L + (has_e ? 4u : 0u)));
        __syncwarp();
        const int ncopy = nact * AE;
        for (int c = lane; c < ncopy; c += 32) {
          const int q = c / AE, a = c - q * AE;
          const int wlo = FWD ? s * kTK : W - s * kTK - npix;
          const long long pix = (long long)(chain0 + q) * W + wlo;  // first pixel, over all images
          if (a < A) {
            const int sid = AGG ? (a == 1 ? dir : inv) : a - 1;
            const float* src = (a == 0 ? p.unary : p.msg_read + (long long)sid * p.slice) + pix * L;
            bulk_g2s(T + (q * A + a) * kTK * L, src, (unsigned)npix * 4u * L, &full[slot]);
          } else if (has_e) {
            bulk_g2s(ET + q * kTK, p.ew + (long long)dir * p.pslice + pix, (unsigned)npix * 4u, &full[slot]);
          }
        }
      }
    }
    return;
  }

  // ---------------------------------- consumers ----------------------------------
  const int wc = warp;
  if (wc >= nact) return;
  const bool act = lane < L;
  // Idle lanes (lane >= L) mirror the last label: same loads, same arithmetic, same `best`, so the
  // warp-wide minimum needs no select; only their stores are masked.
  const int lc = act ? lane : L - 1;
  const unsigned lmask = L >= 32 ? 0xffffffffu : (1u << L) - 1u;
  const float rho = p.rho;
  float cr[LMAX];
#pragma unroll
  for (int f = 0; f < LMAX; ++f) cr[f] = f < L ? ctx_value(p.ctx, p.ctx_rank, L, lc, f) : 0.f;

  int img, fix;  // fix = the coordinate that stays constant along the chain
  if (VERT) {
    img = img0;
    fix = w0 + wc;
  } else {
    img = (chain0 + wc) / H;
    fix = (chain0 + wc) - img * H;
  }
  const long long ibase = (long long)img * H * W;
  float* Mwl = p.msg_write + (long long)dir * p.slice + ibase * L + lc;
  uint8_t* MIl = TRAIN ? p.min_idx + (long long)dir * p.slice + ibase * L + lc : nullptr;
  uint8_t* NI = TRAIN ? p.norm_idx + (long long)dir * p.pslice + ibase : nullptr;
  float* hbuf = hbufs + wc * 64;
  for (int i = lane; i < 64; i += 32) hbuf[i] = kInf;  // labels >= L (LMAX > L) never win
  if (!has_e)  // no edge weights: the producer copies none, every staged weight reads as 1
    for (int i = lane; i < NS * 64; i += 32) etiles[i] = 1.f;
  __syncwarp();
  const int sa = VERT ? kTK * 4 * L : kTK * L;        // stride between staged arrays
  const int sk = (VERT ? 4 * L : L) * (FWD ? 1 : -1);  // stride between consecutive chain pixels
  const int ek = (VERT ? 4 : 1) * (FWD ? 1 : -1);
  const int pstep = VERT ? (FWD ? W : -W) : (FWD ? 1 : -1);
  const int px0 = VERT ? (FWD ? 0 : H - 1) * W + fix : fix * W + (FWD ? 0 : W - 1);  // chain pixel 0
  const int dir_off = (AGG ? 1 : 1 + dir) * sa, inv_off = (AGG ? 2 : 1 + inv) * sa;

  float uu = 0.f, r = 0.f;
  // inputs of one chain pixel -> UU of that pixel (reference order of the additions)
  auto uu_at = [&](const float* t) {
    float sum = t[0];
    if (!AGG) {
#pragma unroll
      for (int a = 1; a <= DT; ++a) sum += t[a * sa];
    }
    sum -= t[dir_off];
    return fmaf(sum, rho, -t[inv_off]);
  };
  // Output rows of the current chain pixel, moved by one pixel per step (running pointers: one
  // 64-bit add each instead of an index multiplication and a widening add per store).
  const long long ostep = (long long)pstep * L;
  float* mw = Mwl + (long long)px0 * L;
  uint8_t* mip = TRAIN ? MIl + (long long)px0 * L : nullptr;
  uint8_t* nip = TRAIN ? NI + px0 : nullptr;
  // message of the current chain pixel from its predecessor's UU (in `uu`) and running message `r`
  auto step = [&](const float* t, float e, int par) {
    const float uu_next = uu_at(t);
    float* hb = hbuf + par * 32;
    if (LT == 0 || LMAX != LT) {
      if (act) hb[lane] = fmaf(rho, r, uu);
    } else {
      hb[lane] = fmaf(rho, r, uu);  // entries >= L are written but never read
    }
    __syncwarp();
    // The warp-wide minimum is issued as soon as the lane's own minimum is known: its latency
    // runs behind the argmin flags, which need only the lane's candidates.
    float val[LMAX];
    minplus_vals<LMAX>(hb, cr, e, val);
    const float best = min_tree<LMAX>(val);
    const float m = warp_min(best);
    int bi = 0;
    if (TRAIN) bi = highest_equal<LMAX>(val, best);
    r = best - m;
    // Unpredicated stores: idle lanes hold the same values as lane L-1 and write the same
    // address, and the normalisation index is warp-uniform.
    *mw = r;
    if (TRAIN) {
      const unsigned bal = __ballot_sync(0xffffffffu, best == m) & lmask;
      *mip = (uint8_t)bi;
      *nip = (uint8_t)(31 - __clz(bal));
    }
    uu = uu_next;
  };
  auto advance = [&]() {
    mw += ostep;
    if (TRAIN) {
      mip += ostep;
      nip += pstep;
    }
  };

  for (int s = 0; s < nstages; ++s) {
    const int slot = s % NS;
    if (!mbar_wait(&full[slot], (s / NS) & 1)) {
      if (lane == 0) atomicExch(p.status, 102);
      return;
    }
    const int npix = len - s * kTK < kTK ? len - s * kTK : kTK;
    const float* T = tiles + slot * tile_floats + lc;
    const float* ET = etiles + slot * 64;
    const float* t0;
    const float* e0;
    if (VERT) {  // box rows ascend in memory; a downward walk starts at the last row of the box
      t0 = T + wc * L + (FWD ? 0 : (kTK - 1) * 4 * L);
      e0 = ET + wc + (FWD ? 0 : (kTK - 1) * 4);
    } else {
      t0 = T + wc * A * kTK * L + (FWD ? 0 : (npix - 1) * L);
      e0 = ET + wc * kTK + (FWD ? 0 : npix - 1);
    }
    if (s > 0 && npix == kTK) {
      // full stage: fully unrolled, every tile offset is an immediate
#pragma unroll
      for (int k = 0; k < kTK; ++k) {
        step(t0 + k * sk, e0[k * ek], k & 1);
        advance();
      }
    } else {
      for (int k = 0; k < npix; ++k) {
        if (s + k == 0) {
          uu = uu_at(t0);  // chain pixel 0 only provides the inputs of pixel 1
        } else {
          step(t0 + k * sk, e0[k * ek], k & 1);
        }
        advance();
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[slot]);
  }
}

// ------------------------------------------------------------------------------------------------
// L > 32: one CTA per chain, thread = label.
// ------------------------------------------------------------------------------------------------
// Barrier over the whole CTA (nthreads == 0) or over its first `nthreads` threads (named barrier
// 1; used where a producer warp of the same CTA must not take part).
__device__ __forceinline__ void cta_sync(int nthreads) {
  if (nthreads == 0) {
    __syncthreads();
  } else {
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
  }
}

// Block-wide min with the index of the HIGHEST thread attaining it.  One barrier inside.
__device__ __forceinline__ void block_min_hi(float v, bool act, int tid, float* red_v, int* red_i,
                                             int nw, float& m, int& n, int bar_threads = 0) {
  const float x = act ? v : kInf;
  const float wm = warp_min(x);
  const unsigned bal = __ballot_sync(0xffffffffu, act && x == wm);
  if ((tid & 31) == 0) {
    red_v[tid >> 5] = wm;
    red_i[tid >> 5] = bal ? (tid & ~31) + 31 - __clz(bal) : -1;
  }
  cta_sync(bar_threads);
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

// State of the label-context evaluation of one CTA-per-chain kernel instance.
template <int MODE>
struct CtaCtx {
  bool windowed;
  int R;
  float cmax;
  float cr[MODE == 2 ? 64 : 1];
};

// One chain step of the CTA-per-chain kernels: publishes h, evaluates best[c] = min_f (h[f] +
// e*ctx(c,f)) with its argmin, and the block-wide normalisation minimum m with its index n.
// Two block barriers.
template <int MODE, bool TRAIN>
__device__ __forceinline__ void cta_minplus(const FwdParams& p, const CtaCtx<MODE>& cc, float h, float e,
                                            bool act, int c, int L, int nw, float* hbuf, const float* ctx1,
                                            float* redA_v, int* redA_i, float* redB_v, int* redB_i,
                                            float& best, int& bi, float& m, int& n, int bar_threads = 0) {
  if (act) hbuf[c] = h;
  best = kInf;
  bi = 0;
  if (MODE == 1 && cc.windowed) {
    const int R = cc.R;
    float hmin;
    int fstar;
    block_min_hi(h, act, c, redA_v, redA_i, nw, hmin, fstar, bar_threads);  // also publishes hbuf
    const float gv = fmaf(e, cc.cmax, hmin);
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
    cta_sync(bar_threads);
    if constexpr (MODE == 2) {
      minplus_regrow<64, TRAIN>(hbuf, cc.cr, e, best, bi);
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
  block_min_hi(best, act, c, redB_v, redB_i, nw, m, n, bar_threads);
}

template <int MODE>
__device__ __forceinline__ void cta_ctx_init(const FwdParams& p, CtaCtx<MODE>& cc, bool act, int c, int L,
                                             float* ctx1) {
  cc.windowed = false;
  cc.R = 0;
  cc.cmax = 0.f;
  if (MODE == 1) {
    ctx1[c] = act ? __ldg(p.ctx + c) : 0.f;
    const CtxInfo inf = *p.info;
    cc.windowed = inf.windowed && (p.ew == nullptr || float_from_order_bits(inf.ew_min_bits) >= 0.f);
    cc.R = inf.R;
    cc.cmax = inf.cmax;
  }
  if constexpr (MODE == 2) {
#pragma unroll
    for (int f = 0; f < 64; ++f) cc.cr[f] = (act && f < L) ? ctx_value(p.ctx, 2, L, c, f) : 0.f;
  }
}

template <int MODE, bool TRAIN>
__global__ void __launch_bounds__(256) fwd_cta_kernel(const __grid_constant__ FwdParams p) {
  extern __shared__ __align__(16) float smem[];
  ChainCtx ch;
  if (!decode_chain(p, blockIdx.x, ch)) return;  // uniform for the CTA
  const int L = p.L, D = p.agg ? 2 : p.D, rows = D + 2, NT = blockDim.x, c = threadIdx.x, nw = NT >> 5;
  float* ring = smem;                  // [kPF][rows][NT]
  float* hbuf = ring + kPF * rows * NT;  // [NT]
  float* ctx1 = hbuf + NT;             // [NT]   (MODE 1)
  float* redA_v = ctx1 + NT;           // [8]
  int* redA_i = reinterpret_cast<int*>(redA_v + 8);
  float* redB_v = redA_v + 16;
  int* redB_i = reinterpret_cast<int*>(redB_v + 8);
  const bool act = c < L;
  CtaCtx<MODE> cc;
  cta_ctx_init<MODE>(p, cc, act, c, L, ctx1);
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
        for (int k = 0; k < D; ++k)
          cp_async4(dst + (1 + k) * NT,
                    Mr + (p.agg ? (k == 0 ? ch.dir : ch.inv) : k) * p.slice + (long long)px * L + c);
      }
      if (E && j >= 1) cp_async4(dst + (D + 1) * NT, E + px);
    }
    cp_async_commit();
  };

#pragma unroll
  for (int j = 0; j < kPF; ++j) issue(j);
  cp_async_wait<kPF - 1>();
  float uu = act ? uu_from_ring(ring, NT, c, D, ch.dir, ch.inv, p.rho, p.agg) : 0.f;
  issue(kPF);
  float r = 0.f;

  for (int i = 1; i < len; ++i) {
    cp_async_wait<kPF - 1>();
    const float* slot = ring + (i & (kPF - 1)) * rows * NT;
    const float e = E ? slot[(D + 1) * NT + c] : 1.f;
    const float uu_next = (act && i < len - 1) ? uu_from_ring(slot, NT, c, D, ch.dir, ch.inv, p.rho, p.agg) : 0.f;
    const float h = act ? fmaf(p.rho, r, uu) : kInf;
    float best, m;
    int bi, n;
    cta_minplus<MODE, TRAIN>(p, cc, h, e, act, c, L, nw, hbuf, ctx1, redA_v, redA_i, redB_v, redB_i, best, bi, m, n);
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

// CTA-per-chain kernel with bulk-copy staging, for L % 4 == 0 (every pixel's label row is then
// 16-byte aligned, in any direction).  The last warp of the CTA is the producer: per stage of K
// chain pixels it issues, for each of the D+1 input arrays, either one cp.async.bulk of K*L floats
// (horizontal chains are contiguous) or K copies of one label row each (all other directions);
// completion on an mbarrier per stage, bounded waits.  Edge weights are fetched one stage ahead by
// the first K consumer threads and published through shared memory.
template <int MODE, bool TRAIN>
__global__ void __launch_bounds__(288) fwd_cta_tma_kernel(const __grid_constant__ FwdParams p) {
  extern __shared__ __align__(128) float smem[];
  ChainCtx ch;
  if (!decode_chain(p, blockIdx.x, ch)) return;  // uniform for the CTA
  const int L = p.L, D = p.agg ? 2 : p.D, A = D + 1, K = p.tma_k, NS = p.tma_stages;
  const int NT = blockDim.x - 32, c = threadIdx.x, nw = NT >> 5;
  const bool producer = c >= NT;
  const int tile_floats = A * K * L;
  float* tiles = smem;                        // [NS][A][K][L]
  float* etile = tiles + NS * tile_floats;    // [2][K]
  float* hbuf = etile + 2 * K;                // [NT]
  float* ctx1 = hbuf + NT;                    // [NT]
  float* redA_v = ctx1 + NT;                  // [8] + [8] + [8] + [8]
  int* redA_i = reinterpret_cast<int*>(redA_v + 8);
  float* redB_v = redA_v + 16;
  int* redB_i = reinterpret_cast<int*>(redB_v + 8);
  unsigned long long* full = reinterpret_cast<unsigned long long*>(redA_v + 32);  // [NS]
  unsigned long long* empty = full + NS;                                          // [NS]
  const bool act = c < L;

  const int len = ch.len;
  const int nstages = (len + K - 1) / K;
  const long long ibase = (long long)ch.img * p.H * p.W;
  const int pix0 = ch.h0 * p.W + ch.w0;
  const bool contiguous = (ch.pstep == 1 || ch.pstep == -1);

  if (c == 0) {
    for (int i = 0; i < NS; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_fence_init();
  }
  CtaCtx<MODE> cc;
  if (!producer) {
    cta_ctx_init<MODE>(p, cc, act, c, L, ctx1);
    hbuf[c] = kInf;  // entries >= L stay +inf
  }
  __syncthreads();

  if (producer) {
    const int lane = c - NT;
    const float* U = p.unary + ibase * L;
    const float* Mr = p.msg_read + ibase * L;
    for (int s = 0; s < nstages; ++s) {
      const int slot = s % NS;
      if (s >= NS && !mbar_wait(&empty[slot], ((s / NS) - 1) & 1)) {
        if (lane == 0) atomicExch(p.status, 111);
        break;
      }
      const int np = len - s * K < K ? len - s * K : K;
      float* T = tiles + slot * tile_floats;
      if (lane == 0) mbar_arrive_expect_tx(&full[slot], (unsigned)(np * A * L) * 4u);
      __syncwarp();
      if (contiguous) {
        // pixels s*K .. s*K+np-1 are adjacent in memory (ascending for pstep=1, descending for -1)
        const int first = ch.pstep == 1 ? pix0 + s * K : pix0 - (s * K + np - 1);
        if (lane < A) {
          const int sid = p.agg ? (lane == 1 ? ch.dir : ch.inv) : lane - 1;
          const float* src = (lane == 0 ? U : Mr + (long long)sid * p.slice) + (long long)first * L;
          bulk_g2s(T + lane * K * L, src, (unsigned)(np * L) * 4u, &full[slot]);
        }
      } else {
        for (int q = lane; q < np * A; q += 32) {
          const int k = q / A, a = q - k * A;
          const int px = pix0 + (s * K + k) * ch.pstep;
          const int sid = p.agg ? (a == 1 ? ch.dir : ch.inv) : a - 1;
          const float* src = (a == 0 ? U : Mr + (long long)sid * p.slice) + (long long)px * L;
          bulk_g2s(T + (a * K + k) * L, src, (unsigned)L * 4u, &full[slot]);
        }
      }
    }
    return;
  }

  // ---------------------------------- consumers ----------------------------------
  float* Mw = p.msg_write + (long long)ch.dir * p.slice + ibase * L;
  const float* E = p.ew ? p.ew + (long long)ch.dir * p.pslice + ibase : nullptr;
  uint8_t* MI = TRAIN ? p.min_idx + (long long)ch.dir * p.slice + ibase * L : nullptr;
  uint8_t* NI = TRAIN ? p.norm_idx + (long long)ch.dir * p.pslice + ibase : nullptr;
  const int dir_off = (p.agg ? 1 : 1 + ch.dir) * K * L, inv_off = (p.agg ? 2 : 1 + ch.inv) * K * L;
  auto load_e = [&](int s) -> float {  // thread k < K: weight of chain pixel s*K + k
    const int j = s * K + c;
    return (E && c < K && j < len && j >= 1) ? E[pix0 + j * ch.pstep] : 1.f;
  };
  if (c < K) etile[c] = load_e(0);
  float e_next = load_e(1);
  float uu = 0.f, r = 0.f;
  for (int s = 0; s < nstages; ++s) {
    const int slot = s % NS;
    if (!mbar_wait(&full[slot], (s / NS) & 1)) {
      if (c == 0) atomicExch(p.status, 112);
      return;
    }
    const int np = len - s * K < K ? len - s * K : K;
    const float* T = tiles + slot * tile_floats;
    const float* et = etile + (s & 1) * K;
    // position of chain pixel s*K + k inside the tile
    const int kbase = (contiguous && ch.pstep == -1) ? np - 1 : 0;
    const int kstep = (contiguous && ch.pstep == -1) ? -1 : 1;
    cta_sync(NT);  // the weights of this stage (written at the end of the previous one) are visible
    for (int k = 0; k < np; ++k) {
      const float* t = T + (kbase + k * kstep) * L + c;
      float uu_next = 0.f;
      if (act) {
        float sum = t[0];
        if (!p.agg)
          for (int a = 1; a <= D; ++a) sum += t[a * K * L];
        sum -= t[dir_off];
        uu_next = fmaf(sum, p.rho, -t[inv_off]);
      }
      if (s + k > 0) {
        const float e = et[k];
        const float h = act ? fmaf(p.rho, r, uu) : kInf;
        float best, m;
        int bi, n;
        cta_minplus<MODE, TRAIN>(p, cc, h, e, act, c, L, nw, hbuf, ctx1, redA_v, redA_i, redB_v, redB_i, best, bi,
                                 m, n, NT);
        r = best - m;
        const int px = pix0 + (s * K + k) * ch.pstep;
        if (act) Mw[(long long)px * L + c] = r;
        if (TRAIN) {
          if (act) MI[(long long)px * L + c] = (uint8_t)bi;
          if (c == 0) NI[px] = (uint8_t)n;
        }
      }
      uu = uu_next;
    }
    if (c < K) etile[((s + 1) & 1) * K + c] = e_next;
    e_next = load_e(s + 2);
    cta_sync(NT);  // every consumer is done with the tile
    if (c == 0) mbar_arrive(&empty[slot]);
  }
}

// ------------------------------------------------------------------------------------------------
// 32 < L <= 64, rank-2 (dense) context, L % 4 == 0: one WARP per chain, TWO labels per lane, both
// context rows of the lane in registers.  No block barrier (the CTA-per-chain kernel needs two per
// step and two warps per chain).  Every warp stages its own inputs: lane-parallel cp.async.bulk
// copies (one per array and stage for horizontal chains, one label row per pixel otherwise) into a
// private ring, completion on the warp's own mbarriers, refilled by the warp itself as soon as it
// has consumed a stage (no producer warp: it would hold as many registers as a consumer).
// ------------------------------------------------------------------------------------------------
constexpr int kPairWarps = 4;  // chains per CTA

template <bool TRAIN>
__global__ void __launch_bounds__(kPairWarps * 32, 1) fwd_pair_kernel(const __grid_constant__ FwdParams p) {
  extern __shared__ __align__(128) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int L = p.L, D = p.agg ? 2 : p.D, A = D + 1, K = p.tma_k, NS = p.tma_stages;
  const int tile_floats = A * K * L;
  const int per_warp = NS * tile_floats + 2 * 64 + 2 * K + 2 * NS + 2;  // floats (barriers are 2 each)
  float* wbase = smem + warp * ((per_warp + 3) & ~3);
  float* tiles = wbase;                               // [NS][A][K][L]
  float* hbuf = tiles + NS * tile_floats;             // [2][64]
  float* etile = hbuf + 128;                          // [2][K]
  unsigned long long* full = reinterpret_cast<unsigned long long*>(etile + 2 * K + ((2 * K) & 1));
  if (lane == 0)
    for (int i = 0; i < NS; ++i) mbar_init(&full[i], 1);
  hbuf[lane] = kInf, hbuf[32 + lane] = kInf, hbuf[64 + lane] = kInf, hbuf[96 + lane] = kInf;
  if (lane == 0) mbar_fence_init();
  __syncwarp();
  ChainCtx ch;
  if (!decode_chain(p, blockIdx.x * kPairWarps + warp, ch)) return;

  const int len = ch.len;
  const int nstages = (len + K - 1) / K;
  const long long ibase = (long long)ch.img * p.H * p.W;
  const int pix0 = ch.h0 * p.W + ch.w0;
  const bool contiguous = (ch.pstep == 1 || ch.pstep == -1);
  const float* U = p.unary + ibase * L;
  const float* Mr = p.msg_read + ibase * L;

  auto issue_stage = [&](int s) {  // copies of stage s into slot s % NS (all lanes call)
    if (s >= nstages) return;
    const int slot = s % NS;
    const int np = len - s * K < K ? len - s * K : K;
    float* T = tiles + slot * tile_floats;
    if (lane == 0) {
      fence_proxy_async_smem();
      mbar_arrive_expect_tx(&full[slot], (unsigned)(np * A * L) * 4u);
    }
    __syncwarp();
    if (contiguous) {
      const int first = ch.pstep == 1 ? pix0 + s * K : pix0 - (s * K + np - 1);
      if (lane < A) {
        const int sid = p.agg ? (lane == 1 ? ch.dir : ch.inv) : lane - 1;
        const float* src = (lane == 0 ? U : Mr + (long long)sid * p.slice) + (long long)first * L;
        bulk_g2s(T + lane * K * L, src, (unsigned)(np * L) * 4u, &full[slot]);
      }
    } else {
      for (int q = lane; q < np * A; q += 32) {
        const int k = q / A, a = q - k * A;
        const int px = pix0 + (s * K + k) * ch.pstep;
        const int sid = p.agg ? (a == 1 ? ch.dir : ch.inv) : a - 1;
        const float* src = (a == 0 ? U : Mr + (long long)sid * p.slice) + (long long)px * L;
        bulk_g2s(T + (a * K + k) * L, src, (unsigned)L * 4u, &full[slot]);
      }
    }
  };

  const int c0 = 2 * lane;          // labels c0, c0 + 1 (L is a multiple of four: both or none exist)
  const bool act = c0 < L;
  const int lc0 = act ? c0 : L - 2;  // idle lanes shadow the last pair: loads need no predicate
  float cr0[64], cr1[64];
#pragma unroll
  for (int f = 0; f < 64; ++f) {
    cr0[f] = (act && f < L) ? ctx_value(p.ctx, p.ctx_rank, L, c0, f) : 0.f;
    cr1[f] = (act && f < L) ? ctx_value(p.ctx, p.ctx_rank, L, c0 + 1, f) : 0.f;
  }
  float* Mw = p.msg_write + (long long)ch.dir * p.slice + ibase * L + c0;
  const float* E = p.ew ? p.ew + (long long)ch.dir * p.pslice + ibase : nullptr;
  uint8_t* MI = TRAIN ? p.min_idx + (long long)ch.dir * p.slice + ibase * L + c0 : nullptr;
  uint8_t* NI = TRAIN ? p.norm_idx + (long long)ch.dir * p.pslice + ibase : nullptr;
  const int dir_off = (p.agg ? 1 : 1 + ch.dir) * K * L, inv_off = (p.agg ? 2 : 1 + ch.inv) * K * L;
  const float rho = p.rho;
  auto load_e = [&](int s) -> float {  // lane k < K: weight of chain pixel s*K + k
    const int j = s * K + lane;
    return (E && lane < K && j < len && j >= 1) ? E[pix0 + j * ch.pstep] : 1.f;
  };
  // The 64 candidates are evaluated as two halves of 32 (the second wins ties: highest index), so
  // that only 32 sums are alive next to the 128 context registers.
  auto eval_label = [&](const float* hb, const float (&cr)[64], float e, float& best, int& bi) {
    float ba, bb;
    int ia, ib;
    minplus_regrow<32, TRAIN, 64, 0>(hb, cr, e, ba, ia);
    minplus_regrow<32, TRAIN, 64, 32>(hb + 32, cr, e, bb, ib);
    best = fminf(ba, bb);
    bi = bb <= ba ? ib + 32 : ia;
  };

  for (int s = 0; s < NS; ++s) issue_stage(s);
  if (lane < K) etile[lane] = load_e(0);
  float e_next = load_e(1);
  float uu0 = 0.f, uu1 = 0.f, r0 = 0.f, r1 = 0.f;
  int po = pix0 * L;             // element offset of the current pixel's label row
  const int postep = ch.pstep * L;
  int px = pix0;
  for (int s = 0; s < nstages; ++s) {
    const int slot = s % NS;
    if (!mbar_wait(&full[slot], (s / NS) & 1)) {
      if (lane == 0) atomicExch(p.status, 131);
      return;
    }
    const int np = len - s * K < K ? len - s * K : K;
    const float* T = tiles + slot * tile_floats + lc0;
    const float* et = etile + (s & 1) * K;
    const bool flip = contiguous && ch.pstep == -1;
    __syncwarp();
    for (int k = 0; k < np; ++k) {
      const float* t = T + (flip ? np - 1 - k : k) * L;
      float2 v = *reinterpret_cast<const float2*>(t);
      if (!p.agg)
        for (int a = 1; a <= D; ++a) {
          const float2 x = *reinterpret_cast<const float2*>(t + a * K * L);
          v.x += x.x, v.y += x.y;
        }
      const float2 md = *reinterpret_cast<const float2*>(t + dir_off);
      const float2 mi = *reinterpret_cast<const float2*>(t + inv_off);
      const float un0 = fmaf(v.x - md.x, rho, -mi.x);
      const float un1 = fmaf(v.y - md.y, rho, -mi.y);
      if (s + k > 0) {
        const float e = et[k];
        float* hb = hbuf + ((s * K + k) & 1) * 64;
        if (act) *reinterpret_cast<float2*>(hb + c0) = make_float2(fmaf(rho, r0, uu0), fmaf(rho, r1, uu1));
        __syncwarp();
        float b0, b1;
        int i0, i1;
        eval_label(hb, cr0, e, b0, i0);
        eval_label(hb, cr1, e, b1, i1);
        const float x0 = act ? b0 : kInf, x1 = act ? b1 : kInf;
        const float m = warp_min(fminf(x0, x1));
        r0 = b0 - m;
        r1 = b1 - m;
        if (act) *reinterpret_cast<float2*>(Mw + po) = make_float2(r0, r1);
        if (TRAIN) {
          const unsigned bal0 = __ballot_sync(0xffffffffu, x0 == m);
          const unsigned bal1 = __ballot_sync(0xffffffffu, x1 == m);
          const int n0 = 2 * (31 - __clz(bal0));      // -2 when no even label attains the minimum
          const int n1 = 2 * (31 - __clz(bal1)) + 1;  // -1 when no odd label does
          if (act) *reinterpret_cast<uchar2*>(MI + po) = make_uchar2((unsigned char)i0, (unsigned char)i1);
          if (lane == 0) NI[px] = (uint8_t)(n0 > n1 ? n0 : n1);
        }
      }
      uu0 = un0;
      uu1 = un1;
      po += postep;
      px += ch.pstep;
    }
    if (lane < K) etile[((s + 1) & 1) * K + lane] = e_next;
    e_next = load_e(s + 2);
    __syncwarp();
    issue_stage(s + NS);  // this warp refills the slot it has just consumed
  }
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

// The same with 16-byte accesses (n, slice multiples of 4, pointers 16-byte aligned); every
// component is summed in the same order as above.
__global__ void __launch_bounds__(256)
aggregate_vec4_kernel(const float4* __restrict__ unary, const float4* __restrict__ msg, float4* __restrict__ cost,
                      long long n4, int D, long long slice4, float factor, int min_a_dir) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 u = unary[i];
    float4 v = make_float4(u.x * factor, u.y * factor, u.z * factor, u.w * factor);
    if (min_a_dir) {
      float4 mm = msg[i];
      for (int k = 1; k < D; ++k) {
        const float4 x = msg[k * slice4 + i];
        if (x.x < mm.x) mm.x = x.x;
        if (x.y < mm.y) mm.y = x.y;
        if (x.z < mm.z) mm.z = x.z;
        if (x.w < mm.w) mm.w = x.w;
      }
      v.x += mm.x, v.y += mm.y, v.z += mm.z, v.w += mm.w;
    } else {
      for (int k = 0; k < D; ++k) {
        const float4 x = msg[k * slice4 + i];
        v.x += x.x, v.y += x.y, v.z += x.z, v.w += x.w;
      }
    }
    cost[i] = v;
  }
}

// The same sums written with the labels FIRST ([nimg, L, H*W] planes, the layout the reference's
// module hands back after its permute, pytorch/MP_module.py:232): one block per 32 pixels of an
// image, through a shared-memory tile so that both sides are coalesced.
__global__ void __launch_bounds__(256)
aggregate_lhw_kernel(const float* __restrict__ unary, const float* __restrict__ msg, float* __restrict__ cost,
                     int L, long long HW, int D, long long slice, float factor, int min_a_dir) {
  extern __shared__ float tile[];  // [L][33]
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long long b = blockIdx.y, p0 = blockIdx.x * 32ll;
  const int np = HW - p0 < 32 ? (int)(HW - p0) : 32;
  const long long base = (b * HW + p0) * L;
  for (int i = threadIdx.x; i < np * L; i += 256) {
    float v = unary[base + i] * factor;
    if (min_a_dir) {
      float mm = msg[base + i];
      for (int k = 1; k < D; ++k) {
        const float x = msg[k * slice + base + i];
        if (x < mm) mm = x;
      }
      v += mm;
    } else {
      for (int k = 0; k < D; ++k) v += msg[k * slice + base + i];
    }
    const int px = i / L, l = i - px * L;
    tile[l * 33 + px] = v;
  }
  __syncthreads();
  float* dst = cost + b * L * HW + p0;
  for (int l = ty; l < L; l += 8)
    if (tx < np) dst[(long long)l * HW + tx] = tile[l * 33 + tx];
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
  const size_t smem = (size_t)wpb * (kPF * ((p.agg ? 2 : p.D) + 2) * 32 + 64) * sizeof(float);
  cudaError_t e = ensure_smem(fwd_warp_kernel<LMAX, DT, TRAIN>, smem);
  if (e != cudaSuccess) return e;
  ProfScope prof(kProfFwdSweep, st);
  fwd_warp_kernel<LMAX, DT, TRAIN><<<(total + wpb - 1) / wpb, wpb * 32, smem, st>>>(p);
  count_launch();
  return cudaGetLastError();
}

template <int LMAX, bool TRAIN>
cudaError_t launch_warp(const FwdParams& p, cudaStream_t st) {
  if (p.agg) return launch_warp_d<LMAX, 0, TRAIN>(p, st);
  if (p.D == 4) return launch_warp_d<LMAX, 4, TRAIN>(p, st);
  if (p.D == 8) return launch_warp_d<LMAX, 8, TRAIN>(p, st);
  return launch_warp_d<LMAX, 0, TRAIN>(p, st);
}

template <int LMAX, bool TRAIN, bool EXACT>
cudaError_t launch_warp_soft(const FwdParams& p, cudaStream_t st) {
  const int total = p.chain_off[p.ndirs];
  const int wpb = total >= 148 * 32 ? 4 : 1;
  const size_t smem = (size_t)wpb * (kPF * (p.D + 2) * 32 + 64 + 32 * 33) * sizeof(float);
  cudaError_t e = ensure_smem(fwd_warp_kernel<LMAX, 0, TRAIN, true, EXACT>, smem);
  if (e != cudaSuccess) return e;
  ProfScope prof(kProfFwdSweep, st);
  fwd_warp_kernel<LMAX, 0, TRAIN, true, EXACT><<<(total + wpb - 1) / wpb, wpb * 32, smem, st>>>(p);
  count_launch();
  return cudaGetLastError();
}

size_t tma_smem_bytes(int L, int D, int stages) {
  return ((size_t)stages * ((size_t)(D + 1) * kTK * 4 * L + 64) + 4 * 64) * sizeof(float) + 2 * stages * 8 + 16 + 128;
}

// Can direction `dir` of this problem use the bulk-copy kernel?  Needs 16-byte aligned row segments.
bool tma_eligible(const FwdParams& p, int dir, int* stages) {
  if (dir > 3 || p.L > 32 || (!p.agg && p.D != 4 && p.D != 8)) return false;
  if ((p.W & 3) || (((long long)p.W * p.L) & 3)) return false;
  const uintptr_t bits = (uintptr_t)p.unary | (uintptr_t)p.msg_read | (uintptr_t)p.ew;
  if (bits & 15) return false;
  int ns = tma_stage_override() ? tma_stage_override() : 4;
  while (ns >= 2 && tma_smem_bytes(p.L, p.agg ? 2 : p.D, ns) > (ns >= 3 ? 110 : 200) * 1024) --ns;
  if (ns < 2) return false;
  *stages = ns;
  return true;
}

template <int LMAX, int LT, int DT, bool TRAIN, bool VERT, bool FWD>
cudaError_t launch_tma_v(FwdParams p, int dir, int stages, cudaStream_t st) {
  p.dir0 = dir;
  p.ndirs = 1;
  p.tma_stages = stages;
  const int groups = VERT ? p.nimg * (p.W >> 2) : (p.nimg * p.H + 3) >> 2;
  const size_t smem = tma_smem_bytes(p.L, DT, stages);
  cudaError_t e = ensure_smem(fwd_tma_kernel<LMAX, LT, DT, TRAIN, VERT, FWD>, smem);
  if (e != cudaSuccess) return e;
  TmaMaps maps{};
  if (VERT) {
    const unsigned long long inner = (unsigned long long)p.W * p.L, rows = (unsigned long long)p.nimg * p.H;
    bool ok = encode_tmap_2d(&maps.a, p.unary, inner, rows, 4 * p.L, kTK) &&
              encode_tmap_2d(&maps.b, p.msg_read, inner, rows * p.D, 4 * p.L, kTK);
    if (ok && p.ew) ok = encode_tmap_2d(&maps.c, p.ew, (unsigned long long)p.W, rows * p.D, 4, kTK);
    if (!ok) return cudaErrorNotSupported;
  }
  ProfScope prof(kProfFwdSweep, st);
  fwd_tma_kernel<LMAX, LT, DT, TRAIN, VERT, FWD><<<groups, 160, smem, st>>>(p, maps);
  count_launch();
  return cudaGetLastError();
}

template <int LMAX, int LT, int DT, bool TRAIN>
cudaError_t launch_tma_d(const FwdParams& p, int dir, int stages, cudaStream_t st) {
  switch (dir) {
    case 0: return launch_tma_v<LMAX, LT, DT, TRAIN, false, true>(p, dir, stages, st);
    case 1: return launch_tma_v<LMAX, LT, DT, TRAIN, false, false>(p, dir, stages, st);
    case 2: return launch_tma_v<LMAX, LT, DT, TRAIN, true, true>(p, dir, stages, st);
    default: return launch_tma_v<LMAX, LT, DT, TRAIN, true, false>(p, dir, stages, st);
  }
}

template <int LMAX, int LT, bool TRAIN>
cudaError_t launch_tma(const FwdParams& p, int dir, int stages, cudaStream_t st) {
  if (p.agg) return launch_tma_d<LMAX, LT, 2, TRAIN>(p, dir, stages, st);
  if (p.D == 4) return launch_tma_d<LMAX, LT, 4, TRAIN>(p, dir, stages, st);
  return launch_tma_d<LMAX, LT, 8, TRAIN>(p, dir, stages, st);
}

template <int MODE, bool TRAIN>
cudaError_t launch_cta(const FwdParams& p, cudaStream_t st) {
  const int total = p.chain_off[p.ndirs];
  const int NT = MODE == 2 ? 64 : ((p.L + 31) / 32) * 32;
  const size_t smem = ((size_t)kPF * ((p.agg ? 2 : p.D) + 2) * NT + 2 * NT + 32) * sizeof(float);
  cudaError_t e = ensure_smem(fwd_cta_kernel<MODE, TRAIN>, smem);
  if (e != cudaSuccess) return e;
  ProfScope prof(kProfFwdSweep, st);
  fwd_cta_kernel<MODE, TRAIN><<<total, NT, smem, st>>>(p);
  count_launch();
  return cudaGetLastError();
}

template <int MODE, bool TRAIN>
cudaError_t launch_cta_tma(FwdParams p, cudaStream_t st) {
  const int total = p.chain_off[p.ndirs];
  const int NT = MODE == 2 ? 64 : ((p.L + 31) / 32) * 32;
  const int A = (p.agg ? 2 : p.D) + 1;
  int K = 16, NS = 3;
  auto bytes = [&](int k, int ns) {
    return ((size_t)ns * A * k * p.L + 2 * k + 2 * NT + 32) * sizeof(float) + 2 * ns * 8 + 16;
  };
  while (K > 4 && bytes(K, NS) > 100 * 1024) K >>= 1;
  if (bytes(K, NS) > 100 * 1024) NS = 2;
  if (tma_stage_override()) NS = tma_stage_override();
  if (bytes(K, NS) > 200 * 1024) return cudaErrorInvalidConfiguration;
  p.tma_k = K;
  p.tma_stages = NS;
  const size_t smem = bytes(K, NS);
  cudaError_t e = ensure_smem(fwd_cta_tma_kernel<MODE, TRAIN>, smem);
  if (e != cudaSuccess) return e;
  ProfScope prof(kProfFwdSweep, st);
  fwd_cta_tma_kernel<MODE, TRAIN><<<total, NT + 32, smem, st>>>(p);
  count_launch();
  return cudaGetLastError();
}

// Variant with the context rows in shared memory (one [64][68] table per CTA; row stride 68 makes
// the per-lane 16-byte row reads conflict-free): 164 registers instead of 255, so three chains
// per SM sub-partition instead of two.  Lane l owns labels l and l + 32.  It is bound by shared
// memory bandwidth (every step reads both 64-float rows of every lane: 16 KB per warp and step)
// and still ~8 % faster than the register variant, which is bound by issue latency at two
// warps per sub-partition.
constexpr int kPairSWarps = 4;
constexpr int kPairRS = 68;

template <bool TRAIN>
__device__ __forceinline__ void minplus_rows32(const float* hb, const float* crow, float e, float& best, int& bi) {
  float cr[32];
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const float4 t = reinterpret_cast<const float4*>(crow)[q];
    cr[4 * q] = t.x, cr[4 * q + 1] = t.y, cr[4 * q + 2] = t.z, cr[4 * q + 3] = t.w;
  }
  minplus_regrow<32, TRAIN>(hb, cr, e, best, bi);
}

template <bool TRAIN>
__global__ void __launch_bounds__(kPairSWarps * 32, 3) fwd_pair_smem_kernel(const __grid_constant__ FwdParams p) {
  extern __shared__ __align__(128) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int L = p.L, D = p.agg ? 2 : p.D, A = D + 1, K = p.tma_k, NS = p.tma_stages;
  float* ctab = smem;  // [64][kPairRS]
  for (int i = threadIdx.x; i < 64 * kPairRS; i += blockDim.x) {
    const int c = i / kPairRS, f = i - c * kPairRS;
    ctab[i] = (c < L && f < L) ? ctx_value(p.ctx, p.ctx_rank, L, c, f) : 0.f;
  }
  const int tile_floats = A * K * L;
  const int per_warp = NS * tile_floats + 2 * 64 + 2 * K + 2 * NS + 2;
  float* wbase = smem + 64 * kPairRS + warp * ((per_warp + 3) & ~3);
  float* tiles = wbase;                               // [NS][A][K][L]
  float* hbuf = tiles + NS * tile_floats;             // [2][64]
  float* etile = hbuf + 128;                          // [2][K]
  unsigned long long* full = reinterpret_cast<unsigned long long*>(etile + 2 * K + ((2 * K) & 1));
  if (lane == 0)
    for (int i = 0; i < NS; ++i) mbar_init(&full[i], 1);
  hbuf[lane] = kInf, hbuf[32 + lane] = kInf, hbuf[64 + lane] = kInf, hbuf[96 + lane] = kInf;
  if (lane == 0) mbar_fence_init();
  __syncthreads();
  ChainCtx ch;
  if (!decode_chain(p, blockIdx.x * kPairSWarps + warp, ch)) return;

  const int len = ch.len;
  const int nstages = (len + K - 1) / K;
  const long long ibase = (long long)ch.img * p.H * p.W;
  const int pix0 = ch.h0 * p.W + ch.w0;
  const bool contiguous = (ch.pstep == 1 || ch.pstep == -1);
  const float* U = p.unary + ibase * L;
  const float* Mr = p.msg_read + ibase * L;

  auto issue_stage = [&](int s) {
    if (s >= nstages) return;
    const int slot = s % NS;
    const int np = len - s * K < K ? len - s * K : K;
    float* T = tiles + slot * tile_floats;
    if (lane == 0) {
      fence_proxy_async_smem();
      mbar_arrive_expect_tx(&full[slot], (unsigned)(np * A * L) * 4u);
    }
    __syncwarp();
    if (contiguous) {
      const int first = ch.pstep == 1 ? pix0 + s * K : pix0 - (s * K + np - 1);
      if (lane < A) {
        const int sid = p.agg ? (lane == 1 ? ch.dir : ch.inv) : lane - 1;
        const float* src = (lane == 0 ? U : Mr + (long long)sid * p.slice) + (long long)first * L;
        bulk_g2s(T + lane * K * L, src, (unsigned)(np * L) * 4u, &full[slot]);
      }
    } else {
      for (int q = lane; q < np * A; q += 32) {
        const int k = q / A, a = q - k * A;
        const int px = pix0 + (s * K + k) * ch.pstep;
        const int sid = p.agg ? (a == 1 ? ch.dir : ch.inv) : a - 1;
        const float* src = (a == 0 ? U : Mr + (long long)sid * p.slice) + (long long)px * L;
        bulk_g2s(T + (a * K + k) * L, src, (unsigned)L * 4u, &full[slot]);
      }
    }
  };

  const int la = lane, lb = lane + 32;
  const bool actb = lb < L;               // la < L always (L > 32)
  const int lbc = actb ? lb : la;         // loads of a missing second label repeat the first
  const float* rowa = ctab + la * kPairRS;
  const float* rowb = ctab + lbc * kPairRS;
  float* Mw = p.msg_write + (long long)ch.dir * p.slice + ibase * L;
  const float* E = p.ew ? p.ew + (long long)ch.dir * p.pslice + ibase : nullptr;
  uint8_t* MI = TRAIN ? p.min_idx + (long long)ch.dir * p.slice + ibase * L : nullptr;
  uint8_t* NI = TRAIN ? p.norm_idx + (long long)ch.dir * p.pslice + ibase : nullptr;
  const int dir_off = (p.agg ? 1 : 1 + ch.dir) * K * L, inv_off = (p.agg ? 2 : 1 + ch.inv) * K * L;
  const float rho = p.rho;
  auto load_e = [&](int s) -> float {
    const int j = s * K + lane;
    return (E && lane < K && j < len && j >= 1) ? E[pix0 + j * ch.pstep] : 1.f;
  };
  auto eval_label = [&](const float* hb, const float* row, float e, float& best, int& bi) {
    float ba, bb;
    int ia, ib;
    minplus_rows32<TRAIN>(hb, row, e, ba, ia);
    minplus_rows32<TRAIN>(hb + 32, row + 32, e, bb, ib);
    best = fminf(ba, bb);
    bi = bb <= ba ? ib + 32 : ia;   // the later half wins ties: highest index
  };

  for (int s = 0; s < NS; ++s) issue_stage(s);
  if (lane < K) etile[lane] = load_e(0);
  float e_next = load_e(1);
  float uu0 = 0.f, uu1 = 0.f, r0 = 0.f, r1 = 0.f;
  // rows of the current chain pixel, moved by one pixel per step (the stage depth is a launch
  // parameter: nothing of it folds into immediates)
  const int postep = ch.pstep * L, KL = K * L;
  float* mwa = Mw + (long long)pix0 * L + la;
  uint8_t* mia = TRAIN ? MI + (long long)pix0 * L + la : nullptr;
  uint8_t* nip = TRAIN ? NI + pix0 : nullptr;
  int hpar = 0;
  bool first = true;
  const bool flip = contiguous && ch.pstep == -1;
  for (int s = 0; s < nstages; ++s) {
    const int slot = s % NS;
    if (!mbar_wait(&full[slot], (s / NS) & 1)) {
      if (lane == 0) atomicExch(p.status, 132);
      return;
    }
    const int np = len - s * K < K ? len - s * K : K;
    const float* T = tiles + slot * tile_floats;
    const float* et = etile + (s & 1) * K;
    __syncwarp();
    const float* t = T + (flip ? np - 1 : 0) * L;
    const int tstep = flip ? -L : L;
    for (int k = 0; k < np; ++k, t += tstep, mwa += postep, hpar ^= 64) {
      float va = t[la], vb = t[lbc];
      if (!p.agg)
        for (int a = 1; a <= D; ++a) va += t[a * KL + la], vb += t[a * KL + lbc];
      const float un0 = fmaf(va - t[dir_off + la], rho, -t[inv_off + la]);
      const float un1 = fmaf(vb - t[dir_off + lbc], rho, -t[inv_off + lbc]);
      if (!first) {
        const float e = et[k];
        float* hb = hbuf + hpar;
        hb[la] = fmaf(rho, r0, uu0);
        if (actb) hb[lb] = fmaf(rho, r1, uu1);
        __syncwarp();
        float b0, b1;
        int i0, i1;
        eval_label(hb, rowa, e, b0, i0);
        eval_label(hb, rowb, e, b1, i1);
        const float x1 = actb ? b1 : kInf;
        const float m = warp_min(fminf(b0, x1));
        r0 = b0 - m;
        r1 = b1 - m;
        mwa[0] = r0;
        if (actb) mwa[32] = r1;
        if (TRAIN) {
          const unsigned bal0 = __ballot_sync(0xffffffffu, b0 == m);
          const unsigned bal1 = __ballot_sync(0xffffffffu, x1 == m);
          mia[0] = (uint8_t)i0;
          if (actb) mia[32] = (uint8_t)i1;
          if (lane == 0) *nip = (uint8_t)(bal1 ? 63 - __clz(bal1) : 31 - __clz(bal0));
        }
      }
      uu0 = un0;
      uu1 = un1;
      first = false;
      if (TRAIN) {
        mia += postep;
        nip += ch.pstep;
      }
    }
    if (lane < K) etile[((s + 1) & 1) * K + lane] = e_next;
    e_next = load_e(s + 2);
    __syncwarp();
    issue_stage(s + NS);
  }
}

template <bool TRAIN>
cudaError_t launch_pair_smem(FwdParams p, cudaStream_t st) {
  const int total = p.chain_off[p.ndirs];
  const int A = (p.agg ? 2 : p.D) + 1;
  int K = 4, NS = 3;
  auto per_warp = [&](int k, int ns) { return ((ns * A * k * p.L + 128 + 2 * k + 2 * ns + 2) + 3) & ~3; };
  auto bytes = [&](int k) { return ((size_t)64 * kPairRS + (size_t)kPairSWarps * per_warp(k, NS)) * sizeof(float); };
  while (K > 1 && bytes(K) > 72 * 1024) K >>= 1;
  p.tma_k = K;
  p.tma_stages = NS;
  const size_t smem = bytes(K);
  cudaError_t e = ensure_smem(fwd_pair_smem_kernel<TRAIN>, smem);
  if (e != cudaSuccess) return e;
  ProfScope prof(kProfFwdSweep, st);
  fwd_pair_smem_kernel<TRAIN><<<(total + kPairSWarps - 1) / kPairSWarps, kPairSWarps * 32, smem, st>>>(p);
  count_launch();
  return cudaGetLastError();
}

template <bool TRAIN>
cudaError_t launch_pair(FwdParams p, cudaStream_t st) {
  // default: context rows in shared memory (three CTAs of four chains per SM); MPL_PAIR_REG=1 selects
  // the variant that keeps both rows of a lane in registers (comparison knob)
  if (!(getenv("MPL_PAIR_REG") && getenv("MPL_PAIR_REG")[0] == '1')) return launch_pair_smem<TRAIN>(p, st);
  const int total = p.chain_off[p.ndirs];
  const int A = (p.agg ? 2 : p.D) + 1;
  int K = 8, NS = 3;
  auto per_warp = [&](int k, int ns) { return ((ns * A * k * p.L + 128 + 2 * k + 2 * ns + 2) + 3) & ~3; };
  while (K > 2 && (size_t)kPairWarps * per_warp(K, NS) * sizeof(float) > 100 * 1024) K >>= 1;
  p.tma_k = K;
  p.tma_stages = NS;
  const size_t smem = (size_t)kPairWarps * per_warp(K, NS) * sizeof(float);
  cudaError_t e = ensure_smem(fwd_pair_kernel<TRAIN>, smem);
  if (e != cudaSuccess) return e;
  ProfScope prof(kProfFwdSweep, st);
  fwd_pair_kernel<TRAIN><<<(total + kPairWarps - 1) / kPairWarps, kPairWarps * 32, smem, st>>>(p);
  count_launch();
  return cudaGetLastError();
}

// Label rows of 16-byte multiples at 16-byte aligned bases: the bulk-copy CTA kernel applies.
bool cta_tma_eligible(const FwdParams& p) {
  if (p.L & 3) return false;
  return (((uintptr_t)p.unary | (uintptr_t)p.msg_read) & 15) == 0;
}

template <int MODE, bool TRAIN>
cudaError_t launch_cta_any(const FwdParams& p, cudaStream_t st) {
  if (cta_tma_eligible(p)) return launch_cta_tma<MODE, TRAIN>(p, st);
  return launch_cta<MODE, TRAIN>(p, st);
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
    // directions with aligned row segments go to the bulk-copy kernel (one launch each), the
    // remaining contiguous range of directions to the generic kernel
    FwdParams rest = p;
    int first_generic = p.dir0;
    // several independent directions (ISGMR) of a small problem: one launch of the generic kernel
    // over all of them beats one small launch per direction
    const bool few_chains = (p.ndirs > 1 && (long long)p.nimg * (p.H < p.W ? p.H : p.W) < 256) || p.parts > 1;
    for (int d = p.dir0; d < p.dir0 + p.ndirs && !few_chains; ++d) {
      int stages = 0;
      if (d != first_generic || !tma_eligible(p, d, &stages)) break;
      cudaError_t e = p.L == 21 ? (train ? launch_tma<21, 21, true>(p, d, stages, st) : launch_tma<21, 21, false>(p, d, stages, st))
                                : (train ? launch_tma<32, 0, true>(p, d, stages, st) : launch_tma<32, 0, false>(p, d, stages, st));
      if (e != cudaSuccess) return e;
      first_generic = d + 1;
    }
    const int nrest = p.dir0 + p.ndirs - first_generic;
    if (nrest == 0) return cudaSuccess;
    const int base = p.chain_off[first_generic - p.dir0];
    rest.dir0 = first_generic;
    rest.ndirs = nrest;
    for (int i = 0; i <= nrest; ++i) rest.chain_off[i] = p.chain_off[first_generic - p.dir0 + i] - base;
    for (int i = 0; i < nrest; ++i) rest.chain_begin[i] = p.chain_begin[first_generic - p.dir0 + i];
    if (p.L == 21) return train ? launch_warp<21, true>(rest, st) : launch_warp<21, false>(rest, st);
    return train ? launch_warp<32, true>(rest, st) : launch_warp<32, false>(rest, st);
  }
  // windowed rank-1 context: warp-per-chain kernel, inference and training (at most 31 candidates per
  // label against the pair kernel's 64: 2.0 against 7.2 ms for a 512 x 512 x 64 training forward)
  static const bool no_wide_train = [] {  // MPL_NO_WIDE_TRAIN=1: tuning / comparison knob
    const char* e = getenv("MPL_NO_WIDE_TRAIN");
    return e && e[0] == '1';
  }();
  if (p.ctx_rank == 1 && (!train || !no_wide_train) && p.host_windowed && p.host_R <= 16 &&
      p.L <= 256 && cta_tma_eligible(p) && (p.agg || p.D != 2)) {
    return launch_forward_wide(p, train, st);
  }
  if (p.L <= 64 && cta_tma_eligible(p) && !pair_kernels_disabled())
    return train ? launch_pair<true>(p, st) : launch_pair<false>(p, st);
  if (p.ctx_rank == 1) return train ? launch_cta_any<1, true>(p, st) : launch_cta_any<1, false>(p, st);
  if (p.L <= 64) return train ? launch_cta_any<2, true>(p, st) : launch_cta_any<2, false>(p, st);
  return train ? launch_cta_any<0, true>(p, st) : launch_cta_any<0, false>(p, st);
}

// Soft TRWP sweep of the directions described by p (L <= 32 only: one warp per chain).
cudaError_t launch_forward_soft_sweep(const FwdParams& p, bool train, cudaStream_t st) {
  if (p.chain_off[p.ndirs] == 0) return cudaSuccess;
  if (p.L > 32) return launch_forward_soft_cta(p, train, st);  // one CTA per chain, up to 64 labels
  if (p.L == 21) return train ? launch_warp_soft<21, true, true>(p, st) : launch_warp_soft<21, false, true>(p, st);
  if (p.L < 21) return train ? launch_warp_soft<21, true, false>(p, st) : launch_warp_soft<21, false, false>(p, st);
  return train ? launch_warp_soft<32, true, false>(p, st) : launch_warp_soft<32, false, false>(p, st);
}

// ------------------------------------------------------------------------------------------------
// Layout glue around the layer: network code holds class scores as [B,L,H,W] planes, the layer wants
// costs [B,H,W,L] with the labels innermost.  The reference does score -> cost (negate, subtract
// the per-pixel minimum), permute, layer, permute, negate as six elementwise passes
// (mpnet.py:161-169, pytorch/MP_module.py:198,232); here each side is one pass through a
// shared-memory tile of 32 pixels x L labels, coalesced on both ends.
//   MODE 0: out = -in            MODE 1: out = max_l(in) - in, argmax saved (lowest index on ties)
//   MODE 2 (backward of 1, direction hwl -> lhw): out[l] = -in[l] + (l == argmax) * sum_l in[l]
//   MODE 3: out = in (the plain layout change of pytorch/MP_module.py:198,232)
// ------------------------------------------------------------------------------------------------
template <int MODE>
__global__ void lhw_to_hwl_kernel(const float* __restrict__ in, float* __restrict__ out, uint8_t* __restrict__ amax,
                                  int L, long long HW) {
  extern __shared__ float tile[];  // [L][33]
  __shared__ float mx[32];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const long long b = blockIdx.y, p0 = blockIdx.x * 32ll;
  const float* src = in + b * L * HW;
  const int np = HW - p0 < 32 ? (int)(HW - p0) : 32;
  for (int l = ty; l < L; l += 8) tile[l * 33 + tx] = tx < np ? src[(long long)l * HW + p0 + tx] : 0.f;
  __syncthreads();
  if (MODE == 1) {
    if (ty == 0) {
      float m = tile[tx];
      int k = 0;
      for (int l = 1; l < L; ++l) {
        const float v = tile[l * 33 + tx];
        if (v > m) m = v, k = l;
      }
      mx[tx] = m;
      if (tx < np) amax[b * HW + p0 + tx] = (uint8_t)k;
    }
    __syncthreads();
  }
  float* dst = out + (b * HW + p0) * L;
  for (int i = threadIdx.x; i < np * L; i += 256) {
    const int px = i / L, l = i - px * L;
    const float v = tile[l * 33 + px];
    dst[i] = MODE == 1 ? mx[px] - v : (MODE == 3 ? v : -v);
  }
}

template <int MODE>
__global__ void hwl_to_lhw_kernel(const float* __restrict__ in, float* __restrict__ out,
                                  const uint8_t* __restrict__ amax, int L, long long HW) {
  extern __shared__ float tile[];  // [L][33]
  __shared__ float sm[32];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long long b = blockIdx.y, p0 = blockIdx.x * 32ll;
  const int np = HW - p0 < 32 ? (int)(HW - p0) : 32;
  const float* src = in + (b * HW + p0) * L;
  for (int i = threadIdx.x; i < np * L; i += 256) {
    const int px = i / L, l = i - px * L;
    tile[l * 33 + px] = src[i];
  }
  __syncthreads();
  if (MODE == 2) {
    if (ty == 0 && tx < np) {
      float s = 0.f;
      for (int l = 0; l < L; ++l) s += tile[l * 33 + tx];
      sm[tx] = s;
    }
    __syncthreads();
  }
  float* dst = out + b * L * HW;
  const int k = (MODE == 2 && tx < np) ? (int)amax[b * HW + p0 + tx] : -1;
  for (int l = ty; l < L; l += 8)
    if (tx < np) {
      const float v = tile[l * 33 + tx];
      dst[(long long)l * HW + p0 + tx] = MODE == 3 ? v : -v + ((MODE == 2 && l == k) ? sm[tx] : 0.f);
    }
}

cudaError_t launch_layout(int kind, const float* in, float* out, uint8_t* amax, int B, int L, long long HW,
                          cudaStream_t st) {
  const dim3 grid((unsigned)((HW + 31) / 32), (unsigned)B);
  const size_t smem = (size_t)L * 33 * sizeof(float);
  ProfScope prof(kProfElementwise, st);
  switch (kind) {
    case 0: lhw_to_hwl_kernel<0><<<grid, 256, smem, st>>>(in, out, amax, L, HW); break;
    case 1: lhw_to_hwl_kernel<1><<<grid, 256, smem, st>>>(in, out, amax, L, HW); break;
    case 2: hwl_to_lhw_kernel<0><<<grid, 256, smem, st>>>(in, out, amax, L, HW); break;
    case 4: lhw_to_hwl_kernel<3><<<grid, 256, smem, st>>>(in, out, amax, L, HW); break;
    case 5: hwl_to_lhw_kernel<3><<<grid, 256, smem, st>>>(in, out, amax, L, HW); break;
    default: hwl_to_lhw_kernel<2><<<grid, 256, smem, st>>>(in, out, amax, L, HW); break;
  }
  count_launch();
  return cudaGetLastError();
}

// Energy of a labelling x on the grid MRF the layers minimise: sum_p U[p, x_p] (out[0]) and
// sum over the undirected edges (p - step_d, p), d even, of E_d[p] * ctx(x_p, x_{p - step_d})
// (out[1]); what the reference's evaluation script computes for the 4-connected case
// (tools/matlab/MRF/calEnergy.m:23-46, right and down links).  One block per 256 pixels writes its
// partial sums (fixed order inside the block), a second kernel adds the partials in order.
__global__ void energy_partial_kernel(const float* __restrict__ unary, const float* __restrict__ ctx,
                                      const float* __restrict__ ew, const uint8_t* __restrict__ label,
                                      long long npix, int H, int W, int L, int D, int rank, double* part) {
  __shared__ double su[256], sp[256];
  const long long px = blockIdx.x * 256ll + threadIdx.x;
  double eu = 0.0, ep = 0.0;
  if (px < npix) {
    const int x = label[px];
    eu = unary[px * L + x];
    const int w = (int)(px % W), h = (int)((px / W) % H);
    for (int d = 0; d < D; d += 2) {
      int hs, ws;
      dir_step(d, hs, ws);
      const int fh = h - hs, fw = w - ws;
      if (fh < 0 || fh >= H || fw < 0 || fw >= W) continue;
      const int xf = label[px - (long long)hs * W - ws];
      const float e = ew ? ew[(long long)d * npix + px] : 1.f;
      ep += (double)(e * ctx_value(ctx, rank, L, x, xf));
    }
  }
  su[threadIdx.x] = eu;
  sp[threadIdx.x] = ep;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      su[threadIdx.x] += su[threadIdx.x + o];
      sp[threadIdx.x] += sp[threadIdx.x + o];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    part[2 * blockIdx.x] = su[0];
    part[2 * blockIdx.x + 1] = sp[0];
  }
}

__global__ void energy_final_kernel(const double* __restrict__ part, int nblocks, double* out) {
  if (threadIdx.x < 2) {
    double s = 0.0;
    for (int b = 0; b < nblocks; ++b) s += part[2 * b + threadIdx.x];
    out[threadIdx.x] = s;
  }
}

cudaError_t launch_energy(const float* unary, const float* ctx, const float* ew, const uint8_t* label,
                          long long npix, int H, int W, int L, int D, int rank, double* part, double* out,
                          cudaStream_t st) {
  const int nblocks = (int)((npix + 255) / 256);
  energy_partial_kernel<<<nblocks, 256, 0, st>>>(unary, ctx, ew, label, npix, H, W, L, D, rank, part);
  count_launch();
  energy_final_kernel<<<1, 32, 0, st>>>(part, nblocks, out);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_aggregate(const float* unary, const float* msg, float* cost, uint8_t* label,
                             long long npix, int L, int D, long long slice, float factor,
                             int min_a_dir, cudaStream_t st) {
  const long long n = npix * L;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  ProfScope prof(kProfElementwise, st);
  const bool vec4 = n % 4 == 0 && slice % 4 == 0 &&
                    ((reinterpret_cast<uintptr_t>(unary) | reinterpret_cast<uintptr_t>(msg) |
                      reinterpret_cast<uintptr_t>(cost)) & 15) == 0;
  if (vec4) {
    long long b4 = (n / 4 + 255) / 256;
    if (b4 > 148 * 16) b4 = 148 * 16;
    aggregate_vec4_kernel<<<(int)b4, 256, 0, st>>>(reinterpret_cast<const float4*>(unary),
                                                   reinterpret_cast<const float4*>(msg),
                                                   reinterpret_cast<float4*>(cost), n / 4, D, slice / 4, factor,
                                                   min_a_dir);
  } else {
    aggregate_kernel<<<(int)blocks, 256, 0, st>>>(unary, msg, cost, n, D, slice, factor, min_a_dir);
  }
  count_launch();
  if (label) {
    label_kernel<<<(int)((npix + 127) / 128), 128, 0, st>>>(cost, label, npix, L);
    count_launch();
  }
  return cudaGetLastError();
}

cudaError_t launch_aggregate_lhw(const float* unary, const float* msg, float* cost, int nimg, int L,
                                 long long HW, int D, long long slice, float factor, int min_a_dir,
                                 cudaStream_t st) {
  const dim3 grid((unsigned)((HW + 31) / 32), (unsigned)nimg);
  const size_t smem = (size_t)L * 33 * sizeof(float);
  ProfScope prof(kProfElementwise, st);
  aggregate_lhw_kernel<<<grid, 256, smem, st>>>(unary, msg, cost, L, HW, D, slice, factor, min_a_dir);
  count_launch();
  return cudaGetLastError();
}

}  // namespace mpl
