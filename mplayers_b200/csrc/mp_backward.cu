// Backward kernels of the TRWP / ISGMR layers for sm_100a.
//
// One backward sweep replays one direction's chains in reverse from the saved argmin indices.
// The reference does it as a chain kernel with four global atomicAdds per label per step
// (MPLayers/TRWP/TRWP_backward.cu:49-275), an elementwise UpdateUnaryKernelBack with D+3 more
// atomics per element (:26-47) and two memsets (:421-422).  Here the whole sweep is one kernel:
//   * the scatter "dUU[front, idx[c]] += t[c]" never leaves the chip: it is evaluated as a gather
//     over the labels of the same pixel (fixed order, so the result is run-to-run identical) and
//     carried to the predecessor pixel in a register;
//   * the elementwise update of the pixel's gradients is applied on the fly (each address is
//     touched once per sweep);
//   * the label-context gradient is accumulated in a per-chain table in shared memory (row c is
//     private to thread c) and flushed once per chain into per-slot partial tables, which a final
//     kernel sums in a fixed order;
//   * per-pixel scalars (normalisation sum, edge weight, normalisation index, edge-weight
//     gradient) are produced for a whole block of steps at once, one step per lane, instead of
//     one warp reduction per step.  The normalisation sum is taken over the stored gradient
//     alone: the part carried from the successor pixel sums to zero (it is itself the output of
//     a normalisation backward), so only rounding noise is dropped.
#include <cstdlib>

#include "mp_common.cuh"
#include "mp_minplus.cuh"

namespace mpl {

namespace {

__device__ __forceinline__ void warp_sum2(float& a, float& b) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
}

// ------------------------------------------------------------------------------------------------
// L <= 32, generic: one warp per chain, lane = label, any direction / alignment.
// DT = compile-time direction count (0: from params); CP = gradient bookkeeping scheme.
//
// The chain is walked in blocks of 32 steps; the stored message gradients of a whole block are
// staged in shared memory one block ahead with cp.async.
// ------------------------------------------------------------------------------------------------
constexpr int kRB = 64;  // ring rows: two blocks of 32 steps
constexpr int kRS = 33;  // padded row stride (conflict-free both along and across rows)

__host__ __device__ inline int bwd_warp_floats(int L, int rank, int cp) {
  const int tab = rank == 2 ? L * (L | 1) : 32;
  return (cp ? 2 : 1) * kRB * kRS + 32 * kRS + 128 + ((tab + 3) & ~3);
}

template <int DT, int SCH>
__global__ void __launch_bounds__(128, 1) bwd_warp_kernel(const __grid_constant__ BwdParams p) {
  constexpr bool CP = SCH == 1;   // C + P bookkeeping
  constexpr bool QM = SCH == 2;   // store the scatter field only
  extern __shared__ __align__(16) float smem[];
  const int wpb = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int L = p.L, D = DT ? DT : p.D;
  const int LS = L | 1;  // odd row stride: private rows without bank conflicts
  // full (symmetric / Toeplitz) context table shared by the CTA
  float* ctab = smem;
  const int ctab_floats = (L * LS + 3) & ~3;
  for (int i = threadIdx.x; i < L * L; i += blockDim.x)
    ctab[(i / L) * LS + (i % L)] = ctx_value(p.ctx, p.ctx_rank, L, i / L, i % L);
  __syncthreads();
  const int g = blockIdx.x * wpb + warp;
  BChain ch;
  if (!decode_bchain(p, g, ch)) return;
  const int dir = ch.dir, inv = dir ^ 1;
  const int tab = p.ctx_rank == 2 ? L * LS : 32;
  float* ring = smem + ctab_floats + warp * bwd_warp_floats(L, p.ctx_rank, CP);  // [kRB][kRS] (x2 if CP)
  float* ring2 = ring + kRB * kRS;                                              // CP: P_dir rows
  float* dtile = ring + (CP ? 2 : 1) * kRB * kRS;                               // [32][kRS]
  float* ts = dtile + 32 * kRS;                                                 // [2][32]
  float* is = ts + 64;                                                          // [2][32] argmin as float
  float* acc = ts + 128;                                                        // context-gradient table
  const bool act = lane < L;
  for (int i = lane; i < tab; i += 32) acc[i] = 0.f;
  is[lane] = -1.f;
  is[32 + lane] = -1.f;

  const long long ibase = (long long)ch.img * p.H * p.W;
  float* DMrl = p.dm_read + (long long)dir * p.slice + ibase * L + lane;  // dM_dir, or P_dir
  float* DMal = p.dm_acc + ibase * L + lane;
  float* DUl = p.dunary + ibase * L + lane;                              // dU, or C
  const float* E = p.ew ? p.ew + (long long)dir * p.pslice + ibase : nullptr;
  float* DE = p.dew ? p.dew + (long long)dir * p.pslice + ibase : nullptr;
  const uint8_t* MIl = p.min_idx + (long long)dir * p.slice + ibase * L + lane;
  const uint8_t* NI = p.norm_idx + (long long)dir * p.pslice + ibase;
  const int len = ch.len;
  const int pstep = ch.pstep, ostep = ch.pstep * L;
  const int pixl = ch.h0 * p.W + ch.w0 + (len - 1) * pstep;  // last pixel of the chain
  const float rho = p.rho;
  const float rinv = rho - 1.f;  // dM_inv += rho*q - q
  const int nsteps = len - 1;    // steps with a predecessor pixel (s = 0 .. len-2)

  // step s visits chain pixel len-1-s at image pixel pixl - s*pstep
  auto stage_block = [&](int b) {  // stored gradients of the 32 steps of block b -> ring rows
    if (act) {
      const int s = 32 * b;
      int o = (pixl - s * pstep) * L;
      float* dst = ring + (s & (kRB - 1)) * kRS + lane;
#pragma unroll 8
      for (int u = 0; u < 32; ++u) {
        // CP also needs the values of the chain-start pixel (its C is rewritten there)
        if (s + u < (CP ? len : nsteps)) {
          cp_async4(dst + u * kRS, CP ? DUl + o : DMrl + o);
          if (CP) cp_async4(dst + kRB * kRS + u * kRS, DMrl + o);
        }
        o -= ostep;
      }
    }
    cp_async_commit();
  };
  auto load_blk = [&](int b, float& eb, int& nb) {  // lane l: scalars of step 32*b + l
    const int s = 32 * b + lane;
    eb = 1.f;
    nb = 0;
    if (s < nsteps) {
      const int px = pixl - s * pstep;
      if (E) eb = E[px];
      nb = NI[px];
    }
  };

  stage_block(0);
  float e_cur, e_nxt;
  int n_cur, n_nxt;
  load_blk(0, e_cur, n_cur);
  int fa[8], fb[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) fa[u] = (u < nsteps && act) ? (int)MIl[(pixl - u * pstep) * L] : -1;

  float q = 0.f;  // lane f: sum of t[c] of the successor pixel over labels c whose argmin was f
  int of = pixl * L;
  const int nblocks = (len + 31) >> 5;
  for (int b = 0; b < nblocks; ++b) {
    stage_block(b + 1);
    load_blk(b + 1, e_nxt, n_nxt);
    cp_async_wait<1>();
    __syncwarp();
    // normalisation sums of this block: lane j sums row j of the staged gradients
    float s_cur = 0.f;
    {
      const float* row = ring + ((32 * b + lane) & (kRB - 1)) * kRS;
      for (int c = 0; c < L; ++c) s_cur += CP ? row[c] + row[kRB * kRS + c] : row[c];
    }
    for (int g8 = 0; g8 < 4; ++g8) {
      const int s0 = 32 * b + 8 * g8;
      if (s0 >= len) break;
#pragma unroll
      for (int u = 0; u < 8; ++u) {  // argmin indices of the next group of 8 steps
        const int s = s0 + 8 + u;
        fb[u] = (s < nsteps && act) ? (int)MIl[(pixl - s * pstep) * L] : -1;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int s = s0 + u;
        if (s < len) {
          const float rq = rho * q;
          float qn = 0.f;
          const float x0 = ring[(s & (kRB - 1)) * kRS + lane];  // dM_dir, or C
          if (s < nsteps) {
            const int sl = s & 31;
            const float e = __shfl_sync(0xffffffffu, e_cur, sl);
            const int n = __shfl_sync(0xffffffffu, n_cur, sl);
            const float S = __shfl_sync(0xffffffffu, s_cur, sl);
            const int f = fa[u];
            const float x = CP ? x0 + ring2[(s & (kRB - 1)) * kRS + lane] : x0;
            const float t0 = act ? x + rq : 0.f;
            const float t = (lane == n) ? t0 - S : t0;  // MPLayers/commonCUDA.cuh:131-145
            float cv = 0.f;
            if (act) {
              cv = ctab[lane * LS + f];
              if (lane != f || p.keep_diag) {
                if (p.ctx_rank == 2) {
                  acc[lane * LS + f] += e * t;
                } else {
                  atomicAdd(acc + (lane > f ? lane - f : f - lane), e * t);
                }
              }
            }
            dtile[sl * kRS + lane] = cv * t;
            float* tb = ts + (s & 1) * 32;
            float* ib = is + (s & 1) * 32;
            tb[lane] = t;
            if (act) ib[lane] = (float)f;
            __syncwarp();
            qn = gather_q<0>(tb, ib, L, (float)lane);
          }
          if (act) {
            if (QM) {
              DMal[(long long)dir * p.slice + of] = q;  // scatter field of this direction at this pixel
            } else if (CP) {
              const float cnew = x0 + rq;  // dU and every dM_k (k != dir, inv) receive rho*q
              DUl[of] = cnew;
              DMrl[of] = -cnew;            // dM_dir = C + P_dir = 0 after its sweep
              atomicAdd(DMal + inv * p.slice + of, -q);
            } else {
              // UpdateUnaryKernelBack (MPLayers/TRWP/TRWP_backward.cu:26-47) applied to this pixel
#pragma unroll
              for (int k = 0; k < (DT ? DT : 16); ++k) {
                if (k < D && k != dir) atomicAdd(DMal + k * p.slice + of, k == inv ? rinv * q : rq);
              }
              atomicAdd(DUl + of, rq);
              DMrl[of] = 0.f;
            }
          }
          q = qn;
          of -= ostep;
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) fa[u] = fb[u];
    }
    // edge-weight gradients of this block: lane j sums row j of the product tile
    __syncwarp();
    if (DE) {
      const int s = 32 * b + lane;
      if (s < nsteps) {
        const float* row = dtile + lane * kRS;
        float de = 0.f;
        for (int c = 0; c < L; ++c) de += row[c];
        atomicAdd(DE + (pixl - s * pstep), de);
      }
    }
    __syncwarp();
    e_cur = e_nxt;
    n_cur = n_nxt;
  }
  cp_async_wait<0>();

  // flush the context-gradient table of this chain
  __syncwarp();
  float* part = p.dctx_part + (long long)(g % p.n_slots) * (p.ctx_rank == 2 ? L * L : L);
  if (p.ctx_rank == 2) {
    for (int i = lane; i < L * L; i += 32) {
      const float v = acc[(i / L) * LS + (i % L)];
      if (v != 0.f) atomicAdd(part + i, v);
    }
  } else if (act) {
    const float v = acc[lane];
    if (v != 0.f) atomicAdd(part + lane, v);
  }
}

// ------------------------------------------------------------------------------------------------
// L <= 32, directions 0..3, 16-byte aligned rows, C + P bookkeeping: bulk-copy staged kernel.
// Same CTA organisation as the forward one: four consumer warps (four neighbouring chains) and a
// producer warp issuing plain cp.async.bulk copies of C and P_dir row segments, kBK steps per
// stage, completion counted on mbarriers; every wait is bounded.
// LT = compile-time label count (0: runtime); VERT = directions 2/3; REV = the backward walk runs
// towards decreasing coordinates (directions 0 and 2, whose forward walk runs upwards).
// ------------------------------------------------------------------------------------------------
constexpr int kBK = 16;
constexpr int kDS = 33;  // row stride of the per-stage product tile

__host__ __device__ inline int bwd_tma_warp_floats(int L, int rank) {
  (void)rank;  // the per-chain table is kept per (c, f) pair for both context conventions
  return kBK * kDS + 128 + ((L * (L | 1) + 3) & ~3);
}

// QM: scatter-field scheme (ISGMR): only the gradient slice of the direction is staged and only the
// scatter field is stored.
template <int LT, bool VERT, bool REV, bool QM = false>
__global__ void __launch_bounds__(160, 1) bwd_tma_kernel(const __grid_constant__ BwdParams p,
                                                         const __grid_constant__ TmaMaps maps) {
  // No static shared memory in this kernel: the dynamic region starts at the CTA's shared window
  // base, which satisfies the 128-byte alignment the tiled TMA destination needs.  (Rounding the
  // pointer up by hand would hide its address space from the compiler and turn every shared
  // access into a slower generic one.)
  extern __shared__ __align__(128) float smem[];
  const int L = LT ? LT : p.L, H = p.H, W = p.W, NS = p.tma_stages;
  const int LS = L | 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int dir = p.dir, inv = dir ^ 1;
  const int len = VERT ? H : W;
  const int nstages = (len + kBK - 1) / kBK;
  const int tile_floats = 2 * kBK * 4 * L;  // C and P_dir, kBK steps, four chains

  float* tiles = smem;                                         // [NS][tile_floats]
  float* ctab = tiles + NS * tile_floats;                      // [L][LS]
  float* wbase = ctab + ((L * LS + 3) & ~3);                   // per-warp areas
  unsigned long long* full =
      reinterpret_cast<unsigned long long*>(wbase + 4 * bwd_tma_warp_floats(L, p.ctx_rank));
  unsigned long long* empty = full + NS;

  int nact, img0 = 0, w0 = 0, chain0 = 0;
  if (VERT) {
    const int gpi = W >> 2;
    img0 = blockIdx.x / gpi;
    w0 = (blockIdx.x - img0 * gpi) << 2;
    nact = 4;
  } else {
    chain0 = blockIdx.x << 2;
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
  for (int i = threadIdx.x; i < L * L; i += blockDim.x)
    ctab[(i / L) * LS + (i % L)] = ctx_value(p.ctx, p.ctx_rank, L, i / L, i % L);
  __syncthreads();

  // step st of the walk visits coordinate (REV ? len-1-st : st) along the chain direction
  if (warp == 4) {
    // ---------------------------------- producer ----------------------------------
    const unsigned row_bytes = 16u * L;
    for (int s = 0; s < nstages; ++s) {
      const int slot = s % NS;
      if (s >= NS && !mbar_wait(&empty[slot], ((s / NS) - 1) & 1)) {
        if (lane == 0) atomicExch(p.status, 201);
        break;
      }
      const int npix = len - s * kBK < kBK ? len - s * kBK : kBK;
      float* T = tiles + slot * tile_floats;
      if (VERT) {
        // 2-D tiled TMA: one copy per array brings kBK image rows of the 4-pixel column group
        if (lane == 0) {
          mbar_arrive_expect_tx(&full[slot], (QM ? 1u : 2u) * kBK * row_bytes);
          const int y0 = img0 * H + (REV ? H - (s + 1) * kBK : s * kBK);
          if (!QM) tma_load_2d(T, &maps.a, w0 * L, y0, &full[slot]);
          tma_load_2d(T + kBK * 4 * L, &maps.b, w0 * L, dir * p.nimg * H + y0, &full[slot]);
        }
      } else {
        if (lane == 0) mbar_arrive_expect_tx(&full[slot], (unsigned)nact * (unsigned)npix * (QM ? 4u : 8u) * L);
        __syncwarp();
        const int ncopy = nact * 2;
        for (int c = lane; c < ncopy; c += 32) {
          const int qd = c >> 1, a = c & 1;
          if (QM && a == 0) continue;
          const int wlo = REV ? W - s * kBK - npix : s * kBK;
          const long long pix = (long long)(chain0 + qd) * W + wlo;
          const float* src = (a == 0 ? p.dunary : p.dm_read + (long long)dir * p.slice) + pix * L;
          bulk_g2s(T + (qd * 2 + a) * kBK * L, src, (unsigned)npix * 4u * L, &full[slot]);
        }
      }
    }
    return;
  }

  // ---------------------------------- consumers ----------------------------------
  const int wc = warp;
  if (wc >= nact) return;
  const bool act = lane < L;
  const int lc = act ? lane : L - 1;  // idle lanes mirror the last label (stores hit the same address)
  float* dtile = wbase + wc * bwd_tma_warp_floats(L, p.ctx_rank);  // [kBK][kDS]
  float* ts = dtile + kBK * kDS;                                   // [2][32]
  float* is = ts + 64;                                             // [2][32] argmin as float
  float* acc = ts + 128;                                           // [L][LS], row c private to lane c
  for (int i = lane; i < L * LS; i += 32) acc[i] = 0.f;
  __syncwarp();

  int img, fix;
  if (VERT) {
    img = img0;
    fix = w0 + wc;
  } else {
    img = (chain0 + wc) / H;
    fix = (chain0 + wc) - img * H;
  }
  const long long ibase = (long long)img * H * W;
  float* Cl = QM ? nullptr : p.dunary + ibase * L + lc;
  float* Pdl = p.dm_read + (long long)dir * p.slice + ibase * L + lc;
  float* Pil = p.dm_read + (long long)inv * p.slice + ibase * L + lc;
  float* Ql = p.dm_acc + (long long)dir * p.slice + ibase * L + lc;   // QM: scatter field of this direction
  const float* E = p.ew ? p.ew + (long long)dir * p.pslice + ibase : nullptr;
  float* DE = p.dew ? p.dew + (long long)dir * p.pslice + ibase : nullptr;
  const uint8_t* MIl = p.min_idx + (long long)dir * p.slice + ibase * L + lc;
  const uint8_t* NI = p.norm_idx + (long long)dir * p.pslice + ibase;
  const float rho = p.rho;
  const int sa = VERT ? kBK * 4 * L : kBK * L;        // C -> P_dir inside a tile
  const int sk = (VERT ? 4 * L : L) * (REV ? -1 : 1);  // consecutive steps inside a tile
  const int pstep = VERT ? (REV ? -W : W) : (REV ? -1 : 1);
  const int px0 = VERT ? (REV ? H - 1 : 0) * W + fix : fix * W + (REV ? W - 1 : 0);  // first step
  const int nsteps = len - 1;  // steps that have a predecessor pixel
  const bool diag_ok = p.keep_diag != 0;
  const bool rank2 = p.ctx_rank == 2;
  const float mef = (float)lc;

  float q = 0.f;
  // per-stage scalars, lane j < kBK: step kBK*s + j
  auto load_scalars = [&](int s, float& es, int& ns) {
    const int st = s * kBK + lane;
    es = 1.f;
    ns = 0;
    if (lane < kBK && st < nsteps) {
      const int px = px0 + st * pstep;
      if (E) es = E[px];
      ns = NI[px];
    }
  };
  auto load_idx = [&](int s, int (&fi)[kBK]) {
    if ((s + 1) * kBK <= nsteps) {  // every step of the stage has a predecessor: no per-load checks
      const uint8_t* b = MIl + (px0 + s * kBK * pstep) * L;
#pragma unroll
      for (int u = 0; u < kBK; ++u) fi[u] = (int)b[u * pstep * L];
    } else {
#pragma unroll
      for (int u = 0; u < kBK; ++u) {
        const int st = s * kBK + u;
        fi[u] = st < nsteps ? (int)MIl[(px0 + st * pstep) * L] : 0;
      }
    }
  };
  float e_st, e_nx;
  int n_st, n_nx;
  int fa[kBK], fb[kBK];
  load_scalars(0, e_st, n_st);
  load_idx(0, fa);

  // output rows of the current pixel, moved by one pixel per step
  const long long ostep = (long long)pstep * L;
  float* pC = QM ? nullptr : Cl + (long long)px0 * L;
  float* pPd = Pdl + (long long)px0 * L;
  float* pPi = Pil + (long long)px0 * L;
  float* pQ = Ql + (long long)px0 * L;
  // one step: t = tile pointer of this pixel (C at t[0], P_dir at t[sa]), k = step inside the stage
  auto step = [&](const float* t, int k, int f, float S_st, bool has_front) {
    const float cval = QM ? 0.f : t[0];
    const float rq = rho * q;
    float qn = 0.f;
    if (has_front) {
      const float e = __shfl_sync(0xffffffffu, e_st, k);
      const int n = __shfl_sync(0xffffffffu, n_st, k);
      const float S = __shfl_sync(0xffffffffu, S_st, k);
      const float t0 = (cval + t[sa]) + rq;
      const float tt = (lc == n) ? t0 - S : t0;  // MPLayers/commonCUDA.cuh:131-145
      const float cv = ctab[lc * LS + f];
      dtile[k * kDS + lane] = cv * tt;
      // the diagonal (c == f) is accumulated like every other cell and dropped at the flush unless
      // it is wanted; idle lanes repeat lane L-1's read-modify-write in lockstep
      acc[lc * LS + f] = fmaf(e, tt, acc[lc * LS + f]);
      float* tb = ts + (k & 1) * 32;
      float* ib = is + (k & 1) * 32;
      tb[lane] = tt;
      ib[lane] = (float)f;
      __syncwarp();
      qn = gather_q<LT>(tb, ib, L, mef);
    }
    if constexpr (QM) {
      *pQ = q;
      pQ += ostep;
    } else {
      const float cnew = cval + rq;  // dU and every dM_k (k != dir, inv) receive rho*q
      *pC = cnew;
      *pPd = -cnew;                  // dM_dir = C + P_dir = 0 after its sweep
      if (act) atomicAdd(pPi, -q);
      pC += ostep;
      pPd += ostep;
      pPi += ostep;
    }
    q = qn;
  };

  for (int s = 0; s < nstages; ++s) {
    const int slot = s % NS;
    load_scalars(s + 1, e_nx, n_nx);
    load_idx(s + 1, fb);
    if (!mbar_wait(&full[slot], (s / NS) & 1)) {
      if (lane == 0) atomicExch(p.status, 202);
      return;
    }
    const int npix = len - s * kBK < kBK ? len - s * kBK : kBK;
    const float* T = tiles + slot * tile_floats;
    const float* t0p;
    if (VERT) {  // box rows ascend in memory; a downward walk starts at the last row of the box
      t0p = T + wc * L + (REV ? (kBK - 1) * 4 * L : 0);
    } else {
      t0p = T + wc * 2 * kBK * L + (REV ? (npix - 1) * L : 0);
    }
    // normalisation sums of the stage: lane j sums (C + P_dir) over the labels of step j
    float S_st = 0.f;
    if (lane < npix) {
      const float* row = t0p + lane * sk;
      if constexpr (LT > 0) {
#pragma unroll
        for (int c = 0; c < LT; ++c) S_st += QM ? row[sa + c] : row[c] + row[sa + c];
      } else {
        for (int c = 0; c < L; ++c) S_st += QM ? row[sa + c] : row[c] + row[sa + c];
      }
    }
    const float* tl = t0p + lc;
    const int pxs = px0 + s * kBK * pstep;
    if (npix == kBK && s != nstages - 1) {
#pragma unroll
      for (int k = 0; k < kBK; ++k) step(tl + k * sk, k, fa[k], S_st, true);
    } else {
#pragma unroll
      for (int k = 0; k < kBK; ++k)
        if (k < npix) step(tl + k * sk, k, fa[k], S_st, s * kBK + k < nsteps);
    }
    // edge-weight gradients of this stage: lane j sums row j of the product tile
    __syncwarp();
    if (DE && lane < kBK && s * kBK + lane < nsteps)
      atomicAdd(DE + (pxs + lane * pstep), row_sum<LT>(dtile + lane * kDS, L));
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[slot]);
    e_st = e_nx;
    n_st = n_nx;
#pragma unroll
    for (int u = 0; u < kBK; ++u) fa[u] = fb[u];
  }

  // flush the context-gradient table of this chain
  __syncwarp();
  const int gchain = blockIdx.x * 4 + wc;
  float* part = p.dctx_part + (long long)(gchain % p.n_slots) * (rank2 ? L * L : L);
  if (rank2) {
    for (int i = lane; i < L * L; i += 32) {
      const int c = i / L, f = i - c * L;
      const float v = acc[c * LS + f];
      if (v != 0.f && (c != f || diag_ok)) atomicAdd(part + i, v);
    }
  } else if (act && (lane > 0 || diag_ok)) {  // rank 1: lane k folds every (c, f) with |c - f| == k, in a fixed order
    float v = 0.f;
    for (int c = 0; c < L; ++c) {
      if (c - lane >= 0) v += acc[c * LS + c - lane];
      if (lane > 0 && c + lane < L) v += acc[c * LS + c + lane];
    }
    if (v != 0.f) atomicAdd(part + lane, v);
  }
}

// ------------------------------------------------------------------------------------------------
// 32 < L <= 64, L % 4 == 0: one WARP per chain, TWO labels per lane (2*lane, 2*lane + 1), schemes
// 1 (C + P) and 2 (scatter field).  No block barrier: the CTA-per-chain kernel pays two per step
// plus a cross-warp reduction.  The stored gradients are staged kPB steps per stage by the warp
// itself (lane-parallel cp.async.bulk copies: one per array and stage for horizontal chains, one
// label row per pixel otherwise) with completion on the warp's own mbarriers, bounded waits.
// ------------------------------------------------------------------------------------------------
constexpr int kPB = 16;   // steps per stage (and per block of per-pixel scalars)
constexpr int kPNS = 2;   // stages in flight

// floats of shared memory per warp (the CTA adds one [L][L|1] context table)
__host__ __device__ inline int bwd_pair_floats(int L, int rank, int sch) {
  const int tab = rank == 2 ? L * (L | 1) : 64;
  return kPNS * (sch == 1 ? 2 : 1) * kPB * L + kPNS * kPB * L / 4 + kPB * 33 + 256 + ((tab + 3) & ~3) + 2 * kPNS + 2;
}

// q0 / q1: scatter sums of labels me0, me0 + 1 over the 64 (padded) labels of one pixel.
// FULL: all 64 labels exist (no loop bound to test).
template <bool FULL>
__device__ __forceinline__ void gather_q2(const float* tb, const float* ib, int L, float me0, float& q0,
                                          float& q1) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f;
  const float me1 = me0 + 1.f;
  auto body = [&](int v) {  // four labels c: packed fmas over (c, c+1), accumulators a* for me0, b* for me1
    const float4 t = reinterpret_cast<const float4*>(tb)[v];
    const float4 i = reinterpret_cast<const float4*>(ib)[v];
    ffma2(a0, a1, eq_flag(i.x, me0), eq_flag(i.y, me0), t.x, t.y, a0, a1);
    ffma2(b0, b1, eq_flag(i.x, me1), eq_flag(i.y, me1), t.x, t.y, b0, b1);
    ffma2(a2, a3, eq_flag(i.z, me0), eq_flag(i.w, me0), t.z, t.w, a2, a3);
    ffma2(b2, b3, eq_flag(i.z, me1), eq_flag(i.w, me1), t.z, t.w, b2, b3);
  };
  if constexpr (FULL) {
#pragma unroll
    for (int v = 0; v < 16; ++v) body(v);
  } else {
    const int nv = L >> 2;
#pragma unroll 3
    for (int v = 0; v < nv; ++v) body(v);
  }
  q0 = (a0 + a1) + (a2 + a3);
  q1 = (b0 + b1) + (b2 + b3);
}

// Nothing in the step loop loads from global memory into registers except the per-block scalars:
// gradients arrive by bulk copy, argmin indices by cp.async, context values come from a table in
// shared memory.  (Register prefetches of several kinds share the few hardware scoreboards, and a
// use of a cached value then waits for the DRAM loads issued next to it.)
template <int SCH, bool FULL>
__global__ void __launch_bounds__(256, 1) bwd_pair_kernel(const __grid_constant__ BwdParams p) {
  constexpr bool CP = SCH == 1;
  constexpr int NA = CP ? 2 : 1;  // staged arrays: (C, P_dir) or the gradient slice of the direction
  extern __shared__ __align__(128) float smem[];
  const int wpb = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int L = FULL ? 64 : p.L, LS = L | 1;
  const int ctab_floats = (L * LS + 3) & ~3;
  float* ctab = smem;                              // [L][LS] full context table of the CTA
  for (int i = threadIdx.x; i < L * L; i += blockDim.x)
    ctab[(i / L) * LS + (i % L)] = ctx_value(p.ctx, p.ctx_rank, L, i / L, i % L);
  const int per_warp = (bwd_pair_floats(L, p.ctx_rank, SCH) + 3) & ~3;
  float* ring = smem + ctab_floats + warp * per_warp;  // [kPNS][NA][kPB][L]
  const int stage_floats = NA * kPB * L;
  uint8_t* itile = reinterpret_cast<uint8_t*>(ring + kPNS * stage_floats);  // [kPNS][kPB][L] argmin indices
  float* dtile = ring + kPNS * stage_floats + kPNS * kPB * L / 4;           // [kPB][33]
  float* ts = dtile + kPB * 33;                    // [2][64]  (kPB * 33 is a multiple of 4)
  float* is = ts + 128;                            // [2][64] argmin as float
  float* acc = is + 128;                           // context-gradient table of this chain
  const int tab = p.ctx_rank == 2 ? L * LS : 64;
  unsigned long long* full = reinterpret_cast<unsigned long long*>(acc + ((tab + 3) & ~3));
  if (lane == 0) {
    for (int i = 0; i < kPNS; ++i) mbar_init(&full[i], 1);
    mbar_fence_init();
  }
  for (int i = lane; i < tab; i += 32) acc[i] = 0.f;
  for (int i = lane; i < 128; i += 32) ts[i] = 0.f, is[i] = -1.f;
  __syncthreads();
  const int g = blockIdx.x * wpb + warp;
  BChain ch;
  if (!decode_bchain(p, g, ch)) return;
  const int dir = ch.dir, inv = dir ^ 1;
  const int c0 = 2 * lane;
  const bool act = c0 < L;  // L is even: a lane owns two labels or none

  const long long ibase = (long long)ch.img * p.H * p.W;
  float* DMr = p.dm_read + (long long)dir * p.slice + ibase * L;  // dM_dir, or P_dir
  float* DMa = p.dm_acc + ibase * L;
  float* DU = p.dunary + ibase * L;                               // dU, or C
  const float* E = p.ew ? p.ew + (long long)dir * p.pslice + ibase : nullptr;
  float* DE = p.dew ? p.dew + (long long)dir * p.pslice + ibase : nullptr;
  const uint8_t* MI = p.min_idx + (long long)dir * p.slice + ibase * L;
  const uint8_t* NI = p.norm_idx + (long long)dir * p.pslice + ibase;
  const int len = ch.len, pstep = ch.pstep, ostep = pstep * L;
  const int pixl = ch.h0 * p.W + ch.w0 + (len - 1) * pstep;  // last pixel of the chain
  const float rho = p.rho;
  const int nsteps = len - 1;               // steps with a predecessor pixel
  const int nrows = CP ? len : nsteps;      // staged pixels (C + P also rewrites the chain-start pixel)
  const bool contiguous = pstep == 1 || pstep == -1;
  const int nblocks = (len + kPB - 1) / kPB;

  auto stage_rows = [&](int b) {
    const int r = nrows - kPB * b;
    return r < 0 ? 0 : (r > kPB ? kPB : r);
  };
  // step s = kPB*b + u visits image pixel pixl - s*pstep; its row in the stage tile is u, except
  // for chains walked towards decreasing addresses in one copy (pstep == +1), which land reversed
  auto issue_stage = [&](int b) {
    const int rows = stage_rows(b);
    const int slot = b % kPNS;
    const int s0 = kPB * b;
    if (rows > 0) {
      float* T = ring + slot * stage_floats;
      if (lane == 0) {
        fence_proxy_async_smem();
        mbar_arrive_expect_tx(&full[slot], (unsigned)(rows * NA * L) * 4u);
      }
      __syncwarp();
      if (contiguous) {
        const int first = pstep == 1 ? pixl - (s0 + rows - 1) : pixl + s0;
        if (lane < NA)
          bulk_g2s(T + lane * kPB * L, (CP && lane == 0 ? DU : DMr) + (long long)first * L,
                   (unsigned)(rows * L) * 4u, &full[slot]);
      } else {
        for (int q = lane; q < rows * NA; q += 32) {
          const int u = q / NA, a = q - u * NA;
          const int px = pixl - (s0 + u) * pstep;
          bulk_g2s(T + (a * kPB + u) * L, (CP && a == 0 ? DU : DMr) + (long long)px * L, (unsigned)L * 4u,
                   &full[slot]);
        }
      }
    }
    // argmin indices of the steps with a predecessor: four labels per lane and step
    if (4 * lane < L) {
      uint8_t* dst = itile + (slot * kPB) * L + 4 * lane;
      const uint8_t* src = MI + (long long)(pixl - s0 * pstep) * L + 4 * lane;
#pragma unroll 4
      for (int u = 0; u < kPB; ++u) {
        if (s0 + u < nsteps)
          cp_async4(reinterpret_cast<float*>(dst + u * L), reinterpret_cast<const float*>(src - (long long)u * ostep));
      }
    }
    cp_async_commit();
  };
  auto load_blk = [&](int b, float& eb, int& nb) {  // lane l: scalars of step kPB*b + (l & 15)
    const int s = kPB * b + (lane & (kPB - 1));
    eb = 1.f;
    nb = 0;
    if (s < nsteps) {
      const int px = pixl - s * pstep;
      if (E) eb = E[px];
      nb = NI[px];
    }
  };

  for (int b = 0; b < kPNS; ++b) issue_stage(b);
  float e_cur, e_nxt;
  int n_cur, n_nxt;
  load_blk(0, e_cur, n_cur);

  float q0 = 0.f, q1 = 0.f;  // scatter sums carried from the successor pixel (labels c0, c0 + 1)
  // output rows of the current pixel (labels c0, c0 + 1), moved by one pixel per step
  float* pA = (CP ? DU : DMa + (long long)dir * p.slice) + (long long)pixl * L + c0;  // C, or the scatter field
  float* pB = DMr + (long long)pixl * L + c0;                                         // P_dir
  float* pI = DMa + (long long)inv * p.slice + (long long)pixl * L + c0;              // P_inv
  for (int b = 0; b < nblocks; ++b) {
    load_blk(b + 1, e_nxt, n_nxt);
    const int rows = stage_rows(b);
    const int slot = b % kPNS;
    const float* T = ring + slot * stage_floats;
    const uint8_t* IT = itile + (slot * kPB) * L + c0;
    cp_async_wait<kPNS - 1>();
    if (rows > 0 && !mbar_wait(&full[slot], (b / kPNS) & 1)) {
      if (lane == 0) atomicExch(p.status, 141);
      return;
    }
    __syncwarp();
    const bool flip = contiguous && pstep == 1;
    // normalisation sums of the block: lanes j and j + 16 each sum one half of the row of step j
    float s_cur = 0.f;
    {
      const int u = lane & (kPB - 1), half = lane >> 4;
      if (u < rows) {
        const int hl = L >> 1;  // even halves (L % 4 == 0)
        const float* row = T + (flip ? rows - 1 - u : u) * L + half * hl;
        float sa = 0.f, sb = 0.f;
        int c = lane >= hl ? lane - hl : lane;  // rotated start: lanes hit distinct banks
#pragma unroll 4
        for (int i = 0; i < hl; i += 2) {
          sa += CP ? row[c] + row[c + kPB * L] : row[c];
          c = c + 1 >= hl ? 0 : c + 1;
          sb += CP ? row[c] + row[c + kPB * L] : row[c];
          c = c + 1 >= hl ? 0 : c + 1;
        }
        s_cur = sa + sb;
      }
      s_cur += __shfl_xor_sync(0xffffffffu, s_cur, 16);
    }
    const int send = len - kPB * b < kPB ? len - kPB * b : kPB;
    const float* row = T + (flip ? rows - 1 : 0) * L + c0;
    const int rstep = flip ? -L : L;
    const uint8_t* irow = IT;
    float* drow = dtile + lane;
    for (int sl = 0; sl < send; ++sl, row += rstep, irow += L, drow += 33, pA -= ostep, pB -= ostep, pI -= ostep) {
      const int s = kPB * b + sl;
      const float rq0 = rho * q0, rq1 = rho * q1;
      float qn0 = 0.f, qn1 = 0.f;
      float2 x0 = make_float2(0.f, 0.f), x1 = make_float2(0.f, 0.f);
      if (act && sl < rows) {
        x0 = *reinterpret_cast<const float2*>(row);
        if (CP) x1 = *reinterpret_cast<const float2*>(row + kPB * L);
      }
      if (s < nsteps) {
        const float e = __shfl_sync(0xffffffffu, e_cur, sl);
        const int n = __shfl_sync(0xffffffffu, n_cur, sl);
        const float S = __shfl_sync(0xffffffffu, s_cur, sl);
        float t0 = 0.f, t1 = 0.f, cv0 = 0.f, cv1 = 0.f;
        if (act) {
          const uchar2 fi = *reinterpret_cast<const uchar2*>(irow);
          const int f0 = fi.x, f1 = fi.y;
          t0 = x0.x + x1.x + rq0;
          t1 = x0.y + x1.y + rq1;
          t0 = (c0 == n) ? t0 - S : t0;  // MPLayers/commonCUDA.cuh:131-145
          t1 = (c0 + 1 == n) ? t1 - S : t1;
          cv0 = ctab[c0 * LS + f0];
          cv1 = ctab[(c0 + 1) * LS + f1];
          if (p.ctx_rank == 2) {
            // the diagonal is accumulated like every other cell and dropped at the flush unless wanted
            acc[c0 * LS + f0] = fmaf(e, t0, acc[c0 * LS + f0]);
            acc[(c0 + 1) * LS + f1] = fmaf(e, t1, acc[(c0 + 1) * LS + f1]);
          } else {
            if (c0 != f0 || p.keep_diag) atomicAdd(acc + (c0 > f0 ? c0 - f0 : f0 - c0), e * t0);
            if (c0 + 1 != f1 || p.keep_diag) atomicAdd(acc + (c0 + 1 > f1 ? c0 + 1 - f1 : f1 - c0 - 1), e * t1);
          }
          float* tb = ts + (s & 1) * 64;
          float* ib = is + (s & 1) * 64;
          *reinterpret_cast<float2*>(tb + c0) = make_float2(t0, t1);
          *reinterpret_cast<float2*>(ib + c0) = make_float2((float)f0, (float)f1);
        }
        *drow = fmaf(cv0, t0, cv1 * t1);
        __syncwarp();
        gather_q2<FULL>(ts + (s & 1) * 64, is + (s & 1) * 64, L, (float)c0, qn0, qn1);
      }
      if (act) {
        if (!CP) {
          // scatter field of this direction at this pixel
          *reinterpret_cast<float2*>(pA) = make_float2(q0, q1);
        } else {
          const float2 cn = make_float2(x0.x + rq0, x0.y + rq1);  // dU and every dM_k (k != dir, inv) receive rho*q
          *reinterpret_cast<float2*>(pA) = cn;
          *reinterpret_cast<float2*>(pB) = make_float2(-cn.x, -cn.y);  // dM_dir = C + P_dir = 0 after its sweep
          atomicAdd(pI, -q0);
          atomicAdd(pI + 1, -q1);
        }
      }
      q0 = qn0;
      q1 = qn1;
    }
    // edge-weight gradients of this block: lane j sums row j of the product tile
    __syncwarp();
    if (DE && lane < kPB) {
      const int s = kPB * b + lane;
      if (s < nsteps) {
        const float* row = dtile + lane * 33;
        float da = 0.f, db = 0.f;
#pragma unroll 8
        for (int c = 0; c < 32; c += 2) da += row[c], db += row[c + 1];
        atomicAdd(DE + (pixl - s * pstep), da + db);
      }
    }
    __syncwarp();
    issue_stage(b + kPNS);  // this warp refills the slot it has just consumed
    e_cur = e_nxt;
    n_cur = n_nxt;
  }
  cp_async_wait<0>();

  // flush the context-gradient table of this chain
  __syncwarp();
  float* part = p.dctx_part + (long long)(g % p.n_slots) * (p.ctx_rank == 2 ? L * L : L);
  if (p.ctx_rank == 2) {
    for (int i = lane; i < L * L; i += 32) {
      const int c = i / L, f = i - c * L;
      const float v = acc[c * LS + f];
      if (v != 0.f && (c != f || p.keep_diag)) atomicAdd(part + i, v);
    }
  } else {
    for (int i = lane; i < L; i += 32) {
      const float v = acc[i];
      if (v != 0.f) atomicAdd(part + i, v);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Soft (expected-value) TRWP backward, L <= 32: one warp per chain, lane = label c, C + P scheme.
// Per step the softmin weights of every label are recomputed from the saved edge values,
//   d(value[c][f]) = t[c] * w[c][f] * (1 - value[c][f] + message[c]),
// the scatter q[f] = sum_c d(value[c][f]) goes through a shared-memory transpose and is carried to
// the predecessor pixel in a register; the label-context gradient of row c lives in registers of
// lane c for the whole chain (diagonal included, as in the reference,
// MPLayers/TRWP_hard_soft/TRWP_backward_soft.cu:100-127).
// ------------------------------------------------------------------------------------------------
constexpr int kSoftPF = 4;  // pixels staged ahead (power of two)

__host__ __device__ inline int bwd_soft_slot_floats(int L) {
  // L*L edge values copied as the 16-byte aligned superset of their (4-byte aligned) tile: up to 3
  // floats of slack in front, rounded up to 16 bytes; then the C and P_dir rows (32 floats each)
  return ((L * L + 6) & ~3) + 64;
}
__host__ __device__ inline int bwd_soft_warp_floats(int L) {
  // ring of kSoftPF slots, transpose tile [32][33], kSoftPF mbarriers (2 floats each)
  return kSoftPF * bwd_soft_slot_floats(L) + 32 * 33 + 3 + 2 * kSoftPF;
}

template <int LMAX, bool EXACT>  // EXACT: L == LMAX, every "f < L" test folds away
__global__ void __launch_bounds__(128, 1) bwd_soft_kernel(const __grid_constant__ BwdParams p) {
  extern __shared__ __align__(16) float smem[];
  const int wpb = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = blockIdx.x * wpb + warp;
  BChain ch;
  if (!decode_bchain(p, g, ch)) return;
  const int L = EXACT ? LMAX : p.L, dir = ch.dir, inv = dir ^ 1;
  const int n2 = L * L, slot_floats = bwd_soft_slot_floats(L);
  float* ring = smem + warp * ((bwd_soft_warp_floats(L) + 3) & ~3);   // [kSoftPF][slot_floats]
  float* tile = ring + kSoftPF * slot_floats;            // [32][33]
  unsigned long long* full = reinterpret_cast<unsigned long long*>(
      ring + kSoftPF * slot_floats + ((32 * 33 + 1) & ~1));
  if (lane == 0) {
    for (int i = 0; i < kSoftPF; ++i) mbar_init(&full[i], 1);
    mbar_fence_init();
  }
  __syncwarp();
  const bool act = lane < L;
  const int lc = act ? lane : L - 1;
  const bool l2r = (dir & 1) == 0;

  float cr[LMAX], acc[LMAX];
#pragma unroll
  for (int f = 0; f < LMAX; ++f) {
    cr[f] = (act && f < L) ? ctx_value(p.ctx, p.ctx_rank, L, lane, f) : 0.f;
    acc[f] = 0.f;
  }
  const long long ibase = (long long)ch.img * p.H * p.W;
  float* C = p.dunary + ibase * L + lc;                                   // common part of dM_k
  float* Pd = p.dm_read + (long long)dir * p.slice + ibase * L + lc;      // P_dir
  float* Pi = p.dm_read + (long long)inv * p.slice + ibase * L + lc;      // P_inv
  const float* E = p.ew ? p.ew + (long long)dir * p.pslice + ibase : nullptr;
  float* DE = p.dew ? p.dew + (long long)dir * p.pslice + ibase : nullptr;
  const uint8_t* NI = p.norm_idx + (long long)dir * p.pslice + ibase;
  const float* EL = p.edge_label + ((long long)dir * p.pslice + ibase) * n2;
  const int len = ch.len, pstep = ch.pstep;
  const int pixl = ch.h0 * p.W + ch.w0 + (len - 1) * pstep;  // last pixel of the chain
  const float rho = p.rho;

  // Staging of step s (pixel pixl - s*pstep), kSoftPF steps ahead: its L*L edge values by ONE bulk
  // copy of the 16-byte aligned superset of the tile (the tile itself is only 4-byte aligned; the
  // consumer skips the slack), completion on the warp's own mbarrier; its C and P_dir rows by
  // 4-byte cp.async.  Nothing in the step loop loads from global memory into a register except the
  // per-block scalars.  A superset that would reach past the end of the saved tensor (the very
  // last pixel) is copied element by element instead.
  auto tile_src = [&](int s, unsigned& off_floats, unsigned& bytes, bool& bulk) -> const float* {
    const float* src = EL + (long long)(pixl - s * pstep) * n2;
    const uintptr_t a = reinterpret_cast<uintptr_t>(src);
    off_floats = (unsigned)(a & 15) >> 2;
    bytes = (unsigned)((off_floats + n2) * 4 + 15) & ~15u;
    const float* al = src - off_floats;
    bulk = reinterpret_cast<uintptr_t>(al) + bytes <= reinterpret_cast<uintptr_t>(p.edge_label_end);
    return bulk ? al : src;
  };
  auto issue = [&](int s) {
    if (s < len) {
      const int pxs = pixl - s * pstep;
      const int slot = s & (kSoftPF - 1);
      float* dst = ring + slot * slot_floats;
      if (s < len - 1) {
        unsigned off, bytes;
        bool bulk;
        const float* src = tile_src(s, off, bytes, bulk);
        if (lane == 0) {
          fence_proxy_async_smem();
          mbar_arrive_expect_tx(&full[slot], bulk ? bytes : 0u);
          if (bulk) bulk_g2s(dst, src, bytes, &full[slot]);
        }
        if (!bulk)
          for (int i = lane; i < n2; i += 32) cp_async4(dst + i, src + i);
      }
      if (act) {
        cp_async4(dst + slot_floats - 64 + lane, C + pxs * L);
        cp_async4(dst + slot_floats - 32 + lane, Pd + pxs * L);
      }
    }
    cp_async_commit();
  };
  auto load_blk = [&](int b, float& eb, int& nb) {  // lane l: scalars of step 32*b + l
    const int s = 32 * b + lane;
    eb = 1.f;
    nb = 0;
    if (s < len - 1) {
      const int pxs = pixl - s * pstep;
      if (E) eb = E[pxs];
      nb = NI[pxs];
    }
  };

#pragma unroll
  for (int s = 0; s < kSoftPF; ++s) issue(s);
  float e_cur, e_nxt;
  int n_cur, n_nxt;
  load_blk(0, e_cur, n_cur);
  load_blk(1, e_nxt, n_nxt);

  float q = 0.f;
  int px = pixl;
  for (int s = 0; s < len; ++s) {
    if ((s & 31) == 0 && s) {
      e_cur = e_nxt;
      n_cur = n_nxt;
      load_blk((s >> 5) + 1, e_nxt, n_nxt);
    }
    cp_async_wait<kSoftPF - 1>();
    const float* sl = ring + (s & (kSoftPF - 1)) * slot_floats;
    const float* ev = sl;   // edge values of this pixel inside the slot
    if (s < len - 1) {
      unsigned off, bytes;
      bool bulk;
      tile_src(s, off, bytes, bulk);
      if (!mbar_wait(&full[s & (kSoftPF - 1)], (s / kSoftPF) & 1)) {
        if (lane == 0) atomicExch(p.status, 151);
        return;
      }
      ev = sl + (bulk ? off : 0u);
    }
    __syncwarp();
    const int of = px * L;
    const float c_old = sl[slot_floats - 64 + lc];
    const float x0 = c_old + sl[slot_floats - 32 + lc];   // C + P_dir of this pixel
    const float rq = rho * q;
    float qn = 0.f;
    if (s < len - 1) {
      const float e = __shfl_sync(0xffffffffu, e_cur, s & 31);
      const int n = __shfl_sync(0xffffffffu, n_cur, s & 31);
      float d[LMAX];
#pragma unroll
      for (int f = 0; f < LMAX; ++f) d[f] = (f < L) ? (l2r ? ev[f * L + lc] : ev[lc * L + f]) : kInf;
      float t = act ? x0 + rq : 0.f;
      const float S = warp_sum(t);
      t = (lane == n) ? t - S : t;
      // softmin weights of row c
      float m = d[0];
#pragma unroll
      for (int f = 1; f < LMAX; ++f) m = fminf(m, d[f]);
      float ex[LMAX], se = 0.f, ms = 0.f;
#pragma unroll
      for (int f = 0; f < LMAX; ++f) {
        ex[f] = (f < L) ? __expf(m - d[f]) : 0.f;
        se += ex[f];
      }
      const float inv_se = 1.f / se;
#pragma unroll
      for (int f = 0; f < LMAX; ++f) {
        ex[f] *= inv_se;   // now the weight of candidate f
        ms = (f < L) ? fmaf(ex[f], d[f], ms) : ms;
      }
      float de = 0.f;
#pragma unroll
      for (int f = 0; f < LMAX; ++f) {
        const float dd = (f < L && act) ? t * ex[f] * (1.f - d[f] + ms) : 0.f;
        tile[lane * 33 + f] = dd;
        de = fmaf(cr[f], dd, de);
        acc[f] = fmaf(e, dd, acc[f]);
      }
      de = warp_sum(de);
      if (DE && lane == 0) atomicAdd(DE + px, de);
      __syncwarp();
      if (act) {
        float qa = 0.f, qb = 0.f;
        int c = 0;
        for (; c + 1 < L; c += 2) {
          qa += tile[c * 33 + lane];
          qb += tile[(c + 1) * 33 + lane];
        }
        if (c < L) qa += tile[c * 33 + lane];
        qn = qa + qb;
      }
    }
    if (act) {
      const float cnew = c_old + rq;  // dU and every dM_k (k != dir, inv) receive rho*q
      C[of] = cnew;
      Pd[of] = -cnew;                 // dM_dir = C + P_dir = 0 after its sweep
      atomicAdd(Pi + of, -q);
    }
    __syncwarp();
    issue(s + kSoftPF);
    q = qn;
    px -= pstep;
  }
  cp_async_wait<0>();

  // flush the label-context gradient of this chain (row c = lane)
  float* part = p.dctx_part + (long long)(g % p.n_slots) * (p.ctx_rank == 2 ? L * L : L);
  if (act) {
#pragma unroll
    for (int f = 0; f < LMAX; ++f) {
      if (f < L && acc[f] != 0.f) {
        if (p.ctx_rank == 2) {
          atomicAdd(part + lane * L + f, acc[f]);
        } else {
          atomicAdd(part + (lane > f ? lane - f : f - lane), acc[f]);
        }
      }
    }
  }
}

constexpr int kPFB = 8;  // CTA kernel: pixels of dM_d staged ahead (power of two)

// ------------------------------------------------------------------------------------------------
// L > 32: one CTA per chain, thread = label.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) bwd_cta_kernel(const __grid_constant__ BwdParams p) {
  extern __shared__ __align__(16) float smem[];
  BChain ch;
  if (!decode_bchain(p, blockIdx.x, ch)) return;  // uniform
  const int L = p.L, D = p.D, dir = ch.dir, inv = dir ^ 1, NT = blockDim.x, c = threadIdx.x;
  const int nw = NT >> 5, lane = c & 31, warp = c >> 5;
  const bool qmode = p.cp_scheme == 2;
  const int LS = L | 1;
  float* ring = smem;                          // [kPFB][NT]
  float* ts = ring + kPFB * NT;                // [2][NT]
  int* is = reinterpret_cast<int*>(ts + 2 * NT);  // [2][NT]
  float* red = ts + 4 * NT;                    // [2][16] partial sums, [32..33] cv of the norm label
  float* acc = red + 40;                       // table (rank 2 in smem: L*LS, rank 1: L)
  const bool act = c < L;
  const int tab = p.ctx_rank == 2 ? (p.table_in_smem ? L * LS : 0) : L;
  for (int i = c; i < tab; i += NT) acc[i] = 0.f;
  is[c] = -1;
  is[NT + c] = -1;
  __syncthreads();

  const long long ibase = (long long)ch.img * p.H * p.W;
  float* DMr = p.dm_read + (long long)dir * p.slice + ibase * L;
  float* DMa = p.dm_acc + ibase * L;
  float* DU = p.dunary + ibase * L;
  const float* E = p.ew ? p.ew + (long long)dir * p.pslice + ibase : nullptr;
  float* DE = p.dew ? p.dew + (long long)dir * p.pslice + ibase : nullptr;
  const uint8_t* MI = p.min_idx + (long long)dir * p.slice + ibase * L;
  const uint8_t* NI = p.norm_idx + (long long)dir * p.pslice + ibase;
  const int len = ch.len;
  const int pixl = ch.h0 * p.W + ch.w0 + (len - 1) * ch.pstep;
  const float rho = p.rho;
  float* part = p.dctx_part + (long long)(blockIdx.x % p.n_slots) * (p.ctx_rank == 2 ? L * L : L);

  auto issue = [&](int s) {
    if (s < len - 1 && act)
      cp_async4(ring + (s & (kPFB - 1)) * NT + c, DMr + (long long)(pixl - s * ch.pstep) * L + c);
    cp_async_commit();
  };
  auto load_idx = [&](int s) -> int {
    return (s < len - 1 && act) ? (int)MI[(long long)(pixl - s * ch.pstep) * L + c] : -1;
  };
  auto load_blk = [&](int b, float& eb, int& nb) {
    const int s = 32 * b + lane;
    eb = 1.f;
    nb = 0;
    if (s < len - 1) {
      const int px = pixl - s * ch.pstep;
      if (E) eb = E[px];
      nb = NI[px];
    }
  };

#pragma unroll
  for (int s = 0; s < kPFB; ++s) issue(s);
  int i0 = load_idx(0), i1 = load_idx(1), i2 = load_idx(2), i3 = load_idx(3);
  float e_cur, e_nxt;
  int n_cur, n_nxt;
  load_blk(0, e_cur, n_cur);
  load_blk(1, e_nxt, n_nxt);

  float q = 0.f;
  for (int s = 0; s < len; ++s) {
    if ((s & 31) == 0 && s) {
      e_cur = e_nxt;
      n_cur = n_nxt;
      load_blk((s >> 5) + 1, e_nxt, n_nxt);
    }
    cp_async_wait<kPFB - 1>();
    const int px = pixl - s * ch.pstep;
    const long long o = (long long)px * L + c;
    const bool has_front = s < len - 1;
    const float rq = rho * q;
    float qn = 0.f;
    if (has_front) {
      const float e = __shfl_sync(0xffffffffu, e_cur, s & 31);
      const int n = __shfl_sync(0xffffffffu, n_cur, s & 31);
      const int f = i0;
      const float t0 = act ? ring[(s & (kPFB - 1)) * NT + c] + rq : 0.f;
      const float cv = act ? ctx_value(p.ctx, p.ctx_rank, L, c, f) : 0.f;
      float S = t0, P = cv * t0;
      warp_sum2(S, P);
      float* rb = red + (s & 1) * 16;
      if (lane == 0) {
        rb[warp] = S;
        rb[8 + warp] = P;
      }
      if (c == n) red[32 + (s & 1)] = cv;
      __syncthreads();
      S = 0.f;
      P = 0.f;
      for (int w = 0; w < nw; ++w) {
        S += rb[w];
        P += rb[8 + w];
      }
      const float cn = red[32 + (s & 1)];
      const float t = (c == n) ? t0 - S : t0;
      if (DE && c == 0) atomicAdd(DE + px, P - cn * S);
      if (act && (c != f || p.keep_diag)) {
        if (p.ctx_rank == 2) {
          if (p.table_in_smem) {
            acc[c * LS + f] += e * t;
          } else {
            atomicAdd(part + c * L + f, e * t);
          }
        } else {
          atomicAdd(acc + (c > f ? c - f : f - c), e * t);
        }
      }
      float* tb = ts + (s & 1) * NT;
      int* ib = is + (s & 1) * NT;
      tb[c] = t;
      if (act) ib[c] = f;
      __syncthreads();
      for (int k = 0; k < L; ++k)
        if (ib[k] == c) qn += tb[k];
    }
    if (act) {
      if (qmode) {
        DMa[(long long)dir * p.slice + o] = q;  // scatter field of this direction at this pixel
      } else {
        for (int k = 0; k < D; ++k) {
          if (k == dir) continue;
          atomicAdd(DMa + k * p.slice + o, k == inv ? fmaf(rho, q, -q) : rq);
        }
        atomicAdd(DU + o, rq);
        DMr[o] = 0.f;
      }
    }
    issue(s + kPFB);
    i0 = i1;
    i1 = i2;
    i2 = i3;
    i3 = load_idx(s + 4);
    q = qn;
  }
  cp_async_wait<0>();

  __syncthreads();
  if (p.ctx_rank == 2) {
    if (p.table_in_smem)
      for (int i = c; i < L * L; i += NT) {
        const float v = acc[(i / L) * LS + (i % L)];
        if (v != 0.f) atomicAdd(part + i, v);
      }
  } else if (act) {
    const float v = acc[c];
    if (v != 0.f) atomicAdd(part + c, v);
  }
}

// Prologue.  cp_scheme 0: dunary = factor * g, dM_k = g for every k (MPLayers/TRWP/TRWP_backward.cu:8-24,
// MPLayers/ISGMR/ISGMR_backward.cu:18-37).  cp_scheme 1: C = g, P_k = 0.
__global__ void backward_init_kernel(const float* __restrict__ g, float* __restrict__ dunary,
                                     float* __restrict__ dm, long long n, int D, float factor, int cp) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = g[i];
    dunary[i] = cp ? v : factor * v;
    for (int k = 0; k < D; ++k) dm[k * n + i] = cp ? 0.f : v;
  }
}

// The same prologue reading g with the labels first ([nimg, L, H*W] planes): one block per 32 pixels
// of an image, through a shared-memory tile.
__global__ void __launch_bounds__(256)
backward_init_lhw_kernel(const float* __restrict__ g, float* __restrict__ dunary, float* __restrict__ dm, int L,
                         long long HW, long long n, int D, float factor, int cp) {
  extern __shared__ float tile[];  // [L][33]
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long long b = blockIdx.y, p0 = blockIdx.x * 32ll;
  const int np = HW - p0 < 32 ? (int)(HW - p0) : 32;
  const float* src = g + b * L * HW + p0;
  for (int l = ty; l < L; l += 8) tile[l * 33 + tx] = tx < np ? src[(long long)l * HW + tx] : 0.f;
  __syncthreads();
  const long long base = (b * HW + p0) * L;
  for (int i = threadIdx.x; i < np * L; i += 256) {
    const int px = i / L, l = i - px * L;
    const float v = tile[l * 33 + px];
    dunary[base + i] = cp ? v : factor * v;
    for (int k = 0; k < D; ++k) dm[k * n + base + i] = cp ? 0.f : v;
  }
}

// ISGMR, cp_scheme 2: after the D independent sweeps of an iteration have stored their scatter
// fields q_d, the gradients of the messages that iteration read are
//   dM_k = rho * Q - rho * q_k - q_inv(k),   Q = sum_d q_d,   and   dU += rho * Q
// (what the reference accumulates with D+3 atomics per element and sweep,
// MPLayers/ISGMR/ISGMR_backward.cu:39-60, followed by SumMsgKernel and a copy, :482-483).
__global__ void isgmr_combine_kernel(const float* __restrict__ q, float* __restrict__ dm,
                                     float* __restrict__ dunary, long long n, int D, float rho) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float qv[16];
    float Q = 0.f;
    for (int d = D - 1; d >= 0; --d) {  // the order in which the reference's sweeps add
      qv[d] = q[d * n + i];
      Q += qv[d];
    }
    const float rQ = rho * Q;
    dunary[i] += rQ;
    for (int k = 0; k < D; ++k) dm[k * n + i] = (rQ - rho * qv[k]) - qv[k ^ 1];
  }
}

// The same with Q given (summed over ALL directions, possibly on other GPUs) and only the
// directions [dir0, dir0 + ndirs) held here; dunary may be null (then only the messages' part).
__global__ void isgmr_combine_total_kernel(const float* __restrict__ Qt, const float* __restrict__ q,
                                           float* __restrict__ dm, float* __restrict__ dunary, long long n,
                                           int dir0, int ndirs, float rho) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float rQ = rho * Qt[i];
    if (dunary) dunary[i] += rQ;
    for (int k = dir0; k < dir0 + ndirs; ++k) dm[k * n + i] = (rQ - rho * q[k * n + i]) - q[(k ^ 1) * n + i];
  }
}

// out = base * factor + sum of nf consecutive fields (base may be null: plain sum), ascending order
__global__ void sum_fields_kernel(const float* __restrict__ base, float factor, const float* __restrict__ f,
                                  int nf, long long n, long long stride, float* __restrict__ out) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float v = base ? base[i] * factor : 0.f;
    for (int k = 0; k < nf; ++k) v += f[k * stride + i];
    out[i] = v;
  }
}

// Sums the per-slot partial tables in slot order (two fixed-order levels) and folds them into the
// caller's dcontext with the reference's addressing (MPLayers/TRWP/TRWP_backward.cu:102-112):
// rank 2 -> cell [min(c,f)][max(c,f)], rank 1 -> cell |c-f|.
constexpr int kRedChunks = 64;

__global__ void dctx_reduce1_kernel(float* __restrict__ part, int n_slots, int CT) {
  // chunk y sums slots y, y + kRedChunks, ... into slot y (in place; slot y is only read by chunk y)
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int y = blockIdx.y;
  if (i >= CT || y >= n_slots) return;
  float s = 0.f;
  for (int k = y; k < n_slots; k += kRedChunks) s += part[(long long)k * CT + i];
  part[(long long)y * CT + i] = s;
}

__global__ void dctx_reduce2_kernel(const float* __restrict__ part, int n_slots, int L, int rank,
                                    float* __restrict__ dctx) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int CT = rank == 2 ? L * L : L;
  if (i >= CT) return;
  const int n = n_slots < kRedChunks ? n_slots : kRedChunks;
  if (rank == 2) {
    const int a = i / L, b = i % L;
    if (a > b) return;
    float s = 0.f;
    if (a == b) {
      for (int k = 0; k < n; ++k) s += part[(long long)k * CT + i];
    } else {
      const int j = b * L + a;
      for (int k = 0; k < n; ++k) s += part[(long long)k * CT + i] + part[(long long)k * CT + j];
    }
    dctx[i] += s;
  } else {
    float s = 0.f;
    for (int k = 0; k < n; ++k) s += part[(long long)k * CT + i];
    dctx[i] += s;
  }
}

constexpr int kSmemTableMaxL = 128;  // rank-2 table L*(L|1) floats fits next to the staging ring

size_t bwd_tma_smem_bytes(int L, int rank, int stages) {
  return ((size_t)stages * 2 * kBK * 4 * L + ((L * (L | 1) + 3) & ~3) + 4 * (size_t)bwd_tma_warp_floats(L, rank)) *
             sizeof(float) +
         2 * stages * 8 + 16 + 128;
}

bool bwd_tma_eligible(const BwdParams& p) {
  if (p.cp_scheme == 0 || p.dir > 3 || p.L > 32 || p.ndirs > 1) return false;
  if ((p.W & 3) || (((long long)p.W * p.L) & 3)) return false;
  if (((uintptr_t)(p.cp_scheme == 1 ? p.dunary : nullptr) | (uintptr_t)p.dm_read) & 15) return false;
  return true;
}

bool bwd_pair_eligible(const BwdParams& p) {
  if (p.L <= 32 || p.L > 64 || (p.L & 3) || p.cp_scheme == 0) return false;
  if (((uintptr_t)p.dunary | (uintptr_t)p.dm_read | (uintptr_t)p.dm_acc) & 15) return false;
  const char* e = getenv("MPL_NO_PAIR");  // tuning / comparison knob
  return !(e && e[0] == '1');
}

template <int LT>
cudaError_t launch_bwd_tma(const BwdParams& p, cudaStream_t st) {
  const bool vert = p.dir >= 2;
  const bool rev = (p.dir & 1) == 0;  // forward walk upwards -> backward walk downwards
  const int groups = vert ? p.nimg * (p.W >> 2) : (p.nimg * p.H + 3) >> 2;
  const size_t smem = bwd_tma_smem_bytes(p.L, p.ctx_rank, p.tma_stages);
  TmaMaps maps{};
  const bool qm = p.cp_scheme == 2;
  if (vert) {
    const unsigned long long inner = (unsigned long long)p.W * p.L, rows = (unsigned long long)p.nimg * p.H;
    if ((!qm && !encode_tmap_2d(&maps.a, p.dunary, inner, rows, 4 * p.L, kBK)) ||
        !encode_tmap_2d(&maps.b, p.dm_read, inner, rows * p.D, 4 * p.L, kBK))
      return cudaErrorNotSupported;
  }
  auto go = [&](auto kernel) -> cudaError_t {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
    }
    kernel<<<groups, 160, smem, st>>>(p, maps);
    return cudaSuccess;
  };
  if (qm) {
    if (vert) return rev ? go(bwd_tma_kernel<LT, true, true, true>) : go(bwd_tma_kernel<LT, true, false, true>);
    return rev ? go(bwd_tma_kernel<LT, false, true, true>) : go(bwd_tma_kernel<LT, false, false, true>);
  }
  if (vert) return rev ? go(bwd_tma_kernel<LT, true, true>) : go(bwd_tma_kernel<LT, true, false>);
  return rev ? go(bwd_tma_kernel<LT, false, true>) : go(bwd_tma_kernel<LT, false, false>);
}

}  // namespace

cudaError_t launch_isgmr_combine(const float* q, float* dm, float* dunary, long long n, int D, float rho,
                                 cudaStream_t st) {
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  ProfScope prof(kProfElementwise, st);
  isgmr_combine_kernel<<<(int)blocks, 256, 0, st>>>(q, dm, dunary, n, D, rho);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_isgmr_combine_total(const float* q_total, const float* q, float* dm, float* dunary, long long n,
                                       int dir0, int ndirs, float rho, cudaStream_t st) {
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  ProfScope prof(kProfElementwise, st);
  isgmr_combine_total_kernel<<<(int)blocks, 256, 0, st>>>(q_total, q, dm, dunary, n, dir0, ndirs, rho);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_sum_fields(const float* base, float factor, const float* fields, int nf, long long n,
                              long long stride, float* out, cudaStream_t st) {
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  ProfScope prof(kProfElementwise, st);
  sum_fields_kernel<<<(int)blocks, 256, 0, st>>>(base, factor, fields, nf, n, stride, out);
  count_launch();
  return cudaGetLastError();
}

int backward_slots(int H, int W, int L, int D, int nimg, int rank) {
  // One partial table per chain of a launch, so that every table has a single writer per launch and
  // the sums are run-to-run identical.  A launch covers one direction (TRWP) or all of them (ISGMR);
  // the call does not know which, so the larger count is provisioned while the tables stay within
  // 256 MB, else the largest direction's count, else 4096 slots shared through atomic adds (then
  // the order of the additions, and with it the last bits of the gradient, can vary between runs).
  long long mx = 1, sum = 0;
  for (int d = 0; d < D; ++d) {
    const long long n = (long long)make_geom(d, H, W).n_chains * nimg;
    if (n > mx) mx = n;
    sum += n;
  }
  const long long table = (long long)(rank == 2 ? L * L : L) * (long long)sizeof(float);
  const long long budget = 256ll << 20;
  if (sum * table <= budget || sum <= 4096) return (int)sum;
  if (mx * table <= budget || mx <= 4096) return (int)mx;
  return 4096;
}

cudaError_t launch_backward_init(const float* dcost, float* dunary, float* dm, long long n, int D,
                                 float factor, int cp_scheme, cudaStream_t st) {
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  ProfScope prof(kProfElementwise, st);
  backward_init_kernel<<<(int)blocks, 256, 0, st>>>(dcost, dunary, dm, n, D, factor, cp_scheme);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_backward_init_lhw(const float* dcost, float* dunary, float* dm, int nimg, int L, long long HW,
                                     int D, float factor, int cp_scheme, cudaStream_t st) {
  const dim3 grid((unsigned)((HW + 31) / 32), (unsigned)nimg);
  const size_t smem = (size_t)L * 33 * sizeof(float);
  ProfScope prof(kProfElementwise, st);
  backward_init_lhw_kernel<<<grid, 256, smem, st>>>(dcost, dunary, dm, L, HW, (long long)nimg * HW * L, D, factor,
                                                    cp_scheme);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_backward_sweep(const BwdParams& p0, cudaStream_t st) {
  BwdParams p = p0;
  if (p.ndirs < 1) p.ndirs = 1;
  if (p.cp_scheme == 2 && p.L <= 32 && p.ndirs > 1 && p.parts <= 1 &&
      (long long)p.nimg * (p.H < p.W ? p.H : p.W) >= 256) {
    // ISGMR, L <= 32: the axis directions whose rows are 16-byte aligned go to the bulk-copy kernel
    // one by one (the sweeps are independent), the rest to one launch of the generic kernel.
    // Small problems (few chains per direction) stay with one launch over all directions.
    int d = p.dir;
    const int end = p.dir + p.ndirs;
    for (; d < end && d <= 3; ++d) {
      BwdParams one = p;
      one.dir = d;
      one.ndirs = 1;
      if (!bwd_tma_eligible(one)) break;
      cudaError_t e = launch_backward_sweep(one, st);
      if (e != cudaSuccess) return e;
    }
    if (d == end) return cudaSuccess;
    p.ndirs = end - d;  // the remaining range continues below
    p.dir = d;
  }
  p.chain_off[0] = 0;
  for (int i = 0; i < p.ndirs; ++i) {
    int begin, count;
    chain_part((long long)make_geom(p.dir + i, p.H, p.W).n_chains * p.nimg, p.part, p.parts, begin, count);
    p.chain_begin[i] = begin;
    p.chain_off[i + 1] = p.chain_off[i] + count;
  }
  const int total = p.chain_off[p.ndirs];
  if (total == 0) return cudaSuccess;
  const int L = p.L, LS = L | 1;
  ProfScope prof(kProfBwdSweep, st);
  if (L <= 32 && p.parts <= 1 && bwd_tma_eligible(p)) {
    p.tma_stages = tma_stage_override() ? tma_stage_override() : 4;
    cudaError_t e = L == 21 ? launch_bwd_tma<21>(p, st) : launch_bwd_tma<0>(p, st);
    if (e != cudaSuccess) return e;
  } else if (L <= 32) {
    const int wpb = total >= 148 * 32 ? 4 : 1;
    const size_t smem = ((size_t)((L * LS + 3) & ~3) + (size_t)wpb * bwd_warp_floats(L, p.ctx_rank, p.cp_scheme == 1)) *
                        sizeof(float);
    auto go = [&](auto kernel) -> cudaError_t {
      if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
      }
      kernel<<<(total + wpb - 1) / wpb, wpb * 32, smem, st>>>(p);
      return cudaSuccess;
    };
    cudaError_t e;
    if (p.cp_scheme == 1) {
      e = go(bwd_warp_kernel<0, 1>);
    } else if (p.cp_scheme == 2) {
      e = go(bwd_warp_kernel<0, 2>);
    } else {
      e = p.D == 4 ? go(bwd_warp_kernel<4, 0>) : p.D == 8 ? go(bwd_warp_kernel<8, 0>) : go(bwd_warp_kernel<0, 0>);
    }
    if (e != cudaSuccess) return e;
  } else if (bwd_wide_eligible(L, p.ctx_rank, p.cp_scheme, p.dunary, p.dm_read, p.dm_acc)) {
    // rank-1 context, 32 < L <= 256: several labels per lane, scatter split into near and far indices
    cudaError_t e = launch_backward_wide(p, total, st);
    if (e != cudaSuccess) return e;
  } else if (bwd_pair_eligible(p)) {
    const size_t per_warp = (size_t)((bwd_pair_floats(L, p.ctx_rank, p.cp_scheme) + 3) & ~3) * sizeof(float);
    const size_t table = (size_t)((L * LS + 3) & ~3) * sizeof(float);
    int wpb = (int)((227 * 1024 - table) / per_warp);
    wpb = wpb > 8 ? 8 : wpb;
    const size_t smem = table + per_warp * wpb;
    auto go = [&](auto kernel) -> cudaError_t {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      kernel<<<(total + wpb - 1) / wpb, wpb * 32, smem, st>>>(p);
      return cudaSuccess;
    };
    cudaError_t e;
    if (L == 64) {
      e = p.cp_scheme == 1 ? go(bwd_pair_kernel<1, true>) : go(bwd_pair_kernel<2, true>);
    } else {
      e = p.cp_scheme == 1 ? go(bwd_pair_kernel<1, false>) : go(bwd_pair_kernel<2, false>);
    }
    if (e != cudaSuccess) return e;
  } else {
    const int NT = ((L + 31) / 32) * 32;
    p.table_in_smem = (p.ctx_rank == 2 && L <= kSmemTableMaxL) ? 1 : 0;
    const int tab = p.ctx_rank == 2 ? (p.table_in_smem ? L * LS : 0) : L;
    const size_t smem = ((size_t)kPFB * NT + 4 * NT + 40 + tab + 4) * sizeof(float);
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(bwd_cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
    }
    bwd_cta_kernel<<<total, NT, smem, st>>>(p);
  }
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_backward_soft_sweep(const BwdParams& p0, cudaStream_t st) {
  BwdParams p = p0;
  p.ndirs = 1;
  p.parts = 0;
  p.chain_begin[0] = 0;
  p.chain_off[0] = 0;
  p.chain_off[1] = make_geom(p.dir, p.H, p.W).n_chains * p.nimg;
  const int total = p.chain_off[1];
  if (total == 0) return cudaSuccess;
  if (p.cp_scheme != 1) return cudaErrorNotSupported;
  if (p.L > 32) return launch_backward_soft_cta(p, total, st);  // one CTA per chain, up to 64 labels
  const int wpb = 4;
  const size_t smem = (size_t)wpb * ((bwd_soft_warp_floats(p.L) + 3) & ~3) * sizeof(float);
  auto go = [&](auto kernel) -> cudaError_t {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
    }
    kernel<<<(total + wpb - 1) / wpb, wpb * 32, smem, st>>>(p);
    return cudaSuccess;
  };
  ProfScope prof(kProfBwdSweep, st);
  cudaError_t e = p.L == 21 ? go(bwd_soft_kernel<21, true>)
                  : p.L < 21 ? go(bwd_soft_kernel<21, false>) : go(bwd_soft_kernel<32, false>);
  if (e != cudaSuccess) return e;
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_dctx_reduce(float* part, int n_slots, int L, int rank, int keep_diag, float* dctx,
                               cudaStream_t st) {
  (void)keep_diag;  // the diagonal is filtered where the table is accumulated
  const int CT = rank == 2 ? L * L : L;
  if (n_slots > kRedChunks) {
    dctx_reduce1_kernel<<<dim3((CT + 127) / 128, kRedChunks), 128, 0, st>>>(part, n_slots, CT);
    count_launch();
  }
  dctx_reduce2_kernel<<<(CT + 127) / 128, 128, 0, st>>>(part, n_slots, L, rank, dctx);
  count_launch();
  return cudaGetLastError();
}

}  // namespace mpl
