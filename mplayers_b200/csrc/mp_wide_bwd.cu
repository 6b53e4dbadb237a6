// Backward sweep for a rank-1 context with 32 < L <= 256 labels, L % 4 == 0 (learning a truncated
// linear / quadratic function on stereo- or denoising-sized label sets): one WARP per chain, LPT
// consecutive labels per lane, schemes 1 (C + P bookkeeping, TRWP) and 2 (scatter field, ISGMR).
// Replaces, for those problems, the reference's backward chain kernels with one thread per label,
// a block barrier per candidate and D + 1 global reductions per label and step
// (MPLayers/TRWP/TRWP_backward.cu:26-275).
#include <cstdlib>
#include <type_traits>

#include "mp_common.cuh"
#include "mp_minplus.cuh"

namespace mpl {

namespace {

constexpr int kWNS = 2;  // stages in flight per warp

// Floats of shared memory per warp: staged gradients [kWNS][NA][K][L], argmin indices
// [kWNS][K][L] bytes, product tile [16][33], t and index-as-float windows [2][2][LP + 2G], the
// chain's label-context gradient table by SIGNED offset c - f [2L], the far scatter buffer [LP],
// kWNS mbarriers.
__host__ __device__ inline int bwd_wide_floats(int L, int lp, int g, int K, int na) {
  return kWNS * na * K * L + kWNS * K * L / 4 + 16 * 33 + 4 * (lp + 2 * g) + ((2 * L + 3) & ~3) + lp + 2 * kWNS + 2;
}

// Two adjacent floats added to global memory with one reduction (8-byte aligned address).
__device__ __forceinline__ void red_add_v2(float* addr, float a, float b) {
  asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(__cvta_generic_to_global(addr)), "f"(a), "f"(b)
               : "memory");
}

// ------------------------------------------------------------------------------------------------
// One step of the replay at pixel `cur` with saved indices f[c] = argmin of label c:
//   t[c]  = dM_dir[cur][c] + rho * q[c];  t[n] -= sum_c t[c]          (n = normalisation index)
//   q'[f] = sum over c with f[c] == f of t[c]                          (carried to the predecessor)
//   dE[cur] += sum_c ctx[|c - f[c]|] * t[c];   dctx[|c - f[c]|] += E * t[c]
// The scatter q' is split by the distance |c - f[c]|:
//  * near (< RW): lane-local gather over the 2 RW - 1 neighbours of each of its labels from a
//    window of t and f in shared memory -- per candidate one compare-to-flag, one multiply and two
//    adds, the second add accumulating the per-offset sums of the label-context gradient in
//    registers;
//  * far: with a context that saturates, every label whose minimum came through the saturated value
//    points at the SAME label (the one with the smallest h), so the far labels that share the
//    target of the first of them are summed with one warp reduction and handed to the target's
//    lane; whatever is left after that round (other targets: possible only among exactly tied
//    candidates, or with a context that does not saturate) goes through shared-memory atomics.
//    The label-context gradient of the far labels is kept by SIGNED offset c - f: the labels that
//    share a target then own distinct cells, so the round adds to them without atomics (float
//    atomics on shared memory are compare-and-swap loops); the two signs are folded at the end.
// With RW == 2 the only neighbours outside a lane are one label on each side: they come by
// shuffle, the gather compares integer indices in registers, and nothing goes through shared memory.
// RW is a tuning parameter only: any split gives the same sums.
// ------------------------------------------------------------------------------------------------
template <int LPT, int RW, int SCH>
__global__ void __launch_bounds__(32, 8) bwd_wide_kernel(const __grid_constant__ BwdParams p) {
  constexpr bool CP = SCH == 1;
  constexpr int NA = CP ? 2 : 1;  // staged arrays: (C, P_dir) or the gradient slice of the direction
  constexpr int LP = 32 * LPT;
  constexpr int G = RW & ~1;      // guard band (floats, even) on both sides of the window buffers
  constexpr int WB = LP + 2 * G;
  constexpr int NWV = (LPT + 2 * G) / 2;  // float2 loads covering a lane's window
  extern __shared__ __align__(128) float smem[];
  const int lane = threadIdx.x;
  const int L = p.L, K = p.tma_k;
  float* ring = smem;                                        // [kWNS][NA][K][L]
  const int stage_floats = NA * K * L;
  uint8_t* itile = reinterpret_cast<uint8_t*>(ring + kWNS * stage_floats);  // [kWNS][K][L]
  float* dtile = ring + kWNS * stage_floats + kWNS * K * L / 4;             // [16][33]
  float* tbuf = dtile + 16 * 33;                             // [2][WB]
  float* ibuf = tbuf + 2 * WB;                               // [2][WB] argmin as float
  float* acc = ibuf + 2 * WB;                                // [2L] label-context gradient of the chain, cell L + c - f
  float* qfar = acc + ((2 * L + 3) & ~3);                    // [LP]
  unsigned long long* full = reinterpret_cast<unsigned long long*>(qfar + LP);
  float* ctab = reinterpret_cast<float*>(full + kWNS + 1);   // [L] the context
  if (lane == 0) {
    for (int i = 0; i < kWNS; ++i) mbar_init(&full[i], 1);
    mbar_fence_init();
  }
  for (int i = lane; i < L; i += 32) {
    acc[i] = 0.f;
    acc[L + i] = 0.f;
    ctab[i] = __ldg(p.ctx + i);
  }
  for (int i = lane; i < 2 * WB; i += 32) tbuf[i] = 0.f, ibuf[i] = -1.f;
  for (int i = lane; i < LP; i += 32) qfar[i] = 0.f;
  __syncwarp();
  BChain ch;
  if (!decode_bchain(p, blockIdx.x, ch)) return;
  const int dir = ch.dir, inv = dir ^ 1;
  const int c0 = LPT * lane;
  const int nl = L - c0 < 0 ? 0 : (L - c0 < LPT ? L - c0 : LPT);  // labels of this lane that exist
  const bool whole = nl == LPT;

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
  const int nblocks = (len + K - 1) / K;

  auto stage_rows = [&](int b) {
    const int r = nrows - K * b;
    return r < 0 ? 0 : (r > K ? K : r);
  };
  // step s = K*b + u visits image pixel pixl - s*pstep; its row in the stage tile is u, except for
  // chains walked towards decreasing addresses in one copy (pstep == +1), which land reversed
  auto issue_stage = [&](int b) {
    const int rows = stage_rows(b);
    const int slot = b % kWNS;
    const int s0 = K * b;
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
          bulk_g2s(T + lane * K * L, (CP && lane == 0 ? DU : DMr) + (long long)first * L,
                   (unsigned)(rows * L) * 4u, &full[slot]);
      } else {
        for (int q = lane; q < rows * NA; q += 32) {
          const int u = q / NA, a = q - u * NA;
          const int px = pixl - (s0 + u) * pstep;
          bulk_g2s(T + (a * K + u) * L, (CP && a == 0 ? DU : DMr) + (long long)px * L, (unsigned)L * 4u,
                   &full[slot]);
        }
      }
    }
    // argmin indices of the steps with a predecessor
    for (int u = 0; u < K; ++u) {
      if (s0 + u >= nsteps) break;
      uint8_t* dst = itile + (slot * K + u) * L;
      const uint8_t* src = MI + (long long)(pixl - (s0 + u) * pstep) * L;
      for (int j = 4 * lane; j < L; j += 128)
        cp_async4(reinterpret_cast<float*>(dst + j), reinterpret_cast<const float*>(src + j));
    }
    cp_async_commit();
  };
  auto load_blk = [&](int b, float& eb, int& nb) {  // lane l: scalars of step K*b + (l & (K - 1))
    const int s = K * b + (lane & (K - 1));
    eb = 1.f;
    nb = 0;
    if (s < nsteps) {
      const int px = pixl - s * pstep;
      if (E) eb = E[px];
      nb = NI[px];
    }
  };

  for (int b = 0; b < kWNS; ++b) issue_stage(b);
  float e_cur, e_nxt;
  int n_cur, n_nxt;
  load_blk(0, e_cur, n_cur);

  float q[LPT], ack[RW];
#pragma unroll
  for (int i = 0; i < LPT; ++i) q[i] = 0.f;  // scatter sums carried from the successor pixel
#pragma unroll
  for (int k = 0; k < RW; ++k) ack[k] = 0.f;  // near offsets of the label-context gradient (this lane's share)
  // output pointers of the current pixel (label c0), moved by one pixel per step
  float* pA = (CP ? DU : DMa + (long long)dir * p.slice) + (long long)pixl * L + c0;  // C, or the scatter field
  float* pB = DMr + (long long)pixl * L + c0;                                         // P_dir
  float* pI = DMa + (long long)inv * p.slice + (long long)pixl * L + c0;              // P_inv
  const bool flip = contiguous && pstep == 1;

  // One step.  FULL (warp-uniform): all 32 * LPT labels exist, no per-label bounds tests.  FRONT: the
  // pixel has a predecessor on the chain (all but the chain's first pixel, which only stores).
  auto step = [&](auto full_c, auto front_c, const float* row, const uint8_t* irow, float* drow, int sl) {
    constexpr bool FULL = decltype(full_c)::value;
    constexpr bool has_front = decltype(front_c)::value;
    constexpr bool staged = has_front || CP;  // the scatter-field scheme stages no row for the first pixel
    float rq[LPT], x0[LPT], x1[LPT], qn[LPT];
#pragma unroll
    for (int i = 0; i < LPT; ++i) rq[i] = rho * q[i], x0[i] = 0.f, x1[i] = 0.f, qn[i] = 0.f;
    if (staged) {
      if (FULL || whole) {
#pragma unroll
        for (int v = 0; v < LPT / 2; ++v) {
          const float2 a = reinterpret_cast<const float2*>(row)[v];
          x0[2 * v] = a.x, x0[2 * v + 1] = a.y;
          if (CP) {
            const float2 c = reinterpret_cast<const float2*>(row + K * L)[v];
            x1[2 * v] = c.x, x1[2 * v + 1] = c.y;
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < LPT; ++i) {
          if (i < nl) {
            x0[i] = row[i];
            if (CP) x1[i] = row[K * L + i];
          }
        }
      }
    }
    if constexpr (has_front) {
      const float e = __shfl_sync(0xffffffffu, e_cur, sl);
      const int n = __shfl_sync(0xffffffffu, n_cur, sl);
      float xs[LPT];
#pragma unroll
      for (int i = 0; i < LPT; ++i) xs[i] = CP ? x0[i] + x1[i] : x0[i];
      // normalisation sum over the stored gradient of this pixel
      float ps = 0.f;
#pragma unroll
      for (int i = 0; i < LPT; ++i) ps += xs[i];
      const float S = warp_sum(ps);
      int f[LPT], kd[LPT];
      float t[LPT];
      if (FULL || whole) {
#pragma unroll
        for (int v = 0; v < LPT / 2; ++v) {
          const uchar2 fi = *reinterpret_cast<const uchar2*>(irow + 2 * v);
          f[2 * v] = fi.x, f[2 * v + 1] = fi.y;
        }
      } else {
#pragma unroll
        for (int i = 0; i < LPT; ++i) f[i] = i < nl ? (int)irow[i] : c0 + i;
      }
      float de = 0.f;
      const int jn = n - c0;  // position of the normalisation label inside this lane, if it is here
#pragma unroll
      for (int i = 0; i < LPT; ++i) {
        const float ti = xs[i] + rq[i];
        t[i] = (i == jn) ? ti - S : ti;  // MPLayers/commonCUDA.cuh:131-145
        const int d = c0 + i - f[i];
        kd[i] = d < 0 ? -d : d;
        if (FULL || i < nl) de = fmaf(ctab[kd[i]], t[i], de);
      }
      *drow = de;
      // ---- near: gather over the window of each label of this lane ----
      if constexpr (RW == 2) {
        const float tl = __shfl_up_sync(0xffffffffu, t[LPT - 1], 1), tr = __shfl_down_sync(0xffffffffu, t[0], 1);
        int fl = __shfl_up_sync(0xffffffffu, f[LPT - 1], 1), fr = __shfl_down_sync(0xffffffffu, f[0], 1);
        fl = lane == 0 ? -1 : fl;
        fr = lane == 31 ? -1 : fr;
        float sk0 = 0.f, sk1 = 0.f;
#pragma unroll
        for (int i = 0; i < LPT; ++i) {
          const int me = c0 + i;
          const float tlv = i == 0 ? tl : t[i == 0 ? 0 : i - 1];
          const int flv = i == 0 ? fl : f[i == 0 ? 0 : i - 1];
          const float trv = i == LPT - 1 ? tr : t[i == LPT - 1 ? i : i + 1];
          const int frv = i == LPT - 1 ? fr : f[i == LPT - 1 ? i : i + 1];
          const float a = flv == me ? tlv : 0.f, b = f[i] == me ? t[i] : 0.f, c = frv == me ? trv : 0.f;
          const float ac = a + c;
          qn[i] = ac + b;
          sk0 += b;
          sk1 += ac;
        }
        ack[0] = fmaf(e, sk0, ack[0]);
        ack[1] = fmaf(e, sk1, ack[1]);
        __syncwarp();  // orders the table updates of successive steps
      } else {
        float* tb = tbuf + (sl & 1) * WB + G;
        float* ib = ibuf + (sl & 1) * WB + G;
        if (FULL || whole) {
#pragma unroll
          for (int v = 0; v < LPT / 2; ++v) {
            reinterpret_cast<float2*>(tb + c0)[v] = make_float2(t[2 * v], t[2 * v + 1]);
            reinterpret_cast<float2*>(ib + c0)[v] = make_float2((float)f[2 * v], (float)f[2 * v + 1]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < LPT; ++i)
            if (i < nl) tb[c0 + i] = t[i], ib[c0 + i] = (float)f[i];
        }
        __syncwarp();
        float wt[NWV * 2], wi[NWV * 2];
#pragma unroll
        for (int v = 0; v < NWV; ++v) {
          const float2 a = reinterpret_cast<const float2*>(tb + c0 - G)[v];
          const float2 c = reinterpret_cast<const float2*>(ib + c0 - G)[v];
          wt[2 * v] = a.x, wt[2 * v + 1] = a.y;
          wi[2 * v] = c.x, wi[2 * v + 1] = c.y;
        }
        float sk[RW];
#pragma unroll
        for (int k = 0; k < RW; ++k) sk[k] = 0.f;
#pragma unroll
        for (int i = 0; i < LPT; ++i) {
          const float me = (float)(c0 + i);
#pragma unroll
          for (int o = -(RW - 1); o <= RW - 1; ++o) {
            const float pr = eq_flag(wi[G + i + o], me) * wt[G + i + o];
            qn[i] += pr;
            sk[o < 0 ? -o : o] += pr;
          }
        }
#pragma unroll
        for (int k = 0; k < RW; ++k) ack[k] = fmaf(e, sk[k], ack[k]);
      }
      // ---- far ----
      bool pend[LPT];
      bool any = false;
#pragma unroll
      for (int i = 0; i < LPT; ++i) {
        pend[i] = (FULL || i < nl) && kd[i] >= RW;
        any |= pend[i];
      }
      const unsigned anyb = __ballot_sync(0xffffffffu, any);
      if (anyb) {
        int ft = 0;
#pragma unroll
        for (int i = LPT - 1; i >= 0; --i) ft = pend[i] ? f[i] : ft;
        const int tg = __shfl_sync(0xffffffffu, ft, __ffs(anyb) - 1);
        float part = 0.f;
        bool left = false;
        // signed offset: distinct labels, distinct cells (lanes without a far label keep away: the
        // cells of labels that do not exist may lie outside the table)
        float* cell = acc + (any ? L + c0 - tg : L);
#pragma unroll
        for (int i = 0; i < LPT; ++i) {
          const bool hit = pend[i] && f[i] == tg;
          const float ht = hit ? t[i] : 0.f;
          part += ht;
          const float cv = fmaf(e, ht, cell[i]);
          if (hit) cell[i] = cv;
          pend[i] = pend[i] && !hit;
          left |= pend[i];
        }
        const float tot = warp_sum(part);
        const int jt = tg - c0;
#pragma unroll
        for (int i = 0; i < LPT; ++i) qn[i] += (i == jt) ? tot : 0.f;
        if (__ballot_sync(0xffffffffu, left)) {
          __syncwarp();
#pragma unroll
          for (int i = 0; i < LPT; ++i) {
            if (pend[i]) {
              atomicAdd(qfar + f[i], t[i]);
              atomicAdd(acc + (L + c0 + i - f[i]), e * t[i]);
            }
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < LPT; ++i) qn[i] += qfar[c0 + i];
          __syncwarp();
#pragma unroll
          for (int i = 0; i < LPT; ++i) qfar[c0 + i] = 0.f;
        }
      }
    }
    if (FULL || nl > 0) {
      if (!CP) {
        // scatter field of this direction at this pixel
        if (FULL || whole) {
#pragma unroll
          for (int v = 0; v < LPT / 2; ++v) reinterpret_cast<float2*>(pA)[v] = make_float2(q[2 * v], q[2 * v + 1]);
        } else {
#pragma unroll
          for (int i = 0; i < LPT; ++i)
            if (i < nl) pA[i] = q[i];
        }
      } else {
        // dU and every dM_k (k != dir, inv) receive rho*q; dM_dir = C + P_dir = 0 after its sweep
        float cn[LPT];
#pragma unroll
        for (int i = 0; i < LPT; ++i) cn[i] = x0[i] + rq[i];
        if (FULL || whole) {
#pragma unroll
          for (int v = 0; v < LPT / 2; ++v) {
            reinterpret_cast<float2*>(pA)[v] = make_float2(cn[2 * v], cn[2 * v + 1]);
            reinterpret_cast<float2*>(pB)[v] = make_float2(-cn[2 * v], -cn[2 * v + 1]);
          }
#pragma unroll
          for (int v = 0; v < LPT / 2; ++v) red_add_v2(pI + 2 * v, -q[2 * v], -q[2 * v + 1]);
        } else {
#pragma unroll
          for (int i = 0; i < LPT; ++i) {
            if (i < nl) {
              pA[i] = cn[i];
              pB[i] = -cn[i];
              atomicAdd(pI + i, -q[i]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < LPT; ++i) q[i] = qn[i];
    pA -= ostep;
    pB -= ostep;
    pI -= ostep;
  };

  const bool all_whole = L == LP;  // warp-uniform
  for (int b = 0; b < nblocks; ++b) {
    load_blk(b + 1, e_nxt, n_nxt);
    const int rows = stage_rows(b);
    const int slot = b % kWNS;
    cp_async_wait<kWNS - 1>();
    if (rows > 0 && !mbar_wait(&full[slot], (b / kWNS) & 1)) {
      if (lane == 0) atomicExch(p.status, 161);
      return;
    }
    __syncwarp();
    const int send = len - K * b < K ? len - K * b : K;
    const float* row = ring + slot * stage_floats + (flip ? rows - 1 : 0) * L + c0;
    const int rstep = flip ? -L : L;
    const uint8_t* irow = itile + (slot * K) * L + c0;
    float* drow = dtile + lane;
    for (int sl = 0; sl < send; ++sl) {
      const int s = K * b + sl;
      if (s < nsteps) {
        if (all_whole) {
          step(std::true_type{}, std::true_type{}, row, irow, drow, sl);
        } else {
          step(std::false_type{}, std::true_type{}, row, irow, drow, sl);
        }
      } else {
        step(std::false_type{}, std::false_type{}, row, irow, drow, sl);
      }
      row += rstep;
      irow += L;
      drow += 33;
    }
    // edge-weight gradients of this block: lane j sums row j of the product tile
    __syncwarp();
    if (DE && lane < K) {
      const int s = K * b + lane;
      if (s < nsteps) {
        const float* dr = dtile + lane * 33;
        float da = 0.f, db = 0.f;
#pragma unroll 8
        for (int c = 0; c < 32; c += 2) da += dr[c], db += dr[c + 1];
        atomicAdd(DE + (pixl - s * pstep), da + db);
      }
    }
    __syncwarp();
    issue_stage(b + kWNS);  // the warp refills the slot it has just consumed
    e_cur = e_nxt;
    n_cur = n_nxt;
  }
  cp_async_wait<0>();

  // flush the label-context gradient of this chain: near offsets from the registers, then the table
  __syncwarp();
#pragma unroll
  for (int k = 0; k < RW; ++k) {
    const float v = warp_sum(ack[k]);
    if (lane == 0 && k < L && (k > 0 || p.keep_diag)) acc[L + k] += v;
  }
  __syncwarp();
  float* part = p.dctx_part + (long long)(blockIdx.x % p.n_slots) * L;
  for (int i = lane; i < L; i += 32) {
    const float v = i > 0 ? acc[L + i] + acc[L - i] : acc[L];  // fold the two signs of the offset
    if (v != 0.f) atomicAdd(part + i, v);
  }
}

template <int LPT, int RW, int SCH>
cudaError_t launch_bw(BwdParams p, int total, cudaStream_t st) {
  constexpr int LP = 32 * LPT, G = RW & ~1, NA = SCH == 1 ? 2 : 1;
  auto bytes = [&](int k) {
    return ((size_t)bwd_wide_floats(p.L, LP, G, k, NA) + ((p.L + 3) & ~3) + 4) * sizeof(float);
  };
  // every chain of the launch resident at once where possible: the stage depth shrinks first
  const int per_sm = (total + 147) / 148;
  const size_t budget = (size_t)225 * 1024 / (per_sm > 0 ? per_sm : 1);
  int K = 16;
  while (K > 2 && bytes(K) + 1024 > budget) K >>= 1;
  p.tma_k = K;
  const size_t smem = bytes(K);
  auto kernel = bwd_wide_kernel<LPT, RW, SCH>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                       (int)cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return e;
  kernel<<<total, 32, smem, st>>>(p);
  return cudaGetLastError();
}

template <int LPT, int SCH>
cudaError_t launch_bw_r(const BwdParams& p, int total, cudaStream_t st) {
  const int w = p.window > 0 ? p.window : 4;  // without a statement about the context: a middle width
  if (w <= 2) return launch_bw<LPT, 2, SCH>(p, total, st);
  if (w <= 4) return launch_bw<LPT, 4, SCH>(p, total, st);
  if (w <= 8) return launch_bw<LPT, 8, SCH>(p, total, st);
  return launch_bw<LPT, 16, SCH>(p, total, st);
}

template <int SCH>
cudaError_t launch_bw_l(const BwdParams& p, int total, cudaStream_t st) {
  switch (2 * ((p.L + 63) / 64)) {
    case 2: return launch_bw_r<2, SCH>(p, total, st);
    case 4: return launch_bw_r<4, SCH>(p, total, st);
    case 6: return launch_bw_r<6, SCH>(p, total, st);
    default: return launch_bw_r<8, SCH>(p, total, st);
  }
}

}  // namespace

bool bwd_wide_eligible(int L, int ctx_rank, int cp_scheme, const void* dunary, const void* dm_read,
                       const void* dm_acc) {
  static const int min_l = [] {  // MPL_WIDE_BWD_MIN_L: tuning / comparison knob (first label count taken)
    const char* e = getenv("MPL_WIDE_BWD_MIN_L");
    return e ? atoi(e) : 33;
  }();
  if (ctx_rank != 1 || L < min_l || L > 256 || (L & 3) || cp_scheme == 0) return false;
  if (((uintptr_t)dunary | (uintptr_t)dm_read | (uintptr_t)dm_acc) & 15) return false;
  return !pair_kernels_disabled();
}

// `total` chains as described by p.chain_off / chain_begin (filled by launch_backward_sweep).
cudaError_t launch_backward_wide(const BwdParams& p, int total, cudaStream_t st) {
  return p.cp_scheme == 1 ? launch_bw_l<1>(p, total, st) : launch_bw_l<2>(p, total, st);
}

}  // namespace mpl
