// Shared device/host helpers of the TRWP / ISGMR kernels (sm_100a).
#pragma once
#include <cuda.h>  // CUtensorMap (types only; the encoder is fetched through the runtime)
#include <cuda_runtime.h>
#include <cstdlib>
#include <stdint.h>

namespace mpl {

// Direction table, identical to the reference's (MPLayers/common.cpp:28-76): step of direction d;
// a message in direction d at pixel `cur` comes from `front = cur - step`; dir_inv = d ^ 1.
namespace detail {
constexpr int kHs[16] = {0, 0, 1, -1, 1, -1, 1, -1, 1, -1, 2, -2, 2, -2, 1, -1};
constexpr int kWs[16] = {1, -1, 0, 0, 1, -1, -1, 1, 2, -2, 1, -1, -1, 1, -2, 2};
constexpr unsigned long long pack16(const int* v) {
  unsigned long long r = 0;
  for (int i = 0; i < 16; ++i) r |= (unsigned long long)(v[i] + 2) << (4 * i);
  return r;
}
constexpr unsigned long long kHsPacked = pack16(kHs), kWsPacked = pack16(kWs);
}  // namespace detail

__host__ __device__ inline void dir_step(int dir, int& hs, int& ws) {
  hs = (int)((detail::kHsPacked >> (4 * dir)) & 15) - 2;  // nibble table: no local-memory array
  ws = (int)((detail::kWsPacked >> (4 * dir)) & 15) - 2;
}

// Chains of one direction inside one image.  A chain starts at every pixel whose `front` lies
// outside the image and follows +step until it leaves the image, so every pixel belongs to exactly
// one chain per direction.  (The reference enumerates "trees" and skips out-of-image steps,
// MPLayers/TRWP/TRWP_forward.cu:201-218,310-312; the visited pixel sequences are the same.)
struct DirGeom {
  int hs, ws;     // step
  int ah, aw;     // min(|hs|, H), min(|ws|, W)
  int n_first;    // chains starting in the first ah rows (all columns)
  int n_chains;   // chains per image
};

__host__ __device__ inline DirGeom make_geom(int dir, int H, int W) {
  DirGeom g;
  dir_step(dir, g.hs, g.ws);
  const int ahs = g.hs < 0 ? -g.hs : g.hs, aws = g.ws < 0 ? -g.ws : g.ws;
  g.ah = ahs < H ? ahs : H;
  g.aw = aws < W ? aws : W;
  g.n_first = g.ah * W;
  g.n_chains = g.n_first + (H - g.ah) * g.aw;
  return g;
}

// Start pixel (h0, w0) and number of pixels `len` of chain t (0 <= t < n_chains).
__host__ __device__ inline void chain_start(const DirGeom& g, int H, int W, int t, int& h0, int& w0,
                                            int& len) {
  if (t < g.n_first) {
    const int rr = t / W;
    h0 = g.hs > 0 ? rr : H - 1 - rr;
    w0 = t - rr * W;
  } else {
    const int t2 = t - g.n_first;
    const int rr = g.ah + t2 / g.aw;
    const int ci = t2 - (t2 / g.aw) * g.aw;
    h0 = g.hs < 0 ? H - 1 - rr : rr;
    w0 = g.ws > 0 ? ci : W - 1 - ci;
  }
  int nh = 0x7fffffff, nw = 0x7fffffff;
  if (g.hs > 0) nh = (H - 1 - h0) / g.hs;
  if (g.hs < 0) nh = h0 / (-g.hs);
  if (g.ws > 0) nw = (W - 1 - w0) / g.ws;
  if (g.ws < 0) nw = w0 / (-g.ws);
  len = 1 + (nh < nw ? nh : nw);
}

// Chains [begin, begin + count) of `total` that part `part` of `parts` covers (parts <= 1: all).
__host__ __device__ inline void chain_part(long long total, int part, int parts, int& begin, int& count) {
  if (parts <= 1) {
    begin = 0;
    count = (int)total;
    return;
  }
  begin = (int)(total * part / parts);
  count = (int)(total * (part + 1) / parts) - begin;
}

// What the device learned about a rank-1 context and the edge weights (written by
// analyze kernels, read by the sweep kernels; lives in the caller's workspace).
struct CtxInfo {
  int windowed;   // 1: ctx[k] <= ctx[L-1] for k < R, ctx[k] == ctx[L-1] for k >= R, and 2R-1 < L
  int R;          // first offset at which ctx has reached its final value
  float cmax;     // ctx[L-1]
  int ew_min_bits;  // order-preserving int image of min(edge weight)
};

struct FwdParams {
  const float* unary;     // [nimg,H,W,L]
  const float* msg_read;  // [D,nimg,H,W,L] messages entering UU
  float* msg_write;       // [D,nimg,H,W,L] slice `dir` receives the new messages
  const float* ctx;
  const float* ew;        // [D,nimg,H,W] or nullptr (= 1)
  float* edge_label;      // soft TRWP, training: [D,nimg,H,W,L,L] edge values of this iteration, else nullptr
  uint8_t* min_idx;       // [D,nimg,H,W,L] of this iteration, or nullptr
  uint8_t* norm_idx;      // [D,nimg,H,W]
  const CtxInfo* info;
  int* status;            // device word: 0 = ok, else the code of a wait that gave up
  int H, W, L, D, nimg;
  long long slice;        // nimg*H*W*L
  long long pslice;       // nimg*H*W
  float rho;
  int ctx_rank;
  int tma_stages;         // bulk-copy kernels: ring depth
  int tma_k;              // bulk-copy CTA kernel: chain pixels per stage
  int tma_box;            // wide kernel: vertical chains are staged with 2-D tiled TMA boxes
  // agg != 0 (ISGMR): `unary` holds the per-iteration aggregate A = U + sum_k M_k of the messages
  // being read (computed once per iteration in the reference order of the additions), so a sweep
  // stages A, M_dir and M_inv only: UU = (A - M_dir) * rho - M_inv, bit-identical to the
  // reference's ((U + M_0 + ... + M_{D-1}) - M_dir) * rho - M_inv.
  int agg;
  int host_windowed;      // host copy of the context analysis (rank-1, L > 32): windowed path is exact
  int host_R;             //   ... and its window half-width
  int dir0, ndirs;        // this launch covers directions dir0 .. dir0+ndirs-1
  int chain_off[17];      // prefix sums of the chain counts of those directions in this launch
  int chain_begin[16];    // first chain (of nimg*n_chains) of each of those directions in this launch
  int part, parts;        // the launch covers part `part` of `parts` of every direction's chains (parts <= 1: all)
};

struct BwdParams {
  const float* ctx;
  const float* ew;        // or nullptr (= 1)
  const float* edge_label; // soft TRWP: [D,nimg,H,W,L,L] edge values saved by the forward, else nullptr
  const float* edge_label_end;  // one past the last element of the whole saved tensor (all iterations)
  const uint8_t* min_idx; // [D,nimg,H,W,L] of this iteration
  const uint8_t* norm_idx; // [D,nimg,H,W]
  float* dm_read;         // [D,...]: slice `dir` holds the gradient of this sweep's messages; zeroed here
  float* dm_acc;          // [D,...]: gradient of the messages the sweep read (TRWP: == dm_read)
  float* dunary;
  float* dew;             // [D,nimg,H,W], or nullptr
  float* dctx_part;       // [n_slots, ctx_table] partial tables
  int n_slots;
  int H, W, L, D, nimg;
  long long slice, pslice;
  float rho;
  int ctx_rank, keep_diag;
  int dir;                // first direction of this launch
  int ndirs;              // directions covered (more than one only with cp_scheme == 2)
  int chain_off[17];      // prefix sums of the chain counts of those directions in this launch
  int chain_begin[16];    // first chain (of nimg*n_chains) of each of those directions in this launch
  int part, parts;        // part `part` of `parts` of every direction's chains (parts <= 1: all)
  int table_in_smem;      // CTA kernel: 1 = [L][L|1] table in shared memory
  // Gradient bookkeeping.  cp_scheme == 0: `dunary` and the D slices of `dm_acc` are updated with
  // one reduction each per pixel (the reference's UpdateUnaryKernelBack).  cp_scheme == 1 (TRWP,
  // L <= 32): the message gradients are kept as dM_k = C + P_k with the common part C stored in
  // `dunary` (dU and every dM_k receive the same increment rho*q) and P_k in `dm_read`; a sweep
  // then rewrites C and P_dir and corrects P_inv only.  cp_scheme == 2 (ISGMR): a sweep only stores
  // its scatter field q_dir (into slice `dir` of `dm_acc`); the D sweeps of an iteration are
  // independent and run in one launch, and isgmr_combine_kernel afterwards forms
  // dM_k = rho*Q - rho*q_k - q_inv(k), dU += rho*Q with Q = sum_d q_d.
  int cp_scheme;
  int tma_stages;
  int tma_k;              // wide kernel: chain steps per stage
  int window;             // wide kernel: the caller's statement about a rank-1 context (mpl_problem::context_window), or 0
  int* status;            // device word: 0 = ok, else the code of a wait that gave up
};

__device__ __forceinline__ float ctx_value(const float* ctx, int rank, int L, int c, int f) {
  if (rank == 2) {
    const int a = c < f ? c : f, b = c < f ? f : c;
    return __ldg(ctx + a * L + b);
  }
  const int k = c - f;
  return __ldg(ctx + (k < 0 ? -k : k));
}

// Two independent fp32 fused multiply-adds in one instruction (fma.rn.f32x2, sm_100): d = a*b + c
// on both halves, each rounded exactly like fmaf.  The chain kernels are bound by instruction
// issue, not by the FMA pipe, so halving the count of their fmas shortens a step.
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0,
                                      float c1) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %5};\n\t"
      "mov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}

// Warp-wide float min in one instruction (sm_100a).
__device__ __forceinline__ float warp_min(float v) {
  float m;
  asm volatile("redux.sync.min.f32 %0, %1, 0xffffffff;" : "=f"(m) : "f"(v));
  return m;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void cp_async4(float* smem_dst, const float* gmem_src) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ int float_order_bits(float x) {
  const int b = __float_as_int(x);
  return b >= 0 ? b : b ^ 0x7fffffff;
}
__device__ __forceinline__ float float_from_order_bits(int b) {
  return __int_as_float(b >= 0 ? b : b ^ 0x7fffffff);
}

constexpr float kInf = __builtin_huge_valf();

// ---- mbarrier / bulk-copy (TMA) primitives; every wait is bounded --------------------------------
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// Waits for the phase with the given parity; gives up after `limit` clocks (default: about a second)
// and returns false.  Each try may leave the thread suspended for up to kMbarSuspendNs (it resumes
// as soon as the phase completes), so a warp that is far ahead of its partner (a producer with a
// full ring) does not spend issue slots of its scheduler on polling.
constexpr unsigned kMbarSuspendNs = 20000;
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity,
                                          long long limit = 2000000000ll) {
  const unsigned a = smem_u32(bar);
  const long long t0 = clock64();
  for (;;) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(a), "r"(parity), "r"(kMbarSuspendNs)
        : "memory");
    if (ok) return true;
    if (clock64() - t0 > limit) return false;
  }
}
// Tensor maps of the vertical-direction kernels (2-D tiled TMA: one copy brings kTK image rows of
// a four-pixel-wide column group).  Passed as a __grid_constant__ kernel parameter.
struct alignas(64) TmaMaps {
  CUtensorMap a;  // forward: unary            backward: C (dunary)
  CUtensorMap b;  // forward: message slices   backward: P (message-gradient slices)
  CUtensorMap c;  // forward: edge weights
};
// Encodes a 2-D fp32 map: `inner` contiguous floats per row, `rows` rows, box = box_inner x box_rows.
// Returns false if the driver entry point is unavailable or the encode fails.
bool encode_tmap_2d(CUtensorMap* m, const void* base, unsigned long long inner, unsigned long long rows,
                    unsigned box_inner, unsigned box_rows);

// 2-D tiled TMA load (no multicast): box at (x, y) -> shared memory, completion in bytes on `bar`.
// dst 128-byte aligned; x * 4 bytes a multiple of 16.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y,
                                            unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// MPL_NO_PAIR=1 keeps 32 < L <= 64 on the CTA-per-chain kernels (tuning / comparison knob).
inline bool pair_kernels_disabled() {
  const char* e = getenv("MPL_NO_PAIR");
  return e && e[0] == '1';
}

// Orders this thread's earlier generic-proxy accesses to shared memory before later async-proxy
// (bulk-copy) accesses; used by warps that refill a tile they have just finished reading.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Global -> shared bulk copy (no multicast), completion counted in bytes on `bar`.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Host-side launchers (mp_forward.cu / mp_backward.cu).  Return cudaGetLastError() of the launch.
cudaError_t launch_analyze(const float* ctx, int L, int rank, const float* ew, long long n_ew,
                           CtxInfo* info, cudaStream_t st);
cudaError_t launch_forward_sweep(const FwdParams& p, bool train, cudaStream_t st);
cudaError_t launch_forward_wide(const FwdParams& p, bool train, cudaStream_t st);  // mp_wide.cu
cudaError_t launch_aggregate(const float* unary, const float* msg, float* cost, uint8_t* label,
                             long long npix, int L, int D, long long slice, float factor,
                             int min_a_dir, cudaStream_t st);
cudaError_t launch_backward_init(const float* dcost, float* dunary, float* dm, long long n, int D,
                                 float factor, int cp_scheme, cudaStream_t st);
// labels-first variants (mpl_problem::cost_labels_first): cost / dcost as [nimg, L, H*W] planes
cudaError_t launch_aggregate_lhw(const float* unary, const float* msg, float* cost, int nimg, int L,
                                 long long HW, int D, long long slice, float factor, int min_a_dir,
                                 cudaStream_t st);
cudaError_t launch_backward_init_lhw(const float* dcost, float* dunary, float* dm, int nimg, int L, long long HW,
                                     int D, float factor, int cp_scheme, cudaStream_t st);
cudaError_t launch_backward_sweep(const BwdParams& p, cudaStream_t st);
// mp_wide_bwd.cu: rank-1 context, 32 < L <= 256, L % 4 == 0, schemes 1 and 2
bool bwd_wide_eligible(int L, int ctx_rank, int cp_scheme, const void* dunary, const void* dm_read,
                       const void* dm_acc);
cudaError_t launch_backward_wide(const BwdParams& p, int total, cudaStream_t st);
cudaError_t launch_isgmr_combine_total(const float* q_total, const float* q, float* dm, float* dunary, long long n,
                                       int dir0, int ndirs, float rho, cudaStream_t st);
cudaError_t launch_forward_soft_sweep(const FwdParams& p, bool train, cudaStream_t st);
cudaError_t launch_backward_soft_sweep(const BwdParams& p, cudaStream_t st);
// Soft TRWP for 32 < L <= 64 (mp_soft_cta.cu).
cudaError_t launch_forward_soft_cta(const FwdParams& p, bool train, cudaStream_t st);
cudaError_t launch_backward_soft_cta(const BwdParams& p, int total, cudaStream_t st);
// Stand-alone soft-weighted message ops (mp_swbp.cu).
cudaError_t launch_soft_weighted_message(const float* msg, long long n_tables, int L, float* norm,
                                         uint8_t* min_ind, cudaStream_t st);
cudaError_t launch_soft_weighted_message_back(const float* dnorm, const float* msg, const uint8_t* min_ind,
                                              long long n_tables, int L, float* dmsg, cudaStream_t st);
// Input builders (mp_terms.cu).
cudaError_t launch_stereo_data_cost(const uint8_t* left, const uint8_t* right, int H, int W, int nB, int L,
                                    int birchfield, int squared, int trunc, float* out, cudaStream_t st);
cudaError_t launch_gradient_cues(const uint8_t* img, int H, int W, int nB, int grad_thresh, int grad_penalty,
                                 int compact, float* hcue, float* vcue, cudaStream_t st);
cudaError_t launch_smoothness_context(int L, int method, float smax, float* out, cudaStream_t st);
bool edge_weights_reduces(int mode);
cudaError_t launch_edge_weights(const float* img, int B, int C, int H, int W, int D, int mode, float sigma,
                                float threshold, float penalty, float* out, double* sums, cudaStream_t st);
cudaError_t launch_layout(int kind, const float* in, float* out, uint8_t* amax, int B, int L, long long HW,
                          cudaStream_t st);
cudaError_t launch_energy(const float* unary, const float* ctx, const float* ew, const uint8_t* label,
                          long long npix, int H, int W, int L, int D, int rank, double* part, double* out,
                          cudaStream_t st);
cudaError_t launch_sum_fields(const float* base, float factor, const float* fields, int nf, long long n,
                              long long stride, float* out, cudaStream_t st);
cudaError_t launch_isgmr_combine(const float* q, float* dm, float* dunary, long long n, int D, float rho,
                                 cudaStream_t st);
cudaError_t launch_dctx_reduce(float* part, int n_slots, int L, int rank, int keep_diag,
                               float* dctx, cudaStream_t st);
int backward_slots(int H, int W, int L, int D, int nimg, int rank);
int tma_stage_override();  // MPL_TMA_STAGES environment variable (tuning knob), 0 = not set
void count_launch(int n = 1);

// Optional per-launch timing (mpl_profile_enable): CUDA events recorded on the launching stream
// directly before and after a kernel launch, summed per kernel kind when read.
enum ProfKind { kProfFwdSweep = 0, kProfBwdSweep = 1, kProfElementwise = 2, kProfKinds = 3 };
struct ProfScope {
  ProfScope(int kind, cudaStream_t st);
  ~ProfScope();
  int kind_;
  cudaStream_t st_;
  cudaEvent_t a_, b_;
  bool on_;
};

}  // namespace mpl
