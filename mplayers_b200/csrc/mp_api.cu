// C ABI of libmplayers_b200 (declared in include/mplayers_b200.h): argument validation and the
// host loops over iterations and directions.  The loop ORDER is the reference's
// (MPLayers/TRWP/TRWP_forward.cu:440-548, MPLayers/TRWP/TRWP_backward.cu:337-424,
// MPLayers/ISGMR/ISGMR_forward.cu:506-654, MPLayers/ISGMR/ISGMR_backward.cu:353-484); what runs
// inside each step is one fused kernel instead of the reference's kernel + memcpy/memset pairs.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/mplayers_b200.h"
#include "mp_common.cuh"

namespace mpl {
int tma_stage_override() {
  static const int v = [] {
    const char* e = getenv("MPL_TMA_STAGES");
    const int n = e ? atoi(e) : 0;
    return (n >= 2 && n <= 8) ? n : 0;
  }();
  return v;
}
bool encode_tmap_2d(CUtensorMap* m, const void* base, unsigned long long inner, unsigned long long rows,
                    unsigned box_inner, unsigned box_rows) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeFn>(f);
  }();
  if (!fn) return false;
  // A descriptor depends only on (address, shape, box); encoding costs tens of microseconds on the
  // host, so the last few are kept (training loops present the same buffers again and again).
  struct Entry {
    const void* base;
    unsigned long long inner, rows;
    unsigned bi, br;
    CUtensorMap map;
  };
  static std::mutex mu;
  static Entry cache[32];
  static int n_cached = 0, next_slot = 0;
  {
    std::lock_guard<std::mutex> lk(mu);
    for (int i = 0; i < n_cached; ++i) {
      const Entry& e = cache[i];
      if (e.base == base && e.inner == inner && e.rows == rows && e.bi == box_inner && e.br == box_rows) {
        *m = e.map;
        return true;
      }
    }
  }
  const cuuint64_t dims[2] = {inner, rows};
  const cuuint64_t strides[1] = {inner * sizeof(float)};
  const cuuint32_t box[2] = {box_inner, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  if (fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  std::lock_guard<std::mutex> lk(mu);
  Entry& e = cache[next_slot];
  e.base = base, e.inner = inner, e.rows = rows, e.bi = box_inner, e.br = box_rows, e.map = *m;
  next_slot = (next_slot + 1) % 32;
  if (n_cached < 32) ++n_cached;
  return true;
}

static std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

static std::atomic<int> g_prof_on{0};
static std::mutex g_prof_mu;
struct ProfPair {
  int kind;
  cudaEvent_t a, b;
};
static std::vector<ProfPair> g_prof_pending;
static double g_prof_ms[kProfKinds];
static long long g_prof_n[kProfKinds];

ProfScope::ProfScope(int kind, cudaStream_t st) : kind_(kind), st_(st), a_(nullptr), b_(nullptr), on_(false) {
  if (!g_prof_on.load(std::memory_order_relaxed)) return;
  if (cudaEventCreate(&a_) != cudaSuccess || cudaEventCreate(&b_) != cudaSuccess) return;
  on_ = cudaEventRecord(a_, st_) == cudaSuccess;
}
ProfScope::~ProfScope() {
  if (!on_) return;
  cudaEventRecord(b_, st_);
  std::lock_guard<std::mutex> lk(g_prof_mu);
  g_prof_pending.push_back({kind_, a_, b_});
}
}  // namespace mpl

namespace {

thread_local std::string g_err;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(MPL_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define MPL_CUDA(expr)                                   \
  do {                                                   \
    cudaError_t e__ = (expr);                            \
    if (e__ != cudaSuccess) return cuda_fail(e__, #expr); \
  } while (0)

struct Dims {
  long long nimg, npix, slice;
  int ctx_elems;
};

int validate(const mpl_problem* p, Dims* d) {
  if (!p) return fail(MPL_ERR_INVALID, "problem is NULL");
  if (p->n_iter < 0 || p->batch < 1 || p->n_cv < 1 || p->height < 1 || p->width < 1)
    return fail(MPL_ERR_INVALID, "bad shape: n_iter=%d batch=%d n_cv=%d height=%d width=%d", p->n_iter,
                p->batch, p->n_cv, p->height, p->width);
  if (p->n_disp < 1 || p->n_disp > 256)
    return fail(MPL_ERR_UNSUPPORTED, "n_disp=%d outside 1..256 (argmin indices are 8-bit)", p->n_disp);
  if (p->n_dir < 2 || p->n_dir > 16 || (p->n_dir & 1))
    return fail(MPL_ERR_UNSUPPORTED, "n_dir=%d: must be even and in 2..16", p->n_dir);
  if (p->context_rank != 1 && p->context_rank != 2)
    return fail(MPL_ERR_INVALID, "context_rank=%d: must be 1 or 2", p->context_rank);
  const long long per_img = (long long)p->height * p->width * p->n_disp;
  if (per_img >= (1ll << 31))
    return fail(MPL_ERR_UNSUPPORTED, "height*width*n_disp=%lld must be below 2^31", per_img);
  d->nimg = (long long)p->batch * p->n_cv;
  d->npix = d->nimg * p->height * p->width;
  d->slice = d->npix * p->n_disp;
  if (d->nimg * 4096ll >= (1ll << 31) || d->npix >= (1ll << 40))
    return fail(MPL_ERR_UNSUPPORTED, "batch*n_cv=%lld too large", d->nimg);
  d->ctx_elems = p->context_rank == 2 ? p->n_disp * p->n_disp : p->n_disp;
  if (p->chain_parts > 1 && (p->chain_part < 0 || p->chain_part >= p->chain_parts))
    return fail(MPL_ERR_INVALID, "chain_part=%d outside 0..%d", p->chain_part, p->chain_parts - 1);
  return MPL_OK;
}

int check_chain_count(const mpl_problem* p, const Dims& d) {
  for (int k = 0; k < p->n_dir; ++k) {
    const long long n = (long long)mpl::make_geom(k, p->height, p->width).n_chains * d.nimg;
    if (n * p->n_dir >= (1ll << 31)) return fail(MPL_ERR_UNSUPPORTED, "too many chains (%lld)", n);
  }
  return MPL_OK;
}

void fill_forward(mpl::FwdParams& fp, const mpl_problem* p, const Dims& d, const float* unary,
                  const float* ctx, const float* ew, void* workspace) {
  fp.unary = unary;
  fp.ctx = ctx;
  fp.ew = ew;
  fp.info = static_cast<const mpl::CtxInfo*>(workspace);
  fp.status = reinterpret_cast<int*>(static_cast<char*>(workspace) + 64);  // kStatusOffset
  fp.H = p->height;
  fp.W = p->width;
  fp.L = p->n_disp;
  fp.D = p->n_dir;
  fp.nimg = (int)d.nimg;
  fp.slice = d.slice;
  fp.pslice = d.npix;
  fp.rho = p->rho;
  fp.ctx_rank = p->context_rank;
}

void set_dirs(mpl::FwdParams& fp, int dir0, int ndirs) {
  fp.dir0 = dir0;
  fp.ndirs = ndirs;
  fp.chain_off[0] = 0;
  for (int i = 0; i < ndirs; ++i) {
    int begin, count;
    mpl::chain_part((long long)mpl::make_geom(dir0 + i, fp.H, fp.W).n_chains * fp.nimg, fp.part, fp.parts, begin, count);
    fp.chain_begin[i] = begin;
    fp.chain_off[i + 1] = fp.chain_off[i] + count;
  }
}

// Result of the device-side analysis (launch_analyze, in `workspace`): *window = R > 0 if the
// windowed evaluation is exact, else -1.  Waits for the stream.
int read_window(const void* workspace, bool has_weights, int* window, cudaStream_t st) {
  mpl::CtxInfo hi;
  MPL_CUDA(cudaMemcpyAsync(&hi, workspace, sizeof(hi), cudaMemcpyDeviceToHost, st));
  MPL_CUDA(cudaStreamSynchronize(st));
  const bool ew_ok = !has_weights || hi.ew_min_bits >= 0;  // order bits: negative <=> negative float
  *window = (hi.windowed && ew_ok && hi.R > 0) ? hi.R : -1;
  return MPL_OK;
}

// Fills the sweep parameters, clears the status word and runs the context / edge-weight analysis
// (and, where a rank-1 context may take the windowed kernel, reads its result back: one small
// synchronising copy).
int prepare_forward(mpl::FwdParams& fp, const mpl_problem* p, const Dims& d, const float* unary,
                    const float* context, const float* edge_weights, void* workspace, bool train,
                    cudaStream_t st) {
  const int D = p->n_dir, L = p->n_disp;
  fill_forward(fp, p, d, unary, context, edge_weights, workspace);
  MPL_CUDA(cudaMemsetAsync(fp.status, 0, sizeof(int), st));
  MPL_CUDA(mpl::launch_analyze(context, L, p->context_rank, edge_weights, d.npix * D,
                               static_cast<mpl::CtxInfo*>(workspace), st));
  if (p->context_rank == 1 && L > 32) {
    // Rank-1 context with more than 32 labels: the wide windowed kernel is chosen on the host.  With a
    // statement from the caller (mpl_problem::context_window) nothing is read back; without one the
    // result of the device-side analysis is copied to the host, which waits for the stream --
    // unless the stream is being captured, where waiting is not allowed: then all candidates are
    // evaluated.
    if (p->context_window > 0) {
      fp.host_windowed = 1;
      fp.host_R = p->context_window;
    } else if (p->context_window == 0) {
      cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
      MPL_CUDA(cudaStreamIsCapturing(st, &cap));
      if (cap == cudaStreamCaptureStatusNone) {
        int w = -1;
        if (int rc = read_window(workspace, edge_weights != nullptr, &w, st)) return rc;
        fp.host_windowed = w > 0;
        fp.host_R = w > 0 ? w : 0;
      }
    }
  }
  return MPL_OK;
}

int forward_common(bool isgmr, const mpl_problem* p, const float* unary, const float* context,
                   const float* edge_weights, float* msg, float* msg_update, float* cost_final,
                   uint8_t* msg_min_index, uint8_t* msg_norm_index, uint8_t* label_all,
                   void* workspace, size_t workspace_bytes, void* stream) {
  Dims d;
  if (int rc = validate(p, &d)) return rc;
  if (int rc = check_chain_count(p, d)) return rc;
  if (!unary || !context || !msg || !cost_final || (isgmr && !msg_update))
    return fail(MPL_ERR_INVALID, "NULL tensor pointer");
  if ((msg_min_index == nullptr) != (msg_norm_index == nullptr))
    return fail(MPL_ERR_INVALID, "msg_min_index and msg_norm_index must both be given or both be NULL");
  if (!workspace || workspace_bytes < mpl_forward_workspace_bytes(p))
    return fail(MPL_ERR_INVALID, "workspace too small: %zu < %zu", workspace_bytes,
                mpl_forward_workspace_bytes(p));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool train = msg_min_index != nullptr;
  const int D = p->n_dir, L = p->n_disp;

  mpl::FwdParams fp{};
  if (int rc = prepare_forward(fp, p, d, unary, context, edge_weights, workspace, train, st)) return rc;

  const float factor = (isgmr && p->enable_sgm) ? (float)D : 1.f;
  // ISGMR alternates between the two message buffers so that the last iteration writes `msg`.
  float* rd = msg;
  float* wr = msg;
  if (isgmr) {
    const bool last_writes_msg_when_first_writes_msg = (p->n_iter % 2) == 1;
    wr = last_writes_msg_when_first_writes_msg ? msg : msg_update;
    rd = wr == msg ? msg_update : msg;
    // The iterations start from the messages in `msg`, as in the reference.  With an odd iteration
    // count the first sweep writes `msg`, so its input moves to `msg_update` first.
    if (rd != msg && p->n_iter > 0)
      MPL_CUDA(cudaMemcpyAsync(msg_update, msg, (size_t)D * d.slice * sizeof(float), cudaMemcpyDeviceToDevice, st));
  }
  for (int it = 0; it < p->n_iter; ++it) {
    fp.min_idx = train ? msg_min_index + (long long)it * D * d.slice : nullptr;
    fp.norm_idx = train ? msg_norm_index + (long long)it * D * d.npix : nullptr;
    fp.msg_read = rd;
    fp.msg_write = wr;
    if (isgmr) {
      // Every direction reads the previous iteration's messages.  Their sum with the unaries is
      // formed once (in `cost_final`, which is otherwise unused until the end) so that a sweep
      // stages three arrays instead of D+1.  The first iteration forms it too: the messages the
      // caller passes in count, as they do in the reference and in the other path.
      // With few labels and directions the sweep sums U + sum_k M_k itself faster than a separate
      // pass over all messages does (measured 5.13 -> 4.99 ms on 2x512x512, L = 21, D = 4); with
      // 256 labels the extra staged rows cost more than the pass (28.4 -> 29.2 ms).
      const bool use_agg = !(L <= 32 && D <= 4);
      fp.agg = use_agg ? 1 : 0;
      fp.unary = unary;
      if (use_agg) {
        MPL_CUDA(mpl::launch_aggregate(unary, rd, cost_final, nullptr, d.npix, L, D, d.slice, 1.f, 0, st));
        fp.unary = cost_final;
      }
      set_dirs(fp, 0, D);
      MPL_CUDA(mpl::launch_forward_sweep(fp, train, st));
      float* t = rd;
      rd = wr;
      wr = t;
    } else {
      for (int dir = 0; dir < D; ++dir) {  // later directions see earlier ones' new messages
        set_dirs(fp, dir, 1);
        MPL_CUDA(mpl::launch_forward_sweep(fp, train, st));
      }
    }
    if (label_all) {
      const float* cur = isgmr ? rd : msg;  // after the swap `rd` holds this iteration's messages
      MPL_CUDA(mpl::launch_aggregate(unary, cur, cost_final, label_all + (long long)it * d.npix, d.npix,
                                     L, D, d.slice, factor, p->enable_min_a_dir, st));
    }
  }
  const float* fin = isgmr ? rd : msg;
  if (isgmr && p->n_iter > 0 && fin != msg)
    return fail(MPL_ERR_CUDA, "internal: ISGMR buffer parity");
  if (p->cost_labels_first) {
    MPL_CUDA(mpl::launch_aggregate_lhw(unary, msg, cost_final, (int)d.nimg, L, (long long)p->height * p->width, D,
                                       d.slice, factor, p->enable_min_a_dir, st));
  } else {
    MPL_CUDA(mpl::launch_aggregate(unary, msg, cost_final, nullptr, d.npix, L, D, d.slice, factor,
                                   p->enable_min_a_dir, st));
  }
  return MPL_OK;
}

// Layout of every workspace (forward, backward, the built-in scratch): bytes [0, 64) context
// analysis, [64, 68) the device status word, [256, ...) the backward's partial label-context tables.
constexpr size_t kStatusOffset = 64, kTablesOffset = 256;
inline float* ws_tables(void* workspace) { return reinterpret_cast<float*>(static_cast<char*>(workspace) + kTablesOffset); }
inline int* ws_status(void* workspace) { return reinterpret_cast<int*>(static_cast<char*>(workspace) + kStatusOffset); }

void fill_backward(mpl::BwdParams& bp, const mpl_problem* p, const Dims& d, const float* context,
                   const float* edge_weights, float* dunary, float* part, int n_slots, int cp, int* status) {
  bp.ctx = context;
  bp.ew = edge_weights;
  bp.dunary = dunary;
  bp.dctx_part = part;
  bp.n_slots = n_slots;
  bp.H = p->height;
  bp.W = p->width;
  bp.L = p->n_disp;
  bp.D = p->n_dir;
  bp.nimg = (int)d.nimg;
  bp.slice = d.slice;
  bp.pslice = d.npix;
  bp.rho = p->rho;
  bp.ctx_rank = p->context_rank;
  bp.keep_diag = p->keep_diag;
  bp.cp_scheme = cp;
  bp.window = p->context_window > 0 ? p->context_window : 0;
  bp.status = status;
}

int backward_common(bool isgmr, const mpl_problem* p, const float* context, const float* edge_weights,
                    const float* dcost_final, const uint8_t* msg_min_index,
                    const uint8_t* msg_norm_index, float* dunary, float* dcontext,
                    float* dedge_weights, float* dmsg, float* dmsg_update, void* workspace,
                    size_t workspace_bytes, void* stream) {
  Dims d;
  if (int rc = validate(p, &d)) return rc;
  if (int rc = check_chain_count(p, d)) return rc;
  if (!context || !dcost_final || !msg_min_index || !msg_norm_index || !dunary || !dcontext || !dmsg ||
      (isgmr && !dmsg_update))
    return fail(MPL_ERR_INVALID, "NULL tensor pointer");
  if (edge_weights && !dedge_weights)
    return fail(MPL_ERR_INVALID, "dedge_weights is NULL although edge_weights is given");
  if (!workspace || workspace_bytes < mpl_backward_workspace_bytes(p))
    return fail(MPL_ERR_INVALID, "workspace too small: %zu < %zu", workspace_bytes,
                mpl_backward_workspace_bytes(p));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int D = p->n_dir, L = p->n_disp;
  const int n_slots = mpl::backward_slots(p->height, p->width, L, D, (int)d.nimg, p->context_rank);
  float* part = ws_tables(workspace);
  MPL_CUDA(cudaMemsetAsync(part, 0, (size_t)n_slots * d.ctx_elems * sizeof(float), st));

  const float factor = (isgmr && p->enable_sgm) ? (float)D : 1.f;
  // TRWP with L <= 32 keeps the message gradients as dM_k = C + P_k (C in `dunary`, P in `dmsg`),
  // see BwdParams::cp_scheme; everything else updates dunary and the D slices directly.
  // (L <= 64 in multiples of four at 16-byte aligned buffers runs the two-labels-per-lane kernel,
  // which knows the C + P scheme as well.)
  const bool pair_cp = L <= 64 && (L & 3) == 0 && ((((uintptr_t)dunary | (uintptr_t)dmsg) & 15) == 0) &&
                       !mpl::pair_kernels_disabled();
  // (a rank-1 context with 32 < L <= 256 runs the several-labels-per-lane kernel, C + P too)
  const bool wide_cp = mpl::bwd_wide_eligible(L, p->context_rank, 1, dunary, dmsg, dmsg);
  const int cp = isgmr ? 2 : ((L <= 32 || pair_cp || wide_cp) ? 1 : 0);
  float* X = isgmr ? dmsg_update : dmsg;  // gradients of the messages the sweeps produced
  float* Y = isgmr ? dmsg : dmsg;         // gradients of the messages the sweeps read
  if (p->cost_labels_first) {
    MPL_CUDA(mpl::launch_backward_init_lhw(dcost_final, dunary, X, (int)d.nimg, L, (long long)p->height * p->width,
                                           D, factor, cp == 1, st));
  } else {
    MPL_CUDA(mpl::launch_backward_init(dcost_final, dunary, X, d.slice, D, factor, cp == 1, st));
  }
  int* status = ws_status(workspace);
  MPL_CUDA(cudaMemsetAsync(status, 0, sizeof(int), st));

  mpl::BwdParams bp{};
  fill_backward(bp, p, d, context, edge_weights, dunary, part, n_slots, cp, status);
  for (int it = p->n_iter - 1; it >= 0; --it) {
    bp.min_idx = msg_min_index + (long long)it * D * d.slice;
    bp.norm_idx = msg_norm_index + (long long)it * D * d.npix;
    bp.dew = (edge_weights && dedge_weights) ? dedge_weights : nullptr;
    if (isgmr) {
      // The D sweeps of an iteration are independent: one launch reads dMU (X) and stores the
      // scatter fields q_d (Y); the combine kernel then rewrites X with the gradients of the
      // messages this iteration read and adds rho * sum_d q_d to dunary.
      bp.dir = 0;
      bp.ndirs = D;
      bp.dm_read = X;
      bp.dm_acc = Y;
      MPL_CUDA(mpl::launch_backward_sweep(bp, st));
      MPL_CUDA(mpl::launch_isgmr_combine(Y, X, dunary, d.slice, D, p->rho, st));
    } else {
      for (int dir = D - 1; dir >= 0; --dir) {
        bp.dir = dir;
        bp.ndirs = 1;
        bp.dm_read = X;
        bp.dm_acc = Y;
        MPL_CUDA(mpl::launch_backward_sweep(bp, st));
      }
    }
  }
  MPL_CUDA(mpl::launch_dctx_reduce(part, n_slots, L, p->context_rank, p->keep_diag, dcontext, st));
  return MPL_OK;
}

}  // namespace

extern "C" {

int mpl_analyze_context(const mpl_problem* p, const float* context, const float* edge_weights,
                        int32_t* window, void* workspace, size_t workspace_bytes, void* stream) {
  Dims d;
  if (int rc = validate(p, &d)) return rc;
  if (!context || !window) return fail(MPL_ERR_INVALID, "NULL pointer");
  if (!workspace || workspace_bytes < mpl_forward_workspace_bytes(p))
    return fail(MPL_ERR_INVALID, "workspace too small: %zu < %zu", workspace_bytes,
                mpl_forward_workspace_bytes(p));
  *window = -1;
  if (p->context_rank != 1 || p->n_disp <= 32) return MPL_OK;  // only those sweeps have a windowed form
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MPL_CUDA(mpl::launch_analyze(context, p->n_disp, 1, edge_weights, d.npix * p->n_dir,
                               static_cast<mpl::CtxInfo*>(workspace), st));
  int w = -1;
  if (int rc = read_window(workspace, edge_weights != nullptr, &w, st)) return rc;
  *window = w;
  return MPL_OK;
}

size_t mpl_forward_workspace_bytes(const mpl_problem* p) {
  (void)p;
  return 256;
}

size_t mpl_backward_workspace_bytes(const mpl_problem* p) {
  Dims d;
  if (validate(p, &d) != MPL_OK) return 256;
  const int n_slots = mpl::backward_slots(p->height, p->width, p->n_disp, p->n_dir, (int)d.nimg, p->context_rank);
  return kTablesOffset + (size_t)n_slots * d.ctx_elems * sizeof(float);  // header + tables
}

int mpl_trwp_forward(const mpl_problem* p, const float* unary, const float* context,
                     const float* edge_weights, float* msg, float* cost_final, uint8_t* msg_min_index,
                     uint8_t* msg_norm_index, uint8_t* label_all, void* workspace,
                     size_t workspace_bytes, void* stream) {
  return forward_common(false, p, unary, context, edge_weights, msg, nullptr, cost_final, msg_min_index,
                        msg_norm_index, label_all, workspace, workspace_bytes, stream);
}

int mpl_isgmr_forward(const mpl_problem* p, const float* unary, const float* context,
                      const float* edge_weights, float* msg, float* msg_update, float* cost_final,
                      uint8_t* msg_min_index, uint8_t* msg_norm_index, uint8_t* label_all,
                      void* workspace, size_t workspace_bytes, void* stream) {
  return forward_common(true, p, unary, context, edge_weights, msg, msg_update, cost_final,
                        msg_min_index, msg_norm_index, label_all, workspace, workspace_bytes, stream);
}

int mpl_trwp_backward(const mpl_problem* p, const float* context, const float* edge_weights,
                      const float* dcost_final, const uint8_t* msg_min_index,
                      const uint8_t* msg_norm_index, float* dunary, float* dcontext,
                      float* dedge_weights, float* dmsg, void* workspace, size_t workspace_bytes,
                      void* stream) {
  return backward_common(false, p, context, edge_weights, dcost_final, msg_min_index, msg_norm_index,
                         dunary, dcontext, dedge_weights, dmsg, nullptr, workspace, workspace_bytes,
                         stream);
}

int mpl_isgmr_backward(const mpl_problem* p, const float* context, const float* edge_weights,
                       const float* dcost_final, const uint8_t* msg_min_index,
                       const uint8_t* msg_norm_index, float* dunary, float* dcontext,
                       float* dedge_weights, float* dmsg, float* dmsg_update, void* workspace,
                       size_t workspace_bytes, void* stream) {
  return backward_common(true, p, context, edge_weights, dcost_final, msg_min_index, msg_norm_index,
                         dunary, dcontext, dedge_weights, dmsg, dmsg_update, workspace,
                         workspace_bytes, stream);
}

// ---- ISGMR one iteration at a time over a subset of directions (direction sharding) -------------
namespace {
int check_dir_range(const mpl_problem* p, int32_t dir_first, int32_t dir_count) {
  if (dir_first < 0 || dir_count < 0 || (dir_first & 1) || (dir_count & 1) || dir_first + dir_count > p->n_dir)
    return fail(MPL_ERR_INVALID,
                "directions [%d, %d) of %d: the range must start and end on a pair (d, d^1) boundary",
                dir_first, dir_first + dir_count, p->n_dir);
  return MPL_OK;
}
}  // namespace

int mpl_isgmr_forward_directions(const mpl_problem* p, int32_t dir_first, int32_t dir_count,
                                 const float* aggregate, const float* context, const float* edge_weights,
                                 const float* msg_read, float* msg_write, uint8_t* msg_min_index,
                                 uint8_t* msg_norm_index, void* workspace, size_t workspace_bytes,
                                 void* stream) {
  Dims d;
  if (int rc = validate(p, &d)) return rc;
  if (int rc = check_chain_count(p, d)) return rc;
  if (int rc = check_dir_range(p, dir_first, dir_count)) return rc;
  if (!aggregate || !context || !msg_read || !msg_write) return fail(MPL_ERR_INVALID, "NULL tensor pointer");
  if (msg_read == msg_write) return fail(MPL_ERR_INVALID, "msg_read and msg_write must be different buffers");
  if ((msg_min_index == nullptr) != (msg_norm_index == nullptr))
    return fail(MPL_ERR_INVALID, "msg_min_index and msg_norm_index must both be given or both be NULL");
  if (!workspace || workspace_bytes < mpl_forward_workspace_bytes(p))
    return fail(MPL_ERR_INVALID, "workspace too small: %zu < %zu", workspace_bytes,
                mpl_forward_workspace_bytes(p));
  if (dir_count == 0) return MPL_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool train = msg_min_index != nullptr;
  mpl::FwdParams fp{};
  if (int rc = prepare_forward(fp, p, d, aggregate, context, edge_weights, workspace, train, st)) return rc;
  fp.agg = 1;
  fp.min_idx = msg_min_index;
  fp.norm_idx = msg_norm_index;
  fp.msg_read = msg_read;
  fp.msg_write = msg_write;
  fp.part = p->chain_part;
  fp.parts = p->chain_parts;
  set_dirs(fp, dir_first, dir_count);
  MPL_CUDA(mpl::launch_forward_sweep(fp, train, st));
  return MPL_OK;
}

int mpl_sum_directions(const mpl_problem* p, int32_t dir_first, int32_t dir_count, const float* base,
                       float base_factor, const float* fields, float* out, void* stream) {
  Dims d;
  if (int rc = validate(p, &d)) return rc;
  if (dir_first < 0 || dir_count < 0 || dir_first + dir_count > p->n_dir)
    return fail(MPL_ERR_INVALID, "directions [%d, %d) of %d", dir_first, dir_first + dir_count, p->n_dir);
  if (!out || (dir_count > 0 && !fields)) return fail(MPL_ERR_INVALID, "NULL tensor pointer");
  MPL_CUDA(mpl::launch_sum_fields(base, base_factor, fields ? fields + (long long)dir_first * d.slice : nullptr,
                                  dir_count, d.slice, d.slice, out, static_cast<cudaStream_t>(stream)));
  return MPL_OK;
}

int mpl_sum_directions_range(const mpl_problem* p, int32_t dir_first, int32_t dir_count, const float* base,
                             float base_factor, const float* fields, float* out, int64_t first_element,
                             int64_t n_elements, void* stream) {
  Dims d;
  if (int rc = validate(p, &d)) return rc;
  if (dir_first < 0 || dir_count < 0 || dir_first + dir_count > p->n_dir)
    return fail(MPL_ERR_INVALID, "directions [%d, %d) of %d", dir_first, dir_first + dir_count, p->n_dir);
  if (!out || (dir_count > 0 && !fields)) return fail(MPL_ERR_INVALID, "NULL tensor pointer");
  if (first_element < 0 || n_elements < 0 || first_element + n_elements > d.slice)
    return fail(MPL_ERR_INVALID, "elements [%lld, %lld) outside the field of %lld",
                (long long)first_element, (long long)(first_element + n_elements), d.slice);
  if (n_elements == 0) return MPL_OK;
  MPL_CUDA(mpl::launch_sum_fields(base ? base + first_element : nullptr, base_factor,
                                  fields ? fields + (long long)dir_first * d.slice + first_element : nullptr,
                                  dir_count, n_elements, d.slice, out + first_element,
                                  static_cast<cudaStream_t>(stream)));
  return MPL_OK;
}

int mpl_isgmr_backward_directions(const mpl_problem* p, int32_t dir_first, int32_t dir_count,
                                  const float* context, const float* edge_weights, float* dmsg_update,
                                  const uint8_t* msg_min_index, const uint8_t* msg_norm_index,
                                  float* scatter, float* dedge_weights, void* workspace,
                                  size_t workspace_bytes, int32_t clear_workspace, void* stream) {
  Dims d;
  if (int rc = validate(p, &d)) return rc;
  if (int rc = check_chain_count(p, d)) return rc;
  if (int rc = check_dir_range(p, dir_first, dir_count)) return rc;
  if (!context || !dmsg_update || !msg_min_index || !msg_norm_index || !scatter)
    return fail(MPL_ERR_INVALID, "NULL tensor pointer");
  if (edge_weights && !dedge_weights)
    return fail(MPL_ERR_INVALID, "dedge_weights is NULL although edge_weights is given");
  if (!workspace || workspace_bytes < mpl_backward_workspace_bytes(p))
    return fail(MPL_ERR_INVALID, "workspace too small: %zu < %zu", workspace_bytes,
                mpl_backward_workspace_bytes(p));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int n_slots = mpl::backward_slots(p->height, p->width, p->n_disp, p->n_dir, (int)d.nimg, p->context_rank);
  float* part = ws_tables(workspace);
  int* status = ws_status(workspace);
  if (clear_workspace) {
    MPL_CUDA(cudaMemsetAsync(part, 0, (size_t)n_slots * d.ctx_elems * sizeof(float), st));
    MPL_CUDA(cudaMemsetAsync(status, 0, sizeof(int), st));
  }
  if (dir_count == 0) return MPL_OK;
  mpl::BwdParams bp{};
  fill_backward(bp, p, d, context, edge_weights, nullptr, part, n_slots, 2, status);
  bp.min_idx = msg_min_index;
  bp.norm_idx = msg_norm_index;
  bp.dew = (edge_weights && dedge_weights) ? dedge_weights : nullptr;
  bp.dir = dir_first;
  bp.ndirs = dir_count;
  bp.part = p->chain_part;
  bp.parts = p->chain_parts;
  bp.dm_read = dmsg_update;
  bp.dm_acc = scatter;
  MPL_CUDA(mpl::launch_backward_sweep(bp, st));
  return MPL_OK;
}

int mpl_isgmr_backward_combine(const mpl_problem* p, int32_t dir_first, int32_t dir_count,
                               const float* scatter_total, const float* scatter, float* dmsg_update,
                               float* dunary, void* stream) {
  Dims d;
  if (int rc = validate(p, &d)) return rc;
  if (int rc = check_dir_range(p, dir_first, dir_count)) return rc;
  if (!scatter_total || (dir_count > 0 && (!scatter || !dmsg_update)))
    return fail(MPL_ERR_INVALID, "NULL tensor pointer");
  MPL_CUDA(mpl::launch_isgmr_combine_total(scatter_total, scatter, dmsg_update, dunary, d.slice, dir_first,
                                           dir_count, p->rho, static_cast<cudaStream_t>(stream)));
  return MPL_OK;
}

int mpl_backward_context_finish(const mpl_problem* p, void* workspace, size_t workspace_bytes,
                                float* dcontext, void* stream) {
  Dims d;
  if (int rc = validate(p, &d)) return rc;
  if (!dcontext) return fail(MPL_ERR_INVALID, "NULL tensor pointer");
  if (!workspace || workspace_bytes < mpl_backward_workspace_bytes(p))
    return fail(MPL_ERR_INVALID, "workspace too small: %zu < %zu", workspace_bytes,
                mpl_backward_workspace_bytes(p));
  const int n_slots = mpl::backward_slots(p->height, p->width, p->n_disp, p->n_dir, (int)d.nimg, p->context_rank);
  MPL_CUDA(mpl::launch_dctx_reduce(ws_tables(workspace), n_slots, p->n_disp, p->context_rank,
                                   p->keep_diag, dcontext, static_cast<cudaStream_t>(stream)));
  return MPL_OK;
}

// ---- soft (expected-value) TRWP ------------------------------------------------------------------
int mpl_trwp_soft_forward(const mpl_problem* p, const float* unary, const float* context,
                          const float* edge_weights, float* msg, float* cost_final, float* msg_edge_label,
                          uint8_t* msg_norm_index, uint8_t* label_all, void* workspace,
                          size_t workspace_bytes, void* stream) {
  Dims d;
  if (int rc = validate(p, &d)) return rc;
  if (int rc = check_chain_count(p, d)) return rc;
  if (p->n_disp > 64)
    return fail(MPL_ERR_UNSUPPORTED, "soft TRWP is built for n_disp <= 64 (got %d): it saves n_disp^2 values per "
                                     "pixel, direction and iteration", p->n_disp);
  if (!unary || !context || !msg || !cost_final) return fail(MPL_ERR_INVALID, "NULL tensor pointer");
  if ((msg_edge_label == nullptr) != (msg_norm_index == nullptr))
    return fail(MPL_ERR_INVALID, "msg_edge_label and msg_norm_index must both be given or both be NULL");
  if (!workspace || workspace_bytes < mpl_forward_workspace_bytes(p))
    return fail(MPL_ERR_INVALID, "workspace too small: %zu < %zu", workspace_bytes,
                mpl_forward_workspace_bytes(p));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool train = msg_edge_label != nullptr;
  const int D = p->n_dir, L = p->n_disp;
  mpl::FwdParams fp{};
  fill_forward(fp, p, d, unary, context, edge_weights, workspace);
  MPL_CUDA(cudaMemsetAsync(fp.status, 0, sizeof(int), st));
  fp.msg_read = msg;
  fp.msg_write = msg;
  for (int it = 0; it < p->n_iter; ++it) {
    fp.norm_idx = train ? msg_norm_index + (long long)it * D * d.npix : nullptr;
    fp.edge_label = train ? msg_edge_label + (long long)it * D * d.npix * L * L : nullptr;
    for (int dir = 0; dir < D; ++dir) {  // later directions see earlier ones' new messages
      set_dirs(fp, dir, 1);
      MPL_CUDA(mpl::launch_forward_soft_sweep(fp, train, st));
    }
    if (label_all)
      MPL_CUDA(mpl::launch_aggregate(unary, msg, cost_final, label_all + (long long)it * d.npix, d.npix, L, D,
                                     d.slice, 1.f, 0, st));
  }
  MPL_CUDA(mpl::launch_aggregate(unary, msg, cost_final, nullptr, d.npix, L, D, d.slice, 1.f, 0, st));
  return MPL_OK;
}

int mpl_trwp_soft_backward(const mpl_problem* p, const float* context, const float* edge_weights,
                           const float* dcost_final, const float* msg_edge_label,
                           const uint8_t* msg_norm_index, float* dunary, float* dcontext,
                           float* dedge_weights, float* dmsg, void* workspace, size_t workspace_bytes,
                           void* stream) {
  Dims d;
  if (int rc = validate(p, &d)) return rc;
  if (int rc = check_chain_count(p, d)) return rc;
  if (p->n_disp > 64) return fail(MPL_ERR_UNSUPPORTED, "soft TRWP is built for n_disp <= 64 (got %d)", p->n_disp);
  if (!context || !dcost_final || !msg_edge_label || !msg_norm_index || !dunary || !dcontext || !dmsg)
    return fail(MPL_ERR_INVALID, "NULL tensor pointer");
  if (edge_weights && !dedge_weights)
    return fail(MPL_ERR_INVALID, "dedge_weights is NULL although edge_weights is given");
  if (!workspace || workspace_bytes < mpl_backward_workspace_bytes(p))
    return fail(MPL_ERR_INVALID, "workspace too small: %zu < %zu", workspace_bytes,
                mpl_backward_workspace_bytes(p));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int D = p->n_dir, L = p->n_disp;
  const int n_slots = mpl::backward_slots(p->height, p->width, L, D, (int)d.nimg, p->context_rank);
  float* part = ws_tables(workspace);
  int* status = ws_status(workspace);
  MPL_CUDA(cudaMemsetAsync(part, 0, (size_t)n_slots * d.ctx_elems * sizeof(float), st));
  MPL_CUDA(cudaMemsetAsync(status, 0, sizeof(int), st));
  // C + P bookkeeping (BwdParams::cp_scheme == 1): C in dunary, P_k in dmsg
  MPL_CUDA(mpl::launch_backward_init(dcost_final, dunary, dmsg, d.slice, D, 1.f, 1, st));
  mpl::BwdParams bp{};
  fill_backward(bp, p, d, context, edge_weights, dunary, part, n_slots, 1, status);
  bp.dm_read = dmsg;
  bp.dm_acc = dmsg;
  bp.dew = (edge_weights && dedge_weights) ? dedge_weights : nullptr;
  for (int it = p->n_iter - 1; it >= 0; --it) {
    bp.norm_idx = msg_norm_index + (long long)it * D * d.npix;
    bp.edge_label = msg_edge_label + (long long)it * D * d.npix * L * L;
    bp.edge_label_end = msg_edge_label + (long long)p->n_iter * D * d.npix * L * L;
    for (int dir = D - 1; dir >= 0; --dir) {
      bp.dir = dir;
      MPL_CUDA(mpl::launch_backward_soft_sweep(bp, st));
    }
  }
  MPL_CUDA(mpl::launch_dctx_reduce(part, n_slots, L, p->context_rank, 1, dcontext, st));
  return MPL_OK;
}

// ---- layout glue: class scores [B,L,H,W] <-> costs [B,H,W,L] -------------------------------------
namespace {
int layout_call(int kind, const float* in, float* out, uint8_t* amax, int32_t batch, int32_t n_disp,
                int32_t height, int32_t width, void* stream) {
  if (!in || !out || ((kind == 1 || kind == 3) && !amax)) return fail(MPL_ERR_INVALID, "NULL tensor pointer");
  if (batch < 1 || height < 1 || width < 1 || n_disp < 1 || n_disp > 256 || batch > 65535)
    return fail(MPL_ERR_INVALID, "bad shape: batch=%d n_disp=%d height=%d width=%d", batch, n_disp, height, width);
  MPL_CUDA(mpl::launch_layout(kind, in, out, amax, batch, n_disp, (long long)height * width,
                              static_cast<cudaStream_t>(stream)));
  return MPL_OK;
}
}  // namespace

int mpl_scores_to_costs(const float* scores, float* costs, uint8_t* argmax, int32_t batch, int32_t n_disp,
                        int32_t height, int32_t width, void* stream) {
  return layout_call(1, scores, costs, argmax, batch, n_disp, height, width, stream);
}
int mpl_scores_to_costs_backward(const float* dcosts, const uint8_t* argmax, float* dscores, int32_t batch,
                                 int32_t n_disp, int32_t height, int32_t width, void* stream) {
  return layout_call(3, dcosts, dscores, const_cast<uint8_t*>(argmax), batch, n_disp, height, width, stream);
}
int mpl_negate_lhw_to_hwl(const float* in, float* out, int32_t batch, int32_t n_disp, int32_t height,
                          int32_t width, void* stream) {
  return layout_call(0, in, out, nullptr, batch, n_disp, height, width, stream);
}
int mpl_negate_hwl_to_lhw(const float* in, float* out, int32_t batch, int32_t n_disp, int32_t height,
                          int32_t width, void* stream) {
  return layout_call(2, in, out, nullptr, batch, n_disp, height, width, stream);
}

int mpl_permute_lhw_to_hwl(const float* in, float* out, int32_t batch, int32_t n_disp, int32_t height,
                           int32_t width, void* stream) {
  return layout_call(4, in, out, nullptr, batch, n_disp, height, width, stream);
}
int mpl_permute_hwl_to_lhw(const float* in, float* out, int32_t batch, int32_t n_disp, int32_t height,
                           int32_t width, void* stream) {
  return layout_call(5, in, out, nullptr, batch, n_disp, height, width, stream);
}

// ---- energy of labellings (evaluation of the minimisation, not part of the layer) -----------------
size_t mpl_energy_workspace_bytes(const mpl_problem* p) {
  Dims d;
  if (validate(p, &d) != MPL_OK) return 256;
  return (size_t)((d.npix + 255) / 256) * 2 * sizeof(double) + 256;
}

int mpl_labeling_energy(const mpl_problem* p, const float* unary, const float* context,
                        const float* edge_weights, const uint8_t* labels, int32_t n_labelings,
                        double* energy, void* workspace, size_t workspace_bytes, void* stream) {
  Dims d;
  if (int rc = validate(p, &d)) return rc;
  if (!unary || !context || !labels || !energy || n_labelings < 0)
    return fail(MPL_ERR_INVALID, "NULL tensor pointer or negative count");
  if (!workspace || workspace_bytes < mpl_energy_workspace_bytes(p))
    return fail(MPL_ERR_INVALID, "workspace too small: %zu < %zu", workspace_bytes, mpl_energy_workspace_bytes(p));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  for (int i = 0; i < n_labelings; ++i)
    MPL_CUDA(mpl::launch_energy(unary, context, edge_weights, labels + (long long)i * d.npix, d.npix, p->height,
                                p->width, p->n_disp, p->n_dir, p->context_rank, static_cast<double*>(workspace),
                                energy + 2 * i, st));
  return MPL_OK;
}

// ---- stand-alone soft-weighted message ops ---------------------------------------------------------
int mpl_soft_weighted_message(const float* message, int64_t n_tables, int32_t n_disp,
                              float* message_soft_sum_norm, uint8_t* message_soft_sum_min_ind, void* stream) {
  if (n_tables < 0 || n_tables >= (1ll << 31)) return fail(MPL_ERR_INVALID, "n_tables=%lld", (long long)n_tables);
  if (n_disp < 1 || n_disp > 256) return fail(MPL_ERR_UNSUPPORTED, "n_disp=%d outside 1..256", n_disp);
  if (n_tables == 0) return MPL_OK;
  if (!message || !message_soft_sum_norm || !message_soft_sum_min_ind)
    return fail(MPL_ERR_INVALID, "NULL tensor pointer");
  MPL_CUDA(mpl::launch_soft_weighted_message(message, n_tables, n_disp, message_soft_sum_norm,
                                             message_soft_sum_min_ind, static_cast<cudaStream_t>(stream)));
  return MPL_OK;
}

int mpl_soft_weighted_message_backward(const float* dmessage_soft_sum_norm, const float* message,
                                       const uint8_t* message_soft_sum_min_ind, int64_t n_tables,
                                       int32_t n_disp, float* dmessage, void* stream) {
  if (n_tables < 0 || n_tables >= (1ll << 31)) return fail(MPL_ERR_INVALID, "n_tables=%lld", (long long)n_tables);
  if (n_disp < 1 || n_disp > 256) return fail(MPL_ERR_UNSUPPORTED, "n_disp=%d outside 1..256", n_disp);
  if (n_tables == 0) return MPL_OK;
  if (!dmessage_soft_sum_norm || !message || !message_soft_sum_min_ind || !dmessage)
    return fail(MPL_ERR_INVALID, "NULL tensor pointer");
  MPL_CUDA(mpl::launch_soft_weighted_message_back(dmessage_soft_sum_norm, message, message_soft_sum_min_ind,
                                                  n_tables, n_disp, dmessage, static_cast<cudaStream_t>(stream)));
  return MPL_OK;
}

// ---- input builders -----------------------------------------------------------------------------
int mpl_stereo_data_cost(const uint8_t* left, const uint8_t* right, int32_t height, int32_t width,
                         int32_t channels, int32_t n_disp, int32_t birchfield, int32_t squared_diffs,
                         int32_t trunc_diffs, float* data_cost, void* stream) {
  if (!left || !right || !data_cost) return fail(MPL_ERR_INVALID, "NULL tensor pointer");
  if (height < 1 || width < 1 || channels < 1 || n_disp < 1)
    return fail(MPL_ERR_INVALID, "bad shape: height=%d width=%d channels=%d n_disp=%d", height, width, channels,
                n_disp);
  if (n_disp > 256) return fail(MPL_ERR_UNSUPPORTED, "n_disp=%d outside 1..256", n_disp);
  if (height > 65535) return fail(MPL_ERR_UNSUPPORTED, "height=%d above 65535", height);
  if ((long long)height * width * n_disp >= (1ll << 40)) return fail(MPL_ERR_UNSUPPORTED, "volume too large");
  if (trunc_diffs < -32767 || trunc_diffs > 32767) return fail(MPL_ERR_INVALID, "trunc_diffs=%d", trunc_diffs);
  MPL_CUDA(mpl::launch_stereo_data_cost(left, right, height, width, channels, n_disp, birchfield != 0,
                                        squared_diffs != 0, trunc_diffs, data_cost,
                                        static_cast<cudaStream_t>(stream)));
  return MPL_OK;
}

int mpl_gradient_cues(const uint8_t* image, int32_t height, int32_t width, int32_t channels,
                      int32_t grad_thresh, int32_t grad_penalty, int32_t compact, float* h_cue, float* v_cue,
                      void* stream) {
  if (!image || !h_cue || !v_cue) return fail(MPL_ERR_INVALID, "NULL tensor pointer");
  if (height < 1 || width < 1 || channels < 1)
    return fail(MPL_ERR_INVALID, "bad shape: height=%d width=%d channels=%d", height, width, channels);
  if (grad_thresh < -10000 || grad_thresh > 10000) return fail(MPL_ERR_INVALID, "grad_thresh=%d", grad_thresh);
  if ((long long)height * width >= (1ll << 31)) return fail(MPL_ERR_UNSUPPORTED, "height*width must be below 2^31");
  MPL_CUDA(mpl::launch_gradient_cues(image, height, width, channels, grad_thresh, grad_penalty, compact != 0,
                                     h_cue, v_cue, static_cast<cudaStream_t>(stream)));
  return MPL_OK;
}

int mpl_smoothness_context(int32_t n_disp, const char* method, float smoothness_max, float* context,
                           void* stream) {
  static const char* const kNames[] = {"L", "Q", "TL", "TQ", "Cauchy", "Huber"};
  if (!method || !context) return fail(MPL_ERR_INVALID, "NULL pointer");
  if (n_disp < 1 || n_disp > 256) return fail(MPL_ERR_UNSUPPORTED, "n_disp=%d outside 1..256", n_disp);
  int id = -1;
  for (int i = 0; i < 6; ++i)
    if (!strcmp(method, kNames[i])) id = i;
  if (id < 0) return fail(MPL_ERR_UNSUPPORTED, "smoothness method \"%s\" (known: L Q TL TQ Cauchy Huber)", method);
  MPL_CUDA(mpl::launch_smoothness_context(n_disp, id, smoothness_max, context, static_cast<cudaStream_t>(stream)));
  return MPL_OK;
}

int32_t mpl_edge_mode(const char* name) {
  static const struct { const char* name; int id; } kModes[] = {
      {"gt_edge", 0}, {"superpixel_edge", 1}, {"canny", 2}, {"sobel", 3}, {"edge_net_sigmoid", 3},
      {"edge_net", 4}, {"kernel_cue_real", 5}, {"kernel_cue_binary", 6}, {"threshold", 7},
      {"shifted", 8}, {"cue_penalty", 9}};
  if (!name) return -1;
  for (const auto& m : kModes)
    if (!strcmp(name, m.name)) return m.id;
  return -1;
}

int32_t mpl_edge_mode_channels(int32_t mode, int32_t channels) {
  if (mode < 0 || mode > 9 || channels < 1) return -1;
  return mpl::edge_weights_reduces(mode) ? 1 : channels;
}

int mpl_edge_weights(int32_t mode, const float* image, int32_t batch, int32_t channels, int32_t height,
                     int32_t width, int32_t n_dir, float sigma, float threshold, float penalty,
                     float* edge_weights, void* workspace, size_t workspace_bytes, void* stream) {
  if (!image || !edge_weights) return fail(MPL_ERR_INVALID, "NULL tensor pointer");
  if (mode < 0 || mode > 9) return fail(MPL_ERR_INVALID, "edge mode %d outside 0..9", mode);
  if (batch < 1 || channels < 1 || height < 1 || width < 1)
    return fail(MPL_ERR_INVALID, "bad shape: batch=%d channels=%d height=%d width=%d", batch, channels, height,
                width);
  if (n_dir < 1 || n_dir > 16) return fail(MPL_ERR_UNSUPPORTED, "n_dir=%d outside 1..16", n_dir);
  if ((long long)height * width >= (1ll << 31) || batch > 65535)
    return fail(MPL_ERR_UNSUPPORTED, "height*width must be below 2^31 and batch at most 65535");
  if (mode == 6 && (!workspace || workspace_bytes < sizeof(double) * 16))
    return fail(MPL_ERR_INVALID, "kernel_cue_binary needs a workspace of 128 bytes");
  if ((mode == 5 || mode == 6) && !(sigma != 0.f)) return fail(MPL_ERR_INVALID, "sigma must be non-zero");
  MPL_CUDA(mpl::launch_edge_weights(image, batch, channels, height, width, n_dir, mode, sigma, threshold, penalty,
                                    edge_weights, static_cast<double*>(workspace),
                                    static_cast<cudaStream_t>(stream)));
  return MPL_OK;
}

int mpl_workspace_status(const void* workspace, int32_t* status) {
  if (!workspace || !status) return fail(MPL_ERR_INVALID, "NULL pointer");
  MPL_CUDA(cudaMemcpy(status, static_cast<const char*>(workspace) + kStatusOffset, sizeof(int32_t),
                      cudaMemcpyDeviceToHost));
  return MPL_OK;
}

int mpl_forward_status(const void* workspace, int32_t* status) { return mpl_workspace_status(workspace, status); }

size_t mpl_workspace_status_offset(void) { return kStatusOffset; }

}  // extern "C"

namespace {
// One warp waits on an mbarrier that nothing ever arrives at, with a limit of `limit_cycles`
// clocks: the wait must give up, record its code and let the kernel return.
__global__ void selftest_wait_kernel(int* status, long long limit_cycles) {
  __shared__ unsigned long long bar;
  if (threadIdx.x == 0) {
    mpl::mbar_init(&bar, 1);
    mpl::mbar_fence_init();
  }
  __syncwarp();
  if (!mpl::mbar_wait(&bar, 0, limit_cycles)) {
    if (threadIdx.x == 0) atomicExch(status, 901);
  }
}
}  // namespace

extern "C" {

int mpl_selftest_bounded_wait(void* workspace, size_t workspace_bytes, int64_t limit_cycles, void* stream) {
  if (!workspace || workspace_bytes < 256) return fail(MPL_ERR_INVALID, "workspace of at least 256 bytes needed");
  if (limit_cycles < 1 || limit_cycles > 2000000000ll)
    return fail(MPL_ERR_INVALID, "limit_cycles=%lld outside 1..2e9", (long long)limit_cycles);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MPL_CUDA(cudaMemsetAsync(ws_status(workspace), 0, sizeof(int), st));
  selftest_wait_kernel<<<1, 32, 0, st>>>(ws_status(workspace), (long long)limit_cycles);
  mpl::count_launch();
  MPL_CUDA(cudaGetLastError());
  return MPL_OK;
}

// ---- TRWP backward for callers that cannot allocate device memory ------------------------------
// The scratch of mpl_trwp_backward (per-chain label-context partial tables + a status word) lives
// in this file-scope device array instead of a caller-provided workspace.  The array's name is only
// a host-side handle; kernels need its device address, fetched once per device below.
#define MPL_STATIC_SCRATCH_BYTES (8u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[MPL_STATIC_SCRATCH_BYTES];

size_t mpl_static_scratch_bytes(void) { return MPL_STATIC_SCRATCH_BYTES; }

int mpl_trwp_backward_static(const mpl_problem* p, const float* context, const float* edge_weights,
                             const float* dcost_final, const uint8_t* msg_min_index,
                             const uint8_t* msg_norm_index, float* dunary, float* dcontext,
                             float* dedge_weights, float* dmsg, void* stream) {
  Dims d;
  if (int rc = validate(p, &d)) return rc;
  const size_t need = mpl_backward_workspace_bytes(p);
  if (need > MPL_STATIC_SCRATCH_BYTES)
    return fail(MPL_ERR_UNSUPPORTED,
                "problem needs %zu bytes of scratch, the built-in scratch holds %u; use mpl_trwp_backward "
                "with a caller-provided workspace",
                need, MPL_STATIC_SCRATCH_BYTES);
  // one-time set-up per device (with that device current): resolve the array's device address
  static std::mutex mu;
  static void* addr[64] = {nullptr};
  int dev = 0;
  MPL_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(MPL_ERR_UNSUPPORTED, "device ordinal %d not supported", dev);
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lk(mu);
    if (!addr[dev]) {
      void* ptr = nullptr;
      MPL_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
      addr[dev] = ptr;
    }
    scratch = addr[dev];
  }
  // backward_common clears the part of the scratch it uses (partial tables and status word)
  return backward_common(false, p, context, edge_weights, dcost_final, msg_min_index, msg_norm_index, dunary,
                         dcontext, dedge_weights, dmsg, nullptr, scratch, MPL_STATIC_SCRATCH_BYTES, stream);
}

int mpl_static_scratch_status(int32_t* status) {
  if (!status) return fail(MPL_ERR_INVALID, "NULL pointer");
  void* ptr = nullptr;
  MPL_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
  return mpl_workspace_status(ptr, status);
}

const char* mpl_last_error(void) { return g_err.c_str(); }

int64_t mpl_kernel_launches(void) { return mpl::g_launches.load(std::memory_order_relaxed); }

int32_t mpl_version(void) { return 100; }

int32_t mpl_chain_count(int32_t dir, int32_t height, int32_t width) {
  if (dir < 0 || dir > 15 || height < 1 || width < 1) return -1;
  return mpl::make_geom(dir, height, width).n_chains;
}

int32_t mpl_chain_geometry(int32_t dir, int32_t height, int32_t width, int32_t chain, int32_t* out5) {
  if (dir < 0 || dir > 15 || height < 1 || width < 1 || !out5) return MPL_ERR_INVALID;
  const mpl::DirGeom g = mpl::make_geom(dir, height, width);
  if (chain < 0 || chain >= g.n_chains) return MPL_ERR_INVALID;
  int h0, w0, len;
  mpl::chain_start(g, height, width, chain, h0, w0, len);
  out5[0] = h0;
  out5[1] = w0;
  out5[2] = len;
  out5[3] = g.hs;
  out5[4] = g.ws;
  return MPL_OK;
}

void mpl_profile_enable(int32_t on) { mpl::g_prof_on.store(on ? 1 : 0); }

int32_t mpl_profile_read(int32_t kind, double* total_ms, int64_t* launches) {
  if (kind < 0 || kind >= mpl::kProfKinds) return MPL_ERR_INVALID;
  std::lock_guard<std::mutex> lk(mpl::g_prof_mu);
  for (auto& pr : mpl::g_prof_pending) {
    float ms = 0.f;
    if (cudaEventSynchronize(pr.b) == cudaSuccess && cudaEventElapsedTime(&ms, pr.a, pr.b) == cudaSuccess) {
      mpl::g_prof_ms[pr.kind] += ms;
      mpl::g_prof_n[pr.kind] += 1;
    }
    cudaEventDestroy(pr.a);
    cudaEventDestroy(pr.b);
  }
  mpl::g_prof_pending.clear();
  if (total_ms) *total_ms = mpl::g_prof_ms[kind];
  if (launches) *launches = mpl::g_prof_n[kind];
  return MPL_OK;
}

void mpl_profile_reset(void) {
  mpl_profile_read(0, nullptr, nullptr);
  std::lock_guard<std::mutex> lk(mpl::g_prof_mu);
  for (int k = 0; k < mpl::kProfKinds; ++k) {
    mpl::g_prof_ms[k] = 0.0;
    mpl::g_prof_n[k] = 0;
  }
}

}  // extern "C"
