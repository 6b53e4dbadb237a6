/*
 * mplayers_b200 -- C ABI of the TRWP / ISGMR min-sum message-passing layers for NVIDIA B200
 * (sm_100a).  Plain pointers and sizes only; every pointer is DEVICE memory of the current CUDA
 * device unless stated otherwise, and every call is asynchronous on `stream` (a cudaStream_t
 * passed as void*; NULL = the legacy default stream).
 *
 * Tensor layouts are the reference extension's (all contiguous, fp32 values, u8 indices):
 *   unary, cost_final, dcost_final, dunary ....... [B, cv, H, W, L]
 *   msg, msg_update, dmsg, dmsg_update ........... [D, B, cv, H, W, L]
 *   edge_weights, dedge_weights .................. [D, B, cv, H, W]   (weight of edge front->cur at cur)
 *   msg_min_index ................................ [I, D, B, cv, H, W, L]   u8
 *   msg_norm_index ............................... [I, D, B, cv, H, W]      u8
 *   label_all .................................... [I, B, cv, H, W]         u8
 *   context ...................................... [L] (rank 1: ctx[|c-f|]) or [L, L] (rank 2: read
 *                                                  as ctx[min(c,f)][max(c,f)], upper triangle)
 * The reference selects the context convention by `L == 21`; here it is `context_rank`.
 *
 * Every function returns MPL_OK or an error code; mpl_last_error() gives the message of the last
 * failure on the calling thread.  Nothing is computed on the CPU: without a CUDA device the
 * compute entry points fail with MPL_ERR_CUDA.
 */
#ifndef MPLAYERS_B200_H_
#define MPLAYERS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MPL_OK 0
#define MPL_ERR_INVALID 1     /* bad shape, NULL pointer, workspace too small */
#define MPL_ERR_UNSUPPORTED 2 /* e.g. n_disp > 256, odd n_dir */
#define MPL_ERR_CUDA 3        /* a CUDA runtime call failed */

/* Problem description.  Replaces the shape reads the reference does from its at::Tensor
 * arguments (MPLayers/TRWP/TRWP_forward.cu:390-408, MPLayers/TRWP/TRWP_backward.cu:288-294) and
 * the scalar arguments of Forward()/Backward() (MPLayers/TRWP/TRWP.cpp:245-256,285-295;
 * MPLayers/ISGMR/ISGMR.cpp:300-313,344-356). */
typedef struct mpl_problem {
  int32_t n_iter;           /* I */
  int32_t n_dir;            /* D: 2..16, even; directions 0..D-1 of MPLayers/common.cpp:28-76 */
  int32_t batch;            /* B */
  int32_t n_cv;             /* cv (second batch-like axis) */
  int32_t height;           /* H */
  int32_t width;            /* W */
  int32_t n_disp;           /* L: 1..256 */
  int32_t context_rank;     /* 1 or 2 */
  int32_t enable_min_a_dir; /* cost = U + min_d M_d instead of U + sum_d M_d */
  int32_t enable_sgm;       /* ISGMR only: cost = D*U + sum_d M_d */
  int32_t keep_diag;        /* backward: 1 = also accumulate dcontext where c == f (what
                               MPLayers/TRWP_hard_soft does), 0 = skip it (TRWP / ISGMR libs,
                               MPLayers/TRWP/TRWP_backward.cu:111-112) */
  float rho;                /* 0.5 for TRWP, 1 for ISGMR (pytorch/MP_module.py:172) */
  int32_t context_window;   /* rank-1 context with more than 32 labels only; else ignored.
                               0: unknown -- the forward call analyses context and edge weights on the
                                  device and reads the result back, i.e. it waits for `stream` once;
                                  while `stream` is being captured it does not wait and evaluates all
                                  L candidates per label instead;
                               R > 0: the caller states that context[k] is non-decreasing for k < R,
                                  equal to context[L-1] for k >= R, and that no edge weight is negative
                                  (what mpl_analyze_context reports) -- no read-back, fully
                                  asynchronous; a wrong statement gives wrong results;
                               -1: evaluate all L candidates per label.
                               Backward calls never read anything back; there a value R > 0 is only a
                               hint for how the scatter of a rank-1 context with more than 32 labels
                               is split (any value gives the same sums). */
  int32_t chain_part;       /* iteration-level ISGMR entry points only (mpl_isgmr_forward_directions, */
  int32_t chain_parts;      /* mpl_isgmr_backward_directions): the call runs part chain_part of
                               chain_parts of the chains of each of its directions (chains of the even
                               direction of a pair in the order of mpl_chain_geometry, images outermost;
                               the odd direction walks the same lines from their other end, so that a
                               part holds both messages of every line it owns); chain_parts <= 1: all chains.
                               Lets more ranks than direction pairs share one image: pixels a call
                               does not visit are left untouched in every output. */
  int32_t cost_labels_first; /* mpl_trwp_forward / mpl_isgmr_forward and their backward calls: 1 = cost_final and
                               dcost_final are [B, cv, L, H, W] (the layout pytorch/MP_module.py:232 hands back
                               after its permute) instead of [B, cv, H, W, L]; the final aggregation writes and
                               the backward prologue reads that layout directly, so the caller needs no
                               separate layout pass.  Every other tensor keeps the labels last. */
} mpl_problem;

/* Analyses a rank-1 context (and the edge weights, may be NULL) for mpl_problem::context_window:
 * *window receives R > 0 if min over the 2R-1 nearest labels plus one global term is exact (see
 * above), else -1.  Synchronous (waits for `stream`); call it once per context, not per step.
 * The reference evaluates all L candidates always (MPLayers/TRWP/TRWP_forward.cu:126-152). */
int mpl_analyze_context(const mpl_problem* p, const float* context, const float* edge_weights,
                        int32_t* window, void* workspace, size_t workspace_bytes, void* stream);

/* Bytes of device scratch the forward / backward entry points need for `p` (never 0). */
size_t mpl_forward_workspace_bytes(const mpl_problem* p);
size_t mpl_backward_workspace_bytes(const mpl_problem* p);

/* TRWP forward.  Replaces TRWP.forward of the reference extension
 * (MPLayers/TRWP/TRWP.cpp:245-283,323-326 -> ForwardCUDA, MPLayers/TRWP/TRWP_forward.cu:378-564).
 *   msg            in/out: the messages the first iteration starts from -- zero as the reference
 *                  allocates them (pytorch/MP_module.py:26), or those of an earlier call (pixels
 *                  without a predecessor must hold 0: no sweep writes them); holds the final
 *                  messages on exit
 *   edge_weights   NULL = every weight is 1
 *   msg_min_index, msg_norm_index   both NULL = inference (nothing saved); both non-NULL = training
 *   label_all      NULL = do not save per-iteration labels
 * The reference's `unary_update` scratch argument has no counterpart (the update is fused). */
int mpl_trwp_forward(const mpl_problem* p, const float* unary, const float* context,
                     const float* edge_weights, float* msg, float* cost_final,
                     uint8_t* msg_min_index, uint8_t* msg_norm_index, uint8_t* label_all,
                     void* workspace, size_t workspace_bytes, void* stream);

/* TRWP backward.  Replaces TRWP.backward (MPLayers/TRWP/TRWP.cpp:285-321 -> BackwardCUDA,
 * MPLayers/TRWP/TRWP_backward.cu:277-437).
 *   dunary          out (overwritten)
 *   dcontext        accumulated into ([L] or [L,L]; zero it for a plain gradient)
 *   dedge_weights   accumulated into; may be NULL when edge_weights is NULL
 *   dmsg            scratch [D,B,cv,H,W,L], contents on entry ignored
 * The reference's `dunary_update` scratch argument has no counterpart. */
int mpl_trwp_backward(const mpl_problem* p, const float* context, const float* edge_weights,
                      const float* dcost_final, const uint8_t* msg_min_index,
                      const uint8_t* msg_norm_index, float* dunary, float* dcontext,
                      float* dedge_weights, float* dmsg, void* workspace, size_t workspace_bytes,
                      void* stream);

/* ISGMR (and SGM) forward.  Replaces ISGMR.forward (MPLayers/ISGMR/ISGMR.cpp:300-342,399-404 ->
 * ForwardCUDA, MPLayers/ISGMR/ISGMR_forward.cu:433-665).  The iterations start from the messages in
 * `msg` (zero as the reference allocates them, or those of an earlier call), whatever the label and
 * direction counts; msg_update must hold 0 at the pixels without a predecessor (zero it once).  The
 * two buffers are used alternately instead of being copied every iteration (an odd n_iter costs one
 * copy at the start); on exit `msg` holds the final messages, `msg_update` those of the iteration
 * before. */
int mpl_isgmr_forward(const mpl_problem* p, const float* unary, const float* context,
                      const float* edge_weights, float* msg, float* msg_update, float* cost_final,
                      uint8_t* msg_min_index, uint8_t* msg_norm_index, uint8_t* label_all,
                      void* workspace, size_t workspace_bytes, void* stream);

/* ISGMR backward.  Replaces ISGMR.backward (MPLayers/ISGMR/ISGMR.cpp:344-397 -> BackwardCUDA,
 * MPLayers/ISGMR/ISGMR_backward.cu:290-497).  dmsg and dmsg_update are scratch [D,B,cv,H,W,L],
 * contents on entry ignored. */
int mpl_isgmr_backward(const mpl_problem* p, const float* context, const float* edge_weights,
                       const float* dcost_final, const uint8_t* msg_min_index,
                       const uint8_t* msg_norm_index, float* dunary, float* dcontext,
                       float* dedge_weights, float* dmsg, float* dmsg_update, void* workspace,
                       size_t workspace_bytes, void* stream);

/* ---- Soft (expected-value) TRWP ------------------------------------------------------------------
 * The message is the expectation of the edge values under softmin weights instead of their
 * minimum.  Replaces TRWP_hard_soft.forward_soft / backward_soft of the reference
 * (MPLayers/TRWP_hard_soft/TRWP.cpp:433-436 -> ForwardCUDASoft / BackwardCUDASoft,
 * MPLayers/TRWP_hard_soft/TRWP_forward_soft.cu:418-558, TRWP_backward_soft.cu:400-551).
 *   msg_edge_label [I,D,B,cv,H,W,L,L] f32: the edge values of every visited pixel, entry [f][c]
 *                  (front label f, label c) for even directions and [c][f] for odd ones, as the
 *                  reference stores them; msg_norm_index [I,D,B,cv,H,W] u8.  Both NULL = inference.
 *   n_disp <= 64 (MPL_ERR_UNSUPPORTED beyond: L*L values are saved per pixel, direction, iteration;
 *   up to 32 labels one warp per chain, 33..64 one CTA of 64 threads per chain).
 * Forward values agree with the reference kernels bit for bit (same intrinsics, same reduction
 * order); the backward accumulates dcontext on the diagonal too, as the reference does
 * (TRWP_backward_soft.cu:114-126).  dmsg is scratch [D,B,cv,H,W,L]. */
int mpl_trwp_soft_forward(const mpl_problem* p, const float* unary, const float* context,
                          const float* edge_weights, float* msg, float* cost_final,
                          float* msg_edge_label, uint8_t* msg_norm_index, uint8_t* label_all,
                          void* workspace, size_t workspace_bytes, void* stream);
int mpl_trwp_soft_backward(const mpl_problem* p, const float* context, const float* edge_weights,
                           const float* dcost_final, const float* msg_edge_label,
                           const uint8_t* msg_norm_index, float* dunary, float* dcontext,
                           float* dedge_weights, float* dmsg, void* workspace,
                           size_t workspace_bytes, void* stream);

/* ---- ISGMR one iteration at a time, over a subset of directions --------------------------------
 * The D sweeps of an ISGMR iteration only read the previous iteration's messages
 * (MPLayers/ISGMR/ISGMR_forward.cu:506-622), so they can run on different GPUs; what couples them
 * is the per-pixel sum over ALL directions that the next iteration's update needs (and, in the
 * backward, the sum of all scatter fields).  These entry points do one iteration for the
 * directions [dir_first, dir_first + dir_count) -- whole pairs (d, d^1): dir_first and dir_count
 * even -- and leave the two sums to the caller, who forms them with mpl_sum_directions and one
 * all-reduce per iteration (mplayers_b200/parallel.py does it over torch.distributed).  The
 * monolithic mpl_isgmr_forward / mpl_isgmr_backward are these loops with dir_count = D.  They
 * replace, per iteration, the loop bodies of ForwardCUDA / BackwardCUDA of the reference
 * (MPLayers/ISGMR/ISGMR_forward.cu:506-647, MPLayers/ISGMR/ISGMR_backward.cu:353-484). */

/* Forward sweeps of one iteration.
 *   aggregate   [B,cv,H,W,L]: unary + sum over ALL D directions of the previous messages
 *               (the unaries themselves in the first iteration, when the messages are zero)
 *   msg_read    [D,...] previous messages; only the slices d and d^1 of the given directions are read
 *   msg_write   [D,...] (another buffer); the slices of the given directions are written
 *   msg_min_index [D,B,cv,H,W,L], msg_norm_index [D,B,cv,H,W]: THIS iteration's part of the saved
 *               indices (both NULL = inference); only the given directions' slices are written */
int mpl_isgmr_forward_directions(const mpl_problem* p, int32_t dir_first, int32_t dir_count,
                                 const float* aggregate, const float* context,
                                 const float* edge_weights, const float* msg_read, float* msg_write,
                                 uint8_t* msg_min_index, uint8_t* msg_norm_index, void* workspace,
                                 size_t workspace_bytes, void* stream);

/* out[B,cv,H,W,L] = base * base_factor + sum over the given directions of fields[d]
 * (fields [D,B,cv,H,W,L]; base may be NULL: plain sum; any dir_first / dir_count inside 0..D). */
int mpl_sum_directions(const mpl_problem* p, int32_t dir_first, int32_t dir_count, const float* base,
                       float base_factor, const float* fields, float* out, void* stream);
/* The same for elements [first_element, first_element + n_elements) of the field only (the same
 * pointers as above): lets a caller form the sum chunk by chunk and hand each chunk to a
 * collective while the next one is being summed. */
int mpl_sum_directions_range(const mpl_problem* p, int32_t dir_first, int32_t dir_count, const float* base,
                             float base_factor, const float* fields, float* out, int64_t first_element,
                             int64_t n_elements, void* stream);

/* Backward sweeps of one iteration: replays the given directions' chains from this iteration's
 * saved indices.
 *   dmsg_update [D,...] gradient w.r.t. the messages this iteration produced; given slices read
 *   scatter     [D,...] out: slice d receives the field q_d the sweep scatters to the pixels'
 *               predecessors (what the reference adds into dunary_update, ISGMR_backward.cu:101-103)
 *   dedge_weights accumulated into (given slices); may be NULL when edge_weights is NULL
 *   workspace   of mpl_backward_workspace_bytes(p): label-context partial tables, accumulated over
 *               calls; pass clear_workspace = 1 on the first call of a backward pass */
int mpl_isgmr_backward_directions(const mpl_problem* p, int32_t dir_first, int32_t dir_count,
                                  const float* context, const float* edge_weights,
                                  float* dmsg_update, const uint8_t* msg_min_index,
                                  const uint8_t* msg_norm_index, float* scatter,
                                  float* dedge_weights, void* workspace, size_t workspace_bytes,
                                  int32_t clear_workspace, void* stream);

/* After the scatter fields of ALL directions have been summed into scatter_total [B,cv,H,W,L]:
 * dmsg_update[k] = rho*Q - rho*q_k - q_(k^1) for the given directions (now the gradient w.r.t. the
 * messages the iteration read) and dunary += rho*Q (skipped when dunary is NULL).  Restates
 * UpdateUnaryKernelBack + SumMsgKernel (MPLayers/ISGMR/ISGMR_backward.cu:39-60,8-16). */
int mpl_isgmr_backward_combine(const mpl_problem* p, int32_t dir_first, int32_t dir_count,
                               const float* scatter_total, const float* scatter, float* dmsg_update,
                               float* dunary, void* stream);

/* Sums the label-context partial tables of `workspace` into dcontext (accumulating), with the
 * reference's cell addressing (MPLayers/ISGMR/ISGMR_backward.cu:104-115). */
int mpl_backward_context_finish(const mpl_problem* p, void* workspace, size_t workspace_bytes,
                                float* dcontext, void* stream);

/* Layout glue around the layer.  Network code holds class scores as [B,L,H,W] planes; the layer
 * takes costs [B,(cv=1),H,W,L].  The reference converts with six elementwise passes: costs = -scores,
 * minus the per-pixel minimum, permute, layer, permute back, negate (mpnet.py:161-169,
 * pytorch/MP_module.py:198,232).  Each of these is one pass, coalesced on both sides:
 *   mpl_scores_to_costs            costs[b,p,l] = max_l scores[b,:,p] - scores[b,l,p]; argmax [B,H,W] u8
 *                                  saved for the backward (lowest index among equal maxima)
 *   mpl_scores_to_costs_backward   dscores[b,l,p] = -dcosts[b,p,l] + (l == argmax[b,p]) * sum_l dcosts[b,p,:]
 *   mpl_negate_hwl_to_lhw          scores_out[b,l,p] = -cost_final[b,p,l]   (and its backward:)
 *   mpl_negate_lhw_to_hwl          out[b,p,l] = -in[b,l,p]
 *   mpl_permute_lhw_to_hwl / mpl_permute_hwl_to_lhw   the plain layout change of the module call,
 *                                  unary [B*cv,L,H,W] -> [B*cv,H,W,L] and back (pytorch/MP_module.py:198,232) */
int mpl_scores_to_costs(const float* scores, float* costs, uint8_t* argmax, int32_t batch,
                        int32_t n_disp, int32_t height, int32_t width, void* stream);
int mpl_scores_to_costs_backward(const float* dcosts, const uint8_t* argmax, float* dscores,
                                 int32_t batch, int32_t n_disp, int32_t height, int32_t width,
                                 void* stream);
int mpl_negate_lhw_to_hwl(const float* in, float* out, int32_t batch, int32_t n_disp, int32_t height,
                          int32_t width, void* stream);
int mpl_negate_hwl_to_lhw(const float* in, float* out, int32_t batch, int32_t n_disp, int32_t height,
                          int32_t width, void* stream);
int mpl_permute_lhw_to_hwl(const float* in, float* out, int32_t batch, int32_t n_disp, int32_t height,
                           int32_t width, void* stream);
int mpl_permute_hwl_to_lhw(const float* in, float* out, int32_t batch, int32_t n_disp, int32_t height,
                           int32_t width, void* stream);

/* Energy of labellings on the MRF the layers minimise, for energy-versus-iteration curves from the
 * per-iteration labels `label_all` of a forward call.  energy [n_labelings, 2] (f64, device):
 * {sum_p U[p, x_p], sum over undirected edges (p - step_d, p), d even, of E_d[p] * ctx(x_p, x_front)}.
 * For 4 directions this is what the reference's evaluation script computes from the saved
 * labellings (tools/matlab/MRF/calEnergy.m:23-46: right and down links); the reference has no GPU
 * counterpart.  labels [n_labelings, B, cv, H, W] u8; workspace of mpl_energy_workspace_bytes(p). */
size_t mpl_energy_workspace_bytes(const mpl_problem* p);
int mpl_labeling_energy(const mpl_problem* p, const float* unary, const float* context,
                        const float* edge_weights, const uint8_t* labels, int32_t n_labelings,
                        double* energy, void* workspace, size_t workspace_bytes, void* stream);

/* TRWP backward without any device allocation.  It has no counterpart in the reference.
 *
 * Same computation and arguments as mpl_trwp_backward, minus the workspace: the scratch (partial
 * label-context tables, one per chain, and a status word) is a fixed array of
 * mpl_static_scratch_bytes() = 8 MiB that is part of the library image, so every GPU that loads
 * the library carries it until the process exits.  Meant for callers that must not allocate on the
 * device at call time -- code running inside a memory pool that is already fully handed out, a
 * capture-safe or real-time section where cudaMalloc's implicit synchronisation is unacceptable,
 * a plugin whose host forbids allocator calls.  The function itself calls no cudaMalloc/cudaFree
 * and no allocating library routine.
 *   - Problems whose mpl_backward_workspace_bytes() exceeds the 8 MiB are rejected with
 *     MPL_ERR_UNSUPPORTED and a message naming both sizes (the segmentation configuration, 2 x
 *     512 x 512 pixels with 21 labels, needs 7.2 MB).
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress) with that device current; make that first call outside any stream
 *     capture.
 *   - All calls on a device share the one array; each call clears what it uses first, but two
 *     calls whose kernels overlap on the GPU (different streams) race on it.  Serialise them. */
size_t mpl_static_scratch_bytes(void);
int mpl_trwp_backward_static(const mpl_problem* p, const float* context, const float* edge_weights,
                             const float* dcost_final, const uint8_t* msg_min_index,
                             const uint8_t* msg_norm_index, float* dunary, float* dcontext,
                             float* dedge_weights, float* dmsg, void* stream);

/* Device status word.  The bulk-copy staged kernels wait on mbarriers; every such wait is bounded
 * (about a second) and, when it gives up, records a code in the status word of the call's
 * workspace and lets its warp return, so that the context stays usable.  The word sits at byte
 * mpl_workspace_status_offset() (= 64) of every workspace, forward or backward; every call clears
 * it first.  mpl_workspace_status reads it back (synchronously: it waits for the device) after the
 * call that used the workspace: 0 = every kernel ran to completion, otherwise the code of the wait
 * that gave up -- forward staging 101 / 102 (labels <= 32), 111 / 112 and 121 / 122 (one CTA per
 * chain, many labels per lane), 131 / 132 (two labels per lane); backward staging 201 / 202
 * (labels <= 32), 141 (two labels per lane), 161 (several labels per lane), 151 (soft TRWP); 901 the
 * self-test below -- and the call's outputs must be discarded.  mpl_static_scratch_status
 * does the same for the built-in scratch of mpl_trwp_backward_static on the current device.
 * mpl_forward_status is the older name of mpl_workspace_status.  No counterpart in the reference,
 * whose kernels never wait on anything.
 *
 * mpl_selftest_bounded_wait launches one warp that waits, with a limit of `limit_cycles` clocks, on
 * an mbarrier nothing ever arrives at, so that the give-up path (status code 901) can be exercised
 * without a fault, a trap or an unbounded spin. */
int mpl_workspace_status(const void* workspace, int32_t* status);
int mpl_forward_status(const void* workspace, int32_t* status);
int mpl_static_scratch_status(int32_t* status);
size_t mpl_workspace_status_offset(void);
int mpl_selftest_bounded_wait(void* workspace, size_t workspace_bytes, int64_t limit_cycles, void* stream);

/* Stand-alone soft-weighted message ops of the reference's TRWP_hard_soft extension
 * (`soft_weighted_message`, `soft_weighted_message_back`: MPLayers/TRWP_hard_soft/TRWP.cpp:382-419,
 * kernels TRWP_swbp.cu:135-245).  message [n_tables, n_disp(front), n_disp(current)]:
 *   soft[t,c] = sum_f softmax_f(-message[t,:,c])[f] * message[t,f,c];  min_ind[t] = argmin_c soft[t,c]
 *   (highest index among equal minima);  norm[t,c] = soft[t,c] - soft[t,min_ind[t]].
 * The backward call writes dmessage [n_tables,n_disp,n_disp] = d norm / d message applied to
 * dmessage_soft_sum_norm [n_tables,n_disp]. */
int mpl_soft_weighted_message(const float* message, int64_t n_tables, int32_t n_disp,
                              float* message_soft_sum_norm, uint8_t* message_soft_sum_min_ind, void* stream);
int mpl_soft_weighted_message_backward(const float* dmessage_soft_sum_norm, const float* message,
                                       const uint8_t* message_soft_sum_min_ind, int64_t n_tables,
                                       int32_t n_disp, float* dmessage, void* stream);

/* Builders of the layers' inputs.  The reference builds them on the host CPU
 * (MPLayers/aux/aux.cpp, called through MPLayers/aux/auxPy.cpp:9-112) or with chains of torch
 * slicing ops (utils/edge_weights.py); here each is one pass whose output is already in the layout
 * the layers read.  Images are device buffers; reading image files stays with the caller.
 *
 * mpl_stereo_data_cost   computeDSI (aux.cpp:6-91): matching cost of left pixel x against right
 *     pixel x - d for d in [0, n_disp), summed over min(3, channels) colours, either the
 *     Birchfield-Tomasi sampling-insensitive difference (integer half-sample neighbours) or the
 *     absolute difference, optionally squared, truncated at trunc_diffs (per colour when not
 *     squared), and the truncation value where x - d < 0.  left/right: u8 [height,width,channels]
 *     interleaved; data_cost: f32 [height,width,n_disp] = the layers' unary [1,1,H,W,L].  Values
 *     are integers and identical to the reference's.
 * mpl_gradient_cues      computeCues (aux.cpp:93-158): grad_penalty where the squared colour
 *     difference to the right (h_cue) / lower (v_cue) neighbour is below channels*grad_thresh^2,
 *     else 1.  compact = 0: both [height,width]; compact = 1: what the reference returns to Python
 *     (auxPy.cpp:86-99), h_cue [height*(width-1)] row-major, v_cue [(height-1)*width] column-major.
 * mpl_smoothness_context computeSmoothnessContext (aux.cpp:160-214): context [n_disp,n_disp] for
 *     method "L", "Q", "TL", "TQ", "Cauchy" or "Huber" with truncation smoothness_max.
 * mpl_edge_weights       getEdgeShift (utils/edge_weights.py:45-111): for each direction d the weight
 *     of the edge (p - step_d, p) stored at p, 0 where p - step_d is outside; image f32
 *     [batch,channels,height,width]; mode from mpl_edge_mode(name), the reference's edge_mode
 *     strings plus "shifted" (its fall-through branch) and "cue_penalty"
 *     (MPLayers/extra_exp_edge_weights.py:115-121).  Output [n_dir,batch,Cout,height,width] with
 *     Cout = mpl_edge_mode_channels(mode, channels): 1 for the modes that reduce over channels
 *     (superpixel_edge, kernel_cue_real, kernel_cue_binary, threshold, cue_penalty) -- the layers'
 *     edge_weights [D,B,cv=1,H,W] -- else `channels`.  kernel_cue_binary needs a 128-byte workspace. */
int mpl_stereo_data_cost(const uint8_t* left, const uint8_t* right, int32_t height, int32_t width,
                         int32_t channels, int32_t n_disp, int32_t birchfield, int32_t squared_diffs,
                         int32_t trunc_diffs, float* data_cost, void* stream);
int mpl_gradient_cues(const uint8_t* image, int32_t height, int32_t width, int32_t channels,
                      int32_t grad_thresh, int32_t grad_penalty, int32_t compact, float* h_cue, float* v_cue,
                      void* stream);
int mpl_smoothness_context(int32_t n_disp, const char* method, float smoothness_max, float* context,
                           void* stream);
int32_t mpl_edge_mode(const char* name);                       /* -1 for an unknown name */
int32_t mpl_edge_mode_channels(int32_t mode, int32_t channels); /* -1 on bad arguments */
int mpl_edge_weights(int32_t mode, const float* image, int32_t batch, int32_t channels, int32_t height,
                     int32_t width, int32_t n_dir, float sigma, float threshold, float penalty,
                     float* edge_weights, void* workspace, size_t workspace_bytes, void* stream);

/* Message of the last error on the calling thread ("" if none).  Replaces the reference's
 * printf-and-return error reporting (MPLayers/TRWP/TRWP.cpp:269-273,316). */
const char* mpl_last_error(void);

/* Number of CUDA kernels this library has launched in this process so far (all threads). */
int64_t mpl_kernel_launches(void);

/* Library version (major*10000 + minor*100 + patch). */
int32_t mpl_version(void);

/* Chain enumeration used by every kernel (host-side copy, for tests and callers that want to
 * inspect the traversal).  Counterpart of the reference's n_trees / tree_id -> start mapping
 * (MPLayers/common.cpp:78-87, MPLayers/TRWP/TRWP_forward.cu:201-218,310-312), restated as: a
 * chain starts at every pixel whose predecessor lies outside the image.
 * mpl_chain_count: chains per image of direction `dir` (-1 on bad arguments).
 * mpl_chain_geometry: out5 = {h_start, w_start, n_pixels, h_step, w_step} of chain `chain`. */
int32_t mpl_chain_count(int32_t dir, int32_t height, int32_t width);
int32_t mpl_chain_geometry(int32_t dir, int32_t height, int32_t width, int32_t chain, int32_t* out5);

/* Per-launch timing for benchmarks (no counterpart in the reference, which times with
 * time.time() around whole calls, MPLayers/main.py:271-300).  While enabled, every sweep and
 * elementwise kernel launch is bracketed by CUDA events on its stream.  mpl_profile_read waits
 * for the recorded events and returns the summed device time and launch count of one kind:
 * 0 = forward sweep, 1 = backward sweep, 2 = elementwise (aggregation, backward prologue). */
void mpl_profile_enable(int32_t on);
int32_t mpl_profile_read(int32_t kind, double* total_ms, int64_t* launches);
void mpl_profile_reset(void);

#ifdef __cplusplus
}
#endif
#endif /* MPLAYERS_B200_H_ */
