// Training step of the expert-parallel layer: the forward pass of ep_layer.cu in the training
// layout (every local expert's rows start at a multiple of 64 rows of the receive buffer and are
// followed by zero rows, so that the weight-gradient GEMMs reduce over whole 64-row blocks), with
// the activations the backward pass needs kept where they were produced, and the backward pass
// as the same exchange run in reverse:
//
//   forward   router -> permute + dispatch of x rows (region A) -> segment tables, zero padding
//             -> gate/up GEMM (g, u, h stay on the expert's rank) -> down GEMM -> return of the
//             fp32 expert rows -> combine on the token's rank (o rows stay there for the gate
//             gradient); auxiliary-loss statistics from the count table every rank already holds.
//   backward  token's rank: d_o = gate * dOut per slot, d_gate = <dOut, o>  -> dispatch of the d_o
//             rows (region B, same placement as the forward rows) -> expert's rank: dH / dG / dU,
//             dXp and the three weight gradients of its own experts -> return of the fp32 dXp rows
//             -> token's rank: router gradient, dX.
//
// Region A keeps the forward rows until the backward pass has used them.  A peer that runs ahead
// into its next forward step cannot overwrite them: it writes rows only after it has seen the
// counts of ALL ranks for that step, and a rank posts its counts when its own stream gets there,
// i.e. after its weight-gradient GEMMs.  That is why the dXp rows may travel home (and their flag
// be raised) on a side stream while the weight gradients are still being computed.
//
// What the caller still reduces over the ranks (replicated parameters): d_router_w,
// d_router_bias, the shared experts' weight gradients and the auxiliary loss are this rank's
// share; their sum over the ranks is the gradient / the loss.  Routed experts' weight gradients
// are complete on the rank that owns the expert.  Shared experts (replicated) are applied to the
// rank's own tokens without communication, forward and backward, in the gaps the exchange leaves.
//
// The reference engine is single-GPU and has no MoE backward (core/src/CUDA/kernel/
// backward_pass.cu:1701-2005 covers the dense FFN); conventions as in backward.cu.
#include <cstdlib>

#include "router.cuh"

namespace axm {

int validate_ep_layer(const AxmEpLayout* l, const AxmMoeDesc* d);
int launch_expert_ffn(const AxmMoeDesc* d, const void* x_perm, int32_t a_rows, const void* x_alt,
                      int32_t alt_rows, const AxmSegment* segments, int32_t num_segments,
                      const void* w_gate, const void* w_up, const void* w_down,
                      const void* shared_gate, const void* shared_up, const void* shared_down,
                      void* h, void* o, int32_t rows_total, int32_t* status, cudaStream_t st,
                      cudaEvent_t between, const AxmRemoteOut* remote, void* save_g, void* save_u);
int launch_ep_permute_dispatch(const AxmEpLayout* l, uint32_t step, const void* x, const int32_t* topk_idx,
                               const int32_t* block_counts, int32_t* histogram, int32_t* offsets,
                               int32_t* row_src, int32_t* slot_dst, int32_t* done_counter, int T, int k,
                               int hist_accumulate, int32_t* status, cudaStream_t st);
int launch_ep_segments_split(const AxmEpLayout* l, uint32_t step, AxmSegment* segments, AxmSegment* ret_segments,
                             int32_t* rows_received, AxmSegment* seg_halves, int32_t* split_rows,
                             int32_t* status, cudaStream_t st);
int launch_ep_zero_pad(const AxmEpLayout* l, uint32_t step, void* buf, cudaStream_t st);
int launch_expert_ffn_backward(const AxmMoeDesc* desc, const AxmSegment* segments, int32_t num_segments,
                               int32_t rows_total, const void* x_perm, const void* h, const void* g, const void* u,
                               const void* d_o, const void* w_gate, const void* w_up, const void* w_down, void* d_g,
                               void* d_u, void* d_xp, void* d_w_gate, void* d_w_up, void* d_w_down, int32_t* status,
                               void* stream, int phases);
size_t dwr_partial_floats(int D, int E);
int launch_aux_partial(const float* logits, float* partial, int T, int E, cudaStream_t st);
int bwd_source_limits(int E, int router_dtype);
int launch_bwd_prepare(const float* d_out, const float* o, const int32_t* row_src, const float* gate,
                       const int32_t* offsets, void* d_o, float* d_gate, int D, int E, int k, cudaStream_t st);
int launch_bwd_source_tail(const AxmMoeDesc* desc, const AxmMoeTrain* t, const float* logits,
                           const int32_t* topk_idx, const float* d_gate, const float* aux_coef, float* dz,
                           float* bias_partial, float* dwr_partial, const float* d_xp, const int32_t* slot_dst,
                           cudaStream_t st, int S, const float* d_xp_shared, int shared_stride);
int launch_train_shared_rows(const void* x, void* x_perm, AxmSegment* segments, int T, int Tp, int D, int E, int S,
                             int row0, cudaStream_t st);
int launch_bwd_prepare_shared(const float* d_out, void* d_o, int T, int Tp, int D, int S, int row0, cudaStream_t st);
int launch_combine_strided(const AxmMoeDesc* desc, const void* x, const void* o, const void* o_shared,
                           int shared_stride, const int32_t* slot_dst, const float* topk_gate, void* y, void* out,
                           cudaStream_t st);

namespace {

constexpr int kEpTrainAlign = 64;

size_t up256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

struct EpTrainWs {
  int32_t* status;
  int32_t* scratch;  // 2 counters of the exchange kernels (zero between calls)
  int32_t* rows_received;
  float* logits;
  int32_t* topk_idx;
  float* topk_gate;
  int32_t* block_counts;
  int32_t* offsets;
  int32_t* row_src;
  int32_t* slot_dst;
  AxmSegment* segments;      // [G * El] as the exchange kernels write them
  AxmSegment* ret_segments;  // [G * El]
  AxmSegment* expert_segs;   // [El]: one segment per local expert, padded rows
  float* aux_partial;        // [296][E]; the backward pass reuses it for the bias partial sums
  float* aux_coef;           // [E]
  int32_t* counts_global;    // [E]: tokens per expert over all ranks (from the count table)
  float* d_gate;             // [T * k]
  float* dz;                 // [T][E]
  float* dwr_partial;
  void* d_o_local;           // [T * k][D] bf16: gate-scaled upstream rows in local expert order
  void *g, *u, *h;           // [cap][F] bf16, saved by the forward pass
  void *d_g, *d_u;           // [cap][F] bf16
  void* o;                   // [cap][D] fp32: expert rows (forward), dXp rows (backward)
  // shared experts (replicated; they see this rank's tokens only): S runs of Tp rows each, Tp =
  // the tokens padded to a multiple of 64
  AxmSegment* shared_segs;   // [S]
  void* xs;                  // [S * Tp][D] bf16: a copy of the token rows per shared expert
  void *gs, *us, *hs;        // [S * Tp][F] bf16
  void *dgs, *dus;           // [S * Tp][F] bf16
  void* dos;                 // [S * Tp][D] bf16
  void* os;                  // [S * Tp][D] fp32: outputs (forward), dXp rows (backward)
  int shared_rows;           // Tp
  void* router_scratch;
  size_t router_scratch_bytes;
  size_t zero_bytes;
  size_t bytes;
};

EpTrainWs carve(const AxmEpLayout* l, const AxmMoeDesc* d, void* base) {
  EpTrainWs w;
  size_t off = 0;
  auto take = [&](size_t n) {
    void* p = base ? static_cast<char*>(base) + off : nullptr;
    off += up256(n);
    return p;
  };
  const size_t T = d->tokens, D = d->d_model, F = d->d_ff, E = d->num_experts, k = d->top_k, S = d->num_shared;
  const size_t G = l->world, El = E / G, cap = (size_t)l->cap;
  const size_t Tp = (T + kEpTrainAlign - 1) / kEpTrainAlign * kEpTrainAlign;
  w.status = static_cast<int32_t*>(take(4));
  w.scratch = static_cast<int32_t*>(take(8));
  w.zero_bytes = off;
  w.rows_received = static_cast<int32_t*>(take(4));
  w.logits = static_cast<float*>(take(4 * T * E));
  w.topk_idx = static_cast<int32_t*>(take(4 * T * k));
  w.topk_gate = static_cast<float*>(take(4 * T * k));
  w.block_counts = static_cast<int32_t*>(take(4 * (size_t)AXM_ROUTE_BLOCKS * E));
  w.offsets = static_cast<int32_t*>(take(4 * (E + 1)));
  w.row_src = static_cast<int32_t*>(take(4 * T * k));
  w.slot_dst = static_cast<int32_t*>(take(4 * T * k));
  w.segments = static_cast<AxmSegment*>(take(sizeof(AxmSegment) * G * El));
  w.ret_segments = static_cast<AxmSegment*>(take(sizeof(AxmSegment) * G * El));
  w.expert_segs = static_cast<AxmSegment*>(take(sizeof(AxmSegment) * El));
  w.aux_partial = static_cast<float*>(take(4 * (size_t)AXM_ROUTE_BLOCKS * E));
  w.aux_coef = static_cast<float*>(take(4 * E));
  w.counts_global = static_cast<int32_t*>(take(4 * E));
  w.d_gate = static_cast<float*>(take(4 * T * k));
  w.dz = static_cast<float*>(take(4 * T * E));
  w.dwr_partial = static_cast<float*>(take(4 * dwr_partial_floats((int)D, (int)E)));
  w.d_o_local = take(2 * T * k * D);
  w.g = take(2 * cap * F);
  w.u = take(2 * cap * F);
  w.h = take(2 * cap * F);
  w.d_g = take(2 * cap * F);
  w.d_u = take(2 * cap * F);
  w.o = take(4 * cap * D);
  w.shared_rows = (int)Tp;
  w.shared_segs = static_cast<AxmSegment*>(take(sizeof(AxmSegment) * (S ? S : 1)));
  w.xs = take(2 * S * Tp * D);
  w.gs = take(2 * S * Tp * F);
  w.us = take(2 * S * Tp * F);
  w.hs = take(2 * S * Tp * F);
  w.dgs = take(2 * S * Tp * F);
  w.dus = take(2 * S * Tp * F);
  w.dos = take(2 * S * Tp * D);
  w.os = take(4 * S * Tp * D);
  w.router_scratch_bytes = 0;
  axm_moe_router_scratch_bytes(d, &w.router_scratch_bytes);
  w.router_scratch = take(w.router_scratch_bytes);
  w.bytes = off;
  return w;
}

int validate_ep_train(const AxmEpLayout* l, const AxmMoeDesc* d, int32_t tokens_global) {
  if (int rc = validate_ep_layer(l, d)) return rc;
  if (d->tokens <= 0) return fail(AXM_ERR_ARGUMENT, "tokens %d must be positive", d->tokens);
  if (tokens_global < d->tokens)
    return fail(AXM_ERR_ARGUMENT, "tokens_global %d is smaller than this rank's %d tokens", tokens_global, d->tokens);
  if (l->row_align != kEpTrainAlign)
    return fail(AXM_ERR_ARGUMENT, "the training step needs row_align %d in the exchange layout, got %d", kEpTrainAlign,
                l->row_align);
  const long long need = (long long)d->tokens * d->top_k * l->world +
                         (long long)(kEpTrainAlign - 1) * (d->num_experts / l->world);
  if (l->cap < need)
    return fail(AXM_ERR_ARGUMENT, "receive buffer of %d rows; %lld needed with padding", l->cap, need);
  return AXM_OK;
}

// counts[e] = tokens of all ranks routed to expert e (every rank's counts were posted into this
// rank's table by the dispatch).  Runs before this rank's return flag lets a peer move on to a
// step that rewrites the table.
// In the same launch: expert_segs[j] = the merged segment of local expert j (entry j * G of the
// exchange table).  One block of 256 threads (E <= 256, at most 64 experts per rank).
__global__ void train_tables_kernel(const int32_t* __restrict__ table, int G, int E, int32_t* __restrict__ counts,
                                    const AxmSegment* __restrict__ segments, AxmSegment* __restrict__ expert_segs,
                                    int El) {
  const int e = threadIdx.x;
  if (e < El) expert_segs[e] = segments[e * G];
  if (e >= E) return;
  int cnt = 0;
  for (int s = 0; s < G; ++s) cnt += __ldcg(table + s * E + e);
  counts[e] = cnt;
}

// One block: f_e from the counts of all ranks, the constant alpha * E * f_e / T that the router
// backward adds to dp[t, e], and this rank's share of the loss alpha * E * sum_e f_e * P_e (P_e =
// mean over ALL tokens; the share sums this rank's probabilities only).  T is the token count
// over all ranks.
__global__ void aux_final_ep_kernel(const float* __restrict__ partial, const int32_t* __restrict__ counts,
                                    float* __restrict__ aux_coef, float* __restrict__ aux_loss, int T, int E, int k,
                                    float alpha) {
  __shared__ float term[256];
  const int e = threadIdx.x;
  float v = 0.0f;
  if (e < E) {
    float P = 0.0f;
    for (int b = 0; b < AXM_ROUTE_BLOCKS; ++b) P += partial[(size_t)b * E + e];
    P /= (float)T;
    const float f = (float)counts[e] / ((float)T * (float)k);
    v = f * P;
    aux_coef[e] = alpha * (float)E * f / (float)T;
  }
  term[threadIdx.x] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float acc = 0.0f;
    for (int i = 0; i < E; ++i) acc += term[i];
    if (aux_loss != nullptr) *aux_loss = alpha * (float)E * acc;
  }
}

// High-priority side stream for the return of the dXp rows under the weight-gradient GEMMs,
// created once per device and thread.
struct TrainPipe {
  cudaStream_t side = nullptr;
  cudaEvent_t dx_done = nullptr, side_done = nullptr;
  bool ok = false;
};
TrainPipe* train_pipe() {
  static thread_local TrainPipe pipes[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  TrainPipe& p = pipes[dev];
  if (!p.ok) {
    int prio_lo = 0, prio_hi = 0;
    if (cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi) != cudaSuccess) return nullptr;
    if (cudaStreamCreateWithPriority(&p.side, cudaStreamNonBlocking, prio_hi) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&p.dx_done, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&p.side_done, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    p.ok = true;
  }
  return &p;
}

struct Call {
  EpTrainWs w;
  AxmEpLayout l;       // this call's row counts
  AxmMoeDesc d_route;  // local tokens, all experts
  AxmMoeDesc d_ffn;    // this rank's experts
  int El;
};

int prepare(const AxmEpLayout* layout, const AxmMoeDesc* desc, const AxmMoeTrain* t, int32_t tokens_global,
            void* workspace, size_t workspace_bytes, uint32_t step, Call* c) {
  if (int rc = validate_ep_train(layout, desc, tokens_global)) return rc;
  if (t == nullptr) return fail(AXM_ERR_ARGUMENT, "tensors is null");
  if (layout->peers == nullptr || layout->local_region == nullptr)
    return fail(AXM_ERR_ARGUMENT, "the peer table or the local region is null");
  if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(AXM_ERR_WORKSPACE, "workspace is null or not 256-byte aligned");
  c->w = carve(layout, desc, workspace);
  if (workspace_bytes < c->w.bytes)
    return fail(AXM_ERR_WORKSPACE, "workspace has %zu bytes, %zu needed", workspace_bytes, c->w.bytes);
  if (step == 0) return fail(AXM_ERR_ARGUMENT, "step starts at 1 and grows by one per call");
  c->El = desc->num_experts / layout->world;
  c->l = *layout;
  c->l.return_rows = layout->return_rows > layout->slots ? layout->return_rows : layout->slots;
  c->l.slots = desc->tokens * desc->top_k;
  c->l.tokens_local = desc->tokens;
  c->l.num_shared = 0;  // the exchange carries routed rows only; shared experts stay on their rank
  c->d_route = *desc;
  c->d_route.num_shared = 0;
  // the saved h of the training layout is one bf16 term; the histogram is this call's
  c->d_route.flags &= ~(AXM_FLAG_HIST_ACCUMULATE | AXM_FLAG_H_EXACT);
  c->d_ffn = c->d_route;
  c->d_ffn.num_experts = c->El;
  c->d_ffn.top_k = desc->top_k < c->El ? desc->top_k : c->El;
  return AXM_OK;
}

}  // namespace
}  // namespace axm

using namespace axm;

extern "C" int axm_moe_ep_train_workspace_bytes(const AxmEpLayout* layout, const AxmMoeDesc* desc, size_t* bytes,
                                                size_t* zero_bytes) {
  if (layout == nullptr || desc == nullptr) return fail(AXM_ERR_ARGUMENT, "layout or desc is null");
  if (int rc = validate_ep_train(layout, desc, desc->tokens)) return rc;
  if (bytes == nullptr) return fail(AXM_ERR_ARGUMENT, "bytes is null");
  EpTrainWs w = carve(layout, desc, nullptr);
  *bytes = w.bytes;
  if (zero_bytes) *zero_bytes = w.zero_bytes;
  return AXM_OK;
}

extern "C" int axm_moe_ep_train_status_word(const AxmEpLayout* layout, const AxmMoeDesc* desc, void* workspace,
                                            int32_t** status, int32_t** rows_received) {
  if (layout == nullptr || desc == nullptr) return fail(AXM_ERR_ARGUMENT, "layout or desc is null");
  if (int rc = validate_ep_train(layout, desc, desc->tokens)) return rc;
  if (!workspace) return fail(AXM_ERR_ARGUMENT, "axm_moe_ep_train_status_word: null pointer");
  EpTrainWs w = carve(layout, desc, workspace);
  if (status) *status = w.status;
  if (rows_received) *rows_received = w.rows_received;
  return AXM_OK;
}

extern "C" int axm_moe_ep_forward_train(const AxmEpLayout* layout, const AxmMoeDesc* desc, const AxmMoeTrain* t,
                                        int32_t tokens_global, void* workspace, size_t workspace_bytes,
                                        uint32_t step, void* stream) {
  if (layout == nullptr || desc == nullptr) return fail(AXM_ERR_ARGUMENT, "layout or desc is null");
  Call c;
  if (int rc = prepare(layout, desc, t, tokens_global, workspace, workspace_bytes, step, &c)) return rc;
  if (!t->x || !t->router_w || !t->w_gate || !t->w_up || !t->w_down || !t->out)
    return fail(AXM_ERR_ARGUMENT, "axm_moe_ep_forward_train: x, router_w, w_gate, w_up, w_down, out are required");
  const int S = desc->num_shared;
  if (S > 0 && (!t->shared_gate || !t->shared_up || !t->shared_down))
    return fail(AXM_ERR_ARGUMENT, "num_shared > 0 needs shared_gate, shared_up and shared_down");
  if (int rc = require_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  EpTrainWs& w = c.w;
  const int T = desc->tokens, E = desc->num_experts, k = desc->top_k, G = layout->world;
  char* region = static_cast<char*>(layout->local_region);
  void* recv = region + layout->off_recv;
  const void* o_back = region + layout->off_oback;
  const int32_t* table = reinterpret_cast<const int32_t*>(region + layout->off_counts);

  int rc = launch_router_auto(&c.d_route, t->x, t->router_w, t->router_bias, w.logits, w.topk_idx, w.topk_gate,
                              w.block_counts, w.router_scratch, w.router_scratch_bytes, nullptr, stream, nullptr);
  if (rc) return rc;
  if ((rc = launch_ep_permute_dispatch(&c.l, step, t->x, w.topk_idx, w.block_counts, t->histogram, w.offsets,
                                       w.row_src, w.slot_dst, w.scratch, T, k, 0, w.status, st)))
    return rc;
  AxmMoeDesc d_shared = c.d_route;
  d_shared.num_experts = S > 0 ? S : 1;
  d_shared.top_k = 1;
  if (S > 0) {
    // the shared experts need this rank's tokens only: their GEMMs fill the time in which the
    // routed rows of the peers arrive
    if ((rc = launch_train_shared_rows(t->x, w.xs, w.shared_segs, T, w.shared_rows, desc->d_model, 0, S, 0, st)))
      return rc;
    if ((rc = launch_expert_ffn(&d_shared, w.xs, S * w.shared_rows, nullptr, 0, w.shared_segs, S, t->shared_gate,
                                t->shared_up, t->shared_down, nullptr, nullptr, nullptr, w.hs, w.os,
                                S * w.shared_rows, w.status, st, nullptr, nullptr, w.gs, w.us)))
      return rc;
  }
  if ((rc = launch_ep_segments_split(&c.l, step, w.segments, w.ret_segments, w.rows_received, nullptr, nullptr,
                                     w.status, st)))
    return rc;
  train_tables_kernel<<<1, 256, 0, st>>>(table, G, E, w.counts_global, w.segments, w.expert_segs, c.El);
  if ((rc = launch_ep_zero_pad(&c.l, step, recv, st))) return rc;
  if ((rc = launch_expert_ffn(&c.d_ffn, recv, c.l.cap, nullptr, 0, w.expert_segs, c.El, t->w_gate, t->w_up,
                              t->w_down, nullptr, nullptr, nullptr, w.h, w.o, c.l.cap, w.status, st, nullptr,
                              nullptr, w.g, w.u)))
    return rc;
  if ((rc = axm_ep_return(&c.l, step, w.ret_segments, w.o, w.scratch, w.status, stream))) return rc;
  // the auxiliary-loss statistics fill the time in which the peers' rows come back
  if ((rc = launch_aux_partial(w.logits, w.aux_partial, T, E, st))) return rc;
  aux_final_ep_kernel<<<1, 256, 0, st>>>(w.aux_partial, w.counts_global, w.aux_coef, t->aux_loss, tokens_global, E, k,
                                         t->aux_alpha);
  if ((rc = axm_ep_wait_return(&c.l, step, w.status, stream))) return rc;
  AxmMoeDesc d_comb = c.d_route;
  d_comb.num_shared = S;
  if ((rc = launch_combine_strided(&d_comb, t->x, o_back, S > 0 ? w.os : nullptr, w.shared_rows, w.slot_dst,
                                   w.topk_gate, nullptr, t->out, st)))
    return rc;
  return check_launch("ep_forward_train");
}

extern "C" int axm_moe_ep_backward(const AxmEpLayout* fwd_layout, const AxmEpLayout* bwd_layout,
                                   const AxmMoeDesc* desc, const AxmMoeTrain* t, int32_t tokens_global,
                                   void* workspace, size_t workspace_bytes, uint32_t step, void* stream) {
  if (fwd_layout == nullptr || bwd_layout == nullptr || desc == nullptr)
    return fail(AXM_ERR_ARGUMENT, "layout or desc is null");
  Call c;
  if (int rc = prepare(fwd_layout, desc, t, tokens_global, workspace, workspace_bytes, step, &c)) return rc;
  if (int rc = validate_ep_train(bwd_layout, desc, tokens_global)) return rc;
  if (bwd_layout->peers == nullptr || bwd_layout->local_region == nullptr)
    return fail(AXM_ERR_ARGUMENT, "the backward region's peer table or local region is null");
  if (bwd_layout->local_region == fwd_layout->local_region)
    return fail(AXM_ERR_ARGUMENT, "the backward pass needs an exchange region of its own");
  if (bwd_layout->cap != fwd_layout->cap || bwd_layout->world != fwd_layout->world ||
      bwd_layout->rank != fwd_layout->rank)
    return fail(AXM_ERR_ARGUMENT, "forward and backward regions differ in cap, world or rank");
  if (!t->x || !t->router_w || !t->w_gate || !t->w_up || !t->w_down || !t->d_out || !t->d_x)
    return fail(AXM_ERR_ARGUMENT, "axm_moe_ep_backward: x, weights, d_out and d_x are required");
  const bool wgrad = t->d_w_gate || t->d_w_up || t->d_w_down;
  if (wgrad && !(t->d_w_gate && t->d_w_up && t->d_w_down))
    return fail(AXM_ERR_ARGUMENT, "weight gradients: give all three or none");
  const int S = desc->num_shared;
  if (S > 0) {
    if (!t->shared_gate || !t->shared_up || !t->shared_down)
      return fail(AXM_ERR_ARGUMENT, "num_shared > 0 needs shared_gate, shared_up and shared_down");
    const bool shared_all = t->d_shared_gate && t->d_shared_up && t->d_shared_down;
    const bool shared_any = t->d_shared_gate || t->d_shared_up || t->d_shared_down;
    if (wgrad != shared_any || shared_any != shared_all)
      return fail(AXM_ERR_ARGUMENT, "shared experts' weight gradients: all three exactly when the routed experts' are given");
  }
  if (int rc = require_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  EpTrainWs& w = c.w;
  const int D = desc->d_model, E = desc->num_experts, k = desc->top_k;
  AxmEpLayout lb = *bwd_layout;
  lb.return_rows = bwd_layout->return_rows > bwd_layout->slots ? bwd_layout->return_rows : bwd_layout->slots;
  lb.slots = c.l.slots;
  lb.tokens_local = c.l.tokens_local;
  lb.num_shared = 0;
  const void* x_recv = static_cast<const char*>(fwd_layout->local_region) + fwd_layout->off_recv;
  const float* o_back = reinterpret_cast<const float*>(static_cast<const char*>(fwd_layout->local_region) +
                                                       fwd_layout->off_oback);
  void* do_recv = static_cast<char*>(bwd_layout->local_region) + bwd_layout->off_recv;
  const float* dxp_back = reinterpret_cast<const float*>(static_cast<const char*>(bwd_layout->local_region) +
                                                         bwd_layout->off_oback);

  int rc;
  if ((rc = bwd_source_limits(E, desc->router_dtype))) return rc;
  // where the tokens live: offsets[E] = T * k rows in local expert order, no padding rows
  if ((rc = launch_bwd_prepare(t->d_out, o_back, w.row_src, w.topk_gate, w.offsets, w.d_o_local, w.d_gate, D, E, k,
                               st)))
    return rc;
  if ((rc = axm_ep_dispatch(&lb, step, w.offsets, w.d_o_local, w.scratch, w.status, stream))) return rc;
  if (S > 0) {
    // shared experts: local rows only (their weight gradients are this rank's share, like the
    // router's); computed while the gradient rows of the peers arrive
    AxmMoeDesc d_shared = c.d_route;
    d_shared.num_experts = S;
    d_shared.top_k = 1;
    if ((rc = launch_bwd_prepare_shared(t->d_out, w.dos, desc->tokens, w.shared_rows, D, S, 0, st))) return rc;
    if ((rc = launch_expert_ffn_backward(&d_shared, w.shared_segs, S, S * w.shared_rows, w.xs, w.hs, w.gs, w.us, w.dos,
                                         t->shared_gate, t->shared_up, t->shared_down, w.dgs, w.dus, w.os,
                                         t->d_shared_gate, t->d_shared_up, t->d_shared_down, w.status, stream, 3)))
      return rc;
  }
  // where the experts live: the same tables as in the forward pass (the counts are the same)
  if ((rc = launch_ep_segments_split(&lb, step, w.segments, w.ret_segments, w.rows_received, nullptr, nullptr,
                                     w.status, st)))
    return rc;
  // w.expert_segs still holds the forward pass's one-segment-per-expert table
  if ((rc = launch_ep_zero_pad(&lb, step, do_recv, st))) return rc;
  // AXM_EP_TRAIN_OVERLAP=0 keeps everything on the caller's stream (return after the weight gradients)
  static const bool overlap = [] {
    const char* e = getenv("AXM_EP_TRAIN_OVERLAP");
    return !(e != nullptr && e[0] == '0');
  }();
  TrainPipe* pipe = (overlap && wgrad) ? train_pipe() : nullptr;
  if ((rc = launch_expert_ffn_backward(&c.d_ffn, w.expert_segs, c.El, lb.cap, x_recv, w.h, w.g, w.u, do_recv,
                                       t->w_gate, t->w_up, t->w_down, w.d_g, w.d_u, w.o, t->d_w_gate, t->d_w_up,
                                       t->d_w_down, w.status, stream, pipe ? 1 : 3)))
    return rc;
  if (pipe != nullptr) {
    // The dXp rows go home on a side stream while the weight gradients are computed.  Raising the
    // return flag before the weight gradients have read the forward rows is safe: a source writes
    // new rows into this rank's receive buffer only after it has seen the counts of ALL ranks for
    // the next step, and this rank posts its own only when its stream has reached that step.
    AXM_CUDA(cudaEventRecord(pipe->dx_done, st));
    AXM_CUDA(cudaStreamWaitEvent(pipe->side, pipe->dx_done, 0));
    if ((rc = axm_ep_return(&lb, step, w.ret_segments, w.o, w.scratch, w.status, pipe->side))) return rc;
    AXM_CUDA(cudaEventRecord(pipe->side_done, pipe->side));
    if ((rc = launch_expert_ffn_backward(&c.d_ffn, w.expert_segs, c.El, lb.cap, x_recv, w.h, w.g, w.u, do_recv,
                                         t->w_gate, t->w_up, t->w_down, w.d_g, w.d_u, w.o, t->d_w_gate, t->d_w_up,
                                         t->d_w_down, w.status, stream, 2)))
      return rc;
    AXM_CUDA(cudaStreamWaitEvent(st, pipe->side_done, 0));
  } else {
    if ((rc = axm_ep_return(&lb, step, w.ret_segments, w.o, w.scratch, w.status, stream))) return rc;
  }
  if ((rc = axm_ep_wait_return(&lb, step, w.status, stream))) return rc;
  return launch_bwd_source_tail(&c.d_route, t, w.logits, w.topk_idx, w.d_gate, w.aux_coef, w.dz, w.aux_partial,
                                w.dwr_partial, dxp_back, w.slot_dst, st, S, static_cast<const float*>(w.os),
                                w.shared_rows);
}
