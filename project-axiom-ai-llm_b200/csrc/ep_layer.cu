// The expert-parallel layer behind the C ABI: one call per rank and layer enqueues
//   router -> permute + dispatch (rows stored straight into the owners' receive buffers)
//   -> segment tables -> gate/up GEMM -> down GEMM -> return of the expert rows to their
//   source ranks -> wait for the rows coming back -> combine.
// (Optionally the down GEMM runs in two halves with the first half's rows travelling back
// while the second half is computed; see split_return below.)
// The reference engine is single-GPU (no communication library anywhere in core/src); this is
// the sharded form of its forward_mixture_experts (core/src/CUDA/kernel/moe_router.cu:205-320)
// with the host logic in C++: validation before any launch, caller-provided workspace, all
// work enqueued, no host synchronisation.  The host program only allocates the exchange
// regions in memory its peers can address and hands over the table of their addresses.
#include <cstdlib>
#include <cstring>

#include "router.cuh"

namespace axm {

int launch_expert_ffn_phases(const AxmMoeDesc* d, const void* x_perm, int32_t a_rows, const void* x_alt,
                             int32_t alt_rows, const AxmSegment* segments, int32_t num_segments,
                             const void* w_gate, const void* w_up, const void* w_down,
                             const void* shared_gate, const void* shared_up, const void* shared_down,
                             void* h, void* o, int32_t rows_total, int32_t* status, cudaStream_t st,
                             cudaEvent_t between, const AxmRemoteOut* remote, void* save_g, void* save_u,
                             int phases);
int launch_ep_permute_dispatch(const AxmEpLayout* l, uint32_t step, const void* x, const int32_t* topk_idx,
                               const int32_t* block_counts, int32_t* histogram, int32_t* offsets,
                               int32_t* row_src, int32_t* slot_dst, int32_t* done_counter, int T, int k,
                               int hist_accumulate, int32_t* status, cudaStream_t st);
int launch_ep_segments_split(const AxmEpLayout* l, uint32_t step, AxmSegment* segments, AxmSegment* ret_segments,
                             int32_t* rows_received, AxmSegment* seg_halves, int32_t* split_rows,
                             int32_t* status, cudaStream_t st);
int launch_ep_return_half(const AxmEpLayout* l, uint32_t step, const AxmSegment* ret_segments, const void* o,
                          int32_t* done_counter, const int32_t* split_rows, int half, int signal,
                          int32_t* status, cudaStream_t st);

// Arguments of one expert-parallel layer call against the exchange layout (also used by ep_train.cu).
int validate_ep_layer(const AxmEpLayout* l, const AxmMoeDesc* d) {
  if (l == nullptr || d == nullptr) return fail(AXM_ERR_ARGUMENT, "layout or desc is null");
  if (l->world <= 0 || l->world > 64 || l->rank < 0 || l->rank >= l->world)
    return fail(AXM_ERR_ARGUMENT, "rank %d / world %d out of range", l->rank, l->world);
  if (d->tokens < 0) return fail(AXM_ERR_ARGUMENT, "tokens %d negative", d->tokens);
  if (d->d_model <= 0 || d->d_ff <= 0 || d->d_model % 8 || d->d_ff % 8)
    return fail(AXM_ERR_ARGUMENT, "d_model %d and d_ff %d must be positive multiples of 8", d->d_model, d->d_ff);
  if (d->num_experts <= 0 || d->num_experts > 256 || d->num_experts % l->world != 0)
    return fail(AXM_ERR_ARGUMENT, "num_experts %d must be in 1..256 and a multiple of world %d", d->num_experts,
                l->world);
  if (d->num_experts / l->world > 64) return fail(AXM_ERR_ARGUMENT, "more than 64 experts per rank");
  if (d->top_k <= 0 || d->top_k > 8 || d->top_k > d->num_experts)
    return fail(AXM_ERR_ARGUMENT, "top_k %d not in 1..min(num_experts, 8)", d->top_k);
  if (d->num_shared < 0 || d->num_shared > 8) return fail(AXM_ERR_ARGUMENT, "num_shared %d not in 0..8", d->num_shared);
  if (d->router_dtype != AXM_ROUTER_BF16 && d->router_dtype != AXM_ROUTER_FP32)
    return fail(AXM_ERR_ARGUMENT, "router_dtype %d unknown", d->router_dtype);
  if (l->num_experts != d->num_experts || l->d_model != d->d_model)
    return fail(AXM_ERR_ARGUMENT, "layout was sized for %d experts / d_model %d, desc says %d / %d", l->num_experts,
                l->d_model, d->num_experts, d->d_model);
  if ((long long)d->tokens * d->top_k > l->slots)
    return fail(AXM_ERR_ARGUMENT, "%d tokens x top-%d exceed the %d slots the exchange region was sized for",
                d->tokens, d->top_k, l->slots);
  if ((long long)l->cap + (long long)d->num_shared * d->tokens > 0x7fffffffLL)
    return fail(AXM_ERR_ARGUMENT, "row count overflows int32");
  return AXM_OK;
}

namespace {

size_t up256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

struct EpWs {
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
  AxmSegment* segments;      // [G * El + S]
  AxmSegment* ret_segments;  // [G * El]
  AxmSegment* seg_halves;    // [2 * El + S]
  int32_t* split_rows;       // [El]
  void* x_perm;              // only the two-kernel dispatch uses it
  void* h;
  void* o;
  void* router_scratch;
  size_t router_scratch_bytes;
  size_t zero_bytes;  // leading bytes that must be zero before the first call
  size_t bytes;
};

EpWs carve_ep(const AxmEpLayout* l, const AxmMoeDesc* d, void* base) {
  EpWs w;
  size_t off = 0;
  auto take = [&](size_t n) {
    void* p = base ? static_cast<char*>(base) + off : nullptr;
    off += up256(n);
    return p;
  };
  const size_t T = d->tokens, D = d->d_model, F = d->d_ff, E = d->num_experts, k = d->top_k, S = d->num_shared;
  const size_t G = l->world, El = E / G;
  const size_t rows_total = (size_t)l->cap + S * T;
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
  w.segments = static_cast<AxmSegment*>(take(sizeof(AxmSegment) * (G * El + S)));
  w.ret_segments = static_cast<AxmSegment*>(take(sizeof(AxmSegment) * G * El));
  w.seg_halves = static_cast<AxmSegment*>(take(sizeof(AxmSegment) * (2 * El + S)));
  w.split_rows = static_cast<int32_t*>(take(4 * El));
  w.x_perm = take(2 * T * k * D);
  w.h = take(((d->flags & AXM_FLAG_H_EXACT) ? 4 : 2) * rows_total * F);
  w.o = take(4 * rows_total * D);
  w.router_scratch_bytes = 0;
  axm_moe_router_scratch_bytes(d, &w.router_scratch_bytes);
  w.router_scratch = take(w.router_scratch_bytes);
  w.bytes = off;
  return w;
}

int env_flag(const char* name, int dflt) {
  const char* e = getenv(name);
  return e == nullptr ? dflt : (e[0] != '0');
}

// Side stream and events for the overlapped return, created once per device and thread.
struct EpPipe {
  cudaStream_t side = nullptr, in = nullptr, out = nullptr;
  cudaEvent_t half_done = nullptr, side_done = nullptr, start = nullptr;
  cudaEvent_t arrived[8] = {}, done[8] = {};
  bool ok = false;
};
EpPipe* ep_pipe() {
  static thread_local EpPipe pipes[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  EpPipe& p = pipes[dev];
  if (!p.ok) {
    // the side stream carries small copy kernels that must get onto the SMs beside a persistent
    // GEMM that becomes runnable at the same moment: highest priority
    int prio_lo = 0, prio_hi = 0;
    if (cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi) != cudaSuccess) return nullptr;
    if (cudaStreamCreateWithPriority(&p.side, cudaStreamNonBlocking, prio_hi) != cudaSuccess) return nullptr;
    if (cudaStreamCreateWithFlags(&p.in, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaStreamCreateWithFlags(&p.out, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    cudaEvent_t* evs[] = {&p.half_done, &p.side_done, &p.start};
    for (cudaEvent_t* e : evs)
      if (cudaEventCreateWithFlags(e, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    for (int i = 0; i < 8; ++i) {
      if (cudaEventCreateWithFlags(&p.arrived[i], cudaEventDisableTiming) != cudaSuccess) return nullptr;
      if (cudaEventCreateWithFlags(&p.done[i], cudaEventDisableTiming) != cudaSuccess) return nullptr;
    }
    p.ok = true;
  }
  return &p;
}

// ev: optional 10 timing events: 0..7 recorded on the caller's stream between the phases
// (0 = start ... 7 = end), 8 and 9 on the side stream around the first half's return copy
int ep_forward_impl(const AxmEpLayout* layout, const AxmMoeDesc* desc, const AxmEpTensors* t, void* workspace,
                    size_t workspace_bytes, uint32_t step, void* stream, cudaEvent_t* ev) {
  if (int rc = validate_ep_layer(layout, desc)) return rc;
  if (t == nullptr) return fail(AXM_ERR_ARGUMENT, "tensors is null");
  if (!t->x || !t->router_w || !t->w_gate || !t->w_up || !t->w_down || !t->out)
    return fail(AXM_ERR_ARGUMENT, "x, router_w, w_gate, w_up, w_down and out are required");
  if (desc->num_shared > 0 && (!t->shared_gate || !t->shared_up || !t->shared_down))
    return fail(AXM_ERR_ARGUMENT, "num_shared > 0 needs shared_gate, shared_up and shared_down");
  if (layout->peers == nullptr) return fail(AXM_ERR_ARGUMENT, "the peer table is null");
  if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(AXM_ERR_WORKSPACE, "workspace is null or not 256-byte aligned");
  EpWs w = carve_ep(layout, desc, workspace);
  if (workspace_bytes < w.bytes)
    return fail(AXM_ERR_WORKSPACE, "workspace has %zu bytes, %zu needed", workspace_bytes, w.bytes);
  if (step == 0) return fail(AXM_ERR_ARGUMENT, "step starts at 1 and grows by one per call");
  if (int rc = require_device()) return rc;

  static const int fused_dispatch = env_flag("AXM_EP_FUSED_DISPATCH", 1);
  // Off by default.  Measured on 8 GPUs (T 8192, D 4096, E 8, F 14336): the first half's copy
  // does run under the second half's GEMM (98 - 135 us after the down projection starts), but two
  // launches of 64 tile pairs on 74 CTA pairs take 205 us where one launch of 128 takes 180, and
  // the ranks drift further apart: 0.774 ms per step against 0.690.  AXM_EP_SPLIT_RETURN=1 enables it.
  static const int split_return = env_flag("AXM_EP_SPLIT_RETURN", 0);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int T = desc->tokens, D = desc->d_model, E = desc->num_experts, k = desc->top_k, S = desc->num_shared;
  const int G = layout->world, El = E / G;
  AxmEpLayout l = *layout;  // this call's row counts (a chunk may hold fewer tokens than the region was sized for)
  l.return_rows = layout->return_rows > layout->slots ? layout->return_rows : layout->slots;
  l.slots = T * k;
  l.tokens_local = T;
  l.num_shared = S;
  EpPipe* pipe = split_return ? ep_pipe() : nullptr;

  float* logits = t->logits ? t->logits : w.logits;
  int32_t* idx = t->topk_idx ? t->topk_idx : w.topk_idx;
  float* gate = t->topk_gate ? t->topk_gate : w.topk_gate;
  AxmMoeDesc d_route = *desc;
  d_route.num_shared = 0;
  AxmMoeDesc d_ffn = *desc;
  d_ffn.num_experts = El;
  d_ffn.top_k = k < El ? k : El;
  const int rows_total = l.cap + S * T;
  const int n_seg = G * El + S;
  auto mark = [&](int i) { if (ev) cudaEventRecord(ev[i], st); };

  mark(0);
  int rc = launch_router_auto(&d_route, t->x, t->router_w, t->router_bias, logits, idx, gate, w.block_counts,
                              w.router_scratch, w.router_scratch_bytes, nullptr, stream, nullptr);
  if (rc) return rc;
  mark(1);
  if (fused_dispatch) {
    rc = launch_ep_permute_dispatch(&l, step, t->x, idx, w.block_counts, t->histogram, w.offsets, w.row_src,
                                    w.slot_dst, w.scratch, T, k, (desc->flags & AXM_FLAG_HIST_ACCUMULATE) ? 1 : 0,
                                    w.status, st);
    if (rc) return rc;
  } else {
    if ((rc = axm_moe_permute(&d_route, t->x, idx, w.block_counts, t->histogram, w.offsets, w.row_src, w.slot_dst,
                              w.x_perm, stream)))
      return rc;
    if ((rc = axm_ep_dispatch(&l, step, w.offsets, w.x_perm, w.scratch, w.status, stream))) return rc;
  }
  mark(2);
  if ((rc = launch_ep_segments_split(&l, step, w.segments, w.ret_segments, w.rows_received, w.seg_halves,
                                     w.split_rows, w.status, st)))
    return rc;
  mark(3);
  const void* recv = static_cast<const char*>(layout->local_region) + layout->off_recv;
  const void* o_back = static_cast<const char*>(layout->local_region) + layout->off_oback;
  auto ffn = [&](const AxmSegment* segs, int n, int phases) {
    return launch_expert_ffn_phases(&d_ffn, recv, l.cap, t->x, T, segs, n, t->w_gate, t->w_up, t->w_down,
                                    t->shared_gate, t->shared_up, t->shared_down, w.h, w.o, rows_total, w.status,
                                    st, nullptr, nullptr, nullptr, nullptr, phases);
  };
  if ((rc = ffn(w.segments, n_seg, 1))) return rc;
  mark(4);
  if (pipe != nullptr) {
    // first halves: down projection, then their rows go home on the side stream while the
    // second halves (and the shared experts) are projected
    if ((rc = ffn(w.seg_halves, El, 2))) return rc;
    AXM_CUDA(cudaEventRecord(pipe->half_done, st));
    AXM_CUDA(cudaStreamWaitEvent(pipe->side, pipe->half_done, 0));
    if (ev) cudaEventRecord(ev[8], pipe->side);
    if ((rc = launch_ep_return_half(&l, step, w.ret_segments, w.o, w.scratch + 1, w.split_rows, 0, 0, w.status,
                                    pipe->side)))
      return rc;
    if (ev) cudaEventRecord(ev[9], pipe->side);
    AXM_CUDA(cudaEventRecord(pipe->side_done, pipe->side));
    if ((rc = ffn(w.seg_halves + El, El + S, 2))) return rc;
    mark(5);
    AXM_CUDA(cudaStreamWaitEvent(st, pipe->side_done, 0));
    if ((rc = launch_ep_return_half(&l, step, w.ret_segments, w.o, w.scratch + 1, w.split_rows, 1, 1, w.status, st)))
      return rc;
  } else {
    if ((rc = ffn(w.segments, n_seg, 2))) return rc;
    mark(5);
    if ((rc = axm_ep_return(&l, step, w.ret_segments, w.o, w.scratch, w.status, stream))) return rc;
  }
  mark(6);
  if ((rc = axm_ep_wait_return(&l, step, w.status, stream))) return rc;
  AxmMoeDesc d_comb = *desc;
  const float* o_shared = S > 0 ? static_cast<const float*>(w.o) + (size_t)l.cap * D : nullptr;
  rc = axm_moe_combine(&d_comb, t->x, o_back, o_shared, w.slot_dst, gate, t->y, t->out, stream);
  mark(7);
  return rc;
}

}  // namespace
}  // namespace axm

using namespace axm;

extern "C" int axm_moe_ep_workspace_bytes(const AxmEpLayout* layout, const AxmMoeDesc* desc, size_t* bytes,
                                          size_t* zero_bytes) {
  if (int rc = validate_ep_layer(layout, desc)) return rc;
  if (bytes == nullptr) return fail(AXM_ERR_ARGUMENT, "bytes is null");
  EpWs w = carve_ep(layout, desc, nullptr);
  *bytes = w.bytes;
  if (zero_bytes) *zero_bytes = w.zero_bytes;
  return AXM_OK;
}

extern "C" int axm_moe_ep_status_word(const AxmEpLayout* layout, const AxmMoeDesc* desc, void* workspace,
                                      int32_t** status, int32_t** rows_received) {
  if (int rc = validate_ep_layer(layout, desc)) return rc;
  if (!workspace) return fail(AXM_ERR_ARGUMENT, "axm_moe_ep_status_word: null pointer");
  EpWs w = carve_ep(layout, desc, workspace);
  if (status) *status = w.status;
  if (rows_received) *rows_received = w.rows_received;
  return AXM_OK;
}

extern "C" int axm_moe_ep_forward(const AxmEpLayout* layout, const AxmMoeDesc* desc, const AxmEpTensors* tensors,
                                  void* workspace, size_t workspace_bytes, uint32_t step, void* stream) {
  return ep_forward_impl(layout, desc, tensors, workspace, workspace_bytes, step, stream, nullptr);
}

extern "C" int axm_moe_ep_forward_profiled(const AxmEpLayout* layout, const AxmMoeDesc* desc,
                                           const AxmEpTensors* tensors, void* workspace, size_t workspace_bytes,
                                           uint32_t step, void* stream, float* stage_ms) {
  if (stage_ms == nullptr) return fail(AXM_ERR_ARGUMENT, "stage_ms is null");
  for (int i = 0; i < 9; ++i) stage_ms[i] = 0.0f;
  cudaEvent_t ev[10];
  for (int i = 0; i < 10; ++i)
    if (cudaEventCreate(&ev[i]) != cudaSuccess) return fail(AXM_ERR_LAUNCH, "cudaEventCreate failed");
  int rc = ep_forward_impl(layout, desc, tensors, workspace, workspace_bytes, step, stream, ev);
  if (rc == AXM_OK) {
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) rc = fail(AXM_ERR_LAUNCH, "synchronise: %s", cudaGetErrorString(e));
    else {
      for (int i = 0; i < 7; ++i) cudaEventElapsedTime(&stage_ms[i], ev[i], ev[i + 1]);
      // the overlapped copy: when it started and ended, counted from the start of the down GEMM
      if (cudaEventQuery(ev[8]) == cudaSuccess && cudaEventQuery(ev[9]) == cudaSuccess) {
        cudaEventElapsedTime(&stage_ms[7], ev[4], ev[8]);
        cudaEventElapsedTime(&stage_ms[8], ev[4], ev[9]);
      }
      cudaGetLastError();
    }
  }
  for (int i = 0; i < 10; ++i) cudaEventDestroy(ev[i]);
  return rc;
}

// Host-buffer form: the rank's tokens are cut into `chunks` equal parts (the same number on
// every rank - also with chunks = 0, so the ranks must then hold the same number of tokens or
// at least all lie on one side of 4096; every part is one complete exchange step); part c + 1 comes in over PCIe and
// part c - 1 goes out while part c is computed.  *step is the first step number to use and is
// advanced by the number of parts.  Synchronises the stream before returning.
extern "C" int axm_moe_ep_forward_host(const AxmEpLayout* layout, const AxmMoeDesc* desc,
                                       const AxmEpTensors* tensors, const void* h_x, void* h_out, void* d_x,
                                       void* d_out, void* workspace, size_t workspace_bytes, int32_t chunks,
                                       uint32_t* step, void* stream) {
  if (int rc = validate_ep_layer(layout, desc)) return rc;
  if (!tensors || !h_x || !h_out || !d_x || !d_out || !step)
    return fail(AXM_ERR_ARGUMENT, "axm_moe_ep_forward_host: null pointer");
  if (chunks < 0 || chunks > 8) return fail(AXM_ERR_ARGUMENT, "chunks %d not in 0..8", chunks);
  // 0 = this library's choice.  Every part is a whole exchange step, whose fixed cost (about 0.2 ms)
  // has to be won back by the copy it hides: measured for T 8192, D 4096, F 14336 over 2 GPUs
  // (4096 tokens per rank) 3.83 ms in two parts against 4.06 in one; over 4 GPUs 2.60 against 2.51.
  if (chunks == 0) chunks = desc->tokens >= 4096 ? 2 : 1;
  if (*step == 0) return fail(AXM_ERR_ARGUMENT, "step starts at 1");
  if (int rc = require_device()) return rc;
  EpPipe* pipe = ep_pipe();
  if (pipe == nullptr) return fail(AXM_ERR_LAUNCH, "could not create the copy streams");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int T = desc->tokens, E = desc->num_experts, k = desc->top_k;
  const size_t row_bytes = (size_t)desc->d_model * 2;
  AXM_CUDA(cudaEventRecord(pipe->start, st));
  AXM_CUDA(cudaStreamWaitEvent(pipe->in, pipe->start, 0));
  AXM_CUDA(cudaStreamWaitEvent(pipe->out, pipe->start, 0));
  const int per = (T + chunks - 1) / chunks;
  for (int c = 0; c < chunks; ++c) {
    // every rank runs the same number of exchange steps, also when its last parts are empty
    const int t0 = c * per < T ? c * per : T;
    const int n = (c + 1) * per < T ? per : T - t0;
    const size_t off = (size_t)t0 * row_bytes;
    if (n > 0)
      AXM_CUDA(cudaMemcpyAsync(static_cast<char*>(d_x) + off, static_cast<const char*>(h_x) + off,
                               (size_t)n * row_bytes, cudaMemcpyHostToDevice, pipe->in));
    AXM_CUDA(cudaEventRecord(pipe->arrived[c], pipe->in));
    AXM_CUDA(cudaStreamWaitEvent(st, pipe->arrived[c], 0));
    AxmMoeDesc d = *desc;
    d.tokens = n;
    if (c > 0) d.flags |= AXM_FLAG_HIST_ACCUMULATE;
    AxmEpTensors tt = *tensors;
    tt.x = static_cast<char*>(d_x) + off;
    tt.out = static_cast<char*>(d_out) + off;
    if (tensors->y) tt.y = static_cast<char*>(tensors->y) + off;
    if (tensors->logits) tt.logits = tensors->logits + (size_t)t0 * E;
    if (tensors->topk_idx) tt.topk_idx = tensors->topk_idx + (size_t)t0 * k;
    if (tensors->topk_gate) tt.topk_gate = tensors->topk_gate + (size_t)t0 * k;
    // the workspace was sized for the whole batch: a part needs no more
    if (int rc = ep_forward_impl(layout, &d, &tt, workspace, workspace_bytes, *step, stream, nullptr)) return rc;
    *step += 1;
    AXM_CUDA(cudaEventRecord(pipe->done[c], st));
    AXM_CUDA(cudaStreamWaitEvent(pipe->out, pipe->done[c], 0));
    if (n > 0)
      AXM_CUDA(cudaMemcpyAsync(static_cast<char*>(h_out) + off, static_cast<char*>(d_out) + off,
                               (size_t)n * row_bytes, cudaMemcpyDeviceToHost, pipe->out));
  }
  cudaError_t e = cudaStreamSynchronize(pipe->out);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return fail(AXM_ERR_LAUNCH, "pipelined expert-parallel host call: %s", cudaGetErrorString(e));
  return AXM_OK;
}
