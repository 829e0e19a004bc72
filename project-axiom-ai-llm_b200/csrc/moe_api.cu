// Host side of the C ABI: error text, device checks, workspace carving and the
// whole-layer call.  Mirrors the host logic of forward_mixture_experts in the
// reference engine (core/src/CUDA/kernel/moe_router.cu:205-320): validate, then
// enqueue router -> dispatch -> expert FFN -> combine on the caller's stream and
// report only enqueue-time errors.  Unlike the engine it allocates nothing: all
// scratch comes from the caller's workspace.
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "router.cuh"

namespace axm {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return status;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(AXM_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  return AXM_OK;
}

struct DeviceInfo {
  int checked_device = -1;
  int major = 0;
  int sms = 0;
  cudaError_t err = cudaSuccess;
};

static DeviceInfo& device_info() {
  static thread_local DeviceInfo info;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    info.err = e;
    info.checked_device = -1;
    cudaGetLastError();
    return info;
  }
  if (dev != info.checked_device) {
    cudaDeviceProp p;
    info.err = cudaGetDeviceProperties(&p, dev);
    if (info.err == cudaSuccess) {
      info.major = p.major;
      info.sms = p.multiProcessorCount;
      info.checked_device = dev;
    } else {
      cudaGetLastError();
    }
  }
  return info;
}

int require_device() {
  DeviceInfo& i = device_info();
  if (i.err != cudaSuccess)
    return fail(AXM_ERR_DEVICE, "no usable CUDA device: %s", cudaGetErrorString(i.err));
  if (i.major != 10)
    return fail(AXM_ERR_DEVICE, "device has compute capability %d.x; this library is sm_100a only", i.major);
  return AXM_OK;
}

int sm_count() { return device_info().sms > 0 ? device_info().sms : 148; }

int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return dev;
}

int cuda_status(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return AXM_OK;
  cudaGetLastError();  // the error is reported here; do not leave it for a later launch check
  return fail(AXM_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
}

int ensure_dynamic_smem(const void* kernel, size_t bytes, SmemLimitCache* cache, const char* what) {
  if (bytes <= 48u * 1024u) return AXM_OK;  // within the default limit
  const int dev = current_device();
  // Racing threads may both ask the runtime; the attribute only ever grows, so that is harmless.
  if (dev >= 0 && dev < 64 && cache->granted[dev] >= (int)bytes) return AXM_OK;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(AXM_ERR_LAUNCH, "%s: %zu bytes of shared memory refused: %s", what, bytes, cudaGetErrorString(e));
  }
  if (dev >= 0 && dev < 64) cache->granted[dev] = (int)bytes;
  return AXM_OK;
}

int launch_expert_ffn(const AxmMoeDesc* d, const void* x_perm, int32_t a_rows, const void* x_alt,
                      int32_t alt_rows, const AxmSegment* segments, int32_t num_segments,
                      const void* w_gate, const void* w_up, const void* w_down,
                      const void* shared_gate, const void* shared_up, const void* shared_down,
                      void* h, void* o, int32_t rows_total, int32_t* status, cudaStream_t st,
                      cudaEvent_t between, const AxmRemoteOut* remote, void* save_g, void* save_u);

// Scratch of the split down projection of calls with a handful of tokens (grouped_ffn_2sm.cu).
void set_down_split_scratch(void* p, size_t bytes);
size_t down_split_scratch_bytes(const AxmMoeDesc* d);
int down_splits_for(const AxmMoeDesc* d, int pairs);
bool use_2sm_kernels();

static size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

// Carves the workspace.  With base == nullptr it only measures.
struct Workspace {
  float* logits;
  int32_t* topk_idx;
  float* topk_gate;
  int32_t* block_counts;
  int32_t* offsets;
  int32_t* row_src;
  int32_t* slot_dst;
  AxmSegment* segments;
  int32_t* status;
  void* x_perm;
  void* h;
  void* o;
  void* router_scratch;  // split, transposed router weights of the tensor-core router (may be empty)
  size_t router_scratch_bytes;
  float* rstd;           // [T] per-token 1/rms of the fused pre-norm call
  void* down_split;      // partial sums of the split down projection (empty beyond eight tokens)
  size_t down_split_bytes;
  size_t bytes;
};

static Workspace carve(const AxmMoeDesc* d, void* base) {
  Workspace w;
  size_t off = 0;
  auto take = [&](size_t n) {
    void* p = base ? static_cast<char*>(base) + off : nullptr;
    off += align256(n);
    return p;
  };
  const size_t T = d->tokens, D = d->d_model, F = d->d_ff, E = d->num_experts, k = d->top_k,
               S = d->num_shared;
  const size_t rows = T * k + T * S;
  w.status = static_cast<int32_t*>(take(sizeof(int32_t)));
  w.logits = static_cast<float*>(take(sizeof(float) * T * E));
  w.topk_idx = static_cast<int32_t*>(take(sizeof(int32_t) * T * k));
  w.topk_gate = static_cast<float*>(take(sizeof(float) * T * k));
  w.block_counts = static_cast<int32_t*>(take(sizeof(int32_t) * AXM_ROUTE_BLOCKS * E));
  w.offsets = static_cast<int32_t*>(take(sizeof(int32_t) * (E + 1)));
  w.row_src = static_cast<int32_t*>(take(sizeof(int32_t) * T * k));
  w.slot_dst = static_cast<int32_t*>(take(sizeof(int32_t) * T * k));
  w.segments = static_cast<AxmSegment*>(take(sizeof(AxmSegment) * (E + S)));
  w.x_perm = take(2 * T * k * D);
  w.h = take(((d->flags & AXM_FLAG_H_EXACT) ? 4 : 2) * rows * F);  // one or two bf16 terms per element
  w.o = take(4 * rows * D);
  w.router_scratch_bytes = 0;
  axm_moe_router_scratch_bytes(d, &w.router_scratch_bytes);
  w.router_scratch = take(w.router_scratch_bytes);
  w.rstd = static_cast<float*>(take(sizeof(float) * T));
  w.down_split_bytes = down_split_scratch_bytes(d);
  w.down_split = take(w.down_split_bytes);
  w.bytes = off;
  return w;
}

static int validate_forward(const AxmMoeDesc* d) {
  if (d == nullptr) return fail(AXM_ERR_ARGUMENT, "desc is null");
  if (d->tokens < 0) return fail(AXM_ERR_ARGUMENT, "tokens %d negative", d->tokens);
  if (d->d_model <= 0 || d->d_ff <= 0 || d->d_model % 8 || d->d_ff % 8)
    return fail(AXM_ERR_ARGUMENT, "d_model %d and d_ff %d must be positive multiples of 8", d->d_model, d->d_ff);
  if (d->num_experts <= 0 || d->num_experts > 256)
    return fail(AXM_ERR_ARGUMENT, "num_experts %d not in 1..256", d->num_experts);
  if (d->top_k <= 0 || d->top_k > 8 || d->top_k > d->num_experts)
    return fail(AXM_ERR_ARGUMENT, "top_k %d not in 1..min(num_experts, 8)", d->top_k);
  if (d->num_shared < 0 || d->num_shared > 8)
    return fail(AXM_ERR_ARGUMENT, "num_shared %d not in 0..8", d->num_shared);
  if (d->router_dtype != AXM_ROUTER_BF16 && d->router_dtype != AXM_ROUTER_FP32)
    return fail(AXM_ERR_ARGUMENT, "router_dtype %d unknown", d->router_dtype);
  if ((long long)d->tokens * (d->top_k + d->num_shared) > 0x7fffffffLL)
    return fail(AXM_ERR_ARGUMENT, "row count overflows int32");
  return AXM_OK;
}

}  // namespace axm

using namespace axm;

extern "C" const char* axm_last_error(void) { return g_err; }

extern "C" const char* axm_version(void) { return "axm_moe 0.1 sm_100a"; }

extern "C" int axm_moe_forward_launches(const AxmMoeDesc* desc) {
  if (validate_forward(desc) != AXM_OK) return AXM_ERR_ARGUMENT;
  if (desc->tokens == 0) return 0;
  size_t scratch = 0;
  axm_moe_router_scratch_bytes(desc, &scratch);
  // router (preceded by its weight-preparation kernel on the tensor-core path), permute,
  // gate/up GEMM, down GEMM (plus the sum of its ranges when a handful of tokens makes it split
  // the reduction; counted for the 74 CTA pairs of a B200), combine
  const int split = (use_2sm_kernels() && down_splits_for(desc, 74) > 1) ? 1 : 0;
  return (scratch > 0 ? 6 : 5) + split;
}

extern "C" int axm_moe_workspace_bytes(const AxmMoeDesc* desc, size_t* bytes) {
  if (int rc = validate_forward(desc)) return rc;
  if (bytes == nullptr) return fail(AXM_ERR_ARGUMENT, "bytes is null");
  *bytes = carve(desc, nullptr).bytes;
  return AXM_OK;
}

extern "C" int axm_moe_status_word(const AxmMoeDesc* desc, void* workspace, int32_t** status) {
  if (int rc = validate_forward(desc)) return rc;
  if (!workspace || !status) return fail(AXM_ERR_ARGUMENT, "axm_moe_status_word: null pointer");
  *status = carve(desc, workspace).status;
  return AXM_OK;
}

static int launch_rms_stats(const void* x, float* rstd, int tokens, int d_model, float eps, cudaStream_t st);

// residual_src: what the combine adds to y (t->x for the plain layer; the un-normalised
// block input when x is the output of a preceding RMSNorm).
// norm_gamma / norm_eps (norm_eps > 0): fused pre-norm form - t->x is the un-normalised block
// input; one statistics pass stores 1/rms per token, the router and the permute kernel apply
// the normalisation as they read x, nothing normalised is written to memory.
static int forward_impl(const AxmMoeDesc* desc, const AxmMoeTensors* t, void* workspace,
                        size_t workspace_bytes, void* stream, cudaEvent_t* ev,
                        const void* residual_src = nullptr, const float* norm_gamma = nullptr,
                        float norm_eps = 0.0f) {
  if (int rc = validate_forward(desc)) return rc;
  if (t == nullptr) return fail(AXM_ERR_ARGUMENT, "tensors is null");
  if (desc->tokens == 0) return AXM_OK;  // empty input: nothing to enqueue
  if (!t->x || !t->router_w || !t->w_gate || !t->w_up || !t->w_down || !t->out)
    return fail(AXM_ERR_ARGUMENT, "x, router_w, w_gate, w_up, w_down and out are required");
  if (desc->num_shared > 0 && (!t->shared_gate || !t->shared_up || !t->shared_down))
    return fail(AXM_ERR_ARGUMENT, "num_shared > 0 needs shared_gate, shared_up and shared_down");
  if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(AXM_ERR_WORKSPACE, "workspace is null or not 256-byte aligned");
  Workspace w = carve(desc, workspace);
  if (workspace_bytes < w.bytes)
    return fail(AXM_ERR_WORKSPACE, "workspace has %zu bytes, %zu needed", workspace_bytes, w.bytes);
  if (int rc = require_device()) return rc;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* logits = t->logits ? t->logits : w.logits;
  int32_t* idx = t->topk_idx ? t->topk_idx : w.topk_idx;
  float* gate = t->topk_gate ? t->topk_gate : w.topk_gate;
  int32_t* offsets = t->offsets ? t->offsets : w.offsets;
  int32_t* row_src = t->row_src ? t->row_src : w.row_src;
  int32_t* slot_dst = t->slot_dst ? t->slot_dst : w.slot_dst;
  const int T = desc->tokens, k = desc->top_k, S = desc->num_shared, E = desc->num_experts;

  if (ev) cudaEventRecord(ev[0], st);
  bool router_cleared_status = false;  // the tensor-core router's preparation kernel clears the word
  int rc;
  const float* rstd = nullptr;
  if (norm_eps > 0.0f) {
    const RouterTcPlan plan = router_tc_plan(desc);
    if (!plan.ok || w.router_scratch_bytes < plan.scratch_bytes || (reinterpret_cast<uintptr_t>(t->x) & 15) != 0)
      return fail(AXM_ERR_ARGUMENT, "the fused pre-norm form needs the tensor-core router (at most 80 experts with "
                                    "fp32 router weights, 16-byte aligned x); pass x_norm to run the two-kernel form");
    if ((rc = launch_rms_stats(t->x, w.rstd, T, desc->d_model, norm_eps, st))) return rc;
    rstd = w.rstd;
    rc = launch_router_tc(desc, plan, t->x, t->router_w, t->router_bias, logits, idx, gate, w.block_counts,
                          w.router_scratch, w.status, st, rstd, norm_gamma);
    router_cleared_status = true;
  } else {
    rc = launch_router_auto(desc, t->x, t->router_w, t->router_bias, logits, idx, gate, w.block_counts,
                            w.router_scratch, w.router_scratch_bytes, w.status, stream, &router_cleared_status);
  }
  if (rc) return rc;
  if (ev) cudaEventRecord(ev[1], st);
  rc = launch_permute(desc, t->x, idx, w.block_counts, t->histogram, offsets, row_src, slot_dst,
                      w.x_perm, w.segments, router_cleared_status ? nullptr : w.status, st, 1, rstd, norm_gamma);
  if (rc) return rc;
  if (ev) cudaEventRecord(ev[2], st);
  set_down_split_scratch(w.down_split, w.down_split_bytes);
  rc = launch_expert_ffn(desc, w.x_perm, T * k, t->x, T, w.segments, E + S, t->w_gate, t->w_up,
                         t->w_down, t->shared_gate, t->shared_up, t->shared_down, w.h, w.o,
                         T * k + T * S, w.status, st, ev ? ev[3] : nullptr, nullptr, nullptr, nullptr);
  set_down_split_scratch(nullptr, 0);
  if (rc) return rc;
  if (ev) cudaEventRecord(ev[4], st);
  const float* o_shared =
      S > 0 ? static_cast<const float*>(w.o) + (size_t)T * k * desc->d_model : nullptr;
  rc = axm_moe_combine(desc, residual_src ? residual_src : t->x, w.o, o_shared, slot_dst, gate, t->y, t->out,
                       stream);
  if (ev) cudaEventRecord(ev[5], st);
  return rc;
}

extern "C" int axm_moe_forward(const AxmMoeDesc* desc, const AxmMoeTensors* t, void* workspace,
                               size_t workspace_bytes, void* stream) {
  return forward_impl(desc, t, workspace, workspace_bytes, stream, nullptr);
}

// y[t, :] = bf16(x[t, :] * rsqrt(mean(x[t, :]^2) + eps) * gamma).  One warp per token:
// the row stays in registers between the sum of squares and the scaling.
// kWrite = false: only rstd[t] = rsqrt(mean(x[t]^2) + eps) is stored (same sum order, hence the
// same bits, as in the writing form); the router and the permute kernel then apply it on load.
constexpr int kNormMaxChunks = 16;  // 16-byte pieces per lane kept in registers (D <= 4096)
template <bool kWrite>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma,
               __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int T, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (blockDim.x >> 5);
  const int chunks = D / 8;
  for (int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < T; t += warps) {
    const uint4* row = reinterpret_cast<const uint4*>(x + (size_t)t * D);
    uint4 v[kNormMaxChunks];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < kNormMaxChunks; ++i) {
      const int c = lane + 32 * i;
      v[i] = make_uint4(0, 0, 0, 0);
      if (c < chunks) v[i] = __ldg(row + c);
      const uint32_t w4[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        ss = fmaf(bf16_lo(w4[j]), bf16_lo(w4[j]), ss);
        ss = fmaf(bf16_hi(w4[j]), bf16_hi(w4[j]), ss);
      }
    }
    for (int c = lane + 32 * kNormMaxChunks; c < chunks; c += 32) {  // rows longer than the register tile
      const uint4 u = __ldg(row + c);
      const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
      for (int j = 0; j < 4; ++j) {
        ss = fmaf(bf16_lo(w4[j]), bf16_lo(w4[j]), ss);
        ss = fmaf(bf16_hi(w4[j]), bf16_hi(w4[j]), ss);
      }
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
    const float rstd = rsqrtf(ss / (float)D + eps);
    if (!kWrite) {
      if (lane == 0) rstd_out[t] = rstd;
      continue;
    }
    uint4* out = reinterpret_cast<uint4*>(y + (size_t)t * D);
    auto scale = [&](uint4 u, int c) {
      const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
      uint32_t r[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int d = c * 8 + 2 * j;
        const float g0 = gamma ? __ldg(gamma + d) : 1.0f, g1 = gamma ? __ldg(gamma + d + 1) : 1.0f;
        r[j] = pack_bf16(bf16_lo(w4[j]) * rstd * g0, bf16_hi(w4[j]) * rstd * g1);
      }
      return make_uint4(r[0], r[1], r[2], r[3]);
    };
#pragma unroll
    for (int i = 0; i < kNormMaxChunks; ++i) {
      const int c = lane + 32 * i;
      if (c < chunks) out[c] = scale(v[i], c);
    }
    for (int c = lane + 32 * kNormMaxChunks; c < chunks; c += 32) out[c] = scale(__ldg(row + c), c);
  }
}

extern "C" int axm_moe_rmsnorm(const void* x, const float* gamma, void* y, int32_t tokens,
                               int32_t d_model, float eps, void* stream) {
  if (!x || !y) return fail(AXM_ERR_ARGUMENT, "axm_moe_rmsnorm: null pointer");
  if (tokens < 0 || d_model <= 0 || d_model % 8) return fail(AXM_ERR_ARGUMENT, "axm_moe_rmsnorm: bad shape");
  if (tokens == 0) return AXM_OK;
  if (int rc = require_device()) return rc;
  int blocks = (tokens + 7) / 8;
  if (blocks > 8 * sm_count()) blocks = 8 * sm_count();
  rmsnorm_kernel<true><<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), gamma, static_cast<__nv_bfloat16*>(y), nullptr, tokens, d_model, eps);
  return check_launch("rmsnorm_kernel");
}

// rstd[t] alone (device buffer of `tokens` floats): the statistics pass of the fused pre-norm call.
static int launch_rms_stats(const void* x, float* rstd, int tokens, int d_model, float eps, cudaStream_t st) {
  int blocks = (tokens + 7) / 8;
  if (blocks > 8 * sm_count()) blocks = 8 * sm_count();
  rmsnorm_kernel<false><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), nullptr, nullptr, rstd, tokens,
                                                d_model, eps);
  return check_launch("rmsnorm_kernel(stats)");
}

extern "C" int axm_moe_forward_prenorm(const AxmMoeDesc* desc, const AxmMoeTensors* t, const float* gamma,
                                       float eps, void* x_norm, void* workspace, size_t workspace_bytes,
                                       void* stream) {
  if (int rc = validate_forward(desc)) return rc;
  if (!t || !t->x) return fail(AXM_ERR_ARGUMENT, "axm_moe_forward_prenorm: null pointer");
  if (!(eps > 0.0f)) return fail(AXM_ERR_ARGUMENT, "axm_moe_forward_prenorm: eps must be positive");
  if (x_norm == nullptr) {
    // fused form: the normalised activations are never written; shared experts would need them
    // as a GEMM operand in memory
    if (desc->num_shared > 0)
      return fail(AXM_ERR_ARGUMENT, "axm_moe_forward_prenorm without x_norm does not take shared experts");
    return forward_impl(desc, t, workspace, workspace_bytes, stream, nullptr, t->x, gamma, eps);
  }
  if (x_norm == t->out) return fail(AXM_ERR_ARGUMENT, "x_norm must not alias out");
  if (int rc = axm_moe_rmsnorm(t->x, gamma, x_norm, desc->tokens, desc->d_model, eps, stream)) return rc;
  AxmMoeTensors tt = *t;
  tt.x = x_norm;  // the experts and the router see the normalised activations ...
  return forward_impl(desc, &tt, workspace, workspace_bytes, stream, nullptr, t->x);  // ... the residual does not
}

extern "C" int axm_moe_forward_profiled(const AxmMoeDesc* desc, const AxmMoeTensors* t,
                                        void* workspace, size_t workspace_bytes, void* stream,
                                        float* stage_ms) {
  if (stage_ms == nullptr) return fail(AXM_ERR_ARGUMENT, "stage_ms is null");
  for (int i = 0; i < 5; ++i) stage_ms[i] = 0.0f;
  cudaEvent_t ev[6];
  for (int i = 0; i < 6; ++i)
    if (cudaEventCreate(&ev[i]) != cudaSuccess) return fail(AXM_ERR_LAUNCH, "cudaEventCreate failed");
  int rc = forward_impl(desc, t, workspace, workspace_bytes, stream, ev);
  if (rc == AXM_OK && desc->tokens > 0) {
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) rc = fail(AXM_ERR_LAUNCH, "synchronise: %s", cudaGetErrorString(e));
    else
      for (int i = 0; i < 5; ++i) cudaEventElapsedTime(&stage_ms[i], ev[i], ev[i + 1]);
  }
  for (int i = 0; i < 6; ++i) cudaEventDestroy(ev[i]);
  return rc;
}

// Copy streams and events of the pipelined host-buffer call, created once per device.
namespace {
constexpr int kHostChunksMax = 8;
struct HostPipe {
  cudaStream_t in = nullptr, out = nullptr;
  cudaEvent_t arrived[kHostChunksMax] = {}, done[kHostChunksMax] = {}, start = nullptr;
  cudaEvent_t copied[2] = {};  // batch pipeline: the copy out of slot b has read its device buffer
  bool ok = false;
};
HostPipe* host_pipe() {
  static thread_local HostPipe pipes[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  HostPipe& p = pipes[dev];
  if (!p.ok) {
    if (cudaStreamCreateWithFlags(&p.in, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaStreamCreateWithFlags(&p.out, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&p.start, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    for (int i = 0; i < 2; ++i)
      if (cudaEventCreateWithFlags(&p.copied[i], cudaEventDisableTiming) != cudaSuccess) return nullptr;
    for (int i = 0; i < kHostChunksMax; ++i) {
      if (cudaEventCreateWithFlags(&p.arrived[i], cudaEventDisableTiming) != cudaSuccess) return nullptr;
      if (cudaEventCreateWithFlags(&p.done[i], cudaEventDisableTiming) != cudaSuccess) return nullptr;
    }
    p.ok = true;
  }
  return &p;
}
}  // namespace

// Chunk sizes for the host pipeline when every expert holds a handful of 256-row tile pairs per
// chunk (few experts, routing close to uniform: no logit bias, no shared experts).  A chunk of t
// tokens gives an expert about t k / E rows, with a binomial spread; it costs the expert
// pairs(t) = ceil((mean + 2.5 sigma) / 256) tile pairs whether they are full or not.  Even chunks
// waste pairs (three chunks of 2731 tokens of an 8192-token, 8-expert, top-2 batch need 3 pairs
// per expert for 683 rows each).  Instead: a first chunk of one pair per expert, so that little
// copy-in time is exposed, then the remaining pairs in two chunks as full as their pairs allow.
// Writes the three token counts to `tokens` and returns true, or returns false when the batch
// does not fit that pattern.  Measured on 8192 tokens, d_model 4096, 8 experts of 14336 with the
// GPU at its sustained clocks: 5.78 - 5.98 ms per call against 6.09 - 6.24 for three even chunks
// (5.00 device-resident).
static bool tile_aware_schedule(int T, int E, int k, int* tokens) {
  auto pairs = [&](int t) {
    const double mean = (double)t * k / E;
    const double sigma = sqrt(mean * (1.0 - 1.0 / E));
    return (int)ceil((mean + 2.5 * sigma) / 256.0);
  };
  auto cap = [&](int p) {  // most tokens (a multiple of 64) that p pairs per expert hold
    int t = (int)((double)p * 256.0 * E / k) / 64 * 64;
    while (t > 0 && pairs(t) > p) t -= 64;
    return t;
  };
  const int p_total = pairs(T);
  if (p_total < 3 || p_total > 24) return false;
  const int t1 = cap(1);
  if (t1 < 256 || t1 >= T) return false;
  const int p_rest = p_total - 1, p2 = (p_rest + 1) / 2, p3 = p_rest - p2;
  int t2 = cap(p2);
  if (t2 > T - t1) t2 = T - t1;
  const int t3 = T - t1 - t2;
  if (t3 <= 0 || t3 > cap(p3)) return false;
  tokens[0] = t1;
  tokens[1] = t2;
  tokens[2] = t3;
  return true;
}

// Tokens are independent, so the batch is cut into chunks and pipelined: while chunk c
// is computed on the caller's stream, chunk c+1 comes in over PCIe on a copy stream and
// chunk c-1 goes out on another.  Per-token results do not depend on the chunking.
// Chunking needs the permutation outputs (offsets, row_src, slot_dst), which describe
// the whole batch, not to be requested, and two chunk workspaces to fit into the
// caller's workspace; otherwise the call runs as one piece.
extern "C" int axm_moe_forward_host(const AxmMoeDesc* desc, const AxmMoeTensors* t,
                                    const void* h_x, void* h_out, void* d_x, void* d_out,
                                    void* workspace, size_t workspace_bytes, void* stream) {
  if (int rc = validate_forward(desc)) return rc;
  if (!t || !h_x || !h_out || !d_x || !d_out)
    return fail(AXM_ERR_ARGUMENT, "axm_moe_forward_host: null pointer");
  if (desc->tokens == 0) return AXM_OK;
  if (int rc = require_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int T = desc->tokens, D = desc->d_model, E = desc->num_experts, k = desc->top_k;
  const size_t row_bytes = (size_t)D * 2;

  // Chunk sizes.  Only the first chunk's copy in and the last chunk's copy out are not
  // hidden behind compute, which asks for many small chunks; but every chunk streams all
  // expert weights from HBM once more, which asks for few.  Measured on the largest
  // workload (8192 tokens, d_model 4096, 8 experts of 14336: 2.8 GB of weights; host link
  // 29 GB/s in, 57 GB/s out): three even chunks 6.03 ms, 1:3:3:1 6.23, four even 6.43,
  // 2:3:3:2 6.55, six 7.04, against 4.6 ms for the layer alone.  Where the copies take as
  // long as the compute (smaller layers), more chunks pay.  So: from 4096 tokens on, three
  // chunks if the estimated compute time is well above the copy-in time, else four; two
  // from 1024 tokens; with few experts and near-uniform routing the three chunks are sized in tile
  // pairs instead (tile_aware_schedule above).  AXM_HOST_CHUNKS = n (1..8) asks for n even chunks,
  // AXM_HOST_SCHEDULE = "a,b,..." (up to 8 positive integers) for chunks in those
  // proportions; a schedule whose largest chunk does not fit twice into the workspace
  // falls back to even chunks of the same count.
  int weights[kHostChunksMax] = {0};
  int chunks = T >= 4096 ? 4 : (T >= 1024 ? 2 : 1);
  bool uneven = false;
  if (T >= 4096) {
    const double compute_s = 6.0 * T * (double)(k + desc->num_shared) * D * (double)desc->d_ff / 1.3e15;
    const double copy_in_s = (double)T * row_bytes / 28e9;
    if (compute_s > 1.5 * copy_in_s) chunks = 3;
    // Few experts with many rows each: the cost of a chunk is set by how many 256-row tile pairs
    // each expert needs, so the chunks are sized in tile pairs (see tile_aware_schedule).
    if (t->router_bias == nullptr && desc->num_shared == 0 && tile_aware_schedule(T, E, k, weights)) {
      chunks = 3;
      uneven = true;
    }
  }
  if (const char* env = getenv("AXM_HOST_CHUNKS")) {
    int v = atoi(env);
    if (v >= 1 && v <= kHostChunksMax) {
      chunks = v;
      uneven = false;
    }
  }
  if (const char* env = getenv("AXM_HOST_SCHEDULE")) {
    int n = 0;
    bool ok = true;
    for (const char* p = env; *p && ok;) {
      char* end = nullptr;
      long v = strtol(p, &end, 10);
      if (end == p || v <= 0 || v > 1000 || n == kHostChunksMax) {
        ok = false;
        break;
      }
      weights[n++] = (int)v;
      p = (*end == ',') ? end + 1 : end;
      if (*end != ',' && *end != 0) ok = false;
    }
    if (ok && n >= 1) {
      chunks = n;
      uneven = n > 1;
    }
  }
  if (t->offsets || t->row_src || t->slot_dst || d_x == d_out) chunks = 1;
  HostPipe* pipe = chunks > 1 ? host_pipe() : nullptr;
  if (pipe == nullptr) chunks = 1;
  AxmMoeDesc cd = *desc;
  size_t chunk_ws = 0;
  int bounds[kHostChunksMax + 1] = {0};
  for (int attempt = 0; attempt < 2 && chunks > 1; ++attempt) {
    if (uneven) {
      long long total = 0, acc = 0;
      for (int c = 0; c < chunks; ++c) total += weights[c];
      for (int c = 0; c < chunks; ++c) {
        acc += weights[c];
        long long b = ((long long)T * acc / total + 63) & ~63LL;  // any size is valid; keep rows tidy
        bounds[c + 1] = (c + 1 == chunks || b > T) ? T : (int)b;
      }
    } else {
      const int per = (T + chunks - 1) / chunks;
      for (int c = 1; c <= chunks; ++c) bounds[c] = c * per < T ? c * per : T;
    }
    int largest = 0;
    for (int c = 0; c < chunks; ++c) largest = bounds[c + 1] - bounds[c] > largest ? bounds[c + 1] - bounds[c] : largest;
    cd.tokens = largest;
    chunk_ws = carve(&cd, nullptr).bytes;
    // two chunk workspaces and, behind them, one status word per chunk
    if (workspace != nullptr && 2 * chunk_ws + 256 <= workspace_bytes) break;
    if (uneven) {
      uneven = false;  // the largest chunks do not fit twice: try even chunks
    } else {
      chunks = 1;
    }
  }
  if (chunks > 1 && (workspace == nullptr || 2 * chunk_ws + 256 > workspace_bytes)) chunks = 1;
  if (chunks == 1) {
    const size_t bytes = (size_t)T * row_bytes;
    cudaError_t e = cudaMemcpyAsync(d_x, h_x, bytes, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return fail(AXM_ERR_LAUNCH, "H2D copy: %s", cudaGetErrorString(e));
    AxmMoeTensors tt = *t;
    tt.x = d_x;
    tt.out = d_out;
    if (int rc = axm_moe_forward(desc, &tt, workspace, workspace_bytes, stream)) return rc;
    e = cudaMemcpyAsync(h_out, d_out, bytes, cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return fail(AXM_ERR_LAUNCH, "D2H copy: %s", cudaGetErrorString(e));
    int32_t status = 0;
    e = cudaMemcpyAsync(&status, carve(desc, workspace).status, sizeof(int32_t),
                        cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail(AXM_ERR_LAUNCH, "synchronise: %s", cudaGetErrorString(e));
    if (status != 0) return fail(AXM_ERR_TIMEOUT, "a bounded wait in GEMM kernel %d gave up", status);
    return AXM_OK;
  }

  // the copy streams start after whatever the caller already queued on its stream
  AXM_CUDA(cudaEventRecord(pipe->start, st));
  AXM_CUDA(cudaStreamWaitEvent(pipe->in, pipe->start, 0));
  AXM_CUDA(cudaStreamWaitEvent(pipe->out, pipe->start, 0));
  int32_t status[kHostChunksMax] = {};
  int32_t* status_all = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) + 2 * chunk_ws);
  for (int c = 0; c < chunks; ++c) {
    const int t0 = bounds[c], n = bounds[c + 1] - bounds[c];
    if (n <= 0) {
      chunks = c;
      break;
    }
    const size_t off = (size_t)t0 * row_bytes;
    AXM_CUDA(cudaMemcpyAsync(static_cast<char*>(d_x) + off, static_cast<const char*>(h_x) + off, (size_t)n * row_bytes, cudaMemcpyHostToDevice, pipe->in));
    AXM_CUDA(cudaEventRecord(pipe->arrived[c], pipe->in));
    AXM_CUDA(cudaStreamWaitEvent(st, pipe->arrived[c], 0));
    AxmMoeDesc d = *desc;
    d.tokens = n;
    if (c > 0) d.flags |= AXM_FLAG_HIST_ACCUMULATE;  // the histogram covers the whole batch
    AxmMoeTensors tt = *t;
    tt.x = static_cast<char*>(d_x) + off;
    tt.out = static_cast<char*>(d_out) + off;
    if (t->y) tt.y = static_cast<char*>(t->y) + off;
    if (t->logits) tt.logits = t->logits + (size_t)t0 * E;
    if (t->topk_idx) tt.topk_idx = t->topk_idx + (size_t)t0 * k;
    if (t->topk_gate) tt.topk_gate = t->topk_gate + (size_t)t0 * k;
    void* ws = static_cast<char*>(workspace) + (size_t)(c & 1) * chunk_ws;
    if (int rc = axm_moe_forward(&d, &tt, ws, chunk_ws, stream)) return rc;
    AXM_CUDA(cudaMemcpyAsync(status_all + c, carve(&d, ws).status, sizeof(int32_t), cudaMemcpyDeviceToDevice, st));
    AXM_CUDA(cudaEventRecord(pipe->done[c], st));
    AXM_CUDA(cudaStreamWaitEvent(pipe->out, pipe->done[c], 0));
    AXM_CUDA(cudaMemcpyAsync(static_cast<char*>(h_out) + off, static_cast<char*>(d_out) + off, (size_t)n * row_bytes, cudaMemcpyDeviceToHost, pipe->out));
  }
  cudaError_t e = cudaStreamSynchronize(pipe->out);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e == cudaSuccess) e = cudaMemcpy(status, status_all, sizeof(int32_t) * chunks, cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(AXM_ERR_LAUNCH, "pipelined host call: %s", cudaGetErrorString(e));
  for (int c = 0; c < chunks; ++c)
    if (status[c] != 0) return fail(AXM_ERR_TIMEOUT, "a bounded wait in GEMM kernel %d gave up", status[c]);
  return AXM_OK;
}

// A run of batches from host memory, double-buffered on the device: batch i + 1 comes in over
// PCIe while batch i is computed and batch i - 1 goes out, so in steady state a batch costs the
// longer of its compute and its copies instead of their sum.  Every batch is a complete layer
// call over desc->tokens tokens (same arithmetic as axm_moe_forward).  d_x2 and d_out2 hold two
// batches each; the workspace is one layer workspace plus 256 bytes.  Optional per-token outputs
// in `t` (logits, indices, gates, permutation) are refused: they would describe the last batch
// only.  Synchronises before returning.
extern "C" int axm_moe_forward_host_batches(const AxmMoeDesc* desc, const AxmMoeTensors* t,
                                            const void* const* h_x, void* const* h_out, int32_t n_batches,
                                            void* d_x2, void* d_out2, void* workspace, size_t workspace_bytes,
                                            void* stream) {
  if (int rc = validate_forward(desc)) return rc;
  if (!t || !h_x || !h_out || !d_x2 || !d_out2)
    return fail(AXM_ERR_ARGUMENT, "axm_moe_forward_host_batches: null pointer");
  if (n_batches < 0 || n_batches > 64) return fail(AXM_ERR_ARGUMENT, "n_batches %d not in 0..64", n_batches);
  if (t->logits || t->topk_idx || t->topk_gate || t->offsets || t->row_src || t->slot_dst || t->y)
    return fail(AXM_ERR_ARGUMENT, "axm_moe_forward_host_batches: per-token outputs are not kept per batch");
  for (int i = 0; i < n_batches; ++i)
    if (!h_x[i] || !h_out[i]) return fail(AXM_ERR_ARGUMENT, "axm_moe_forward_host_batches: batch %d has a null buffer", i);
  if (d_x2 == d_out2) return fail(AXM_ERR_ARGUMENT, "axm_moe_forward_host_batches: d_x2 and d_out2 must differ");
  if (n_batches == 0 || desc->tokens == 0) return AXM_OK;
  const size_t ws_bytes = carve(desc, nullptr).bytes;
  if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0 || workspace_bytes < ws_bytes + 256)
    return fail(AXM_ERR_WORKSPACE, "workspace is null, not 256-byte aligned or smaller than %zu bytes", ws_bytes + 256);
  if (int rc = require_device()) return rc;
  HostPipe* pipe = host_pipe();
  if (pipe == nullptr) return fail(AXM_ERR_LAUNCH, "could not create the copy streams");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t batch_bytes = (size_t)desc->tokens * desc->d_model * 2;
  int32_t* status_all = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) + ws_bytes);  // [64]
  AXM_CUDA(cudaEventRecord(pipe->start, st));
  AXM_CUDA(cudaStreamWaitEvent(pipe->in, pipe->start, 0));
  AXM_CUDA(cudaStreamWaitEvent(pipe->out, pipe->start, 0));
  for (int i = 0; i < n_batches; ++i) {
    const int b = i & 1;
    char* dx = static_cast<char*>(d_x2) + (size_t)b * batch_bytes;
    char* dout = static_cast<char*>(d_out2) + (size_t)b * batch_bytes;
    // slot b's input was last read by the layer call of batch i - 2
    if (i >= 2) AXM_CUDA(cudaStreamWaitEvent(pipe->in, pipe->done[b], 0));
    AXM_CUDA(cudaMemcpyAsync(dx, h_x[i], batch_bytes, cudaMemcpyHostToDevice, pipe->in));
    AXM_CUDA(cudaEventRecord(pipe->arrived[b], pipe->in));
    AXM_CUDA(cudaStreamWaitEvent(st, pipe->arrived[b], 0));
    // slot b's output was last read by the copy out of batch i - 2
    if (i >= 2) AXM_CUDA(cudaStreamWaitEvent(st, pipe->copied[b], 0));
    AxmMoeTensors tt = *t;
    tt.x = dx;
    tt.out = dout;
    if (int rc = axm_moe_forward(desc, &tt, workspace, ws_bytes, stream)) return rc;
    AXM_CUDA(cudaMemcpyAsync(status_all + i, carve(desc, workspace).status, sizeof(int32_t), cudaMemcpyDeviceToDevice, st));
    AXM_CUDA(cudaEventRecord(pipe->done[b], st));
    AXM_CUDA(cudaStreamWaitEvent(pipe->out, pipe->done[b], 0));
    AXM_CUDA(cudaMemcpyAsync(h_out[i], dout, batch_bytes, cudaMemcpyDeviceToHost, pipe->out));
    AXM_CUDA(cudaEventRecord(pipe->copied[b], pipe->out));
  }
  int32_t status[64] = {};
  cudaError_t e = cudaStreamSynchronize(pipe->out);
  if (e == cudaSuccess) e = cudaStreamSynchronize(pipe->in);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e == cudaSuccess) e = cudaMemcpy(status, status_all, sizeof(int32_t) * n_batches, cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(AXM_ERR_LAUNCH, "batch pipeline: %s", cudaGetErrorString(e));
  for (int i = 0; i < n_batches; ++i)
    if (status[i] != 0) return fail(AXM_ERR_TIMEOUT, "a bounded wait in GEMM kernel %d gave up (batch %d)", status[i], i);
  return AXM_OK;
}
