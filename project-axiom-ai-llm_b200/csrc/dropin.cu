// Drop-in library: the three C symbols through which the reference engine
// reaches its MoE layer (core/src/CUDA/kernel/moe_router.cuh:30-44), implemented
// on top of axm_moe_forward.  A build of the engine that leaves moe_router.cu out
// and links this library instead runs its MoE branch
// (core/src/CUDA/kernel/forward_pass.cu:1590-1598, core/src/ai.cpp:593-656) on
// the tensor-core path unchanged.
//
// The engine passes its weight and activation structs by pointer.  Their
// definitions are not copied here; the fields used are read at the byte offsets
// they have on Linux x86-64 (measured by compiling a probe against the engine's
// header, see oracle/build_ref.sh).  Semantics kept from the engine:
//   * hidden_states is overwritten with x + MoE(x); d_residual_out gets a copy,
//     d_ffn_output the weighted expert sum before the residual;
//   * the eight published buffers are allocated here on first use, stored into
//     the caller's struct and freed by the caller (free_gpu_activations); they
//     come from the engine's own allocate_vram when that symbol is loaded in the
//     process, so that its free_vram accepts them, else from cudaMalloc;
//   * the histogram is zeroed when allocated and accumulates across calls until
//     reset_expert_histogram;
//   * top-2 routing, bf16 router weights, everything enqueued on the caller's
//     stream, the return value reflects enqueue-time errors only;
//   * the SwiGLU intermediate keeps 16 mantissa bits (AXM_FLAG_H_EXACT) so that every
//     output element is within the layer tolerance of the engine's fp32 intermediate.
// Private scratch (workspace, [T][2] index and gate arrays) is kept per device and
// activation struct and re-sized when a call needs more; what it replaces is freed.
// One deliberate difference: the engine looks at the first 16 experts only and
// ignores the rest; this library refuses expert_count > 16 instead of routing to
// a different set of experts than the weights describe.
#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace {

// Byte offsets on Linux x86-64 (struct sizes 472 and 328).
constexpr size_t kW_expert_count = 336, kW_router = 344, kW_gate = 376, kW_up = 384, kW_down = 392;
constexpr size_t kA_ffn_output = 144, kA_residual_out = 160, kA_logits = 216, kA_first = 224,
                 kA_second = 232, kA_w_first = 240, kA_w_second = 248, kA_histogram = 256;

template <typename T>
T load_field(const void* base, size_t off) {
  T v;
  memcpy(&v, static_cast<const char*>(base) + off, sizeof(T));
  return v;
}
void store_ptr(void* base, size_t off, void* p) { memcpy(static_cast<char*>(base) + off, &p, sizeof(p)); }

typedef void* (*AllocFn)(size_t, void*);
typedef void (*FreeFn)(void*, void*);

// The engine's allocator when its symbols are loaded in the process (then its
// free_gpu_activations / free_vram accept what is published here), else the runtime's.
AllocFn engine_alloc() {
  static AllocFn fn = reinterpret_cast<AllocFn>(dlsym(RTLD_DEFAULT, "allocate_vram"));
  return fn;
}
FreeFn engine_free() {
  static FreeFn fn = reinterpret_cast<FreeFn>(dlsym(RTLD_DEFAULT, "free_vram"));
  return fn;
}

void* vram_alloc(size_t bytes, void* stream) {
  if (engine_alloc() != nullptr && engine_free() != nullptr) return engine_alloc()(bytes, stream);
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}

// Releases a buffer this library allocated and has outgrown.  Work that still uses it
// was enqueued on `stream`: the engine's free is ordered on that stream, cudaFree
// waits for the device.
void vram_free(void* p, void* stream) {
  if (p == nullptr) return;
  if (engine_alloc() != nullptr && engine_free() != nullptr) {
    engine_free()(p, stream);
    return;
  }
  if (cudaFree(p) != cudaSuccess) cudaGetLastError();
}

// What this library keeps per (device, activation struct): its private scratch and the
// token / expert counts the published buffers of that struct were sized for.  The engine
// runs one forward at a time per activation struct (its own buffers have the same
// restriction), so calls on the same struct must not overlap; different structs, or the
// same process driving several GPUs, get separate state.
struct Instance {
  int device = -1;
  const void* acts = nullptr;
  void* workspace = nullptr;
  size_t workspace_bytes = 0;
  int32_t* idx = nullptr;  // [T][2]
  float* gate = nullptr;   // [T][2]
  size_t scratch_tokens = 0;
  size_t pub_tokens = 0, pub_experts = 0, pub_dim = 0;  // 0: nothing published yet
};

constexpr int kMaxInstances = 64;
std::mutex g_mutex;
Instance g_instances[kMaxInstances];
int g_num_instances = 0;

Instance* instance_for(int device, const void* acts) {
  for (int i = 0; i < g_num_instances; ++i)
    if (g_instances[i].device == device && g_instances[i].acts == acts) return &g_instances[i];
  if (g_num_instances == kMaxInstances) return nullptr;
  Instance* in = &g_instances[g_num_instances++];
  *in = Instance();
  in->device = device;
  in->acts = acts;
  return in;
}

bool h_exact_mode() {
  // The engine keeps the SwiGLU intermediate in fp32; the two-term intermediate is what
  // meets its tolerance on every element, so it is the default behind the engine's
  // interface.  AXM_DROPIN_H_EXACT=0 selects the faster one-term form.
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("AXM_DROPIN_H_EXACT");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

__global__ void split_top2_kernel(const int32_t* __restrict__ idx, const float* __restrict__ gate,
                                  int32_t* __restrict__ first, int32_t* __restrict__ second,
                                  float* __restrict__ w_first, float* __restrict__ w_second, int T) {
  int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < T) {
    first[t] = idx[2 * t];
    second[t] = idx[2 * t + 1];
    w_first[t] = gate[2 * t];
    w_second[t] = gate[2 * t + 1];
  }
}

bool report(const char* what) {
  fprintf(stderr, "axm_moe drop-in: %s: %s\n", what, axm_last_error());
  return false;
}

}  // namespace

extern "C" AXM_API bool forward_mixture_experts(void* hidden_states, const void* gpu_weights,
                                                void* gpu_activations, size_t sequence_length,
                                                size_t embedding_dim,
                                                size_t feedforward_network_dimension, void* stream) {
  if (!hidden_states || !gpu_weights || !gpu_activations || sequence_length == 0 ||
      embedding_dim == 0 || feedforward_network_dimension == 0)
    return false;
  const size_t E = load_field<size_t>(gpu_weights, kW_expert_count);
  void* router = load_field<void*>(gpu_weights, kW_router);
  void* gate_w = load_field<void*>(gpu_weights, kW_gate);
  void* up_w = load_field<void*>(gpu_weights, kW_up);
  void* down_w = load_field<void*>(gpu_weights, kW_down);
  if (E < 2 || !router || !gate_w || !up_w || !down_w) return false;
  if (E > 16) {
    fprintf(stderr, "axm_moe drop-in: expert_count %zu > 16 is not supported through this interface\n", E);
    return false;
  }
  const size_t T = sequence_length, D = embedding_dim, F = feedforward_network_dimension;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  AxmMoeDesc d = {(int32_t)T, (int32_t)D, (int32_t)F, (int32_t)E, 2, 0, AXM_ROUTER_BF16,
                  AXM_FLAG_RESIDUAL | AXM_FLAG_HIST_ACCUMULATE | (h_exact_mode() ? AXM_FLAG_H_EXACT : 0)};
  size_t need = 0;
  if (axm_moe_workspace_bytes(&d, &need) != AXM_OK) return report("shape");
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }

  std::lock_guard<std::mutex> lock(g_mutex);
  Instance* in = instance_for(device, gpu_activations);
  if (in == nullptr) {
    fprintf(stderr, "axm_moe drop-in: more than %d activation structs in one process\n", kMaxInstances);
    return false;
  }
  // published buffers: allocate the ones the caller's struct does not hold yet
  struct Buf { size_t off; size_t bytes; bool zero; };
  const Buf bufs[] = {
      {kA_logits, sizeof(float) * T * E, false},   {kA_first, sizeof(int32_t) * T, false},
      {kA_second, sizeof(int32_t) * T, false},     {kA_w_first, sizeof(float) * T, false},
      {kA_w_second, sizeof(float) * T, false},     {kA_histogram, sizeof(int32_t) * E, true},
      {kA_ffn_output, 2 * T * D, false},           {kA_residual_out, 2 * T * D, false}};
  bool any_present = false;
  for (const Buf& b : bufs) any_present = any_present || load_field<void*>(gpu_activations, b.off) != nullptr;
  // The engine sizes these buffers on the first call and never again
  // (core/src/CUDA/kernel/moe_router.cu:223-250), so a later call with more tokens or
  // experts would write past them.  This library remembers the sizes and refuses.
  if (any_present && in->pub_tokens != 0 && (T > in->pub_tokens || E > in->pub_experts || D > in->pub_dim)) {
    fprintf(stderr,
            "axm_moe drop-in: the published buffers of this activation struct hold %zu tokens x %zu "
            "experts x %zu columns; a call with %zu x %zu x %zu does not fit (free them first)\n",
            in->pub_tokens, in->pub_experts, in->pub_dim, T, E, D);
    return false;
  }
  if (!any_present) in->pub_tokens = in->pub_experts = in->pub_dim = 0;  // the caller freed them
  for (const Buf& b : bufs) {
    if (load_field<void*>(gpu_activations, b.off) != nullptr) continue;
    void* p = vram_alloc(b.bytes, stream);
    if (p == nullptr) return false;
    if (b.zero && cudaMemsetAsync(p, 0, b.bytes, st) != cudaSuccess) return false;
    store_ptr(gpu_activations, b.off, p);
  }
  if (in->pub_tokens == 0) {
    in->pub_tokens = T;
    in->pub_experts = E;
    in->pub_dim = D;
  }
  if (need > in->workspace_bytes) {
    void* p = vram_alloc(need + 256, stream);
    if (p == nullptr) return false;
    vram_free(in->workspace, stream);
    in->workspace = p;
    in->workspace_bytes = need;
  }
  if (T > in->scratch_tokens) {
    int32_t* ni = static_cast<int32_t*>(vram_alloc(sizeof(int32_t) * 2 * T, stream));
    float* ng = static_cast<float*>(vram_alloc(sizeof(float) * 2 * T, stream));
    if (!ni || !ng) {
      vram_free(ni, stream);
      vram_free(ng, stream);
      return false;
    }
    vram_free(in->idx, stream);
    vram_free(in->gate, stream);
    in->idx = ni;
    in->gate = ng;
    in->scratch_tokens = T;
  }
  void* ws = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(in->workspace) + 255) & ~uintptr_t(255));
  int32_t* g_idx = in->idx;
  float* g_gate = in->gate;
  const size_t g_workspace_bytes = in->workspace_bytes;

  AxmMoeTensors t;
  memset(&t, 0, sizeof(t));
  t.x = hidden_states;
  t.out = hidden_states;  // in place, as the engine does
  t.router_w = router;
  t.w_gate = gate_w;
  t.w_up = up_w;
  t.w_down = down_w;
  t.logits = load_field<float*>(gpu_activations, kA_logits);
  t.topk_idx = g_idx;
  t.topk_gate = g_gate;
  t.histogram = load_field<int32_t*>(gpu_activations, kA_histogram);
  t.y = load_field<void*>(gpu_activations, kA_ffn_output);
  if (axm_moe_forward(&d, &t, ws, g_workspace_bytes, stream) != AXM_OK) return report("forward");
  split_top2_kernel<<<(unsigned)((T + 255) / 256), 256, 0, st>>>(
      g_idx, g_gate, load_field<int32_t*>(gpu_activations, kA_first),
      load_field<int32_t*>(gpu_activations, kA_second), load_field<float*>(gpu_activations, kA_w_first),
      load_field<float*>(gpu_activations, kA_w_second), (int)T);
  if (cudaMemcpyAsync(load_field<void*>(gpu_activations, kA_residual_out), hidden_states, 2 * T * D,
                      cudaMemcpyDeviceToDevice, st) != cudaSuccess)
    return false;
  return cudaGetLastError() == cudaSuccess;
}

extern "C" AXM_API bool download_expert_counts(const void* gpu_activations, int32_t* h_histogram,
                                               size_t num_experts) {
  if (!gpu_activations || !h_histogram || num_experts == 0) return false;
  const int32_t* hist = load_field<const int32_t*>(gpu_activations, kA_histogram);
  if (hist == nullptr) return false;
  return cudaMemcpy(h_histogram, hist, sizeof(int32_t) * num_experts, cudaMemcpyDeviceToHost) == cudaSuccess;
}

extern "C" AXM_API bool reset_expert_histogram(void* gpu_activations, size_t num_experts, void* stream) {
  if (!gpu_activations || num_experts == 0) return false;
  int32_t* hist = load_field<int32_t*>(gpu_activations, kA_histogram);
  if (hist == nullptr) return false;
  return cudaMemsetAsync(hist, 0, sizeof(int32_t) * num_experts, static_cast<cudaStream_t>(stream)) ==
         cudaSuccess;
}
