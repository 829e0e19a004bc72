// A host program in plain C++ that drives the MoE layer through the C ABI alone
// (include/axm_moe.h + the CUDA runtime): no Python, no torch.  It mirrors what the
// reference engine's host wrapper does around forward_mixture_experts
// (core/src/ai.cpp:593-623): upload activations, run the layer, download the output
// and the histogram, check the invariants the engine's own test checks
// (core/test/test_ai.cpp:944-1015: histogram sums to k*T, no dead expert at this
// size, every output finite) and that two calls give identical bytes.
// Built and run by tests/test_cabi_host_gpu.py.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "axm_moe.h"

static uint16_t to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static float from_bf16(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

#define CK(x)                                                                 \
  do {                                                                        \
    cudaError_t e_ = (x);                                                     \
    if (e_ != cudaSuccess) {                                                  \
      fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_));                \
      return 2;                                                               \
    }                                                                         \
  } while (0)

template <typename T>
static int upload(const std::vector<T>& h, void** d) {
  CK(cudaMalloc(d, h.size() * sizeof(T)));
  CK(cudaMemcpy(*d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
  return 0;
}

int main() {
  const int T = 256, D = 256, E = 8, K = 2, F = 512;
  std::mt19937 rng(1337);
  std::normal_distribution<float> act(0.f, 1.f), wgt(0.f, 0.02f);
  std::vector<uint16_t> x(T * D), wg((size_t)E * D * F), wu((size_t)E * D * F), wd((size_t)E * F * D);
  std::vector<float> wr(D * E);
  for (auto& v : x) v = to_bf16(act(rng));
  for (auto& v : wr) v = wgt(rng);
  for (auto& v : wg) v = to_bf16(wgt(rng));
  for (auto& v : wu) v = to_bf16(wgt(rng));
  for (auto& v : wd) v = to_bf16(wgt(rng));

  void *d_x, *d_wr, *d_wg, *d_wu, *d_wd, *d_out, *d_hist, *d_ws;
  if (upload(x, &d_x) || upload(wr, &d_wr) || upload(wg, &d_wg) || upload(wu, &d_wu) || upload(wd, &d_wd)) return 2;
  CK(cudaMalloc(&d_out, (size_t)T * D * 2));
  CK(cudaMalloc(&d_hist, E * sizeof(int32_t)));

  AxmMoeDesc desc = {T, D, F, E, K, 0, AXM_ROUTER_FP32, AXM_FLAG_RESIDUAL};
  size_t ws_bytes = 0;
  if (axm_moe_workspace_bytes(&desc, &ws_bytes) != AXM_OK) {
    fprintf(stderr, "workspace: %s\n", axm_last_error());
    return 3;
  }
  CK(cudaMalloc(&d_ws, ws_bytes));
  AxmMoeTensors t;
  memset(&t, 0, sizeof(t));
  t.x = d_x;
  t.router_w = d_wr;
  t.w_gate = d_wg;
  t.w_up = d_wu;
  t.w_down = d_wd;
  t.histogram = static_cast<int32_t*>(d_hist);
  t.out = d_out;

  cudaStream_t st;
  CK(cudaStreamCreate(&st));
  std::vector<uint16_t> out1(T * D), out2(T * D);
  std::vector<int32_t> hist(E);
  for (int rep = 0; rep < 2; ++rep) {
    if (axm_moe_forward(&desc, &t, d_ws, ws_bytes, st) != AXM_OK) {
      fprintf(stderr, "forward: %s\n", axm_last_error());
      return 3;
    }
    CK(cudaStreamSynchronize(st));
    CK(cudaMemcpy((rep ? out2 : out1).data(), d_out, (size_t)T * D * 2, cudaMemcpyDeviceToHost));
  }
  CK(cudaMemcpy(hist.data(), d_hist, E * sizeof(int32_t), cudaMemcpyDeviceToHost));
  int32_t* d_status = nullptr;
  int32_t status = -1;
  if (axm_moe_status_word(&desc, d_ws, &d_status) != AXM_OK) return 3;
  CK(cudaMemcpy(&status, d_status, 4, cudaMemcpyDeviceToHost));

  long sum = 0;
  int dead = 0;
  for (int e = 0; e < E; ++e) {
    sum += hist[e];
    dead += hist[e] == 0;
  }
  int bad = 0, moved = 0;
  for (int i = 0; i < T * D; ++i) {
    float v = from_bf16(out1[i]);
    bad += !std::isfinite(v);
    moved += out1[i] != x[i];
  }
  const bool same = memcmp(out1.data(), out2.data(), out1.size() * 2) == 0;
  printf("%s histogram_sum=%ld dead=%d nonfinite=%d changed=%d deterministic=%d status=%d\n", axm_version(), sum,
         dead, bad, moved, (int)same, status);
  // a null argument is refused with a message, not a crash
  t.out = nullptr;
  const int rc = axm_moe_forward(&desc, &t, d_ws, ws_bytes, st);
  printf("null out -> %d (%s)\n", rc, axm_last_error());
  const bool ok = sum == (long)K * T && dead == 0 && bad == 0 && moved > T * D / 2 && same && status == 0 &&
                  rc == AXM_ERR_ARGUMENT;
  printf(ok ? "OK\n" : "FAILED\n");
  return ok ? 0 : 1;
}
