// The part of the router whose results must be bit-identical wherever it runs: softmax,
// top-k with the lowest index winning ties, renormalised gates, following the fp32
// operation order of the reference engine's router kernel
// (core/src/CUDA/kernel/moe_router.cu:59-110).  Shared by the routing-from-logits kernel,
// the CUDA-core fused router (router.cu) and the tensor-core router (router_tc.cu).
// Translation units that include this file must be compiled without fast-math.
#pragma once

#include "common.cuh"

namespace axm {

constexpr int kRouteMaxK = 8;

// Softmax / top-k / gates for one token whose logits sit in shared memory
// (row `z`, overwritten with probabilities and then scratched).  `hist` receives one
// atomic increment per selected expert (shared or global memory).
template <int K_MAX>
__device__ __forceinline__ void route_one_token(float* z, int E, int k, int32_t* idx_out,
                                                float* gate_out, int* hist_s) {
  float m = z[0];
  for (int e = 1; e < E; ++e) m = z[e] > m ? z[e] : m;
  float s = 0.0f;
  for (int e = 0; e < E; ++e) {
    float p = expf(z[e] - m);
    z[e] = p;
    s += p;
  }
  float inv = 1.0f / (s + 1e-9f);
  for (int e = 0; e < E; ++e) z[e] *= inv;

  int sel[K_MAX];
  float pv[K_MAX];
  float sel_sum = 0.0f;
#pragma unroll
  for (int i = 0; i < K_MAX; ++i) {
    if (i < k) {
      int best = 0;
      float bv = -1.0f;
      for (int e = 0; e < E; ++e) {
        float p = z[e];
        if (p > bv) {
          bv = p;
          best = e;
        }
      }
      z[best] = -2.0f;  // taken
      sel[i] = best;
      pv[i] = bv;
      sel_sum += bv;
    }
  }
  float denom = sel_sum + 1e-9f;
#pragma unroll
  for (int i = 0; i < K_MAX; ++i) {
    if (i < k) {
      idx_out[i] = sel[i];
      gate_out[i] = pv[i] / denom;
      atomicAdd(&hist_s[sel[i]], 1);
    }
  }
}


// ---- tensor-core router (router_tc.cu): launch plan and host entry ------------------------
struct RouterTcPlan {
  bool ok;          // false: this shape is served by the CUDA-core kernel
  int epad, terms, n_cols, stages, stage_bytes, tmem_cols, exch_bytes, tile_bytes, cs;
  size_t smem_bytes, scratch_bytes;
};
RouterTcPlan router_tc_plan(const AxmMoeDesc* d);
// The tensor-core router when the shape and the scratch allow it (*used_tc = true; its
// preparation kernel also clears *status), else the CUDA-core kernel.
int launch_router_auto(const AxmMoeDesc* desc, const void* x, const void* router_w, const float* router_bias,
                       float* logits, int32_t* topk_idx, float* topk_gate, int32_t* block_counts,
                       void* scratch, size_t scratch_bytes, int32_t* status, void* stream, bool* used_tc);
// norm_rstd / norm_gamma: pre-norm form (the router sees bf16(x * rstd[t] * gamma) without it
// being materialised); both NULL for the plain form.
int launch_router_tc(const AxmMoeDesc* d, const RouterTcPlan& p, const void* x, const void* router_w,
                     const float* bias, float* logits, int32_t* idx, float* gate, int32_t* block_counts,
                     void* scratch, int32_t* status, cudaStream_t st, const float* norm_rstd = nullptr,
                     const float* norm_gamma = nullptr);

}  // namespace axm
