// Fused router: fp32 logits, softmax, top-k (lowest index wins ties),
// renormalised gates and per-block expert counts.
//
// Stands in for top2_router_kernel of the reference engine
// (core/src/CUDA/kernel/moe_router.cu:27-111), generalised to any k and E and
// to fp32 router weights.  Everything after the logits follows that kernel's
// fp32 operation order exactly, because expert indices and gates have to come
// out bit-identical for identical logits:
//     m = max_e z_e;  p_e = expf(z_e - m);  s = sum_e p_e (ascending e);
//     p_e *= 1 / (s + 1e-9f);  k scans with strict '>' from e = 0;
//     gate_i = p_i / (sum of the selected p + 1e-9f).
// This file must be compiled without fast-math.
//
// Work split: the token range is cut into AXM_ROUTE_BLOCKS contiguous blocks,
// one CTA each.  The permute kernel uses the same split, so the per-block
// counts written here give it a stable placement without atomics on global
// memory.
#include "router.cuh"

namespace axm {

constexpr int kRouterThreads = 256;
constexpr int kTokSub = 64;   // tokens handled per pass inside a block
constexpr int kEC = 8;        // experts per register chunk
constexpr int kTB = 4;        // tokens whose loads are in flight together
constexpr int kMaxK = kRouteMaxK;

__host__ __device__ inline int route_block_begin(int b, int T) {
  return (int)(((long long)b * T) / AXM_ROUTE_BLOCKS);
}

template <typename WT>
__device__ __forceinline__ float load_w(const WT* p);
template <>
__device__ __forceinline__ float load_w<float>(const float* p) {
  return __ldg(p);
}
template <>
__device__ __forceinline__ float load_w<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}

// ---- tensor-core logits for many experts --------------------------------------------
// For E >= 16 the CUDA-core path above spends ~100 instructions per (token, 8 experts,
// warp); mma.sync does the same GEMV-batch as a small GEMM.  x is bf16 already; an fp32
// router weight is split exactly into three bf16 terms (hi + mid + lo carry its 24
// mantissa bits), so three m16n8k16 MMAs with fp32 accumulation reproduce the fp32
// product sum to accumulation-order noise.  Warp w reduces over its eighth of d for all
// tokens of the sub-block and 32 experts at a time; the eight partial sums are added in
// warp order (deterministic).
constexpr int kMmaNC = 4;                 // n-tiles (of 8 experts) per pass
constexpr int kMmaPartE = 8 * kMmaNC;     // experts per pass

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename WT>
__device__ __forceinline__ void split_pair(const WT* p0, const WT* p1, bool ok0, bool ok1, uint32_t (&out)[3]);
template <>
__device__ __forceinline__ void split_pair<float>(const float* p0, const float* p1, bool ok0, bool ok1,
                                                  uint32_t (&out)[3]) {
  float w0 = ok0 ? __ldg(p0) : 0.0f, w1 = ok1 ? __ldg(p1) : 0.0f;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    __nv_bfloat16 h0 = __float2bfloat16_rn(w0), h1 = __float2bfloat16_rn(w1);
    out[i] = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
    w0 -= __bfloat162float(h0);
    w1 -= __bfloat162float(h1);
  }
}
template <>
__device__ __forceinline__ void split_pair<__nv_bfloat16>(const __nv_bfloat16* p0, const __nv_bfloat16* p1,
                                                          bool ok0, bool ok1, uint32_t (&out)[3]) {
  uint32_t h0 = ok0 ? (uint32_t)__bfloat16_as_ushort(*p0) : 0u, h1 = ok1 ? (uint32_t)__bfloat16_as_ushort(*p1) : 0u;
  out[0] = h0 | (h1 << 16);
  out[1] = out[2] = 0u;
}

// z_s[tt][e] (zeroed by the caller) += sum_d x[ts + tt][d] * wr[d][e] for tt < nt.
template <typename WT>
__device__ __forceinline__ void logits_mma(const __nv_bfloat16* __restrict__ x, const WT* __restrict__ wr,
                                           float* z_s, float* part_s, int ts, int nt, int D, int E, int EP) {
  constexpr int kTerms = sizeof(WT) == 4 ? 3 : 1;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int slice = ((D + 7) / 8 + 15) / 16 * 16;  // d per warp, a multiple of 16
  const int k_begin = warp * slice, k_end = min(D, k_begin + slice);
  for (int e0 = 0; e0 < E; e0 += kMmaPartE) {
    float acc[4][kMmaNC][4];
#pragma unroll
    for (int m = 0; m < 4; ++m)
#pragma unroll
      for (int n = 0; n < kMmaNC; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[m][n][i] = 0.0f;
    for (int k0 = k_begin; k0 < k_end; k0 += 16) {
      uint32_t a[4][4];
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const int r0 = m * 16 + g, r1 = r0 + 8;
        const int ka = k0 + 2 * tq, kb = ka + 8;
        const uint32_t* p0 = reinterpret_cast<const uint32_t*>(x + (size_t)(ts + r0) * D);
        const uint32_t* p1 = reinterpret_cast<const uint32_t*>(x + (size_t)(ts + r1) * D);
        a[m][0] = (r0 < nt && ka < D) ? __ldg(p0 + (ka >> 1)) : 0u;
        a[m][1] = (r1 < nt && ka < D) ? __ldg(p1 + (ka >> 1)) : 0u;
        a[m][2] = (r0 < nt && kb < D) ? __ldg(p0 + (kb >> 1)) : 0u;
        a[m][3] = (r1 < nt && kb < D) ? __ldg(p1 + (kb >> 1)) : 0u;
      }
#pragma unroll
      for (int n = 0; n < kMmaNC; ++n) {
        const int e = e0 + n * 8 + g;
        const bool e_ok = e < E;
        const int ka = k0 + 2 * tq, kb = ka + 8;
        uint32_t b0[3], b1[3];
        split_pair<WT>(wr + (size_t)ka * E + e, wr + (size_t)(ka + 1) * E + e, e_ok && ka < D, e_ok && ka + 1 < D, b0);
        split_pair<WT>(wr + (size_t)kb * E + e, wr + (size_t)(kb + 1) * E + e, e_ok && kb < D, e_ok && kb + 1 < D, b1);
#pragma unroll
        for (int i = 0; i < kTerms; ++i)
#pragma unroll
          for (int m = 0; m < 4; ++m) mma_bf16_16816(acc[m][n], a[m], b0[i], b1[i]);
      }
    }
    // C fragment: c0,c1 -> row g, experts 2tq, 2tq+1; c2,c3 -> row g + 8
#pragma unroll
    for (int m = 0; m < 4; ++m)
#pragma unroll
      for (int n = 0; n < kMmaNC; ++n) {
        float* p = part_s + ((size_t)warp * kTokSub + m * 16 + g) * kMmaPartE + n * 8 + 2 * tq;
        p[0] = acc[m][n][0];
        p[1] = acc[m][n][1];
        p[8 * kMmaPartE] = acc[m][n][2];
        p[8 * kMmaPartE + 1] = acc[m][n][3];
      }
    __syncthreads();
    for (int i = tid; i < nt * kMmaPartE; i += kRouterThreads) {
      const int tt = i / kMmaPartE, e = i - tt * kMmaPartE;
      if (e0 + e < E) {
        float sum = 0.0f;
#pragma unroll
        for (int wv = 0; wv < 8; ++wv) sum += part_s[((size_t)wv * kTokSub + tt) * kMmaPartE + e];
        z_s[tt * EP + e0 + e] = sum;
      }
    }
    __syncthreads();
  }
}

// kFromLogits: skip the GEMV and read z from `logits_in`.
template <typename WT, bool kFromLogits, bool kMma>
__global__ void __launch_bounds__(kRouterThreads, kMma ? 1 : 2)
router_kernel(const __nv_bfloat16* __restrict__ x, const WT* __restrict__ wr,
              const float* __restrict__ bias, const float* __restrict__ logits_in,
              float* __restrict__ logits_out, int32_t* __restrict__ topk_idx,
              float* __restrict__ topk_gate, int32_t* __restrict__ block_counts, int T, int D,
              int E, int k) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int EP = E + 1;  // padded row, so that threads walking rows hit distinct banks
  float* z_s = reinterpret_cast<float*>(smem_raw);                 // [kTokSub][EP]
  constexpr int kPartE = kMma ? kMmaPartE : kEC;
  float* part_s = z_s + kTokSub * EP;                              // [8 warps][kTokSub][kPartE]
  int* hist_s = reinterpret_cast<int*>(part_s + 8 * kTokSub * kPartE);  // [E]

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int t_begin = route_block_begin(blockIdx.x, T);
  const int t_end = route_block_begin(blockIdx.x + 1, T);

  for (int e = tid; e < E; e += kRouterThreads) hist_s[e] = 0;
  __syncthreads();

  for (int ts = t_begin; ts < t_end; ts += kTokSub) {
    const int nt = min(kTokSub, t_end - ts);

    if constexpr (kFromLogits) {
      for (int i = tid; i < nt * E; i += kRouterThreads) {
        int tt = i / E, e = i - tt * E;
        z_s[tt * EP + e] = logits_in[(size_t)(ts + tt) * E + e];
      }
    } else {
      for (int i = tid; i < nt * EP; i += kRouterThreads) z_s[i] = 0.0f;
      __syncthreads();
      if constexpr (kMma) {
        logits_mma<WT>(x, wr, z_s, part_s, ts, nt, D, E, EP);
      } else {
      // Each thread owns four pairs of consecutive d in every 2048-wide slab
      // (d0 + 512*j + 2*tid + {0,1}) and keeps the matching 8 x kEC weights in
      // registers while it walks the tokens.  With that interleaving a warp's
      // weight loads and its 4-byte activation loads are both contiguous.
      for (int e0 = 0; e0 < E; e0 += kEC) {
        for (int d0 = 0; d0 < D; d0 += kRouterThreads * 8) {
          float w[8][kEC];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int d = d0 + 512 * j + 2 * tid;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              float* wrow = w[2 * j + i];
#pragma unroll
              for (int e = 0; e < kEC; ++e) wrow[e] = 0.0f;
              if (d + i < D) {
                const WT* rowp = wr + (size_t)(d + i) * E + e0;
                if (sizeof(WT) == 4 && (E & 3) == 0) {
#pragma unroll
                  for (int hq = 0; hq < 2; ++hq)
                    if (e0 + 4 * hq < E) {
                      float4 v = __ldg(reinterpret_cast<const float4*>(rowp) + hq);
                      wrow[4 * hq + 0] = v.x;
                      wrow[4 * hq + 1] = v.y;
                      wrow[4 * hq + 2] = v.z;
                      wrow[4 * hq + 3] = v.w;
                    }
                } else if (sizeof(WT) == 2 && (E & 7) == 0) {
                  uint4 v = __ldg(reinterpret_cast<const uint4*>(rowp));
                  wrow[0] = bf16_lo(v.x);
                  wrow[1] = bf16_hi(v.x);
                  wrow[2] = bf16_lo(v.y);
                  wrow[3] = bf16_hi(v.y);
                  wrow[4] = bf16_lo(v.z);
                  wrow[5] = bf16_hi(v.z);
                  wrow[6] = bf16_lo(v.w);
                  wrow[7] = bf16_hi(v.w);
                } else {
#pragma unroll
                  for (int e = 0; e < kEC; ++e)
                    if (e0 + e < E) wrow[e] = load_w<WT>(rowp + e);
                }
              }
            }
          }
          // Tokens go through in batches of kTB, software-pipelined: the loads of batch
          // i + 1 are issued before batch i is worked on, so 4 * kTB loads per thread are
          // always in flight and their latency hides behind the arithmetic.
          uint32_t xn[kTB][4];
          auto load_batch = [&](int tb) {
#pragma unroll
            for (int b = 0; b < kTB; ++b)
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int d = d0 + 512 * j + 2 * tid;
                xn[b][j] = 0u;
                if (d < D && tb + b < nt)
                  xn[b][j] = __ldg(reinterpret_cast<const uint32_t*>(x + (size_t)(ts + tb + b) * D + d));
              }
          };
          load_batch(0);
          for (int tb = 0; tb < nt; tb += kTB) {
            uint32_t xv[kTB][4];
#pragma unroll
            for (int b = 0; b < kTB; ++b)
#pragma unroll
              for (int j = 0; j < 4; ++j) xv[b][j] = xn[b][j];
            load_batch(tb + kTB);
#pragma unroll
            for (int b = 0; b < kTB; ++b) {
              const int tt = tb + b;
              float xf[8] = {bf16_lo(xv[b][0]), bf16_hi(xv[b][0]), bf16_lo(xv[b][1]), bf16_hi(xv[b][1]),
                             bf16_lo(xv[b][2]), bf16_hi(xv[b][2]), bf16_lo(xv[b][3]), bf16_hi(xv[b][3])};
              float acc[kEC];
#pragma unroll
              for (int e = 0; e < kEC; ++e) acc[e] = 0.0f;
#pragma unroll
              for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < kEC; ++e) acc[e] = fmaf(xf[j], w[j][e], acc[e]);
              // Transposed butterfly: 8 values on 32 lanes -> one value per lane after
              // three exchange steps, then two plain steps.  Fixed tree, so the sum
              // order (and the logits) are reproducible.
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                bool up = lane & 16;
                float send = up ? acc[i] : acc[i + 4];
                float keep = up ? acc[i + 4] : acc[i];
                acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
              }
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                bool up = lane & 8;
                float send = up ? acc[i] : acc[i + 2];
                float keep = up ? acc[i + 2] : acc[i];
                acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
              }
              {
                bool up = lane & 4;
                float send = up ? acc[0] : acc[1];
                float keep = up ? acc[1] : acc[0];
                acc[0] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
              }
              acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 2);
              acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 1);
              if ((lane & 3) == 0 && tt < nt) {
                int e = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
                part_s[(warp * kTokSub + tt) * kEC + e] = acc[0];
              }
            }
          }
          __syncthreads();
          for (int i = tid; i < nt * kEC; i += kRouterThreads) {
            int tt = i / kEC, e = i - tt * kEC;
            if (e0 + e < E) {
              float sum = z_s[tt * EP + e0 + e];
#pragma unroll
              for (int wv = 0; wv < 8; ++wv) sum += part_s[(wv * kTokSub + tt) * kEC + e];
              z_s[tt * EP + e0 + e] = sum;
            }
          }
          __syncthreads();
        }
      }
      }
      if (bias != nullptr)
        for (int i = tid; i < nt * E; i += kRouterThreads) {
          int tt = i / E, e = i - tt * E;
          z_s[tt * EP + e] += bias[e];
        }
    }
    __syncthreads();
    if (logits_out != nullptr)
      for (int i = tid; i < nt * E; i += kRouterThreads) {
        int tt = i / E, e = i - tt * E;
        logits_out[(size_t)(ts + tt) * E + e] = z_s[tt * EP + e];
      }
    __syncthreads();
    if (tid < nt) {
      int t = ts + tid;
      route_one_token<kMaxK>(z_s + tid * EP, E, k, topk_idx + (size_t)t * k,
                             topk_gate + (size_t)t * k, hist_s);
    }
    __syncthreads();
  }
  for (int e = tid; e < E; e += kRouterThreads)
    block_counts[(size_t)blockIdx.x * E + e] = hist_s[e];
}

static size_t router_smem_bytes(int E, bool mma = false) {
  return sizeof(float) * ((size_t)kTokSub * (E + 1) + 8 * kTokSub * (mma ? kMmaPartE : kEC)) +
         sizeof(int) * (size_t)E;
}

// The tensor-core logits pay off from 32 experts on (multiples of 8): measured 94 vs 207 us at
// E = 64 (T 16384, D 2048), but 46 vs 35 us at E = 16.
static bool router_use_mma(int E) { return E >= 32 && E % 8 == 0; }

template <typename WT>
static int launch_router(bool mma, size_t smem, cudaStream_t st, const __nv_bfloat16* x, const WT* w,
                          const float* bias, float* logits, int32_t* idx, float* gate, int32_t* bc,
                          const AxmMoeDesc* d) {
  if (mma) {
    auto kern = router_kernel<WT, false, true>;
    static SmemLimitCache cache = {};
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem, &cache, "router_kernel")) return rc;
    kern<<<AXM_ROUTE_BLOCKS, kRouterThreads, smem, st>>>(x, w, bias, nullptr, logits, idx, gate, bc,
                                                         d->tokens, d->d_model, d->num_experts, d->top_k);
  } else {
    auto kern = router_kernel<WT, false, false>;
    static SmemLimitCache cache = {};
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem, &cache, "router_kernel")) return rc;
    kern<<<AXM_ROUTE_BLOCKS, kRouterThreads, smem, st>>>(x, w, bias, nullptr, logits, idx, gate, bc,
                                                         d->tokens, d->d_model, d->num_experts, d->top_k);
  }
  return check_launch("router_kernel");
}

int validate_route(const AxmMoeDesc* d) {
  if (d == nullptr) return fail(AXM_ERR_ARGUMENT, "desc is null");
  if (d->tokens < 0 || d->d_model <= 0 || d->num_experts <= 0 || d->top_k <= 0)
    return fail(AXM_ERR_ARGUMENT, "tokens/d_model/num_experts/top_k must be positive");
  if (d->num_experts > 256) return fail(AXM_ERR_ARGUMENT, "num_experts %d > 256", d->num_experts);
  if (d->top_k > kMaxK || d->top_k > d->num_experts)
    return fail(AXM_ERR_ARGUMENT, "top_k %d must be <= min(num_experts, %d)", d->top_k, kMaxK);
  if (d->d_model % 8 != 0) return fail(AXM_ERR_ARGUMENT, "d_model %d not a multiple of 8", d->d_model);
  return AXM_OK;
}

}  // namespace axm

using namespace axm;

extern "C" int axm_moe_router(const AxmMoeDesc* desc, const void* x, const void* router_w,
                              const float* router_bias, float* logits, int32_t* topk_idx,
                              float* topk_gate, int32_t* block_counts, void* stream) {
  if (int rc = validate_route(desc)) return rc;
  if (!x || !router_w || !topk_idx || !topk_gate || !block_counts)
    return fail(AXM_ERR_ARGUMENT, "axm_moe_router: null pointer");
  if (int rc = require_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool mma = router_use_mma(desc->num_experts);
  size_t smem = router_smem_bytes(desc->num_experts, mma);
  const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
  if (desc->router_dtype == AXM_ROUTER_FP32)
    return launch_router<float>(mma, smem, st, xb, static_cast<const float*>(router_w), router_bias, logits,
                                topk_idx, topk_gate, block_counts, desc);
  if (desc->router_dtype == AXM_ROUTER_BF16)
    return launch_router<__nv_bfloat16>(mma, smem, st, xb, static_cast<const __nv_bfloat16*>(router_w),
                                        router_bias, logits, topk_idx, topk_gate, block_counts, desc);
  return fail(AXM_ERR_ARGUMENT, "router_dtype %d unknown", desc->router_dtype);
}

extern "C" int axm_moe_router_scratch_bytes(const AxmMoeDesc* desc, size_t* bytes) {
  if (int rc = validate_route(desc)) return rc;
  if (bytes == nullptr) return fail(AXM_ERR_ARGUMENT, "bytes is null");
  if (desc->router_dtype != AXM_ROUTER_FP32 && desc->router_dtype != AXM_ROUTER_BF16)
    return fail(AXM_ERR_ARGUMENT, "router_dtype %d unknown", desc->router_dtype);
  const RouterTcPlan p = router_tc_plan(desc);
  *bytes = p.ok ? p.scratch_bytes : 0;
  return AXM_OK;
}

namespace axm {
int launch_router_auto(const AxmMoeDesc* desc, const void* x, const void* router_w, const float* router_bias,
                       float* logits, int32_t* topk_idx, float* topk_gate, int32_t* block_counts,
                       void* scratch, size_t scratch_bytes, int32_t* status, void* stream, bool* used_tc) {
  if (used_tc) *used_tc = false;
  if (int rc = validate_route(desc)) return rc;
  if (!x || !router_w || !topk_idx || !topk_gate || !block_counts)
    return fail(AXM_ERR_ARGUMENT, "axm_moe_router_ws: null pointer");
  if (desc->router_dtype != AXM_ROUTER_FP32 && desc->router_dtype != AXM_ROUTER_BF16)
    return fail(AXM_ERR_ARGUMENT, "router_dtype %d unknown", desc->router_dtype);
  const RouterTcPlan p = router_tc_plan(desc);
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(scratch)) & 15) == 0;
  if (!p.ok || scratch == nullptr || scratch_bytes < p.scratch_bytes || !aligned || desc->tokens == 0)
    return axm_moe_router(desc, x, router_w, router_bias, logits, topk_idx, topk_gate, block_counts, stream);
  if (int rc = require_device()) return rc;
  if (used_tc) *used_tc = true;
  return launch_router_tc(desc, p, x, router_w, router_bias, logits, topk_idx, topk_gate, block_counts,
                          scratch, status, static_cast<cudaStream_t>(stream));
}
}  // namespace axm

extern "C" int axm_moe_router_ws(const AxmMoeDesc* desc, const void* x, const void* router_w,
                                 const float* router_bias, float* logits, int32_t* topk_idx,
                                 float* topk_gate, int32_t* block_counts, void* scratch,
                                 size_t scratch_bytes, int32_t* status, void* stream) {
  return launch_router_auto(desc, x, router_w, router_bias, logits, topk_idx, topk_gate, block_counts, scratch,
                            scratch_bytes, status, stream, nullptr);
}

extern "C" int axm_moe_route_from_logits(const AxmMoeDesc* desc, const float* logits,
                                         int32_t* topk_idx, float* topk_gate,
                                         int32_t* block_counts, void* stream) {
  if (int rc = validate_route(desc)) return rc;
  if (!logits || !topk_idx || !topk_gate || !block_counts)
    return fail(AXM_ERR_ARGUMENT, "axm_moe_route_from_logits: null pointer");
  if (int rc = require_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  size_t smem = router_smem_bytes(desc->num_experts);
  auto kern = router_kernel<float, true, false>;
  static SmemLimitCache cache = {};
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem, &cache, "router_kernel(from logits)"))
    return rc;
  kern<<<AXM_ROUTE_BLOCKS, kRouterThreads, smem, st>>>(nullptr, nullptr, nullptr, logits, nullptr,
                                                       topk_idx, topk_gate, block_counts,
                                                       desc->tokens, desc->d_model,
                                                       desc->num_experts, desc->top_k);
  return check_launch("router_kernel(from logits)");
}
