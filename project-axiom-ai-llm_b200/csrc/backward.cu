// Training step of the MoE layer: forward pass that keeps what the backward pass
// needs, Switch-style load-balancing loss, and the backward pass (upstream
// gradient -> dX, router and expert weight gradients).
//
// The reference engine has neither (its MoE branch is forward only and its backward
// pass handles the dense FFN, core/src/CUDA/kernel/backward_pass.cu:1701-2005; an
// auxiliary loss is listed as future work in document/AI_CONTEXT.md:217).  The maths
// follows the layer's forward conventions (core/src/CUDA/kernel/moe_router.cu:59-105
// for softmax / gates) and the engine's dense-backward conventions: fp32 weight
// gradients in the weights' layout (backward_pass.cu:1013-1048) and the SiLU*mul
// derivative of core/src/CUDA/kernel/swiglu.cu:34-55.  Unlike the dense backward no
// gradient is clamped and bf16 weights (not fp32 masters) feed the input gradients.
//
//   L = sum(dOut * out) + aux,  out = x + y,  aux = alpha * E * sum_e f_e * P_e,
//   f_e = count_e / (T k) (constant), P_e = mean_t p[t, e].
#include "router.cuh"

namespace axm {

__host__ __device__ inline int train_block_begin(int b, int T) {
  return (int)(((long long)b * T) / AXM_ROUTE_BLOCKS);
}

// p = softmax(z) with the forward pass's operation order; returns the row maximum's sum etc. in place.
__device__ __forceinline__ void softmax_row(const float* __restrict__ z, float* p, int E) {
  float m = z[0];
  for (int e = 1; e < E; ++e) m = z[e] > m ? z[e] : m;
  float s = 0.0f;
  for (int e = 0; e < E; ++e) {
    p[e] = expf(z[e] - m);
    s += p[e];
  }
  const float inv = 1.0f / (s + 1e-9f);
  for (int e = 0; e < E; ++e) p[e] *= inv;
}

// Stage 1 of the auxiliary loss: per token block, column sums of the probabilities.
// One thread per token keeps its row in shared memory; fixed summation order.
constexpr int kAuxThreads = 128;
__global__ void __launch_bounds__(kAuxThreads)
aux_partial_kernel(const float* __restrict__ logits, float* __restrict__ partial, int T, int E) {
  extern __shared__ float sm[];  // [kAuxThreads][E + 1]
  const int EP = E + 1;
  const int t0 = train_block_begin(blockIdx.x, T), t1 = train_block_begin(blockIdx.x + 1, T);
  float* mine = sm + threadIdx.x * EP;
  for (int e = threadIdx.x; e < E; e += kAuxThreads) partial[(size_t)blockIdx.x * E + e] = 0.0f;
  __syncthreads();
  for (int ts = t0; ts < t1; ts += kAuxThreads) {
    const int t = ts + threadIdx.x;
    if (t < t1) softmax_row(logits + (size_t)t * E, mine, E);
    __syncthreads();
    const int nt = min(kAuxThreads, t1 - ts);
    for (int e = threadIdx.x; e < E; e += kAuxThreads) {
      float acc = partial[(size_t)blockIdx.x * E + e];
      for (int i = 0; i < nt; ++i) acc += sm[i * EP + e];
      partial[(size_t)blockIdx.x * E + e] = acc;
    }
    __syncthreads();
  }
}

// Stage 2: P_e, f_e, the loss, and the per-expert constant alpha * E * f_e / T that the
// router backward adds to every dp[t, e].
__global__ void aux_final_kernel(const float* __restrict__ partial, const int32_t* __restrict__ counts,
                                 float* __restrict__ aux_coef, float* __restrict__ aux_loss, int T,
                                 int E, int k, float alpha) {
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

// One warp per permuted row r: the gate-scaled upstream gradient row (bf16, zero for
// padding rows) and the gate gradient dgate[slot] = <dOut[t], o[r]>.
__global__ void __launch_bounds__(256)
bwd_prepare_kernel(const float* __restrict__ d_out, const float* __restrict__ o,
                   const int32_t* __restrict__ row_src, const float* __restrict__ gate,
                   const int32_t* __restrict__ offsets, __nv_bfloat16* __restrict__ d_o,
                   float* __restrict__ d_gate, int D, int E, int k) {
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (blockDim.x >> 5);
  const int rows = offsets[E];
  for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
    const int slot = row_src[r];
    uint2* dst = reinterpret_cast<uint2*>(d_o + (size_t)r * D);
    if (slot < 0) {
      for (int c = lane; c < D / 4; c += 32) dst[c] = make_uint2(0u, 0u);
      continue;
    }
    const int t = slot / k;
    const float w = gate[slot];
    const float4* dy = reinterpret_cast<const float4*>(d_out + (size_t)t * D);
    const float4* orow = reinterpret_cast<const float4*>(o + (size_t)r * D);
    float dot = 0.0f;
    for (int c = lane; c < D / 4; c += 32) {
      const float4 a = __ldg(dy + c), b = __ldg(orow + c);
      dot = fmaf(a.x, b.x, dot);
      dot = fmaf(a.y, b.y, dot);
      dot = fmaf(a.z, b.z, dot);
      dot = fmaf(a.w, b.w, dot);
      dst[c] = make_uint2(pack_bf16(w * a.x, w * a.y), pack_bf16(w * a.z, w * a.w));
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
    if (lane == 0) d_gate[slot] = dot;
  }
}

// One thread per token: gate gradients -> probability gradients (through the
// renormalisation over the selected experts, plus the auxiliary-loss term) ->
// logit gradients through the softmax.  dz[t, e] = p_e * (dp_e - sum_j p_j dp_j).
constexpr int kRbThreads = 128;  // at most; fewer when E rows of p and dp per thread would not fit
// Threads per block such that blockDim * 2 * (E + 1) floats fit in 200 KB of shared memory
// (E = 256: 96 threads), a multiple of a warp.
static int router_bwd_threads(int E) {
  int t = (int)((200u * 1024u) / (8u * (unsigned)(E + 1)));
  t = t > kRbThreads ? kRbThreads : t;
  return t / 32 * 32;
}
__global__ void __launch_bounds__(kRbThreads)
router_bwd_kernel(const float* __restrict__ logits, const int32_t* __restrict__ topk_idx,
                  const float* __restrict__ d_gate, const float* __restrict__ aux_coef,
                  float* __restrict__ dz, int T, int E, int k) {
  extern __shared__ float sm[];  // [blockDim.x][2][E + 1]
  const int EP = E + 1;
  float* p = sm + threadIdx.x * 2 * EP;
  float* dp = p + EP;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  softmax_row(logits + (size_t)t * E, p, E);
  float sel = 0.0f, dot = 0.0f;
  for (int i = 0; i < k; ++i) sel += p[topk_idx[(size_t)t * k + i]];
  const float denom = sel + 1e-9f;
  for (int i = 0; i < k; ++i) dot += d_gate[(size_t)t * k + i] * p[topk_idx[(size_t)t * k + i]];
  for (int e = 0; e < E; ++e) dp[e] = aux_coef[e];
  for (int i = 0; i < k; ++i)
    dp[topk_idx[(size_t)t * k + i]] += d_gate[(size_t)t * k + i] / denom - dot / (denom * denom);
  float pd = 0.0f;
  for (int e = 0; e < E; ++e) pd += p[e] * dp[e];
  for (int e = 0; e < E; ++e) dz[(size_t)t * E + e] = p[e] * (dp[e] - pd);
}

// Gradient of the router bias: d_bias[e] = sum_t dz[t, e] (the bias is added to the logits).
// Two passes with a fixed order: kBiasChunks blocks sum their token ranges, one block adds the
// partial sums in chunk order.  Deterministic.
constexpr int kBiasChunks = 64;
__global__ void __launch_bounds__(256)
dbias_partial_kernel(const float* __restrict__ dz, float* __restrict__ partial, int T, int E) {
  const int c = blockIdx.x;
  const int t0 = (int)(((long long)c * T) / kBiasChunks), t1 = (int)(((long long)(c + 1) * T) / kBiasChunks);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float acc = 0.0f;
    for (int t = t0; t < t1; ++t) acc += dz[(size_t)t * E + e];
    partial[(size_t)c * E + e] = acc;
  }
}
__global__ void __launch_bounds__(256)
dbias_reduce_kernel(const float* __restrict__ partial, float* __restrict__ d_bias, int E) {
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float acc = 0.0f;
    for (int c = 0; c < kBiasChunks; ++c) acc += partial[(size_t)c * E + e];
    d_bias[e] = acc;
  }
}

// dWr[d, e] = sum_t x[t, d] * dz[t, e].  grid (ceil(D / 256), chunks): a thread sums its chunk of
// tokens in order; dwr_reduce adds the chunks in order.  Deterministic.
constexpr int kDwrChunks = 128;
// A thread owns two adjacent d (one 4-byte load per token, a warp reads 128 contiguous bytes of the
// row) and EC experts; eight tokens per trip keep eight loads in flight.  The partial sums are laid
// out [chunk][e][d], so that neighbouring threads write neighbouring words.
template <int EC>
__global__ void __launch_bounds__(128)
dwr_partial_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ dz,
                   float* __restrict__ partial, int T, int D, int E) {
  const int d = (blockIdx.x * 128 + threadIdx.x) * 2;
  const int c = blockIdx.y;
  const int chunks = gridDim.y;  // at most kDwrChunks
  const int t0 = (int)(((long long)c * T) / chunks), t1 = (int)(((long long)(c + 1) * T) / chunks);
  if (d >= D) return;  // D is a multiple of 8: a thread's two columns are both inside or both outside
  for (int e0 = 0; e0 < E; e0 += EC) {
    float acc0[EC], acc1[EC];
#pragma unroll
    for (int j = 0; j < EC; ++j) acc0[j] = acc1[j] = 0.0f;
    const bool vec = (E & 3) == 0 && e0 + EC <= E;
    int t = t0;
    for (; t + 7 < t1; t += 8) {
      uint32_t xv[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) xv[q] = __ldg(reinterpret_cast<const uint32_t*>(x + (size_t)(t + q) * D + d));
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float x0 = bf16_lo(xv[q]), x1 = bf16_hi(xv[q]);
        const float* z = dz + (size_t)(t + q) * E + e0;
        if (vec) {
#pragma unroll
          for (int j4 = 0; j4 < EC / 4; ++j4) {
            const float4 zz = __ldg(reinterpret_cast<const float4*>(z) + j4);
            const float zv[4] = {zz.x, zz.y, zz.z, zz.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              acc0[4 * j4 + i] = fmaf(x0, zv[i], acc0[4 * j4 + i]);
              acc1[4 * j4 + i] = fmaf(x1, zv[i], acc1[4 * j4 + i]);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < EC; ++j)
            if (e0 + j < E) {
              const float zv = __ldg(z + j);
              acc0[j] = fmaf(x0, zv, acc0[j]);
              acc1[j] = fmaf(x1, zv, acc1[j]);
            }
        }
      }
    }
    for (; t < t1; ++t) {
      const uint32_t xv = __ldg(reinterpret_cast<const uint32_t*>(x + (size_t)t * D + d));
      const float x0 = bf16_lo(xv), x1 = bf16_hi(xv);
      const float* z = dz + (size_t)t * E + e0;
#pragma unroll
      for (int j = 0; j < EC; ++j)
        if (e0 + j < E) {
          const float zv = __ldg(z + j);
          acc0[j] = fmaf(x0, zv, acc0[j]);
          acc1[j] = fmaf(x1, zv, acc1[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < EC; ++j)
      if (e0 + j < E)
        *reinterpret_cast<float2*>(partial + ((size_t)c * E + e0 + j) * D + d) = make_float2(acc0[j], acc1[j]);
  }
}

// d_wr[d][e] = sum over the chunks, in chunk order, of partial[chunk][e][d].
__global__ void dwr_reduce_kernel(const float* __restrict__ partial, float* __restrict__ d_wr, int D, int E,
                                  int chunks) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= D * E) return;
  const int e = i / D, d = i - e * D;
  float acc = 0.0f;
#pragma unroll 16
  for (int c = 0; c < chunks; ++c) acc += __ldg(partial + ((size_t)c * E + e) * D + d);  // loads ahead, adds in order
  d_wr[(size_t)d * E + e] = acc;
}

// dX[t, d] = dOut[t, d] (residual) + sum_i dXp[slot_dst[t, i], d] + sum_e Wr[d, e] * dz[t, e].
// grid (D / d_tile, token chunks); a thread owns 4 consecutive d and works on four tokens
// at a time, so that their gathers are in flight together and one shared-memory read of
// the router weights serves four tokens.  The block's slice of the router weights sits in
// shared memory as [E][d_tile] (conflict-free float4 reads); dz[t, :] is the same address
// for the whole block (broadcast).
constexpr int kFinTokens = 4;

// ER > 0: E == ER and the thread keeps its 4 x ER router weights in registers (no shared memory);
// ER == 0: any E, the block's weight slice sits in shared memory.
template <typename WT, int ER>
__global__ void __launch_bounds__(128)
bwd_finalize_kernel(const float* __restrict__ d_out, const float* __restrict__ d_xp,
                    const int32_t* __restrict__ slot_dst, const WT* __restrict__ wr,
                    const float* __restrict__ dz, float* __restrict__ d_x, int T, int D, int E, int k,
                    int residual, int d_tile, int S, const float* __restrict__ d_xp_shared, int shared_stride) {
  extern __shared__ __align__(16) float w_s[];  // [E][d_tile] (ER == 0)
  const int d0 = blockIdx.x * d_tile;
  if (ER == 0) {
    // a warp fills 32 consecutive d of one expert: no bank conflicts; the strided reads of
    // Wr stay in L1/L2 (the slice is E * d_tile elements)
    for (int i = threadIdx.x; i < E * d_tile; i += blockDim.x) {
      const int e = i / d_tile, dd = i - e * d_tile;
      w_s[i] = d0 + dd < D ? (float)wr[(size_t)(d0 + dd) * E + e] : 0.0f;
    }
    __syncthreads();
  }
  const int dl = threadIdx.x * 4;
  if (dl >= d_tile || d0 + dl >= D) return;
  float4 w_r[ER > 0 ? ER : 1];
  if (ER > 0) {  // D is a multiple of 8: the thread's four d are all inside
#pragma unroll
    for (int e = 0; e < ER; ++e) {
      const WT* row = wr + (size_t)(d0 + dl) * ER + e;
      w_r[e] = make_float4((float)row[0], (float)row[ER], (float)row[2 * ER], (float)row[3 * ER]);
    }
  }
  const int c = (d0 + dl) / 4;
  const int t0 = (int)(((long long)blockIdx.y * T) / gridDim.y);
  const int t1 = (int)(((long long)(blockIdx.y + 1) * T) / gridDim.y);
  for (int t = t0; t < t1; t += kFinTokens) {
    float4 acc[kFinTokens], rt[kFinTokens];
    int tq[kFinTokens];
#pragma unroll
    for (int q = 0; q < kFinTokens; ++q) {
      tq[q] = min(t + q, t1 - 1);  // a short last group repeats its last token; stores are masked
      acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
      rt[q] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (residual) acc[q] = __ldg(reinterpret_cast<const float4*>(d_out + (size_t)tq[q] * D) + c);
    }
    for (int i = 0; i < k; ++i) {
      float4 v[kFinTokens];
#pragma unroll
      for (int q = 0; q < kFinTokens; ++q) {
        const int r = __ldg(slot_dst + (size_t)tq[q] * k + i);
        v[q] = __ldg(reinterpret_cast<const float4*>(d_xp + (size_t)r * D) + c);
      }
#pragma unroll
      for (int q = 0; q < kFinTokens; ++q) {
        acc[q].x += v[q].x;
        acc[q].y += v[q].y;
        acc[q].z += v[q].z;
        acc[q].w += v[q].w;
      }
    }
    for (int s = 0; s < S; ++s) {  // shared experts: row s * shared_stride + t of d_xp_shared
      float4 v[kFinTokens];
#pragma unroll
      for (int q = 0; q < kFinTokens; ++q)
        v[q] = __ldg(reinterpret_cast<const float4*>(d_xp_shared + ((size_t)s * shared_stride + tq[q]) * D) + c);
#pragma unroll
      for (int q = 0; q < kFinTokens; ++q) {
        acc[q].x += v[q].x;
        acc[q].y += v[q].y;
        acc[q].z += v[q].z;
        acc[q].w += v[q].w;
      }
    }
    auto add_e = [&](int e, int q, float zv) {
      const float4 wv = ER > 0 ? w_r[e] : *reinterpret_cast<const float4*>(w_s + e * d_tile + dl);
      rt[q].x = fmaf(wv.x, zv, rt[q].x);
      rt[q].y = fmaf(wv.y, zv, rt[q].y);
      rt[q].z = fmaf(wv.z, zv, rt[q].z);
      rt[q].w = fmaf(wv.w, zv, rt[q].w);
    };
    if (ER > 0) {
#pragma unroll
      for (int e = 0; e < ER; e += 4) {
        float4 zz[kFinTokens];
#pragma unroll
        for (int q = 0; q < kFinTokens; ++q)
          zz[q] = __ldg(reinterpret_cast<const float4*>(dz + (size_t)tq[q] * ER + e));
#pragma unroll
        for (int q = 0; q < kFinTokens; ++q) {
          add_e(e, q, zz[q].x);
          add_e(e + 1, q, zz[q].y);
          add_e(e + 2, q, zz[q].z);
          add_e(e + 3, q, zz[q].w);
        }
      }
    } else if ((E & 3) == 0) {
      for (int e = 0; e < E; e += 4) {
        float4 zz[kFinTokens];
#pragma unroll
        for (int q = 0; q < kFinTokens; ++q)
          zz[q] = __ldg(reinterpret_cast<const float4*>(dz + (size_t)tq[q] * E + e));
#pragma unroll
        for (int q = 0; q < kFinTokens; ++q) {
          add_e(e, q, zz[q].x);
          add_e(e + 1, q, zz[q].y);
          add_e(e + 2, q, zz[q].z);
          add_e(e + 3, q, zz[q].w);
        }
      }
    } else {
      for (int e = 0; e < E; ++e)
#pragma unroll
        for (int q = 0; q < kFinTokens; ++q) add_e(e, q, __ldg(dz + (size_t)tq[q] * E + e));
    }
#pragma unroll
    for (int q = 0; q < kFinTokens; ++q) {
      if (t + q >= t1) break;
      acc[q].x += rt[q].x;
      acc[q].y += rt[q].y;
      acc[q].z += rt[q].z;
      acc[q].w += rt[q].w;
      reinterpret_cast<float4*>(d_x + (size_t)tq[q] * D)[c] = acc[q];
    }
  }
}

int launch_expert_ffn(const AxmMoeDesc* d, const void* x_perm, int32_t a_rows, const void* x_alt,
                      int32_t alt_rows, const AxmSegment* segments, int32_t num_segments,
                      const void* w_gate, const void* w_up, const void* w_down,
                      const void* shared_gate, const void* shared_up, const void* shared_down,
                      void* h, void* o, int32_t rows_total, int32_t* status, cudaStream_t st,
                      cudaEvent_t between, const AxmRemoteOut* remote, void* save_g, void* save_u);

// ---- pieces of the backward pass that run where the tokens live (shared with the
// expert-parallel training step, ep_train.cu) ------------------------------------------
size_t dwr_partial_floats(int D, int E) { return (size_t)kDwrChunks * D * E; }

int launch_aux_partial(const float* logits, float* partial, int T, int E, cudaStream_t st) {
  const size_t sm = sizeof(float) * kAuxThreads * (E + 1);
  static SmemLimitCache aux_cache = {};
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(aux_partial_kernel), sm, &aux_cache, "aux_partial_kernel"))
    return rc;
  aux_partial_kernel<<<AXM_ROUTE_BLOCKS, kAuxThreads, sm, st>>>(logits, partial, T, E);
  return check_launch("aux_partial_kernel");
}

static int finalize_tile(int E) { return E <= 64 ? 512 : 128; }

// Raises the dynamic shared-memory limits of router_bwd_kernel and bwd_finalize_kernel.
int bwd_source_limits(int E, int router_dtype) {
  const int rb_threads = router_bwd_threads(E);
  const size_t sm = sizeof(float) * (size_t)rb_threads * 2 * (E + 1);
  static SmemLimitCache rb_cache = {};
  int rc;
  if ((rc = ensure_dynamic_smem(reinterpret_cast<const void*>(router_bwd_kernel), sm, &rb_cache, "router_bwd_kernel")))
    return rc;
  if (E == 8 || E == 16) return AXM_OK;  // weights in registers: no dynamic shared memory
  const size_t fsm = sizeof(float) * (size_t)E * finalize_tile(E);
  static SmemLimitCache cache32 = {}, cache16 = {};
  if (router_dtype == AXM_ROUTER_FP32)
    return ensure_dynamic_smem(reinterpret_cast<const void*>(bwd_finalize_kernel<float, 0>), fsm, &cache32, "bwd_finalize_kernel");
  return ensure_dynamic_smem(reinterpret_cast<const void*>(bwd_finalize_kernel<__nv_bfloat16, 0>), fsm, &cache16, "bwd_finalize_kernel");
}

// d_o[r] = bf16(gate * dOut[token of r]) and d_gate[slot] = <dOut[t], o[r]> over the rows
// [0, offsets[E]) of the expert-contiguous order (row_src[r] < 0: zero row).
int launch_bwd_prepare(const float* d_out, const float* o, const int32_t* row_src, const float* gate,
                       const int32_t* offsets, void* d_o, float* d_gate, int D, int E, int k, cudaStream_t st) {
  bwd_prepare_kernel<<<4 * sm_count(), 256, 0, st>>>(d_out, o, row_src, gate, offsets,
                                                     static_cast<__nv_bfloat16*>(d_o), d_gate, D, E, k);
  return check_launch("bwd_prepare_kernel");
}

// Gate gradients -> logit gradients -> router bias / weight gradients -> dX, over desc->tokens
// tokens.  bias_partial holds at least [64][E] floats, dwr_partial dwr_partial_floats(D, E).
// bwd_source_limits must have succeeded for this E and router dtype.
int launch_bwd_source_tail(const AxmMoeDesc* desc, const AxmMoeTrain* t, const float* logits,
                           const int32_t* topk_idx, const float* d_gate, const float* aux_coef, float* dz,
                           float* bias_partial, float* dwr_partial, const float* d_xp, const int32_t* slot_dst,
                           cudaStream_t st, int S, const float* d_xp_shared, int shared_stride) {
  const int T = desc->tokens, D = desc->d_model, E = desc->num_experts, k = desc->top_k;
  const int residual = (desc->flags & AXM_FLAG_RESIDUAL) ? 1 : 0;
  const int rb_threads = router_bwd_threads(E);
  const size_t sm = sizeof(float) * (size_t)rb_threads * 2 * (E + 1);
  const int d_tile = finalize_tile(E);
  const size_t fsm = sizeof(float) * (size_t)E * d_tile;
  router_bwd_kernel<<<(T + rb_threads - 1) / rb_threads, rb_threads, sm, st>>>(logits, topk_idx, d_gate, aux_coef,
                                                                              dz, T, E, k);
  if (t->d_router_bias != nullptr) {
    dbias_partial_kernel<<<kBiasChunks, 256, 0, st>>>(dz, bias_partial, T, E);
    dbias_reduce_kernel<<<1, 256, 0, st>>>(bias_partial, t->d_router_bias, E);
  }
  if (t->d_router_w != nullptr) {
    // about 64 tokens per chunk, at most kDwrChunks chunks: a small batch (a rank's share under
    // expert parallelism) does not pay for 128 partial sums per element
    int chunks = T / 64;
    chunks = chunks < 8 ? 8 : (chunks > kDwrChunks ? kDwrChunks : chunks);
    dim3 grid((D / 2 + 127) / 128, chunks);
    dwr_partial_kernel<16><<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(t->x), dz, dwr_partial, T, D, E);
    dwr_reduce_kernel<<<(D * E + 63) / 64, 64, 0, st>>>(dwr_partial, t->d_router_w, D, E, chunks);  // many small blocks: the sums are latency-bound
  }
  dim3 fgrid((D + d_tile - 1) / d_tile, 1);
  const bool in_regs = E == 8 || E == 16;
  // one wave: as many blocks per SM as the weight slices fit (about 200 KB of shared memory);
  // with the weights in registers, what the register file holds
  int per_sm = in_regs ? 3 : (int)((200u * 1024u) / (fsm + 1024));
  per_sm = per_sm < 1 ? 1 : (per_sm > 12 ? 12 : per_sm);
  fgrid.y = (unsigned)((per_sm * sm_count() + fgrid.x - 1) / fgrid.x);
  if ((int)fgrid.y > T) fgrid.y = T;
  auto launch = [&](auto kern, const auto* wr_typed, size_t smem) {
    kern<<<fgrid, 128, smem, st>>>(t->d_out, d_xp, slot_dst, wr_typed, dz, t->d_x, T, D, E, k, residual, d_tile, S,
                                   d_xp_shared, shared_stride);
  };
  if (desc->router_dtype == AXM_ROUTER_FP32) {
    const float* w = static_cast<const float*>(t->router_w);
    if (E == 8) launch(bwd_finalize_kernel<float, 8>, w, 0);
    else if (E == 16) launch(bwd_finalize_kernel<float, 16>, w, 0);
    else launch(bwd_finalize_kernel<float, 0>, w, fsm);
  } else {
    const __nv_bfloat16* w = static_cast<const __nv_bfloat16*>(t->router_w);
    if (E == 8) launch(bwd_finalize_kernel<__nv_bfloat16, 8>, w, 0);
    else if (E == 16) launch(bwd_finalize_kernel<__nv_bfloat16, 16>, w, 0);
    else launch(bwd_finalize_kernel<__nv_bfloat16, 0>, w, fsm);
  }
  return check_launch("backward");
}

constexpr int kTrainAlign = 64;

int launch_combine_strided(const AxmMoeDesc* desc, const void* x, const void* o, const void* o_shared,
                           int shared_stride, const int32_t* slot_dst, const float* topk_gate, void* y, void* out,
                           cudaStream_t st);

// Shared experts in the training layout: every shared expert s gets its own copy of the token
// rows at rows [row0 + s * Tp, row0 + s * Tp + T) of x_perm, followed by zero rows up to Tp (a
// multiple of 64), and one ordinary segment {a_row0 = out_row0 = row0 + s * Tp, rows = Tp,
// expert = s} behind the routed experts' segments.  With that every backward kernel treats a
// shared expert like a routed one that received all tokens.
__global__ void __launch_bounds__(256)
train_shared_rows_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ x_perm,
                         AxmSegment* __restrict__ segments, int T, int Tp, int D, int E, int S, int row0) {
  if (blockIdx.x == 0 && (int)threadIdx.x < S) {
    AxmSegment sg;
    sg.a_row0 = sg.out_row0 = row0 + (int)threadIdx.x * Tp;
    sg.rows = Tp;
    sg.expert = threadIdx.x;
    segments[E + threadIdx.x] = sg;
  }
  const int chunks = D / 8;
  const long long total = (long long)Tp * chunks;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / chunks), c = (int)(i - (long long)t * chunks);
    const uint4 v = t < T ? __ldg(reinterpret_cast<const uint4*>(x + (size_t)t * D) + c) : make_uint4(0u, 0u, 0u, 0u);
    for (int s = 0; s < S; ++s)
      reinterpret_cast<uint4*>(x_perm + ((size_t)row0 + (size_t)s * Tp + t) * D)[c] = v;
  }
}

// Upstream gradient of the shared experts' rows: d_o[row0 + s * Tp + t] = bf16(dOut[t]) (they
// enter the output with weight 1), zero rows behind the tokens.
__global__ void __launch_bounds__(256)
bwd_prepare_shared_kernel(const float* __restrict__ d_out, __nv_bfloat16* __restrict__ d_o, int T, int Tp, int D,
                          int S, int row0) {
  const int chunks = D / 4;
  const long long total = (long long)Tp * chunks;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / chunks), c = (int)(i - (long long)t * chunks);
    uint2 v = make_uint2(0u, 0u);
    if (t < T) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(d_out + (size_t)t * D) + c);
      v = make_uint2(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w));
    }
    for (int s = 0; s < S; ++s)
      reinterpret_cast<uint2*>(d_o + ((size_t)row0 + (size_t)s * Tp + t) * D)[c] = v;
  }
}

// Launchers of the two kernels above for callers outside this file (the expert-parallel training
// step keeps the shared experts' rows in buffers of their own: row0 = 0, E = 0 there).
int launch_train_shared_rows(const void* x, void* x_perm, AxmSegment* segments, int T, int Tp, int D, int E, int S,
                             int row0, cudaStream_t st) {
  train_shared_rows_kernel<<<2 * sm_count(), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                           static_cast<__nv_bfloat16*>(x_perm), segments, T, Tp, D, E, S,
                                                           row0);
  return check_launch("train_shared_rows_kernel");
}
int launch_bwd_prepare_shared(const float* d_out, void* d_o, int T, int Tp, int D, int S, int row0, cudaStream_t st) {
  bwd_prepare_shared_kernel<<<2 * sm_count(), 256, 0, st>>>(d_out, static_cast<__nv_bfloat16*>(d_o), T, Tp, D, S, row0);
  return check_launch("bwd_prepare_shared_kernel");
}

struct TrainWs {
  int32_t* status;
  float* logits;
  int32_t* topk_idx;
  float* topk_gate;
  int32_t* block_counts;
  int32_t* counts;
  int32_t* offsets;
  int32_t* row_src;
  int32_t* slot_dst;
  AxmSegment* segments;
  float* aux_partial;
  float* aux_coef;
  float* d_gate;
  float* dz;
  float* dwr_partial;
  void *x_perm, *g, *u, *h, *o, *d_o, *d_g, *d_u, *d_xp;
  void* router_scratch;
  size_t router_scratch_bytes;
  int rows_max;     // rows of every row buffer: routed rows (padded) + shared experts' rows
  int shared_row0;  // first row of shared expert 0 (a fixed place behind the routed rows)
  int shared_rows;  // rows per shared expert: the tokens padded to a multiple of 64
  size_t bytes;
};

static TrainWs carve_train(const AxmMoeDesc* d, void* base) {
  TrainWs w;
  size_t off = 0;
  auto take = [&](size_t n) {
    void* p = base ? static_cast<char*>(base) + off : nullptr;
    off += (n + 255) & ~static_cast<size_t>(255);
    return p;
  };
  const size_t T = d->tokens, D = d->d_model, F = d->d_ff, E = d->num_experts, k = d->top_k, S = d->num_shared;
  const size_t R0 = (T * k + (kTrainAlign - 1) * E + kTrainAlign - 1) / kTrainAlign * kTrainAlign;
  const size_t Tp = (T + kTrainAlign - 1) / kTrainAlign * kTrainAlign;
  const size_t R = R0 + S * Tp;
  w.rows_max = (int)R;
  w.shared_row0 = (int)R0;
  w.shared_rows = (int)Tp;
  w.status = static_cast<int32_t*>(take(4));
  w.logits = static_cast<float*>(take(4 * T * E));
  w.topk_idx = static_cast<int32_t*>(take(4 * T * k));
  w.topk_gate = static_cast<float*>(take(4 * T * k));
  w.block_counts = static_cast<int32_t*>(take(4 * AXM_ROUTE_BLOCKS * E));
  w.counts = static_cast<int32_t*>(take(4 * E));
  w.offsets = static_cast<int32_t*>(take(4 * (E + 1)));
  w.row_src = static_cast<int32_t*>(take(4 * R0));
  w.slot_dst = static_cast<int32_t*>(take(4 * T * k));
  w.segments = static_cast<AxmSegment*>(take(sizeof(AxmSegment) * (E + S)));
  w.aux_partial = static_cast<float*>(take(4 * AXM_ROUTE_BLOCKS * E));
  w.aux_coef = static_cast<float*>(take(4 * E));
  w.d_gate = static_cast<float*>(take(4 * T * k));
  w.dz = static_cast<float*>(take(4 * T * E));
  w.dwr_partial = static_cast<float*>(take(4 * (size_t)kDwrChunks * D * E));
  w.x_perm = take(2 * R * D);
  w.g = take(2 * R * F);
  w.u = take(2 * R * F);
  w.h = take(2 * R * F);
  w.o = take(4 * R * D);
  w.d_o = take(2 * R * D);
  w.d_g = take(2 * R * F);
  w.d_u = take(2 * R * F);
  w.d_xp = take(4 * R * D);
  w.router_scratch_bytes = 0;
  axm_moe_router_scratch_bytes(d, &w.router_scratch_bytes);
  w.router_scratch = take(w.router_scratch_bytes);
  w.bytes = off;
  return w;
}

static int validate_train(const AxmMoeDesc* d) {
  if (d == nullptr) return fail(AXM_ERR_ARGUMENT, "desc is null");
  if (d->tokens <= 0) return fail(AXM_ERR_ARGUMENT, "tokens %d must be positive", d->tokens);
  if (d->d_model <= 0 || d->d_ff <= 0 || d->d_model % 8 || d->d_ff % 8)
    return fail(AXM_ERR_ARGUMENT, "d_model %d and d_ff %d must be positive multiples of 8", d->d_model, d->d_ff);
  if (d->num_experts <= 0 || d->num_experts > 256)
    return fail(AXM_ERR_ARGUMENT, "num_experts %d not in 1..256", d->num_experts);
  if (d->top_k <= 0 || d->top_k > 8 || d->top_k > d->num_experts)
    return fail(AXM_ERR_ARGUMENT, "top_k %d not in 1..min(num_experts, 8)", d->top_k);
  if (d->num_shared < 0 || d->num_shared > 8) return fail(AXM_ERR_ARGUMENT, "num_shared %d not in 0..8", d->num_shared);
  if (d->router_dtype != AXM_ROUTER_BF16 && d->router_dtype != AXM_ROUTER_FP32)
    return fail(AXM_ERR_ARGUMENT, "router_dtype %d unknown", d->router_dtype);
  if ((long long)d->tokens * d->top_k + 64LL * d->num_experts + ((long long)d->tokens + 64) * d->num_shared > 0x7fffffffLL)
    return fail(AXM_ERR_ARGUMENT, "row count overflows int32");
  return AXM_OK;
}

static int check_ws(const AxmMoeDesc* d, void* ws, size_t bytes, TrainWs* out) {
  if (ws == nullptr || (reinterpret_cast<uintptr_t>(ws) & 255) != 0)
    return fail(AXM_ERR_WORKSPACE, "workspace is null or not 256-byte aligned");
  *out = carve_train(d, ws);
  if (bytes < out->bytes) return fail(AXM_ERR_WORKSPACE, "workspace has %zu bytes, %zu needed", bytes, out->bytes);
  return AXM_OK;
}

}  // namespace axm

using namespace axm;

extern "C" int axm_moe_train_workspace_bytes(const AxmMoeDesc* desc, size_t* bytes) {
  if (int rc = validate_train(desc)) return rc;
  if (bytes == nullptr) return fail(AXM_ERR_ARGUMENT, "bytes is null");
  *bytes = carve_train(desc, nullptr).bytes;
  return AXM_OK;
}

extern "C" int axm_moe_forward_train(const AxmMoeDesc* desc, const AxmMoeTrain* t, void* workspace,
                                     size_t workspace_bytes, void* stream) {
  if (int rc = validate_train(desc)) return rc;
  if (!t || !t->x || !t->router_w || !t->w_gate || !t->w_up || !t->w_down || !t->out)
    return fail(AXM_ERR_ARGUMENT, "axm_moe_forward_train: x, router_w, w_gate, w_up, w_down, out are required");
  if (desc->num_shared > 0 && (!t->shared_gate || !t->shared_up || !t->shared_down))
    return fail(AXM_ERR_ARGUMENT, "num_shared > 0 needs shared_gate, shared_up and shared_down");
  TrainWs w;
  if (int rc = check_ws(desc, workspace, workspace_bytes, &w)) return rc;
  if (int rc = require_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int T = desc->tokens, E = desc->num_experts, k = desc->top_k, S = desc->num_shared;
  AxmMoeDesc d = *desc;
  // ws.counts holds this call's counts; the saved h of the training layout is one bf16 term
  d.flags &= ~(AXM_FLAG_HIST_ACCUMULATE | AXM_FLAG_H_EXACT);
  d.num_shared = 0;  // the routed part; the shared experts follow as ordinary segments of their own
  bool router_cleared_status = false;
  int rc = launch_router_auto(&d, t->x, t->router_w, t->router_bias, w.logits, w.topk_idx, w.topk_gate,
                              w.block_counts, w.router_scratch, w.router_scratch_bytes, w.status, stream,
                              &router_cleared_status);
  if (rc) return rc;
  if ((rc = launch_permute(&d, t->x, w.topk_idx, w.block_counts, w.counts, w.offsets, w.row_src,
                           w.slot_dst, w.x_perm, w.segments, router_cleared_status ? nullptr : w.status, st,
                           kTrainAlign)))
    return rc;
  if ((rc = launch_expert_ffn(&d, w.x_perm, w.rows_max, nullptr, 0, w.segments, E, t->w_gate, t->w_up,
                              t->w_down, nullptr, nullptr, nullptr, w.h, w.o, w.rows_max, w.status, st,
                              nullptr, nullptr, w.g, w.u)))
    return rc;
  if (S > 0) {
    train_shared_rows_kernel<<<2 * sm_count(), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(t->x),
                                                             static_cast<__nv_bfloat16*>(w.x_perm), w.segments, T,
                                                             w.shared_rows, desc->d_model, E, S, w.shared_row0);
    AxmMoeDesc ds = d;
    ds.num_experts = S;
    ds.top_k = 1;
    if ((rc = launch_expert_ffn(&ds, w.x_perm, w.rows_max, nullptr, 0, w.segments + E, S, t->shared_gate,
                                t->shared_up, t->shared_down, nullptr, nullptr, nullptr, w.h, w.o, w.rows_max,
                                w.status, st, nullptr, nullptr, w.g, w.u)))
      return rc;
  }
  AxmMoeDesc dc = *desc;
  dc.flags &= ~(AXM_FLAG_HIST_ACCUMULATE | AXM_FLAG_H_EXACT);
  const float* o_shared = S > 0 ? static_cast<const float*>(w.o) + (size_t)w.shared_row0 * desc->d_model : nullptr;
  if ((rc = launch_combine_strided(&dc, t->x, w.o, o_shared, w.shared_rows, w.slot_dst, w.topk_gate, nullptr, t->out,
                                   st)))
    return rc;
  // auxiliary loss and the constants its gradient needs
  if (int rc2 = launch_aux_partial(w.logits, w.aux_partial, T, E, st)) return rc2;
  aux_final_kernel<<<1, 256, 0, st>>>(w.aux_partial, w.counts, w.aux_coef, t->aux_loss, T, E, k,
                                      t->aux_alpha);
  if (t->histogram != nullptr)
    AXM_CUDA(cudaMemcpyAsync(t->histogram, w.counts, sizeof(int32_t) * E, cudaMemcpyDeviceToDevice, st));
  return check_launch("forward_train");
}

extern "C" int axm_moe_backward(const AxmMoeDesc* desc, const AxmMoeTrain* t, void* workspace,
                                size_t workspace_bytes, void* stream) {
  if (int rc = validate_train(desc)) return rc;
  if (!t || !t->x || !t->router_w || !t->w_gate || !t->w_up || !t->w_down || !t->d_out || !t->d_x)
    return fail(AXM_ERR_ARGUMENT, "axm_moe_backward: x, weights, d_out and d_x are required");
  const int S = desc->num_shared;
  if (S > 0) {
    if (!t->shared_gate || !t->shared_up || !t->shared_down)
      return fail(AXM_ERR_ARGUMENT, "num_shared > 0 needs shared_gate, shared_up and shared_down");
    const bool routed = t->d_w_gate || t->d_w_up || t->d_w_down;
    const bool shared_all = t->d_shared_gate && t->d_shared_up && t->d_shared_down;
    const bool shared_any = t->d_shared_gate || t->d_shared_up || t->d_shared_down;
    if (routed != shared_any || shared_any != shared_all)
      return fail(AXM_ERR_ARGUMENT, "shared experts' weight gradients: all three exactly when the routed experts' are given");
  }
  TrainWs w;
  if (int rc = check_ws(desc, workspace, workspace_bytes, &w)) return rc;
  if (int rc = require_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int D = desc->d_model, E = desc->num_experts, k = desc->top_k;

  // Shared-memory limits of the two router-gradient kernels are settled before anything is
  // launched, so that a refusal leaves no half-finished backward pass behind.
  int rc;
  if ((rc = bwd_source_limits(E, desc->router_dtype))) return rc;
  if ((rc = launch_bwd_prepare(t->d_out, static_cast<const float*>(w.o), w.row_src, w.topk_gate, w.offsets, w.d_o,
                               w.d_gate, D, E, k, st)))
    return rc;
  AxmMoeDesc dr = *desc;
  dr.num_shared = 0;  // the routed experts; the shared ones follow as experts of their own
  if ((rc = axm_moe_expert_ffn_backward(&dr, w.segments, E, w.rows_max, w.x_perm, w.h, w.g, w.u, w.d_o,
                                        t->w_gate, t->w_up, t->w_down, w.d_g, w.d_u, w.d_xp,
                                        t->d_w_gate, t->d_w_up, t->d_w_down, w.status, stream)))
    return rc;
  if (S > 0) {
    bwd_prepare_shared_kernel<<<2 * sm_count(), 256, 0, st>>>(t->d_out, static_cast<__nv_bfloat16*>(w.d_o),
                                                              desc->tokens, w.shared_rows, D, S, w.shared_row0);
    AxmMoeDesc ds = *desc;
    ds.num_experts = S;
    ds.num_shared = 0;
    ds.top_k = 1;
    if ((rc = axm_moe_expert_ffn_backward(&ds, w.segments + E, S, w.rows_max, w.x_perm, w.h, w.g, w.u, w.d_o,
                                          t->shared_gate, t->shared_up, t->shared_down, w.d_g, w.d_u, w.d_xp,
                                          t->d_shared_gate, t->d_shared_up, t->d_shared_down, w.status, stream)))
      return rc;
  }
  return launch_bwd_source_tail(desc, t, w.logits, w.topk_idx, w.d_gate, w.aux_coef, w.dz, w.aux_partial,
                                w.dwr_partial, static_cast<const float*>(w.d_xp), w.slot_dst, st, S,
                                static_cast<const float*>(w.d_xp) + (size_t)w.shared_row0 * D, w.shared_rows);
}

// ---- optimizer step for the MoE weights ---------------------------------------------
// AdamW with decoupled weight decay over an fp32 master copy, two fp32 moments and the
// bf16 working copy the kernels read - the storage the engine keeps for every MoE matrix
// (core/src/CUDA/util/gpu_types.cuh:148-168; its fused AdamW for the dense weights is
// core/src/CUDA/kernel/backward_pass.cu:812-852).  Textbook update, bias-corrected:
//   m = b1 m + (1 - b1) g;  v = b2 v + (1 - b2) g^2;
//   w -= lr * ( (m / (1 - b1^t)) / (sqrt(v / (1 - b2^t)) + eps) + wd * w );  w_bf16 = bf16(w).
//
// kEngine selects the conventions of the engine's own fused AdamW, so that an engine
// checkpoint trains the same way under either optimiser:
//   g: non-finite -> 0, then clamped to [-100, 100];  m, v updated with that g;
//   bias corrections 1 - b^t replaced by 1 when they are <= 1e-7;
//   step size lr * rsqrt(in_dim) (in_dim = rows of the [in][out] matrix);
//   w' = w - step * (m_hat / (sqrt(v_hat) + eps) + wd * w); if w' is finite it is clamped to
//   [-2, 2] and stored (master and bf16 copy), else the weight is left as it was.
// The host passes lr already scaled and c1, c2 already floored.
namespace axm {
template <bool kEngine>
__device__ __forceinline__ void adamw_one(float g, float& mj, float& vj, float& wj, bool& store, float lr,
                                          float b1, float b2, float eps, float wd, float c1, float c2) {
  if (kEngine) {
    if (!isfinite(g)) g = 0.0f;
    g = fmaxf(-100.0f, fminf(100.0f, g));
  }
  mj = b1 * mj + (1.0f - b1) * g;
  vj = b2 * vj + (1.0f - b2) * g * g;
  if (kEngine) {
    const float upd = (mj / c1) / (sqrtf(vj / c2) + eps);
    const float w_new = wj - lr * (upd + wd * wj);
    store = isfinite(w_new);
    if (store) wj = fmaxf(-2.0f, fminf(2.0f, w_new));
  } else {
    wj -= lr * ((mj / c1) / (sqrtf(vj / c2) + eps) + wd * wj);
    store = true;
  }
}

template <bool kEngine>
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
             const float* __restrict__ grad, __nv_bfloat16* __restrict__ w_bf16, long long n, float lr,
             float b1, float b2, float eps, float wd, float c1, float c2) {
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n;
       i += (long long)gridDim.x * blockDim.x * 4) {
    if (i + 3 < n) {
      float4 g = __ldg(reinterpret_cast<const float4*>(grad + i));
      float4 mm = *reinterpret_cast<float4*>(m + i), vv = *reinterpret_cast<float4*>(v + i);
      float4 ww = *reinterpret_cast<float4*>(master + i);
      float* gp = &g.x; float* mp = &mm.x; float* vp = &vv.x; float* wp = &ww.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        bool st;
        adamw_one<kEngine>(gp[j], mp[j], vp[j], wp[j], st, lr, b1, b2, eps, wd, c1, c2);
      }
      *reinterpret_cast<float4*>(m + i) = mm;
      *reinterpret_cast<float4*>(v + i) = vv;
      // a weight whose update was refused keeps its value (wp[j] untouched) and its bf16 copy
      // is the rounding of that unchanged master: storing both changes nothing
      *reinterpret_cast<float4*>(master + i) = ww;
      *reinterpret_cast<uint2*>(w_bf16 + i) = make_uint2(pack_bf16(ww.x, ww.y), pack_bf16(ww.z, ww.w));
    } else {
      for (long long e = i; e < n; ++e) {
        float mj = m[e], vj = v[e], wj = master[e];
        bool st;
        adamw_one<kEngine>(grad[e], mj, vj, wj, st, lr, b1, b2, eps, wd, c1, c2);
        m[e] = mj;
        v[e] = vj;
        master[e] = wj;
        w_bf16[e] = __float2bfloat16_rn(wj);
      }
    }
  }
}
}  // namespace axm

static int adamw_launch(bool engine, float* master, float* m, float* v, const float* grad, void* w_bf16,
                        int64_t n, float lr, float beta1, float beta2, float eps, float weight_decay,
                        int64_t step, int64_t in_dim, void* stream) {
  if (!master || !m || !v || !grad || !w_bf16) return fail(AXM_ERR_ARGUMENT, "axm_moe_adamw_step: null pointer");
  if (n < 0 || (!engine && step < 1)) return fail(AXM_ERR_ARGUMENT, "axm_moe_adamw_step: n must be >= 0 and step >= 1");
  if ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(grad)) & 15)
    return fail(AXM_ERR_ARGUMENT, "axm_moe_adamw_step: fp32 buffers must be 16-byte aligned");
  // the kernel stores four bf16 values at a time
  if (reinterpret_cast<uintptr_t>(w_bf16) & 7)
    return fail(AXM_ERR_ARGUMENT, "axm_moe_adamw_step: the bf16 copy must be 8-byte aligned");
  if (n == 0) return AXM_OK;
  if (int rc = require_device()) return rc;
  float c1 = 1.0f - powf(beta1, (float)(step > 0 ? step : 1)), c2 = 1.0f - powf(beta2, (float)(step > 0 ? step : 1));
  if (engine) {
    if (!(c1 > 1e-7f)) c1 = 1.0f;
    if (!(c2 > 1e-7f)) c2 = 1.0f;
    lr = lr * (1.0f / sqrtf((float)(in_dim > 0 ? in_dim : 1)));
  }
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 16LL * sm_count()) blocks = 16LL * sm_count();
  if (blocks < 1) blocks = 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (engine)
    adamw_kernel<true><<<(unsigned)blocks, 256, 0, st>>>(master, m, v, grad, static_cast<__nv_bfloat16*>(w_bf16), n,
                                                         lr, beta1, beta2, eps, weight_decay, c1, c2);
  else
    adamw_kernel<false><<<(unsigned)blocks, 256, 0, st>>>(master, m, v, grad, static_cast<__nv_bfloat16*>(w_bf16), n,
                                                          lr, beta1, beta2, eps, weight_decay, c1, c2);
  return check_launch("adamw_kernel");
}

extern "C" int axm_moe_adamw_step(float* master, float* m, float* v, const float* grad, void* w_bf16,
                                  int64_t n, float lr, float beta1, float beta2, float eps,
                                  float weight_decay, int32_t step, void* stream) {
  return adamw_launch(false, master, m, v, grad, w_bf16, n, lr, beta1, beta2, eps, weight_decay, step, 1, stream);
}

extern "C" int axm_moe_adamw_step_engine(float* master, float* m, float* v, const float* grad, void* w_bf16,
                                         int64_t n, int64_t in_dim, float lr, float beta1, float beta2,
                                         float eps, float weight_decay, int64_t step, void* stream) {
  return adamw_launch(true, master, m, v, grad, w_bf16, n, lr, beta1, beta2, eps, weight_decay, step, in_dim,
                      stream);
}
