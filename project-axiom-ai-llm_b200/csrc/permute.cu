// Dispatch (histogram -> exclusive scan -> stable expert-contiguous placement ->
// 16-byte row copies) and the weighted combine with residual.
//
// The reference engine has no permutation: its dispatch kernel walks tokens one
// CTA each (core/src/CUDA/kernel/moe_router.cu:113-191).  The placement rule
// implemented here is the one that reproduces its routing in expert-contiguous
// form: rows of an expert ordered by token index, then by slot.  The histogram
// has the engine's meaning (one count per selection,
// core/src/CUDA/kernel/moe_router.cu:107-110); accumulation across calls is the
// caller's choice (AXM_FLAG_HIST_ACCUMULATE).  The combine kernel reads fp32 expert
// rows, computes bf16(sum_i gate_i * o_i) and then bf16(x + y), the two rounding points of
// core/src/CUDA/kernel/moe_router.cu:186-203.
#include "common.cuh"

namespace axm {

__host__ __device__ inline int route_block_begin2(int b, int T) {
  return (int)(((long long)b * T) / AXM_ROUTE_BLOCKS);
}

constexpr int kPermThreads = 256;
constexpr int kPermTokSub = 128;  // tokens placed per pass
constexpr int kMaxE = 256;

// One CTA per router block.  Shared memory: total[E], base[E], run[E], dst[kPermTokSub*k].
__global__ void __launch_bounds__(kPermThreads)
permute_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ topk_idx,
               const int32_t* __restrict__ block_counts, int32_t* __restrict__ histogram,
               int32_t* __restrict__ offsets, int32_t* __restrict__ row_src,
               int32_t* __restrict__ slot_dst, __nv_bfloat16* __restrict__ x_perm,
               AxmSegment* __restrict__ segments, int32_t* __restrict__ status, int T, int D,
               int E, int k, int S, int hist_accumulate, int row_align,
               const float* __restrict__ norm_rstd, const float* __restrict__ norm_gamma) {
  __shared__ int total_s[kMaxE];
  __shared__ int run_s[kMaxE];   // next free row per expert for this block
  __shared__ int scan_s[kMaxE + 1];
  __shared__ int dst_s[kPermTokSub * 8];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x;

  for (int e = tid; e < E; e += kPermThreads) {
    total_s[e] = 0;
    run_s[e] = 0;
  }
  __syncthreads();
  // Column sums of block_counts: all blocks -> total, blocks before this one -> run.
  const int n_cells = AXM_ROUTE_BLOCKS * E;
  for (int i = tid; i < n_cells; i += kPermThreads) {
    int bb = i / E, e = i - bb * E;
    int c = block_counts[i];
    if (c != 0) {
      atomicAdd(&total_s[e], c);
      if (bb < b) atomicAdd(&run_s[e], c);
    }
  }
  __syncthreads();
  // Exclusive scan over experts (E <= 256: one warp walks it in chunks of 32).
  if (warp == 0) {
    int carry = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      int e = e0 + lane;
      // training layout: every expert's rows start at a multiple of row_align
      int v = e < E ? (total_s[e] + row_align - 1) / row_align * row_align : 0;
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
      }
      if (e < E) scan_s[e] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) scan_s[E] = carry;
  }
  __syncthreads();
  for (int e = tid; e < E; e += kPermThreads) run_s[e] += scan_s[e];
  if (b == 0) {
    for (int e = tid; e <= E; e += kPermThreads) {
      if (offsets != nullptr) offsets[e] = scan_s[e];
      if (e < E && histogram != nullptr)
        histogram[e] = (hist_accumulate ? histogram[e] : 0) + total_s[e];
    }
    if (segments != nullptr) {
      for (int e = tid; e < E + S; e += kPermThreads) {
        AxmSegment sg;
        if (e < E) {
          sg.a_row0 = scan_s[e];
          sg.out_row0 = scan_s[e];
          sg.rows = scan_s[e + 1] - scan_s[e];  // padded rows (equal to the count when row_align is 1)
          sg.expert = e;
        } else {
          sg.a_row0 = 0;
          sg.out_row0 = T * k + (e - E) * T;
          sg.rows = T;
          sg.expert = e | AXM_SEG_ALT_A;
        }
        segments[e] = sg;
      }
    }
    if (status != nullptr && tid == 0) *status = 0;
  }
  // Padding rows (row_align > 1) are zero rows that belong to no slot: block e fills expert e's.
  if (row_align > 1 && b < E) {
    const int pad0 = scan_s[b] + total_s[b], pad1 = scan_s[b + 1];
    const int chunks = D / 8;
    for (int r = pad0; r < pad1; ++r) {
      if (row_src != nullptr && tid == 0) row_src[r] = -1;
      if (x_perm != nullptr)
        for (int c = tid; c < chunks; c += kPermThreads)
          reinterpret_cast<uint4*>(x_perm + (size_t)r * D)[c] = make_uint4(0, 0, 0, 0);
    }
  }
  __syncthreads();

  const int t_begin = route_block_begin2(b, T);
  const int t_end = route_block_begin2(b + 1, T);
  for (int ts = t_begin; ts < t_end; ts += kPermTokSub) {
    const int nt = min(kPermTokSub, t_end - ts);
    const int n_ent = nt * k;
    // Stable placement: one warp walks the (token, slot) entries in order, 32 at
    // a time; equal experts inside a chunk are ranked by a match + popcount.
    if (warp == 0) {
      for (int c0 = 0; c0 < n_ent; c0 += 32) {
        int i = c0 + lane;
        bool live = i < n_ent;
        int e = live ? topk_idx[(size_t)ts * k + i] : -1;
        unsigned peers = __match_any_sync(0xffffffffu, e);
        int rank = __popc(peers & ((1u << lane) - 1u));
        int dst = -1;
        if (live) {
          dst = run_s[e] + rank;
          dst_s[i] = dst;
        }
        __syncwarp();
        if (live && rank == __popc(peers) - 1) run_s[e] += rank + 1;  // last peer advances
        __syncwarp();
        if (live) {
          size_t slot = (size_t)ts * k + i;
          if (slot_dst != nullptr) slot_dst[slot] = dst;
          if (row_src != nullptr) row_src[dst] = (int32_t)slot;
        }
      }
    }
    __syncthreads();
    // Row copies: a warp takes a token, reads its row once in 16-byte pieces and
    // stores it to each of its k destinations.
    if (x_perm != nullptr) {
      const int chunks = D / 8;
      for (int tt = warp; tt < nt; tt += kPermThreads / 32) {
        const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(ts + tt) * D);
        for (int c0 = 0; c0 < chunks; c0 += 128) {
          uint4 v[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            int c = c0 + j * 32 + lane;
            if (c < chunks) v[j] = __ldg(src + c);
          }
          if (norm_rstd != nullptr) {
            // pre-norm form: the rows dispatched are RMSNorm(x), formed here exactly as the
            // RMSNorm kernel forms them, bf16(x * rstd * gamma)
            const float rs = __ldg(norm_rstd + ts + tt);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int c = c0 + j * 32 + lane;
              if (c < chunks) {
                const uint32_t w4[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
                uint32_t r4[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const int d = c * 8 + 2 * q;
                  const float g0 = norm_gamma ? __ldg(norm_gamma + d) : 1.0f, g1 = norm_gamma ? __ldg(norm_gamma + d + 1) : 1.0f;
                  r4[q] = pack_bf16(bf16_lo(w4[q]) * rs * g0, bf16_hi(w4[q]) * rs * g1);
                }
                v[j] = make_uint4(r4[0], r4[1], r4[2], r4[3]);
              }
            }
          }
          for (int i = 0; i < k; ++i) {
            uint4* dstp = reinterpret_cast<uint4*>(x_perm + (size_t)dst_s[tt * k + i] * D);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              int c = c0 + j * 32 + lane;
              if (c < chunks) dstp[c] = v[j];
            }
          }
        }
      }
    }
    __syncthreads();
  }
}

__global__ void build_segments_kernel(const int32_t* __restrict__ offsets,
                                      AxmSegment* __restrict__ segments, int T, int E, int k,
                                      int S) {
  for (int e = threadIdx.x; e < E + S; e += blockDim.x) {
    AxmSegment sg;
    if (e < E) {
      sg.a_row0 = offsets[e];
      sg.out_row0 = offsets[e];
      sg.rows = offsets[e + 1] - offsets[e];
      sg.expert = e;
    } else {
      sg.a_row0 = 0;
      sg.out_row0 = T * k + (e - E) * T;
      sg.rows = T;
      sg.expert = e | AXM_SEG_ALT_A;
    }
    segments[e] = sg;
  }
}

// One thread per 16-byte piece of an output row.  K is the exact top-k, so the
// gathered row pieces live in 2*K float4 registers and all of them are in flight
// together.
template <int K>
__global__ void __launch_bounds__(256)
combine_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ o,
               const float* __restrict__ o_shared, const int32_t* __restrict__ slot_dst,
               const float* __restrict__ topk_gate, __nv_bfloat16* __restrict__ y,
               __nv_bfloat16* __restrict__ out, int T, int D, int S, int residual, int shared_stride) {
  const int chunks = D / 8;
  const long long total = (long long)T * chunks;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < total;
       g += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(g / chunks);
    const int c = (int)(g - (long long)t * chunks);
    int r[K];
    float gw[K];
#pragma unroll
    for (int i = 0; i < K; ++i) {
      r[i] = __ldg(slot_dst + (size_t)t * K + i);
      gw[i] = __ldg(topk_gate + (size_t)t * K + i);
    }
    uint4 xv = make_uint4(0, 0, 0, 0);
    if (residual) xv = __ldg(reinterpret_cast<const uint4*>(x + (size_t)t * D) + c);
    float4 va[K], vb[K];
#pragma unroll
    for (int i = 0; i < K; ++i) {
      const float4* row = reinterpret_cast<const float4*>(o + (size_t)r[i] * D) + 2 * c;
      va[i] = __ldg(row);
      vb[i] = __ldg(row + 1);
    }
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
#pragma unroll
    for (int i = 0; i < K; ++i) {
      acc[0] = fmaf(gw[i], va[i].x, acc[0]);
      acc[1] = fmaf(gw[i], va[i].y, acc[1]);
      acc[2] = fmaf(gw[i], va[i].z, acc[2]);
      acc[3] = fmaf(gw[i], va[i].w, acc[3]);
      acc[4] = fmaf(gw[i], vb[i].x, acc[4]);
      acc[5] = fmaf(gw[i], vb[i].y, acc[5]);
      acc[6] = fmaf(gw[i], vb[i].z, acc[6]);
      acc[7] = fmaf(gw[i], vb[i].w, acc[7]);
    }
    for (int s = 0; s < S; ++s) {
      const float4* row = reinterpret_cast<const float4*>(o_shared + ((size_t)s * shared_stride + t) * D) + 2 * c;
      float4 a = __ldg(row), b = __ldg(row + 1);
      acc[0] += a.x;
      acc[1] += a.y;
      acc[2] += a.z;
      acc[3] += a.w;
      acc[4] += b.x;
      acc[5] += b.y;
      acc[6] += b.z;
      acc[7] += b.w;
    }
    uint4 yv;
    yv.x = pack_bf16(acc[0], acc[1]);
    yv.y = pack_bf16(acc[2], acc[3]);
    yv.z = pack_bf16(acc[4], acc[5]);
    yv.w = pack_bf16(acc[6], acc[7]);
    if (y != nullptr) reinterpret_cast<uint4*>(y + (size_t)t * D)[c] = yv;
    if (residual) {
      uint4 rr;
      rr.x = pack_bf16(bf16_lo(xv.x) + bf16_lo(yv.x), bf16_hi(xv.x) + bf16_hi(yv.x));
      rr.y = pack_bf16(bf16_lo(xv.y) + bf16_lo(yv.y), bf16_hi(xv.y) + bf16_hi(yv.y));
      rr.z = pack_bf16(bf16_lo(xv.z) + bf16_lo(yv.z), bf16_hi(xv.z) + bf16_hi(yv.z));
      rr.w = pack_bf16(bf16_lo(xv.w) + bf16_lo(yv.w), bf16_hi(xv.w) + bf16_hi(yv.w));
      reinterpret_cast<uint4*>(out + (size_t)t * D)[c] = rr;
    } else {
      reinterpret_cast<uint4*>(out + (size_t)t * D)[c] = yv;
    }
  }
}

template <int K>
static void launch_combine(int blocks, cudaStream_t st, const void* x, const void* o,
                           const void* o_shared, const int32_t* slot_dst, const float* topk_gate,
                           void* y, void* out, const AxmMoeDesc* d, int residual, int shared_stride) {
  combine_kernel<K><<<blocks, 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(o),
      static_cast<const float*>(o_shared), slot_dst, topk_gate, static_cast<__nv_bfloat16*>(y),
      static_cast<__nv_bfloat16*>(out), d->tokens, d->d_model, d->num_shared, residual, shared_stride);
}

int launch_permute(const AxmMoeDesc* d, const void* x, const int32_t* topk_idx,
                   const int32_t* block_counts, int32_t* histogram, int32_t* offsets,
                   int32_t* row_src, int32_t* slot_dst, void* x_perm, AxmSegment* segments,
                   int32_t* status, cudaStream_t st, int row_align, const float* norm_rstd,
                   const float* norm_gamma) {
  permute_kernel<<<AXM_ROUTE_BLOCKS, kPermThreads, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), topk_idx, block_counts, histogram, offsets, row_src,
      slot_dst, static_cast<__nv_bfloat16*>(x_perm), segments, status, d->tokens, d->d_model,
      d->num_experts, d->top_k, d->num_shared, (d->flags & AXM_FLAG_HIST_ACCUMULATE) ? 1 : 0,
      row_align < 1 ? 1 : row_align, norm_rstd, norm_gamma);
  return check_launch("permute_kernel");
}

}  // namespace axm

namespace axm {
int validate_perm(const AxmMoeDesc* d) {
  if (d == nullptr) return fail(AXM_ERR_ARGUMENT, "desc is null");
  if (d->tokens < 0 || d->d_model <= 0 || d->num_experts <= 0 || d->top_k <= 0)
    return fail(AXM_ERR_ARGUMENT, "tokens/d_model/num_experts/top_k must be positive");
  if (d->num_experts > kMaxE) return fail(AXM_ERR_ARGUMENT, "num_experts %d > %d", d->num_experts, kMaxE);
  if (d->top_k > 8) return fail(AXM_ERR_ARGUMENT, "top_k %d > 8", d->top_k);
  if (d->num_shared < 0 || d->num_shared > 8) return fail(AXM_ERR_ARGUMENT, "num_shared %d not in 0..8", d->num_shared);
  if (d->d_model % 8 != 0) return fail(AXM_ERR_ARGUMENT, "d_model %d not a multiple of 8", d->d_model);
  if ((long long)d->tokens * d->top_k + (long long)d->tokens * d->num_shared > 0x7fffffffLL)
    return fail(AXM_ERR_ARGUMENT, "row count overflows int32");
  return AXM_OK;
}
}  // namespace axm

namespace axm {
// Combine with the shared experts' rows `shared_stride` rows apart ([S][shared_stride][D] fp32; the
// public entry point passes the token count, the training layout its padded token count).
int launch_combine_strided(const AxmMoeDesc* desc, const void* x, const void* o, const void* o_shared,
                           int shared_stride, const int32_t* slot_dst, const float* topk_gate, void* y, void* out,
                           cudaStream_t st) {
  if (int rc = validate_perm(desc)) return rc;
  if (!o || !slot_dst || !topk_gate || !out) return fail(AXM_ERR_ARGUMENT, "axm_moe_combine: null pointer");
  const int residual = (desc->flags & AXM_FLAG_RESIDUAL) ? 1 : 0;
  if (residual && !x) return fail(AXM_ERR_ARGUMENT, "axm_moe_combine: residual without x");
  if (desc->num_shared > 0 && !o_shared) return fail(AXM_ERR_ARGUMENT, "axm_moe_combine: shared experts without o_shared");
  if (desc->tokens == 0) return AXM_OK;
  if (int rc = require_device()) return rc;
  long long total = (long long)desc->tokens * (desc->d_model / 8);
  int blocks = (int)((total + 255) / 256);
  int cap = sm_count() * 16;
  if (blocks > cap) blocks = cap;
  switch (desc->top_k) {
#define AXM_COMBINE_CASE(K) \
  case K: launch_combine<K>(blocks, st, x, o, o_shared, slot_dst, topk_gate, y, out, desc, residual, shared_stride); break;
    AXM_COMBINE_CASE(1)
    AXM_COMBINE_CASE(2)
    AXM_COMBINE_CASE(3)
    AXM_COMBINE_CASE(4)
    AXM_COMBINE_CASE(5)
    AXM_COMBINE_CASE(6)
    AXM_COMBINE_CASE(7)
    AXM_COMBINE_CASE(8)
#undef AXM_COMBINE_CASE
    default: return fail(AXM_ERR_ARGUMENT, "top_k %d not in 1..8", desc->top_k);
  }
  return check_launch("combine_kernel");
}
}  // namespace axm

using namespace axm;

extern "C" int axm_moe_permute(const AxmMoeDesc* desc, const void* x, const int32_t* topk_idx,
                               const int32_t* block_counts, int32_t* histogram, int32_t* offsets,
                               int32_t* row_src, int32_t* slot_dst, void* x_perm, void* stream) {
  if (int rc = validate_perm(desc)) return rc;
  if (!topk_idx || !block_counts) return fail(AXM_ERR_ARGUMENT, "axm_moe_permute: null pointer");
  if (x_perm != nullptr && x == nullptr) return fail(AXM_ERR_ARGUMENT, "axm_moe_permute: x_perm without x");
  if (int rc = require_device()) return rc;
  return launch_permute(desc, x, topk_idx, block_counts, histogram, offsets, row_src, slot_dst,
                        x_perm, nullptr, nullptr, static_cast<cudaStream_t>(stream), 1, nullptr, nullptr);
}

extern "C" int axm_moe_permute_padded(const AxmMoeDesc* desc, const void* x, const int32_t* topk_idx,
                                      const int32_t* block_counts, int32_t* histogram,
                                      int32_t* offsets, int32_t* row_src, int32_t* slot_dst,
                                      void* x_perm, AxmSegment* segments, int32_t row_align,
                                      void* stream) {
  if (int rc = validate_perm(desc)) return rc;
  if (!topk_idx || !block_counts) return fail(AXM_ERR_ARGUMENT, "axm_moe_permute_padded: null pointer");
  if (x_perm != nullptr && x == nullptr) return fail(AXM_ERR_ARGUMENT, "axm_moe_permute_padded: x_perm without x");
  if (row_align < 1 || row_align > 1024) return fail(AXM_ERR_ARGUMENT, "row_align %d not in 1..1024", row_align);
  if (int rc = require_device()) return rc;
  return launch_permute(desc, x, topk_idx, block_counts, histogram, offsets, row_src, slot_dst,
                        x_perm, segments, nullptr, static_cast<cudaStream_t>(stream), row_align, nullptr, nullptr);
}

extern "C" int axm_moe_build_segments(const AxmMoeDesc* desc, const int32_t* offsets,
                                      AxmSegment* segments, void* stream) {
  if (int rc = validate_perm(desc)) return rc;
  if (!offsets || !segments) return fail(AXM_ERR_ARGUMENT, "axm_moe_build_segments: null pointer");
  if (int rc = require_device()) return rc;
  build_segments_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      offsets, segments, desc->tokens, desc->num_experts, desc->top_k, desc->num_shared);
  return check_launch("build_segments_kernel");
}

extern "C" int axm_moe_combine(const AxmMoeDesc* desc, const void* x, const void* o,
                               const void* o_shared, const int32_t* slot_dst,
                               const float* topk_gate, void* y, void* out, void* stream) {
  return launch_combine_strided(desc, x, o, o_shared, desc ? desc->tokens : 0, slot_dst, topk_gate, y, out,
                                static_cast<cudaStream_t>(stream));
}
