// Expert FFN for decode-sized calls (at most kDecodeTokens tokens): with one to four tokens an
// expert holds one to four rows, only k experts' weights are touched at all, and the 256-row
// tensor-core tiles of grouped_ffn_2sm.cu leave most SMs without a tile (one token, top-2 of 8
// experts: 32 tile pairs for the down projection on 74 CTA pairs).  The work is a pure weight
// stream, so these kernels are GEMV-style on the CUDA cores: every CTA streams one 256-column
// slice of one expert's weight matrix from HBM exactly once with 16-byte loads, keeps the
// expert's few activation rows in shared memory, and its eight warps split the reduction
// dimension; the partial sums meet in shared memory in warp order (deterministic).
//
//   decode_gate_up_kernel   h[r, f] = SiLU(x_r . Wg[e][:, f]) * (x_r . Wu[e][:, f])    -> bf16 (hi | lo)
//   decode_down_kernel      partial[z][r, d] = sum over the z-th quarter of f of h[r, f] * Wd[e][f, d]
//   decode_reduce_kernel    o[r, d] = sum_z partial[z][r, d]                             -> fp32
//
// The down projection splits f over kDecodeSplits CTAs so that one token still gives 128 CTAs.
// Same conventions as the tensor-core path (core/src/CUDA/kernel/moe_router.cu:155-190 of the
// reference engine is what both replace): bf16 inputs, fp32 accumulation, h rounded to bf16
// between the projections (two bf16 terms with AXM_FLAG_H_EXACT), fp32 expert rows out.  The
// summation order differs from the tensor cores', so results agree to rounding, not bit for bit.
// The reference engine's decode path is dense-only (core/src/ai.cpp:944-1052).
#include <cstdlib>

#include "common.cuh"

namespace axm {

constexpr int kDecodeTokens = 4;   // rows an expert can hold (a token picks an expert at most once)
constexpr int kDecodeSplits = 4;   // CTAs that share the reduction of one down-projection slice
constexpr int kDecodeWarps = 8;
constexpr int kDecodeCols = 256;   // columns per CTA: 32 lanes x 8 bf16

struct DecodeArgs {
  const AxmSegment* segments;
  int routed_experts;
  int D, F;
  const __nv_bfloat16* x_perm;  // rows of routed segments
  const __nv_bfloat16* x_alt;   // rows of AXM_SEG_ALT_A segments (shared experts read the tokens themselves)
  const __nv_bfloat16 *w_gate, *w_up, *w_down, *s_gate, *s_up, *s_down;
  __nv_bfloat16* h;             // [rows][h_ld]
  int h_ld, lo_off;             // lo_off != 0: second bf16 term at column lo_off + f
  float* partial;               // [kDecodeSplits][rows_total][D]
  int rows_total;
};

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
  f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}

__device__ __forceinline__ uint4 ldg_stream(const __nv_bfloat16* p) {
  uint4 v;  // weights are read once: keep them out of L1
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// grid (ceil(F / 256), segments); 256 threads.  Dynamic shared memory: x rows [4][D] bf16, then
// the partial sums [8 warps][4 rows][256 columns][gate, up] fp32.
__global__ void __launch_bounds__(kDecodeWarps * 32)
decode_gate_up_kernel(DecodeArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  const AxmSegment sg = a.segments[blockIdx.y];
  const int rows = sg.rows < kDecodeTokens ? sg.rows : kDecodeTokens;
  if (rows <= 0) return;
  const int D = a.D, F = a.F;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem);
  float* red = reinterpret_cast<float*>(smem + (size_t)kDecodeTokens * D * 2);
  const int e_raw = sg.expert & ~AXM_SEG_ALT_A;
  const bool shared_w = e_raw >= a.routed_experts;
  const int e = shared_w ? e_raw - a.routed_experts : e_raw;
  const __nv_bfloat16* src = (sg.expert & AXM_SEG_ALT_A) ? a.x_alt : a.x_perm;
  const __nv_bfloat16* wg = (shared_w ? a.s_gate : a.w_gate) + (size_t)e * D * F;
  const __nv_bfloat16* wu = (shared_w ? a.s_up : a.w_up) + (size_t)e * D * F;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < kDecodeTokens * (D / 8); i += blockDim.x) {
    const int r = i / (D / 8), c = i - r * (D / 8);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows) v = __ldg(reinterpret_cast<const uint4*>(src + (size_t)(sg.a_row0 + r) * D) + c);
    reinterpret_cast<uint4*>(xs + (size_t)r * D)[c] = v;
  }
  __syncthreads();
  const int f = blockIdx.x * kDecodeCols + lane * 8;
  const bool live = f < F;  // F is a multiple of 8: a lane's eight columns are all inside or all outside
  const int d_per = (D + kDecodeWarps - 1) / kDecodeWarps;
  const int d0 = warp * d_per, d1 = (d0 + d_per < D) ? d0 + d_per : D;
  float ag[kDecodeTokens][8], au[kDecodeTokens][8];
#pragma unroll
  for (int r = 0; r < kDecodeTokens; ++r)
#pragma unroll
    for (int j = 0; j < 8; ++j) ag[r][j] = au[r][j] = 0.0f;
  if (live) {
    const __nv_bfloat16* pg = wg + (size_t)d0 * F + f;
    const __nv_bfloat16* pu = wu + (size_t)d0 * F + f;
    int d = d0;
    for (; d + 3 < d1; d += 4) {  // eight 16-byte loads in flight per lane
      uint4 vg[4], vu[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        vg[q] = ldg_stream(pg + (size_t)q * F);
        vu[q] = ldg_stream(pu + (size_t)q * F);
      }
      pg += (size_t)4 * F;
      pu += (size_t)4 * F;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float g8[8], u8[8];
        unpack8(vg[q], g8);
        unpack8(vu[q], u8);
#pragma unroll
        for (int r = 0; r < kDecodeTokens; ++r) {
          const float xv = __bfloat162float(xs[(size_t)r * D + d + q]);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            ag[r][j] = fmaf(xv, g8[j], ag[r][j]);
            au[r][j] = fmaf(xv, u8[j], au[r][j]);
          }
        }
      }
    }
    for (; d < d1; ++d) {
      float g8[8], u8[8];
      unpack8(ldg_stream(pg), g8);
      unpack8(ldg_stream(pu), u8);
      pg += F;
      pu += F;
#pragma unroll
      for (int r = 0; r < kDecodeTokens; ++r) {
        const float xv = __bfloat162float(xs[(size_t)r * D + d]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ag[r][j] = fmaf(xv, g8[j], ag[r][j]);
          au[r][j] = fmaf(xv, u8[j], au[r][j]);
        }
      }
    }
  }
  // red[warp][r][column][2]
#pragma unroll
  for (int r = 0; r < kDecodeTokens; ++r)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float2* p = reinterpret_cast<float2*>(red) + ((size_t)(warp * kDecodeTokens + r) * kDecodeCols + lane * 8 + j);
      *p = make_float2(ag[r][j], au[r][j]);
    }
  __syncthreads();
  for (int i = tid; i < rows * kDecodeCols; i += blockDim.x) {
    const int r = i / kDecodeCols, c = i - r * kDecodeCols;
    const int fc = blockIdx.x * kDecodeCols + c;
    if (fc >= F) continue;
    float g = 0.0f, u = 0.0f;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) {  // warp order: deterministic
      const float2 v = reinterpret_cast<const float2*>(red)[(size_t)(w * kDecodeTokens + r) * kDecodeCols + c];
      g += v.x;
      u += v.y;
    }
    const float hv = __fdividef(g, 1.0f + __expf(-g)) * u;  // the tensor-core epilogue's form
    __nv_bfloat16* out = a.h + (size_t)(sg.out_row0 + r) * a.h_ld + fc;
    const __nv_bfloat16 hi = __float2bfloat16_rn(hv);
    *out = hi;
    if (a.lo_off != 0) out[a.lo_off] = __float2bfloat16_rn(hv - __bfloat162float(hi));
  }
}

// grid (ceil(D / 256), segments, kDecodeSplits); 256 threads.  Dynamic shared memory: the split's
// part of the h rows as fp32 [4][f_len], then the partial sums [8 warps][4 rows][256 columns].
__global__ void __launch_bounds__(kDecodeWarps * 32)
decode_down_kernel(DecodeArgs a, int f_len) {
  extern __shared__ __align__(16) unsigned char smem[];
  const AxmSegment sg = a.segments[blockIdx.y];
  const int rows = sg.rows < kDecodeTokens ? sg.rows : kDecodeTokens;
  if (rows <= 0) return;
  const int D = a.D, F = a.F;
  const int f_lo = blockIdx.z * f_len;
  const int f_hi = f_lo + f_len < F ? f_lo + f_len : F;
  float* hs = reinterpret_cast<float*>(smem);
  float* red = hs + (size_t)kDecodeTokens * f_len;
  const int e_raw = sg.expert & ~AXM_SEG_ALT_A;
  const bool shared_w = e_raw >= a.routed_experts;
  const int e = shared_w ? e_raw - a.routed_experts : e_raw;
  const __nv_bfloat16* wd = (shared_w ? a.s_down : a.w_down) + (size_t)e * F * D;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < kDecodeTokens * f_len; i += blockDim.x) {
    const int r = i / f_len, c = i - r * f_len;
    float v = 0.0f;
    if (r < rows && f_lo + c < f_hi) {
      const __nv_bfloat16* p = a.h + (size_t)(sg.out_row0 + r) * a.h_ld + f_lo + c;
      v = __bfloat162float(*p);
      if (a.lo_off != 0) v += __bfloat162float(p[a.lo_off]);
    }
    hs[i] = v;
  }
  __syncthreads();
  const int dc = blockIdx.x * kDecodeCols + lane * 8;
  const bool live = dc < D;
  const int n = f_hi > f_lo ? f_hi - f_lo : 0;
  const int per = (n + kDecodeWarps - 1) / kDecodeWarps;
  const int c0 = warp * per, c1 = (c0 + per < n) ? c0 + per : n;
  float acc[kDecodeTokens][8];
#pragma unroll
  for (int r = 0; r < kDecodeTokens; ++r)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[r][j] = 0.0f;
  if (live) {
    const __nv_bfloat16* p = wd + (size_t)(f_lo + c0) * D + dc;
    int c = c0;
    for (; c + 7 < c1; c += 8) {  // eight 16-byte loads in flight per lane
      uint4 v[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] = ldg_stream(p + (size_t)q * D);
      p += (size_t)8 * D;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float w8[8];
        unpack8(v[q], w8);
#pragma unroll
        for (int r = 0; r < kDecodeTokens; ++r) {
          const float hv = hs[(size_t)r * f_len + c + q];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[r][j] = fmaf(hv, w8[j], acc[r][j]);
        }
      }
    }
    for (; c < c1; ++c) {
      float w8[8];
      unpack8(ldg_stream(p), w8);
      p += D;
#pragma unroll
      for (int r = 0; r < kDecodeTokens; ++r) {
        const float hv = hs[(size_t)r * f_len + c];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[r][j] = fmaf(hv, w8[j], acc[r][j]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kDecodeTokens; ++r)
#pragma unroll
    for (int j = 0; j < 8; ++j) red[(size_t)(warp * kDecodeTokens + r) * kDecodeCols + lane * 8 + j] = acc[r][j];
  __syncthreads();
  for (int i = tid; i < rows * kDecodeCols; i += blockDim.x) {
    const int r = i / kDecodeCols, c = i - r * kDecodeCols;
    const int d = blockIdx.x * kDecodeCols + c;
    if (d >= D) continue;
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) s += red[(size_t)(w * kDecodeTokens + r) * kDecodeCols + c];
    a.partial[((size_t)blockIdx.z * a.rows_total + sg.out_row0 + r) * D + d] = s;
  }
}

// o[row][d] = sum over the splits, in split order.
__global__ void __launch_bounds__(256)
decode_reduce_kernel(const float* __restrict__ partial, float* __restrict__ o, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.0f;
#pragma unroll
  for (int z = 0; z < kDecodeSplits; ++z) s += partial[(size_t)z * n + i];
  o[i] = s;
}

size_t decode_partial_bytes(const AxmMoeDesc* d) {
  if (d->tokens <= 0 || d->tokens > kDecodeTokens) return 0;
  const size_t rows = (size_t)d->tokens * (d->top_k + d->num_shared);
  return sizeof(float) * kDecodeSplits * rows * d->d_model;
}

// Whether a call of this shape takes the kernels above: few tokens, and shared memory for the
// activation rows (AXM_DECODE_GEMV=0 keeps the tensor-core kernels).
bool decode_path_wanted(const AxmMoeDesc* d) {
  static const bool enabled = [] {
    const char* e = getenv("AXM_DECODE_GEMV");
    return !(e != nullptr && e[0] == '0');
  }();
  if (!enabled || d->tokens <= 0 || d->tokens > kDecodeTokens) return false;
  const size_t red = sizeof(float) * kDecodeWarps * kDecodeTokens * kDecodeCols;
  const size_t gu = (size_t)kDecodeTokens * d->d_model * 2 + 2 * red;
  const size_t f_len = ((size_t)d->d_ff + kDecodeSplits - 1) / kDecodeSplits;
  const size_t dn = sizeof(float) * kDecodeTokens * f_len + red;
  return gu <= 200 * 1024 && dn <= 200 * 1024;
}

// h and o as axm_moe_expert_ffn leaves them, for a segment table whose segments hold at most
// kDecodeTokens rows each.  partial: decode_partial_bytes() of scratch.
int launch_decode_ffn(const AxmMoeDesc* d, const void* x_perm, const void* x_alt, const AxmSegment* segments,
                      int32_t num_segments, const void* w_gate, const void* w_up, const void* w_down,
                      const void* shared_gate, const void* shared_up, const void* shared_down, void* h, void* o,
                      void* partial, int32_t rows_total, cudaStream_t st, cudaEvent_t between) {
  if (!partial) return fail(AXM_ERR_WORKSPACE, "decode path without its scratch");
  if (num_segments <= 0 || rows_total <= 0) return AXM_OK;
  const int D = d->d_model, F = d->d_ff;
  const bool exact = (d->flags & AXM_FLAG_H_EXACT) != 0;
  DecodeArgs a;
  a.segments = segments;
  a.routed_experts = d->num_experts;
  a.D = D;
  a.F = F;
  a.x_perm = static_cast<const __nv_bfloat16*>(x_perm);
  a.x_alt = static_cast<const __nv_bfloat16*>(x_alt);
  a.w_gate = static_cast<const __nv_bfloat16*>(w_gate);
  a.w_up = static_cast<const __nv_bfloat16*>(w_up);
  a.w_down = static_cast<const __nv_bfloat16*>(w_down);
  a.s_gate = static_cast<const __nv_bfloat16*>(shared_gate);
  a.s_up = static_cast<const __nv_bfloat16*>(shared_up);
  a.s_down = static_cast<const __nv_bfloat16*>(shared_down);
  a.h = static_cast<__nv_bfloat16*>(h);
  a.h_ld = exact ? 2 * F : F;
  a.lo_off = exact ? F : 0;
  a.partial = static_cast<float*>(partial);
  a.rows_total = rows_total;
  const size_t red = sizeof(float) * kDecodeWarps * kDecodeTokens * kDecodeCols;
  const size_t gu_smem = (size_t)kDecodeTokens * D * 2 + 2 * red;
  const int f_len = (F + kDecodeSplits - 1) / kDecodeSplits;
  const size_t dn_smem = sizeof(float) * kDecodeTokens * f_len + red;
  static SmemLimitCache gu_cache = {}, dn_cache = {};
  int rc;
  if ((rc = ensure_dynamic_smem(reinterpret_cast<const void*>(decode_gate_up_kernel), gu_smem, &gu_cache, "decode_gate_up_kernel")))
    return rc;
  if ((rc = ensure_dynamic_smem(reinterpret_cast<const void*>(decode_down_kernel), dn_smem, &dn_cache, "decode_down_kernel")))
    return rc;
  decode_gate_up_kernel<<<dim3((F + kDecodeCols - 1) / kDecodeCols, num_segments), kDecodeWarps * 32, gu_smem, st>>>(a);
  if ((rc = check_launch("decode_gate_up_kernel"))) return rc;
  if (between) cudaEventRecord(between, st);
  decode_down_kernel<<<dim3((D + kDecodeCols - 1) / kDecodeCols, num_segments, kDecodeSplits), kDecodeWarps * 32,
                       dn_smem, st>>>(a, f_len);
  if ((rc = check_launch("decode_down_kernel"))) return rc;
  const long long n = (long long)rows_total * D;
  decode_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(static_cast<const float*>(partial),
                                                                   static_cast<float*>(o), n);
  return check_launch("decode_reduce_kernel");
}

}  // namespace axm
