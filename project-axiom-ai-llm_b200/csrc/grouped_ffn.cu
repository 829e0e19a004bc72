// Grouped SwiGLU expert GEMMs for sm_100a: tcgen05.mma with the accumulator in
// tensor memory, operands staged in shared memory by TMA, one persistent CTA per
// SM walking a tile list built from the segment table.
//
// Stands in for the two phases of the reference engine's per-token dispatch
// kernel (core/src/CUDA/kernel/moe_router.cu:155-173 gate/up + SiLU*mul,
// 177-190 down projection), which run on CUDA cores there.  The weight layouts
// are consumed as the engine stores them ([E][D][F] and [E][F][D] with the
// output dimension contiguous, core/src/CUDA/util/gpu_types.cuh:152-157): the B
// operand is therefore "MN-major" and is described to the tensor core with the
// transposed canonical shared-memory layout; no weight re-layout happens.
//
//   kernel<true>  : h[r, f]  = SiLU(x_r . Wg[e][:, f]) * (x_r . Wu[e][:, f])   (bf16)
//   kernel<false> : o[r, d]  = h_r . Wd[e][:, d]                               (fp32)
//
// Tile: 128 rows x 256 accumulator columns x 64 reduction elements per stage.
// In the SwiGLU kernel the 256 columns are 128 gate columns followed by the 128
// up columns of the same f range, so one MMA produces both and the epilogue
// needs nothing but its own thread's registers.
//
// Roles (192 threads): warp 0 = TMA producer (one lane), warp 1 = MMA issuer
// (one lane) and TMEM owner, warps 2-5 = epilogue (TMEM -> registers -> global).
// Two 256-column accumulators alternate so that the epilogue of tile i overlaps
// the MMAs of tile i+1.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "gemm_common.cuh"

namespace axm {

struct GemmArgs {
  const AxmSegment* segments;
  int num_segments;
  int n_total;        // output columns: F (SwiGLU) or D (down)
  int k_total;        // reduction length: D (SwiGLU) or F (down)
  int routed_experts; // expert ids >= this address the shared-expert weights
  void* out;          // bf16 rows (SwiGLU) or fp32 rows (down)
  const AxmRemoteOut* remote;  // down kernel only: per-segment output redirect, or null
  __nv_bfloat16* save_g;  // SwiGLU kernel, training: also store the gate and up
  __nv_bfloat16* save_u;  // pre-activations (bf16, same shape as h), or null
  int* status;
  // Two-term SwiGLU intermediate (AXM_FLAG_H_EXACT): h rows are [hi | lo], hi = bf16(h),
  // lo = bf16(h - hi).  SwiGLU kernel: h_ld = row stride of h in elements, lo_off = column
  // offset of the lo half (0: one term).  Down kernel: with two_term every weight k-block is
  // used twice, against the hi rows (tm_a) and the lo rows (tm_a_alt).
  int h_ld;
  int lo_off;
  int two_term;
};


// Instruction descriptor: fp32 accumulate, bf16 A and B, A K-major, B MN-major,
// N = 256, M = 128.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | (0u << 15) | (1u << 16) |
                                ((uint32_t)(UMMA_N >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);


template <bool kSwiGLU>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_a_alt,
                    const __grid_constant__ CUtensorMap tm_b0, const __grid_constant__ CUtensorMap tm_b1,
                    const __grid_constant__ CUtensorMap tm_b0_sh, const __grid_constant__ CUtensorMap tm_b1_sh,
                    GemmArgs args) {
  extern __shared__ unsigned char smem_raw[];
  // 128-byte-swizzled tiles need 1024-byte alignment.
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  GemmShared* sh = reinterpret_cast<GemmShared*>(tiles + (size_t)kStages * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int BN_OUT = kSwiGLU ? 128 : 256;
  const int n_tiles = (args.n_total + BN_OUT - 1) / BN_OUT;
  const bool two_term = !kSwiGLU && args.two_term != 0;
  const int k_blocks = (two_term ? 2 : 1) * ((args.k_total + BK - 1) / BK);
  const int nseg = args.num_segments;

  // ---- set-up -------------------------------------------------------------------
  for (int s = threadIdx.x; s < nseg; s += kGemmThreads) sh->seg[s] = args.segments[s];
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&sh->full[i], 1);
      mbar_init(&sh->empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh->tmem_full[i], 1);
      mbar_init(&sh->tmem_empty[i], 4);
    }
    sh->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b0);
    if (kSwiGLU) tma_prefetch_desc(&tm_b1);
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(&sh->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int s = 0; s < nseg; ++s) {
      sh->tile_prefix[s] = acc;
      int rows = sh->seg[s].rows;
      acc += rows > 0 ? (rows + BM - 1) / BM : 0;
    }
    sh->tile_prefix[nseg] = acc;
    sh->total_tiles = acc * n_tiles;
    int ng = 0;
    for (int s = 0; s < nseg; ++s)
      if (s == 0 || sh->seg[s].expert != sh->seg[s - 1].expert) sh->group_first[ng++] = s;
    sh->group_first[ng] = nseg;
    sh->num_groups = ng;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const int total_tiles = sh->total_tiles;
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->abort_flag;

  if (warp == 0) {
    // ---- TMA producer ------------------------------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        TileCoord tc = decode_tile(sh, nseg, n_tiles, tile);
        const AxmSegment sg = sh->seg[tc.seg];
        const int e_raw = sg.expert & 0xffff;
        const bool shared_w = e_raw >= args.routed_experts;
        const int e = shared_w ? e_raw - args.routed_experts : e_raw;
        const bool alt_a = kSwiGLU && (sg.expert & AXM_SEG_ALT_A);
        const int a_row = (kSwiGLU ? sg.a_row0 : sg.out_row0) + tc.m_tile * BM;
        const CUtensorMap* ma = alt_a ? &tm_a_alt : &tm_a;
        const CUtensorMap* mb0 = shared_w ? &tm_b0_sh : &tm_b0;
        const CUtensorMap* mb1 = shared_w ? &tm_b1_sh : &tm_b1;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          unsigned char* sa = tiles + (size_t)stage * kStageBytes;
          unsigned char* sb = sa + kABytes;
          mbar_expect_tx(&sh->full[stage], kStageBytes);
          const int kk = (two_term ? (kb >> 1) : kb) * BK;
          tma_load_2d(sa, (two_term && (kb & 1)) ? &tm_a_alt : ma, &sh->full[stage], kk, a_row);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (kSwiGLU) {
              const CUtensorMap* mb = c < 2 ? mb0 : mb1;
              tma_load_3d(sb + c * kBChunkBytes, mb, &sh->full[stage],
                          tc.n_tile * BN_OUT + (c & 1) * 64, kk, e);
            } else {
              tma_load_3d(sb + c * kBChunkBytes, mb0, &sh->full[stage],
                          tc.n_tile * BN_OUT + c * 64, kk, e);
            }
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer --------------------------------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        if (!mbar_wait(&sh->tmem_empty[acc], acc_phase ^ 1u, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)acc * UMMA_N;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&sh->full[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + (size_t)stage * kStageBytes);
          const uint32_t sb = sa + kABytes;
          // A: K-major, 8-row groups 1024 bytes apart.  B: MN-major, 64-column
          // chunks 8192 bytes apart (leading), 8-k groups 1024 bytes apart (stride).
          const uint64_t da = make_smem_desc(sa, 16, 1024);
          const uint64_t db = make_smem_desc(sb, kBChunkBytes, 1024);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j) {
            // +32 bytes along K for A; +16 k-rows x 128 bytes for B
            tc_mma_bf16(d_tmem, da + (uint64_t)(j * 2), db + (uint64_t)(j * 128), kInstrDesc,
                        (kb > 0 || j > 0) ? 1u : 0u);
          }
          tc_commit(&sh->empty[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit(&sh->tmem_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ---- epilogue ------------------------------------------------------------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      TileCoord tc = decode_tile(sh, nseg, n_tiles, tile);
      const AxmSegment sg = sh->seg[tc.seg];
      // warp-uniform outcome: the tcgen05.ld below needs the whole warp
      if (!__all_sync(0xffffffffu, mbar_wait(&sh->tmem_full[acc], acc_phase, abort_flag))) break;
      tc_fence_after();
      const int row_in_seg = tc.m_tile * BM + quad * 32 + lane;
      const bool row_ok = row_in_seg < sg.rows;
      const int n0 = tc.n_tile * BN_OUT;
      size_t out_elem = (size_t)(sg.out_row0 + (row_ok ? row_in_seg : 0)) * args.n_total + n0;
      void* out_base = args.out;
      if constexpr (!kSwiGLU) {
        // Fused return: this segment's rows go straight into another buffer (a
        // peer GPU's return buffer under expert parallelism) with plain stores.
        if (args.remote != nullptr) {
          const AxmRemoteOut ro = args.remote[tc.seg];
          if (ro.base != nullptr) {
            out_base = ro.base;
            out_elem = (size_t)(ro.row0 + (row_ok ? row_in_seg : 0)) * args.n_total + n0;
          }
        }
      }
      const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)acc * UMMA_N;
#pragma unroll 1
      for (int c0 = 0; c0 < BN_OUT; c0 += 32) {
        uint32_t g[32];
        tmem_ld32(t_addr + c0, g);
        if constexpr (kSwiGLU) {
          uint32_t u[32];
          tmem_ld32(t_addr + 128 + c0, u);
          tmem_ld_wait();
          uint32_t packed[16], packed_lo[16];
          const bool with_lo = args.lo_off != 0;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
            float u0 = __uint_as_float(u[2 * j]), u1 = __uint_as_float(u[2 * j + 1]);
            float h0 = __fdividef(g0, 1.0f + __expf(-g0)) * u0;
            float h1 = __fdividef(g1, 1.0f + __expf(-g1)) * u1;
            packed[j] = pack_bf16(h0, h1);
            // second term: what the first bf16 rounding dropped
            packed_lo[j] = with_lo ? pack_bf16(h0 - bf16_lo(packed[j]), h1 - bf16_hi(packed[j])) : 0u;
          }
          if (row_ok) {
            __nv_bfloat16* out_row = static_cast<__nv_bfloat16*>(out_base) +
                                     (size_t)(sg.out_row0 + row_in_seg) * args.h_ld + n0;
#pragma unroll
            for (int q = 0; q < 4; ++q)
              if (n0 + c0 + q * 8 < args.n_total) {
                *reinterpret_cast<uint4*>(out_row + c0 + q * 8) =
                    make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                if (with_lo)
                  *reinterpret_cast<uint4*>(out_row + args.lo_off + c0 + q * 8) =
                      make_uint4(packed_lo[4 * q], packed_lo[4 * q + 1], packed_lo[4 * q + 2],
                                 packed_lo[4 * q + 3]);
              }
            if (args.save_g != nullptr) {
#pragma unroll
              for (int q = 0; q < 4; ++q)
                if (n0 + c0 + q * 8 < args.n_total) {
                  uint4 gv, uv;
                  gv.x = pack_bf16(__uint_as_float(g[8 * q + 0]), __uint_as_float(g[8 * q + 1]));
                  gv.y = pack_bf16(__uint_as_float(g[8 * q + 2]), __uint_as_float(g[8 * q + 3]));
                  gv.z = pack_bf16(__uint_as_float(g[8 * q + 4]), __uint_as_float(g[8 * q + 5]));
                  gv.w = pack_bf16(__uint_as_float(g[8 * q + 6]), __uint_as_float(g[8 * q + 7]));
                  uv.x = pack_bf16(__uint_as_float(u[8 * q + 0]), __uint_as_float(u[8 * q + 1]));
                  uv.y = pack_bf16(__uint_as_float(u[8 * q + 2]), __uint_as_float(u[8 * q + 3]));
                  uv.z = pack_bf16(__uint_as_float(u[8 * q + 4]), __uint_as_float(u[8 * q + 5]));
                  uv.w = pack_bf16(__uint_as_float(u[8 * q + 6]), __uint_as_float(u[8 * q + 7]));
                  *reinterpret_cast<uint4*>(args.save_g + out_elem + c0 + q * 8) = gv;
                  *reinterpret_cast<uint4*>(args.save_u + out_elem + c0 + q * 8) = uv;
                }
            }
          }
        } else {
          tmem_ld_wait();
          if (row_ok) {
            float* out_row = static_cast<float*>(out_base) + out_elem;
#pragma unroll
            for (int q = 0; q < 8; ++q)
              if (n0 + c0 + q * 4 < args.n_total)
                *reinterpret_cast<uint4*>(out_row + c0 + q * 4) =
                    make_uint4(g[4 * q], g[4 * q + 1], g[4 * q + 2], g[4 * q + 3]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->tmem_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // ---- drain -----------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (sh->abort_flag != 0) {
    // A wait gave up.  Give copies that are still in flight a bounded time to
    // land in this CTA's shared memory before it is released, then report.
    long long t0 = clock64();
    while (clock64() - t0 < 4000000LL) {
    }
    if (threadIdx.x == 0 && args.status != nullptr) atomicExch(args.status, kSwiGLU ? 1 : 2);
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host side ------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
        qr == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

static int encode_tensor_map_typed(CUtensorMap* m, CUtensorMapDataType type, const void* base, int rank,
                                   const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                                   CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  if (encode_fn() == nullptr) return fail(AXM_ERR_DEVICE, "cuTensorMapEncodeTiled entry point not found");
  cuuint64_t d[3], st[2];
  cuuint32_t b[3], es[3] = {1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    if (i + 1 < rank) st[i] = strides_bytes[i];
  }
  CUresult r = encode_fn()(m, type, (cuuint32_t)rank, const_cast<void*>(base),
                           d, st, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(AXM_ERR_ARGUMENT, "cuTensorMapEncodeTiled(rank %d) failed: %d", rank, (int)r);
  return AXM_OK;
}

int encode_tensor_map(CUtensorMap* m, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box) {
  return encode_tensor_map_typed(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, rank, dims, strides_bytes, box);
}

int encode_tensor_map_sw64(CUtensorMap* m, const void* base, int rank, const uint64_t* dims,
                           const uint64_t* strides_bytes, const uint32_t* box) {
  return encode_tensor_map_typed(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, rank, dims, strides_bytes, box,
                                 CU_TENSOR_MAP_SWIZZLE_64B);
}

int encode_tensor_map_f32(CUtensorMap* m, const void* base, int rank, const uint64_t* dims,
                          const uint64_t* strides_bytes, const uint32_t* box) {
  return encode_tensor_map_typed(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, rank, dims, strides_bytes, box);
}

int launch_expert_ffn_2sm(const AxmMoeDesc* d, const void* x_perm, int32_t a_rows, const void* x_alt,
                          int32_t alt_rows, const AxmSegment* segments, int32_t num_segments,
                          const void* w_gate, const void* w_up, const void* w_down,
                          const void* shared_gate, const void* shared_up, const void* shared_down,
                          void* h, void* o, int32_t rows_total, int32_t* status, cudaStream_t st,
                          cudaEvent_t between, void* save_g, void* save_u, int phases);

bool use_2sm_kernels() {
  static int v = -1;
  if (v < 0) {
    // two-SM (cta_group::2) kernels are the default forward path; AXM_GEMM_2SM=0 selects
    // the one-SM kernels of this file (which the fused return always uses)
    const char* e = getenv("AXM_GEMM_2SM");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

// Row-major bf16 matrix [rows][cols]; box = 64 columns x box_rows rows.
static int make_map_2d(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols,
                       uint32_t box_rows, uint64_t ld = 0) {
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {(ld ? ld : cols) * 2};  // ld: distance between rows in elements
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                           strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(AXM_ERR_ARGUMENT, "cuTensorMapEncodeTiled(2d) failed: %d", (int)r);
  return AXM_OK;
}

// Weights [experts][k_rows][n_cols] bf16, n contiguous; box = 64 n x 64 k x 1 expert.
static int make_map_3d(CUtensorMap* m, const void* base, uint64_t experts, uint64_t k_rows,
                       uint64_t n_cols) {
  cuuint64_t dims[3] = {n_cols, k_rows, experts};
  cuuint64_t strides[2] = {n_cols * 2, n_cols * k_rows * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)BK, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims,
                           strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(AXM_ERR_ARGUMENT, "cuTensorMapEncodeTiled(3d) failed: %d", (int)r);
  return AXM_OK;
}

// phases: bit 0 = gate/up projection with the SiLU*mul epilogue (writes h), bit 1 = down
// projection (reads h, writes o).  Callers that overlap other work with the down projection
// launch the two separately, with different segment tables if they like.
int launch_expert_ffn_phases(const AxmMoeDesc* d, const void* x_perm, int32_t a_rows, const void* x_alt,
                             int32_t alt_rows, const AxmSegment* segments, int32_t num_segments,
                             const void* w_gate, const void* w_up, const void* w_down,
                             const void* shared_gate, const void* shared_up, const void* shared_down,
                             void* h, void* o, int32_t rows_total, int32_t* status, cudaStream_t st,
                             cudaEvent_t between, const AxmRemoteOut* remote, void* save_g, void* save_u,
                             int phases);

int launch_expert_ffn(const AxmMoeDesc* d, const void* x_perm, int32_t a_rows, const void* x_alt,
                      int32_t alt_rows, const AxmSegment* segments, int32_t num_segments,
                      const void* w_gate, const void* w_up, const void* w_down,
                      const void* shared_gate, const void* shared_up, const void* shared_down,
                      void* h, void* o, int32_t rows_total, int32_t* status, cudaStream_t st,
                      cudaEvent_t between, const AxmRemoteOut* remote, void* save_g, void* save_u) {
  return launch_expert_ffn_phases(d, x_perm, a_rows, x_alt, alt_rows, segments, num_segments, w_gate, w_up, w_down,
                                  shared_gate, shared_up, shared_down, h, o, rows_total, status, st, between,
                                  remote, save_g, save_u, 3);
}

int launch_expert_ffn_phases(const AxmMoeDesc* d, const void* x_perm, int32_t a_rows, const void* x_alt,
                             int32_t alt_rows, const AxmSegment* segments, int32_t num_segments,
                             const void* w_gate, const void* w_up, const void* w_down,
                             const void* shared_gate, const void* shared_up, const void* shared_down,
                             void* h, void* o, int32_t rows_total, int32_t* status, cudaStream_t st,
                             cudaEvent_t between, const AxmRemoteOut* remote, void* save_g, void* save_u,
                             int phases) {
  if (remote == nullptr && use_2sm_kernels())
    return launch_expert_ffn_2sm(d, x_perm, a_rows, x_alt, alt_rows, segments, num_segments, w_gate, w_up,
                                 w_down, shared_gate, shared_up, shared_down, h, o, rows_total, status, st,
                                 between, save_g, save_u, phases);
  if (encode_fn() == nullptr) return fail(AXM_ERR_DEVICE, "cuTensorMapEncodeTiled entry point not found");
  const int D = d->d_model, F = d->d_ff, E = d->num_experts, S = d->num_shared;
  CUtensorMap a1, a1_alt, g, u, g_sh, u_sh, a2, dn, dn_sh;
  int rc;
  if ((rc = make_map_2d(&a1, x_perm, (uint64_t)(a_rows > 0 ? a_rows : 1), D, BM))) return rc;
  if (x_alt != nullptr && alt_rows > 0) {
    if ((rc = make_map_2d(&a1_alt, x_alt, alt_rows, D, BM))) return rc;
  } else {
    a1_alt = a1;
  }
  if ((rc = make_map_3d(&g, w_gate, E, D, F))) return rc;
  if ((rc = make_map_3d(&u, w_up, E, D, F))) return rc;
  if ((rc = make_map_3d(&dn, w_down, E, F, D))) return rc;
  if (S > 0) {
    if ((rc = make_map_3d(&g_sh, shared_gate, S, D, F))) return rc;
    if ((rc = make_map_3d(&u_sh, shared_up, S, D, F))) return rc;
    if ((rc = make_map_3d(&dn_sh, shared_down, S, F, D))) return rc;
  } else {
    g_sh = g;
    u_sh = u;
    dn_sh = dn;
  }
  const bool exact = (d->flags & AXM_FLAG_H_EXACT) != 0;
  const uint64_t h_ld = exact ? 2 * (uint64_t)F : (uint64_t)F;
  CUtensorMap a2_lo;
  if ((rc = make_map_2d(&a2, h, rows_total, F, BM, h_ld))) return rc;
  a2_lo = a2;
  if (exact && (rc = make_map_2d(&a2_lo, static_cast<const __nv_bfloat16*>(h) + F, rows_total, F, BM, h_ld)))
    return rc;

  static SmemLimitCache smem_swiglu = {}, smem_down = {};
  if ((rc = ensure_dynamic_smem(reinterpret_cast<const void*>(grouped_gemm_kernel<true>), kGemmSmemBytes,
                                &smem_swiglu, "grouped_gemm_kernel<SwiGLU>")))
    return rc;
  if ((rc = ensure_dynamic_smem(reinterpret_cast<const void*>(grouped_gemm_kernel<false>), kGemmSmemBytes,
                                &smem_down, "grouped_gemm_kernel<down>")))
    return rc;
  const int grid = sm_count();
  GemmArgs ga;
  ga.segments = segments;
  ga.num_segments = num_segments;
  ga.routed_experts = E;
  ga.status = status;
  ga.remote = nullptr;
  ga.save_g = static_cast<__nv_bfloat16*>(save_g);
  ga.save_u = static_cast<__nv_bfloat16*>(save_u);
  ga.n_total = F;
  ga.k_total = D;
  ga.out = h;
  ga.h_ld = (int)h_ld;
  ga.lo_off = exact ? F : 0;
  ga.two_term = 0;
  if (phases & 1) {
    grouped_gemm_kernel<true><<<grid, kGemmThreads, kGemmSmemBytes, st>>>(a1, a1_alt, g, u, g_sh, u_sh, ga);
    if ((rc = check_launch("grouped_gemm_kernel<swiglu>"))) return rc;
  }
  if (between != nullptr) cudaEventRecord(between, st);
  if (!(phases & 2)) return AXM_OK;
  ga.n_total = D;
  ga.k_total = F;
  ga.out = o;
  ga.remote = remote;
  ga.save_g = nullptr;
  ga.save_u = nullptr;
  ga.two_term = exact ? 1 : 0;
  grouped_gemm_kernel<false><<<grid, kGemmThreads, kGemmSmemBytes, st>>>(a2, a2_lo, dn, dn, dn_sh, dn_sh, ga);
  return check_launch("grouped_gemm_kernel<down>");
}

}  // namespace axm

using namespace axm;

extern "C" int axm_moe_expert_ffn(const AxmMoeDesc* desc, const void* x_perm, int32_t a_rows,
                                  const void* x_alt, int32_t alt_rows,
                                  const AxmSegment* segments, int32_t num_segments,
                                  const void* w_gate, const void* w_up, const void* w_down,
                                  const void* shared_gate, const void* shared_up,
                                  const void* shared_down, void* h, void* o, int32_t rows_total,
                                  int32_t* status, void* stream) {
  if (desc == nullptr) return fail(AXM_ERR_ARGUMENT, "desc is null");
  if (desc->d_model <= 0 || desc->d_ff <= 0 || desc->d_model % 8 || desc->d_ff % 8)
    return fail(AXM_ERR_ARGUMENT, "d_model and d_ff must be positive multiples of 8");
  if (desc->num_experts <= 0) return fail(AXM_ERR_ARGUMENT, "num_experts must be positive");
  if (num_segments < 0 || num_segments > kMaxSegments)
    return fail(AXM_ERR_ARGUMENT, "num_segments %d not in 0..%d", num_segments, kMaxSegments);
  if (!x_perm || !segments || !w_gate || !w_up || !w_down || !h || !o)
    return fail(AXM_ERR_ARGUMENT, "axm_moe_expert_ffn: null pointer");
  if (desc->num_shared > 0 && (!shared_gate || !shared_up || !shared_down))
    return fail(AXM_ERR_ARGUMENT, "axm_moe_expert_ffn: shared experts without weights");
  if (rows_total <= 0 || num_segments == 0) return AXM_OK;
  if (int rc = require_device()) return rc;
  return launch_expert_ffn(desc, x_perm, a_rows, x_alt, alt_rows, segments, num_segments, w_gate,
                           w_up, w_down, shared_gate, shared_up, shared_down, h, o, rows_total,
                           status, static_cast<cudaStream_t>(stream), nullptr, nullptr, nullptr, nullptr);
}

extern "C" int axm_moe_expert_ffn_remote(const AxmMoeDesc* desc, const void* x_perm, int32_t a_rows,
                                         const void* x_alt, int32_t alt_rows,
                                         const AxmSegment* segments, int32_t num_segments,
                                         const void* w_gate, const void* w_up, const void* w_down,
                                         const void* shared_gate, const void* shared_up,
                                         const void* shared_down, void* h, void* o,
                                         int32_t rows_total, const AxmRemoteOut* remote_out,
                                         int32_t* status, void* stream) {
  if (int rc = axm_moe_expert_ffn(desc, x_perm, a_rows, x_alt, alt_rows, segments, 0, w_gate, w_up,
                                  w_down, shared_gate, shared_up, shared_down, h, o, rows_total,
                                  status, stream))
    return rc;  // argument checks only: zero segments launch nothing
  if (num_segments < 0 || num_segments > kMaxSegments)
    return fail(AXM_ERR_ARGUMENT, "num_segments %d not in 0..%d", num_segments, kMaxSegments);
  if (rows_total <= 0 || num_segments == 0) return AXM_OK;
  if (int rc = require_device()) return rc;
  return launch_expert_ffn(desc, x_perm, a_rows, x_alt, alt_rows, segments, num_segments, w_gate,
                           w_up, w_down, shared_gate, shared_up, shared_down, h, o, rows_total,
                           status, static_cast<cudaStream_t>(stream), nullptr, remote_out, nullptr, nullptr);
}
