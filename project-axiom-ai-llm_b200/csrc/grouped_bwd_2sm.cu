// Weight gradients of the expert FFN on CTA pairs (tcgen05.mma.cta_group::2):
//   dW[e][m, n] = sum over the expert's rows r of A[r, m] * B[r, n]
// used for dWd = h^T dO, dWg = x^T dG, dWu = x^T dU.  Both operands are MN-major (the rows
// are the reduction index), the output is fp32 in the weight's own [in][out] layout, as the
// reference engine's dense backward produces for its FFN weights
// (core/src/CUDA/kernel/backward_pass.cu:1013-1048; the engine has no MoE backward).
//
// Same product as kWGRAD of grouped_bwd.cu, which stays as the fallback.  There a CTA
// fills 48 KB of operands per k-block; here the two CTAs of a pair compute a 256 x 256
// tile together, each staging its own 128 rows of A^T and only half of B's columns:
// 32 KB per k-block and CTA, six stages instead of four.  A unit is (expert, n-tile,
// pair of m-tiles); with an odd number of m-tiles the last pair's second half idles.
// Segments must be padded to a multiple of 64 rows with zero rows (training layout).
// The fp32 tile leaves through a per-warp staging block and TMA stores, which clip at the
// matrix edge.  All waits are bounded; a wait that gives up winds both CTAs down and sets
// the status word to 9.
#include "gemm_2sm.cuh"

namespace axm {

namespace {

struct __align__(8) WgradShared2 {
  uint64_t full[kStages2];    // used in the leader: bytes of both CTAs land here
  uint64_t empty[kStages2];   // own: the leader's MMA commit arrives in both CTAs
  uint64_t tmem_full[2];      // own
  uint64_t tmem_empty[2];     // used in the leader: 4 epilogue warps of each CTA
  uint32_t tmem_base;
  int abort_flag;
  AxmSegment seg[kMaxSegments];
};

constexpr int kWgradStagingBytes = 4 * 4096;  // one 32 x 32 fp32 block per epilogue warp
constexpr size_t kWgrad2SmemBytes =
    1024 + (size_t)kStages2 * kStageBytes2 + kWgradStagingBytes + sizeof(WgradShared2);
static_assert(kWgrad2SmemBytes <= 227u * 1024u, "shared memory of the pair weight-gradient kernel");

struct Wgrad2Args {
  const AxmSegment* segments;
  int num_segments;
  int m_total;  // rows of one expert's gradient
  int n_total;  // columns
  int* status;
};

// fp32 accumulate, bf16 A and B both MN-major, N = 256, M = 256 over the pair
constexpr uint32_t kInstrDescWgrad2 = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) |
                                      ((uint32_t)(UMMA_N >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);

struct WgradUnit {
  int seg, n_tile, m_tile, a_m_tile;
  bool live;  // false: this half of the pair has no tile (odd number of m-tiles)
};

__device__ __forceinline__ WgradUnit decode_wgrad(int unit, int pairs_w, int n_tiles, int m_tiles, int rank) {
  const int per = pairs_w * n_tiles;
  WgradUnit u;
  u.seg = unit / per;
  const int local = unit - u.seg * per;
  u.n_tile = local / pairs_w;
  const int p = local - u.n_tile * pairs_w;
  u.m_tile = 2 * p + rank;
  u.live = u.m_tile < m_tiles;
  u.a_m_tile = u.live ? u.m_tile : 2 * p;  // an idle half still stages (the leader's) rows
  return u;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
grouped_wgrad_2sm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                         const __grid_constant__ CUtensorMap tm_out, Wgrad2Args args) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  unsigned char* staging = tiles + (size_t)kStages2 * kStageBytes2;  // 1024-byte aligned
  WgradShared2* sh = reinterpret_cast<WgradShared2*>(staging + kWgradStagingBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const uint32_t peer = rank ^ 1u;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;
  const int n_tiles = (args.n_total + UMMA_N - 1) / UMMA_N;
  const int m_tiles = (args.m_total + BM - 1) / BM;
  const int pairs_w = (m_tiles + 1) / 2;
  const int nseg = args.num_segments;
  const int total_units = nseg * pairs_w * n_tiles;

  for (int s = threadIdx.x; s < nseg; s += kGemmThreads) sh->seg[s] = args.segments[s];
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages2; ++i) {
      mbar_init(&sh->full[i], 1);
      mbar_init(&sh->empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh->tmem_full[i], 1);
      mbar_init(&sh->tmem_empty[i], 8);
    }
    sh->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
    tma_prefetch_desc(&tm_out);
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_alloc2(&sh->tmem_base, kTmemCols);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // barriers of both CTAs are initialised before anyone signals across
  tc_fence_after();

  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->abort_flag;
  auto raise_abort = [&]() {  // tell the peer too, so that the pair winds down together
    st_cluster_u32(map_to_cta(smem_u32(&sh->abort_flag), peer), 1u);
  };

  if (warp == 0) {
    // ---- TMA producer: own 128 columns of A^T, own half of B ---------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = cluster_id; ok && unit < total_units; unit += num_clusters) {
        const WgradUnit u = decode_wgrad(unit, pairs_w, n_tiles, m_tiles, (int)rank);
        const AxmSegment sg = sh->seg[u.seg];
        const int k_blocks = (sg.rows + BK - 1) / BK;
        const int a_col = u.a_m_tile * BM;
        const int b_col = u.n_tile * UMMA_N + (int)rank * 128;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1u, abort_flag)) {
            raise_abort();
            ok = false;
            break;
          }
          unsigned char* sa = tiles + (size_t)stage * kStageBytes2;
          unsigned char* sb = sa + kABytes;
          if (rank == 0) mbar_expect_tx(&sh->full[stage], 2 * kStageBytes2);
          const uint32_t bar = map_to_cta(smem_u32(&sh->full[stage]), 0);
          const int row = sg.a_row0 + kb * BK;
#pragma unroll
          for (int c = 0; c < 2; ++c) tma2_load_2d(sa + c * kBChunkBytes, &tm_a, bar, a_col + c * 64, row);
#pragma unroll
          for (int c = 0; c < 2; ++c) tma2_load_2d(sb + c * kBChunkBytes, &tm_b, bar, b_col + c * 64, row);
          if (++stage == kStages2) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the leader CTA only ---------------------------------------------
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int unit = cluster_id; ok && unit < total_units; unit += num_clusters) {
        const WgradUnit u = decode_wgrad(unit, pairs_w, n_tiles, m_tiles, 0);
        const int k_blocks = (sh->seg[u.seg].rows + BK - 1) / BK;
        if (!mbar_wait(&sh->tmem_empty[acc], acc_phase ^ 1u, abort_flag)) {
          raise_abort();
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)acc * UMMA_N;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&sh->full[stage], phase, abort_flag)) {
            raise_abort();
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + (size_t)stage * kStageBytes2);
          const uint32_t sb = sa + kABytes;
          // MN-major operands: 64-wide chunks 8192 B apart, 8-k groups 1024 B apart, +2048 B per 16 k
          const uint64_t da = make_smem_desc(sa, kBChunkBytes, 1024);
          const uint64_t db = make_smem_desc(sb, kBChunkBytes, 1024);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j)
            tc_mma2_bf16(d_tmem, da + (uint64_t)(j * 128), db + (uint64_t)(j * 128), kInstrDescWgrad2,
                         (kb > 0 || j > 0) ? 1u : 0u);
          tc_commit2(map_to_cta(smem_u32(&sh->empty[stage]), 0));
          tc_commit2(map_to_cta(smem_u32(&sh->empty[stage]), 1));
          if (++stage == kStages2) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        // with no rows nothing was issued and the commits arrive at once; the epilogue writes zeros
        tc_commit2(map_to_cta(smem_u32(&sh->tmem_full[acc]), 0));
        tc_commit2(map_to_cta(smem_u32(&sh->tmem_full[acc]), 1));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ---- epilogue: every CTA drains its own 128 accumulator rows -----------------------
    const int quad = warp & 3;
    unsigned char* stage_w = staging + (size_t)((warp - 2) & 3) * 4096;
    int acc = 0;
    uint32_t acc_phase = 0;
    const uint32_t leader_tmem_empty0 = map_to_cta(smem_u32(&sh->tmem_empty[0]), 0);
    const uint32_t leader_tmem_empty1 = map_to_cta(smem_u32(&sh->tmem_empty[1]), 0);
    for (int unit = cluster_id; unit < total_units; unit += num_clusters) {
      const WgradUnit u = decode_wgrad(unit, pairs_w, n_tiles, m_tiles, (int)rank);
      const AxmSegment sg = sh->seg[u.seg];
      const int k_blocks = (sg.rows + BK - 1) / BK;
      if (!__all_sync(0xffffffffu, mbar_wait(&sh->tmem_full[acc], acc_phase, abort_flag))) break;
      tc_fence_after();
      const int n0 = u.n_tile * UMMA_N;
      const int block_row0 = u.m_tile * BM + quad * 32;
      const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)acc * UMMA_N;
      if (u.live) {
#pragma unroll 1
        for (int c0 = 0; c0 < UMMA_N; c0 += 32) {
          uint32_t v[32];
          __syncwarp();
          tmem_ld32(t_addr + c0, v);
          tmem_ld_wait();
          if (k_blocks == 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0u;
          }
          // Lane = row of the 32 x 32 block; piece q of row r sits at q ^ (r & 7), the 128-byte
          // swizzle of the output map (and free of bank conflicts); one TMA store per block.
          if (lane == 0) bulk_wait_read();  // the previous block's store has read the buffer
          __syncwarp();
          if (n0 + c0 < args.n_total && block_row0 < args.m_total) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<uint4*>(stage_w + lane * 128 + ((q ^ (lane & 7)) << 4)) =
                  make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              tma_store_3d(&tm_out, stage_w, n0 + c0, block_row0, sg.expert & 0xffff);
              bulk_commit_group();
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc == 0 ? leader_tmem_empty0 : leader_tmem_empty1);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (lane == 0) bulk_wait_all();
  }

  // ---- drain: nobody leaves while the peer may still touch its shared memory or TMEM -----
  tc_fence_before();
  __syncthreads();
  if (sh->abort_flag != 0) {
    long long t0 = clock64();
    while (clock64() - t0 < 4000000LL) {
    }
    if (threadIdx.x == 0 && args.status != nullptr) atomicExch(args.status, 9);
  }
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc2(tmem_base, kTmemCols);
  }
}

// Row-major bf16 matrix [rows][cols]; box = 64 columns x 64 rows (rows = reduction index).
int map_kbox(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols) {
  const uint64_t dims[2] = {cols, rows};
  const uint64_t strides[1] = {cols * 2};
  const uint32_t box[2] = {64, 64};
  return encode_tensor_map(m, base, 2, dims, strides, box);
}

}  // namespace

// dW[e] = A^T . B over each segment's rows: A [rows_total][m_total], B [rows_total][n_total]
// (bf16), dW [experts][m_total][n_total] fp32.  AXM_ERR_DEVICE when pairs cannot be
// scheduled, so that the caller can fall back to the one-SM kernel.
int launch_wgrad_2sm(const AxmSegment* segments, int32_t num_segments, int32_t rows_total, int32_t experts,
                     const void* a, int32_t m_total, const void* b, int32_t n_total, void* d_w,
                     int32_t* status, cudaStream_t st) {
  static SmemLimitCache smem = {};
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(grouped_wgrad_2sm_kernel), kWgrad2SmemBytes,
                                   &smem, "grouped_wgrad_2sm_kernel"))
    return rc;
  const int grid = grid_2sm();
  if (grid < 0) return grid;
  if (grid < 2) return fail(AXM_ERR_DEVICE, "two-SM clusters cannot be scheduled on this device");
  CUtensorMap ma, mb, mo;
  int rc;
  if ((rc = map_kbox(&ma, a, (uint64_t)rows_total, (uint64_t)m_total))) return rc;
  if ((rc = map_kbox(&mb, b, (uint64_t)rows_total, (uint64_t)n_total))) return rc;
  const uint64_t dims[3] = {(uint64_t)n_total, (uint64_t)m_total, (uint64_t)experts};
  const uint64_t strides[2] = {(uint64_t)n_total * 4, (uint64_t)n_total * (uint64_t)m_total * 4};
  const uint32_t box[3] = {32, 32, 1};
  if ((rc = encode_tensor_map_f32(&mo, d_w, 3, dims, strides, box))) return rc;
  Wgrad2Args wa;
  wa.segments = segments;
  wa.num_segments = num_segments;
  wa.m_total = m_total;
  wa.n_total = n_total;
  wa.status = status;
  grouped_wgrad_2sm_kernel<<<grid, kGemmThreads, kWgrad2SmemBytes, st>>>(ma, mb, mo, wa);
  return check_launch("grouped_wgrad_2sm_kernel");
}

}  // namespace axm
