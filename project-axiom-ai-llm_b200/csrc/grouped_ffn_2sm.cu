// Two-SM form of the forward grouped GEMMs: thread-block clusters of two CTAs issue
// tcgen05.mma.cta_group::2 (M = 256 across the pair, N = 256).  Each CTA stages its
// own 128 activation rows and only HALF of the weight tile (128 of the 256 columns);
// the tensor core of the leader CTA reads both halves, so the shared-memory fill per
// FLOP drops from 48 KB to 32 KB per k-block and the pipeline gets six stages.
// No cluster multicast is used anywhere: every CTA issues its own TMA loads, and the
// leader signals the peer's barriers with ordinary (non-multicast) tcgen05.commit
// instructions addressed to the peer's shared memory.
//
// Same operator as grouped_ffn.cu (core/src/CUDA/kernel/moe_router.cu:155-190 of the
// reference engine); same weight layouts consumed as stored (MN-major B operand).
// The two m-tiles of a pair are any two consecutive m-tiles of one expert group, so
// ragged experts cost no extra padding; an odd tile count leaves one half idle.
//
// Modes: kModeDown (h . Wd, fp32 rows), kModeSwiGLU (x . [Wg | Wu] -> h), and kModeDX, the
// backward input gradient dXp = dG . Wg^T + dU . Wu^T: one accumulator over a reduction of
// 2F (first dG with Wg, then dU with Wu), the weights read K-major as stored ([E][D][F], the
// reduction index f contiguous), each CTA staging 128 of the tile's 256 output columns d.
// kModeDH is the other backward product on the rows, dH = dO . Wd^T (Wd as stored, [E][F][D], is
// K-major for it), with the SwiGLU derivative in the epilogue: the saved g, u come in and dG, dU
// go out through a per-warp staging block in row-contiguous 64-byte runs (see grouped_bwd.cu).
// The one-SM kernels move 48 KB per k-block and CTA through L2; at about 16 TB/s summed over
// the SMs that, not the tensor pipe, bounds them - the pair form moves 32 KB.
#include <mutex>

#include "gemm_2sm.cuh"

namespace axm {

enum { kModeDown = 0, kModeSwiGLU = 1, kModeDX = 2, kModeDH = 3 };

struct Gemm2Args {
  const AxmSegment* segments;
  int num_segments;
  int n_total;
  int k_total;
  int routed_experts;
  void* out;
  __nv_bfloat16* save_g;  // training: also store the gate / up pre-activations (bf16), or null;
  __nv_bfloat16* save_u;  //   kModeDH: the saved pre-activations, read
  void* out1;             // kModeDH: dU (out is dG)
  int* status;
  // Two-term SwiGLU intermediate (AXM_FLAG_H_EXACT): h rows are [hi | lo] of 2 * n_total bf16,
  // hi = bf16(h), lo = bf16(h - hi).  kModeSwiGLU: h_ld is the row stride of h in elements and
  // lo_off the column offset of the lo half (0: one term).  kModeDown: with two_term the
  // reduction runs over both halves, k-block by k-block (hi, lo, hi, lo, ...) against the same
  // weight rows, so the accumulator receives (hi + lo) . Wd.
  int h_ld;
  int lo_off;
  int two_term;
  // kModeDown, calls with so few rows that the tile list would leave most CTA pairs idle: the
  // reduction is cut into k_splits ranges of k-blocks, every (tile, range) is a unit of its own,
  // and range z stores its partial sums at out + z * split_stride floats (a small kernel adds
  // them in range order).  1: the whole reduction in one unit, stored at out.
  int k_splits;
  long long split_stride;
};

constexpr int kStagesDh = 5;  // operand stages of kModeDH (one stage's room goes to its epilogue blocks)
constexpr int kDhSlots = 3;   // 4 KiB slots (g / dG block + u / dU block) per epilogue warp

// fp32 accumulate, bf16 A (K-major) and B (MN-major), N = 256, M = 256 over the pair
constexpr uint32_t kInstrDesc2 = (1u << 4) | (1u << 7) | (1u << 10) | (0u << 15) | (1u << 16) |
                                 ((uint32_t)(UMMA_N >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);

// the same with a K-major B operand (kModeDX)
constexpr uint32_t kInstrDesc2KB = kInstrDesc2 & ~(1u << 16);

struct UnitCoord {
  int seg;      // segment of this CTA's m-tile (valid only if live)
  int m_tile;
  int n_tile;
  int seg0;     // first segment of the group (for the weights' expert id)
  bool live;    // false: this half of the pair has no tile
  int a_seg, a_m_tile;  // rows to load even when not live (the pair's first tile)
};

__device__ __forceinline__ void find_tile(const GemmShared2* sh, int s0, int s1, int m_idx, int* seg,
                                          int* m_tile) {
  int a = s0, b = s1 - 1;
  while (a < b) {
    int mid = (a + b + 1) >> 1;
    if (sh->tile_prefix[mid] <= m_idx) a = mid; else b = mid - 1;
  }
  *seg = a;
  *m_tile = m_idx - sh->tile_prefix[a];
}

__device__ __forceinline__ UnitCoord decode_unit(const GemmShared2* sh, int n_tiles, int unit, int rank) {
  int lo = 0, hi = sh->num_groups - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (sh->pair_prefix[mid] * n_tiles <= unit) lo = mid; else hi = mid - 1;
  }
  const int s0 = sh->group_first[lo], s1 = sh->group_first[lo + 1];
  const int base = sh->tile_prefix[s0];
  const int mt = sh->tile_prefix[s1] - base;
  const int pairs = sh->pair_prefix[lo + 1] - sh->pair_prefix[lo];
  const int local = unit - sh->pair_prefix[lo] * n_tiles;
  UnitCoord uc;
  uc.n_tile = local / pairs;
  const int p = local - uc.n_tile * pairs;
  uc.seg0 = s0;
  find_tile(sh, s0, s1, base + 2 * p, &uc.a_seg, &uc.a_m_tile);
  uc.live = 2 * p + rank < mt;
  if (uc.live) {
    find_tile(sh, s0, s1, base + 2 * p + rank, &uc.seg, &uc.m_tile);
    uc.a_seg = uc.seg;
    uc.a_m_tile = uc.m_tile;
  } else {
    uc.seg = uc.a_seg;
    uc.m_tile = uc.a_m_tile;
  }
  return uc;
}

template <int kMode>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
grouped_gemm_2sm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_a_alt,
                        const __grid_constant__ CUtensorMap tm_b0, const __grid_constant__ CUtensorMap tm_b1,
                        const __grid_constant__ CUtensorMap tm_b0_sh, const __grid_constant__ CUtensorMap tm_b1_sh,
                        const __grid_constant__ CUtensorMap tm_g, const __grid_constant__ CUtensorMap tm_u,
                        const __grid_constant__ CUtensorMap tm_dg, const __grid_constant__ CUtensorMap tm_du,
                        Gemm2Args args) {
  constexpr bool kSwiGLU = kMode == kModeSwiGLU;
  constexpr bool kDX = kMode == kModeDX;
  constexpr bool kDH = kMode == kModeDH;
  constexpr bool kBKmajor = kDX || kDH;  // weights read K-major: one box of 64 k x 128 columns per CTA
  // kModeDH gives one operand stage to the epilogue's g / u / dG / dU blocks
  constexpr int kSt = kDH ? kStagesDh : kStages2;
  extern __shared__ unsigned char smem_raw[];
  // both CTAs of a pair compute the same offsets, so their tiles sit at the same place
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  GemmShared2* sh = reinterpret_cast<GemmShared2*>(tiles + (size_t)kSt * kStageBytes2);
  // kModeDH: behind the control block, 1024-byte aligned, per epilogue warp kDhSlots slots of
  // 4 KiB (a 32 x 32 bf16 block of g / dG and one of u / dU, filled and drained by TMA with
  // 64-byte swizzle), then one mbarrier per warp and slot
  unsigned char* staging = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(sh + 1) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* dh_bars = reinterpret_cast<uint64_t*>(staging + (size_t)4 * kDhSlots * 4096);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const uint32_t peer = rank ^ 1u;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;
  constexpr int BN_OUT = kSwiGLU ? 128 : 256;
  const int k_splits = (kMode == kModeDown && args.k_splits > 1) ? args.k_splits : 1;
  // with k_splits > 1 the "column tile" index that orders the units carries the split in its
  // low part: n_tiles counts (column tile, split) pairs
  const int n_tiles = ((args.n_total + BN_OUT - 1) / BN_OUT) * k_splits;
  const int kb_half = (args.k_total + BK - 1) / BK;
  const bool two_term = kMode == kModeDown && args.two_term != 0;
  // kModeDX: dG x Wg, then dU x Wu; two-term down: every weight k-block twice (hi rows, lo rows)
  const int k_blocks = (kDX || two_term) ? 2 * kb_half : kb_half;
  const int nseg = args.num_segments;

  for (int s = threadIdx.x; s < nseg; s += kGemmThreads) sh->seg[s] = args.segments[s];
  if (threadIdx.x == 0) {
    for (int i = 0; i < kSt; ++i) {
      mbar_init(&sh->full[i], 1);
      mbar_init(&sh->empty[i], 1);
    }
    if (kDH) {
      for (int i = 0; i < 4 * kDhSlots; ++i) mbar_init(&dh_bars[i], 1);
      tma_prefetch_desc(&tm_g);
      tma_prefetch_desc(&tm_u);
      tma_prefetch_desc(&tm_dg);
      tma_prefetch_desc(&tm_du);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh->tmem_full[i], 1);
      mbar_init(&sh->tmem_empty[i], 8);
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
    tmem_alloc2(&sh->tmem_base, kTmemCols);
    tmem_relinquish2();
  }
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int s = 0; s < nseg; ++s) {
      sh->tile_prefix[s] = acc;
      int rows = sh->seg[s].rows;
      acc += rows > 0 ? (rows + BM - 1) / BM : 0;
    }
    sh->tile_prefix[nseg] = acc;
    int ng = 0;
    for (int s = 0; s < nseg; ++s)
      if (s == 0 || sh->seg[s].expert != sh->seg[s - 1].expert) sh->group_first[ng++] = s;
    sh->group_first[ng] = nseg;
    sh->num_groups = ng;
    int pairs = 0;
    for (int g = 0; g < ng; ++g) {
      sh->pair_prefix[g] = pairs;
      int mt = sh->tile_prefix[sh->group_first[g + 1]] - sh->tile_prefix[sh->group_first[g]];
      pairs += (mt + 1) / 2;
    }
    sh->pair_prefix[ng] = pairs;
    sh->total_units = pairs * n_tiles;
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // barriers of both CTAs are initialised before anyone signals across
  tc_fence_after();

  const int total_units = sh->total_units;
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->abort_flag;
  auto raise_abort = [&]() {  // tell the peer too, so that the pair winds down together
    st_cluster_u32(map_to_cta(smem_u32(&sh->abort_flag), peer), 1u);
  };

  if (warp == 0) {
    // ---- TMA producer (each CTA: its rows of A, its half of B) ---------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = cluster_id; ok && unit < total_units; unit += num_clusters) {
        const UnitCoord uc = decode_unit(sh, n_tiles, unit, (int)rank);
        const AxmSegment sg = sh->seg[uc.a_seg];
        const int e_raw = sh->seg[uc.seg0].expert & 0xffff;
        const bool shared_w = e_raw >= args.routed_experts;
        const int e = shared_w ? e_raw - args.routed_experts : e_raw;
        const bool alt_a = kSwiGLU && (sg.expert & AXM_SEG_ALT_A);
        const int a_row = (kSwiGLU ? sg.a_row0 : sg.out_row0) + uc.a_m_tile * BM;
        const CUtensorMap* ma = alt_a ? &tm_a_alt : &tm_a;
        // SwiGLU: the leader stages the gate columns, the peer the up columns of the same f range;
        // down: the leader stages columns n0..n0+127, the peer n0+128..n0+255
        const CUtensorMap* mb = kSwiGLU ? (rank == 0 ? (shared_w ? &tm_b0_sh : &tm_b0)
                                                     : (shared_w ? &tm_b1_sh : &tm_b1))
                                        : (shared_w ? &tm_b0_sh : &tm_b0);
        const int n_col = (uc.n_tile / k_splits) * BN_OUT + (kSwiGLU ? 0 : (int)rank * 128);
        const int kb_per = (k_blocks + k_splits - 1) / k_splits;
        const int kb0 = (uc.n_tile % k_splits) * kb_per;
        const int kb1 = kb0 + kb_per < k_blocks ? kb0 + kb_per : k_blocks;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1u, abort_flag)) {
            raise_abort();
            ok = false;
            break;
          }
          unsigned char* sa = tiles + (size_t)stage * kStageBytes2;
          unsigned char* sb = sa + kABytes;
          // the leader's barrier counts the bytes of both CTAs
          if (rank == 0) mbar_expect_tx(&sh->full[stage], 2 * kStageBytes2);
          const uint32_t bar = map_to_cta(smem_u32(&sh->full[stage]), 0);
          if constexpr (kDH) {
            tma2_load_2d(sa, &tm_a, bar, kb * BK, a_row);
            tma2_load_3d(sb, &tm_b0, bar, kb * BK, n_col, e);
          } else if constexpr (kDX) {
            const bool second = kb >= kb_half;
            const int kk = (second ? kb - kb_half : kb) * BK;
            tma2_load_2d(sa, second ? &tm_a_alt : &tm_a, bar, kk, a_row);
            // K-major weights: one box of 64 k x 128 output columns
            tma2_load_3d(sb, second ? &tm_b1 : &tm_b0, bar, kk, n_col, e);
          } else {
            const int kk = (two_term ? (kb >> 1) : kb) * BK;
            tma2_load_2d(sa, (two_term && (kb & 1)) ? &tm_a_alt : ma, bar, kk, a_row);
            tma2_load_3d(sb, mb, bar, n_col, kk, e);
            tma2_load_3d(sb + kBChunkBytes, mb, bar, n_col + 64, kk, e);
          }
          if (++stage == kSt) {
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
        if (!mbar_wait(&sh->tmem_empty[acc], acc_phase ^ 1u, abort_flag)) {
          raise_abort();
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)acc * UMMA_N;
        int kb0 = 0, kb1 = k_blocks;
        if (k_splits > 1) {
          const UnitCoord uc = decode_unit(sh, n_tiles, unit, 0);
          const int kb_per = (k_blocks + k_splits - 1) / k_splits;
          kb0 = (uc.n_tile % k_splits) * kb_per;
          kb1 = kb0 + kb_per < k_blocks ? kb0 + kb_per : k_blocks;
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&sh->full[stage], phase, abort_flag)) {
            raise_abort();
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + (size_t)stage * kStageBytes2);
          const uint32_t sb = sa + kABytes;
          const uint64_t da = make_smem_desc(sa, 16, 1024);
          // MN-major B: 64-wide chunks 8192 B apart, +2048 B per 16 k; K-major B (kModeDX): like A
          const uint64_t db = kBKmajor ? make_smem_desc(sb, 16, 1024) : make_smem_desc(sb, kBChunkBytes, 1024);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j)
            tc_mma2_bf16(d_tmem, da + (uint64_t)(j * 2), db + (uint64_t)(j * (kBKmajor ? 2 : 128)),
                         kBKmajor ? kInstrDesc2KB : kInstrDesc2, (kb > kb0 || j > 0) ? 1u : 0u);
          // free this stage in both CTAs once the MMAs that read it are done
          tc_commit2(map_to_cta(smem_u32(&sh->empty[stage]), 0));
          tc_commit2(map_to_cta(smem_u32(&sh->empty[stage]), 1));
          if (++stage == kSt) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit2(map_to_cta(smem_u32(&sh->tmem_full[acc]), 0));
        tc_commit2(map_to_cta(smem_u32(&sh->tmem_full[acc]), 1));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ---- epilogue: every CTA drains its own 128 accumulator rows -----------------------
    const int quad = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t dh_issued = 0, dh_used = 0;  // kModeDH: blocks of g / u requested (lane 0) and consumed
    const uint32_t leader_tmem_empty0 = map_to_cta(smem_u32(&sh->tmem_empty[0]), 0);
    const uint32_t leader_tmem_empty1 = map_to_cta(smem_u32(&sh->tmem_empty[1]), 0);
    for (int unit = cluster_id; unit < total_units; unit += num_clusters) {
      const UnitCoord uc = decode_unit(sh, n_tiles, unit, (int)rank);
      const AxmSegment sg = sh->seg[uc.seg];
      // kModeDH: this warp's 32 rows of the tile, and the loads of its first two blocks of g / u,
      // requested before the accumulator is waited for
      const int dh_row0 = sg.out_row0 + uc.m_tile * BM + quad * 32;
      const int dh_rows_left = uc.live ? sg.rows - (uc.m_tile * BM + quad * 32) : 0;
      const bool dh_full = dh_rows_left >= 32;
      const int dh_n0 = uc.n_tile * BN_OUT;
      auto dh_valid = [&](int jb) { return dh_rows_left > 0 && dh_n0 + jb * 32 < args.n_total; };
      auto dh_issue = [&](int jb) {  // lane 0 only; blocks are issued in the order they are used
        const int slot = (int)(dh_issued % kDhSlots);
        unsigned char* dst = staging + (size_t)(((warp - 2) & 3) * kDhSlots + slot) * 4096;
        uint64_t* bar = &dh_bars[((warp - 2) & 3) * kDhSlots + slot];
        mbar_expect_tx(bar, 4096);
        tma_load_2d(dst, &tm_g, bar, dh_n0 + jb * 32, dh_row0);
        tma_load_2d(dst + 2048, &tm_u, bar, dh_n0 + jb * 32, dh_row0);
        ++dh_issued;
      };
      if constexpr (kDH) {
        if (dh_full && lane == 0) {
          bulk_wait_read();  // the previous tile's last stores have read their slots
          if (dh_valid(0)) dh_issue(0);
          if (dh_valid(1)) dh_issue(1);
        }
      }
      if (!__all_sync(0xffffffffu, mbar_wait(&sh->tmem_full[acc], acc_phase, abort_flag))) break;
      tc_fence_after();
      const int row_in_seg = uc.m_tile * BM + quad * 32 + lane;
      const bool row_ok = uc.live && row_in_seg < sg.rows;
      const int n0 = (uc.n_tile / k_splits) * BN_OUT;
      // range z of a split reduction stores into its own copy of the output
      const size_t out_elem = (size_t)(sg.out_row0 + (row_ok ? row_in_seg : 0)) * args.n_total + n0 +
                              (k_splits > 1 ? (size_t)(uc.n_tile % k_splits) * (size_t)args.split_stride : 0);
      const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)acc * UMMA_N;
      if constexpr (kDH) {
        // The SwiGLU derivative with the saved g, u: dG = dH u s (1 + g (1 - s)), dU = dH g s,
        // s = sigmoid(g) (core/src/CUDA/kernel/swiglu.cu:34-55 of the reference engine).
        // g and u come in, and dG and dU go out, as 32 x 32 bf16 blocks moved by TMA (64-byte
        // swizzle: 16-byte piece q of row r sits at r * 64 + ((q ^ (r / 2 % 4)) * 16, so a lane
        // reading its own row meets no bank conflict): the epilogue warps issue no global loads
        // or stores of their own.  Each warp owns kDhSlots slots; the loads run two blocks ahead.
        unsigned char* slots = staging + (size_t)((warp - 2) & 3) * kDhSlots * 4096;
        auto piece_smem = [&](int row, int piece) { return row * 64 + ((piece ^ ((row >> 1) & 3)) << 4); };
#pragma unroll 1
        for (int jb = 0; jb < BN_OUT / 32; ++jb) {
          if (!dh_valid(jb)) break;  // columns ascend: nothing valid follows
          const int slot = (int)(dh_used % kDhSlots);
          unsigned char* g_s = slots + (size_t)slot * 4096;
          unsigned char* u_s = g_s + 2048;
          const int c0 = jb * 32;
          uint32_t v[32];
          if (dh_full) {
            if (!__all_sync(0xffffffffu, mbar_wait(&dh_bars[((warp - 2) & 3) * kDhSlots + slot],
                                                   (dh_used / kDhSlots) & 1u, abort_flag)))
              break;
          } else {
            // a block with fewer than 32 rows of the segment (segments not padded to 32 rows):
            // the lane fetches its own row, and stores it itself below
            __syncwarp();
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 gv = make_uint4(0, 0, 0, 0), uv = make_uint4(0, 0, 0, 0);
              if (lane < dh_rows_left && n0 + c0 + q * 8 < args.n_total) {
                const size_t el = (size_t)(dh_row0 + lane) * args.n_total + n0 + c0 + q * 8;
                gv = __ldg(reinterpret_cast<const uint4*>(args.save_g + el));
                uv = __ldg(reinterpret_cast<const uint4*>(args.save_u + el));
              }
              *reinterpret_cast<uint4*>(g_s + piece_smem(lane, q)) = gv;
              *reinterpret_cast<uint4*>(u_s + piece_smem(lane, q)) = uv;
            }
          }
          __syncwarp();
          tmem_ld32(t_addr + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4* gp = reinterpret_cast<uint4*>(g_s + piece_smem(lane, q));
            uint4* up = reinterpret_cast<uint4*>(u_s + piece_smem(lane, q));
            const uint4 gv = *gp;
            const uint4 uv = *up;
            const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
            const uint32_t uw[4] = {uv.x, uv.y, uv.z, uv.w};
            uint32_t dgw[4], duw[4];
#pragma unroll
            for (int pp = 0; pp < 4; ++pp) {
              float r0[2], r1[2];
#pragma unroll
              for (int hh = 0; hh < 2; ++hh) {
                const float gval = hh ? bf16_hi(gw[pp]) : bf16_lo(gw[pp]);
                const float uval = hh ? bf16_hi(uw[pp]) : bf16_lo(uw[pp]);
                const float dh = __uint_as_float(v[q * 8 + pp * 2 + hh]);
                const float sg_ = __fdividef(1.0f, 1.0f + __expf(-gval));
                r0[hh] = dh * uval * (sg_ * (1.0f + gval * (1.0f - sg_)));  // dG
                r1[hh] = dh * gval * sg_;                                    // dU
              }
              dgw[pp] = pack_bf16(r0[0], r0[1]);
              duw[pp] = pack_bf16(r1[0], r1[1]);
            }
            if (dh_full) {
              *gp = make_uint4(dgw[0], dgw[1], dgw[2], dgw[3]);  // in place: the lane's own row
              *up = make_uint4(duw[0], duw[1], duw[2], duw[3]);
            } else if (lane < dh_rows_left && n0 + c0 + q * 8 < args.n_total) {
              const size_t el = (size_t)(dh_row0 + lane) * args.n_total + n0 + c0 + q * 8;
              *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(args.out) + el) = make_uint4(dgw[0], dgw[1], dgw[2], dgw[3]);
              *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(args.out1) + el) = make_uint4(duw[0], duw[1], duw[2], duw[3]);
            }
          }
          if (dh_full) {
            fence_proxy_async();  // the stores below read these bytes through the async proxy
            __syncwarp();
            if (lane == 0) {
              // the slot two blocks ahead is the one block jb - 1 was stored from: that store
              // was issued a whole block ago and has read its bytes
              if (jb + 2 < BN_OUT / 32 && dh_valid(jb + 2)) {
                bulk_wait_read();
                dh_issue(jb + 2);
              }
              tma_store_2d(&tm_dg, g_s, n0 + c0, dh_row0);
              tma_store_2d(&tm_du, u_s, n0 + c0, dh_row0);
              bulk_commit_group();
            }
            ++dh_used;
          }
        }
      } else if (uc.live) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN_OUT; c0 += 32) {
          uint32_t g[32];
          __syncwarp();
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
              __nv_bfloat16* out_row = static_cast<__nv_bfloat16*>(args.out) +
                                       (size_t)(sg.out_row0 + row_in_seg) * args.h_ld + n0;
#pragma unroll
              for (int q = 0; q < 4; ++q)
                if (n0 + c0 + q * 8 < args.n_total) {
                  // streaming store: h is not read again by this kernel and must not push
                  // the activations and weights the other CTAs share out of L2
                  __stcs(reinterpret_cast<uint4*>(out_row + c0 + q * 8),
                         make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]));
                  if (with_lo)
                    __stcs(reinterpret_cast<uint4*>(out_row + args.lo_off + c0 + q * 8),
                           make_uint4(packed_lo[4 * q], packed_lo[4 * q + 1], packed_lo[4 * q + 2],
                                      packed_lo[4 * q + 3]));
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
                    __stcs(reinterpret_cast<uint4*>(args.save_g + out_elem + c0 + q * 8), gv);
                    __stcs(reinterpret_cast<uint4*>(args.save_u + out_elem + c0 + q * 8), uv);
                  }
              }
            }
          } else {
            tmem_ld_wait();
            if (row_ok) {
              float* out_row = static_cast<float*>(args.out) + out_elem;
#pragma unroll
              for (int q = 0; q < 8; ++q)
                if (n0 + c0 + q * 4 < args.n_total)
                  __stcs(reinterpret_cast<uint4*>(out_row + c0 + q * 4),
                         make_uint4(g[4 * q], g[4 * q + 1], g[4 * q + 2], g[4 * q + 3]));
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
    if (kDH && lane == 0) bulk_wait_all();  // the last dG / dU blocks have left shared memory
  }

  // ---- drain: nobody leaves while the peer may still touch its shared memory or TMEM -----
  tc_fence_before();
  __syncthreads();
  if (sh->abort_flag != 0) {
    long long t0 = clock64();
    while (clock64() - t0 < 4000000LL) {
    }
    if (threadIdx.x == 0 && args.status != nullptr) atomicExch(args.status, kSwiGLU ? 6 : (kDX ? 8 : (kDH ? 10 : 7)));
  }
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc2(tmem_base, kTmemCols);
  }
}

// o[i] = sum over the ranges of a split down projection, in range order.
__global__ void __launch_bounds__(256)
down_split_reduce_kernel(const float* __restrict__ partial, float* __restrict__ o, long long n, int splits) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.0f;
  for (int z = 0; z < splits; ++z) s += partial[(size_t)z * n + i];
  o[i] = s;
}

// Scratch for the partial sums of a split down projection, lent for the duration of one layer
// call by a caller that owns a workspace (axm_moe_forward); other callers run unsplit.
constexpr int kSplitTokensMax = 8;
constexpr int kSplitsMax = 4;
static thread_local void* g_split_scratch = nullptr;
static thread_local size_t g_split_scratch_bytes = 0;
void set_down_split_scratch(void* p, size_t bytes) {
  g_split_scratch = p;
  g_split_scratch_bytes = bytes;
}
// Ranges the down projection of this call is cut into on `pairs` CTA pairs (1: not split).
int down_splits_for(const AxmMoeDesc* d, int pairs) {
  const int D = d->d_model, F = d->d_ff, E = d->num_experts, S = d->num_shared;
  if ((d->flags & AXM_FLAG_H_EXACT) || d->tokens <= 0 || d->tokens > kSplitTokensMax || pairs <= 0) return 1;
  const long long rows_max = (long long)d->tokens * (d->top_k + S);
  const int n_tiles = (D + 255) / 256, k_blocks = (F + BK - 1) / BK;
  const long long units_max = (rows_max < E + S ? rows_max : (long long)(E + S)) * n_tiles;
  if (units_max <= 0) return 1;
  int splits = (int)((2LL * pairs + units_max - 1) / units_max);  // about two units per CTA pair
  if (splits > kSplitsMax) splits = kSplitsMax;
  while (splits > 1 && (splits - 1) * ((k_blocks + splits - 1) / splits) >= k_blocks) --splits;  // no empty range
  return splits < 1 ? 1 : splits;
}
size_t down_split_scratch_bytes(const AxmMoeDesc* d) {
  if (d->tokens <= 0 || d->tokens > kSplitTokensMax) return 0;
  return sizeof(float) * kSplitsMax * (size_t)d->tokens * (d->top_k + d->num_shared) * d->d_model;
}

// Row-major bf16 matrix of `rows` x `cols` whose rows are `ld` elements apart (0: cols).
static int map2_rows(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint64_t ld = 0) {
  const uint64_t dims[2] = {cols, rows};
  const uint64_t strides[1] = {(ld ? ld : cols) * 2};
  const uint32_t box[2] = {64, (uint32_t)BM};
  return encode_tensor_map(m, base, 2, dims, strides, box);
}
static int map2_weights(CUtensorMap* m, const void* base, uint64_t experts, uint64_t k_rows, uint64_t n_cols) {
  const uint64_t dims[3] = {n_cols, k_rows, experts};
  const uint64_t strides[2] = {n_cols * 2, n_cols * k_rows * 2};
  const uint32_t box[3] = {64, (uint32_t)BK, 1};
  return encode_tensor_map(m, base, 3, dims, strides, box);
}

// Number of CTAs to launch (two per cluster), or 0 when pairs cannot be scheduled; a
// negative status when the shared-memory limit could not be raised.  Function attributes
// and the occupancy answer belong to a device's context, so both are kept per device.
int grid_2sm() {
  static SmemLimitCache smem_swiglu = {}, smem_down = {};
  static int cached[64];  // 0 = not asked yet, else grid + 1
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(grouped_gemm_2sm_kernel<kModeSwiGLU>), kGemm2SmemBytes,
                                   &smem_swiglu, "grouped_gemm_2sm_kernel<SwiGLU>"))
    return rc;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(grouped_gemm_2sm_kernel<kModeDown>), kGemm2SmemBytes,
                                   &smem_down, "grouped_gemm_2sm_kernel<down>"))
    return rc;
  const int dev = current_device();
  if (dev >= 0 && dev < 64 && cached[dev] != 0) return cached[dev] - 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(sm_count() & ~1), 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = kGemm2SmemBytes;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, grouped_gemm_2sm_kernel<kModeSwiGLU>, &cfg);
  if (e != cudaSuccess) {
    cudaGetLastError();
    clusters = 0;
  }
  const int want = sm_count() / 2;
  const int grid = 2 * (clusters < want ? clusters : want);
  if (dev >= 0 && dev < 64) cached[dev] = grid + 1;
  return grid;
}

int launch_expert_ffn_2sm(const AxmMoeDesc* d, const void* x_perm, int32_t a_rows, const void* x_alt,
                          int32_t alt_rows, const AxmSegment* segments, int32_t num_segments,
                          const void* w_gate, const void* w_up, const void* w_down,
                          const void* shared_gate, const void* shared_up, const void* shared_down,
                          void* h, void* o, int32_t rows_total, int32_t* status, cudaStream_t st,
                          cudaEvent_t between, void* save_g, void* save_u, int phases) {
  const int grid = grid_2sm();
  if (grid < 0) return grid;  // status, message already set
  if (grid < 2) return fail(AXM_ERR_DEVICE, "two-SM clusters cannot be scheduled on this device");
  const int D = d->d_model, F = d->d_ff, E = d->num_experts, S = d->num_shared;
  CUtensorMap a1, a1_alt, g, u, g_sh, u_sh, a2, dn, dn_sh;
  int rc;
  if ((rc = map2_rows(&a1, x_perm, (uint64_t)(a_rows > 0 ? a_rows : 1), D))) return rc;
  if (x_alt != nullptr && alt_rows > 0) {
    if ((rc = map2_rows(&a1_alt, x_alt, alt_rows, D))) return rc;
  } else {
    a1_alt = a1;
  }
  if ((rc = map2_weights(&g, w_gate, E, D, F))) return rc;
  if ((rc = map2_weights(&u, w_up, E, D, F))) return rc;
  if ((rc = map2_weights(&dn, w_down, E, F, D))) return rc;
  if (S > 0) {
    if ((rc = map2_weights(&g_sh, shared_gate, S, D, F))) return rc;
    if ((rc = map2_weights(&u_sh, shared_up, S, D, F))) return rc;
    if ((rc = map2_weights(&dn_sh, shared_down, S, F, D))) return rc;
  } else {
    g_sh = g;
    u_sh = u;
    dn_sh = dn;
  }
  const bool exact = (d->flags & AXM_FLAG_H_EXACT) != 0;
  const uint64_t h_ld = exact ? 2 * (uint64_t)F : (uint64_t)F;
  CUtensorMap a2_lo;
  if ((rc = map2_rows(&a2, h, rows_total, F, h_ld))) return rc;
  a2_lo = a2;
  if (exact && (rc = map2_rows(&a2_lo, static_cast<const __nv_bfloat16*>(h) + F, rows_total, F, h_ld))) return rc;
  Gemm2Args ga;
  ga.h_ld = (int)h_ld;
  ga.lo_off = exact ? F : 0;
  ga.two_term = 0;
  ga.k_splits = 1;
  ga.split_stride = 0;
  ga.segments = segments;
  ga.num_segments = num_segments;
  ga.routed_experts = E;
  ga.status = status;
  ga.n_total = F;
  ga.k_total = D;
  ga.out = h;
  ga.save_g = static_cast<__nv_bfloat16*>(save_g);
  ga.save_u = static_cast<__nv_bfloat16*>(save_u);
  if (phases & 1) {
    grouped_gemm_2sm_kernel<kModeSwiGLU><<<grid, kGemmThreads, kGemm2SmemBytes, st>>>(a1, a1_alt, g, u, g_sh, u_sh, a1,
                                                                                      a1, a1, a1, ga);
    if ((rc = check_launch("grouped_gemm_2sm_kernel<swiglu>"))) return rc;
  }
  if (between != nullptr) cudaEventRecord(between, st);
  if (!(phases & 2)) return AXM_OK;
  ga.n_total = D;
  ga.k_total = F;
  ga.out = o;
  ga.save_g = nullptr;
  ga.save_u = nullptr;
  ga.out1 = nullptr;
  ga.two_term = exact ? 1 : 0;
  ga.k_splits = 1;
  ga.split_stride = 0;
  // A call with a handful of tokens touches few experts, each with one tile pair: fewer units than
  // CTA pairs (one token, top-2, D = 4096: 32 units for 74 pairs).  The reduction is then cut
  // into up to four ranges that run as units of their own and are added afterwards, if the
  // caller has lent the scratch for their partial sums.
  int splits = down_splits_for(d, grid / 2);
  const size_t split_bytes = sizeof(float) * (size_t)splits * rows_total * D;
  if (splits > 1 && (g_split_scratch == nullptr || g_split_scratch_bytes < split_bytes)) splits = 1;
  if (splits > 1) {
    ga.k_splits = splits;
    ga.split_stride = (long long)rows_total * D;
    ga.out = g_split_scratch;
  }
  grouped_gemm_2sm_kernel<kModeDown><<<grid, kGemmThreads, kGemm2SmemBytes, st>>>(a2, a2_lo, dn, dn, dn_sh, dn_sh, a2,
                                                                                  a2, a2, a2, ga);
  if (int rc2 = check_launch("grouped_gemm_2sm_kernel<down>")) return rc2;
  if (splits > 1) {
    const long long n = (long long)rows_total * D;
    down_split_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(static_cast<const float*>(g_split_scratch),
                                                                         static_cast<float*>(o), n, splits);
    return check_launch("down_split_reduce_kernel");
  }
  return AXM_OK;
}

// Weights [experts][n_rows][k_cols] read K-major by a CTA pair: box = 64 k x 128 n x 1 expert.
static int map2_weights_kmajor(CUtensorMap* m, const void* base, uint64_t experts, uint64_t n_rows,
                               uint64_t k_cols) {
  const uint64_t dims[3] = {k_cols, n_rows, experts};
  const uint64_t strides[2] = {k_cols * 2, k_cols * n_rows * 2};
  const uint32_t box[3] = {64, 128, 1};
  return encode_tensor_map(m, base, 3, dims, strides, box);
}

// dH = dO . Wd[e]^T with the SwiGLU derivative in the epilogue: dG, dU (bf16) from the saved g, u.
// AXM_ERR_DEVICE when pairs cannot be scheduled, so that the caller can fall back.
constexpr size_t kGemm2DhSmemBytes = 1024 + (size_t)kStagesDh * kStageBytes2 + sizeof(GemmShared2) + 1024 +
                                     (size_t)4 * kDhSlots * 4096 + 8 * 4 * kDhSlots;
static_assert(kGemm2DhSmemBytes <= 227u * 1024u, "shared memory of the pair dH kernel");

int launch_bwd_dh_2sm(const AxmMoeDesc* d, const AxmSegment* segments, int32_t num_segments,
                      int32_t rows_total, const void* d_o, const void* w_down, const void* g, const void* u,
                      void* d_g, void* d_u, int32_t* status, cudaStream_t st) {
  static SmemLimitCache smem_dh = {};
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(grouped_gemm_2sm_kernel<kModeDH>), kGemm2DhSmemBytes,
                                   &smem_dh, "grouped_gemm_2sm_kernel<dH>"))
    return rc;
  const int grid = grid_2sm();
  if (grid < 0) return grid;
  if (grid < 2) return fail(AXM_ERR_DEVICE, "two-SM clusters cannot be scheduled on this device");
  const int D = d->d_model, F = d->d_ff, E = d->num_experts;
  CUtensorMap m_do, m_wd, m_g, m_u, m_dg, m_du;
  int rc;
  if ((rc = map2_rows(&m_do, d_o, (uint64_t)rows_total, D))) return rc;
  if ((rc = map2_weights_kmajor(&m_wd, w_down, E, F, D))) return rc;
  {
    // 32 x 32 bf16 blocks of the [rows][F] tensors the epilogue reads and writes, 64-byte swizzle
    const uint64_t dims[2] = {(uint64_t)F, (uint64_t)rows_total};
    const uint64_t strides[1] = {(uint64_t)F * 2};
    const uint32_t box[2] = {32, 32};
    if ((rc = encode_tensor_map_sw64(&m_g, g, 2, dims, strides, box))) return rc;
    if ((rc = encode_tensor_map_sw64(&m_u, u, 2, dims, strides, box))) return rc;
    if ((rc = encode_tensor_map_sw64(&m_dg, d_g, 2, dims, strides, box))) return rc;
    if ((rc = encode_tensor_map_sw64(&m_du, d_u, 2, dims, strides, box))) return rc;
  }
  Gemm2Args ga;
  ga.segments = segments;
  ga.num_segments = num_segments;
  ga.routed_experts = E;
  ga.status = status;
  ga.n_total = F;
  ga.k_total = D;
  ga.out = d_g;
  ga.out1 = d_u;
  ga.save_g = static_cast<__nv_bfloat16*>(const_cast<void*>(g));
  ga.save_u = static_cast<__nv_bfloat16*>(const_cast<void*>(u));
  ga.h_ld = F;
  ga.lo_off = 0;
  ga.two_term = 0;
  ga.k_splits = 1;
  ga.split_stride = 0;
  grouped_gemm_2sm_kernel<kModeDH><<<grid, kGemmThreads, kGemm2DhSmemBytes, st>>>(m_do, m_do, m_wd, m_wd, m_wd,
                                                                                  m_wd, m_g, m_u, m_dg, m_du, ga);
  return check_launch("grouped_gemm_2sm_kernel<dH>");
}

// dXp[r, :] = dG[r, :] . Wg[e]^T + dU[r, :] . Wu[e]^T over the segments' rows (fp32 out).
// Returns AXM_ERR_DEVICE when pairs cannot be scheduled, so that the caller can fall back.
int launch_bwd_dx_2sm(const AxmMoeDesc* d, const AxmSegment* segments, int32_t num_segments,
                      int32_t rows_total, const void* d_g, const void* d_u, const void* w_gate,
                      const void* w_up, void* d_xp, int32_t* status, cudaStream_t st) {
  static SmemLimitCache smem_dx = {};
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(grouped_gemm_2sm_kernel<kModeDX>), kGemm2SmemBytes,
                                   &smem_dx, "grouped_gemm_2sm_kernel<dX>"))
    return rc;
  const int grid = grid_2sm();
  if (grid < 0) return grid;
  if (grid < 2) return fail(AXM_ERR_DEVICE, "two-SM clusters cannot be scheduled on this device");
  const int D = d->d_model, F = d->d_ff, E = d->num_experts;
  CUtensorMap m_dg, m_du, m_wg, m_wu;
  int rc;
  if ((rc = map2_rows(&m_dg, d_g, (uint64_t)rows_total, F))) return rc;
  if ((rc = map2_rows(&m_du, d_u, (uint64_t)rows_total, F))) return rc;
  if ((rc = map2_weights_kmajor(&m_wg, w_gate, E, D, F))) return rc;
  if ((rc = map2_weights_kmajor(&m_wu, w_up, E, D, F))) return rc;
  Gemm2Args ga;
  ga.segments = segments;
  ga.num_segments = num_segments;
  ga.routed_experts = E;
  ga.status = status;
  ga.n_total = D;
  ga.k_total = F;
  ga.out = d_xp;
  ga.save_g = nullptr;
  ga.save_u = nullptr;
  ga.out1 = nullptr;
  ga.h_ld = D;
  ga.lo_off = 0;
  ga.two_term = 0;
  ga.k_splits = 1;
  ga.split_stride = 0;
  grouped_gemm_2sm_kernel<kModeDX><<<grid, kGemmThreads, kGemm2SmemBytes, st>>>(m_dg, m_du, m_wg, m_wu, m_wg,
                                                                                m_wu, m_dg, m_dg, m_dg, m_dg, ga);
  return check_launch("grouped_gemm_2sm_kernel<dX>");
}

}  // namespace axm
