// Backward grouped GEMMs of the expert FFN on the sm_100a tensor cores: same
// persistent, warp-specialised tcgen05 / TMEM / TMA skeleton as the forward
// kernels (grouped_ffn.cu), with the operand forms the gradients need.
//
// The reference engine has no MoE backward (its backward pass covers the dense
// FFN only, core/src/CUDA/kernel/backward_pass.cu:1701-2005); the three products
// follow its dense conventions: fp32 weight gradients in the weights' own
// [in][out] layout (backward_pass.cu:1013-1048) and the SiLU*mul derivative of
// core/src/CUDA/kernel/swiglu.cu:34-55.
//
//   kDH    dH[r, f] = dO_r . Wd[e][f, :]        A rows K-major, B = Wd as stored is
//          K-major ([F][D], reduction over D contiguous).  The epilogue applies the
//          SwiGLU derivative with the saved g, u and stores dG, dU (bf16).
//   kDX    dXp[r, d] = dG_r . Wg[e][d, :] + dU_r . Wu[e][d, :]   one accumulator,
//          reduction over 2F (first dG x Wg, then dU x Wu); B K-major; fp32 out.
//          By default this product runs on CTA pairs instead (kModeDX of
//          grouped_ffn_2sm.cu); the kernel here is the one-SM fallback.
//   kWGRAD dW[e][m, n] = sum_r A[r, m] * B[r, n] over the expert's rows: both
//          operands MN-major (rows are the reduction index).  Used for
//          dWd = h^T dO, dWg = x^T dG, dWu = x^T dU.  Segments must be padded to
//          a multiple of 64 rows with zero rows (training layout), so that the
//          reduction has no ragged tail.  Its fp32 tiles leave through shared
//          memory and TMA stores (whole 128-byte row pieces) instead of per-lane
//          stores, which had kept the L1 store path busier than the tensor pipe.
//
// kDH's epilogue reads g, u and writes dG, dU through a per-warp staging block in shared
// memory so that global requests are row-contiguous; with one 16-byte piece of a different
// row per lane the L1 path, not the tensor pipe, had set the pace (eight epilogue warps
// instead of four did not help, which is how that showed).
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "gemm_common.cuh"

namespace axm {

enum { kDH = 0, kDX = 1, kWGRAD = 2 };

struct BwdArgs {
  const AxmSegment* segments;
  int num_segments;
  int n_total;  // output columns: F (kDH), D (kDX), N of the weight gradient (kWGRAD)
  int k_total;  // reduction length: D (kDH), F per half (kDX); unused for kWGRAD
  int m_total;  // kWGRAD: rows of one expert's weight gradient
  void* out0;   // kDH: dG (bf16)   kDX: dXp (fp32)   kWGRAD: dW (fp32 [E][m_total][n_total])
  void* out1;   // kDH: dU (bf16)
  const __nv_bfloat16* g;  // kDH: saved pre-activations [rows][F]
  const __nv_bfloat16* u;
  int* status;
};

template <int MODE>
struct BwdCfg {
  static constexpr int kEpiWarps = 4;
  static constexpr int kThreads = 64 + 32 * kEpiWarps;
  // per epilogue warp 4 KiB: kWGRAD one 32 x 32 fp32 block (128-byte swizzled rows),
  // kDH two 32 x 32 bf16 blocks (g / dG and u / dU)
  static constexpr int kStagingBytes = MODE == kDX ? 0 : 4 * 4096;
  static constexpr size_t kSmemBytes = kGemmSmemBytes + kStagingBytes;
};

template <int MODE>
__device__ __forceinline__ TileCoord decode_bwd(const GemmShared* sh, int nseg, int n_tiles,
                                                int m_tiles, int linear) {
  if constexpr (MODE == kWGRAD) {
    TileCoord tc;
    const int per = m_tiles * n_tiles;
    tc.seg = linear / per;
    const int local = linear - tc.seg * per;
    tc.n_tile = local / m_tiles;
    tc.m_tile = local - tc.n_tile * m_tiles;
    return tc;
  } else {
    return decode_tile(sh, nseg, n_tiles, linear);
  }
}

// tm_a1 carries, for kWGRAD, the fp32 map of the output [E][m_total][n_total] (box 32 x 32 x 1).
template <int MODE>
__global__ void __launch_bounds__(BwdCfg<MODE>::kThreads, 1)
grouped_bwd_kernel(const __grid_constant__ CUtensorMap tm_a0, const __grid_constant__ CUtensorMap tm_a1,
                   const __grid_constant__ CUtensorMap tm_b0, const __grid_constant__ CUtensorMap tm_b1,
                   BwdArgs args) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  unsigned char* staging = tiles + (size_t)kStages * kStageBytes;  // 1024-byte aligned
  GemmShared* sh = reinterpret_cast<GemmShared*>(staging + BwdCfg<MODE>::kStagingBytes);
  constexpr int kThreads = BwdCfg<MODE>::kThreads;
  constexpr int kEpiWarps = BwdCfg<MODE>::kEpiWarps;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles = (args.n_total + UMMA_N - 1) / UMMA_N;
  const int m_tiles_w = (args.m_total + BM - 1) / BM;  // kWGRAD only
  const int kb_half = (args.k_total + BK - 1) / BK;
  const int nseg = args.num_segments;

  for (int s = threadIdx.x; s < nseg; s += kThreads) sh->seg[s] = args.segments[s];
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&sh->full[i], 1);
      mbar_init(&sh->empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh->tmem_full[i], 1);
      mbar_init(&sh->tmem_empty[i], kEpiWarps);
    }
    sh->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_a0);
    tma_prefetch_desc(&tm_b0);
    if (MODE == kWGRAD) tma_prefetch_desc(&tm_a1);
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
    int ng = 0;
    for (int s = 0; s < nseg; ++s)
      if (s == 0 || sh->seg[s].expert != sh->seg[s - 1].expert) sh->group_first[ng++] = s;
    sh->group_first[ng] = nseg;
    sh->num_groups = ng;
    sh->total_tiles = MODE == kWGRAD ? nseg * m_tiles_w * n_tiles : acc * n_tiles;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const int total_tiles = sh->total_tiles;
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->abort_flag;

  // k-blocks of a tile: fixed for the dgrad kernels, the expert's rows for kWGRAD
  auto tile_k_blocks = [&](const AxmSegment& sg) {
    if constexpr (MODE == kDH) return kb_half;
    else if constexpr (MODE == kDX) return 2 * kb_half;
    else return (sg.rows + BK - 1) / BK;
  };

  if (warp == 0) {
    // ---- TMA producer ------------------------------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const TileCoord tc = decode_bwd<MODE>(sh, nseg, n_tiles, m_tiles_w, tile);
        const AxmSegment sg = sh->seg[tc.seg];
        const int e = sg.expert & 0xffff;
        const int k_blocks = tile_k_blocks(sg);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          unsigned char* sa = tiles + (size_t)stage * kStageBytes;
          unsigned char* sb = sa + kABytes;
          mbar_expect_tx(&sh->full[stage], kStageBytes);
          if constexpr (MODE == kDH) {
            tma_load_2d(sa, &tm_a0, &sh->full[stage], kb * BK, sg.a_row0 + tc.m_tile * BM);
            tma_load_3d(sb, &tm_b0, &sh->full[stage], kb * BK, tc.n_tile * UMMA_N, e);
          } else if constexpr (MODE == kDX) {
            const bool second = kb >= kb_half;
            const int kk = (second ? kb - kb_half : kb) * BK;
            tma_load_2d(sa, second ? &tm_a1 : &tm_a0, &sh->full[stage], kk, sg.a_row0 + tc.m_tile * BM);
            tma_load_3d(sb, second ? &tm_b1 : &tm_b0, &sh->full[stage], kk, tc.n_tile * UMMA_N, e);
          } else {
            const int row = sg.a_row0 + kb * BK;
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tma_load_2d(sa + c * kBChunkBytes, &tm_a0, &sh->full[stage], tc.m_tile * BM + c * 64, row);
#pragma unroll
            for (int c = 0; c < 4; ++c)
              tma_load_2d(sb + c * kBChunkBytes, &tm_b0, &sh->full[stage], tc.n_tile * UMMA_N + c * 64, row);
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
      constexpr bool kAmn = MODE == kWGRAD, kBmn = MODE == kWGRAD;
      constexpr uint32_t idesc = instr_desc(kAmn, kBmn);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const TileCoord tc = decode_bwd<MODE>(sh, nseg, n_tiles, m_tiles_w, tile);
        const int k_blocks = tile_k_blocks(sh->seg[tc.seg]);
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
          // K-major operand: 8-row groups 1024 B apart, +32 B per 16 k.
          // MN-major operand: 64-wide chunks 8192 B apart, 8-k groups 1024 B apart, +2048 B per 16 k.
          const uint64_t da = kAmn ? make_smem_desc(sa, kBChunkBytes, 1024) : make_smem_desc(sa, 16, 1024);
          const uint64_t db = kBmn ? make_smem_desc(sb, kBChunkBytes, 1024) : make_smem_desc(sb, 16, 1024);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j)
            tc_mma_bf16(d_tmem, da + (uint64_t)(j * (kAmn ? 128 : 2)), db + (uint64_t)(j * (kBmn ? 128 : 2)),
                        idesc, (kb > 0 || j > 0) ? 1u : 0u);
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
    const int quad = warp & 3;  // the TMEM lanes a warp may read: 32 * (warp id mod 4)
    constexpr int kColsPerWarp = UMMA_N / (kEpiWarps / 4);
    const int c_begin = ((warp - 2) >> 2) * kColsPerWarp, c_end = c_begin + kColsPerWarp;
    unsigned char* stage_w = staging + (size_t)((warp - 2) & 3) * 4096;  // kWGRAD, kDH
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const TileCoord tc = decode_bwd<MODE>(sh, nseg, n_tiles, m_tiles_w, tile);
      const AxmSegment sg = sh->seg[tc.seg];
      const int k_blocks = tile_k_blocks(sg);
      const int n0 = tc.n_tile * UMMA_N;
      // kDH: g, u, dG, dU move between global memory and the warp's staging block in
      // row-contiguous 64-byte runs (a request touches 8 rows, not 32), and each lane
      // works on its own row out of shared memory.  Piece p of a 32 x 32 bf16 block:
      // row p / 4, 16-byte piece p % 4; in shared memory at row * 64 + ((piece ^ (row / 2 % 4)) * 16,
      // which keeps both access patterns free of bank conflicts.  g and u stream from HBM, so
      // their pieces are fetched two blocks ahead, the first two before the accumulator is
      // even waited for: with one block of lead every block had cost a memory latency.
      uint4 g_q0[4], u_q0[4], g_q1[4], u_q1[4];  // 128 pieces per 32 x 32 block: four per lane and tensor
      const int rows_left = sg.rows - (tc.m_tile * BM + quad * 32);  // rows of this warp's block
      auto piece_ok = [&](int p, int c0) {
        return (p >> 2) < rows_left && c0 < c_end && n0 + c0 + (p & 3) * 8 < args.n_total;
      };
      auto piece_elem = [&](int p, int c0) {
        return (size_t)(sg.out_row0 + tc.m_tile * BM + quad * 32 + (p >> 2)) * args.n_total + n0 + c0 +
               (p & 3) * 8;
      };
      auto piece_smem = [&](int row, int piece) { return row * 64 + ((piece ^ ((row >> 1) & 3)) << 4); };
      auto fetch_gu = [&](int c0, uint4 (&gq)[4], uint4 (&uq)[4]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int p = lane + 32 * i;
          gq[i] = make_uint4(0, 0, 0, 0);
          uq[i] = make_uint4(0, 0, 0, 0);
          if (piece_ok(p, c0)) {
            gq[i] = __ldg(reinterpret_cast<const uint4*>(args.g + piece_elem(p, c0)));
            uq[i] = __ldg(reinterpret_cast<const uint4*>(args.u + piece_elem(p, c0)));
          }
        }
      };
      if constexpr (MODE == kDH) {
        fetch_gu(c_begin, g_q0, u_q0);
        fetch_gu(c_begin + 32, g_q1, u_q1);
      }
      if (!__all_sync(0xffffffffu, mbar_wait(&sh->tmem_full[acc], acc_phase, abort_flag))) break;
      tc_fence_after();
      const int row_in_tile = tc.m_tile * BM + quad * 32 + lane;
      bool row_ok;
      size_t out_elem;
      if constexpr (MODE == kWGRAD) {
        row_ok = row_in_tile < args.m_total;
        out_elem = ((size_t)(sg.expert & 0xffff) * args.m_total + (row_ok ? row_in_tile : 0)) * args.n_total + n0;
      } else {
        row_ok = row_in_tile < sg.rows;
        out_elem = (size_t)(sg.out_row0 + (row_ok ? row_in_tile : 0)) * args.n_total + n0;
      }
      const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)acc * UMMA_N;
      if constexpr (MODE == kDH) {
        unsigned char* g_s = stage_w;
        unsigned char* u_s = stage_w + 2048;
        auto dh_block = [&](int c0, uint4 (&gq)[4], uint4 (&uq)[4]) {
          uint32_t v[32];
          __syncwarp();  // the previous block's read-back is done; also rejoins the warp for tcgen05.ld
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int p = lane + 32 * i;
            *reinterpret_cast<uint4*>(g_s + piece_smem(p >> 2, p & 3)) = gq[i];
            *reinterpret_cast<uint4*>(u_s + piece_smem(p >> 2, p & 3)) = uq[i];
          }
          fetch_gu(c0 + 64, gq, uq);  // this queue's next block is two blocks on
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
            *gp = make_uint4(dgw[0], dgw[1], dgw[2], dgw[3]);  // in place: the lane's own row
            *up = make_uint4(duw[0], duw[1], duw[2], duw[3]);
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int p = lane + 32 * i;
            if (piece_ok(p, c0)) {
              *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(args.out0) + piece_elem(p, c0)) =
                  *reinterpret_cast<const uint4*>(g_s + piece_smem(p >> 2, p & 3));
              *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(args.out1) + piece_elem(p, c0)) =
                  *reinterpret_cast<const uint4*>(u_s + piece_smem(p >> 2, p & 3));
            }
          }
        };
#pragma unroll 1
        for (int c0 = c_begin; c0 < c_end; c0 += 64) {
          dh_block(c0, g_q0, u_q0);
          dh_block(c0 + 32, g_q1, u_q1);
        }
      }
#pragma unroll 1
      for (int c0 = c_begin; MODE != kDH && c0 < c_end; c0 += 32) {
        uint32_t v[32];
        __syncwarp();  // tcgen05.ld is warp-wide: rejoin lanes that skipped the stores
        tmem_ld32(t_addr + c0, v);
        tmem_ld_wait();
        if (MODE == kWGRAD && k_blocks == 0) {
          // an expert without rows: its weight gradient is zero, the accumulator was never written
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
        }
        if constexpr (MODE == kWGRAD) {
          // Lane = row of the block.  Its eight 16-byte pieces go to shared memory in the
          // 128-byte-swizzle pattern of the output map (piece q of row r at q ^ (r & 7)),
          // which also keeps the eight lanes of a store phase on different banks; then one
          // TMA store writes the 32 x 32 block.  The map clips rows beyond m_total and
          // columns beyond n_total.
          if (lane == 0) bulk_wait_read();  // the previous block's store has read the buffer
          __syncwarp();
          if (n0 + c0 < args.n_total && tc.m_tile * BM + quad * 32 < args.m_total) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<uint4*>(stage_w + lane * 128 + ((q ^ (lane & 7)) << 4)) =
                  make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              tma_store_3d(&tm_a1, stage_w, n0 + c0, tc.m_tile * BM + quad * 32, sg.expert & 0xffff);
              bulk_commit_group();
            }
          }
          continue;
        }
        if (!row_ok) continue;
        {
          float* out_row = static_cast<float*>(args.out0) + out_elem;
#pragma unroll
          for (int q = 0; q < 8; ++q)
            if (n0 + c0 + q * 4 < args.n_total)
              *reinterpret_cast<uint4*>(out_row + c0 + q * 4) =
                  make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
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
  if (MODE == kWGRAD && warp >= 2 && lane == 0) bulk_wait_all();
  tc_fence_before();
  __syncthreads();
  if (sh->abort_flag != 0) {
    long long t0 = clock64();
    while (clock64() - t0 < 4000000LL) {
    }
    if (threadIdx.x == 0 && args.status != nullptr) atomicExch(args.status, 3 + MODE);
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host side ------------------------------------------------------------------------

static int map_rows(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  const uint64_t dims[2] = {cols, rows};
  const uint64_t strides[1] = {cols * 2};
  const uint32_t box[2] = {64, box_rows};
  return encode_tensor_map(m, base, 2, dims, strides, box);
}

// Weights [experts][n_rows][k_cols] read K-major: box = 64 k x 256 n x 1 expert.
static int map_weights_kmajor(CUtensorMap* m, const void* base, uint64_t experts, uint64_t n_rows,
                              uint64_t k_cols) {
  const uint64_t dims[3] = {k_cols, n_rows, experts};
  const uint64_t strides[2] = {k_cols * 2, k_cols * n_rows * 2};
  const uint32_t box[3] = {64, 256, 1};
  return encode_tensor_map(m, base, 3, dims, strides, box);
}

// fp32 weight gradient [experts][m][n]: box = 32 columns (128 bytes) x 32 rows x 1 expert.
static int map_wgrad_out(CUtensorMap* m, void* base, uint64_t experts, uint64_t rows, uint64_t cols) {
  const uint64_t dims[3] = {cols, rows, experts};
  const uint64_t strides[2] = {cols * 4, cols * rows * 4};
  const uint32_t box[3] = {32, 32, 1};
  return encode_tensor_map_f32(m, base, 3, dims, strides, box);
}

template <int MODE>
static int launch_bwd(const CUtensorMap& a0, const CUtensorMap& a1, const CUtensorMap& b0,
                      const CUtensorMap& b1, const BwdArgs& args, cudaStream_t st, const char* what) {
  static SmemLimitCache smem = {};
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(grouped_bwd_kernel<MODE>),
                                   BwdCfg<MODE>::kSmemBytes, &smem, what))
    return rc;
  grouped_bwd_kernel<MODE><<<sm_count(), BwdCfg<MODE>::kThreads, BwdCfg<MODE>::kSmemBytes, st>>>(a0, a1, b0, b1,
                                                                                               args);
  return check_launch(what);
}

}  // namespace axm

using namespace axm;

namespace axm {
// phases: bit 0 = the two input-gradient products (dH with the SwiGLU derivative, then dXp),
// bit 1 = the three weight gradients.  The expert-parallel backward runs them as two calls so
// that the dXp rows can travel home while the weight gradients are computed.
int launch_expert_ffn_backward(const AxmMoeDesc* desc, const AxmSegment* segments, int32_t num_segments,
                               int32_t rows_total, const void* x_perm, const void* h, const void* g, const void* u,
                               const void* d_o, const void* w_gate, const void* w_up, const void* w_down, void* d_g,
                               void* d_u, void* d_xp, void* d_w_gate, void* d_w_up, void* d_w_down, int32_t* status,
                               void* stream, int phases) {
  if (desc == nullptr) return fail(AXM_ERR_ARGUMENT, "desc is null");
  const int D = desc->d_model, F = desc->d_ff, E = desc->num_experts;
  if (D <= 0 || F <= 0 || D % 8 || F % 8 || E <= 0)
    return fail(AXM_ERR_ARGUMENT, "d_model and d_ff must be positive multiples of 8, num_experts positive");
  if (num_segments < 0 || num_segments > kMaxSegments)
    return fail(AXM_ERR_ARGUMENT, "num_segments %d not in 0..%d", num_segments, kMaxSegments);
  if (!segments || !x_perm || !h || !g || !u || !d_o || !w_gate || !w_up || !w_down || !d_g || !d_u || !d_xp)
    return fail(AXM_ERR_ARGUMENT, "axm_moe_expert_ffn_backward: null pointer");
  const bool wgrad = d_w_gate || d_w_up || d_w_down;
  if (wgrad && !(d_w_gate && d_w_up && d_w_down))
    return fail(AXM_ERR_ARGUMENT, "weight gradients: give all three or none");
  if (rows_total <= 0 || num_segments == 0) return AXM_OK;
  if (int rc = require_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint64_t R = (uint64_t)rows_total;
  int rc;
  CUtensorMap m_do, m_dg, m_du, m_wd, m_wg, m_wu;
  if ((rc = map_rows(&m_do, d_o, R, D, BM))) return rc;
  if ((rc = map_rows(&m_dg, d_g, R, F, BM))) return rc;
  if ((rc = map_rows(&m_du, d_u, R, F, BM))) return rc;
  if ((rc = map_weights_kmajor(&m_wd, w_down, E, F, D))) return rc;
  if ((rc = map_weights_kmajor(&m_wg, w_gate, E, D, F))) return rc;
  if ((rc = map_weights_kmajor(&m_wu, w_up, E, D, F))) return rc;

  BwdArgs a;
  a.segments = segments;
  a.num_segments = num_segments;
  a.status = status;
  a.m_total = 0;
  a.g = static_cast<const __nv_bfloat16*>(g);
  a.u = static_cast<const __nv_bfloat16*>(u);
  // dH = dO . Wd^T, SwiGLU derivative in the epilogue -> dG, dU
  a.n_total = F;
  a.k_total = D;
  a.out0 = d_g;
  a.out1 = d_u;
  if (phases & 1) {
  rc = AXM_ERR_DEVICE;
  static const bool dh_pairs = [] {  // CTA pairs with TMA-moved epilogue blocks by default; AXM_DH_2SM=0 opts out
    const char* e = getenv("AXM_DH_2SM");
    return !(e != nullptr && e[0] == '0');
  }();
  if (dh_pairs && use_2sm_kernels())
    rc = launch_bwd_dh_2sm(desc, segments, num_segments, rows_total, d_o, w_down, g, u, d_g, d_u, status, st);
  if (rc == AXM_ERR_DEVICE)  // pairs not wanted or not schedulable: the one-SM kernel
    rc = launch_bwd<kDH>(m_do, m_do, m_wd, m_wd, a, st, "grouped_bwd_kernel<dH>");
  if (rc) return rc;
  // dXp = dG . Wg^T + dU . Wu^T
  a.n_total = D;
  a.k_total = F;
  a.out0 = d_xp;
  a.out1 = nullptr;
  rc = AXM_ERR_DEVICE;
  if (use_2sm_kernels())
    rc = launch_bwd_dx_2sm(desc, segments, num_segments, rows_total, d_g, d_u, w_gate, w_up, d_xp, status, st);
  if (rc == AXM_ERR_DEVICE)  // pairs not wanted or not schedulable: the one-SM kernel
    rc = launch_bwd<kDX>(m_dg, m_du, m_wg, m_wu, a, st, "grouped_bwd_kernel<dX>");
  if (rc) return rc;
  }
  if (!wgrad || !(phases & 2)) return AXM_OK;

  CUtensorMap k_h, k_do, k_x, k_dg, k_du;  // 64-row boxes: rows are the reduction index
  if ((rc = map_rows(&k_h, h, R, F, 64))) return rc;
  if ((rc = map_rows(&k_do, d_o, R, D, 64))) return rc;
  if ((rc = map_rows(&k_x, x_perm, R, D, 64))) return rc;
  if ((rc = map_rows(&k_dg, d_g, R, F, 64))) return rc;
  if ((rc = map_rows(&k_du, d_u, R, F, 64))) return rc;
  CUtensorMap o_wd, o_wg, o_wu;  // fp32 outputs, stored tile by tile through TMA
  if ((rc = map_wgrad_out(&o_wd, d_w_down, E, F, D))) return rc;
  if ((rc = map_wgrad_out(&o_wg, d_w_gate, E, D, F))) return rc;
  if ((rc = map_wgrad_out(&o_wu, d_w_up, E, D, F))) return rc;
  a.k_total = 0;
  // each product on CTA pairs by default, on the one-SM kernel if pairs are not wanted or not schedulable
  auto wgrad_one = [&](const void* am, const CUtensorMap& ka, int m_total, const void* bm, const CUtensorMap& kb,
                       int n_total, void* out, const CUtensorMap& omap, const char* what) -> int {
    int r = AXM_ERR_DEVICE;
    if (use_2sm_kernels())
      r = launch_wgrad_2sm(segments, num_segments, rows_total, E, am, m_total, bm, n_total, out, status, st);
    if (r != AXM_ERR_DEVICE) return r;
    a.m_total = m_total;
    a.n_total = n_total;
    a.out0 = out;
    return launch_bwd<kWGRAD>(ka, omap, kb, kb, a, st, what);
  };
  if ((rc = wgrad_one(h, k_h, F, d_o, k_do, D, d_w_down, o_wd, "grouped_bwd_kernel<dWd>"))) return rc;  // h^T dO : [F][D]
  if ((rc = wgrad_one(x_perm, k_x, D, d_g, k_dg, F, d_w_gate, o_wg, "grouped_bwd_kernel<dWg>"))) return rc;  // x^T dG : [D][F]
  return wgrad_one(x_perm, k_x, D, d_u, k_du, F, d_w_up, o_wu, "grouped_bwd_kernel<dWu>");
}
}  // namespace axm

extern "C" int axm_moe_expert_ffn_backward(const AxmMoeDesc* desc, const AxmSegment* segments,
                                           int32_t num_segments, int32_t rows_total,
                                           const void* x_perm, const void* h, const void* g,
                                           const void* u, const void* d_o, const void* w_gate,
                                           const void* w_up, const void* w_down, void* d_g, void* d_u,
                                           void* d_xp, void* d_w_gate, void* d_w_up, void* d_w_down,
                                           int32_t* status, void* stream) {
  return axm::launch_expert_ffn_backward(desc, segments, num_segments, rows_total, x_perm, h, g, u, d_o, w_gate, w_up,
                                         w_down, d_g, d_u, d_xp, d_w_gate, d_w_up, d_w_down, status, stream, 3);
}
