// Pieces shared by the grouped tensor-core kernels (forward and backward):
// tile geometry, the shared-memory control block, the sm_100 shared-memory matrix
// descriptor and the tile decoder.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace axm {

constexpr int BM = 128;             // rows per tile
constexpr int BK = 64;              // reduction elements per stage (128 bytes of bf16)
constexpr int UMMA_N = 256;         // accumulator columns per tile
constexpr int UMMA_K = 16;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;          // 16 KiB
constexpr int kBChunkBytes = 64 * BK * 2;     // 64 output columns x 64 k: 8 KiB
constexpr int kBBytes = 4 * kBChunkBytes;     // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kMaxSegments = 512;
constexpr int kGemmThreads = 192;
constexpr int kTmemCols = 512;

struct __align__(8) GemmShared {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int total_tiles;
  int tile_prefix[kMaxSegments + 1];  // m-tiles before segment s
  int num_groups;                     // runs of consecutive segments with one expert
  int group_first[kMaxSegments + 1];  // first segment of group g
  AxmSegment seg[kMaxSegments];
};

constexpr size_t kGemmSmemBytes = 1024 /*alignment slack*/ + (size_t)kStages * kStageBytes + sizeof(GemmShared);

// Shared-memory matrix descriptor (sm_100 format): start address, leading and
// stride byte offsets in 16-byte units, descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;  // version
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

struct TileCoord {
  int seg;
  int m_tile;
  int n_tile;
};

// Tiles are ordered group by group, where a group is a run of consecutive
// segments that use the same expert (one segment on a single GPU; one per source
// rank under expert parallelism).  Inside a group the order is n-tile major and
// m-tile minor over ALL the group's m-tiles, so CTAs that run together share a
// weight column block and each weight tile is fetched from HBM about once.
__device__ __forceinline__ TileCoord decode_tile(const GemmShared* sh, int num_segments,
                                                 int n_tiles, int linear) {
  int lo = 0, hi = sh->num_groups - 1;
  while (lo < hi) {  // largest g whose first tile is <= linear
    int mid = (lo + hi + 1) >> 1;
    if (sh->tile_prefix[sh->group_first[mid]] * n_tiles <= linear) lo = mid; else hi = mid - 1;
  }
  const int s0 = sh->group_first[lo], s1 = sh->group_first[lo + 1];
  const int base = sh->tile_prefix[s0];
  const int mt = sh->tile_prefix[s1] - base;
  const int local = linear - base * n_tiles;
  TileCoord tc;
  tc.n_tile = local / mt;
  const int m_idx = base + (local - tc.n_tile * mt);
  int a = s0, b = s1 - 1;
  while (a < b) {  // largest s in the group with tile_prefix[s] <= m_idx
    int mid = (a + b + 1) >> 1;
    if (sh->tile_prefix[mid] <= m_idx) a = mid; else b = mid - 1;
  }
  tc.seg = a;
  tc.m_tile = m_idx - sh->tile_prefix[a];
  return tc;
}


// Instruction descriptor of tcgen05.mma kind::f16: fp32 accumulate, bf16 A and B,
// M = 128, N = 256; a_mn / b_mn select the MN-major (transposed) operand form.
__host__ __device__ constexpr uint32_t instr_desc(bool a_mn, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(UMMA_N >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// bf16 tensor map with 128-byte swizzle and zero fill: dims / box innermost first,
// strides in bytes for dimensions 1.. (rank - 1).  Defined in grouped_ffn.cu.
int encode_tensor_map(CUtensorMap* m, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box);
// The same for an fp32 tensor (used for TMA stores of fp32 tiles; box inner extent 32 = 128 bytes).
int encode_tensor_map_f32(CUtensorMap* m, const void* base, int rank, const uint64_t* dims,
                          const uint64_t* strides_bytes, const uint32_t* box);

// bf16 map with 64-byte swizzle (box inner extent 32 elements): the epilogue blocks of the dH kernel.
int encode_tensor_map_sw64(CUtensorMap* m, const void* base, int rank, const uint64_t* dims,
                           const uint64_t* strides_bytes, const uint32_t* box);

// Two-SM (cta_group::2) kernels are the default; AXM_GEMM_2SM=0 selects the one-SM kernels.
bool use_2sm_kernels();
// Input-gradient GEMM of the backward pass on CTA pairs (grouped_ffn_2sm.cu).
int launch_bwd_dx_2sm(const AxmMoeDesc* d, const AxmSegment* segments, int32_t num_segments,
                      int32_t rows_total, const void* d_g, const void* d_u, const void* w_gate,
                      const void* w_up, void* d_xp, int32_t* status, cudaStream_t st);
// dH GEMM of the backward pass with the SwiGLU derivative, on CTA pairs (grouped_ffn_2sm.cu).
int launch_bwd_dh_2sm(const AxmMoeDesc* d, const AxmSegment* segments, int32_t num_segments,
                      int32_t rows_total, const void* d_o, const void* w_down, const void* g, const void* u,
                      void* d_g, void* d_u, int32_t* status, cudaStream_t st);
// Weight-gradient GEMM of the backward pass on CTA pairs (grouped_bwd_2sm.cu).
int launch_wgrad_2sm(const AxmSegment* segments, int32_t num_segments, int32_t rows_total, int32_t experts,
                     const void* a, int32_t m_total, const void* b, int32_t n_total, void* d_w,
                     int32_t* status, cudaStream_t st);

}  // namespace axm
