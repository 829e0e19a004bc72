// Pieces shared by the kernels that run on CTA pairs (thread-block clusters of two,
// tcgen05.mma.cta_group::2): stage geometry, the shared-memory control block and the PTX
// wrappers.  No cluster multicast: every CTA issues its own TMA loads, and the leader
// signals the peer's barriers with ordinary tcgen05.commit instructions addressed to the
// peer's shared memory.
#pragma once

#include "gemm_common.cuh"

namespace axm {

constexpr int kStages2 = 6;
constexpr int kBHalfBytes = 2 * kBChunkBytes;              // 128 columns x 64 k
constexpr int kStageBytes2 = kABytes + kBHalfBytes;        // 32 KiB per CTA and stage

struct __align__(8) GemmShared2 {
  uint64_t full[kStages2];      // used in the leader: bytes of both CTAs land here
  uint64_t empty[kStages2];     // own: the leader's MMA commit arrives in both CTAs
  uint64_t tmem_full[2];        // own
  uint64_t tmem_empty[2];       // used in the leader: 4 epilogue warps of each CTA
  uint32_t tmem_base;
  int abort_flag;
  int total_units;
  int num_groups;
  int tile_prefix[kMaxSegments + 1];
  int group_first[kMaxSegments + 1];
  int pair_prefix[kMaxSegments + 1];  // pairs before group g
  AxmSegment seg[kMaxSegments];
};

constexpr size_t kGemm2SmemBytes = 1024 + (size_t)kStages2 * kStageBytes2 + sizeof(GemmShared2);

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// TMA loads of a CTA pair: the completion bytes are counted on the mbarrier at
// `bar_cluster_addr`, which may live in the peer CTA (the leader's barrier).
__device__ __forceinline__ void tma2_load_2d(void* dst, const void* tmap, uint32_t bar_cluster_addr,
                                             int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma2_load_3d(void* dst, const void* tmap, uint32_t bar_cluster_addr,
                                             int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(dst)),
      "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// arrives on the mbarrier at a shared::cluster address once the pair's MMAs issued so far are done
__device__ __forceinline__ void tc_commit2(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tc_mma2_bf16(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}


// Number of CTAs to launch (two per cluster), 0 when pairs cannot be scheduled, or a
// negative status (defined in grouped_ffn_2sm.cu).
int grid_2sm();

}  // namespace axm
