// Expert-parallel exchange over NVLink peer memory: dispatch of permuted token
// rows to the ranks that own their experts, and return of the expert outputs,
// written as plain peer stores by this GPU's own kernels, with flags in peer
// memory instead of host synchronisation.
//
// The reference engine is single-GPU; this is the sharded form of its
// forward_mixture_experts (core/src/CUDA/kernel/moe_router.cu:205-320): each
// rank routes and permutes its own tokens, the rows travel to the expert's
// rank, the grouped GEMMs run on local memory only, the fp32 expert rows travel
// back and are combined where the gates are.
//
// Every rank owns one "exchange region" of identical layout (AxmEpLayout) and
// knows the address of every peer's region (peer access enabled by whoever
// allocated them).  Per layer call, with `step` a counter the host increments:
//   axm_ep_dispatch   post my per-expert counts to all peers, flag; wait for all
//                     peers' counts; copy my permuted rows into each owner's
//                     receive buffer at the offset the counts imply; flag.  The
//                     receive buffer is expert-major (all sources' rows of local
//                     expert 0, then of expert 1 ...; inside an expert by source
//                     rank), so one expert's rows are one contiguous run.
//   axm_ep_segments   wait for all sources' rows; build the segment table (one
//                     merged segment per local expert, so the GEMMs tile the rows
//                     exactly as on a single GPU) and the return map.
//   (grouped GEMMs over the receive buffer - local TMA only)
//   axm_ep_return     copy fp32 expert rows back into each source's buffer, flag.
//   axm_ep_wait_return wait for all owners' rows before the combine.
// Flags only ever grow (they hold the step number), so nothing is reset and a
// buffer is never overwritten before its reader has signalled: the return flag of
// step n from rank B tells rank A that B has finished reading everything A sent
// in step n.
//
// All waits are bounded (about two seconds); a wait that gives up stores a code
// in the status word and the kernel carries on, so a missing peer cannot hang the
// GPU.  No multicast, no TMA on peer memory: peers are reached with ordinary
// 16-byte stores.
#include "common.cuh"

namespace axm {

struct EpArgs {
  char* const* peers;   // device array [G]: base of every rank's exchange region
  int rank, G, E, El;   // El = experts per rank
  int D;                // d_model
  int slots;            // T_local * k of this call
  int ret_rows;         // rows of a rank's return buffer (>= any rank's slots)
  int cap;              // rows the receive buffer holds
  int S, T_local;       // shared experts, local tokens
  int align;            // every local expert's run in the receive buffer starts at a multiple of this
  uint32_t step;
  long long off_counts, off_flags, off_recv, off_oback;  // byte offsets inside a region
  int32_t* status;
};

// flags: [3][G] uint32 = {counts posted, rows delivered, outputs returned}
__device__ __forceinline__ uint32_t* flag_ptr(const EpArgs& a, int owner, int kind, int src) {
  return reinterpret_cast<uint32_t*>(a.peers[owner] + a.off_flags) + kind * a.G + src;
}

__device__ __forceinline__ void store_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Waits until flag >= step (wrap-safe).  Returns false when the wait ran out.
__device__ __forceinline__ bool wait_flag(const uint32_t* p, uint32_t step) {
  long long t0 = clock64();
  while ((int32_t)(load_acquire_sys(p) - step) < 0) {
    if (clock64() - t0 > kWaitCycles) return false;
    __nanosleep(64);
  }
  return true;
}

// Thread s < G waits for flag (kind, s) of this rank; the block then syncs.
__device__ __forceinline__ void wait_all_sources(const EpArgs& a, int kind, int code) {
  if ((int)threadIdx.x < a.G) {
    if (!wait_flag(flag_ptr(a, a.rank, kind, threadIdx.x), a.step) && a.status != nullptr)
      atomicExch(a.status, code);
  }
  __syncthreads();
}

__device__ __forceinline__ int round_up_rows(int v, int align) { return (v + align - 1) / align * align; }

// Row of `owner_first .. e`'s receive buffer where the rows that rank `rank` sends to expert e
// start: the (aligned) runs of the owner's earlier experts, then the rows lower ranks send to e.
__device__ __forceinline__ int dispatch_base(const EpArgs& a, const int32_t* table, int e) {
  const int e_first = (e / a.El) * a.El;  // the owner's first expert
  int base = 0;
  for (int q = e_first; q < e; ++q) {
    int tot = 0;
    for (int s = 0; s < a.G; ++s) tot += __ldcg(table + s * a.E + q);
    base += round_up_rows(tot, a.align);
  }
  for (int s = 0; s < a.rank; ++s) base += __ldcg(table + s * a.E + e);
  return base;
}

constexpr int kEpThreads = 256;
constexpr int kEpMaxRanks = 64;
constexpr int kEpMaxExperts = 4096;  // 64 ranks x 64 experts per rank

__global__ void __launch_bounds__(kEpThreads)
ep_dispatch_kernel(EpArgs a, const int32_t* __restrict__ offsets,
                   const __nv_bfloat16* __restrict__ x_perm, int32_t* __restrict__ done_counter) {
  __shared__ int off_s[kEpMaxExperts + 1];  // my permuted rows of expert e start here
  __shared__ int dst_base[kEpMaxExperts];   // row in the owner's receive buffer where they go
  const int tid = threadIdx.x;

  // 1. post my counts into every peer's table (row = my rank) and flag them
  if (blockIdx.x == 0) {
    for (int i = tid; i < a.E * a.G; i += kEpThreads) {
      int g = i / a.E, e = i - g * a.E;
      int32_t* table = reinterpret_cast<int32_t*>(a.peers[g] + a.off_counts);
      table[a.rank * a.E + e] = offsets[e + 1] - offsets[e];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < a.G) store_release_sys(flag_ptr(a, tid, 0, a.rank), a.step);
  }
  // 2. wait for everybody's counts (each block on its own: no block depends on another)
  wait_all_sources(a, 0, 11);
  // 3. where do my rows go: the owner's buffer holds, expert by expert, the rows of
  //    source 0, 1, ... - mine start after all rows of the owner's earlier experts and
  //    the rows that lower ranks send to this expert
  const int32_t* table = reinterpret_cast<const int32_t*>(a.peers[a.rank] + a.off_counts);
  for (int e = tid; e <= a.E; e += kEpThreads) off_s[e] = offsets[e];
  for (int e = tid; e < a.E; e += kEpThreads) dst_base[e] = dispatch_base(a, table, e);
  __syncthreads();
  // 4. copy: one warp per row, 16-byte pieces, plain stores into the owner's memory
  const int warp = tid >> 5, lane = tid & 31;
  const int warps_total = gridDim.x * (kEpThreads / 32);
  const int chunks = a.D / 8;
  int e = 0;
  for (int r = blockIdx.x * (kEpThreads / 32) + warp; r < a.slots; r += warps_total) {
    while (e + 1 < a.E && r >= off_s[e + 1]) ++e;  // rows ascend, so does the expert
    const int dst_row = dst_base[e] + (r - off_s[e]);
    if (dst_row < 0 || dst_row >= a.cap) continue;  // cannot happen with cap = slots * G; never write outside
    const uint4* src = reinterpret_cast<const uint4*>(x_perm + (size_t)r * a.D);
    uint4* dst = reinterpret_cast<uint4*>(a.peers[e / a.El] + a.off_recv) + (size_t)dst_row * chunks;
    for (int c0 = 0; c0 < chunks; c0 += 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (c0 + u * 32 + lane < chunks) v[u] = __ldg(src + c0 + u * 32 + lane);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (c0 + u * 32 + lane < chunks) dst[c0 + u * 32 + lane] = v[u];
    }
  }
  // 5. when every block is done, tell every owner that my rows have landed
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    int prev = atomicAdd(done_counter, 1);
    if (prev == (int)gridDim.x - 1) {
      *done_counter = 0;
      __threadfence_system();
      for (int o = 0; o < a.G; ++o) store_release_sys(flag_ptr(a, o, 1, a.rank), a.step);
    }
  }
}

// Permute and dispatch in one kernel: the placement of axm_moe_permute (histogram, exclusive
// scan, stable ranks: rows of an expert ordered by token, then slot) with the rows written
// straight into the owners' receive buffers instead of a local x_perm that a second kernel
// would read back.  One CTA per router block, like the permute kernel.  Block 0 posts this
// rank's counts to all peers as soon as they are known; every block then waits for the
// peers' counts (bounded), derives where this rank's rows of each expert start in the
// owner's buffer, places its tokens and copies each row once per selected expert with
// 16-byte stores (local for this rank's own experts, over NVLink otherwise).  slot_dst and
// row_src describe the LOCAL expert-contiguous order (row r of this rank's virtual x_perm),
// which is also the row of the return buffer where the expert output of that slot lands.
constexpr int kFusedTokSub = 128;
constexpr int kFusedMaxE = 256;
__global__ void __launch_bounds__(kEpThreads)
ep_permute_dispatch_kernel(EpArgs a, const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ topk_idx,
                           const int32_t* __restrict__ block_counts, int32_t* __restrict__ histogram,
                           int32_t* __restrict__ offsets, int32_t* __restrict__ row_src,
                           int32_t* __restrict__ slot_dst, int32_t* __restrict__ done_counter, int T, int k,
                           int hist_accumulate) {
  __shared__ int total_s[kFusedMaxE];
  __shared__ int run_s[kFusedMaxE];      // next free LOCAL row per expert for this block
  __shared__ int scan_s[kFusedMaxE + 1];  // local offsets
  __shared__ int base_s[kFusedMaxE];      // row in the owner's receive buffer of my first row of expert e
  __shared__ int dst_s[kFusedTokSub * 8];  // destination row in the owner's buffer
  __shared__ unsigned char own_s[kFusedTokSub * 8];  // owner rank
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x, E = a.E;

  for (int e = tid; e < E; e += kEpThreads) {
    total_s[e] = 0;
    run_s[e] = 0;
  }
  __syncthreads();
  const int n_cells = AXM_ROUTE_BLOCKS * E;
  for (int i = tid; i < n_cells; i += kEpThreads) {
    const int bb = i / E, e = i - bb * E;
    const int c = block_counts[i];
    if (c != 0) {
      atomicAdd(&total_s[e], c);
      if (bb < b) atomicAdd(&run_s[e], c);
    }
  }
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      const int v = e < E ? total_s[e] : 0;
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
      }
      if (e < E) scan_s[e] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) scan_s[E] = carry;
  }
  __syncthreads();
  for (int e = tid; e < E; e += kEpThreads) run_s[e] += scan_s[e];
  if (b == 0) {
    // publish: local outputs, and my counts into every peer's table (row = my rank)
    for (int e = tid; e <= E; e += kEpThreads) {
      if (offsets != nullptr) offsets[e] = scan_s[e];
      if (e < E && histogram != nullptr) histogram[e] = (hist_accumulate ? histogram[e] : 0) + total_s[e];
    }
    for (int i = tid; i < E * a.G; i += kEpThreads) {
      const int g = i / E, e = i - g * E;
      int32_t* table = reinterpret_cast<int32_t*>(a.peers[g] + a.off_counts);
      table[a.rank * E + e] = total_s[e];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < a.G) store_release_sys(flag_ptr(a, tid, 0, a.rank), a.step);
  }
  wait_all_sources(a, 0, 11);
  {
    const int32_t* table = reinterpret_cast<const int32_t*>(a.peers[a.rank] + a.off_counts);
    for (int e = tid; e < E; e += kEpThreads) base_s[e] = dispatch_base(a, table, e);
  }
  __syncthreads();

  const int t_begin = (int)(((long long)b * T) / AXM_ROUTE_BLOCKS);
  const int t_end = (int)(((long long)(b + 1) * T) / AXM_ROUTE_BLOCKS);
  const int chunks = a.D / 8;
  for (int ts = t_begin; ts < t_end; ts += kFusedTokSub) {
    const int nt = min(kFusedTokSub, t_end - ts);
    const int n_ent = nt * k;
    if (warp == 0) {
      for (int c0 = 0; c0 < n_ent; c0 += 32) {
        const int i = c0 + lane;
        const bool live = i < n_ent;
        const int e = live ? topk_idx[(size_t)ts * k + i] : -1;
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        const int rank_in = __popc(peers & ((1u << lane) - 1u));
        int local_row = -1;
        if (live) {
          local_row = run_s[e] + rank_in;
          dst_s[i] = base_s[e] + (local_row - scan_s[e]);
          own_s[i] = (unsigned char)(e / a.El);
        }
        __syncwarp();
        if (live && rank_in == __popc(peers) - 1) run_s[e] += rank_in + 1;
        __syncwarp();
        if (live) {
          const size_t slot = (size_t)ts * k + i;
          if (slot_dst != nullptr) slot_dst[slot] = local_row;
          if (row_src != nullptr) row_src[local_row] = (int32_t)slot;
        }
      }
    }
    __syncthreads();
    for (int tt = warp; tt < nt; tt += kEpThreads / 32) {
      const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(ts + tt) * a.D);
      for (int c0 = 0; c0 < chunks; c0 += 128) {
        uint4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = c0 + j * 32 + lane;
          if (c < chunks) v[j] = __ldg(src + c);
        }
        for (int i = 0; i < k; ++i) {
          const int dst_row = dst_s[tt * k + i];
          if (dst_row < 0 || dst_row >= a.cap) continue;  // never write outside the receive buffer
          uint4* dstp = reinterpret_cast<uint4*>(a.peers[own_s[tt * k + i]] + a.off_recv) + (size_t)dst_row * chunks;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c = c0 + j * 32 + lane;
            if (c < chunks) dstp[c] = v[j];
          }
        }
      }
    }
    __syncthreads();
  }
  // when every block is done, tell every owner that my rows have landed
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    const int prev = atomicAdd(done_counter, 1);
    if (prev == (int)gridDim.x - 1) {
      *done_counter = 0;
      __threadfence_system();
      for (int o = 0; o < a.G; ++o) store_release_sys(flag_ptr(a, o, 1, a.rank), a.step);
    }
  }
}

// One block.  The receive buffer is expert-major: all sources' rows of local expert 0
// (source 0 first), then of expert 1, ...  Two tables over that buffer, both indexed
// j * G + s (local expert j, source rank s), which is also ascending row order:
//   segments     for the grouped GEMMs.  Without a remote-output table the rows of one
//                expert are ONE segment (entry j * G holds all of them, the other G - 1
//                entries of that expert hold zero rows), so the m-tiles are cut exactly as
//                on a single GPU instead of once per source.  With a remote-output table
//                (the down GEMM stores into the sources' buffers itself) every source keeps
//                its own segment, because a segment has one destination.
//   ret_segments for the return copy: {a_row0 = row in the source's return buffer,
//                out_row0 = row here, rows, expert = source rank}.
__global__ void __launch_bounds__(kEpThreads)
ep_segments_kernel(EpArgs a, AxmSegment* __restrict__ segments,
                   AxmSegment* __restrict__ ret_segments, AxmRemoteOut* __restrict__ remote_out,
                   int32_t* __restrict__ rows_received, AxmSegment* __restrict__ seg_halves,
                   int32_t* __restrict__ split_rows) {
  __shared__ int rows_s[kEpMaxRanks * 64];
  __shared__ int start_s[kEpMaxRanks * 64];
  wait_all_sources(a, 1, 12);
  const int32_t* table = reinterpret_cast<const int32_t*>(a.peers[a.rank] + a.off_counts);
  const int n = a.G * a.El;
  for (int i = threadIdx.x; i < n; i += kEpThreads) {
    int j = i / a.G, s = i - j * a.G;
    rows_s[i] = __ldcg(table + s * a.E + a.rank * a.El + j);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int i = 0; i < n; ++i) {
      if (i % a.G == 0) acc = round_up_rows(acc, a.align);  // a new expert's run
      start_s[i] = acc;
      acc += rows_s[i];
    }
    if (rows_received != nullptr) *rows_received = acc;
    for (int s = 0; s < a.S; ++s) {
      AxmSegment sg;
      sg.a_row0 = 0;
      sg.out_row0 = a.cap + s * a.T_local;
      sg.rows = a.T_local;
      sg.expert = (a.El + s) | AXM_SEG_ALT_A;
      segments[n + s] = sg;
      if (seg_halves != nullptr) seg_halves[2 * a.El + s] = sg;  // projected with the second halves
      if (remote_out != nullptr) {
        AxmRemoteOut ro;
        ro.base = nullptr;  // shared experts stay in the local output buffer
        ro.row0 = 0;
        ro.reserved = 0;
        remote_out[n + s] = ro;
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += kEpThreads) {
    int j = i / a.G, s = i - j * a.G;
    int before = 0;  // source s's own offset of expert rank*El + j
    for (int e = 0; e < a.rank * a.El + j; ++e) before += __ldcg(table + s * a.E + e);
    AxmSegment rs;
    rs.a_row0 = before;
    rs.out_row0 = start_s[i];
    rs.rows = rows_s[i];
    rs.expert = s;
    ret_segments[i] = rs;
    AxmSegment sg;
    sg.expert = j;
    if (remote_out != nullptr) {
      sg.a_row0 = start_s[i];
      sg.out_row0 = start_s[i];
      sg.rows = rows_s[i];
      AxmRemoteOut ro;
      ro.base = a.peers[s] + a.off_oback;
      ro.row0 = before;
      ro.reserved = 0;
      remote_out[i] = ro;
    } else {
      const int first = j * a.G;  // the expert's run starts where its source 0 starts
      // with an alignment the run is padded to a whole number of aligned blocks (zero rows)
      const int end = (j + 1 < a.El) ? start_s[first + a.G]
                                     : round_up_rows(start_s[n - 1] + rows_s[n - 1], a.align);
      sg.a_row0 = start_s[first];
      sg.out_row0 = start_s[first];
      sg.rows = (s == 0) ? end - start_s[first] : 0;
      // The same rows as two segments per expert, cut at a multiple of 256 rows (a pair of
      // m-tiles) near the middle: the down projection of the first halves can be returned
      // while the second halves are still being computed.  seg_halves: [2][El].
      if (seg_halves != nullptr && s == 0) {
        const int rows = end - start_s[first];
        const int pairs = (rows + 255) / 256;
        int cut = ((pairs + 1) / 2) * 256;
        if (cut > rows) cut = rows;
        AxmSegment ha = sg, hb = sg;
        ha.rows = cut;
        hb.a_row0 = hb.out_row0 = start_s[first] + cut;
        hb.rows = rows - cut;
        seg_halves[j] = ha;
        seg_halves[a.El + j] = hb;
        if (split_rows != nullptr) split_rows[j] = start_s[first] + cut;
      }
    }
    segments[i] = sg;
  }
}

__global__ void __launch_bounds__(kEpThreads)
ep_return_kernel(EpArgs a, const AxmSegment* __restrict__ ret_segments,
                 const float* __restrict__ o, int32_t* __restrict__ done_counter,
                 const int32_t* __restrict__ split_rows, int half, int signal) {
  // half: -1 = all rows; 0 = rows of each local expert before split_rows[j]; 1 = the rest.
  // signal: flag the sources when done (the last of the launches that cover a step).
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * (kEpThreads / 32);
  const int chunks = a.D / 4;  // 16-byte pieces of an fp32 row
  const int n = a.G * a.El;
  int seg = 0;
  AxmSegment sg = ret_segments[0];
  for (int r = blockIdx.x * (kEpThreads / 32) + warp;; r += warps_total) {
    while (seg < n && r >= sg.out_row0 + sg.rows) {
      ++seg;
      if (seg < n) sg = ret_segments[seg];
    }
    if (seg >= n) break;
    if (r < sg.out_row0) continue;  // a padding row between two experts' runs (training layout)
    if (half >= 0) {
      const int cut = split_rows[seg / a.G];  // entries are ordered (local expert, source)
      if ((half == 0) != (r < cut)) continue;
    }
    const int dst_row = sg.a_row0 + (r - sg.out_row0);
    if (dst_row >= a.ret_rows) continue;  // the source's buffer, not this rank's row count
    const uint4* src = reinterpret_cast<const uint4*>(o + (size_t)r * a.D);
    uint4* dst = reinterpret_cast<uint4*>(a.peers[sg.expert] + a.off_oback) + (size_t)dst_row * chunks;
    for (int c0 = 0; c0 < chunks; c0 += 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (c0 + u * 32 + lane < chunks) v[u] = __ldg(src + c0 + u * 32 + lane);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (c0 + u * 32 + lane < chunks) dst[c0 + u * 32 + lane] = v[u];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (signal && threadIdx.x == 0) {
    int prev = atomicAdd(done_counter, 1);
    if (prev == (int)gridDim.x - 1) {
      *done_counter = 0;
      __threadfence_system();
      for (int s = 0; s < a.G; ++s) store_release_sys(flag_ptr(a, s, 2, a.rank), a.step);
    }
  }
}

__global__ void ep_wait_return_kernel(EpArgs a) { wait_all_sources(a, 2, 13); }

// Training layout (align > 1): zero the padding rows between one local expert's last row and
// the next aligned start in a [cap][D] bf16 buffer laid out like the receive buffer.  Runs after
// ep_segments_kernel on the same stream (the counts are complete then).  grid (El, parts).
__global__ void __launch_bounds__(kEpThreads)
ep_zero_pad_kernel(EpArgs a, __nv_bfloat16* __restrict__ buf) {
  const int32_t* table = reinterpret_cast<const int32_t*>(a.peers[a.rank] + a.off_counts);
  const int j = blockIdx.x;
  int start = 0, tot = 0;
  for (int q = 0; q <= j; ++q) {
    start += round_up_rows(tot, a.align);
    tot = 0;
    for (int s = 0; s < a.G; ++s) tot += __ldcg(table + s * a.E + a.rank * a.El + q);
  }
  const int pad0 = start + tot;
  int pad1 = start + round_up_rows(tot, a.align);
  if (pad1 > a.cap) pad1 = a.cap;
  const int chunks = a.D / 8;
  const long long pieces = (long long)(pad1 > pad0 ? pad1 - pad0 : 0) * chunks;
  uint4* dst = reinterpret_cast<uint4*>(buf + (size_t)pad0 * a.D);
  for (long long i = (long long)blockIdx.y * kEpThreads + threadIdx.x; i < pieces;
       i += (long long)gridDim.y * kEpThreads)
    dst[i] = make_uint4(0u, 0u, 0u, 0u);
}

// After a down GEMM that stored its rows into the sources' return buffers itself:
// the kernel boundary has made those stores visible; tell every source.
__global__ void ep_signal_return_kernel(EpArgs a) {
  __threadfence_system();
  if ((int)threadIdx.x < a.G) store_release_sys(flag_ptr(a, threadIdx.x, 2, a.rank), a.step);
}

static int validate_ep(const AxmEpLayout* l) {
  if (l == nullptr || l->peers == nullptr) return fail(AXM_ERR_ARGUMENT, "exchange layout or peer table is null");
  if (l->world <= 0 || l->world > kEpMaxRanks || l->rank < 0 || l->rank >= l->world)
    return fail(AXM_ERR_ARGUMENT, "rank %d / world %d out of range (at most %d ranks)", l->rank, l->world, kEpMaxRanks);
  if (l->num_experts <= 0 || l->num_experts % l->world != 0)
    return fail(AXM_ERR_ARGUMENT, "num_experts %d must be a positive multiple of world %d", l->num_experts, l->world);
  if (l->num_experts / l->world > 64) return fail(AXM_ERR_ARGUMENT, "more than 64 experts per rank");
  if (l->d_model <= 0 || l->d_model % 8 != 0) return fail(AXM_ERR_ARGUMENT, "d_model %d not a multiple of 8", l->d_model);
  if (l->slots < 0 || l->cap < 0) return fail(AXM_ERR_ARGUMENT, "negative row count");
  if (l->row_align < 0 || l->row_align > 1024) return fail(AXM_ERR_ARGUMENT, "row_align %d not in 0..1024", l->row_align);
  return AXM_OK;
}

static EpArgs make_args(const AxmEpLayout* l, uint32_t step, int32_t* status) {
  EpArgs a;
  a.peers = reinterpret_cast<char* const*>(const_cast<void* const*>(l->peers));
  a.rank = l->rank;
  a.G = l->world;
  a.E = l->num_experts;
  a.El = l->num_experts / l->world;
  a.D = l->d_model;
  a.slots = l->slots;
  a.ret_rows = l->return_rows > l->slots ? l->return_rows : l->slots;
  a.cap = l->cap;
  a.S = l->num_shared;
  a.T_local = l->tokens_local;
  a.align = l->row_align > 1 ? l->row_align : 1;
  a.step = step;
  a.off_counts = l->off_counts;
  a.off_flags = l->off_flags;
  a.off_recv = l->off_recv;
  a.off_oback = l->off_oback;
  a.status = status;
  return a;
}

int launch_ep_permute_dispatch(const AxmEpLayout* l, uint32_t step, const void* x, const int32_t* topk_idx,
                               const int32_t* block_counts, int32_t* histogram, int32_t* offsets,
                               int32_t* row_src, int32_t* slot_dst, int32_t* done_counter, int T, int k,
                               int hist_accumulate, int32_t* status, cudaStream_t st) {
  if (int rc = validate_ep(l)) return rc;
  if (l->num_experts > kFusedMaxE) return fail(AXM_ERR_ARGUMENT, "num_experts %d > %d", l->num_experts, kFusedMaxE);
  EpArgs a = make_args(l, step, status);
  ep_permute_dispatch_kernel<<<AXM_ROUTE_BLOCKS, kEpThreads, 0, st>>>(
      a, static_cast<const __nv_bfloat16*>(x), topk_idx, block_counts, histogram, offsets, row_src, slot_dst,
      done_counter, T, k, hist_accumulate);
  return check_launch("ep_permute_dispatch_kernel");
}

int launch_ep_segments_split(const AxmEpLayout* l, uint32_t step, AxmSegment* segments, AxmSegment* ret_segments,
                             int32_t* rows_received, AxmSegment* seg_halves, int32_t* split_rows,
                             int32_t* status, cudaStream_t st) {
  if (int rc = validate_ep(l)) return rc;
  EpArgs a = make_args(l, step, status);
  ep_segments_kernel<<<1, kEpThreads, 0, st>>>(a, segments, ret_segments, nullptr, rows_received, seg_halves,
                                              split_rows);
  return check_launch("ep_segments_kernel");
}

int launch_ep_return_half(const AxmEpLayout* l, uint32_t step, const AxmSegment* ret_segments, const void* o,
                          int32_t* done_counter, const int32_t* split_rows, int half, int signal,
                          int32_t* status, cudaStream_t st) {
  if (int rc = validate_ep(l)) return rc;
  EpArgs a = make_args(l, step, status);
  ep_return_kernel<<<2 * sm_count(), kEpThreads, 0, st>>>(a, ret_segments, static_cast<const float*>(o),
                                                         done_counter, split_rows, half, signal);
  return check_launch("ep_return_kernel");
}

// Zero rows behind every local expert's run in `buf` ([cap][D] bf16, receive-buffer layout).
int launch_ep_zero_pad(const AxmEpLayout* l, uint32_t step, void* buf, cudaStream_t st) {
  if (int rc = validate_ep(l)) return rc;
  if (l->row_align <= 1) return AXM_OK;
  EpArgs a = make_args(l, step, nullptr);
  ep_zero_pad_kernel<<<dim3(a.El, 8), kEpThreads, 0, st>>>(a, static_cast<__nv_bfloat16*>(buf));
  return check_launch("ep_zero_pad_kernel");
}

}  // namespace axm

using namespace axm;

extern "C" int axm_ep_region_bytes(int32_t world, int32_t num_experts, int32_t d_model,
                                   int32_t slots, int32_t cap, AxmEpLayout* layout,
                                   size_t* bytes) {
  if (!layout || !bytes) return fail(AXM_ERR_ARGUMENT, "axm_ep_region_bytes: null pointer");
  if (world <= 0 || num_experts <= 0 || d_model <= 0 || slots < 0 || cap < 0)
    return fail(AXM_ERR_ARGUMENT, "axm_ep_region_bytes: bad sizes");
  auto up = [](long long v) { return (v + 255) & ~255LL; };
  long long off = 0;
  layout->off_flags = off;
  off = up(off + 4LL * 3 * world);
  layout->off_counts = off;
  off = up(off + 4LL * world * num_experts);
  layout->off_recv = off;
  off = up(off + 2LL * cap * d_model);
  layout->off_oback = off;
  off = up(off + 4LL * slots * d_model);
  layout->world = world;
  layout->num_experts = num_experts;
  layout->d_model = d_model;
  layout->slots = slots;
  layout->cap = cap;
  layout->row_align = 1;
  layout->return_rows = 0;
  *bytes = (size_t)off;
  return AXM_OK;
}

extern "C" int axm_ep_dispatch(const AxmEpLayout* layout, uint32_t step, const int32_t* offsets,
                               const void* x_perm, int32_t* scratch, int32_t* status, void* stream) {
  if (int rc = validate_ep(layout)) return rc;
  if (!offsets || !x_perm || !scratch) return fail(AXM_ERR_ARGUMENT, "axm_ep_dispatch: null pointer");
  if (int rc = require_device()) return rc;
  EpArgs a = make_args(layout, step, status);
  ep_dispatch_kernel<<<2 * sm_count(), kEpThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      a, offsets, static_cast<const __nv_bfloat16*>(x_perm), scratch);
  return check_launch("ep_dispatch_kernel");
}

extern "C" int axm_ep_segments(const AxmEpLayout* layout, uint32_t step, AxmSegment* segments,
                               AxmSegment* ret_segments, AxmRemoteOut* remote_out,
                               int32_t* rows_received, int32_t* status, void* stream) {
  if (int rc = validate_ep(layout)) return rc;
  if (!segments || !ret_segments) return fail(AXM_ERR_ARGUMENT, "axm_ep_segments: null pointer");
  if (int rc = require_device()) return rc;
  EpArgs a = make_args(layout, step, status);
  ep_segments_kernel<<<1, kEpThreads, 0, static_cast<cudaStream_t>(stream)>>>(a, segments, ret_segments,
                                                                             remote_out, rows_received, nullptr,
                                                                             nullptr);
  return check_launch("ep_segments_kernel");
}

extern "C" int axm_ep_return(const AxmEpLayout* layout, uint32_t step,
                             const AxmSegment* ret_segments, const void* o, int32_t* scratch,
                             int32_t* status, void* stream) {
  if (int rc = validate_ep(layout)) return rc;
  if (!ret_segments || !o || !scratch) return fail(AXM_ERR_ARGUMENT, "axm_ep_return: null pointer");
  if (int rc = require_device()) return rc;
  EpArgs a = make_args(layout, step, status);
  ep_return_kernel<<<2 * sm_count(), kEpThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      a, ret_segments, static_cast<const float*>(o), scratch + 1, nullptr, -1, 1);
  return check_launch("ep_return_kernel");
}

extern "C" int axm_ep_signal_return(const AxmEpLayout* layout, uint32_t step, void* stream) {
  if (int rc = validate_ep(layout)) return rc;
  if (int rc = require_device()) return rc;
  EpArgs a = make_args(layout, step, nullptr);
  ep_signal_return_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return check_launch("ep_signal_return_kernel");
}

extern "C" int axm_ep_wait_return(const AxmEpLayout* layout, uint32_t step, int32_t* status,
                                  void* stream) {
  if (int rc = validate_ep(layout)) return rc;
  if (int rc = require_device()) return rc;
  EpArgs a = make_args(layout, step, status);
  ep_wait_return_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return check_launch("ep_wait_return_kernel");
}
