// Streaming router: the logits as a tall-skinny tensor-core product, softmax / top-k /
// gates in the epilogue, all of x read from HBM exactly once.
//
// Stands in for top2_router_kernel of the reference engine
// (core/src/CUDA/kernel/moe_router.cu:27-111).  Everything after the logits is the same
// device function the routing-from-logits entry point runs (route_one_token, router.cuh),
// so expert indices and gates are bit-identical for identical logits; the logits differ
// from a sequential fp32 sum only by summation order (|dz| <= 1e-4 * max(1, |z|)).
//
// Why a tensor-core kernel for a memory-bound stage: with E experts every bf16 element of
// x costs E multiply-adds.  On CUDA cores that is as long as the HBM time already at E = 8
// and six times longer at E = 64; on the tensor core it is a few per cent of it.
//
// Shape of the product: a tile is 128 tokens (M) x N columns x D (K), bf16 in, fp32
// accumulate in tensor memory.  fp32 router weights are split exactly into three bf16
// terms w = hi + mid + lo (8 + 8 + 8 mantissa bits) by a small preparation kernel that
// also transposes them to K-major; the three terms sit side by side along N
// (N = 3 * Epad, Epad = E rounded up to 16), so one tcgen05.mma per 16 k produces all
// three partial products and the epilogue adds them.  bf16 router weights use one term.
//
// Work split: one thread-block cluster of CS CTAs (1, 2 or 4) per tile, each reducing over
// its share of D, so that two CTAs per SM keep 100+ KB of x in flight per SM even for a few
// thousand tokens.  CS depends on the layer's shape only, never on the
// number of tokens: a token's logits have the same summation order whatever batch it is
// in (expert-parallel ranks and the single-GPU layer must route identically).  CTA r takes
// the 64-wide blocks r, r + CS, ... of d_model.  After the reduction loop one cluster barrier
// makes every CTA's stage memory reusable; each thread adds its row's three terms and stores
// the row's partial logits into the CTA that owns the row (plain st.shared::cluster stores,
// then an arrival on the owner's mbarrier); CTA r owns rows [r * 128 / CS, (r + 1) * 128 / CS)
// of the tile: it adds the slices in rank order, adds the bias, writes the logits and routes
// one token per thread.
//
// Per-block expert counts for the permute kernel go to block_counts with integer atomics
// (order-independent, hence deterministic); the preparation kernel zeroes the table.
// The main kernel is launched with programmatic stream serialization: its prologue and its
// first loads of x overlap the preparation kernel, and griddepcontrol.wait orders
// everything that depends on it.
#include <cuda.h>

#include <cstdlib>

#include "gemm_common.cuh"
#include "router.cuh"

namespace axm {

constexpr int kRtThreads = 192;     // warp 0: TMA producer, warp 1: MMA issuer, warps 2-5: epilogue
constexpr int kRtMaxStages = 8;
constexpr int kRtTileRows = 128;
constexpr int kRtABytes = kRtTileRows * BK * 2;   // 16 KiB
constexpr int kRtStageBudget = 100 * 1024;        // two CTAs per SM

struct __align__(8) RouterTcShared {
  uint64_t full[kRtMaxStages];
  uint64_t empty[kRtMaxStages];
  uint64_t tmem_full;
  uint64_t exch_full;   // 128 arrivals: every row of this CTA's slice of the tile, from every CTA of the cluster
  uint32_t tmem_base;
  int abort_flag;
};

struct RouterTcArgs {
  // Pre-norm form: the router sees RMSNorm(x) without anybody having written it to memory.
  // norm_rstd[t] = rsqrt(mean(x[t]^2) + eps); the epilogue warps then load x themselves,
  // form bf16(x * rstd * gamma) exactly as the RMSNorm kernel does and store it in the layout
  // the tensor core reads; the TMA producer only brings the weight tiles.  NULL: x by TMA.
  const __nv_bfloat16* x;
  const float* norm_rstd;
  const float* norm_gamma;  // [D] or NULL (ones)
  const float* bias;
  float* logits_out;
  int32_t* topk_idx;
  float* topk_gate;
  int32_t* block_counts;
  int32_t* status;
  int T, D, E, k;
  int epad;        // E rounded up to a multiple of 16
  int terms;       // 3 (fp32 weights) or 1 (bf16 weights)
  int n_cols;      // terms * epad: N of the MMA
  int stages;
  int stage_bytes; // A tile + B tile, a multiple of 1024
  int tmem_cols;   // power of two >= max(32, n_cols)
  int exch_bytes;  // bytes of the exchange buffer [CS][128 / CS][epad + 4] floats, 16-byte multiple
  int tile_bytes;  // bytes of the region shared by the pipeline stages and, later, exchange buffer + logits
};

__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t rt_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void rt_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t rt_map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void rt_st_cluster_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}
// 32 lanes x 16 consecutive fp32 columns of tensor memory
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void rt_mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Bounded wait on a barrier whose arrivals come from other CTAs of the cluster.
__device__ __forceinline__ bool rt_mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const uint32_t addr = smem_u32(bar);
  long long t0 = clock64();
  while (true) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) {
      *abort_flag = 1;
      return false;
    }
  }
}
__device__ __forceinline__ void epilogue_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// fp32 accumulate, bf16 A and B, both K-major, M = 128, N = n
__device__ __forceinline__ uint32_t rt_instr_desc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kRtTileRows >> 4) << 24);
}

// ---- preparation: split + transpose the router weights, zero the count table ------------
// bt[(term * epad + e) * D + d] = term-th bf16 piece of w[d][e]; rows e >= E are zero.
template <typename WT>
__global__ void __launch_bounds__(256)
router_prep_kernel(const WT* __restrict__ w, __nv_bfloat16* __restrict__ bt, int32_t* __restrict__ block_counts,
                   int32_t* __restrict__ status, int D, int E, int epad, int n_counts) {
  griddep_launch();  // the router kernel may start its prologue now; it waits before it depends on this grid
  if (status != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *status = 0;  // first kernel of a layer call
  constexpr int kTerms = sizeof(WT) == 4 ? 3 : 1;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (long long i = tid; i < n_counts; i += stride) block_counts[i] = 0;
  const long long total = (long long)epad * D;
  for (long long i = tid; i < total; i += stride) {
    const int e = (int)(i / D), d = (int)(i - (long long)e * D);
    if (kTerms == 3) {
      float v = e < E ? __ldg(reinterpret_cast<const float*>(w) + (size_t)d * E + e) : 0.0f;
#pragma unroll
      for (int t = 0; t < 3; ++t) {
        const __nv_bfloat16 h = __float2bfloat16_rn(v);
        bt[((size_t)t * epad + e) * D + d] = h;
        v -= __bfloat162float(h);  // exact: the residual has fewer significant bits each time
      }
    } else {
      const __nv_bfloat16* wb = reinterpret_cast<const __nv_bfloat16*>(w);
      bt[(size_t)e * D + d] = e < E ? wb[(size_t)d * E + e] : __float2bfloat16_rn(0.0f);
    }
  }
}

// ---- the router ---------------------------------------------------------------------------
template <int CS>
__global__ void __launch_bounds__(kRtThreads)
router_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_b,
                 RouterTcArgs a) {
  constexpr int RP = kRtTileRows / CS;  // rows of the tile this CTA routes
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  // After the reduction loop the stage memory is reused: exchange buffer [CS][RP][epad + 4]
  // floats, then this CTA's logits [RP][E + 1].
  float* exch = reinterpret_cast<float*>(tiles);
  float* z_s = reinterpret_cast<float*>(tiles + a.exch_bytes);
  RouterTcShared* sh = reinterpret_cast<RouterTcShared*>(tiles + a.tile_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = CS > 1 ? rt_cluster_rank() : 0u;
  const int tile = blockIdx.x / CS;
  const int row0 = tile * kRtTileRows;
  const int kb_total = (a.D + BK - 1) / BK;
  // Which 64-wide blocks of d_model this CTA reduces over: rank, rank + CS, ...  The CTAs of a
  // cluster run in step, so together they ask HBM for CS adjacent 128-byte pieces of a row.
  const int kb_count = max(0, (kb_total - (int)rank + CS - 1) / CS);
  const int EP = a.E + 1;
  const int xld = a.epad + 4;  // row pitch of the exchange buffer in floats (conflict-free 16-byte stores)

  if (threadIdx.x == 0) {
    for (int i = 0; i < a.stages; ++i) {
      mbar_init(&sh->full[i], a.norm_rstd != nullptr ? 129 : 1);  // + the 128 loading threads
      mbar_init(&sh->empty[i], 1);
    }
    mbar_init(&sh->tmem_full, 1);
    mbar_init(&sh->exch_full, kRtTileRows);  // one arrival per row of the tile slice this CTA owns, from every CTA
    sh->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_b);
  }
  __syncthreads();
  // The producer warp starts requesting tiles at once; tensor memory is allocated meanwhile
  // and only the MMA and epilogue warps (160 threads, named barrier 2) wait for its address.
  uint32_t tmem_base = 0;
  if (warp >= 1) {
    if (warp == 1) {
      tmem_alloc(&sh->tmem_base, (uint32_t)a.tmem_cols);
      tmem_relinquish();
    }
    tc_fence_before();
    asm volatile("bar.sync 2, 160;" ::: "memory");
    tc_fence_after();
    tmem_base = sh->tmem_base;
  }
  volatile int* abort_flag = &sh->abort_flag;
  const bool by_warps = a.norm_rstd != nullptr;  // activation tiles produced by the epilogue warps
  const uint32_t stage_tx = (uint32_t)((by_warps ? 0 : kRtABytes) + a.n_cols * BK * 2);

  if (warp == 0) {
    // ---- TMA producer -----------------------------------------------------------------
    if (lane == 0) {
      // x does not depend on the preparation kernel: the first ring of activation tiles is
      // requested before the wait, the weight tiles of those stages after it
      const int early = min(a.stages, kb_count);
      for (int i = 0; i < early; ++i) {
        mbar_expect_tx(&sh->full[i], stage_tx);
        if (!by_warps)
          tma_load_2d(tiles + (size_t)i * a.stage_bytes, &tm_x, &sh->full[i], ((int)rank + i * CS) * BK, row0);
      }
      griddep_wait();
      for (int i = 0; i < early; ++i)
        tma_load_2d(tiles + (size_t)i * a.stage_bytes + kRtABytes, &tm_b, &sh->full[i], ((int)rank + i * CS) * BK, 0);
      int stage = early == a.stages ? 0 : early;
      uint32_t phase = early == a.stages ? 1u : 0u;
      for (int i = early; i < kb_count; ++i) {
        if (!mbar_wait(&sh->empty[stage], phase ^ 1u, abort_flag)) break;
        unsigned char* sa = tiles + (size_t)stage * a.stage_bytes;
        mbar_expect_tx(&sh->full[stage], stage_tx);
        if (!by_warps) tma_load_2d(sa, &tm_x, &sh->full[stage], ((int)rank + i * CS) * BK, row0);
        tma_load_2d(sa + kRtABytes, &tm_b, &sh->full[stage], ((int)rank + i * CS) * BK, 0);
        if (++stage == a.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer -------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = rt_instr_desc(a.n_cols);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = 0; i < kb_count; ++i) {
        if (!mbar_wait(&sh->full[stage], phase, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(tiles + (size_t)stage * a.stage_bytes);
        const uint64_t da = make_smem_desc(sa, 16, 1024);
        const uint64_t db = make_smem_desc(sa + kRtABytes, 16, 1024);
#pragma unroll
        for (int j = 0; j < BK / UMMA_K; ++j)
          tc_mma_bf16(tmem_base, da + (uint64_t)(j * 2), db + (uint64_t)(j * 2), idesc, (i > 0 || j > 0) ? 1u : 0u);
        tc_commit(&sh->empty[stage]);
        if (++stage == a.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) tc_commit(&sh->tmem_full);
    }
  }

  if (warp >= 2) {
    // ---- pre-norm form: these warps produce the activation tiles -----------------------------
    // A row's 128 bytes of a k-block are loaded by eight neighbouring lanes (16 bytes each),
    // scaled and rounded like the RMSNorm kernel, and stored with the 128-byte swizzle of the
    // tensor-core layout: 16-byte piece c of row r at r * 128 + ((c ^ (r & 7)) * 16).
    if (by_warps) {
      const int lt = (warp - 2) * 32 + lane;
      const int c = lt & 7, rsub = lt >> 3;  // piece of the row, row within a group of 16
      const int chunks = a.D / 8;
      float rstd[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int r = row0 + rsub + 16 * j;
        rstd[j] = r < a.T ? __ldg(a.norm_rstd + r) : 0.0f;
      }
      auto fetch = [&](int i, uint4 (&v)[8]) {
        const int piece = ((int)rank + i * CS) * 8 + c;  // 16-byte piece index inside a row of x
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int r = row0 + rsub + 16 * j;
          v[j] = make_uint4(0, 0, 0, 0);
          if (r < a.T && piece < chunks) v[j] = __ldg(reinterpret_cast<const uint4*>(a.x + (size_t)r * a.D) + piece);
        }
      };
      uint4 cur[8], nxt[8];
      if (kb_count > 0) fetch(0, cur);
      for (int i = 0; i < kb_count; ++i) {
        if (i + 1 < kb_count) fetch(i + 1, nxt);
        const int stage = i % a.stages;
        const uint32_t use = (uint32_t)(i / a.stages);
        if (!__all_sync(0xffffffffu, mbar_wait(&sh->empty[stage], (use & 1u) ^ 1u, abort_flag))) break;
        unsigned char* sa = tiles + (size_t)stage * a.stage_bytes;
        const int d0 = (((int)rank + i * CS) * 8 + c) * 8;  // first of this lane's eight columns
        float gm[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) gm[q] = (a.norm_gamma != nullptr && d0 + q < a.D) ? __ldg(a.norm_gamma + d0 + q) : 1.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int r = rsub + 16 * j;
          const uint32_t w4[4] = {cur[j].x, cur[j].y, cur[j].z, cur[j].w};
          uint32_t o4[4];
#pragma unroll
          for (int q = 0; q < 4; ++q)
            o4[q] = pack_bf16(bf16_lo(w4[q]) * rstd[j] * gm[2 * q], bf16_hi(w4[q]) * rstd[j] * gm[2 * q + 1]);
          *reinterpret_cast<uint4*>(sa + r * 128 + ((c ^ (r & 7)) << 4)) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
        }
        fence_proxy_async();  // the tensor core reads these bytes through the async proxy
        mbar_arrive(&sh->full[stage]);
#pragma unroll
        for (int j = 0; j < 8; ++j) cur[j] = nxt[j];
      }
    }
    // ---- epilogue: 128 threads, thread = accumulator row ----------------------------------
    const int quad = warp & 3;
    bool acc_ok = true;
    if (kb_count > 0) {
      acc_ok = __all_sync(0xffffffffu, mbar_wait(&sh->tmem_full, 0u, abort_flag));
      tc_fence_after();
    }
    // One cluster barrier per kernel: a thread arrives when its part of the reduction loop is
    // over (for these warps: the accumulator is complete, so every tile this CTA requested has
    // landed and been read).  Once it completes, the stage memory of every CTA of the cluster
    // is free to receive the partial sums.
    if (CS > 1) {
      asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    {
      // this CTA's partial logits of row r, (hi + mid) + lo, 16 experts at a time, stored into
      // the row's owner
      const int r = quad * 32 + lane;
      const int owner = r / RP, lr = r - owner * RP;
      const uint32_t dst_local = smem_u32(exch + ((size_t)rank * RP + lr) * xld);
      const uint32_t dst = CS > 1 ? rt_map_to_cta(dst_local, (uint32_t)owner) : dst_local;
      const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
      const bool have = kb_count > 0 && acc_ok;  // a CTA without k-blocks contributes zeros
      for (int c0 = 0; c0 < a.epad; c0 += 16) {
        float part[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) part[j] = 0.0f;
        if (have) {
          uint32_t hi[16], mid[16], lo[16];
          const uint32_t col = t_addr + (uint32_t)c0;
          tmem_ld16(col, hi);
          if (a.terms == 3) {
            tmem_ld16(col + (uint32_t)a.epad, mid);
            tmem_ld16(col + (uint32_t)(2 * a.epad), lo);
          }
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float v = __uint_as_float(hi[j]);
            if (a.terms == 3) v = (v + __uint_as_float(mid[j])) + __uint_as_float(lo[j]);
            part[j] = v;
          }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q)
          rt_st_cluster_v4(dst + (uint32_t)(c0 + 4 * q) * 4u, __float_as_uint(part[4 * q]),
                           __float_as_uint(part[4 * q + 1]), __float_as_uint(part[4 * q + 2]),
                           __float_as_uint(part[4 * q + 3]));
      }
      tc_fence_before();
      // tell the owner that this row's slice has landed (release at cluster scope orders the stores)
      const uint32_t bar_local = smem_u32(&sh->exch_full);
      rt_mbar_arrive_cluster(CS > 1 ? rt_map_to_cta(bar_local, (uint32_t)owner) : bar_local);
    }
    const bool got_all = __all_sync(0xffffffffu, rt_mbar_wait_cluster(&sh->exch_full, 0u, abort_flag));
    griddep_wait();  // the count table was zeroed by the preparation kernel
    const int et = (warp - 2) * 32 + lane;  // 0..127
    const int t_first = row0 + (int)rank * RP;
    const int rows_here = got_all ? max(0, min(RP, a.T - t_first)) : 0;
    // z = sum over the CTAs' slices in rank order, then + bias
    for (int i = et; i < rows_here * a.E; i += 128) {
      const int lr = i / a.E, e = i - lr * a.E;
      float z = 0.0f;
#pragma unroll
      for (int s = 0; s < CS; ++s) z += exch[((size_t)s * RP + lr) * xld + e];
      if (a.bias != nullptr) z += __ldg(a.bias + e);
      z_s[lr * EP + e] = z;
      if (a.logits_out != nullptr) a.logits_out[(size_t)t_first * a.E + i] = z;
    }
    epilogue_bar_sync();
    if (et < rows_here) {
      const int t = t_first + et;
      const int b = (int)((((long long)t + 1) * AXM_ROUTE_BLOCKS - 1) / a.T);  // the token's block of the permute split
      route_one_token<kRouteMaxK>(z_s + et * EP, a.E, a.k, a.topk_idx + (size_t)t * a.k,
                                  a.topk_gate + (size_t)t * a.k, a.block_counts + (size_t)b * a.E);
    }
  } else {
    __syncwarp();
    if (CS > 1) {
      asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
  }

  // ---- teardown ------------------------------------------------------------------------
  // Nobody stores into this CTA's shared memory any more: its exchange barrier has seen all
  // 128 arrivals (or a wait gave up and the status word says so).
  __syncthreads();
  if (sh->abort_flag != 0) {
    long long t0 = clock64();
    while (clock64() - t0 < 4000000LL) {
    }
    if (threadIdx.x == 0 && a.status != nullptr) atomicExch(a.status, 14);
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)a.tmem_cols);
  }
}

// ---- host side ----------------------------------------------------------------------------

static bool router_tc_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("AXM_ROUTER_TC");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

RouterTcPlan router_tc_plan(const AxmMoeDesc* d) {
  RouterTcPlan p = {};
  p.terms = d->router_dtype == AXM_ROUTER_FP32 ? 3 : 1;
  p.epad = (d->num_experts + 15) / 16 * 16;
  p.n_cols = p.terms * p.epad;
  if (!router_tc_enabled() || p.n_cols > 256 || d->d_model % 8 != 0) return p;  // ok = false
  const int b_bytes = (p.n_cols * BK * 2 + 1023) / 1024 * 1024;
  p.stage_bytes = kRtABytes + b_bytes;
  const int kb_total = (d->d_model + BK - 1) / BK;
  // CTAs per cluster = slices of d_model: a function of the layer's shape alone, never of the
  // token count.  Four slices where the exchange is cheap (few columns); with many experts the
  // epilogue (exchange, per-token top-k over E) weighs more than the stream and two are faster
  // (measured at T 16384, D 2048, E 64: 31 us against 45).
  p.cs = kb_total >= 16 && p.n_cols <= 64 ? 4 : (kb_total >= 4 ? 2 : 1);
  p.exch_bytes = kRtTileRows * (p.epad + 4) * 4;
  p.stages = kRtStageBudget / p.stage_bytes;
  p.stages = p.stages < 2 ? 2 : (p.stages > kRtMaxStages ? kRtMaxStages : p.stages);
  p.tmem_cols = 32;
  while (p.tmem_cols < p.n_cols) p.tmem_cols *= 2;
  const int after_loop = p.exch_bytes + 4 * (kRtTileRows / p.cs) * (d->num_experts + 1);
  p.tile_bytes = p.stages * p.stage_bytes > after_loop ? p.stages * p.stage_bytes : (after_loop + 1023) / 1024 * 1024;
  p.smem_bytes = 1024 + (size_t)p.tile_bytes + sizeof(RouterTcShared);
  p.scratch_bytes = ((size_t)p.n_cols * d->d_model * 2 + 255) & ~(size_t)255;
  p.ok = p.smem_bytes <= 227u * 1024u;
  return p;
}

template <int CS>
static int launch_router_tc_cs(const RouterTcPlan& p, const CUtensorMap& mx, const CUtensorMap& mb,
                               const RouterTcArgs& args, int tiles, cudaStream_t st) {
  static SmemLimitCache cache = {};
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(router_tc_kernel<CS>), p.smem_bytes, &cache,
                                   "router_tc_kernel"))
    return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * CS), 1, 1);
  cfg.blockDim = dim3(kRtThreads, 1, 1);
  cfg.dynamicSmemBytes = p.smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attrs[2];
  int n = 0;
  attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[n].val.programmaticStreamSerializationAllowed = 1;
  ++n;
  if (CS > 1) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = CS;
    attrs[n].val.clusterDim.y = 1;
    attrs[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  return cuda_status(cudaLaunchKernelEx(&cfg, router_tc_kernel<CS>, mx, mb, args), "router_tc_kernel");
}

// Returns AXM_OK after enqueueing the preparation and router kernels.
int launch_router_tc(const AxmMoeDesc* d, const RouterTcPlan& p, const void* x, const void* router_w,
                     const float* bias, float* logits, int32_t* idx, float* gate, int32_t* block_counts,
                     void* scratch, int32_t* status, cudaStream_t st, const float* norm_rstd,
                     const float* norm_gamma) {
  const int T = d->tokens, D = d->d_model, E = d->num_experts;
  CUtensorMap mx, mb;
  {
    const uint64_t dims[2] = {(uint64_t)D, (uint64_t)(T > 0 ? T : 1)};
    const uint64_t strides[1] = {(uint64_t)D * 2};
    const uint32_t box[2] = {(uint32_t)BK, (uint32_t)kRtTileRows};
    if (int rc = encode_tensor_map(&mx, x, 2, dims, strides, box)) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)D, (uint64_t)p.n_cols};
    const uint64_t strides[1] = {(uint64_t)D * 2};
    const uint32_t box[2] = {(uint32_t)BK, (uint32_t)p.n_cols};
    if (int rc = encode_tensor_map(&mb, scratch, 2, dims, strides, box)) return rc;
  }
  const int n_counts = AXM_ROUTE_BLOCKS * E;
  long long work = (long long)p.epad * D;
  int blocks = (int)((work + 255) / 256);
  if (blocks > 2 * sm_count()) blocks = 2 * sm_count();
  if (d->router_dtype == AXM_ROUTER_FP32)
    router_prep_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(router_w),
                                                      static_cast<__nv_bfloat16*>(scratch), block_counts, status,
                                                      D, E, p.epad, n_counts);
  else
    router_prep_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(router_w),
                                                              static_cast<__nv_bfloat16*>(scratch), block_counts,
                                                              status, D, E, p.epad, n_counts);
  if (int rc = check_launch("router_prep_kernel")) return rc;
  RouterTcArgs a;
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.norm_rstd = norm_rstd;
  a.norm_gamma = norm_gamma;
  a.bias = bias;
  a.logits_out = logits;
  a.topk_idx = idx;
  a.topk_gate = gate;
  a.block_counts = block_counts;
  a.status = status;
  a.T = T;
  a.D = D;
  a.E = E;
  a.k = d->top_k;
  a.epad = p.epad;
  a.terms = p.terms;
  a.n_cols = p.n_cols;
  a.stages = p.stages;
  a.stage_bytes = p.stage_bytes;
  a.tmem_cols = p.tmem_cols;
  a.exch_bytes = p.exch_bytes;
  a.tile_bytes = p.tile_bytes;
  const int tiles = (T + kRtTileRows - 1) / kRtTileRows;
  switch (p.cs) {
    case 4: return launch_router_tc_cs<4>(p, mx, mb, a, tiles, st);
    case 2: return launch_router_tc_cs<2>(p, mx, mb, a, tiles, st);
    default: return launch_router_tc_cs<1>(p, mx, mb, a, tiles, st);
  }
}

}  // namespace axm

