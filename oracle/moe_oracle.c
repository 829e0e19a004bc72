/*
 * CPU oracle for the mixture-of-experts layer (router -> dispatch -> expert
 * SwiGLU FFN -> combine).
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or
 * calls this file; it exists so that the CUDA path can be checked against an
 * independent scalar statement of the layer's arithmetic, and so that a CPU
 * timing can be printed beside the GPU number.
 *
 * It is written from the layer's specification (softmax router, top-k with the
 * lowest index winning ties, renormalised gates, per-expert histogram, SwiGLU
 * experts with fp32 accumulation, weighted combine, residual) and follows the
 * operator conventions of the engine it stands in for.  The citations below
 * name where that engine defines each convention (paths inside its project);
 * no text of it is reproduced here.
 *
 *   router logits, sequential fp32 sum over d ....... core/src/CUDA/kernel/moe_router.cu:42-57
 *   softmax with 1/(sum + 1e-9f) .................... core/src/CUDA/kernel/moe_router.cu:59-76
 *   top-1 / top-2 by strict '>' ascending scan ...... core/src/CUDA/kernel/moe_router.cu:78-95
 *   gates p_i / (sum of selected p + 1e-9f) ......... core/src/CUDA/kernel/moe_router.cu:97-105
 *   histogram, accumulating across calls ............ core/src/CUDA/kernel/moe_router.cu:107-110
 *   expert FFN, SiLU(g)*u kept in fp32 .............. core/src/CUDA/kernel/moe_router.cu:155-173
 *   down projection, gate-weighted sum, one rounding  core/src/CUDA/kernel/moe_router.cu:177-190
 *   residual add with a second bf16 rounding ........ core/src/CUDA/kernel/moe_router.cu:193-203
 *   weight layouts [D][E], [E][D][F], [E][F][D] ..... core/src/CUDA/util/gpu_types.cuh:147-157
 *   SiLU*mul and its derivative ..................... core/src/CUDA/kernel/swiglu.cu:19-55
 *   AdamW as the engine's fused kernel applies it ... core/src/CUDA/kernel/backward_pass.cu:812-852
 *
 * Parity status: the engine's own tests hold no numeric vectors for this layer
 * (only "histogram sums to 2T, no dead expert, outputs finite").  The oracle is
 * pinned by running the engine's unmodified kernels next to it on a GPU (see
 * oracle/build_ref.sh and tests/test_reference_parity_gpu.py); where that binary is
 * not present those tests skip with the reason "parity unpinned".
 *
 * All tensors are row-major.  bf16 values travel as uint16_t.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* round-to-nearest-even, the conversion CUDA's __float2bfloat16_rn performs */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

static inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Number of threads the parallel loops use from now on (n <= 0: leave as is).  A launcher
 * may have set OMP_NUM_THREADS=1 for its workers; a timing run asks for the cores it wants. */
ORC_API void orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

ORC_API void orc_f32_to_bf16(const float* src, uint16_t* dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_bf16(src[i]);
}

ORC_API void orc_bf16_to_f32(const uint16_t* src, float* dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = bf16_to_f32(src[i]);
}

/* ------------------------------------------------------------------ router */

/*
 * z[t,e] = sum_d x[t,d] * Wr[d,e] (+ bias[e]), one fused multiply-add per d in
 * ascending d.  wr_is_fp32 selects the router-weight dtype: bf16 is what the
 * drop-in interface carries, fp32 is what the benchmark configurations use.
 * With bf16 weights every product is exact in fp32, so fused and unfused
 * multiply-add give the same bits.
 */
ORC_API void orc_router_logits(const uint16_t* x, const void* wr, int wr_is_fp32,
                               const float* bias, int T, int D, int E, float* logits) {
  const float* wf = (const float*)wr;
  const uint16_t* wh = (const uint16_t*)wr;
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t) {
    float* z = logits + (size_t)t * E;
    for (int e = 0; e < E; ++e) z[e] = 0.0f;
    for (int d = 0; d < D; ++d) {
      float xv = bf16_to_f32(x[(size_t)t * D + d]);
      if (wr_is_fp32) {
        const float* w = wf + (size_t)d * E;
        for (int e = 0; e < E; ++e) z[e] = fmaf(xv, w[e], z[e]);
      } else {
        const uint16_t* w = wh + (size_t)d * E;
        for (int e = 0; e < E; ++e) z[e] = fmaf(xv, bf16_to_f32(w[e]), z[e]);
      }
    }
    if (bias)
      for (int e = 0; e < E; ++e) z[e] += bias[e];
  }
}

static inline int32_t float_order(float f) { /* monotone map of non-negative floats */
  int32_t i;
  memcpy(&i, &f, 4);
  return i;
}

/*
 * Softmax, top-k, gates and histogram from given fp32 logits.
 *   idx   [T][k] int32, slot 0 = best
 *   gates [T][k] fp32
 *   probs [T][E] fp32 or NULL
 *   counts[E]    int32, INCREMENTED (the histogram accumulates across calls)
 *   near_tie [T] uint8 or NULL: 1 where two of the k+1 largest probabilities lie
 *            within 4 units in the last place of each other, i.e. where an exp
 *            implementation that differs by an ulp may legitimately pick another
 *            expert.
 */
ORC_API void orc_route_from_logits(const float* logits, int T, int E, int k, int32_t* idx,
                                   float* gates, float* probs, int32_t* counts,
                                   uint8_t* near_tie) {
  float* p = (float*)malloc(sizeof(float) * (size_t)E);
  uint8_t* taken = (uint8_t*)malloc((size_t)E);
  for (int t = 0; t < T; ++t) {
    const float* z = logits + (size_t)t * E;
    float m = z[0];
    for (int e = 1; e < E; ++e)
      if (z[e] > m) m = z[e];
    float s = 0.0f;
    for (int e = 0; e < E; ++e) {
      p[e] = expf(z[e] - m);
      s += p[e];
    }
    float inv = 1.0f / (s + 1e-9f);
    for (int e = 0; e < E; ++e) p[e] *= inv;
    if (probs) memcpy(probs + (size_t)t * E, p, sizeof(float) * (size_t)E);

    memset(taken, 0, (size_t)E);
    float sel_sum = 0.0f;
    float prev = 0.0f;
    int tie = 0;
    for (int i = 0; i < k; ++i) {
      int best = -1;
      float bv = -1.0f;
      for (int e = 0; e < E; ++e) {
        if (taken[e]) continue;
        if (p[e] > bv) { /* strict: the lowest index keeps a tie */
          bv = p[e];
          best = e;
        }
      }
      taken[best] = 1;
      idx[(size_t)t * k + i] = best;
      sel_sum += bv;
      if (i > 0 && abs(float_order(prev) - float_order(bv)) <= 4) tie = 1;
      prev = bv;
    }
    if (k < E) {
      float bv = -1.0f;
      for (int e = 0; e < E; ++e)
        if (!taken[e] && p[e] > bv) bv = p[e];
      if (abs(float_order(prev) - float_order(bv)) <= 4) tie = 1;
    }
    float denom = sel_sum + 1e-9f;
    for (int i = 0; i < k; ++i) {
      int e = idx[(size_t)t * k + i];
      gates[(size_t)t * k + i] = p[e] / denom;
      if (counts) counts[e] += 1;
    }
    if (near_tie) near_tie[t] = (uint8_t)tie;
  }
  free(p);
  free(taken);
}

/*
 * Expert-contiguous row order.  offsets[e] is the exclusive scan of the
 * per-expert counts (offsets[E] = T*k).  Within an expert rows are ordered by
 * token index and then by slot.  row_src[r] = t*k + slot for destination row r,
 * slot_dst[t*k + slot] = r.
 */
ORC_API void orc_build_permutation(const int32_t* idx, int T, int E, int k, int32_t* offsets,
                                   int32_t* row_src, int32_t* slot_dst) {
  int32_t* cnt = (int32_t*)calloc((size_t)E + 1, sizeof(int32_t));
  for (int64_t i = 0; i < (int64_t)T * k; ++i) cnt[idx[i]] += 1;
  offsets[0] = 0;
  for (int e = 0; e < E; ++e) offsets[e + 1] = offsets[e] + cnt[e];
  int32_t* cur = (int32_t*)malloc(sizeof(int32_t) * (size_t)E);
  memcpy(cur, offsets, sizeof(int32_t) * (size_t)E);
  for (int64_t i = 0; i < (int64_t)T * k; ++i) {
    int32_t r = cur[idx[i]]++;
    if (row_src) row_src[r] = (int32_t)i;
    if (slot_dst) slot_dst[i] = r;
  }
  free(cnt);
  free(cur);
}

/* Switch-style load-balancing loss: alpha * E * sum_e f_e * P_e, with
 * f_e = count_e / (T*k) and P_e = mean_t p[t,e]. */
ORC_API float orc_aux_loss(const float* probs, const int32_t* idx, int T, int E, int k,
                           float alpha) {
  double* P = (double*)calloc((size_t)E, sizeof(double));
  double* f = (double*)calloc((size_t)E, sizeof(double));
  for (int t = 0; t < T; ++t)
    for (int e = 0; e < E; ++e) P[e] += probs[(size_t)t * E + e];
  for (int64_t i = 0; i < (int64_t)T * k; ++i) f[idx[i]] += 1.0;
  double acc = 0.0;
  for (int e = 0; e < E; ++e) acc += (f[e] / ((double)T * k)) * (P[e] / T);
  free(P);
  free(f);
  return (float)(alpha * E * acc);
}

/* --------------------------------------------------------------- expert FFN */

/*
 * One expert applied to n rows.  rows[i] indexes x.  Result o[i][0..D) in fp32.
 * Accumulation for every output element is a chain of fused multiply-adds in
 * ascending reduction index.  h_bf16 != 0 rounds SiLU(g)*u to bf16 before the
 * down projection (what a two-GEMM pipeline with a bf16 intermediate does);
 * 0 keeps it in fp32.
 */
static void expert_ffn_rows(const uint16_t* x, const int32_t* rows, int n, int D, int F,
                            const uint16_t* wg, const uint16_t* wu, const uint16_t* wd,
                            int h_bf16, float* o /* [n][D] */) {
  enum { RB = 8 };
#pragma omp parallel
  {
    float* g = (float*)malloc(sizeof(float) * (size_t)RB * F);
    float* u = (float*)malloc(sizeof(float) * (size_t)RB * F);
    float* wrow = (float*)malloc(sizeof(float) * (size_t)(F > D ? F : D) * 2);
    float* wrow2 = wrow + (F > D ? F : D);
#pragma omp for schedule(dynamic, 1)
    for (int r0 = 0; r0 < n; r0 += RB) {
      int nr = n - r0 < RB ? n - r0 : RB;
      memset(g, 0, sizeof(float) * (size_t)RB * F);
      memset(u, 0, sizeof(float) * (size_t)RB * F);
      for (int d = 0; d < D; ++d) {
        const uint16_t* wgr = wg + (size_t)d * F;
        const uint16_t* wur = wu + (size_t)d * F;
        for (int f = 0; f < F; ++f) {
          wrow[f] = bf16_to_f32(wgr[f]);
          wrow2[f] = bf16_to_f32(wur[f]);
        }
        for (int r = 0; r < nr; ++r) {
          float xv = bf16_to_f32(x[(size_t)rows[r0 + r] * D + d]);
          float* gr = g + (size_t)r * F;
          float* ur = u + (size_t)r * F;
          for (int f = 0; f < F; ++f) {
            gr[f] = fmaf(xv, wrow[f], gr[f]);
            ur[f] = fmaf(xv, wrow2[f], ur[f]);
          }
        }
      }
      for (int r = 0; r < nr; ++r) {
        float* gr = g + (size_t)r * F;
        float* ur = u + (size_t)r * F;
        for (int f = 0; f < F; ++f) {
          float gv = gr[f];
          float h = (gv / (1.0f + expf(-gv))) * ur[f];
          gr[f] = h_bf16 ? round_bf16(h) : h;
        }
        memset(o + (size_t)(r0 + r) * D, 0, sizeof(float) * (size_t)D);
      }
      for (int f = 0; f < F; ++f) {
        const uint16_t* wdr = wd + (size_t)f * D;
        for (int d = 0; d < D; ++d) wrow[d] = bf16_to_f32(wdr[d]);
        for (int r = 0; r < nr; ++r) {
          float hv = g[(size_t)r * F + f];
          float* orow = o + (size_t)(r0 + r) * D;
          for (int d = 0; d < D; ++d) orow[d] = fmaf(hv, wrow[d], orow[d]);
        }
      }
    }
    free(g);
    free(u);
    free(wrow);
  }
}

/* One expert's FFN over n consecutive rows of x ([n][D] bf16): o[n][D] fp32. */
ORC_API void orc_expert_ffn(const uint16_t* x, int n, int D, int F, const uint16_t* wg,
                            const uint16_t* wu, const uint16_t* wd, int h_bf16, float* o) {
  int32_t* rows = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n > 0 ? n : 1));
  for (int i = 0; i < n; ++i) rows[i] = i;
  if (n > 0) expert_ffn_rows(x, rows, n, D, F, wg, wu, wd, h_bf16, o);
  free(rows);
}

/*
 * Whole layer from given routing.
 *   x        [T][D] bf16
 *   wg, wu   [E][D][F] bf16 ; wd [E][F][D] bf16
 *   idx      [T][k], gates [T][k]
 *   S shared experts (weights swg/swu [S][D][F], swd [S][F][D]) are applied to
 *     every token and added unweighted.
 *   h_bf16 / o_bf16: round the SwiGLU intermediate / each expert's output row to
 *     bf16 (the rounding points of a GEMM pipeline); 0/0 is the fp32-throughout
 *     convention with a single rounding of the weighted sum.
 *   y_out    [T][D] bf16: weighted expert sum (+ shared) rounded once.
 *   out      [T][D] bf16: bf16(float(x) + float(y_out)).
 *   tok_lo..tok_hi restricts the evaluation to a token range (others untouched),
 *     so that large configurations can be checked on a slice.
 */
ORC_API void orc_moe_forward(const uint16_t* x, const uint16_t* wg, const uint16_t* wu,
                             const uint16_t* wd, const int32_t* idx, const float* gates,
                             int T, int D, int E, int k, int F, int S, const uint16_t* swg,
                             const uint16_t* swu, const uint16_t* swd, int h_bf16, int o_bf16,
                             int tok_lo, int tok_hi, uint16_t* y_out, uint16_t* out) {
  if (tok_hi > T) tok_hi = T;
  if (tok_lo < 0) tok_lo = 0;
  int nt = tok_hi - tok_lo;
  if (nt <= 0) return;
  /* per-(token,slot) fp32 expert outputs, slot k.. are the shared experts */
  int slots = k + S;
  float* o_all = (float*)malloc(sizeof(float) * (size_t)nt * slots * D);
  int32_t* rows = (int32_t*)malloc(sizeof(int32_t) * (size_t)nt);
  int32_t* where = (int32_t*)malloc(sizeof(int32_t) * (size_t)nt);
  float* o_tmp = (float*)malloc(sizeof(float) * (size_t)nt * D);
  for (int e = 0; e < E + S; ++e) {
    int n = 0;
    for (int t = tok_lo; t < tok_hi; ++t) {
      if (e < E) {
        for (int i = 0; i < k; ++i)
          if (idx[(size_t)t * k + i] == e) {
            rows[n] = t;
            where[n] = (t - tok_lo) * slots + i;
            ++n;
          }
      } else {
        rows[n] = t;
        where[n] = (t - tok_lo) * slots + k + (e - E);
        ++n;
      }
    }
    if (n == 0) continue;
    const uint16_t *g_, *u_, *d_;
    if (e < E) {
      g_ = wg + (size_t)e * D * F;
      u_ = wu + (size_t)e * D * F;
      d_ = wd + (size_t)e * F * D;
    } else {
      g_ = swg + (size_t)(e - E) * D * F;
      u_ = swu + (size_t)(e - E) * D * F;
      d_ = swd + (size_t)(e - E) * F * D;
    }
    expert_ffn_rows(x, rows, n, D, F, g_, u_, d_, h_bf16, o_tmp);
    for (int i = 0; i < n; ++i)
      memcpy(o_all + (size_t)where[i] * D, o_tmp + (size_t)i * D, sizeof(float) * (size_t)D);
  }
#pragma omp parallel for schedule(static)
  for (int t = tok_lo; t < tok_hi; ++t) {
    const float* ot = o_all + (size_t)(t - tok_lo) * slots * D;
    for (int d = 0; d < D; ++d) {
      float acc = 0.0f;
      for (int i = 0; i < k; ++i) {
        float ov = ot[(size_t)i * D + d];
        if (o_bf16) ov = round_bf16(ov);
        acc = fmaf(gates[(size_t)t * k + i], ov, acc);
      }
      for (int s = 0; s < S; ++s) {
        float ov = ot[(size_t)(k + s) * D + d];
        if (o_bf16) ov = round_bf16(ov);
        acc += ov;
      }
      uint16_t yb = f32_to_bf16(acc);
      if (y_out) y_out[(size_t)t * D + d] = yb;
      if (out) out[(size_t)t * D + d] = f32_to_bf16(bf16_to_f32(x[(size_t)t * D + d]) + bf16_to_f32(yb));
    }
  }
  free(o_all);
  free(rows);
  free(where);
  free(o_tmp);
}

/* ------------------------------------------------------------------ backward */

/*
 * Gradients of  L = sum(dY * out) + aux  with  out = x + y  (residual) and
 * aux = alpha * E * sum_e f_e * P_e  (f_e treated as a constant, gradient through
 * P_e = mean_t p[t,e] only).  No reference counterpart: the engine's backward pass
 * covers the dense FFN only (core/src/CUDA/kernel/backward_pass.cu:1701-2005); the
 * SiLU*mul derivative is the one of core/src/CUDA/kernel/swiglu.cu:34-55.
 *
 *   probs [T][E]: router probabilities of the forward pass
 *   dY    [T][D] fp32 upstream gradient
 *   act_bf16 != 0 rounds the tensors a GEMM pipeline stores as bf16 (g, u, h,
 *   gate-scaled dY rows, dG, dU) at the points where it stores them.
 * Outputs (all fp32, overwritten): dX [T][D], dWg/dWu [E][D][F], dWd [E][F][D],
 * dWr [D][E], dgate [T][k], dlogits [T][E].  Any output pointer may be NULL.
 */
ORC_API void orc_moe_backward(const uint16_t* x, const void* wr, int wr_is_fp32,
                              const uint16_t* wg, const uint16_t* wu, const uint16_t* wd,
                              const int32_t* idx, const float* gates, const float* probs,
                              const float* dY, int T, int D, int E, int k, int F, float alpha,
                              int act_bf16, float* dX, float* dWg, float* dWu, float* dWd,
                              float* dWr, float* dgate, float* dlogits) {
  const size_t DF = (size_t)D * F;
  if (dX) memcpy(dX, dY, sizeof(float) * (size_t)T * D); /* residual path */
  if (dWg) memset(dWg, 0, sizeof(float) * (size_t)E * DF);
  if (dWu) memset(dWu, 0, sizeof(float) * (size_t)E * DF);
  if (dWd) memset(dWd, 0, sizeof(float) * (size_t)E * DF);
  if (dWr) memset(dWr, 0, sizeof(float) * (size_t)D * E);
  float* f_e = (float*)calloc((size_t)E, sizeof(float));
  for (int64_t i = 0; i < (int64_t)T * k; ++i) f_e[idx[i]] += 1.0f / ((float)T * k);
  float* dw_all = (float*)calloc((size_t)T * k, sizeof(float));
  float* dx_slots = (float*)calloc((size_t)T * k * D, sizeof(float)); /* summed in slot order below */

  /* experts one at a time so that the weight gradients need no atomics */
#pragma omp parallel for schedule(dynamic, 1)
  for (int e = 0; e < E; ++e) {
    const uint16_t* Wg = wg + (size_t)e * DF;
    const uint16_t* Wu = wu + (size_t)e * DF;
    const uint16_t* Wd = wd + (size_t)e * DF;
    float* g = (float*)malloc(sizeof(float) * F);
    float* u = (float*)malloc(sizeof(float) * F);
    float* h = (float*)malloc(sizeof(float) * F);
    float* dh = (float*)malloc(sizeof(float) * F);
    float* dg = (float*)malloc(sizeof(float) * F);
    float* du = (float*)malloc(sizeof(float) * F);
    float* dO = (float*)malloc(sizeof(float) * D);
    float* o = (float*)malloc(sizeof(float) * D);
    float* dx = (float*)malloc(sizeof(float) * D);
    for (int t = 0; t < T; ++t)
      for (int i = 0; i < k; ++i) {
        if (idx[(size_t)t * k + i] != e) continue;
        const uint16_t* xt = x + (size_t)t * D;
        const float w = gates[(size_t)t * k + i];
        /* forward recomputation */
        for (int f = 0; f < F; ++f) g[f] = u[f] = 0.0f;
        for (int d = 0; d < D; ++d) {
          float xv = bf16_to_f32(xt[d]);
          const uint16_t* a = Wg + (size_t)d * F;
          const uint16_t* b = Wu + (size_t)d * F;
          for (int f = 0; f < F; ++f) {
            g[f] = fmaf(xv, bf16_to_f32(a[f]), g[f]);
            u[f] = fmaf(xv, bf16_to_f32(b[f]), u[f]);
          }
        }
        for (int f = 0; f < F; ++f) {
          float hv = (g[f] / (1.0f + expf(-g[f]))) * u[f];
          if (act_bf16) {
            g[f] = round_bf16(g[f]);
            u[f] = round_bf16(u[f]);
            hv = round_bf16(hv);
          }
          h[f] = hv;
        }
        for (int d = 0; d < D; ++d) o[d] = 0.0f;
        for (int f = 0; f < F; ++f) {
          const uint16_t* c = Wd + (size_t)f * D;
          for (int d = 0; d < D; ++d) o[d] = fmaf(h[f], bf16_to_f32(c[d]), o[d]);
        }
        /* gate gradient and the gate-scaled upstream rows */
        float dw = 0.0f;
        for (int d = 0; d < D; ++d) {
          float dy = dY[(size_t)t * D + d];
          dw = fmaf(dy, o[d], dw);
          dO[d] = act_bf16 ? round_bf16(w * dy) : w * dy;
        }
        dw_all[(size_t)t * k + i] = dw;
        /* dh = dO . Wd^T ; SwiGLU derivative */
        for (int f = 0; f < F; ++f) {
          const uint16_t* c = Wd + (size_t)f * D;
          float acc = 0.0f;
          for (int d = 0; d < D; ++d) acc = fmaf(dO[d], bf16_to_f32(c[d]), acc);
          dh[f] = acc;
          float s = 1.0f / (1.0f + expf(-g[f]));
          float silu = g[f] * s;
          float dgv = acc * u[f] * (s * (1.0f + g[f] * (1.0f - s)));
          float duv = acc * silu;
          dg[f] = act_bf16 ? round_bf16(dgv) : dgv;
          du[f] = act_bf16 ? round_bf16(duv) : duv;
        }
        /* dx = dg . Wg^T + du . Wu^T */
        for (int d = 0; d < D; ++d) {
          const uint16_t* a = Wg + (size_t)d * F;
          const uint16_t* b = Wu + (size_t)d * F;
          float acc = 0.0f;
          for (int f = 0; f < F; ++f) acc = fmaf(dg[f], bf16_to_f32(a[f]), acc);
          for (int f = 0; f < F; ++f) acc = fmaf(du[f], bf16_to_f32(b[f]), acc);
          dx[d] = acc;
        }
        memcpy(dx_slots + ((size_t)t * k + i) * D, dx, sizeof(float) * (size_t)D);
        /* weight gradients */
        if (dWd)
          for (int f = 0; f < F; ++f) {
            float* r = dWd + (size_t)e * DF + (size_t)f * D;
            for (int d = 0; d < D; ++d) r[d] = fmaf(h[f], dO[d], r[d]);
          }
        if (dWg || dWu)
          for (int d = 0; d < D; ++d) {
            float xv = bf16_to_f32(xt[d]);
            if (dWg) {
              float* r = dWg + (size_t)e * DF + (size_t)d * F;
              for (int f = 0; f < F; ++f) r[f] = fmaf(xv, dg[f], r[f]);
            }
            if (dWu) {
              float* r = dWu + (size_t)e * DF + (size_t)d * F;
              for (int f = 0; f < F; ++f) r[f] = fmaf(xv, du[f], r[f]);
            }
          }
      }
    free(g); free(u); free(h); free(dh); free(dg); free(du); free(dO); free(o); free(dx);
  }
  if (dgate) memcpy(dgate, dw_all, sizeof(float) * (size_t)T * k);
  if (dX)
    for (int t = 0; t < T; ++t)
      for (int i = 0; i < k; ++i)
        for (int d = 0; d < D; ++d) dX[(size_t)t * D + d] += dx_slots[((size_t)t * k + i) * D + d];
  free(dx_slots);

  /* router: gates -> probabilities -> logits -> router weights and x */
  float* dp = (float*)malloc(sizeof(float) * E);
  float* dz = (float*)malloc(sizeof(float) * E);
  for (int t = 0; t < T; ++t) {
    const float* p = probs + (size_t)t * E;
    float sel = 0.0f, dot = 0.0f;
    for (int i = 0; i < k; ++i) sel += p[idx[(size_t)t * k + i]];
    float denom = sel + 1e-9f;
    for (int i = 0; i < k; ++i) dot += dw_all[(size_t)t * k + i] * p[idx[(size_t)t * k + i]];
    for (int e = 0; e < E; ++e) dp[e] = alpha * (float)E * f_e[e] / (float)T;
    for (int i = 0; i < k; ++i)
      dp[idx[(size_t)t * k + i]] += dw_all[(size_t)t * k + i] / denom - dot / (denom * denom);
    float pd = 0.0f;
    for (int e = 0; e < E; ++e) pd += p[e] * dp[e];
    for (int e = 0; e < E; ++e) dz[e] = p[e] * (dp[e] - pd);
    if (dlogits) memcpy(dlogits + (size_t)t * E, dz, sizeof(float) * E);
    for (int d = 0; d < D; ++d) {
      float xv = bf16_to_f32(x[(size_t)t * D + d]);
      float acc = 0.0f;
      for (int e = 0; e < E; ++e) {
        float wv = wr_is_fp32 ? ((const float*)wr)[(size_t)d * E + e]
                              : bf16_to_f32(((const uint16_t*)wr)[(size_t)d * E + e]);
        acc = fmaf(wv, dz[e], acc);
        if (dWr) dWr[(size_t)d * E + e] = fmaf(xv, dz[e], dWr[(size_t)d * E + e]);
      }
      if (dX) dX[(size_t)t * D + d] += acc;
    }
  }
  free(dp); free(dz); free(f_e); free(dw_all);
}

/* RMSNorm of each row: y = bf16(x * rstd * gamma), rstd = 1 / sqrt(mean(x^2) + eps), fp32
 * throughout, sum of squares in ascending d.  gamma may be NULL (ones).  Placement and role
 * in the block: core/src/CUDA/kernel/forward_pass.cu:404-461,1580-1598 of the engine. */
ORC_API void orc_rmsnorm(const uint16_t* x, const float* gamma, int T, int D, float eps, uint16_t* y) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t) {
    float ss = 0.0f;
    for (int d = 0; d < D; ++d) {
      float v = bf16_to_f32(x[(size_t)t * D + d]);
      ss = fmaf(v, v, ss);
    }
    float rstd = 1.0f / sqrtf(ss / (float)D + eps);
    for (int d = 0; d < D; ++d) {
      float v = bf16_to_f32(x[(size_t)t * D + d]) * rstd * (gamma ? gamma[d] : 1.0f);
      y[(size_t)t * D + d] = f32_to_bf16(v);
    }
  }
}

/* One AdamW step over a weight matrix kept as fp32 master + two fp32 moments + bf16 working
 * copy, with the conventions of the engine's fused optimiser kernel
 * (core/src/CUDA/kernel/backward_pass.cu:812-852): a non-finite gradient counts as zero,
 * gradients are clamped to [-100, 100], the step size is lr / sqrt(in_dim), each bias
 * correction 1 - beta^step is replaced by 1 when it is not above 1e-7 (and step 0 counts as
 * 1), the moments are always written, and the weight is written (clamped to [-2, 2]) only
 * when the new value is finite. */
ORC_API void orc_adamw_engine(float* master, float* m, float* v, const float* grad, uint16_t* w_bf16,
                              int64_t n, int64_t in_dim, float lr, float beta1, float beta2, float eps,
                              float weight_decay, int64_t step) {
  const float t = (float)(step > 0 ? step : 1);
  float c1 = 1.0f - powf(beta1, t), c2 = 1.0f - powf(beta2, t);
  if (!(c1 > 1e-7f)) c1 = 1.0f;
  if (!(c2 > 1e-7f)) c2 = 1.0f;
  const float step_size = lr * (1.0f / sqrtf((float)(in_dim > 0 ? in_dim : 1)));
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    float g = grad[i];
    if (!isfinite(g)) g = 0.0f;
    g = fmaxf(-100.0f, fminf(100.0f, g));
    const float mi = beta1 * m[i] + (1.0f - beta1) * g;
    const float vi = beta2 * v[i] + (1.0f - beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    const float upd = (mi / c1) / (sqrtf(vi / c2) + eps);
    const float w_new = master[i] - step_size * (upd + weight_decay * master[i]);
    if (isfinite(w_new)) {
      master[i] = fmaxf(-2.0f, fminf(2.0f, w_new));
      w_bf16[i] = f32_to_bf16(master[i]);
    }
  }
}
