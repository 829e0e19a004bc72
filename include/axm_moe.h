/*
 * axm_moe.h — C ABI of the B200 (sm_100a) mixture-of-experts layer.
 *
 * One layer call is   router -> permute (dispatch) -> grouped SwiGLU expert FFN
 * -> weighted combine (+ residual).  Every entry point takes plain device
 * pointers and sizes, enqueues its kernels on the caller's stream, never
 * synchronises and never allocates: scratch memory comes from the caller as one
 * workspace whose size axm_moe_workspace_bytes() reports.
 *
 * The layer replaces the MoE branch of PROJECT-AXIOM's CUDA library.  Each
 * declaration names the interface of that engine it stands in for, as
 * file:line inside the engine's source tree.  Tensor layouts are the engine's:
 *
 *   x, out            [T][D]      bf16, row-major        (core/src/CUDA/kernel/moe_router.cu:205-220)
 *   router weights    [D][E]      bf16 or fp32, E contiguous (core/src/CUDA/util/gpu_types.cuh:147-148)
 *   gate, up weights  [E][D][F]   bf16, F contiguous     (core/src/CUDA/util/gpu_types.cuh:152-155)
 *   down weights      [E][F][D]   bf16, D contiguous     (core/src/CUDA/util/gpu_types.cuh:156-157)
 *   logits            [T][E]      fp32
 *   expert indices    [T][k]      int32, slot 0 = largest probability
 *   gate weights      [T][k]      fp32
 *   histogram         [E]         int32
 *
 * All functions return AXM_OK (0) or a negative AxmStatus; axm_last_error()
 * returns a thread-local description of the last failure.  There is no CPU
 * fallback: on a machine without a usable sm_100 device every compute entry
 * point fails with AXM_ERR_DEVICE.
 */
#ifndef AXM_MOE_H
#define AXM_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define AXM_API __attribute__((visibility("default")))
#else
#define AXM_API
#endif

typedef enum AxmStatus {
  AXM_OK = 0,
  AXM_ERR_ARGUMENT = -1,  /* null pointer, zero or unsupported dimension */
  AXM_ERR_WORKSPACE = -2, /* workspace missing, misaligned or too small */
  AXM_ERR_DEVICE = -3,    /* no sm_100 device / driver entry point missing */
  AXM_ERR_LAUNCH = -4,    /* cudaGetLastError() after an enqueue */
  AXM_ERR_TIMEOUT = -5    /* a bounded device-side wait gave up (status word) */
} AxmStatus;

enum { AXM_ROUTER_BF16 = 0, AXM_ROUTER_FP32 = 1 };

enum {
  AXM_FLAG_RESIDUAL = 1,        /* out = bf16(x + y), else out = y            */
  AXM_FLAG_HIST_ACCUMULATE = 2, /* histogram[e] += counts, else histogram = counts */
  /* The reference keeps the SwiGLU intermediate h = SiLU(g) * u in fp32 between its two
   * projections (core/src/CUDA/kernel/moe_router.cu:155-190).  By default this library
   * stores h as one bf16 value, which leaves a few outputs per million just outside
   * 1e-2 + 2e-2 * |ref| where two large expert outputs cancel.  With this flag h is
   * stored as two bf16 terms (hi = bf16(h), lo = bf16(h - hi): 16 mantissa bits) and the
   * down projection multiplies both by the same weights, so every output meets that
   * bound; the down projection then does twice the tensor-core work and h takes twice
   * the room (workspace sizes follow the flag).  Inference entry points only. */
  AXM_FLAG_H_EXACT = 4
};

/* Problem shape.  D and F must be multiples of 8 (16-byte rows); E <= 256;
 * 1 <= k <= min(E, 8); S <= 8. */
typedef struct AxmMoeDesc {
  int32_t tokens;       /* T */
  int32_t d_model;      /* D */
  int32_t d_ff;         /* F */
  int32_t num_experts;  /* E, routed experts */
  int32_t top_k;        /* k */
  int32_t num_shared;   /* S, always-on experts added unweighted */
  int32_t router_dtype; /* AXM_ROUTER_BF16 | AXM_ROUTER_FP32 */
  int32_t flags;        /* AXM_FLAG_* */
} AxmMoeDesc;

/* Device pointers.  Inputs first; outputs the caller wants published may be
 * NULL, in which case the layer keeps them in its workspace. */
typedef struct AxmMoeTensors {
  const void* x;             /* [T][D] bf16 */
  const void* router_w;      /* [D][E] */
  const float* router_bias;  /* [E] fp32 added to the logits, or NULL */
  const void* w_gate;        /* [E][D][F] bf16 */
  const void* w_up;          /* [E][D][F] bf16 */
  const void* w_down;        /* [E][F][D] bf16 */
  const void* shared_gate;   /* [S][D][F] bf16 or NULL when S == 0 */
  const void* shared_up;     /* [S][D][F] */
  const void* shared_down;   /* [S][F][D] */
  float* logits;             /* [T][E] fp32, optional */
  int32_t* topk_idx;         /* [T][k], optional */
  float* topk_gate;          /* [T][k], optional */
  int32_t* histogram;        /* [E], optional */
  int32_t* offsets;          /* [E+1] exclusive scan of this call's counts, optional */
  int32_t* row_src;          /* [T*k] permuted row r came from slot t*k+i, optional */
  int32_t* slot_dst;         /* [T*k] slot t*k+i went to permuted row r, optional */
  void* y;                   /* [T][D] bf16 weighted expert sum before the residual, optional */
  void* out;                 /* [T][D] bf16, required; may alias x */
} AxmMoeTensors;

/* Thread-local text of the last error returned on this thread. */
AXM_API const char* axm_last_error(void);

/* Library / build identification: "axm_moe <version> sm_100a". */
AXM_API const char* axm_version(void);

/* Number of kernels one axm_moe_forward() call enqueues for this shape. */
AXM_API int axm_moe_forward_launches(const AxmMoeDesc* desc);

/* Bytes of scratch axm_moe_forward() needs for this shape (256-byte aligned
 * base required).  Replaces the lazily allocated activation buffers of
 * core/src/CUDA/kernel/moe_router.cu:222-261. */
AXM_API int axm_moe_workspace_bytes(const AxmMoeDesc* desc, size_t* bytes);

/* The whole layer.  Replaces forward_mixture_experts
 * (core/src/CUDA/kernel/moe_router.cuh:30-36, moe_router.cu:205-320). */
AXM_API int axm_moe_forward(const AxmMoeDesc* desc, const AxmMoeTensors* tensors,
                            void* workspace, size_t workspace_bytes, void* stream);

/* The layer at its call site in a pre-norm transformer block:
 *   out = x + MoE(RMSNorm(x)),  RMSNorm(x) = bf16(x * rsqrt(mean(x^2) + eps) * gamma).
 * The engine normalises before its MoE branch (core/src/CUDA/kernel/forward_pass.cu:1580-1598,
 * RMSNorm at forward_pass.cu:404-461) but then adds the NORMALISED activations as the
 * residual and leaves the block's hidden state untouched; this entry point wires the
 * residual to the block input, which is what a pre-norm block means.  gamma is fp32 [D]
 * or NULL (ones).  x_norm is a caller buffer of T*D bf16 that receives RMSNorm(x), or NULL:
 * then the normalisation is folded into the reads of the router and of the permute kernel
 * (one statistics pass stores 1/rms per token, nothing normalised is written to memory; same
 * bits as the two-kernel form).  The folded form needs num_shared == 0 and a shape the
 * tensor-core router serves (AXM_ERR_ARGUMENT otherwise).  eps > 0. */
AXM_API int axm_moe_forward_prenorm(const AxmMoeDesc* desc, const AxmMoeTensors* tensors,
                                    const float* gamma, float eps, void* x_norm, void* workspace,
                                    size_t workspace_bytes, void* stream);

/* RMSNorm alone (the first kernel of axm_moe_forward_prenorm). */
AXM_API int axm_moe_rmsnorm(const void* x, const float* gamma, void* y, int32_t tokens,
                            int32_t d_model, float eps, void* stream);

/* axm_moe_forward with CUDA events between its five kernels; synchronises the
 * stream and returns the device time of each stage in milliseconds:
 * stage_ms[0..4] = router, permute, gate/up GEMM, down GEMM, combine.  A
 * measuring aid with no reference counterpart. */
AXM_API int axm_moe_forward_profiled(const AxmMoeDesc* desc, const AxmMoeTensors* tensors,
                                     void* workspace, size_t workspace_bytes, void* stream,
                                     float* stage_ms);

/* The same call for a caller whose activations live in host memory: copies x
 * from (pinned) host memory, runs the layer, copies out back, all on `stream`,
 * and synchronises the stream before returning.  Weights stay device pointers.
 * Mirrors the host wrapper AI::forward_mixture_experts (core/src/ai.cpp:593-623).
 * d_x / d_out are device staging buffers of T*D bf16 each.  From 1024 tokens on, if
 * d_x != d_out and offsets / row_src / slot_dst are not requested, the batch is cut
 * into chunks whose copies in, compute and copies out overlap (results per token are
 * the same; the histogram still covers the whole batch). */
AXM_API int axm_moe_forward_host(const AxmMoeDesc* desc, const AxmMoeTensors* tensors,
                                 const void* h_x, void* h_out, void* d_x, void* d_out,
                                 void* workspace, size_t workspace_bytes, void* stream);

/* A run of n_batches (<= 64) batches from pinned host memory, double-buffered on the device:
 * batch i + 1 is copied in while batch i is computed and batch i - 1 is copied out, so in
 * steady state a batch costs the longer of its compute and its copies.  Every batch is one
 * axm_moe_forward over desc->tokens tokens (same bytes out).  h_x[i] / h_out[i]: [T][D] bf16
 * host buffers; d_x2, d_out2: device buffers of two batches each; workspace: the layer's
 * workspace plus 256 bytes.  Per-token outputs in `tensors` must be NULL (histogram is allowed
 * and follows AXM_FLAG_HIST_ACCUMULATE).  Synchronises before returning.  The reference's call
 * site copies nothing (device-resident activations, core/src/CUDA/kernel/forward_pass.cu:1585-1598);
 * this is for hosts that feed the layer from host memory. */
AXM_API int axm_moe_forward_host_batches(const AxmMoeDesc* desc, const AxmMoeTensors* tensors,
                                         const void* const* h_x, void* const* h_out, int32_t n_batches,
                                         void* d_x2, void* d_out2, void* workspace,
                                         size_t workspace_bytes, void* stream);

/* Device address of the int32 status word inside a workspace.  The GEMM kernels
 * store a non-zero code there when one of their bounded waits gives up; a
 * caller that synchronises can read it back.  No reference counterpart (the
 * engine reports enqueue-time errors only, core/src/CUDA/kernel/moe_router.cu:319). */
AXM_API int axm_moe_status_word(const AxmMoeDesc* desc, void* workspace, int32_t** status);

/* ---- stages, callable on their own (tests, expert-parallel drivers) ---- */

/* Fused router: logits (+bias), softmax, top-k, gates, per-block counts.
 * Replaces top2_router_kernel (core/src/CUDA/kernel/moe_router.cu:27-111).
 * block_counts: [AXM_ROUTE_BLOCKS][E] int32 scratch consumed by axm_moe_permute. */
AXM_API int axm_moe_router(const AxmMoeDesc* desc, const void* x, const void* router_w,
                           const float* router_bias, float* logits, int32_t* topk_idx,
                           float* topk_gate, int32_t* block_counts, void* stream);

/* The same router with scratch memory for its tensor-core form: the logits are computed as
 * a tcgen05 product streamed through TMA (x is read from HBM once, at bandwidth), which needs
 * the router weights split into bf16 terms and transposed - `scratch`, of
 * axm_moe_router_scratch_bytes() bytes (16-byte aligned), written by a small preparation
 * kernel at every call.  0 bytes means the shape is not served by that kernel (more than 80
 * experts with fp32 weights); then, and when scratch is NULL or too small, the call runs
 * axm_moe_router.  `status` (optional int32 device word): cleared at the start of the call on
 * the tensor-core path, then set to a non-zero code if a bounded wait gave up. */
AXM_API int axm_moe_router_scratch_bytes(const AxmMoeDesc* desc, size_t* bytes);
AXM_API int axm_moe_router_ws(const AxmMoeDesc* desc, const void* x, const void* router_w,
                              const float* router_bias, float* logits, int32_t* topk_idx,
                              float* topk_gate, int32_t* block_counts, void* scratch,
                              size_t scratch_bytes, int32_t* status, void* stream);

/* Routing from caller-supplied fp32 logits: the part of the router whose
 * results must equal the reference bit for bit
 * (core/src/CUDA/kernel/moe_router.cu:59-110). */
AXM_API int axm_moe_route_from_logits(const AxmMoeDesc* desc, const float* logits,
                                      int32_t* topk_idx, float* topk_gate,
                                      int32_t* block_counts, void* stream);

/* Histogram, exclusive-scan offsets, stable expert-contiguous placement and the
 * 16-byte row copies.  No counterpart kernel in the reference (its dispatch is
 * per token, core/src/CUDA/kernel/moe_router.cu:113-191); the histogram follows
 * moe_router.cu:107-110.  x_perm: [T*k][D] bf16 or NULL to skip the row copies. */
AXM_API int axm_moe_permute(const AxmMoeDesc* desc, const void* x, const int32_t* topk_idx,
                            const int32_t* block_counts, int32_t* histogram, int32_t* offsets,
                            int32_t* row_src, int32_t* slot_dst, void* x_perm, void* stream);

struct AxmSegment;
/* axm_moe_permute in the training layout: every expert's rows start at a multiple
 * of row_align (64 for the backward kernels); the rows between an expert's last
 * row and the next expert's first are zero in x_perm and have row_src = -1.
 * offsets[e] is the padded start, offsets[E] the padded total (<= T*k +
 * (row_align - 1) * E); the histogram still holds the true counts.  `segments`
 * ([E], optional) receives one segment per expert with the padded row count. */
AXM_API int axm_moe_permute_padded(const AxmMoeDesc* desc, const void* x, const int32_t* topk_idx,
                                   const int32_t* block_counts, int32_t* histogram,
                                   int32_t* offsets, int32_t* row_src, int32_t* slot_dst,
                                   void* x_perm, struct AxmSegment* segments, int32_t row_align,
                                   void* stream);

/* One segment of rows that share an expert, for the grouped GEMMs.  Expert ids
 * >= E address the shared experts. */
typedef struct AxmSegment {
  int32_t a_row0;   /* first row in the A operand */
  int32_t out_row0; /* first row in the output */
  int32_t rows;
  int32_t expert;   /* bit 30 set: A rows come from the alternate A tensor */
} AxmSegment;
#define AXM_SEG_ALT_A (1 << 30)

/* Builds the segment table of a single-GPU layer call on the device from the
 * offsets array: one segment per routed expert, then one per shared expert. */
AXM_API int axm_moe_build_segments(const AxmMoeDesc* desc, const int32_t* offsets,
                                   AxmSegment* segments, void* stream);

/* Grouped SwiGLU expert FFN over `num_segments` segments read from device memory:
 *   h   = SiLU(A . Wg[e]) * (A . Wu[e])     -> bf16 [rows_total][F]
 *                                             ([rows_total][2F], hi | lo, with AXM_FLAG_H_EXACT)
 *   o   = h . Wd[e]                         -> fp32 [rows_total][D]
 * tcgen05 tensor-core kernels, bf16 in, fp32 accumulate in tensor memory.
 * Replaces moe_top2_dispatch_kernel phases A and B
 * (core/src/CUDA/kernel/moe_router.cu:155-190).
 * a_rows / alt_rows are the row counts of x_perm and x_alt (tensor-map extents);
 * rows_total is the row count of h and o. status is an int32 device word that
 * receives a non-zero code if a bounded wait inside a kernel gave up. */
AXM_API int axm_moe_expert_ffn(const AxmMoeDesc* desc, const void* x_perm, int32_t a_rows,
                               const void* x_alt, int32_t alt_rows, const AxmSegment* segments,
                               int32_t num_segments, const void* w_gate, const void* w_up,
                               const void* w_down, const void* shared_gate,
                               const void* shared_up, const void* shared_down, void* h,
                               void* o, int32_t rows_total, int32_t* status, void* stream);

/* Backward of the grouped expert FFN over a segment table whose segments are padded
 * to multiples of 64 rows with zero rows (training layout; a_row0 == out_row0):
 *   dH  = d_o . Wd[e]^T ; dG = dH * u * silu'(g), dU = dH * silu(g)   -> d_g, d_u bf16 [rows][F]
 *   dXp = dG . Wg[e]^T + dU . Wu[e]^T                                  -> d_xp fp32 [rows][D]
 *   dWd[e] = h^T d_o, dWg[e] = x_perm^T dG, dWu[e] = x_perm^T dU       -> fp32, weight layouts
 * d_o is the gate-scaled upstream gradient per permuted row (bf16 [rows][D]); g, u, h
 * are what the forward pass saved.  The three weight gradients may all be NULL.
 * tcgen05 kernels.  No reference counterpart (the engine's backward covers the dense
 * FFN only, core/src/CUDA/kernel/backward_pass.cu:1701-2005); gradients follow its
 * conventions: fp32, same [in][out] layout as the weights (backward_pass.cu:1013-1048),
 * SiLU*mul derivative of core/src/CUDA/kernel/swiglu.cu:34-55. */
AXM_API int axm_moe_expert_ffn_backward(const AxmMoeDesc* desc, const AxmSegment* segments,
                                        int32_t num_segments, int32_t rows_total,
                                        const void* x_perm, const void* h, const void* g,
                                        const void* u, const void* d_o, const void* w_gate,
                                        const void* w_up, const void* w_down, void* d_g, void* d_u,
                                        void* d_xp, void* d_w_gate, void* d_w_up, void* d_w_down,
                                        int32_t* status, void* stream);

/* ---- training step -------------------------------------------------------------
 * No reference counterpart: the engine's MoE branch is forward only, its backward
 * pass covers the dense FFN (core/src/CUDA/kernel/backward_pass.cu:1701-2005) and a
 * load-balancing loss is future work there (document/AI_CONTEXT.md:217).
 *   L = sum(d_out * out) + aux,  out = x + MoE(x),
 *   aux = aux_alpha * E * sum_e f_e * P_e  (f_e = share of the T*k selections that
 *   went to expert e, a constant; P_e = mean over tokens of the router probability).
 * axm_moe_forward_train runs the forward pass, keeps the activations the backward
 * needs in the workspace (training layout: experts padded to 64 rows) and writes
 * the auxiliary loss; axm_moe_backward must follow with the same desc, tensors and
 * workspace.  Gradients are fp32 in the layouts of what they belong to; they are
 * overwritten, not accumulated.  Shared experts are not supported here. */
typedef struct AxmMoeTrain {
  const void* x;            /* [T][D] bf16 */
  const void* router_w;     /* [D][E] bf16 or fp32 */
  const float* router_bias; /* [E] or NULL */
  const void* w_gate;       /* [E][D][F] bf16 */
  const void* w_up;         /* [E][D][F] bf16 */
  const void* w_down;       /* [E][F][D] bf16 */
  void* out;                /* [T][D] bf16 (forward) */
  float* aux_loss;          /* device scalar, optional (forward) */
  int32_t* histogram;       /* [E] this call's counts, optional (forward) */
  float aux_alpha;
  const float* d_out;       /* [T][D] fp32 upstream gradient (backward) */
  float* d_x;               /* [T][D] fp32 */
  float* d_router_w;        /* [D][E] fp32, optional */
  float* d_w_gate;          /* [E][D][F] fp32; the three expert gradients together or none */
  float* d_w_up;            /* [E][D][F] fp32 */
  float* d_w_down;          /* [E][F][D] fp32 */
  float* d_router_bias;     /* [E] fp32 gradient of router_bias (sum over tokens of the logit
                             * gradients), optional; NULL leaves the bias untrained */
  const void* shared_gate;  /* [S][D][F] bf16: shared experts (desc->num_shared > 0), applied to every
                             * token with weight 1 as in the forward call */
  const void* shared_up;    /* [S][D][F] bf16 */
  const void* shared_down;  /* [S][F][D] bf16 */
  float* d_shared_gate;     /* [S][D][F] fp32: given exactly when the routed experts' gradients are */
  float* d_shared_up;       /* [S][D][F] fp32 */
  float* d_shared_down;     /* [S][F][D] fp32 */
} AxmMoeTrain;

AXM_API int axm_moe_train_workspace_bytes(const AxmMoeDesc* desc, size_t* bytes);
AXM_API int axm_moe_forward_train(const AxmMoeDesc* desc, const AxmMoeTrain* tensors,
                                  void* workspace, size_t workspace_bytes, void* stream);
AXM_API int axm_moe_backward(const AxmMoeDesc* desc, const AxmMoeTrain* tensors, void* workspace,
                             size_t workspace_bytes, void* stream);

/* AdamW step (decoupled weight decay, bias correction with `step` >= 1) over one MoE
 * weight matrix as the engine stores it: fp32 master, two fp32 moments, bf16 working
 * copy (core/src/CUDA/util/gpu_types.cuh:148-168); `grad` is what axm_moe_backward
 * wrote.  Follows the textbook update (axm_moe_adamw_step_engine below follows the
 * engine's own fused AdamW, core/src/CUDA/kernel/backward_pass.cu:812-852).  n elements,
 * fp32 buffers 16-byte aligned, the bf16 copy 8-byte aligned (else AXM_ERR_ARGUMENT). */
AXM_API int axm_moe_adamw_step(float* master, float* m, float* v, const float* grad, void* w_bf16,
                               int64_t n, float lr, float beta1, float beta2, float eps,
                               float weight_decay, int32_t step, void* stream);

/* The same step with the conventions of the engine's own fused AdamW kernel
 * (core/src/CUDA/kernel/backward_pass.cu:812-852), so that weights of an engine
 * checkpoint move exactly as the engine's optimiser would move them:
 *   a non-finite gradient counts as 0 and gradients are clamped to [-100, 100];
 *   the step size is lr / sqrt(in_dim), in_dim = the matrix's input dimension
 *   (D for router, gate and up weights, F for down weights);
 *   a bias-correction term 1 - beta^step that is <= 1e-7 is replaced by 1 (step 0 counts as 1);
 *   the new weight is clamped to [-2, 2]; if it is not finite the weight is left unchanged
 *   (the moments are still updated).
 * Also requires the bf16 copy to be 8-byte aligned, like axm_moe_adamw_step. */
AXM_API int axm_moe_adamw_step_engine(float* master, float* m, float* v, const float* grad,
                                      void* w_bf16, int64_t n, int64_t in_dim, float lr, float beta1,
                                      float beta2, float eps, float weight_decay, int64_t step,
                                      void* stream);

/* ---- MoE block of the engine's checkpoint file ----------------------------------
 * The engine's `weights.axiom` (56-byte packed header "AXIOM_V1", fp32 weights, bias,
 * embeddings, optional transformer block tagged "TXFM"; core/include/config.hpp:41-55,92,
 * writer core/src/training.cpp:283-392, loader core/src/ai.cpp:273-491) holds no router
 * or expert tensors, so a model with MoE layers cannot be saved or resumed.  These
 * entry points keep the MoE weights in a tagged block appended AFTER the transformer
 * block; the stock loader stops reading after the transformer block, so a file with
 * the MoE block still loads there.  All of it is host code: no GPU is needed.
 *
 * Block layout (little-endian, packed):
 *   u64 magic = 0x4D4F4558 ("MOEX", written like the engine's 0x5458464D "TXFM" tag)
 *   u64 version = 1
 *   u64 d_model, d_ff, num_experts, top_k, num_shared
 *   u64 flags            bit 0: router bias present
 *   u64 payload_bytes    bytes of the tensors that follow
 *   fp32 router_w [D][E]; router_bias [E] (if flagged); w_gate [E][D][F]; w_up [E][D][F];
 *        w_down [E][F][D]; shared_gate, shared_up [S][D][F]; shared_down [S][F][D] (if S > 0)
 *   u64 checksum         sum of the payload's 32-bit words, modulo 2^64
 * fp32 because the engine checkpoints its fp32 master copies; the bf16 working copy
 * is rebuilt with axm_moe_cast_master.
 *
 * save: `path` must be an existing checkpoint WITH a transformer block (the stock
 *   loader rejects any other tag at that position).  An MoE block already present is
 *   replaced.  Like the engine's writer: refuses non-finite values, writes
 *   `path`.tmp, then renames over `path`; on any failure the .tmp is removed and
 *   `path` is untouched.
 * probe: fills desc->{d_model, d_ff, num_experts, top_k, num_shared} and *has_bias
 *   from the block; AXM_ERR_ARGUMENT if the file has none or is damaged.
 * load: `desc` must match the block; fills the host buffers; verifies sizes, the
 *   checksum and that every value is finite before anything is returned as valid. */
typedef struct AxmMoeCheckpoint {
  float* router_w;    /* HOST fp32, layouts as in AxmMoeTensors */
  float* router_bias; /* [E] or NULL */
  float* w_gate;
  float* w_up;
  float* w_down;
  float* shared_gate; /* NULL when num_shared == 0 */
  float* shared_up;
  float* shared_down;
} AxmMoeCheckpoint;

AXM_API int axm_moe_checkpoint_save(const char* path, const AxmMoeDesc* desc,
                                    const AxmMoeCheckpoint* tensors);
AXM_API int axm_moe_checkpoint_probe(const char* path, AxmMoeDesc* desc, int32_t* has_bias);
AXM_API int axm_moe_checkpoint_load(const char* path, const AxmMoeDesc* desc,
                                    const AxmMoeCheckpoint* tensors);

/* bf16 working copy of an fp32 master matrix (both on the device), n elements,
 * round-to-nearest-even: what the kernels read after a checkpoint was loaded. */
AXM_API int axm_moe_cast_master(const float* master, void* w_bf16, size_t n, void* stream);


/* Per-segment redirect of the down projection's output: rows of segment s are
 * stored at base + (row0 + i) * D floats instead of into `o` (base == NULL keeps
 * the segment in `o`).  Under expert parallelism base is the source rank's return
 * buffer in peer memory, so the expert outputs leave the GPU from the GEMM
 * epilogue itself (plain stores over NVLink) and no separate return copy runs. */
typedef struct AxmRemoteOut {
  void* base;
  int32_t row0;
  int32_t reserved;
} AxmRemoteOut;

/* axm_moe_expert_ffn with the redirect table remote_out[num_segments] (device
 * memory).  No reference counterpart. */
AXM_API int axm_moe_expert_ffn_remote(const AxmMoeDesc* desc, const void* x_perm, int32_t a_rows,
                                      const void* x_alt, int32_t alt_rows,
                                      const AxmSegment* segments, int32_t num_segments,
                                      const void* w_gate, const void* w_up, const void* w_down,
                                      const void* shared_gate, const void* shared_up,
                                      const void* shared_down, void* h, void* o,
                                      int32_t rows_total, const AxmRemoteOut* remote_out,
                                      int32_t* status, void* stream);

/* Weighted combine over fp32 expert rows:
 * y[t] = bf16(sum_i gate[t,i] * o[slot_dst[t,i]] + sum_s o_shared[s][t]),
 * out[t] = bf16(x[t] + y[t]) with AXM_FLAG_RESIDUAL.  Replaces the gate-weighted
 * sum and the residual add (core/src/CUDA/kernel/moe_router.cu:186-203,304-317).
 * o is fp32 [T*k][D]; o_shared points at the first shared expert's fp32 rows
 * ([S][T][D]) or NULL. */
AXM_API int axm_moe_combine(const AxmMoeDesc* desc, const void* x, const void* o,
                            const void* o_shared, const int32_t* slot_dst,
                            const float* topk_gate, void* y, void* out, void* stream);

/* ---- expert-parallel exchange over NVLink peer memory ------------------------
 * No reference counterpart: the engine is single-GPU (no NCCL/MPI in core/src).
 * Every rank allocates one exchange region of identical layout in memory its
 * peers can address (peer access / symmetric memory; the allocation is the
 * host's) and passes the table of all regions' base addresses.  The kernels reach
 * peers with plain 16-byte stores and bounded flag waits; see csrc/ep_exchange.cu.
 * `step` must grow by one per layer call, starting at 1, on every rank alike.
 * The region must be zero-filled once before the first call (flags).
 * `scratch` is 2 zero-initialised int32 in local memory, private to the layer. */
typedef struct AxmEpLayout {
  const void* const* peers; /* DEVICE array [world]: base address of every rank's region */
  int32_t rank, world;
  int32_t num_experts;      /* E over all ranks; E / world experts per rank */
  int32_t d_model;
  int32_t slots;            /* T_local * k: rows this rank sends and gets back */
  int32_t cap;              /* rows the receive buffer holds (slots * world covers every case) */
  int32_t num_shared;       /* shared experts, run on the local tokens */
  int32_t tokens_local;
  int64_t off_flags, off_counts, off_recv, off_oback; /* byte offsets inside a region */
  void* local_region;       /* this rank's own region (= peers[rank]), readable by the host code of
                             * axm_moe_ep_forward; the stage entry points below do not use it */
  int32_t row_align;        /* 0 or 1: rows packed.  64: training layout - every local expert's run in the
                             * receive buffer starts at a multiple of 64 rows and is followed by zero rows
                             * up to the next multiple; cap must then hold slots * world + 63 * (E / world) */
  int32_t return_rows;      /* rows every rank's return buffer holds when `slots` carries one call's (smaller)
                             * row count; 0: the same as slots.  Ranks may hold different numbers of tokens in
                             * a call, so a rank bounds its stores into a peer's return buffer by this. */
} AxmEpLayout;

/* Fills the offsets / sizes of `layout` and returns the bytes one region needs:
 * flags [3][world] u32, counts [world][E] i32, receive buffer [cap][D] bf16,
 * return buffer [slots][D] fp32. */
AXM_API int axm_ep_region_bytes(int32_t world, int32_t num_experts, int32_t d_model,
                                int32_t slots, int32_t cap, AxmEpLayout* layout, size_t* bytes);

/* Dispatch: posts this rank's per-expert counts (from `offsets`, [E+1]) to all
 * peers, waits for theirs, copies the permuted rows (x_perm [slots][D] bf16) into
 * the owners' receive buffers and flags them.  A receive buffer is expert-major:
 * the rows of the owner's first expert from source 0, 1, ..., then its second
 * expert's, so one expert's rows are one contiguous run. */
AXM_API int axm_ep_dispatch(const AxmEpLayout* layout, uint32_t step, const int32_t* offsets,
                            const void* x_perm, int32_t* scratch, int32_t* status, void* stream);

/* Waits for every source's rows, then writes two tables over the receive buffer
 * (world * E/world entries each, entry j * world + s for local expert j and source
 * rank s, which is ascending row order): `segments` for axm_moe_expert_ffn,
 * followed by num_shared segments over the local tokens with output rows from
 * `cap` on; and `ret_segments` for axm_ep_return ({a_row0 = row in the source's
 * return buffer, out_row0 = row here, rows, expert = source rank}).
 * With remote_out == NULL the rows of one expert form ONE segment (entry j * world;
 * the expert's other entries hold zero rows), so the GEMMs cut their m-tiles as on
 * a single GPU.  If remote_out is not NULL every source keeps its own segment and
 * remote_out receives, in the order of `segments`, the redirect table that makes
 * axm_moe_expert_ffn_remote store each segment straight into its source's return
 * buffer.  Also the number of rows received. */
AXM_API int axm_ep_segments(const AxmEpLayout* layout, uint32_t step, AxmSegment* segments,
                            AxmSegment* ret_segments, AxmRemoteOut* remote_out,
                            int32_t* rows_received, int32_t* status, void* stream);

/* Return: copies the fp32 expert rows `o` back into each source rank's return
 * buffer at the rows its own permutation expects, and flags the sources. */
AXM_API int axm_ep_return(const AxmEpLayout* layout, uint32_t step,
                          const AxmSegment* ret_segments, const void* o, int32_t* scratch,
                          int32_t* status, void* stream);

/* Fused return: after axm_moe_expert_ffn_remote has stored the rows itself, flags
 * every source (replaces axm_ep_return). */
AXM_API int axm_ep_signal_return(const AxmEpLayout* layout, uint32_t step, void* stream);

/* Waits until every owner has returned this rank's rows (run before axm_moe_combine
 * on the return buffer). */
AXM_API int axm_ep_wait_return(const AxmEpLayout* layout, uint32_t step, int32_t* status,
                               void* stream);

/* ---- the expert-parallel layer as one call ------------------------------------------
 * axm_moe_ep_forward runs, for this rank's tokens (desc->tokens = T_local; desc->num_experts
 * = E over all ranks), router -> permute fused with the dispatch (rows are stored straight
 * into the owners' receive buffers) -> segment tables -> gate/up GEMM -> down GEMM -> return
 * of the expert rows -> wait for the returned rows -> combine.  Everything is enqueued on
 * `stream`; no host synchronisation.  (With AXM_EP_SPLIT_RETURN=1 in the environment the down
 * GEMM runs in two halves and the first half's rows return on an internal side stream while
 * the second half is computed; measured slower on 8 GPUs, so it is off by default.)  `layout` as for the stage calls, with local_region set;
 * layout->slots and cap are what the regions were SIZED for, the call may carry fewer tokens.
 * `step` starts at 1 and grows by one per call on every rank alike.
 * The workspace is private to the rank; its first *zero_bytes bytes must be zero before the
 * first call (counters) and are left zero by every call.  The status word (first int32 of
 * the workspace, axm_moe_ep_status_word) is sticky: a bounded wait that gave up stores a
 * non-zero code and nothing clears it but the caller.
 * No reference counterpart: the engine is single-GPU. */
typedef struct AxmEpTensors {
  const void* x;            /* [T_local][D] bf16 */
  const void* router_w;     /* [D][E], replicated */
  const float* router_bias; /* [E] or NULL */
  const void* w_gate;       /* [E / world][D][F]: this rank's experts */
  const void* w_up;
  const void* w_down;       /* [E / world][F][D] */
  const void* shared_gate;  /* [S][D][F] replicated, or NULL */
  const void* shared_up;
  const void* shared_down;
  float* logits;            /* [T_local][E], optional */
  int32_t* topk_idx;        /* [T_local][k], optional */
  float* topk_gate;         /* [T_local][k], optional */
  int32_t* histogram;       /* [E]: this rank's tokens per expert, optional */
  void* y;                  /* [T_local][D] bf16, optional */
  void* out;                /* [T_local][D] bf16 */
} AxmEpTensors;

AXM_API int axm_moe_ep_workspace_bytes(const AxmEpLayout* layout, const AxmMoeDesc* desc, size_t* bytes,
                                       size_t* zero_bytes);
AXM_API int axm_moe_ep_forward(const AxmEpLayout* layout, const AxmMoeDesc* desc,
                               const AxmEpTensors* tensors, void* workspace, size_t workspace_bytes,
                               uint32_t step, void* stream);
/* ---- training step of the expert-parallel layer -------------------------------------------
 * The sharded form of axm_moe_forward_train / axm_moe_backward; no reference counterpart (the
 * engine is single-GPU and its backward covers the dense FFN only,
 * core/src/CUDA/kernel/backward_pass.cu:1701-2005).  AxmMoeTrain is read per rank: x, out,
 * d_out, d_x cover this rank's desc->tokens tokens; w_gate / w_up / w_down and their gradients
 * cover this rank's E / world experts; router_w, router_bias and the shared experts are
 * replicated (shared experts are applied to the rank's own tokens without communication).
 * Two exchange regions of equal size are needed, both with row_align = 64 and
 * cap >= slots * world + 63 * (E / world): `layout` carries the forward rows and keeps them
 * until the backward pass has read them, `bwd_layout` carries the gradient rows.  The same
 * `step` is passed to the forward and the backward call of one training step; it grows by one
 * per training step on every rank alike.  tokens_global is the token count over all ranks.
 * Left to the caller (sums over the ranks of replicated quantities): d_router_w, d_router_bias,
 * d_shared_gate / d_shared_up / d_shared_down and aux_loss hold this rank's share.  Routed
 * experts' weight gradients are complete on their rank.
 * The workspace holds the saved activations between the two calls; its leading zero_bytes must
 * be zero before the first call. */
AXM_API int axm_moe_ep_train_workspace_bytes(const AxmEpLayout* layout, const AxmMoeDesc* desc, size_t* bytes,
                                             size_t* zero_bytes);
AXM_API int axm_moe_ep_forward_train(const AxmEpLayout* layout, const AxmMoeDesc* desc,
                                     const AxmMoeTrain* tensors, int32_t tokens_global, void* workspace,
                                     size_t workspace_bytes, uint32_t step, void* stream);
AXM_API int axm_moe_ep_backward(const AxmEpLayout* layout, const AxmEpLayout* bwd_layout,
                                const AxmMoeDesc* desc, const AxmMoeTrain* tensors, int32_t tokens_global,
                                void* workspace, size_t workspace_bytes, uint32_t step, void* stream);
AXM_API int axm_moe_ep_train_status_word(const AxmEpLayout* layout, const AxmMoeDesc* desc, void* workspace,
                                         int32_t** status, int32_t** rows_received);

/* Device addresses of the sticky status word and of the number of rows this rank received
 * in the last call (either pointer may be NULL). */
AXM_API int axm_moe_ep_status_word(const AxmEpLayout* layout, const AxmMoeDesc* desc, void* workspace,
                                   int32_t** status, int32_t** rows_received);
/* axm_moe_ep_forward with CUDA events between its phases; synchronises the stream and returns
 * device times in milliseconds: router, permute + dispatch, wait for rows + segment
 * tables, gate/up GEMM, down GEMM, return copy (of the second half when the return is
 * split), wait for returned rows + combine; stage_ms[7] and [8] are the
 * start and the end of the first half's return copy (side stream), counted from the start
 * of the down GEMM (both 0 when the return is not split).  stage_ms holds 9 floats.  A
 * measuring aid. */
AXM_API int axm_moe_ep_forward_profiled(const AxmEpLayout* layout, const AxmMoeDesc* desc,
                                        const AxmEpTensors* tensors, void* workspace,
                                        size_t workspace_bytes, uint32_t step, void* stream,
                                        float* stage_ms);
/* The same layer for activations in (pinned) host memory, mirroring the engine's host wrapper
 * (core/src/ai.cpp:593-623): the rank's tokens are cut into `chunks` equal parts (1..8, the
 * same on every rank; each part is one exchange step), part c + 1 is copied in and part c - 1
 * copied out while part c is computed.  chunks = 0 lets the library choose (two parts from 4096
 * tokens per rank on, else one; every rank must then arrive at the same number).  d_x / d_out:
 * device staging buffers of T_local * D bf16.  *step is the first step number to use and is
 * advanced by the number of parts.  Synchronises. */
AXM_API int axm_moe_ep_forward_host(const AxmEpLayout* layout, const AxmMoeDesc* desc,
                                    const AxmEpTensors* tensors, const void* h_x, void* h_out, void* d_x,
                                    void* d_out, void* workspace, size_t workspace_bytes, int32_t chunks,
                                    uint32_t* step, void* stream);

/* Number of token blocks the router splits T into (rows of block_counts). */
#define AXM_ROUTE_BLOCKS 296

/* Routing from fp32 logits followed by the dispatch (axm_moe_route_from_logits +
 * axm_moe_permute in one call) for callers that may not allocate device memory
 * and have no scratch buffer to lend: servers that give all of HBM to their own
 * arena at start-up, plug-ins living in someone else's process, code on a path
 * where cudaMalloc's implicit synchronisation is not acceptable.  The block-count
 * scratch is a fixed array inside the library (AXM_NOALLOC_SCRATCH_BYTES of device
 * memory on every GPU that loads the library, held until the process exits), so
 * the call allocates nothing and asks the caller only for inputs and outputs
 * (same meaning as in the two calls it replaces; histogram, offsets, row_src,
 * slot_dst and x_perm may be NULL, x is needed only with x_perm).
 * Limits: num_experts <= AXM_NOALLOC_MAX_EXPERTS, else AXM_ERR_ARGUMENT and
 * nothing is launched.  All calls on a GPU share the array: every call rewrites
 * the whole part it later reads, so no stale contents are ever used, but calls
 * whose kernels overlap on the GPU race - serialise them (one stream, or events).
 * The first call on each device resolves the array's address and may initialise
 * the CUDA context; make it before any stream capture begins.
 * This entry point has no counterpart in the reference engine. */
#define AXM_NOALLOC_MAX_EXPERTS 128
#define AXM_NOALLOC_SCRATCH_BYTES (4 * AXM_ROUTE_BLOCKS * AXM_NOALLOC_MAX_EXPERTS)
AXM_API int axm_moe_route_dispatch_noalloc(const AxmMoeDesc* desc, const float* logits,
                                           const void* x, int32_t* topk_idx, float* topk_gate,
                                           int32_t* histogram, int32_t* offsets,
                                           int32_t* row_src, int32_t* slot_dst, void* x_perm,
                                           void* stream);

#ifdef __cplusplus
}
#endif
#endif /* AXM_MOE_H */
