/*
 * axm_moe_dropin.h — the reference engine's own MoE entry points, as exported by
 * libaxm_moe_dropin.so.  Names, argument order and meaning are those of
 * core/src/CUDA/kernel/moe_router.cuh:30-44 of PROJECT-AXIOM; the struct
 * arguments are the engine's GpuWeights / GpuActivations, passed here as opaque
 * pointers (fields are read at their Linux x86-64 byte offsets, the definitions
 * stay in the engine's core/src/CUDA/util/gpu_types.cuh:144-168,225-232).
 * An engine build that links this library instead of compiling moe_router.cu
 * keeps every caller unchanged.
 */
#ifndef AXM_MOE_DROPIN_H
#define AXM_MOE_DROPIN_H

#include <stddef.h>
#include <stdint.h>

#include "axm_moe.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Replaces forward_mixture_experts (core/src/CUDA/kernel/moe_router.cuh:30-36,
 * moe_router.cu:205-320): hidden_states [T][D] bf16 is overwritten with
 * x + MoE(x); logits, top-2 indices and gates, histogram, weighted expert sum and
 * final output are published in the activation struct (allocated on first use). */
AXM_API bool forward_mixture_experts(void* hidden_states, const void* gpu_weights,
                                     void* gpu_activations, size_t sequence_length,
                                     size_t embedding_dim, size_t feedforward_network_dimension,
                                     void* stream);

/* Replaces download_expert_counts (core/src/CUDA/kernel/moe_router.cuh:38-40,
 * moe_router.cu:322-333): synchronous copy of the histogram to host memory. */
AXM_API bool download_expert_counts(const void* gpu_activations, int32_t* h_histogram,
                                    size_t num_experts);

/* Replaces reset_expert_histogram (core/src/CUDA/kernel/moe_router.cuh:42-44,
 * moe_router.cu:335-349): zeroes the histogram on the given stream. */
AXM_API bool reset_expert_histogram(void* gpu_activations, size_t num_experts, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* AXM_MOE_DROPIN_H */
