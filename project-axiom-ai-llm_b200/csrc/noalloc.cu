// Routing + dispatch for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at all: an inference server
// that hands every byte of HBM to its own arena at start-up and forbids later
// driver allocations, a plug-in loaded into a process whose memory is owned by
// someone else, or code that runs where an allocation would stall the whole
// device (it synchronises).  The regular entry points already take their scratch
// from the caller; this one needs no scratch from anybody.  The only scratch the
// routing and dispatch kernels use - the per-block expert counts that the router
// writes and the permute kernel scans - lives in a fixed array inside the
// library image instead.
//
// Cost and limits, so nobody is surprised:
//   * the array is part of the module: every GPU that loads the library holds
//     AXM_NOALLOC_SCRATCH_BYTES (148 KiB) of device memory until the process exits;
//   * it is sized for at most AXM_NOALLOC_MAX_EXPERTS experts; a larger
//     num_experts is refused with AXM_ERR_ARGUMENT, nothing is launched;
//   * all calls on one GPU share the array.  Each call overwrites all of the part
//     it reads (the router kernel stores a count for every block and expert,
//     zeros included), so nothing has to be cleared between calls and nothing
//     left over from an earlier call is ever read; but two calls whose kernels
//     overlap on the GPU (different streams, no dependency) race on it.  Order
//     such calls yourself;
//   * the first call on each device looks up the array's device address
//     (cudaGetSymbolAddress, which may load the module and create the context).
//     Make that first call outside any stream capture.
#include <mutex>

#include "common.cuh"

namespace axm {

constexpr int kNoAllocMaxExperts = AXM_NOALLOC_MAX_EXPERTS;
constexpr int kMaxDevices = 64;

// [AXM_ROUTE_BLOCKS][kNoAllocMaxExperts] int32.  In host code this name is only a
// handle for the runtime, not a device address: the address is resolved below.
static __device__ __align__(256) int32_t g_block_counts_scratch[AXM_ROUTE_BLOCKS * kNoAllocMaxExperts];

static_assert(sizeof(int32_t) * AXM_ROUTE_BLOCKS * kNoAllocMaxExperts == AXM_NOALLOC_SCRATCH_BYTES,
              "AXM_NOALLOC_SCRATCH_BYTES in the header is out of date");

static std::mutex g_scratch_mutex;
static int32_t* g_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch array on the current device, resolved once per
// device with that device current.
static int scratch_for_current_device(int32_t** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(AXM_ERR_DEVICE, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(AXM_ERR_DEVICE, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_block_counts_scratch);
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return fail(AXM_ERR_DEVICE, "cudaGetSymbolAddress(scratch) on device %d: %s", dev,
                  cudaGetErrorString(e));
    }
    g_scratch_ptr[dev] = static_cast<int32_t*>(p);
  }
  *out = g_scratch_ptr[dev];
  return AXM_OK;
}

}  // namespace axm

using namespace axm;

extern "C" int axm_moe_route_dispatch_noalloc(const AxmMoeDesc* desc, const float* logits,
                                              const void* x, int32_t* topk_idx, float* topk_gate,
                                              int32_t* histogram, int32_t* offsets,
                                              int32_t* row_src, int32_t* slot_dst, void* x_perm,
                                              void* stream) {
  if (desc == nullptr) return fail(AXM_ERR_ARGUMENT, "desc is null");
  if (desc->num_experts > kNoAllocMaxExperts)
    return fail(AXM_ERR_ARGUMENT,
                "axm_moe_route_dispatch_noalloc: num_experts %d exceeds the built-in scratch "
                "(at most %d experts); use axm_moe_route_from_logits + axm_moe_permute with "
                "caller-provided scratch",
                desc->num_experts, kNoAllocMaxExperts);
  // Everything both stages check is checked here, before the first launch: a call that
  // is going to be refused must not have written routing results already.
  if (int rc = validate_route(desc)) return rc;
  if (int rc = validate_perm(desc)) return rc;
  if (!logits || !topk_idx || !topk_gate)
    return fail(AXM_ERR_ARGUMENT, "axm_moe_route_dispatch_noalloc: null pointer");
  if (x_perm != nullptr && x == nullptr)
    return fail(AXM_ERR_ARGUMENT, "axm_moe_route_dispatch_noalloc: x_perm without x");
  if (int rc = require_device()) return rc;
  int32_t* scratch = nullptr;
  if (int rc = scratch_for_current_device(&scratch)) return rc;
  // Same kernels as the regular entry points, with the library's own array as
  // the block-count scratch.
  if (int rc = axm_moe_route_from_logits(desc, logits, topk_idx, topk_gate, scratch, stream)) return rc;
  return axm_moe_permute(desc, x, topk_idx, scratch, histogram, offsets, row_src, slot_dst, x_perm,
                         stream);
}
