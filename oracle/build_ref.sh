#!/bin/sh
# Builds the reference engine's MoE kernels, UNMODIFIED, from the sources where
# they lie (the directory named by REF) into oracle/_ref/ as a second checker
# beside the CPU oracle.  Nothing of the reference is copied into this
# repository: the output directory is git-ignored and holds only a binary and a
# small JSON of struct offsets measured by compiling a probe against the
# reference's own header.
#
# The reference is source-available under its own licence, which allows building
# the unmodified source and running it locally for evaluation.  Its build system
# asks for an explicit acceptance (AXIOM_ACCEPT_LICENSE=ON); this script asks for
# the same variable and does nothing without it.  Read $REF/LICENSE first.
set -e
if [ -z "${REF}" ]; then
  echo "build_ref.sh: set REF to the directory that holds the reference engine's sources" >&2
  exit 2
fi
HERE="$(cd "$(dirname "$0")" && pwd)"
if [ "${AXIOM_ACCEPT_LICENSE}" != "ON" ]; then
  echo "build_ref.sh: set AXIOM_ACCEPT_LICENSE=ON to accept ${REF}/LICENSE and build the reference kernels" >&2
  exit 3
fi
if [ ! -f "${REF}/core/src/CUDA/kernel/moe_router.cu" ]; then
  echo "build_ref.sh: reference sources not found under ${REF}" >&2
  exit 4
fi
NVCC="${NVCC:-$(command -v nvcc || echo /usr/local/cuda/bin/nvcc)}"
mkdir -p "${HERE}/_ref"
"${NVCC}" -arch=sm_100a --std=c++20 -O3 -D'__declspec(x)=' -DBUILDING_CUDA_DLL \
  -I"${REF}/core/include" -I"${REF}/core/src/CUDA/util" --expt-relaxed-constexpr \
  -Xcompiler -fPIC -shared -cudart shared -o "${HERE}/_ref/libaxiom_moe_ref.so" \
  "${REF}/core/src/CUDA/kernel/moe_router.cu" \
  "${REF}/core/src/CUDA/util/caching_allocator.cu" \
  "${REF}/core/src/CUDA/util/memory_allocation.cu"
"${NVCC}" --std=c++20 -D'__declspec(x)=' -I"${REF}/core/include" -I"${REF}/core/src/CUDA/util" \
  -DREF_TYPES_HEADER="\"${REF}/core/src/CUDA/util/gpu_types.cuh\"" \
  -o "${HERE}/_ref/ref_offsets_probe" "${HERE}/ref_offsets_probe.cu"
"${HERE}/_ref/ref_offsets_probe" > "${HERE}/_ref/ref_offsets.json"
rm -f "${HERE}/_ref/ref_offsets_probe"
echo "built ${HERE}/_ref/libaxiom_moe_ref.so and ref_offsets.json"
