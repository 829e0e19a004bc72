"""Drives the reference engine's unmodified MoE kernels (oracle/_ref, built by
oracle/build_ref.sh) on torch CUDA tensors.  Tests and the benchmark's optional
reference leg only.  The caller-side structs are opaque byte blobs; the offsets
of the fields come from oracle/_ref/ref_offsets.json, which the build measures
against the reference's own header (core/src/CUDA/util/gpu_types.cuh)."""
import ctypes
import json
import os
import struct

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")
REF_LIB = os.path.join(REF_DIR, "libaxiom_moe_ref.so")
REF_OFFSETS = os.path.join(REF_DIR, "ref_offsets.json")


# Field offsets of the engine's structs on Linux x86-64, as measured by
# oracle/ref_offsets_probe.cu against the engine's header.  Used when the
# reference build (and its JSON) is absent, e.g. to drive the drop-in library.
OFFSETS_LINUX_X86_64 = {
    "sizeof_GpuWeights": 472, "sizeof_GpuActivations": 328, "w.enable_moe": 328,
    "w.expert_count": 336, "w.d_router_weights": 344, "w.d_expert_gate": 376, "w.d_expert_up": 384,
    "w.d_expert_down": 392, "a.d_ffn_output": 144, "a.d_residual_out": 160,
    "a.d_router_logits": 216, "a.d_expert_first": 224, "a.d_expert_second": 232,
    "a.d_weight_first": 240, "a.d_weight_second": 248, "a.d_expert_histogram": 256,
}


def available():
    return os.path.exists(REF_LIB) and os.path.exists(REF_OFFSETS)


class ReferenceMoe:
    """forward_mixture_experts / download_expert_counts / reset_expert_histogram
    (core/src/CUDA/kernel/moe_router.cuh:30-44) of the reference build, or of any
    other library that exports the same three symbols (lib_path)."""

    def __init__(self, lib_path=None):
        self.lib = ctypes.CDLL(lib_path or REF_LIB)
        self.off = (json.load(open(REF_OFFSETS)) if lib_path is None and os.path.exists(REF_OFFSETS)
                    else dict(OFFSETS_LINUX_X86_64))
        vp, sz = ctypes.c_void_p, ctypes.c_size_t
        self.lib.forward_mixture_experts.argtypes = [vp, vp, vp, sz, sz, sz, vp]
        self.lib.forward_mixture_experts.restype = ctypes.c_bool
        self.lib.download_expert_counts.argtypes = [vp, vp, sz]
        self.lib.download_expert_counts.restype = ctypes.c_bool
        self.lib.reset_expert_histogram.argtypes = [vp, sz, vp]
        self.lib.reset_expert_histogram.restype = ctypes.c_bool
        self.cudart = ctypes.CDLL("libcudart.so.12")
        self.cudart.cudaMemcpy.argtypes = [vp, vp, sz, ctypes.c_int]
        self.weights = ctypes.create_string_buffer(self.off["sizeof_GpuWeights"])
        self.acts = ctypes.create_string_buffer(self.off["sizeof_GpuActivations"])
        self.keep = None

    def set_weights(self, router_w_bf16, w_gate, w_up, w_down):
        E = w_gate.shape[0]
        self.keep = (router_w_bf16, w_gate, w_up, w_down)
        o = self.off
        struct.pack_into("?", self.weights, o["w.enable_moe"], True)
        struct.pack_into("Q", self.weights, o["w.expert_count"], E)
        for name, t in (("w.d_router_weights", router_w_bf16), ("w.d_expert_gate", w_gate),
                        ("w.d_expert_up", w_up), ("w.d_expert_down", w_down)):
            assert t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous()
            struct.pack_into("Q", self.weights, o[name], t.data_ptr())
        self.E = E

    def forward(self, hidden, F):
        """In place on `hidden` ([T][D] bf16, CUDA), on the legacy default stream."""
        T, D = hidden.shape
        ok = self.lib.forward_mixture_experts(hidden.data_ptr(), ctypes.addressof(self.weights),
                                              ctypes.addressof(self.acts), T, D, F, None)
        torch.cuda.synchronize()
        return bool(ok)

    def _field(self, name, shape, dtype):
        p = struct.unpack_from("Q", self.acts, self.off[name])[0]
        assert p != 0, f"reference did not allocate {name}"
        t = torch.empty(shape, dtype=dtype, device="cuda")
        rc = self.cudart.cudaMemcpy(t.data_ptr(), p, t.numel() * t.element_size(), 3)
        assert rc == 0
        torch.cuda.synchronize()
        return t

    def outputs(self, T, D):
        E = self.E
        return {
            "logits": self._field("a.d_router_logits", (T, E), torch.float32),
            "first": self._field("a.d_expert_first", (T,), torch.int32),
            "second": self._field("a.d_expert_second", (T,), torch.int32),
            "w_first": self._field("a.d_weight_first", (T,), torch.float32),
            "w_second": self._field("a.d_weight_second", (T,), torch.float32),
            "histogram": self._field("a.d_expert_histogram", (E,), torch.int32),
            "ffn_output": self._field("a.d_ffn_output", (T, D), torch.bfloat16),
            "residual_out": self._field("a.d_residual_out", (T, D), torch.bfloat16),
        }

    def download_counts(self):
        buf = (ctypes.c_int32 * self.E)()
        ok = self.lib.download_expert_counts(ctypes.addressof(self.acts), buf, self.E)
        return bool(ok), list(buf)

    def reset_histogram(self):
        ok = self.lib.reset_expert_histogram(ctypes.addressof(self.acts), self.E, None)
        torch.cuda.synchronize()
        return bool(ok)
