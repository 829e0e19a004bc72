"""Python host helper over the C ABI of the B200 MoE layer (include/axm_moe.h).

The product is the shared library; this module only loads it with ctypes and
offers the call shape of the reference engine's host wrapper
AI::forward_mixture_experts (core/src/ai.cpp:593-623): give it activations, get
the layer output and the per-expert histogram back.  PyTorch is used for device
memory and streams, nothing else.  There is no fallback: if the library is not
built, or no sm_100 device is present, calls raise.
"""
import ctypes
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libaxm_moe.so")
DROPIN_PATH = os.path.join(HERE, "libaxm_moe_dropin.so")
HEADER_PATH = os.path.join(HERE, "..", "include", "axm_moe.h")

AXM_OK = 0
AXM_ERR_ARGUMENT = -1
AXM_ERR_WORKSPACE = -2
AXM_ERR_DEVICE = -3
AXM_ERR_LAUNCH = -4
AXM_ERR_TIMEOUT = -5
ROUTER_BF16 = 0
ROUTER_FP32 = 1
FLAG_RESIDUAL = 1
FLAG_HIST_ACCUMULATE = 2
FLAG_H_EXACT = 4
ROUTE_BLOCKS = 296
SEG_ALT_A = 1 << 30
NOALLOC_MAX_EXPERTS = 128


class AxmError(RuntimeError):
    def __init__(self, status, text):
        super().__init__(f"axm_moe status {status}: {text}")
        self.status = status


class MoeDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in (
        "tokens", "d_model", "d_ff", "num_experts", "top_k", "num_shared", "router_dtype", "flags")]


class MoeTensors(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in (
        "x", "router_w", "router_bias", "w_gate", "w_up", "w_down", "shared_gate", "shared_up",
        "shared_down", "logits", "topk_idx", "topk_gate", "histogram", "offsets", "row_src",
        "slot_dst", "y", "out")]


class EpLayout(ctypes.Structure):
    _fields_ = ([("peers", ctypes.c_void_p)] +
                [(n, ctypes.c_int32) for n in ("rank", "world", "num_experts", "d_model", "slots",
                                               "cap", "num_shared", "tokens_local")] +
                [(n, ctypes.c_int64) for n in ("off_flags", "off_counts", "off_recv", "off_oback")] +
                [("local_region", ctypes.c_void_p), ("row_align", ctypes.c_int32),
                 ("return_rows", ctypes.c_int32)])


class EpTensors(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in (
        "x", "router_w", "router_bias", "w_gate", "w_up", "w_down", "shared_gate", "shared_up",
        "shared_down", "logits", "topk_idx", "topk_gate", "histogram", "y", "out")]


class MoeTrain(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_void_p) for n in ("x", "router_w", "router_bias", "w_gate", "w_up",
                                                "w_down", "out", "aux_loss", "histogram")] +
                [("aux_alpha", ctypes.c_float)] +
                [(n, ctypes.c_void_p) for n in ("d_out", "d_x", "d_router_w", "d_w_gate", "d_w_up",
                                                "d_w_down", "d_router_bias", "shared_gate", "shared_up",
                                                "shared_down", "d_shared_gate", "d_shared_up",
                                                "d_shared_down")])


class MoeCheckpoint(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in ("router_w", "router_bias", "w_gate", "w_up", "w_down",
                                               "shared_gate", "shared_up", "shared_down")]


class Segment(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("a_row0", "out_row0", "rows", "expert")]


_lib = None


def load():
    """Loads libaxm_moe.so (once) and declares its prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is not built; run `python project-axiom-ai-llm_b200/build.py`")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i32, sz = ctypes.c_void_p, ctypes.c_int32, ctypes.c_size_t
    dp = ctypes.POINTER(MoeDesc)
    lib.axm_last_error.restype = ctypes.c_char_p
    lib.axm_version.restype = ctypes.c_char_p
    lib.axm_moe_forward_launches.argtypes = [dp]
    lib.axm_moe_workspace_bytes.argtypes = [dp, ctypes.POINTER(sz)]
    lib.axm_moe_forward.argtypes = [dp, ctypes.POINTER(MoeTensors), vp, sz, vp]
    lib.axm_moe_forward_profiled.argtypes = [dp, ctypes.POINTER(MoeTensors), vp, sz, vp,
                                             ctypes.POINTER(ctypes.c_float)]
    lib.axm_moe_forward_prenorm.argtypes = [dp, ctypes.POINTER(MoeTensors), vp, ctypes.c_float, vp, vp, sz, vp]
    lib.axm_moe_rmsnorm.argtypes = [vp, vp, vp, i32, i32, ctypes.c_float, vp]
    lib.axm_moe_forward_host.argtypes = [dp, ctypes.POINTER(MoeTensors), vp, vp, vp, vp, vp, sz, vp]
    lib.axm_moe_forward_host_batches.argtypes = [dp, ctypes.POINTER(MoeTensors), ctypes.POINTER(vp),
                                                 ctypes.POINTER(vp), i32, vp, vp, vp, sz, vp]
    lib.axm_moe_status_word.argtypes = [dp, vp, ctypes.POINTER(vp)]
    lib.axm_moe_router.argtypes = [dp, vp, vp, vp, vp, vp, vp, vp, vp]
    lib.axm_moe_router_scratch_bytes.argtypes = [dp, ctypes.POINTER(sz)]
    lib.axm_moe_router_ws.argtypes = [dp, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp, vp]
    lib.axm_moe_route_from_logits.argtypes = [dp, vp, vp, vp, vp, vp]
    lib.axm_moe_permute.argtypes = [dp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
    lib.axm_moe_build_segments.argtypes = [dp, vp, vp, vp]
    lib.axm_moe_expert_ffn.argtypes = [dp, vp, i32, vp, i32, vp, i32, vp, vp, vp, vp, vp, vp, vp,
                                       vp, i32, vp, vp]
    lib.axm_moe_combine.argtypes = [dp, vp, vp, vp, vp, vp, vp, vp, vp]
    tp = ctypes.POINTER(MoeTrain)
    lib.axm_moe_train_workspace_bytes.argtypes = [dp, ctypes.POINTER(sz)]
    lib.axm_moe_forward_train.argtypes = [dp, tp, vp, sz, vp]
    lib.axm_moe_backward.argtypes = [dp, tp, vp, sz, vp]
    lib.axm_moe_permute_padded.argtypes = [dp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, vp]
    lib.axm_moe_adamw_step.argtypes = [vp, vp, vp, vp, vp, ctypes.c_int64] + [ctypes.c_float] * 5 + [i32, vp]
    lib.axm_moe_adamw_step_engine.argtypes = ([vp] * 5 + [ctypes.c_int64, ctypes.c_int64] +
                                              [ctypes.c_float] * 5 + [ctypes.c_int64, vp])
    lib.axm_moe_expert_ffn_backward.argtypes = [dp, vp, i32, i32] + [vp] * 16
    lp, u32 = ctypes.POINTER(EpLayout), ctypes.c_uint32
    lib.axm_ep_region_bytes.argtypes = [i32, i32, i32, i32, i32, lp, ctypes.POINTER(sz)]
    lib.axm_ep_dispatch.argtypes = [lp, u32, vp, vp, vp, vp, vp]
    lib.axm_ep_segments.argtypes = [lp, u32, vp, vp, vp, vp, vp, vp]
    lib.axm_ep_signal_return.argtypes = [lp, u32, vp]
    lib.axm_moe_expert_ffn_remote.argtypes = [dp, vp, i32, vp, i32, vp, i32, vp, vp, vp, vp, vp, vp,
                                              vp, vp, i32, vp, vp, vp]
    lib.axm_ep_return.argtypes = [lp, u32, vp, vp, vp, vp, vp]
    lib.axm_ep_wait_return.argtypes = [lp, u32, vp, vp]
    ept = ctypes.POINTER(EpTensors)
    lib.axm_moe_ep_workspace_bytes.argtypes = [lp, dp, ctypes.POINTER(sz), ctypes.POINTER(sz)]
    lib.axm_moe_ep_forward.argtypes = [lp, dp, ept, vp, sz, u32, vp]
    lib.axm_moe_ep_status_word.argtypes = [lp, dp, vp, ctypes.POINTER(vp), ctypes.POINTER(vp)]
    lib.axm_moe_ep_forward_profiled.argtypes = [lp, dp, ept, vp, sz, u32, vp, ctypes.POINTER(ctypes.c_float)]
    lib.axm_moe_ep_forward_host.argtypes = [lp, dp, ept, vp, vp, vp, vp, vp, sz, i32, ctypes.POINTER(u32), vp]
    lib.axm_moe_ep_train_workspace_bytes.argtypes = [lp, dp, ctypes.POINTER(sz), ctypes.POINTER(sz)]
    lib.axm_moe_ep_forward_train.argtypes = [lp, dp, tp, i32, vp, sz, u32, vp]
    lib.axm_moe_ep_backward.argtypes = [lp, lp, dp, tp, i32, vp, sz, u32, vp]
    lib.axm_moe_ep_train_status_word.argtypes = [lp, dp, vp, ctypes.POINTER(vp), ctypes.POINTER(vp)]
    lib.axm_moe_route_dispatch_noalloc.argtypes = [dp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
    cp = ctypes.POINTER(MoeCheckpoint)
    lib.axm_moe_checkpoint_save.argtypes = [ctypes.c_char_p, dp, cp]
    lib.axm_moe_checkpoint_probe.argtypes = [ctypes.c_char_p, dp, ctypes.POINTER(i32)]
    lib.axm_moe_checkpoint_load.argtypes = [ctypes.c_char_p, dp, cp]
    lib.axm_moe_cast_master.argtypes = [vp, vp, sz, vp]
    _lib = lib
    return lib


def check(status):
    if status != AXM_OK:
        raise AxmError(status, load().axm_last_error().decode())
    return status


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def current_stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def make_desc(tokens, d_model, d_ff, num_experts, top_k, num_shared=0, router_dtype=ROUTER_FP32,
              flags=FLAG_RESIDUAL):
    return MoeDesc(tokens, d_model, d_ff, num_experts, top_k, num_shared, router_dtype, flags)


def router_scratch_bytes(desc):
    """Bytes of scratch axm_moe_router_ws wants for this shape (0: no tensor-core router for it)."""
    n = ctypes.c_size_t(0)
    check(load().axm_moe_router_scratch_bytes(ctypes.byref(desc), ctypes.byref(n)))
    return n.value


def workspace_bytes(desc):
    n = ctypes.c_size_t(0)
    check(load().axm_moe_workspace_bytes(ctypes.byref(desc), ctypes.byref(n)))
    return n.value


class MoeLayer:
    """One MoE layer bound to its weights, with a workspace sized for `tokens`.

    forward(x) returns (out, histogram) like the reference host wrapper; the
    routing tensors of the last call stay readable as attributes.  h_exact keeps
    the SwiGLU intermediate in two bf16 terms (AXM_FLAG_H_EXACT): every output
    element then meets the layer tolerance against an fp32 intermediate.
    """

    def __init__(self, weights, tokens, top_k, residual=True, hist_accumulate=False,
                 device="cuda", publish_y=True, h_exact=False):
        self.lib = load()
        self.w = weights
        wr = weights["router_w"]
        D, E = wr.shape
        F = weights["w_gate"].shape[2]
        S = 0 if weights.get("shared_gate") is None else weights["shared_gate"].shape[0]
        flags = ((FLAG_RESIDUAL if residual else 0) | (FLAG_HIST_ACCUMULATE if hist_accumulate else 0) |
                 (FLAG_H_EXACT if h_exact else 0))
        rdt = ROUTER_FP32 if wr.dtype == torch.float32 else ROUTER_BF16
        self.desc = make_desc(tokens, D, F, E, top_k, S, rdt, flags)
        self.T, self.D, self.F, self.E, self.k, self.S = tokens, D, F, E, top_k, S
        self.device = torch.device(device)
        # 256 spare bytes: the batch pipeline keeps one status word per batch behind the workspace
        self.workspace = torch.empty(max(workspace_bytes(self.desc), 256) + 256, dtype=torch.uint8,
                                     device=self.device)
        dev = self.device
        self.logits = torch.empty(tokens, E, dtype=torch.float32, device=dev)
        self.topk_idx = torch.empty(tokens, top_k, dtype=torch.int32, device=dev)
        self.topk_gate = torch.empty(tokens, top_k, dtype=torch.float32, device=dev)
        self.histogram = torch.zeros(E, dtype=torch.int32, device=dev)
        self.offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
        self.row_src = torch.empty(tokens * top_k, dtype=torch.int32, device=dev)
        self.slot_dst = torch.empty(tokens * top_k, dtype=torch.int32, device=dev)
        self.y = torch.empty(tokens, D, dtype=torch.bfloat16, device=dev) if publish_y else None

    def tensors(self, x, out):
        w = self.w
        return MoeTensors(
            x.data_ptr(), w["router_w"].data_ptr(),
            None if w.get("router_bias") is None else w["router_bias"].data_ptr(),
            w["w_gate"].data_ptr(), w["w_up"].data_ptr(), w["w_down"].data_ptr(),
            None if self.S == 0 else w["shared_gate"].data_ptr(),
            None if self.S == 0 else w["shared_up"].data_ptr(),
            None if self.S == 0 else w["shared_down"].data_ptr(),
            self.logits.data_ptr(), self.topk_idx.data_ptr(), self.topk_gate.data_ptr(),
            self.histogram.data_ptr(), self.offsets.data_ptr(), self.row_src.data_ptr(),
            self.slot_dst.data_ptr(), None if self.y is None else self.y.data_ptr(), out.data_ptr())

    def forward(self, x, out=None):
        assert x.is_cuda and x.dtype == torch.bfloat16 and x.shape == (self.T, self.D)
        assert x.is_contiguous()
        if out is None:
            out = torch.empty_like(x)
        t = self.tensors(x, out)
        check(self.lib.axm_moe_forward(ctypes.byref(self.desc), ctypes.byref(t), ptr(self.workspace),
                                       self.workspace.numel(), current_stream()))
        return out, self.histogram

    def forward_prenorm(self, x, gamma, eps, x_norm, out=None):
        """out = x + MoE(RMSNorm(x)); x_norm receives the normalised activations (None: the
        normalisation is folded into the router's and the permute kernel's reads)."""
        if out is None:
            out = torch.empty_like(x)
        t = self.tensors(x, out)
        check(self.lib.axm_moe_forward_prenorm(ctypes.byref(self.desc), ctypes.byref(t), ptr(gamma), eps,
                                               ptr(x_norm), ptr(self.workspace), self.workspace.numel(),
                                               current_stream()))
        return out

    def forward_profiled(self, x, out=None):
        """forward() with per-stage device times: returns (out, [ms] * 5)."""
        if out is None:
            out = torch.empty_like(x)
        t = self.tensors(x, out)
        ms = (ctypes.c_float * 5)()
        check(self.lib.axm_moe_forward_profiled(ctypes.byref(self.desc), ctypes.byref(t),
                                                ptr(self.workspace), self.workspace.numel(),
                                                current_stream(), ms))
        return out, list(ms)

    def forward_host(self, h_x, h_out, d_x, d_out, keep_permutation=False):
        """Activations in (pinned) host memory; synchronises before returning."""
        t = self.tensors(d_x, d_out)
        if not keep_permutation:   # lets the call pipeline copies and compute in chunks
            t.offsets = t.row_src = t.slot_dst = None
        check(self.lib.axm_moe_forward_host(
            ctypes.byref(self.desc), ctypes.byref(t), ptr(h_x), ptr(h_out), ptr(d_x), ptr(d_out),
            ptr(self.workspace), self.workspace.numel(), current_stream()))
        return h_out

    def forward_host_batches(self, h_xs, h_outs, d_x2, d_out2):
        """A run of batches from pinned host memory, double-buffered on the device (batch i + 1
        comes in while batch i is computed and batch i - 1 goes out); synchronises."""
        n = len(h_xs)
        assert n == len(h_outs) and d_x2.shape[0] == 2 * self.T and d_out2.shape[0] == 2 * self.T
        t = self.tensors(d_x2, d_out2)
        t.logits = t.topk_idx = t.topk_gate = t.offsets = t.row_src = t.slot_dst = t.y = None
        xs = (ctypes.c_void_p * n)(*[h.data_ptr() for h in h_xs])
        outs = (ctypes.c_void_p * n)(*[h.data_ptr() for h in h_outs])
        check(self.lib.axm_moe_forward_host_batches(
            ctypes.byref(self.desc), ctypes.byref(t), xs, outs, n, ptr(d_x2), ptr(d_out2),
            ptr(self.workspace), self.workspace.numel(), current_stream()))
        return h_outs

    def status(self):
        """Reads the workspace status word (synchronises)."""
        p = ctypes.c_void_p()
        check(self.lib.axm_moe_status_word(ctypes.byref(self.desc), ptr(self.workspace),
                                           ctypes.byref(p)))
        off = p.value - self.workspace.data_ptr()
        torch.cuda.synchronize()
        return int(self.workspace[off:off + 4].view(torch.int32).item())


class MoeTrainLayer:
    """Forward + backward of one MoE layer (training step).  step(x, d_out) returns
    (out, aux_loss, grads) with grads = dict(d_x, d_router_w, d_w_gate, d_w_up, d_w_down)."""

    def __init__(self, weights, tokens, top_k, aux_alpha=0.01, device="cuda", weight_grads=True):
        self.lib = load()
        self.w = weights
        wr = weights["router_w"]
        D, E = wr.shape
        F = weights["w_gate"].shape[2]
        rdt = ROUTER_FP32 if wr.dtype == torch.float32 else ROUTER_BF16
        S = self.S = 0 if weights.get("shared_gate") is None else weights["shared_gate"].shape[0]
        self.desc = make_desc(tokens, D, F, E, top_k, S, rdt, FLAG_RESIDUAL)
        dev = torch.device(device)
        n = ctypes.c_size_t(0)
        check(self.lib.axm_moe_train_workspace_bytes(ctypes.byref(self.desc), ctypes.byref(n)))
        self.workspace = torch.empty(n.value, dtype=torch.uint8, device=dev)
        f32 = torch.float32
        self.out = torch.empty(tokens, D, dtype=torch.bfloat16, device=dev)
        self.aux = torch.zeros(1, dtype=f32, device=dev)
        self.histogram = torch.zeros(E, dtype=torch.int32, device=dev)
        self.d_x = torch.empty(tokens, D, dtype=f32, device=dev)
        self.d_router_w = torch.empty(D, E, dtype=f32, device=dev)
        self.d_router_bias = (torch.empty(E, dtype=f32, device=dev)
                              if weights.get("router_bias") is not None else None)
        self.weight_grads = weight_grads
        if weight_grads:
            self.d_w_gate = torch.empty(E, D, F, dtype=f32, device=dev)
            self.d_w_up = torch.empty(E, D, F, dtype=f32, device=dev)
            self.d_w_down = torch.empty(E, F, D, dtype=f32, device=dev)
            if S:
                self.d_shared_gate = torch.empty(S, D, F, dtype=f32, device=dev)
                self.d_shared_up = torch.empty(S, D, F, dtype=f32, device=dev)
                self.d_shared_down = torch.empty(S, F, D, dtype=f32, device=dev)
        self.aux_alpha = aux_alpha

    def tensors(self, x, d_out):
        w = self.w
        g = self.weight_grads
        return MoeTrain(
            x.data_ptr(), w["router_w"].data_ptr(),
            None if w.get("router_bias") is None else w["router_bias"].data_ptr(),
            w["w_gate"].data_ptr(), w["w_up"].data_ptr(), w["w_down"].data_ptr(),
            self.out.data_ptr(), self.aux.data_ptr(), self.histogram.data_ptr(), self.aux_alpha,
            None if d_out is None else d_out.data_ptr(), self.d_x.data_ptr(),
            self.d_router_w.data_ptr(), self.d_w_gate.data_ptr() if g else None,
            self.d_w_up.data_ptr() if g else None, self.d_w_down.data_ptr() if g else None,
            None if self.d_router_bias is None else self.d_router_bias.data_ptr(),
            w["shared_gate"].data_ptr() if self.S else None, w["shared_up"].data_ptr() if self.S else None,
            w["shared_down"].data_ptr() if self.S else None,
            self.d_shared_gate.data_ptr() if g and self.S else None,
            self.d_shared_up.data_ptr() if g and self.S else None,
            self.d_shared_down.data_ptr() if g and self.S else None)

    def forward(self, x):
        t = self.tensors(x, None)
        check(self.lib.axm_moe_forward_train(ctypes.byref(self.desc), ctypes.byref(t),
                                             ptr(self.workspace), self.workspace.numel(),
                                             current_stream()))
        return self.out

    def backward(self, x, d_out):
        t = self.tensors(x, d_out)
        check(self.lib.axm_moe_backward(ctypes.byref(self.desc), ctypes.byref(t), ptr(self.workspace),
                                        self.workspace.numel(), current_stream()))
        return self.d_x

    def step(self, x, d_out):
        self.forward(x)
        self.backward(x, d_out)
        grads = {"d_x": self.d_x, "d_router_w": self.d_router_w}
        if self.d_router_bias is not None:
            grads["d_router_bias"] = self.d_router_bias
        if self.weight_grads:
            grads.update(d_w_gate=self.d_w_gate, d_w_up=self.d_w_up, d_w_down=self.d_w_down)
            if self.S:
                grads.update(d_shared_gate=self.d_shared_gate, d_shared_up=self.d_shared_up,
                             d_shared_down=self.d_shared_down)
        return self.out, self.aux, grads
