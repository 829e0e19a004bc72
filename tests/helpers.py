"""Thin callers of the C-ABI stage functions on torch CUDA tensors (tests only)."""
import ctypes

import numpy as np
import torch


def desc_for(axm, cfg, router_dtype=None, flags=None, tokens=None):
    return axm.make_desc(cfg.tokens if tokens is None else tokens, cfg.d_model, cfg.d_ff,
                         cfg.num_experts, cfg.top_k, cfg.num_shared,
                         axm.ROUTER_FP32 if router_dtype is None else router_dtype,
                         axm.FLAG_RESIDUAL if flags is None else flags)


def run_router(axm, desc, x, wr, bias=None, tensor_core=True):
    """The fused router: with scratch (tensor-core kernel where the shape allows it) or, with
    tensor_core=False, through axm_moe_router (CUDA-core kernel)."""
    lib = axm.load()
    T, E, k = desc.tokens, desc.num_experts, desc.top_k
    dev = x.device
    logits = torch.full((T, E), float("nan"), dtype=torch.float32, device=dev)
    idx = torch.full((T, k), -1, dtype=torch.int32, device=dev)
    gate = torch.empty(T, k, dtype=torch.float32, device=dev)
    bc = torch.full((axm.ROUTE_BLOCKS, E), 12345, dtype=torch.int32, device=dev)
    if tensor_core:
        need = axm.router_scratch_bytes(desc)
        scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        axm.check(lib.axm_moe_router_ws(ctypes.byref(desc), axm.ptr(x), axm.ptr(wr), axm.ptr(bias),
                                        axm.ptr(logits), axm.ptr(idx), axm.ptr(gate), axm.ptr(bc),
                                        axm.ptr(scratch), need, axm.ptr(status), axm.current_stream()))
        torch.cuda.synchronize()
        assert int(status.item()) == 0, f"router reported a timed-out wait: {int(status.item())}"
    else:
        axm.check(lib.axm_moe_router(ctypes.byref(desc), axm.ptr(x), axm.ptr(wr), axm.ptr(bias),
                                     axm.ptr(logits), axm.ptr(idx), axm.ptr(gate), axm.ptr(bc),
                                     axm.current_stream()))
    return logits, idx, gate, bc


def run_route_from_logits(axm, desc, logits):
    lib = axm.load()
    T, E, k = desc.tokens, desc.num_experts, desc.top_k
    dev = logits.device
    idx = torch.empty(T, k, dtype=torch.int32, device=dev)
    gate = torch.empty(T, k, dtype=torch.float32, device=dev)
    bc = torch.empty(axm.ROUTE_BLOCKS, E, dtype=torch.int32, device=dev)
    axm.check(lib.axm_moe_route_from_logits(ctypes.byref(desc), axm.ptr(logits), axm.ptr(idx),
                                            axm.ptr(gate), axm.ptr(bc), axm.current_stream()))
    return idx, gate, bc


def run_permute(axm, desc, x, idx, bc, histogram=None, copy_rows=True):
    lib = axm.load()
    T, E, k, D = desc.tokens, desc.num_experts, desc.top_k, desc.d_model
    dev = idx.device
    if histogram is None:
        histogram = torch.zeros(E, dtype=torch.int32, device=dev)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    row_src = torch.full((T * k,), -1, dtype=torch.int32, device=dev)
    slot_dst = torch.full((T * k,), -1, dtype=torch.int32, device=dev)
    xp = torch.zeros(T * k, D, dtype=torch.bfloat16, device=dev) if copy_rows else None
    axm.check(lib.axm_moe_permute(ctypes.byref(desc), axm.ptr(x), axm.ptr(idx), axm.ptr(bc),
                                  axm.ptr(histogram), axm.ptr(offsets), axm.ptr(row_src),
                                  axm.ptr(slot_dst), axm.ptr(xp), axm.current_stream()))
    return histogram, offsets, row_src, slot_dst, xp


def run_build_segments(axm, desc, offsets):
    lib = axm.load()
    n = desc.num_experts + desc.num_shared
    seg = torch.empty(n, 4, dtype=torch.int32, device=offsets.device)
    axm.check(lib.axm_moe_build_segments(ctypes.byref(desc), axm.ptr(offsets), axm.ptr(seg),
                                         axm.current_stream()))
    return seg


def run_expert_ffn(axm, desc, xp, x_alt, seg, w, rows_total):
    lib = axm.load()
    dev = xp.device
    h = torch.zeros(rows_total, desc.d_ff, dtype=torch.bfloat16, device=dev)
    o = torch.zeros(rows_total, desc.d_model, dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    S = desc.num_shared
    axm.check(lib.axm_moe_expert_ffn(
        ctypes.byref(desc), axm.ptr(xp), xp.shape[0], axm.ptr(x_alt),
        0 if x_alt is None else x_alt.shape[0], axm.ptr(seg), seg.shape[0],
        axm.ptr(w["w_gate"]), axm.ptr(w["w_up"]), axm.ptr(w["w_down"]),
        axm.ptr(w["shared_gate"]) if S else None, axm.ptr(w["shared_up"]) if S else None,
        axm.ptr(w["shared_down"]) if S else None, axm.ptr(h), axm.ptr(o), rows_total,
        axm.ptr(status), axm.current_stream()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"GEMM kernel reported a timed-out wait: {int(status.item())}"
    return h, o


def run_combine(axm, desc, x, o, o_shared, slot_dst, gate):
    lib = axm.load()
    y = torch.empty(desc.tokens, desc.d_model, dtype=torch.bfloat16, device=o.device)
    out = torch.empty_like(y)
    axm.check(lib.axm_moe_combine(ctypes.byref(desc), axm.ptr(x), axm.ptr(o), axm.ptr(o_shared),
                                  axm.ptr(slot_dst), axm.ptr(gate), axm.ptr(y), axm.ptr(out),
                                  axm.current_stream()))
    return y, out


def to_dev(w, dev):
    return {k: (v.to(dev) if v is not None else None) for k, v in w.items()}


def _check(err, bound, what, detail, allow_frac, hard_factor):
    bad = err > bound
    n_bad = int(bad.sum())
    worst = float((err / bound).max()) if err.numel() else 0.0
    assert n_bad <= allow_frac * err.numel() and worst <= hard_factor, (
        f"{what}: {n_bad} of {err.numel()} elements outside {detail} "
        f"(allowed {allow_frac:g} of them), worst err/bound {worst:.3f} (limit {hard_factor}), "
        f"max err {float(err.max()):.4g}")
    return n_bad


def assert_close_layer(got, ref, rel=2e-2, abs_=1e-2, what="layer output", allow_frac=0.0,
                       hard_factor=1.0):
    """|got - ref| <= abs_ + rel * |ref| element-wise (the layer tolerance).

    allow_frac / hard_factor: against a reference that keeps the SwiGLU
    intermediate in fp32, a pipeline that stores it as bf16 leaves a thin tail
    (a few elements per million at d_model 4096, d_ff 14336, where two large
    expert outputs cancel) just outside the bound; such a comparison allows that
    fraction of elements to exceed the bound, and none by more than hard_factor."""
    g, r = got.float().cpu(), ref.float().cpu()
    err = (g - r).abs()
    bound = abs_ + rel * r.abs()
    _check(err, bound, what, f"{abs_} + {rel}*|ref|", allow_frac, max(hard_factor, 1.0))
    return float(err.max()) if err.numel() else 0.0


def assert_close_out(got_out, ref_out, ref_y, rel=2e-2, abs_=1e-2, what="out", allow_frac=0.0,
                     hard_factor=1.0, out_step=2.0 ** -7):
    """Tolerance for out = bf16(x + y).  The layer tolerance applies to y; the
    residual add can cancel, so the same absolute error in y may be large
    relative to a small |x + y|.  The bound is therefore the y tolerance plus the
    rounding of the sum: |d| <= abs_ + rel * |y_ref| + out_step * |out_ref|, where
    out_step = 2^-7 covers the two bf16 roundings (half a step, 2^-8 * |out|, on
    each side); the strict comparisons pass 2^-8."""
    g, r, y = got_out.float().cpu(), ref_out.float().cpu(), ref_y.float().cpu()
    err = (g - r).abs()
    bound = abs_ + rel * y.abs() + out_step * r.abs()
    _check(err, bound, what, f"{abs_} + {rel}*|y_ref| + {out_step:g}*|out_ref|", allow_frac,
           max(hard_factor, 1.0))
    return float(err.max()) if err.numel() else 0.0
