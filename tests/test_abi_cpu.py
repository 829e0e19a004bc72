"""The C-ABI library loads, exports every symbol its header declares, validates
arguments, and refuses to compute without an sm_100 device (no CPU fallback)."""
import ctypes
import os
import re

import pytest
import torch


def declared_symbols(path):
    text = open(path).read()
    return sorted(set(re.findall(r"AXM_API\s+[\w\s\*]+?\b(axm_\w+)\s*\(", text)))


def test_exports_every_declared_symbol(axm):
    lib = axm.load()
    names = declared_symbols(axm.HEADER_PATH)
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/axm_moe.h but not exported"
    assert b"sm_100a" in lib.axm_version()


def test_dropin_exports_the_reference_symbols(axm):
    """libaxm_moe_dropin.so exports exactly what include/axm_moe_dropin.h declares."""
    header = os.path.join(os.path.dirname(axm.HEADER_PATH), "axm_moe_dropin.h")
    text = open(header).read()
    names = sorted(set(re.findall(r"AXM_API\s+bool\s+(\w+)\s*\(", text)))
    assert names == ["download_expert_counts", "forward_mixture_experts", "reset_expert_histogram"]
    lib = ctypes.CDLL(axm.DROPIN_PATH)
    for n in names:
        assert hasattr(lib, n)
    lib.forward_mixture_experts.restype = ctypes.c_bool
    lib.forward_mixture_experts.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_size_t] * 3 + [ctypes.c_void_p]
    # argument validation happens before any CUDA call
    assert lib.forward_mixture_experts(None, None, None, 1, 1, 1, None) is False
    blob = ctypes.create_string_buffer(512)
    assert lib.forward_mixture_experts(ctypes.addressof(blob), ctypes.addressof(blob),
                                       ctypes.addressof(blob), 0, 8, 8, None) is False


def test_struct_sizes_match_header(axm):
    assert ctypes.sizeof(axm.MoeDesc) == 32
    assert ctypes.sizeof(axm.MoeTensors) == 18 * 8
    assert ctypes.sizeof(axm.Segment) == 16
    assert ctypes.sizeof(axm.MoeTrain) == 23 * 8       # 22 pointers and one float, padded
    assert ctypes.sizeof(axm.EpLayout) == 8 + 8 * 4 + 4 * 8 + 8 + 2 * 4
    assert ctypes.sizeof(axm.EpTensors) == 15 * 8


def test_workspace_size_and_launch_count(axm):
    d = axm.make_desc(4096, 2048, 5632, 8, 2)
    n = axm.workspace_bytes(d)
    rows = 4096 * 2
    assert n >= 2 * rows * (2048 + 5632 + 2048)
    assert n % 256 == 0
    # router (with its weight-preparation kernel on the tensor-core path), permute, two GEMMs, combine
    assert axm.load().axm_moe_forward_launches(ctypes.byref(d)) == 6
    assert axm.router_scratch_bytes(d) == 3 * 16 * 2048 * 2      # three bf16 terms of 16 padded experts
    wide = axm.make_desc(4096, 2048, 5632, 128, 2)                 # 3 * 128 columns exceed one MMA
    assert axm.router_scratch_bytes(wide) == 0
    assert axm.load().axm_moe_forward_launches(ctypes.byref(wide)) == 5
    d0 = axm.make_desc(0, 2048, 5632, 8, 2)
    assert axm.load().axm_moe_forward_launches(ctypes.byref(d0)) == 0
    # up to eight tokens the down projection splits its reduction (one more launch: the sum of the
    # ranges) and the workspace holds the ranges' partial sums; not in the strict-tolerance mode
    few = axm.make_desc(1, 4096, 14336, 8, 2)
    assert axm.load().axm_moe_forward_launches(ctypes.byref(few)) == 7
    assert axm.load().axm_moe_forward_launches(ctypes.byref(axm.make_desc(16, 4096, 14336, 8, 2))) == 6
    few_x = axm.make_desc(1, 4096, 14336, 8, 2, flags=axm.FLAG_RESIDUAL | axm.FLAG_H_EXACT)
    assert axm.load().axm_moe_forward_launches(ctypes.byref(few_x)) == 6
    assert axm.workspace_bytes(few) >= 4 * 2 * 4096 * 4


@pytest.mark.parametrize("kw", [
    dict(d_model=2047), dict(d_ff=12), dict(num_experts=0), dict(num_experts=257), dict(top_k=0),
    dict(top_k=9), dict(top_k=3, num_experts=2), dict(num_shared=9), dict(tokens=-1),
    dict(router_dtype=7),
])
def test_bad_shapes_are_rejected(axm, kw):
    base = dict(tokens=64, d_model=256, d_ff=512, num_experts=8, top_k=2)
    base.update(kw)
    d = axm.make_desc(**base)
    n = ctypes.c_size_t(0)
    rc = axm.load().axm_moe_workspace_bytes(ctypes.byref(d), ctypes.byref(n))
    assert rc == axm.AXM_ERR_ARGUMENT
    assert len(axm.load().axm_last_error()) > 0


def test_null_pointers_are_rejected(axm):
    lib = axm.load()
    d = axm.make_desc(64, 256, 512, 8, 2)
    t = axm.MoeTensors()
    assert lib.axm_moe_forward(ctypes.byref(d), ctypes.byref(t), None, 0, None) == axm.AXM_ERR_ARGUMENT
    assert lib.axm_moe_forward(ctypes.byref(d), None, None, 0, None) == axm.AXM_ERR_ARGUMENT
    assert lib.axm_moe_router(ctypes.byref(d), None, None, None, None, None, None, None, None) \
        == axm.AXM_ERR_ARGUMENT
    assert lib.axm_moe_permute(ctypes.byref(d), None, None, None, None, None, None, None, None,
                               None) == axm.AXM_ERR_ARGUMENT
    assert lib.axm_moe_combine(ctypes.byref(d), None, None, None, None, None, None, None, None) \
        == axm.AXM_ERR_ARGUMENT


def test_workspace_checks(axm):
    lib = axm.load()
    d = axm.make_desc(64, 256, 512, 8, 2)
    fake = ctypes.c_void_p(0x1000)
    t = axm.MoeTensors(*([0x1000] * 18))
    assert lib.axm_moe_forward(ctypes.byref(d), ctypes.byref(t), None, 0, None) == axm.AXM_ERR_WORKSPACE
    assert lib.axm_moe_forward(ctypes.byref(d), ctypes.byref(t), ctypes.c_void_p(0x1010), 1 << 30,
                               None) == axm.AXM_ERR_WORKSPACE
    assert lib.axm_moe_forward(ctypes.byref(d), ctypes.byref(t), fake, 16, None) == axm.AXM_ERR_WORKSPACE


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour without a GPU")
def test_no_cpu_fallback(axm):
    """With valid arguments but no sm_100 device the layer fails loudly."""
    lib = axm.load()
    d = axm.make_desc(64, 256, 512, 8, 2)
    fake = ctypes.c_void_p(0x1000)
    t = axm.MoeTensors(*([0x1000] * 18))
    rc = lib.axm_moe_forward(ctypes.byref(d), ctypes.byref(t), fake, 1 << 30, None)
    assert rc == axm.AXM_ERR_DEVICE
    with pytest.raises(axm.AxmError):
        axm.check(rc)


def test_exact_intermediate_flag_doubles_the_h_region(axm):
    """AXM_FLAG_H_EXACT keeps the SwiGLU intermediate as two bf16 terms: T*k*F more elements."""
    d = axm.make_desc(4096, 2048, 5632, 8, 2)
    dx = axm.make_desc(4096, 2048, 5632, 8, 2, flags=axm.FLAG_RESIDUAL | axm.FLAG_H_EXACT)
    assert axm.workspace_bytes(dx) - axm.workspace_bytes(d) == 2 * 4096 * 2 * 5632


def test_adamw_argument_checks(axm):
    """Refusals happen before any CUDA call: null pointers, a step below 1, fp32 buffers off a
    16-byte boundary, and a bf16 working copy off an 8-byte boundary (the kernel stores four
    bf16 values at a time; a misaligned store would fault on the device)."""
    lib = axm.load()
    a = ctypes.c_void_p(0x10000)
    args = (64, 1e-3, 0.9, 0.95, 1e-8, 0.0, 1, None)
    assert lib.axm_moe_adamw_step(None, a, a, a, a, *args) == axm.AXM_ERR_ARGUMENT
    assert lib.axm_moe_adamw_step(a, a, a, a, a, 64, 1e-3, 0.9, 0.95, 1e-8, 0.0, 0, None) == axm.AXM_ERR_ARGUMENT
    assert lib.axm_moe_adamw_step(ctypes.c_void_p(0x10004), a, a, a, a, *args) == axm.AXM_ERR_ARGUMENT
    assert lib.axm_moe_adamw_step(a, a, a, a, ctypes.c_void_p(0x10002), *args) == axm.AXM_ERR_ARGUMENT
    assert b"8-byte aligned" in lib.axm_last_error()
    assert lib.axm_moe_adamw_step_engine(a, a, a, a, ctypes.c_void_p(0x10004), 64, 2048, 1e-3, 0.9, 0.95,
                                         1e-8, 0.0, 1, None) == axm.AXM_ERR_ARGUMENT
    assert lib.axm_moe_adamw_step(a, a, a, a, a, 0, 1e-3, 0.9, 0.95, 1e-8, 0.0, 1, None) == axm.AXM_OK


def test_ep_training_layout_checks(axm):
    """The sharded training step refuses, before any CUDA call, a layout that is not in the 64-row
    training form, a receive buffer without room for the padding, and a token count over all ranks
    below this rank's."""
    lib = axm.load()
    world, E, D, F, T, k = 2, 8, 256, 512, 64, 2
    slots = T * k

    def layout(cap, align):
        lo = axm.EpLayout()
        n = ctypes.c_size_t(0)
        assert lib.axm_ep_region_bytes(world, E, D, slots, cap, ctypes.byref(lo), ctypes.byref(n)) == axm.AXM_OK
        assert lo.row_align == 1           # packed rows unless the caller asks for the training form
        lo.rank, lo.row_align = 0, align
        return lo

    d = axm.make_desc(T, D, F, E, k)
    nb, zb = ctypes.c_size_t(0), ctypes.c_size_t(0)
    need = slots * world + 63 * (E // world)
    good = layout(need, 64)
    assert lib.axm_moe_ep_train_workspace_bytes(ctypes.byref(good), ctypes.byref(d), ctypes.byref(nb),
                                                ctypes.byref(zb)) == axm.AXM_OK
    assert nb.value > 5 * 2 * need * F and 0 < zb.value <= 512
    for bad in (layout(need, 1), layout(need - 1, 64)):
        assert lib.axm_moe_ep_train_workspace_bytes(ctypes.byref(bad), ctypes.byref(d), ctypes.byref(nb),
                                                    ctypes.byref(zb)) == axm.AXM_ERR_ARGUMENT
    plain = nb.value
    shared = axm.make_desc(T, D, F, E, k, num_shared=1)          # one replicated expert over this rank's tokens
    assert lib.axm_moe_ep_train_workspace_bytes(ctypes.byref(good), ctypes.byref(shared), ctypes.byref(nb),
                                                ctypes.byref(zb)) == axm.AXM_OK
    assert nb.value - plain >= 64 * (5 * 2 * F + (2 + 2 + 4) * D)    # its rows: x, g, u, h, dG, dU, dO, o
    t = axm.MoeTrain()
    assert lib.axm_moe_ep_forward_train(ctypes.byref(good), ctypes.byref(d), ctypes.byref(t), T - 1, None, 0, 1,
                                        None) == axm.AXM_ERR_ARGUMENT
    assert b"tokens_global" in lib.axm_last_error()
    # the backward pass wants an exchange region of its own
    good.peers = good.local_region = 0x10000
    t2 = axm.MoeTrain(*([0x1000] * 9), 0.01, *([0x1000] * 7), *([None] * 6))
    assert lib.axm_moe_ep_backward(ctypes.byref(good), ctypes.byref(good), ctypes.byref(d), ctypes.byref(t2), T * world,
                                   ctypes.c_void_p(0x100000), 1 << 40, 1, None) == axm.AXM_ERR_ARGUMENT
    assert b"region of its own" in lib.axm_last_error()


def test_host_batches_argument_checks(axm):
    lib = axm.load()
    d = axm.make_desc(64, 256, 512, 8, 2)
    a = 0x10000
    t = axm.MoeTensors(*([a] * 18))
    two = (ctypes.c_void_p * 2)(a, a)
    call = lambda tt, xs, n, dx=a, dout=a + 4096, ws=a, nbytes=1 << 40: lib.axm_moe_forward_host_batches(
        ctypes.byref(d), ctypes.byref(tt), xs, two, n, ctypes.c_void_p(dx), ctypes.c_void_p(dout),
        ctypes.c_void_p(ws), nbytes, None)
    assert call(t, two, 2) == axm.AXM_ERR_ARGUMENT and b"per-token outputs" in lib.axm_last_error()
    t.logits = t.topk_idx = t.topk_gate = t.offsets = t.row_src = t.slot_dst = t.y = None
    assert call(t, two, 65) == axm.AXM_ERR_ARGUMENT
    assert call(t, (ctypes.c_void_p * 2)(a, None), 2) == axm.AXM_ERR_ARGUMENT
    assert call(t, two, 2, dx=a, dout=a) == axm.AXM_ERR_ARGUMENT
    assert call(t, two, 2, nbytes=1024) == axm.AXM_ERR_WORKSPACE
    assert call(t, two, 0) == axm.AXM_OK          # nothing to do: no device needed
