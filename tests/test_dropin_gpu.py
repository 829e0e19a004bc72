"""The drop-in library (the reference's three symbols over this layer) driven the
way the reference's host wrapper drives its own: opaque struct blobs, in-place
hidden states, lazily allocated published buffers, accumulating histogram.
Compared with the oracle, and with the reference binary where it is built."""
import numpy as np
import pytest
import torch

import helpers
import reference_binding

pytestmark = pytest.mark.gpu


def drive(lib_path, workloads, cuda_device, cfg, axm):
    x, w = workloads.make_inputs(cfg, router_bf16=True)
    wd = helpers.to_dev(w, cuda_device)
    m = reference_binding.ReferenceMoe(lib_path)
    m.set_weights(wd["router_w"], wd["w_gate"], wd["w_up"], wd["w_down"])
    hidden = x.to(cuda_device).clone()
    assert m.forward(hidden, cfg.d_ff)
    r = m.outputs(cfg.tokens, cfg.d_model)
    r["final"] = hidden
    return x, w, m, r


@pytest.mark.parametrize("kw", [dict(tokens=256, d_model=32, d_ff=64), dict(), dict(tokens=2048, d_model=2048, d_ff=5632)])
def test_dropin_against_oracle(axm, workloads, oracle, cuda_device, kw):
    cfg = workloads.scaled(workloads.CONFIGS["C1"], **kw)
    x, w, m, r = drive(axm.DROPIN_PATH, workloads, cuda_device, cfg, axm)
    T, E = cfg.tokens, cfg.num_experts
    z = oracle.router_logits(x, w["router_w"])
    zl = r["logits"].cpu().numpy()
    assert (np.abs(zl - z) <= 1e-4 * np.maximum(1.0, np.abs(z))).all()
    oi, og, _, oc, tie = oracle.route(zl, 2)
    idx = torch.stack([r["first"], r["second"]], 1).cpu().numpy()
    gate = torch.stack([r["w_first"], r["w_second"]], 1).cpu().numpy()
    mism = (oi != idx).any(axis=1)
    assert not (mism & (tie == 0)).any()
    assert (r["histogram"].cpu().numpy() == np.bincount(idx.ravel(), minlength=E)).all()
    y_ref, out_ref = oracle.forward(x, w, idx, gate)   # fp32 intermediate, like the engine
    helpers.assert_close_layer(r["ffn_output"], y_ref, what="d_ffn_output vs oracle")
    helpers.assert_close_out(r["final"], out_ref, y_ref, what="hidden_states vs oracle", out_step=2.0 ** -8)
    assert torch.equal(r["final"], r["residual_out"])
    # second call: histogram accumulates; download and reset behave like the reference's
    hidden = x.to(cuda_device).clone()
    assert m.forward(hidden, cfg.d_ff)
    ok, twice = m.download_counts()
    assert ok and (np.array(twice) == 2 * r["histogram"].cpu().numpy()).all()
    assert m.reset_histogram()
    ok, zero = m.download_counts()
    assert ok and not any(zero)
    assert torch.equal(hidden, r["final"])


@pytest.mark.skipif(not reference_binding.available(),
                    reason="parity unpinned: oracle/_ref not built (oracle/build_ref.sh)")
@pytest.mark.parametrize("name,kw", [("C1", dict(tokens=256, d_model=32, d_ff=64)), ("C1", dict()),
                                     ("C2", dict(tokens=512)), ("C2", dict())])   # the last: C2 at full size
def test_dropin_against_reference_binary(axm, workloads, cuda_device, name, kw):
    cfg = workloads.scaled(workloads.CONFIGS[name], **kw)
    x, w, m_new, new = drive(axm.DROPIN_PATH, workloads, cuda_device, cfg, axm)
    _, _, m_ref, ref = drive(None, workloads, cuda_device, cfg, axm)
    same = (new["first"] == ref["first"]) & (new["second"] == ref["second"])
    assert int((~same).sum()) <= max(1, cfg.tokens // 500)
    assert torch.equal(new["histogram"], ref["histogram"]) or int((~same).sum()) >= 1
    # the drop-in runs the two-term SwiGLU intermediate: every element inside the bound
    helpers.assert_close_layer(new["ffn_output"][same], ref["ffn_output"][same],
                               what="d_ffn_output vs reference")
    helpers.assert_close_out(new["final"][same], ref["final"][same], ref["ffn_output"][same],
                             what="hidden_states vs reference", out_step=2.0 ** -8)
    g_new = torch.stack([new["w_first"], new["w_second"]], 1)[same]
    g_ref = torch.stack([ref["w_first"], ref["w_second"]], 1)[same]
    assert float((g_new - g_ref).abs().max()) <= 1e-5


def test_dropin_refuses_what_it_cannot_do(axm, workloads, cuda_device):
    cfg = workloads.scaled(workloads.CONFIGS["C1"], tokens=64, d_model=64, d_ff=64, num_experts=32)
    x, w = workloads.make_inputs(cfg, router_bf16=True)
    wd = helpers.to_dev(w, cuda_device)
    m = reference_binding.ReferenceMoe(axm.DROPIN_PATH)
    m.set_weights(wd["router_w"], wd["w_gate"], wd["w_up"], wd["w_down"])
    hidden = x.to(cuda_device).clone()
    assert m.forward(hidden, cfg.d_ff) is False      # more than 16 experts
    assert torch.equal(hidden.cpu(), x)


def test_engine_moe_test_through_the_dropin(axm, cuda_device):
    """The engine's own MoE test (core/test/test_ai.cpp:944-1015) against the drop-in library:
    same shape and checks (histogram of 8 entries summing to 2 * 256, no dead expert,
    AI::verify_routing_balance's ratio below 3, finite in-place output)."""
    from test_oracle_cpu import engine_test_inputs, routing_balance_ok
    x, w = engine_test_inputs()
    wd = helpers.to_dev(w, cuda_device)
    m = reference_binding.ReferenceMoe(axm.DROPIN_PATH)
    m.set_weights(wd["router_w"], wd["w_gate"], wd["w_up"], wd["w_down"])
    hidden = x.to(cuda_device).clone()
    assert m.forward(hidden, 64)
    ok, hist = m.download_counts()
    assert ok and len(hist) == 8
    assert sum(hist) == 512 and min(hist) > 0
    assert routing_balance_ok(hist, 256, 8)
    assert torch.isfinite(hidden.float()).all()
    assert not torch.equal(hidden, x.to(cuda_device)), "the hidden states are updated in place"


def _free_published(m):
    """What the engine's free_gpu_activations does for the MoE fields: free and null them."""
    import ctypes
    import struct
    m.cudart.cudaFree.argtypes = [ctypes.c_void_p]
    for name in ("a.d_router_logits", "a.d_expert_first", "a.d_expert_second", "a.d_weight_first",
                 "a.d_weight_second", "a.d_expert_histogram", "a.d_ffn_output", "a.d_residual_out"):
        p = struct.unpack_from("Q", m.acts, m.off[name])[0]
        if p:
            assert m.cudart.cudaFree(p) == 0
        struct.pack_into("Q", m.acts, m.off[name], 0)


def test_dropin_state_is_per_activation_struct_and_checks_sizes(axm, workloads, cuda_device):
    """Two activation structs in one process keep separate scratch; a call with more tokens
    than the published buffers were sized for is refused (the engine would write past them,
    core/src/CUDA/kernel/moe_router.cu:223-250) and works again once the caller has freed them."""
    small = workloads.scaled(workloads.CONFIGS["C1"], tokens=64)
    big = workloads.scaled(workloads.CONFIGS["C1"], tokens=320)
    xs, w = workloads.make_inputs(small, router_bf16=True)
    xb, _ = workloads.make_inputs(big, router_bf16=True)
    wd = helpers.to_dev(w, cuda_device)
    m1 = reference_binding.ReferenceMoe(axm.DROPIN_PATH)
    m2 = reference_binding.ReferenceMoe(axm.DROPIN_PATH)
    for m in (m1, m2):
        m.set_weights(wd["router_w"], wd["w_gate"], wd["w_up"], wd["w_down"])

    def expect(x):
        layer = axm.MoeLayer(wd, x.shape[0], 2, h_exact=True)
        out, _ = layer.forward(x.to(cuda_device))
        return out.clone()

    h1 = xs.to(cuda_device).clone()
    h2 = xb.to(cuda_device).clone()
    assert m1.forward(h1, small.d_ff) and m2.forward(h2, big.d_ff)
    assert torch.equal(h1, expect(xs)) and torch.equal(h2, expect(xb))
    # interleaved again: neither call disturbed the other's state
    h1b = xs.to(cuda_device).clone()
    assert m1.forward(h1b, small.d_ff)
    assert torch.equal(h1b, h1)
    # m1's buffers hold 64 tokens: 320 do not fit
    h_grow = xb.to(cuda_device).clone()
    assert m1.forward(h_grow, big.d_ff) is False
    assert torch.equal(h_grow.cpu(), xb), "a refused call must not touch the hidden states"
    # fewer tokens fit
    h_less = xs[:32].to(cuda_device).clone()
    assert m1.forward(h_less, small.d_ff)
    assert torch.equal(h_less, expect(xs[:32]))
    _free_published(m1)
    assert m1.forward(h_grow, big.d_ff)
    assert torch.equal(h_grow, h2)
    ok, hist = m1.download_counts()
    assert ok and sum(hist) == 2 * big.tokens, "a freshly allocated histogram starts at zero"


def test_dropin_on_two_devices(axm, workloads):
    """One process, two GPUs: the scratch of one device is never handed to the other."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    cfg = workloads.scaled(workloads.CONFIGS["C1"], tokens=128)
    x, w = workloads.make_inputs(cfg, router_bf16=True)
    outs = []
    for dev in (torch.device("cuda:0"), torch.device("cuda:1")):
        with torch.cuda.device(dev):
            wd = helpers.to_dev(w, dev)
            m = reference_binding.ReferenceMoe(axm.DROPIN_PATH)
            m.set_weights(wd["router_w"], wd["w_gate"], wd["w_up"], wd["w_down"])
            hidden = x.to(dev).clone()
            assert m.forward(hidden, cfg.d_ff)
            torch.cuda.synchronize(dev)
            outs.append(hidden.cpu())
    assert torch.equal(outs[0], outs[1])
