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
    y_ref, out_ref = oracle.forward(x, w, idx, gate, h_bf16=True)
    helpers.assert_close_layer(r["ffn_output"], y_ref, what="d_ffn_output vs oracle")
    helpers.assert_close_out(r["final"], out_ref, y_ref, what="hidden_states vs oracle")
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
def test_dropin_against_reference_binary(axm, workloads, cuda_device):
    cfg = workloads.scaled(workloads.CONFIGS["C1"], tokens=256, d_model=32, d_ff=64)
    x, w, m_new, new = drive(axm.DROPIN_PATH, workloads, cuda_device, cfg, axm)
    _, _, m_ref, ref = drive(None, workloads, cuda_device, cfg, axm)
    same = (new["first"] == ref["first"]) & (new["second"] == ref["second"])
    assert int((~same).sum()) <= 1
    assert torch.equal(new["histogram"], ref["histogram"]) or int((~same).sum()) == 1
    helpers.assert_close_layer(new["ffn_output"][same], ref["ffn_output"][same],
                               what="d_ffn_output vs reference", allow_frac=1e-4, hard_factor=2.0)
    helpers.assert_close_out(new["final"][same], ref["final"][same], ref["ffn_output"][same],
                             what="hidden_states vs reference", allow_frac=1e-4, hard_factor=2.0)
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
