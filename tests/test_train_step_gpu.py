"""Training step (forward + backward + auxiliary loss) through the C ABI against the
CPU oracle's backward pass on the same routing.  Floating point; every gradient
tensor is checked element-wise with |err| <= 2e-2 * |ref| + 1e-2 * max|ref|
against the oracle with fp32 intermediates, and with half that bound against the
oracle rounding g, u, h, dO, dG, dU to bf16 where this pipeline stores them."""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def close(got, ref, what, factor=1.0):
    g = got.float().cpu().numpy() if torch.is_tensor(got) else got
    err = np.abs(g - ref)
    bound = factor * (2e-2 * np.abs(ref) + 1e-2 * np.abs(ref).max())
    bad = err > bound
    assert not bad.any(), (f"{what}: {int(bad.sum())} of {bad.size} outside the bound, max err "
                           f"{err.max():.4g}, max |ref| {np.abs(ref).max():.4g}")


@pytest.mark.parametrize("name,kw", [
    ("C1", dict(tokens=96, num_experts=8)),
    ("C5", dict(tokens=256, d_model=512, d_ff=1024)),
    ("C5", dict(tokens=192)),                       # C5's d_model 2048, d_ff 4096, E 16
    ("C1", dict(tokens=70, d_model=72, d_ff=200, num_experts=5, top_k=3)),
])
@pytest.mark.parametrize("router_bf16", [False, True])
def test_train_step_matches_oracle(axm, workloads, oracle, cuda_device, name, kw, router_bf16):
    cfg = workloads.scaled(workloads.CONFIGS[name], **kw)
    if router_bf16 and cfg.d_model > 1024:
        pytest.skip("bf16 router covered on the smaller shapes")
    alpha = 0.01
    x, w = workloads.make_inputs(cfg, router_bf16=router_bf16)
    dY = torch.randn(cfg.tokens, cfg.d_model, generator=torch.Generator().manual_seed(cfg.seed + 100))
    wd = helpers.to_dev(w, cuda_device)
    layer = axm.MoeTrainLayer(wd, cfg.tokens, cfg.top_k, aux_alpha=alpha)
    xd, dYd = x.to(cuda_device), dY.to(cuda_device)
    out, aux, grads = layer.step(xd, dYd)
    torch.cuda.synchronize()

    # the routing the GPU used, recovered through the oracle from the GPU's logits
    z = oracle.router_logits(x, w["router_w"])
    desc = helpers.desc_for(axm, cfg, axm.ROUTER_BF16 if router_bf16 else axm.ROUTER_FP32)
    logits, idx_d, gate_d, _ = helpers.run_router(axm, desc, xd, wd["router_w"])
    zl = logits.cpu().numpy()
    assert (np.abs(zl - z) <= 1e-4 * np.maximum(1.0, np.abs(z))).all()
    idx, gates = idx_d.cpu().numpy(), gate_d.cpu().numpy()
    _, _, probs, counts, _ = oracle.route(zl, cfg.top_k)
    assert (layer.histogram.cpu().numpy() == np.bincount(idx.ravel(), minlength=cfg.num_experts)).all()

    # forward output and auxiliary loss
    y_ref, out_ref = oracle.forward(x, w, idx, gates, h_bf16=True)
    helpers.assert_close_out(out, out_ref, y_ref, what="training forward out")
    aux_ref = oracle.aux_loss(probs, idx, alpha)
    assert abs(float(aux.item()) - aux_ref) <= 1e-5 * max(1.0, abs(aux_ref))

    names = {"d_x": "dX", "d_router_w": "dWr", "d_w_gate": "dWg", "d_w_up": "dWu", "d_w_down": "dWd"}
    ref32 = oracle.backward(x, w, idx, gates, probs, dY.numpy(), alpha=alpha)
    refbf = oracle.backward(x, w, idx, gates, probs, dY.numpy(), alpha=alpha, act_bf16=True)
    for gname, oname in names.items():
        got = grads[gname]
        if gname == "d_x":   # compare the part that went through the layer, not the residual copy
            got = got.cpu() - dY
            r32, rbf = ref32[oname] - dY.numpy(), refbf[oname] - dY.numpy()
        else:
            r32, rbf = ref32[oname], refbf[oname]
        close(got, r32, f"{oname} vs oracle (fp32 intermediates)")
        close(got, rbf, f"{oname} vs oracle (bf16 rounding points)", factor=0.5)


def test_train_step_is_deterministic_and_matches_inference_forward(axm, workloads, cuda_device):
    cfg = workloads.scaled(workloads.CONFIGS["C5"], tokens=1024)
    x, w = workloads.make_inputs(cfg, device=cuda_device)
    dY = torch.randn(cfg.tokens, cfg.d_model, device=cuda_device)
    layer = axm.MoeTrainLayer(w, cfg.tokens, cfg.top_k)
    out1, aux1, g1 = layer.step(x, dY)
    keep = {k: v.clone() for k, v in g1.items()}
    out1 = out1.clone()
    out2, aux2, g2 = layer.step(x, dY)
    assert torch.equal(out1, out2)
    for k in keep:
        assert torch.equal(keep[k], g2[k]), k
    inf = axm.MoeLayer(w, cfg.tokens, cfg.top_k)
    out3, _ = inf.forward(x)
    assert torch.equal(out3, out1)          # padded layout, same arithmetic per row
    assert torch.isfinite(keep["d_x"]).all() and torch.isfinite(keep["d_w_down"]).all()


def test_full_size_c5_step_matches_oracle(axm, workloads, oracle, cuda_device):
    """The training step at the full size of the forward + backward workload (8192 tokens,
    d_model 2048, 16 experts of d_ff 4096, top-2: about 1024 rows per expert, so several
    m-tiles per expert, 16 k-blocks per weight-gradient tile, CTA-pair kernels) against the
    CPU oracle's backward on the same routing: every element of dX, dWr, dWg, dWu, dWd.
    The oracle needs about a minute of host time for this size."""
    cfg = workloads.CONFIGS["C5"]
    alpha = cfg.aux_alpha
    x, w = workloads.make_inputs(cfg)
    dY = torch.randn(cfg.tokens, cfg.d_model, generator=torch.Generator().manual_seed(cfg.seed + 100))
    wd = helpers.to_dev(w, cuda_device)
    layer = axm.MoeTrainLayer(wd, cfg.tokens, cfg.top_k, aux_alpha=alpha)
    xd, dYd = x.to(cuda_device), dY.to(cuda_device)
    out, aux, grads = layer.step(xd, dYd)
    torch.cuda.synchronize()
    assert int(layer.workspace[:4].view(torch.int32).item()) == 0, "a GEMM kernel reported a timed-out wait"

    desc = helpers.desc_for(axm, cfg)
    logits, idx_d, gate_d, _ = helpers.run_router(axm, desc, xd, wd["router_w"])
    zl = logits.cpu().numpy()
    idx, gates = idx_d.cpu().numpy(), gate_d.cpu().numpy()
    _, _, probs, _, _ = oracle.route(zl, cfg.top_k)
    hist = np.bincount(idx.ravel(), minlength=cfg.num_experts)
    assert (layer.histogram.cpu().numpy() == hist).all()
    assert hist.max() > 2 * 128 and hist.min() > 128, "every expert spans several m-tiles at this size"
    aux_ref = oracle.aux_loss(probs, idx, alpha)
    assert abs(float(aux.item()) - aux_ref) <= 1e-5 * max(1.0, abs(aux_ref))

    ref = oracle.backward(x, w, idx, gates, probs, dY.numpy(), alpha=alpha)
    close(grads["d_x"].cpu() - dY, ref["dX"] - dY.numpy(), "dX at full size")
    close(grads["d_router_w"], ref["dWr"], "dWr at full size")
    for gname, oname in (("d_w_gate", "dWg"), ("d_w_up", "dWu"), ("d_w_down", "dWd")):
        for e in range(cfg.num_experts):    # one expert at a time keeps the host copies small
            close(grads[gname][e], ref[oname][e], f"{oname}[{e}] at full size")
    # forward output of the same step on a token slice
    lo, hi = 4000, 4064
    y_ref, out_ref = oracle.forward(x, w, idx, gates, h_bf16=True, tok_range=(lo, hi))
    helpers.assert_close_out(out[lo:hi], out_ref[lo:hi], y_ref[lo:hi], what="training forward out (slice)")


def test_router_bias_is_trained(axm, workloads, oracle, cuda_device):
    """With a router bias (added to the logits before the softmax) the backward pass also
    returns its gradient, the sum over tokens of the logit gradients; the other gradients see
    the bias through the routing and the probabilities."""
    cfg = workloads.scaled(workloads.CONFIGS["C4"], tokens=200, d_model=128, d_ff=256, num_experts=16, top_k=3,
                           num_shared=0)
    alpha = 0.01
    x, w = workloads.make_inputs(cfg)
    assert w.get("router_bias") is not None
    dY = torch.randn(cfg.tokens, cfg.d_model, generator=torch.Generator().manual_seed(11))
    wd = helpers.to_dev(w, cuda_device)
    layer = axm.MoeTrainLayer(wd, cfg.tokens, cfg.top_k, aux_alpha=alpha)
    xd, dYd = x.to(cuda_device), dY.to(cuda_device)
    out, aux, grads = layer.step(xd, dYd)
    torch.cuda.synchronize()
    desc = axm.make_desc(cfg.tokens, cfg.d_model, cfg.d_ff, cfg.num_experts, cfg.top_k)
    logits, idx_d, gate_d, _ = helpers.run_router(axm, desc, xd, wd["router_w"], wd["router_bias"])
    zl = logits.cpu().numpy()
    idx, gates = idx_d.cpu().numpy(), gate_d.cpu().numpy()
    _, _, probs, _, _ = oracle.route(zl, cfg.top_k)
    ref = oracle.backward(x, w, idx, gates, probs, dY.numpy(), alpha=alpha)
    close(grads["d_router_bias"], ref["dlogits"].sum(0), "d_router_bias")
    close(grads["d_router_w"], ref["dWr"], "dWr with a router bias")
    close(grads["d_x"].cpu() - dY, ref["dX"] - dY.numpy(), "dX with a router bias")


@pytest.mark.parametrize("tokens,shared", [(200, 2), (128, 1)])
def test_train_step_with_shared_experts(axm, workloads, oracle, cuda_device, tokens, shared):
    """Shared experts (every token, weight 1) in the training step.  The oracle's backward covers
    routed experts; a shared expert is the same arithmetic with every token routed to it at gate 1,
    so the reference is the routed backward plus, per shared expert, the backward of a one-expert
    top-1 layer with unit gates and probabilities (its router gradient vanishes identically)."""
    cfg = workloads.scaled(workloads.CONFIGS["C4"], tokens=tokens, d_model=128, d_ff=256, num_experts=16, top_k=3,
                           num_shared=shared)
    alpha = 0.01
    x, w = workloads.make_inputs(cfg)
    S = cfg.num_shared
    assert w["shared_gate"].shape[0] == S
    dY = torch.randn(cfg.tokens, cfg.d_model, generator=torch.Generator().manual_seed(12))
    wd = helpers.to_dev(w, cuda_device)
    layer = axm.MoeTrainLayer(wd, cfg.tokens, cfg.top_k, aux_alpha=alpha)
    xd, dYd = x.to(cuda_device), dY.to(cuda_device)
    out, aux, grads = layer.step(xd, dYd)
    keep = {k: v.clone() for k, v in grads.items()}
    out2, _, grads2 = layer.step(xd, dYd)           # buffers reused; deterministic
    torch.cuda.synchronize()
    assert int(layer.workspace[:4].view(torch.int32).item()) == 0
    for k_, v in keep.items():
        assert torch.equal(v, grads2[k_]), k_

    desc = axm.make_desc(cfg.tokens, cfg.d_model, cfg.d_ff, cfg.num_experts, cfg.top_k)
    logits, idx_d, gate_d, _ = helpers.run_router(axm, desc, xd, wd["router_w"], wd["router_bias"])
    zl = logits.cpu().numpy()
    idx, gates = idx_d.cpu().numpy(), gate_d.cpu().numpy()
    _, _, probs, _, _ = oracle.route(zl, cfg.top_k)

    # forward: the oracle applies the shared experts itself; the inference layer gives the same bytes
    y_ref, out_ref = oracle.forward(x, w, idx, gates, h_bf16=True)
    helpers.assert_close_out(out, out_ref, y_ref, what="training forward out with shared experts")
    inf = axm.MoeLayer(wd, cfg.tokens, cfg.top_k)
    out_inf, _ = inf.forward(xd)
    assert torch.equal(out_inf, out2)

    routed = {k_: v for k_, v in w.items() if not k_.startswith("shared_")}
    ones = np.ones((cfg.tokens, 1), np.float32)
    zero_idx = np.zeros((cfg.tokens, 1), np.int32)
    for act_bf16, factor in ((False, 1.0), (True, 0.5)):
        ref = oracle.backward(x, routed, idx, gates, probs, dY.numpy(), alpha=alpha, act_bf16=act_bf16)
        dx_ref = ref["dX"] - dY.numpy()
        for s in range(S):
            ws = {"router_w": torch.zeros(cfg.d_model, 1), "w_gate": w["shared_gate"][s:s + 1],
                  "w_up": w["shared_up"][s:s + 1], "w_down": w["shared_down"][s:s + 1]}
            rs = oracle.backward(x, ws, zero_idx, ones, ones, dY.numpy(), alpha=0.0, act_bf16=act_bf16)
            dx_ref = dx_ref + (rs["dX"] - dY.numpy())
            close(grads["d_shared_gate"][s], rs["dWg"][0], f"d_shared_gate[{s}] (bf16 points {act_bf16})", factor)
            close(grads["d_shared_up"][s], rs["dWu"][0], f"d_shared_up[{s}] (bf16 points {act_bf16})", factor)
            close(grads["d_shared_down"][s], rs["dWd"][0], f"d_shared_down[{s}] (bf16 points {act_bf16})", factor)
        close(grads["d_x"].cpu() - dY, dx_ref, f"dX with shared experts (bf16 points {act_bf16})", factor)
        for gname, oname in (("d_router_w", "dWr"), ("d_w_gate", "dWg"), ("d_w_up", "dWu"), ("d_w_down", "dWd")):
            close(grads[gname], ref[oname], f"{oname} beside shared experts (bf16 points {act_bf16})", factor)
