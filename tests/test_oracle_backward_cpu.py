"""The oracle's backward pass against torch autograd in float64 on the same
routing (an independent statement of the layer: softmax, fixed top-k selection,
renormalised gates, SwiGLU experts, residual, Switch-style auxiliary loss)."""
import numpy as np
import torch


def autograd_reference(x, w, idx, dY, alpha):
    x64 = x.double().requires_grad_(True)
    wr = w["router_w"].double().requires_grad_(True)
    wg = w["w_gate"].double().requires_grad_(True)
    wu = w["w_up"].double().requires_grad_(True)
    wd = w["w_down"].double().requires_grad_(True)
    T, E, k = x.shape[0], wr.shape[1], idx.shape[1]
    p = torch.softmax(x64 @ wr, -1)
    sel = torch.gather(p, 1, idx)
    gates = sel / (sel.sum(1, keepdim=True) + 1e-9)
    y = torch.zeros_like(x64)
    for t in range(T):
        for i in range(k):
            e = int(idx[t, i])
            h = torch.nn.functional.silu(x64[t] @ wg[e]) * (x64[t] @ wu[e])
            y[t] = y[t] + gates[t, i] * (h @ wd[e])
    out = x64 + y
    f = torch.bincount(idx.flatten(), minlength=E).double() / (T * k)
    aux = alpha * E * (f * p.mean(0)).sum()
    loss = (out * dY.double()).sum() + aux
    loss.backward()
    return {"dX": x64.grad, "dWr": wr.grad, "dWg": wg.grad, "dWu": wu.grad, "dWd": wd.grad}


def test_backward_matches_autograd(oracle, workloads):
    cfg = workloads.MoeConfig("bwd", tokens=24, d_model=32, num_experts=6, top_k=2, d_ff=48, seed=21)
    x, w = workloads.make_inputs(cfg)
    # larger weights than the benchmark's so that every gradient path is well above fp32 noise
    for n in ("w_gate", "w_up", "w_down"):
        w[n] = (w[n].float() * 8).bfloat16()
    w["router_w"] = w["router_w"] * 8
    z = oracle.router_logits(x, w["router_w"])
    idx, gates, probs, _, _ = oracle.route(z, cfg.top_k)
    dY = torch.randn(cfg.tokens, cfg.d_model, generator=torch.Generator().manual_seed(3))
    got = oracle.backward(x, w, idx, gates, probs, dY.numpy(), alpha=0.01)
    ref = autograd_reference(x, w, torch.from_numpy(idx).long(), dY, 0.01)
    for n in ("dX", "dWr", "dWg", "dWu", "dWd"):
        r = ref[n].numpy()
        err = np.abs(got[n] - r).max()
        assert err <= 2e-4 * max(1.0, np.abs(r).max()), f"{n}: max err {err}, max |ref| {np.abs(r).max()}"


def test_backward_bf16_rounding_points_stay_close(oracle, workloads):
    cfg = workloads.MoeConfig("bwd2", tokens=32, d_model=64, num_experts=4, top_k=2, d_ff=64, seed=22)
    x, w = workloads.make_inputs(cfg)
    z = oracle.router_logits(x, w["router_w"])
    idx, gates, probs, _, _ = oracle.route(z, cfg.top_k)
    dY = torch.randn(cfg.tokens, cfg.d_model, generator=torch.Generator().manual_seed(4)).numpy()
    a = oracle.backward(x, w, idx, gates, probs, dY, alpha=0.01)
    b = oracle.backward(x, w, idx, gates, probs, dY, alpha=0.01, act_bf16=True)
    for n in ("dX", "dWg", "dWu", "dWd", "dWr"):
        scale = np.abs(a[n]).max()
        assert np.abs(a[n] - b[n]).max() <= 2e-2 * scale + 1e-6, n


def test_golden_small_backward(oracle):
    """The committed gradients (tests/golden/make_golden.py) of the committed forward case are
    reproduced: the oracle's backward sums in a fixed order per output element, so only the
    last bits may differ between builds (1e-6 relative)."""
    import os
    import torch
    gdir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    f = np.load(os.path.join(gdir, "moe_small.npz"))
    b = np.load(os.path.join(gdir, "moe_small_bwd.npz"))
    x = torch.from_numpy(f["x_bits"].view(np.int16).copy()).view(torch.bfloat16)
    w = {n: torch.from_numpy(f[n + "_bits"].view(np.int16).copy()).view(torch.bfloat16)
         for n in ("w_gate", "w_up", "w_down")}
    w["router_w"] = torch.from_numpy(f["router_w"].copy())
    z = oracle.router_logits(x, w["router_w"])
    idx, gates, probs, _, _ = oracle.route(z, int(f["top_k"]))
    assert (idx == f["topk_idx"]).all()
    assert abs(oracle.aux_loss(probs, idx, float(b["aux_alpha"])) - float(b["aux_loss"])) < 1e-7
    got = oracle.backward(x, w, idx, gates, probs, b["d_y"], alpha=float(b["aux_alpha"]))
    for name in ("dX", "dWr", "dWg", "dWu", "dWd", "dgate", "dlogits"):
        ref = b[name]
        err = np.abs(got[name] - ref).max()
        assert err <= 1e-6 * max(1.0, float(np.abs(ref).max())), (name, err)
