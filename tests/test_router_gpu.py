"""Router parity on the GPU, through the C ABI.

Bit-exactness is asked of everything that follows the logits: the oracle is fed
the kernel's own fp32 logits and must choose the same experts.  The oracle's
expf is glibc's and the kernel's is CUDA's, which differ by an ulp now and then,
so gates are compared within 16 ulp (k probabilities, each an ulp or two off, enter
the renormalisation), and an index difference is accepted only on
a token the oracle flags as a near-tie (two candidate probabilities within 4 ulp).
"""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def ulp_diff(a, b):
    return np.abs(a.view(np.int32).astype(np.int64) - b.view(np.int32).astype(np.int64))


def check_routing(oracle, logits_np, idx, gate, bc, k):
    oi, og, _, oc, tie = oracle.route(logits_np, k)
    gi, gg = idx.cpu().numpy(), gate.cpu().numpy()
    mism = (gi != oi).any(axis=1)
    assert not (mism & (tie == 0)).any(), f"{int((mism & (tie == 0)).sum())} index mismatches that are not near-ties"
    same = ~mism
    assert ulp_diff(gg[same], og[same]).max(initial=0) <= 16
    counts = bc.sum(0).cpu().numpy()
    assert (counts == np.bincount(gi.ravel(), minlength=counts.shape[0])).all()
    return int(mism.sum())


CASES = [
    ("C1", None, {}), ("C2", None, {}), ("C3", 1024, {}), ("C4", 2048, {}), ("C5", 1024, {}),
    ("C2", 1, {}), ("C2", 295, {}), ("C2", 297, {}), ("C1", 1000, dict(num_experts=3, top_k=3)),
    ("C1", 512, dict(num_experts=256, top_k=8)), ("C1", 300, dict(d_model=72, num_experts=5, top_k=1)),
    ("C3", 300, dict(d_model=4104)),
]


@pytest.mark.parametrize("name,tokens,kw", CASES)
@pytest.mark.parametrize("router_bf16", [False, True])
@pytest.mark.parametrize("kernel", ["tensor-core", "cuda-core"])
def test_fused_router(axm, workloads, oracle, cuda_device, name, tokens, kw, router_bf16, kernel):
    """Both forms of the fused router: the streaming tcgen05 kernel (taken whenever the caller
    lends scratch and terms * E <= 256) and the CUDA-core kernel behind axm_moe_router."""
    if kernel == "cuda-core" and name == "C3":
        pytest.skip("the CUDA-core kernel is covered on the smaller shapes")
    cfg = workloads.scaled(workloads.CONFIGS[name], tokens=tokens, **kw)
    x, w = workloads.make_inputs(cfg, router_bf16=router_bf16)
    xd, wd = x.to(cuda_device), helpers.to_dev(w, cuda_device)
    desc = helpers.desc_for(axm, cfg, axm.ROUTER_BF16 if router_bf16 else axm.ROUTER_FP32)
    logits, idx, gate, bc = helpers.run_router(axm, desc, xd, wd["router_w"], wd.get("router_bias"),
                                               tensor_core=(kernel == "tensor-core"))
    torch.cuda.synchronize()
    z = oracle.router_logits(x, w["router_w"], w.get("router_bias"))
    zl = logits.cpu().numpy()
    # summation order differs by design (tree vs sequential): |dz| <= 1e-4 * max(1, |z|)
    assert (np.abs(zl - z) <= 1e-4 * np.maximum(1.0, np.abs(z))).all()
    check_routing(oracle, zl, idx, gate, bc, cfg.top_k)
    # the per-block counts are what the permute kernel places rows by: block b covers tokens
    # [b * T / 296, (b + 1) * T / 296)
    gi = idx.cpu().numpy()
    T = cfg.tokens
    bounds = [(b * T) // axm.ROUTE_BLOCKS for b in range(axm.ROUTE_BLOCKS + 1)]
    bcn = bc.cpu().numpy()
    for b in (0, 1, 147, 294, 295):
        want = np.bincount(gi[bounds[b]:bounds[b + 1]].ravel(), minlength=cfg.num_experts)
        assert (bcn[b] == want).all(), f"block {b}"
    # same tokens in a different batch: identical logits bits (the reduction order over
    # d_model does not depend on the batch), hence identical routing
    if T >= 300:
        half = workloads.scaled(cfg, tokens=T // 3)
        d2 = helpers.desc_for(axm, half, axm.ROUTER_BF16 if router_bf16 else axm.ROUTER_FP32)
        l2, i2, g2, _ = helpers.run_router(axm, d2, xd[T // 3:2 * (T // 3)].contiguous(), wd["router_w"],
                                           wd.get("router_bias"), tensor_core=(kernel == "tensor-core"))
        assert torch.equal(l2.view(torch.int32), logits[T // 3:2 * (T // 3)].view(torch.int32))
        assert torch.equal(i2, idx[T // 3:2 * (T // 3)])


def test_route_from_logits_ties_and_extremes(axm, workloads, oracle, cuda_device):
    """Exact ties, huge spreads and constant rows: lowest index must win."""
    rng = np.random.default_rng(7)
    T, E, k = 4096, 16, 2
    z = rng.standard_normal((T, E)).astype(np.float32)
    z[0:512] = np.round(z[0:512])                 # many exact ties
    z[512:600] = 0.0                              # all equal
    z[600:700] *= 50.0                            # saturating softmax, many zero probabilities
    z[700:800, 3] = z[700:800, 9]                 # a forced pair
    cfg = workloads.scaled(workloads.CONFIGS["C2"], tokens=T, num_experts=E, top_k=k)
    desc = helpers.desc_for(axm, cfg)
    idx, gate, bc = helpers.run_route_from_logits(axm, desc, torch.from_numpy(z).to(cuda_device))
    torch.cuda.synchronize()
    oi, og, _, _, tie = oracle.route(z, k)
    gi = idx.cpu().numpy()
    # exact ties resolve identically on both sides; only rows where distinct
    # logits give nearly equal probabilities may differ
    exact_tie_rows = np.zeros(T, dtype=bool)
    exact_tie_rows[0:600] = True
    assert (gi[512:600] == np.array([0, 1])).all()
    mism = (gi != oi).any(axis=1)
    assert not (mism & (tie == 0)).any()
    assert ulp_diff(gate.cpu().numpy()[~mism], og[~mism]).max() <= 16
    assert int(bc.sum()) == T * k


def test_route_from_logits_top6_of_64(axm, workloads, oracle, cuda_device):
    cfg = workloads.scaled(workloads.CONFIGS["C4"], tokens=8192)
    x, w = workloads.make_inputs(cfg)
    z = oracle.router_logits(x, w["router_w"], w["router_bias"])
    desc = helpers.desc_for(axm, cfg)
    idx, gate, bc = helpers.run_route_from_logits(axm, desc, torch.from_numpy(z).to(cuda_device))
    torch.cuda.synchronize()
    check_routing(oracle, z, idx, gate, bc, cfg.top_k)
    hist = bc.sum(0).cpu().numpy()
    assert hist.max() > 4 * hist.mean()          # the Zipf bias really skews the load
