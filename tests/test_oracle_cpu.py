"""CPU checks of the oracle itself: against an independent torch fp32 statement
of the layer, against its committed golden vectors, and its routing rules."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_router_matches_torch(oracle, workloads):
    cfg = workloads.CONFIGS["C1"]
    x, w = workloads.make_inputs(cfg)
    z = oracle.router_logits(x, w["router_w"])
    zt = (x.double() @ w["router_w"].double()).numpy()
    assert np.abs(z - zt).max() <= 1e-5
    idx, gates, probs, counts, tie = oracle.route(z, cfg.top_k)
    p = torch.softmax(torch.from_numpy(z), -1)
    tv, ti = torch.topk(p, cfg.top_k, dim=-1)
    assert (ti.numpy() == idx).all()
    assert np.abs(gates - (tv / tv.sum(-1, keepdim=True)).numpy()).max() < 1e-6
    assert counts.sum() == cfg.tokens * cfg.top_k
    assert (np.bincount(idx.ravel(), minlength=cfg.num_experts) == counts).all()


def test_lowest_index_wins_ties(oracle):
    z = np.zeros((5, 6), dtype=np.float32)
    z[1, [4, 2]] = 1.0          # two equal maxima -> 2 first, then 4
    z[2, 5] = 3.0               # one maximum, the rest tie -> 5, then 0
    z[3] = [0.5, 0.5, 0.5, 0.25, 0.5, 0.5]
    z[4] = [-1, -1, -2, -1, -3, -1]
    idx, gates, _, counts, tie = oracle.route(z, 3)
    assert idx[0].tolist() == [0, 1, 2]
    assert idx[1].tolist() == [2, 4, 0]
    assert idx[2].tolist() == [5, 0, 1]
    assert idx[3].tolist() == [0, 1, 2]
    assert idx[4].tolist() == [0, 1, 3]
    assert tie.all()            # every row has exact ties among its candidates
    assert np.allclose(gates.sum(1), 1.0, atol=1e-6)
    assert counts.sum() == 15


def test_histogram_accumulates(oracle):
    z = np.random.default_rng(0).standard_normal((100, 8)).astype(np.float32)
    _, _, _, counts, _ = oracle.route(z, 2)
    _, _, _, counts2, _ = oracle.route(z, 2, counts=counts.copy())
    assert (counts2 == 2 * counts).all()


def test_permutation_rule(oracle):
    rng = np.random.default_rng(1)
    T, E, k = 333, 7, 3
    idx = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    offsets, row_src, slot_dst = oracle.permutation(idx, E)
    assert offsets[0] == 0 and offsets[-1] == T * k
    assert sorted(row_src.tolist()) == list(range(T * k))
    assert (row_src[slot_dst] == np.arange(T * k)).all()
    flat = idx.ravel()
    for e in range(E):
        rows = row_src[offsets[e]:offsets[e + 1]]
        assert (flat[rows] == e).all()
        assert (np.diff(rows) > 0).all()      # ordered by token, then slot


def test_permutation_with_empty_experts(oracle):
    idx = np.array([[3, 1], [3, 1], [1, 3]], dtype=np.int32)
    offsets, row_src, slot_dst = oracle.permutation(idx, 5)
    assert offsets.tolist() == [0, 0, 3, 3, 6, 6]
    assert row_src.tolist() == [1, 3, 4, 0, 2, 5]


def test_forward_matches_torch(oracle, workloads):
    cfg = workloads.scaled(workloads.CONFIGS["C1"], tokens=24)
    x, w = workloads.make_inputs(cfg)
    z = oracle.router_logits(x, w["router_w"])
    idx, gates, _, _, _ = oracle.route(z, cfg.top_k)
    y, out = oracle.forward(x, w, idx, gates)
    xf = x.double()
    yref = torch.zeros_like(xf)
    for t in range(cfg.tokens):
        for i in range(cfg.top_k):
            e = int(idx[t, i])
            g = xf[t] @ w["w_gate"][e].double()
            u = xf[t] @ w["w_up"][e].double()
            yref[t] += float(gates[t, i]) * ((torch.nn.functional.silu(g) * u) @ w["w_down"][e].double())
    assert (y.double() - yref).abs().max() < 2e-3 * max(1.0, float(yref.abs().max()))
    outref = (x.float() + y.float()).bfloat16()
    assert torch.equal(out, outref)
    # rounding the intermediates like a two-GEMM bf16 pipeline stays well inside the tolerance
    y2, _ = oracle.forward(x, w, idx, gates, h_bf16=True, o_bf16=True)
    assert (y2.float() - y.float()).abs().max() <= 1e-2


def test_forward_shared_experts_and_token_range(oracle, workloads):
    cfg = workloads.scaled(workloads.CONFIGS["C4"], tokens=16, d_model=64, d_ff=96, num_experts=8,
                           top_k=3)
    x, w = workloads.make_inputs(cfg)
    z = oracle.router_logits(x, w["router_w"], w["router_bias"])
    idx, gates, _, _, _ = oracle.route(z, cfg.top_k)
    y, out = oracle.forward(x, w, idx, gates)
    xf = x.double()
    yref = torch.zeros_like(xf)
    for t in range(cfg.tokens):
        for i in range(cfg.top_k):
            e = int(idx[t, i])
            h = torch.nn.functional.silu(xf[t] @ w["w_gate"][e].double()) * (xf[t] @ w["w_up"][e].double())
            yref[t] += float(gates[t, i]) * (h @ w["w_down"][e].double())
        for s in range(cfg.num_shared):
            h = torch.nn.functional.silu(xf[t] @ w["shared_gate"][s].double()) * (xf[t] @ w["shared_up"][s].double())
            yref[t] += h @ w["shared_down"][s].double()
    assert (y.double() - yref).abs().max() < 2e-3 * max(1.0, float(yref.abs().max()))
    y_part, _ = oracle.forward(x, w, idx, gates, tok_range=(4, 9))
    assert torch.equal(y_part[4:9], y[4:9])
    assert float(y_part[:4].abs().max()) == 0.0 and float(y_part[9:].abs().max()) == 0.0


def test_aux_loss(oracle):
    rng = np.random.default_rng(2)
    z = rng.standard_normal((64, 8)).astype(np.float32)
    idx, _, probs, counts, _ = oracle.route(z, 2)
    f = counts / counts.sum()
    P = probs.mean(0)
    want = 0.01 * 8 * float((f * P).sum())
    assert abs(oracle.aux_loss(probs, idx, 0.01) - want) < 1e-7


def test_golden_small(oracle):
    """The committed vectors (tests/golden/make_golden.py) are reproduced bit for bit."""
    g = np.load(os.path.join(GOLDEN, "moe_small.npz"))
    x = torch.from_numpy(g["x_bits"].view(np.int16).copy()).view(torch.bfloat16)
    w = {n: torch.from_numpy(g[n + "_bits"].view(np.int16).copy()).view(torch.bfloat16)
         for n in ("w_gate", "w_up", "w_down")}
    w["router_w"] = torch.from_numpy(g["router_w"].copy())
    z = oracle.router_logits(x, w["router_w"])
    assert (z == g["logits"]).all()
    idx, gates, _, counts, _ = oracle.route(z, int(g["top_k"]))
    assert (idx == g["topk_idx"]).all()
    assert (gates.view(np.int32) == g["topk_gate"].view(np.int32)).all()
    assert (counts == g["histogram"]).all()
    offsets, row_src, slot_dst = oracle.permutation(idx, w["router_w"].shape[1])
    assert (offsets == g["offsets"]).all() and (row_src == g["row_src"]).all()
    y, out = oracle.forward(x, w, idx, gates)
    assert (out.view(torch.int16).numpy().view(np.uint16) == g["out_bits"]).all()
    assert (y.view(torch.int16).numpy().view(np.uint16) == g["y_bits"]).all()


def engine_test_inputs():
    """The shape of the engine's own MoE test (core/test/test_ai.cpp:944-1015): 256 tokens drawn
    uniformly from (-1, 1) in a 32-dim space, 8 experts of width 64, top-2, weights uniform in
    +-1/sqrt(D) drawn in the order router, gate, up, down as allocate_expert_weights does
    (core/src/CUDA/util/memory_allocation.cu:543-569).  Seeded Mersenne twisters as there; the draws
    themselves differ from libstdc++'s distributions, so only the structural checks carry over."""
    T, D, F, E = 256, 32, 64, 8
    x = torch.from_numpy(np.random.RandomState(1337).uniform(-1.0, 1.0, (T, D)).astype(np.float32)).bfloat16()
    rs = np.random.RandomState(1337)
    lim = 1.0 / np.sqrt(D)
    draw = lambda *shape: torch.from_numpy(rs.uniform(-lim, lim, shape).astype(np.float32)).bfloat16()
    w = {"router_w": draw(D, E), "w_gate": draw(E, D, F), "w_up": draw(E, D, F), "w_down": draw(E, F, D)}
    return x, w


def routing_balance_ok(hist, tokens, experts):
    """The engine's acceptance rule for a routing histogram (AI::verify_routing_balance,
    core/src/ai.cpp:625-656): every selection counted, no dead expert, hottest expert below
    three times the mean load."""
    hist = [int(c) for c in hist]
    if len(hist) != experts or tokens == 0 or sum(hist) != 2 * tokens or min(hist) <= 0:
        return False
    return max(hist) / (sum(hist) / experts) < 3.0


def test_engine_moe_test_invariants_hold_for_the_oracle(oracle):
    x, w = engine_test_inputs()
    z = oracle.router_logits(x, w["router_w"])
    idx, gates, _, counts, _ = oracle.route(z, 2)
    assert len(counts) == 8 and counts.sum() == 512
    assert (counts > 0).all(), "dead expert"
    assert routing_balance_ok(counts, 256, 8)
    assert (idx[:, 0] != idx[:, 1]).all()
    _, out = oracle.forward(x, w, idx, gates)
    assert torch.isfinite(out.float()).all()
    assert not routing_balance_ok([512, 0, 0, 0, 0, 0, 0, 0], 256, 8)
    assert not routing_balance_ok([200, 45, 45, 45, 45, 44, 44, 44], 256, 8)


def test_adamw_engine_statement():
    """The oracle's AdamW with the engine's conventions against the same update spelled out
    in numpy fp32 (step size lr / sqrt(in_dim), clamps, floored bias corrections)."""
    import oracle_binding
    orc = oracle_binding.load()
    rng = np.random.default_rng(5)
    n, in_dim = 1000, 256
    w = (rng.standard_normal(n) * 0.5).astype(np.float32)
    m = (rng.standard_normal(n) * 0.1).astype(np.float32)
    v = np.abs(rng.standard_normal(n)).astype(np.float32)
    g = (rng.standard_normal(n) * 60).astype(np.float32)
    g[::7] = np.nan
    g[1::9] = np.inf
    lr, b1, b2, eps, wd, step = (np.float32(a) for a in (0.5, 0.9, 0.999, 1e-8, 0.01, 3))
    gc = np.where(np.isfinite(g), g, np.float32(0)).clip(-100, 100).astype(np.float32)
    m_ref = b1 * m + (np.float32(1) - b1) * gc
    v_ref = b2 * v + (np.float32(1) - b2) * gc * gc
    c1 = np.float32(1) - b1 ** step
    c2 = np.float32(1) - b2 ** step
    size = lr * (np.float32(1) / np.sqrt(np.float32(in_dim)))
    w_ref = (w - size * ((m_ref / c1) / (np.sqrt(v_ref / c2) + eps) + wd * w)).clip(-2, 2).astype(np.float32)
    wb = np.zeros(n, np.uint16)
    orc.adamw_engine(w, m, v, g, wb, in_dim, float(lr), float(b1), float(b2), float(eps), float(wd), 3)
    assert np.abs(m - m_ref).max() <= 1e-6 * np.abs(m_ref).max()
    assert np.abs(v - v_ref).max() <= 1e-6 * np.abs(v_ref).max()
    assert np.abs(w - w_ref).max() <= 1e-6
    assert (wb == (torch.from_numpy(w).bfloat16().view(torch.int16).numpy().view(np.uint16))).all()
    # a bias correction that underflows counts as 1: beta = 1 makes 1 - beta^t = 0
    w2, m2, v2 = np.ones(4, np.float32), np.zeros(4, np.float32), np.zeros(4, np.float32)
    orc.adamw_engine(w2, m2, v2, np.ones(4, np.float32), np.zeros(4, np.uint16), 1, 0.1, 1.0, 1.0, 1e-8, 0.0, 5)
    assert np.isfinite(w2).all() and (m2 == 0).all() and (v2 == 0).all()
