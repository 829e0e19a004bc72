"""Grouped SwiGLU expert GEMMs (tcgen05) against a torch fp32 statement of the
same two products, segment by segment.  Floating point, fp32 accumulation: h is
stored as bf16 and o as fp32, so an element may differ by bf16 rounding of h
plus accumulation-order noise: |err| <= 2^-7 * |ref| + 2e-3 * max|ref|."""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def ffn_reference(xp, seg_rows, w, E):
    """Per-segment fp32 reference; h is rounded to bf16 before the down product."""
    outs_h, outs_o = [], []
    for (a0, rows, e, a_src) in seg_rows:
        a = a_src[a0:a0 + rows].float()
        if e < E:
            g, u, d = w["w_gate"][e], w["w_up"][e], w["w_down"][e]
        else:
            g, u, d = w["shared_gate"][e - E], w["shared_up"][e - E], w["shared_down"][e - E]
        h = torch.nn.functional.silu(a @ g.float()) * (a @ u.float())
        outs_h.append(h)
        outs_o.append(h.bfloat16().float() @ d.float())
    return outs_h, outs_o


def close(got, ref, what):
    if ref.numel() == 0:
        return
    err = (got.float() - ref).abs()
    bound = 2.0 ** -7 * ref.abs() + 2e-3 * ref.abs().max()
    assert (err <= bound).all(), f"{what}: max err {float(err.max()):.4g}, max |ref| {float(ref.abs().max()):.4g}"


@pytest.mark.parametrize("D,F,E,S,rows", [
    (256, 512, 8, 0, [18, 16, 18, 19, 15, 12, 16, 14]),       # C1-like, every expert under one tile
    (2048, 5632, 8, 0, [130, 0, 128, 1, 257, 0, 127, 64]),    # C2 dims, ragged, empty experts
    (2048, 1408, 8, 2, [5, 300, 0, 0, 129, 77, 0, 12]),       # C4 dims with shared experts
    (4096, 1024, 2, 0, [200, 100]),                           # C3 d_model
    (264, 200, 3, 0, [33, 140, 7]),                           # nothing a multiple of the tile
    (64, 64, 1, 1, [1]),                                      # smallest
])
def test_expert_ffn(axm, cuda_device, D, F, E, S, rows):
    g = torch.Generator(device=cuda_device).manual_seed(D + F)
    T = 96 if S else 0
    w = {
        "w_gate": (torch.randn(E, D, F, device=cuda_device, generator=g) * 0.02).bfloat16(),
        "w_up": (torch.randn(E, D, F, device=cuda_device, generator=g) * 0.02).bfloat16(),
        "w_down": (torch.randn(E, F, D, device=cuda_device, generator=g) * 0.02).bfloat16(),
    }
    if S:
        w["shared_gate"] = (torch.randn(S, D, F, device=cuda_device, generator=g) * 0.02).bfloat16()
        w["shared_up"] = (torch.randn(S, D, F, device=cuda_device, generator=g) * 0.02).bfloat16()
        w["shared_down"] = (torch.randn(S, F, D, device=cuda_device, generator=g) * 0.02).bfloat16()
    n_routed = sum(rows)
    xp = torch.randn(max(n_routed, 1), D, device=cuda_device, generator=g).bfloat16()
    x_alt = torch.randn(T, D, device=cuda_device, generator=g).bfloat16() if S else None
    off = np.concatenate([[0], np.cumsum(rows)]).astype(np.int32)
    seg, seg_rows = [], []
    for e in range(E):
        seg.append([off[e], off[e], rows[e], e])
        seg_rows.append((int(off[e]), rows[e], e, xp))
    for s in range(S):
        seg.append([0, n_routed + s * T, T, (E + s) | axm.SEG_ALT_A])
        seg_rows.append((0, T, E + s, x_alt))
    seg_t = torch.tensor(seg, dtype=torch.int32, device=cuda_device)
    rows_total = n_routed + S * T
    desc = axm.make_desc(T, D, F, E, 1, S)
    h, o = helpers.run_expert_ffn(axm, desc, xp, x_alt, seg_t, w, rows_total)
    ref_h, ref_o = ffn_reference(xp, seg_rows, w, E)
    for (sg, rh, ro) in zip(seg, ref_h, ref_o):
        r0, n = sg[1], sg[2]
        close(h[r0:r0 + n], rh, f"h of expert {sg[3] & 0xffff}")
        close(o[r0:r0 + n], ro, f"o of expert {sg[3] & 0xffff}")


def test_expert_ffn_leaves_other_rows_alone(axm, cuda_device):
    """Rows that belong to no segment keep their previous contents (masked tails)."""
    D, F, E = 128, 256, 2
    g = torch.Generator(device=cuda_device).manual_seed(1)
    w = {n: (torch.randn(E, *s, device=cuda_device, generator=g) * 0.02).bfloat16()
         for n, s in (("w_gate", (D, F)), ("w_up", (D, F)), ("w_down", (F, D)))}
    xp = torch.randn(300, D, device=cuda_device, generator=g).bfloat16()
    seg = torch.tensor([[0, 0, 100, 0], [150, 150, 50, 1]], dtype=torch.int32, device=cuda_device)
    desc = axm.make_desc(0, D, F, E, 1, 0)
    h, o = helpers.run_expert_ffn(axm, desc, xp, None, seg, w, 300)
    assert float(h[100:150].abs().max()) == 0.0 and float(h[200:].abs().max()) == 0.0
    assert float(o[100:150].abs().max()) == 0.0 and float(o[200:].abs().max()) == 0.0
    assert float(o[:100].abs().max()) > 0.0
