"""Backward grouped GEMMs (tcgen05; K-major weights for the input gradients,
transposed operands for the weight gradients) against torch fp32, expert by expert,
on segments padded to multiples of 64 rows.  bf16 inputs, fp32 accumulation:
|err| <= 2^-7 * |ref| + 4e-3 * max|ref| per tensor."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def close(got, ref, what):
    err = (got.float() - ref).abs()
    bound = 2.0 ** -7 * ref.abs() + 4e-3 * ref.abs().max()
    assert (err <= bound).all(), f"{what}: max err {float(err.max()):.4g}, max |ref| {float(ref.abs().max()):.4g}"


@pytest.mark.parametrize("D,F,E,rows", [
    (256, 512, 4, [70, 0, 128, 5]),
    (2048, 4096, 3, [300, 64, 129]),
    (136, 200, 2, [33, 64]),
])
def test_expert_ffn_backward(axm, cuda_device, D, F, E, rows):
    lib = axm.load()
    dev = cuda_device
    gen = torch.Generator(device=dev).manual_seed(D + F)
    rnd = lambda *s, scale=1.0: (torch.randn(*s, device=dev, generator=gen) * scale)
    wg, wu = rnd(E, D, F, scale=0.02).bfloat16(), rnd(E, D, F, scale=0.02).bfloat16()
    wd = rnd(E, F, D, scale=0.02).bfloat16()
    padded = [(r + 63) // 64 * 64 for r in rows]
    off = np.concatenate([[0], np.cumsum(padded)]).astype(int)
    R = int(off[-1])
    x = torch.zeros(R, D, device=dev, dtype=torch.bfloat16)
    d_o = torch.zeros(R, D, device=dev, dtype=torch.bfloat16)
    for e in range(E):
        x[off[e]:off[e] + rows[e]] = rnd(rows[e], D).bfloat16()
        d_o[off[e]:off[e] + rows[e]] = rnd(rows[e], D).bfloat16()
    # forward quantities the backward consumes (pad rows stay zero)
    g = torch.zeros(R, F, device=dev, dtype=torch.bfloat16)
    u = torch.zeros_like(g)
    h = torch.zeros_like(g)
    for e in range(E):
        sl = slice(off[e], off[e + 1])
        gf, uf = x[sl].float() @ wg[e].float(), x[sl].float() @ wu[e].float()
        g[sl], u[sl] = gf.bfloat16(), uf.bfloat16()
        h[sl] = (torch.nn.functional.silu(gf) * uf).bfloat16()
    seg = torch.tensor([[off[e], off[e], padded[e], e] for e in range(E)], dtype=torch.int32, device=dev)
    d_g = torch.full((R, F), 7.0, device=dev, dtype=torch.bfloat16)
    d_u = torch.full_like(d_g, 7.0)
    d_xp = torch.full((R, D), 7.0, device=dev, dtype=torch.float32)
    dwg = torch.full((E, D, F), 7.0, device=dev, dtype=torch.float32)
    dwu = torch.full_like(dwg, 7.0)
    dwd = torch.full((E, F, D), 7.0, device=dev, dtype=torch.float32)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    desc = axm.make_desc(0, D, F, E, 1)
    p = axm.ptr
    axm.check(lib.axm_moe_expert_ffn_backward(
        ctypes.byref(desc), p(seg), E, R, p(x), p(h), p(g), p(u), p(d_o), p(wg), p(wu), p(wd),
        p(d_g), p(d_u), p(d_xp), p(dwg), p(dwu), p(dwd), p(status), axm.current_stream()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for e in range(E):
        sl = slice(off[e], off[e + 1])
        gf, uf = g[sl].float(), u[sl].float()
        dh = d_o[sl].float() @ wd[e].float().t()
        s = torch.sigmoid(gf)
        dg_ref = dh * uf * (s * (1 + gf * (1 - s)))
        du_ref = dh * gf * s
        if padded[e]:
            close(d_g[sl], dg_ref, f"dG expert {e}")
            close(d_u[sl], du_ref, f"dU expert {e}")
            dx_ref = d_g[sl].float() @ wg[e].float().t() + d_u[sl].float() @ wu[e].float().t()
            close(d_xp[sl], dx_ref, f"dXp expert {e}")
        close(dwd[e], h[sl].float().t() @ d_o[sl].float(), f"dWd expert {e}") if padded[e] else None
        if padded[e] == 0:
            assert float(dwd[e].abs().max()) == 0.0 and float(dwg[e].abs().max()) == 0.0
            continue
        close(dwg[e], x[sl].float().t() @ d_g[sl].float(), f"dWg expert {e}")
        close(dwu[e], x[sl].float().t() @ d_u[sl].float(), f"dWu expert {e}")
