"""AdamW step over an MoE weight matrix (fp32 master + moments, bf16 working copy)
against the same update written in numpy fp32.  Elementwise fp32: |err| <= 1e-6 * max(1, |ref|);
the bf16 copy must be the rounding of the GPU's own master."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [1, 7, 4096, 1000003])
def test_adamw_step(axm, cuda_device, n):
    lib = axm.load()
    rng = np.random.default_rng(n)
    w = (rng.standard_normal(n) * 0.02).astype(np.float32)
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    lr, b1, b2, eps, wd = np.float32(1e-3), np.float32(0.9), np.float32(0.95), np.float32(1e-8), np.float32(0.1)
    dw, dm, dv = (torch.from_numpy(a.copy()).to(cuda_device) for a in (w, m, v))
    wb = torch.empty(n, dtype=torch.bfloat16, device=cuda_device)
    for step in (1, 2, 3):
        g = rng.standard_normal(n).astype(np.float32)
        dg = torch.from_numpy(g).to(cuda_device)
        axm.check(lib.axm_moe_adamw_step(axm.ptr(dw), axm.ptr(dm), axm.ptr(dv), axm.ptr(dg), axm.ptr(wb), n,
                                         float(lr), float(b1), float(b2), float(eps), float(wd), step,
                                         axm.current_stream()))
        c1 = np.float32(1) - np.float32(b1) ** np.float32(step)
        c2 = np.float32(1) - np.float32(b2) ** np.float32(step)
        m = b1 * m + (np.float32(1) - b1) * g
        v = b2 * v + (np.float32(1) - b2) * g * g
        w = w - lr * ((m / c1) / (np.sqrt(v / c2) + eps) + wd * w)
        torch.cuda.synchronize()
        for got, ref in ((dw, w), (dm, m), (dv, v)):
            err = np.abs(got.cpu().numpy() - ref)
            assert (err <= 1e-6 * np.maximum(1.0, np.abs(ref))).all()
        assert torch.equal(wb, dw.bfloat16())


@pytest.mark.parametrize("n,in_dim", [(5, 1), (4099, 2048), (300001, 4096)])
def test_adamw_engine_conventions_match_oracle(axm, oracle, cuda_device, n, in_dim):
    """axm_moe_adamw_step_engine against the oracle's statement of the engine's optimiser
    (lr / sqrt(in_dim), gradient clamp and non-finite -> 0, floored bias corrections, weight
    clamp, update skipped when not finite).  fp32 throughout; the kernel's sqrt and divisions
    are IEEE and powf runs on the host, so the two differ only by fused multiply-adds."""
    lib = axm.load()
    rng = np.random.default_rng(n)
    w = (rng.standard_normal(n) * 0.5).astype(np.float32)
    w[::97] = 1.9999                       # next to the weight clamp
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    wb_ref = np.zeros(n, np.uint16)
    lr, b1, b2, eps, wd = 0.3, 0.9, 0.95, 1e-8, 0.1
    dw, dm, dv = (torch.from_numpy(a.copy()).to(cuda_device) for a in (w, m, v))
    wb = torch.zeros(n, dtype=torch.bfloat16, device=cuda_device)
    for step in (0, 1, 2, 3):               # the engine counts step 0 as 1
        g = (rng.standard_normal(n) * 30.0).astype(np.float32)
        g[::11] = 1e4                       # clamped to 100
        g[3::13] = np.nan                   # counts as zero
        g[5::17] = -np.inf
        dg = torch.from_numpy(g).to(cuda_device)
        axm.check(lib.axm_moe_adamw_step_engine(axm.ptr(dw), axm.ptr(dm), axm.ptr(dv), axm.ptr(dg), axm.ptr(wb),
                                                n, in_dim, lr, b1, b2, eps, wd, step, axm.current_stream()))
        oracle.adamw_engine(w, m, v, g, wb_ref, in_dim, lr, b1, b2, eps, wd, step)
        torch.cuda.synchronize()
        # m = b1 * m + (1 - b1) * g adds terms of magnitude up to 100 that may cancel, and the
        # kernel contracts it into a fused multiply-add: absolute 1e-5 there; v sums positive
        # terms and w moves by a small step: relative 1e-6
        for got, ref, what, tol in ((dw, w, "w", 1e-6 * np.maximum(1.0, np.abs(w))), (dm, m, "m", 1e-5),
                                    (dv, v, "v", 1e-6 * np.maximum(1.0, np.abs(v)))):
            err = np.abs(got.cpu().numpy() - ref)
            assert (err <= tol).all(), what
        assert np.isfinite(dw.cpu().numpy()).all() and float(dw.abs().max()) <= 2.0
        assert torch.equal(wb, dw.bfloat16())

