"""Dispatch parity: histogram, offsets, placement and row copies are integer /
byte work and must equal the oracle's exactly."""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def block_counts_from_idx(axm, idx_np, T, E):
    """Per-router-block expert counts, the scratch the router hands to permute."""
    bc = np.zeros((axm.ROUTE_BLOCKS, E), dtype=np.int32)
    for b in range(axm.ROUTE_BLOCKS):
        lo, hi = (b * T) // axm.ROUTE_BLOCKS, ((b + 1) * T) // axm.ROUTE_BLOCKS
        if hi > lo:
            bc[b] = np.bincount(idx_np[lo:hi].ravel(), minlength=E)
    return bc


def random_idx(rng, T, E, k, dead=()):
    live = np.array([e for e in range(E) if e not in dead])
    return np.stack([rng.permutation(live)[:k] for _ in range(T)]).astype(np.int32)


@pytest.mark.parametrize("T,E,k,D,dead", [
    (64, 8, 2, 256, ()), (4096, 8, 2, 2048, ()), (2048, 64, 6, 2048, ()), (1, 8, 2, 64, ()),
    (295, 8, 2, 64, ()), (1000, 8, 2, 136, (0, 7)), (5000, 16, 1, 64, (3,)), (777, 256, 8, 72, ()),
    (20000, 4, 4, 64, ()),
])
def test_permute_matches_oracle(axm, oracle, cuda_device, T, E, k, D, dead):
    rng = np.random.default_rng(T + E)
    idx = random_idx(rng, T, E, k, dead)
    x = torch.randn(T, D, generator=torch.Generator().manual_seed(T)).bfloat16()
    desc = axm.make_desc(T, D, 64, E, k)
    bc = torch.from_numpy(block_counts_from_idx(axm, idx, T, E)).to(cuda_device)
    hist, offsets, row_src, slot_dst, xp = helpers.run_permute(
        axm, desc, x.to(cuda_device), torch.from_numpy(idx).to(cuda_device), bc)
    torch.cuda.synchronize()
    ooff, ors, osd = oracle.permutation(idx, E)
    assert (offsets.cpu().numpy() == ooff).all()
    assert (row_src.cpu().numpy() == ors).all()
    assert (slot_dst.cpu().numpy() == osd).all()
    assert (hist.cpu().numpy() == np.bincount(idx.ravel(), minlength=E)).all()
    assert torch.equal(xp.cpu(), x[torch.from_numpy(ors // k).long()])
    seg = helpers.run_build_segments(axm, desc, offsets).cpu().numpy()
    assert (seg[:, 0] == ooff[:-1]).all() and (seg[:, 2] == np.diff(ooff)).all()
    assert (seg[:, 3] == np.arange(E)).all()


def test_histogram_accumulate_flag(axm, cuda_device):
    rng = np.random.default_rng(3)
    T, E, k = 512, 8, 2
    idx = random_idx(rng, T, E, k)
    bc = torch.from_numpy(block_counts_from_idx(axm, idx, T, E)).to(cuda_device)
    idx_d = torch.from_numpy(idx).to(cuda_device)
    want = np.bincount(idx.ravel(), minlength=E)
    hist = torch.full((E,), 5, dtype=torch.int32, device=cuda_device)
    d_set = axm.make_desc(T, 64, 64, E, k, flags=0)
    helpers.run_permute(axm, d_set, None, idx_d, bc, histogram=hist, copy_rows=False)
    assert (hist.cpu().numpy() == want).all()
    d_acc = axm.make_desc(T, 64, 64, E, k, flags=axm.FLAG_HIST_ACCUMULATE)
    helpers.run_permute(axm, d_acc, None, idx_d, bc, histogram=hist, copy_rows=False)
    helpers.run_permute(axm, d_acc, None, idx_d, bc, histogram=hist, copy_rows=False)
    assert (hist.cpu().numpy() == 3 * want).all()
