"""The entry point for callers that cannot allocate device memory
(axm_moe_route_dispatch_noalloc) against the regular pair of calls it replaces.

Such callers - a server whose arena owns all of HBM, a plug-in inside another
process, a latency path that must not hit cudaMalloc's synchronisation - get the
router's block-count scratch from a fixed array inside the library.  The results
are integer and index work plus fp32 gates computed by the same kernels, so they
must equal the regular entry points' bit for bit.  Two calls in a row with
different shapes share that array; the second must not see anything of the first.
This file sorts last on purpose, so that a run that stops at the first failure
has already run everything else."""
import ctypes

import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def regular(axm, desc, logits, x):
    idx, gate, bc = helpers.run_route_from_logits(axm, desc, logits)
    hist, offsets, row_src, slot_dst, xp = helpers.run_permute(axm, desc, x, idx, bc)
    torch.cuda.synchronize()
    return idx, gate, hist, offsets, row_src, slot_dst, xp


def no_alloc(axm, desc, logits, x):
    lib = axm.load()
    T, E, k, D = desc.tokens, desc.num_experts, desc.top_k, desc.d_model
    dev = logits.device
    idx = torch.full((T, k), -1, dtype=torch.int32, device=dev)
    gate = torch.zeros(T, k, dtype=torch.float32, device=dev)
    hist = torch.zeros(E, dtype=torch.int32, device=dev)
    offsets = torch.full((E + 1,), -1, dtype=torch.int32, device=dev)
    row_src = torch.full((T * k,), -1, dtype=torch.int32, device=dev)
    slot_dst = torch.full((T * k,), -1, dtype=torch.int32, device=dev)
    xp = torch.zeros(T * k, D, dtype=torch.bfloat16, device=dev)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    axm.check(lib.axm_moe_route_dispatch_noalloc(
        ctypes.byref(desc), axm.ptr(logits), axm.ptr(x), axm.ptr(idx), axm.ptr(gate), axm.ptr(hist),
        axm.ptr(offsets), axm.ptr(row_src), axm.ptr(slot_dst), axm.ptr(xp), axm.current_stream()))
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    return idx, gate, hist, offsets, row_src, slot_dst, xp


def case(axm, cuda_device, T, D, E, k, seed):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g).to(cuda_device)
    x = torch.randn(T, D, generator=g).bfloat16().to(cuda_device)
    desc = axm.make_desc(T, D, 64, E, k, flags=0)
    return desc, logits, x


def test_two_calls_in_a_row_match_the_regular_entry_points(axm, oracle, cuda_device):
    # a wide case first, then a narrower one that reuses the front of the same scratch
    for (T, D, E, k, seed) in [(3000, 128, 128, 6, 1), (1111, 64, 8, 2, 2)]:
        desc, logits, x = case(axm, cuda_device, T, D, E, k, seed)
        want = regular(axm, desc, logits, x)
        got = no_alloc(axm, desc, logits, x)
        names = ["topk_idx", "topk_gate", "histogram", "offsets", "row_src", "slot_dst", "x_perm"]
        for n, a, b in zip(names, got, want):
            if a.dtype.is_floating_point:   # same kernel, same inputs: identical bits
                assert torch.equal(a.view(torch.int32) if a.dtype == torch.float32
                                   else a.view(torch.int16),
                                   b.view(torch.int32) if b.dtype == torch.float32
                                   else b.view(torch.int16)), n
            else:
                assert torch.equal(a, b), n
        assert int(got[2].sum()) == T * k
        # and against the CPU oracle from the same logits: the same experts except where it
        # flags a near-tie (CPU and GPU expf may differ in the last bit), and the placement
        # rule applied to the indices this call produced
        idx = got[0].cpu().numpy()
        oi, og, _, oc, tie = oracle.route(logits.cpu().numpy(), k)
        mism = (oi != idx).any(axis=1)
        assert not (mism & (tie == 0)).any()
        ooff, ors, osd = oracle.permutation(idx, E)
        assert (got[3].cpu().numpy() == ooff).all()
        assert (got[4].cpu().numpy() == ors).all() and (got[5].cpu().numpy() == osd).all()
        assert (got[2].cpu().numpy() == np.bincount(idx.ravel(), minlength=E)).all()
        rows = got[6].cpu()
        assert torch.equal(rows, x.cpu()[torch.from_numpy(ors).long() // k])


def test_more_experts_than_the_builtin_scratch_holds_is_refused(axm, cuda_device):
    E = axm.NOALLOC_MAX_EXPERTS + 1
    desc, logits, x = case(axm, cuda_device, 64, 64, E, 2, 3)
    lib = axm.load()
    idx = torch.full((64, 2), -7, dtype=torch.int32, device=cuda_device)
    gate = torch.zeros(64, 2, dtype=torch.float32, device=cuda_device)
    rc = lib.axm_moe_route_dispatch_noalloc(ctypes.byref(desc), axm.ptr(logits), axm.ptr(x),
                                            axm.ptr(idx), axm.ptr(gate), None, None, None, None,
                                            None, axm.current_stream())
    torch.cuda.synchronize()
    assert rc == axm.AXM_ERR_ARGUMENT
    assert b"exceeds the built-in scratch" in lib.axm_last_error()
    assert int((idx != -7).sum()) == 0          # nothing was launched


def test_a_refused_call_has_launched_nothing(axm, cuda_device):
    """Every argument is checked before the first kernel: x_perm without x is refused
    with the routing outputs untouched."""
    desc, logits, x = case(axm, cuda_device, 64, 64, 8, 2, 4)
    lib = axm.load()
    idx = torch.full((64, 2), -7, dtype=torch.int32, device=cuda_device)
    gate = torch.zeros(64, 2, dtype=torch.float32, device=cuda_device)
    xp = torch.zeros(128, 64, dtype=torch.bfloat16, device=cuda_device)
    rc = lib.axm_moe_route_dispatch_noalloc(ctypes.byref(desc), axm.ptr(logits), None,
                                            axm.ptr(idx), axm.ptr(gate), None, None, None, None,
                                            axm.ptr(xp), axm.current_stream())
    torch.cuda.synchronize()
    assert rc == axm.AXM_ERR_ARGUMENT
    assert int((idx != -7).sum()) == 0
