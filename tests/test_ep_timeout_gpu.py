"""Failure detection of the expert-parallel exchange without any GPU fault: a
wait on a flag that no peer ever sets runs out after its bound (about two
seconds), the kernel returns, the status word holds the code of the wait that
gave up, and the context stays usable."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_for_a_peer_that_never_answers_gives_up(axm, cuda_device):
    lib = axm.load()
    layout = axm.EpLayout()
    nbytes = ctypes.c_size_t(0)
    world, E, D, slots = 2, 4, 64, 8
    axm.check(lib.axm_ep_region_bytes(world, E, D, slots, slots * world, ctypes.byref(layout),
                                      ctypes.byref(nbytes)))
    region = torch.zeros(nbytes.value, dtype=torch.uint8, device=cuda_device)
    # a two-rank layout whose "peer" is this GPU's own region: rank 1 never runs, so the
    # flags it would set stay 0
    peers = torch.tensor([region.data_ptr(), region.data_ptr()], dtype=torch.int64, device=cuda_device)
    layout.peers = peers.data_ptr()
    layout.rank = 0
    layout.num_shared = 0
    layout.tokens_local = 4
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    t0 = time.time()
    axm.check(lib.axm_ep_wait_return(ctypes.byref(layout), 1, axm.ptr(status), axm.current_stream()))
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert int(status.item()) == 13          # the return wait gave up
    assert 0.5 < waited < 10.0
    # the context is intact: ordinary work still runs and gives right answers
    a = torch.arange(1024, device=cuda_device, dtype=torch.float32)
    assert float((a * 2).sum().item()) == float(1023 * 1024)
    # once the flag is there the same call returns at once and reports nothing
    flags = region[layout.off_flags:layout.off_flags + 4 * 3 * world].view(torch.int32)
    flags[2 * world + 0] = 1
    flags[2 * world + 1] = 1
    status.zero_()
    t0 = time.time()
    axm.check(lib.axm_ep_wait_return(ctypes.byref(layout), 1, axm.ptr(status), axm.current_stream()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and time.time() - t0 < 0.5
