"""Checkpoint block -> device: the fp32 master tensors loaded from the file are cast to
the bf16 working copy by the library (round-to-nearest-even, as torch does) and the
layer built from them gives the same bits as the layer built from the original weights."""
import importlib
import struct

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_resume_from_checkpoint(axm, workloads, cuda_device, tmp_path):
    ckpt = importlib.import_module("project_axiom_ai_llm_b200.checkpoint")
    cfg = workloads.scaled(workloads.CONFIGS["C1"], tokens=64)
    x, w = workloads.make_inputs(cfg, device=cuda_device)
    # fp32 masters: the bf16 weights widened (exactly representable), the router as it is
    master = {n: t.float().cpu().numpy() for n, t in w.items()}
    path = str(tmp_path / "weights.axiom")
    rng = np.random.default_rng(0)
    with open(path, "wb") as f:  # a minimal stock checkpoint with a transformer block
        f.write(b"AXIOM_V1" + struct.pack("<6Q", 2, 2, 0, 0, 0, 0))
        f.write(struct.pack("<3Q", 0x5458464D, 2, 3))
        f.write(rng.standard_normal(4 * 4 + 3 * 6).astype(np.float32).tobytes())
    ckpt.save_moe_block(path, master, top_k=cfg.top_k)
    info, loaded = ckpt.load_moe_block(path)
    assert info["num_experts"] == cfg.num_experts and info["d_ff"] == cfg.d_ff

    lib = axm.load()
    resumed = {}
    for n, t in w.items():
        dev_master = torch.from_numpy(loaded[n]).to(cuda_device)
        if t.dtype == torch.bfloat16:
            out = torch.empty_like(t)
            axm.check(lib.axm_moe_cast_master(axm.ptr(dev_master), axm.ptr(out), dev_master.numel(),
                                              axm.current_stream()))
            assert torch.equal(out, dev_master.bfloat16())
            resumed[n] = out
        else:
            resumed[n] = dev_master
    torch.cuda.synchronize()
    a, _ = axm.MoeLayer(w, cfg.tokens, cfg.top_k).forward(x)
    b, _ = axm.MoeLayer(resumed, cfg.tokens, cfg.top_k).forward(x)
    torch.cuda.synchronize()
    assert torch.equal(a, b)

    # the cast rounds to nearest even like torch for values that are not bf16-exact
    v = torch.randn(100003, device=cuda_device)
    o = torch.empty(100003, device=cuda_device, dtype=torch.bfloat16)
    axm.check(lib.axm_moe_cast_master(axm.ptr(v), axm.ptr(o), v.numel(), axm.current_stream()))
    torch.cuda.synchronize()
    assert torch.equal(o, v.bfloat16())
