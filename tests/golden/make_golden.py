"""Writes tests/golden/moe_small.npz: a small MoE layer case (inputs and every
published output) computed by the CPU oracle, and tests/golden/moe_small_bwd.npz: the
gradients of the same case for a stored upstream gradient (auxiliary-loss weight 0.01).
Run from the repository root:

    python tests/golden/make_golden.py

The inputs are stored with the outputs, so the vectors do not depend on a random
number generator staying the same.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import conftest  # noqa: E402
import oracle_binding  # noqa: E402


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main():
    conftest.load_package()
    import importlib
    wl = importlib.import_module("project_axiom_ai_llm_b200.workloads")
    orc = oracle_binding.load()
    cfg = wl.MoeConfig("small", tokens=96, d_model=64, num_experts=8, top_k=2, d_ff=128, seed=11)
    x, w = wl.make_inputs(cfg)
    z = orc.router_logits(x, w["router_w"])
    idx, gates, probs, counts, tie = orc.route(z, cfg.top_k)
    offsets, row_src, slot_dst = orc.permutation(idx, cfg.num_experts)
    y, out = orc.forward(x, w, idx, gates)
    np.savez_compressed(
        os.path.join(HERE, "moe_small.npz"), top_k=cfg.top_k, x_bits=bits(x),
        router_w=w["router_w"].numpy(), w_gate_bits=bits(w["w_gate"]), w_up_bits=bits(w["w_up"]),
        w_down_bits=bits(w["w_down"]), logits=z, topk_idx=idx, topk_gate=gates, histogram=counts,
        offsets=offsets, row_src=row_src, slot_dst=slot_dst, y_bits=bits(y), out_bits=bits(out))
    print("wrote moe_small.npz", os.path.getsize(os.path.join(HERE, "moe_small.npz")), "bytes")
    g = torch.Generator().manual_seed(12)
    d_y = torch.randn(cfg.tokens, cfg.d_model, generator=g).numpy()
    grads = orc.backward(x, w, idx, gates, probs, d_y, alpha=0.01)
    np.savez_compressed(os.path.join(HERE, "moe_small_bwd.npz"), d_y=d_y, aux_alpha=0.01,
                        aux_loss=orc.aux_loss(probs, idx, 0.01), **grads)
    print("wrote moe_small_bwd.npz", os.path.getsize(os.path.join(HERE, "moe_small_bwd.npz")), "bytes")


if __name__ == "__main__":
    main()
