"""Expert-parallel host logic on CPU: two gloo ranks with the oracle standing in
for the CUDA stages must reproduce the single-process oracle layer bit for bit."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, cfg_kw, out_dir):
    sys.path.insert(0, HERE)
    import importlib
    import conftest
    conftest.load_package()
    wl = importlib.import_module("project_axiom_ai_llm_b200.workloads")
    ep = importlib.import_module("project_axiom_ai_llm_b200.expert_parallel")
    import cpu_stages
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = wl.MoeConfig(**cfg_kw)
        x, w = wl.make_inputs(cfg)
        tl = cfg.tokens // world
        layer = ep.ExpertParallelMoe(ep.shard_weights(w, rank, world), tl, cfg.num_experts,
                                     cfg.top_k, stages=cpu_stages.OracleStages())
        out = layer.forward(x[rank * tl:(rank + 1) * tl].contiguous())
        torch.save({"out": out, "idx": layer.idx, "hist": layer.histogram,
                    "rows": layer.last_rows_received}, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cfg_kw", [
    dict(name="ep_small", tokens=64, d_model=64, num_experts=8, top_k=2, d_ff=96, seed=5),
    dict(name="ep_skew", tokens=96, d_model=64, num_experts=16, top_k=6, d_ff=64, seed=6,
         num_shared=2, zipf_s=1.2, zipf_c=3.0),
    dict(name="ep_k1", tokens=32, d_model=32, num_experts=2, top_k=1, d_ff=32, seed=7),
])
def test_two_ranks_match_single_process(tmp_path, oracle, workloads, cfg_kw):
    world = 2
    mp.start_processes(_worker, args=(world, _free_port(), cfg_kw, str(tmp_path)), nprocs=world,
                       join=True, start_method="spawn")
    cfg = workloads.MoeConfig(**cfg_kw)
    x, w = workloads.make_inputs(cfg)
    z = oracle.router_logits(x, w["router_w"], w.get("router_bias"))
    idx, gates, _, counts, _ = oracle.route(z, cfg.top_k)
    _, ref = oracle.forward(x, w, idx, gates)
    parts = [torch.load(os.path.join(str(tmp_path), f"r{r}.pt")) for r in range(world)]
    out = torch.cat([p["out"] for p in parts])
    assert (torch.cat([p["idx"] for p in parts]).numpy() == idx).all()
    assert (sum(p["hist"] for p in parts).numpy() == counts).all()
    # rows received by rank r = selections of its experts over all tokens
    el = cfg.num_experts // world
    for r, p in enumerate(parts):
        assert p["rows"] == int(counts[r * el:(r + 1) * el].sum())
    assert torch.equal(out, ref)


def test_segment_table(workloads, axm):
    import importlib
    ep = importlib.import_module("project_axiom_ai_llm_b200.expert_parallel")

    class Shell(ep.ExpertParallelMoe):
        def __init__(self):
            self.El, self.world, self.S, self.Tl, self.cap = 3, 2, 2, 10, 40

    seg = Shell().build_segments(torch.tensor([[4, 0, 2], [1, 5, 0]], dtype=torch.int32))
    assert seg.dtype == torch.int32
    # rows arrive source-major: (s0,e0)=4 (s0,e1)=0 (s0,e2)=2 (s1,e0)=1 (s1,e1)=5 (s1,e2)=0;
    # the table is expert-major
    assert seg[:6, 0].tolist() == [0, 6, 4, 7, 4, 12]
    assert seg[:6, 2].tolist() == [4, 1, 0, 5, 2, 0]
    assert seg[:6, 3].tolist() == [0, 0, 1, 1, 2, 2]
    assert seg[6].tolist() == [0, 40, 10, 3 | axm.SEG_ALT_A]
    assert seg[7].tolist() == [0, 50, 10, 4 | axm.SEG_ALT_A]
