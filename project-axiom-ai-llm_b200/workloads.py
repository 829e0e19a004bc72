"""The benchmark configurations of the MoE layer and their seeded synthetic inputs.

Activations are bf16 ~ N(0, 1); expert weights bf16 ~ N(0, 0.02^2); router
weights fp32 ~ N(0, 0.02^2).  One generator per configuration draws, in this
order: x, router weights, gate, up, down, shared gate/up/down, bias permutation.
Layouts are the reference engine's (core/src/CUDA/util/gpu_types.cuh:147-157):
router [D][E], gate/up [E][D][F], down [E][F][D].  No public dataset is involved.
"""
from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class MoeConfig:
    name: str
    tokens: int
    d_model: int
    num_experts: int
    top_k: int
    d_ff: int
    seed: int
    num_shared: int = 0
    zipf_s: float = 0.0       # > 0: additive per-expert logit bias c * rank^-s
    zipf_c: float = 0.0
    training: bool = False
    aux_alpha: float = 0.0

    @property
    def gemm_flops(self):
        """6*T*k*D*F for the routed experts plus 6*T*S*D*F for the shared ones."""
        return 6 * self.tokens * (self.top_k + self.num_shared) * self.d_model * self.d_ff

    @property
    def weight_bytes(self):
        return 6 * (self.num_experts + self.num_shared) * self.d_model * self.d_ff

    def stage_bytes(self, router_w_bytes=4):
        """Algorithmic HBM bytes of the memory-bound stages of one layer call."""
        T, D, E, k, S = self.tokens, self.d_model, self.num_experts, self.top_k, self.num_shared
        return {
            "router": 2 * T * D + router_w_bytes * D * E + 4 * T * E + 8 * T * k + 4 * E,
            "permute": 2 * T * D + 2 * T * k * D + 8 * T * k,
            "combine": 2 * T * (k + S) * D + 8 * T * k + 2 * T * D + 2 * T * D,
        }


CONFIGS = {
    "C1": MoeConfig("C1", 64, 256, 8, 2, 512, seed=0),
    "C2": MoeConfig("C2", 4096, 2048, 8, 2, 5632, seed=1),
    "C3": MoeConfig("C3", 8192, 4096, 8, 2, 14336, seed=2),
    "C4": MoeConfig("C4", 16384, 2048, 64, 6, 1408, seed=3, num_shared=2, zipf_s=1.2, zipf_c=3.0),
    "C5": MoeConfig("C5", 8192, 2048, 16, 2, 4096, seed=4, training=True, aux_alpha=0.01),
}


def scaled(cfg, tokens=None, **kw):
    """A copy of cfg with fewer tokens or other fields replaced (parity-test sizes)."""
    d = dict(cfg.__dict__)
    if tokens is not None:
        d["tokens"] = tokens
    d.update(kw)
    return MoeConfig(**d)


def make_inputs(cfg, device="cpu", router_bf16=False):
    """Seeded tensors for cfg.  Drawn on `device` (the values depend on it)."""
    dev = torch.device(device)
    g = torch.Generator(device=dev)
    g.manual_seed(cfg.seed)
    T, D, E, F, S = cfg.tokens, cfg.d_model, cfg.num_experts, cfg.d_ff, cfg.num_shared

    def normal(shape, std, dtype):
        t = torch.empty(shape, dtype=torch.float32, device=dev)
        t.normal_(0.0, std, generator=g)
        return t.to(dtype)

    w = {}
    x = normal((T, D), 1.0, torch.bfloat16)
    wr = normal((D, E), 0.02, torch.float32)
    w["router_w"] = wr.to(torch.bfloat16) if router_bf16 else wr
    w["w_gate"] = normal((E, D, F), 0.02, torch.bfloat16)
    w["w_up"] = normal((E, D, F), 0.02, torch.bfloat16)
    w["w_down"] = normal((E, F, D), 0.02, torch.bfloat16)
    if S > 0:
        w["shared_gate"] = normal((S, D, F), 0.02, torch.bfloat16)
        w["shared_up"] = normal((S, D, F), 0.02, torch.bfloat16)
        w["shared_down"] = normal((S, F, D), 0.02, torch.bfloat16)
    if cfg.zipf_s > 0:
        perm = torch.randperm(E, generator=g, device=dev)
        rank = torch.empty(E, dtype=torch.float32, device=dev)
        rank[perm] = torch.arange(1, E + 1, dtype=torch.float32, device=dev)
        w["router_bias"] = (cfg.zipf_c * rank.pow(-cfg.zipf_s)).contiguous()
    return x, w
