"""CPU stand-in for the four compute stages of the expert-parallel layer, built on
the oracle.  Lets the exchange logic of ExpertParallelMoe (counts, splits, segment
table, row order) run under gloo without a GPU.  Tests only."""
import numpy as np
import torch

import oracle_binding


class OracleStages:
    def __init__(self):
        self.orc = oracle_binding.load()

    def router(self, desc, x, w, logits, idx, gate, block_counts):
        z = self.orc.router_logits(x, w["router_w"], w.get("router_bias"))
        i, g, _, _, _ = self.orc.route(z, desc.top_k)
        logits.copy_(torch.from_numpy(z))
        idx.copy_(torch.from_numpy(i))
        gate.copy_(torch.from_numpy(g))
        block_counts.zero_()

    def permute(self, desc, x, idx, block_counts, histogram, offsets, row_src, slot_dst, x_perm):
        i = idx.numpy()
        off, rs, sd = self.orc.permutation(i, desc.num_experts)
        offsets.copy_(torch.from_numpy(off))
        row_src.copy_(torch.from_numpy(rs))
        slot_dst.copy_(torch.from_numpy(sd))
        histogram.copy_(torch.from_numpy(np.diff(off).astype(np.int32)))
        x_perm.copy_(x[torch.from_numpy(rs // desc.top_k).long()])

    def expert_ffn(self, desc, a, a_rows, x_alt, alt_rows, segments, w, h, o, rows_total, status):
        E = desc.num_experts
        for a0, o0, rows, ex in segments.tolist():
            if rows == 0:
                continue
            e = ex & 0xffff
            src = x_alt if (ex >> 30) & 1 else a
            if e < E:
                wg, wu, wd = w["w_gate"][e], w["w_up"][e], w["w_down"][e]
            else:
                wg, wu, wd = w["shared_gate"][e - E], w["shared_up"][e - E], w["shared_down"][e - E]
            res = self.orc.expert_ffn(src[a0:a0 + rows], wg, wu, wd)
            o[o0:o0 + rows] = torch.from_numpy(res)

    def combine(self, desc, x, o, o_shared, slot_dst, gate, y, out):
        T, k, S = desc.tokens, desc.top_k, desc.num_shared
        rows = o[slot_dst.long()].view(T, k, -1)
        acc = torch.zeros(T, rows.shape[2], dtype=torch.float32)
        for i in range(k):   # fused multiply-add chain in slot order, like the oracle
            acc = _fma(gate[:, i:i + 1], rows[:, i], acc)
        for s in range(S):
            acc = acc + o_shared[s * T:(s + 1) * T]
        yb = acc.bfloat16()
        y.copy_(yb)
        out.copy_((x.float() + yb.float()).bfloat16() if desc.flags & 1 else yb)


def _fma(a, b, c):
    """Element-wise fused multiply-add in fp32 (via fp64: exact product, one rounding)."""
    return (a.double() * b.double() + c.double()).float()
