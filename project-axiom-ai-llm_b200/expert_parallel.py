"""Expert-parallel MoE layer: tokens and experts sharded over the ranks of one
node, one process per GPU, two all-to-all exchanges per layer call.

The reference engine is single-GPU (no NCCL anywhere in core/src); this module
is the sharded form of its forward_mixture_experts call
(core/src/CUDA/kernel/moe_router.cu:205-320):

  rank r owns tokens [r*T/G, (r+1)*T/G) and experts [r*E/G, (r+1)*E/G);
  router + permute run on the local tokens (router weights replicated);
  counts all-to-all -> row all-to-all (dispatch) into local HBM, one segment per
  (source rank, local expert) -> grouped SwiGLU GEMMs on local memory only ->
  row all-to-all back -> weighted combine on the source rank (gates never move).
  Shared experts are replicated and applied to the local tokens, no traffic.

torch.distributed (NCCL over NVLink on GPUs, gloo in CPU tests) carries the
exchanges.  The compute stages come from a `stages` object: CudaStages calls the
C ABI; tests substitute a CPU stand-in to exercise the exchange logic with gloo.
"""
import ctypes

import torch
import torch.distributed as dist

from . import (AXM_ERR_TIMEOUT, FLAG_H_EXACT, FLAG_RESIDUAL, ROUTER_BF16, ROUTER_FP32, ROUTE_BLOCKS, SEG_ALT_A,
               AxmError, EpLayout, EpTensors, MoeTrain, check, current_stream, load, make_desc, ptr, router_scratch_bytes)


class CudaStages:
    """The four compute stages through the C ABI, on the current CUDA device."""

    def __init__(self):
        self.lib = load()
        self.router_scratch = None   # split router weights of the tensor-core router, sized on first use

    def router(self, desc, x, w, logits, idx, gate, block_counts):
        need = router_scratch_bytes(desc)
        if need and (self.router_scratch is None or self.router_scratch.numel() < need
                     or self.router_scratch.device != x.device):
            self.router_scratch = torch.empty(need, dtype=torch.uint8, device=x.device)
        check(self.lib.axm_moe_router_ws(ctypes.byref(desc), ptr(x), ptr(w["router_w"]),
                                         ptr(w.get("router_bias")), ptr(logits), ptr(idx), ptr(gate),
                                         ptr(block_counts), ptr(self.router_scratch) if need else None,
                                         need, None, current_stream()))

    def permute(self, desc, x, idx, block_counts, histogram, offsets, row_src, slot_dst, x_perm):
        check(self.lib.axm_moe_permute(ctypes.byref(desc), ptr(x), ptr(idx), ptr(block_counts),
                                       ptr(histogram), ptr(offsets), ptr(row_src), ptr(slot_dst),
                                       ptr(x_perm), current_stream()))

    def expert_ffn(self, desc, a, a_rows, x_alt, alt_rows, segments, w, h, o, rows_total, status):
        S = desc.num_shared
        check(self.lib.axm_moe_expert_ffn(
            ctypes.byref(desc), ptr(a), a_rows, ptr(x_alt), alt_rows, ptr(segments),
            segments.shape[0], ptr(w["w_gate"]), ptr(w["w_up"]), ptr(w["w_down"]),
            ptr(w["shared_gate"]) if S else None, ptr(w["shared_up"]) if S else None,
            ptr(w["shared_down"]) if S else None, ptr(h), ptr(o), rows_total, ptr(status),
            current_stream()))

    def combine(self, desc, x, o, o_shared, slot_dst, gate, y, out):
        check(self.lib.axm_moe_combine(ctypes.byref(desc), ptr(x), ptr(o), ptr(o_shared),
                                       ptr(slot_dst), ptr(gate), ptr(y), ptr(out),
                                       current_stream()))


def shard_weights(w, rank, world):
    """This rank's slice of the expert weights; router, bias and shared experts replicated."""
    E = w["w_gate"].shape[0]
    assert E % world == 0, "num_experts must divide by the number of ranks"
    el = E // world
    out = dict(w)
    for n in ("w_gate", "w_up", "w_down"):
        out[n] = w[n][rank * el:(rank + 1) * el].contiguous()
    return out


class ExpertParallelMoe:
    """forward(x_local) -> out_local for this rank's T/G tokens."""

    def __init__(self, local_weights, tokens_local, num_experts, top_k, group=None, stages=None,
                 residual=True):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.stages = stages if stages is not None else CudaStages()
        self.w = local_weights
        wr = local_weights["router_w"]
        self.dev = wr.device
        D = wr.shape[0]
        F = local_weights["w_gate"].shape[2]
        self.E, self.k, self.D, self.F = num_experts, top_k, D, F
        self.El = num_experts // self.world
        assert self.El * self.world == num_experts
        assert local_weights["w_gate"].shape[0] == self.El
        self.S = 0 if local_weights.get("shared_gate") is None else local_weights["shared_gate"].shape[0]
        self.Tl = tokens_local
        rdt = ROUTER_FP32 if wr.dtype == torch.float32 else ROUTER_BF16
        flags = FLAG_RESIDUAL if residual else 0
        # routing runs over the global expert set, the FFN over the local one
        self.desc_route = make_desc(tokens_local, D, F, num_experts, top_k, 0, rdt, flags)
        self.desc_ffn = make_desc(tokens_local, D, F, self.El, min(top_k, self.El), self.S, rdt, flags)
        self.desc_comb = make_desc(tokens_local, D, F, num_experts, top_k, self.S, rdt, flags)
        dev, i32, bf = self.dev, torch.int32, torch.bfloat16
        n_slots = tokens_local * top_k
        # worst case: every slot of every rank lands on this rank's experts
        self.cap = n_slots * self.world
        self.rows_total = self.cap + self.S * tokens_local
        self.logits = torch.empty(tokens_local, num_experts, dtype=torch.float32, device=dev)
        self.idx = torch.empty(tokens_local, top_k, dtype=i32, device=dev)
        self.gate = torch.empty(tokens_local, top_k, dtype=torch.float32, device=dev)
        self.block_counts = torch.empty(ROUTE_BLOCKS, num_experts, dtype=i32, device=dev)
        self.histogram = torch.zeros(num_experts, dtype=i32, device=dev)
        self.offsets = torch.empty(num_experts + 1, dtype=i32, device=dev)
        self.row_src = torch.empty(n_slots, dtype=i32, device=dev)
        self.slot_dst = torch.empty(n_slots, dtype=i32, device=dev)
        self.x_perm = torch.empty(n_slots, D, dtype=bf, device=dev)
        self.recv = torch.empty(self.cap, D, dtype=bf, device=dev)
        self.h = torch.empty(self.rows_total, F, dtype=bf, device=dev)
        self.o = torch.empty(self.rows_total, D, dtype=torch.float32, device=dev)
        self.o_back = torch.empty(n_slots, D, dtype=torch.float32, device=dev)
        self.y = torch.empty(tokens_local, D, dtype=bf, device=dev)
        self.status = torch.zeros(1, dtype=i32, device=dev)
        self.recv_counts = torch.empty(self.world, self.El, dtype=i32, device=dev)
        self.last_rows_received = 0

    def build_segments(self, recv_counts):
        """Segment table for the rows received: one per (source rank, local expert).
        Rows sit in arrival order (source-major); the table lists them expert-major so
        that the GEMM kernel sees one expert's segments side by side and shares its
        weight tiles among them.  Then one segment per shared expert over the local tokens."""
        flat = recv_counts.reshape(-1).to(torch.int64)
        starts = torch.cumsum(flat, 0) - flat
        expert = torch.arange(self.El, device=flat.device).repeat(self.world)
        seg = torch.stack([starts, starts, flat, expert], dim=1)
        seg = seg.view(self.world, self.El, 4).transpose(0, 1).reshape(-1, 4)
        if self.S:
            s = torch.arange(self.S, device=flat.device)
            shared = torch.stack([torch.zeros_like(s), self.cap + s * self.Tl,
                                  torch.full_like(s, self.Tl), (self.El + s) | SEG_ALT_A], dim=1)
            seg = torch.cat([seg, shared], 0)
        return seg.to(torch.int32).contiguous()

    def forward(self, x, out=None, events=None):
        """events: optional list that receives (name, torch.cuda.Event) marks between phases."""
        st, G, El = self.stages, self.world, self.El

        def mark(name):
            if events is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                events.append((name, ev))

        if out is None:
            out = torch.empty_like(x)
        mark("start")
        st.router(self.desc_route, x, self.w, self.logits, self.idx, self.gate, self.block_counts)
        st.permute(self.desc_route, x, self.idx, self.block_counts, self.histogram, self.offsets,
                   self.row_src, self.slot_dst, self.x_perm)
        mark("router+permute")
        # counts: send[g][j] = my rows for expert g*El + j; recv[g][j] = rows rank g sends me
        send_counts = (self.offsets[1:] - self.offsets[:-1]).reshape(G, El).contiguous()
        dist.all_to_all_single(self.recv_counts, send_counts, group=self.group)
        both = torch.stack([send_counts.sum(1), self.recv_counts.sum(1)]).cpu()  # one host sync
        in_splits, out_splits = both[0].tolist(), both[1].tolist()
        n_recv = sum(out_splits)
        self.last_rows_received = n_recv
        mark("counts exchange + host sync")
        dist.all_to_all_single(self.recv[:n_recv], self.x_perm, out_splits, in_splits,
                               group=self.group)
        mark("dispatch all-to-all")
        seg = self.build_segments(self.recv_counts)
        st.expert_ffn(self.desc_ffn, self.recv, self.cap, x, self.Tl, seg, self.w, self.h, self.o,
                      self.rows_total, self.status)
        mark("segments + expert GEMMs")
        dist.all_to_all_single(self.o_back, self.o[:n_recv], in_splits, out_splits,
                               group=self.group)
        mark("return all-to-all")
        o_shared = self.o[self.cap:] if self.S else None
        st.combine(self.desc_comb, x, self.o_back, o_shared, self.slot_dst, self.gate, self.y, out)
        mark("combine")
        return out


class ExpertParallelMoeP2P:
    """The same sharded layer with the two exchanges done by this library's own
    kernels over NVLink peer memory (csrc/ep_exchange.cu) instead of NCCL
    all-to-alls: no host synchronisation inside a layer call, seven kernels in all.

    The exchange region is symmetric memory (torch.distributed._symmetric_memory):
    one allocation per rank, every rank holding the addresses of all of them.
    forward(x_local) -> out_local.  GPU only.

    fused_return=True lets the down GEMM's epilogue store the expert rows into the
    sources' buffers itself.  Measured on 8 B200s it is slower than the separate
    copy kernel (the epilogue writes one 128-byte piece per lane, which NVLink
    carries poorly; the copy kernel writes 512 contiguous bytes per warp), so the
    copy kernel is the default.
    """

    def __init__(self, local_weights, tokens_local, num_experts, top_k, group=None, residual=True,
                 fused_return=False, c_layer=True, h_exact=False):
        import torch.distributed._symmetric_memory as symm_mem
        self.fused_return = fused_return
        # c_layer: the whole call behind axm_moe_ep_forward (permute fused with the dispatch);
        # otherwise the stage-by-stage sequence below, which the fused-return variant also uses
        self.c_layer = c_layer and not fused_return
        self.lib = load()
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.stages = CudaStages()
        self.w = local_weights
        wr = local_weights["router_w"]
        self.dev = wr.device
        D = wr.shape[0]
        F = local_weights["w_gate"].shape[2]
        self.E, self.k, self.D, self.F = num_experts, top_k, D, F
        self.El = num_experts // self.world
        assert self.El * self.world == num_experts and local_weights["w_gate"].shape[0] == self.El
        self.S = 0 if local_weights.get("shared_gate") is None else local_weights["shared_gate"].shape[0]
        self.Tl = tokens_local
        rdt = ROUTER_FP32 if wr.dtype == torch.float32 else ROUTER_BF16
        flags = (FLAG_RESIDUAL if residual else 0) | (FLAG_H_EXACT if h_exact else 0)
        self.desc_route = make_desc(tokens_local, D, F, num_experts, top_k, 0, rdt, flags)
        self.desc_ffn = make_desc(tokens_local, D, F, self.El, min(top_k, self.El), self.S, rdt, flags)
        self.desc_comb = make_desc(tokens_local, D, F, num_experts, top_k, self.S, rdt, flags)
        self.desc_layer = make_desc(tokens_local, D, F, num_experts, top_k, self.S, rdt, flags)
        dev, i32, bf = self.dev, torch.int32, torch.bfloat16
        n_slots = tokens_local * top_k
        self.slots = n_slots
        self.cap = n_slots * self.world
        self.rows_total = self.cap + self.S * tokens_local
        self.n_seg = self.world * self.El + self.S

        self.layout = EpLayout()
        nbytes = ctypes.c_size_t(0)
        check(self.lib.axm_ep_region_bytes(self.world, num_experts, D, n_slots, self.cap,
                                           ctypes.byref(self.layout), ctypes.byref(nbytes)))
        self.region = symm_mem.empty(nbytes.value, dtype=torch.uint8, device=dev)
        self.handle = symm_mem.rendezvous(self.region, self.group)
        self.region.zero_()
        torch.cuda.synchronize()
        dist.barrier(self.group)
        self.layout.peers = self.handle.buffer_ptrs_dev
        self.layout.rank = self.rank
        self.layout.num_shared = self.S
        self.layout.tokens_local = tokens_local
        self.layout.local_region = self.region.data_ptr()
        lo = self.layout
        self.recv = self.region[lo.off_recv:lo.off_recv + 2 * self.cap * D].view(bf).view(self.cap, D)
        self.o_back = self.region[lo.off_oback:lo.off_oback + 4 * n_slots * D].view(
            torch.float32).view(n_slots, D)

        self.logits = torch.empty(tokens_local, num_experts, dtype=torch.float32, device=dev)
        self.idx = torch.empty(tokens_local, top_k, dtype=i32, device=dev)
        self.gate = torch.empty(tokens_local, top_k, dtype=torch.float32, device=dev)
        self.block_counts = torch.empty(ROUTE_BLOCKS, num_experts, dtype=i32, device=dev)
        self.histogram = torch.zeros(num_experts, dtype=i32, device=dev)
        self.offsets = torch.empty(num_experts + 1, dtype=i32, device=dev)
        self.row_src = torch.empty(n_slots, dtype=i32, device=dev)
        self.slot_dst = torch.empty(n_slots, dtype=i32, device=dev)
        self.x_perm = torch.empty(n_slots, D, dtype=bf, device=dev)
        self.y = torch.empty(tokens_local, D, dtype=bf, device=dev)
        self.step = 0
        if self.c_layer:
            nb, zb = ctypes.c_size_t(0), ctypes.c_size_t(0)
            check(self.lib.axm_moe_ep_workspace_bytes(ctypes.byref(self.layout), ctypes.byref(self.desc_layer),
                                                      ctypes.byref(nb), ctypes.byref(zb)))
            self.workspace = torch.empty(nb.value, dtype=torch.uint8, device=dev)
            self.workspace[:zb.value].zero_()
            ps, pr = ctypes.c_void_p(), ctypes.c_void_p()
            check(self.lib.axm_moe_ep_status_word(ctypes.byref(self.layout), ctypes.byref(self.desc_layer),
                                                  ptr(self.workspace), ctypes.byref(ps), ctypes.byref(pr)))
            base = self.workspace.data_ptr()
            self.status = self.workspace[ps.value - base:ps.value - base + 4].view(i32)
            self.rows_received = self.workspace[pr.value - base:pr.value - base + 4].view(i32)
            self.rows_received.zero_()
            return
        self.h = torch.empty(self.rows_total, F * (2 if h_exact else 1), dtype=bf, device=dev)
        self.o = torch.empty(self.rows_total, D, dtype=torch.float32, device=dev)
        self.status = torch.zeros(1, dtype=i32, device=dev)
        self.scratch = torch.zeros(2, dtype=i32, device=dev)
        self.segments = torch.zeros(self.n_seg, 4, dtype=i32, device=dev)
        self.ret_segments = torch.zeros(self.world * self.El, 4, dtype=i32, device=dev)
        self.remote_out = torch.zeros(self.n_seg, 2, dtype=torch.int64, device=dev)
        self.rows_received = torch.zeros(1, dtype=i32, device=dev)

    @property
    def last_rows_received(self):
        return int(self.rows_received.item())

    def check_status(self):
        """Reads the status word (synchronises this rank's stream) and raises AxmError with
        AXM_ERR_TIMEOUT if a bounded wait of an exchange or GEMM kernel gave up since the last
        check: the outputs of the calls in between must then be thrown away.  forward() never
        synchronises, so a caller decides how often to look (every step costs one host sync;
        once per optimiser step or per request batch is the usual place)."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise AxmError(AXM_ERR_TIMEOUT, f"a bounded device-side wait gave up (kernel code {code}) "
                                            f"on rank {self.rank}")

    def ep_tensors(self, x, out):
        w, S = self.w, self.S
        return EpTensors(
            x.data_ptr(), w["router_w"].data_ptr(),
            None if w.get("router_bias") is None else w["router_bias"].data_ptr(),
            w["w_gate"].data_ptr(), w["w_up"].data_ptr(), w["w_down"].data_ptr(),
            w["shared_gate"].data_ptr() if S else None, w["shared_up"].data_ptr() if S else None,
            w["shared_down"].data_ptr() if S else None, self.logits.data_ptr(), self.idx.data_ptr(),
            self.gate.data_ptr(), self.histogram.data_ptr(), self.y.data_ptr(), out.data_ptr())

    def forward_profiled(self, x, out=None):
        """forward() with device times of its seven phases (synchronises): returns (out, {name: ms})."""
        assert self.c_layer
        if out is None:
            out = torch.empty_like(x)
        self.step += 1
        t = self.ep_tensors(x, out)
        ms = (ctypes.c_float * 9)()
        check(self.lib.axm_moe_ep_forward_profiled(
            ctypes.byref(self.layout), ctypes.byref(self.desc_layer), ctypes.byref(t), ptr(self.workspace),
            self.workspace.numel(), self.step, current_stream(), ms))
        names = ["router", "permute + dispatch (peer stores)", "wait rows + segments", "gate/up GEMM",
                 "down GEMM", "return (peer stores)", "wait return + combine"]
        stages = dict(zip(names, list(ms)[:7]))
        if ms[8] > 0:   # the split return (AXM_EP_SPLIT_RETURN=1): when the first half's copy ran
            stages["first half's return: start after down GEMM start"] = ms[7]
            stages["first half's return: end after down GEMM start"] = ms[8]
        return out, stages

    def forward_host(self, h_x, h_out, d_x, d_out, chunks=0):
        """Activations in pinned host memory, copies pipelined with the exchange steps; synchronises.
        chunks = 0 leaves the number of parts to the library (two from 4096 tokens per rank on)."""
        assert self.c_layer
        t = self.ep_tensors(d_x, d_out)
        step = ctypes.c_uint32(self.step + 1)
        check(self.lib.axm_moe_ep_forward_host(
            ctypes.byref(self.layout), ctypes.byref(self.desc_layer), ctypes.byref(t), ptr(h_x), ptr(h_out),
            ptr(d_x), ptr(d_out), ptr(self.workspace), self.workspace.numel(), chunks, ctypes.byref(step),
            current_stream()))
        self.step = step.value - 1
        return h_out

    def forward(self, x, out=None, events=None):
        if self.c_layer:
            if out is None:
                out = torch.empty_like(x)
            self.step += 1
            t = self.ep_tensors(x, out)
            desc = self.desc_layer
            if x.shape[0] != self.Tl:
                # fewer tokens than the regions were sized for (an uneven last batch; the ranks need
                # not hold the same number): the call carries its own token count
                assert x.shape[0] <= self.Tl
                desc = make_desc(x.shape[0], self.D, self.F, self.E, self.k, self.S, desc.router_dtype, desc.flags)
            check(self.lib.axm_moe_ep_forward(ctypes.byref(self.layout), ctypes.byref(desc),
                                              ctypes.byref(t), ptr(self.workspace), self.workspace.numel(),
                                              self.step, current_stream()))
            return out
        st, lib, lo = self.stages, self.lib, ctypes.byref(self.layout)

        def mark(name):
            if events is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                events.append((name, ev))

        if out is None:
            out = torch.empty_like(x)
        self.step += 1
        stream = current_stream()
        mark("start")
        st.router(self.desc_route, x, self.w, self.logits, self.idx, self.gate, self.block_counts)
        st.permute(self.desc_route, x, self.idx, self.block_counts, self.histogram, self.offsets,
                   self.row_src, self.slot_dst, self.x_perm)
        mark("router+permute")
        check(lib.axm_ep_dispatch(lo, self.step, ptr(self.offsets), ptr(self.x_perm),
                                  ptr(self.scratch), ptr(self.status), stream))
        mark("dispatch (peer stores)")
        check(lib.axm_ep_segments(lo, self.step, ptr(self.segments), ptr(self.ret_segments),
                                  ptr(self.remote_out) if self.fused_return else None,
                                  ptr(self.rows_received), ptr(self.status), stream))
        mark("wait rows + segments")
        w, S = self.w, self.S
        if self.fused_return:
            # the down GEMM's epilogue stores each row into its source rank's return buffer
            check(lib.axm_moe_expert_ffn_remote(
                ctypes.byref(self.desc_ffn), ptr(self.recv), self.cap, ptr(x), self.Tl,
                ptr(self.segments), self.n_seg, ptr(w["w_gate"]), ptr(w["w_up"]), ptr(w["w_down"]),
                ptr(w["shared_gate"]) if S else None, ptr(w["shared_up"]) if S else None,
                ptr(w["shared_down"]) if S else None, ptr(self.h), ptr(self.o), self.rows_total,
                ptr(self.remote_out), ptr(self.status), stream))
            mark("expert GEMMs (return fused)")
            check(lib.axm_ep_signal_return(lo, self.step, stream))
        else:
            st.expert_ffn(self.desc_ffn, self.recv, self.cap, x, self.Tl, self.segments, self.w,
                          self.h, self.o, self.rows_total, self.status)
            mark("expert GEMMs")
            check(lib.axm_ep_return(lo, self.step, ptr(self.ret_segments), ptr(self.o),
                                    ptr(self.scratch), ptr(self.status), stream))
            mark("return (peer stores)")
        check(lib.axm_ep_wait_return(lo, self.step, ptr(self.status), stream))
        o_shared = self.o[self.cap:] if self.S else None
        st.combine(self.desc_comb, x, self.o_back, o_shared, self.slot_dst, self.gate, self.y, out)
        mark("wait return + combine")
        return out


class ExpertParallelTrainP2P:
    """Training step of the sharded layer (csrc/ep_train.cu): forward with the activations kept
    where they were produced, backward as the same exchange in reverse.  Two symmetric-memory
    regions (forward rows / gradient rows), both in the 64-row training layout.

    step(x_local, d_out_local) -> (out_local, aux_loss, grads): grads["d_x"] covers this rank's
    tokens, d_w_gate / d_w_up / d_w_down this rank's experts; d_router_w, d_router_bias and the
    auxiliary loss are summed over the ranks here (they share one buffer: one small all-reduce),
    because the router is replicated.  GPU only."""

    ALIGN = 64

    def __init__(self, local_weights, tokens_local, num_experts, top_k, group=None, aux_alpha=0.01,
                 weight_grads=True, tokens_global=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.lib = load()
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.w = local_weights
        wr = local_weights["router_w"]
        dev = self.dev = wr.device
        D = wr.shape[0]
        F = local_weights["w_gate"].shape[2]
        self.E, self.k, self.D, self.F = num_experts, top_k, D, F
        self.El = num_experts // self.world
        assert self.El * self.world == num_experts and local_weights["w_gate"].shape[0] == self.El
        self.Tl = tokens_local
        self.tokens_global = tokens_global if tokens_global is not None else tokens_local * self.world
        rdt = ROUTER_FP32 if wr.dtype == torch.float32 else ROUTER_BF16
        self.S = 0 if local_weights.get("shared_gate") is None else local_weights["shared_gate"].shape[0]
        self.desc = make_desc(tokens_local, D, F, num_experts, top_k, self.S, rdt, FLAG_RESIDUAL)
        n_slots = tokens_local * top_k
        cap = n_slots * self.world + (self.ALIGN - 1) * self.El
        self.cap = (cap + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        self.layouts, self.regions, self.handles = [], [], []
        for _ in range(2):   # forward rows, gradient rows
            lo = EpLayout()
            nbytes = ctypes.c_size_t(0)
            check(self.lib.axm_ep_region_bytes(self.world, num_experts, D, n_slots, self.cap,
                                               ctypes.byref(lo), ctypes.byref(nbytes)))
            region = symm_mem.empty(nbytes.value, dtype=torch.uint8, device=dev)
            handle = symm_mem.rendezvous(region, self.group)
            region.zero_()
            lo.peers = handle.buffer_ptrs_dev
            lo.rank = self.rank
            lo.num_shared = 0
            lo.tokens_local = tokens_local
            lo.local_region = region.data_ptr()
            lo.row_align = self.ALIGN
            self.layouts.append(lo)
            self.regions.append(region)
            self.handles.append(handle)
        torch.cuda.synchronize()
        dist.barrier(self.group)
        nb, zb = ctypes.c_size_t(0), ctypes.c_size_t(0)
        check(self.lib.axm_moe_ep_train_workspace_bytes(ctypes.byref(self.layouts[0]), ctypes.byref(self.desc),
                                                        ctypes.byref(nb), ctypes.byref(zb)))
        self.workspace = torch.empty(nb.value, dtype=torch.uint8, device=dev)
        self.workspace[:zb.value].zero_()
        ps, pr = ctypes.c_void_p(), ctypes.c_void_p()
        check(self.lib.axm_moe_ep_train_status_word(ctypes.byref(self.layouts[0]), ctypes.byref(self.desc),
                                                    ptr(self.workspace), ctypes.byref(ps), ctypes.byref(pr)))
        base = self.workspace.data_ptr()
        self.status = self.workspace[ps.value - base:ps.value - base + 4].view(torch.int32)
        self.rows_received = self.workspace[pr.value - base:pr.value - base + 4].view(torch.int32)
        self.rows_received.zero_()
        f32 = torch.float32
        self.out = torch.empty(tokens_local, D, dtype=torch.bfloat16, device=dev)
        # the three quantities that are summed over the ranks live in one buffer: one all-reduce
        has_bias = local_weights.get("router_bias") is not None
        n_wr = D * num_experts
        n_wr_pad = (n_wr + 3) // 4 * 4                    # keeps the bias gradient 16-byte aligned
        self.replicated = torch.zeros(n_wr_pad + (num_experts if has_bias else 0) + 1, dtype=f32, device=dev)
        self.d_router_w = self.replicated[:n_wr].view(D, num_experts)
        self.d_router_bias = self.replicated[n_wr_pad:n_wr_pad + num_experts] if has_bias else None
        self.aux = self.replicated[-1:]
        self.histogram = torch.zeros(num_experts, dtype=torch.int32, device=dev)
        self.d_x = torch.empty(tokens_local, D, dtype=f32, device=dev)
        self.weight_grads = weight_grads
        if weight_grads:
            self.d_w_gate = torch.empty(self.El, D, F, dtype=f32, device=dev)
            self.d_w_up = torch.empty(self.El, D, F, dtype=f32, device=dev)
            self.d_w_down = torch.empty(self.El, F, D, dtype=f32, device=dev)
            if self.S:      # replicated like the router: this rank's share, summed in backward()
                self.d_shared = torch.empty(self.S * (2 * D * F + F * D), dtype=f32, device=dev)
                n1 = self.S * D * F
                self.d_shared_gate = self.d_shared[:n1].view(self.S, D, F)
                self.d_shared_up = self.d_shared[n1:2 * n1].view(self.S, D, F)
                self.d_shared_down = self.d_shared[2 * n1:].view(self.S, F, D)
        self.aux_alpha = aux_alpha
        self.step_no = 0

    def check_status(self):
        """Raises AxmError(AXM_ERR_TIMEOUT) if a bounded device-side wait gave up since the last check
        (synchronises this rank's stream)."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise AxmError(AXM_ERR_TIMEOUT, f"a bounded device-side wait gave up (kernel code {code}) "
                                            f"on rank {self.rank}")

    def tensors(self, x, d_out):
        w, g = self.w, self.weight_grads
        return MoeTrain(
            x.data_ptr(), w["router_w"].data_ptr(),
            None if w.get("router_bias") is None else w["router_bias"].data_ptr(),
            w["w_gate"].data_ptr(), w["w_up"].data_ptr(), w["w_down"].data_ptr(),
            self.out.data_ptr(), self.aux.data_ptr(), self.histogram.data_ptr(), self.aux_alpha,
            None if d_out is None else d_out.data_ptr(), self.d_x.data_ptr(),
            self.d_router_w.data_ptr(), self.d_w_gate.data_ptr() if g else None,
            self.d_w_up.data_ptr() if g else None, self.d_w_down.data_ptr() if g else None,
            None if self.d_router_bias is None else self.d_router_bias.data_ptr(),
            w["shared_gate"].data_ptr() if self.S else None, w["shared_up"].data_ptr() if self.S else None,
            w["shared_down"].data_ptr() if self.S else None,
            self.d_shared_gate.data_ptr() if g and self.S else None,
            self.d_shared_up.data_ptr() if g and self.S else None,
            self.d_shared_down.data_ptr() if g and self.S else None)

    def forward(self, x, tokens_global=None):
        """Enqueues the forward pass; self.aux then holds this rank's share of the auxiliary loss.
        A rank may bring fewer tokens than the layer was sized for (an uneven last batch); then
        tokens_global is this step's token count over all ranks and out / d_x are used up to
        x.shape[0] rows."""
        self.step_no += 1
        t = self.tensors(x, None)
        self.step_desc, self.step_tokens = self.desc, self.tokens_global
        if x.shape[0] != self.Tl or tokens_global is not None:
            assert x.shape[0] <= self.Tl and tokens_global is not None
            d = self.desc
            self.step_desc = make_desc(x.shape[0], self.D, self.F, self.E, self.k, self.S, d.router_dtype, d.flags)
            self.step_tokens = tokens_global
        check(self.lib.axm_moe_ep_forward_train(ctypes.byref(self.layouts[0]), ctypes.byref(self.step_desc),
                                                ctypes.byref(t), self.step_tokens, ptr(self.workspace),
                                                self.workspace.numel(), self.step_no, current_stream()))
        return self.out[:x.shape[0]]

    def backward(self, x, d_out, reduce=True):
        """Enqueues the backward pass of the last forward(); reduce=True adds the replicated
        router's gradients (and the auxiliary loss) over the ranks."""
        t = self.tensors(x, d_out)
        check(self.lib.axm_moe_ep_backward(ctypes.byref(self.layouts[0]), ctypes.byref(self.layouts[1]),
                                           ctypes.byref(self.step_desc), ctypes.byref(t), self.step_tokens,
                                           ptr(self.workspace), self.workspace.numel(), self.step_no,
                                           current_stream()))
        if reduce:
            dist.all_reduce(self.replicated, group=self.group)
            if self.S and self.weight_grads:
                dist.all_reduce(self.d_shared, group=self.group)
        return self.d_x[:x.shape[0]]

    def step(self, x, d_out, reduce=True, tokens_global=None):
        out = self.forward(x, tokens_global=tokens_global)
        self.backward(x, d_out, reduce=reduce)
        grads = {"d_x": self.d_x[:x.shape[0]], "d_router_w": self.d_router_w}
        if self.d_router_bias is not None:
            grads["d_router_bias"] = self.d_router_bias
        if self.weight_grads:
            grads.update(d_w_gate=self.d_w_gate, d_w_up=self.d_w_up, d_w_down=self.d_w_down)
            if self.S:
                grads.update(d_shared_gate=self.d_shared_gate, d_shared_up=self.d_shared_up,
                             d_shared_down=self.d_shared_down)
        return out, self.aux, grads
