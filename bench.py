"""Benchmark of the MoE-layer hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--config C3] [--impl reference]

A step is one forward call of the layer over one batch of seeded synthetic
tokens.  N = 1 runs the whole layer on one GPU; N > 1 (under torchrun) runs it
expert-parallel: T/N tokens and E/N experts per rank, all-to-all dispatch and
return.  Rank 0 prints one JSON line.  `--impl reference` times the CPU
statement of the layer (the reference engine has no CPU implementation of its
own and its GPU kernels are single-GPU CUDA-core code) on the host cores.
"""
import argparse
import ctypes
import importlib
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG_DIR = os.path.join(ROOT, "project-axiom-ai-llm_b200")

# Fallback peaks, used only if MEASURED_PEAKS.json is absent.
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0

TRAFFIC_FILE = os.path.join(ROOT, "profiles", "dram_traffic_of_dominant_kernel.md")


def ncu_traffic(workload):
    """DRAM bytes (read + write) per launch of the gate/up GEMM for `workload`, from the
    committed ncu summary: lines of the form
    `traffic: workload=C3 ... read_bytes=N write_bytes=M commit=H`.  None when the file
    has no line for the workload."""
    import re
    try:
        text = open(TRAFFIC_FILE).read()
    except OSError:
        return None, None
    for line in text.splitlines():
        m = re.match(r"\s*traffic:\s+workload=(\S+)\s.*read_bytes=(\d+)\s+write_bytes=(\d+)\s+commit=(\S+)", line)
        if m and m.group(1) == workload:
            return int(m.group(2)) + int(m.group(3)), m.group(4)
    return None, None


def load_package():
    name = "project_axiom_ai_llm_b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(
        name, os.path.join(PKG_DIR, "__init__.py"), submodule_search_locations=[PKG_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS,
            "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50", "-i", str(self.index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        self.proc.wait()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        self.file.close()
        os.unlink(self.file.name)
        busy = [v for v in sm if v > 0.5 * max(sm)] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


def cpu_baseline(cfg, x, w, sample_tokens, repeats=1):
    """The CPU oracle timed on the first `sample_tokens` tokens of the batch."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_binding
    orc = oracle_binding.load()
    # every core this process may run on, whatever OMP_NUM_THREADS a launcher exported
    orc.set_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    n = min(sample_tokens, cfg.tokens)
    xs = x[:n].cpu()
    wc = {k: (v.cpu() if v is not None else None) for k, v in w.items()}
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        z = orc.router_logits(xs, wc["router_w"], wc.get("router_bias"))
        idx, gates, _, _, _ = orc.route(z, cfg.top_k)
        orc.permutation(idx, cfg.num_experts)
        orc.forward(xs, wc, idx, gates)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": n / best, "unit": "tokens/s", "cores": orc.threads(), "kind": "port",
            "sample": f"first {n} tokens of the batch through router, permutation and expert FFN "
                      f"(C, OpenMP, fp32 accumulate), {best:.2f} s; tokens/s = {n} / that time, i.e. scaled "
                      f"linearly in T, every slice streaming all expert weights once"}


def reference_gpu(cfg, wl, dev, repeats=30):
    """The reference engine's own, unmodified GPU kernels (oracle/_ref, built by
    oracle/build_ref.sh) timed on this GPU with CUDA events around forward_mixture_experts:
    median of `repeats` calls after warm-up, the hidden states restored before each call
    (the reference works in place), the histogram reset first.  Only the shapes it can run."""
    import ctypes
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import reference_binding
    if cfg.num_shared or cfg.top_k != 2 or cfg.num_experts > 16 or cfg.training:
        return {"unavailable": "the reference kernels do top-2 over at most 16 experts, forward only, "
                               "without shared experts or router bias"}
    if 2 * cfg.d_ff * 4 > 48 * 1024:
        return {"unavailable": f"the reference dispatch kernel needs {2 * cfg.d_ff * 4} bytes of dynamic shared "
                               "memory and never raises the 48 KiB default limit: its launch fails at this d_ff"}
    if not reference_binding.available():
        return {"unavailable": "oracle/_ref is not built (oracle/build_ref.sh)"}
    x, w = wl.make_inputs(cfg, device=dev, router_bf16=True)
    ref = reference_binding.ReferenceMoe()
    ref.set_weights(w["router_w"], w["w_gate"], w["w_up"], w["w_down"])
    hidden = x.clone()
    for _ in range(3):
        hidden.copy_(x)
        if not ref.forward(hidden, cfg.d_ff):
            return {"unavailable": "forward_mixture_experts returned false"}
    ref.reset_histogram()
    times = []
    for _ in range(repeats):
        hidden.copy_(x)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()            # torch's default stream is the legacy stream the reference enqueues on
        ok = bool(ref.lib.forward_mixture_experts(hidden.data_ptr(), ctypes.addressof(ref.weights),
                                                  ctypes.addressof(ref.acts), cfg.tokens, cfg.d_model,
                                                  cfg.d_ff, None))
        e1.record()
        torch.cuda.synchronize()
        if not ok:
            return {"unavailable": "forward_mixture_experts returned false"}
        times.append(e0.elapsed_time(e1))
    ms = statistics.median(times)
    return {"ms_per_step": ms, "value": cfg.tokens / (ms / 1000.0), "unit": "tokens/s", "calls": repeats,
            "what": "unmodified reference kernels (router, per-token dispatch on CUDA cores, residual) "
                    "compiled for sm_100a, bf16 router weights, device-resident inputs"}


def run_reference(args, wl):
    """--impl reference: the CPU statement of the layer on the host cores, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    cfg = wl.CONFIGS[args.config]
    sample = args.reference_tokens
    small = wl.scaled(cfg, tokens=sample)
    x, w = wl.make_inputs(small)
    times = []
    info = None
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        info = cpu_baseline(small, x, w, sample)
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    ms = 1000.0 * sum(times) / len(times)
    value = sample / (ms / 1000.0)
    info["value"] = value
    line = {
        "impl": "reference", "metric": "MoE-layer tokens/s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "gpu_launches": 0,
        "config": workload_config(cfg, args.gpus),
        "cpu_baseline": info,
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference engine has no CPU MoE path; this is the CPU port of its layer "
                "semantics (oracle/), all host threads",
    }
    print(json.dumps(line), flush=True)


def workload_config(cfg, n_gpus):
    l2_note = ("inputs larger than L2 (expert weights "
               f"{cfg.weight_bytes / n_gpus / 1e9:.2f} GB per GPU); no flush")
    return {
        "workload": f"{cfg.name}: MoE layer {'training step (forward + backward)' if cfg.training else 'forward'}, T={cfg.tokens} d_model={cfg.d_model} "
                    f"E={cfg.num_experts}+{cfg.num_shared} shared top-{cfg.top_k} d_ff={cfg.d_ff}, "
                    f"seed {cfg.seed}",
        "tokens": cfg.tokens, "d_model": cfg.d_model, "num_experts": cfg.num_experts,
        "top_k": cfg.top_k, "d_ff": cfg.d_ff, "num_shared": cfg.num_shared,
        "parallelism": "single GPU" if n_gpus == 1 else f"expert-parallel ep{n_gpus} "
                       f"({cfg.num_experts // n_gpus} experts and {cfg.tokens // n_gpus} tokens per GPU)",
        "l2": l2_note,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--config", default="C3", choices=["C1", "C2", "C3", "C4", "C5"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-tokens", type=int, default=512, help="tokens in the CPU baseline sample")
    ap.add_argument("--reference-tokens", type=int, default=512)
    ap.add_argument("--sustained-seconds", type=float, default=2.0,
                    help="length of the extra back-to-back loop that gives the steady-state rate (0: skip)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tokens", type=int, default=0,
                    help="override the workload's token count (e.g. 16 for a decode-sized batch)")
    ap.add_argument("--ep-transport", default="p2p", choices=["p2p", "nccl"],
                    help="N > 1: own peer-memory exchange kernels, or NCCL all-to-all")
    ap.add_argument("--ep-host-chunks", type=int, default=0,
                    help="N > 1: parts the host-buffer call cuts each rank's tokens into (every part is a "
                         "whole exchange step, whose fixed cost outweighs the hidden copies at 8 GPUs)")
    ap.add_argument("--ep-stages", action="store_true",
                    help="p2p transport: the stage-by-stage sequence from Python instead of axm_moe_ep_forward")
    ap.add_argument("--ep-return", default="copy", choices=["fused", "copy"],
                    help="p2p transport: expert rows returned from the down GEMM's epilogue, or "
                         "by a separate copy kernel")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    axm = load_package()
    wl = importlib.import_module("project_axiom_ai_llm_b200.workloads")
    if args.impl == "reference":
        run_reference(args, wl)
        return

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torchrun")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the MoE layer has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    cfg = wl.CONFIGS[args.config]
    if args.tokens > 0:
        cfg = wl.scaled(cfg, tokens=args.tokens, name=f"{cfg.name}@T{args.tokens}")
    peaks = measured_peaks()
    T, D, k = cfg.tokens, cfg.d_model, cfg.top_k
    x, w = wl.make_inputs(cfg, device=dev)  # same seed on every rank -> same tensors
    launches_per_step = 0

    training = cfg.training
    if training and world > 1:
        # the same step sharded: tokens and experts over the ranks, both exchanges by this library's
        # peer-memory kernels, the replicated router's gradients summed with one small all-reduce
        ep = importlib.import_module("project_axiom_ai_llm_b200.expert_parallel")
        assert T % world == 0 and cfg.num_experts % world == 0
        tl = T // world
        x_local = x[rank * tl:(rank + 1) * tl].contiguous()
        wloc = ep.shard_weights(w, rank, world)
        del w
        layer = ep.ExpertParallelTrainP2P(wloc, tl, cfg.num_experts, k, aux_alpha=cfg.aux_alpha)
        d_out = torch.randn(T, D, device=dev, generator=torch.Generator(device=dev).manual_seed(cfg.seed))
        d_out = d_out[rank * tl:(rank + 1) * tl].contiguous()
        out = layer.out
        step = lambda: layer.step(x_local, d_out)
        # forward: router, permute + dispatch, segment tables (2), padding, two GEMMs, auxiliary loss (2),
        # return, wait, combine; backward: prepare, dispatch, segment tables (2), padding, dH, dX, three
        # weight-gradient GEMMs, return, wait, router gradient, dWr (2), dX assembly
        launches_per_step = 12 + 16 + (1 if axm.router_scratch_bytes(layer.desc) else 0)
    elif training:
        # forward (saving activations) + auxiliary loss + backward with all weight gradients
        layer = axm.MoeTrainLayer(w, T, k, aux_alpha=cfg.aux_alpha)
        x_local = x
        d_out = torch.randn(T, D, device=dev, generator=torch.Generator(device=dev).manual_seed(cfg.seed))
        out = layer.out
        step = lambda: layer.step(x_local, d_out)
        launches_per_step = 17 + (1 if axm.router_scratch_bytes(layer.desc) else 0)
    elif world == 1:
        layer = axm.MoeLayer(w, T, k, publish_y=False)
        out = torch.empty_like(x)
        x_local = x
        step = lambda: layer.forward(x_local, out)
        launches_per_step = layer.lib.axm_moe_forward_launches(ctypes.byref(layer.desc))
    else:
        ep = importlib.import_module("project_axiom_ai_llm_b200.expert_parallel")
        assert T % world == 0 and cfg.num_experts % world == 0
        tl = T // world
        x_local = x[rank * tl:(rank + 1) * tl].contiguous()
        wloc = ep.shard_weights(w, rank, world)
        del w
        if args.ep_transport == "p2p":
            layer = ep.ExpertParallelMoeP2P(wloc, tl, cfg.num_experts, k,
                                            fused_return=(args.ep_return == "fused"),
                                            c_layer=not args.ep_stages)
        else:
            layer = ep.ExpertParallelMoe(wloc, tl, cfg.num_experts, k)
        out = torch.empty_like(x_local)
        step = lambda: layer.forward(x_local, out)
        # p2p behind axm_moe_ep_forward: router (+ its preparation kernel), permute fused with the
        # dispatch, segment tables, gate/up GEMM, down GEMM, return copy, wait, combine.
        # nccl: router, permute, two GEMMs, combine plus library collectives.
        c_layer = getattr(layer, "c_layer", False)
        launches_per_step = (8 if c_layer else (9 if args.ep_transport == "p2p" else 5)) + \
            (1 if axm.router_scratch_bytes(layer.desc_route) else 0)
    del x
    torch.cuda.empty_cache()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = T / (ms_step / 1000.0)

    # ---- steady state: the same step back to back for a few seconds ---------------
    sustained = None
    if args.sustained_seconds > 0:
        n_loop = max(args.steps, int(args.sustained_seconds * 1000.0 / ms_step) + 1)
        s_sampler = ClockSampler(local_rank)
        barrier()
        if rank == 0:
            s_sampler.start()
        e0.record()
        for _ in range(n_loop):
            step()
        e1.record()
        barrier()
        s_ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([s_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            s_ms = float(t.item())
        if rank == 0:
            sc = s_sampler.stop()
            s_step = s_ms / n_loop
            sustained = {"steps": n_loop, "seconds": s_ms / 1000.0, "ms_per_step": s_step,
                         "value": T / (s_step / 1000.0), "unit": "tokens/s", "clocks": sc,
                         "ms_x_sm_mhz": s_step * sc["sm_mhz"] if sc.get("sm_mhz") else None}

    # ---- the strict-tolerance mode (two-term SwiGLU intermediate) -------------------
    h_exact = None
    if world == 1 and not training:
        layer_x = axm.MoeLayer(layer.w, T, k, publish_y=False, h_exact=True)
        for _ in range(3):
            layer_x.forward(x_local, out)
        barrier()
        e0.record()
        for _ in range(args.steps):
            layer_x.forward(x_local, out)
        e1.record()
        barrier()
        hx_ms = e0.elapsed_time(e1) / args.steps
        if layer_x.status() != 0:
            raise SystemExit("GEMM kernel reported a timed-out wait (exact mode)")
        h_exact = {"ms_per_step": hx_ms, "value": T / (hx_ms / 1000.0), "unit": "tokens/s",
                   "what": "AXM_FLAG_H_EXACT: SwiGLU intermediate kept as two bf16 terms, every output "
                           "element within 1e-2 + 2e-2*|ref| of an fp32 intermediate"}
        del layer_x
        torch.cuda.empty_cache()

    # ---- end to end: host buffers, copies inside the timed region ----------------
    h_x = x_local.cpu().pin_memory()
    h_out = torch.empty_like(h_x).pin_memory()
    d_x = torch.empty_like(x_local)
    if training:
        h_dy = d_out.cpu().pin_memory()
        h_dx = torch.empty_like(h_dy).pin_memory()
        d_dy = torch.empty_like(d_out)

        copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
        ev_dy, ev_fwd, ev_free = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()

        def e2e_step():
            # the upstream gradient comes in while the forward pass runs, the output goes out while
            # the backward pass runs; x in and d_x out are the exposed copies
            cur = torch.cuda.current_stream()
            ev_free.record(cur)                  # the previous step's reads of d_dy are done
            copy_in.wait_event(ev_free)
            d_x.copy_(h_x, non_blocking=True)
            with torch.cuda.stream(copy_in):
                d_dy.copy_(h_dy, non_blocking=True)
                ev_dy.record(copy_in)
            layer.forward(d_x)
            ev_fwd.record(cur)
            copy_out.wait_event(ev_fwd)
            with torch.cuda.stream(copy_out):
                h_out.copy_(layer.out, non_blocking=True)
            cur.wait_event(ev_dy)
            layer.backward(d_x, d_dy)
            h_dx.copy_(layer.d_x, non_blocking=True)
            cur.synchronize()
            copy_out.synchronize()
    elif world == 1:
        e2e_step = lambda: layer.forward_host(h_x, h_out, d_x, out)
    elif getattr(layer, "c_layer", False):
        # host buffers through axm_moe_ep_forward_host
        e2e_step = lambda: layer.forward_host(h_x, h_out, d_x, out, chunks=args.ep_host_chunks)
    else:
        def e2e_step():
            d_x.copy_(h_x, non_blocking=True)
            layer.forward(d_x, out)
            h_out.copy_(out, non_blocking=True)
            torch.cuda.current_stream().synchronize()
    for _ in range(3):
        e2e_step()
    barrier()
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_ms /= args.steps
    # ---- the same with a run of batches in flight: axm_moe_forward_host_batches ------------
    e2e_stream = None
    if world == 1 and not training:
        n_b = max(2, min(args.steps, 64))
        h_x_b = torch.empty_like(h_x).pin_memory()
        h_x_b.copy_(h_x)
        h_out_b = torch.empty_like(h_out).pin_memory()
        d_x2 = torch.empty(2 * T, D, dtype=torch.bfloat16, device=dev)
        d_out2 = torch.empty_like(d_x2)
        h_xs = [h_x if i % 2 == 0 else h_x_b for i in range(n_b)]
        h_outs = [h_out if i % 2 == 0 else h_out_b for i in range(n_b)]
        layer.forward_host_batches(h_xs[:3], h_outs[:3], d_x2, d_out2)
        barrier()
        e0.record()
        layer.forward_host_batches(h_xs, h_outs, d_x2, d_out2)
        e1.record()
        barrier()
        es_ms = e0.elapsed_time(e1) / n_b
        e2e_stream = {"value": T / (es_ms / 1000.0), "unit": "tokens/s", "ms_per_step": es_ms, "batches": n_b,
                      "h2d_bytes_per_step": h_x.numel() * 2, "d2h_bytes_per_step": h_x.numel() * 2,
                      "what": "one call over a run of host batches, double-buffered on the device: every "
                              "batch is copied in, computed and copied out inside the timed region, batch "
                              "i + 1's copy in and batch i - 1's copy out overlap batch i's compute"}
        del d_x2, d_out2
    clocks = sampler.stop() if rank == 0 else None
    copy_bytes = h_x.numel() * 2 * world
    h2d_bytes = copy_bytes + (h_dy.numel() * 4 * world if training else 0)
    d2h_bytes = copy_bytes + (h_dx.numel() * 4 * world if training else 0)

    # ---- roofline of the dominant kernel (gate/up grouped GEMM) ---------------------
    roofline = None
    stages = None
    if training:
        # nine grouped tensor-core GEMMs per step: 6TkDF forward, 12TkDF backward
        fl = 3.0 * cfg.gemm_flops
        tf = fl / (ms_step * 1e-3) / 1e12
        roofline = {"kernel": "all grouped GEMMs of the training step (whole-step time)",
                    "bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"] * world, "unit": "TFLOP/s",
                    "frac": tf / (peaks["bf16_tflops"] * world),
                    "peak_source": peaks["source"] + (" (burst)" if world == 1 else f" (burst) x {world} GPUs"),
                    "traffic": None}
        status = int(layer.status.item()) if world > 1 else int(layer.workspace[:4].view(torch.int32).item())
        if status != 0:
            raise SystemExit(f"a GEMM kernel reported a timed-out wait (status {status})")
    elif world == 1:
        acc = [0.0] * 5
        reps = 10
        for _ in range(reps):
            _, ms = layer.forward_profiled(x_local, out)
            acc = [a + m for a, m in zip(acc, ms)]
        stage_ms = [a / reps for a in acc]
        names = ["router", "permute", "gate_up_gemm", "down_gemm", "combine"]
        sb = cfg.stage_bytes(4)
        rows = T * (k + cfg.num_shared)
        flops_gu = 4.0 * rows * D * cfg.d_ff
        flops_dn = 2.0 * rows * D * cfg.d_ff
        stages = {n: {"ms": m} for n, m in zip(names, stage_ms)}
        for n in ("router", "permute", "combine"):
            gbs = sb[n] / (stages[n]["ms"] * 1e-3) / 1e9
            stages[n].update({"bytes": sb[n], "gb_s": gbs, "frac_hbm": gbs / peaks["hbm_gbs"]})
        for n, fl in (("gate_up_gemm", flops_gu), ("down_gemm", flops_dn)):
            tf = fl / (stages[n]["ms"] * 1e-3) / 1e12
            stages[n].update({"flops": fl, "tflop_s": tf, "frac_tensor": tf / peaks["bf16_tflops"]})
        a = stages["gate_up_gemm"]["tflop_s"]
        two_sm = os.environ.get("AXM_GEMM_2SM", "1")[:1] != "0"
        roofline = {"kernel": ("grouped_gemm_2sm_kernel<SwiGLU>" if two_sm else "grouped_gemm_kernel<SwiGLU>") +
                              " (gate/up)", "bound": "tensor",
                    "achieved": a, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": a / peaks["bf16_tflops"], "peak_source": peaks["source"] + " (burst)",
                    "frac_of_sustained": a / peaks["bf16_tflops_sustained"] if peaks["bf16_tflops_sustained"] else None,
                    "traffic": ncu_traffic(cfg.name)[0], "traffic_commit": ncu_traffic(cfg.name)[1]}
        status = layer.status()
        if status != 0:
            raise SystemExit(f"GEMM kernel reported a timed-out wait (status {status})")

    ep_stages = None
    if world > 1 and training:
        # forward and backward halves of the sharded step (rank 0's events; each includes waiting for peers)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        acc = [0.0, 0.0]
        reps = 10
        for _ in range(reps):
            barrier()
            ev[0].record()
            layer.forward(x_local)
            ev[1].record()
            layer.backward(x_local, d_out)
            ev[2].record()
            torch.cuda.synchronize()
            acc[0] += ev[0].elapsed_time(ev[1]) / reps
            acc[1] += ev[1].elapsed_time(ev[2]) / reps
        ep_stages = {"forward (saves activations, auxiliary loss)": {"ms": acc[0]},
                     "backward (incl. the all-reduce of the router gradients)": {"ms": acc[1]},
                     "rows_received_rank0": int(layer.rows_received.item())}
    if world > 1 and not training:
        acc = {}
        reps = 10
        for _ in range(reps):
            if getattr(layer, "c_layer", False):
                _, ms = layer.forward_profiled(x_local, out)
                for n, v in ms.items():
                    acc[n] = acc.get(n, 0.0) + v / reps
            else:
                evs = []
                layer.forward(x_local, out, events=evs)
                torch.cuda.synchronize()
                for (_, a), (n, b) in zip(evs[:-1], evs[1:]):
                    acc[n] = acc.get(n, 0.0) + a.elapsed_time(b) / reps
        ep_stages = {n: {"ms": v} for n, v in acc.items()}
        ep_stages["rows_received_rank0"] = layer.last_rows_received

    # ---- expert parallel: the answer itself, against the single-GPU layer ------------
    ep_check = None
    ep_failed = False
    if world > 1 and training:
        # the sharded training step against the single-GPU step on the same seeded batch: output
        # and input gradient bit for bit
        layer.check_status()
        layer.step(x_local, d_out)
        mine = [layer.out.clone(), layer.d_x.clone()]
        gathered = []
        for t_ in mine:
            parts = [torch.empty_like(t_) for _ in range(world)] if rank == 0 else None
            dist.gather(t_, parts, dst=0)
            gathered.append(parts)
        verdict = torch.zeros(1, dtype=torch.int32, device=dev)
        if rank == 0:
            xs, ws = wl.make_inputs(cfg, device=dev)
            dy = torch.randn(T, D, device=dev, generator=torch.Generator(device=dev).manual_seed(cfg.seed))
            single = axm.MoeTrainLayer(ws, T, k, aux_alpha=cfg.aux_alpha, weight_grads=False)
            single.step(xs, dy)
            torch.cuda.synchronize()
            same = (torch.equal(torch.cat(gathered[0]), single.out) and
                    torch.equal(torch.cat(gathered[1]), single.d_x))
            ep_check = "bit-equal (out, d_x)" if same else "MISMATCH"
            verdict[0] = 0 if same else 1
            del single, ws, xs, dy, gathered
        dist.broadcast(verdict, src=0)
        ep_failed = int(verdict.item()) != 0
    elif world > 1:
        if hasattr(layer, "check_status"):
            layer.check_status()
        out_final = layer.forward(x_local, out).clone()
        gathered = [torch.empty_like(out_final) for _ in range(world)] if rank == 0 else None
        dist.gather(out_final, gathered, dst=0)
        verdict = torch.zeros(1, dtype=torch.int32, device=dev)
        if rank == 0:
            xs, ws = wl.make_inputs(cfg, device=dev)      # the same seeded batch, all experts
            single = axm.MoeLayer(ws, T, k, publish_y=False)
            ref_out, _ = single.forward(xs)
            torch.cuda.synchronize()
            same = torch.equal(torch.cat(gathered), ref_out)
            ep_check = "bit-equal" if same else "MISMATCH"
            if not same:
                diff = (torch.cat(gathered).float() - ref_out.float()).abs()
                ep_check += f": {int((diff > 0).sum())} elements differ, max |diff| {float(diff.max()):.4g}"
            verdict[0] = 0 if same else 1
            del single, ws, xs, ref_out, gathered
        dist.broadcast(verdict, src=0)
        ep_failed = int(verdict.item()) != 0

    cpu = None
    if world == 1 and rank == 0 and not args.no_cpu_baseline and not training:
        cpu = cpu_baseline(cfg, x_local, layer.w, args.cpu_tokens)
    ref_gpu = None
    if world == 1 and rank == 0 and not training:
        ref_gpu = reference_gpu(cfg, wl, dev)

    if rank == 0:
        line = {
            "metric": "MoE-layer tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": workload_config(cfg, world),
            "e2e": {"value": T / (e2e_ms / 1000.0), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes},
            "gpu_launches": launches_per_step * args.steps * world,
            "clocks": clocks,
            "gemm_tflops_layer": (3 if training else 1) * cfg.gemm_flops / (ms_step * 1e-3) / 1e12,
            "gemm_frac_of_peak_layer": (3 if training else 1) * cfg.gemm_flops / (ms_step * 1e-3) / 1e12
                                       / (peaks["bf16_tflops"] * world),
        }
        if training:
            line["metric"] = "MoE-layer training step tokens/s (forward + backward)"
        if roofline is not None:
            line["roofline"] = roofline
        if stages is not None:
            line["stages"] = stages
        if world > 1 and training:
            line["config"]["ep_transport"] = "p2p"
        if ep_stages is not None and training:
            line["stages_rank0"] = ep_stages
        elif ep_stages is not None:
            line["stages_rank0"] = ep_stages
            line["config"]["ep_transport"] = args.ep_transport
            if args.ep_transport == "p2p":
                line["config"]["ep_return"] = args.ep_return
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if ref_gpu is not None:
            line["reference_gpu"] = ref_gpu
        if sustained is not None:
            line["sustained"] = sustained
        if h_exact is not None:
            line["h_exact"] = h_exact
        if e2e_stream is not None:
            line["e2e_stream"] = e2e_stream
        if ep_check is not None:
            line["ep_check"] = ep_check
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if ep_failed:
        raise SystemExit("expert-parallel output differs from the single-GPU layer's")


if __name__ == "__main__":
    main()
