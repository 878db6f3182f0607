#!/usr/bin/env python
"""Benchmark of the paged-KV decode hot path: K/V append + paged decode attention over
every layer of one decode step, on synthetic data with the shapes of the benchmark
configurations.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg3|cfg2|cfg1|cfg5]
                    [--impl ours|reference] [--no-graph]

One JSON line is printed by rank 0.  A "step" is one pass of the hot path over one batch:
for every layer, append the batch's new K/V rows to their slots, then run paged decode
attention for every sequence over its whole (fragmented) history.  Weak scaling: every
rank owns its own block pool and its own batch (same shapes, different seed); there is no
data-path collective, only a barrier and a max-reduction of the device time.

  value     tokens/s with every input resident in HBM when the timed region starts
            (CUDA-graph replay of the step unless --no-graph).
  e2e       the same step driven from HOST buffers through the public operators: per
            step the index arrays and every layer's q/k/v rows go host->device from
            pinned memory and every layer's attention output comes back.
  roofline  achieved HBM GB/s of the decode attention kernel: algorithmic bytes per launch
            divided by the mean launch time, CUDA events around each launch in an
            instrumented pass that follows the timed region.
  cpu_baseline  the reference's own CPU path (oracle/_ref, built from its sources) or the C
            restatement, timed on this host on a bounded sample (N=1, rank 0 only).
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOAD_TEXT = {
    "cfg1": "one Qwen2.5-0.5B attention layer (14q/2kv heads, d64), fp32 KV, 8 seqs, ctx U[64,512], block 16, 4096-block shuffled pool",
    "cfg2": "Qwen2.5-0.5B decode step: 24 layers, 14q/2kv heads, d64, bf16 KV, 64 seqs, ctx U[256,2048], block 16, shuffled pool",
    "cfg3": "TinyLlama-1.1B decode step: 22 layers, 32q/4kv heads, d64, bf16 KV, 256 seqs, ctx log-uniform [128,8192], block 16, fragmented 65536-block pool per layer",
    "cfg4": "chunked prefill, Qwen2.5-0.5B attention shapes (14q/2kv heads, d64), bf16: 32 seqs, cached context U[0,1536] + 512-token chunk, causal over cached+new, block 16, shuffled tables; one step = append + prefill attention for 24 layers",
    "cfg5": "prefix-cache decode: TinyLlama shapes, 22 layers, 128 seqs sharing a 512-token prefix + suffix U[32,256], bf16 KV, block 16",
}
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) per launch of the decode attention kernel, from the
# ncu captures summarised under profiles/ (same per-launch workload as the default seed of each configuration).
NCU_TRAFFIC = {
    "cfg3": {"bytes": 429279488, "source": "profiles/decode_tma_kernel_cfg3_ncu_full.md (421.21 MB read + 8.07 MB written)"},
}
METRIC = "decode tok/s (K/V append + paged decode attention over all layers)"


def peaks(key="hbm_gbs", fallback=6650.0):
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)[key]), "measured (MEASURED_PEAKS.json)"
    return fallback, "fallback (earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs (read-only NVML)."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.002)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


# ------------------------------------------------------------------------------------
# CPU arm: the reference's own implementation of the path on the host cores.
# ------------------------------------------------------------------------------------
def cpu_step_sample(w, checker, threads, layer_pools=None, seed=0):
    """Times ONE layer of the step (append + attention for every sequence) on the host and
    returns (seconds for that layer, description).  Pools are fp32, as in the reference's CPU
    backend; bf16 workloads are rounded to bf16 and widened first."""
    import oracle
    orc = oracle.load_orc()
    pkv = importlib.import_module("llm-engine_b200")
    rng = np.random.default_rng(seed)
    bs, kv_dim = w.block_size, w.kv_dim
    tabs, pos, _ = w.step_tokens()
    idx = pkv.pack_step(tabs, pos, bs)
    N = idx.n_tokens
    slots_total = w.num_blocks * bs
    if layer_pools is not None:
        kc, vc = layer_pools
    else:
        # Only slots that some sequence owns are read; filling the whole pool costs host time for nothing.
        kc = np.zeros((slots_total, kv_dim), dtype=np.float32)
        vc = np.zeros((slots_total, kv_dim), dtype=np.float32)
        used = np.unique(idx.block_tables)
        rows = (used[:, None].astype(np.int64) * bs + np.arange(bs)[None, :]).reshape(-1)
        for a in (kc, vc):
            vals = rng.standard_normal((rows.size, kv_dim), dtype=np.float32)
            a[rows] = orc.from_bf16_bits(orc.to_bf16_bits(vals)) if w.dtype == "bf16" else vals
    cast = (lambda a: orc.from_bf16_bits(orc.to_bf16_bits(a))) if w.dtype == "bf16" else (lambda a: a)
    q = cast(rng.standard_normal((N, w.q_heads * w.head_dim), dtype=np.float32))
    k = cast(rng.standard_normal((N, kv_dim), dtype=np.float32))
    v = cast(rng.standard_normal((N, kv_dim), dtype=np.float32))

    def one_layer():
        t0 = time.perf_counter()
        checker.append(k, v, idx.slots, kc, vc)
        checker.paged_attention(q, kc, vc, idx.block_tables, idx.table_offset, idx.token_seq, idx.token_pos,
                                w.q_heads, w.kv_heads, w.head_dim, bs, w.scale, threads=threads)
        return time.perf_counter() - t0

    return one_layer, N


def run_reference_arm(args, rank, world):
    """--impl reference: the reference's CPU implementation, all host threads, bounded sample per step."""
    if rank != 0:
        return
    import oracle
    wl = importlib.import_module("llm-engine_b200.workloads")
    checker = oracle.load_ref()
    kind = "reference"
    if checker is None:
        checker, kind = oracle.load_orc(), "port"
    threads = oracle.ref_default_thread_count()
    w = wl.make(args.workload)
    one_layer, N = cpu_step_sample(w, checker, threads)
    for _ in range(max(1, min(args.warmup, 1))):
        one_layer()
    steps = max(1, min(args.steps, 5))
    times = [one_layer() for _ in range(steps)]
    t_layer = float(np.mean(times))
    t_step = t_layer * w.layers
    value = N / t_step
    sample = f"each step = 1 of {w.layers} layers over all {w.n_seqs} sequences (append + attention), scaled x{w.layers}; {steps} steps timed"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": 1, "ms_per_step": t_step * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {WORKLOAD_TEXT[args.workload]}", "device": "host CPU",
                   "note": "the reference's CPU backend is fp32; bf16 inputs are rounded to bf16 and widened"},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------
def run_ours(args, rank, local_rank, world):
    import torch
    import torch.distributed as dist

    pkv = importlib.import_module("llm-engine_b200")
    wl = importlib.import_module("llm-engine_b200.workloads")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    sh = importlib.import_module("llm-engine_b200.sharding")
    # Weak scaling: every rank gets the configuration's batch with the SAME lengths and table shapes
    # (fixed work per GPU); only the tensor contents differ per rank (generator seeds below).
    w = wl.make(args.workload, layers=args.layers)
    tdt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[w.dtype]
    bs, kv_dim, L = w.block_size, w.kv_dim, w.layers
    H = w.q_heads * w.head_dim
    tabs, pos, _ = w.step_tokens()
    idx = pkv.pack_step(tabs, pos, bs)
    N = idx.n_tokens
    slots_total = w.num_blocks * bs

    g = torch.Generator(device=dev).manual_seed(77 + rank)
    pools = torch.empty((L, 2, slots_total, kv_dim), dtype=tdt, device=dev)
    for l in range(L):       # N(0,1) values, generated layer by layer to bound the fp32 temporary
        for j in range(2):
            pools[l, j].copy_(torch.randn((slots_total, kv_dim), generator=g, device=dev, dtype=torch.float32))
    q = torch.randn((L, N, H), generator=g, device=dev, dtype=torch.float32).to(tdt)
    k = torch.randn((L, N, kv_dim), generator=g, device=dev, dtype=torch.float32).to(tdt)
    v = torch.randn((L, N, kv_dim), generator=g, device=dev, dtype=torch.float32).to(tdt)
    out = torch.zeros((L, N, H), dtype=tdt, device=dev)
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
    d_slots, d_seq, d_pos = i32(idx.slots), i32(idx.token_seq), i32(idx.token_pos)
    d_tab, d_off = i32(idx.block_tables), i32(idx.table_offset)
    plan = pkv.DecodePlan(N, w.q_heads, w.kv_heads, w.head_dim, device=dev)
    # per-layer views made once, so the timed loops only issue launches
    kc_l, vc_l = [pools[l, 0] for l in range(L)], [pools[l, 1] for l in range(L)]
    q_l, k_l, v_l, out_l = [q[l] for l in range(L)], [k[l] for l in range(L)], [v[l] for l in range(L)], [out[l] for l in range(L)]

    # Decode steps on the TMA kernel can take the append inside the attention launch (one kernel per
    # layer fewer).  That pays where the launch chain dominates (configuration 2: +11 %); on
    # configuration 3 it measures the same as the reference's two calls per layer, which then stay the
    # default so that the attention launch is timed by itself.  --append fused|separate overrides.
    fused = w.dtype != "f32" and (args.append == "fused" or (args.append == "auto" and N * w.kv_heads < 1024))

    def layer(l, qq, kk, vv, oo):
        if fused:
            plan.append_attention(qq, kk, vv, d_slots, kc_l[l], vc_l[l], d_tab, d_off, d_seq, d_pos, oo, bs, w.scale)
        else:
            pkv.launch_store_kv(kk, vv, d_slots, kc_l[l], vc_l[l], N, kv_dim)
            plan.attention(qq, kc_l[l], vc_l[l], d_tab, d_off, d_seq, d_pos, oo, bs, w.scale)

    def step_resident():
        plan.build_host(idx.token_pos)
        for l in range(L):
            layer(l, q_l[l], k_l[l], v_l[l], out_l[l])

    launches_per_step = (2 if fused else 3) * L      # kernels: [append,] attention, merge

    # ---- end-to-end step: host buffers in, host buffers out --------------------------
    pin = lambda t: t.cpu().pin_memory()
    h_q, h_k, h_v = pin(q), pin(k), pin(v)
    h_out = torch.empty((L, N, H), dtype=tdt).pin_memory()
    h_idx = [torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).pin_memory()
             for a in (idx.slots, idx.token_seq, idx.token_pos, idx.block_tables, idx.table_offset)]
    d_idx = [d_slots, d_seq, d_pos, d_tab, d_off]
    e_q, e_k, e_v = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    e_out = torch.empty_like(out)
    h2d_bytes = sum(t.numel() * t.element_size() for t in (h_q, h_k, h_v)) + sum(t.numel() * 4 for t in h_idx)
    d2h_bytes = h_out.numel() * h_out.element_size()
    copy_stream = torch.cuda.Stream(device=dev)
    out_stream = torch.cuda.Stream(device=dev)

    def step_e2e():
        """Index arrays first, then layer l's q/k/v rows are uploaded on a copy stream while layer
        l-1 computes, and layer l's output goes back while layer l+1 computes."""
        main = torch.cuda.current_stream()
        for hs, ds in zip(h_idx, d_idx):
            ds.copy_(hs, non_blocking=True)
        plan.build_host(idx.token_pos)
        up_done = []
        copy_stream.wait_stream(main)
        with torch.cuda.stream(copy_stream):
            for l in range(L):
                e_q[l].copy_(h_q[l], non_blocking=True)
                e_k[l].copy_(h_k[l], non_blocking=True)
                e_v[l].copy_(h_v[l], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_stream)
                up_done.append(ev)
        for l in range(L):
            main.wait_event(up_done[l])
            layer(l, e_q[l], e_k[l], e_v[l], e_out[l])
            ev = torch.cuda.Event()
            ev.record(main)
            out_stream.wait_event(ev)
            with torch.cuda.stream(out_stream):
                h_out[l].copy_(e_out[l], non_blocking=True)
        main.wait_stream(out_stream)
        main.wait_stream(copy_stream)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        barrier()
        return max_over_ranks(a.elapsed_time(b))

    # ---- resident timing (CUDA graph of one step unless --no-graph) ----------------------
    step_resident()
    torch.cuda.synchronize()
    use_graph = not args.no_graph
    replay = step_resident
    if use_graph:
        try:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step_resident()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step_resident()
            replay = graph.replay
        except Exception as e:   # report it, do not hide it
            use_graph = False
            replay = step_resident
            sys.stderr.write(f"[bench] CUDA graph capture failed, timing eager launches: {e}\n")
            torch.cuda.synchronize()

    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    ms_total = timed(replay, args.steps, args.warmup)
    clocks = sampler.stop()
    ms_step = ms_total / args.steps
    tokens_all = sum_over_ranks(float(N))
    value = tokens_all / (ms_step * 1e-3)

    # ---- per-launch time of the decode attention kernel (instrumented pass) ---------------
    plan.build_host(idx.token_pos)
    evs = []
    torch.cuda.synchronize()
    for _ in range(args.steps):
        for l in range(L):
            if not fused:
                pkv.launch_store_kv(k_l[l], v_l[l], d_slots, kc_l[l], vc_l[l], N, kv_dim)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            if fused:
                plan.append_attention(q_l[l], k_l[l], v_l[l], d_slots, kc_l[l], vc_l[l], d_tab, d_off, d_seq, d_pos, out_l[l], bs, w.scale)
            else:
                plan.attention(q_l[l], kc_l[l], vc_l[l], d_tab, d_off, d_seq, d_pos, out_l[l], bs, w.scale)
            b.record()
            evs.append((a, b))
    torch.cuda.synchronize()
    attn_ms = float(np.mean([a.elapsed_time(b) for a, b in evs]))
    peak, peak_src = peaks()
    algo_bytes = w.decode_bytes_per_layer()
    achieved = algo_bytes / (attn_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": ("decode_tma_kernel + decode_combine_kernel" if w.dtype != "f32" else "decode_simt_kernel + decode_combine_kernel"),
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": NCU_TRAFFIC.get(args.workload, {}).get("bytes"),
                "traffic_source": NCU_TRAFFIC.get(args.workload, {}).get("source"),
                "peak_source": peak_src, "algorithmic_bytes_per_launch": algo_bytes,
                "us_per_launch": attn_ms * 1e3, "launches_timed": len(evs),
                "frac_of_nominal_8TBs": achieved / 8000.0}

    # ---- end to end ---------------------------------------------------------------------
    e2e = None
    if not args.no_e2e:
        ms_e2e = timed(step_e2e, args.steps, max(args.warmup, 3)) / args.steps
        e2e_value = tokens_all / (ms_e2e * 1e-3)
        ok = torch.equal(e_out, out)       # same inputs through both routes: identical bits
        e2e = {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": int(h2d_bytes), "d2h_bytes_per_step": int(d2h_bytes),
               "ms_per_step": ms_e2e, "matches_resident_output": bool(ok)}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        import oracle
        checker = oracle.load_ref()
        kind = "reference"
        if checker is None:
            checker, kind = oracle.load_orc(), "port"
        threads = oracle.ref_default_thread_count()
        w0 = wl.make(args.workload)
        one_layer, n0 = cpu_step_sample(w0, checker, threads)
        one_layer()
        t = min(one_layer() for _ in range(3))
        cpu = {"value": n0 / (t * w0.layers), "unit": "tok/s", "cores": threads, "kind": kind,
               "sample": f"1 of {w0.layers} layers over all {w0.n_seqs} sequences (append + attention), best of 3, scaled x{w0.layers}"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w.dtype,
            "data": "synthetic",
            "config": {"workload": f"{args.workload}: {WORKLOAD_TEXT[args.workload]}", "tokens_per_step_per_gpu": N,
                       "layers": L, "sharding": "by sequence: each rank owns its pool and its batch, no collective",
                       "l2": f"per-step working set {algo_bytes * L / 1e9:.2f} GB across {L} distinct per-layer pools, far larger than the 126 MB L2",
                       "launch": "cuda graph replay" if use_graph else "eager launches",
                       "append": "inside the attention launch (pkv_append_decode_attn_planned)" if fused else "separate launch (pkv_append)",
                       **({"layers_override": args.layers} if args.layers else {})},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "step_hbm_gbs": (algo_bytes + w.append_bytes_per_layer()) * L / (ms_step * 1e-3) / 1e9,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_prefill(args, rank, local_rank, world):
    """--workload cfg4: chunked paged prefill.  One step = for every layer, append the chunk's K/V rows
    and run the tcgen05 prefill attention kernel.  Metric: prompt tokens/s; roofline: tensor."""
    import torch
    import torch.distributed as dist

    pkv = importlib.import_module("llm-engine_b200")
    wl = importlib.import_module("llm-engine_b200.workloads")
    sh = importlib.import_module("llm-engine_b200.sharding")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = args.layers or 24
    w = wl.make("cfg4", layers=L)
    tdt = torch.bfloat16
    bs, kv_dim = w.block_size, w.kv_dim
    H = w.q_heads * w.head_dim
    tabs, pos, _ = w.step_tokens()
    idx = pkv.pack_step(tabs, pos, bs)
    N = idx.n_tokens
    slots_total = w.num_blocks * bs
    g = torch.Generator(device=dev).manual_seed(91 + rank)
    rnd = lambda *shape: torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(tdt)
    pools = rnd(L, 2, slots_total, kv_dim)
    q, k, v = rnd(L, N, H), rnd(L, N, kv_dim), rnd(L, N, kv_dim)
    out = torch.zeros((L, N, H), dtype=tdt, device=dev)
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
    d_slots, d_tab, d_off = i32(idx.slots), i32(idx.block_tables), i32(idx.table_offset)
    q_len = w.new.astype(np.int32)
    q_start = np.concatenate([[0], np.cumsum(q_len)[:-1]]).astype(np.int32)
    d_qs, d_ql, d_ctx = i32(q_start), i32(q_len), i32(w.ctx.astype(np.int32))
    maxq = int(q_len.max())

    def attn(l, q_l, out_l):
        pkv.launch_attention_prefill(q_l, pools[l, 0], pools[l, 1], d_tab, d_off, d_qs, d_ql, d_ctx, out_l, N,
                                     w.n_seqs, maxq, w.q_heads, w.kv_heads, w.head_dim, bs, w.num_blocks, w.scale)

    def step():
        for l in range(L):
            pkv.launch_store_kv(k[l], v[l], d_slots, pools[l, 0], pools[l, 1], N, kv_dim)
            attn(l, q[l], out[l])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        barrier()
        _, ms = sh.reduce_step(0.0, a.elapsed_time(b), dist if world > 1 else None, dev)
        return ms

    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    ms_step = timed(step, args.steps, args.warmup) / args.steps
    clocks = sampler.stop()
    tokens_all, _ = sh.reduce_step(float(N), 0.0, dist if world > 1 else None, dev)
    value = tokens_all / (ms_step * 1e-3)
    # per-launch time of the prefill kernel
    evs = []
    for _ in range(max(1, args.steps // 2)):
        for l in range(L):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            attn(l, q[l], out[l])
            b.record()
            evs.append((a, b))
    torch.cuda.synchronize()
    k_ms = float(np.mean([a.elapsed_time(b) for a, b in evs]))
    flops = w.prefill_flops_per_layer()
    peak, src = peaks("bf16_tflops", 1590.0)
    sust, _ = peaks("bf16_tflops_sustained", 1400.0)
    ach = flops / (k_ms * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": "prefill_tc_kernel", "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                "frac": ach / peak, "frac_of_sustained": ach / sust, "traffic": None, "peak_source": src,
                "algorithmic_flops_per_launch": flops, "us_per_launch": k_ms * 1e3, "launches_timed": len(evs)}
    # end to end: the chunk's q/k/v rows from pinned host memory, outputs back
    e2e = None
    if not args.no_e2e:
        pin = lambda t: t.cpu().pin_memory()
        h_q, h_k, h_v = pin(q), pin(k), pin(v)
        h_out = torch.empty((L, N, H), dtype=tdt).pin_memory()
        e_q, e_k, e_v, e_out = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v), torch.empty_like(out)
        h_slots = torch.from_numpy(idx.slots).pin_memory()

        def step_e2e():
            d_slots.copy_(h_slots, non_blocking=True)
            for l in range(L):
                e_q[l].copy_(h_q[l], non_blocking=True)
                e_k[l].copy_(h_k[l], non_blocking=True)
                e_v[l].copy_(h_v[l], non_blocking=True)
                pkv.launch_store_kv(e_k[l], e_v[l], d_slots, pools[l, 0], pools[l, 1], N, kv_dim)
                attn(l, e_q[l], e_out[l])
                h_out[l].copy_(e_out[l], non_blocking=True)

        ms_e = timed(step_e2e, args.steps, args.warmup) / args.steps
        e2e = {"value": tokens_all / (ms_e * 1e-3), "unit": "tok/s", "ms_per_step": ms_e,
               "h2d_bytes_per_step": int(sum(t.numel() * t.element_size() for t in (h_q, h_k, h_v)) + h_slots.numel() * 4),
               "d2h_bytes_per_step": int(h_out.numel() * h_out.element_size()),
               "matches_resident_output": bool(torch.equal(e_out, out))}
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        import oracle
        checker = oracle.load_ref() or oracle.load_orc()
        kind = "reference" if checker.kind == "reference" else "port"
        threads = oracle.ref_default_thread_count()
        # bounded sample: every 16th chunk token of every sequence, one layer, scaled
        orc = oracle.load_orc()
        rng = np.random.default_rng(0)
        kc = orc.from_bf16_bits(orc.to_bf16_bits(rng.standard_normal((slots_total, kv_dim), dtype=np.float32)))
        vc = orc.from_bf16_bits(orc.to_bf16_bits(rng.standard_normal((slots_total, kv_dim), dtype=np.float32)))
        sample = np.arange(0, N, 16)
        qs = orc.from_bf16_bits(orc.to_bf16_bits(rng.standard_normal((sample.size, H), dtype=np.float32)))
        t0 = time.perf_counter()
        checker.paged_attention(qs, kc, vc, idx.block_tables, idx.table_offset, idx.token_seq[sample],
                                idx.token_pos[sample], w.q_heads, w.kv_heads, w.head_dim, bs, w.scale, threads=threads)
        t = time.perf_counter() - t0
        cpu = {"value": N / (t * 16 * L), "unit": "tok/s", "cores": threads, "kind": kind,
               "sample": f"attention for every 16th chunk token of all {w.n_seqs} sequences, 1 of {L} layers, scaled x16 x{L}"}
    if rank == 0:
        line = {"metric": "chunked prefill tok/s (K/V append + paged prefill attention over all layers)", "value": value,
                "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"cfg4: {WORKLOAD_TEXT['cfg4']}", "tokens_per_step_per_gpu": N, "layers": L,
                           "l2": "24 distinct per-layer pools and q/k/v/out sets (2.4 GB per step), larger than the 126 MB L2",
                           "launch": "eager launches"},
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": 2 * L * args.steps, "clocks": clocks}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def long_prompt_tables(S, prefix_blocks, bs, seed=1240):
    """S sequences that share prefix_blocks leading blocks and have 32..256 tokens of their own."""
    rng = np.random.default_rng(seed)
    ctx = prefix_blocks * bs + rng.integers(32, 257, size=S)
    own = (ctx + 1 + bs - 1) // bs - prefix_blocks
    nb = int(own.sum()) + prefix_blocks + 8
    perm = rng.permutation(nb).astype(np.int32)
    tables, at = [], prefix_blocks
    for n in own:
        tables.append(np.concatenate([perm[:prefix_blocks], perm[at:at + n]]).astype(np.int32))
        at += n
    return tables, ctx.tolist()


def compare_shared_plan(pkv, torch, dev, tables, positions, qh, kvh, hd, bs, nb, layers):
    """us per layer of attention + merge with the ordinary plan and with the shared-prefix plan."""
    S = len(tables)
    nb = nb or int(max(int(t.max()) for t in tables)) + 1
    kv_dim, H = kvh * hd, qh * hd
    idx = pkv.pack_step(tables, positions, bs, tok_keys=list(range(S)))
    pools = torch.randn((layers, 2, nb * bs, kv_dim), device=dev, dtype=torch.float32).to(torch.bfloat16)
    q = torch.randn((layers, S, H), device=dev, dtype=torch.float32).to(torch.bfloat16)
    out = torch.zeros((layers, S, H), device=dev, dtype=torch.bfloat16)
    i32 = lambda x: torch.from_numpy(np.ascontiguousarray(x, dtype=np.int32)).to(dev)
    d = [i32(idx.block_tables), i32(idx.table_offset), i32(idx.token_seq), i32(idx.token_pos)]
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    res = {"per_sequence_bytes_per_layer": int(sum(2 * (p + 1) * kv_dim * 2 for p in positions))}
    for name in ("ordinary", "shared"):
        pl = pkv.DecodePlan(S, qh, kvh, hd, device=dev)
        pl.build_host(idx.token_pos) if name == "ordinary" else pl.build_host_shared(idx, bs, min_saved_bytes=0)

        def run_layers():
            for l in range(layers):
                pl.attention(q[l], pools[l, 0], pools[l, 1], *d, out[l], bs, 1.0 / float(np.sqrt(hd)))
        for _ in range(3):
            run_layers()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            run_layers()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        a.record()
        for _ in range(20):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        res[name] = {"us_per_layer": a.elapsed_time(b) / 20 / layers * 1e3, "shared_units": pl.n_shared_units,
                     "items": int(pl.plan.n_items), "chunk": int(pl.plan.chunk)}
    pl = pkv.DecodePlan(S, qh, kvh, hd, device=dev)
    res["default_rule_picks"] = "shared" if pl.build_host_shared(idx, bs).n_shared_units > 0 else "ordinary"
    return res


def run_head_sharded(args, rank, local_rank, world):
    """--sharding head (cfg3, 2 or 4 GPUs): ONE batch for the whole job; rank r keeps the pools and the
    query columns of kv heads [r*kvh/world, (r+1)*kvh/world) and computes them for all 256 sequences,
    and every rank ends each layer with the full attention output.  Strong scaling.  --exchange peer
    (default): the exchange is fused into the merge kernel (peer stores over NVLink + bounded flag
    wait); --exchange nccl: local output, then an NCCL all-gather, for comparison."""
    import torch
    import torch.distributed as dist
    pkv = importlib.import_module("llm-engine_b200")
    wl = importlib.import_module("llm-engine_b200.workloads")
    sh = importlib.import_module("llm-engine_b200.sharding")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    w = wl.make(args.workload, layers=args.layers)
    if w.kv_heads % world:
        raise SystemExit(f"--sharding head: {w.kv_heads} kv heads do not divide over {world} GPUs")
    tdt = {"bf16": torch.bfloat16, "f16": torch.float16}[w.dtype]
    bs, L, hd = w.block_size, w.layers, w.head_dim
    q0, ql, kv0, kvl = sh.head_slices(w.q_heads, w.kv_heads, world, rank)
    kv_dim_l, H_l, H = kvl * hd, ql * hd, w.q_heads * hd
    tabs, pos, _ = w.step_tokens()
    idx = pkv.pack_step(tabs, pos, bs)
    N = idx.n_tokens
    slots_total = w.num_blocks * bs
    g = torch.Generator(device=dev).manual_seed(77 + rank)
    pools = torch.empty((L, 2, slots_total, kv_dim_l), dtype=tdt, device=dev)
    for l in range(L):
        for j in range(2):
            pools[l, j].copy_(torch.randn((slots_total, kv_dim_l), generator=g, device=dev, dtype=torch.float32))
    q = torch.randn((L, N, H_l), generator=g, device=dev, dtype=torch.float32).to(tdt)
    k = torch.randn((L, N, kv_dim_l), generator=g, device=dev, dtype=torch.float32).to(tdt)
    v = torch.randn((L, N, kv_dim_l), generator=g, device=dev, dtype=torch.float32).to(tdt)
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
    d_slots, d_seq, d_pos = i32(idx.slots), i32(idx.token_seq), i32(idx.token_pos)
    d_tab, d_off = i32(idx.block_tables), i32(idx.table_offset)
    plan = pkv.DecodePlan(N, ql, kvl, hd, device=dev)
    ex = sh.HeadShardedExchange(N, w.q_heads, hd, tdt, dist, dev)
    out_local = torch.zeros((N, H_l), dtype=tdt, device=dev)
    out_full = torch.zeros((world, N, H_l), dtype=tdt, device=dev)

    def step():
        plan.build_host(idx.token_pos)
        for l in range(L):
            pkv.launch_store_kv(k[l], v[l], d_slots, pools[l, 0], pools[l, 1], N, kv_dim_l)
            if args.exchange == "peer":
                ex.attention(plan, q[l], pools[l, 0], pools[l, 1], d_tab, d_off, d_seq, d_pos, bs, w.scale)
            else:
                plan.attention(q[l], pools[l, 0], pools[l, 1], d_tab, d_off, d_seq, d_pos, out_local, bs, w.scale)
                dist.all_gather_into_tensor(out_full, out_local)

    def barrier():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    replay = step
    if not args.no_graph:
        plan.build_host(idx.token_pos)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        replay = graph.replay
        for _ in range(3):
            replay()
        barrier()
    # agreement of the two exchanges on the last layer (rank-major columns in the all-gather buffer)
    if args.exchange == "peer":
        plan.attention(q[L - 1], pools[L - 1, 0], pools[L - 1, 1], d_tab, d_off, d_seq, d_pos, out_local, bs, w.scale)
        dist.all_gather_into_tensor(out_full, out_local)
        torch.cuda.synchronize()
        same = bool(torch.equal(out_full.permute(1, 0, 2).reshape(N, H).view(torch.int16), ex.out.view(torch.int16)))
    else:
        same = None
    barrier()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        replay()
    b.record()
    barrier()
    clocks = sampler.stop()
    ms = torch.tensor([a.elapsed_time(b) / args.steps], dtype=torch.float64, device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_step = float(ms.item())
    flags = pkv.debug_device_flags()
    peak, src = peaks()
    byts = w.decode_bytes_per_layer() / world            # this rank's share of the K/V bytes of a layer
    if rank == 0:
        print(json.dumps({
            "metric": "decode tok/s (K/V append + paged decode attention over all layers)", "value": N / (ms_step * 1e-3),
            "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
            "config": {"workload": f"{args.workload}: {WORKLOAD_TEXT[args.workload]}", "layers": L,
                       "sharding": f"by head: each rank holds {kvl} of {w.kv_heads} kv heads for all {N} sequences; every rank "
                                   f"ends each layer with the full output",
                       "exchange": "fused into the merge kernel: peer stores over NVLink + bounded flag wait" if args.exchange == "peer"
                                   else "NCCL all-gather after the local attention",
                       "launch": "eager launches" if args.no_graph else "cuda graph replay"},
            "roofline": {"bound": "hbm", "kernel": "decode_tma_kernel + decode_combine_kernel (+ exchange), whole step",
                         "achieved": byts * L / (ms_step * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": byts * L / (ms_step * 1e-3) / 1e9 / peak, "traffic": None, "peak_source": src},
            "exchange_bytes_per_layer_per_gpu": N * H_l * 2 * (world - 1), "peer_result_equals_nccl_result": same,
            "device_error_flags": flags, "cpu_baseline": None, "e2e": None, "gpu_launches": 3 * L * args.steps, "clocks": clocks}), flush=True)
    # Tear-down: the captured graph (it holds NCCL kernels in --exchange nccl) goes first; a watchdog
    # ends the process if a collective's tear-down does not return.
    sys.stdout.flush()
    threading.Timer(20.0, lambda: os._exit(0)).start()
    replay = None
    if not args.no_graph:
        del graph
    torch.cuda.synchronize()
    ex.close()
    dist.destroy_process_group()
    os._exit(0)


def run_prefix_cow(args, rank, local_rank, world):
    """--workload cfg5: 128 sequences forked from one parent that holds a 512-token prefix plus a partial
    block; the first divergent write of each child triggers a copy-on-write block copy on every pool
    (timed: CoW GB/s), then each sequence gets its seeded suffix and 64 decode steps with appends run
    (timed: decode tok/s, host bookkeeping + packing + planning included, eager launches)."""
    import torch
    pkv = importlib.import_module("llm-engine_b200")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    rng = np.random.default_rng(1239 + 1000 * rank)
    L, qh, kvh, hd, bs, nb, S = (args.layers or 22), 32, 4, 64, 16, 8192, 128
    kv_dim, H = kvh * hd, qh * hd
    scale = 1.0 / float(np.sqrt(hd))
    mgr = pkv.KVCacheManager(nb, bs, True)
    parent = mgr.new_table()
    prefix = rng.integers(0, 32000, size=520).astype(np.int32).tolist()      # 32 full blocks + 8 tokens
    mgr.allocate_prompt(parent, prefix)
    mgr.commit_computed(parent, prefix, 520)
    seqs = [parent] + [mgr.new_table() for _ in range(S - 1)]
    for t in seqs[1:]:
        mgr.fork(parent, t)
    pools = torch.randn((L, 2, nb * bs, kv_dim), device=dev, dtype=torch.float32).to(torch.bfloat16)
    ptrs = torch.tensor([pools[l, j].data_ptr() for l in range(L) for j in range(2)], dtype=torch.int64, device=dev)
    pairs = []
    for t in seqs:
        r = mgr.cow(t, 520)
        if r[0] >= 0:
            pairs.append(r)
    pa = torch.from_numpy(np.asarray(pairs, dtype=np.int32)).to(dev)
    block_bytes = bs * kv_dim * 2
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 20
    for _ in range(3):
        pkv.launch_copy_blocks_layers(ptrs, 2 * L, pa, len(pairs), block_bytes)
    torch.cuda.synchronize()
    a.record()
    for _ in range(reps):
        pkv.launch_copy_blocks_layers(ptrs, 2 * L, pa, len(pairs), block_bytes)
    b.record()
    torch.cuda.synchronize()
    cow_us = a.elapsed_time(b) / reps * 1e3
    cow_bytes = 2 * len(pairs) * block_bytes * 2 * L          # read + write, K and V, every layer
    # suffixes (their K/V are whatever the pool holds: values do not matter for timing)
    lens = []
    for t in seqs:
        n = 520 + int(rng.integers(32, 257))
        for m in range(521, n + 1):
            mgr.ensure_slot(t, m)
        lens.append(n)
    q = torch.randn((L, S, H), device=dev, dtype=torch.float32).to(torch.bfloat16)
    k = torch.randn((L, S, kv_dim), device=dev, dtype=torch.float32).to(torch.bfloat16)
    v = torch.randn((L, S, kv_dim), device=dev, dtype=torch.float32).to(torch.bfloat16)
    out = torch.zeros((L, S, H), device=dev, dtype=torch.bfloat16)
    plan = pkv.DecodePlan(S, qh, kvh, hd, device=dev)
    i32 = lambda x: torch.from_numpy(np.ascontiguousarray(x, dtype=np.int32)).to(dev, non_blocking=True)

    # Index build on the device (pkv_step_pack_device): the tables stay resident, a step sends only
    # the newly appended block ids and one (row, position, 1) triple per sequence.  --host-pack uses the
    # host routine and five copies per step instead, as the reference does.
    max_row = max(t.num_blocks() for t in seqs) + 8
    packer = pkv.DeviceStepPacker(S, max_row, bs, max_tokens=S, max_table_entries=S * max_row, device=dev)
    for i, t in enumerate(seqs):
        packer.set_table(i, t.blocks)

    def decode_step():
        if args.host_pack:
            for t, n in zip(seqs, lens):
                mgr.ensure_slot(t, n + 1)
            idx = pkv.pack_step([t.blocks for t in seqs], lens, bs, tok_keys=list(range(S)))
            d = [i32(idx.block_tables), i32(idx.table_offset), i32(idx.token_seq), i32(idx.token_pos)]
            d_slots = i32(idx.slots)
            plan.build_host(idx.token_pos)
        else:
            for i, (t, n) in enumerate(zip(seqs, lens)):
                mgr.ensure_slot(t, n + 1)
                if n % bs == 0:                       # position n opened a new block
                    packer.set_block(i, n // bs, int(t.blocks[-1]))
            packer.pack([(i, lens[i], 1) for i in range(S)])
            d = [packer.tables, packer.table_offset, packer.token_seq, packer.positions]
            d_slots = packer.slots
            plan.build_device(packer.positions)
        for l in range(L):
            pkv.launch_store_kv(k[l], v[l], d_slots, pools[l, 0], pools[l, 1], S, kv_dim)
            plan.attention(q[l], pools[l, 0], pools[l, 1], *d, out[l], bs, scale)
        for i in range(S):
            lens[i] += 1

    for _ in range(3):
        decode_step()
    torch.cuda.synchronize()
    steps = 64
    t0 = time.perf_counter()
    a.record()
    byts = 0
    for _ in range(steps):
        n_before = list(lens)
        decode_step()
        byts += sum(2 * (n + 1) * kv_dim * 2 for n in n_before) * L
    b.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    ms_step = a.elapsed_time(b) / steps
    peak, src = peaks()
    # Shared-prefix-aware plan against the ordinary one (attention + merge per layer, indices and plan
    # resident, CUDA-graph replay, CUDA events): on the state the 64 steps left, and on a long shared
    # prompt where the saving outweighs the extra launch.
    del pools, q, k, v, out
    torch.cuda.empty_cache()
    shared_cmp = {"cfg5_after_64_steps": compare_shared_plan(pkv, torch, dev, [np.asarray(t.blocks) for t in seqs],
                                                             [n - 1 for n in lens], qh, kvh, hd, bs, nb, min(L, 4)),
                  "long_prompt_256_seqs_x_8192_shared": compare_shared_plan(pkv, torch, dev, *long_prompt_tables(256, 512, bs),
                                                                            qh, kvh, hd, bs, None, min(L, 4))}
    line = {"metric": "prefix-cache decode tok/s (bookkeeping + append + paged decode attention, 64 steps) and CoW copy GB/s",
            "value": S / (ms_step * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": 3, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"cfg5: {WORKLOAD_TEXT['cfg5']}", "layers": L, "launch": "eager launches, host bookkeeping in the timed region",
                       "index_build": "host (pkv_step_pack + five copies)" if args.host_pack else "device (pkv_step_pack_device, one copy)",
                       "note": "the reference never shares a partial block (docs/design.md:36); the CoW trigger is this library's additive fork()/cow()"},
            "cow": {"pairs": len(pairs), "pools": 2 * L, "us_per_wave": cow_us, "bytes_read_plus_written": cow_bytes,
                    "GBps": cow_bytes / cow_us / 1e3, "frac_of_measured_hbm": cow_bytes / cow_us / 1e3 / peak},
            "roofline": {"bound": "hbm", "kernel": "decode_tma_kernel + decode_combine_kernel (whole step incl. host)",
                         "achieved": byts / steps / (ms_step * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": byts / steps / (ms_step * 1e-3) / 1e9 / peak, "traffic": None, "peak_source": src},
            "shared_prefix_plan": shared_cmp,
            "cpu_baseline": None, "e2e": {"value": S * steps / wall, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                                          "note": "wall clock over the same 64 steps"},
            "gpu_launches": 3 * L * steps}
    if rank == 0:
        print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="cfg3", choices=sorted(WORKLOAD_TEXT))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--append", choices=("auto", "fused", "separate"), default="auto",
                    help="decode: K/V append inside the attention launch, as its own launch (as the reference calls it), or by step size")
    ap.add_argument("--sharding", choices=("sequence", "head"), default="sequence",
                    help="multi-GPU: independent batches per GPU (default, weak scaling) or one batch split by kv head")
    ap.add_argument("--exchange", choices=("peer", "nccl"), default="peer", help="--sharding head: how the output slices are exchanged")
    ap.add_argument("--host-pack", action="store_true", help="cfg5: build the step indices on the host instead of on the device")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiling runs)")
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (profiling runs only; noted in config)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if world != args.gpus:
        if args.gpus > 1 and world == 1:
            raise SystemExit("--gpus N > 1 is launched with torch.distributed.run --nproc-per-node N")
    if args.sharding == "head" and world > 1 and args.workload in ("cfg2", "cfg3"):
        run_head_sharded(args, rank, local_rank, world)
    elif args.workload == "cfg4":
        run_prefill(args, rank, local_rank, world)
    elif args.workload == "cfg5":
        run_prefix_cow(args, rank, local_rank, world)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
