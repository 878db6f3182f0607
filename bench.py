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
    "mixed": "one attention call on a mixed step as llm-engine's forward pass packs it: two 300-token prefill chunks (1,200 and 700 cached tokens) + 20 decode tokens, Qwen2.5-0.5B shapes (14q/2kv heads, d64), f16, block 16",
    "cow": "copy-on-write block copy alone: TinyLlama shapes (4 kv heads, d64, bf16, block 16: 8 KiB blocks), 22 layers x 2 pools of 8192 blocks, 127 block pairs per wave on every pool in one launch, 8 disjoint pair lists in rotation",
}
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) per launch of the decode attention kernel, from the
# ncu captures summarised under profiles/ (same per-launch workload as the default seed of each configuration).
NCU_TRAFFIC = {
    "cfg3": {"bytes": 428955648, "source": "profiles/decode_tma_kernel_cfg3_ncu_full.md (421.21 MB read + 7.75 MB written)"},
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
def load_workloads_standalone():
    """The workload generator, loaded from its file so that the CPU arm never imports the product
    package (and therefore never loads libpkv.so)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("pkv_workloads", os.path.join(ROOT, "llm-engine_b200", "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["pkv_workloads"] = mod
    spec.loader.exec_module(mod)
    return mod


def pack_step_numpy(w):
    """Index arrays of the step as CudaModel::upload_step_indices builds them
    (src/model/cuda/cuda_model.cu:453-473), in numpy: sequences in packed order, each table once."""
    bs = w.block_size
    seq = np.repeat(np.arange(w.n_seqs, dtype=np.int32), w.new.astype(np.int64))
    first = np.concatenate([[0], np.cumsum(w.new)[:-1]])
    pos = (np.repeat(w.ctx, w.new.astype(np.int64)) + (np.arange(seq.size) - np.repeat(first, w.new.astype(np.int64)))).astype(np.int32)
    tables = np.concatenate([np.asarray(t, dtype=np.int32) for t in w.tables])
    off = np.concatenate([[0], np.cumsum([len(t) for t in w.tables])[:-1]]).astype(np.int32)
    slots = (tables[off[seq] + pos // bs].astype(np.int64) * bs + pos % bs).astype(np.int32)
    return {"slots": slots, "token_seq": seq, "token_pos": pos, "block_tables": tables, "table_offset": off, "n_tokens": int(seq.size)}


def cpu_step_fn(w, checker, threads, seed=0):
    """Returns (step, n_tokens): step() runs the WHOLE step on the host -- for every layer, append the
    batch's K/V rows and run paged attention for every sequence -- and returns its wall time.  Pools
    are fp32, as in the reference's CPU backend (bf16 workloads are rounded to bf16 and widened first);
    one K pool and one V pool are reused by every layer: configuration 3 reads 0.8 GB of their rows per
    layer, far beyond the last-level cache, so reuse does not flatter the number."""
    import oracle
    orc = oracle.load_orc()
    rng = np.random.default_rng(seed)
    bs, kv_dim = w.block_size, w.kv_dim
    idx = pack_step_numpy(w)
    N = idx["n_tokens"]
    slots_total = w.num_blocks * bs
    # Only slots that some sequence owns are read; filling the whole pool costs host time for nothing.
    kc = np.zeros((slots_total, kv_dim), dtype=np.float32)
    vc = np.zeros((slots_total, kv_dim), dtype=np.float32)
    used = np.unique(idx["block_tables"])
    rows = (used[:, None].astype(np.int64) * bs + np.arange(bs)[None, :]).reshape(-1)
    cast = (lambda a: orc.from_bf16_bits(orc.to_bf16_bits(a))) if w.dtype == "bf16" else (lambda a: a)
    for a in (kc, vc):
        a[rows] = cast(rng.standard_normal((rows.size, kv_dim), dtype=np.float32))
    q = cast(rng.standard_normal((N, w.q_heads * w.head_dim), dtype=np.float32))
    k = cast(rng.standard_normal((N, kv_dim), dtype=np.float32))
    v = cast(rng.standard_normal((N, kv_dim), dtype=np.float32))

    def step():
        t0 = time.perf_counter()
        for _ in range(w.layers):
            checker.append(k, v, idx["slots"], kc, vc)
            checker.paged_attention(q, kc, vc, idx["block_tables"], idx["table_offset"], idx["token_seq"], idx["token_pos"],
                                    w.q_heads, w.kv_heads, w.head_dim, bs, w.scale, threads=threads)
        return time.perf_counter() - t0

    step.pool_gb_read_per_layer = rows.size * kv_dim * 4 * 2 / 1e9
    return step, N


def run_reference_arm(args, rank, world):
    """--impl reference: the reference's CPU implementation (oracle/_ref, compiled from its sources; the
    C restatement if that is absent), all host threads, every layer of the step, --steps timed steps
    after --warmup untimed ones.  Nothing of the product is imported or loaded."""
    if rank != 0:
        return
    import oracle
    wl = load_workloads_standalone()
    checker = oracle.load_ref()
    kind = "reference"
    if checker is None:
        checker, kind = oracle.load_orc(), "port"
    threads = oracle.ref_default_thread_count()
    w = wl.make(args.workload)
    step, N = cpu_step_fn(w, checker, threads)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    t_step = (time.perf_counter() - t0) / args.steps
    value = N / t_step
    sample = f"every step = all {w.layers} layers over all {w.n_seqs} sequences (append + attention); {args.steps} steps timed after {args.warmup} warm-up steps"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t_step * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {WORKLOAD_TEXT[args.workload]}", "tokens_per_step_per_gpu": N, "layers": w.layers,
                   "device": "host CPU",
                   "note": "the reference's CPU backend is fp32; bf16 inputs are rounded to bf16 and widened; one K/V pool pair reused by "
                           f"every layer ({step.pool_gb_read_per_layer:.2f} GB of rows read per layer)"},
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

    plan.build_host(idx.token_pos)
    cluster_form = int(plan.plan.cluster)            # > 0: small-step form, the merge happens inside the attention launch
    launches_per_step = ((2 if fused else 3) - (1 if cluster_form else 0)) * L      # kernels: [append,] attention [, merge]

    # ---- end-to-end step: host buffers in, host buffers out --------------------------
    # Host side: one pinned staging buffer per layer holding that layer's q | k | v rows back to back
    # (one upload per layer), one for the five index arrays, the planner's own pinned staging, and one
    # for every layer's output.  Device side: mirrors of the same shape, with contiguous q/k/v views.
    row = H + 2 * kv_dim
    h_qkv = torch.empty((L, N * row), dtype=tdt).pin_memory()
    e_qkv = torch.empty((L, N * row), dtype=tdt, device=dev)
    for l in range(L):
        h_qkv[l, :N * H].copy_(q[l].reshape(-1))
        h_qkv[l, N * H:N * (H + kv_dim)].copy_(k[l].reshape(-1))
        h_qkv[l, N * (H + kv_dim):].copy_(v[l].reshape(-1))
    e_q = [e_qkv[l, :N * H].view(N, H) for l in range(L)]
    e_k = [e_qkv[l, N * H:N * (H + kv_dim)].view(N, kv_dim) for l in range(L)]
    e_v = [e_qkv[l, N * (H + kv_dim):].view(N, kv_dim) for l in range(L)]
    h_out = torch.empty((L, N, H), dtype=tdt).pin_memory()
    e_out = torch.empty_like(out)
    idx_arrays = [idx.slots, idx.token_seq, idx.token_pos, idx.block_tables, idx.table_offset]
    idx_off = np.concatenate([[0], np.cumsum([((a.size + 63) // 64) * 64 for a in idx_arrays])])
    h_idx = torch.zeros(int(idx_off[-1]), dtype=torch.int32).pin_memory()
    e_idx = torch.zeros(int(idx_off[-1]), dtype=torch.int32, device=dev)
    for a, o in zip(idx_arrays, idx_off):
        h_idx[int(o):int(o) + a.size].copy_(torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)))
    e_slots, e_seq, e_pos, e_tab, e_off = [e_idx[int(o):int(o) + a.size] for a, o in zip(idx_arrays, idx_off)]
    plan_e = pkv.DecodePlan(N, w.q_heads, w.kv_heads, w.head_dim, device=dev)
    h2d_bytes = h_qkv.numel() * h_qkv.element_size() + h_idx.numel() * 4 + plan_e.staging.numel()
    d2h_bytes = h_out.numel() * h_out.element_size()
    copy_stream = torch.cuda.Stream(device=dev)
    out_stream = torch.cuda.Stream(device=dev)

    def layer_e(l):
        if fused:
            plan_e.append_attention(e_q[l], e_k[l], e_v[l], e_slots, kc_l[l], vc_l[l], e_tab, e_off, e_seq, e_pos, e_out[l], bs, w.scale)
        else:
            pkv.launch_store_kv(e_k[l], e_v[l], e_slots, kc_l[l], vc_l[l], N, kv_dim)
            plan_e.attention(e_q[l], kc_l[l], vc_l[l], e_tab, e_off, e_seq, e_pos, e_out[l], bs, w.scale)

    def e2e_device_part():
        """Everything of an end-to-end step that runs on the device: the index arrays and the plan image
        go up first, layer l's q|k|v rows are uploaded on a copy stream while layer l-1 computes, and
        layer l's output goes back while layer l+1 computes.  Capturable: no host work in here."""
        main = torch.cuda.current_stream()
        e_idx.copy_(h_idx, non_blocking=True)
        plan_e.workspace[:plan_e.staging.numel()].copy_(plan_e.staging, non_blocking=True)
        up_done = []
        copy_stream.wait_stream(main)
        with torch.cuda.stream(copy_stream):
            for l in range(L):
                e_qkv[l].copy_(h_qkv[l], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_stream)
                up_done.append(ev)
        # The uploads run far ahead of the kernels (26 us each against 76 us of compute per layer), so the
        # kernels need not wait for them layer by layer: a wait before layers 0, 1, 3, 7, 15 covers the
        # uploads of the layers up to the next wait.  Every wait is an extra dependency on that layer's first
        # kernel, which then cannot start early on its predecessor (programmatic dependent launch).
        covered = -1
        for l in range(L):
            if l > covered:
                covered = min(L - 1, max(l, 2 * l))
                main.wait_event(up_done[covered])
            layer_e(l)
            ev = torch.cuda.Event()
            ev.record(main)
            out_stream.wait_event(ev)
            with torch.cuda.stream(out_stream):
                h_out[l].copy_(e_out[l], non_blocking=True)
        main.wait_stream(out_stream)
        main.wait_stream(copy_stream)

    e2e_graph = [None]

    def step_e2e():
        """One serving step as a caller of the library makes it: plan on the host from the host copy of
        the positions (into pinned staging), then the device part -- a replay of its captured graph
        when capture worked, eager launches otherwise -- then wait for the outputs to be in host
        memory, as a decode loop must before it can sample."""
        plan_e.build_host_image(idx.token_pos)
        if e2e_graph[0] is not None:
            e2e_graph[0].replay()
        else:
            e2e_device_part()
        torch.cuda.current_stream().synchronize()

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
        plan_e.build_host_image(idx.token_pos)
        e2e_device_part()                      # eager once: warms every path the capture will take
        torch.cuda.synchronize()
        e2e_launch = "eager launches"
        if not args.no_graph:
            try:
                g2 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g2):
                    e2e_device_part()
                e2e_graph[0] = g2
                e2e_launch = "cuda graph replay (copies are nodes of the graph)"
            except Exception as e:
                e2e_graph[0] = None
                sys.stderr.write(f"[bench] capture of the end-to-end step failed, timing eager launches: {e}\n")
                torch.cuda.synchronize()
        h_out.zero_()
        ms_e2e = timed(step_e2e, args.steps, max(args.warmup, 3)) / args.steps
        e2e_value = tokens_all / (ms_e2e * 1e-3)
        ok = torch.equal(e_out, out) and torch.equal(h_out.to(dev), out)   # same inputs through both routes: identical bits, on the device and back on the host
        e2e = {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": int(h2d_bytes), "d2h_bytes_per_step": int(d2h_bytes),
               "ms_per_step": ms_e2e, "matches_resident_output": bool(ok), "launch": e2e_launch,
               "per_step": "host: split-K plan from the host positions into pinned staging; device: index arrays + plan image + one "
                           f"q|k|v upload per layer ({L + 2} host-to-device copies), {launches_per_step} kernels, {L} device-to-host copies; "
                           "then a stream synchronise (the outputs are needed on the host)"}

    # ---- strong scaling: ONE batch of the configuration dealt over the ranks ----------------
    # BASELINE words configuration 3 as "batch 256 ... sequence-sharded across 1/2/4/8 GPUs".  The weak
    # line above gives every rank the whole batch; here the same batch is dealt once, longest context
    # first to the least loaded rank (sharding.deal_sequences, "balanced"), each rank runs the step on
    # its share out of its own pool, and the job's time is the slowest rank's.  One GPU: the deal is the
    # whole batch, i.e. the weak measurement itself.
    strong = None

    def strong_share(world_v, rank_v):
        """Rank rank_v's share of the batch dealt over world_v GPUs, timed on THIS GPU out of its own pools:
        (ms per step, sequences, K/V bytes per layer, whether the append ran inside the attention launch)."""
        sel = sh.deal_sequences(w.ctx, world_v, rank_v, "balanced")
        tabs_s = [w.tables[i] for i in sel]
        pos_s = np.asarray([int(w.ctx[i]) for i in sel], dtype=np.int32)
        idx_s = pkv.pack_step(tabs_s, pos_s, bs)
        Ns = idx_s.n_tokens
        s_slots, s_seq, s_pos = i32(idx_s.slots), i32(idx_s.token_seq), i32(idx_s.token_pos)
        s_tab, s_off = i32(idx_s.block_tables), i32(idx_s.table_offset)
        plan_s = pkv.DecodePlan(Ns, w.q_heads, w.kv_heads, w.head_dim, device=dev)
        fused_s = w.dtype != "f32" and (args.append == "fused" or (args.append == "auto" and Ns * w.kv_heads < 1024))
        qs, ks, vs, os_ = [q[l][:Ns] for l in range(L)], [k[l][:Ns] for l in range(L)], [v[l][:Ns] for l in range(L)], [out[l][:Ns] for l in range(L)]

        def step_strong():
            plan_s.build_host(idx_s.token_pos)
            for l in range(L):
                if fused_s:
                    plan_s.append_attention(qs[l], ks[l], vs[l], s_slots, kc_l[l], vc_l[l], s_tab, s_off, s_seq, s_pos, os_[l], bs, w.scale)
                else:
                    pkv.launch_store_kv(ks[l], vs[l], s_slots, kc_l[l], vc_l[l], Ns, kv_dim)
                    plan_s.attention(qs[l], kc_l[l], vc_l[l], s_tab, s_off, s_seq, s_pos, os_[l], bs, w.scale)

        step_strong()
        torch.cuda.synchronize()
        replay_s = step_strong
        if not args.no_graph:
            try:
                gs = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gs):
                    step_strong()
                replay_s = gs.replay
            except Exception as e:
                sys.stderr.write(f"[bench] capture of the strong-scaling step failed, timing eager launches: {e}\n")
                torch.cuda.synchronize()
        ms = timed(replay_s, args.steps, args.warmup) / args.steps
        L_all = (w.ctx + w.new).astype(np.int64)
        my_bytes = float((2 * L_all[sel] * w.kv_heads * w.head_dim * w.elem_bytes).sum())
        return ms, int(Ns), my_bytes, fused_s

    if not args.no_strong:
        if world == 1:
            strong = {"value": value, "unit": "tok/s", "ms_per_step": ms_step, "sequences_per_rank": [N],
                      "efficiency_vs_one_gpu": 1.0, "policy": "balanced (one rank: the whole batch)"}
            if args.workload == "cfg3":
                # What the deal over 2, 4 and 8 GPUs would give, from rank 0's share timed on this one GPU (the
                # shares hold the same K/V bytes to 1e-5 and no collective is involved, so the slowest rank's time
                # is this time up to run-to-run noise): the real multi-GPU figure is the `strong` block of a
                # --gpus N run.
                proj = {}
                for wv in (2, 4, 8):
                    ms_v, n_v, b_v, f_v = strong_share(wv, 0)
                    proj[str(wv)] = {"sequences": n_v, "kv_bytes_per_layer": b_v, "ms_per_step": ms_v, "us_per_layer": ms_v * 1e3 / L,
                                     "projected_tok_s": N / (ms_v * 1e-3), "projected_efficiency": (ms_step / wv) / ms_v,
                                     "append": "inside the attention launch" if f_v else "separate launch"}
                strong["one_gpu_share_of_a_deal_over"] = proj
        else:
            ms_s, Ns, my_bytes, fused_s = strong_share(world, rank)
            gather = [None] * world
            dist.all_gather_object(gather, (int(Ns), my_bytes))
            strong = {"value": N / (ms_s * 1e-3), "unit": "tok/s", "ms_per_step": ms_s,
                      "sequences_per_rank": [g_[0] for g_ in gather],
                      "kv_bytes_per_layer_per_rank": [g_[1] for g_ in gather],
                      "hbm_gbs_slowest_rank": max(g_[1] for g_ in gather) * L / (ms_s * 1e-3) / 1e9,
                      "frac_of_peak_slowest_rank": max(g_[1] for g_ in gather) * L / (ms_s * 1e-3) / 1e9 / peak,
                      "efficiency_vs_one_gpu": (ms_step / world) / ms_s,
                      "one_gpu_ms_per_step": ms_step,
                      "append": "inside the attention launch" if fused_s else "separate launch",
                      "policy": "balanced: longest context first to the least loaded rank; total batch fixed at "
                                f"{N} sequences; one-GPU time = this run's whole-batch step on one rank"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        import oracle
        checker = oracle.load_ref()
        kind = "reference"
        if checker is None:
            checker, kind = oracle.load_orc(), "port"
        threads = oracle.ref_default_thread_count()
        w0 = wl.make(args.workload)
        cpu_step, n0 = cpu_step_fn(w0, checker, threads)
        cpu_step()
        t = min(cpu_step() for _ in range(2))
        cpu = {"value": n0 / t, "unit": "tok/s", "cores": threads, "kind": kind,
               "sample": f"whole steps (all {w0.layers} layers over all {w0.n_seqs} sequences, append + attention), one warm-up, best of 2"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w.dtype,
            "data": "synthetic",
            "config": {"workload": f"{args.workload}: {WORKLOAD_TEXT[args.workload]}", "tokens_per_step_per_gpu": N,
                       "layers": L, "sharding": "by sequence: each rank owns its pool and its batch, no collective",
                       "l2": f"per-step working set {algo_bytes * L / 1e9:.2f} GB across {L} distinct per-layer pools, far larger than the 126 MB L2",
                       "launch": "cuda graph replay" if use_graph else "eager launches",
                       "plan": "split-K plan built on the host once, at capture, and its upload replayed: `value` holds no per-step host "
                               "planning (positions change every step in serving); `e2e` re-plans on the host every step",
                       "cpu_affinity": getattr(args, "affinity_note", None),
                       "append": "inside the attention launch (pkv_append_decode_attn_planned)" if fused else "separate launch (pkv_append)",
                       "attention_form": (f"clusters of {cluster_form} blocks per (token, kv head), merge inside the launch"
                                          if cluster_form else "split-K units + merge launch"),
                       **({"layers_override": args.layers} if args.layers else {})},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "step_hbm_gbs": (algo_bytes + w.append_bytes_per_layer()) * L / (ms_step * 1e-3) / 1e9,
            "strong": strong,
        }
        if getattr(args, "return_line", False):
            return line
        if world == 1 and not args.no_secondary:
            line["secondary"] = secondary_measurements(args, pkv, wl, torch, dev, pools, w)
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
        if getattr(args, "return_line", False):
            return line
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
    pkv.launch_copy_blocks_layers(ptrs, 2 * L, pa, len(pairs), block_bytes)      # the workload's own copy-on-write wave
    torch.cuda.synchronize()
    # Its speed is measured on waves of the same shape over rotating disjoint pair lists: repeating the one
    # wave (92 MB read + written) would time the 126 MB L2, not HBM.
    import types
    cow = measure_cow_rotated(pkv, torch, dev, pools, types.SimpleNamespace(block_size=bs, kv_dim=kv_dim, elem_bytes=2, num_blocks=nb),
                              pairs_per_set=len(pairs))
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
            "cow": cow,
            "roofline": {"bound": "hbm", "kernel": "decode_tma_kernel + decode_combine_kernel (whole step incl. host)",
                         "achieved": byts / steps / (ms_step * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": byts / steps / (ms_step * 1e-3) / 1e9 / peak, "traffic": None, "peak_source": src},
            "shared_prefix_plan": shared_cmp,
            "cpu_baseline": None, "e2e": {"value": S * steps / wall, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                                          "note": "wall clock over the same 64 steps"},
            "gpu_launches": 3 * L * steps}
    if rank == 0:
        print(json.dumps(line), flush=True)


def measure_cow_rotated(pkv, torch, dev, pools, w, sets=8, pairs_per_set=127, waves=40):
    """Copy-on-write block copy at HBM speed rather than out of L2: `sets` disjoint lists of block pairs
    are copied in rotation over every pool of the model in one launch each, so that a block is touched
    again only after sets x pairs x pools x 2 x block_bytes (several times the 126 MB L2) of other
    traffic.  Pool contents are overwritten (blocks copied over blocks): call it last."""
    L = pools.shape[0]
    block_bytes = w.block_size * w.kv_dim * w.elem_bytes
    ptrs = torch.tensor([pools[l, j].data_ptr() for l in range(L) for j in range(2)], dtype=torch.int64, device=dev)
    ids = np.random.default_rng(5).permutation(w.num_blocks)[:2 * sets * pairs_per_set].astype(np.int32)
    lists = [torch.from_numpy(np.ascontiguousarray(ids[2 * i * pairs_per_set:2 * (i + 1) * pairs_per_set].reshape(-1, 2))).to(dev)
             for i in range(sets)]
    wave_bytes = 2 * pairs_per_set * block_bytes * 2 * L
    for i in range(sets):
        pkv.launch_copy_blocks_layers(ptrs, 2 * L, lists[i], pairs_per_set, block_bytes)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(waves):
        pkv.launch_copy_blocks_layers(ptrs, 2 * L, lists[i % sets], pairs_per_set, block_bytes)
    b.record()
    torch.cuda.synchronize()
    us = a.elapsed_time(b) / waves * 1e3
    peak, _ = peaks()
    return {"kernel": "copy_blocks_kernel", "pairs_per_wave": pairs_per_set, "pools": 2 * L, "disjoint_pair_sets_in_rotation": sets,
            "bytes_read_plus_written_per_wave": wave_bytes, "bytes_between_reuse_of_a_block": wave_bytes * sets,
            "us_per_wave": us, "GBps": wave_bytes / us / 1e3, "frac_of_measured_hbm": wave_bytes / us / 1e3 / peak}


def measure_mixed_step(pkv, torch, dev):
    """A step as llm-engine's forward pass hands it to launch_attention_decode: two 300-token prefill chunks
    plus 20 decode tokens (Qwen2.5-0.5B shapes, f16).  Timed per attention call: through the mixed entry
    point (chunks routed to the tensor-core prefill kernel on the device) and through the decode entry
    point (every chunk token a decode unit that re-reads its whole history, which is what the
    reference's launcher does)."""
    qh, kvh, hd, bs = 14, 2, 64, 16
    rng = np.random.default_rng(21)
    ctx = [1200, 700] + [int(x) for x in rng.integers(200, 3000, size=20)]
    new = [300, 300] + [1] * 20
    nb = sum((c + n + bs - 1) // bs for c, n in zip(ctx, new)) + 8
    perm = rng.permutation(nb).astype(np.int32)
    tabs, pos, at = [], [], 0
    for c, n in zip(ctx, new):
        kb = (c + n + bs - 1) // bs
        t = perm[at:at + kb].copy()
        at += kb
        for i in range(n):
            tabs.append(t)
            pos.append(c + i)
    idx = pkv.pack_step(tabs, pos, bs)
    N = idx.n_tokens
    f16 = lambda *shape: torch.randn(shape, device=dev, dtype=torch.float32).to(torch.float16)
    kc, vc, q = f16(nb * bs, kvh * hd), f16(nb * bs, kvh * hd), f16(N, qh * hd)
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
    d = [i32(idx.block_tables), i32(idx.table_offset), i32(idx.token_seq), i32(idx.token_pos)]
    out_m, out_d = torch.zeros_like(q), torch.zeros_like(q)
    ws = torch.empty(pkv.mixed_workspace_bytes(N, qh, kvh, hd), dtype=torch.uint8, device=dev)
    scale = 1.0 / float(np.sqrt(hd))
    mixed = lambda: pkv.launch_attention_mixed(q, kc, vc, *d, out_m, N, qh, kvh, hd, bs, scale, ws, num_blocks=nb)
    plain = lambda: pkv.launch_attention_decode(q, kc, vc, *d, out_d, N, qh, kvh, hd, bs, scale, workspace=ws)
    res = {}
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name, fn in (("mixed_entry_point", mixed), ("decode_entry_point", plain)):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        a.record()
        for _ in range(30):
            fn()
        b.record()
        torch.cuda.synchronize()
        res[name + "_us_per_call"] = a.elapsed_time(b) / 30 * 1e3
    diff = (out_m.float() - out_d.float()).abs().max().item()
    res.update({"step": "2 x 300-token chunks (cached 1,200 and 700) + 20 decode tokens, 14q/2kv heads, d64, f16", "tokens": N,
                "max_abs_difference_between_the_two": diff,
                "speedup": res["decode_entry_point_us_per_call"] / res["mixed_entry_point_us_per_call"]})
    return res


def run_cow(args, rank, local_rank, world):
    """--workload cow: the block copy of configuration 5 by itself, out of HBM (rotating pair lists)."""
    import torch
    pkv = importlib.import_module("llm-engine_b200")
    wl = importlib.import_module("llm-engine_b200.workloads")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    w = wl.make("cfg5", layers=args.layers or 22)
    pools = torch.randn((w.layers, 2, w.num_blocks * w.block_size, w.kv_dim), device=dev, dtype=torch.float32).to(torch.bfloat16)
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    res = measure_cow_rotated(pkv, torch, dev, pools, w, waves=max(args.steps, 8) * 4)
    clocks = sampler.stop()
    if rank == 0:
        peak, src = peaks()
        print(json.dumps({"metric": "copy-on-write block copy GB/s (read + written)", "value": res["GBps"], "unit": "GB/s", "n_gpus": world,
                          "steps": max(args.steps, 8) * 4, "warmup": 8, "ms_per_step": res["us_per_wave"] / 1e3, "higher_is_better": True,
                          "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
                          "config": {"workload": f"cow: {WORKLOAD_TEXT['cow']}", "l2": "a block is touched again only after 8 waves (733 MB) of other traffic"},
                          "roofline": {"bound": "hbm", "kernel": "copy_blocks_kernel", "achieved": res["GBps"], "peak": peak, "unit": "GB/s",
                                       "frac": res["GBps"] / peak, "traffic": None, "peak_source": src,
                                       "algorithmic_bytes_per_launch": res["bytes_read_plus_written_per_wave"], "us_per_launch": res["us_per_wave"]},
                          "cpu_baseline": None, "e2e": None, "gpu_launches": max(args.steps, 8) * 4, "clocks": clocks, "detail": res}), flush=True)


def run_mixed(args, rank, local_rank, world):
    """--workload mixed: the mixed step by itself (the router's kernels are easiest to profile this way)."""
    import torch
    pkv = importlib.import_module("llm-engine_b200")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    res = measure_mixed_step(pkv, torch, dev)
    clocks = sampler.stop()
    if rank == 0:
        us = res["mixed_entry_point_us_per_call"]
        print(json.dumps({"metric": "mixed-step attention calls per second (prefill chunks routed to the tensor-core kernel)", "value": 1e6 / us,
                          "unit": "calls/s", "n_gpus": world, "steps": 30, "warmup": 5, "ms_per_step": us / 1e3,
                          "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                          "config": {"workload": f"mixed: {WORKLOAD_TEXT['mixed']}"}, "roofline": None, "cpu_baseline": None, "e2e": None,
                          "gpu_launches": None, "clocks": clocks, "detail": res}), flush=True)


def secondary_measurements(args, pkv, wl, torch, dev, pools, w):
    """Short runs of the other kernels on the box the default line is measured on (one GPU only): the
    tcgen05 prefill kernel on configuration 4's launch, the small-batch decode step of configuration 2,
    the copy-on-write block copy out of HBM, and a mixed step through both attention entry points."""
    import copy
    sec = {}
    a2 = copy.copy(args)
    a2.return_line, a2.no_cpu, a2.no_e2e, a2.no_strong, a2.no_secondary = True, True, True, True, True
    try:
        a2.workload, a2.layers, a2.steps, a2.warmup = "cfg4", 4, 8, 3
        ln = run_prefill(a2, 0, dev.index, 1)
        r = ln["roofline"]
        sec["cfg4_prefill"] = {"kernel": r["kernel"], "us_per_launch": r["us_per_launch"], "TFLOPs": r["achieved"], "frac_of_burst_peak": r["frac"],
                               "frac_of_sustained_peak": r["frac_of_sustained"], "algorithmic_flops_per_launch": r["algorithmic_flops_per_launch"],
                               "layers_run": 4, "clocks": ln["clocks"]}
    except Exception as e:
        sec["cfg4_prefill"] = {"error": repr(e)}
    try:
        a2.workload, a2.layers, a2.steps, a2.warmup = "cfg2", None, 20, 5
        ln = run_ours(a2, 0, dev.index, 1)
        r = ln["roofline"]
        sec["cfg2_decode"] = {"value_tok_s": ln["value"], "ms_per_step": ln["ms_per_step"], "us_per_layer_in_graph": ln["ms_per_step"] * 1e3 / ln["config"]["layers"],
                              "step_hbm_gbs": ln["step_hbm_gbs"], "frac_of_peak_whole_step": ln["step_hbm_gbs"] / r["peak"],
                              "attention_us_per_launch_eager": r["us_per_launch"], "attention_frac_eager": r["frac"],
                              "append": ln["config"]["append"], "launch": ln["config"]["launch"],
                              "attention_form": ln["config"]["attention_form"]}
    except Exception as e:
        sec["cfg2_decode"] = {"error": repr(e)}
    prev_env = None
    try:
        # the same step with the cluster form switched off: append + attention, then the merge launch
        prev_env = os.environ.get("PKV_DECODE_CLUSTER")
        os.environ["PKV_DECODE_CLUSTER"] = "0"
        ln = run_ours(a2, 0, dev.index, 1)
        sec["cfg2_decode_ordinary_form"] = {"value_tok_s": ln["value"], "us_per_layer_in_graph": ln["ms_per_step"] * 1e3 / ln["config"]["layers"],
                                           "attention_us_per_launch_eager": ln["roofline"]["us_per_launch"],
                                           "attention_form": ln["config"]["attention_form"]}
    except Exception as e:
        sec["cfg2_decode_ordinary_form"] = {"error": repr(e)}
    finally:
        if prev_env is None:
            os.environ.pop("PKV_DECODE_CLUSTER", None)
        else:
            os.environ["PKV_DECODE_CLUSTER"] = prev_env
    try:
        sec["mixed_step"] = measure_mixed_step(pkv, torch, dev)
    except Exception as e:
        sec["mixed_step"] = {"error": repr(e)}
    try:
        sec["cow_copy"] = measure_cow_rotated(pkv, torch, dev, pools, w)
    except Exception as e:
        sec["cow_copy"] = {"error": repr(e)}
    return sec


def bind_rank_to_cores(local_rank, world):
    """One process per GPU on a host whose cores all sit behind one NUMA node: give every rank its own
    slice of the cores this job may use, so that eight launch loops do not migrate over each other."""
    try:
        cores = sorted(os.sched_getaffinity(0))
        per = len(cores) // world
        if world > 1 and per >= 1:
            mine = cores[local_rank * per:(local_rank + 1) * per]
            os.sched_setaffinity(0, mine)
            return f"rank bound to {len(mine)} of {len(cores)} cores ({mine[0]}-{mine[-1]})"
    except Exception:
        pass
    return None


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
    ap.add_argument("--no-strong", action="store_true", help="skip the strong-scaling block (one batch dealt over the ranks)")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary block (prefill, small-batch decode, block copy, mixed step)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    args.affinity_note = bind_rank_to_cores(local_rank, world)
    if world != args.gpus:
        if args.gpus > 1 and world == 1:
            raise SystemExit("--gpus N > 1 is launched with torch.distributed.run --nproc-per-node N")
    if args.sharding == "head" and world > 1 and args.workload in ("cfg2", "cfg3"):
        run_head_sharded(args, rank, local_rank, world)
    elif args.workload == "cfg4":
        run_prefill(args, rank, local_rank, world)
    elif args.workload == "cfg5":
        run_prefix_cow(args, rank, local_rank, world)
    elif args.workload == "cow":
        run_cow(args, rank, local_rank, world)
    elif args.workload == "mixed":
        run_mixed(args, rank, local_rank, world)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
