#!/usr/bin/env python
"""Headline benchmark: GDN single-token decode at production batch (B=256, Hqk=16, HV=32,
d=128, fp32 k-last state pool of 1024 slots) — state traffic in GB/s against the HBM peak.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One process per GPU (torchrun for N>1). With N GPUs the value heads (and the matching
q/k heads and pool shard) are split across ranks; there is no data-path collective, only
the barrier that brackets the timed region. A "step" is one decode step of the whole
batch: every (request, value head) 128x128 fp32 state is read once and written once.

value : steps timed back to back with inputs resident in HBM (CUDA events on the launch stream).
e2e   : the same step through the public op with the step's activations (packed q|k|v, a, b)
        copied from pinned host memory and the output rows copied back, every step; the copies
        of neighbouring steps overlap the kernel (three streams, double-buffered) and the host
        waits for step i-1's rows while step i runs. The state pool is the engine's resident
        cache, not a per-step input, so it stays in HBM in both measurements.
roofline.achieved : algorithmic state bytes per launch (2 * B * HV_local * 65536) / average
        launch time. cpu_baseline: the CPU oracle (a port of the reference's fp32 PyTorch
        recurrence) timed on the host cores on a bounded sample of the same requests.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

B, HQK, HV, D, SLOTS = 256, 16, 32, 128, 1024
TILE_BYTES = D * D * 4
SEED = 20261125 + 1
METRIC = "gdn_decode_state_bandwidth_B256"
UNIT = "GB/s"
WORKLOAD = "config1: GDN decode B=256 Hqk=16 HV=32 d=128, fp32 k-last pool 1024 slots, random non-consecutive slots"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the full workload (B=256, 32 heads: 8192 tiles),
# from the one-pass ncu capture summarised in profiles/: 541.4 MB read + 476.2 MB written = 1017.6 MB for
# 1073.7 MB of algorithmic bytes (the last ~60 MB written are still dirty in L2 when the kernel ends).
# Reported for that workload only (smaller launches leave a larger share of their writes in L2).
TRAFFIC_BYTES_FULL_LAUNCH = 541374720 + 476201728


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_inputs(hv_lo: int, hv_hi: int, device):
    """Seeded synthetic inputs of config 1 restricted to value heads [hv_lo, hv_hi)."""
    g = torch.Generator().manual_seed(SEED)
    ratio = HV // HQK
    h_lo, h_hi = hv_lo // ratio, (hv_hi + ratio - 1) // ratio
    q = torch.nn.functional.normalize(torch.randn(B, HQK, D, generator=g), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(B, HQK, D, generator=g), dim=-1)
    v = torch.randn(B, HV, D, generator=g)
    a = torch.randn(B, HV, generator=g)
    b = torch.randn(B, HV, generator=g)
    A_log = torch.rand(HV, generator=g) * math.log(16.0)
    dt_bias = torch.randn(HV, generator=g) * 0.1
    perm = torch.randperm(SLOTS, generator=g)                  # SGLang padding rule: slot 0 is an ordinary slot
    slot_sets = [perm[i * B:(i + 1) * B].to(torch.int32) for i in range(SLOTS // B)]   # disjoint sets (4 at B=256)
    hl = h_hi - h_lo
    hvl = hv_hi - hv_lo
    mixed = torch.cat([q[:, h_lo:h_hi].reshape(B, hl * D), k[:, h_lo:h_hi].reshape(B, hl * D),
                       v[:, hv_lo:hv_hi].reshape(B, hvl * D)], dim=1).bfloat16()
    host = dict(mixed=mixed, a=a[:, hv_lo:hv_hi].contiguous().bfloat16(), b=b[:, hv_lo:hv_hi].contiguous().bfloat16())
    const = dict(A_log=A_log[hv_lo:hv_hi].contiguous(), dt_bias=dt_bias[hv_lo:hv_hi].contiguous().bfloat16())
    return host, const, slot_sets, hl, hvl


def run_ours(args):
    from pla_b200.decode import fused_sigmoid_gating_delta_rule_forward_k_last_packed as packed
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    assert HV % world == 0
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    hv_lo, hv_hi = rank * HV // world, (rank + 1) * HV // world
    host, const, slot_sets, hl, hvl = make_inputs(hv_lo, hv_hi, dev)
    pinned = {k_: v_.pin_memory() for k_, v_ in host.items()}
    dev_in = {k_: v_.to(dev) for k_, v_ in host.items()}
    const = {k_: v_.to(dev) for k_, v_ in const.items()}
    g = torch.Generator(device=dev).manual_seed(SEED + rank)
    pool = torch.empty(SLOTS, hvl, D, D, device=dev)
    pool.normal_(0.0, 0.02, generator=g)
    slot_sets = [s.to(dev) for s in slot_sets]
    cu = torch.arange(B + 1, dtype=torch.int32, device=dev)
    out = torch.empty(B, 1, hvl, D, dtype=torch.bfloat16, device=dev)
    out_host = torch.empty(B, 1, hvl, D, dtype=torch.bfloat16).pin_memory()
    scale = D ** -0.5
    stream = torch.cuda.current_stream()

    def step(i, inp):
        packed(inp["mixed"], inp["a"], inp["b"], const["A_log"], const["dt_bias"], 1.0, 20.0, scale, pool,
               slot_sets[i % len(slot_sets)], out, True, cu, False, True, rows_per_cta=args.rows)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ----
    # The K steps are replayed from a CUDA graph of G consecutive steps (G divides K, slot sets keep
    # rotating inside the graph), as a serving engine replays its decode step: at 8 GPUs a step is
    # ~25 us of kernel time and per-call host overhead would otherwise be what is measured.
    for i in range(args.warmup):
        step(i, dev_in)
    G = max(g_ for g_ in range(1, 41) if args.steps % g_ == 0)     # 40 steps per graph at the default 2000
    graph = None
    if not args.no_graph:
        side = torch.cuda.Stream()
        side.wait_stream(stream)
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(G):
                    step(i, dev_in)
        stream.wait_stream(side)
        graph.replay()
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    if graph is not None:
        for _ in range(args.steps // G):
            graph.replay()
    else:
        for i in range(args.steps):
            step(i, dev_in)
    e1.record(stream)
    barrier()
    ms_dev = e0.elapsed_time(e1)

    # ---- end to end: pinned host activations in, output rows out, every step ----
    # A serving engine overlaps the copies of neighbouring steps with the kernel: three streams (H2D,
    # compute, D2H) over double-buffered staging / output buffers. Every step still copies its own inputs
    # from pinned memory and its own output rows back, and the host waits for the previous step's rows
    # before it enqueues the step after next.
    s_in, s_c, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    stages = [{k_: torch.empty_like(v_) for k_, v_ in dev_in.items()} for _ in range(2)]
    outs = [torch.empty_like(out) for _ in range(2)]
    out_hosts = [torch.empty(B, 1, hvl, D, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_c = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i):
        b_ = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_c[b_])          # the kernel that read this staging buffer has finished
            for k_ in stages[b_]:
                stages[b_][k_].copy_(pinned[k_], non_blocking=True)
            ev_in[b_].record(s_in)
        with torch.cuda.stream(s_c):
            s_c.wait_event(ev_in[b_])
            s_c.wait_event(ev_out[b_])         # this output buffer has been copied out
            inp = stages[b_]
            packed(inp["mixed"], inp["a"], inp["b"], const["A_log"], const["dt_bias"], 1.0, 20.0, scale, pool,
                   slot_sets[i % len(slot_sets)], outs[b_], True, cu, False, True, rows_per_cta=args.rows)
            ev_c[b_].record(s_c)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_c[b_])
            out_hosts[b_].copy_(outs[b_], non_blocking=True)
            ev_out[b_].record(s_out)
        ev_out[b_ ^ 1].synchronize()           # the host consumes the previous step's rows

    for s_ in (s_in, s_c, s_out):
        s_.wait_stream(stream)
    for i in range(args.warmup):
        e2e_step(i)
    barrier()
    e2 = torch.cuda.Event(enable_timing=True)
    e3 = torch.cuda.Event(enable_timing=True)
    e2.record(s_in)
    for i in range(args.steps):
        e2e_step(i)
    e3.record(s_out)
    barrier()
    ms_e2e = e2.elapsed_time(e3)   # first H2D enqueued .. last D2H done, host-side gaps included
    clocks = sampler.stop() if rank == 0 else None

    times = torch.tensor([ms_dev, ms_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_dev, ms_e2e = times.tolist()

    total_state_bytes = 2 * B * HV * TILE_BYTES                      # whole job, per step
    local_state_bytes = 2 * B * hvl * TILE_BYTES                     # this GPU's launch
    value = total_state_bytes * args.steps / (ms_dev * 1e-3) / 1e9
    e2e_value = total_state_bytes * args.steps / (ms_e2e * 1e-3) / 1e9
    peak, peak_src = measured_peaks()
    per_launch_s = ms_dev * 1e-3 / args.steps
    achieved = local_state_bytes / per_launch_s / 1e9
    h2d = sum(v_.numel() * v_.element_size() for v_ in host.values())
    d2h = out_host.numel() * out_host.element_size()

    line = None
    if rank == 0:
        cpu = None if args.no_cpu else cpu_baseline_sample()
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_dev / args.steps, 5), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "layout": "k-last packed-QKV op", "launch": ("host call per step" if args.no_graph else f"CUDA graph of {G} steps"), "sharding": f"value heads / {world}",
                       "l2": "each step touches 1 GiB/n_gpus of state; slot sets rotate over disjoint sets of B slots",
                       "frac_of_nominal_8TBps": round(achieved / 8000.0, 4)},
            "e2e": {"value": round(e2e_value, 1), "unit": UNIT, "h2d_bytes_per_step": h2d * world,
                    "d2h_bytes_per_step": d2h * world, "ms_per_step": round(ms_e2e / args.steps, 5),
                    "pipeline": "H2D / kernel / D2H on three streams, double-buffered; host waits for step i-1's rows"},
            "gpu_launches": args.steps,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "peak_source": f"of {peak_src}",
                         "traffic": TRAFFIC_BYTES_FULL_LAUNCH if (B == 256 and hvl == HV and world == 1) else None,
                         "algorithmic_bytes_per_launch": local_state_bytes},
            "cpu_baseline": cpu,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return line


def cpu_oracle_step(n_req: int, reps: int):
    """Times the CPU oracle on the first ``n_req`` requests of the workload (all 32 value heads)."""
    from oracle import decode as odec
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    host, const, slot_sets, hl, hvl = make_inputs(0, HV, "cpu")
    mixed = host["mixed"][:n_req]
    q = mixed[:, : HQK * D].reshape(n_req, HQK, D)
    k = mixed[:, HQK * D: 2 * HQK * D].reshape(n_req, HQK, D)
    v = mixed[:, 2 * HQK * D:].reshape(n_req, HV, D)
    g = torch.Generator().manual_seed(SEED)
    pool = torch.randn(n_req, HV, D, D, generator=g) * 0.02      # pool pre-gathered to the active slots
    idx = list(range(n_req))
    best = float("inf")
    for _ in range(reps + 1):                                    # first pass is warm-up
        t0 = time.perf_counter()
        odec.klast_forward(q=q, k=k, v=v, a=host["a"][:n_req], b=host["b"][:n_req], A_log=const["A_log"],
                           dt_bias=const["dt_bias"], state=pool, slot_indices=idx, lengths=[1] * n_req,
                           scale=D ** -0.5)
        best = min(best, time.perf_counter() - t0)
    gbs = 2 * n_req * HV * TILE_BYTES / best / 1e9
    return gbs, best, threads


def cpu_baseline_sample():
    n_req, reps = 32, 3
    gbs, sec, threads = cpu_oracle_step(n_req, reps)
    return {"value": round(gbs, 3), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"CPU oracle (fp32 torch recurrence) on {n_req} of the 256 requests, best of {reps}; "
                      f"{sec * 1e3:.1f} ms per sample step; state pre-gathered to the active slots"}


def run_reference(args):
    """Reference arm: the reference's own CPU implementation of the path — its fp32 PyTorch
    recurrence, restated in oracle/ because the reference tree is not on the GPU box — on all
    host threads. Rank 0 only."""
    if int(os.environ.get("RANK", 0)) != 0:
        return
    n_req = 32 if args.steps <= 200 else 8           # keeps the whole run within a few minutes
    threads = os.cpu_count() or 1
    for _ in range(args.warmup):
        cpu_oracle_step(n_req, 0)
    total = 0.0
    for _ in range(args.steps):
        _, sec, threads = cpu_oracle_step(n_req, 0)
        total += sec
    value = 2 * n_req * HV * TILE_BYTES * args.steps / total / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(total / args.steps * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": f"{n_req} of 256 requests per step"},
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{n_req} of the 256 requests per step, all host threads"},
        "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _time_steps(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run_prefill(args):
    """Secondary line (not the headline metric): config 3, GDN packed varlen prefill, 8 sequences with
    lengths ~U[512, 8192], Hqk=16, HV=32, indexed fp32 pool; Mtok/s on one GPU."""
    from pla_b200.prefill.flashqla import gdn_prefill_packed_qkv_fwd
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(20261125 + 3)
    lengths = torch.randint(512, 8193, (8,), generator=g).tolist()
    T = sum(lengths)
    width = 2 * HQK * D + HV * D
    storage = torch.empty(T, width + 64, dtype=torch.bfloat16, device=dev)
    packed = storage[:, 17:17 + width]
    gd = torch.Generator(device=dev).manual_seed(5)
    packed.normal_(0.0, 1.0, generator=gd)
    for lo in (0, HQK * D):   # q, k L2-normalised per head, as in config 0
        blk = packed[:, lo:lo + HQK * D].float().view(T, HQK, D)
        packed[:, lo:lo + HQK * D] = torch.nn.functional.normalize(blk, dim=-1).view(T, HQK * D).bfloat16()
    gates = torch.randn(T, 2 * HV, generator=g).bfloat16().to(dev)
    A_log = (torch.rand(HV, generator=g) * math.log(16.0)).to(dev)
    dt_bias = (torch.randn(HV, generator=g) * 0.1).to(dev)
    pool = (torch.randn(16, HV, D, D, generator=g) * 0.02).to(dev)
    idx = torch.tensor([1, 3, 5, 7, 9, 11, 13, 15], dtype=torch.int32, device=dev)
    offs = [0]
    for n in lengths:
        offs.append(offs[-1] + n)
    cu = torch.tensor(offs, dtype=torch.int32, device=dev)

    def step():
        gdn_prefill_packed_qkv_fwd(packed, gates[:, :HV], gates[:, HV:], A_log, dt_bias, cu, num_qk_heads=HQK,
                                   num_v_heads=HV, initial_state=pool, initial_state_indices=idx,
                                   output_final_state=False, raw_cu_seqlens=tuple(offs))

    ms = _time_steps(step, args.steps, max(args.warmup, 3))
    flops = T * (HV * 133803 + HQK * 32768)
    print(json.dumps({"metric": "gdn_prefill_throughput_32K_varlen", "value": round(T / ms / 1e3, 3), "unit": "Mtok/s",
                      "n_gpus": 1, "steps": args.steps, "ms_per_step": round(ms, 4), "higher_is_better": True,
                      "dtype": "f32", "data": "synthetic",
                      "config": {"workload": f"config3: 8 sequences {lengths}, T={T}, Hqk=16 HV=32, chunk 64 on the tensor cores (tf32)",
                                 "chunk_equivalent_tflops": round(flops / ms / 1e9, 2),
                                 "algorithmic_GBps": round(T * 24.7e3 / ms / 1e6, 1)}}), flush=True)


def run_prefill_cp(args):
    """Secondary lines for config 4, one long sequence cut into contiguous token ranges over the ranks
    (prescan -> all-gather of (offset, transition) -> fold -> segment pass):
    prefill_cp      GDN, 64K tokens, Hqk=8, HV=24, chunk-64 tensor-core kernels;
    prefill_cp_kda  KDA, 128K tokens, 32 heads, per-channel softplus gate with weak decay
                    (A_log ~ U(-4, -2)), token-recurrent kernel."""
    import torch.distributed as dist
    from pla_b200._ops import ops
    from pla_b200.prefill.context_parallel import gdn_prefill_context_parallel, kda_prefill_context_parallel
    kda = args.workload == "prefill_cp_kda"
    rank, world, local = (int(os.environ.get(k_, d_)) for k_, d_ in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    T, Hg, H = (131072, 32, 32) if kda else (65536, 8, 24)
    if args.tokens:
        T = args.tokens          # profiling aid; the workload string then says so
    per = (T // world + 63) // 64 * 64
    lo, hi = min(rank * per, T), min((rank + 1) * per, T)
    gd = torch.Generator(device=dev).manual_seed(44)

    def draw(*shape):
        """Every rank draws the whole tensor from the same seed and keeps its token range (rank 0 keeps all
        of it for the single-pass comparison)."""
        full = torch.randn(*shape, generator=gd, device=dev)
        return full if rank == 0 else full[lo:hi].clone()

    q = torch.nn.functional.normalize(draw(T, Hg, D), dim=-1).bfloat16()
    k = torch.nn.functional.normalize(draw(T, Hg, D), dim=-1).bfloat16()
    v = draw(T, H, D).bfloat16()
    gate = (draw(T, H, D) if kda else draw(T, H)).bfloat16()
    beta = draw(T, H).bfloat16()
    u = torch.rand(H, generator=gd, device=dev)
    A_log = (-4.0 + 2.0 * u) if kda else u * math.log(16.0)
    dt_bias = torch.randn(H, D, generator=gd, device=dev) * 0.1 if kda else torch.randn(H, generator=gd, device=dev) * 0.1
    S0 = torch.randn(H, D, D, generator=gd, device=dev) * 0.02
    sl = slice(lo, hi) if rank == 0 else slice(None)
    mine = [x[sl] for x in (q, k, v, gate, beta)]
    steps = min(args.steps, 5) if (kda and args.kda_backend == "recurrent") else args.steps

    ranges_on_one_gpu = world == 1 and (not kda or args.kda_backend == "chunked")
    if ranges_on_one_gpu:
        # one GPU: the same prescan / fold / segment scheme over token ranges inside the GPU, through the facade
        from pla_b200.prefill.flashqla import ops as fq
        pool1 = S0[None].clone()
        slot0 = torch.zeros(1, dtype=torch.int32, device=dev)
        cu1 = torch.tensor([0, T], dtype=torch.int32, device=dev)

    if ranges_on_one_gpu and kda:
        from pla_b200.prefill.flashkdapro import flashkda_fwd
        out1 = torch.empty(T, H, D, dtype=torch.bfloat16, device=dev)
        status1 = torch.zeros(1, dtype=torch.int32, device=dev)

    def step():
        if ranges_on_one_gpu and kda:
            flashkda_fwd(q, k, v, gate, beta, A_log, dt_bias, out1, None, None, state_pool=pool1, state_indices=slot0,
                         raw_cu_seqlens=(0, T), backend="chunked", status=status1)
            return out1, pool1[0]
        if ranges_on_one_gpu:
            res = fq.chunk_gated_delta_rule_fwd(q[None], k[None], v[None], None, None, initial_state=pool1,
                                                initial_state_indices=slot0, cu_seqlens=cu1, output_final_state=False,
                                                auto_cp=True, normalize_qk=True, raw_cu_seqlens=(0, T), raw_gate_a=gate,
                                                raw_beta_b=beta, A_log=A_log, dt_bias=dt_bias)
            return res[2][0], pool1[0]
        if kda:
            return kda_prefill_context_parallel(*mine, A_log, dt_bias, None, initial_state=S0, backend=args.kda_backend)
        return gdn_prefill_context_parallel(*mine, A_log, dt_bias, initial_state=S0)

    for _ in range(1 if (kda and args.kda_backend == "recurrent") else max(args.warmup, 3)):
        o, final = step()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        o, final = step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    if ranges_on_one_gpu:
        pool1.copy_(S0[None])             # the pool is updated in place: restart from S0 for the comparison
        o, final = step()
    if rank == 0:
        # the same kernels in a single pass over the whole sequence, for comparison
        one = torch.empty(T, H, D, dtype=torch.bfloat16, device=dev)
        fin = torch.empty(1, H, D, D, dtype=torch.float32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        if kda and args.kda_backend == "chunked":
            ops.kda_prefill_chunked(q, k, v, gate, beta, A_log, dt_bias, one, cu, S0[None].contiguous(), None, fin, None,
                                    None, False, True, D ** -0.5, None, False, T // 64, 0, False, status)
        elif kda:
            ops.prefill_recurrent(q, k, v, gate, beta, A_log, dt_bias, one, cu, S0[None].contiguous(), None, fin, None,
                                  False, True, True, D ** -0.5, None, False, False, status)
        else:
            ops.gdn_prefill_chunked(q, k, v, gate, beta, A_log, dt_bias, one, None, cu, S0[None].contiguous(), None, fin,
                                    None, False, True, D ** -0.5, False, False, T // 64, 0, status)
        rel = lambda a, b: float((a.float() - b.float()).norm() / b.float().norm())
        what = (f"config4 (KDA part): 1 sequence, T={T}, 32 heads, softplus gate, A_log~U(-4,-2), "
                + ("chunk 64 (tf32) tensor-core kernels" if args.kda_backend == "chunked" else "token-recurrent kernel")
                if kda else f"config4 (GDN part): 1 sequence, T={T}, Hqk=8 HV=24, chunk 64 (tf32)")
        if args.tokens:
            what = "REDUCED (profiling aid) " + what
        print(json.dumps({"metric": "kda_prefill_context_parallel_128K" if kda else "gdn_prefill_context_parallel_64K",
                          "value": round(T / ms / 1e3, 3),
                          "unit": "Mtok/s", "n_gpus": world, "steps": steps, "ms_per_step": round(ms, 4),
                          "higher_is_better": True, "scaling": "strong", "dtype": "f32", "data": "synthetic",
                          "config": {"workload": (f"{what}, {len(fq.plan_token_ranges([0, T], H, 148)[2])} token ranges "
                                                  "inside the GPU (prescan, fold, segment pass)") if ranges_on_one_gpu else
                                                 (f"{what}, {per} tokens per rank, one all-gather of "
                                                  f"[{H},2,128,128] fp32 per rank"),
                                     "out_rel_l2_vs_single_pass": rel(o, one[lo:hi]),
                                     "state_rel_l2_vs_single_pass": rel(final, fin[0]),
                                     "status": int(status.item())}}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def run_vlast(args):
    """Secondary line: config 1 in the v-last layout ([slots, HV, K, V] pool) through
    pla_b200.decode.gdn.v_last, one GPU, device-resident steps."""
    from pla_b200.decode.gdn.v_last import fused_sigmoid_gating_delta_rule
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(SEED)
    q = torch.nn.functional.normalize(torch.randn(B, 1, HQK, D, generator=g), dim=-1).bfloat16().to(dev)
    k = torch.nn.functional.normalize(torch.randn(B, 1, HQK, D, generator=g), dim=-1).bfloat16().to(dev)
    v = torch.randn(B, 1, HV, D, generator=g).bfloat16().to(dev)
    a = torch.randn(B, HV, generator=g).bfloat16().to(dev)
    b = torch.randn(B, HV, generator=g).bfloat16().to(dev)
    A_log = (torch.rand(HV, generator=g) * math.log(16.0)).to(dev)
    dt_bias = (torch.randn(HV, generator=g) * 0.1).bfloat16().to(dev)
    perm = torch.randperm(SLOTS, generator=g)
    sets = [perm[i * B:(i + 1) * B].to(torch.int32).to(dev) for i in range(SLOTS // B)]
    pool = torch.empty(SLOTS, HV, D, D, device=dev).normal_(0.0, 0.02, generator=torch.Generator(device=dev).manual_seed(1))
    o = torch.empty(B, 1, HV, D, dtype=torch.bfloat16, device=dev)
    i_ = [0]

    def step():
        fused_sigmoid_gating_delta_rule(A_log, a, dt_bias, q, k, v, b, o, pool, sets[i_[0] % len(sets)], None, 1.0, 20.0,
                                        D ** -0.5, 1, B, HQK, HV, D, D, True, True, False)
        i_[0] += 1

    ms = _time_steps(step, args.steps, max(args.warmup, 3))
    gbs = 2 * B * HV * TILE_BYTES / (ms * 1e-3) / 1e9
    print(json.dumps({"metric": "gdn_decode_state_bandwidth_B256_vlast", "value": round(gbs, 1), "unit": "GB/s",
                      "n_gpus": 1, "steps": args.steps, "ms_per_step": round(ms, 5), "higher_is_better": True,
                      "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "config1 (v-last half): GDN decode B=256 Hqk=16 HV=32 d=128, fp32 v-last pool "
                                             "1024 slots, 4 disjoint slot sets rotated", "launch": "host call per step"},
                      "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": measured_peaks()[0], "unit": "GB/s",
                                   "frac": round(gbs / measured_peaks()[0], 4),
                                   "peak_source": "of " + measured_peaks()[1]}}),
          flush=True)


def run_conv(args):
    """Secondary line: the causal conv in front of config 3's prefill (8 sequences, ~32K token rows of the packed
    q|k|v width 8192, bf16), history pool of 64 slots; algorithmic bytes = one read and one write of every row."""
    from pla_b200.prefill.causal_conv import causal_conv1d_fn
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(SEED + 3)
    lengths = torch.randint(512, 8193, (8,), generator=g).tolist()
    T, C = sum(lengths), 8192
    offs = [0]
    for n in lengths:
        offs.append(offs[-1] + n)
    x = torch.randn(T, C, generator=g).bfloat16().to(dev)
    w = (torch.randn(C, 4, generator=g) * 0.2).to(dev)
    state = torch.zeros(64, 3, C, dtype=torch.bfloat16, device=dev).transpose(1, 2)
    idx = torch.randperm(64, generator=g)[:8].to(torch.int32).to(dev)
    cu = torch.tensor(offs, dtype=torch.int32, device=dev)
    y = torch.empty_like(x)

    def step():
        causal_conv1d_fn(x, w, None, state, cu, idx, None, "silu", out=y)

    ms = _time_steps(step, args.steps, max(args.warmup, 3))
    gbs = 2 * T * C * 2 / (ms * 1e-3) / 1e9
    print(json.dumps({"metric": "causal_conv_prefill_bandwidth", "value": round(gbs, 1), "unit": "GB/s", "n_gpus": 1,
                      "steps": args.steps, "ms_per_step": round(ms, 5), "higher_is_better": True, "dtype": "f32",
                      "data": "synthetic",
                      "config": {"workload": f"causal conv (width 4, SiLU) in front of config3: 8 sequences {lengths}, "
                                             f"T={T}, {C} channels bf16, 1.3 GB touched per step (> L2)"},
                      "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": measured_peaks()[0], "unit": "GB/s",
                                   "frac": round(gbs / measured_peaks()[0], 4),
                                   "peak_source": "of " + measured_peaks()[1]}}), flush=True)


def run_replay(args):
    """Secondary line: config 2, KDA ReplaySSM verify + commit, 32 heads, 64 rows x 4 tokens, 512 pages."""
    import numpy as np
    sys.path.insert(0, str(ROOT / "tests" / "golden"))
    import cases
    from pla_b200.decode.kda_replayssm_vllm import KDAReplayCommitContext, KDAReplayRecords, kda_replay_verify
    H, N, Q, pages = 32, 64, 4, 512
    rs = np.random.RandomState(20261125 + 2)
    layer = cases.replay_layer(rs, pages, H, Q, "SD", device="cuda")
    x = cases.replay_inputs(rs, H, N * Q, device="cuda")
    layer.replay_records = KDAReplayRecords.allocate(N, H, Q, "cuda")
    slots = torch.tensor((rs.permutation(pages - 1)[:N] + 1).astype("int32"), device="cuda")
    cu = torch.arange(0, N * Q + 1, Q, dtype=torch.int32, device="cuda")
    sampled = torch.tensor(rs.randint(1, Q + 1, N).astype("int32"), device="cuda")
    out = torch.empty(N * Q, H * D, dtype=torch.bfloat16, device="cuda")
    ctx = KDAReplayCommitContext.create([layer], Q, N, conv_state_layout="SD")
    kw = {k_: v_ for k_, v_ in x.items() if k_ != "storage"}

    def verify():
        kda_replay_verify(**kw, conv_state=layer.kv_cache[0], checkpoint_state=layer.kv_cache[1],
                          records=layer.replay_records, query_start_loc=cu, state_indices=slots,
                          conv_state_layout="SD", out=out)

    def commit():
        ctx.commit(sampled, slots, cu, token_capacity=N * Q)

    ms_v = _time_steps(verify, args.steps, max(args.warmup, 3))
    ms_c = _time_steps(commit, args.steps, max(args.warmup, 3))
    state_v, state_c = N * H * TILE_BYTES, 2 * N * H * TILE_BYTES
    print(json.dumps({"metric": "kda_replay_verify_commit_state_bandwidth", "unit": "GB/s",
                      "value": round((state_v + state_c) / ((ms_v + ms_c) * 1e-3) / 1e9, 1),
                      "n_gpus": 1, "steps": args.steps, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "config2: H=32, 64 rows x 4 tokens, 512 pages, accepted ~U{1..4}",
                                 "verify_ms": round(ms_v, 4), "commit_ms": round(ms_c, 4),
                                 "verify_GBps": round(state_v / ms_v / 1e6, 1),
                                 "commit_GBps": round(state_c / ms_c / 1e6, 1)}}), flush=True)


def main():
    global B, SLOTS, WORKLOAD
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="decode", choices=["decode", "decode_vlast", "prefill", "prefill_cp", "prefill_cp_kda", "replay", "conv"],
                    help="decode = the headline metric; prefill / replay print secondary lines (1 GPU)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=0,
                    help="prefill_cp / prefill_cp_kda: sequence length override (profiling aid, multiple of 64)")
    ap.add_argument("--kda-backend", default="chunked", choices=["chunked", "recurrent"],
                    help="prefill_cp_kda: chunk-64 tensor-core kernels or the exact token recurrence")
    ap.add_argument("--rows", type=int, default=0, help="state rows per CTA (0 = library default)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample (tuning runs)")
    ap.add_argument("--no-graph", action="store_true", help="launch every step from the host instead of a CUDA graph")
    ap.add_argument("--batch", type=int, default=B, help="requests per step (profiling aid; the metric is quoted at 256)")
    ap.add_argument("--slots", type=int, default=SLOTS, help="pool slots (profiling aid; default 1024)")
    args = ap.parse_args()
    if (args.batch, args.slots) != (B, SLOTS):
        B, SLOTS = args.batch, args.slots
        WORKLOAD = f"REDUCED (not the headline): GDN decode B={B} Hqk=16 HV=32 d=128, fp32 k-last pool {SLOTS} slots"
    if args.workload in ("prefill_cp", "prefill_cp_kda"):
        args.steps = min(args.steps, 50)
        run_prefill_cp(args)
        return
    if args.workload != "decode":
        if int(os.environ.get("RANK", 0)) == 0:
            args.steps = min(args.steps, 50)
            {"prefill": run_prefill, "replay": run_replay, "decode_vlast": run_vlast, "conv": run_conv}[args.workload](args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        if args.warmup < 3:
            args.warmup = 3
        run_ours(args)


if __name__ == "__main__":
    main()
