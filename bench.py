#!/usr/bin/env python
"""Benchmark of the linear-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One process per GPU (torchrun for N > 1). One JSON line comes out of rank 0. Its headline keys are the first
half of the metric -- GDN single-token decode at production batch (B=256, Hqk=16, HV=32, d=128, fp32 k-last
pool of 1024 slots): state traffic in GB/s against the HBM peak -- and the object ``prefill`` carries the second
half: chunked GDN prefill of ~32K packed varlen tokens in Mtok/s. With N GPUs the value heads (and the matching
q/k heads and pool shard) are split across the ranks for both; neither has a data-path collective. The objects
``prefill_cp`` / ``prefill_cp_kda`` time one long sequence cut into token ranges over the ranks (one NCCL
all-gather of chunk-boundary state pairs inside the timed region), ``secondary`` holds short runs of the other
operators of the path (v-last layout, bf16 pool, ReplaySSM verify + commit, causal conv, fused KDA decode step).

A decode "step" is one decode step of the whole batch: every (request, value head) 128x128 fp32 state is read
once and written once. A prefill "step" is one pass over the packed batch.

value : K steps timed back to back with inputs resident in HBM (CUDA events on the launch stream), the K-step
        block repeated and the MEDIAN block reported (``spread`` gives min / max / repeats).
e2e   : the same step through the public op with the step's inputs copied from ONE pinned host buffer (one
        copy per step) and the step's output rows copied back, every step. The copies of neighbouring steps
        overlap the kernel (three streams, double-buffered), captured in a CUDA graph so that the host enqueues
        nothing per step. The state pool is the engine's resident cache, not a per-step input.
roofline.achieved : algorithmic bytes (decode) or chunk-equivalent flops (prefill) per step / step time.
cpu_baseline : the CPU oracle (a port of the reference's fp32 PyTorch recurrence) timed on the host cores on a
        bounded sample of the same workload, at N = 1 only and before any GPU work starts.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the full decode workload (B=256, 32 heads: 8192
# tiles), from the one-pass ncu capture summarised in profiles/ (mean of three launches): 541.3 MB read + 479.4 MB
# written = 1020.7 MB for 1073.7 MB of algorithmic bytes (the last ~57 MB written are still dirty in L2 when the
# kernel ends). Reported for that workload only (smaller launches leave a larger share of their writes in L2).
TRAFFIC_BYTES_FULL_LAUNCH = 541260885 + 479420075
# The same sum over the kernels of one config-3 prefill step (prepare, inverse, chain: one launch each), from profiles/.
PREFILL_TRAFFIC_BYTES = 4_081_566_208
PREFILL_FLOP_PER_TOKEN_HV = 133803     # chunk-equivalent tensor work per token and value head
PREFILL_FLOP_PER_TOKEN_HQK = 32768     # ... and per q/k head (K K^T and Q K^T)


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["hbm_gbs"]), float(d["bf16_tflops_sustained"]), "measured"
        except Exception:
            pass
    return 6650.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi for as long as the GPU work of the bench runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,utilization.gpu")

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
        sm, mx, busy, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clk, top, util = float(parts[0]), float(parts[1]), float(parts[6])
            except ValueError:
                continue
            sm.append(clk)
            mx.append(top)
            if util > 0:
                busy.append(clk)
            for n, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        under_load = busy or sm
        return {"sm_mhz": statistics.median(under_load) if under_load else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "samples_under_load": len(busy), "reasons": sorted(reasons)}


class Ranks:
    """Rank bookkeeping plus the barrier / rank-max helpers every section uses."""

    def __init__(self, gpus: int):
        self.rank = int(os.environ.get("RANK", 0))
        self.world = int(os.environ.get("WORLD_SIZE", 1))
        self.local = int(os.environ.get("LOCAL_RANK", 0))
        assert self.world == gpus, f"--gpus {gpus} but WORLD_SIZE={self.world}"
        self.dev = torch.device("cuda", self.local)

    def init(self):
        import torch.distributed as dist
        torch.cuda.set_device(self.local)
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            from datetime import timedelta
            # a short collective timeout: a rank that dies must not leave the others waiting for ten minutes
            dist.init_process_group("nccl", device_id=self.dev, timeout=timedelta(seconds=240))

    def barrier(self):
        torch.cuda.synchronize()
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def rank_max(self, values):
        t = torch.tensor(values, device=self.dev, dtype=torch.float64)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def finish(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()


def timed_blocks(ranks: Ranks, run_block, stream, repeats: int):
    """``repeats`` timed blocks, each bracketed by a barrier + synchronize on both sides; per block the time is the
    maximum over the ranks. Returns the list of block times in ms."""
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(repeats)]
    for e0, e1 in pairs:
        ranks.barrier()
        e0.record(stream)
        run_block()
        e1.record(stream)
        ranks.barrier()
    return ranks.rank_max([e0.elapsed_time(e1) for e0, e1 in pairs])


def summary(ms_blocks):
    return {"min_ms": round(min(ms_blocks), 5), "max_ms": round(max(ms_blocks), 5), "repeats": len(ms_blocks)}


def pick_repeats(block_ms: float, lo: int = 5, hi: int = 60, target_ms: float = 250.0) -> int:
    return int(min(hi, max(lo, math.ceil(target_ms / max(block_ms, 1e-3)))))


# ------------------------------------------------------------------------------------------------ decode
def make_decode_inputs(hv_lo: int, hv_hi: int):
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


class Staging:
    """The step's activations (packed q|k|v rows, then a, then b) in ONE buffer, so that a step is one
    host-to-device copy; ``views`` are the three tensors the op takes."""

    def __init__(self, host: dict, device=None, pinned=False):
        self.shapes = {k_: tuple(v_.shape) for k_, v_ in host.items()}
        self.sizes = {k_: v_.numel() for k_, v_ in host.items()}
        total = sum(self.sizes.values())
        if device is None:
            self.flat = torch.empty(total, dtype=torch.bfloat16)
            if pinned:
                self.flat = self.flat.pin_memory()
            off = 0
            for k_, v_ in host.items():
                self.flat[off:off + self.sizes[k_]].copy_(v_.reshape(-1))
                off += self.sizes[k_]
        else:
            self.flat = torch.empty(total, dtype=torch.bfloat16, device=device)
        self.views = {}
        off = 0
        for k_ in host:
            self.views[k_] = self.flat[off:off + self.sizes[k_]].view(self.shapes[k_])
            off += self.sizes[k_]
        self.bytes = total * 2


def bench_decode(ranks: Ranks, args, state_dtype=torch.float32, with_e2e=True, steps=None):
    from pla_b200.decode import fused_sigmoid_gating_delta_rule_forward_k_last_packed as packed
    world, rank, dev = ranks.world, ranks.rank, ranks.dev
    steps = steps or args.steps
    assert HV % world == 0
    hv_lo, hv_hi = rank * HV // world, (rank + 1) * HV // world
    host, const, slot_sets, hl, hvl = make_decode_inputs(hv_lo, hv_hi)
    pinned = Staging(host, pinned=True)
    resident = Staging(host, device=dev)
    resident.flat.copy_(pinned.flat)
    const = {k_: v_.to(dev) for k_, v_ in const.items()}
    g = torch.Generator(device=dev).manual_seed(SEED + rank)
    pool = torch.empty(SLOTS, hvl, D, D, device=dev)
    pool.normal_(0.0, 0.02, generator=g)
    if state_dtype != torch.float32:
        pool = pool.to(state_dtype)
    slot_sets = [s.to(dev) for s in slot_sets]
    cu = torch.arange(B + 1, dtype=torch.int32, device=dev)
    out = torch.empty(B, 1, hvl, D, dtype=torch.bfloat16, device=dev)
    scale = D ** -0.5
    stream = torch.cuda.current_stream()
    esz = pool.element_size()

    def step(i, inp, dst):
        packed(inp["mixed"], inp["a"], inp["b"], const["A_log"], const["dt_bias"], 1.0, 20.0, scale, pool,
               slot_sets[i % len(slot_sets)], dst, True, cu, False, True, rows_per_cta=args.rows)

    # ---- device-resident timing ----
    # The K steps are replayed from a CUDA graph of G consecutive steps (G divides K, slot sets keep
    # rotating inside the graph), as a serving engine replays its decode step: at 8 GPUs a step is
    # ~25 us of kernel time and per-call host overhead would otherwise be what is measured.
    for i in range(args.warmup):
        step(i, resident.views, out)
    G = max(g_ for g_ in range(1, 41) if steps % g_ == 0)     # 40 steps per graph at the default 2000
    graph = None
    if not args.no_graph:
        side = torch.cuda.Stream()
        side.wait_stream(stream)
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(G):
                    step(i, resident.views, out)
        stream.wait_stream(side)

    def block():
        if graph is not None:
            for _ in range(steps // G):
                graph.replay()
        else:
            for i in range(steps):
                step(i, resident.views, out)

    ranks.barrier()
    t0 = time.perf_counter()
    block()                                                    # one untimed block: sizes the number of repeats
    torch.cuda.synchronize()
    est_ms = ranks.rank_max([(time.perf_counter() - t0) * 1e3])[0]
    repeats = pick_repeats(est_ms)
    blocks = timed_blocks(ranks, block, stream, repeats)
    ms_dev = statistics.median(blocks)

    local_state_bytes = 2 * B * hvl * D * D * esz                # this GPU's launch
    total_state_bytes = local_state_bytes * world                # whole job, per step
    res = {"ms_dev": ms_dev, "blocks": blocks, "G": G, "steps": steps, "hvl": hvl,
           "local_state_bytes": local_state_bytes, "total_state_bytes": total_state_bytes,
           "value": total_state_bytes * steps / (ms_dev * 1e-3) / 1e9,
           "achieved": local_state_bytes * steps / (ms_dev * 1e-3) / 1e9}
    if not with_e2e:
        return res

    # ---- end to end: one pinned staging buffer in, output rows out, every step ----
    # Three streams (H2D, compute, D2H) over double-buffered staging / output buffers, as a serving engine
    # overlaps the copies of neighbouring steps with the kernel. The whole pipeline of G2 steps is captured into
    # one CUDA graph (the copies become memcpy nodes), so the host enqueues one graph launch per G2 steps.
    s_in, s_c, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    stages = [Staging(host, device=dev) for _ in range(2)]
    outs = [torch.empty_like(out) for _ in range(2)]
    out_hosts = [torch.empty(B, 1, hvl, D, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_c = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def pipeline(n_steps, first):
        """Enqueues n_steps pipelined steps; s_c is the stream the caller forks from and joins into."""
        s_in.wait_stream(s_c)
        s_out.wait_stream(s_c)
        for i in range(n_steps):
            b_ = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_c[b_])          # the kernel that read this staging buffer has finished
                stages[b_].flat.copy_(pinned.flat, non_blocking=True)
                ev_in[b_].record(s_in)
            with torch.cuda.stream(s_c):
                s_c.wait_event(ev_in[b_])
                if i >= 2:
                    s_c.wait_event(ev_out[b_])         # this output buffer has been copied out
                step(first + i, stages[b_].views, outs[b_])
                ev_c[b_].record(s_c)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_c[b_])
                out_hosts[b_].copy_(outs[b_], non_blocking=True)
                ev_out[b_].record(s_out)
        s_c.wait_stream(s_in)
        s_c.wait_stream(s_out)

    s_c.wait_stream(stream)
    with torch.cuda.stream(s_c):
        pipeline(max(args.warmup, 4), 0)
    torch.cuda.synchronize()
    G2 = G
    e2e_graph, how = None, "host-enqueued"
    if not args.no_graph:
        try:
            e2e_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(e2e_graph, stream=s_c):
                pipeline(G2, 0)
            how = f"CUDA graph of {G2} pipelined steps"
        except Exception as exc:   # a capture problem must not cost the measurement: fall back to host enqueue
            e2e_graph, how = None, f"host-enqueued (graph capture failed: {type(exc).__name__})"
            torch.cuda.synchronize()

    def e2e_block():
        if e2e_graph is not None:
            for _ in range(steps // G2):
                e2e_graph.replay()
        else:
            pipeline(steps, 0)

    with torch.cuda.stream(s_c):
        ranks.barrier()
        t0 = time.perf_counter()
        e2e_block()
        torch.cuda.synchronize()
        est_ms = ranks.rank_max([(time.perf_counter() - t0) * 1e3])[0]
        e2e_blocks = timed_blocks(ranks, e2e_block, s_c, pick_repeats(est_ms))
    ms_e2e = statistics.median(e2e_blocks)
    stream.wait_stream(s_c)
    check = float(out_hosts[0].float().abs().sum())               # the rows did arrive on the host
    res.update({"ms_e2e": ms_e2e, "e2e_blocks": e2e_blocks, "e2e_how": how, "h2d": pinned.bytes,
                "d2h": out_hosts[0].numel() * 2, "e2e_value": total_state_bytes * steps / (ms_e2e * 1e-3) / 1e9,
                "e2e_rows_nonzero": check > 0.0})
    return res


def cpu_oracle_step(n_req: int, reps: int):
    """Times the CPU oracle on the first ``n_req`` requests of the workload (all 32 value heads)."""
    from oracle import decode as odec
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    host, const, slot_sets, hl, hvl = make_decode_inputs(0, HV)
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
                      f"{sec * 1e3:.1f} ms per sample step; state pre-gathered to the active slots; "
                      "taken before any GPU work"}


# ------------------------------------------------------------------------------------------------ prefill (config 3)
def prefill_lengths():
    g = torch.Generator().manual_seed(20261125 + 3)
    lengths = torch.randint(512, 8193, (8,), generator=g).tolist()
    return lengths, g


def cpu_prefill_sample(tokens: int = 2048):
    """The CPU oracle on the first ``tokens`` tokens of config 3's first sequence, all 16 / 32 heads."""
    from oracle import decode as odec
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(77)
    q = torch.nn.functional.normalize(torch.randn(tokens, HQK, D, generator=g), dim=-1).bfloat16()
    k = torch.nn.functional.normalize(torch.randn(tokens, HQK, D, generator=g), dim=-1).bfloat16()
    v = torch.randn(tokens, HV, D, generator=g).bfloat16()
    a = torch.randn(tokens, HV, generator=g).bfloat16()
    b = torch.randn(tokens, HV, generator=g).bfloat16()
    A_log = torch.rand(HV, generator=g) * math.log(16.0)
    dt_bias = torch.randn(HV, generator=g) * 0.1
    pool = torch.randn(1, HV, D, D, generator=g) * 0.02
    t0 = time.perf_counter()
    odec.klast_forward(q=q, k=k, v=v, a=a, b=b, A_log=A_log, dt_bias=dt_bias, state=pool, slot_indices=[0],
                       lengths=[tokens], scale=D ** -0.5)
    sec = time.perf_counter() - t0
    return {"value": round(tokens / sec / 1e6, 6), "unit": "Mtok/s", "cores": threads, "kind": "port",
            "sample": f"CPU oracle (fp32 torch token recurrence, all {HQK}/{HV} heads) on one sequence of {tokens} tokens, "
                      f"{sec:.2f} s; throughput per token is independent of the batch; taken before any GPU work"}


def bench_prefill(ranks: Ranks, args):
    """Config 3 through gdn_prefill_packed_qkv_fwd: 8 packed sequences with lengths ~U[512, 8192], indexed fp32 pool
    with non-consecutive slots. Heads are sharded over the ranks like decode."""
    from pla_b200.prefill.flashqla import gdn_prefill_packed_qkv_fwd
    world, rank, dev = ranks.world, ranks.rank, ranks.dev
    lengths, g = prefill_lengths()
    T = sum(lengths)
    ratio = HV // HQK
    hvl = HV // world
    hl = max(1, hvl // ratio)
    width = 2 * hl * D + hvl * D
    # packed rows in a wider allocation, starting 34 bytes off 16-byte alignment: the layout a conv output
    # with a padded pitch hands to the op
    storage = torch.empty(T, width + 64, dtype=torch.bfloat16, device=dev)
    packed = storage[:, 17:17 + width]
    gd = torch.Generator(device=dev).manual_seed(5 + rank)
    packed.normal_(0.0, 1.0, generator=gd)
    for lo in (0, hl * D):   # q, k L2-normalised per head, as in config 0
        blk = packed[:, lo:lo + hl * D].float().view(T, hl, D)
        packed[:, lo:lo + hl * D] = torch.nn.functional.normalize(blk, dim=-1).view(T, hl * D).bfloat16()
    gates = torch.randn(T, 2 * hvl, generator=g).bfloat16().to(dev)
    A_log = (torch.rand(HV, generator=g) * math.log(16.0))[rank * hvl:(rank + 1) * hvl].contiguous().to(dev)
    dt_bias = (torch.randn(HV, generator=g) * 0.1)[rank * hvl:(rank + 1) * hvl].contiguous().to(dev)
    pool = (torch.randn(16, hvl, D, D, generator=g) * 0.02).to(dev)
    idx = torch.tensor([1, 3, 5, 7, 9, 11, 13, 15], dtype=torch.int32, device=dev)
    offs = [0]
    for n in lengths:
        offs.append(offs[-1] + n)
    cu = torch.tensor(offs, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream()
    steps = max(1, min(args.steps, 20))

    def run(rows, gate_rows):
        return gdn_prefill_packed_qkv_fwd(rows, gate_rows[:, :hvl], gate_rows[:, hvl:], A_log, dt_bias, cu,
                                          num_qk_heads=hl, num_v_heads=hvl, initial_state=pool,
                                          initial_state_indices=idx, output_final_state=False,
                                          raw_cu_seqlens=tuple(offs))[2]

    for _ in range(max(args.warmup, 3)):
        run(packed, gates)

    def block():
        for _ in range(steps):
            run(packed, gates)

    blocks = timed_blocks(ranks, block, stream, 5)
    ms = statistics.median(blocks) / steps

    # ---- end to end: the packed rows and the gate rows come from pinned host memory every step and the output
    # rows go back; H2D of step i+1, the kernels of step i and D2H of step i-1 overlap (three streams) ----
    host_rows = torch.empty(T, width, dtype=torch.bfloat16).pin_memory()
    host_rows.copy_(packed)
    host_gates = torch.empty(T, 2 * hvl, dtype=torch.bfloat16).pin_memory()
    host_gates.copy_(gates)
    host_out = [torch.empty(T, hvl, D, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    stage_rows = [torch.empty(T, width + 64, dtype=torch.bfloat16, device=dev)[:, 17:17 + width] for _ in range(2)]
    stage_gates = [torch.empty_like(gates) for _ in range(2)]
    s_in, s_c, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_c = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    outs = [None, None]
    e2e_steps = max(2, min(steps, 10))

    def e2e_block():
        s_in.wait_stream(s_c)
        s_out.wait_stream(s_c)
        for i in range(e2e_steps):
            b_ = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_c[b_])
                stage_rows[b_].copy_(host_rows, non_blocking=True)
                stage_gates[b_].copy_(host_gates, non_blocking=True)
                ev_in[b_].record(s_in)
            with torch.cuda.stream(s_c):
                s_c.wait_event(ev_in[b_])
                if i >= 2:
                    s_c.wait_event(ev_out[b_])
                outs[b_] = run(stage_rows[b_], stage_gates[b_])
                ev_c[b_].record(s_c)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_c[b_])
                host_out[b_].copy_(outs[b_].view(T, hvl, D), non_blocking=True)
                ev_out[b_].record(s_out)
        s_c.wait_stream(s_in)
        s_c.wait_stream(s_out)

    s_c.wait_stream(stream)
    with torch.cuda.stream(s_c):
        e2e_block()
        torch.cuda.synchronize()
        e2e_blocks = timed_blocks(ranks, e2e_block, s_c, 3)
    stream.wait_stream(s_c)
    ms_e2e = statistics.median(e2e_blocks) / e2e_steps

    hbm, tflops, src = measured_peaks()
    flops_local = T * (hvl * PREFILL_FLOP_PER_TOKEN_HV + hl * PREFILL_FLOP_PER_TOKEN_HQK)
    alg_bytes = T * ((2 * hl + 2 * hvl) * 256 + 4 * hvl)
    achieved = flops_local / (ms * 1e-3) / 1e12
    h2d = host_rows.numel() * 2 + host_gates.numel() * 2
    d2h = host_out[0].numel() * 2
    return {
        "metric": "gdn_prefill_throughput_32K_varlen", "value": round(T / ms / 1e3, 3), "unit": "Mtok/s",
        "ms_per_step": round(ms, 4), "steps": steps, "spread": summary([b_ / steps for b_ in blocks]),
        "higher_is_better": True, "dtype": "tf32 operands, f32 accumulate", "data": "synthetic",
        "config": {"workload": f"config3: GDN packed varlen prefill, 8 sequences {lengths}, T={T} tokens exactly, Hqk=16 HV=32 "
                               "d=128, chunk 64, indexed fp32 pool with non-consecutive slots, packed q|k|v rows 34 bytes off "
                               "16-byte alignment", "sharding": f"value heads / {world}",
                   "l2": "0.67 GB of activations / n_gpus per step plus the chunk workspace, both larger than L2"},
        "roofline": {"bound": "tensor", "achieved": round(achieved, 2), "peak": tflops, "unit": "TFLOP/s",
                     "frac": round(achieved / tflops, 4), "peak_source": f"of {src} (sustained bf16 GEMM rate)",
                     "flops_per_step": flops_local, "traffic": PREFILL_TRAFFIC_BYTES if world == 1 else None,
                     "algorithmic_bytes": alg_bytes,
                     "algorithmic_GBps": round(alg_bytes / (ms * 1e-3) / 1e9, 1),
                     "frac_of_hbm": round(alg_bytes / (ms * 1e-3) / 1e9 / hbm, 4)},
        "e2e": {"value": round(T / ms_e2e / 1e3, 3), "unit": "Mtok/s", "ms_per_step": round(ms_e2e, 4),
                "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
                "pipeline": "H2D / kernels / D2H on three streams, double-buffered, host-enqueued"},
        "gpu_launches_per_step": 2,
    }


# ------------------------------------------------------------------------------------------------ config 4
def bench_prefill_cp(ranks: Ranks, args, kda: bool):
    """Config 4: one long sequence cut into contiguous token ranges over the ranks (prescan -> one all-gather of
    (offset, transition) pairs -> fold -> segment pass); on one GPU the same scheme over ranges inside the GPU.
    GDN: 64K tokens, Hqk=8, HV=24. KDA: 128K tokens, 32 heads, per-channel softplus gate, A_log ~ U(-4, -2)."""
    from pla_b200._ops import ops
    from pla_b200.prefill.context_parallel import gdn_prefill_context_parallel, kda_prefill_context_parallel
    from pla_b200.prefill.flashqla import ops as fq
    from pla_b200.prefill.flashkdapro import flashkda_fwd
    world, rank, dev = ranks.world, ranks.rank, ranks.dev
    T, Hg, H = (131072, 32, 32) if kda else (65536, 8, 24)
    if args.tokens:
        T = args.tokens          # profiling aid; the workload string then says so
    per = (T // world + 63) // 64 * 64
    lo, hi = min(rank * per, T), min((rank + 1) * per, T)
    steps = max(1, min(args.steps, 10))

    def one_config(weak: bool, timed: bool):
        gd = torch.Generator(device=dev).manual_seed(44 + int(weak))

        def draw(*shape):
            """Every rank draws the whole tensor from the same seed and keeps its token range (rank 0 keeps all
            of it for the single-pass comparison)."""
            full = torch.randn(*shape, generator=gd, device=dev)
            return full if rank == 0 else full[lo:hi].clone()

        q = torch.nn.functional.normalize(draw(T, Hg, D), dim=-1).bfloat16()
        k = torch.nn.functional.normalize(draw(T, Hg, D), dim=-1).bfloat16()
        v = draw(T, H, D).bfloat16()
        gate = (draw(T, H, D) if kda else draw(T, H)).bfloat16()
        beta = draw(T, H)
        if weak:
            beta = beta - 5.0        # small beta keeps the product of (I - beta k k^T) of order one over a range
        beta = beta.bfloat16()
        u = torch.rand(H, generator=gd, device=dev)
        if weak:
            A_log = -10.0 + u        # ~5e-5 nats per token: a range's transition matrix stays of order one
        else:
            A_log = (-4.0 + 2.0 * u) if kda else u * math.log(16.0)
        dt_bias = torch.randn(H, D, generator=gd, device=dev) * 0.1 if kda else torch.randn(H, generator=gd, device=dev) * 0.1
        S0 = torch.randn(H, D, D, generator=gd, device=dev) * 0.02
        sl = slice(lo, hi) if rank == 0 else slice(None)
        mine = [x[sl] for x in (q, k, v, gate, beta)]
        one_gpu = world == 1
        if one_gpu:
            pool1 = S0[None].clone()
            slot0 = torch.zeros(1, dtype=torch.int32, device=dev)
            cu1 = torch.tensor([0, T], dtype=torch.int32, device=dev)
            out1 = torch.empty(T, H, D, dtype=torch.bfloat16, device=dev)
            status1 = torch.zeros(1, dtype=torch.int32, device=dev)

        def step():
            if one_gpu and kda:
                flashkda_fwd(q, k, v, gate, beta, A_log, dt_bias, out1, None, None, state_pool=pool1, state_indices=slot0,
                             raw_cu_seqlens=(0, T), backend="chunked", status=status1)
                return out1, pool1[0]
            if one_gpu:
                res = fq.chunk_gated_delta_rule_fwd(q[None], k[None], v[None], None, None, initial_state=pool1,
                                                    initial_state_indices=slot0, cu_seqlens=cu1, output_final_state=False,
                                                    auto_cp=True, normalize_qk=True, raw_cu_seqlens=(0, T), raw_gate_a=gate,
                                                    raw_beta_b=beta, A_log=A_log, dt_bias=dt_bias)
                return res[2][0], pool1[0]
            if kda:
                return kda_prefill_context_parallel(*mine, A_log, dt_bias, None, initial_state=S0, backend="chunked")
            return gdn_prefill_context_parallel(*mine, A_log, dt_bias, initial_state=S0)

        ms, blocks = None, None
        if timed:
            for _ in range(max(args.warmup, 3)):
                step()

            def block():
                for _ in range(steps):
                    step()

            blocks = timed_blocks(ranks, block, torch.cuda.current_stream(), 3)
            ms = statistics.median(blocks) / steps
        if one_gpu:
            pool1.copy_(S0[None])             # the pool is updated in place: restart from S0 for the comparison
        o, final = step()
        torch.cuda.synchronize()
        rel_o = rel_s = status_code = None
        if rank == 0:
            # the same kernels in a single pass over the whole sequence, for comparison
            one = torch.empty(T, H, D, dtype=torch.bfloat16, device=dev)
            fin = torch.empty(1, H, D, D, dtype=torch.float32, device=dev)
            status = torch.zeros(1, dtype=torch.int32, device=dev)
            cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
            if kda:
                ops.kda_prefill_chunked(q, k, v, gate, beta, A_log, dt_bias, one, cu, S0[None].contiguous(), None, fin, None,
                                        None, False, True, D ** -0.5, None, False, T // 64, 0, False, status)
            else:
                ops.gdn_prefill_chunked(q, k, v, gate, beta, A_log, dt_bias, one, None, cu, S0[None].contiguous(), None, fin,
                                        None, False, True, D ** -0.5, False, False, T // 64, 0, status)
            rel = lambda a_, b_: float((a_.float() - b_.float()).norm() / b_.float().norm())
            rel_o, rel_s, status_code = rel(o, one[lo:hi]), rel(final, fin[0]), int(status.item())
            # how much of the final state comes from the incoming one: rerun the single pass from zero
            fin0 = torch.empty_like(fin)
            if kda:
                ops.kda_prefill_chunked(q, k, v, gate, beta, A_log, dt_bias, one, cu, None, None, fin0, None,
                                        None, False, True, D ** -0.5, None, False, T // 64, 0, False, status)
            else:
                ops.gdn_prefill_chunked(q, k, v, gate, beta, A_log, dt_bias, one, None, cu, None, None, fin0,
                                        None, False, True, D ** -0.5, False, False, T // 64, 0, status)
            carried = rel(fin0[0], fin[0])
            del one, fin, fin0
        else:
            carried = None
        del q, k, v, gate, beta, mine
        torch.cuda.empty_cache()
        return ms, blocks, rel_o, rel_s, status_code, carried

    ms, blocks, rel_o, rel_s, status_code, carried = one_config(False, True)
    _, _, wrel_o, wrel_s, wstatus, wcarried = one_config(True, False)
    if kda:
        what = f"config4 (KDA part): 1 sequence, T={T}, 32 heads, softplus gate, A_log~U(-4,-2), chunk 64 (tf32) tensor-core kernels"
    else:
        what = f"config4 (GDN part): 1 sequence, T={T}, Hqk=8 HV=24, chunk 64 (tf32) tensor-core kernels"
    if args.tokens:
        what = "REDUCED (profiling aid) " + what
    if world == 1:
        plan = fq.plan_token_ranges([0, T], H, torch.cuda.get_device_properties(dev).multi_processor_count)
        how = f"{len(plan[2]) if plan else 1} token ranges inside the GPU (prescan, fold, segment pass)"
    else:
        how = f"{per} tokens per rank, one NCCL all-gather of [{H},2,128,128] fp32 per rank inside the timed region"
    return {"metric": "kda_prefill_context_parallel_128K" if kda else "gdn_prefill_context_parallel_64K",
            "value": round(T / ms / 1e3, 3), "unit": "Mtok/s", "ms_per_step": round(ms, 4), "steps": steps,
            "spread": summary([b_ / steps for b_ in blocks]), "higher_is_better": True, "scaling": "strong",
            "config": {"workload": what, "split": how},
            "vs_single_pass": {"out_rel_l2": rel_o, "state_rel_l2": rel_s, "status": status_code,
                               "state_share_not_from_initial_state": carried},
            "vs_single_pass_weak_decay": {
                "gates": "A_log ~ U(-10,-9), beta logits - 5: transitions of order one over a whole range",
                "out_rel_l2": wrel_o, "state_rel_l2": wrel_s, "status": wstatus,
                "state_share_not_from_initial_state": wcarried}}


# ------------------------------------------------------------------------------------------------ secondary operators
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


def run_vlast(args):
    """Config 1 in the v-last layout ([slots, HV, K, V] pool) through pla_b200.decode.gdn.v_last, one GPU,
    device-resident steps."""
    from pla_b200.decode.gdn.v_last import fused_sigmoid_gating_delta_rule
    dev = torch.device("cuda", torch.cuda.current_device())
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

    steps = min(args.steps, 200)
    ms = _time_steps(step, steps, max(args.warmup, 3))
    gbs = 2 * B * HV * TILE_BYTES / (ms * 1e-3) / 1e9
    hbm, _, src = measured_peaks()
    return {"metric": "gdn_decode_state_bandwidth_B256_vlast", "value": round(gbs, 1), "unit": "GB/s",
            "n_gpus": 1, "steps": steps, "ms_per_step": round(ms, 5), "higher_is_better": True,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "config1 (v-last half): GDN decode B=256 Hqk=16 HV=32 d=128, fp32 v-last pool "
                                   "1024 slots, 4 disjoint slot sets rotated", "launch": "host call per step"},
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": hbm, "unit": "GB/s",
                         "frac": round(gbs / hbm, 4), "peak_source": "of " + src}}


def run_conv(args):
    """The causal conv in front of config 3's prefill (8 sequences, ~32K token rows of the packed q|k|v width
    8192, bf16), history pool of 64 slots; algorithmic bytes = one read and one write of every row."""
    from pla_b200.prefill.causal_conv import causal_conv1d_fn
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator().manual_seed(SEED + 3)
    lengths = torch.randint(512, 8193, (8,), generator=g).tolist()
    T, C = sum(lengths), 8192
    offs = [0]
    for n in lengths:
        offs.append(offs[-1] + n)
    x = torch.randn(T, C, generator=torch.Generator(device=dev).manual_seed(3), device=dev).bfloat16()
    w = (torch.randn(C, 4, generator=g) * 0.2).to(dev)
    state = torch.zeros(64, 3, C, dtype=torch.bfloat16, device=dev).transpose(1, 2)
    idx = torch.randperm(64, generator=g)[:8].to(torch.int32).to(dev)
    cu = torch.tensor(offs, dtype=torch.int32, device=dev)
    y = torch.empty_like(x)

    def step():
        causal_conv1d_fn(x, w, None, state, cu, idx, None, "silu", out=y)

    steps = min(args.steps, 50)
    ms = _time_steps(step, steps, max(args.warmup, 3))
    gbs = 2 * T * C * 2 / (ms * 1e-3) / 1e9
    hbm, _, src = measured_peaks()
    return {"metric": "causal_conv_prefill_bandwidth", "value": round(gbs, 1), "unit": "GB/s", "n_gpus": 1,
            "steps": steps, "ms_per_step": round(ms, 5), "higher_is_better": True, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": f"causal conv (width 4, SiLU) in front of config3: 8 sequences {lengths}, "
                                   f"T={T}, {C} channels bf16, 1.3 GB touched per step (> L2)"},
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": hbm, "unit": "GB/s",
                         "frac": round(gbs / hbm, 4), "peak_source": "of " + src}}


def run_replay(args):
    """Config 2, KDA ReplaySSM verify + commit, 32 heads, 64 rows x 4 tokens, 512 pages, softplus gate."""
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

    steps = min(args.steps, 100)
    ms_v = _time_steps(verify, steps, max(args.warmup, 3))
    ms_c = _time_steps(commit, steps, max(args.warmup, 3))
    state_v, state_c = N * H * TILE_BYTES, 2 * N * H * TILE_BYTES
    hbm, _, src = measured_peaks()
    return {"metric": "kda_replay_verify_commit_state_bandwidth", "unit": "GB/s",
            "value": round((state_v + state_c) / ((ms_v + ms_c) * 1e-3) / 1e9, 1),
            "n_gpus": 1, "steps": steps, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "config2: H=32, 64 rows x 4 tokens, 512 pages, accepted ~U{1..4}",
                       "verify_ms": round(ms_v, 4), "commit_ms": round(ms_c, 4),
                       "verify_GBps": round(state_v / ms_v / 1e6, 1), "commit_GBps": round(state_c / ms_c / 1e6, 1),
                       "verify_frac_of_hbm": round(state_v / ms_v / 1e6 / hbm, 4),
                       "commit_frac_of_hbm": round(state_c / ms_c / 1e6 / hbm, 4), "peak_source": "of " + src}}


def run_mega(args):
    """The fused KDA decode step (conv + SiLU + shift, gate, recurrence, gated RMSNorm) at B=256, 32 heads."""
    from pla_b200.decode.kda import fused_kda_decode_mega_forward
    dev = torch.device("cuda", torch.cuda.current_device())
    H, Bm, slots = 32, 256, 1024
    g = torch.Generator(device=dev).manual_seed(9)
    dim = H * D
    x = torch.randn(Bm, 3 * dim, generator=g, device=dev).bfloat16()
    weight = torch.randn(3, 4, dim, generator=g, device=dev) * 0.3
    conv_state = torch.randn(slots, 3 * dim, 3, generator=g, device=dev).bfloat16()
    raw_g = torch.randn(1, Bm, H, D, generator=g, device=dev).bfloat16()
    raw_beta = torch.randn(1, Bm, H, generator=g, device=dev).bfloat16()
    A_log = torch.rand(H, generator=g, device=dev)
    dt_bias = torch.randn(dim, generator=g, device=dev) * 0.1
    state = torch.randn(slots, H, D, D, generator=g, device=dev) * 0.02
    out_gate = torch.randn(Bm, H, D, generator=g, device=dev).bfloat16()
    norm_w = torch.rand(D, generator=g, device=dev) + 0.5
    perm = torch.randperm(slots, generator=g, device=dev).to(torch.int32)
    sets = [perm[i * Bm:(i + 1) * Bm].contiguous() for i in range(slots // Bm)]
    out = torch.empty(1, Bm, H, D, dtype=torch.bfloat16, device=dev)
    i_ = [0]

    def step():
        fused_kda_decode_mega_forward(x, weight, None, conv_state, raw_g, raw_beta, A_log, dt_bias, sets[i_[0] % len(sets)],
                                      state, out, output_gate=out_gate, norm_weight=norm_w, norm_eps=1e-5, lower_bound=-5.0)
        i_[0] += 1

    steps = min(args.steps, 200)
    ms = _time_steps(step, steps, max(args.warmup, 3))
    gbs = 2 * Bm * H * TILE_BYTES / (ms * 1e-3) / 1e9
    hbm, _, src = measured_peaks()
    return {"metric": "kda_decode_mega_state_bandwidth_B256", "value": round(gbs, 1), "unit": "GB/s", "n_gpus": 1,
            "steps": steps, "ms_per_step": round(ms, 5), "higher_is_better": True, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "fused KDA decode step: B=256, 32 heads, conv width 4 + SiLU, safe gate, gated output "
                                   "RMSNorm, fp32 k-last pool 1024 slots, 4 disjoint slot sets rotated",
                       "launch": "host call per step"},
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": hbm, "unit": "GB/s",
                         "frac": round(gbs / hbm, 4), "peak_source": "of " + src}}


SECONDARY = {"decode_vlast": run_vlast, "replay": run_replay, "conv": run_conv, "mega": run_mega}


def guarded(name, fn, *a):
    """A secondary section must not cost the headline line: its failure is reported in its place."""
    try:
        return fn(*a)
    except Exception as exc:                       # noqa: BLE001
        torch.cuda.synchronize()
        return {"error": f"{name}: {type(exc).__name__}: {str(exc)[:300]}"}


# ------------------------------------------------------------------------------------------------ arms
def run_ours(args):
    ranks = Ranks(args.gpus)
    world, rank = ranks.world, ranks.rank
    sections = set(args.sections.split(",")) if args.sections else {"decode", "prefill", "cp", "secondary"}
    # the CPU samples first, on an otherwise idle host (rank 0 of a one-GPU run only: under torchrun the other
    # ranks would compete for the cores)
    cpu_decode = cpu_prefill = None
    if world == 1 and not args.no_cpu:
        cpu_decode = cpu_baseline_sample()
        if "prefill" in sections:
            cpu_prefill = cpu_prefill_sample()
    sampler = ClockSampler(ranks.local)
    if rank == 0:
        sampler.start()
    ranks.init()
    dev = ranks.dev

    dec = bench_decode(ranks, args)
    line = None
    hbm, _, peak_src = measured_peaks()
    if rank == 0:
        steps, hvl = dec["steps"], dec["hvl"]
        achieved = dec["achieved"]
        line = {
            "metric": METRIC, "value": round(dec["value"], 1), "unit": UNIT, "n_gpus": world, "steps": steps,
            "warmup": args.warmup, "ms_per_step": round(dec["ms_dev"] / steps, 5), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "spread": {**summary([b_ / steps for b_ in dec["blocks"]]), "what": "ms per step of each timed K-step block; value is the median block"},
            "config": {"workload": WORKLOAD, "layout": "k-last packed-QKV op",
                       "launch": ("host call per step" if args.no_graph else f"CUDA graph of {dec['G']} steps"),
                       "sharding": f"value heads / {world}",
                       "l2": "each step touches 1 GiB/n_gpus of state; slot sets rotate over disjoint sets of B slots",
                       "frac_of_nominal_8TBps": round(achieved / 8000.0, 4)},
            "e2e": {"value": round(dec["e2e_value"], 1), "unit": UNIT, "h2d_bytes_per_step": dec["h2d"] * world,
                    "d2h_bytes_per_step": dec["d2h"] * world, "ms_per_step": round(dec["ms_e2e"] / steps, 5),
                    "spread": summary([b_ / steps for b_ in dec["e2e_blocks"]]),
                    "pipeline": "one H2D copy per step from one pinned buffer / kernel / D2H of the output rows on three "
                                "streams, double-buffered; " + dec["e2e_how"],
                    "output_rows_on_host_nonzero": dec["e2e_rows_nonzero"]},
            "gpu_launches": steps,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm, "unit": "GB/s",
                         "frac": round(achieved / hbm, 4), "peak_source": f"of {peak_src}",
                         "traffic": TRAFFIC_BYTES_FULL_LAUNCH if (B == 256 and hvl == HV and world == 1) else None,
                         "algorithmic_bytes_per_launch": dec["local_state_bytes"]},
            "cpu_baseline": cpu_decode if cpu_decode is not None else
            {"value": None, "note": "taken at n_gpus = 1 only: under torchrun the other ranks compete for the host cores"},
        }
    if "prefill" in sections:
        pre = guarded("prefill", bench_prefill, ranks, args)
        if rank == 0:
            if "error" not in pre:
                pre["cpu_baseline"] = cpu_prefill if cpu_prefill is not None else {"value": None, "note": "n_gpus = 1 only"}
            line["prefill"] = pre
    if "cp" in sections:
        for key, kda in (("prefill_cp", False), ("prefill_cp_kda", True)):
            res = guarded(key, bench_prefill_cp, ranks, args, kda)
            if rank == 0:
                line[key] = res
    if "secondary" in sections:
        sec = {}
        d16 = guarded("decode_bf16_pool", bench_decode, ranks, args, torch.bfloat16, False, min(args.steps, 200))
        if rank == 0:
            if "error" in d16:
                sec["decode_bf16_pool"] = d16
            else:
                st = d16["steps"]
                sec["decode_bf16_pool"] = {
                    "metric": "gdn_decode_state_bandwidth_B256_bf16_pool", "value": round(d16["value"], 1), "unit": UNIT,
                    "ms_per_step": round(d16["ms_dev"] / st, 5), "steps": st,
                    "roofline": {"bound": "hbm", "achieved": round(d16["achieved"], 1), "peak": hbm,
                                 "frac": round(d16["achieved"] / hbm, 4), "peak_source": f"of {peak_src}",
                                 "algorithmic_bytes_per_launch": d16["local_state_bytes"]},
                    "config": {"workload": "config1 with a bf16 k-last pool (half the state bytes per step), heads / n_gpus"}}
            for name, fn in SECONDARY.items():          # one GPU each; rank 0 runs them while the others wait
                sec[name] = guarded(name, fn, args)
            line["secondary"] = sec
        ranks.barrier()
    if rank == 0:
        line["clocks"] = sampler.stop()
        print(json.dumps(line), flush=True)
    ranks.finish()
    return line


def run_reference(args):
    """Reference arm: the reference's own CPU implementation of the path -- its fp32 PyTorch
    recurrence, restated in oracle/ because the reference tree is not on the GPU box -- on all
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
    pre = cpu_prefill_sample(1024)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(total / args.steps * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": f"{n_req} of 256 requests per step"},
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{n_req} of the 256 requests per step, all host threads"},
        "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "prefill": {"metric": "gdn_prefill_throughput_32K_varlen", "value": pre["value"], "unit": "Mtok/s",
                    "cpu_baseline": pre, "e2e": {"value": pre["value"], "unit": "Mtok/s", "h2d_bytes_per_step": 0,
                                                 "d2h_bytes_per_step": 0}},
    }
    print(json.dumps(line), flush=True)


def main():
    global B, SLOTS, WORKLOAD
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="all",
                    choices=["all", "decode", "prefill", "prefill_cp", "prefill_cp_kda"] + sorted(SECONDARY),
                    help="all = the full line; decode / prefill / prefill_cp* = that section only; the others print "
                         "one secondary line (1 GPU)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sections", default="", help="comma list out of decode,prefill,cp,secondary (default: all four)")
    ap.add_argument("--tokens", type=int, default=0,
                    help="prefill_cp / prefill_cp_kda: sequence length override (profiling aid, multiple of 64)")
    ap.add_argument("--rows", type=int, default=0, help="k-last decode kernel choice (0 = library default)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline samples (tuning runs)")
    ap.add_argument("--no-graph", action="store_true", help="launch every step from the host instead of a CUDA graph")
    ap.add_argument("--batch", type=int, default=B, help="requests per step (profiling aid; the metric is quoted at 256)")
    ap.add_argument("--slots", type=int, default=SLOTS, help="pool slots (profiling aid; default 1024)")
    args = ap.parse_args()
    if (args.batch, args.slots) != (B, SLOTS):
        B, SLOTS = args.batch, args.slots
        WORKLOAD = f"REDUCED (not the headline): GDN decode B={B} Hqk=16 HV=32 d=128, fp32 k-last pool {SLOTS} slots"
    if args.impl == "reference":
        run_reference(args)
        return
    if args.warmup < 3:
        args.warmup = 3
    if args.workload in SECONDARY:
        if int(os.environ.get("RANK", 0)) == 0:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
            print(json.dumps(SECONDARY[args.workload](args)), flush=True)
        return
    if args.workload in ("prefill", "prefill_cp", "prefill_cp_kda"):
        ranks = Ranks(args.gpus)
        ranks.init()
        res = bench_prefill(ranks, args) if args.workload == "prefill" else \
            bench_prefill_cp(ranks, args, args.workload == "prefill_cp_kda")
        if ranks.rank == 0:
            res["n_gpus"] = ranks.world
            print(json.dumps(res), flush=True)
        ranks.finish()
        return
    if args.workload == "decode" and not args.sections:
        args.sections = "decode"
    run_ours(args)


if __name__ == "__main__":
    main()
