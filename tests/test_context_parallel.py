"""Host side of the context-parallel prefill on CPU: gloo ranks exchange (offset, transition) pairs
computed by the oracle recurrence and must reproduce the serial recurrence."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import OracleSegmentKernels
from oracle import decode as odec
from pla_b200.prefill import context_parallel as cp

D = 128


def make_inputs(T, Hg, H, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, Hg, D, generator=g).bfloat16()
    k = torch.randn(T, Hg, D, generator=g).bfloat16()
    v = torch.randn(T, H, D, generator=g).bfloat16()
    gate = torch.randn(T, H, generator=g).bfloat16()
    beta = torch.randn(T, H, generator=g).bfloat16()
    A_log = torch.rand(H, generator=g) * 2.0
    dt_bias = torch.randn(H, generator=g) * 0.1
    S0 = torch.randn(H, D, D, generator=g) * 0.05
    return q, k, v, gate, beta, A_log, dt_bias, S0


def _worker(rank, world, port, splits, with_state, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        T = sum(splits)
        q, k, v, gate, beta, A_log, dt_bias, S0 = make_inputs(T, 1, 2, 5)
        lo = sum(splits[:rank])
        hi = lo + splits[rank]
        sl = slice(lo, hi)
        kern = OracleSegmentKernels(q[sl], k[sl], v[sl], gate[sl], beta[sl], A_log, dt_bias, D ** -0.5)
        o, final = cp.gdn_prefill_context_parallel(q[sl], k[sl], v[sl], gate[sl], beta[sl], A_log, dt_bias,
                                                   initial_state=S0 if with_state else None, segment_kernels=kern)
        torch.save({"o": o, "final": final}, os.path.join(result_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("splits,with_state", [((37, 43), True), ((30, 0, 25), False)])
def test_gloo_ranks_reproduce_the_serial_recurrence(tmp_path, splits, with_state):
    world = len(splits)
    mp.spawn(_worker, args=(world, _free_port(), splits, with_state, str(tmp_path)), nprocs=world, join=True)
    T = sum(splits)
    q, k, v, gate, beta, A_log, dt_bias, S0 = make_inputs(T, 1, 2, 5)
    state = S0 if with_state else torch.zeros_like(S0)
    exp_out, exp_state, _ = odec.klast_forward(q=q, k=k, v=v, a=gate, b=beta, A_log=A_log, dt_bias=dt_bias,
                                               state=state[None], slot_indices=[0], lengths=[T], scale=D ** -0.5)
    outs = []
    for r in range(world):
        res = torch.load(os.path.join(tmp_path, f"rank{r}.pt"))
        assert res["o"].shape[0] == splits[r]
        outs.append(res["o"].float())
        torch.testing.assert_close(res["final"], exp_state[0], rtol=1e-4, atol=1e-5)   # same on every rank
    torch.testing.assert_close(torch.cat(outs), exp_out.float(), rtol=2e-2, atol=2e-2)


def test_fold_is_the_composition_of_affine_maps():
    g = torch.Generator().manual_seed(0)
    H, W = 3, 4
    gathered = torch.randn(W, H, 2, D, D, generator=g) * 0.1
    S0 = torch.randn(H, D, D, generator=g)
    s = S0.clone()
    for r in range(W):
        torch.testing.assert_close(cp.fold_transfers(S0, gathered, r), s)
        s = s @ gathered[r, :, 1] + gathered[r, :, 0]
    ident = cp.identity_transfer(H, "cpu")
    torch.testing.assert_close(cp.fold_transfers(S0, ident[None], 1), S0)
    assert torch.equal(cp.fold_transfers(None, gathered, 0), torch.zeros(H, D, D))


def _decode_shard_worker(rank, world, port, result_dir):
    """Rank r of the decode bench: value heads [r*HV/world, (r+1)*HV/world) of every request, its pool shard, no
    data-path collective; the oracle stands in for the kernel."""
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import bench
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        bench.B, bench.SLOTS = 6, 12
        hv_lo, hv_hi = rank * bench.HV // world, (rank + 1) * bench.HV // world
        host, const, slot_sets, hl, hvl = bench.make_decode_inputs(hv_lo, hv_hi)
        g = torch.Generator().manual_seed(99)
        pool = (torch.randn(bench.SLOTS, bench.HV, D, D, generator=g) * 0.02)[:, hv_lo:hv_hi].contiguous()
        mixed = host["mixed"]
        q = mixed[:, :hl * D].view(bench.B, hl, D)
        k = mixed[:, hl * D:2 * hl * D].view(bench.B, hl, D)
        v = mixed[:, 2 * hl * D:].view(bench.B, hvl, D)
        out, state, _ = odec.klast_forward(q=q, k=k, v=v, a=host["a"], b=host["b"], A_log=const["A_log"],
                                           dt_bias=const["dt_bias"], state=pool, slot_indices=slot_sets[0].tolist(),
                                           lengths=[1] * bench.B, scale=D ** -0.5)
        dist.barrier()                      # the only collective of the sharded decode: the timing barrier
        torch.save({"out": out, "state": state, "slots": slot_sets[0]}, os.path.join(result_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_decode_head_shards_reassemble_to_the_unsharded_step(tmp_path):
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import bench
    world = 2
    mp.spawn(_decode_shard_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    saved = (bench.B, bench.SLOTS)
    try:
        bench.B, bench.SLOTS = 6, 12
        host, const, slot_sets, hl, hvl = bench.make_decode_inputs(0, bench.HV)
        g = torch.Generator().manual_seed(99)
        pool = torch.randn(bench.SLOTS, bench.HV, D, D, generator=g) * 0.02
        mixed = host["mixed"]
        q = mixed[:, :hl * D].view(bench.B, hl, D)
        k = mixed[:, hl * D:2 * hl * D].view(bench.B, hl, D)
        v = mixed[:, 2 * hl * D:].view(bench.B, hvl, D)
        out, state, _ = odec.klast_forward(q=q, k=k, v=v, a=host["a"], b=host["b"], A_log=const["A_log"],
                                           dt_bias=const["dt_bias"], state=pool, slot_indices=slot_sets[0].tolist(),
                                           lengths=[1] * bench.B, scale=D ** -0.5)
    finally:
        bench.B, bench.SLOTS = saved
    parts = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(world)]
    assert all(torch.equal(p["slots"], parts[0]["slots"]) for p in parts)      # every rank draws the same slot map
    torch.testing.assert_close(torch.cat([p["out"] for p in parts], dim=1).float(), out.float(), rtol=0, atol=0)
    torch.testing.assert_close(torch.cat([p["state"] for p in parts], dim=1), state, rtol=0, atol=0)


def test_token_range_plan_properties():
    """The host planner: ranges tile every sequence in order, cut on 64-token chunk boundaries counted from the
    sequence start, at least 16 chunks long, never more chains than SMs, nothing split when SMs are busy."""
    import importlib
    fq = importlib.import_module("pla_b200.prefill.flashqla.ops")
    assert fq.plan_token_ranges([0, 4000, 8000], 32, 148) is None           # 64 chains: two ranges each would not pay
    offs = [0, 65536]
    ranges, seg_first, last, seq_of = fq.plan_token_ranges(offs, 24, 148)   # 24 chains: four ranges halve the time
    assert seg_first == [0, 4] and last == [False] * 3 + [True] and ranges[0] == 0 and ranges[-1] == 65536
    assert all((b - a) % 64 == 0 and b - a >= 16 * 64 for a, b in zip(ranges, ranges[1:]))
    offs = [0, 3000, 3000, 9001, 9100]
    ranges, seg_first, last, seq_of = fq.plan_token_ranges(offs, 4, 148)
    assert len(seg_first) == len(offs) and seg_first[-1] == len(last) == len(seq_of)
    for s in range(len(offs) - 1):
        mine = ranges[seg_first[s]:seg_first[s + 1] + 1]
        assert mine[0] == offs[s] and mine[-1] == offs[s + 1] and mine == sorted(mine)
        assert all((x - offs[s]) % 64 == 0 for x in mine[1:-1])
        assert last[seg_first[s]:seg_first[s + 1]] == [False] * (seg_first[s + 1] - seg_first[s] - 1) + [True]
    assert len(last) * 4 <= 2 * 148


def test_rank_range_plan_properties():
    """Ranges inside a rank: chunk-aligned cuts that tile the rank's tokens, at least 16 chunks each, none when the
    rank is short or already has enough chains."""
    from pla_b200.prefill.context_parallel import plan_rank_ranges
    assert plan_rank_ranges(1000, 4, 148) is None                 # 16 chunks: nothing to cut
    assert plan_rank_ranges(65536, 296, 148) is None              # two full waves of chains already
    for tokens, chains in [(65536, 24), (8192, 24), (131072, 32), (2240, 2), (40001, 8)]:
        offs = plan_rank_ranges(tokens, chains, 148)
        assert offs is not None and offs[0] == 0 and offs[-1] == tokens
        assert all(b > a for a, b in zip(offs, offs[1:])) and all(x % 64 == 0 for x in offs[:-1])
        assert all(b - a >= 16 * 64 or b == tokens for a, b in zip(offs, offs[1:]))
    assert len(plan_rank_ranges(65536, 24, 148)) - 1 == 6         # 24 chains: six ranges, a quarter of the chain steps
