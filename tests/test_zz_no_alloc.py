"""The allocation-free commit-plan entry point, called straight through the C ABI.

Some runners cannot hand the planner a scratch buffer: they create their commit state only after
every free byte of the GPU has gone to their cache pools, or from code that is not allowed to call
the allocator. ``pla_b200_kda_replay_plan_static`` keeps its candidate buffer inside the library
instead. The plan it writes must be identical to the one the ordinary entry point writes with a
caller-provided buffer -- checked here on two different batches in a row, because the built-in
buffer is shared between calls and still holds the previous call's candidates.
"""
import ctypes

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu


def _args(sc, plan, candidate, keep):
    from pla_b200 import capi
    dev = "cuda"

    def vec(values):
        t = torch.tensor(values, dtype=torch.int64, device=dev)
        keep.append(t)
        return t

    a = capi.KdaCommitArgs()
    a.candidate = candidate.data_ptr() if candidate is not None else None
    a.plan = plan.data_ptr()
    a.sampled = capi.index_of(vec(sc["counts"]))
    a.source = capi.index_of(vec(sc["sources"]))
    a.cu = capi.index_of(vec(sc["offsets"]))
    a.mapping = capi.index_of(None)
    batch = len(sc["sources"])
    if sc["table"] is not None:
        table = torch.tensor(sc["table"], dtype=torch.int64, device=dev)
        keep.append(table)
        a.blocks = capi.Index(table.data_ptr(), 1, 1)
        a.block_row_stride, a.block_col_stride = table.stride(0), table.stride(1)
        a.block_rows, a.block_cols = table.shape
        a.computed = capi.index_of(vec(sc["positions"]))
        a.block_size = sc["block_size"]
    else:
        a.blocks = capi.index_of(None)
        a.computed = capi.index_of(None)
    a.N, a.capacity, a.sampler_rows = batch, sc["capacity"], batch
    a.H, a.slots, a.Q, a.null_block_id = 1, sc["slots"], sc["q"], 0
    a.token_capacity = sc["token_capacity"]
    return a


def test_static_plan_equals_plan_with_caller_buffer_twice_in_a_row(native_built):
    from pla_b200 import capi
    lib = capi.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    scenarios = {s["name"]: s for s in cases.plan_scenarios()}
    # two different batches back to back: a large aligned one with a conflict, then a small plain one
    for name in ("boundary_source_b40_align", "disjoint_b5_plain", "duplicate_final_b40_align"):
        sc = scenarios[name]
        keep = []
        cap = sc["capacity"]
        want = torch.full((4, cap), -3, dtype=torch.int32, device="cuda")
        got = torch.full((4, cap), -5, dtype=torch.int32, device="cuda")
        candidate = torch.empty((4, cap), dtype=torch.int32, device="cuda")
        rc = lib.pla_b200_kda_replay_plan(ctypes.byref(_args(sc, want, candidate, keep)), stream)
        assert rc == 0, lib.pla_b200_last_error()
        rc = lib.pla_b200_kda_replay_plan_static(ctypes.byref(_args(sc, got, None, keep)), stream)
        assert rc == 0, lib.pla_b200_last_error()
        torch.cuda.synchronize()
        assert torch.equal(got, want), name
        assert got[0].sum().item() >= 0 and (got != -5).all()


def test_static_plan_rejects_more_rows_than_its_buffer_holds(native_built):
    from pla_b200 import capi
    lib = capi.load()
    sc = dict(next(s for s in cases.plan_scenarios() if s["name"] == "disjoint_b5_plain"))
    sc["capacity"] = 4097
    plan = torch.zeros((4, 4097), dtype=torch.int32, device="cuda")
    rc = lib.pla_b200_kda_replay_plan_static(ctypes.byref(_args(sc, plan, None, [])), None)
    assert rc == -5
    assert b"4096" in lib.pla_b200_last_error()
