"""k-last decode / verify on the GPU against the CPU oracle and the reference fixtures.

Mirrors the reference's tests/test_k_last_state_dtype.py: page-strided pool with a
256-element gap per slot, slots [3, 0, -1], poisoned snapshot cache, bit-exact
untouched regions.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

import cases
from helpers import assert_out_close, assert_state_close
from oracle import decode as odec

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def to_cuda(args, backing):
    dev = "cuda"
    backing_d = backing.to(dev)
    out = {}
    for key, val in args.items():
        out[key] = val.to(dev) if isinstance(val, torch.Tensor) else val
    HV = args["v"].shape[2]
    out["initial_state_source"] = backing_d[:, : HV * 128 * 128].view(backing.shape[0], HV, 128, 128)
    return out, backing_d


@pytest.mark.parametrize("rows", [0, 1, 16, 17, 32, 64, 128])
@pytest.mark.parametrize("name", sorted(cases.KLAST_CASES))
def test_klast_matches_oracle_and_fixture(native_built, name, rows):
    """Every kernel choice (0 = the library's pick, 1 = row-per-thread, 16 / 17 = streaming with sixteen / twelve
    warps, 32 / 64 / 128 = one block per CTA) on fp32 and bf16 pools (tests/test_k_last_state_dtype.py:159-220)."""
    from pla_b200.decode import fused_sigmoid_gating_delta_rule_forward_k_last as forward
    args, backing, lengths, state_ids, cache_ids = cases.klast_case(name)
    if rows in (1, 16, 17) and cases.KLAST_CASES[name]["mode"] != "decode":
        dargs, _ = to_cuda(args, backing)
        with pytest.raises(RuntimeError, match="single-token decode kernels"):
            forward(**dargs, rows_per_cta=rows)   # these kernels only take plain single-token calls
        return
    if rows == 1 and backing.dtype != torch.float32:
        dargs, _ = to_cuda(args, backing)
        with pytest.raises(RuntimeError, match="fp32 pool"):
            forward(**dargs, rows_per_cta=rows)
        return
    exp_out, exp_state, exp_cache = odec.klast_forward(**cases.oracle_kwargs(args, lengths, state_ids, cache_ids))
    dargs, dbacking = to_cuda(args, backing)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    state_ptr = dargs["initial_state_source"].data_ptr()
    out = forward(**dargs, status=status, rows_per_cta=rows)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert out.shape == args["v"].shape and out.dtype == args["v"].dtype
    assert dargs["initial_state_source"].data_ptr() == state_ptr
    assert dargs["initial_state_source"].dtype == backing.dtype
    assert_out_close(out[0], exp_out, "out vs oracle")
    state = dargs["initial_state_source"].cpu()
    assert_state_close(state, exp_state, "state vs oracle")
    gold = np.load(GOLDEN / f"klast_{name}.npz")
    assert_out_close(out[0], torch.from_numpy(gold["out"][0]), "out vs reference fixture")
    assert_state_close(torch.from_numpy(cases.subsample(state)), torch.from_numpy(gold["state"]), "state vs fixture")
    # bit-exact: slot padding, and every slot no active request owns
    hb = dbacking.cpu()
    assert torch.equal(hb[:, -256:], backing[:, -256:])
    touched = {s for s, n in zip(state_ids, lengths) if n > 0 and (s >= 0 if args.get("is_sglang", True) else s > 0)}
    if args["disable_state_update"]:
        assert torch.equal(hb, backing)
    else:
        for s in range(hb.shape[0]):
            if s not in touched:
                assert torch.equal(hb[s], backing[s]), f"slot {s} must be untouched"
    if exp_cache is not None:
        cache = dargs["intermediate_states_buffer"].cpu()
        untouched = exp_cache == -7.0
        assert torch.equal(cache[untouched], exp_cache[untouched])
        assert_state_close(cache[~untouched], exp_cache[~untouched], "snapshot cache vs oracle")
        assert_state_close(torch.from_numpy(cases.subsample(cache)), torch.from_numpy(gold["cache"]), "cache vs fixture",
                           tol=1e-3)


def _config0(B=8, H=16, HV=32, slots=64, seed=20261125, pad_one=False):
    """BASELINE config 0: q,k,v ~N(0,1) with q,k L2-normalised, a,b ~N(0,1), A_log ~U(0,log16),
    dt_bias ~N(0,0.1), pool ~N(0,0.02), seeded slot permutation."""
    g = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(B, H, 128, generator=g), dim=-1).bfloat16()
    k = torch.nn.functional.normalize(torch.randn(B, H, 128, generator=g), dim=-1).bfloat16()
    v = torch.randn(B, HV, 128, generator=g).bfloat16()
    a = torch.randn(B, HV, generator=g).bfloat16()
    b = torch.randn(B, HV, generator=g).bfloat16()
    A_log = torch.rand(HV, generator=g) * float(np.log(16.0))
    dt_bias = (torch.randn(HV, generator=g) * 0.1).bfloat16()
    pool = torch.randn(slots, HV, 128, 128, generator=g) * 0.02
    idx = torch.randperm(slots, generator=g)[:B].to(torch.int32)
    if pad_one:
        idx[B // 2] = -1
    return dict(q=q, k=k, v=v, a=a, b=b, A_log=A_log, dt_bias=dt_bias, pool=pool, idx=idx)


@pytest.mark.parametrize("pad_one", [False, True])
def test_config0_gdn_decode(native_built, pad_one):
    from pla_b200.decode import fused_sigmoid_gating_delta_rule_forward_k_last as forward
    c = _config0(pad_one=pad_one)
    B = c["q"].shape[0]
    exp_out, exp_state, _ = odec.klast_forward(
        q=c["q"], k=c["k"], v=c["v"], a=c["a"], b=c["b"], A_log=c["A_log"], dt_bias=c["dt_bias"],
        state=c["pool"], slot_indices=c["idx"].tolist(), lengths=[1] * B, scale=128 ** -0.5)
    d = {k_: v_.cuda() for k_, v_ in c.items()}
    cu = torch.arange(B + 1, dtype=torch.int32, device="cuda")
    out = forward(d["A_log"], d["a"][None], d["dt_bias"], 1.0, 20.0, d["q"][None], d["k"][None], d["v"][None],
                  d["b"][None], d["pool"], d["idx"], 128 ** -0.5, True, cu, False, False, None, None, None, None)
    torch.cuda.synchronize()
    assert_out_close(out[0], exp_out)
    pool = d["pool"].cpu()
    assert_state_close(pool, exp_state)
    used = set(i for i in c["idx"].tolist() if i >= 0)
    for s in range(pool.shape[0]):
        if s not in used:
            assert torch.equal(pool[s], c["pool"][s])
    if pad_one:
        assert torch.count_nonzero(out[0, B // 2]) == 0


@pytest.mark.parametrize("state_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("is_kda", [False, True])
def test_stream_unit_ranges_cut_tiles_anywhere(native_built, is_kda, state_dtype):
    """150 requests x 6 heads = 14,400 units of 8 rows over 148 x 16 warps: every warp's range (6 or 7 units) starts
    and ends in the middle of a tile; padded requests and an out-of-pool slot sit inside the ranges."""
    from pla_b200.decode import fused_sigmoid_gating_delta_rule_forward_k_last as forward
    B, H, HV, slots = 150, 2, 6, 160
    g = torch.Generator().manual_seed(31)
    q = torch.randn(B, H, 128, generator=g).bfloat16()
    k = torch.randn(B, H, 128, generator=g).bfloat16()
    v = torch.randn(B, HV, 128, generator=g).bfloat16()
    a = torch.randn(B, HV * 128 if is_kda else HV, generator=g).bfloat16().view(B, HV, -1).squeeze(-1)
    b = torch.randn(B, HV, generator=g).bfloat16()
    A_log = torch.rand(HV, generator=g) * 2.0
    dt_bias = (torch.randn(HV * 128 if is_kda else HV, generator=g) * 0.1).bfloat16()
    pool = (torch.randn(slots, HV, 128, 128, generator=g) * 0.05).to(state_dtype)
    idx = torch.randperm(slots, generator=g)[:B].to(torch.int32)
    idx[7] = -1
    idx[8] = -1
    idx[93] = -1
    exp_out, exp_state, _ = odec.klast_forward(
        q=q, k=k, v=v, a=a, b=b, A_log=A_log, dt_bias=dt_bias.view(HV, -1).squeeze(-1), state=pool,
        slot_indices=idx.tolist(), lengths=[1] * B, scale=128 ** -0.5, is_kda=is_kda)
    dpool = pool.cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cu = torch.arange(B + 1, dtype=torch.int32, device="cuda")
    for rows in (16, 17) if state_dtype == torch.float32 else (16,):
        dpool.copy_(pool)
        out = forward(A_log.cuda(), a.cuda()[None], dt_bias.cuda(), 1.0, 20.0, q.cuda()[None], k.cuda()[None],
                      v.cuda()[None], b.cuda()[None], dpool, idx.cuda(), 128 ** -0.5, True, cu, is_kda, False, None, None,
                      None, None, status=status, rows_per_cta=rows)
        torch.cuda.synchronize()
        assert status.item() == 0
        assert_out_close(out[0], exp_out)
        assert_state_close(dpool.cpu(), exp_state)
        assert torch.count_nonzero(out[0, [7, 8, 93]]) == 0
        used = set(i for i in idx.tolist() if i >= 0)
        host = dpool.cpu()
        for s_ in range(slots):
            if s_ not in used:
                assert torch.equal(host[s_], pool[s_])


@pytest.mark.parametrize("is_kda", [False, True])
def test_packed_matches_unpacked(native_built, is_kda):
    from pla_b200.decode import (fused_sigmoid_gating_delta_rule_forward_k_last as forward,
                                 fused_sigmoid_gating_delta_rule_forward_k_last_packed as packed)
    B, H, HV = 5, 2, 4
    g = torch.Generator().manual_seed(7)
    width = 2 * H * 128 + HV * 128
    buf = torch.randn(B, width + 64, generator=g).bfloat16().cuda()
    mixed = buf[:, :width]                          # padded token stride
    a = (torch.randn(B, HV * 128 if is_kda else HV, generator=g)).bfloat16().cuda()
    b = torch.randn(B, HV, generator=g).bfloat16().cuda()
    A_log = torch.randn(HV, generator=g).cuda()
    dt_bias = torch.randn(HV * 128 if is_kda else HV, generator=g).bfloat16().cuda()
    pool = (torch.randn(9, HV, 128, 128, generator=g) * 0.1).cuda()
    idx = torch.tensor([4, 0, -1, 7, 2], dtype=torch.int32).cuda()
    cu = torch.arange(B + 1, dtype=torch.int32).cuda()
    pool2 = pool.clone()
    pool0 = pool.cpu().clone()
    out = torch.full((B, 1, HV, 128), 5.0, dtype=torch.bfloat16, device="cuda")
    ret = packed(mixed, a, b, A_log, dt_bias, 1.0, 20.0, 128 ** -0.5, pool, idx, out, True, cu, is_kda)
    assert ret.data_ptr() == out.data_ptr()
    q = mixed[:, : H * 128].reshape(B, H, 128).contiguous()
    k = mixed[:, H * 128: 2 * H * 128].reshape(B, H, 128).contiguous()
    v = mixed[:, 2 * H * 128:].reshape(B, HV, 128).contiguous()
    out2 = forward(A_log, a[None], dt_bias, 1.0, 20.0, q[None], k[None], v[None], b[None], pool2, idx,
                   128 ** -0.5, True, cu, is_kda, False, None, None, None, None)
    torch.cuda.synchronize()
    assert torch.equal(out[:, 0], out2[0])
    assert torch.equal(pool, pool2)
    exp_out, exp_state, _ = odec.klast_forward(
        q=q.cpu(), k=k.cpu(), v=v.cpu(), a=a.cpu(), b=b.cpu(), A_log=A_log.cpu(), dt_bias=dt_bias.cpu(),
        state=pool0, slot_indices=idx.tolist(), lengths=[1] * B, scale=128 ** -0.5, is_kda=is_kda)
    assert_out_close(out[:, 0], exp_out)
    assert_state_close(pool.cpu(), exp_state)
    assert torch.equal(out[2, 0].cpu(), torch.zeros(HV, 128, dtype=torch.bfloat16))  # slot -1 -> zeros


def test_vllm_slot_table_writes_each_draft_token_slot(native_built):
    """2-D slot table: start from column num_accepted-1, snapshot step t into column t's slot
    (src/decode/k-last/fused_sigmoid_gating_k_last_kernel.cuh:218-225, :856-863)."""
    from pla_b200.decode import fused_sigmoid_gating_delta_rule_forward_k_last as forward
    B, T, H, HV = 3, 3, 1, 2
    g = torch.Generator().manual_seed(11)
    q = torch.randn(1, B * T, H, 128, generator=g).bfloat16()
    k = torch.randn(1, B * T, H, 128, generator=g).bfloat16()
    v = torch.randn(1, B * T, HV, 128, generator=g).bfloat16()
    a = torch.randn(1, B * T, HV, generator=g).bfloat16()
    b = torch.randn(1, B * T, HV, generator=g).bfloat16()
    A_log = torch.randn(HV, generator=g)
    dt_bias = torch.randn(HV, generator=g).bfloat16()
    pool = torch.randn(12, HV, 128, 128, generator=g) * 0.1
    table = torch.tensor([[1, 2, 3], [4, 0, 5], [0, 6, 7]], dtype=torch.int32)
    accepted = torch.tensor([2, 1, 1], dtype=torch.int32)
    cu = torch.arange(0, B * T + 1, T, dtype=torch.int32)
    exp_out, exp_state, _ = odec.klast_forward(
        q=q[0], k=k[0], v=v[0], a=a[0], b=b[0], A_log=A_log, dt_bias=dt_bias, state=pool, slot_indices=table,
        lengths=[T] * B, scale=128 ** -0.5, is_sglang=False, disable_state_update=True, num_accepted=accepted.tolist())
    dpool = pool.cuda()
    out = forward(A_log.cuda(), a.cuda(), dt_bias.cuda(), 1.0, 20.0, q.cuda(), k.cuda(), v.cuda(), b.cuda(), dpool,
                  table.cuda(), 128 ** -0.5, True, cu.cuda(), False, True, None, None, accepted.cuda(), None,
                  is_sglang=False)
    torch.cuda.synchronize()
    assert_out_close(out[0], exp_out)
    assert_state_close(dpool.cpu(), exp_state)
    for s in (0, 8, 9, 10, 11):
        assert torch.equal(dpool[s].cpu(), pool[s])
    assert torch.count_nonzero(out[0, 2 * T:]) == 0  # request 2 starts from slot 0 = vLLM padding


def test_bad_interval_sets_status_instead_of_trapping(native_built):
    from pla_b200.decode import fused_sigmoid_gating_delta_rule_forward_k_last as forward
    c = _config0(B=2, H=1, HV=2, slots=4)
    d = {k_: v_.cuda() for k_, v_ in c.items()}
    cu = torch.tensor([0, 2, 2], dtype=torch.int32, device="cuda")   # first interval longer than t_max = 1
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    before = d["pool"].clone()
    forward(d["A_log"], d["a"][None], d["dt_bias"], 1.0, 20.0, d["q"][None], d["k"][None], d["v"][None],
            d["b"][None], d["pool"], d["idx"], 1.0, True, cu, False, False, None, None, None, None, status=status)
    torch.cuda.synchronize()
    assert status.item() & 1
    assert torch.equal(d["pool"], before)
