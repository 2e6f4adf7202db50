"""Width-4 causal conv (+ SiLU) over packed varlen rows with a 3-tap history per request: the oracle against
the fixtures made by the reference's conv oracle, the CUDA op against both."""
from pathlib import Path

import numpy as np
import pytest
import torch

import cases
from oracle import conv as oconv

GOLDEN = Path(__file__).resolve().parent / "golden"


def oracle_of(kw, **extra):
    return oconv.causal_conv_prefill(kw["x"], kw["weight"], kw["bias"], kw["conv_state"], kw["offsets"],
                                     kw["state_indices"].tolist(),
                                     None if kw["has_initial_state"] is None else kw["has_initial_state"].tolist(), **extra)


def tol(dtype):
    return dict(rtol=1e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=2e-3, atol=4e-3)


@pytest.mark.parametrize("name", sorted(cases.CONV_CASES))
def test_oracle_matches_reference_fixture(name):
    kw, c = cases.conv_case(name)
    gold = np.load(GOLDEN / f"{name}.npz")
    y, state = oracle_of(kw)
    total = kw["offsets"][-1]
    torch.testing.assert_close(y.float(), torch.from_numpy(gold["y"]), **tol(y.dtype))      # one rounding to 16 bits
    assert torch.count_nonzero(y[total:]) == 0
    assert torch.equal(state.float(), torch.from_numpy(gold["final"]))                      # histories are copies: exact


def test_oracle_sequence_equals_token_by_token():
    """Running a sequence in one call and one token at a time through the kept history give the same rows."""
    kw, _ = cases.conv_case("conv_ds_fp16")
    y_all, st_all = oracle_of(kw)
    state = kw["conv_state"].clone()
    offs = kw["offsets"]
    for s, (beg, end) in enumerate(zip(offs, offs[1:])):
        for t in range(beg, end):
            y1, state = oconv.causal_conv_prefill(kw["x"][t:t + 1], kw["weight"], kw["bias"], state, [0, 1],
                                                  [int(kw["state_indices"][s])])
            assert torch.equal(y1[0], y_all[t])
    assert torch.equal(state, st_all)


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(cases.CONV_CASES))
def test_cuda_conv_matches_oracle_and_fixture(native_built, name):
    from pla_b200._ops import ops
    kw, c = cases.conv_case(name)
    d, _ = cases.conv_case(name, device="cuda")
    exp_y, exp_state = oracle_of(kw)
    cu = torch.tensor(kw["offsets"], dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    pool_before = d["conv_state"].clone()
    y = ops.causal_conv_prefill(d["x"], d["weight"], d["bias"], d["conv_state"], cu, d["state_indices"],
                                d["has_initial_state"], True, False, None, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    torch.testing.assert_close(y.cpu().float(), exp_y.float(), **tol(exp_y.dtype))
    assert torch.count_nonzero(y[kw["offsets"][-1]:]) == 0
    assert torch.equal(d["conv_state"].cpu(), exp_state)                     # histories are copies of inputs: bit-exact
    gold = np.load(GOLDEN / f"{name}.npz")
    torch.testing.assert_close(y.cpu().float(), torch.from_numpy(gold["y"]), **tol(exp_y.dtype))
    assert torch.equal(d["conv_state"].cpu().float(), torch.from_numpy(gold["final"]))
    used = {int(s) for s, n in zip(kw["state_indices"], c["lengths"]) if s >= 0 and n > 0}
    for s in range(c["slots"]):
        if s not in used:
            assert torch.equal(d["conv_state"][s], pool_before[s])


@pytest.mark.gpu
@pytest.mark.parametrize("tokens,channels", [(1500, 1024), (9, 4096), (4200, 264)])
def test_cuda_conv_tiles_and_facade(native_built, tokens, channels):
    """Every tile size the launcher picks, sequences that start one and two rows before a tile edge, the
    channels-first view the serving stacks pass, the vLLM null block, and a call without any history."""
    from pla_b200.prefill.causal_conv import causal_conv1d_fn
    g = torch.Generator().manual_seed(tokens + channels)
    cuts = sorted({0, tokens} | {int(t) for t in torch.randint(0, tokens, (6,), generator=g)} | {t for t in (63, 126, 127) if t < tokens})
    lengths = [b - a for a, b in zip(cuts, cuts[1:])]
    x = torch.randn(tokens + 3, channels, generator=g).bfloat16()
    w = (torch.randn(channels, 4, generator=g) * 0.4).bfloat16()
    bias = (torch.randn(channels, generator=g) * 0.1).bfloat16()
    state = (torch.randn(len(lengths) + 1, 3, channels, generator=g) * 0.5).bfloat16().transpose(1, 2)
    idx = torch.randperm(len(lengths) + 1, generator=g)[:len(lengths)].to(torch.int32)
    has = torch.rand(len(lengths), generator=g) < 0.7
    exp_y, exp_state = oconv.causal_conv_prefill(x, w.float(), bias.float(), state, cuts, idx.tolist(), has.tolist(),
                                                 vllm_pad=True)
    dstate = state.transpose(1, 2).contiguous().cuda().transpose(1, 2)
    dx = x.cuda()
    y = causal_conv1d_fn(dx.t(), w.cuda(), bias.cuda(), dstate, torch.tensor(cuts, dtype=torch.int32, device="cuda"),
                         idx.cuda(), has.cuda(), "silu", pad_slot_id=0)
    torch.cuda.synchronize()
    assert y.shape == (channels, tokens + 3) and y.stride(0) == 1
    torch.testing.assert_close(y.t().cpu().float(), exp_y.float(), **tol(torch.bfloat16))
    assert torch.equal(dstate.cpu(), exp_state)
    # no history at all: every sequence starts from zeros, nothing kept; no activation
    exp_plain, _ = oconv.causal_conv_prefill(x, w.float(), None, None, cuts, silu=False)
    y2 = causal_conv1d_fn(dx, w.cuda(), None, None, torch.tensor(cuts, dtype=torch.int32, device="cuda"), activation=None)
    torch.testing.assert_close(y2.cpu().float(), exp_plain.float(), **tol(torch.bfloat16))


@pytest.mark.gpu
def test_cuda_conv_contract_errors(native_built):
    from pla_b200._ops import ops
    x = torch.zeros(8, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(64, 4, device="cuda")
    cu = torch.tensor([0, 8], dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="in place"):
        ops.causal_conv_prefill(x, w, None, None, cu, None, None, True, False, x, None)
    with pytest.raises(RuntimeError, match="multiple of 8"):
        ops.causal_conv_prefill(x[:, :60], w[:60], None, None, cu, None, None, True, False, None, None)
    with pytest.raises(RuntimeError, match="aligned"):
        ops.causal_conv_prefill(x[:, 4:60], w[:56].contiguous(), None, None, cu, None, None, True, False, None, None)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    state = torch.ones(2, 64, 3, dtype=torch.bfloat16, device="cuda")
    y = ops.causal_conv_prefill(x, w, None, state, cu, torch.tensor([5], dtype=torch.int32, device="cuda"), None, True, False,
                                None, status)
    torch.cuda.synchronize()
    assert status.item() == 8 and torch.count_nonzero(y) == 0 and torch.all(state == 1)   # bad slot: flagged, nothing kept


@pytest.mark.gpu
def test_cuda_conv_empty_inputs(native_built):
    """No rows, no sequences, only empty sequences: nothing faults, rows outside every sequence are zero and the
    histories stay as they were."""
    from pla_b200._ops import ops
    w = torch.ones(64, 4, device="cuda")
    state = torch.full((3, 64, 3), 2.0, dtype=torch.bfloat16, device="cuda")
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    y = ops.causal_conv_prefill(torch.zeros(0, 64, dtype=torch.bfloat16, device="cuda"), w, None, state, i32([0, 0]), i32([1]),
                                None, True, False, None, None)
    assert y.shape == (0, 64)
    x = torch.ones(70, 64, dtype=torch.bfloat16, device="cuda")
    y = ops.causal_conv_prefill(x, w, None, state, i32([0]), i32([]), None, True, False, None, None)
    assert torch.count_nonzero(y) == 0
    y = ops.causal_conv_prefill(x, w, None, state, i32([0, 0, 0]), i32([2, 0]), None, True, False, None, None)
    torch.cuda.synchronize()
    assert torch.count_nonzero(y) == 0 and torch.all(state == 2.0)
    # one row after two empty sequences: history 2,2,2 then the row: 2 + 2 + 2 + 1 = 7, no activation
    y = ops.causal_conv_prefill(x[:1], w, None, state, i32([0, 0, 0, 1]), i32([2, 0, 1]), None, False, False, None, None)
    torch.cuda.synchronize()
    assert torch.all(y == 7.0) and torch.all(state[1, :, 2] == 1.0) and torch.all(state[1, :, :2] == 2.0)
    assert torch.all(state[0] == 2.0) and torch.all(state[2] == 2.0)
