"""Prefill: CPU oracle against reference fixtures (not gpu), and the GPU ops against both (gpu)."""
from pathlib import Path

import numpy as np
import pytest
import torch

import cases
from helpers import assert_out_close, assert_state_close
from oracle import decode as odec

GOLDEN = Path(__file__).resolve().parent / "golden"
D = 128


def kda_oracle(c):
    return odec.klast_forward(
        q=c["q"], k=c["k"], v=c["v"], a=c["g"], b=c["beta"], A_log=c["A_log"], dt_bias=c["dt_bias"], state=c["init"],
        slot_indices=list(range(len(c["lengths"]))), lengths=c["lengths"], scale=D ** -0.5, use_qk_l2norm=True,
        is_kda=True, lower_bound=c["lower_bound"])


@pytest.mark.parametrize("name", sorted(cases.PREFILL_CASES))
def test_gdn_token_recurrence_matches_chunked_reference(name):
    c = cases.gdn_prefill_case(name)
    out, state, _ = odec.klast_forward(**cases.gdn_prefill_oracle_kwargs(c))
    gold = np.load(GOLDEN / f"prefill_{name}.npz")
    n_real = c["cu"][-1]
    np.testing.assert_allclose(out[:n_real].float().numpy(), gold["out"], rtol=2e-2, atol=2e-3)
    assert torch.count_nonzero(out[n_real:]) == 0
    np.testing.assert_allclose(cases.subsample(state[c["slots"]]), gold["final"], rtol=1e-3, atol=1e-5)


@pytest.mark.parametrize("softplus", [False, True])
@pytest.mark.parametrize("name", sorted(cases.KDA_PREFILL_CASES))
def test_kda_token_recurrence_matches_reference(name, softplus):
    c = cases.kda_prefill_case(name, softplus=softplus)
    out, state, _ = kda_oracle(c)
    gold = np.load(GOLDEN / f"prefill_{name}_{'softplus' if softplus else 'safe'}.npz")
    n_real = c["cu"][-1]
    np.testing.assert_allclose(out[:n_real].float().numpy(), gold["out"], rtol=2e-2, atol=2e-3)
    np.testing.assert_allclose(cases.subsample(state), gold["final"], rtol=1e-3, atol=1e-5)


# ------------------------------------------------------------------------------------------ GPU
@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(cases.PREFILL_CASES))
def test_gdn_packed_prefill_indexed_pool(native_built, name):
    from pla_b200.prefill.flashqla import gdn_prefill_packed_qkv_fwd
    c = cases.gdn_prefill_case(name, device="cuda")
    cpu = cases.gdn_prefill_case(name)
    exp_out, exp_state, _ = odec.klast_forward(**cases.gdn_prefill_oracle_kwargs(cpu))
    assert c["packed"].data_ptr() % 4 != 0          # rows are only 2-byte aligned
    idx = torch.tensor(c["slots"], dtype=torch.int32, device="cuda")
    cu = torch.tensor(c["cu"], dtype=torch.int32, device="cuda")
    storage_before = c["storage"].clone()
    g_cum, A, o, none, final = gdn_prefill_packed_qkv_fwd(
        c["packed"], c["a"], c["b"], c["A_log"], c["dt_bias"], cu, num_qk_heads=c["Hg"], num_v_heads=c["H"],
        initial_state=c["pool"], initial_state_indices=idx, raw_cu_seqlens=tuple(c["cu"]))
    torch.cuda.synchronize()
    assert none is None and o.shape == (1, c["T"], c["H"], D)
    n_real = c["cu"][-1]
    assert_out_close(o[0, :n_real], exp_out[:n_real])
    assert torch.count_nonzero(o[0, n_real:]) == 0                       # padded suffix exactly zero
    assert_state_close(c["pool"].cpu(), exp_state)
    assert torch.equal(final, c["pool"][idx.long()])
    for s in range(16):
        if s not in c["slots"]:
            assert torch.equal(c["pool"][s].cpu(), cpu["pool"][s])
    assert torch.equal(c["storage"], storage_before)
    gold = np.load(GOLDEN / f"prefill_{name}.npz")
    assert_out_close(o[0, :n_real], torch.from_numpy(gold["out"]), "out vs chunked reference fixture")
    assert_state_close(torch.from_numpy(cases.subsample(c["pool"][idx.long()].cpu())), torch.from_numpy(gold["final"]),
                       "state vs chunked reference fixture")


@pytest.mark.gpu
@pytest.mark.parametrize("state_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("with_state", [False, True])
def test_gdn_legacy_state_and_activated_gates(native_built, with_state, state_dtype):
    """Legacy [N,H,DK,DV] state (transposed w.r.t. the pool), pre-activated fp32 g / beta, q/k already normalised."""
    from pla_b200.prefill.flashqla import chunk_gated_delta_rule_fwd
    cpu = cases.gdn_prefill_case("gdn_two_seqs")
    kw = cases.gdn_prefill_oracle_kwargs(cpu)
    T, H = cpu["T"], cpu["H"]
    g = (-cpu["A_log"].exp() * torch.nn.functional.softplus(cpu["a"].float() + cpu["dt_bias"])).contiguous()
    beta = torch.sigmoid(cpu["b"].float()).contiguous()
    init = cpu["pool"][cpu["slots"]].to(state_dtype)                      # [N,H,DV,DK]
    kw["q"] = torch.nn.functional.normalize(kw["q"].float(), dim=-1).bfloat16()
    kw["k"] = torch.nn.functional.normalize(kw["k"].float(), dim=-1).bfloat16()
    exp_out, exp_state, _ = odec.klast_forward(
        q=kw["q"], k=kw["k"], v=kw["v"], a=cpu["a"], b=cpu["b"], A_log=cpu["A_log"], dt_bias=cpu["dt_bias"],
        state=(init.float() if with_state else torch.zeros_like(init, dtype=torch.float32)),
        slot_indices=[0, 1], lengths=cpu["lengths"], scale=D ** -0.5, use_qk_l2norm=False)
    legacy = init.transpose(-1, -2).contiguous().cuda() if with_state else None
    cu = torch.tensor(cpu["cu"], dtype=torch.int32, device="cuda")
    _, _, o, _, final = chunk_gated_delta_rule_fwd(
        kw["q"].contiguous().cuda()[None], kw["k"].contiguous().cuda()[None], kw["v"].contiguous().cuda()[None],
        g.cuda()[None], beta.cuda()[None], initial_state=legacy, cu_seqlens=cu, final_state_dtype=state_dtype)
    torch.cuda.synchronize()
    n_real = cpu["cu"][-1]
    assert_out_close(o[0, :n_real], exp_out[:n_real])
    assert final.shape == (2, H, D, D) and final.dtype == state_dtype
    assert_state_close(final.float().cpu().transpose(-1, -2), exp_state,
                       tol=1e-3 if state_dtype == torch.float32 else 8e-3)
    if with_state:
        assert torch.equal(legacy.cpu(), init.transpose(-1, -2))         # the incoming legacy state is not modified


@pytest.mark.gpu
@pytest.mark.parametrize("backend", ["recurrent", "chunked"])
@pytest.mark.parametrize("softplus", [False, True])
@pytest.mark.parametrize("name", sorted(cases.KDA_PREFILL_CASES))
def test_kda_prefill(native_built, name, softplus, backend):
    from pla_b200.prefill.flashkdapro import flashkda_fwd
    cpu = cases.kda_prefill_case(name, softplus=softplus)
    c = cases.kda_prefill_case(name, softplus=softplus, device="cuda")
    exp_out, exp_state, _ = kda_oracle(cpu)
    out = torch.full((c["T"], c["H"], D), 3.0, dtype=torch.bfloat16, device="cuda")
    final = torch.empty_like(c["init"])
    init_before = c["init"].clone()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    flashkda_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"], c["A_log"], c["dt_bias"], out,
                 lower_bound=c["lower_bound"], initial_state=c["init"], final_state=final,
                 cu_seqlens=torch.tensor(c["cu"], dtype=torch.int64, device="cuda"), backend=backend, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    n_real = c["cu"][-1]
    assert_out_close(out[:n_real], exp_out[:n_real])
    assert torch.count_nonzero(out[n_real:]) == 0
    assert_state_close(final.cpu(), exp_state)
    assert torch.equal(c["init"], init_before)
    gold = np.load(GOLDEN / f"prefill_{name}_{'softplus' if softplus else 'safe'}.npz")
    assert_out_close(out[:n_real], torch.from_numpy(gold["out"]), "out vs reference fixture")
    # pool form: in place, by slot
    pool = torch.zeros(6, c["H"], D, D, device="cuda")
    slots = torch.tensor([4, 1][:len(c["lengths"])], dtype=torch.int32, device="cuda")
    pool[slots.long()] = c["init"]
    out2 = torch.empty_like(out)
    flashkda_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"], c["A_log"], c["dt_bias"], out2,
                 lower_bound=c["lower_bound"], cu_seqlens=torch.tensor(c["cu"], dtype=torch.int32, device="cuda"),
                 state_pool=pool, state_indices=slots, backend=backend)
    torch.cuda.synchronize()
    assert torch.equal(out2, out)
    assert torch.equal(pool[slots.long()], final)
    with pytest.raises(ValueError, match="mutually exclusive"):
        flashkda_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"], c["A_log"], c["dt_bias"], out2, state_pool=pool,
                     state_indices=slots, final_state=final)


@pytest.mark.gpu
@pytest.mark.parametrize("lower_bound,a_lo,a_hi", [(-5.0, 0.0, 2.5), (-1.0, -1.0, 1.0), (None, -4.0, -2.0)])
def test_kda_chunked_long_unaligned(native_built, lower_bound, a_lo, a_hi):
    """Chunked KDA on many chunks per chain with rows 2 bytes off 16-byte alignment, strong decay (safe gate
    down to -5 per token) and the weak softplus decay of the long-sequence config, against the oracle."""
    from pla_b200.prefill.flashkdapro import flashkda_fwd
    g = torch.Generator().manual_seed(123)
    H, lengths = 2, [1100, 77]
    T = sum(lengths)
    width = 4 * H * D
    packed = torch.randn(T, width + 8, generator=g).bfloat16()
    gates = torch.randn(T, H, generator=g).bfloat16()
    A_log = a_lo + (a_hi - a_lo) * torch.rand(H, generator=g)
    dt_bias = torch.randn(H, D, generator=g) * 0.1
    init = torch.randn(2, H, D, D, generator=g) * 0.05
    views = lambda t: [t[:, 1 + i * H * D:1 + (i + 1) * H * D].unflatten(1, (H, D)) for i in range(4)]
    q, k, v, gg = views(packed)
    exp_out, exp_state, _ = odec.klast_forward(q=q, k=k, v=v, a=gg, b=gates, A_log=A_log, dt_bias=dt_bias.reshape(-1),
                                               state=init, slot_indices=[0, 1], lengths=lengths, scale=D ** -0.5,
                                               is_kda=True, lower_bound=lower_bound)
    dq, dk, dv, dg = views(packed.cuda())
    assert dq.data_ptr() % 16 == 2
    out = torch.empty(T, H, D, dtype=torch.bfloat16, device="cuda")
    final = torch.empty(2, H, D, D, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    flashkda_fwd(dq, dk, dv, dg, gates.cuda(), A_log.cuda(), dt_bias.cuda(), out, lower_bound=lower_bound,
                 initial_state=init.cuda(), final_state=final, raw_cu_seqlens=(0, lengths[0], T), backend="chunked",
                 status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert_out_close(out, exp_out)
    assert_state_close(final.cpu(), exp_state)


@pytest.mark.gpu
@pytest.mark.parametrize("lower_bound,a_lo,a_hi", [(-5.0, 0.0, 2.5), (None, -4.0, -2.0)])
def test_kda_token_ranges_inside_the_gpu(native_built, lower_bound, a_lo, a_hi):
    """auto_cp of the KDA facade: a 3300-token sequence of a small batch runs as three token ranges (prescan,
    fold, parallel ranges); the pool is updated in place exactly as by the single chains, against the oracle."""
    from pla_b200.prefill.flashkdapro import flashkda_fwd
    from pla_b200.prefill.flashqla import ops as fq
    g = torch.Generator().manual_seed(321)
    H, lengths = 2, [3300, 0, 1300, 70]
    T = sum(lengths)
    offs = [0]
    for n in lengths:
        offs.append(offs[-1] + n)
    plan = fq.plan_token_ranges(offs, H, 148)
    assert plan is not None and plan[1][1] == 3
    q, k, v, gg = (torch.randn(T, H, D, generator=g).bfloat16() for _ in range(4))
    gates = torch.randn(T, H, generator=g)
    if lower_bound is None:
        gates -= 3.0                                   # small beta: the transitions of the ranges stay of order one
    gates = gates.bfloat16()
    A_log = a_lo + (a_hi - a_lo) * torch.rand(H, generator=g)
    dt_bias = torch.randn(H, D, generator=g) * 0.1
    pool = torch.randn(6, H, D, D, generator=g) * 0.3
    slots = [4, 0, 2, 5]
    exp_out, exp_state, _ = odec.klast_forward(q=q, k=k, v=v, a=gg, b=gates, A_log=A_log, dt_bias=dt_bias.reshape(-1),
                                               state=pool, slot_indices=slots, lengths=lengths, scale=D ** -0.5,
                                               is_kda=True, lower_bound=lower_bound)
    outs = {}
    for auto_cp in (False, True):
        dpool = pool.cuda()
        out = torch.empty(T, H, D, dtype=torch.bfloat16, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        flashkda_fwd(q.cuda(), k.cuda(), v.cuda(), gg.cuda(), gates.cuda(), A_log.cuda(), dt_bias.cuda(), out,
                     lower_bound=lower_bound, state_pool=dpool,
                     state_indices=torch.tensor(slots, dtype=torch.int32, device="cuda"), raw_cu_seqlens=tuple(offs),
                     backend="chunked", status=status, auto_cp=auto_cp)
        torch.cuda.synchronize()
        assert status.item() == 0
        assert_out_close(out, exp_out, f"auto_cp={auto_cp}")
        assert_state_close(dpool.cpu(), exp_state, f"auto_cp={auto_cp}")
        outs[auto_cp] = out.cpu()
    assert_out_close(outs[True], outs[False], "ranges vs single chains")


@pytest.mark.gpu
def test_kda_chunked_reports_decay_out_of_range(native_built):
    """An unbounded softplus gate that decays a channel by more than 80 nats inside 16 tokens cannot be
    represented by the sub-block references: the call flags it instead of returning silently wrong numbers."""
    from pla_b200.prefill.flashkdapro import flashkda_fwd
    g = torch.Generator().manual_seed(5)
    H, T = 1, 64
    q, k, v = (torch.randn(T, H, D, generator=g).bfloat16().cuda() for _ in range(3))
    gate = (torch.randn(T, H, D, generator=g) + 3.0).bfloat16().cuda()
    beta = torch.randn(T, H, generator=g).bfloat16().cuda()
    out = torch.empty(T, H, D, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    flashkda_fwd(q, k, v, gate, beta, torch.full((H,), 2.5).cuda(), torch.zeros(H, D).cuda(), out, lower_bound=None,
                 backend="chunked", status=status)
    torch.cuda.synchronize()
    assert status.item() & 16


def test_auto_backend_bound_for_the_softplus_gate(native_built):
    """``backend="auto"`` sends a softplus gate to the chunk-64 tensor-core kernels exactly when its parameters keep
    the decay of 16 tokens within 80 nats for gate inputs up to 20 (16 exp(max A_log) softplus(20 + max dt_bias) <= 80):
    the benchmark's weak-decay gates A_log ~ U(-4, -2) qualify, A_log = -1 does not."""
    from pla_b200.prefill.flashkdapro.ops import _softplus_decay_is_bounded
    weak = -4.0 + 2.0 * torch.rand(32, generator=torch.Generator().manual_seed(1))
    bias = torch.randn(32, 128, generator=torch.Generator().manual_seed(2)) * 0.1
    assert _softplus_decay_is_bounded(weak, bias)
    assert _softplus_decay_is_bounded(torch.full((4,), -1.5), torch.zeros(4, 128))
    assert not _softplus_decay_is_bounded(torch.full((4,), -1.0), torch.zeros(4, 128))
    assert not _softplus_decay_is_bounded(torch.tensor([-4.0, 1.0]), torch.zeros(2, 128))
    assert not _softplus_decay_is_bounded(torch.full((4,), -1.5), torch.full((4, 128), 6.0))


@pytest.mark.gpu
def test_auto_backend_runs_the_chunked_kernels_for_weak_softplus_gates(native_built):
    from pla_b200.prefill.flashkdapro import flashkda_fwd
    H, T = 2, 300
    g = torch.Generator(device="cuda").manual_seed(4)
    rn = lambda *s: torch.randn(*s, generator=g, device="cuda")
    q, k, v, gate = (rn(T, H, D).bfloat16() for _ in range(4))
    beta = rn(T, H).bfloat16()
    A_log = -4.0 + 2.0 * torch.rand(H, generator=g, device="cuda")
    dt_bias = rn(H, D) * 0.1
    outs = {}
    for backend in ("auto", "chunked", "recurrent"):
        out = torch.empty(T, H, D, dtype=torch.bfloat16, device="cuda")
        final = torch.empty(1, H, D, D, device="cuda")
        flashkda_fwd(q, k, v, gate, beta, A_log, dt_bias, out, None, None, final_state=final, backend=backend)
        outs[backend] = (out.float(), final)
    torch.cuda.synchronize()
    assert torch.equal(outs["auto"][0], outs["chunked"][0]) and torch.equal(outs["auto"][1], outs["chunked"][1])
    assert_out_close(outs["auto"][0], outs["recurrent"][0], "chunked vs token recurrence")
    assert_state_close(outs["auto"][1], outs["recurrent"][1], "chunked vs token recurrence")
