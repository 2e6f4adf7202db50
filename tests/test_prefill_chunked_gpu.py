"""Chunked (chunk 64) tensor-core GDN prefill: the prepare stage's operand images against fp32 torch,
and the whole op against the CPU oracle and the chunked reference fixtures."""
from pathlib import Path

import numpy as np
import pytest
import torch

import cases
from helpers import assert_out_close, assert_state_close
from oracle import decode as odec

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
D, C = 128, 64
KQ_BYTES, KNT_BYTES, TM_BYTES, PM_BYTES, VEC_BYTES = 128 * 128 * 4, 128 * 64 * 4, 64 * 64 * 4, 64 * 64 * 4, 1024
HBLOB, VBLOB = KQ_BYTES + KNT_BYTES, TM_BYTES + PM_BYTES + VEC_BYTES


def image_to_tile(img, rows, kdim):
    """Operand image [K/4][rows][4] -> [rows, K]."""
    return img.view(kdim // 4, rows, 4).permute(1, 0, 2).reshape(rows, kdim)


def run_op(c, stage, state=True):
    from pla_b200._ops import ops
    Hg, H, T = c["Hg"], c["H"], c["T"]
    p = c["packed"]
    q = p.as_strided((T, Hg, D), (p.stride(0), D, 1), p.storage_offset())
    k = p.as_strided((T, Hg, D), (p.stride(0), D, 1), p.storage_offset() + Hg * D)
    v = p.as_strided((T, H, D), (p.stride(0), D, 1), p.storage_offset() + 2 * Hg * D)
    out = torch.full((T, H, D), 7.0, dtype=torch.bfloat16, device="cuda")
    g_cum = torch.zeros(T, H, device="cuda")
    cu = torch.tensor(c["cu"], dtype=torch.int32, device="cuda")
    idx = torch.tensor(c["slots"], dtype=torch.int32, device="cuda")
    max_chunks = sum((n + C - 1) // C for n in c["lengths"])
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ws = ops.gdn_prefill_chunked(q, k, v, c["a"], c["b"], c["A_log"], c["dt_bias"], out, g_cum, cu,
                                 c["pool"] if state else None, idx if state else None, None, None, False, True,
                                 D ** -0.5, False, state, max_chunks, stage, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    return ws, out, g_cum, max_chunks


@pytest.mark.parametrize("name", sorted(cases.PREFILL_CASES))
def test_prepare_stage_operand_images(native_built, name):
    c = cases.gdn_prefill_case(name, device="cuda")
    cpu = cases.gdn_prefill_case(name)
    ws, _, g_cum, max_chunks = run_op(c, stage=1)
    ws = ws.cpu()
    kw = cases.gdn_prefill_oracle_kwargs(cpu)
    Hg, H = cpu["Hg"], cpu["H"]
    R = H // Hg
    qn = odec.l2norm(kw["q"].float()) * D ** -0.5
    kn = odec.l2norm(kw["k"].float())
    g = odec.log_decay(cpu["a"].float() + cpu["dt_bias"], cpu["A_log"][None], None)      # [T,H]
    beta = torch.sigmoid(cpu["b"].float())
    gc = 0
    for s, n_seq in enumerate(cpu["lengths"]):
        for ci in range((n_seq + C - 1) // C):
            t0 = cpu["cu"][s] + ci * C
            n = min(C, n_seq - ci * C)
            for h in range(Hg):
                blob = ws[(gc * Hg + h) * HBLOB:(gc * Hg + h + 1) * HBLOB]
                kq = image_to_tile(blob[:KQ_BYTES].view(torch.float32), 128, 128)
                knt = image_to_tile(blob[KQ_BYTES:].view(torch.float32), 128, 64)
                Kn = torch.zeros(C, D); Qn = torch.zeros(C, D)
                Kn[:n] = kn[t0:t0 + n, h]; Qn[:n] = qn[t0:t0 + n, h]
                torch.testing.assert_close(kq[:64], Kn, rtol=1e-3, atol=1e-4)
                torch.testing.assert_close(kq[64:], Qn, rtol=1e-3, atol=1e-5)
                assert torch.equal(knt, kq[:64].t())
                A = Kn @ Kn.t()
                QK = Qn @ Kn.t()
                for r in range(R):
                    hv = h * R + r
                    off = max_chunks * Hg * HBLOB + (gc * H + hv) * VBLOB
                    vb = ws[off:off + VBLOB]
                    # of column group jg only rows 4 jg .. 63 are stored (the rows above are zero by construction
                    # and are never written to or copied from the workspace)
                    stored = torch.arange(C)[:, None] >= (torch.arange(C)[None, :] // 4) * 4
                    Tm = torch.where(stored, image_to_tile(vb[:TM_BYTES].view(torch.float32), 64, 64), 0.0)
                    Pm = torch.where(stored, image_to_tile(vb[TM_BYTES:TM_BYTES + PM_BYTES].view(torch.float32), 64, 64), 0.0)
                    vec = vb[TM_BYTES + PM_BYTES:].view(torch.float32)
                    G = torch.zeros(C); b = torch.zeros(C)
                    G[:n] = torch.cumsum(g[t0:t0 + n, hv], 0); G[n:] = G[n - 1]
                    b[:n] = beta[t0:t0 + n, hv]
                    torch.testing.assert_close(vec[:64], b * torch.exp(G), rtol=1e-4, atol=1e-6)
                    torch.testing.assert_close(vec[64:128], b, rtol=1e-4, atol=1e-6)
                    torch.testing.assert_close(g_cum[t0:t0 + n, hv].cpu(), G[:n], rtol=1e-4, atol=1e-5)
                    Gam = torch.exp(G[:, None] - G[None, :])
                    L = torch.tril(b[:, None] * A * Gam, -1)
                    T_ref = torch.linalg.solve_triangular(torch.eye(C) + L, torch.eye(C), upper=False)
                    P_ref = torch.tril(QK * Gam)
                    P_ref[n:] = 0
                    torch.testing.assert_close(Tm, T_ref, rtol=5e-3, atol=2e-3)
                    torch.testing.assert_close(Pm, P_ref, rtol=5e-3, atol=1e-4)
            gc += 1


@pytest.mark.parametrize("with_state", [True, False])
@pytest.mark.parametrize("name", sorted(cases.PREFILL_CASES))
def test_chunked_prefill_matches_oracle_and_fixture(native_built, name, with_state):
    c = cases.gdn_prefill_case(name, device="cuda")
    cpu = cases.gdn_prefill_case(name)
    kw = cases.gdn_prefill_oracle_kwargs(cpu)
    if not with_state:
        kw["state"] = torch.zeros_like(cpu["pool"])
    exp_out, exp_state, _ = odec.klast_forward(**kw)
    pool_before = c["pool"].clone()
    _, out, _, _ = run_op(c, stage=0, state=with_state)
    n_real = cpu["cu"][-1]
    assert_out_close(out[:n_real], exp_out[:n_real])
    assert torch.count_nonzero(out[n_real:]) == 0
    if with_state:
        assert_state_close(c["pool"].cpu(), exp_state)
        for s in range(16):
            if s not in cpu["slots"]:
                assert torch.equal(c["pool"][s], pool_before[s])
        gold = np.load(GOLDEN / f"prefill_{name}.npz")
        assert_out_close(out[:n_real], torch.from_numpy(gold["out"]), "out vs chunked reference fixture")
        idx = torch.tensor(cpu["slots"])
        assert_state_close(torch.from_numpy(cases.subsample(c["pool"].cpu()[idx])), torch.from_numpy(gold["final"]),
                           "state vs chunked reference fixture")
    else:
        assert torch.equal(c["pool"], pool_before)          # no state given: nothing written


def test_chunked_prefill_long_sequences_against_token_recurrence(native_built):
    """Many chunks per chain (barrier phases wrap, errors accumulate): the tensor-core path against the
    CPU oracle on a 2048-token sequence and against the token-recurrent GPU kernel at 8 x ~4K tokens."""
    from pla_b200._ops import ops
    g = torch.Generator().manual_seed(77)
    Hg, H = 1, 2
    lengths = [2048, 333]
    T = sum(lengths)
    width = 2 * Hg * D + H * D
    packed = torch.randn(T, width, generator=g).bfloat16()
    gates = torch.randn(T, 2 * H, generator=g).bfloat16()
    A_log = torch.rand(H, generator=g) * float(np.log(16.0))
    dt_bias = torch.randn(H, generator=g) * 0.1
    pool = torch.randn(4, H, D, D, generator=g) * 0.02
    cu = [0, 2048, T]
    q = packed[:, :Hg * D].reshape(T, Hg, D)
    k = packed[:, Hg * D:2 * Hg * D].reshape(T, Hg, D)
    v = packed[:, 2 * Hg * D:].reshape(T, H, D)
    exp_out, exp_state, _ = odec.klast_forward(q=q, k=k, v=v, a=gates[:, :H], b=gates[:, H:], A_log=A_log,
                                               dt_bias=dt_bias, state=pool, slot_indices=[2, 0], lengths=lengths,
                                               scale=D ** -0.5)
    dp = packed.cuda()
    dq = dp.as_strided((T, Hg, D), (width, D, 1), 0)
    dk = dp.as_strided((T, Hg, D), (width, D, 1), Hg * D)
    dv = dp.as_strided((T, H, D), (width, D, 1), 2 * Hg * D)
    dg = gates.cuda()
    dpool = pool.cuda()
    out = torch.empty(T, H, D, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.gdn_prefill_chunked(dq, dk, dv, dg[:, :H], dg[:, H:], A_log.cuda(), dt_bias.cuda(), out, None,
                            torch.tensor(cu, dtype=torch.int32, device="cuda"), dpool,
                            torch.tensor([2, 0], dtype=torch.int32, device="cuda"), None, None, False, True,
                            D ** -0.5, False, True, sum((n + C - 1) // C for n in lengths), 0, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert_out_close(out, exp_out)
    assert_state_close(dpool.cpu(), exp_state)

    # config-3 sized: both GPU evaluations of the same recurrence must agree
    Hg, H = 16, 32
    lengths = torch.randint(512, 8193, (8,), generator=g).tolist()
    T = sum(lengths)
    width = 2 * Hg * D + H * D
    dp = torch.empty(T, width, dtype=torch.bfloat16, device="cuda").normal_(generator=torch.Generator("cuda").manual_seed(3))
    dq = dp.as_strided((T, Hg, D), (width, D, 1), 0)
    dk = dp.as_strided((T, Hg, D), (width, D, 1), Hg * D)
    dv = dp.as_strided((T, H, D), (width, D, 1), 2 * Hg * D)
    dg = torch.randn(T, 2 * H, generator=g).bfloat16().cuda()
    A_log = (torch.rand(H, generator=g) * float(np.log(16.0))).cuda()
    dt_bias = (torch.randn(H, generator=g) * 0.1).cuda()
    pool_a = (torch.randn(16, H, D, D, generator=g) * 0.02).cuda()
    pool_b = pool_a.clone()
    idx = torch.arange(1, 16, 2, dtype=torch.int32, device="cuda")
    offs = [0]
    for n in lengths:
        offs.append(offs[-1] + n)
    cu = torch.tensor(offs, dtype=torch.int32, device="cuda")
    out_a = torch.empty(T, H, D, dtype=torch.bfloat16, device="cuda")
    out_b = torch.empty_like(out_a)
    ops.gdn_prefill_chunked(dq, dk, dv, dg[:, :H], dg[:, H:], A_log, dt_bias, out_a, None, cu, pool_a, idx, None, None,
                            False, True, D ** -0.5, False, True, sum((n + C - 1) // C for n in lengths), 0, status)
    ops.prefill_recurrent(dq, dk, dv, dg[:, :H], dg[:, H:], A_log, dt_bias, out_b, cu, pool_b, idx, None, None, False,
                          False, True, D ** -0.5, None, False, True, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert_out_close(out_a, out_b, "chunked vs token-recurrent output")
    assert_state_close(pool_a, pool_b, "chunked vs token-recurrent state")


def test_chunked_prefill_every_state_scaling_mode(native_built):
    """The chain keeps the state as S / sigma and decides per chunk, from the chunk's total decay, between three modes:
    carry sigma along (weak decay), rescale the accumulator (sigma about to leave [2^-40, 1]) or overwrite it (the
    chunk alone decays below 2^-40). One value head per decay strength from e^-0.02 to e^-700 per chunk, 24 chunks
    each, so that every mode and every transition between modes occurs; outputs and states against the CPU oracle,
    head by head."""
    from pla_b200._ops import ops
    g = torch.Generator().manual_seed(2040)
    Hg, H = 2, 16
    lengths = [1536, 700]
    T = sum(lengths)
    width = 2 * Hg * D + H * D
    packed = torch.randn(T, width, generator=g).bfloat16()
    gates = torch.randn(T, 2 * H, generator=g).bfloat16()
    # mean log decay per token about -0.7 e^{A_log}: per chunk from -0.02 (A_log = -7.7) to -700 (A_log = 2.75)
    A_log = torch.linspace(-7.7, 2.75, H)
    dt_bias = torch.randn(H, generator=g) * 0.1
    pool = torch.randn(4, H, D, D, generator=g) * 0.02
    cu = [0, lengths[0], T]
    q = packed[:, :Hg * D].reshape(T, Hg, D)
    k = packed[:, Hg * D:2 * Hg * D].reshape(T, Hg, D)
    v = packed[:, 2 * Hg * D:].reshape(T, H, D)
    exp_out, exp_state, _ = odec.klast_forward(q=q, k=k, v=v, a=gates[:, :H], b=gates[:, H:], A_log=A_log,
                                               dt_bias=dt_bias, state=pool, slot_indices=[3, 1], lengths=lengths,
                                               scale=D ** -0.5)
    dp = packed.cuda()
    dq = dp.as_strided((T, Hg, D), (width, D, 1), 0)
    dk = dp.as_strided((T, Hg, D), (width, D, 1), Hg * D)
    dv = dp.as_strided((T, H, D), (width, D, 1), 2 * Hg * D)
    dg = gates.cuda()
    dpool = pool.cuda()
    out = torch.empty(T, H, D, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.gdn_prefill_chunked(dq, dk, dv, dg[:, :H], dg[:, H:], A_log.cuda(), dt_bias.cuda(), out, None,
                            torch.tensor(cu, dtype=torch.int32, device="cuda"), dpool,
                            torch.tensor([3, 1], dtype=torch.int32, device="cuda"), None, None, False, True,
                            D ** -0.5, False, True, sum((n + C - 1) // C for n in lengths), 0, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    got = dpool.cpu()
    for h in range(H):
        assert_out_close(out[:, h].cpu(), exp_out[:, h], f"value head {h} (A_log {A_log[h]:.2f})")
        for slot in (3, 1):
            assert_state_close(got[slot, h], exp_state[slot, h], f"value head {h} (A_log {A_log[h]:.2f}), slot {slot}")
    assert torch.equal(got[[0, 2]], pool[[0, 2]])


def test_chunked_prefill_rows_ending_at_the_allocation_end(native_built):
    """q, k, v that fill their allocations exactly (2 MiB each, 16-byte aligned rows): the staged row
    copies must not touch a byte past the last row."""
    from pla_b200._ops import ops
    g = torch.Generator().manual_seed(9)
    T, Hg, H = 1024, 8, 8
    q, k, v = (torch.randn(T, n, D, generator=g).bfloat16() for n in (Hg, Hg, H))
    gates = torch.randn(T, 2 * H, generator=g).bfloat16()
    A_log = torch.rand(H, generator=g) * float(np.log(16.0))
    dt_bias = torch.randn(H, generator=g) * 0.1
    exp_out, exp_state, _ = odec.klast_forward(q=q, k=k, v=v, a=gates[:, :H], b=gates[:, H:], A_log=A_log,
                                               dt_bias=dt_bias, state=torch.zeros(1, H, D, D), slot_indices=[0],
                                               lengths=[T], scale=D ** -0.5)
    dq, dk, dv = q.cuda(), k.cuda(), v.cuda()
    assert all(x.numel() * 2 == 2 << 20 and x.data_ptr() % 16 == 0 for x in (dq, dk, dv))
    dg = gates.cuda()
    out = torch.empty(T, H, D, dtype=torch.bfloat16, device="cuda")
    final = torch.empty(1, H, D, D, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.gdn_prefill_chunked(dq, dk, dv, dg[:, :H], dg[:, H:], A_log.cuda(), dt_bias.cuda(), out, None,
                            torch.tensor([0, T], dtype=torch.int32, device="cuda"), None, None, final, None, False,
                            True, D ** -0.5, False, False, T // C, 0, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert_out_close(out, exp_out)
    assert_state_close(final.cpu()[0], exp_state[0])


@pytest.mark.parametrize("dtype,Hg,H", [(torch.float16, 1, 2), (torch.bfloat16, 1, 12), (torch.bfloat16, 2, 6)])
def test_chunked_prefill_head_groups_and_fp16(native_built, dtype, Hg, H):
    """fp16 activations, and value-head groups of 2, 3 and 12 per q/k head (more than one pass of eight heads
    inside the prepare kernel), against the oracle."""
    from pla_b200._ops import ops
    g = torch.Generator().manual_seed(41)
    lengths = [130, 64, 1]
    T = sum(lengths)
    q, k, v = (torch.randn(T, n, D, generator=g).to(dtype) for n in (Hg, Hg, H))
    gates = torch.randn(T, 2 * H, generator=g).to(dtype)
    A_log = torch.rand(H, generator=g) * float(np.log(16.0))
    dt_bias = torch.randn(H, generator=g) * 0.1
    pool = torch.randn(5, H, D, D, generator=g) * 0.05
    slots = [3, 0, 4]
    exp_out, exp_state, _ = odec.klast_forward(q=q, k=k, v=v, a=gates[:, :H], b=gates[:, H:], A_log=A_log,
                                               dt_bias=dt_bias, state=pool, slot_indices=slots, lengths=lengths,
                                               scale=D ** -0.5)
    dg, dpool = gates.cuda(), pool.cuda()
    out = torch.empty(T, H, D, dtype=dtype, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cu = torch.tensor([0, 130, 194, 195], dtype=torch.int32, device="cuda")
    ops.gdn_prefill_chunked(q.cuda(), k.cuda(), v.cuda(), dg[:, :H], dg[:, H:], A_log.cuda(), dt_bias.cuda(), out, None,
                            cu, dpool, torch.tensor(slots, dtype=torch.int32, device="cuda"), None, None, False, True,
                            D ** -0.5, False, True, T // C + 3, 0, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert_out_close(out, exp_out)
    assert_state_close(dpool.cpu(), exp_state)
    untouched = [s for s in range(5) if s not in slots]
    assert torch.equal(dpool[untouched].cpu(), pool[untouched])


@pytest.mark.parametrize("weak_decay", [False, True])
def test_intra_gpu_token_ranges_match_single_chains(native_built, weak_decay):
    """auto_cp: long sequences cut into token ranges (prescan, fold, parallel ranges) against the same
    sequences run as single chains and against the oracle; pool updated in place either way. With weak decay
    and small beta the transition of a 1088-token range stays of order one, so the incoming state of the later
    ranges depends on the folded transitions and not only on the offsets."""
    from pla_b200.prefill.flashqla import ops as fq
    g = torch.Generator().manual_seed(17)
    Hg, H = 1, 2
    lengths = [3300, 0, 1300, 70]
    T = sum(lengths)
    offs = [0]
    for n in lengths:
        offs.append(offs[-1] + n)
    plan = fq.plan_token_ranges(offs, H, 148)
    assert plan is not None and plan[1][1] > 1 and plan[1][-1] == len(plan[2])   # the 3300-token sequence becomes three ranges
    q, k, v = (torch.randn(1, T, n, D, generator=g).bfloat16() for n in (Hg, Hg, H))
    gates = torch.randn(T, 2 * H, generator=g)
    A_log = torch.rand(H, generator=g) * float(np.log(16.0))
    if weak_decay:
        gates[:, H:] -= 4.0
        A_log = -8.0 + torch.rand(H, generator=g)
    gates = gates.bfloat16()
    dt_bias = torch.randn(H, generator=g) * 0.1
    pool = torch.randn(6, H, D, D, generator=g) * (0.5 if weak_decay else 0.05)
    slots = [4, 0, 2, 5]
    exp_out, exp_state, _ = odec.klast_forward(q=q[0], k=k[0], v=v[0], a=gates[:, :H], b=gates[:, H:], A_log=A_log,
                                               dt_bias=dt_bias, state=pool, slot_indices=slots, lengths=lengths,
                                               scale=D ** -0.5)
    dev = "cuda"
    results = {}
    for auto_cp in (False, True):
        dpool = pool.to(dev)
        dg = gates.to(dev)
        res = fq.chunk_gated_delta_rule_fwd(
            q.to(dev), k.to(dev), v.to(dev), None, None, initial_state=dpool,
            initial_state_indices=torch.tensor(slots, dtype=torch.int32, device=dev),
            cu_seqlens=torch.tensor(offs, dtype=torch.int32, device=dev), output_final_state=True, auto_cp=auto_cp,
            normalize_qk=True, raw_cu_seqlens=tuple(offs), raw_gate_a=dg[:, :H], raw_beta_b=dg[:, H:],
            A_log=A_log.to(dev), dt_bias=dt_bias.to(dev))
        torch.cuda.synchronize()
        results[auto_cp] = (res[2][0].cpu(), dpool.cpu(), res[4].cpu(), res[0].cpu())
        assert_out_close(res[2][0], exp_out, f"auto_cp={auto_cp}")
        assert_state_close(dpool.cpu(), exp_state, f"auto_cp={auto_cp}")
        assert torch.equal(res[4].cpu(), dpool.cpu()[slots])
    assert torch.equal(results[True][3], results[False][3])                  # g_cum is the same by-product
    assert_out_close(results[True][0], results[False][0], "ranges vs single chains")


def test_negative_slot_is_padding_with_and_without_token_ranges(native_built):
    """A sequence whose slot index is negative is padding in both evaluations of the same call: zero output rows,
    no slot read or written, zero rows in the returned final states; the other sequences are unaffected."""
    from pla_b200.prefill.flashqla import ops as fq
    g = torch.Generator().manual_seed(23)
    Hg, H = 1, 2
    lengths = [3300, 1300, 70]
    T = sum(lengths)
    offs = [0, 3300, 4600, 4670]
    assert fq.plan_token_ranges(offs, H, 148) is not None
    q, k, v = (torch.randn(1, T, n, D, generator=g).bfloat16() for n in (Hg, Hg, H))
    gates = torch.randn(T, 2 * H, generator=g).bfloat16()
    A_log = torch.rand(H, generator=g) * 2.0
    dt_bias = torch.randn(H, generator=g) * 0.1
    pool = torch.randn(6, H, D, D, generator=g) * 0.05
    slots = [-1, 2, 5]
    live = torch.arange(T) >= offs[1]
    exp_out, exp_state, _ = odec.klast_forward(q=q[0], k=k[0], v=v[0], a=gates[:, :H], b=gates[:, H:], A_log=A_log,
                                               dt_bias=dt_bias, state=pool, slot_indices=slots, lengths=lengths,
                                               scale=D ** -0.5)
    dev = "cuda"
    outs = {}
    for auto_cp in (False, True):
        dpool = pool.to(dev)
        dg = gates.to(dev)
        res = fq.chunk_gated_delta_rule_fwd(
            q.to(dev), k.to(dev), v.to(dev), None, None, initial_state=dpool,
            initial_state_indices=torch.tensor(slots, dtype=torch.int32, device=dev),
            cu_seqlens=torch.tensor(offs, dtype=torch.int32, device=dev), output_final_state=True, auto_cp=auto_cp,
            normalize_qk=True, raw_cu_seqlens=tuple(offs), raw_gate_a=dg[:, :H], raw_beta_b=dg[:, H:],
            A_log=A_log.to(dev), dt_bias=dt_bias.to(dev))
        torch.cuda.synchronize()
        out, final = res[2][0].cpu(), res[4].cpu()
        assert torch.count_nonzero(out[~live]) == 0, f"auto_cp={auto_cp}: the padding sequence must give zero rows"
        assert_out_close(out[live], exp_out[live], f"auto_cp={auto_cp}")
        assert_state_close(dpool.cpu(), exp_state, f"auto_cp={auto_cp}")
        for s_ in (0, 1, 3, 4):
            assert torch.equal(dpool[s_].cpu(), pool[s_])
        assert torch.count_nonzero(final[0]) == 0 and torch.equal(final[1:], dpool.cpu()[[2, 5]])
        outs[auto_cp] = out
    assert_out_close(outs[True], outs[False], "ranges vs single chains")


@pytest.mark.parametrize("name", sorted(cases.PREFILL_CASES))
def test_chunk_factor_by_product(native_built, name):
    """``A`` of the facade's return tuple (pla/prefill/flashqla/ops.py:247-248 of the reference returns it second): a
    deferred object that lays the chunk-64 factor out as [1, T, H, 64] on first use -- each token's row of
    (I + tril(diag(beta) K K^T . Gamma, -1))^-1, zero rows past the last sequence."""
    from pla_b200.prefill.flashqla import gdn_prefill_packed_qkv_fwd
    from pla_b200.prefill.flashqla.ops import ChunkFactor
    c = cases.gdn_prefill_case(name, device="cuda")
    cpu = cases.gdn_prefill_case(name)
    Hg, H, T = cpu["Hg"], cpu["H"], cpu["T"]
    g_cum, A, o, none, final = gdn_prefill_packed_qkv_fwd(
        c["packed"], c["a"], c["b"], c["A_log"], c["dt_bias"], torch.tensor(cpu["cu"], dtype=torch.int32, device="cuda"),
        num_qk_heads=Hg, num_v_heads=H, initial_state=c["pool"],
        initial_state_indices=torch.tensor(cpu["slots"], dtype=torch.int32, device="cuda"), output_final_state=False,
        raw_cu_seqlens=tuple(cpu["cu"]))
    assert isinstance(A, ChunkFactor) and none is None
    assert tuple(A.shape) == (1, T, H, C) and A.dtype == torch.float32       # touching it lays it out
    got = (A * 1.0)[0].cpu()                                                   # operators and torch functions
    assert torch.equal(got, A[0].cpu()) and torch.equal(torch.mul(A, 1.0)[0].cpu(), got)
    kw = cases.gdn_prefill_oracle_kwargs(cpu)
    kn = odec.l2norm(kw["k"].float())
    g = odec.log_decay(cpu["a"].float() + cpu["dt_bias"], cpu["A_log"][None], None)
    beta = torch.sigmoid(cpu["b"].float())
    R = H // Hg
    for s, n_seq in enumerate(cpu["lengths"]):
        for ci in range((n_seq + C - 1) // C):
            t0 = cpu["cu"][s] + ci * C
            n = min(C, n_seq - ci * C)
            for hv in range(H):
                K = kn[t0:t0 + n, hv // R]
                G = torch.cumsum(g[t0:t0 + n, hv], 0)
                L = torch.tril(beta[t0:t0 + n, hv, None] * (K @ K.t()) * torch.exp(G[:, None] - G[None, :]), -1)
                T_ref = torch.linalg.solve_triangular(torch.eye(n) + L, torch.eye(n), upper=False)
                torch.testing.assert_close(got[t0:t0 + n, hv, :n], T_ref, rtol=5e-3, atol=2e-3)
    assert torch.count_nonzero(got[cpu["cu"][-1]:]) == 0
