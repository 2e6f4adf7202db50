"""Parity at the full benchmark sizes, against the CPU oracle on head subsets (value heads are independent, so the
oracle on two or three of them over all tokens costs seconds) and through size-independent properties: the decode
step is jointly linear in (state, v); slots a step does not address stay bit-identical; a sequence's prefill result
does not depend on the batch around it; the chunked evaluation agrees with the exact token recurrence on the GPU."""
import math
from types import SimpleNamespace

import pytest
import torch

from helpers import assert_out_close, assert_state_close
from oracle import decode as odec

pytestmark = pytest.mark.gpu
D = 128


def test_config1_decode_is_linear_in_state_and_v_and_leaves_other_slots_alone(native_built):
    from pla_b200.decode import fused_sigmoid_gating_delta_rule_forward_k_last as forward
    B, H, HV, SLOTS = 256, 16, 32, 1024
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(20261125 + 1)
    rn = lambda *s: torch.randn(*s, generator=g, device=dev)
    q, k = rn(1, B, H, D).bfloat16(), rn(1, B, H, D).bfloat16()
    a, b = rn(1, B, HV).bfloat16(), rn(1, B, HV).bfloat16()
    A_log = torch.rand(HV, generator=g, device=dev) * math.log(16.0)
    dt_bias = (rn(HV) * 0.1).bfloat16()
    idx = torch.randperm(SLOTS, generator=g, device=dev)[:B].to(torch.int32)
    cu = torch.arange(B + 1, dtype=torch.int32, device=dev)
    # v1, v2 and v1 + v2 all exactly representable in bf16: multiples of 1/8 below 4
    v1 = (torch.randint(-16, 17, (1, B, HV, D), generator=g, device=dev).float() / 8).bfloat16()
    v2 = (torch.randint(-16, 17, (1, B, HV, D), generator=g, device=dev).float() / 8).bfloat16()
    S1 = rn(SLOTS, HV, D, D) * 0.02
    S2 = rn(SLOTS, HV, D, D) * 0.02
    outs, pools = [], []
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for S, v in ((S1, v1), (S2, v2), (S1 + S2, (v1.float() + v2.float()).bfloat16())):
        pool = S.clone()
        o = forward(A_log, a, dt_bias, 1.0, 20.0, q, k, v, b, pool, idx, D ** -0.5, True, cu, False, False, None, None,
                    None, None, status=status)
        outs.append(o.float())
        pools.append(pool)
    torch.cuda.synchronize()
    assert status.item() == 0
    used = idx.long()
    lin = (pools[0][used] + pools[1][used] - pools[2][used]).norm() / pools[2][used].norm()
    assert lin.item() <= 1e-5, lin.item()
    # outputs are rounded to bf16 once each: the sum of two roundings against one
    assert (outs[0] + outs[1] - outs[2]).abs().max().item() <= 2e-2
    others = torch.ones(SLOTS, dtype=torch.bool, device=dev)
    others[used] = False
    assert torch.equal(pools[0][others], S1[others]) and torch.equal(pools[2][others], (S1 + S2)[others])
    # four sampled requests of the full launch against the CPU oracle
    pick = [0, 77, 128, 255]
    sel = torch.tensor(pick, device=dev)
    exp_out, exp_state, _ = odec.klast_forward(
        q=q[0, sel].cpu(), k=k[0, sel].cpu(), v=v1[0, sel].cpu(), a=a[0, sel].cpu(), b=b[0, sel].cpu(), A_log=A_log.cpu(),
        dt_bias=dt_bias.cpu(), state=S1[used[sel]].cpu(), slot_indices=list(range(len(pick))), lengths=[1] * len(pick),
        scale=D ** -0.5)
    assert_out_close(outs[0][0, sel].cpu(), exp_out)
    assert_state_close(pools[0][used[sel]].cpu(), exp_state)
    # the packed-QKV op (the benchmark's op) on the same step: one mixed row per request, bit-identical results
    from pla_b200.decode import fused_sigmoid_gating_delta_rule_forward_k_last_packed as packed
    mixed = torch.cat([q[0].reshape(B, H * D), k[0].reshape(B, H * D), v1[0].reshape(B, HV * D)], dim=1).contiguous()
    pool_p = S1.clone()
    out_p = torch.empty(B, 1, HV, D, dtype=torch.bfloat16, device=dev)
    packed(mixed, a[0], b[0], A_log, dt_bias, 1.0, 20.0, D ** -0.5, pool_p, idx, out_p, True, cu, False, True,
           status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert torch.equal(out_p[:, 0].float(), outs[0][0]) and torch.equal(pool_p, pools[0])
    # the v-last layout ([slots, HV, K, V] pool) through its own op: same recurrence on the transposed tiles
    from pla_b200.decode.gdn.v_last import fused_sigmoid_gating_delta_rule as vlast
    pool_v = S1.transpose(-1, -2).contiguous()
    out_v = torch.empty(B, 1, HV, D, dtype=torch.bfloat16, device=dev)
    vlast(A_log, a[0], dt_bias, q[0][:, None], k[0][:, None], v1[0][:, None], b[0], out_v, pool_v, idx, None, 1.0, 20.0,
          D ** -0.5, 1, B, H, HV, D, D, True, True, False)
    torch.cuda.synchronize()
    assert_out_close(out_v[sel, 0].cpu(), exp_out, "v-last vs oracle")
    assert_state_close(pool_v[used[sel]].transpose(-1, -2).cpu(), exp_state, "v-last vs oracle")
    assert_out_close(out_v[:, 0], outs[0][0], "v-last vs k-last, all requests")
    assert_state_close(pool_v[used].transpose(-1, -2), pools[0][used], "v-last vs k-last, all requests")
    assert torch.equal(pool_v[others], S1.transpose(-1, -2)[others])


def test_config3_prefill_sequences_do_not_depend_on_the_batch_and_match_the_recurrence(native_built):
    from pla_b200._ops import ops
    from pla_b200.prefill.flashqla import ops as fq
    dev = "cuda"
    g = torch.Generator().manual_seed(20261125 + 3)
    lengths = torch.randint(512, 8193, (8,), generator=g).tolist()
    T, Hg, H = sum(lengths), 16, 32
    offs = [0]
    for n in lengths:
        offs.append(offs[-1] + n)
    gd = torch.Generator(device=dev).manual_seed(7)
    rn = lambda *s: torch.randn(*s, generator=gd, device=dev)
    q, k, v = rn(1, T, Hg, D).bfloat16(), rn(1, T, Hg, D).bfloat16(), rn(1, T, H, D).bfloat16()
    ga, gb = rn(T, H).bfloat16(), rn(T, H).bfloat16()
    A_log = torch.rand(H, generator=gd, device=dev) * math.log(16.0)
    dt_bias = rn(H) * 0.1
    pool0 = rn(16, H, D, D) * 0.02
    slots = torch.randperm(16, generator=g)[:8].to(torch.int32).to(dev)

    def run(sl, offsets, idx, pool):
        return fq.chunk_gated_delta_rule_fwd(
            q[:, sl], k[:, sl], v[:, sl], None, None, initial_state=pool, initial_state_indices=idx,
            cu_seqlens=torch.tensor(offsets, dtype=torch.int32, device=dev), output_final_state=False, auto_cp=False,
            normalize_qk=True, raw_cu_seqlens=tuple(offsets), raw_gate_a=ga[sl], raw_beta_b=gb[sl], A_log=A_log,
            dt_bias=dt_bias)[2][0]

    pool = pool0.clone()
    out = run(slice(0, T), offs, slots, pool)
    for s in (2, 7):                                   # the same sequences alone: bit-identical rows and states
        alone = pool0.clone()
        o = run(slice(offs[s], offs[s + 1]), [0, lengths[s]], slots[s:s + 1], alone)
        assert torch.equal(o, out[offs[s]:offs[s + 1]])
        assert torch.equal(alone[slots[s].item()], pool[slots[s].item()])
    # the exact token recurrence on the GPU over the whole batch
    ref_pool = pool0.clone()
    ref = torch.empty(T, H, D, dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.prefill_recurrent(q[0], k[0], v[0], ga, gb, A_log, dt_bias, ref, torch.tensor(offs, dtype=torch.int32, device=dev),
                          ref_pool, slots, None, None, False, False, True, D ** -0.5, None, False, True, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert_out_close(out, ref, "chunked vs token recurrence")
    assert_state_close(pool[slots.long()], ref_pool[slots.long()], "chunked vs token recurrence")
    untouched = [s for s in range(16) if s not in slots.tolist()]
    assert torch.equal(pool[untouched], pool0[untouched])
    # the CPU oracle on value heads 6, 7 (q/k head 3) of all eight sequences: outputs and final states
    hv_sel, h_sel = [6, 7], [3]
    exp_out, exp_state, _ = odec.klast_forward(
        q=q[0][:, h_sel].cpu(), k=k[0][:, h_sel].cpu(), v=v[0][:, hv_sel].cpu(), a=ga[:, hv_sel].cpu(),
        b=gb[:, hv_sel].cpu(), A_log=A_log[hv_sel].cpu(), dt_bias=dt_bias[hv_sel].cpu(),
        state=pool0[:, hv_sel].cpu().contiguous(), slot_indices=slots.tolist(), lengths=lengths, scale=D ** -0.5)
    assert_out_close(out[:, hv_sel].cpu(), exp_out, "chunked vs CPU oracle, value heads 6-7")
    assert_state_close(pool[slots.long()][:, hv_sel].cpu(), exp_state[slots.long().cpu()], "chunked vs CPU oracle")
    for s in range(8):                                 # per sequence, so that a short one cannot hide behind the long
        assert_state_close(pool[slots[s].item(), hv_sel].cpu(), exp_state[slots[s].item()], f"sequence {s} vs CPU oracle")
    # the packed-row entry (the benchmark's call): rows 34 bytes off 16-byte alignment, same results bit for bit
    width = 2 * Hg * D + H * D
    storage = torch.empty(T, width + 64, dtype=torch.bfloat16, device=dev)
    rows = storage[:, 17:17 + width]
    rows.copy_(torch.cat([q[0].reshape(T, Hg * D), k[0].reshape(T, Hg * D), v[0].reshape(T, H * D)], dim=1))
    pool_p = pool0.clone()
    out_p = fq.gdn_prefill_packed_qkv_fwd(rows, ga, gb, A_log, dt_bias, torch.tensor(offs, dtype=torch.int32, device=dev),
                                          num_qk_heads=Hg, num_v_heads=H, initial_state=pool_p,
                                          initial_state_indices=slots, output_final_state=False, auto_cp=False,
                                          raw_cu_seqlens=tuple(offs))[2][0]
    torch.cuda.synchronize()
    assert_out_close(out_p[:, hv_sel].cpu(), exp_out, "packed rows vs CPU oracle")
    assert_out_close(out_p, out, "packed rows vs separate tensors")
    assert_state_close(pool_p[slots.long()], pool[slots.long()], "packed rows vs separate tensors")


def _host_layer(layer):
    """CPU twin of a paged layer that lives on the GPU: same bytes, same strided views."""
    from types import SimpleNamespace
    raw = layer.raw.cpu()
    conv, state = layer.kv_cache
    c = raw.view(torch.bfloat16).as_strided(conv.shape, conv.stride(), conv.storage_offset())
    st = raw.view(torch.float32).as_strided(state.shape, state.stride(), state.storage_offset())
    return SimpleNamespace(raw=raw, kv_cache=(c, st), heads=layer.heads, q=layer.q, layout=layer.layout,
                           page_bytes=layer.page_bytes)


@pytest.mark.parametrize("softplus", [True, False])
def test_config2_verify_then_commit_at_full_size(native_built, softplus):
    """ReplaySSM at the benchmark size (32 heads, 64 request rows x 4 draft tokens, 512 pages; the softplus gate of
    the benchmark and the safe gate): verify's outputs and every record of every row against the fp64 oracle
    (tests/test_kda_replayssm_vllm.py:98-178 is the reference's form of this check), checkpoints and conv
    histories untouched by verify; then the commit against the oracle's plan and the oracle's fold of the ORACLE's
    records, conv histories bit-exact, other pages untouched."""
    import numpy as np

    import cases
    from oracle import replay as orep
    from pla_b200.decode.kda_replayssm_vllm import KDAReplayCommitContext, KDAReplayRecords, kda_replay_verify
    from test_kda_replay_gpu import close
    from test_oracle_replay import oracle_verify
    H, N, Q, pages = 32, 64, 4, 512
    rs = np.random.RandomState(20261125 + 2)
    layer = cases.replay_layer(rs, pages, H, Q, "SD", device="cuda")
    x = cases.replay_inputs(rs, H, N * Q, softplus=softplus, device="cuda")
    layer.replay_records = KDAReplayRecords.allocate(N, H, Q, "cuda")
    slot_list = (rs.permutation(pages - 1)[:N] + 1).astype("int32").tolist()
    offsets = list(range(0, N * Q + 1, Q))
    counts = rs.randint(1, Q + 1, N).astype("int32").tolist()
    slots = torch.tensor(slot_list, dtype=torch.int32, device="cuda")
    cu = torch.tensor(offsets, dtype=torch.int32, device="cuda")
    sampled = torch.tensor(counts, dtype=torch.int32, device="cuda")
    out = torch.empty(N * Q, H * D, dtype=torch.bfloat16, device="cuda")
    ctx = KDAReplayCommitContext.create([layer], Q, N, conv_state_layout="SD")
    old_state = layer.kv_cache[1].clone()
    old_conv = cases.conv_ds(layer).clone()
    # the fp64 oracle on the same bytes
    host_layer = _host_layer(layer)
    host_x = {k_: (v_.cpu() if isinstance(v_, torch.Tensor) else v_) for k_, v_ in x.items()}
    want_out, want = oracle_verify(host_layer, host_x, offsets, slot_list)

    kw = {k_: v_ for k_, v_ in x.items() if k_ != "storage"}
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    kda_replay_verify(**kw, conv_state=layer.kv_cache[0], checkpoint_state=layer.kv_cache[1],
                      records=layer.replay_records, query_start_loc=cu, state_indices=slots, conv_state_layout="SD",
                      out=out, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert torch.equal(layer.kv_cache[1], old_state) and torch.equal(cases.conv_ds(layer), old_conv)
    close(out, want_out, what="verify out vs fp64 oracle")
    rec = layer.replay_records
    for key, tol in (("rawv", 6e-3), ("rawk", 6e-3), ("g", 5e-6), ("beta", 5e-6)):
        close(getattr(rec, key), getattr(want, key), tol, key)
        for row in (0, 17, 63):                        # and row by row, so that one bad row cannot hide
            close(getattr(rec, key)[row], getattr(want, key)[row], tol, f"{key} row {row}")
    assert torch.equal(rec.conv.cpu(), want.conv), "conv windows must be bit-exact"

    plan = ctx.commit(sampled, slots, cu, token_capacity=N * Q)
    torch.cuda.synchronize()
    plan_l = [getattr(plan, k).tolist() for k in ("commit_lens", "final_state_indices", "boundary_state_indices",
                                                  "boundary_recovery_lens")]
    want_plan = orep.commit_plan(sampled=counts, source=slot_list, offsets=offsets, capacity=N, slots=pages, Q=Q,
                                 null_block_id=0, token_capacity=N * Q)
    assert plan_l == want_plan
    assert plan_l[0] == counts
    state, conv = orep.commit_apply(old_state.cpu(), old_conv.cpu(), want, want_plan, slot_list)
    got = layer.kv_cache[1].cpu()
    used = slots.long().cpu()
    # the device folds its own bf16 records, the oracle its own: they differ by record rounding (<= 6e-3 of a
    # record), hence the record bar here; against the fold of the DEVICE's records the bar is 5e-6
    close(got[used], state[used], 6e-3, "committed checkpoints vs oracle fold of oracle records")
    host_rec = SimpleNamespace(**{k: getattr(rec, k).cpu() for k in ("rawv", "rawk", "g", "beta", "conv")})
    state_d, conv_d = orep.commit_apply(old_state.cpu(), old_conv.cpu(), host_rec, plan_l, slot_list)
    err = ((got[used] - state_d[used]).norm() / state_d[used].norm()).item()
    assert err <= 5e-6, err
    others = torch.ones(pages, dtype=torch.bool)
    others[used] = False
    assert torch.equal(got[others], old_state.cpu()[others])
    assert torch.equal(cases.conv_ds(layer).cpu(), conv)
    assert torch.equal(conv, conv_d)


@pytest.mark.parametrize("kda", [False, True])
def test_config4_token_ranges_match_single_chains_at_full_size(native_built, kda):
    """One long sequence (GDN 64K tokens, 8 / 24 heads; KDA 128K tokens, 32 heads, weak softplus decay so that the
    transitions of the ranges matter): running it as token ranges inside the GPU gives the outputs and the final
    state of the single chain per head."""
    dev = "cuda"
    T, Hg, H = (131072, 32, 32) if kda else (65536, 8, 24)
    g = torch.Generator(device=dev).manual_seed(44)
    rn = lambda *s: torch.randn(*s, generator=g, device=dev)
    q = torch.nn.functional.normalize(rn(T, Hg, D), dim=-1).bfloat16()
    k = torch.nn.functional.normalize(rn(T, Hg, D), dim=-1).bfloat16()
    v = rn(T, H, D).bfloat16()
    gate = (rn(T, H, D) if kda else rn(T, H)).bfloat16()
    # small beta and very weak decay: erasure and decay over a whole range stay of order one, so the state entering
    # a range is still visible at its end (with the benchmark's gates it is forgotten and the two runs are bit-equal)
    beta = (rn(T, H) - (6.0 if kda else 4.0)).bfloat16()  # KDA ranges are 43K tokens long
    u = torch.rand(H, generator=g, device=dev)
    A_log = -9.0 + u
    dt_bias = rn(H, D) * 0.1 if kda else rn(H) * 0.1
    S0 = rn(1, H, D, D) * 0.5
    slot0 = torch.zeros(1, dtype=torch.int32, device=dev)
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
    res = {}
    for auto_cp in (False, True):
        pool = S0.clone()
        if kda:
            from pla_b200.prefill.flashkdapro import flashkda_fwd
            out = torch.empty(T, H, D, dtype=torch.bfloat16, device=dev)
            status = torch.zeros(1, dtype=torch.int32, device=dev)
            flashkda_fwd(q, k, v, gate, beta, A_log, dt_bias, out, None, None, state_pool=pool, state_indices=slot0,
                         raw_cu_seqlens=(0, T), backend="chunked", status=status, auto_cp=auto_cp)
            assert status.item() == 0
        else:
            from pla_b200.prefill.flashqla import ops as fq
            out = fq.chunk_gated_delta_rule_fwd(q[None], k[None], v[None], None, None, initial_state=pool,
                                                initial_state_indices=slot0, cu_seqlens=cu, output_final_state=False,
                                                auto_cp=auto_cp, normalize_qk=True, raw_cu_seqlens=(0, T),
                                                raw_gate_a=gate, raw_beta_b=beta, A_log=A_log, dt_bias=dt_bias)[2][0]
        torch.cuda.synchronize()
        res[auto_cp] = (out.float(), pool)
    assert torch.isfinite(res[True][0]).all()
    assert not torch.equal(res[True][0], res[False][0])          # the ranges really ran (different rounding)
    assert_out_close(res[True][0], res[False][0], "ranges vs single chains")
    assert_state_close(res[True][1], res[False][1], "ranges vs single chains")


@pytest.mark.parametrize("kda", [False, True])
def test_config4_benchmark_gates_against_the_cpu_oracle(native_built, kda):
    """Config 4 with the benchmark's own gates (KDA: 128K tokens, 32 heads, softplus gate with A_log ~ U(-4, -2);
    GDN: 64K tokens, 8 / 24 heads, A_log ~ U(0, log 16)): the single chain per head, the token ranges inside the
    GPU and an 8-rank split (ranks emulated one after another, the gathered pairs stacked by hand) all against the
    CPU oracle's token recurrence on a head subset -- outputs of every token and the final state."""
    from pla_b200.prefill import context_parallel as cp
    dev = "cuda"
    T, Hg, H = (131072, 32, 32) if kda else (65536, 8, 24)
    g = torch.Generator(device=dev).manual_seed(45)
    rn = lambda *s: torch.randn(*s, generator=g, device=dev)
    q = torch.nn.functional.normalize(rn(T, Hg, D), dim=-1).bfloat16()
    k = torch.nn.functional.normalize(rn(T, Hg, D), dim=-1).bfloat16()
    v = rn(T, H, D).bfloat16()
    gate = (rn(T, H, D) if kda else rn(T, H)).bfloat16()
    beta = rn(T, H).bfloat16()
    u = torch.rand(H, generator=g, device=dev)
    A_log = (-4.0 + 2.0 * u) if kda else u * math.log(16.0)
    dt_bias = rn(H, D) * 0.1 if kda else rn(H) * 0.1
    S0 = rn(1, H, D, D) * 0.02
    slot0 = torch.zeros(1, dtype=torch.int32, device=dev)
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)

    # CPU oracle on a head subset: KDA heads 5 and 17; GDN value heads 9-11 (q/k head 3)
    hv_sel, h_sel = ([5, 17], [5, 17]) if kda else ([9, 10, 11], [3])
    exp_out, exp_state, _ = odec.klast_forward(
        q=q[:, h_sel].cpu(), k=k[:, h_sel].cpu(), v=v[:, hv_sel].cpu(), a=gate[:, hv_sel].cpu(), b=beta[:, hv_sel].cpu(),
        A_log=A_log[hv_sel].cpu(), dt_bias=dt_bias[hv_sel].cpu(), state=S0[:, hv_sel].cpu().contiguous(), slot_indices=[0],
        lengths=[T], scale=D ** -0.5, is_kda=kda)

    def check(out, state, what):
        assert_out_close(out[:, hv_sel].cpu(), exp_out, f"{what}: outputs vs CPU oracle")
        assert_state_close(state[hv_sel].cpu(), exp_state[0], f"{what}: final state vs CPU oracle")

    # (1) one chain per head, (2) token ranges inside the GPU
    for auto_cp in (False, True):
        pool = S0.clone()
        if kda:
            from pla_b200.prefill.flashkdapro import flashkda_fwd
            out = torch.empty(T, H, D, dtype=torch.bfloat16, device=dev)
            status = torch.zeros(1, dtype=torch.int32, device=dev)
            flashkda_fwd(q, k, v, gate, beta, A_log, dt_bias, out, None, None, state_pool=pool, state_indices=slot0,
                         raw_cu_seqlens=(0, T), backend="chunked", status=status, auto_cp=auto_cp)
            assert status.item() == 0
        else:
            from pla_b200.prefill.flashqla import ops as fq
            out = fq.chunk_gated_delta_rule_fwd(q[None], k[None], v[None], None, None, initial_state=pool,
                                                initial_state_indices=slot0, cu_seqlens=cu, output_final_state=False,
                                                auto_cp=auto_cp, normalize_qk=True, raw_cu_seqlens=(0, T),
                                                raw_gate_a=gate, raw_beta_b=beta, A_log=A_log, dt_bias=dt_bias)[2][0]
        torch.cuda.synchronize()
        check(out, pool[0], "token ranges inside the GPU" if auto_cp else "single chain")
        del out, pool

    # (3) eight ranks, one after another
    W = 8
    per = T // W
    plans = []
    for r in range(W):
        sl = slice(r * per, (r + 1) * per)
        if kda:
            kern = cp.KdaChunkedSegmentKernels(q[sl], k[sl], v[sl], gate[sl], beta[sl], A_log, dt_bias, D ** -0.5, True, None)
        else:
            kern = cp.CudaSegmentKernels(q[sl], k[sl], v[sl], gate[sl], beta[sl], A_log, dt_bias, D ** -0.5, True, False)
        plans.append(cp.begin_segment(kern, r, W, per, H, torch.device(dev)))
    gathered = torch.stack([p.transfer for p in plans])
    outs, state = [], None
    for p in plans:
        o, state = cp.finish_segment(p, S0[0], gathered)
        outs.append(o)
        p.kernels.check()
    torch.cuda.synchronize()
    check(torch.cat(outs), state, "eight emulated ranks")
