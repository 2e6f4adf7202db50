"""fp64 restatement of KDA ReplaySSM verify / commit and the integer commit plan (CPU).

Follows the reference's fp64 oracle (scripts/decode/kda_mtp_sglang/private/_reference.py:67-216)
and the plan kernels (src/decode/kda_replayssm_vllm/commit_plan.cu:18-115). Written
independently and checked against that oracle's outputs in tests/test_oracle_golden.py.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

D = 128
EPS = 1e-6


def causal_conv_silu(x: torch.Tensor, hist: torch.Tensor, w: torch.Tensor):
    """Width-4 causal conv + SiLU per channel over [hist(3) | x].

    x [T,C], hist [C,3] (oldest first), w [C,4] (tap 3 multiplies the current token).
    Returns (y [T,C], windows [T,C,3]) where windows[t] is the history AFTER token t
    (_reference.py:67-89).
    """
    T, C = x.shape
    seq = torch.cat([hist.transpose(0, 1), x], dim=0)              # [3+T, C]
    taps = torch.stack([seq[j:j + T] for j in range(4)], dim=-1)   # [T, C, 4]
    acc = (taps * w[None]).sum(-1)
    y = acc * torch.sigmoid(acc)
    windows = torch.stack([seq[1 + j:1 + j + T] for j in range(3)], dim=-1)
    return y, windows


def gate_log_decay(x, A_log, lower_bound, softplus_beta=1.0, softplus_threshold=20.0):
    eA = torch.exp(A_log)
    if lower_bound is not None:
        return float(lower_bound) * torch.sigmoid(eA * x)
    return -eA * torch.nn.functional.softplus(x, beta=softplus_beta, threshold=softplus_threshold)


def verify_request(xq, xk, xv, raw_g, raw_beta, wq, wk, wv, cq, ck, cv, A_log, dt_bias, state, scale,
                   lower_bound):
    """One request, all heads, fp64. x*: [T,H,128]; raw_g [T,H,128]; raw_beta [T,H]; w*: [H*128,4];
    c*: conv history [H*128,3]; state [H,128(V),128(K)]. Returns dict(out [T,H,128], rawk, rawv,
    g [H,T,128], beta [H,T], win_q/k/v [T,H*128,3]) (_reference.py:92-180)."""
    f = torch.float64
    T, H, _ = xq.shape
    qc, qw = causal_conv_silu(xq.reshape(T, -1).to(f), cq.to(f), wq.to(f))
    kc, kw = causal_conv_silu(xk.reshape(T, -1).to(f), ck.to(f), wk.to(f))
    vc, vw = causal_conv_silu(xv.reshape(T, -1).to(f), cv.to(f), wv.to(f))
    qc, kc, vc = (t.reshape(T, H, D) for t in (qc, kc, vc))
    qn = qc / torch.sqrt((qc * qc).sum(-1, keepdim=True) + EPS) * scale
    kn = kc / torch.sqrt((kc * kc).sum(-1, keepdim=True) + EPS)
    beta = torch.sigmoid(raw_beta.to(f))                                    # [T,H]
    g = gate_log_decay(raw_g.to(f) + dt_bias.to(f).reshape(1, H, D), A_log.to(f).reshape(1, H, 1), lower_bound)
    decay = torch.exp(g)
    S = state.to(f).clone()
    out = torch.zeros(T, H, D, dtype=f)
    for t in range(T):
        S = S * decay[t][:, None, :]
        d = torch.einsum("hvk,hk->hv", S, kn[t])
        vn = (vc[t] - d) * beta[t][:, None]
        S = S + vn[:, :, None] * kn[t][:, None, :]
        out[t] = torch.einsum("hvk,hk->hv", S, qn[t])
    return dict(out=out, rawk=kc.transpose(0, 1), rawv=vc.transpose(0, 1), g=g.transpose(0, 1),
                beta=beta.transpose(0, 1), win_q=qw, win_k=kw, win_v=vw, final_state=S)


def fold_state(state, rawk, rawv, g, beta, n: int):
    """Replay n recorded steps on state [H,V,K] in fp64 with the division-form norm of the
    RECORDED k (_reference.py:183-216). rawk/rawv/g: [H,Q,128]; beta [H,Q]."""
    f = torch.float64
    S = state.to(f).clone()
    for t in range(n):
        kk = rawk[:, t].to(f)
        kk = kk / torch.sqrt((kk * kk).sum(-1, keepdim=True) + EPS)
        S = S * torch.exp(g[:, t].to(f))[:, None, :]
        vv = (rawv[:, t].to(f) - torch.einsum("hvk,hk->hv", S, kk)) * beta[:, t].to(f)[:, None]
        S = S + vv[:, :, None] * kk[:, None, :]
    return S


def commit_plan(*, sampled: Sequence[int], source: Sequence[int], offsets: Sequence[int], capacity: int,
                slots: int, Q: int, null_block_id: int, token_capacity: int,
                mapping: Optional[Sequence[int]] = None, block_table=None, computed=None, block_size: int = 0):
    """Integer commit plan, row by row, then symmetric conflict masking
    (commit_plan.cu:18-115). Returns four lists of length ``capacity``:
    commit_len, final slot, boundary slot, boundary len."""
    N = len(source)
    INT64_MAX = (1 << 63) - 1

    def valid_slot(s):
        return s > null_block_id and 0 <= s < slots

    def valid_interval(b, e):
        return b >= 0 and e > b and e <= token_capacity and e - b <= Q

    cand = [[0] * capacity for _ in range(4)]
    for b in range(capacity):
        count = final = boundary = bc = 0
        if b < N:
            row = mapping[b] if mapping is not None else b
            src, begin, end = source[b], offsets[b], offsets[b + 1]
            if offsets[0] == 0 and 0 <= row < len(sampled) and valid_slot(src) and valid_interval(begin, end):
                s = sampled[row]
                count = 0 if s <= 0 else min(s, end - begin)
                final = src
                if count and block_size:
                    rows = len(block_table)
                    cols = len(block_table[0]) if rows else 0
                    if row >= rows:
                        count = 0
                    else:
                        pos = computed[row]
                        if pos < 0 or pos > INT64_MAX - Q:
                            count = 0
                        else:
                            col = min((pos + count - 1) // block_size, cols - 1)
                            f = block_table[row][col]
                            if not valid_slot(f):
                                count = 0
                            else:
                                final = f
                            distance = block_size - pos % block_size
                            if count and count >= distance:
                                bcol = pos // block_size
                                if bcol >= cols:
                                    count = 0
                                else:
                                    dest = block_table[row][bcol]
                                    if not valid_slot(dest) or (dest == final and distance != count):
                                        count = 0
                                    else:
                                        boundary, bc = dest, distance
        cand[0][b] = count
        cand[1][b] = final if count else 0
        cand[2][b] = boundary if count else 0
        cand[3][b] = bc if count else 0

    def wrap32(v):  # the device stores candidates as int32
        v &= 0xFFFFFFFF
        return v - (1 << 32) if v >= (1 << 31) else v

    cand = [[wrap32(v) for v in col] for col in cand]
    plan = [[0] * capacity for _ in range(4)]
    for b in range(capacity):
        conflict = False
        if cand[0][b]:
            src, f, d, has_d = source[b], cand[1][b], cand[2][b], cand[3][b] > 0
            for o in range(N):
                if o == b:
                    continue
                os_ = source[o]
                if valid_slot(os_) and valid_interval(offsets[o], offsets[o + 1]):
                    conflict |= f == os_ or (has_d and d == os_)
                if not cand[0][o]:
                    continue
                of, od, has_od = cand[1][o], cand[2][o], cand[3][o] > 0
                conflict |= (f == os_ or f == of or (has_od and f == od)
                             or (has_d and (d == os_ or d == of or (has_od and d == od)))
                             or src == of or (has_od and src == od))
        if not conflict:
            for c in range(4):
                plan[c][b] = cand[c][b]
    return plan


def commit_apply(state, conv_ds, records, plan, source, null_block_id=0):
    """Apply a plan: state [slots,H,V,K] fp32 pool and conv history viewed [slots,C,history]
    (both cloned); records with rawv/rawk/g/beta/conv per REQUEST ROW. Returns (state, conv)."""
    new_state, new_conv = state.clone(), conv_ds.clone()
    old = state.clone()
    for b, src in enumerate(source):
        n = plan[0][b]
        if n <= 0 or src <= null_block_id:
            continue
        final, boundary, bc = plan[1][b], plan[2][b], plan[3][b]
        args = (records.rawk[b], records.rawv[b], records.g[b], records.beta[b])
        if bc > 0:
            new_state[boundary] = fold_state(old[src], *args, bc).float()
            new_conv[boundary, :, :3] = records.conv[b, bc - 1]
        new_state[final] = fold_state(old[src], *args, n).float()
        new_conv[final, :, :3] = records.conv[b, n - 1]
    return new_state, new_conv


# ---- SGLang contract: rings addressed by state slot, conv windows by scratch row ----

def ring_verify(vi: dict) -> dict:
    """fused_kda_decode_mtp_dspark in fp64 over an input dict with the entry point's keyword names
    (_reference.py:92-180): returns out [1,T,H,128], the four rings and the three conv-window tensors
    as they are after the call (inputs are not modified). Requests with a slot < 0 are skipped."""
    f = torch.float64
    x_q = vi["x_q"][0]
    T, H, _ = x_q.shape
    slots = [int(s) for s in vi["ssm_state_indices"]]
    scratch = [int(s) for s in vi["intermediate_state_indices"]]
    cu = [int(c) for c in vi["cu_seqlens"]]
    out = torch.zeros(1, T, H, D, dtype=f)
    rings = {k: vi[k].to(f).clone() for k in ("replayssm_rawv", "replayssm_rawk", "replayssm_g", "replayssm_beta")}
    wins = {k: vi[k].to(f).clone() for k in ("intermediate_conv_q", "intermediate_conv_k", "intermediate_conv_v")}
    for n, slot in enumerate(slots):
        if slot < 0:
            continue
        b, e = cu[n], cu[n + 1]
        if e <= b:
            continue
        r = verify_request(vi["x_q"][0, b:e], vi["x_k"][0, b:e], vi["x_v"][0, b:e], vi["g"][0, b:e], vi["beta"][0, b:e],
                           vi["w_q"], vi["w_k"], vi["w_v"], vi["cs_q"][slot], vi["cs_k"][slot], vi["cs_v"][slot],
                           vi["A_log"], vi["dt_bias"], vi["recurrent_state"][slot], float(vi["scale"]),
                           vi["lower_bound"])
        n_tok = e - b
        out[0, b:e] = r["out"]
        rings["replayssm_rawv"][slot, :, :n_tok] = r["rawv"]
        rings["replayssm_rawk"][slot, :, :n_tok] = r["rawk"]
        rings["replayssm_g"][slot, :, :n_tok] = r["g"]
        rings["replayssm_beta"][slot, :, :n_tok] = r["beta"]
        wins["intermediate_conv_q"][scratch[n], :n_tok] = r["win_q"]
        wins["intermediate_conv_k"][scratch[n], :n_tok] = r["win_k"]
        wins["intermediate_conv_v"][scratch[n], :n_tok] = r["win_v"]
    if vi.get("onorm_gate") is not None:
        # gated RMSNorm over the value channels, from the unrounded output (_reference.py:170-175)
        gate = torch.sigmoid(vi["onorm_gate"][0].to(f))
        rms = torch.rsqrt((out[0] * out[0]).mean(-1, keepdim=True) + float(vi["onorm_eps"]))
        out = (out[0] * rms * vi["onorm_weight"].to(f)[None, None, :] * gate)[None]
    return dict(out=out, **rings, **wins)


def fold_layers(temporal, rawv, rawk, gk, beta, slot_idx, accept_lens, track_idx=None, track_step=None,
                null_block_id: int = -1):
    """commit-time exact fold for all layers (_reference.py:183-216; tracking as in
    src/decode/kda_replayssm/kda_mtp_fold.cu:470-485: the state after 0-based step track_step[b] also
    goes to slot track_idx[b]). temporal [layers,slots,HV,V,K]; rawk has H <= HV heads. Returns the
    folded copy in fp64."""
    f = torch.float64
    new = temporal.to(f).clone()
    layers, _, HV = temporal.shape[:3]
    grp = HV // rawk.shape[2]
    for l in range(layers):
        for b, slot in enumerate(int(s) for s in slot_idx):
            n = int(accept_lens[b])
            if slot <= null_block_id or n <= 0:
                continue
            kk = rawk[l, slot].repeat_interleave(grp, dim=0)
            if track_idx is not None:
                tt, ts = int(track_step[b]), int(track_idx[b])
                if 0 <= tt < n and ts > null_block_id:
                    new[l, ts] = fold_state(temporal[l, slot], kk, rawv[l, slot], gk[l, slot], beta[l, slot], tt + 1)
            new[l, slot] = fold_state(temporal[l, slot], kk, rawv[l, slot], gk[l, slot], beta[l, slot], n)
    return new


def conv_window_scatter(dst, src, dst_idx, step_idx):
    """dst[layer, dst_idx[n]] = src[layer, n, step_idx[n]] for requests with step >= 0 and a valid
    destination (src/decode/kda_replayssm/kda_mtp_fold.cu:595-618). Returns the updated copy."""
    new = dst.clone()
    for n, (d, s) in enumerate(zip((int(x) for x in dst_idx), (int(x) for x in step_idx))):
        if s < 0 or d < 0 or d >= dst.shape[1] or n >= src.shape[1] or s >= src.shape[2]:
            continue
        new[:, d] = src[:, n, s]
    return new
