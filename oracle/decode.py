"""fp32 token-by-token delta-rule recurrence on slot-indexed state pools (CPU, torch).

Restates the behaviour of ``reference()`` in the reference's
tests/test_k_last_state_dtype.py:108-155 (k-last GDN/KDA decode, chain and
tree MTP, SGLang / vLLM padding conventions) and, for the vLLM 2-D slot table,
the kernel's own rules (src/decode/k-last/fused_sigmoid_gating_k_last_kernel.cuh:218-225,
:850-863, :1049-1054). Written independently; checked against that function's
outputs in tests/test_oracle_golden.py.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn.functional as F


def log_decay(x: torch.Tensor, A_log: torch.Tensor, lower_bound: Optional[float],
              softplus_beta: float = 1.0, softplus_threshold: float = 20.0) -> torch.Tensor:
    """log of the per-step decay factor (src/pla_device_helpers.cuh:215-246).

    softplus form: -exp(A_log) * softplus(x); safe form: lower_bound * sigmoid(exp(A_log) * x).
    ``A_log`` must already broadcast against ``x``.
    """
    eA = A_log.float().exp()
    if lower_bound is not None:
        return float(lower_bound) * torch.sigmoid(eA * x)
    return -eA * F.softplus(x, beta=softplus_beta, threshold=softplus_threshold)


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """x * rsqrt(sum x^2 + eps) over the last axis (k-last kernel :455-470)."""
    return x * torch.rsqrt(x.square().sum(-1, keepdim=True) + eps)


def step(S: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
         gamma: torch.Tensor, beta: torch.Tensor):
    """One delta-rule step on S[HV, V, K] (k-last kernel :561-605).

    q,k: [HV,K] (already normalised / scaled), v: [HV,V], gamma: [HV,1] or [HV,K], beta: [HV].
    Returns (S_new, o[HV,V]).
    """
    S = S * gamma[:, None, :]
    delta = torch.einsum("hvk,hk->hv", S, k)
    vn = (v - delta) * beta[:, None]
    S = S + vn[:, :, None] * k[:, None, :]
    o = torch.einsum("hvk,hk->hv", S, q)
    return S, o


def klast_forward(
    *, q, k, v, a, b, A_log, dt_bias, state, slot_indices, lengths: Sequence[int],
    scale: float, use_qk_l2norm: bool = True, is_kda: bool = False,
    lower_bound: Optional[float] = None, softplus_beta: float = 1.0, softplus_threshold: float = 20.0,
    is_sglang: bool = True, disable_state_update: bool = False,
    cache: Optional[torch.Tensor] = None, cache_indices: Optional[Sequence[int]] = None,
    parents: Optional[torch.Tensor] = None, num_accepted: Optional[Sequence[int]] = None,
):
    """k-last decode / verify over packed tokens.

    q,k: [tokens,H,128]; v: [tokens,HV,128]; a: [tokens,HV] or [tokens,HV,128]; b: [tokens,HV];
    state: [slots,HV,128(V),128(K)] (a strided view is fine); slot_indices: [N] or [N,S] ints.
    Returns (out[tokens,HV,128] in v's dtype, new_state (clone), new_cache (clone or None)).
    """
    qf, kf, vf = q.float(), k.float(), v.float()
    if use_qk_l2norm:
        qf, kf = l2norm(qf), l2norm(kf)
    qf = qf * scale
    HV, H = v.shape[1], q.shape[1]
    rep = HV // H
    qf = qf.repeat_interleave(rep, dim=1)
    kf = kf.repeat_interleave(rep, dim=1)
    x = a.float().reshape(a.shape[0], HV, -1) + dt_bias.float().reshape(1, HV, -1)
    gamma = log_decay(x, A_log.float().reshape(1, HV, 1), lower_bound, softplus_beta, softplus_threshold).exp()
    beta = torch.sigmoid(b.float())
    new_state = state.clone()
    new_cache = None if cache is None else cache.clone()
    out = torch.zeros_like(vf)
    slots = torch.as_tensor(slot_indices)
    table2d = slots.dim() == 2
    bos = 0
    for n, T in enumerate(lengths):
        if T == 0:
            continue
        if table2d:
            acc = 1 if num_accepted is None else int(num_accepted[n])
            slot = int(slots[n, max(acc, 1) - 1])
        else:
            slot = int(slots[n])
        pad = slot < 0 if is_sglang else slot <= 0
        if pad:
            bos += T
            continue
        S = new_state[slot].float()
        for t in range(T):
            if parents is not None and t > 0 and new_cache is not None:
                par = int(parents[n, t])
                if 0 <= par != t - 1:
                    S = new_cache[int(cache_indices[n]), par].float()
            i = bos + t
            S, o = step(S, qf[i], kf[i], vf[i], gamma[i], beta[i])
            out[i] = o
            if is_sglang:
                if new_cache is not None and int(cache_indices[n]) >= 0:
                    new_cache[int(cache_indices[n]), t] = S.to(new_cache.dtype)
            elif table2d:
                ss = int(slots[n, t])
                if ss > 0:
                    new_state[ss] = S.to(new_state.dtype)
        if not disable_state_update:
            new_state[slot] = S.to(new_state.dtype)
        bos += T
    return out.to(v.dtype), new_state, new_cache


def vlast_forward(*, q, k, v, a, b, A_log, dt_bias, state, slot_indices, scale: float,
                  use_qk_l2norm: bool = True, softplus_beta: float = 1.0, softplus_threshold: float = 20.0,
                  out_init: Optional[torch.Tensor] = None):
    """v-last GDN decode, one token per request: the k-last recurrence on the
    transposed pool [slots,HV,K,V]; a slot < 0 leaves the request's output row as it was
    (src/decode/v-last/fused_sigmoid_gating_bigbatch_kernel.cuh:452-460).
    """
    B = q.shape[0]
    out, st, _ = klast_forward(
        q=q, k=k, v=v, a=a, b=b, A_log=A_log, dt_bias=dt_bias, state=state.transpose(-1, -2),
        slot_indices=slot_indices, lengths=[1] * B, scale=scale, use_qk_l2norm=use_qk_l2norm,
        softplus_beta=softplus_beta, softplus_threshold=softplus_threshold, is_sglang=True)
    if out_init is not None:
        keep = torch.as_tensor(slot_indices)[:B] < 0
        out[keep] = out_init[keep]
    return out, st.transpose(-1, -2).contiguous()


def kda_mega_forward(*, x, weight, bias, conv_state, raw_g, raw_beta, A_log, dt_bias, state_indices, state,
                     lower_bound: Optional[float], output_gate=None, norm_weight=None, norm_eps: float = 1e-5):
    """Fused KDA decode step in fp32 (scripts/decode/kda_fusion/compare_kda_decode_fusion.py:252-308):
    width-4 causal conv + SiLU over the packed q|k|v row with the 3-tap history shifted, L2 norms
    (q scaled by 128^-0.5), per-channel decay (safe gate when ``lower_bound`` is given, softplus otherwise),
    one delta-rule step per head on the k-last state, optional gated RMSNorm of the output.

    x [B, 3*H*128]; weight [3, 4, H*128]; conv_state [slots, 3*H*128, 3]; raw_g [1, B, H, 128];
    raw_beta [1, B, H]; state [slots, H, 128(V), 128(K)]; output_gate [B, H, 128].
    Rows with a negative slot give zeros and change nothing.
    Returns (out [B, H, 128] fp32, new_state, new_conv_state in conv_state's dtype)."""
    B, dim3 = x.shape
    dim = dim3 // 3
    H = dim // 128
    new_state = state.clone().float()
    new_conv = conv_state.clone()
    out = torch.zeros(B, H, 128)
    w = weight.float()                                       # [3, 4, dim]
    for b in range(B):
        slot = int(state_indices[b])
        if slot < 0:
            continue
        taps = new_conv[slot].float()                        # [3*dim, 3]
        xn = x[b].float()
        window = torch.cat([taps, xn[:, None]], dim=1)       # [3*dim, 4]
        wflat = w.permute(0, 2, 1).reshape(3 * dim, 4)       # [3*dim, 4]
        acc = (window * wflat).sum(-1)
        if bias is not None:
            acc = acc + bias.float()
        mixed = acc * torch.sigmoid(acc)
        new_conv[slot] = torch.cat([new_conv[slot][:, 1:], x[b][:, None].to(new_conv.dtype)], dim=1)
        q, k, v = (mixed[i * dim:(i + 1) * dim].view(H, 128) for i in range(3))
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * 128 ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        g = log_decay(raw_g[0, b].float() + dt_bias.float().view(H, 128), A_log.float().view(H, 1), lower_bound)
        S, o = step(new_state[slot], q, k, v, g.exp(), torch.sigmoid(raw_beta[0, b].float()))
        new_state[slot] = S
        if output_gate is not None:
            rstd = torch.rsqrt((o * o).mean(-1, keepdim=True) + norm_eps)
            o = o * rstd * norm_weight.float()[None, :] * torch.sigmoid(output_gate.reshape(B, H, 128)[b].float())
        out[b] = o
    return out, new_state, new_conv
