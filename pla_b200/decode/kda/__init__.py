"""KDA decode entry points of ``pla.decode.kda`` (pla/decode/kda/__init__.py).

``fused_recurrent_kda`` keeps vLLM's signature plus the trailing ``is_sglang`` switch
(src/decode/k-last/fused_recurrent_kda.cpp:146-161) and the reference's exception types:
``ValueError`` / ``NotImplementedError`` for argument validation (:88-96).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..._ops import ops
from ...caselist import show_call

__all__ = ["fused_recurrent_kda", "fused_kda_decode_mega_forward"]


def fused_recurrent_kda(
    q: torch.Tensor,                       # [1, T, H, K]
    k: torch.Tensor,                       # [1, T, H, K]
    v: torch.Tensor,                       # [1, T, H, V]
    raw_g: torch.Tensor,                   # [1, T, H, K] raw gate projection
    raw_beta: torch.Tensor,                # [1, T, H] raw beta logits
    A_log: torch.Tensor,                   # [H]
    dt_bias: Optional[torch.Tensor],       # [H, K] or [H*K], fp32
    lower_bound: Optional[float],          # safe-gate lower bound; None = softplus gate
    initial_state: torch.Tensor,           # [slots, H, V, K] fp32 k-last pool, updated in place
    cu_seqlens: torch.Tensor,              # [N+1]
    ssm_state_indices: torch.Tensor,       # [N] or [N, S] (one slot per draft token)
    num_accepted_tokens: Optional[torch.Tensor] = None,   # [N], with a 2-D table
    out: Optional[torch.Tensor] = None,    # [1, T, H, V] to fill
    fuse_gate: Optional[bool] = None,      # must be true / unset
    is_sglang: bool = False,
    *,
    status: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Recurrent KDA from raw gate / beta inputs. Returns ``(out, initial_state)``: the returned state
    is the pool that was updated in place. Pad slots (``< 0`` for SGLang, ``<= 0`` for vLLM) give zero
    output rows and leave the pool alone. ``status`` (int32[1], keyword-only, not in the reference)
    receives device-detected metadata errors."""
    if fuse_gate is not None and not fuse_gate:
        raise NotImplementedError(
            "pla.decode.kda.fused_recurrent_kda only implements the fused-gate path (fuse_gate=True): pass the raw "
            "gate projection plus A_log/dt_bias and drop the separate gate call.")
    if dt_bias is None:
        raise ValueError("dt_bias is required by the fused-gate kernel path.")
    if q.dim() != 4:
        raise ValueError(f"q must be packed as [1, T, H, K], got {q.dim()}D.")
    if q.shape[0] != 1:
        raise ValueError(f"q must be packed as [1, T, H, K], got batch {q.shape[0]}.")
    K, V = q.shape[3], v.shape[-1]
    if K != 128 or V != 128:
        raise NotImplementedError(
            f"pla.decode.kda.fused_recurrent_kda requires head_dim K == V == 128, got K={K}, V={V}.")
    if initial_state.dtype != torch.float32:
        raise ValueError(f"initial_state must be float32, got {initial_state.dtype}.")
    if ssm_state_indices.dim() not in (1, 2):
        raise ValueError(f"ssm_state_indices must be 1D or 2D, got {ssm_state_indices.dim()}D")
    if ssm_state_indices.dim() == 2 and is_sglang:
        raise ValueError("a 2D ssm_state_indices is the vLLM spec-decode layout; sglang uses a 1D table plus its "
                         "own intermediate-state buffer.")
    if dt_bias.dtype != torch.float32:
        raise ValueError(f"dt_bias must be float32, got {dt_bias.dtype}.")
    if out is None:
        out = torch.empty(v.shape, dtype=v.dtype, device=v.device)
    elif out.shape != v.shape or out.dtype != v.dtype:
        raise ValueError("out must match v in shape and dtype")
    show_call(q, v, True, cu_seqlens, lower_bound=lower_bound)
    ops.fused_recurrent_kda(q, k, v, raw_g, raw_beta, A_log, dt_bias,
                            None if lower_bound is None else float(lower_bound), initial_state, cu_seqlens,
                            ssm_state_indices, num_accepted_tokens, out, bool(is_sglang), status)
    return out, initial_state


def fused_kda_decode_mega_forward(
    x: torch.Tensor,                        # [B, 3*H*128] fp16/bf16, channel-contiguous packed q|k|v projections
    weight: torch.Tensor,                   # fp32 [3, 4, H*128]: segment, tap (3 = current token), channel
    bias: Optional[torch.Tensor] = None,    # fp32 [3*H*128]
    conv_state: torch.Tensor = None,        # activation dtype [slots, 3*H*128, 3], shifted in place
    raw_g: torch.Tensor = None,             # [1, B, H, 128]
    raw_beta: torch.Tensor = None,          # [1, B, H]
    a_log: torch.Tensor = None,             # fp32 [H]
    dt_bias: torch.Tensor = None,           # fp32 [H, 128]
    state_indices: torch.Tensor = None,     # int32 [B]; < 0 = padding row
    state: torch.Tensor = None,             # fp32 [slots, H, 128, 128], updated in place
    out: torch.Tensor = None,               # activation dtype [1, B, H, 128], written
    lower_bound: Optional[float] = None,    # safe gate when given, softplus gate otherwise
    output_gate: Optional[torch.Tensor] = None,   # [B, H, 128] or [1, B, H, 128]
    norm_weight: Optional[torch.Tensor] = None,   # fp32 [128]
    norm_eps: float = 1e-5,
    *,
    status: Optional[torch.Tensor] = None,
) -> None:
    """Kimi K3 fused decode step (docs/readme.md:232-267 of the reference): causal conv + SiLU, gating,
    single-token KDA recurrence and optional gated output RMSNorm; writes ``conv_state``, ``state`` and
    ``out`` in place and returns ``None``. ``output_gate`` and ``norm_weight`` come together. Rows whose
    slot is negative produce a zero output row and touch nothing; slot 0 is an ordinary slot."""
    for name, t in (("conv_state", conv_state), ("raw_g", raw_g), ("raw_beta", raw_beta), ("a_log", a_log),
                    ("dt_bias", dt_bias), ("state_indices", state_indices), ("state", state), ("out", out)):
        if t is None:
            raise TypeError(f"fused_kda_decode_mega_forward() missing required argument: '{name}'")
    ops.kda_decode_mega(x, weight, bias, conv_state, raw_g, raw_beta, a_log, dt_bias, state_indices, state, out,
                        None if lower_bound is None else float(lower_bound), output_gate, norm_weight,
                        float(norm_eps), status)
    return None
