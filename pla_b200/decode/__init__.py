"""k-last GDN / KDA decode — the surface of ``pla.decode`` (pla/decode/__init__.py:63-96).

Both functions keep the reference's positional order
(src/decode/k-last/fused_sigmoid_gating.cpp:164-203).
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from .._ops import ops
from ..caselist import show_call

__all__ = [
    "fused_sigmoid_gating_delta_rule_forward_k_last",
    "fused_sigmoid_gating_delta_rule_forward_k_last_packed",
]


def fused_sigmoid_gating_delta_rule_forward_k_last(
    A_log: torch.Tensor,
    a: torch.Tensor,
    dt_bias: torch.Tensor,
    softplus_beta: float,
    softplus_threshold: float,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    b: torch.Tensor,
    initial_state_source: Optional[torch.Tensor],
    initial_state_indices: Optional[torch.Tensor],
    scale: Optional[float],
    use_qk_l2norm_in_kernel: bool,
    cu_seqlens: Optional[torch.Tensor],
    is_kda: bool,
    disable_state_update: bool,
    intermediate_states_buffer: Optional[torch.Tensor],
    intermediate_state_indices: Optional[torch.Tensor],
    cache_steps_or_num_accept: Union[None, int, torch.Tensor],
    retrieve_parent_token: Optional[torch.Tensor],
    lower_bound: Optional[float] = None,
    is_sglang: Optional[bool] = None,
    out: Optional[torch.Tensor] = None,
    *,
    status: Optional[torch.Tensor] = None,
    rows_per_cta: int = 0,
) -> torch.Tensor:
    """GDN/KDA decode and single-chain / tree MTP verify on a k-last state pool.

    Returns ``out`` (allocated with ``v``'s shape when not supplied) and updates
    the pool in place unless ``disable_state_update``. ``status`` (int32[1],
    keyword-only, not in the reference) receives device-detected metadata errors
    instead of a trap.
    """
    if initial_state_source is None or initial_state_indices is None:
        raise RuntimeError("initial_state_source and initial_state_indices are required")
    if not (q.dim() == 4 and k.dim() == 4 and v.dim() == 4):
        raise RuntimeError("q, k, v must have shape [B, T, heads, dim]")
    cache_steps = None
    num_accepted = None
    if isinstance(cache_steps_or_num_accept, torch.Tensor):
        num_accepted = cache_steps_or_num_accept
    elif cache_steps_or_num_accept is not None:
        cache_steps = int(cache_steps_or_num_accept)
    if scale is None:
        scale = float(k.shape[-1]) ** -0.5
    if out is None:
        out = torch.empty(v.shape, dtype=v.dtype, device=v.device)
    elif out.shape != v.shape or out.dtype != v.dtype:
        raise RuntimeError("out must match v in shape and dtype")
    show_call(q, v, bool(is_kda), cu_seqlens, lower_bound=lower_bound)
    ops.decode_k_last(
        A_log, a, dt_bias, float(softplus_beta), float(softplus_threshold), q, k, v, b,
        initial_state_source, initial_state_indices, float(scale), bool(use_qk_l2norm_in_kernel),
        cu_seqlens, bool(is_kda), bool(disable_state_update), intermediate_states_buffer,
        intermediate_state_indices, cache_steps, num_accepted, retrieve_parent_token,
        None if lower_bound is None else float(lower_bound),
        True if is_sglang is None else bool(is_sglang), out, status, int(rows_per_cta))
    return out


def fused_sigmoid_gating_delta_rule_forward_k_last_packed(
    mixed_qkv: torch.Tensor,
    a: torch.Tensor,
    b: torch.Tensor,
    A_log: torch.Tensor,
    dt_bias: torch.Tensor,
    softplus_beta: float,
    softplus_threshold: float,
    scale: float,
    initial_state_source: torch.Tensor,
    initial_state_indices: torch.Tensor,
    out: torch.Tensor,
    use_qk_l2norm_in_kernel: bool,
    cu_seqlens: Optional[torch.Tensor],
    is_kda: bool,
    is_sglang: Optional[bool] = None,
    *,
    status: Optional[torch.Tensor] = None,
    rows_per_cta: int = 0,
) -> torch.Tensor:
    """One token per request, q|k|v read from one ``mixed_qkv`` row; returns ``out``."""
    ops.decode_k_last_packed(
        mixed_qkv, a, b, A_log, dt_bias, float(softplus_beta), float(softplus_threshold), float(scale),
        initial_state_source, initial_state_indices, out, bool(use_qk_l2norm_in_kernel), cu_seqlens,
        bool(is_kda), True if is_sglang is None else bool(is_sglang), status, int(rows_per_cta))
    return out
