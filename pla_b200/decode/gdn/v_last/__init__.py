"""v-last GDN decode — the surface of ``pla.decode.gdn.v_last``
(pla/decode/gdn/v_last/__init__.py:43-132)."""
from __future__ import annotations

from typing import Optional

import torch

from ...._ops import ops

__all__ = ["fused_sigmoid_gating_delta_rule", "fused_sigmoid_gating_delta_rule_forward"]


def fused_sigmoid_gating_delta_rule_forward(
    A_log, a, dt_bias, softplus_beta, softplus_threshold, q, k, v, b, h0_source, o, h0_indices,
    cu_seqlens, scale, T, B, H, HV, K, V, use_initial_state, use_qk_l2norm_in_kernel, is_varlen,
    *, status: Optional[torch.Tensor] = None,
) -> None:
    """Positional twin of the reference's ``_C.fused_sigmoid_gating_delta_rule_forward``; writes ``o`` and the pool."""
    ops.decode_v_last(
        A_log, a, dt_bias, float(softplus_beta), float(softplus_threshold), q, k, v, b, h0_source, o,
        h0_indices, cu_seqlens, float(scale), int(T), int(B), int(H), int(HV), int(K), int(V),
        bool(use_initial_state), bool(use_qk_l2norm_in_kernel), bool(is_varlen), status)


def fused_sigmoid_gating_delta_rule(
    A_log: torch.Tensor,
    a: torch.Tensor,
    dt_bias: torch.Tensor,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    b: torch.Tensor,
    o: torch.Tensor,
    h0_source: torch.Tensor,
    h0_indices: Optional[torch.Tensor] = None,
    cu_seqlens: Optional[torch.Tensor] = None,
    softplus_beta: float = 1.0,
    softplus_threshold: float = 20.0,
    scale: float = 1.0,
    T: int = 1,
    B: int = 1,
    H: int = 1,
    HV: int = 1,
    K: int = 1,
    V: int = 1,
    use_initial_state: bool = False,
    use_qk_l2norm_in_kernel: bool = False,
    is_varlen: bool = False,
) -> torch.Tensor:
    """Forward-only functional wrapper; returns ``o``."""
    fused_sigmoid_gating_delta_rule_forward(
        A_log, a, dt_bias, softplus_beta, softplus_threshold, q, k, v, b, h0_source, o, h0_indices,
        cu_seqlens, scale, T, B, H, HV, K, V, use_initial_state, use_qk_l2norm_in_kernel, is_varlen)
    return o
