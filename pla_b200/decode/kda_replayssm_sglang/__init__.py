"""KDA ReplaySSM under the SGLang contract: ``pla.decode.kda_replayssm_sglang``
(pla/decode/kda_replayssm_sglang/__init__.py:74-211).

``fused_kda_decode_mtp_dspark``   verify: conv + SiLU, safe gate, recurrence on a private copy of the
    state, outputs, ring records (addressed by state slot) and conv-window snapshots (addressed by
    scratch row); persistent recurrent / conv states are read-only; optional fused gated RMSNorm.
``commit_kda_replayssm_after_verify``   exact fold of each request's accepted ring prefix into the
    fp32 state of all layers in one launch, then the conv-state rollback.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..._ops import ops

__all__ = ["fused_kda_decode_mtp_dspark", "commit_kda_replayssm_after_verify"]

TILE_K = 128


def fused_kda_decode_mtp_dspark(
    *,
    x_q: torch.Tensor,
    x_k: torch.Tensor,
    x_v: torch.Tensor,
    w_q: torch.Tensor,
    w_k: torch.Tensor,
    w_v: torch.Tensor,
    cs_q: torch.Tensor,
    cs_k: torch.Tensor,
    cs_v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    A_log: torch.Tensor,
    dt_bias: torch.Tensor,
    recurrent_state: torch.Tensor,
    intermediate_ssm: Optional[torch.Tensor] = None,
    intermediate_state_indices: torch.Tensor,
    intermediate_conv_q: torch.Tensor,
    intermediate_conv_k: torch.Tensor,
    intermediate_conv_v: torch.Tensor,
    ssm_state_indices: torch.Tensor,
    cu_seqlens: torch.Tensor,
    lower_bound: Optional[float],
    scale: Optional[float] = None,
    replayssm_rawv: Optional[torch.Tensor] = None,
    replayssm_rawk: Optional[torch.Tensor] = None,
    replayssm_g: Optional[torch.Tensor] = None,
    replayssm_beta: Optional[torch.Tensor] = None,
    onorm_gate: Optional[torch.Tensor] = None,
    onorm_weight: Optional[torch.Tensor] = None,
    onorm_eps: Optional[float] = None,
    out: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """KDA verify, ring-cache mode. Keyword-only like SGLang's entry point; returns ``out``
    (allocated when not supplied). All four ``replayssm_*`` rings are required; ``intermediate_ssm``
    is not consumed. Passing all three ``onorm_*`` arguments fuses
    ``out = o * rsqrt(mean(o**2) + onorm_eps) * onorm_weight * sigmoid(onorm_gate)`` computed from the
    fp32 attention output. ``lower_bound=None`` (not in the reference, which requires the safe gate)
    selects the softplus gate. ``status`` (int32[1], not in the reference) receives device-detected
    errors."""
    records = {"replayssm_rawv": replayssm_rawv, "replayssm_rawk": replayssm_rawk, "replayssm_g": replayssm_g,
               "replayssm_beta": replayssm_beta}
    absent = [name for name, ring in records.items() if ring is None]
    if absent:
        raise ValueError("the verify step records into the four replay rings (ring-cache mode is the only one built); "
                         f"missing: {', '.join(absent)}")
    gate, weight, eps = _output_norm(onorm_gate, onorm_weight, onorm_eps)
    result = out if out is not None else torch.empty_like(x_v, memory_format=torch.contiguous_format)
    ops.kda_ring_verify(
        x_q, x_k, x_v, g, beta, w_q.contiguous(), w_k.contiguous(), w_v.contiguous(), cs_q, cs_k, cs_v,
        A_log.contiguous(), dt_bias.contiguous(), recurrent_state, result,
        intermediate_conv_q, intermediate_conv_k, intermediate_conv_v,
        records["replayssm_rawv"], records["replayssm_rawk"], records["replayssm_g"], records["replayssm_beta"],
        ssm_state_indices, intermediate_state_indices, cu_seqlens, float(TILE_K ** -0.5 if scale is None else scale),
        None if lower_bound is None else float(lower_bound), gate, weight, eps, status)
    return result


def _output_norm(gate, weight, eps):
    """The fused output norm takes its three arguments together or not at all."""
    given = [value is not None for value in (gate, weight, eps)]
    if not any(given):
        return None, None, None
    if not all(given):
        raise ValueError("the fused output norm needs onorm_gate, onorm_weight and onorm_eps together")
    return gate, weight, float(eps)


def commit_kda_replayssm_after_verify(
    *,
    spec_state,
    state_batch_indices: torch.Tensor,
    accept_lens: torch.Tensor,
    last_correct_step_indices: torch.Tensor,
    mamba_track_indices: Optional[torch.Tensor] = None,
    mamba_steps_to_track: Optional[torch.Tensor] = None,
    null_block_id: int = -1,
    conv_state_layout: str = "dim_width",
    status: Optional[torch.Tensor] = None,
) -> None:
    """Fold each layer's accepted window into ``spec_state.temporal`` and roll the conv state back.

    ``spec_state`` carries ``temporal [layers, slots, HV, 128, 128]``, ``replayssm_rawv/rawk/g/beta``,
    and the lists ``conv`` / ``intermediate_conv_window``. ``conv_state_layout="width_dim"`` takes
    conv pools ``[layers, slots, width, dim]`` and scratch through transpose views."""
    layouts = {"dim_width": False, "width_dim": True}
    if conv_state_layout not in layouts:
        raise AssertionError(f"conv_state_layout is one of {sorted(layouts)}, got {conv_state_layout!r}")
    pools, windows = list(spec_state.conv), list(spec_state.intermediate_conv_window)
    if len(pools) != len(windows):
        raise AssertionError(f"{len(pools)} conv pools but {len(windows)} conv-window scratch tensors")
    ops.kda_fold_all_layers(
        spec_state.temporal, spec_state.replayssm_rawv, spec_state.replayssm_rawk, spec_state.replayssm_g,
        spec_state.replayssm_beta, state_batch_indices, accept_lens, mamba_track_indices, mamba_steps_to_track,
        int(spec_state.replayssm_rawk.shape[2]), int(null_block_id), status)
    # conv rollback: the window after the last accepted step goes to the request's slot, and the window after the
    # tracked step to the tracking slot when tracking is on
    targets = [(state_batch_indices, last_correct_step_indices)]
    if mamba_track_indices is not None and mamba_steps_to_track is not None:
        targets.append((mamba_track_indices, mamba_steps_to_track))
    width_major = layouts[conv_state_layout]
    for pool, window in zip(pools, windows):
        if width_major:     # [.., width, dim] pools: the op addresses [.., dim, width] through transposed views
            pool, window = pool.transpose(-1, -2), window.transpose(-1, -2)
        for slots, steps in targets:
            ops.kda_conv_window_scatter(pool, window, slots, steps)
