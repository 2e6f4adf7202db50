"""Causal conv in front of the prefill ops: packed varlen rows in, packed q|k|v rows out, per-request 3-tap
history kept in the serving stack's conv cache. Call shape of the stacks' ``causal_conv1d_fn`` (the prefill
counterpart of the conv that the reference fuses into its decode step,
src/decode/k-last/fused_kda_decode_mega_kernel.cuh:36-79)."""
from __future__ import annotations

import weakref
from typing import Optional

import torch

from .._ops import ops

_weight_cache: dict = {}


def _taps_fp32(weight: torch.Tensor) -> torch.Tensor:
    """[channels, 4] fp32 copy of the taps, cached per live weight tensor and version (weights do not change while
    serving). The entry holds a weak reference to the tensor it was made from: a new tensor that happens to reuse
    the address and id of a freed one never matches."""
    if weight.dtype == torch.float32 and weight.is_contiguous():
        return weight
    hit = _weight_cache.get(id(weight))
    if hit is not None and hit[0]() is weight and hit[1] == weight._version:
        return hit[2]
    if len(_weight_cache) >= 64:
        _weight_cache.clear()
    taps = weight.float().contiguous()
    _weight_cache[id(weight)] = (weakref.ref(weight), weight._version, taps)
    return taps


def causal_conv1d_fn(
    x: torch.Tensor,                            # [tokens, channels], or the stacks' [channels, tokens] view of it
    weight: torch.Tensor,                       # [channels, 4]; tap 3 multiplies the current token
    bias: Optional[torch.Tensor] = None,        # [channels]
    conv_states: Optional[torch.Tensor] = None, # [slots, channels, 3] view in any layout (updated in place)
    query_start_loc: Optional[torch.Tensor] = None,   # [N + 1] int32
    cache_indices: Optional[torch.Tensor] = None,     # [N] int32
    has_initial_state: Optional[torch.Tensor] = None, # [N] bool
    activation: Optional[str] = "silu",
    pad_slot_id: int = -1,
    *,
    channels_first: Optional[bool] = None,
    out: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """``y_t = act(bias + h0 w0 + h1 w1 + h2 w2 + x_t w3)`` along every sequence of the packed batch; the history of a
    request is read from ``conv_states[cache_indices[n]]`` (zero when ``has_initial_state[n]`` is false or the slot is
    padding) and holds the request's last three inputs afterwards. ``pad_slot_id = -1``: negative slots are
    padding; ``pad_slot_id = 0``: slot 0 is padding as well (the null block of a paged cache). ``x`` may be the
    ``[channels, tokens]`` transposed view the serving stacks pass (detected by its unit stride, or forced with
    ``channels_first``); the result then has the same orientation. Rows past ``query_start_loc[-1]`` are zero."""
    if activation not in (None, "silu", "swish"):
        raise ValueError("activation must be None, silu or swish")
    if pad_slot_id not in (-1, 0):
        raise ValueError("pad_slot_id must be -1 or 0")
    if not x.is_cuda:
        raise ValueError("x must be a CUDA tensor")
    if x.ndim != 2 or weight.ndim != 2 or weight.size(1) != 4:
        raise ValueError("x must be 2-D and weight [channels, 4]")
    if channels_first is None:
        channels_first = x.size(0) == weight.size(0) and x.stride(0) == 1 and (x.size(1) != weight.size(0) or x.stride(1) != 1)
    rows = x.t() if channels_first else x
    if rows.size(1) != weight.size(0):
        raise ValueError("x and weight disagree on the channel count")
    if rows.size(0) > 0 and rows.stride(1) != 1:
        rows = rows.contiguous()
    T = rows.size(0)
    if query_start_loc is None:
        query_start_loc = torch.tensor([0, T], dtype=torch.int32, device=x.device)
    elif query_start_loc.dtype != torch.int32:
        query_start_loc = query_start_loc.to(torch.int32)
    if cache_indices is not None and cache_indices.dtype != torch.int32:
        cache_indices = cache_indices.to(torch.int32)
    if conv_states is not None and conv_states.ndim != 3:
        raise ValueError("conv_states must be [slots, channels, 3]")
    y_rows = None
    if out is not None:
        y_rows = out.t() if channels_first else out
    y = ops.causal_conv_prefill(rows, _taps_fp32(weight), None if bias is None else bias.float().contiguous(), conv_states,
                                query_start_loc.contiguous(), None if cache_indices is None else cache_indices.contiguous(),
                                has_initial_state, activation is not None, pad_slot_id == 0, y_rows, status)
    return y.t() if channels_first else y
