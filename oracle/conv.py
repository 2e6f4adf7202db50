"""CPU restatement of the width-4 causal conv (+ SiLU) over packed varlen token rows with a 3-tap history per
request: the step in front of the prefill ops that produces their packed q|k|v rows.

TEST INFRASTRUCTURE ONLY (see the package docstring). The per-token arithmetic is the reference's
``_causal_conv_silu`` (scripts/decode/kda_mtp_sglang/private/_reference.py:67-89) applied to every sequence of the
batch; the history convention (three inputs, oldest first, shifted on every token) is the one of its fused decode
step (src/decode/k-last/fused_kda_decode_mega_kernel.cuh:36-79). Pinned by ``tests/golden/conv_*.npz``, which hold
the outputs of that reference function on the cases of ``tests/golden/cases.py``.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch


def causal_conv_prefill(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                        conv_state: Optional[torch.Tensor], offsets: Sequence[int],
                        state_indices: Optional[Sequence[int]] = None,
                        has_initial_state: Optional[Sequence[bool]] = None, silu: bool = True,
                        vllm_pad: bool = False):
    """x [rows, C]; weight [C, 4] (tap 3 multiplies the current token); conv_state [slots, C, 3] or None.
    Returns (y [rows, C] in x's dtype with rows at or past offsets[-1] zero, conv_state after the call).
    A padding slot (< 0, or <= 0 under the vLLM convention) reads a zero history and keeps none."""
    rows, C = x.shape
    y = torch.zeros(rows, C, dtype=x.dtype)
    new_state = None if conv_state is None else conv_state.clone()
    w = weight.double()
    for s, (beg, end) in enumerate(zip(offsets, offsets[1:])):
        n = int(end) - int(beg)
        if n <= 0:
            continue
        slot = s if state_indices is None else int(state_indices[s])
        pad = conv_state is None or (slot <= 0 if vllm_pad else slot < 0)
        reads = not pad and (has_initial_state is None or bool(has_initial_state[s]))
        hist = conv_state[slot].double() if reads else torch.zeros(C, 3, dtype=torch.float64)
        seq = torch.cat([hist.transpose(0, 1), x[beg:end].double()], dim=0)          # [3 + n, C]
        acc = sum(seq[j:j + n] * w[:, j] for j in range(4))
        if bias is not None:
            acc = acc + bias.double()
        y[beg:end] = (acc * torch.sigmoid(acc) if silu else acc).to(x.dtype)
        if not pad:
            new_state[slot] = seq[n:n + 3].transpose(0, 1).to(conv_state.dtype)
    return y, new_state
