"""Request-row KDA replay for a vLLM-style runner — the surface of
``pla.decode.kda_replayssm_vllm`` (pla/decode/kda_replayssm_vllm/__init__.py:20-234).

verify reads a paged FP32 checkpoint read-only and logs replay records; after the
sampler has run, ``KDAReplayCommitContext.commit`` builds the integer commit plan on
the device, folds the accepted prefix into the checkpoints of every layer and
scatters the matching conv windows. Verify and commit must use the same records.
"""
from __future__ import annotations

from dataclasses import dataclass
from numbers import Integral, Real
from typing import Optional

import numpy as np
import torch

from ..._ops import ops

__all__ = ["KDAReplayRecords", "KDAReplayCommitPlan", "KDAReplayCommitContext", "kda_replay_verify"]


@dataclass(frozen=True)
class KDAReplayRecords:
    """Per-layer replay log: post-conv pre-norm v/k (bf16), log-decay g and beta (fp32), and the
    3-tap conv window after each token (bf16)."""
    rawv: torch.Tensor
    rawk: torch.Tensor
    g: torch.Tensor
    beta: torch.Tensor
    conv: torch.Tensor

    @classmethod
    def allocate(cls, max_num_reqs, num_heads, spec_query_len, device):
        if max_num_reqs < 0 or num_heads < 1 or not 1 <= spec_query_len <= 32:
            raise ValueError("records require R >= 0, H > 0 and Q in [1, 32]")
        shape = (max_num_reqs, num_heads, spec_query_len, 128)
        return cls(torch.empty(shape, dtype=torch.bfloat16, device=device),
                   torch.empty(shape, dtype=torch.bfloat16, device=device),
                   torch.empty(shape, dtype=torch.float32, device=device),
                   torch.empty(shape[:-1], dtype=torch.float32, device=device),
                   torch.empty((max_num_reqs, spec_query_len, 3 * num_heads * 128, 3),
                               dtype=torch.bfloat16, device=device))


def kda_replay_verify(*, mixed_qkv, raw_g, raw_beta, conv_weight, conv_state, checkpoint_state, A_log, dt_bias,
                      lower_bound, records, query_start_loc, state_indices, conv_state_layout,
                      out: Optional[torch.Tensor] = None, scale=None, null_block_id=0,
                      status: Optional[torch.Tensor] = None):
    """Verify a speculative window against a paged checkpoint.

    Writes ``out`` (bf16 ``[T, H*128]``; allocated when ``None``) on real query intervals only and
    the replay records of active rows; persistent conv history and checkpoints stay untouched.
    ``lower_bound`` a negative float selects the safe gate ``lower_bound * sigmoid(exp(A_log) * x)``;
    ``None`` (an extension over the reference, which requires a float) selects
    ``-exp(A_log) * softplus(x)``.
    """
    if lower_bound is not None and not isinstance(lower_bound, Real):
        raise TypeError("scale and lower_bound must be host numeric scalars")
    if scale is not None and not isinstance(scale, Real):
        raise TypeError("scale and lower_bound must be host numeric scalars")
    if not isinstance(null_block_id, Integral):
        raise TypeError("null_block_id must be a host integer")
    if out is None:
        out = torch.empty((mixed_qkv.shape[0], checkpoint_state.shape[1] * 128), dtype=torch.bfloat16,
                          device=mixed_qkv.device)
    ops.kda_replay_verify(mixed_qkv, raw_g, raw_beta, conv_weight, conv_state, checkpoint_state, A_log, dt_bias, out,
                          records.rawv, records.rawk, records.g, records.beta, records.conv, query_start_loc,
                          state_indices, conv_state_layout, 128 ** -0.5 if scale is None else float(scale),
                          None if lower_bound is None else float(lower_bound), int(null_block_id), status)
    return out


@dataclass(frozen=True)
class KDAReplayCommitPlan:
    commit_lens: torch.Tensor
    final_state_indices: torch.Tensor
    boundary_state_indices: torch.Tensor
    boundary_recovery_lens: torch.Tensor


def _write_spans(conv, state, layout):
    """Byte intervals [begin, end) that a commit may write for one layer: one interval per state
    page and one per conv page (the bounding span of the first three history items of every
    channel)."""
    item = state.element_size()
    s0 = state.data_ptr() + np.arange(state.size(0), dtype=np.int64) * (state.stride(0) * item)
    s1 = s0 + (state.numel() // state.size(0)) * item
    ds = conv if layout == "DS" else conv.transpose(1, 2)
    ci = conv.element_size()
    extent = ((ds.size(1) - 1) * ds.stride(1) + 2 * ds.stride(2) + 1) * ci
    c0 = ds.data_ptr() + np.arange(ds.size(0), dtype=np.int64) * (ds.stride(0) * ci)
    c1 = c0 + extent
    return np.concatenate([s0, c0]), np.concatenate([s1, c1])


def _spans_overlap(a, b):
    (a0, a1), (b0, b1) = a, b
    order = np.argsort(b0)
    b0, b1 = b0[order], b1[order]
    bmax = np.maximum.accumulate(b1)
    # for every interval of a: the last interval of b that starts before a ends
    pos = np.searchsorted(b0, a1, side="left") - 1
    ok = pos >= 0
    return bool(np.any(bmax[np.clip(pos, 0, None)][ok] > a0[ok]))


class KDAReplayCommitContext:
    """Owns the immutable per-layer pointer table and the reusable device plan buffers.

    Create it outside graph capture and keep cache and record tensors in place for its lifetime;
    writable cache regions of different layers must be disjoint. Commits, reads of the returned
    plan and graph replays captured with one context must be serialised on one stream (the next
    commit overwrites the plan). The plan has ``max_num_reqs`` entries, zeros in unused ones.
    """

    @classmethod
    def create(cls, layers, spec_query_len, max_num_reqs, conv_state_layout="SD", null_block_id=0):
        layers = tuple(layers)
        if not layers or not 1 <= spec_query_len <= 32 or max_num_reqs < 0:
            raise ValueError("context requires layers, R >= 0 and Q in [1, 32]")
        if null_block_id not in (-1, 0):
            raise ValueError("null_block_id must be -1 or 0")
        device = layers[0].kv_cache[1].device
        if device.type != "cuda":
            raise ValueError("commit context requires CUDA tensors")
        with torch.cuda.device(device):
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("create commit context before graph capture")
        slots, heads = layers[0].kv_cache[1].shape[:2]
        descriptors, keepalive, spans = [], [], []
        for index, layer in enumerate(layers):
            conv, state = layer.kv_cache
            rec = layer.replay_records
            tensors = (conv, state, rec.rawv, rec.rawk, rec.g, rec.beta, rec.conv)
            descriptors.append(list(ops.kda_replay_layer_descriptor(
                *tensors, conv_state_layout, int(heads), int(slots), int(spec_query_len), int(max_num_reqs))))
            if any(t.device != device for t in tensors):
                raise ValueError("all context layers must share one device")
            mine = _write_spans(conv, state, conv_state_layout)
            for previous, other in enumerate(spans):
                if _spans_overlap(mine, other) or _spans_overlap(other, mine):
                    raise ValueError(f"context layers {previous} and {index} have overlapping writable caches")
            spans.append(mine)
            keepalive.extend(tensors)
        self = cls()
        self._keepalive = tuple(keepalive)
        self._layers = layers
        self._table = torch.tensor(descriptors, device=device, dtype=torch.int64)
        self._candidate = torch.zeros((4, max_num_reqs), device=device, dtype=torch.int32)
        self._buffer = torch.zeros_like(self._candidate)
        self.plan = KDAReplayCommitPlan(*self._buffer.unbind(0))
        self._heads, self._slots = int(heads), int(slots)
        self._q, self._capacity = int(spec_query_len), int(max_num_reqs)
        self._null = int(null_block_id)
        return self

    def commit(self, num_sampled, state_indices, query_start_loc, request_indices=None, block_table=None,
               num_computed_tokens=None, mamba_block_size=None, *, token_capacity, plan_only=False,
               status: Optional[torch.Tensor] = None):
        """Commit the clamped sampled-token counts (no bonus token is subtracted).

        ``token_capacity`` is the verify projection's ``mixed_qkv.shape[0]``; intervals beyond it are
        skipped. Align mode needs ``block_table``, ``num_computed_tokens`` and
        ``mamba_block_size >= Q`` together. Rows whose source / destination slots collide with
        another active row are masked out of the plan on the device. Returns the plan.
        """
        if not isinstance(token_capacity, Integral):
            raise TypeError("token_capacity must be a host integer")
        align = (block_table is not None, num_computed_tokens is not None, mamba_block_size is not None)
        if any(align) and not all(align):
            raise ValueError("align requires block_table, computed tokens and block size")
        if all(align) and not isinstance(mamba_block_size, Integral):
            raise TypeError("mamba_block_size must be a host integer")
        if all(align) and mamba_block_size < self._q:
            raise ValueError("align block_size must be >= spec_query_len")
        ops.kda_replay_commit(self._table, self._candidate, self._buffer, num_sampled, state_indices,
                              query_start_loc, request_indices, block_table, num_computed_tokens,
                              0 if not all(align) else int(mamba_block_size), self._heads, self._slots, self._q,
                              self._null, int(token_capacity), bool(plan_only), status)
        return self.plan
