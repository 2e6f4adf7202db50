"""KDA prefill entry point with the reference's signature (pla/prefill/flashkdapro/ops.py:66-219)."""
from __future__ import annotations

import math
import weakref
from typing import Optional, Tuple

import torch

from ..._ops import ops
from ...caselist import show_call

DK = 128
DV = 128


def _rows(t: torch.Tensor) -> torch.Tensor:
    """[tokens, H, 128] readable in place when one token's features are contiguous; else materialised."""
    return t if (t.stride(2) == 1 and t.stride(1) == 128) else t.contiguous()


# Largest gate input the static bound below assumes: 16-bit projections of a trained layer stay far inside it,
# and an input beyond it still cannot go unnoticed (the chunked kernel sets PLA_B200_DEV_DECAY_RANGE).
_GATE_INPUT_BOUND = 20.0
_bound_cache = weakref.WeakKeyDictionary()      # A_log tensor object -> (dt_bias object id, versions, verdict)


def _softplus_decay_is_bounded(A_log: torch.Tensor, dt_bias: torch.Tensor) -> bool:
    """True when the softplus gate ``-exp(A_log) * softplus(x + dt_bias)`` cannot decay a key channel by more than
    80 nats inside 16 tokens (what the chunked kernels' 16-token reference points can represent) for inputs
    ``|x| <= 20``:  16 * exp(max A_log) * softplus(20 + max dt_bias) <= 80.  The two maxima are read from the device
    once per pair of parameter tensors: the verdict is remembered for the tensor OBJECTS (and their versions), so a
    layer that passes its parameters pays one device read in its lifetime; a caller that builds new tensors for
    every call pays it every call."""
    stamp = (id(dt_bias), A_log._version, dt_bias._version)
    hit = _bound_cache.get(A_log)
    if hit is not None and hit[0] == stamp:
        return hit[1]
    a_max = float(A_log.detach().float().max())
    b_max = float(dt_bias.detach().float().max())
    x = _GATE_INPUT_BOUND + b_max
    softplus = x if x > 20.0 else math.log1p(math.exp(x))
    verdict = 16.0 * math.exp(a_max) * softplus <= 80.0
    _bound_cache[A_log] = (stamp, verdict)
    return verdict


def flashkda_fwd(
    q: torch.Tensor,                       # [total_tokens, H, DK] bf16
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,                       # [total_tokens, H, DK] bf16 raw gate
    beta: torch.Tensor,                    # [total_tokens, H] bf16 raw
    A_log: torch.Tensor,                   # [H] fp32
    dt_bias: torch.Tensor,                 # [H, DK] fp32
    out: torch.Tensor,                     # [total_tokens, H, DV] bf16 (written)
    scale: Optional[float] = None,
    lower_bound: Optional[float] = -5.0,
    initial_state: Optional[torch.Tensor] = None,   # [N, H, DV, DK]
    final_state: Optional[torch.Tensor] = None,     # [N, H, DV, DK] (written)
    cu_seqlens: Optional[torch.Tensor] = None,
    state_pool: Optional[torch.Tensor] = None,      # [slots, H, DV, DK] (in place)
    state_indices: Optional[torch.Tensor] = None,
    raw_cu_seqlens: Optional[Tuple[int, ...]] = None,
    *,
    backend: str = "auto",
    status: Optional[torch.Tensor] = None,
    auto_cp: bool = True,
) -> None:
    """KDA prefill over packed varlen tokens; writes ``out`` in full (rows past ``cu_seqlens[-1]``
    zero) and ``final_state`` or the pool slots. The gate is the safe gate
    ``lower_bound * sigmoid(exp(A_log) * (g + dt_bias))``; ``lower_bound=None`` (an extension)
    selects ``-exp(A_log) * softplus(g + dt_bias)``. ``None`` initial state starts from zero.

    ``backend`` (keyword-only, not in the reference): ``"chunked"`` = chunk-64 tensor-core kernels (decay
    references every 16 tokens; needs the decay of every key channel to stay within 80 nats per 16 tokens,
    which the safe gate with ``lower_bound >= -5`` guarantees; a violation sets bit 16 of ``status``),
    ``"recurrent"`` = exact fp32 token recurrence, ``"auto"`` = chunked for the safe gate with
    ``-5 <= lower_bound < 0`` and for a softplus gate whose parameters keep the decay inside that range
    (``16 exp(max A_log) softplus(20 + max dt_bias) <= 80``, e.g. ``A_log <= -1.4``; checked once per parameter
    tensor), recurrent otherwise. ``auto_cp`` (keyword-only, default on): with host offsets
    (``raw_cu_seqlens``) and an fp32 ``state_pool``, the chunked backend cuts long sequences of a batch with
    fewer (sequence, head) chains than SMs into token ranges that run in parallel (the job of the reference's
    intra-card planner, src/prefill/flashkdapro/host/torch_extension_cute.cc:179-215).
    """
    if backend not in ("auto", "chunked", "recurrent"):
        raise ValueError("backend must be auto, chunked or recurrent")
    if not q.is_cuda:
        raise ValueError("q must be a CUDA tensor")
    for name, t in (("k", k), ("v", v), ("g", g), ("beta", beta), ("A_log", A_log), ("dt_bias", dt_bias),
                    ("out", out)):
        if t.device != q.device:
            raise ValueError(f"{name} must be on {q.device}, got {t.device}")
    for name, t in (("initial_state", initial_state), ("final_state", final_state), ("cu_seqlens", cu_seqlens),
                    ("state_pool", state_pool), ("state_indices", state_indices)):
        if t is not None and t.device != q.device:
            raise ValueError(f"{name} must be on {q.device}, got {t.device}")
    in_idx = out_idx = None
    in_place = False
    if state_pool is not None:
        if initial_state is not None or final_state is not None:
            raise ValueError("state_pool is mutually exclusive with initial_state/final_state")
        if state_indices is None:
            raise ValueError("state_pool requires state_indices")
        initial_state, in_idx, in_place = state_pool, state_indices, True
    elif state_indices is not None:
        if initial_state is None and final_state is None:
            raise ValueError("state_indices requires state_pool, initial_state, or final_state")
        in_idx = state_indices if initial_state is not None else None
        out_idx = state_indices if final_state is not None else None
    if initial_state is not None and final_state is not None and initial_state.dtype != final_state.dtype:
        raise ValueError("initial_state and final_state dtypes must match")
    if q.ndim != 3 or q.size(2) != DK:
        raise ValueError("q must be [total_tokens, H, 128]")
    T, H = q.size(0), q.size(1)
    if scale is None:
        scale = q.size(-1) ** -0.5
    if cu_seqlens is None:
        cu32 = torch.tensor(raw_cu_seqlens if raw_cu_seqlens is not None else (0, T), dtype=torch.int32,
                            device=q.device)
    else:
        if cu_seqlens.dtype not in (torch.int32, torch.int64):
            raise ValueError("cu_seqlens must be int32 or int64")
        cu32 = cu_seqlens.to(torch.int32).contiguous()
    if raw_cu_seqlens is not None and len(raw_cu_seqlens) != cu32.numel():
        raise ValueError("raw_cu_seqlens must have N+1 entries")
    if not out.is_contiguous() or tuple(out.shape) != (T, H, DV):
        raise ValueError("out must be contiguous [total_tokens, H, DV]")
    show_call(q, v, True, cu32, raw_cu_seqlens, lower_bound, prefill=True)
    bet = beta if beta.stride(-1) == 1 else beta.contiguous()
    gg = g if (g.stride(2) == 1 and g.stride(1) == 128) else g.contiguous()
    lb = None if lower_bound is None else float(lower_bound)
    if backend == "auto":
        if lb is not None:
            backend = "chunked" if -5.0 <= lb < 0.0 else "recurrent"
        else:
            backend = "chunked" if _softplus_decay_is_bounded(A_log, dt_bias) else "recurrent"
    if backend == "chunked":
        max_chunks = T // 64 + (cu32.numel() - 1)
        plan = None
        if (auto_cp and in_place and raw_cu_seqlens is not None and state_pool.dtype == torch.float32
                and state_pool.is_contiguous() and state_indices.dtype == torch.int32):
            # few (sequence, head) chains for the SMs: long sequences run as several token ranges (prescan of every
            # range, fold of the (offset, transition) pairs, then the ranges in parallel); see flashqla.ops
            from ..flashqla.ops import _range_tensors
            offs = [int(x) for x in raw_cu_seqlens]
            plan = _range_tensors(offs, H, q.device)
        if plan is not None:
            cu_ranges, seg_first, prescan_mask, last_mask, seq_of = plan
            chunks = sum((b - a + 63) // 64 for a, b in zip(offs, offs[1:]))
            args = (_rows(q), _rows(k), _rows(v), gg, bet, A_log.contiguous(), dt_bias.contiguous(), out, cu_ranges)
            tail = (False, True, float(scale), lb, False, chunks)
            # a sequence with a negative slot is padding, as in the unsplit kernel: zero output rows, slot untouched
            seq_slot = state_indices[seq_of]
            minus = torch.full_like(prescan_mask, -1)
            ws = ops.kda_prefill_chunked(*args, None, None, None, None, None, *tail, 1, False, status)
            pairs = torch.empty((prescan_mask.numel(), H, 2, DV, DK), dtype=torch.float32, device=q.device)
            ops.kda_prefill_chunked(*args, None, None, pairs, None, ws, *tail, 2, True, status,
                                    torch.where(seq_slot < 0, minus, prescan_mask))
            state_in = ops.cp_fold_segments(pairs, seg_first, state_pool, state_indices.contiguous(), status)
            range_slot = torch.where(seq_slot < 0, minus,
                                     torch.arange(prescan_mask.numel(), dtype=torch.int32, device=q.device))
            out_idx = torch.where(last_mask, seq_slot, minus)
            ops.kda_prefill_chunked(*args, state_in, range_slot, state_pool, out_idx, ws, *tail, 2, False, status)
            return None
        ops.kda_prefill_chunked(
            _rows(q), _rows(k), _rows(v), gg, bet, A_log.contiguous(), dt_bias.contiguous(), out, cu32,
            initial_state, in_idx, None if in_place else final_state, out_idx, None, False, True, float(scale), lb,
            in_place, max_chunks, 0, False, status)
        return None
    ops.prefill_recurrent(
        _rows(q), _rows(k), _rows(v), gg, bet, A_log.contiguous(), dt_bias.contiguous(), out, cu32,
        initial_state, in_idx, None if in_place else final_state, out_idx, False, True, True, float(scale),
        lb, False, in_place, status)
    return None
