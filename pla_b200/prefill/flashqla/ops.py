"""GDN prefill entry points with the reference's signatures
(pla/prefill/flashqla/ops.py:225-738).

State contract: an indexed pool ``[slots, H, DV, DK]`` (k-last) with int32 ``initial_state_indices``
is updated in place, even when ``output_final_state`` is false; the legacy layout
``[N, H, DK, DV]`` is read (or a zero state assumed) and a new final state of that layout returned.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple, Union

import torch

from ..._ops import ops
from ...caselist import show_call

DK = 128
DV = 128
CHUNK_SIZE = 64
_STATE_DTYPES = (torch.float32, torch.bfloat16)


def _offsets(cu_seqlens, num_tokens, raw_cu_seqlens, device):
    if raw_cu_seqlens is not None:
        if isinstance(raw_cu_seqlens, torch.Tensor):
            if (raw_cu_seqlens.device.type != "cpu" or raw_cu_seqlens.ndim != 1
                    or raw_cu_seqlens.dtype not in (torch.int32, torch.int64)):
                raise ValueError("raw_cu_seqlens must be a 1-D CPU int32 or int64 tensor")
            raw_cu_seqlens = raw_cu_seqlens.tolist()
        raw_cu_seqlens = tuple(int(x) for x in raw_cu_seqlens)
        if (len(raw_cu_seqlens) < 2 or raw_cu_seqlens[0] != 0 or raw_cu_seqlens[-1] > num_tokens
                or any(b < a for a, b in zip(raw_cu_seqlens, raw_cu_seqlens[1:]))):
            raise ValueError("raw_cu_seqlens must be monotonic offsets starting at zero within the token count")
    if cu_seqlens is None:
        if raw_cu_seqlens is None:
            raw_cu_seqlens = (0, num_tokens)
        cu_seqlens = torch.tensor(raw_cu_seqlens, dtype=torch.int32, device=device)
    cu32 = cu_seqlens.to(device=device, dtype=torch.int32).contiguous()
    if cu32.ndim != 1:
        raise ValueError("cu_seqlens must be a rank-1 tensor")
    if raw_cu_seqlens is not None and len(raw_cu_seqlens) != cu32.numel():
        raise ValueError("raw_cu_seqlens must have batch+1 entries")
    return cu32


class ChunkFactor:
    """The ``A`` by-product of :func:`chunk_gated_delta_rule_fwd`: per token and value head the token's row of
    ``(I + tril(diag(beta) K K^T . Gamma, -1))^-1`` of its 64-token chunk, ``[1, T, H, 64]`` fp32 (the reference's is
    the same factor of its 32-token chunks, ``[1, T, H, 32]``). The kernels keep it as tensor-core operand images
    in the call's workspace, so it is only laid out as a tensor when somebody looks: any attribute, index or torch
    function applied to this object works on :meth:`materialize`'s result. Rows past ``cu_seqlens[-1]`` are zero.
    Values carry tf32 rounding (they are the operand the tensor core reads)."""

    _KQ_BYTES, _KNT_BYTES, _VBLOB = 128 * 128 * 4, 128 * 64 * 4, 64 * 64 * 4 * 2 + 1024

    def __init__(self, workspace, cu32, tokens, qk_heads, v_heads, max_chunks):
        self._ws, self._cu, self._geom = workspace, cu32, (int(tokens), int(qk_heads), int(v_heads), int(max_chunks))
        self._tensor = None

    def materialize(self) -> torch.Tensor:
        if self._tensor is None:
            T, Hg, H, max_chunks = self._geom
            dev = self._ws.device
            base = max_chunks * Hg * (self._KQ_BYTES + self._KNT_BYTES)
            blobs = self._ws[base:base + max_chunks * H * self._VBLOB].view(max_chunks, H, self._VBLOB)
            # image [column group][row][4 columns] -> [row, column]; only the pieces on or below the diagonal were
            # ever written, the rest of the image is scratch
            tiles = blobs[:, :, :CHUNK_SIZE * CHUNK_SIZE * 4].contiguous().view(torch.float32)
            tiles = tiles.view(max_chunks, H, CHUNK_SIZE // 4, CHUNK_SIZE, 4).permute(0, 1, 3, 2, 4)
            tiles = tiles.reshape(max_chunks, H, CHUNK_SIZE, CHUNK_SIZE)
            lower = torch.ones(CHUNK_SIZE, CHUNK_SIZE, dtype=torch.bool, device=dev).tril()
            tiles = torch.where(lower, tiles, torch.zeros((), device=dev))
            cu = self._cu.to(torch.int64)
            lens = (cu[1:] - cu[:-1]).clamp_min(0)
            first_chunk = torch.cumsum((lens + CHUNK_SIZE - 1) // CHUNK_SIZE, 0) - (lens + CHUNK_SIZE - 1) // CHUNK_SIZE
            tok = torch.arange(T, device=dev)
            seq = torch.searchsorted(cu[1:].contiguous(), tok, right=True).clamp_max(lens.numel() - 1)
            inside = (tok - cu[seq]).clamp_min(0)
            live = (tok >= cu[seq]) & (tok < cu[seq + 1])
            rows = tiles[(first_chunk[seq] + inside // CHUNK_SIZE).clamp_max(max_chunks - 1), :, inside % CHUNK_SIZE]
            self._tensor = torch.where(live[:, None, None], rows, torch.zeros((), device=dev))[None]
        return self._tensor

    def __getattr__(self, name):            # only reached for names this class does not define
        return getattr(self.materialize(), name)

    def __getitem__(self, index):
        return self.materialize()[index]

    def __len__(self):
        return 1

    def __repr__(self):
        state = "materialised" if self._tensor is not None else "deferred"
        return f"ChunkFactor([1, {self._geom[0]}, {self._geom[2]}, {CHUNK_SIZE}], {state})"

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        unwrap = lambda x: x.materialize() if isinstance(x, ChunkFactor) else x
        return func(*[unwrap(a) for a in args], **{k_: unwrap(v_) for k_, v_ in (kwargs or {}).items()})


def _forward_operator(name):
    def method(self, *args):
        return getattr(self.materialize(), name)(*[a.materialize() if isinstance(a, ChunkFactor) else a for a in args])
    method.__name__ = name
    return method


for _op in ("__add__", "__radd__", "__sub__", "__rsub__", "__mul__", "__rmul__", "__truediv__", "__rtruediv__", "__neg__",
            "__matmul__", "__rmatmul__", "__pow__", "__abs__", "__float__", "__iter__"):
    setattr(ChunkFactor, _op, _forward_operator(_op))
del _op


_plan_cache: "OrderedDict" = None  # type: ignore[assignment]


def plan_token_ranges(offsets: Sequence[int], heads: int, n_sm: int, min_chunks: int = 16):
    """Intra-GPU split of long sequences into consecutive token ranges that run as independent chains
    (the job of the reference's planner, pla/prefill/flashqla/private/cp_preprocess.py). Pure host code.

    A (sequence, value head) chain is serial, so a batch with fewer chains than SMs leaves SMs idle. Cutting
    every sequence into ``p`` ranges costs a prescan of the first ``p - 1`` ranges (two chains each) plus the
    ranges themselves, i.e. ``(waves(2 (p-1) n) + waves(p n)) / p`` of the unsplit time per wave, ``n`` = chains
    of the batch, ``waves(x) = ceil(x / n_sm)``; ``p`` grows while that lowers the cost by 10 % or more, and the split is used when
    it saves at least 20 %. Ranges are cut on chunk boundaries counted from the sequence start and are at least
    ``min_chunks`` chunks long. Returns ``(range_offsets, seg_first, last_flags, seq_of_range)`` or ``None``
    when nothing is split."""
    lens = [int(b) - int(a) for a, b in zip(offsets, offsets[1:])]
    live = sum(1 for n in lens if n > 0)
    if live == 0:
        return None
    n = live * heads
    waves = lambda x: -(-x // n_sm)
    most = max((m + CHUNK_SIZE - 1) // CHUNK_SIZE for m in lens) // min_chunks
    best, target = float(waves(n)), 1
    for p in range(2, max(2, min(most, 64)) + 1):
        cost = (waves(2 * (p - 1) * n) + waves(p * n)) / p
        if cost < 0.9 * best:                     # more ranges only for a clear gain: each adds a fold and a prologue
            best, target = cost, p
    if best > 0.8 * waves(n):
        return None
    range_offsets, seg_first, last, seq_of = [int(offsets[0])], [0], [], []
    split = False
    for s, n in enumerate(lens):
        chunks = (n + CHUNK_SIZE - 1) // CHUNK_SIZE
        parts = max(1, min(target, chunks // min_chunks))
        split |= parts > 1
        start = int(offsets[s])
        for part in range(parts):
            end_chunk = chunks * (part + 1) // parts
            end = start + n if part == parts - 1 else start + end_chunk * CHUNK_SIZE
            range_offsets.append(end)
            last.append(part == parts - 1)
            seq_of.append(s)
        seg_first.append(len(last))
    return (range_offsets, seg_first, last, seq_of) if split else None


def _range_tensors(offsets, heads, device):
    """Device copies of the plan, cached for the most recent offset tuples (serving repeats them)."""
    global _plan_cache
    from collections import OrderedDict
    if _plan_cache is None:
        _plan_cache = OrderedDict()
    key = (tuple(int(x) for x in offsets), heads, str(device))
    hit = _plan_cache.get(key)
    if hit is not None:
        _plan_cache.move_to_end(key)
        return hit
    n_sm = torch.cuda.get_device_properties(device).multi_processor_count
    plan = plan_token_ranges(key[0], heads, n_sm)
    if plan is not None:
        range_offsets, seg_first, last, seq_of = plan
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
        plan = (i32(range_offsets), i32(seg_first), i32([-1 if f else 0 for f in last]),
                torch.tensor(last, dtype=torch.bool, device=device), torch.tensor(seq_of, dtype=torch.long, device=device))
    _plan_cache[key] = plan
    while len(_plan_cache) > 8:
        _plan_cache.popitem(last=False)
    return plan


def chunk_gated_delta_rule_fwd(
    q: torch.Tensor,                       # [1, T, Hg, DK]
    k: torch.Tensor,                       # [1, T, Hg, DK]
    v: torch.Tensor,                       # [1, T, H, DV]
    g: Optional[torch.Tensor],             # [1, T, H] fp32 log gate
    beta: Optional[torch.Tensor],          # [1, T, H] fp32 activated beta
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,
    initial_state_indices: Optional[torch.Tensor] = None,
    cu_seqlens: Optional[torch.Tensor] = None,
    output_final_state: bool = True,
    auto_cp: bool = True,
    overlap_warmup_threshold: Optional[float] = None,
    force_tc01_cp_candidate: bool = False,
    normalize_qk: bool = False,
    raw_cu_seqlens: Optional[Union[Sequence[int], torch.Tensor]] = None,
    raw_gate_a: Optional[torch.Tensor] = None,   # [T,H] 16-bit
    raw_beta_b: Optional[torch.Tensor] = None,   # [T,H] 16-bit
    A_log: Optional[torch.Tensor] = None,        # [H] fp32
    dt_bias: Optional[torch.Tensor] = None,      # [H] fp32
    final_state_dtype: Optional[torch.dtype] = None,
) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor], torch.Tensor, None, Optional[torch.Tensor]]:
    """Returns ``(g_cum, A, O, None, final_state)``.

    ``O`` has the physical token shape; rows past ``cu_seqlens[-1]`` are zero and never touch the
    state. With raw gating (``raw_gate_a``, ``raw_beta_b``, ``A_log``, ``dt_bias``) the gate
    ``g = -exp(A_log) * softplus(a + dt_bias)`` and ``beta = sigmoid(b)`` are formed in the kernel.
    Evaluated chunk-wise (chunk 64, WY/UT transform) on the tensor cores. ``g_cum`` is the
    chunk-local cumulative log decay ``[1, T, H]`` fp32 at chunk size 64 (the reference uses 32);
    ``A`` is a :class:`ChunkFactor`: the chunk-64 counterpart ``[1, T, H, 64]`` of the reference's factor, laid out
    as a tensor on first use (inference never reads it, so the call itself does not pay for it). ``auto_cp`` (default on): with host offsets
    (``raw_cu_seqlens``) and an indexed fp32 pool, batches with fewer (sequence, head) chains than SMs have
    their long sequences cut into token ranges that run as independent chains (prescan of every range,
    fold of the (offset, transition) pairs, then the ranges in parallel from their incoming states); a
    a negative slot index marks a padding sequence either way (zero output rows, no state read or written).
    ``overlap_warmup_threshold`` and
    ``force_tc01_cp_candidate`` tune the reference's planner and are accepted and ignored.
    """
    if not q.is_cuda:
        raise ValueError("q must be a CUDA tensor")
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4 or q.size(0) != 1:
        raise ValueError("q, k, v must be [1, T, heads, 128]")
    raw = (raw_gate_a, raw_beta_b, A_log, dt_bias)
    use_raw = any(t is not None for t in raw)
    if use_raw and (any(t is None for t in raw) or g is not None or beta is not None):
        raise ValueError("raw gating needs raw_gate_a, raw_beta_b, A_log and dt_bias, and excludes g/beta")
    if not use_raw and (g is None or beta is None):
        raise ValueError("g and beta are required without raw gating")
    T, Hg, H = q.size(1), k.size(2), v.size(2)
    if q.size(3) != DK or v.size(3) != DV:
        raise ValueError("head dimensions must be 128")
    if scale is None:
        scale = q.size(-1) ** -0.5
    cu32 = _offsets(cu_seqlens, T, raw_cu_seqlens, q.device)
    batch = cu32.numel() - 1
    indexed = initial_state_indices is not None
    if indexed:
        if initial_state is None or initial_state.dtype not in _STATE_DTYPES or not initial_state.is_contiguous():
            raise ValueError("indexed initial_state must be contiguous fp32 or bf16")
        if initial_state.ndim != 4 or tuple(initial_state.shape[1:]) != (H, DV, DK):
            raise ValueError("indexed initial_state must be [num_slots,H,DV,DK]")
        if (initial_state_indices.device != q.device or initial_state_indices.dtype != torch.int32
                or not initial_state_indices.is_contiguous() or initial_state_indices.ndim != 1
                or initial_state_indices.numel() != batch):
            raise ValueError("initial_state_indices must be contiguous int32 [batch] on q.device")
    elif initial_state is not None:
        if initial_state.dtype not in _STATE_DTYPES or not initial_state.is_contiguous():
            raise ValueError("initial_state must be contiguous fp32 or bf16")
        if (initial_state.ndim != 4 or initial_state.size(0) < batch
                or tuple(initial_state.shape[1:]) != (H, DK, DV)):
            raise ValueError("initial_state must be [num_states>=batch,H,DK,DV]")
    if final_state_dtype is None:
        state_dtype = initial_state.dtype if initial_state is not None else torch.float32
    else:
        if final_state_dtype not in _STATE_DTYPES:
            raise ValueError("final_state_dtype must be fp32 or bf16")
        if initial_state is not None and final_state_dtype != initial_state.dtype:
            raise ValueError("final_state_dtype must match the initial_state dtype")
        state_dtype = final_state_dtype

    show_call(q, v, False, cu32, None if isinstance(raw_cu_seqlens, torch.Tensor) else raw_cu_seqlens, prefill=True)
    o = torch.empty((1, T, H, DV), dtype=q.dtype, device=q.device)
    if use_raw:
        gate, bet = raw_gate_a.reshape(T, H) if raw_gate_a.ndim != 2 else raw_gate_a, \
            raw_beta_b.reshape(T, H) if raw_beta_b.ndim != 2 else raw_beta_b
    else:
        gate, bet = g.reshape(T, H), beta.reshape(T, H)
    final_state = None
    state_out = None
    if not indexed and output_final_state:
        state_out = torch.empty((batch, H, DK, DV), dtype=state_dtype, device=q.device)
        final_state = state_out
    # chunk count: exact from trusted host offsets, else the bound T/64 + batch (no device read)
    if raw_cu_seqlens is not None:
        offs = raw_cu_seqlens.tolist() if isinstance(raw_cu_seqlens, torch.Tensor) else list(raw_cu_seqlens)
        max_chunks = sum((int(b) - int(a) + CHUNK_SIZE - 1) // CHUNK_SIZE for a, b in zip(offs, offs[1:]))
    else:
        max_chunks = T // CHUNK_SIZE + batch
    g_cum = torch.zeros((1, T, H), dtype=torch.float32, device=q.device)
    plan = None
    if auto_cp and raw_cu_seqlens is not None and indexed and initial_state.dtype == torch.float32:
        plan = _range_tensors(offs, H, q.device)
    if plan is not None:
        cu_ranges, seg_first, prescan_mask, last_mask, seq_of = plan
        n_ranges = prescan_mask.numel()
        stage_args = (q[0], k[0], v[0], gate, bet, A_log, dt_bias, o[0])
        tail = (False, bool(normalize_qk), float(scale), not use_raw, int(max_chunks))
        # a sequence with a negative slot is padding, exactly as in the unsplit kernel: its ranges are neither
        # prescanned nor run (zero output rows), its slot is never read or written
        seq_slot = initial_state_indices[seq_of]
        minus = torch.full_like(prescan_mask, -1)
        ws = ops.gdn_prefill_chunked_stage(*stage_args, g_cum[0], cu_ranges, None, None, None, *tail, 1, False, None,
                                           None, None)
        pairs = torch.empty((n_ranges, H, 2, DV, DK), dtype=torch.float32, device=q.device)
        ops.gdn_prefill_chunked_stage(*stage_args, None, cu_ranges, None, pairs, ws, *tail, 2, True, None,
                                      torch.where(seq_slot < 0, minus, prescan_mask), None)
        state_in = ops.cp_fold_segments(pairs, seg_first, initial_state, initial_state_indices, None)
        range_slot = torch.where(seq_slot < 0, minus, torch.arange(n_ranges, dtype=torch.int32, device=q.device))
        out_idx = torch.where(last_mask, seq_slot, minus)
        ops.gdn_prefill_chunked_stage(*stage_args, None, cu_ranges, state_in, initial_state, ws, *tail, 2, False, None,
                                      range_slot, out_idx)
        final_state = _gather_final(initial_state, initial_state_indices) if output_final_state else None
        return g_cum, ChunkFactor(ws, cu32, T, Hg, H, max_chunks), o, None, final_state
    ws = ops.gdn_prefill_chunked(
        q[0], k[0], v[0], gate, bet, A_log, dt_bias, o[0], g_cum[0], cu32, initial_state,
        initial_state_indices if indexed else None, state_out, None, not indexed, bool(normalize_qk),
        float(scale), not use_raw, indexed, int(max_chunks), 0, None)
    if indexed and output_final_state:
        final_state = _gather_final(initial_state, initial_state_indices)
    return g_cum, ChunkFactor(ws, cu32, T, Hg, H, max_chunks), o, None, final_state


def _gather_final(pool: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """Final states of the batch out of the indexed pool; a padding sequence (negative slot) gets zeros."""
    idx = slots.long()
    rows = pool[idx.clamp_min(0)]
    return torch.where((idx < 0)[:, None, None, None], torch.zeros((), dtype=pool.dtype, device=pool.device), rows)


def gdn_prefill_packed_qkv_fwd(
    packed_qkv: torch.Tensor,                # [T, 2*Hg*DK + H*DV]
    raw_gate_a: torch.Tensor,                # [T,H]
    raw_beta_b: torch.Tensor,                # [T,H]
    A_log: torch.Tensor,                     # [H] fp32
    dt_bias: torch.Tensor,                   # [H] fp32
    cu_seqlens: torch.Tensor,                # [batch+1] int32
    *,
    num_qk_heads: int,
    num_v_heads: int,
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,
    initial_state_indices: Optional[torch.Tensor] = None,
    output_final_state: bool = True,
    auto_cp: bool = True,
    overlap_warmup_threshold: Optional[float] = None,
    force_tc01_cp_candidate: bool = False,
    raw_cu_seqlens: Optional[Union[Sequence[int], torch.Tensor]] = None,
    final_state_dtype: Optional[torch.dtype] = None,
):
    """GDN prefill directly on a post-convolution ``[T, Q|K|V]`` buffer: features of one token are
    contiguous, the token stride may exceed the row width and the view may start at any element
    (Q/K/V are consumed in place as aliases of the buffer). Same return contract as
    :func:`chunk_gated_delta_rule_fwd`."""
    Hg, H = int(num_qk_heads), int(num_v_heads)
    q, k, v = _packed_views(packed_qkv, Hg, H)
    return chunk_gated_delta_rule_fwd(
        q, k, v, None, None, scale=scale, initial_state=initial_state,
        initial_state_indices=initial_state_indices, cu_seqlens=cu_seqlens,
        output_final_state=output_final_state, auto_cp=auto_cp,
        overlap_warmup_threshold=overlap_warmup_threshold, force_tc01_cp_candidate=force_tc01_cp_candidate,
        normalize_qk=True, raw_cu_seqlens=raw_cu_seqlens, raw_gate_a=raw_gate_a, raw_beta_b=raw_beta_b,
        A_log=A_log, dt_bias=dt_bias, final_state_dtype=final_state_dtype)


def _packed_views(rows: torch.Tensor, Hg: int, H: int):
    """q, k, v of a packed ``[T, Hg*128 | Hg*128 | H*128]`` buffer as ``[1, T, heads, 128]`` views that alias it
    (no copy; the row pitch and the buffer's offset inside its storage carry over)."""
    if Hg <= 0 or H <= 0:
        raise ValueError(f"head counts must be positive, got num_qk_heads={Hg}, num_v_heads={H}")
    problems = []
    if not rows.is_cuda:
        problems.append("it must live on a CUDA device")
    if rows.ndim != 2:
        problems.append(f"it must be [T, Q|K|V], got {rows.ndim} dimensions")
    if rows.dtype not in (torch.float16, torch.bfloat16):
        problems.append(f"it must be fp16 or bf16, got {rows.dtype}")
    if problems:
        raise ValueError("packed_qkv: " + "; ".join(problems))
    want = (2 * Hg + H) * DK
    if rows.size(0) == 0:
        raise ValueError("packed_qkv: an empty token dimension is not supported")
    if rows.size(1) != want:
        raise ValueError(f"packed_qkv: a row holds {rows.size(1)} features, but Hg={Hg}, H={H} need {want}")
    if rows.stride(1) != 1:
        raise ValueError("packed_qkv: the features of a token must be contiguous (the token pitch is free)")
    qk = Hg * DK
    split = lambda lo, heads: rows[:, lo:lo + heads * DK].unflatten(1, (heads, DK)).unsqueeze(0)
    return split(0, Hg), split(qk, Hg), split(2 * qk, H)
