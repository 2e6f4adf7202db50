"""Context-parallel GDN / KDA prefill: one long sequence cut into contiguous token ranges, one per GPU.

Over a token range the gated delta rule is an affine map of the incoming state, row by row of the
k-last state ``S[v, k]``:  ``S_out = S_in @ M + B``  with ``M [K, K]`` the product of the per-token
transitions ``gamma_t (I - beta_t k_t k_t^T)`` and ``B [V, K]`` the state reached from zero
(the reference derives the same pair for its intra-card split:
docs/prefill_flashkdapro_cp_design.md:22-46, src/prefill/flashqla/kernels/prepare_h_cute.cu:59-67).

Per rank:
  1. prepare     chunk operands of the rank's tokens (tensor-core kernel, shared by 2 and 5)
  2. prescan     two chains per value head, no output: B from a zero state, M from the identity with V = 0
  3. all-gather  ``[H, 2, 128, 128]`` fp32 per rank -- the only collective on the path
  4. fold        ``S_in(r) = fold_{j<r}(M_j, B_j)(S_0)``: at most ``world-1`` batched 128^3 products,
                 recomputed on every rank instead of a second collective
  5. segment     the ordinary chain from ``S_in(r)``; the last rank's final state is the sequence's

The last rank's (M, B) is never used, so it skips step 2 and contributes zeros to the gather.
A rank with fewer chains than SMs applies the same scheme once more inside its range (``plan_rank_ranges``).
GDN and KDA (per-channel decay: M = prod diag(gamma_t)(I - beta_t k_t k_t^T), the same row-wise affine form) both
run the chunk-64 tensor-core kernels, whose chain has a prescan mode; for a KDA gate whose decay is not bounded
(``flashkda_fwd`` documents the rule) the token-recurrent kernel's prescan mode takes over.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

D = 128
CHUNK = 64


def plan_rank_ranges(tokens: int, chains: int, n_sm: int, min_chunks: int = 16):
    """Token ranges INSIDE one rank (same idea as the split across ranks, one level down): a rank with fewer
    chains than SMs cuts its tokens into ``p`` ranges on chunk boundaries; it then prescans all ``p`` ranges (two
    chains each), composes their pairs into the rank's pair, and after the exchange runs the ranges in parallel.
    Cost in waves of ``n_sm`` chains: ``(waves(2 p n) + waves(p n)) / p`` against ``waves(2 n) + waves(n)``
    unsplit; ``p`` grows while that lowers the cost by 10 % or more. Returns the range offsets ``[0, ..., tokens]``
    or ``None`` when one range is best. Pure host code."""
    chunks = (tokens + CHUNK - 1) // CHUNK
    waves = lambda x: -(-x // n_sm)
    base = float(waves(2 * chains) + waves(chains))
    best, parts = base, 1
    for p in range(2, max(1, min(chunks // min_chunks, 64)) + 1):
        cost = (waves(2 * p * chains) + waves(p * chains)) / p
        if cost < 0.9 * best:
            best, parts = cost, p
    if parts == 1 or best > 0.8 * base:
        return None
    return [min(tokens, (chunks * i // parts) * CHUNK) for i in range(parts)] + [tokens]


_rank_plans: dict = {}


def _rank_plan_tensors(T: int, H: int, device, split: bool):
    """Device copies of a rank's range plan, kept per (tokens, heads, device): serving repeats the shapes, and
    every small host-to-device copy is a stall on the launch path."""
    key = (T, H, str(device), bool(split))
    hit = _rank_plans.get(key)
    if hit is not None:
        return hit
    offs = None
    if split and device.type == "cuda" and T > 0:
        offs = plan_rank_ranges(T, H, torch.cuda.get_device_properties(device).multi_processor_count)
    parts = 1 if offs is None else len(offs) - 1
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
    plan = dict(parts=parts, cu=i32([0, T] if offs is None else offs), skip_last=i32([0] * (parts - 1) + [-1]),
                seg_first=i32([0, parts]), slot0=i32([0]), last_writes=i32([-1] * (parts - 1) + [0]),
                )
    if len(_rank_plans) >= 32:
        _rank_plans.clear()
    _rank_plans[key] = plan
    return plan


class CudaSegmentKernels:
    """Steps 1, 2 and 5 on the rank's GPU (pla_b200_gdn_prefill_chunked, stages 1 and 2). When the rank has
    fewer chains than SMs its tokens run as several ranges (``plan_rank_ranges``; ``split=False`` turns it off)."""

    def __init__(self, q, k, v, gate, beta, A_log, dt_bias, scale, normalize_qk, gate_activated, split=True):
        from .._ops import ops  # raises ImportError when the native libraries are missing
        self._ops = ops
        self.a = (q, k, v, gate, beta, A_log, dt_bias)
        self.scale, self.normalize_qk, self.gate_activated = float(scale), bool(normalize_qk), bool(gate_activated)
        self._setup(q, v, split)

    def _setup(self, q, v, split):
        T, H = v.shape[0], v.shape[1]
        self.T, self.H = T, H
        self.plan = _rank_plan_tensors(T, H, q.device, split)
        self.parts, self.cu = self.plan["parts"], self.plan["cu"]
        self.max_chunks = (T + CHUNK - 1) // CHUNK
        self.out = torch.empty(T, H, D, dtype=q.dtype, device=q.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=q.device)
        self.ws = None
        self.pairs = None       # [parts, H, 2, 128, 128]: pairs of this rank's ranges

    def _stage(self, stage, prescan, state_in, state_out, range_mask=None, out_indices=None):
        q, k, v, gate, beta, A_log, dt_bias = self.a
        self.ws = self._ops.gdn_prefill_chunked_stage(
            q, k, v, gate, beta, A_log, dt_bias, self.out, None, self.cu, state_in, state_out, self.ws, False,
            self.normalize_qk, self.scale, self.gate_activated, self.max_chunks, stage, prescan, self.status,
            range_mask, out_indices)

    def prepare(self):
        self._stage(1, False, None, None)

    def _prescan_ranges(self, every_range: bool):
        dev = self.out.device
        self.pairs = torch.empty(self.parts, self.H, 2, D, D, dtype=torch.float32, device=dev)
        # the last range's pair is not needed when only the incoming states are wanted
        self._stage(2, True, None, self.pairs[:self.parts], None if every_range else self.plan["skip_last"])

    def prescan(self) -> torch.Tensor:
        dev = self.out.device
        if self.parts == 1:
            mb = torch.empty(1, self.H, 2, D, D, dtype=torch.float32, device=dev)
            self._stage(2, True, None, mb)
            return mb[0]
        # pairs of all ranges, then the rank's pair in one launch: the offset from a zero state through all of them,
        # the transition from the identity through the M_j alone
        self._prescan_ranges(True)
        return self._ops.cp_compose_pairs(self.pairs[:self.parts], self.parts, self.status)

    def segment(self, state_in: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        dev = self.out.device
        final = torch.empty(1, self.H, D, D, dtype=torch.float32, device=dev)
        if self.parts == 1:
            self._stage(2, False, state_in[None].contiguous(), final)
            return self.out, final[0]
        if self.pairs is None:
            self._prescan_ranges(False)
        states = self._ops.cp_fold_segments(self.pairs[:self.parts], self.plan["seg_first"], state_in[None].contiguous(),
                                            self.plan["slot0"], self.status)
        self._stage(2, False, states, final, None, self.plan["last_writes"])
        return self.out, final[0]

    def check(self):
        code = int(self.status.item())
        if code:
            raise RuntimeError(f"chunked prefill reported device status {code:#x}")


class KdaChunkedSegmentKernels:
    """Steps 1, 2 and 5 for KDA with the chunk-64 tensor-core kernels (pla_b200_kda_prefill_chunked); ranges
    inside the rank as for GDN."""

    def __init__(self, q, k, v, gate, beta, A_log, dt_bias, scale, normalize_qk, lower_bound, split=True):
        from .._ops import ops  # raises ImportError when the native libraries are missing
        self._ops = ops
        self.a = (q, k, v, gate, beta, A_log, dt_bias)
        self.scale, self.normalize_qk = float(scale), bool(normalize_qk)
        self.lower_bound = None if lower_bound is None else float(lower_bound)
        self._setup(q, v, split)

    def _stage(self, stage, prescan, state_in, state_out, range_mask=None, out_indices=None):
        q, k, v, gate, beta, A_log, dt_bias = self.a
        self.ws = self._ops.kda_prefill_chunked(
            q, k, v, gate, beta, A_log, dt_bias, self.out, self.cu, state_in, None, state_out, out_indices, self.ws,
            False, self.normalize_qk, self.scale, self.lower_bound, False, self.max_chunks, stage, prescan, self.status,
            range_mask)

    _setup = CudaSegmentKernels._setup
    _prescan_ranges = CudaSegmentKernels._prescan_ranges
    prepare = CudaSegmentKernels.prepare
    prescan = CudaSegmentKernels.prescan
    segment = CudaSegmentKernels.segment
    check = CudaSegmentKernels.check


class RecurrentSegmentKernels:
    """Steps 2 and 5 with the token-recurrent kernel (pla_b200_prefill_recurrent; KDA or GDN)."""

    def __init__(self, q, k, v, gate, beta, A_log, dt_bias, scale, normalize_qk, gate_activated, is_kda, lower_bound):
        from .._ops import ops  # raises ImportError when the native libraries are missing
        self._ops = ops
        self.a = (q, k, v, gate, beta, A_log, dt_bias)
        self.scale, self.normalize_qk, self.gate_activated = float(scale), bool(normalize_qk), bool(gate_activated)
        self.is_kda = bool(is_kda)
        self.lower_bound = None if lower_bound is None else float(lower_bound)
        T, H = v.shape[0], v.shape[1]
        self.T, self.H = T, H
        self.cu = torch.tensor([0, T], dtype=torch.int32, device=q.device)
        self.out = torch.empty(T, H, D, dtype=q.dtype, device=q.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=q.device)

    def prepare(self):
        pass

    def prescan(self) -> torch.Tensor:
        q, k, v, gate, beta, A_log, dt_bias = self.a
        pairs = torch.empty(1, self.H, 2, D, D, dtype=torch.float32, device=self.out.device)
        self._ops.prefill_recurrent_prescan(q, k, v, gate, beta, A_log, dt_bias, self.cu, pairs, self.is_kda,
                                            self.normalize_qk, self.scale, self.lower_bound, self.gate_activated,
                                            self.status)
        return pairs[0]

    def segment(self, state_in: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        q, k, v, gate, beta, A_log, dt_bias = self.a
        final = torch.empty(1, self.H, D, D, dtype=torch.float32, device=self.out.device)
        self._ops.prefill_recurrent(q, k, v, gate, beta, A_log, dt_bias, self.out, self.cu,
                                    state_in[None].contiguous(), None, final, None, False, self.is_kda,
                                    self.normalize_qk, self.scale, self.lower_bound, self.gate_activated, False,
                                    self.status)
        return self.out, final[0]

    check = CudaSegmentKernels.check


class SegmentPlan:
    """State of one rank between the two halves of the algorithm."""

    def __init__(self, kernels, rank, world, tokens, H, device, transfer):
        self.kernels, self.rank, self.world, self.tokens, self.H = kernels, rank, world, tokens, H
        self.device, self.transfer = device, transfer


def identity_transfer(H: int, device) -> torch.Tensor:
    """(B, M) of an empty token range: zero offset, identity transition."""
    mb = torch.zeros(H, 2, D, D, dtype=torch.float32, device=device)
    mb[:, 1] = torch.eye(D, dtype=torch.float32, device=device)
    return mb


def begin_segment(kernels, rank: int, world: int, tokens: int, H: int, device) -> SegmentPlan:
    """Steps 1-2. ``transfer`` is what the rank contributes to the all-gather."""
    if tokens > 0:
        kernels.prepare()
    if rank == world - 1:
        transfer = torch.zeros(H, 2, D, D, dtype=torch.float32, device=device)      # never read
    elif tokens == 0:
        transfer = identity_transfer(H, device)
    else:
        transfer = kernels.prescan()
    return SegmentPlan(kernels, rank, world, tokens, H, device, transfer)


def fold_transfers(initial_state: Optional[torch.Tensor], gathered: torch.Tensor, rank: int) -> torch.Tensor:
    """Step 4: the state entering rank ``rank``'s range. gathered: [world, H, 2, 128, 128] (B, M)."""
    H = gathered.shape[1]
    if initial_state is None:
        state = torch.zeros(H, D, D, dtype=torch.float32, device=gathered.device)
    else:
        state = initial_state.to(torch.float32)
    for j in range(rank):
        state = torch.baddbmm(gathered[j, :, 0], state, gathered[j, :, 1])
    return state


def finish_segment(plan: SegmentPlan, initial_state: Optional[torch.Tensor], gathered: torch.Tensor):
    """Steps 4-5. Returns (o [tokens, H, 128], state leaving this rank's range [H, 128, 128])."""
    ops = getattr(plan.kernels, "_ops", None)
    if ops is not None and gathered.is_cuda:
        # the library's fold kernel (pla_b200_cp_fold_prefix); fold_transfers is the same algebra in torch
        init = None if initial_state is None else initial_state.to(torch.float32).contiguous()
        state_in = ops.cp_fold_prefix(gathered.contiguous(), init, plan.rank, plan.kernels.status)
    else:
        state_in = fold_transfers(initial_state, gathered, plan.rank)
    if plan.tokens == 0:
        return None, state_in
    return plan.kernels.segment(state_in)


def gdn_prefill_context_parallel(
    q: torch.Tensor,                       # [T_rank, Hg, 128] this rank's tokens
    k: torch.Tensor,                       # [T_rank, Hg, 128]
    v: torch.Tensor,                       # [T_rank, H, 128]
    gate: torch.Tensor,                    # [T_rank, H] raw gate input (or fp32 log decay when gate_activated)
    beta: torch.Tensor,                    # [T_rank, H] raw beta input (or fp32 beta when gate_activated)
    A_log: Optional[torch.Tensor] = None,  # [H] fp32
    dt_bias: Optional[torch.Tensor] = None,
    initial_state: Optional[torch.Tensor] = None,   # [H, 128(V), 128(K)] fp32, the same on every rank
    scale: Optional[float] = None,
    normalize_qk: bool = True,
    gate_activated: bool = False,
    output_final_state: bool = True,
    group: Optional[dist.ProcessGroup] = None,
    segment_kernels=None,
):
    """Rank ``r`` of ``group`` holds tokens ``[sum(T_j, j<r), sum(T_j, j<=r))`` of one sequence; ranges
    may have different (even zero) lengths and need no alignment. Returns ``(o, final_state)``:
    this rank's output rows and, when ``output_final_state``, the sequence's final state on every rank.

    ``segment_kernels`` replaces the GPU steps (host-side tests of the exchange); by default the CUDA
    kernels run and a missing native library is an ImportError.
    """
    if scale is None:
        scale = D ** -0.5
    kernels = segment_kernels
    if kernels is None:
        kernels = CudaSegmentKernels(q, k, v, gate, beta, A_log, dt_bias, scale, normalize_qk, gate_activated)
    return run_context_parallel(kernels, v, initial_state, output_final_state, group)


def kda_prefill_context_parallel(
    q: torch.Tensor,                       # [T_rank, H, 128]
    k: torch.Tensor,                       # [T_rank, H, 128]
    v: torch.Tensor,                       # [T_rank, H, 128]
    g: torch.Tensor,                       # [T_rank, H, 128] raw per-channel gate input
    beta: torch.Tensor,                    # [T_rank, H] raw beta input
    A_log: torch.Tensor,                   # [H] fp32
    dt_bias: torch.Tensor,                 # [H, 128] fp32
    lower_bound: Optional[float],          # safe-gate bound, None = softplus gate
    initial_state: Optional[torch.Tensor] = None,   # [H, 128(V), 128(K)] fp32, the same on every rank
    scale: Optional[float] = None,
    normalize_qk: bool = True,
    output_final_state: bool = True,
    group: Optional[dist.ProcessGroup] = None,
    segment_kernels=None,
    backend: str = "auto",
):
    """KDA counterpart of :func:`gdn_prefill_context_parallel` (same ranges, same exchange).
    ``backend``: ``"chunked"`` (tensor-core kernels; decay bounded as ``flashkda_fwd`` documents),
    ``"recurrent"`` (exact token recurrence), ``"auto"`` = the choice ``flashkda_fwd(backend="auto")`` makes:
    chunked for the safe gate with ``-5 <= lower_bound < 0`` and for a softplus gate whose parameters bound the
    decay of 16 tokens by 80 nats."""
    if scale is None:
        scale = D ** -0.5
    kernels = segment_kernels
    if kernels is None:
        if backend == "auto":
            from .flashkdapro.ops import _softplus_decay_is_bounded
            safe = lower_bound is not None and -5.0 <= lower_bound < 0.0
            backend = "chunked" if safe or (lower_bound is None and _softplus_decay_is_bounded(A_log, dt_bias)) else "recurrent"
        if backend == "chunked":
            kernels = KdaChunkedSegmentKernels(q, k, v, g, beta, A_log, dt_bias, scale, normalize_qk, lower_bound)
        else:
            kernels = RecurrentSegmentKernels(q, k, v, g, beta, A_log, dt_bias, scale, normalize_qk, False, True,
                                              lower_bound)
    return run_context_parallel(kernels, v, initial_state, output_final_state, group)


def run_context_parallel(kernels, v, initial_state, output_final_state, group):
    """Steps 1-5 over ``group`` with the given kernel set; ``v`` only supplies shapes, dtype and device."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    T, H = v.shape[0], v.shape[1]
    plan = begin_segment(kernels, rank, world, T, H, v.device)
    gathered = torch.empty(world, H, 2, D, D, dtype=torch.float32, device=v.device)
    dist.all_gather_into_tensor(gathered, plan.transfer[None].contiguous(), group=group)
    o, state_out = finish_segment(plan, initial_state, gathered)
    if o is None:
        o = v.new_empty((0, H, D))
    final = None
    if output_final_state:
        final = state_out.contiguous()
        dist.broadcast(final, src=dist.get_global_rank(group, world - 1) if group is not None else world - 1,
                       group=group)
    if hasattr(kernels, "check"):
        kernels.check()
    return o, final
