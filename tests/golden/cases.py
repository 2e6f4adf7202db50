"""Deterministic small inputs shared by the fixture generator and the tests.

Inputs come from ``numpy.random.RandomState`` (bit-stable across versions) and
are rounded to the activation dtype through torch, so the generator (run where
the reference tree is available) and the tests (run anywhere) see identical
tensors without storing them. Only reference OUTPUTS are stored in the .npz
fixtures, sub-sampled where large (see ``subsample``).
"""
from __future__ import annotations

import numpy as np
import torch

D = 128


def _rs(seed):
    return np.random.RandomState(seed)


def _t(rs, *shape, dtype=torch.bfloat16, scale=1.0):
    return (torch.from_numpy(rs.standard_normal(shape).astype(np.float32)) * scale).to(dtype)


def subsample(x: torch.Tensor, step: int = 4) -> np.ndarray:
    """Every ``step``-th element of the two innermost axes, as float32 numpy."""
    return x.float()[..., ::step, ::step].contiguous().numpy()


# name -> dict(mode, is_kda, H, HV, B, T, act, lower_bound, is_sglang)
KLAST_CASES = {
    "gdn_decode":        dict(mode="decode", is_kda=False, H=2, HV=4, B=3, T=1, act="bf16"),
    "gdn_decode_f16":    dict(mode="decode", is_kda=False, H=2, HV=2, B=3, T=1, act="f16"),
    "kda_decode":        dict(mode="decode", is_kda=True, H=2, HV=4, B=3, T=1, act="bf16"),
    "kda_decode_safe":   dict(mode="decode", is_kda=True, H=2, HV=2, B=3, T=1, act="bf16", lower_bound=-5.0),
    "gdn_decode_vllm":   dict(mode="decode", is_kda=False, H=2, HV=4, B=3, T=1, act="bf16", is_sglang=False),
    "gdn_verify":        dict(mode="verify", is_kda=False, H=2, HV=4, B=3, T=4, act="bf16"),
    "kda_verify":        dict(mode="verify", is_kda=True, H=1, HV=2, B=3, T=4, act="bf16"),
    "gdn_writeback":     dict(mode="writeback", is_kda=False, H=2, HV=2, B=3, T=3, act="bf16"),
    "kda_tree_safe":     dict(mode="tree", is_kda=True, H=1, HV=2, B=3, T=5, act="bf16", lower_bound=-5.0),
    "gdn_tree":          dict(mode="tree", is_kda=False, H=2, HV=2, B=3, T=6, act="bf16"),
    "gdn_ragged":        dict(mode="ragged", is_kda=False, H=2, HV=4, B=3, T=4, act="bf16"),
    "kda_ragged":        dict(mode="ragged", is_kda=True, H=2, HV=2, B=3, T=6, act="f16"),
}


def klast_case(name: str, seed: int = 2026):
    """Arguments in the reference test's layout (tests/test_k_last_state_dtype.py:55-105
    describes the shapes: slot pitch with a 256-element gap, slots [3, 0, -1], a
    poisoned snapshot cache), built on CPU.

    Returns (args, backing, lengths, state_ids, cache_ids).
    """
    c = KLAST_CASES[name]
    rs = _rs(seed + sum(map(ord, name)))
    act = torch.bfloat16 if c["act"] == "bf16" else torch.float16
    H, HV, B, mode, is_kda = c["H"], c["HV"], c["B"], c["mode"], c["is_kda"]
    T = 1 if mode == "decode" else c["T"]
    lengths = [T] * B
    if mode == "ragged":
        lengths = [T, T // 2, 0]
    nt = sum(lengths)
    slots = max(7, B + 2)
    backing = _t(rs, slots, HV * D * D + 256, dtype=torch.float32, scale=0.1)
    state = backing[:, : HV * D * D].view(slots, HV, D, D)
    state_ids = [3, 0, -1]
    cache_ids = [2, 0, 1]
    cache = None
    if mode != "decode":
        cache = torch.full((max(4, B + 1), T + 3, HV, D, D), -7.0, dtype=torch.float32)
    parents = None
    if mode == "tree":
        parents = torch.tensor([[max(0, t - 2) for t in range(T)]] * B, dtype=torch.int32)
    cu = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32)
    args = dict(
        A_log=_t(rs, HV, dtype=torch.float32),
        a=_t(rs, 1, nt, HV, D, dtype=act) if is_kda else _t(rs, 1, nt, HV, dtype=act),
        dt_bias=(_t(rs, HV, D, dtype=torch.float32 if mode != "decode" else act) if is_kda
                 else _t(rs, HV, dtype=act)),
        softplus_beta=1.0, softplus_threshold=20.0,
        q=_t(rs, 1, nt, H, D, dtype=act), k=_t(rs, 1, nt, H, D, dtype=act), v=_t(rs, 1, nt, HV, D, dtype=act),
        b=_t(rs, 1, nt, HV, dtype=act),
        initial_state_source=state,
        initial_state_indices=torch.tensor(state_ids, dtype=torch.int32),
        scale=D ** -0.5, use_qk_l2norm_in_kernel=True, cu_seqlens=cu, is_kda=is_kda,
        disable_state_update=mode not in ("decode", "writeback"),
        intermediate_states_buffer=cache,
        intermediate_state_indices=None if cache is None else torch.tensor(cache_ids, dtype=torch.int32),
        cache_steps_or_num_accept=None if cache is None else T,
        retrieve_parent_token=parents,
    )
    if c.get("lower_bound") is not None:
        args["lower_bound"] = c["lower_bound"]
    if "is_sglang" in c:
        args["is_sglang"] = c["is_sglang"]
    return args, backing, lengths, state_ids, cache_ids


def oracle_kwargs(args, lengths, state_ids, cache_ids):
    """Translate the reference-layout dict into ``oracle.decode.klast_forward`` keywords."""
    return dict(
        q=args["q"][0], k=args["k"][0], v=args["v"][0], a=args["a"][0], b=args["b"][0],
        A_log=args["A_log"], dt_bias=args["dt_bias"], state=args["initial_state_source"],
        slot_indices=state_ids, lengths=lengths, scale=args["scale"],
        use_qk_l2norm=args["use_qk_l2norm_in_kernel"], is_kda=args["is_kda"],
        lower_bound=args.get("lower_bound"), softplus_beta=args["softplus_beta"],
        softplus_threshold=args["softplus_threshold"], is_sglang=args.get("is_sglang", True),
        disable_state_update=args["disable_state_update"], cache=args["intermediate_states_buffer"],
        cache_indices=cache_ids, parents=args["retrieve_parent_token"],
    )
