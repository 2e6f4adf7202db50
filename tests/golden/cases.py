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
    # bf16 state pools (and snapshot caches), the second half of the reference's state_dtype parametrisation
    # (tests/test_k_last_state_dtype.py:159-163)
    "gdn_decode_sbf16":    dict(mode="decode", is_kda=False, H=2, HV=4, B=3, T=1, act="bf16", state="bf16"),
    "kda_decode_sbf16":    dict(mode="decode", is_kda=True, H=2, HV=2, B=3, T=1, act="f16", state="bf16"),
    "gdn_verify_sbf16":    dict(mode="verify", is_kda=False, H=1, HV=2, B=3, T=4, act="bf16", state="bf16"),
    "gdn_writeback_sbf16": dict(mode="writeback", is_kda=False, H=2, HV=2, B=3, T=3, act="f16", state="bf16"),
    "kda_tree_safe_sbf16": dict(mode="tree", is_kda=True, H=1, HV=2, B=3, T=5, act="bf16", lower_bound=-5.0,
                                state="bf16"),
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
    state_dtype = torch.bfloat16 if c.get("state") == "bf16" else torch.float32
    backing = _t(rs, slots, HV * D * D + 256, dtype=torch.float32, scale=0.1).to(state_dtype)
    state = backing[:, : HV * D * D].view(slots, HV, D, D)
    state_ids = [3, 0, -1]
    cache_ids = [2, 0, 1]
    cache = None
    if mode != "decode":
        cache = torch.full((max(4, B + 1), T + 3, HV, D, D), -7.0, dtype=state_dtype)
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


# --------------------------------------------------------------------------- KDA ReplaySSM
from types import SimpleNamespace  # noqa: E402


def replay_layer(rs, slots, heads, q, layout, padding=256, history=None, conv_offset=0, device="cpu"):
    """One layer's paged cache in the geometry the reference tests use
    (tests/test_kda_replayssm_vllm.py:45-63 describes it): every page holds the bf16 conv
    history, then (16-byte aligned) the fp32 [H,128,128] checkpoint, then padding bytes; the
    whole buffer is pre-filled with 0x5A so that stray writes show up."""
    c = 3 * heads * D
    history = q + 2 if history is None else history
    conv_shape = (c, history) if layout == "DS" else (history, c)
    conv_bytes = c * history * 2
    state_bytes = heads * D * D * 4
    state_offset = -(-(conv_offset + conv_bytes) // 16) * 16
    page_bytes = -(-(state_offset + state_bytes + padding) // 16) * 16
    raw = torch.full((slots * page_bytes,), 0x5A, dtype=torch.uint8)
    conv = raw.view(torch.bfloat16).as_strided((slots, *conv_shape),
                                                (page_bytes // 2, conv_shape[1], 1), conv_offset // 2)
    state = raw.view(torch.float32).as_strided((slots, heads, D, D), (page_bytes // 4, D * D, D, 1),
                                               state_offset // 4)
    conv.copy_(_t(rs, *conv.shape, dtype=torch.bfloat16, scale=0.2))
    state.copy_(_t(rs, *state.shape, dtype=torch.float32, scale=0.01))
    raw = raw.to(device)
    conv = raw.view(torch.bfloat16).as_strided(conv.shape, conv.stride(), conv_offset // 2)
    state = raw.view(torch.float32).as_strided(state.shape, state.stride(), state_offset // 4)
    return SimpleNamespace(raw=raw, kv_cache=(conv, state), heads=heads, q=q, layout=layout, page_bytes=page_bytes)


def replay_inputs(rs, heads, capacity, offset=2, softplus=False, device="cpu"):
    """Projection rows [.., q|k|v|g|beta|pad] carved out of a larger buffer (token stride > width,
    nonzero storage offset), conv taps, gate parameters."""
    c = heads * D
    storage = _t(rs, offset + capacity + 2, 4 * c + heads + 3, dtype=torch.bfloat16, scale=0.4).to(device)
    rows = storage[offset:offset + capacity]
    x = dict(mixed_qkv=rows[:, :3 * c], raw_g=rows[:, 3 * c:4 * c], raw_beta=rows[:, 4 * c:4 * c + heads],
             storage=storage, conv_weight=_t(rs, 3 * c, 4, dtype=torch.float32, scale=0.2).to(device),
             A_log=_t(rs, heads, dtype=torch.float32, scale=0.1).to(device),
             dt_bias=_t(rs, c, dtype=torch.float32, scale=0.2).to(device), lower_bound=None if softplus else -5.0)
    return x


def blank_records(rows, heads, q, device="cpu"):
    shape = (rows, heads, q, D)
    return SimpleNamespace(
        rawv=torch.full(shape, -7, dtype=torch.bfloat16, device=device),
        rawk=torch.full(shape, -7, dtype=torch.bfloat16, device=device),
        g=torch.full(shape, -7.0, device=device), beta=torch.full(shape[:-1], -7.0, device=device),
        conv=torch.full((rows, q, 3 * heads * D, 3), -7, dtype=torch.bfloat16, device=device))


def conv_ds(layer):
    c = layer.kv_cache[0]
    return c if layer.layout == "DS" else c.transpose(-1, -2)


# name -> (layout, q, heads): request lengths [q, q-2, 0, 1, 1], slots [7, 2, 5, 0, -1] on 12 pages
REPLAY_VERIFY_CASES = {
    "sd_q4_h2": ("SD", 4, 2), "ds_q4_h2": ("DS", 4, 2), "sd_q1_h1": ("SD", 1, 1), "ds_q5_h1": ("DS", 5, 1),
    "sd_q8_h1": ("SD", 8, 1),
    "ds_q10_h1": ("DS", 10, 1),     # longer than eight tokens: the token-by-token verify kernel
}


def replay_verify_case(name, device="cpu"):
    layout, q, heads = REPLAY_VERIFY_CASES[name]
    rs = _rs(4100 + sum(map(ord, name)))
    lengths = [q, max(q - 2, 0), 0, 1, 1]
    offsets = [0]
    for n in lengths:
        offsets.append(offsets[-1] + n)
    slots = [7, 2, 5, 0, -1]
    layer = replay_layer(rs, 12, heads, q, layout, device=device)
    x = replay_inputs(rs, heads, len(slots) * q + 3, device=device)
    return layer, x, offsets, slots, lengths


# Commit scenarios: 3 request rows on 24 pages, 2 layers, Q = 5, heads = 2.
REPLAY_COMMIT_CASES = {
    "plain_t0": dict(align=False, turn=0), "plain_t1": dict(align=False, turn=1),
    "align_t0": dict(align=True, turn=0), "align_t2": dict(align=True, turn=2),
    "align_t3": dict(align=True, turn=3),
}


def replay_commit_case(name, layout="SD", device="cpu"):
    """Metadata of one commit round: request lengths, sampler mapping, accepted counts and (align
    mode) a block table with 8-token blocks, after the scenario family of the reference's commit
    test (tests/test_kda_replayssm_vllm.py:489-520)."""
    cfg = REPLAY_COMMIT_CASES[name]
    q, heads, rows = 5, 2, 3
    rs = _rs(5700 + sum(map(ord, name)))
    layers = [replay_layer(rs, 24, heads, q, layout, 256 + i * 64, device=device) for i in range(2)]
    x = replay_inputs(rs, heads, rows * q + 2, device=device)
    turn, align = cfg["turn"], cfg["align"]
    lengths = [q, 3, 1] if turn % 2 == 0 else [1, q, 0]
    offsets = [0, lengths[0], sum(lengths[:2]), sum(lengths)]
    mapping = [2, 0, 3]
    counts = ([2, 777, q, 0], [-3, 777, 1, q + 10], [q, 777, 0, 1], [q + 10, 777, 1, 0])[turn % 4]
    table = [[1 + r * 6 + j for j in range(4)] for r in range(4)]
    computed = [6, 1, 7, 8]
    order = [2, 9, 16]
    order = order[(turn + 1) % 3:] + order[:(turn + 1) % 3]
    slots = [table[mapping[b]][(computed[mapping[b]] - 1) // 8] for b in range(rows)] if align else order
    return dict(layers=layers, x=x, q=q, heads=heads, rows=rows, offsets=offsets, slots=slots, mapping=mapping,
                counts=counts, table=table if align else None, computed=computed if align else None,
                block_size=8 if align else None)


def plan_scenarios():
    """Conflict-masking scenarios with their expected plans
    (after tests/test_kda_replayssm_vllm.py:980-1160: a destination equal to another row's source,
    duplicate finals, a boundary slot owned by another row, int64 sources beyond int32, and the
    block-table known answer)."""
    out = []
    for batch in (2, 5, 40):
        for align in (True, False):
            q, capacity = 4, batch + 3
            names = (("c0_owner", "empty_owner", "duplicate_final", "boundary_source", "reverse_source", "disjoint",
                      "wide_source") if align else
                     ("c0_owner", "empty_owner", "duplicate_final", "disjoint", "wide_source", "wide_length"))
            for variant in names:
                sources = list(range(1, batch + 1))
                offsets = [i * q for i in range(batch + 1)]
                counts = [0] * batch
                counts[0] = 1
                table = [[batch + 1 + i, batch + 1 + i] for i in range(batch)]
                positions = [8] * batch
                if variant in ("c0_owner", "empty_owner"):
                    table[0][1] = sources[-1]
                    if variant == "empty_owner":
                        offsets[-1] = offsets[-2]
                elif variant == "duplicate_final":
                    counts[-1] = 1
                    table[-1][1] = table[0][1]
                elif variant == "boundary_source":
                    counts[0], counts[-1], positions[0] = 2, 1, 7
                    table[0][0] = sources[-1]
                elif variant == "reverse_source":
                    counts[-1] = 1
                    table[-1][1] = sources[0]
                elif variant == "disjoint":
                    counts[0], counts[-1] = 2, 1
                else:
                    sources[-1] = 2 ** 32 + table[0][1]
                if not align:
                    if variant in ("c0_owner", "empty_owner", "duplicate_final", "wide_length"):
                        sources[-1] = sources[0]
                    elif variant == "wide_source":
                        sources[-1] = 2 ** 32 + sources[0]
                    if variant == "wide_length":
                        offsets[-1] += 2 ** 32
                out.append(dict(name=f"{variant}_b{batch}_{'align' if align else 'plain'}", sources=sources,
                                offsets=offsets, counts=counts, table=table if align else None,
                                positions=positions if align else None, block_size=8 if align else 0, q=q,
                                capacity=capacity, slots=2 * batch + 8, token_capacity=batch * q,
                                blocked=variant in ("c0_owner", "duplicate_final", "boundary_source",
                                                    "reverse_source")))
    return out


# --------------------------------------------------------------------------- prefill
PREFILL_CASES = {
    # name: (lengths, padded_tokens, Hg, H)
    "gdn_two_seqs": ([97, 50], 3, 1, 2),
    "gdn_chunk_edges": ([64, 1, 129], 0, 2, 4),
}


def gdn_prefill_case(name, device="cpu"):
    """Packed varlen GDN prefill inputs: a [T, Q|K|V] buffer cut out of a wider one (row pitch
    +64 elements, first column 17 -> rows are only 2-byte aligned), raw gates as two column
    slices of one [T, 2H] buffer, fp32 A_log ~ U(0, log 16) and dt_bias ~ N(0, 0.1), an indexed
    fp32 pool [16, H, DV, DK] ~ N(0, 0.02) with non-consecutive slots."""
    lengths, pad, Hg, H = PREFILL_CASES[name]
    rs = _rs(7300 + sum(map(ord, name)))
    T = sum(lengths) + pad
    width = 2 * Hg * D + H * D
    storage = _t(rs, T, width + 64, dtype=torch.bfloat16).to(device)
    packed = storage[:, 17:17 + width]
    gates = _t(rs, T, 2 * H, dtype=torch.bfloat16).to(device)
    A_log = torch.from_numpy(rs.uniform(0.0, np.log(16.0), H).astype(np.float32)).to(device)
    dt_bias = _t(rs, H, dtype=torch.float32, scale=0.1).to(device)
    pool = _t(rs, 16, H, D, D, dtype=torch.float32, scale=0.02).to(device)
    slots = [11, 2, 7, 14][:len(lengths)]
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + n)
    return dict(packed=packed, storage=storage, a=gates[:, :H], b=gates[:, H:], A_log=A_log, dt_bias=dt_bias,
                pool=pool, slots=slots, cu=cu, lengths=lengths, T=T, Hg=Hg, H=H)


def gdn_prefill_oracle_kwargs(c):
    """The case as ``oracle.decode.klast_forward`` keywords (token-level fp32 recurrence)."""
    Hg, H = c["Hg"], c["H"]
    p = c["packed"]
    T = c["T"]
    q = p[:, : Hg * D].reshape(T, Hg, D)
    k = p[:, Hg * D: 2 * Hg * D].reshape(T, Hg, D)
    v = p[:, 2 * Hg * D:].reshape(T, H, D)
    return dict(q=q, k=k, v=v, a=c["a"], b=c["b"], A_log=c["A_log"], dt_bias=c["dt_bias"], state=c["pool"],
                slot_indices=c["slots"], lengths=c["lengths"], scale=D ** -0.5, use_qk_l2norm=True)


KDA_PREFILL_CASES = {"kda_two_seqs": ([70, 41], 2, 2), "kda_one_seq": ([130], 0, 1)}


def kda_prefill_case(name, softplus=False, device="cpu"):
    lengths, pad, H = KDA_PREFILL_CASES[name]
    rs = _rs(8100 + sum(map(ord, name)))
    T = sum(lengths) + pad
    mk = lambda *s, sc=1.0: _t(rs, *s, dtype=torch.bfloat16, scale=sc).to(device)  # noqa: E731
    q, k, v, g = mk(T, H, D), mk(T, H, D), mk(T, H, D), mk(T, H, D)
    beta = mk(T, H)
    A_log = _t(rs, H, dtype=torch.float32, scale=0.3).to(device)
    dt_bias = _t(rs, H, D, dtype=torch.float32, scale=0.2).to(device)
    init = _t(rs, len(lengths), H, D, D, dtype=torch.float32, scale=0.02).to(device)
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + n)
    return dict(q=q, k=k, v=v, g=g, beta=beta, A_log=A_log, dt_bias=dt_bias, init=init, cu=cu, lengths=lengths, T=T,
                H=H, lower_bound=None if softplus else -5.0)


# ---- SGLang ReplaySSM contract (fused_kda_decode_mtp_dspark / commit_kda_replayssm_after_verify) ----
SGLANG_VERIFY_CASES = {"sg_dense": dict(bs=3, dtn=4, heads=2, ring=6, slots=6, onorm=False, pad=False),
                       "sg_onorm_pad": dict(bs=4, dtn=3, heads=2, ring=4, slots=7, onorm=True, pad=True)}


def sglang_verify_case(name, device="cpu"):
    """Input dict with the entry point's keyword names. Slots are a non-trivial permutation, the
    scratch rows are reversed, q/k/v/g are views with a padded token stride."""
    c = SGLANG_VERIFY_CASES[name]
    rs = _rs(sum(map(ord, name)))
    bs, dtn, H, L, slots = c["bs"], c["dtn"], c["heads"], c["ring"], c["slots"]
    T, dim = bs * dtn, c["heads"] * D
    mixed = _t(rs, 1, T, 4 * dim + 64, scale=0.5)                       # q | k | v | g thirds of one row + padding
    x_q, x_k, x_v, g = (mixed[..., i * dim:(i + 1) * dim].view(1, T, H, D) for i in range(4))
    vi = dict(
        x_q=x_q, x_k=x_k, x_v=x_v, g=g, beta=_t(rs, 1, T, H),
        w_q=_t(rs, dim, 4, dtype=torch.float32, scale=0.3), w_k=_t(rs, dim, 4, dtype=torch.float32, scale=0.3),
        w_v=_t(rs, dim, 4, dtype=torch.float32, scale=0.3),
        A_log=torch.from_numpy(rs.uniform(0.5, 1.0, H).astype("float32")),
        dt_bias=_t(rs, dim, dtype=torch.float32, scale=0.1),
        recurrent_state=_t(rs, slots, H, D, D, dtype=torch.float32, scale=0.1),
        lower_bound=-8.0, scale=D ** -0.5, intermediate_ssm=None,
        replayssm_rawv=torch.full((slots, H, L, D), -3.0, dtype=torch.bfloat16),
        replayssm_rawk=torch.full((slots, H, L, D), -3.0, dtype=torch.bfloat16),
        replayssm_g=torch.full((slots, H, L, D), -3.0), replayssm_beta=torch.full((slots, H, L), -3.0),
    )
    conv = _t(rs, slots, 3, 3 * dim, scale=0.3)                          # [slots, width, 3*dim] pool, split + transposed
    vi["cs_q"], vi["cs_k"], vi["cs_v"] = (conv[..., i * dim:(i + 1) * dim].transpose(-1, -2) for i in range(3))
    ic = torch.full((bs + 1, dtn, 3 * dim, 3), -3.0, dtype=torch.bfloat16)
    vi["intermediate_conv_q"], vi["intermediate_conv_k"], vi["intermediate_conv_v"] = (
        ic[:, :, i * dim:(i + 1) * dim] for i in range(3))
    order = rs.permutation(slots)[:bs].astype("int32")
    if c["pad"]:
        order[1] = -1
    vi["ssm_state_indices"] = torch.from_numpy(order)
    vi["intermediate_state_indices"] = torch.arange(bs - 1, -1, -1, dtype=torch.int64)
    vi["cu_seqlens"] = torch.arange(0, T + 1, dtn, dtype=torch.int32)
    if c["onorm"]:
        vi["onorm_gate"] = _t(rs, 1, T, H, D, scale=0.5)
        vi["onorm_weight"] = torch.from_numpy(rs.uniform(0.75, 1.25, D).astype("float32"))
        vi["onorm_eps"] = 1e-6
    if device != "cpu":
        base = {id(mixed): mixed.to(device), id(conv): conv.to(device), id(ic): ic.to(device)}
        dm, dc, di = base[id(mixed)], base[id(conv)], base[id(ic)]
        moved = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in vi.items()}
        for i, key in enumerate(("x_q", "x_k", "x_v", "g")):
            moved[key] = dm[..., i * dim:(i + 1) * dim].view(1, T, H, D)
        for i, key in enumerate(("cs_q", "cs_k", "cs_v")):
            moved[key] = dc[..., i * dim:(i + 1) * dim].transpose(-1, -2)
        for i, key in enumerate(("intermediate_conv_q", "intermediate_conv_k", "intermediate_conv_v")):
            moved[key] = di[:, :, i * dim:(i + 1) * dim]
        vi = moved
    return vi, c


SGLANG_COMMIT_CASES = {"sg_commit": dict(bs=4, dtn=4, heads=2, k_heads=2, ring=5, slots=7, layers=2, track=False),
                       "sg_commit_track_gva": dict(bs=4, dtn=3, heads=4, k_heads=2, ring=4, slots=7, layers=1, track=True)}


def sglang_commit_case(name, device="cpu"):
    """Tensors for commit_kda_replayssm_after_verify: state, rings, one conv pool + window list."""
    c = SGLANG_COMMIT_CASES[name]
    rs = _rs(sum(map(ord, name)))
    bs, dtn, HV, H, L, slots, nl = c["bs"], c["dtn"], c["heads"], c["k_heads"], c["ring"], c["slots"], c["layers"]
    dim = 3 * HV * D
    ci = dict(
        temporal=_t(rs, nl, slots, HV, D, D, dtype=torch.float32, scale=0.1),
        rawv=_t(rs, nl, slots, HV, L, D, scale=0.5), rawk=_t(rs, nl, slots, H, L, D, scale=0.5),
        gk=-torch.from_numpy(rs.uniform(0, 0.5, (nl, slots, HV, L, D)).astype("float32")),
        beta=torch.from_numpy(rs.uniform(0, 1, (nl, slots, HV, L)).astype("float32")),
        conv=[_t(rs, nl, slots, dim, 3)], intermediate_conv_window=[_t(rs, nl, bs, dtn, dim, 3)],
    )
    order = rs.permutation(slots)[:bs].astype("int64")
    order[bs - 1] = -1                                                      # a padding request
    accept = np.array([(i % dtn) + 1 for i in range(bs)], dtype="int32")
    accept[0] = 0                                                           # commits nothing
    ci["state_batch_indices"] = torch.from_numpy(order)
    ci["accept_lens"] = torch.from_numpy(accept)
    ci["last_correct_step_indices"] = torch.from_numpy(accept.astype("int64") - 1)
    if c["track"]:
        free = [s for s in range(slots) if s not in order.tolist()]
        # request 1 snapshots after its first step, request 2 after its last one
        ci["mamba_track_indices"] = torch.tensor([-1, free[0], free[1], -1][:bs], dtype=torch.int64)
        ci["mamba_steps_to_track"] = torch.tensor([0, 0, 2, 0][:bs], dtype=torch.int64)
    if device != "cpu":
        ci = {k: ([t.to(device) for t in v] if isinstance(v, list) else v.to(device)) for k, v in ci.items()}
    return ci, c


# ---- fused KDA decode step (fused_kda_decode_mega_forward) ----
MEGA_CASES = {"mega_h4_norm": dict(H=4, B=3, lower_bound=-5.0, norm=True, dtype="bf16"),
              "mega_h6_softplus": dict(H=6, B=2, lower_bound=None, norm=False, dtype="bf16"),
              "mega_h4_fp16_bias": dict(H=4, B=2, lower_bound=-5.0, norm=True, dtype="fp16")}


def mega_case(name, device="cpu", pad_rows=()):
    """Inputs shaped like the reference's own builder (compare_kda_decode_fusion.py:128-186): padded rows of
    x / raw_beta / output_gate, conv state stored [slots, 3, 3*dim] and viewed [slots, 3*dim, 3], slots in
    descending order (slot 0 included)."""
    c = MEGA_CASES[name]
    rs = _rs(sum(map(ord, name)))
    H, B = c["H"], c["B"]
    dt = torch.bfloat16 if c["dtype"] == "bf16" else torch.float16
    dim, slots = H * D, B + 2
    x = _t(rs, B, 3 * dim + 17, dtype=dt)[:, :3 * dim]
    weight = _t(rs, 3, 4, dim, dtype=torch.float32, scale=0.1)
    bias = _t(rs, 3 * dim, dtype=torch.float32, scale=0.05) if "bias" in name else None
    conv_state = _t(rs, slots, 3, 3 * dim, dtype=dt, scale=0.1).transpose(1, 2)
    raw_g = _t(rs, 1, B, H, D, dtype=dt)
    raw_beta = _t(rs, 1, B, H + 1, dtype=dt)[:, :, :H]
    output_gate = _t(rs, B, dim + 8, dtype=dt)[:, :dim].view(B, H, D)
    norm_weight = _t(rs, D, dtype=torch.float32)
    A_log = _t(rs, H, dtype=torch.float32, scale=0.5)
    dt_bias = _t(rs, dim, dtype=torch.float32, scale=0.1)
    idx = torch.arange(B - 1, -1, -1, dtype=torch.int32)
    for r in pad_rows:
        idx[r] = -1
    state = _t(rs, slots, H, D, D, dtype=torch.float32, scale=0.01)
    kw = dict(x=x, weight=weight, bias=bias, conv_state=conv_state, raw_g=raw_g, raw_beta=raw_beta, a_log=A_log,
              dt_bias=dt_bias, state_indices=idx, state=state, lower_bound=c["lower_bound"],
              output_gate=output_gate if c["norm"] else None, norm_weight=norm_weight if c["norm"] else None,
              norm_eps=1e-5)
    if device != "cpu":
        moved = {}
        for k_, v_ in kw.items():
            if not isinstance(v_, torch.Tensor):
                moved[k_] = v_
            elif k_ in ("x", "raw_beta", "output_gate", "conv_state"):      # keep the padded / transposed views
                base = v_._base if v_._base is not None else v_
                moved[k_] = torch.as_strided(base.to(device), v_.shape, v_.stride(), v_.storage_offset())
            else:
                moved[k_] = v_.to(device)
        kw = moved
    return kw, c


CONV_CASES = {
    # lengths straddle the 8/16/32/64-row tiles; a start one and two rows before a tile edge; an empty sequence
    "conv_mixed": dict(C=256, lengths=[5, 0, 1, 2, 70, 3, 62, 1, 130], slots=12, layout="SD", bias=True, dtype="bf16",
                       extra_rows=5, has_initial=[1, 1, 0, 1, 1, 1, 0, 1, 1], pads=(5,)),
    "conv_ds_fp16": dict(C=136, lengths=[33, 2, 95], slots=5, layout="DS", bias=False, dtype="fp16", extra_rows=0,
                         has_initial=None, pads=()),
}


def conv_case(name, device="cpu"):
    """Packed rows with a row pitch wider than the channel count, history pool stored [slots, 3, C] ("SD", viewed
    [slots, C, 3]) or [slots, C, 3] ("DS"), slots in a scrambled order, optional padding slots (-1)."""
    c = CONV_CASES[name]
    rs = _rs(sum(map(ord, name)))
    C, lengths = c["C"], c["lengths"]
    dt = torch.bfloat16 if c["dtype"] == "bf16" else torch.float16
    total = sum(lengths)
    rows = total + c["extra_rows"]
    x = _t(rs, rows, C + 24, dtype=dt)[:, :C]
    weight = _t(rs, C, 4, dtype=torch.float32, scale=0.4)
    bias = _t(rs, C, dtype=torch.float32, scale=0.1) if c["bias"] else None
    if c["layout"] == "SD":
        conv_state = _t(rs, c["slots"], 3, C, dtype=dt, scale=0.5).transpose(1, 2)
    else:
        conv_state = _t(rs, c["slots"], C, 3, dtype=dt, scale=0.5)
    idx = torch.tensor(rs.permutation(c["slots"])[:len(lengths)].astype("int32"))
    for r in c["pads"]:
        idx[r] = -1
    offsets = [0]
    for n in lengths:
        offsets.append(offsets[-1] + n)
    has = None if c["has_initial"] is None else torch.tensor(c["has_initial"], dtype=torch.bool)
    kw = dict(x=x, weight=weight, bias=bias, conv_state=conv_state, offsets=offsets, state_indices=idx,
              has_initial_state=has)
    if device != "cpu":
        moved = {}
        for k_, v_ in kw.items():
            if not isinstance(v_, torch.Tensor):
                moved[k_] = v_
            elif k_ in ("x", "conv_state"):                                  # keep the padded / transposed views
                base = v_._base if v_._base is not None else v_
                moved[k_] = torch.as_strided(base.to(device), v_.shape, v_.stride(), v_.storage_offset())
            else:
                moved[k_] = v_.to(device)
        kw = moved
    return kw, c
