"""Generates the golden fixtures by running the REFERENCE's own PyTorch oracles.

Run where the reference tree is mounted:
    python tests/golden/make_golden.py /path/to/reference [klast|replay|prefill|sglang|mega|conv]
Nothing from the reference is copied: its functions are loaded from the tree at
run time, fed the seeded inputs of ``cases.py`` and only their outputs are saved.
"""
from __future__ import annotations

import ast
import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import cases  # noqa: E402

if __name__ == "__main__" and len(sys.argv) < 2:
    sys.exit("usage: make_golden.py /path/to/reference [klast|replay|prefill|sglang|mega|conv]")
REF = Path(sys.argv[1]) if len(sys.argv) > 1 else Path("reference")


def load_function(path: Path, name: str, namespace: dict):
    """Compile one top-level function of a reference file without importing the
    module (its imports need the PPU extension)."""
    tree = ast.parse(path.read_text())
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == name)
    exec(compile(ast.Module([fn], []), str(path), "exec"), namespace)
    return namespace[name]


def make_klast():
    reference = load_function(REF / "tests" / "test_k_last_state_dtype.py", "reference", {"torch": torch, "F": F})
    for name in cases.KLAST_CASES:
        args, backing, lengths, state_ids, cache_ids = cases.klast_case(name)
        out, state, cache = reference(args, lengths, state_ids, cache_ids)
        blob = dict(out=out.float().numpy(), state=cases.subsample(state),
                    state_sum=np.float64(state.double().sum().item()))
        if cache is not None:
            blob["cache"] = cases.subsample(cache)
            blob["cache_sum"] = np.float64(cache.double().sum().item())
        np.savez_compressed(HERE / f"klast_{name}.npz", **blob)
        print("klast", name, {k: getattr(v, "shape", None) for k, v in blob.items()})


def load_replay_reference():
    """The reference's vLLM replay test module: its fp64 oracle adapters are plain functions
    (the PPU extension is only imported inside the functions that launch kernels)."""
    import importlib.util
    sys.dont_write_bytecode = True
    sys.path.insert(0, str(REF / "tests"))
    spec = importlib.util.spec_from_file_location("ref_replay_test", REF / "tests" / "test_kda_replayssm_vllm.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def make_replay():
    ref = load_replay_reference()
    import json
    for name in cases.REPLAY_VERIFY_CASES:
        layer, x, offsets, slots, lengths = cases.replay_verify_case(name)
        records = cases.blank_records(len(slots), layer.heads, layer.q)
        out = torch.full((x["mixed_qkv"].shape[0], layer.heads * 128), -11, dtype=torch.bfloat16)
        want_out, want = ref.oracle_verify(layer, x, offsets, slots, records, out, 0)
        np.savez_compressed(HERE / f"replay_verify_{name}.npz", out=want_out.float().numpy(),
                            rawv=want.rawv.float().numpy(), rawk=want.rawk.float().numpy(), g=want.g.numpy(),
                            beta=want.beta.numpy(), conv=want.conv.float().numpy())
        print("replay verify", name, tuple(want_out.shape))
    for name in cases.REPLAY_COMMIT_CASES:
        c = cases.replay_commit_case(name)
        blob = {}
        for li, layer in enumerate(c["layers"]):
            records = cases.blank_records(c["rows"], c["heads"], c["q"])
            out = torch.full((c["x"]["mixed_qkv"].shape[0], c["heads"] * 128), -11, dtype=torch.bfloat16)
            _, want = ref.oracle_verify(layer, c["x"], c["offsets"], c["slots"], records, out, 0)
            state, conv, plan = ref.oracle_commit(layer, want, c["offsets"], c["slots"], c["counts"], c["mapping"],
                                                  c["table"], c["computed"], c["block_size"])
            touched = sorted({s for n, f, b, bc in zip(*plan) if n for s in ([f, b] if bc else [f])})
            blob[f"state_l{li}"] = cases.subsample(state[touched]) if touched else np.zeros((0,), np.float32)
            blob[f"conv_l{li}"] = conv[touched][:, :, :3].float().numpy() if touched else np.zeros((0,), np.float32)
            blob["touched"] = np.array(touched, dtype=np.int64)
            blob["plan"] = np.array(plan, dtype=np.int64)
        np.savez_compressed(HERE / f"replay_commit_{name}.npz", **blob)
        print("replay commit", name, blob["plan"].tolist())
    plans = {}
    for sc in cases.plan_scenarios():
        layer = cases.replay_layer(np.random.RandomState(1), sc["slots"], 1, sc["q"], "DS")
        rec = cases.blank_records(sc["capacity"], 1, sc["q"])
        for key, val in (("rawv", .1), ("rawk", .2), ("g", -.1), ("beta", .5), ("conv", .3)):
            getattr(rec, key).fill_(val)
        batch = len(sc["sources"])
        expected_counts = [0] * batch if sc["blocked"] else sc["counts"]
        _, _, plan = ref.oracle_commit(layer, rec, sc["offsets"], sc["sources"], expected_counts,
                                       block_table=sc["table"], computed=sc["positions"],
                                       block_size=sc["block_size"] or None)
        plans[sc["name"]] = [col + [0] * (sc["capacity"] - batch) for col in plan]
    # known answer stated by the reference for block_table=[[3,4]], computed=[7], block 8, 4 sampled of Q=4
    plans["known_answer_block_boundary"] = [[2], [4], [3], [1]]
    (HERE / "replay_plans.json").write_text(json.dumps(plans, indent=0))
    print("plans", len(plans))


def make_sglang():
    """SGLang-contract verify and fold: the reference's fp64 oracle
    (scripts/decode/kda_mtp_sglang/private/_reference.py:92-216) on the cases of cases.py."""
    import importlib.util
    from types import SimpleNamespace
    spec = importlib.util.spec_from_file_location(
        "ref_sglang", REF / "scripts" / "decode" / "kda_mtp_sglang" / "private" / "_reference.py")
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    for name in cases.SGLANG_VERIFY_CASES:
        vi, c = cases.sglang_verify_case(name)
        cfg = SimpleNamespace(heads=c["heads"], T=c["bs"] * c["dtn"], draft_token_num=c["dtn"], ring_len=c["ring"],
                              slots=c["slots"], bs=c["bs"])
        feed = {k: v for k, v in vi.items() if v is not None}
        want = ref.verify_reference(feed, cfg)
        np.savez_compressed(HERE / f"sglang_verify_{name}.npz", **{k: v.float().numpy() for k, v in want.items()})
        print("sglang verify", name, tuple(want["out"].shape))
    for name in cases.SGLANG_COMMIT_CASES:
        ci, c = cases.sglang_commit_case(name)
        want = ref.fold_reference(ci, None)
        touched = sorted({int(s) for s, n in zip(ci["state_batch_indices"], ci["accept_lens"]) if s >= 0 and n > 0})
        np.savez_compressed(HERE / f"sglang_fold_{name}.npz", touched=np.array(touched),
                            state=cases.subsample(want[:, touched].float()),
                            state_sum=np.float64(want[:, touched].sum().item()))
        print("sglang fold", name, touched)


def make_mega():
    """Fused KDA decode step: the reference's step-by-step fp32 recurrence
    (scripts/decode/kda_fusion/compare_kda_decode_fusion.py:252-308, extracted by name because the module
    imports GPU-only code at its top) on the cases of cases.py. Its result dtype is fp16 by construction."""
    import math
    path = REF / "scripts" / "decode" / "kda_fusion" / "compare_kda_decode_fusion.py"
    ns = {"torch": torch, "math": math, "D": 128, "W": 4, "NORM_EPS": 1e-5, "DEVICE": "cpu",
          "SCALE": 1.0 / math.sqrt(128)}
    load_function(path, "_silu", ns)
    ref = load_function(path, "torch_reference_fp16", ns)
    for name in cases.MEGA_CASES:
        kw, c = cases.mega_case(name)
        assert kw["bias"] is None or name.endswith("bias")
        inp = {"num_seqs": c["B"], "num_heads": c["H"], "packed_x": kw["x"], "fused_weight": kw["weight"],
               "conv_seed": kw["conv_state"], "raw_g": kw["raw_g"], "raw_beta": kw["raw_beta"], "A_log": kw["a_log"],
               "dt_bias": kw["dt_bias"], "state_seed": kw["state"], "state_indices": kw["state_indices"],
               "output_gate": kw["output_gate"] if c["norm"] else torch.zeros(c["B"], c["H"], 128),
               "norm_weight": kw["norm_weight"] if c["norm"] else torch.ones(128)}
        if kw["bias"] is not None:
            continue    # the reference recurrence has no bias term: that case is checked against the oracle only
        out, state, conv = ref(inp, c["lower_bound"], c["norm"])
        touched = sorted(int(s) for s in kw["state_indices"])
        np.savez_compressed(HERE / f"mega_{name}.npz", out=out.float().numpy(),
                            state=cases.subsample(state[touched]), conv=conv[touched].float().numpy(),
                            touched=np.array(touched))
        print("mega", name, tuple(out.shape))


def make_prefill():
    """GDN: the vendored chunked torch reference the reference's own prefill tests compare with
    (scripts/prefill/flashqla/private/ref_gdr.py, chunk 64, called per sequence as in
    tests/prefill_utils.py:272-283). KDA: naive_recurrent_kda with the gate helpers of
    scripts/decode/_kda_reference.py."""
    import importlib.util
    sys.path.insert(0, str(REF / "scripts" / "prefill" / "flashqla"))
    from private import ref_gdr
    for name in cases.PREFILL_CASES:
        c = cases.gdn_prefill_case(name)
        kw = cases.gdn_prefill_oracle_kwargs(c)
        q = kw["q"].float() * torch.rsqrt(kw["q"].float().square().sum(-1, keepdim=True) + 1e-6)
        k = kw["k"].float() * torch.rsqrt(kw["k"].float().square().sum(-1, keepdim=True) + 1e-6)
        g = -c["A_log"].exp() * F.softplus(c["a"].float() + c["dt_bias"])
        beta = torch.sigmoid(c["b"].float())
        outs, finals = [], []
        for i, n in enumerate(c["lengths"]):
            sl = slice(c["cu"][i], c["cu"][i + 1])
            h0 = c["pool"][c["slots"][i]].transpose(-1, -2)[None].float()       # [1,H,DK,DV]
            _, o_i, _, _, h_i = ref_gdr.chunk_gated_delta_rule_fwd(
                q[None, sl], k[None, sl], kw["v"][None, sl].float(), g[None, sl], beta[None, sl],
                cu_seqlens=torch.tensor([0, n]), initial_state=h0, chunk_size=64)
            outs.append(o_i.reshape(n, c["H"], 128))
            finals.append(h_i.reshape(c["H"], 128, 128).transpose(-1, -2))
        np.savez_compressed(HERE / f"prefill_{name}.npz", out=torch.cat(outs).float().numpy(),
                            final=cases.subsample(torch.stack(finals)))
        print("prefill", name, torch.cat(outs).shape)
    spec = importlib.util.spec_from_file_location("ref_kda", REF / "scripts" / "decode" / "_kda_reference.py")
    kda = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(kda)
    for name in cases.KDA_PREFILL_CASES:
        for softplus in (False, True):
            c = cases.kda_prefill_case(name, softplus=softplus)
            if softplus:
                g = kda.naive_kda_gate(c["g"], c["A_log"], c["dt_bias"])
            else:
                g = kda.naive_kda_lowerbound_gate(c["g"], c["A_log"], c["dt_bias"], lower_bound=-5.0)
            qn = c["q"].float() * torch.rsqrt(c["q"].float().square().sum(-1, keepdim=True) + 1e-6)
            kn = c["k"].float() * torch.rsqrt(c["k"].float().square().sum(-1, keepdim=True) + 1e-6)
            outs, finals = [], []
            for i, n in enumerate(c["lengths"]):
                sl = slice(c["cu"][i], c["cu"][i + 1])
                o_i, S = kda.naive_recurrent_kda(qn[None, sl], kn[None, sl], c["v"][None, sl].float(), g[None, sl],
                                                 torch.sigmoid(c["beta"][None, sl].float()),
                                                 initial_state=c["init"][i].transpose(-1, -2)[None],
                                                 output_final_state=True)
                outs.append(o_i[0])
                finals.append(S[0].transpose(-1, -2))
            tag = "softplus" if softplus else "safe"
            np.savez_compressed(HERE / f"prefill_{name}_{tag}.npz", out=torch.cat(outs).float().numpy(),
                                final=cases.subsample(torch.stack(finals)))
            print("prefill", name, tag)


def make_conv():
    """Prefill causal conv: the reference's per-sequence conv oracle (scripts/decode/kda_mtp_sglang/private/
    _reference.py:67-89) run in fp64 over every sequence of the cases of cases.py; the last window is the history
    a request keeps."""
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "ref_sglang", REF / "scripts" / "decode" / "kda_mtp_sglang" / "private" / "_reference.py")
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    for name in cases.CONV_CASES:
        kw, c = cases.conv_case(name)
        x, state, offs = kw["x"], kw["conv_state"], kw["offsets"]
        y = torch.zeros(x.shape, dtype=torch.float64)
        final = state.double().clone()
        for s, (beg, end) in enumerate(zip(offs, offs[1:])):
            if end == beg:
                continue
            slot = int(kw["state_indices"][s])
            reads = slot >= 0 and (kw["has_initial_state"] is None or bool(kw["has_initial_state"][s]))
            hist = state[slot].double() if reads else torch.zeros(c["C"], 3, dtype=torch.float64)
            # the oracle has no bias and always applies SiLU: fold the bias in as a fifth tap on a constant-one input
            out, win = ref._causal_conv_silu(x[beg:end].double(), hist, kw["weight"].double())
            if kw["bias"] is not None:
                pre = sum(torch.cat([hist.t(), x[beg:end].double()])[j:j + end - beg] * kw["weight"].double()[:, j] for j in range(4))
                assert torch.allclose(out, pre * torch.sigmoid(pre), atol=1e-12)
                pre = pre + kw["bias"].double()
                out = pre * torch.sigmoid(pre)
            y[beg:end] = out
            if slot >= 0:
                final[slot] = win[-1]
        np.savez_compressed(HERE / f"{name}.npz", y=y.float().numpy(), final=final.float().numpy())
        print("conv", name, tuple(y.shape))


if __name__ == "__main__":
    torch.manual_seed(0)
    which = sys.argv[2] if len(sys.argv) > 2 else "all"
    if which in ("all", "klast"):
        make_klast()
    if which in ("all", "replay"):
        make_replay()
    if which in ("all", "prefill"):
        make_prefill()
    if which in ("all", "sglang"):
        make_sglang()
    if which in ("all", "mega"):
        make_mega()
    if which in ("all", "conv"):
        make_conv()
