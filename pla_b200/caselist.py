"""Case records of the reference's shape corpus: parse, format, replay.

A record is one line such as
``[GDN]:[D][8]gdn_attn:seqlen_q:1,head_dim_qk:128,head_dim_v:128,num_heads_qk:16,num_heads_v:32,hidden_act:silu,conv_kdim:4,batch_size:8,dtype:bf16.``
or, for packed prefill, ``[KDA]:[P][2,200]kda_attn:...,gate_lower_bound:-5.0,batch_size:2,dtype:bf16,cu_seqlens_q:[0,24,88].``
The grammar is the one the reference's ops print (``generate_ut_tag``, src/op_forge_case.h:149-212) and its test
tools read (``parse_pla_string_re``, tests/utils.py:135-170): a model tag, ``[D]`` (decode / verify, fixed
``seqlen_q`` rows per request, optional ``verify_lens``) or ``[P]`` (packed prefill with ``cu_seqlens_q``), then
``key:value`` pairs. ``replay`` builds seeded synthetic inputs of a record's shape, runs this library's op for it
on the GPU and times it; with ``check=True`` prefill records are also evaluated by the exact token recurrence on
the GPU and the two results compared. ``python -m pla_b200.caselist FILE_OR_DIR`` replays lists. ``build_inputs`` /
``run_inputs`` are the two halves of a replay, for callers that want to judge the results themselves.

``PLA_SHOW_PARAMS=1`` makes the facades print the record of every call (``show_case``), so a serving run on this
library yields lists the reference's tools can replay, and the reverse.
"""
from __future__ import annotations

import ast
import json
import math
import os
import re
import sys
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence

D = 128
_PAIR = re.compile(r"(\w+):(\[.*?\]|[^,]+)")
_HEAD = re.compile(r"\[(\w+)\]:\[([PD])\]\[([\d,\s]*)\](\w+):")


def parse_case(line: str) -> Dict:
    """One record -> dict. Integer, float and list values are converted; unknown keys are kept as they are.
    Adds ``model`` (GDN / KDA / ...), ``phase`` (P / D), ``op`` and ``_raw_line``. Raises ``ValueError`` on a
    line that is not a record."""
    text = line.strip()
    head = _HEAD.search(text)
    if head is None:
        raise ValueError(f"not a case record: {text[:80]!r}")
    case: Dict = {"model": head.group(1), "phase": head.group(2), "op": head.group(4), "_raw_line": text}
    for key, value in _PAIR.findall(text[head.end():].rstrip(".")):
        if value.startswith("["):
            case[key] = ast.literal_eval(value)
            continue
        try:
            case[key] = int(value)
        except ValueError:
            try:
                case[key] = float(value)
            except ValueError:
                case[key] = value
    return case


def offsets_of(case: Dict) -> Optional[List[int]]:
    """Validated packed offsets of a prefill record (``cu_seqlens_q`` or ``cu_seqlens``), or ``None``
    (tests/utils.py:173-205: start at 0, strictly increasing, batch_size + 1 entries)."""
    a, b = case.get("cu_seqlens"), case.get("cu_seqlens_q")
    if a is not None and b is not None and a != b:
        raise ValueError("cu_seqlens and cu_seqlens_q must match when both are provided")
    values = a if a is not None else b
    if values is None:
        return None
    if not isinstance(values, (list, tuple)) or len(values) < 2:
        raise ValueError("cu_seqlens must be a list with at least two offsets")
    if any(isinstance(v, bool) or not isinstance(v, int) for v in values):
        raise ValueError("cu_seqlens offsets must be integers")
    if values[0] != 0:
        raise ValueError("cu_seqlens must start at 0")
    if any(e <= s for s, e in zip(values, values[1:])):
        raise ValueError("cu_seqlens must be strictly increasing")
    if case.get("batch_size") is not None and int(case["batch_size"]) != len(values) - 1:
        raise ValueError(f"batch_size={case['batch_size']} does not match cu_seqlens batch size {len(values) - 1}")
    return list(values)


def format_case(B: int, T: int, K: int, V: int, H: int, HV: int, dtype: str, is_kda: bool = False,
                offsets: Optional[Sequence[int]] = None, gate_lower_bound: float = -5.0,
                force_prefill: bool = False) -> str:
    """The record of a call (src/op_forge_case.h:149-212): decode when every interval of ``offsets`` has one
    token (or there are none and ``force_prefill`` is off), packed prefill otherwise."""
    offs = None if offsets is None else [int(x) for x in offsets]
    if offs is not None:
        if len(offs) != B + 1 or offs[0] != 0 or any(e < s for s, e in zip(offs, offs[1:])):
            raise ValueError("offsets must start at 0, not decrease, and have B + 1 entries")
        if any(e - s != 1 for s, e in zip(offs, offs[1:])):
            force_prefill = True
    elif force_prefill:
        if B != 1:
            raise ValueError("fixed prefill without offsets only supports batch size 1")
        offs = [0, T]
    tag, op = ("KDA", "kda_attn") if is_kda else ("GDN", "gdn_attn")
    out = f"[{tag}]:"
    out += f"[P][{B},200]{op}:" if force_prefill else f"[D][{B}]{op}:seqlen_q:{T},"
    out += f"head_dim_qk:{K},head_dim_v:{V},num_heads_qk:{H},num_heads_v:{HV},hidden_act:silu,conv_kdim:4,"
    if is_kda:
        out += f"gate_lower_bound:{_float_text(gate_lower_bound)},"
    out += f"batch_size:{B},dtype:{dtype}"
    if force_prefill and offs:
        out += ",cu_seqlens_q:[" + ",".join(str(x) for x in offs) + "]"
    return out + "."


def _float_text(x: float) -> str:
    text = repr(float(x))
    return text if ("." in text or "e" in text or "n" in text) else text + ".0"


def show_params() -> bool:
    """``PLA_SHOW_PARAMS`` (non-zero integer): the facades print a record per call."""
    try:
        return int(os.environ.get("PLA_SHOW_PARAMS", "0") or 0) != 0
    except ValueError:
        return False


def show_case(*args, **kwargs) -> None:
    """Print ``format_case(...)`` when ``PLA_SHOW_PARAMS`` is set (no-op otherwise)."""
    if show_params():
        print(format_case(*args, **kwargs), flush=True)


def show_call(q, v, is_kda: bool, cu_seqlens=None, host_offsets=None, lower_bound=None, prefill: bool = False) -> None:
    """Record of a facade call from its tensors (q ``[.., tokens, H, K]``, v ``[.., tokens, HV, V]``). Offsets come
    from ``host_offsets`` when given, else from a device read of ``cu_seqlens`` — skipped while the stream is
    being captured, in which case the record carries the shapes only, as in the reference."""
    if not show_params():
        return
    import torch
    offs = None
    if host_offsets is not None:
        offs = [int(x) for x in host_offsets]
    elif cu_seqlens is not None and not (q.is_cuda and torch.cuda.is_current_stream_capturing()):
        offs = [int(x) for x in cu_seqlens.tolist()]
    rows = q.shape[-3] if q.dim() == 3 or q.shape[0] == 1 else q.shape[0] * q.shape[1]
    B = len(offs) - 1 if offs is not None else (1 if prefill else (q.shape[0] if q.dim() == 4 else rows))
    T = rows if prefill or B == 0 else max(1, rows // max(B, 1))
    name = {"torch.bfloat16": "bf16", "torch.float16": "fp16", "torch.float32": "fp32"}.get(str(q.dtype), str(q.dtype))
    print(format_case(B, T, q.shape[-1], v.shape[-1], q.shape[-2], v.shape[-2], name, is_kda, offs,
                      -5.0 if lower_bound is None else float(lower_bound), prefill), flush=True)


def read_caselist(path) -> List[Dict]:
    """Records of one ``.list`` file (blank lines and ``#`` comments skipped; lines of other operators, which do
    not parse as GDN / KDA records, are skipped as well)."""
    cases = []
    for line in Path(path).read_text().splitlines():
        line = line.strip()
        if not line or line.startswith("#"):
            continue
        try:
            case = parse_case(line)
        except (ValueError, SyntaxError):
            continue
        if case["op"] in ("gdn_attn", "kda_attn"):
            cases.append(case)
    return cases


def collect(path) -> List[Dict]:
    """``[{file, cases}]`` for a ``.list`` file or every ``.list`` file below a directory."""
    root = Path(path)
    files = [root] if root.is_file() else sorted(root.rglob("*.list"))
    found = []
    for f in files:
        cases = read_caselist(f)
        if cases:
            found.append({"file": str(f), "cases": cases})
    return found


# --------------------------------------------------------------------------------------------------------
# replay
# --------------------------------------------------------------------------------------------------------
def _dtype(case):
    import torch
    name = str(case.get("dtype", "bf16"))
    if name in ("bf16", "bfloat16"):
        return torch.bfloat16
    if name in ("fp16", "half", "float16"):
        return torch.float16
    raise ValueError(f"unsupported activation dtype {name}")


def _check_dims(case):
    if case.get("head_dim_qk", D) != D or case.get("head_dim_v", D) != D:
        raise NotImplementedError("head dimensions other than 128")
    H, HV = int(case["num_heads_qk"]), int(case["num_heads_v"])
    if HV % H != 0:
        raise ValueError("num_heads_v must be a multiple of num_heads_qk")
    return H, HV


def _time(fn, steps, warmup):
    import torch
    for _ in range(warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def build_inputs(case: Dict, *, device="cuda", seed: int = 0) -> Dict:
    """Seeded synthetic inputs of a record's shape (q, k, v ~ N(0,1); raw gates ~ N(0,1); A_log ~ U(0, ln 16);
    pool ~ N(0, 0.02); slot 0 left free): everything ``run_inputs`` needs, as a dict of tensors and scalars."""
    import torch
    H, HV = _check_dims(case)
    dt = _dtype(case)
    kda = case["op"] == "kda_attn"
    if kda and H != HV:
        raise NotImplementedError("KDA records have one value head per key head")
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, device=dev)
    B = int(case["batch_size"])
    if case["phase"] == "D":
        Tq = int(case.get("seqlen_q", 1))
        lens = case.get("verify_lens") or [Tq] * B
        offs = [0]
        for n in lens:
            offs.append(offs[-1] + int(n))
    else:
        offs = offsets_of(case)
        if offs is None:
            raise ValueError("a prefill record needs cu_seqlens_q")
    T = offs[-1]
    x = dict(kda=kda, phase=case["phase"], H=H, HV=HV, B=B, T=T, offs=offs, dtype=dt,
             lower_bound=case.get("gate_lower_bound") if kda else None)
    x["cu"] = torch.tensor(offs, dtype=torch.int32, device=dev)
    x["q"], x["k"], x["v"] = rn(T, H, D).to(dt), rn(T, H, D).to(dt), rn(T, HV, D).to(dt)
    x["A_log"] = torch.rand(HV, generator=g, device=dev) * math.log(16.0)
    x["pool"] = rn(B + 1, HV, D, D) * 0.02
    x["idx"] = (torch.randperm(B, generator=g, device=dev) + 1).to(torch.int32)   # slot 0 left free (vLLM null block)
    x["status"] = torch.zeros(1, dtype=torch.int32, device=dev)
    if kda:
        x["gate"], x["beta"], x["dt_bias"] = rn(T, H, D).to(dt), rn(T, H).to(dt), rn(H, D) * 0.1
    else:
        x["gate"], x["beta"] = rn(T, HV).to(dt), rn(T, HV).to(dt)
        # the decode op takes dt_bias in the activation dtype, the prefill ops in fp32
        x["dt_bias"] = (rn(HV) * 0.1).to(dt) if case["phase"] == "D" else rn(HV) * 0.1
    return x


def run_inputs(x: Dict, pool=None, backend: str = "auto"):
    """One call of this library's op for the record behind ``x`` on ``pool`` (default: ``x["pool"]``, updated in
    place). Returns the output rows ``[T, HV, 128]``. ``backend="recurrent"`` evaluates a prefill record with the
    exact token recurrence on the GPU instead of the chunked kernels."""
    import torch
    from .decode import fused_sigmoid_gating_delta_rule_forward_k_last as gdn_decode
    from .decode.kda import fused_recurrent_kda
    from .prefill.flashkdapro.ops import flashkda_fwd
    from .prefill.flashqla.ops import chunk_gated_delta_rule_fwd
    p = x["pool"] if pool is None else pool
    q, k, v, T, H, HV, dt = x["q"], x["k"], x["v"], x["T"], x["H"], x["HV"], x["dtype"]
    if x["phase"] == "D":
        if x["kda"]:
            out, _ = fused_recurrent_kda(q[None], k[None], v[None], x["gate"][None], x["beta"][None], x["A_log"], x["dt_bias"],
                                         x["lower_bound"], p, x["cu"], x["idx"], status=x["status"])
            return out[0]
        return gdn_decode(x["A_log"], x["gate"][None], x["dt_bias"], 1.0, 20.0, q[None], k[None], v[None], x["beta"][None], p,
                          x["idx"], D ** -0.5, True, x["cu"], False, False, None, None, None, None, status=x["status"])[0]
    if x["kda"]:
        out = torch.empty(T, H, D, dtype=dt, device=q.device)
        flashkda_fwd(q, k, v, x["gate"], x["beta"], x["A_log"], x["dt_bias"], out, None, x["lower_bound"], None, None, x["cu"],
                     p, x["idx"], tuple(x["offs"]), backend=backend, status=x["status"])
        return out
    if backend == "recurrent":
        from ._ops import ops
        out = torch.empty(T, HV, D, dtype=dt, device=q.device)
        ops.prefill_recurrent(q, k, v, x["gate"], x["beta"], x["A_log"], x["dt_bias"], out, x["cu"], p, x["idx"], None, None,
                              False, False, True, D ** -0.5, None, False, True, x["status"])
        return out
    return chunk_gated_delta_rule_fwd(q[None], k[None], v[None], None, None, initial_state=p, initial_state_indices=x["idx"],
                                      cu_seqlens=x["cu"], output_final_state=False, normalize_qk=True,
                                      raw_cu_seqlens=tuple(x["offs"]), raw_gate_a=x["gate"], raw_beta_b=x["beta"],
                                      A_log=x["A_log"], dt_bias=x["dt_bias"])[2][0]


def replay(case: Dict, *, device="cuda", steps: int = 20, warmup: int = 3, check: bool = False, seed: int = 0) -> Dict:
    """Run the op of one record on ``build_inputs``' tensors and time it. Returns ``{"tag", "ms", "tokens", ...}``;
    decode records add ``state_GBps`` (fp32 tiles read and written per step), prefill records ``Mtok_per_s``; with
    ``check`` prefill records add the maximum output difference and the relative state difference between the
    chunked kernels and the exact token recurrence, both on the GPU (the test suite checks replayed records against
    its CPU oracle instead: ``tests/test_caselist.py``)."""
    import torch
    x = build_inputs(case, device=device, seed=seed)
    res = {"tag": case.get("_raw_line") or "", "tokens": x["T"], "batch": x["B"]}
    if x["phase"] == "P" and check:
        p1, p2 = x["pool"].clone(), x["pool"].clone()
        o1 = run_inputs(x, p1).float().clone()
        o2 = run_inputs(x, p2, backend="recurrent").float()
        res.update(out_max_abs_diff=float((o1 - o2).abs().max()) if x["T"] else 0.0,
                   state_rel_l2_diff=float((p1 - p2).norm() / p2.norm().clamp_min(1e-30)))
    ms = _time(lambda: run_inputs(x), steps, warmup)
    if x["phase"] == "D":
        res.update(ms=ms, state_GBps=2 * x["B"] * x["HV"] * D * D * 4 / ms / 1e6)
    else:
        res.update(ms=ms, Mtok_per_s=x["T"] / ms / 1e3)
    torch.cuda.synchronize()
    res["status"] = int(x["status"].item())
    return res


def replay_lists(path, *, limit: Optional[int] = None, phase: Optional[str] = None, check: bool = False,
                 steps: int = 20, out=sys.stdout) -> int:
    """Replay the records below ``path``; one JSON line per record. Returns the number of records that failed
    (device status set, exception, or — with ``check`` — a difference above the parity bars 2e-2 / 1e-3)."""
    bad = done = 0
    for group in collect(path):
        for case in group["cases"]:
            if phase and case["phase"] != phase:
                continue
            if limit is not None and done >= limit:
                return bad
            done += 1
            try:
                r = replay(case, check=check, steps=steps)
                r["file"] = os.path.basename(group["file"])
                ok = r["status"] == 0 and r.get("out_max_abs_diff", 0.0) <= 2e-2 and r.get("state_rel_l2_diff", 0.0) <= 1e-3
            except (NotImplementedError, ValueError, RuntimeError) as e:
                r, ok = {"tag": case["_raw_line"], "error": f"{type(e).__name__}: {e}"}, False
            r["ok"] = ok
            bad += 0 if ok else 1
            print(json.dumps(r), file=out, flush=True)
    return bad


def main(argv: Optional[Iterable[str]] = None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description="Replay case lists (the reference's shape corpus format) on this library.")
    ap.add_argument("path", help=".list file or directory")
    ap.add_argument("--limit", type=int, default=None)
    ap.add_argument("--phase", choices=["P", "D"], default=None)
    ap.add_argument("--check", action="store_true", help="prefill: compare with the exact token recurrence")
    ap.add_argument("--steps", type=int, default=20)
    a = ap.parse_args(list(argv) if argv is not None else None)
    return 1 if replay_lists(a.path, limit=a.limit, phase=a.phase, check=a.check, steps=a.steps) else 0


if __name__ == "__main__":
    sys.exit(main())
