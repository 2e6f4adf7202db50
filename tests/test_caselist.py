"""Case records in the reference's corpus grammar: parser, formatter, PLA_SHOW_PARAMS, and the replay of a
sample list through this library's ops (GPU)."""
from pathlib import Path

import pytest
import torch

from pla_b200 import caselist as cl

SAMPLE = Path(__file__).resolve().parent / "golden" / "sample_cases.list"


def test_parse_reads_every_field_and_skips_foreign_records():
    cases = cl.read_caselist(SAMPLE)
    assert [c["phase"] for c in cases] == ["D", "D", "D", "P", "P"]          # comments, blanks, other operators skipped
    assert [c["model"] for c in cases] == ["GDN", "GDN", "KDA", "GDN", "KDA"]
    d = cases[2]
    assert d["seqlen_q"] == 8 and d["verify_lens"] == [3, 8] and d["gate_lower_bound"] == -5.0 and d["dtype"] == "bf16"
    p = cases[3]
    assert p["num_heads_qk"] == 2 and p["num_heads_v"] == 4 and p["norm_eps"] == 1e-06 and p["ssm_dtype"] == "fp32"
    assert cl.offsets_of(p) == [0, 130, 170, 500] and cl.offsets_of(cases[0]) is None
    found = {Path(f["file"]).name: len(f["cases"]) for f in cl.collect(SAMPLE.parent)}
    assert found == {"sample_cases.list": 5, "corpus_sample.list": 320}
    with pytest.raises(ValueError):
        cl.parse_case("seqlen_q:1,batch_size:2")


@pytest.mark.parametrize("bad,why", [
    ({"cu_seqlens_q": [1, 5]}, "start at 0"), ({"cu_seqlens_q": [0, 5, 5]}, "strictly increasing"),
    ({"cu_seqlens_q": [0]}, "at least two"), ({"cu_seqlens_q": [0, 2.5]}, "integers"),
    ({"cu_seqlens_q": [0, 4], "cu_seqlens": [0, 5]}, "must match"),
    ({"cu_seqlens_q": [0, 4, 9], "batch_size": 3}, "does not match")])
def test_offsets_validation(bad, why):
    with pytest.raises(ValueError, match=why):
        cl.offsets_of(bad)


def test_format_round_trips_through_the_parser():
    line = cl.format_case(8, 1, 128, 128, 16, 32, "bf16", offsets=list(range(9)))
    assert line == ("[GDN]:[D][8]gdn_attn:seqlen_q:1,head_dim_qk:128,head_dim_v:128,num_heads_qk:16,num_heads_v:32,"
                    "hidden_act:silu,conv_kdim:4,batch_size:8,dtype:bf16.")
    c = cl.parse_case(line)
    assert (c["phase"], c["batch_size"], c["seqlen_q"], c["num_heads_v"]) == ("D", 8, 1, 32)
    # unequal intervals turn the record into packed prefill and keep the offsets
    line = cl.format_case(2, 0, 128, 128, 4, 4, "fp16", True, [0, 24, 88], gate_lower_bound=-3)
    assert line == ("[KDA]:[P][2,200]kda_attn:head_dim_qk:128,head_dim_v:128,num_heads_qk:4,num_heads_v:4,hidden_act:silu,"
                    "conv_kdim:4,gate_lower_bound:-3.0,batch_size:2,dtype:fp16,cu_seqlens_q:[0,24,88].")
    c = cl.parse_case(line)
    assert c["phase"] == "P" and cl.offsets_of(c) == [0, 24, 88] and c["gate_lower_bound"] == -3.0
    assert cl.format_case(1, 77, 128, 128, 2, 2, "bf16", force_prefill=True).endswith("cu_seqlens_q:[0,77].")
    with pytest.raises(ValueError):
        cl.format_case(2, 77, 128, 128, 2, 2, "bf16", force_prefill=True)
    with pytest.raises(ValueError):
        cl.format_case(2, 1, 128, 128, 2, 2, "bf16", offsets=[0, 1])
    for raw in (c_["_raw_line"] for c_ in cl.read_caselist(SAMPLE)):                  # every sample record re-parses
        again = cl.parse_case(raw)
        assert again["_raw_line"] == raw


def test_show_params_prints_the_record_of_a_call(monkeypatch, capsys):
    q = torch.zeros(1, 6, 2, 128, dtype=torch.bfloat16)
    v = torch.zeros(1, 6, 4, 128, dtype=torch.bfloat16)
    cl.show_call(q, v, False, torch.arange(7))
    assert capsys.readouterr().out == ""                                              # off by default
    monkeypatch.setenv("PLA_SHOW_PARAMS", "1")
    cl.show_call(q, v, False, torch.arange(7, dtype=torch.int32))
    cl.show_call(q, v, True, None, (0, 2, 6), lower_bound=-4.0, prefill=True)
    cl.show_call(q.view(6, 1, 2, 128), v.view(6, 1, 4, 128), False)
    lines = capsys.readouterr().out.splitlines()
    assert lines[0].startswith("[GDN]:[D][6]gdn_attn:seqlen_q:1,") and lines[0].endswith("batch_size:6,dtype:bf16.")
    assert lines[1].startswith("[KDA]:[P][2,200]kda_attn:") and "gate_lower_bound:-4.0" in lines[1] and lines[1].endswith("cu_seqlens_q:[0,2,6].")
    assert lines[2] == lines[0]


@pytest.mark.gpu
def test_replay_of_the_sample_list(native_built):
    import io
    import json
    buf = io.StringIO()
    bad = cl.replay_lists(SAMPLE, check=True, steps=2, out=buf)
    rows = [json.loads(x) for x in buf.getvalue().splitlines()]
    assert len(rows) == 5 and bad == 0, rows
    assert all(r["ok"] and r["status"] == 0 and r["ms"] > 0 for r in rows)
    assert [r["tokens"] for r in rows] == [8, 12, 11, 500, 300]
    for r in rows[3:]:
        assert r["out_max_abs_diff"] <= 2e-2 and r["state_rel_l2_diff"] <= 1e-3


# ---- the reference's corpus: census of all of it, replay of a sample of it --------------------------------------------
GOLDEN = SAMPLE.parent
CORPUS_SAMPLE = GOLDEN / "corpus_sample.list"


def _census():
    import json
    return json.loads((GOLDEN / "corpus_census.json").read_text())


def test_corpus_sample_covers_every_shape_group_of_the_census():
    """The committed sample holds at least two records of every (operator, phase, heads, dtype, query length, gate
    bound) group the corpus has, and every one of them parses; what the formatter prints of it parses back to the same values."""
    import sys
    sys.path.insert(0, str(GOLDEN))
    from make_caselist_sample import group_key
    census = _census()
    assert census["served_records"] == sum(g["records"] for g in census["groups"].values()) == 56467
    assert len(census["groups"]) == 143
    cases = cl.read_caselist(CORPUS_SAMPLE)
    assert len(cases) == 320
    seen = {}
    for c in cases:
        seen[group_key(c)] = seen.get(group_key(c), 0) + 1
        offs = cl.offsets_of(c)
        assert (offs is None) == (c["phase"] == "D")
        again = cl.format_case(c["batch_size"], int(c.get("seqlen_q", 0)), 128, 128, c["num_heads_qk"], c["num_heads_v"],
                               c["dtype"], c["op"] == "kda_attn", offs, gate_lower_bound=c.get("gate_lower_bound", -5.0),
                               force_prefill=c["phase"] == "P")
        back = cl.parse_case(again)       # corpus records carry more fields (norm_eps, ssm_dtype ...) than a call prints
        assert all(c[key] == val for key, val in back.items() if key != "_raw_line" and key in c), (back, c)
    assert set(seen) == set(census["groups"])
    assert all(n >= 2 or census["groups"][k]["records"] == 1 for k, n in seen.items())


def test_census_of_the_whole_reference_corpus():
    """With the reference tree at hand (PLA_REFERENCE_CASELIST = its caselist folder): every one of its records
    parses, and the per-group census equals the committed one."""
    import os
    import sys
    root = os.environ.get("PLA_REFERENCE_CASELIST")
    if not root or not Path(root).is_dir():
        pytest.skip("PLA_REFERENCE_CASELIST does not name the reference's caselist folder")
    sys.path.insert(0, str(GOLDEN))
    from make_caselist_sample import census, pick
    table, groups = census(root)
    assert table == _census()
    assert pick(groups) == [c["_raw_line"] for c in cl.read_caselist(CORPUS_SAMPLE)]


def _oracle_check(x, out, pool_before, pool_after):
    """One value head (the last) of up to three sequences of a replayed record against the CPU oracle: outputs of
    their first ``cap`` tokens (the recurrence is causal), and the final state where the whole sequence fits."""
    from helpers import assert_out_close, assert_state_close
    from oracle import decode as odec
    cap = 320
    hv = x["HV"] - 1
    kh = hv // (x["HV"] // x["H"])
    offs, B = x["offs"], x["B"]
    for n in sorted({0, B // 2, B - 1}):
        lo, full = offs[n], offs[n + 1] - offs[n]
        T = min(full, cap)
        if T == 0:
            continue
        sl = slice(lo, lo + T)
        slot = int(x["idx"][n])
        exp_out, exp_state, _ = odec.klast_forward(
            q=x["q"][sl, kh:kh + 1].cpu(), k=x["k"][sl, kh:kh + 1].cpu(), v=x["v"][sl, hv:hv + 1].cpu(),
            a=x["gate"][sl, hv:hv + 1].cpu(), b=x["beta"][sl, hv:hv + 1].cpu(), A_log=x["A_log"][hv:hv + 1].cpu(),
            dt_bias=x["dt_bias"][hv:hv + 1].float().cpu(), state=pool_before[slot:slot + 1, hv:hv + 1].cpu(),
            slot_indices=[0], lengths=[T], scale=D ** -0.5, is_kda=x["kda"], lower_bound=x["lower_bound"])
        assert_out_close(out[sl, hv:hv + 1].cpu(), exp_out, f"request {n}")
        if T == full:
            assert_state_close(pool_after[slot:slot + 1, hv:hv + 1].cpu(), exp_state, f"request {n}")


D = 128


@pytest.mark.gpu
def test_replay_of_the_corpus_sample_against_the_oracle(native_built):
    """Every sampled record of the reference's corpus through this library's op for it (decode, multi-token verify
    and packed prefill; GDN and KDA; 1 to 4,015 requests; 2 to 32,768 tokens), a head subset against the oracle."""
    cases = cl.read_caselist(CORPUS_SAMPLE)
    done = 0
    for i, case in enumerate(cases):
        x = cl.build_inputs(case, seed=i)
        before = x["pool"].clone()
        out = cl.run_inputs(x)
        torch.cuda.synchronize()
        assert int(x["status"].item()) == 0, case["_raw_line"][:120]
        assert torch.equal(x["pool"][0], before[0]), "slot 0 is never addressed"
        try:
            _oracle_check(x, out, before, x["pool"])
        except AssertionError as e:
            raise AssertionError(f"record {i}: {case['_raw_line'][:160]}: {e}") from e
        done += 1
        del x, before, out
    assert done == 320
