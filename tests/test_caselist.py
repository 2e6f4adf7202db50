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
    found = cl.collect(SAMPLE.parent)
    assert len(found) == 1 and len(found[0]["cases"]) == 5
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
