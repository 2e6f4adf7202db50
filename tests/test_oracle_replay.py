"""The fp64 replay restatement and the integer plan against fixtures made with the reference's oracle."""
import json
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import cases
from oracle import replay as orep

GOLDEN = Path(__file__).resolve().parent / "golden"
D = 128


def oracle_verify(layer, x, offsets, slots, null_block_id=0):
    """Run the restated verify request by request; returns (out fp64 with untouched rows = -11,
    records in their storage dtypes with untouched entries = -7)."""
    H, Q, C = layer.heads, layer.q, layer.heads * D
    rec = cases.blank_records(len(slots), H, Q)
    out = torch.full((x["mixed_qkv"].shape[0], C), -11.0, dtype=torch.float64)
    conv, state = cases.conv_ds(layer), layer.kv_cache[1]
    wq, wk, wv = x["conv_weight"].split(C)
    for row, slot in enumerate(slots):
        b, e = offsets[row], offsets[row + 1]
        if e == b:
            continue
        if slot <= null_block_id:
            out[b:e] = 0
            continue
        xq, xk, xv = (t.reshape(e - b, H, D) for t in x["mixed_qkv"][b:e].split(C, -1))
        cq, ck, cv = (t[:, :3] for t in conv[slot].split(C))
        r = orep.verify_request(xq, xk, xv, x["raw_g"][b:e].reshape(e - b, H, D), x["raw_beta"][b:e], wq, wk, wv,
                                cq, ck, cv, x["A_log"], x["dt_bias"], state[slot], D ** -0.5, x["lower_bound"])
        n = e - b
        out[b:e] = r["out"].reshape(n, C)
        rec.rawk[row, :, :n] = r["rawk"]
        rec.rawv[row, :, :n] = r["rawv"]
        rec.g[row, :, :n] = r["g"]
        rec.beta[row, :, :n] = r["beta"]
        rec.conv[row, :n] = torch.cat([r["win_q"], r["win_k"], r["win_v"]], dim=1)
    return out, rec


@pytest.mark.parametrize("name", sorted(cases.REPLAY_VERIFY_CASES))
def test_verify_restatement_matches_reference_oracle(name):
    layer, x, offsets, slots, lengths = cases.replay_verify_case(name)
    out, rec = oracle_verify(layer, x, offsets, slots)
    gold = np.load(GOLDEN / f"replay_verify_{name}.npz")
    np.testing.assert_allclose(out.numpy(), gold["out"], rtol=1e-5, atol=1e-6)
    for key in ("rawv", "rawk", "g", "beta"):
        np.testing.assert_allclose(getattr(rec, key).float().numpy(), gold[key], rtol=1e-5, atol=1e-6, err_msg=key)
    assert np.array_equal(rec.conv.float().numpy(), gold["conv"])


@pytest.mark.parametrize("name", sorted(cases.REPLAY_COMMIT_CASES))
def test_commit_restatement_matches_reference_oracle(name):
    c = cases.replay_commit_case(name)
    gold = np.load(GOLDEN / f"replay_commit_{name}.npz")
    plan = orep.commit_plan(sampled=c["counts"], source=c["slots"], offsets=c["offsets"], capacity=c["rows"],
                            slots=24, Q=c["q"], null_block_id=0, token_capacity=c["x"]["mixed_qkv"].shape[0],
                            mapping=c["mapping"], block_table=c["table"], computed=c["computed"],
                            block_size=c["block_size"] or 0)
    assert plan == gold["plan"].tolist()
    touched = gold["touched"].tolist()
    for li, layer in enumerate(c["layers"]):
        _, rec = oracle_verify(layer, c["x"], c["offsets"], c["slots"])
        state, conv = orep.commit_apply(layer.kv_cache[1], cases.conv_ds(layer), rec, plan, c["slots"])
        if touched:
            np.testing.assert_allclose(cases.subsample(state[touched]), gold[f"state_l{li}"], rtol=2e-5, atol=1e-7)
            assert np.array_equal(conv[touched][:, :, :3].float().numpy(), gold[f"conv_l{li}"])
        for s in range(state.shape[0]):
            if s not in touched:
                assert torch.equal(state[s], layer.kv_cache[1][s])
                assert torch.equal(conv[s], cases.conv_ds(layer)[s])


def test_plan_scenarios_match_reference_expectations():
    gold = json.loads((GOLDEN / "replay_plans.json").read_text())
    for sc in cases.plan_scenarios():
        plan = orep.commit_plan(sampled=sc["counts"], source=sc["sources"], offsets=sc["offsets"],
                                capacity=sc["capacity"], slots=sc["slots"], Q=sc["q"], null_block_id=0,
                                token_capacity=sc["token_capacity"], block_table=sc["table"],
                                computed=sc["positions"], block_size=sc["block_size"])
        assert plan == gold[sc["name"]], sc["name"]
    # block_table=[[3,4]], computed=[7], block size 8, 2 of 2 tokens accepted: the commit crosses
    # into block 1 after one token
    plan = orep.commit_plan(sampled=[2], source=[2], offsets=[0, 2], capacity=1, slots=8, Q=2, null_block_id=0,
                            token_capacity=2, block_table=[[3, 4]], computed=[7], block_size=8)
    assert plan == gold["known_answer_block_boundary"] == [[2], [4], [3], [1]]
