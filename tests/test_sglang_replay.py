"""KDA ReplaySSM under the SGLang contract: the oracle against fixtures produced by the reference's
fp64 oracle, and ``pla.decode.kda_replayssm_sglang`` on the GPU against the oracle."""
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import cases
from helpers import assert_out_close, assert_state_close, rel_l2
from oracle import replay as orep

GOLD = Path(__file__).parent / "golden"
RINGS = ("replayssm_rawv", "replayssm_rawk", "replayssm_g", "replayssm_beta")
WINS = ("intermediate_conv_q", "intermediate_conv_k", "intermediate_conv_v")
REF_KEYS = {"replayssm_rawv": "ring_rawv", "replayssm_rawk": "ring_rawk", "replayssm_g": "ring_g",
            "replayssm_beta": "ring_beta", "intermediate_conv_q": "ic_q", "intermediate_conv_k": "ic_k",
            "intermediate_conv_v": "ic_v"}


def active_requests(vi, c):
    for n in range(c["bs"]):
        slot = int(vi["ssm_state_indices"][n])
        if slot >= 0:
            yield n, slot, int(vi["intermediate_state_indices"][n])


@pytest.mark.parametrize("name", list(cases.SGLANG_VERIFY_CASES))
def test_oracle_ring_verify_matches_reference_fixture(name):
    vi, c = cases.sglang_verify_case(name)
    got = orep.ring_verify(vi)
    gold = np.load(GOLD / f"sglang_verify_{name}.npz")
    assert rel_l2(got["out"].float(), torch.from_numpy(gold["out"])) < 1e-6
    for n, slot, srow in active_requests(vi, c):
        for key in RINGS:
            torch.testing.assert_close(got[key][slot, :, :c["dtn"]].float(),
                                       torch.from_numpy(gold[REF_KEYS[key]])[slot, :, :c["dtn"]], rtol=1e-6, atol=1e-6)
        for key in WINS:
            assert torch.equal(got[key][srow, :c["dtn"]].float(), torch.from_numpy(gold[REF_KEYS[key]])[srow, :c["dtn"]])


@pytest.mark.parametrize("name", list(cases.SGLANG_COMMIT_CASES))
def test_oracle_fold_layers_matches_reference_fixture(name):
    ci, c = cases.sglang_commit_case(name)
    got = orep.fold_layers(ci["temporal"], ci["rawv"], ci["rawk"], ci["gk"], ci["beta"], ci["state_batch_indices"],
                           ci["accept_lens"])
    gold = np.load(GOLD / f"sglang_fold_{name}.npz")
    touched = gold["touched"].tolist()
    assert rel_l2(torch.from_numpy(cases.subsample(got[:, touched].float())), torch.from_numpy(gold["state"])) < 1e-6
    assert abs(got[:, touched].sum().item() - float(gold["state_sum"])) < 1e-4 * max(1.0, abs(float(gold["state_sum"])))
    untouched = [s for s in range(ci["temporal"].shape[1]) if s not in touched]
    assert torch.equal(got[:, untouched].float(), ci["temporal"][:, untouched])


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(cases.SGLANG_VERIFY_CASES))
def test_fused_kda_decode_mtp_dspark(native_built, name):
    from pla_b200.decode.kda_replayssm_sglang import fused_kda_decode_mtp_dspark
    vi, c = cases.sglang_verify_case(name)
    want = orep.ring_verify(vi)
    dv, _ = cases.sglang_verify_case(name, device="cuda")
    state_before = dv["recurrent_state"].clone()
    conv_before = [dv[k].clone() for k in ("cs_q", "cs_k", "cs_v")]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.full((1, c["bs"] * c["dtn"], c["heads"], 128), -11.0, dtype=torch.bfloat16, device="cuda")
    ret = fused_kda_decode_mtp_dspark(**dv, out=out, status=status)
    torch.cuda.synchronize()
    assert ret is out and status.item() == 0
    assert torch.equal(dv["recurrent_state"], state_before)                      # persistent state is read-only
    assert all(torch.equal(dv[k], b) for k, b in zip(("cs_q", "cs_k", "cs_v"), conv_before))
    assert_out_close(out.cpu(), want["out"].float())
    gold = np.load(GOLD / f"sglang_verify_{name}.npz")
    assert_out_close(out.cpu(), torch.from_numpy(gold["out"]), "out vs reference fixture")
    seen_slots, seen_rows = set(), set()
    for n, slot, srow in active_requests(vi, c):
        seen_slots.add(slot)
        seen_rows.add(srow)
        for key in ("replayssm_rawv", "replayssm_rawk"):
            assert_out_close(dv[key][slot, :, :c["dtn"]].cpu(), want[key][slot, :, :c["dtn"]].float(), key)
        torch.testing.assert_close(dv["replayssm_g"][slot, :, :c["dtn"]].cpu(), want["replayssm_g"][slot, :, :c["dtn"]].float(),
                                   rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(dv["replayssm_beta"][slot, :, :c["dtn"]].cpu(),
                                   want["replayssm_beta"][slot, :, :c["dtn"]].float(), rtol=1e-5, atol=1e-6)
        for key in WINS:                                                         # byte-exact
            assert torch.equal(dv[key][srow, :c["dtn"]].cpu().float(), want[key][srow, :c["dtn"]].float())
    # rows of requests that did not run keep their fill value; padding requests get zero output
    for slot in range(c["slots"]):
        if slot not in seen_slots:
            assert torch.all(dv["replayssm_rawv"][slot] == -3.0) and torch.all(dv["replayssm_beta"][slot] == -3.0)
    for row in range(dv["intermediate_conv_q"].shape[0]):
        if row not in seen_rows:
            assert torch.all(dv["intermediate_conv_q"][row] == -3.0)
    for n in range(c["bs"]):
        if int(vi["ssm_state_indices"][n]) < 0:
            assert torch.all(out[0, n * c["dtn"]:(n + 1) * c["dtn"]] == 0)


@pytest.mark.gpu
@pytest.mark.parametrize("layout", ["dim_width", "width_dim"])
@pytest.mark.parametrize("name", list(cases.SGLANG_COMMIT_CASES))
def test_commit_kda_replayssm_after_verify(native_built, name, layout):
    from pla_b200.decode.kda_replayssm_sglang import commit_kda_replayssm_after_verify
    ci, c = cases.sglang_commit_case(name)
    track = (ci.get("mamba_track_indices"), ci.get("mamba_steps_to_track"))
    want_state = orep.fold_layers(ci["temporal"], ci["rawv"], ci["rawk"], ci["gk"], ci["beta"], ci["state_batch_indices"],
                                  ci["accept_lens"], *track)
    want_conv = orep.conv_window_scatter(ci["conv"][0], ci["intermediate_conv_window"][0], ci["state_batch_indices"],
                                         ci["last_correct_step_indices"])
    if track[0] is not None:
        want_conv = orep.conv_window_scatter(want_conv, ci["intermediate_conv_window"][0], *track)
    d, _ = cases.sglang_commit_case(name, device="cuda")
    conv, window = d["conv"][0], d["intermediate_conv_window"][0]
    if layout == "width_dim":                                                  # pools stored [.., width, dim]
        conv = conv.transpose(-1, -2).contiguous()
        window = window.transpose(-1, -2).contiguous()
    spec = SimpleNamespace(temporal=d["temporal"], replayssm_rawv=d["rawv"], replayssm_rawk=d["rawk"],
                           replayssm_g=d["gk"], replayssm_beta=d["beta"], conv=[conv], intermediate_conv_window=[window])
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    commit_kda_replayssm_after_verify(spec_state=spec, state_batch_indices=d["state_batch_indices"],
                                      accept_lens=d["accept_lens"],
                                      last_correct_step_indices=d["last_correct_step_indices"],
                                      mamba_track_indices=d.get("mamba_track_indices"),
                                      mamba_steps_to_track=d.get("mamba_steps_to_track"),
                                      conv_state_layout=layout, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    got = d["temporal"].cpu()
    changed = [s for s in range(got.shape[1]) if not torch.equal(want_state[:, s].float(), ci["temporal"][:, s])]
    assert changed
    for s in range(got.shape[1]):
        if s in changed:
            assert_state_close(got[:, s], want_state[:, s].float(), f"slot {s}")
        else:
            assert torch.equal(got[:, s], ci["temporal"][:, s])
    got_conv = conv.cpu() if layout == "dim_width" else conv.transpose(-1, -2).cpu()
    assert torch.equal(got_conv, want_conv)
    gold = np.load(GOLD / f"sglang_fold_{name}.npz")
    touched = gold["touched"].tolist()
    assert_state_close(torch.from_numpy(cases.subsample(got[:, touched])), torch.from_numpy(gold["state"]),
                       "state vs reference fixture")
