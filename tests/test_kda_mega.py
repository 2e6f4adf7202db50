"""``fused_kda_decode_mega_forward``: the oracle against fixtures of the reference's own fp32 recurrence, and
the CUDA path against the oracle (output, state, conv state, padding rows)."""
from pathlib import Path

import numpy as np
import pytest
import torch

import cases
from helpers import assert_out_close, assert_state_close, rel_l2
from oracle import decode as odec

GOLD = Path(__file__).parent / "golden"


def oracle_kwargs(kw):
    return {("A_log" if k == "a_log" else k): v for k, v in kw.items()}


@pytest.mark.parametrize("name", [n for n in cases.MEGA_CASES if "bias" not in n])
def test_oracle_matches_reference_fixture(name):
    kw, c = cases.mega_case(name)
    out, state, conv = odec.kda_mega_forward(**oracle_kwargs(kw))
    gold = np.load(GOLD / f"mega_{name}.npz")
    touched = gold["touched"].tolist()
    assert rel_l2(out, torch.from_numpy(gold["out"])[0]) < 2e-3           # the fixture is rounded to fp16
    assert rel_l2(torch.from_numpy(cases.subsample(state[touched])), torch.from_numpy(gold["state"])) < 1e-5
    # the reference stores its conv result as fp16, which flushes the smallest bf16 values: compare by value
    torch.testing.assert_close(conv[touched].float(), torch.from_numpy(gold["conv"]), rtol=0, atol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("pad_rows", [(), (1,)])
@pytest.mark.parametrize("name", list(cases.MEGA_CASES))
def test_fused_kda_decode_mega_forward(native_built, name, pad_rows):
    from pla_b200.decode.kda import fused_kda_decode_mega_forward
    kw, c = cases.mega_case(name, pad_rows=pad_rows)
    want_out, want_state, want_conv = odec.kda_mega_forward(**oracle_kwargs(kw))
    d, _ = cases.mega_case(name, device="cuda", pad_rows=pad_rows)
    out = torch.full((1, c["B"], c["H"], 128), 7.0, dtype=d["x"].dtype, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ret = fused_kda_decode_mega_forward(**d, out=out, status=status)
    torch.cuda.synchronize()
    assert ret is None and status.item() == 0
    assert_out_close(out[0].cpu(), want_out)
    assert_state_close(d["state"].cpu(), want_state)
    assert torch.equal(d["conv_state"].cpu().float(), want_conv.float())    # byte-exact shift
    used = {int(s) for s in kw["state_indices"] if s >= 0}
    for slot in range(kw["state"].shape[0]):
        if slot not in used:
            assert torch.equal(d["state"][slot].cpu(), kw["state"][slot])
            assert torch.equal(d["conv_state"][slot].cpu(), kw["conv_state"][slot])
    for r in pad_rows:
        assert torch.count_nonzero(out[0, r]) == 0
    if not pad_rows and "bias" not in name:
        gold = np.load(GOLD / f"mega_{name}.npz")
        assert_out_close(out[0].cpu(), torch.from_numpy(gold["out"])[0], "out vs reference fixture")
