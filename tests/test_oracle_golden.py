"""The CPU oracle restatement against fixtures produced by the reference's own oracles."""
from pathlib import Path

import numpy as np
import pytest
import torch

import cases
from oracle import decode as odec

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", sorted(cases.KLAST_CASES))
def test_klast_oracle_matches_reference_fixture(name):
    args, backing, lengths, state_ids, cache_ids = cases.klast_case(name)
    out, state, cache = odec.klast_forward(**cases.oracle_kwargs(args, lengths, state_ids, cache_ids))
    gold = np.load(GOLDEN / f"klast_{name}.npz")
    # same fp32 arithmetic in a different evaluation order: a few ulp
    np.testing.assert_allclose(out.float().numpy(), gold["out"][0], rtol=2e-2, atol=2e-3)
    np.testing.assert_allclose(cases.subsample(state), gold["state"], rtol=1e-4, atol=1e-5)
    assert abs(state.double().sum().item() - float(gold["state_sum"])) <= 1e-6 * max(1.0, abs(float(gold["state_sum"])))
    if cache is not None:
        got = cases.subsample(cache)
        np.testing.assert_allclose(got, gold["cache"], rtol=1e-4, atol=1e-5)
        # rows nobody wrote keep the poison value exactly
        assert np.array_equal(got == -7.0, gold["cache"] == -7.0)
    # padding / untouched slots are bit-identical to the input pool
    touched = {s for s, n in zip(state_ids, lengths) if s >= 0 and n > 0}
    if args["disable_state_update"]:
        touched = set()
    if not args.get("is_sglang", True):
        touched.discard(0)
    for s in range(state.shape[0]):
        if s not in touched:
            assert torch.equal(state[s], args["initial_state_source"][s])


def test_vlast_oracle_is_transposed_klast():
    args, backing, lengths, state_ids, cache_ids = cases.klast_case("gdn_decode")
    kw = cases.oracle_kwargs(args, lengths, state_ids, cache_ids)
    out_k, st_k, _ = odec.klast_forward(**kw)
    pool_v = args["initial_state_source"].transpose(-1, -2).contiguous()
    init = torch.full_like(out_k, 3.0)
    out_v, st_v = odec.vlast_forward(
        q=kw["q"], k=kw["k"], v=kw["v"], a=kw["a"], b=kw["b"], A_log=kw["A_log"], dt_bias=kw["dt_bias"],
        state=pool_v, slot_indices=state_ids, scale=kw["scale"], out_init=init)
    assert torch.equal(st_v.transpose(-1, -2), st_k)
    assert torch.equal(out_v[:2], out_k[:2])
    assert torch.equal(out_v[2], init[2])  # slot -1: output row untouched
