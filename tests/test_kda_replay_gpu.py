"""KDA ReplaySSM verify / commit on the GPU against the fp64 oracle.

Follows the discipline of the reference's tests/test_kda_replayssm_vllm.py: paged caches with
padding bytes (0x5A), poisoned records (-7) and outputs (-11), strided int32/int64 index vectors,
bit-exact conv windows, plans and untouched regions. Tolerances are the reference's: max error
relative to the largest reference magnitude <= 6e-3 for out / rawk / rawv, <= 5e-6 for g, beta and
folded checkpoints.
"""
import json
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import cases
from oracle import replay as orep
from test_oracle_replay import oracle_verify

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
D = 128


def close(got, want, tol=6e-3, what=""):
    if got.numel() == 0:
        return
    g, w = got.double().cpu(), want.double().cpu()
    assert torch.isfinite(g).all(), what
    rel = ((g - w).abs().max() / w.abs().max().clamp_min(1e-30)).item()
    assert rel <= tol, f"{what}: max error / max magnitude = {rel:.3e} > {tol}"


def vector(values, dtype=torch.int32, strided=False):
    t = torch.tensor(values, device="cuda", dtype=dtype)
    if strided:
        storage = torch.full((len(values) * 2 + 1,), -99, device="cuda", dtype=dtype)
        storage[1::2] = t
        t = storage[1::2]
    return t


def device_records(rows, heads, q):
    from pla_b200.decode.kda_replayssm_vllm import KDAReplayRecords
    rec = KDAReplayRecords.allocate(rows, heads, q, "cuda")
    for name in ("rawv", "rawk", "g", "beta", "conv"):
        getattr(rec, name).fill_(-7)
    return rec


def run_verify(layer, x, offsets, slots, rec, out, index_dtype=torch.int32, strided=False, null_block_id=0,
               status=None):
    from pla_b200.decode.kda_replayssm_vllm import kda_replay_verify
    args = {k: v for k, v in x.items() if k != "storage"}
    return kda_replay_verify(**args, conv_state=layer.kv_cache[0], checkpoint_state=layer.kv_cache[1], records=rec,
                             query_start_loc=vector(offsets, index_dtype, strided),
                             state_indices=vector(slots, index_dtype, strided), conv_state_layout=layer.layout,
                             out=out, null_block_id=null_block_id, status=status)


@pytest.mark.parametrize("index_dtype,strided", [(torch.int32, False), (torch.int64, True)])
@pytest.mark.parametrize("name", sorted(cases.REPLAY_VERIFY_CASES))
def test_verify_matches_oracle(native_built, name, index_dtype, strided):
    layer, x, offsets, slots, lengths = cases.replay_verify_case(name, device="cuda")
    cpu_layer, cpu_x, *_ = cases.replay_verify_case(name)
    want_out, want = oracle_verify(cpu_layer, cpu_x, offsets, slots)
    rec = device_records(len(slots), layer.heads, layer.q)
    out = torch.full((x["mixed_qkv"].shape[0], layer.heads * D), -11, dtype=torch.bfloat16, device="cuda")
    before, storage_before = layer.raw.clone(), x["storage"].clone()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    run_verify(layer, x, offsets, slots, rec, out, index_dtype, strided, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    last = offsets[-1]
    close(out[:last], want_out[:last], what="out")
    gold = np.load(GOLDEN / f"replay_verify_{name}.npz")
    close(out[:last], torch.from_numpy(gold["out"][:last]), what="out vs reference fixture")
    for key in ("rawv", "rawk", "g", "beta", "conv"):
        got, expected = getattr(rec, key).cpu(), getattr(want, key)
        for b, n in enumerate(lengths):
            if slots[b] > 0 and n:
                act = (b, slice(0, n)) if key == "conv" else (b, slice(None), slice(0, n))
                if key == "conv":
                    assert torch.equal(got[act], expected[act]), key
                else:
                    close(got[act], expected[act], 5e-6 if key in ("g", "beta") else 6e-3, key)
            suffix = got[b, n:] if key == "conv" else got[b, :, n:]
            assert torch.equal(suffix, torch.full_like(suffix, -7)), key
            if slots[b] <= 0 or n == 0:
                assert torch.equal(got[b], torch.full_like(got[b], -7)), key
    assert torch.equal(layer.raw, before), "verify changed persistent pages"
    assert torch.equal(x["storage"], storage_before)
    assert torch.equal(out[last:], torch.full_like(out[last:], -11))
    default_out = run_verify(layer, x, offsets, slots, rec, None)
    close(default_out[:last], want_out[:last], what="allocated out")


def test_verify_softplus_gate_and_null_minus_one(native_built):
    layer, x, offsets, slots, lengths = cases.replay_verify_case("sd_q4_h2", device="cuda")
    cpu_layer, cpu_x, *_ = cases.replay_verify_case("sd_q4_h2")
    x["lower_bound"] = cpu_x["lower_bound"] = None       # g = -exp(A_log) * softplus(x + dt_bias)
    want_out, want = oracle_verify(cpu_layer, cpu_x, offsets, slots, null_block_id=-1)
    rec = device_records(len(slots), layer.heads, layer.q)
    out = torch.full((x["mixed_qkv"].shape[0], layer.heads * D), -11, dtype=torch.bfloat16, device="cuda")
    run_verify(layer, x, offsets, slots, rec, out, null_block_id=-1)
    last = offsets[-1]
    close(out[:last], want_out[:last], what="out")
    close(rec.g[3, :, :1].cpu(), want.g[3, :, :1], 5e-6, "g of the slot-0 row (valid when the null id is -1)")


def _commit_round(c, layers, recs, live):
    from pla_b200.decode.kda_replayssm_vllm import KDAReplayCommitContext
    for layer, rec in zip(layers, recs):
        layer.replay_records = rec
    ctx = KDAReplayCommitContext.create(layers, spec_query_len=c["q"], max_num_reqs=c["rows"],
                                        conv_state_layout=layers[0].layout)
    kwargs = dict(request_indices=vector(c["mapping"], torch.int64, True),
                  token_capacity=c["x"]["mixed_qkv"].shape[0])
    if c["table"] is not None:
        kwargs.update(block_table=torch.tensor(c["table"], device="cuda", dtype=torch.int32),
                      num_computed_tokens=vector(c["computed"]), mamba_block_size=8)
    return ctx.commit(vector(c["counts"], torch.int64, True), vector(c["slots"]),
                      vector(c["offsets"], torch.int64, True), **kwargs)


@pytest.mark.parametrize("layout", ["SD", "DS"])
@pytest.mark.parametrize("name", sorted(cases.REPLAY_COMMIT_CASES))
def test_commit_matches_oracle(native_built, name, layout):
    c = cases.replay_commit_case(name, layout=layout, device="cuda")
    cpu = cases.replay_commit_case(name, layout=layout)
    recs, wants = [], []
    plan_want = orep.commit_plan(sampled=c["counts"], source=c["slots"], offsets=c["offsets"], capacity=c["rows"],
                                 slots=24, Q=c["q"], null_block_id=0, token_capacity=c["x"]["mixed_qkv"].shape[0],
                                 mapping=c["mapping"], block_table=c["table"], computed=c["computed"],
                                 block_size=c["block_size"] or 0)
    if layout == "SD":
        assert plan_want == np.load(GOLDEN / f"replay_commit_{name}.npz")["plan"].tolist()
    for layer, cpu_layer in zip(c["layers"], cpu["layers"]):
        # verify on the device, then fold from the ORACLE's records so the fold is judged alone
        rec = device_records(c["rows"], c["heads"], c["q"])
        out = torch.full((c["x"]["mixed_qkv"].shape[0], c["heads"] * D), -11, dtype=torch.bfloat16, device="cuda")
        run_verify(layer, c["x"], c["offsets"], c["slots"], rec, out)
        _, want_rec = oracle_verify(cpu_layer, cpu["x"], c["offsets"], c["slots"])
        for key in ("rawv", "rawk", "g", "beta", "conv"):
            getattr(rec, key).copy_(getattr(want_rec, key))
        recs.append(rec)
        wants.append(orep.commit_apply(cpu_layer.kv_cache[1], cases.conv_ds(cpu_layer), want_rec, plan_want,
                                       c["slots"]))
    before = [layer.raw.clone() for layer in c["layers"]]
    plan = _commit_round(c, c["layers"], recs, live=False)
    torch.cuda.synchronize()
    got_plan = [getattr(plan, k).tolist() for k in ("commit_lens", "final_state_indices",
                                                    "boundary_state_indices", "boundary_recovery_lens")]
    assert got_plan == plan_want
    touched = {s for n, f, b, bc in zip(*plan_want) if n for s in ([f, b] if bc else [f])}
    for layer, (state, conv), raw_before in zip(c["layers"], wants, before):
        got_state, got_conv = layer.kv_cache[1].cpu(), cases.conv_ds(layer).cpu()
        close(got_state, state, 5e-6, "folded checkpoints")
        for s in range(state.shape[0]):
            if s not in touched:
                assert torch.equal(got_state[s], state[s]), s
        assert torch.equal(got_conv, conv), "conv snapshot scatter is not exact"
        # everything outside the two cache views (page padding included) keeps its bytes
        expected_raw = raw_before.clone()
        c0, s0 = layer.kv_cache
        expected_raw.view(torch.float32).as_strided(s0.shape, s0.stride(), s0.storage_offset()).copy_(s0)
        expected_raw.view(torch.bfloat16).as_strided(c0.shape, c0.stride(), c0.storage_offset()).copy_(c0)
        assert torch.equal(layer.raw, expected_raw), "page padding changed"


def test_verify_then_commit_live_records(native_built):
    """End to end with the device's own records: the committed checkpoint equals an fp64 fold of the
    records the device wrote."""
    c = cases.replay_commit_case("align_t0", device="cuda")
    recs = []
    for layer in c["layers"]:
        rec = device_records(c["rows"], c["heads"], c["q"])
        out = torch.full((c["x"]["mixed_qkv"].shape[0], c["heads"] * D), -11, dtype=torch.bfloat16, device="cuda")
        run_verify(layer, c["x"], c["offsets"], c["slots"], rec, out)
        recs.append(rec)
    olds = [layer.kv_cache[1].cpu().clone() for layer in c["layers"]]
    oldc = [cases.conv_ds(layer).cpu().clone() for layer in c["layers"]]
    plan = _commit_round(c, c["layers"], recs, live=True)
    torch.cuda.synchronize()
    plan_l = [getattr(plan, k).tolist() for k in ("commit_lens", "final_state_indices",
                                                  "boundary_state_indices", "boundary_recovery_lens")]
    for layer, rec, old, oc in zip(c["layers"], recs, olds, oldc):
        host = SimpleNamespace(**{k: getattr(rec, k).cpu() for k in ("rawv", "rawk", "g", "beta", "conv")})
        state, conv = orep.commit_apply(old, oc, host, plan_l, c["slots"])
        close(layer.kv_cache[1].cpu(), state, 5e-6, "live commit")
        assert torch.equal(cases.conv_ds(layer).cpu(), conv)


def test_plan_scenarios_on_device(native_built):
    from pla_b200.decode.kda_replayssm_vllm import KDAReplayCommitContext
    gold = json.loads((GOLDEN / "replay_plans.json").read_text())
    for sc in cases.plan_scenarios():
        batch = len(sc["sources"])
        layer = cases.replay_layer(np.random.RandomState(1), sc["slots"], 1, sc["q"], "DS", device="cuda")
        layer.replay_records = device_records(sc["capacity"], 1, sc["q"])
        ctx = KDAReplayCommitContext.create([layer], sc["q"], sc["capacity"], conv_state_layout="DS")
        kwargs = {}
        if sc["table"] is not None:
            kwargs = dict(block_table=torch.tensor(sc["table"], device="cuda", dtype=torch.int64),
                          num_computed_tokens=vector(sc["positions"], torch.int64, True), mamba_block_size=8)
        before = layer.raw.clone()
        plan = ctx.commit(vector(sc["counts"], torch.int64, True), vector(sc["sources"], torch.int64, True),
                          vector(sc["offsets"], torch.int64, True), token_capacity=sc["token_capacity"],
                          plan_only=True, **kwargs)
        got = [getattr(plan, k).tolist() for k in ("commit_lens", "final_state_indices",
                                                   "boundary_state_indices", "boundary_recovery_lens")]
        assert got == gold[sc["name"]], sc["name"]
        assert torch.equal(layer.raw, before)
        assert batch <= sc["capacity"]


def test_context_rejects_overlapping_layers_and_bad_arguments(native_built):
    from pla_b200.decode.kda_replayssm_vllm import KDAReplayCommitContext, KDAReplayRecords
    layer = cases.replay_layer(np.random.RandomState(2), 6, 1, 2, "SD", device="cuda")
    layer.replay_records = device_records(2, 1, 2)
    twin = SimpleNamespace(kv_cache=layer.kv_cache, replay_records=device_records(2, 1, 2), layout="SD")
    with pytest.raises(ValueError, match="overlapping writable caches"):
        KDAReplayCommitContext.create([layer, twin], 2, 2)
    with pytest.raises(ValueError, match="null_block_id"):
        KDAReplayCommitContext.create([layer], 2, 2, null_block_id=3)
    with pytest.raises(ValueError, match="Q in"):
        KDAReplayRecords.allocate(2, 1, 33, "cuda")
    ctx = KDAReplayCommitContext.create([layer], 2, 2)
    with pytest.raises(ValueError, match="align requires"):
        ctx.commit(vector([1, 1]), vector([1, 2]), vector([0, 2, 4]), block_table=torch.zeros(2, 2, device="cuda"),
                   token_capacity=4)
    with pytest.raises(TypeError):
        ctx.commit(vector([1, 1]), vector([1, 2]), vector([0, 2, 4]), token_capacity=4.5)
