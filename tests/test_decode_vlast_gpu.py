"""v-last GDN decode on the GPU against the CPU oracle (transposed k-last recurrence)."""
import pytest
import torch

from helpers import assert_out_close, assert_state_close
from oracle import decode as odec

pytestmark = pytest.mark.gpu


def _inputs(B, H, HV, slots, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    return dict(
        q=torch.randn(B, 1, H, 128, generator=g).to(dtype), k=torch.randn(B, 1, H, 128, generator=g).to(dtype),
        v=torch.randn(B, 1, HV, 128, generator=g).to(dtype), a=torch.randn(B, HV, generator=g).to(dtype),
        b=torch.randn(B, HV, generator=g).to(dtype), A_log=torch.rand(HV, generator=g) * 2.7,
        dt_bias=(torch.randn(HV, generator=g) * 0.1).to(dtype),
        pool=torch.randn(slots, HV, 128, 128, generator=g) * 0.1)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,HV", [(3, 1, 1), (5, 2, 4), (8, 16, 32)])
@pytest.mark.parametrize("varlen", [False, True])
def test_vlast_matches_oracle(native_built, dtype, B, H, HV, varlen):
    from pla_b200.decode.gdn.v_last import fused_sigmoid_gating_delta_rule
    slots = 2 * B + 1
    c = _inputs(B, H, HV, slots, 3 + B, dtype)
    idx = torch.randperm(slots, generator=torch.Generator().manual_seed(B))[:B].to(torch.int32)
    idx[B // 2] = -1
    o_init = torch.full((B, 1, HV, 128), 9.0, dtype=dtype)
    exp_out, exp_state = odec.vlast_forward(
        q=c["q"][:, 0], k=c["k"][:, 0], v=c["v"][:, 0], a=c["a"], b=c["b"], A_log=c["A_log"], dt_bias=c["dt_bias"],
        state=c["pool"], slot_indices=idx.tolist(), scale=128 ** -0.5, out_init=o_init[:, 0])
    d = {k_: v_.cuda() for k_, v_ in c.items()}
    o = o_init.cuda()
    cu = torch.arange(B + 1, dtype=torch.int32, device="cuda") if varlen else None
    q, k, v = (d[n].view(1, B, -1, 128) if varlen else d[n] for n in ("q", "k", "v"))
    ret = fused_sigmoid_gating_delta_rule(
        A_log=d["A_log"], a=d["a"], dt_bias=d["dt_bias"], q=q, k=k, v=v, b=d["b"], o=o.view(v.shape),
        h0_source=d["pool"], h0_indices=idx.cuda(), cu_seqlens=cu, scale=128 ** -0.5, T=1 if not varlen else B,
        B=B, H=H, HV=HV, K=128, V=128, use_initial_state=True, use_qk_l2norm_in_kernel=True, is_varlen=varlen)
    torch.cuda.synchronize()
    assert ret.data_ptr() == o.data_ptr()
    assert_out_close(o[:, 0], exp_out)
    assert torch.equal(o[B // 2].cpu(), o_init[B // 2])          # padded request: row untouched
    pool = d["pool"].cpu()
    assert_state_close(pool, exp_state)
    used = set(i for i in idx.tolist() if i >= 0)
    for s in range(slots):
        if s not in used:
            assert torch.equal(pool[s], c["pool"][s])


def test_vlast_rejects_unsupported_contracts(native_built):
    from pla_b200.decode.gdn.v_last import fused_sigmoid_gating_delta_rule
    c = {k_: v_.cuda() for k_, v_ in _inputs(2, 1, 1, 3, 0, torch.bfloat16).items()}
    idx = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    o = torch.zeros(2, 1, 1, 128, dtype=torch.bfloat16, device="cuda")
    kw = dict(A_log=c["A_log"], a=c["a"], dt_bias=c["dt_bias"], q=c["q"], k=c["k"], v=c["v"], b=c["b"], o=o,
              h0_indices=idx, T=1, B=2, H=1, HV=1, K=128, V=128, use_qk_l2norm_in_kernel=True)
    with pytest.raises(RuntimeError, match="float32"):
        fused_sigmoid_gating_delta_rule(h0_source=c["pool"].bfloat16(), use_initial_state=True, **kw)
    with pytest.raises(RuntimeError, match="use_initial_state"):
        fused_sigmoid_gating_delta_rule(h0_source=c["pool"], use_initial_state=False, **kw)
