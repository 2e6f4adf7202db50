"""``pla.decode.kda.fused_recurrent_kda`` (vLLM-signature adapter over the k-last KDA op): slot
bookkeeping for 1-D and 2-D tables, both pad conventions, page-padded pools, both gate forms
(cases follow scripts/decode/test_kda_decode.py:147-330 of the reference) and its exception types."""
import pytest
import torch

from helpers import assert_out_close, assert_state_close
from oracle import decode as odec

D = 128


def make(total, H, slots, seed, page_pad=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.rand(1, total, H, D, generator=g).bfloat16()
    k = torch.rand(1, total, H, D, generator=g).bfloat16()
    v = torch.rand(1, total, H, D, generator=g).bfloat16()
    raw_g = torch.randn(1, total, H, D, generator=g).bfloat16()
    raw_beta = torch.randn(1, total, H, generator=g).bfloat16()
    A_log = torch.log(torch.empty(H).uniform_(1, 16, generator=g))
    dt_bias = torch.randn(H * D, generator=g)
    flat = torch.randn(slots, H * D * D + page_pad, generator=g) * 0.1
    pool = flat[:, :H * D * D].view(slots, H, D, D)     # stride(0) > H*V*K when page_pad > 0
    return q, k, v, raw_g, raw_beta, A_log, dt_bias, flat, pool


def run_case(lengths, H, indices, num_accepted, is_sglang, lower_bound, page_pad, seed):
    from pla_b200.decode.kda import fused_recurrent_kda
    total, slots = sum(lengths), 12
    q, k, v, raw_g, raw_beta, A_log, dt_bias, flat, pool = make(total, H, slots, seed, page_pad)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int64)
    idx = torch.tensor(indices, dtype=torch.int64)
    decode_path = idx.dim() == 1 and total == len(lengths)
    bias_seen = dt_bias.bfloat16().float() if decode_path else dt_bias
    exp_out, exp_pool, _ = odec.klast_forward(
        q=q[0], k=k[0], v=v[0], a=raw_g[0], b=raw_beta[0], A_log=A_log, dt_bias=bias_seen, state=pool,
        slot_indices=idx, lengths=lengths, scale=D ** -0.5, is_kda=True, lower_bound=lower_bound,
        is_sglang=is_sglang, disable_state_update=idx.dim() == 2,
        num_accepted=None if num_accepted is None else list(num_accepted))
    dflat = flat.cuda()
    dpool = dflat[:, :H * D * D].view(slots, H, D, D)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    acc = None if num_accepted is None else torch.tensor(num_accepted, dtype=torch.int64, device="cuda")
    out, state = fused_recurrent_kda(q.cuda(), k.cuda(), v.cuda(), raw_g.cuda(), raw_beta.cuda(), A_log.cuda(),
                                     dt_bias.cuda(), lower_bound, dpool, cu.cuda(), idx.cuda(), acc, None, None,
                                     is_sglang, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert state.data_ptr() == dpool.data_ptr()
    assert_out_close(out[0], exp_out)
    assert_state_close(dpool.cpu(), exp_pool)
    if page_pad:
        assert torch.equal(dflat[:, H * D * D:].cpu(), flat[:, H * D * D:])     # page tails untouched


@pytest.mark.gpu
@pytest.mark.parametrize("lower_bound", [None, -5.0])
def test_decode_path_sglang_1d(native_built, lower_bound):
    run_case([1, 1, 1, 1], 4, [5, 0, -1, 9], None, True, lower_bound, 0, 1)


@pytest.mark.gpu
@pytest.mark.parametrize("is_sglang", [True, False])
def test_multi_token_1d(native_built, is_sglang):
    run_case([3, 1, 0, 2], 2, [4, 0, 7, 2], None, is_sglang, -5.0, 0, 2)


@pytest.mark.gpu
@pytest.mark.parametrize("page_pad", [0, 256])
def test_per_token_slots_vllm(native_built, page_pad):
    table = [[1, 2, 3, 4], [5, 6, 7, 8], [0, 0, 0, 0], [9, 10, 11, 0]]
    run_case([4, 2, 4, 3], 2, table, [1, 3, 1, 2], False, None, page_pad, 3)


def test_exception_types(native_built):
    from pla_b200.decode.kda import fused_recurrent_kda
    q, k, v, raw_g, raw_beta, A_log, dt_bias, _, pool = make(2, 1, 2, 0)
    cu = torch.tensor([0, 2])
    idx = torch.tensor([1])
    args = lambda **kw: dict(dict(q=q, k=k, v=v, raw_g=raw_g, raw_beta=raw_beta, A_log=A_log, dt_bias=dt_bias,
                                  lower_bound=None, initial_state=pool, cu_seqlens=cu, ssm_state_indices=idx), **kw)
    with pytest.raises(NotImplementedError):
        fused_recurrent_kda(**args(fuse_gate=False))
    with pytest.raises(ValueError):
        fused_recurrent_kda(**args(dt_bias=None))
    with pytest.raises(ValueError):
        fused_recurrent_kda(**args(q=q[0]))
    with pytest.raises(NotImplementedError):
        fused_recurrent_kda(**args(q=q[..., :64]))
    with pytest.raises(ValueError):
        fused_recurrent_kda(**args(initial_state=pool.bfloat16()))
    with pytest.raises(ValueError):
        fused_recurrent_kda(**args(ssm_state_indices=torch.tensor([[1, 1]]), is_sglang=True))
    with pytest.raises(ValueError):
        fused_recurrent_kda(**args(dt_bias=dt_bias.bfloat16()))
