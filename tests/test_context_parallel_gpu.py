"""Context-parallel prefill kernels on one GPU: the ranks of a group are emulated one after another
(no kernel waits on another), so the prescan pairs, the fold and the segment pass are all checked
against the single-pass kernel and the CPU oracle."""
import pytest
import torch

from helpers import OracleSegmentKernels, assert_out_close, assert_state_close
from oracle import decode as odec

pytestmark = pytest.mark.gpu
D = 128


def make(T, Hg, H, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, Hg, D, generator=g).bfloat16()
    k = torch.randn(T, Hg, D, generator=g).bfloat16()
    v = torch.randn(T, H, D, generator=g).bfloat16()
    gate = torch.randn(T, H, generator=g).bfloat16()
    beta = torch.randn(T, H, generator=g).bfloat16()
    A_log = torch.rand(H, generator=g) * 2.0
    dt_bias = torch.randn(H, generator=g) * 0.1
    S0 = torch.randn(H, D, D, generator=g) * 0.05
    return q, k, v, gate, beta, A_log, dt_bias, S0


@pytest.mark.parametrize("T", [200, 2240])
def test_prescan_pairs_match_the_oracle(native_built, T):
    """T = 2240: the rank runs as two token ranges and composes their pairs into its own."""
    from pla_b200.prefill import context_parallel as cp
    Hg, H = 1, 2
    q, k, v, gate, beta, A_log, dt_bias, _ = make(T, Hg, H, 11)
    ref = OracleSegmentKernels(q, k, v, gate, beta, A_log, dt_bias, D ** -0.5).prescan()
    kern = cp.CudaSegmentKernels(q.cuda(), k.cuda(), v.cuda(), gate.cuda(), beta.cuda(), A_log.cuda(), dt_bias.cuda(),
                                 D ** -0.5, True, False)
    assert kern.parts == (2 if T == 2240 else 1)
    kern.prepare()
    mb = kern.prescan()
    kern.check()
    assert_state_close(mb[:, 0].cpu(), ref[:, 0], "offset B")
    assert_state_close(mb[:, 1].cpu(), ref[:, 1], "transition M")


@pytest.mark.parametrize("splits", [(400, 0, 333, 767), (64, 64), (1000,), (2240, 2300), (2500,)])
def test_emulated_ranks_match_single_pass_and_oracle(native_built, splits):
    from pla_b200._ops import ops
    from pla_b200.prefill import context_parallel as cp
    T, Hg, H, W = sum(splits), 2, 4, len(splits)
    q, k, v, gate, beta, A_log, dt_bias, S0 = make(T, Hg, H, 23)
    dev = torch.device("cuda")
    dq, dk, dv, dg, db = (x.to(dev) for x in (q, k, v, gate, beta))
    dA, dB, dS0 = A_log.to(dev), dt_bias.to(dev), S0.to(dev)
    plans, lo = [], 0
    for r, n in enumerate(splits):
        sl = slice(lo, lo + n)
        kern = cp.CudaSegmentKernels(dq[sl], dk[sl], dv[sl], dg[sl], db[sl], dA, dB, D ** -0.5, True, False)
        plans.append(cp.begin_segment(kern, r, W, n, H, dev))
        lo += n
    gathered = torch.stack([p.transfer for p in plans])
    outs, state = [], None
    for p in plans:
        o, state = cp.finish_segment(p, dS0, gathered)
        if o is not None:
            outs.append(o)
        p.kernels.check()
    out = torch.cat(outs)

    # the same kernels in a single pass
    one = torch.empty(T, H, D, dtype=torch.bfloat16, device=dev)
    final = torch.empty(1, H, D, D, dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.gdn_prefill_chunked(dq, dk, dv, dg, db, dA, dB, one, None, torch.tensor([0, T], dtype=torch.int32, device=dev),
                            dS0[None].contiguous(), None, final, None, False, True, D ** -0.5, False, False,
                            (T + 63) // 64, 0, status)
    assert status.item() == 0
    assert_out_close(out, one, "ranks vs single pass")
    assert_state_close(state, final[0], "ranks vs single pass")

    exp_out, exp_state, _ = odec.klast_forward(q=q, k=k, v=v, a=gate, b=beta, A_log=A_log, dt_bias=dt_bias,
                                               state=S0[None], slot_indices=[0], lengths=[T], scale=D ** -0.5)
    assert_out_close(out, exp_out)
    assert_state_close(state.cpu(), exp_state[0])


def make_kda(T, H, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, H, D, generator=g).bfloat16()
    k = torch.randn(T, H, D, generator=g).bfloat16()
    v = torch.randn(T, H, D, generator=g).bfloat16()
    gate = torch.randn(T, H, D, generator=g).bfloat16()
    beta = torch.randn(T, H, generator=g).bfloat16()
    A_log = -4.0 + 2.0 * torch.rand(H, generator=g)            # weak decay, as the long-sequence config states
    dt_bias = torch.randn(H, D, generator=g) * 0.1
    S0 = torch.randn(H, D, D, generator=g) * 0.05
    return q, k, v, gate, beta, A_log, dt_bias, S0


@pytest.mark.parametrize("chunked,splits", [(False, (90, 37, 0, 61)), (True, (90, 37, 0, 61)), (True, (2240, 2100))])
@pytest.mark.parametrize("lower_bound", [-5.0, None])
def test_kda_emulated_ranks_match_oracle(native_built, lower_bound, chunked, splits):
    """KDA: prescan pairs of the token-recurrent kernel against the oracle, then ranks emulated one after
    another against the serial oracle recurrence. The long split runs every rank as two token ranges."""
    from pla_b200.prefill import context_parallel as cp
    T, H, W = sum(splits), 2, len(splits)
    q, k, v, gate, beta, A_log, dt_bias, S0 = make_kda(T, H, 31)
    dev = torch.device("cuda")
    dq, dk, dv, dg, db = (x.to(dev) for x in (q, k, v, gate, beta))
    dA, dB, dS0 = A_log.to(dev), dt_bias.to(dev), S0.to(dev)
    plans, lo = [], 0
    for r, n in enumerate(splits):
        sl = slice(lo, lo + n)
        if chunked:
            kern = cp.KdaChunkedSegmentKernels(dq[sl], dk[sl], dv[sl], dg[sl], db[sl], dA, dB, D ** -0.5, True,
                                               lower_bound)
        else:
            kern = cp.RecurrentSegmentKernels(dq[sl], dk[sl], dv[sl], dg[sl], db[sl], dA, dB, D ** -0.5, True, False,
                                              True, lower_bound)
        plans.append(cp.begin_segment(kern, r, W, n, H, dev))
        if r == 0:
            ref = OracleSegmentKernels(q[sl], k[sl], v[sl], gate[sl], beta[sl], A_log, dt_bias, D ** -0.5, is_kda=True,
                                       lower_bound=lower_bound).prescan()
            assert_state_close(plans[0].transfer[:, 0].cpu(), ref[:, 0], "offset B")
            # over thousands of tokens the transition shrinks far below the offset, and its tf32 rounding errors
            # (relative to its own small norm) grow with the chunk count; the states it produces are checked below
            assert_state_close(plans[0].transfer[:, 1].cpu(), ref[:, 1], "transition M", tol=1e-3 if n < 1000 else 5e-3)
        lo += n
    gathered = torch.stack([p.transfer for p in plans])
    outs, state = [], None
    for p in plans:
        o, state = cp.finish_segment(p, dS0, gathered)
        if o is not None:
            outs.append(o)
        p.kernels.check()
    exp_out, exp_state, _ = odec.klast_forward(q=q, k=k, v=v, a=gate, b=beta, A_log=A_log, dt_bias=dt_bias,
                                               state=S0[None], slot_indices=[0], lengths=[T], scale=D ** -0.5,
                                               is_kda=True, lower_bound=lower_bound)
    assert_out_close(torch.cat(outs), exp_out)
    assert_state_close(state.cpu(), exp_state[0])


def test_fold_kernel_matches_torch_fold(native_built):
    from pla_b200._ops import ops
    from pla_b200.prefill import context_parallel as cp
    g = torch.Generator().manual_seed(2)
    W, H = 5, 3
    pairs = torch.randn(W, H, 2, D, D, generator=g) * 0.09
    S0 = torch.randn(H, D, D, generator=g)
    dp, dS = pairs.cuda(), S0.cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for rank in range(W):
        for init, dinit in ((S0, dS), (None, None)):
            got = ops.cp_fold_prefix(dp, dinit, rank, status)
            want = cp.fold_transfers(init, pairs, rank)
            torch.testing.assert_close(got.cpu(), want, rtol=1e-4, atol=1e-5)
    # composition of the first n pairs into one: applying it equals applying the n pairs in turn
    for n in range(W + 1):
        one = ops.cp_compose_pairs(dp, n, status).cpu()
        assert one.shape == (H, 2, D, D)
        want = cp.fold_transfers(S0, pairs, n)
        torch.testing.assert_close(torch.baddbmm(one[:, 0], S0, one[:, 1]), want, rtol=1e-4, atol=1e-5)
        if n == 0:
            assert torch.equal(one, cp.identity_transfer(H, "cpu"))
    assert status.item() == 0
