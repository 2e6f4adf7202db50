"""Comparison helpers shared by the tests."""
from __future__ import annotations

import torch

# Parity bars of the target: bf16/fp16 outputs within 2e-2 max-abs and 1e-2
# relative L2; fp32 states within 1e-3 relative L2.
OUT_MAX_ABS = 2e-2
OUT_REL_L2 = 1e-2
STATE_REL_L2 = 1e-3


def rel_l2(x: torch.Tensor, ref: torch.Tensor) -> float:
    x, ref = x.double(), ref.double()
    den = ref.norm().item()
    return (x - ref).norm().item() / max(den, 1e-30)


def assert_out_close(out, ref, what="out"):
    out, ref = out.float().cpu(), ref.float().cpu()
    assert out.shape == ref.shape, (out.shape, ref.shape)
    assert torch.isfinite(out).all(), f"{what}: non-finite values"
    max_abs = (out - ref).abs().max().item() if out.numel() else 0.0
    r = rel_l2(out, ref) if out.numel() else 0.0
    assert max_abs <= OUT_MAX_ABS, f"{what}: max-abs {max_abs:.3e} > {OUT_MAX_ABS}"
    assert r <= OUT_REL_L2, f"{what}: rel-L2 {r:.3e} > {OUT_REL_L2}"


def assert_state_close(state, ref, what="state", tol=STATE_REL_L2):
    state, ref = state.float().cpu(), ref.float().cpu()
    assert state.shape == ref.shape, (state.shape, ref.shape)
    assert torch.isfinite(state).all(), f"{what}: non-finite values"
    r = rel_l2(state, ref)
    assert r <= tol, f"{what}: rel-L2 {r:.3e} > {tol}"


class OracleSegmentKernels:
    """The three GPU steps restated with the oracle's token recurrence (test double)."""

    def __init__(self, q, k, v, gate, beta, A_log, dt_bias, scale, **oracle_kw):
        self.q, self.k, self.v, self.gate, self.beta = q, k, v, gate, beta
        self.A_log, self.dt_bias, self.scale = A_log, dt_bias, scale
        self.H = v.shape[1]
        self.oracle_kw = oracle_kw          # e.g. is_kda=True, lower_bound=-5.0

    def _run(self, v, state):
        out, new_state, _ = _odec().klast_forward(q=self.q, k=self.k, v=v, a=self.gate, b=self.beta, A_log=self.A_log,
                                               dt_bias=self.dt_bias, state=state[None], slot_indices=[0],
                                               lengths=[v.shape[0]], scale=self.scale, **self.oracle_kw)
        return out, new_state[0]

    def prepare(self):
        pass

    def prescan(self):
        zero = torch.zeros(self.H, 128, 128)
        eye = torch.eye(128).expand(self.H, 128, 128).contiguous()
        _, B = self._run(self.v, zero)
        _, M = self._run(torch.zeros_like(self.v), eye)
        return torch.stack([B, M], dim=1)

    def segment(self, state_in):
        return self._run(self.v, state_in)


def _odec():
    from oracle import decode
    return decode
