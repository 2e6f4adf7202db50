"""The C ABI called the way a binding in another language would call it: plain device pointers obtained from the
CUDA runtime, the header's argument structures filled field by field, a raw stream handle -- no torch tensor
anywhere near the library. Results are checked against the CPU oracle. Covers the k-last decode, the v-last decode
and the chunked GDN prefill entries (the three whose structures every serving path fills)."""
import ctypes

import numpy as np
import pytest
import torch

from helpers import assert_out_close, assert_state_close
from oracle import decode as odec

pytestmark = pytest.mark.gpu
D = 128
BF16, F32 = 0, 2


class Device:
    """Device buffers straight from the CUDA runtime (cuda-python), freed when the test ends."""

    def __init__(self):
        from cuda.bindings import runtime as rt
        self.rt, self.ptrs = rt, []
        err, = rt.cudaSetDevice(0)
        assert int(err) == 0

    def put(self, host: torch.Tensor) -> int:
        host = host.contiguous()
        nbytes = host.numel() * host.element_size()
        err, ptr = self.rt.cudaMalloc(max(nbytes, 16))
        assert int(err) == 0
        self.ptrs.append(ptr)
        err, = self.rt.cudaMemcpy(ptr, host.data_ptr(), nbytes, self.rt.cudaMemcpyKind.cudaMemcpyHostToDevice)
        assert int(err) == 0
        return int(ptr)

    def zeros(self, nbytes: int) -> int:
        err, ptr = self.rt.cudaMalloc(max(nbytes, 16))
        assert int(err) == 0
        self.ptrs.append(ptr)
        err, = self.rt.cudaMemset(ptr, 0, max(nbytes, 16))
        assert int(err) == 0
        return int(ptr)

    def get(self, ptr: int, like: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(like).contiguous()
        err, = self.rt.cudaMemcpy(out.data_ptr(), ptr, out.numel() * out.element_size(),
                                  self.rt.cudaMemcpyKind.cudaMemcpyDeviceToHost)   # synchronises with the null stream
        assert int(err) == 0
        return out

    def close(self):
        for p in self.ptrs:
            self.rt.cudaFree(p)


@pytest.fixture
def dev():
    d = Device()
    yield d
    d.close()


def _decode_inputs(B, H, HV, slots, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, D, generator=g).bfloat16()
    k = torch.randn(B, H, D, generator=g).bfloat16()
    v = torch.randn(B, HV, D, generator=g).bfloat16()
    a = torch.randn(B, HV, generator=g).bfloat16()
    b = torch.randn(B, HV, generator=g).bfloat16()
    A_log = torch.rand(HV, generator=g) * 2.0
    dt_bias = (torch.randn(HV, generator=g) * 0.1).bfloat16()
    pool = torch.randn(slots, HV, D, D, generator=g) * 0.05
    idx = torch.randperm(slots, generator=g)[:B].to(torch.int32)
    return q, k, v, a, b, A_log, dt_bias, pool, idx


def test_layout_of_the_mirrored_structures(native_built):
    from pla_b200 import capi
    capi.check_layout(capi.load())


def test_decode_klast_through_the_c_abi(native_built, dev):
    from pla_b200 import capi
    lib = capi.load()
    B, H, HV, slots = 6, 2, 4, 9
    q, k, v, a, b, A_log, dt_bias, pool, idx = _decode_inputs(B, H, HV, slots, 3)
    idx[2] = -1
    exp_out, exp_state, _ = odec.klast_forward(q=q, k=k, v=v, a=a, b=b, A_log=A_log, dt_bias=dt_bias, state=pool,
                                               slot_indices=idx.tolist(), lengths=[1] * B, scale=D ** -0.5)
    x = capi.pla_b200_klast_args()
    x.q, x.k, x.v, x.a, x.b = (dev.put(t) for t in (q, k, v, a, b))
    o_like = torch.empty(B, HV, D, dtype=torch.bfloat16)
    x.o = dev.zeros(o_like.numel() * 2)
    x.q_tok_stride = x.k_tok_stride = H * D
    x.v_tok_stride = HV * D
    x.a_tok_stride = x.b_tok_stride = HV
    x.A_log, x.dt_bias = dev.put(A_log), dev.put(dt_bias)
    x.act_dtype, x.A_log_dtype, x.dt_bias_dtype, x.state_dtype = BF16, F32, BF16, F32
    x.state = dev.put(pool)
    x.state_slot_stride, x.num_slots = HV * D * D, slots
    x.slot_indices = dev.put(idx)
    x.B, x.t_max, x.H, x.HV = B, 1, H, HV
    x.scale, x.softplus_beta, x.softplus_threshold = D ** -0.5, 1.0, 20.0
    x.use_qk_l2norm = 1
    status = dev.zeros(4)
    x.status = status
    rc = lib.pla_b200_decode_klast(ctypes.byref(x), None)      # NULL = the legacy default stream
    assert rc == 0, lib.pla_b200_last_error()
    assert dev.get(status, torch.zeros(1, dtype=torch.int32)).item() == 0
    assert_out_close(dev.get(x.o, o_like), exp_out)
    assert_state_close(dev.get(x.state, pool), exp_state)
    # a contract violation comes back as a code and a message, nothing is launched
    x.HV = 3
    assert lib.pla_b200_decode_klast(ctypes.byref(x), None) == -1
    assert b"multiple of H" in lib.pla_b200_last_error()


def test_decode_vlast_through_the_c_abi(native_built, dev):
    from pla_b200 import capi
    lib = capi.load()
    B, H, HV, slots = 5, 2, 4, 8
    q, k, v, a, b, A_log, dt_bias, pool, idx = _decode_inputs(B, H, HV, slots, 4)
    pool_v = pool.transpose(-1, -2).contiguous()                # [slots, HV, K, V]
    exp_out, exp_state = odec.vlast_forward(q=q, k=k, v=v, a=a, b=b, A_log=A_log, dt_bias=dt_bias, state=pool_v,
                                            slot_indices=idx.tolist(), scale=D ** -0.5)
    x = capi.pla_b200_vlast_args()
    x.q, x.k, x.v, x.a, x.b = (dev.put(t) for t in (q, k, v, a, b))
    o_like = torch.empty(B, HV, D, dtype=torch.bfloat16)
    x.o = dev.zeros(o_like.numel() * 2)
    x.A_log, x.dt_bias = dev.put(A_log), dev.put(dt_bias)
    x.act_dtype, x.A_log_dtype = BF16, F32
    x.state, x.num_slots = dev.put(pool_v), slots
    x.slot_indices = dev.put(idx)
    x.B, x.H, x.HV = B, H, HV
    x.scale, x.softplus_beta, x.softplus_threshold = D ** -0.5, 1.0, 20.0
    x.use_qk_l2norm = 1
    rc = lib.pla_b200_decode_vlast(ctypes.byref(x), None)
    assert rc == 0, lib.pla_b200_last_error()
    assert_out_close(dev.get(x.o, o_like), exp_out)
    assert_state_close(dev.get(x.state, pool_v), exp_state)


def test_gdn_prefill_chunked_through_the_c_abi(native_built, dev):
    from pla_b200 import capi
    lib = capi.load()
    Hg, H, lengths, slots = 1, 2, [150, 70], 5
    T, N = sum(lengths), len(lengths)
    g = torch.Generator().manual_seed(8)
    q = torch.randn(T, Hg, D, generator=g).bfloat16()
    k = torch.randn(T, Hg, D, generator=g).bfloat16()
    v = torch.randn(T, H, D, generator=g).bfloat16()
    gate = torch.randn(T, H, generator=g).bfloat16()
    beta = torch.randn(T, H, generator=g).bfloat16()
    A_log = torch.rand(H, generator=g) * 2.0
    dt_bias = torch.randn(H, generator=g) * 0.1
    pool = torch.randn(slots, H, D, D, generator=g) * 0.05
    idx = torch.tensor([3, 1], dtype=torch.int32)
    cu = torch.tensor([0, 150, T], dtype=torch.int32)
    exp_out, exp_state, _ = odec.klast_forward(q=q, k=k, v=v, a=gate, b=beta, A_log=A_log, dt_bias=dt_bias, state=pool,
                                               slot_indices=idx.tolist(), lengths=lengths, scale=D ** -0.5)
    x = capi.pla_b200_gdn_chunk_args()
    x.q, x.k, x.v = (dev.put(t) for t in (q, k, v))
    x.q_tok_stride = x.k_tok_stride = Hg * D
    x.v_tok_stride = H * D
    x.act_dtype = BF16
    x.gate, x.beta = dev.put(gate), dev.put(beta)
    x.gate_tok_stride = x.beta_tok_stride = H
    x.A_log, x.dt_bias = dev.put(A_log), dev.put(dt_bias)
    o_like = torch.empty(T, H, D, dtype=torch.bfloat16)
    x.o = dev.zeros(o_like.numel() * 2)
    x.state, x.state_dtype = dev.put(pool), F32
    x.state_slot_stride, x.num_slots = H * D * D, slots
    x.slot_indices = dev.put(idx)
    x.write_state = 1
    x.N, x.cu_seqlens, x.T_total = N, dev.put(cu), T
    x.max_chunks = sum((n + 63) // 64 for n in lengths)
    x.H, x.HV = Hg, H
    x.scale, x.normalize_qk = D ** -0.5, 1
    need = lib.pla_b200_gdn_chunk_workspace_bytes(x.max_chunks, Hg, H)
    assert need > 0
    x.workspace, x.workspace_bytes = dev.zeros(need), need
    status = dev.zeros(4)
    x.status = status
    rc = lib.pla_b200_gdn_prefill_chunked(ctypes.byref(x), None)
    assert rc == 0, lib.pla_b200_last_error()
    assert dev.get(status, torch.zeros(1, dtype=torch.int32)).item() == 0
    assert_out_close(dev.get(x.o, o_like), exp_out)
    assert_state_close(dev.get(x.state, pool), exp_state)
    x.workspace_bytes = need - 1
    assert lib.pla_b200_gdn_prefill_chunked(ctypes.byref(x), None) == -1
    assert b"workspace" in lib.pla_b200_last_error()
