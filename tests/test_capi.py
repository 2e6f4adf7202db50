"""The C-ABI library loads and exports every symbol that include/pla_b200.h declares (no GPU needed)."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "pla_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pla_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(native_built):
    from pla_b200 import build
    lib = ctypes.CDLL(str(build.NATIVE_LIB))
    names = declared_symbols()
    assert "pla_b200_decode_klast" in names and "pla_b200_decode_vlast" in names
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    lib.pla_b200_abi_version.restype = ctypes.c_int
    assert lib.pla_b200_abi_version() == 1


def test_null_args_are_rejected_without_a_gpu(native_built):
    from pla_b200 import build
    lib = ctypes.CDLL(str(build.NATIVE_LIB))
    lib.pla_b200_last_error.restype = ctypes.c_char_p
    for name in declared_symbols():
        if name in ("pla_b200_last_error", "pla_b200_abi_version") or name.endswith("_bytes"):
            continue
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        assert fn(None, None) == -1, name
        assert b"NULL" in lib.pla_b200_last_error()


def test_ops_library_registers_the_torch_ops(native_built):
    import torch
    import pla_b200.decode  # noqa: F401
    for op in ("decode_k_last", "decode_k_last_packed", "decode_v_last"):
        assert hasattr(torch.ops.pla_b200, op)


def test_host_contract_errors_raise_runtime_error(native_built):
    import pytest
    import torch
    from pla_b200.decode import fused_sigmoid_gating_delta_rule_forward_k_last as fwd
    x = torch.zeros(1, 1, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        fwd(torch.zeros(2), torch.zeros(1, 1, 2, dtype=torch.bfloat16), torch.zeros(2, dtype=torch.bfloat16), 1.0, 20.0,
            x, x, x, torch.zeros(1, 1, 2, dtype=torch.bfloat16), torch.zeros(2, 2, 128, 128),
            torch.zeros(1, dtype=torch.int32), None, True, None, False, False, None, None, None, None)


def test_every_argument_structure_is_mirrored_with_the_library_layout(native_built):
    """pla_b200/capi.py builds its ctypes structures from the header; the library reports the compiled sizeof and
    offsetof of every field (csrc/abi_layout.cu, generated from the same header): all of them must agree, and the
    generated table must be the one the current header gives."""
    from pla_b200 import capi
    lib = capi.load()
    capi.check_layout(lib)
    assert len(capi.STRUCTS) == 14
    assert (ROOT / "pla_b200" / "csrc" / "abi_layout.cu").read_text() == capi.emit_layout()
    assert lib.pla_b200_struct_size(b"no_such_struct") == -1
    assert lib.pla_b200_field_offset(b"pla_b200_klast_args", b"no_such_field") == -1
