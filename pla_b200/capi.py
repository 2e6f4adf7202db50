"""ctypes view of the C ABI in ``include/pla_b200.h`` (torch-free: plain pointers and sizes).

Every argument structure of the header is mirrored here as a ``ctypes.Structure`` of the same name, built by
reading the header itself, so the two cannot drift apart; ``check_layout`` compares every structure's size and
every field's offset with what the compiled library reports (``pla_b200_struct_size`` /
``pla_b200_field_offset``). A binding in another language would declare the same structures by hand.
"""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "lib" / "libpla_b200.so"
HEADER_PATH = PKG.parent / "include" / "pla_b200.h"

_SCALARS = {"int32_t": ctypes.c_int32, "int64_t": ctypes.c_int64, "float": ctypes.c_float, "uint8_t": ctypes.c_uint8}


def _parse_header(text: str):
    """``typedef struct NAME { ... } NAME;`` blocks -> {name: [(field, ctype), ...]} in declaration order.
    Field types the header uses: pointers (any), int32_t, int64_t, float, and earlier structures by value."""
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    structs = {}
    for name, body in re.findall(r"typedef\s+struct\s+(\w+)\s*\{(.*?)\}\s*\1\s*;", text, flags=re.S):
        fields = []
        for decl in body.split(";"):
            decl = " ".join(decl.split())
            if not decl:
                continue
            base, _, names = decl.rpartition(" ") if "," not in decl else (None, None, None)
            if base is None:       # "type a, b, c" (possibly "type* a, *b")
                first, *rest = [part.strip() for part in decl.split(",")]
                base, _, head = first.rpartition(" ")
                names_list = [head] + rest
            else:
                names_list = [names]
            base = base.replace("const ", "").strip()
            for ident in names_list:
                stars = base.count("*") + ident.count("*")
                ident = ident.replace("*", "").strip()
                kind = base.replace("*", "").strip()
                if stars:
                    ctype = ctypes.c_void_p
                elif kind in _SCALARS:
                    ctype = _SCALARS[kind]
                elif kind in structs:
                    ctype = structs[kind]["class"]
                else:
                    raise ValueError(f"{name}.{ident}: unknown field type {kind!r}")
                fields.append((ident, ctype))
        cls = type(name, (ctypes.Structure,), {"_fields_": fields, "__doc__": f"``{name}`` of include/pla_b200.h."})
        structs[name] = {"class": cls, "fields": fields}
    return structs


STRUCTS = _parse_header(HEADER_PATH.read_text())
globals().update({name: entry["class"] for name, entry in STRUCTS.items()})

# short names used by the tests
Index = STRUCTS["pla_b200_index"]["class"]
KdaCommitArgs = STRUCTS["pla_b200_kda_commit_args"]["class"]

_ENTRY_ARGS = {
    "pla_b200_decode_klast": "pla_b200_klast_args", "pla_b200_prefill_recurrent": "pla_b200_klast_args",
    "pla_b200_decode_vlast": "pla_b200_vlast_args", "pla_b200_gdn_prefill_chunked": "pla_b200_gdn_chunk_args",
    "pla_b200_kda_prefill_chunked": "pla_b200_gdn_chunk_args", "pla_b200_cp_fold_prefix": "pla_b200_cp_fold_args",
    "pla_b200_cp_fold_segments": "pla_b200_cp_fold_segments_args",
    "pla_b200_kda_replay_verify": "pla_b200_kda_verify_args", "pla_b200_kda_ring_verify": "pla_b200_kda_verify_args",
    "pla_b200_kda_fold_layers": "pla_b200_kda_fold_args", "pla_b200_kda_conv_scatter": "pla_b200_kda_conv_scatter_args",
    "pla_b200_kda_replay_plan": "pla_b200_kda_commit_args", "pla_b200_kda_replay_commit": "pla_b200_kda_commit_args",
    "pla_b200_kda_replay_plan_static": "pla_b200_kda_commit_args", "pla_b200_kda_decode_mega": "pla_b200_kda_mega_args",
    "pla_b200_causal_conv_prefill": "pla_b200_conv_prefill_args",
}


def load() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(f"{LIB_PATH} is not built; run `python -m pla_b200.build`")
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.pla_b200_last_error.restype = ctypes.c_char_p
    for name, struct in _ENTRY_ARGS.items():
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.POINTER(STRUCTS[struct]["class"]), ctypes.c_void_p]
    lib.pla_b200_struct_size.restype = ctypes.c_int64
    lib.pla_b200_struct_size.argtypes = [ctypes.c_char_p]
    lib.pla_b200_field_offset.restype = ctypes.c_int64
    lib.pla_b200_field_offset.argtypes = [ctypes.c_char_p, ctypes.c_char_p]
    lib.pla_b200_gdn_chunk_workspace_bytes.restype = ctypes.c_int64
    lib.pla_b200_gdn_chunk_workspace_bytes.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]
    lib.pla_b200_kda_chunk_workspace_bytes.restype = ctypes.c_int64
    lib.pla_b200_kda_chunk_workspace_bytes.argtypes = [ctypes.c_int32, ctypes.c_int32]
    lib.pla_b200_device_status.restype = ctypes.c_int
    lib.pla_b200_device_status.argtypes = [ctypes.POINTER(ctypes.c_int32), ctypes.c_int]
    return lib


def check_layout(lib: ctypes.CDLL) -> None:
    """Raises AssertionError when a mirrored structure differs from the compiled one in size or in any field offset."""
    for name, entry in STRUCTS.items():
        cls = entry["class"]
        want = lib.pla_b200_struct_size(name.encode())
        assert want > 0, f"the library does not know {name}"
        assert ctypes.sizeof(cls) == want, f"sizeof({name}): header mirror {ctypes.sizeof(cls)}, library {want}"
        for field, _ in entry["fields"]:
            off = lib.pla_b200_field_offset(name.encode(), field.encode())
            assert off == getattr(cls, field).offset, f"offsetof({name}, {field}): mirror {getattr(cls, field).offset}, library {off}"


def index_of(tensor) -> "Index":
    """Describe a 1-D torch int32/int64 tensor (any stride) as a ``pla_b200_index``."""
    import torch
    if tensor is None:
        return Index(None, 0, 1)
    assert tensor.dim() == 1 and tensor.dtype in (torch.int32, torch.int64)
    return Index(tensor.data_ptr(), int(tensor.dtype == torch.int64), tensor.stride(0))


def emit_layout() -> str:
    """Source of ``csrc/abi_layout.cu``: the table behind ``pla_b200_struct_size`` / ``pla_b200_field_offset``, one
    ``offsetof`` per field of the header. Regenerate after changing the header:
    ``python -m pla_b200.capi --emit-layout``."""
    out = [
        "// Sizes and field offsets of every argument structure of include/pla_b200.h, so that a binding which mirrors",
        "// the structures in another language can check itself against the compiled library (the Python mirror does).",
        "// Generated from the header, one line per field:  python -m pla_b200.capi --emit-layout",
        "#include <stddef.h>", "#include <string.h>", "", '#include "../../include/pla_b200.h"', "", "namespace {",
        "struct FieldRow {", "  const char* type;", "  const char* field;", "  int64_t offset;", "};",
        "struct SizeRow {", "  const char* type;", "  int64_t size;", "};",
        "#define ROW(T, F) {#T, #F, static_cast<int64_t>(offsetof(T, F))}", "const FieldRow kFields[] = {"]
    for name, entry in STRUCTS.items():
        out += [f"    ROW({name}, {field})," for field, _ in entry["fields"]]
    out += ["};", "const SizeRow kSizes[] = {"]
    out += [f'    {{"{name}", static_cast<int64_t>(sizeof({name}))}},' for name in STRUCTS]
    out += ["};", "}  // namespace", "",
            'extern "C" int64_t pla_b200_struct_size(const char* type) {', "  if (type == nullptr) return -1;",
            "  for (const SizeRow& r : kSizes)", "    if (strcmp(r.type, type) == 0) return r.size;", "  return -1;", "}", "",
            'extern "C" int64_t pla_b200_field_offset(const char* type, const char* field) {',
            "  if (type == nullptr || field == nullptr) return -1;", "  for (const FieldRow& r : kFields)",
            "    if (strcmp(r.type, type) == 0 && strcmp(r.field, field) == 0) return r.offset;", "  return -1;", "}", ""]
    return "\n".join(out)


if __name__ == "__main__":
    import sys
    if "--emit-layout" in sys.argv:
        (PKG / "csrc" / "abi_layout.cu").write_text(emit_layout())
        print(PKG / "csrc" / "abi_layout.cu")
