"""Generates the golden fixtures by running the REFERENCE's own PyTorch oracles.

Run where the reference tree is mounted:
    python tests/golden/make_golden.py [/path/to/reference]
Nothing from the reference is copied: its functions are loaded from the tree at
run time, fed the seeded inputs of ``cases.py`` and only their outputs are saved.
"""
from __future__ import annotations

import ast
import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import cases  # noqa: E402

REF = Path(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")


def load_function(path: Path, name: str, namespace: dict):
    """Compile one top-level function of a reference file without importing the
    module (its imports need the PPU extension)."""
    tree = ast.parse(path.read_text())
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == name)
    exec(compile(ast.Module([fn], []), str(path), "exec"), namespace)
    return namespace[name]


def make_klast():
    reference = load_function(REF / "tests" / "test_k_last_state_dtype.py", "reference", {"torch": torch, "F": F})
    for name in cases.KLAST_CASES:
        args, backing, lengths, state_ids, cache_ids = cases.klast_case(name)
        out, state, cache = reference(args, lengths, state_ids, cache_ids)
        blob = dict(out=out.float().numpy(), state=cases.subsample(state),
                    state_sum=np.float64(state.double().sum().item()))
        if cache is not None:
            blob["cache"] = cases.subsample(cache)
            blob["cache_sum"] = np.float64(cache.double().sum().item())
        np.savez_compressed(HERE / f"klast_{name}.npz", **blob)
        print("klast", name, {k: getattr(v, "shape", None) for k, v in blob.items()})


if __name__ == "__main__":
    torch.manual_seed(0)
    make_klast()
