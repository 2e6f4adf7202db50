"""GDN prefill — the surface of ``pla.prefill.flashqla`` (pla/prefill/flashqla/ops.py:225-738)."""
from .ops import chunk_gated_delta_rule_fwd, gdn_prefill_packed_qkv_fwd  # noqa: F401

__all__ = ["chunk_gated_delta_rule_fwd", "gdn_prefill_packed_qkv_fwd"]
