"""KDA prefill — the surface of ``pla.prefill.flashkdapro`` (pla/prefill/flashkdapro/ops.py:66-219)."""
from .ops import flashkda_fwd  # noqa: F401

__all__ = ["flashkda_fwd"]
