"""Compatibility name of the SGLang ReplaySSM API (pla/decode/kda_mtp_sglang/__init__.py of the reference):
the same two functions as :mod:`pla_b200.decode.kda_replayssm_sglang`."""
from ..kda_replayssm_sglang import commit_kda_replayssm_after_verify, fused_kda_decode_mtp_dspark

__all__ = ["fused_kda_decode_mtp_dspark", "commit_kda_replayssm_after_verify"]
