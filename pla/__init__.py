"""``pla`` — the reference's package name on top of :mod:`pla_b200`.

A serving stack that imports ``pla.decode``, ``pla.decode.gdn.v_last``, ``pla.decode.kda``,
``pla.decode.kda_replayssm_sglang`` / ``kda_mtp_sglang`` / ``kda_replayssm_vllm``, ``pla.prefill.flashqla`` or
``pla.prefill.flashkdapro`` gets the B200 operators with the same function names, argument order and tensor
contracts. Like the reference's root package this one exports nothing itself; every namespace below is the
``pla_b200`` module of the same name (one module object, two names). Importing it loads the native libraries:
there is no fallback, a missing build is an ImportError.
"""
import importlib
import sys

__version__ = "1.1.0"      # the interface version this package mirrors (pla/__init__.py:51 of the reference)
__all__ = []

NAMESPACES = (
    "decode", "decode.gdn", "decode.gdn.v_last", "decode.kda", "decode.kda_replayssm_sglang",
    "decode.kda_mtp_sglang", "decode.kda_replayssm_vllm", "prefill", "prefill.flashqla", "prefill.flashkdapro",
)

for _name in NAMESPACES:
    _module = importlib.import_module("pla_b200." + _name)
    sys.modules[__name__ + "." + _name] = _module
    _parent, _, _leaf = _name.rpartition(".")
    setattr(sys.modules[__name__ + "." + _parent] if _parent else sys.modules[__name__], _leaf, _module)
del _name, _module, _parent, _leaf
