"""pla_b200 — B200 (sm_100a) implementation of the PLA linear-attention hot path.

The sub-packages mirror the operator surface of t-head/pla
(``pla.decode``, ``pla.decode.gdn.v_last``, ``pla.decode.kda``,
``pla.decode.kda_replayssm_{sglang,vllm}``, ``pla.prefill.flashqla``,
``pla.prefill.flashkdapro``): same function names, argument order and tensor
contracts. Every op runs hand-written CUDA through the C ABI declared in
``include/pla_b200.h``; there is no CPU or PyTorch fallback — if the native
libraries are missing, importing any op sub-package raises ImportError.
"""

__version__ = "0.1.0"
