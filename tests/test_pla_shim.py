"""The ``pla`` package name: every namespace of the reference resolves to the pla_b200 module of the same name, and
every facade takes the reference's positional arguments in the reference's order (the pybind argument lists of
src/decode/k-last/fused_sigmoid_gating.cpp:164-259 and the Python signatures of pla/prefill/*/ops.py and
pla/decode/kda_replayssm_*/__init__.py). Loads the native libraries, launches nothing."""
import importlib
import inspect

import pytest


@pytest.fixture(scope="module")
def pla(native_built):
    return importlib.import_module("pla")


def positional(fn):
    return [p.name for p in inspect.signature(fn).parameters.values()
            if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]


K_LAST = ["A_log", "a", "dt_bias", "softplus_beta", "softplus_threshold", "q", "k", "v", "b", "initial_state_source",
          "initial_state_indices", "scale", "use_qk_l2norm_in_kernel", "cu_seqlens", "is_kda", "disable_state_update",
          "intermediate_states_buffer", "intermediate_state_indices", "cache_steps_or_num_accept",
          "retrieve_parent_token", "lower_bound", "is_sglang", "out"]
K_LAST_PACKED = ["mixed_qkv", "a", "b", "A_log", "dt_bias", "softplus_beta", "softplus_threshold", "scale",
                 "initial_state_source", "initial_state_indices", "out", "use_qk_l2norm_in_kernel", "cu_seqlens", "is_kda",
                 "is_sglang"]
MEGA = ["x", "weight", "bias", "conv_state", "raw_g", "raw_beta", "a_log", "dt_bias", "state_indices", "state", "out",
        "lower_bound", "output_gate", "norm_weight", "norm_eps"]
RECURRENT_KDA = ["q", "k", "v", "raw_g", "raw_beta", "A_log", "dt_bias", "lower_bound", "initial_state", "cu_seqlens",
                 "ssm_state_indices", "num_accepted_tokens", "out", "fuse_gate", "is_sglang"]
CHUNK_FWD = ["q", "k", "v", "g", "beta", "scale", "initial_state", "initial_state_indices", "cu_seqlens",
             "output_final_state", "auto_cp", "overlap_warmup_threshold", "force_tc01_cp_candidate", "normalize_qk",
             "raw_cu_seqlens", "raw_gate_a", "raw_beta_b", "A_log", "dt_bias", "final_state_dtype"]
PACKED_PREFILL = ["packed_qkv", "raw_gate_a", "raw_beta_b", "A_log", "dt_bias", "cu_seqlens"]
FLASHKDA = ["q", "k", "v", "g", "beta", "A_log", "dt_bias", "out", "scale", "lower_bound", "initial_state", "final_state",
            "cu_seqlens", "state_pool", "state_indices", "raw_cu_seqlens"]


def test_namespaces_are_the_pla_b200_modules(pla):
    import sys
    for name in pla.NAMESPACES:
        module = importlib.import_module("pla." + name)
        assert module is sys.modules["pla_b200." + name]
    from pla.decode.kda_mtp_sglang import commit_kda_replayssm_after_verify, fused_kda_decode_mtp_dspark
    import pla.decode.kda_replayssm_sglang as sg
    assert fused_kda_decode_mtp_dspark is sg.fused_kda_decode_mtp_dspark
    assert commit_kda_replayssm_after_verify is sg.commit_kda_replayssm_after_verify
    assert pla.__all__ == []


def test_facades_take_the_reference_positional_arguments(pla):
    import pla.decode as dec
    import pla.decode.kda as kda
    import pla.prefill.flashkdapro as fk
    import pla.prefill.flashqla as fq
    assert positional(dec.fused_sigmoid_gating_delta_rule_forward_k_last) == K_LAST
    assert positional(dec.fused_sigmoid_gating_delta_rule_forward_k_last_packed) == K_LAST_PACKED
    assert positional(kda.fused_kda_decode_mega_forward) == MEGA
    assert positional(kda.fused_recurrent_kda) == RECURRENT_KDA
    assert positional(fq.chunk_gated_delta_rule_fwd) == CHUNK_FWD
    assert positional(fq.gdn_prefill_packed_qkv_fwd) == PACKED_PREFILL
    assert positional(fk.flashkda_fwd) == FLASHKDA
    # everything this library adds to a reference signature is keyword-only
    for fn in (dec.fused_sigmoid_gating_delta_rule_forward_k_last, dec.fused_sigmoid_gating_delta_rule_forward_k_last_packed,
               kda.fused_kda_decode_mega_forward, kda.fused_recurrent_kda, fk.flashkda_fwd):
        extra = [p.name for p in inspect.signature(fn).parameters.values() if p.kind == p.KEYWORD_ONLY]
        assert set(extra) <= {"status", "rows_per_cta", "backend", "auto_cp"}, extra
