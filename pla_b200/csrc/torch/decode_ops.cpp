// Host layer of the decode ops: tensor contracts of
//   pla.decode.fused_sigmoid_gating_delta_rule_forward_k_last          (src/decode/k-last/fused_sigmoid_gating_cuda_k_last.cpp:239-435)
//   pla.decode.fused_sigmoid_gating_delta_rule_forward_k_last_packed   (src/decode/k-last/fused_sigmoid_gating_cuda_k_last_packed.cpp:82-204)
//   pla.decode.gdn.v_last.fused_sigmoid_gating_delta_rule_forward      (src/decode/v-last/fused_sigmoid_gating_v_last.cpp:133-235)
// checked with TORCH_CHECK (-> RuntimeError), then one C-ABI call on the
// current stream of the tensors' device. No synchronisation, no D2H.
#include <cmath>

#include "ops_common.h"

namespace pla_ops {
namespace {

struct StateView {
  void* ptr;
  int64_t slot_stride;
  int64_t slots;
  int dtype;
};

// [slots,HV,128,128] (any slot pitch) or a flattened pool row whose stride(0)
// covers one [HV,128,128] block (src/decode/k-last/fused_sigmoid_gating_cuda_k_last.cpp:80-96).
StateView state_view(const at::Tensor& t, int64_t HV, const char* name) {
  const bool physical = t.dim() >= 4 && t.size(-3) == HV && t.size(-2) == 128 && t.size(-1) == 128;
  const bool flattened = t.dim() >= 2 && t.stride(-1) == 1 && t.stride(0) >= HV * 16384;
  TORCH_CHECK(physical || flattened,
              "state/cache head dimensions must match [HV, V, K], or be a flattened pool whose stride(0) "
              "covers HV*V*K with a unit-stride innermost dim");
  TORCH_CHECK(t.scalar_type() == at::kFloat || t.scalar_type() == at::kBFloat16, name,
              ": state dtype must be float32 or bfloat16");
  if (physical) {
    TORCH_CHECK(t.stride(-1) == 1 && t.stride(-2) == 128 && t.stride(-3) == 16384, name,
                ": the [HV, V, K] block of a slot must be contiguous");
  }
  return {t.data_ptr(), t.stride(0), t.size(0), dtype_tag(t, name)};
}

void fill_common(pla_b200_klast_args& g, const at::Tensor& A_log, const at::Tensor& a, const at::Tensor& dt_bias,
                 const at::Tensor& b, int64_t HV, bool is_kda) {
  const int64_t gate_width = is_kda ? HV * 128 : HV;
  TORCH_CHECK(b.dim() >= 2 && b.size(-1) == HV, "b head dimension must match HV");
  TORCH_CHECK(A_log.numel() == HV && dt_bias.numel() == gate_width,
              "A_log/dt_bias head dimensions must match HV and the gate type");
  TORCH_CHECK(A_log.is_contiguous() && dt_bias.is_contiguous(), "A_log and dt_bias must be contiguous");
  TORCH_CHECK(a.scalar_type() == b.scalar_type(), "a and b must share a dtype");
  g.A_log = A_log.data_ptr();
  g.A_log_dtype = dtype_tag(A_log, "A_log");
  g.dt_bias = dt_bias.data_ptr();
  g.dt_bias_dtype = dtype_tag(dt_bias, "dt_bias");
  g.a = a.data_ptr();
  g.b = b.data_ptr();
  g.b_tok_stride = b.stride(b.dim() - 2);
  TORCH_CHECK(b.stride(-1) == 1, "b heads must be contiguous");
}

void decode_k_last(const at::Tensor& A_log, const at::Tensor& a, const at::Tensor& dt_bias, double softplus_beta,
                   double softplus_threshold, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                   const at::Tensor& b, const at::Tensor& state, const at::Tensor& state_indices, double scale,
                   bool use_qk_l2norm, const std::optional<at::Tensor>& cu_seqlens, bool is_kda,
                   bool disable_state_update, const std::optional<at::Tensor>& cache,
                   const std::optional<at::Tensor>& cache_indices, std::optional<int64_t> cache_steps,
                   const std::optional<at::Tensor>& num_accepted, const std::optional<at::Tensor>& parents,
                   std::optional<double> lower_bound, bool is_sglang, at::Tensor out,
                   const std::optional<at::Tensor>& status, int64_t rows_per_cta) {
  check_cuda(q, "q");
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "q, k, v must have shape [B, T, heads, dim]");
  const int64_t H = k.size(2), HV = v.size(2), K = k.size(3), V = v.size(3);
  TORCH_CHECK(H > 0 && HV >= H && HV % H == 0, "HV must be a positive multiple of H, got H=", H, ", HV=", HV);
  TORCH_CHECK(q.sizes() == k.sizes() && v.size(0) == k.size(0) && v.size(1) == k.size(1),
              "q/k shapes and q/k/v token dimensions must match");
  TORCH_CHECK(K == 128 && V == 128,
              "fused_sigmoid_gating_delta_rule_forward_k_last requires head_dim K == V == 128, got K=", K, ", V=", V);
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 || q.scalar_type() == at::kHalf, "q must be fp16 or bf16");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type() &&
                  a.scalar_type() == q.scalar_type() && out.scalar_type() == q.scalar_type(),
              "q, k, v, a, b and out must share the activation dtype");
  TORCH_CHECK(!lower_bound.has_value() || is_kda, "lower_bound is only supported for KDA");
  for (const at::Tensor* t : {&q, &k, &v})
    TORCH_CHECK(t->stride(3) == 1 && t->stride(2) == 128, "q/k/v head and feature axes must be contiguous");
  TORCH_CHECK(a.dim() >= 2 && ((a.dim() == 4 && a.size(2) == HV && a.size(3) == (is_kda ? K : 1)) ||
                               (is_kda && a.dim() == 3 && a.size(1) == HV && a.size(2) == K) ||
                               (a.dim() != 4 && a.size(-1) == (is_kda ? HV * K : HV))),
              "a head dimensions must match HV and the gate type");
  c10::cuda::CUDAGuard guard(q.device());

  pla_b200_klast_args g{};
  fill_common(g, A_log, a, dt_bias, b, HV, is_kda);
  g.a_tok_stride = a.dim() == 4 ? a.stride(1)
                   : (is_kda && a.dim() == 3 && a.size(1) == HV && a.size(2) == K) ? a.stride(0)
                                                                                   : a.stride(a.dim() - 2);
  g.q = q.data_ptr();
  g.k = k.data_ptr();
  g.v = v.data_ptr();
  g.q_tok_stride = q.stride(1);
  g.k_tok_stride = k.stride(1);
  g.v_tok_stride = v.stride(1);
  g.act_dtype = dtype_tag(q, "q");

  const StateView sv = state_view(state, HV, "initial_state_source");
  g.state = sv.ptr;
  g.state_slot_stride = sv.slot_stride;
  g.num_slots = sv.slots;
  g.state_dtype = sv.dtype;

  TORCH_CHECK(state_indices.scalar_type() == at::kInt, "initial_state_indices must be int32");
  TORCH_CHECK(state_indices.dim() == 1 || state_indices.dim() == 2, "initial_state_indices must be [N] or [N, S]");
  TORCH_CHECK(state_indices.stride(-1) == 1, "initial_state_indices columns must be contiguous");
  g.slot_indices = state_indices.data_ptr<int32_t>();
  const bool vllm_spec = state_indices.dim() == 2;
  g.slot_row_stride = vllm_spec ? static_cast<int32_t>(state_indices.stride(0)) : 0;
  g.slot_cols = vllm_spec ? static_cast<int32_t>(state_indices.size(1)) : 0;
  TORCH_CHECK(!vllm_spec || !is_sglang,
              "2D initial_state_indices is the vLLM spec-decode layout; pass is_sglang=False");
  TORCH_CHECK(!(vllm_spec && cache_steps.has_value()),
              "vLLM spec decode expects num_accepted_tokens (a tensor) in cache_steps_or_num_accept, but received "
              "an int");
  g.num_accepted = i32_ptr(num_accepted, "num_accepted_tokens");
  g.cu_seqlens = i32_ptr(cu_seqlens, "cu_seqlens");
  if (cu_seqlens.has_value())
    TORCH_CHECK(cu_seqlens->dim() == 1 && cu_seqlens->is_contiguous(), "cu_seqlens must be contiguous [N+1]");

  const int64_t B = cu_seqlens.has_value() ? cu_seqlens->size(0) - 1 : k.size(0);
  const int64_t tokens = k.size(0) * k.size(1);
  TORCH_CHECK(state_indices.size(0) >= B, "initial_state_indices needs one row per request");
  const bool target_verify = cache.has_value() || cache_indices.has_value() || parents.has_value() ||
                             cache_steps.has_value() || vllm_spec;
  // Longest window a request may have: fixed T without cu_seqlens; otherwise a
  // bound that needs no device read (src/decode/k-last/sanity_checks.h:84-110).
  int64_t t_max;
  if (!cu_seqlens.has_value()) {
    t_max = k.size(1);
  } else {
    TORCH_CHECK(B > 0, "k-last requires at least one sequence");
    if (target_verify && vllm_spec) {
      t_max = state_indices.size(1);
    } else if (k.size(0) == B) {
      t_max = k.size(1);
    } else if (!target_verify && k.size(0) == 1 && k.size(1) == B) {
      t_max = 1;
    } else if (target_verify) {
      if (cache_steps.has_value() && *cache_steps > 0) {
        t_max = *cache_steps;
      } else {
        TORCH_CHECK(k.size(1) % B == 0, "packed target-verify tokens must be divisible by batch size");
        t_max = k.size(1) / B;
      }
    } else {
      t_max = k.size(1);
    }
  }

  if (cache.has_value()) {
    const StateView cv = state_view(*cache, HV, "intermediate_states_buffer");
    TORCH_CHECK(cache->scalar_type() == state.scalar_type(),
                "initial_state_source and intermediate_states_buffer must have the same dtype");
    TORCH_CHECK(cache->is_contiguous(), "intermediate_states_buffer must be contiguous");
    TORCH_CHECK(cache_steps.has_value() || cache->dim() >= 5,
                "the snapshot cache needs an explicit step dimension or cache_steps");
    g.cache = cv.ptr;
    // The request stride is the ALLOCATED step dimension, not the runtime window.
    g.cache_steps = static_cast<int32_t>(cache->dim() >= 5 ? cache->size(1) : *cache_steps);
    TORCH_CHECK(g.cache_steps > 0, "cache_steps must be positive");
  }
  g.cache_indices = i32_ptr(cache_indices, "intermediate_state_indices");
  if (parents.has_value()) {
    TORCH_CHECK(parents->scalar_type() == at::kLong || parents->scalar_type() == at::kInt,
                "retrieve_parent_token dtype should be int32 or int64");
    TORCH_CHECK(parents->dim() == 2, "retrieve_parent_token must be [N, tokens]");
    TORCH_CHECK(cache.has_value(), "a parent table is only valid with the SGLang intermediate cache");
    g.parents = parents->data_ptr();
    g.parents_wide = parents->scalar_type() == at::kLong;
    g.parents_seq_stride = parents->stride(0);
    g.parents_tok_stride = parents->stride(1);
  }

  if (sanity_check()) {
    std::string bad = cu_seqlens.has_value() ? sanity_offsets(*cu_seqlens, tokens, t_max) : std::string();
    if (bad.empty()) bad = sanity_slots(state_indices, sv.slots);
    TORCH_CHECK(bad.empty(), "fused_sigmoid_gating_delta_rule_forward_k_last: sanity check: ", bad);
  }
  const bool mtp = t_max > 1 || disable_state_update || target_verify;
  // dt_bias: activation dtype for plain decode; fp32 for KDA verify
  // (src/decode/k-last/fused_sigmoid_gating_cuda_k_last.cpp:201-217).
  if (is_kda && mtp) {
    TORCH_CHECK(dt_bias.scalar_type() == at::kFloat, "dt_bias must be float32 here: KDA MTP verify reads it as float32");
  } else {
    TORCH_CHECK(dt_bias.scalar_type() == q.scalar_type(), "dt_bias must have q's dtype here (only KDA MTP verify reads float32)");
  }

  TORCH_CHECK(out.is_contiguous() && out.numel() == tokens * HV * 128, "out must be contiguous with v's shape");
  g.o = out.data_ptr();
  g.B = static_cast<int32_t>(B);
  g.t_max = static_cast<int32_t>(t_max);
  g.H = static_cast<int32_t>(H);
  g.HV = static_cast<int32_t>(HV);
  g.scale = static_cast<float>(scale);
  g.softplus_beta = static_cast<float>(softplus_beta);
  g.softplus_threshold = static_cast<float>(softplus_threshold);
  g.lower_bound = static_cast<float>(lower_bound.value_or(0.0));
  g.gate = lower_bound.has_value() ? PLA_B200_GATE_SAFE : PLA_B200_GATE_SOFTPLUS;
  g.is_kda = is_kda;
  g.use_qk_l2norm = use_qk_l2norm;
  g.disable_state_update = disable_state_update;
  g.pad = is_sglang ? PLA_B200_PAD_SGLANG : PLA_B200_PAD_VLLM;
  g.rows_per_cta = static_cast<int32_t>(rows_per_cta);
  g.status = status.has_value() ? const_cast<int32_t*>(i32_ptr(status, "status")) : nullptr;
  if (!bypass_exec()) check_abi(pla_b200_decode_klast(&g, stream_of(q)), "fused_sigmoid_gating_delta_rule_forward_k_last");
}

void decode_k_last_packed(const at::Tensor& mixed_qkv, const at::Tensor& a, const at::Tensor& b,
                          const at::Tensor& A_log, const at::Tensor& dt_bias, double softplus_beta,
                          double softplus_threshold, double scale, const at::Tensor& state,
                          const at::Tensor& state_indices, at::Tensor out, bool use_qk_l2norm,
                          const std::optional<at::Tensor>& cu_seqlens, bool is_kda, bool is_sglang,
                          const std::optional<at::Tensor>& status, int64_t rows_per_cta) {
  check_cuda(mixed_qkv, "mixed_qkv");
  TORCH_CHECK(mixed_qkv.dim() == 2 && mixed_qkv.stride(1) == 1, "mixed_qkv must be [tokens, width] with contiguous rows");
  TORCH_CHECK(out.dim() == 4 && out.size(1) == 1 && out.size(3) == 128 && out.is_contiguous(),
              "out must be contiguous [tokens, 1, HV, 128]");
  const int64_t tokens = mixed_qkv.size(0), HV = out.size(2);
  const int64_t qk_width = mixed_qkv.size(1) - HV * 128;
  TORCH_CHECK(out.size(0) == tokens, "out and mixed_qkv token counts must match");
  TORCH_CHECK(qk_width > 0 && qk_width % 256 == 0, "mixed_qkv width must be 2*H*128 + HV*128");
  const int64_t H = qk_width / 256;
  TORCH_CHECK(HV % H == 0, "HV must be a positive multiple of H, got H=", H, ", HV=", HV);
  TORCH_CHECK(mixed_qkv.scalar_type() == at::kBFloat16 || mixed_qkv.scalar_type() == at::kHalf,
              "mixed_qkv must be fp16 or bf16");
  TORCH_CHECK(a.scalar_type() == mixed_qkv.scalar_type() && out.scalar_type() == mixed_qkv.scalar_type(),
              "mixed_qkv, a, b and out must share the activation dtype");
  TORCH_CHECK(dt_bias.scalar_type() == mixed_qkv.scalar_type(), "dt_bias dtype must match mixed_qkv");
  TORCH_CHECK(a.dim() >= 2 && a.stride(-1) == 1, "a must have contiguous rows");
  c10::cuda::CUDAGuard guard(mixed_qkv.device());

  pla_b200_klast_args g{};
  fill_common(g, A_log, a, dt_bias, b, HV, is_kda);
  const int64_t a_cols = a.numel() / std::max<int64_t>(tokens, 1);
  TORCH_CHECK(a_cols == (is_kda ? HV * 128 : HV), "a head dimensions must match HV and the gate type");
  g.a_tok_stride = (is_kda && a.dim() == 3) ? a.stride(0) : a.stride(a.dim() - 2);
  const auto esz = mixed_qkv.element_size();
  char* base = static_cast<char*>(mixed_qkv.data_ptr());
  g.q = base;
  g.k = base + H * 128 * esz;
  g.v = base + 2 * H * 128 * esz;
  g.q_tok_stride = g.k_tok_stride = g.v_tok_stride = mixed_qkv.stride(0);
  g.act_dtype = dtype_tag(mixed_qkv, "mixed_qkv");
  const StateView sv = state_view(state, HV, "initial_state_source");
  TORCH_CHECK((sv.slot_stride * state.element_size()) % 16 == 0, "state slot pitch must be 16-byte aligned");
  g.state = sv.ptr;
  g.state_slot_stride = sv.slot_stride;
  g.num_slots = sv.slots;
  g.state_dtype = sv.dtype;
  TORCH_CHECK(state_indices.scalar_type() == at::kInt && state_indices.dim() == 1 && state_indices.is_contiguous(),
              "initial_state_indices must be contiguous int32 [N]");
  g.slot_indices = state_indices.data_ptr<int32_t>();
  g.cu_seqlens = i32_ptr(cu_seqlens, "cu_seqlens");
  const int64_t B = cu_seqlens.has_value() ? cu_seqlens->size(0) - 1 : tokens;
  TORCH_CHECK(state_indices.size(0) >= B, "initial_state_indices needs one entry per request");
  g.o = out.data_ptr();
  g.B = static_cast<int32_t>(B);
  g.t_max = 1;
  g.H = static_cast<int32_t>(H);
  g.HV = static_cast<int32_t>(HV);
  g.scale = static_cast<float>(scale);
  g.softplus_beta = static_cast<float>(softplus_beta);
  g.softplus_threshold = static_cast<float>(softplus_threshold);
  g.gate = PLA_B200_GATE_SOFTPLUS;
  g.is_kda = is_kda;
  g.use_qk_l2norm = use_qk_l2norm;
  g.pad = is_sglang ? PLA_B200_PAD_SGLANG : PLA_B200_PAD_VLLM;
  g.rows_per_cta = static_cast<int32_t>(rows_per_cta);
  g.status = status.has_value() ? const_cast<int32_t*>(i32_ptr(status, "status")) : nullptr;
  if (!bypass_exec()) check_abi(pla_b200_decode_klast(&g, stream_of(mixed_qkv)), "fused_sigmoid_gating_delta_rule_forward_k_last_packed");
}

void decode_v_last(const at::Tensor& A_log, const at::Tensor& a, const at::Tensor& dt_bias, double softplus_beta,
                   double softplus_threshold, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                   const at::Tensor& b, const std::optional<at::Tensor>& h0_source, at::Tensor o,
                   const std::optional<at::Tensor>& h0_indices, const std::optional<at::Tensor>& cu_seqlens,
                   double scale, int64_t T, int64_t B, int64_t H, int64_t HV, int64_t K, int64_t V,
                   bool use_initial_state, bool use_qk_l2norm, bool is_varlen,
                   const std::optional<at::Tensor>& status) {
  check_cuda(q, "q");
  TORCH_CHECK(use_initial_state && h0_source.has_value() && h0_indices.has_value(),
              "use_initial_state=True with h0_source and h0_indices is required");
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 || q.scalar_type() == at::kHalf, "q must be fp16 or bf16");
  for (const at::Tensor* t : std::initializer_list<const at::Tensor*>{&k, &v, &a, &b, &dt_bias, &o})
    TORCH_CHECK(t->scalar_type() == q.scalar_type(), "q, k, v, a, b, dt_bias and o must share fp16 or bf16");
  for (const at::Tensor* t : std::initializer_list<const at::Tensor*>{&q, &k, &v, &a, &b, &dt_bias, &o, &A_log})
    TORCH_CHECK(t->is_contiguous(), "v-last decode inputs must be contiguous");
  TORCH_CHECK(h0_source->scalar_type() == at::kFloat, "h0_source must be float32");
  TORCH_CHECK(h0_source->is_contiguous(), "h0_source must be contiguous");
  TORCH_CHECK(K == 128 && V == 128, "v-last decode requires K == V == 128, got K=", K, ", V=", V);
  TORCH_CHECK(H > 0 && HV % H == 0, "HV must be a positive multiple of H, got H=", H, ", HV=", HV);
  TORCH_CHECK(H == 1 || H == 2 || H == 4 || H == 8 || H == 16 || H == 32, "H must be one of {1,2,4,8,16,32}");
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "q, k, v must have shape [batch, tokens, heads, dim]");
  TORCH_CHECK(q.size(2) == H && k.size(2) == H && v.size(2) == HV && q.size(3) == K && v.size(3) == V,
              "H/HV/K/V must match the tensor shapes");
  const int64_t tokens = q.size(0) * q.size(1);
  if (is_varlen) {
    TORCH_CHECK(cu_seqlens.has_value() && cu_seqlens->scalar_type() == at::kInt && cu_seqlens->is_contiguous() &&
                    cu_seqlens->numel() == B + 1,
                "varlen mode requires contiguous int32 cu_seqlens [B+1]");
  } else {
    TORCH_CHECK(T == 1, "fixed-length decode requires T == 1");
    TORCH_CHECK(tokens == B, "B must match the token count");
  }
  TORCH_CHECK(h0_source->dim() == 4 && h0_source->size(1) == HV && h0_source->size(2) == K && h0_source->size(3) == V,
              "h0_source must be [slots, HV, K, V]");
  TORCH_CHECK(h0_indices->scalar_type() == at::kInt && h0_indices->numel() >= B && h0_indices->is_contiguous(),
              "h0_indices must be contiguous int32 with at least B entries");
  TORCH_CHECK(A_log.numel() == HV && dt_bias.numel() == HV, "A_log/dt_bias must have HV elements");
  TORCH_CHECK(a.numel() == tokens * HV && b.numel() == tokens * HV, "a and b must be [tokens, HV]");
  TORCH_CHECK(o.numel() == tokens * HV * V, "o must match v's shape");
  c10::cuda::CUDAGuard guard(q.device());

  pla_b200_vlast_args g{};
  g.q = q.data_ptr();
  g.k = k.data_ptr();
  g.v = v.data_ptr();
  g.a = a.data_ptr();
  g.b = b.data_ptr();
  g.o = o.data_ptr();
  g.A_log = A_log.data_ptr();
  g.dt_bias = dt_bias.data_ptr();
  g.act_dtype = dtype_tag(q, "q");
  g.A_log_dtype = dtype_tag(A_log, "A_log");
  g.state = h0_source->data_ptr<float>();
  g.num_slots = h0_source->size(0);
  g.slot_indices = h0_indices->data_ptr<int32_t>();
  g.cu_seqlens = is_varlen ? cu_seqlens->data_ptr<int32_t>() : nullptr;
  g.B = static_cast<int32_t>(B);
  g.H = static_cast<int32_t>(H);
  g.HV = static_cast<int32_t>(HV);
  g.scale = static_cast<float>(scale);
  g.softplus_beta = static_cast<float>(softplus_beta);
  g.softplus_threshold = static_cast<float>(softplus_threshold);
  g.use_qk_l2norm = use_qk_l2norm;
  g.status = status.has_value() ? const_cast<int32_t*>(i32_ptr(status, "status")) : nullptr;
  if (!bypass_exec()) check_abi(pla_b200_decode_vlast(&g, stream_of(q)), "fused_sigmoid_gating_delta_rule_forward (v-last)");
}

// vLLM-signature KDA adapter (src/decode/k-last/fused_recurrent_kda.cpp:146-314): flattens the raw
// gate to [T, H*128], casts gate inputs to the activation dtype and index vectors to int32, narrows
// the fp32 dt_bias to the activation dtype only when the call takes the plain decode path, and runs
// the k-last op with is_kda. A 2-D slot table (one slot per draft token) means the per-step states
// are the commit, so the start slot is not written again.
void fused_recurrent_kda(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& raw_g,
                         const at::Tensor& raw_beta, const at::Tensor& A_log, const at::Tensor& dt_bias,
                         std::optional<double> lower_bound, const at::Tensor& initial_state,
                         const at::Tensor& cu_seqlens, const at::Tensor& ssm_state_indices,
                         const std::optional<at::Tensor>& num_accepted_tokens, at::Tensor out, bool is_sglang,
                         const std::optional<at::Tensor>& status) {
  TORCH_CHECK(q.dim() == 4 && q.size(0) == 1, "q must be packed as [1, T, H, K]");
  const int64_t T = q.size(1), H = q.size(2), K = q.size(3);
  const auto act = q.scalar_type();
  const bool per_token_slots = ssm_state_indices.dim() == 2;
  at::Tensor a = raw_g.reshape({T, H * K}).to(act).contiguous();
  at::Tensor b = raw_beta.reshape({T, H}).to(act).contiguous();
  at::Tensor cu32 = cu_seqlens.to(at::kInt).contiguous();
  at::Tensor slots = ssm_state_indices.to(at::kInt).contiguous();
  const int64_t B = cu32.numel() - 1;
  TORCH_CHECK(B > 0, "k-last requires at least one sequence");
  // the plain decode path (one token per request, 1-D slots) reads dt_bias at the activation dtype
  const bool mtp = per_token_slots || T != B;
  at::Tensor bias = dt_bias.reshape({H, K});
  if (!mtp) bias = bias.to(act);
  bias = bias.contiguous();
  std::optional<at::Tensor> accepted;
  if (num_accepted_tokens.has_value()) accepted = num_accepted_tokens->to(at::kInt).contiguous();
  at::Tensor o = out.is_contiguous() ? out : at::empty(v.sizes(), v.options());
  decode_k_last(A_log.reshape({-1}).contiguous(), a, bias, 1.0, 20.0, q.contiguous(), k.contiguous(), v.contiguous(), b,
                initial_state, slots, std::pow(static_cast<double>(K), -0.5), true, cu32, true, per_token_slots,
                std::nullopt, std::nullopt, std::nullopt, accepted, std::nullopt, lower_bound, is_sglang, o, status, 0);
  if (!out.is_contiguous()) out.copy_(o);
}

// Fused KDA decode step; tensor contract of fused_kda_decode_mega_forward
// (src/decode/k-last/fused_sigmoid_gating.cpp:136-144, docs/readme.md:232-267). Writes conv_state, state and
// out in place; one kernel, no scratch.
void kda_decode_mega(const at::Tensor& x, const at::Tensor& weight, const std::optional<at::Tensor>& bias,
                     at::Tensor conv_state, const at::Tensor& raw_g, const at::Tensor& raw_beta,
                     const at::Tensor& a_log, const at::Tensor& dt_bias, const at::Tensor& state_indices,
                     at::Tensor state, at::Tensor out, std::optional<double> lower_bound,
                     const std::optional<at::Tensor>& output_gate, const std::optional<at::Tensor>& norm_weight,
                     double norm_eps, const std::optional<at::Tensor>& status) {
  check_cuda(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.size(1) % (3 * 128) == 0 && x.stride(1) == 1,
              "x must be [B, 3*H*128] with contiguous channels");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf, "x must be fp16 or bf16");
  const int64_t B = x.size(0), dim = x.size(1) / 3, H = dim / 128;
  TORCH_CHECK(weight.scalar_type() == at::kFloat && weight.is_contiguous() && weight.dim() == 3 &&
                  weight.size(0) == 3 && weight.size(1) == 4 && weight.size(2) == dim,
              "weight must be contiguous fp32 [3, 4, H*128]");
  if (bias.has_value())
    TORCH_CHECK(bias->scalar_type() == at::kFloat && bias->is_contiguous() && bias->numel() == 3 * dim,
                "bias must be contiguous fp32 [3*H*128]");
  TORCH_CHECK(conv_state.scalar_type() == x.scalar_type() && conv_state.dim() == 3 && conv_state.size(1) == 3 * dim &&
                  conv_state.size(2) == 3,
              "conv_state must be [slots, 3*H*128, 3] in the activation dtype");
  TORCH_CHECK(raw_g.scalar_type() == x.scalar_type() && raw_g.is_contiguous() && raw_g.numel() == B * dim,
              "raw_g must be contiguous [1, B, H, 128] in the activation dtype");
  TORCH_CHECK(raw_beta.scalar_type() == x.scalar_type() && raw_beta.numel() == B * H && raw_beta.dim() == 3 &&
                  raw_beta.size(0) == 1 && raw_beta.stride(2) == 1,
              "raw_beta must be [1, B, H] with contiguous heads in the activation dtype");
  TORCH_CHECK(a_log.scalar_type() == at::kFloat && a_log.is_contiguous() && a_log.numel() == H,
              "a_log must be contiguous fp32 [H]");
  TORCH_CHECK(dt_bias.scalar_type() == at::kFloat && dt_bias.is_contiguous() && dt_bias.numel() == dim,
              "dt_bias must be contiguous fp32 [H, 128]");
  TORCH_CHECK(state_indices.scalar_type() == at::kInt && state_indices.is_contiguous() && state_indices.numel() == B,
              "state_indices must be contiguous int32 [B]");
  TORCH_CHECK(state.scalar_type() == at::kFloat && state.dim() == 4 && state.size(1) == H && state.size(2) == 128 &&
                  state.size(3) == 128 && state.stride(3) == 1 && state.stride(2) == 128 && state.stride(1) == 16384,
              "state must be fp32 [slots, H, 128, 128] with contiguous slot contents");
  TORCH_CHECK(conv_state.size(0) == state.size(0), "conv_state and state must have the same slots");
  TORCH_CHECK(out.scalar_type() == x.scalar_type() && out.is_contiguous() && out.numel() == B * dim,
              "out must be contiguous [1, B, H, 128] in the activation dtype");
  TORCH_CHECK(output_gate.has_value() == norm_weight.has_value(), "output_gate and norm_weight are supplied together");
  for (const at::Tensor* t : std::initializer_list<const at::Tensor*>{&weight, &conv_state, &raw_g, &raw_beta, &a_log,
                                                                     &dt_bias, &state_indices, &state, &out})
    TORCH_CHECK(t->device() == x.device(), "all tensors must be on x's device");
  c10::cuda::CUDAGuard guard(x.device());

  pla_b200_kda_mega_args g{};
  g.x = x.data_ptr();
  g.x_row_stride = x.stride(0);
  g.weight = weight.data_ptr<float>();
  g.bias = bias.has_value() ? bias->data_ptr<float>() : nullptr;
  g.conv_state = conv_state.data_ptr();
  g.conv_strides = {conv_state.stride(0), conv_state.stride(1), conv_state.stride(2)};
  g.raw_g = raw_g.data_ptr();
  g.raw_beta = raw_beta.data_ptr();
  g.beta_row_stride = raw_beta.stride(1);
  g.A_log = a_log.data_ptr<float>();
  g.dt_bias = dt_bias.data_ptr<float>();
  g.state_indices = state_indices.data_ptr<int32_t>();
  g.state = state.data_ptr<float>();
  g.state_slot_stride = state.stride(0);
  g.slots = static_cast<int32_t>(state.size(0));
  g.out = out.data_ptr();
  if (output_gate.has_value()) {
    const at::Tensor& gate = *output_gate;
    TORCH_CHECK(gate.scalar_type() == x.scalar_type() && gate.numel() == B * dim && gate.stride(-1) == 1 &&
                    gate.stride(-2) == 128 && gate.device() == x.device(),
                "output_gate must be [B, H, 128] or [1, B, H, 128] in the activation dtype with contiguous heads");
    TORCH_CHECK(norm_weight->scalar_type() == at::kFloat && norm_weight->is_contiguous() && norm_weight->numel() == 128 &&
                    norm_weight->device() == x.device(),
                "norm_weight must be contiguous fp32 [128]");
    TORCH_CHECK(std::isfinite(norm_eps) && norm_eps >= 0.0, "norm_eps must be finite and non-negative");
    g.output_gate = gate.data_ptr();
    g.gate_row_stride = gate.stride(gate.dim() - 3);
    g.norm_weight = norm_weight->data_ptr<float>();
    g.norm_eps = static_cast<float>(norm_eps);
  }
  g.B = static_cast<int32_t>(B);
  g.H = static_cast<int32_t>(H);
  g.act_dtype = dtype_tag(x, "x");
  g.gate = lower_bound.has_value() ? PLA_B200_GATE_SAFE : PLA_B200_GATE_SOFTPLUS;
  g.lower_bound = static_cast<float>(lower_bound.value_or(0.0));
  g.scale = 1.0f / std::sqrt(128.0f);
  g.status = status.has_value() ? const_cast<int32_t*>(i32_ptr(status, "status")) : nullptr;
  if (!bypass_exec()) check_abi(pla_b200_kda_decode_mega(&g, stream_of(x)), "fused_kda_decode_mega_forward");
}

}  // namespace
}  // namespace pla_ops

TORCH_LIBRARY_FRAGMENT(pla_b200, m) {
  m.def(
      "kda_decode_mega(Tensor x, Tensor weight, Tensor? bias, Tensor(a!) conv_state, Tensor raw_g, Tensor raw_beta, "
      "Tensor a_log, Tensor dt_bias, Tensor state_indices, Tensor(b!) state, Tensor(c!) out, float? lower_bound, "
      "Tensor? output_gate, Tensor? norm_weight, float norm_eps, Tensor(d!)? status) -> ()",
      &pla_ops::kda_decode_mega);
  m.def(
      "fused_recurrent_kda(Tensor q, Tensor k, Tensor v, Tensor raw_g, Tensor raw_beta, Tensor A_log, Tensor dt_bias, "
      "float? lower_bound, Tensor(a!) initial_state, Tensor cu_seqlens, Tensor ssm_state_indices, "
      "Tensor? num_accepted_tokens, Tensor(b!) out, bool is_sglang, Tensor(c!)? status) -> ()",
      &pla_ops::fused_recurrent_kda);
  m.def(
      "decode_k_last(Tensor A_log, Tensor a, Tensor dt_bias, float softplus_beta, float softplus_threshold, "
      "Tensor q, Tensor k, Tensor v, Tensor b, Tensor(a!) initial_state_source, Tensor initial_state_indices, "
      "float scale, bool use_qk_l2norm_in_kernel, Tensor? cu_seqlens, bool is_kda, bool disable_state_update, "
      "Tensor(b!)? intermediate_states_buffer, Tensor? intermediate_state_indices, int? cache_steps, "
      "Tensor? num_accepted, Tensor? retrieve_parent_token, float? lower_bound, bool is_sglang, Tensor(c!) out, "
      "Tensor(d!)? status, int rows_per_cta) -> ()",
      &pla_ops::decode_k_last);
  m.def(
      "decode_k_last_packed(Tensor mixed_qkv, Tensor a, Tensor b, Tensor A_log, Tensor dt_bias, float softplus_beta, "
      "float softplus_threshold, float scale, Tensor(a!) initial_state_source, Tensor initial_state_indices, "
      "Tensor(b!) out, bool use_qk_l2norm_in_kernel, Tensor? cu_seqlens, bool is_kda, bool is_sglang, "
      "Tensor(c!)? status, int rows_per_cta) -> ()",
      &pla_ops::decode_k_last_packed);
  m.def(
      "decode_v_last(Tensor A_log, Tensor a, Tensor dt_bias, float softplus_beta, float softplus_threshold, "
      "Tensor q, Tensor k, Tensor v, Tensor b, Tensor(a!)? h0_source, Tensor(b!) o, Tensor? h0_indices, "
      "Tensor? cu_seqlens, float scale, int T, int B, int H, int HV, int K, int V, bool use_initial_state, "
      "bool use_qk_l2norm_in_kernel, bool is_varlen, Tensor(c!)? status) -> ()",
      &pla_ops::decode_v_last);
}
