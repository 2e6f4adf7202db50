// Host layer of the prefill ops: tensor contracts of
//   pla.prefill.flashqla.chunk_gated_delta_rule_fwd / gdn_prefill_packed_qkv_fwd (pla/prefill/flashqla/ops.py:225-738)
//   pla.prefill.flashkdapro.flashkda_fwd                                          (pla/prefill/flashkdapro/ops.py:66-219)
// mapped onto the chunked (tensor-core) and token-recurrent prefill entries of the C ABI, plus the staged /
// prescan forms used by context parallelism. No sync, no D2H.
#include "ops_common.h"

namespace pla_ops {
namespace {

using Optional = std::optional<at::Tensor>;

void rows_ok(const at::Tensor& t, int64_t heads, const char* name) {
  TORCH_CHECK(t.dim() == 3 && t.size(1) == heads && t.size(2) == 128, name, " must be [tokens, heads, 128]");
  TORCH_CHECK(t.stride(2) == 1 && t.stride(1) == 128, name, ": features inside one token must be contiguous");
}

void state_ok(const at::Tensor& t, int64_t H, const at::Tensor& ref, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.device() == ref.device(), name, " must be on q's device");
  TORCH_CHECK(t.scalar_type() == at::kFloat || t.scalar_type() == at::kBFloat16, name, " must be fp32 or bf16");
  TORCH_CHECK(t.dim() == 4 && t.size(1) == H && t.size(2) == 128 && t.size(3) == 128, name,
              " must be [slots, H, 128, 128]");
  TORCH_CHECK(t.stride(3) == 1 && t.stride(2) == 128 && t.stride(1) == 128 * 128 && t.stride(0) >= H * 16384, name,
              ": the [H,128,128] block of a slot must be contiguous");
}

void run_recurrent(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& gate,
                   const at::Tensor& beta, const Optional& A_log, const Optional& dt_bias, at::Tensor out,
                   const at::Tensor& cu_seqlens, const Optional& state_in, const Optional& in_indices,
                   const Optional& state_out, const Optional& out_indices, bool transposed, bool is_kda,
                   bool normalize_qk, double scale, std::optional<double> lower_bound, bool gate_activated,
                   bool update_in_place, const Optional& status, const Optional& prescan_out) {
  check_cuda(q, "q");
  const int64_t T = q.size(0);
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3, "q, k, v must be [tokens, heads, 128]");
  const int64_t Hg = k.size(1), H = v.size(1);
  rows_ok(q, Hg, "q");
  rows_ok(k, Hg, "k");
  rows_ok(v, H, "v");
  TORCH_CHECK(Hg > 0 && H % Hg == 0, "the value-head count must be a multiple of the q/k head count");
  TORCH_CHECK(k.size(0) == T && v.size(0) == T, "q, k, v token counts must match");
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 || q.scalar_type() == at::kHalf, "q must be fp16 or bf16");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type() &&
                  out.scalar_type() == q.scalar_type(),
              "q, k, v and out must share a dtype");
  TORCH_CHECK(out.is_contiguous() && out.numel() == T * H * 128, "out must be contiguous [tokens, H, 128]");
  TORCH_CHECK(cu_seqlens.scalar_type() == at::kInt && cu_seqlens.dim() == 1 && cu_seqlens.is_contiguous() &&
                  cu_seqlens.numel() >= 2 && cu_seqlens.device() == q.device(),
              "cu_seqlens must be contiguous int32 [batch+1] on q's device");
  const int64_t N = cu_seqlens.numel() - 1;
  c10::cuda::CUDAGuard guard(q.device());

  pla_b200_klast_args g{};
  g.q = q.data_ptr();
  g.k = k.data_ptr();
  g.v = v.data_ptr();
  g.o = out.data_ptr();
  g.q_tok_stride = q.stride(0);
  g.k_tok_stride = k.stride(0);
  g.v_tok_stride = v.stride(0);
  g.act_dtype = dtype_tag(q, "q");
  const int64_t gate_w = is_kda ? H * 128 : H;
  TORCH_CHECK(gate.size(0) == T && gate.numel() == T * gate_w && gate.stride(-1) == 1,
              "gate must be [tokens, H] (GDN) or [tokens, H, 128] (KDA) with contiguous rows");
  if (gate.dim() == 3) TORCH_CHECK(gate.stride(1) == 128, "KDA gate heads must be contiguous");
  TORCH_CHECK(beta.dim() == 2 && beta.size(0) == T && beta.size(1) == H && beta.stride(1) == 1,
              "beta must be [tokens, H] with contiguous heads");
  if (gate_activated) {
    TORCH_CHECK(gate.scalar_type() == at::kFloat && beta.scalar_type() == at::kFloat,
                "activated gates (log-decay g, beta) must be fp32");
  } else {
    TORCH_CHECK(gate.scalar_type() == q.scalar_type() && beta.scalar_type() == q.scalar_type(),
                "raw gate inputs must share q's dtype");
    TORCH_CHECK(A_log.has_value() && dt_bias.has_value(), "raw gating needs A_log and dt_bias");
    TORCH_CHECK(A_log->scalar_type() == at::kFloat && dt_bias->scalar_type() == at::kFloat && A_log->is_contiguous() &&
                    dt_bias->is_contiguous() && A_log->numel() == H && dt_bias->numel() == gate_w,
                "A_log [H] and dt_bias must be contiguous fp32");
    g.A_log = A_log->data_ptr();
    g.dt_bias = dt_bias->data_ptr();
  }
  if (gate_activated) {  // never read, but the entry insists on non-NULL pointers
    g.A_log = gate.data_ptr();
    g.dt_bias = gate.data_ptr();
  }
  g.A_log_dtype = PLA_B200_F32;
  g.dt_bias_dtype = PLA_B200_F32;
  g.a = gate.data_ptr();
  g.b = beta.data_ptr();
  g.a_tok_stride = gate.stride(0);
  g.b_tok_stride = beta.stride(0);
  g.gate_activated = gate_activated;

  g.state_dtype = PLA_B200_F32;
  if (state_in.has_value()) {
    state_ok(*state_in, H, q, "initial state");
    g.state = state_in->data_ptr();
    g.state_slot_stride = state_in->stride(0);
    g.num_slots = state_in->size(0);
    g.state_dtype = dtype_tag(*state_in, "initial state");
  } else {
    g.state_init_zero = 1;
  }
  if (in_indices.has_value()) {
    TORCH_CHECK(state_in.has_value(), "state indices need a state");
    TORCH_CHECK(in_indices->scalar_type() == at::kInt && in_indices->is_contiguous() && in_indices->dim() == 1 &&
                    in_indices->numel() == N && in_indices->device() == q.device(),
                "state indices must be contiguous int32 [batch] on q's device");
    g.slot_indices = in_indices->data_ptr<int32_t>();
  } else {
    g.state_by_request = 1;
    if (state_in.has_value()) TORCH_CHECK(state_in->size(0) >= N, "the initial state needs one slot per sequence");
  }
  if (state_out.has_value()) {
    state_ok(*state_out, H, q, "final state");
    if (state_in.has_value())
      TORCH_CHECK(state_out->scalar_type() == state_in->scalar_type(), "initial and final state dtypes must match");
    g.state_out = state_out->data_ptr();
    g.state_out_slot_stride = state_out->stride(0);
    g.state_dtype = dtype_tag(*state_out, "final state");
    if (out_indices.has_value()) {
      TORCH_CHECK(out_indices->scalar_type() == at::kInt && out_indices->is_contiguous() && out_indices->numel() == N,
                  "final-state indices must be contiguous int32 [batch]");
      g.state_out_indices = out_indices->data_ptr<int32_t>();
    } else {
      TORCH_CHECK(state_out->size(0) >= N, "the final state needs one slot per sequence");
    }
  }
  TORCH_CHECK(!(update_in_place && state_out.has_value()), "in-place update and a separate final state are exclusive");
  TORCH_CHECK(!update_in_place || state_in.has_value(), "an in-place update needs the state pool");
  g.disable_state_update = !(state_out.has_value() || update_in_place);
  g.state_transposed = transposed;
  g.cu_seqlens = cu_seqlens.data_ptr<int32_t>();
  g.B = static_cast<int32_t>(N);
  g.t_max = static_cast<int32_t>(std::max<int64_t>(T, 2));
  g.H = static_cast<int32_t>(Hg);
  g.HV = static_cast<int32_t>(H);
  g.scale = static_cast<float>(scale);
  g.softplus_beta = 1.0f;
  g.softplus_threshold = 20.0f;
  g.lower_bound = static_cast<float>(lower_bound.value_or(0.0));
  g.gate = lower_bound.has_value() ? PLA_B200_GATE_SAFE : PLA_B200_GATE_SOFTPLUS;
  TORCH_CHECK(!lower_bound.has_value() || is_kda, "lower_bound is only supported for KDA");
  g.is_kda = is_kda;
  g.use_qk_l2norm = normalize_qk;
  g.pad = PLA_B200_PAD_SGLANG;
  g.o_total_rows = T;
  g.status = status.has_value() ? const_cast<int32_t*>(i32_ptr(status, "status")) : nullptr;
  if (prescan_out.has_value()) {
    TORCH_CHECK(prescan_out->scalar_type() == at::kFloat && prescan_out->is_contiguous() &&
                    prescan_out->numel() == N * H * 2 * 128 * 128 && prescan_out->device() == q.device(),
                "a prescan stores contiguous fp32 [batch, H, 2, 128, 128] on q's device");
    g.prescan = 1;
    g.state = nullptr;
    g.state_out = prescan_out->data_ptr();
    g.state_out_indices = nullptr;
    g.slot_indices = nullptr;
    g.state_dtype = PLA_B200_F32;
    g.state_transposed = 0;
    g.o_total_rows = 0;
  }
  if (!bypass_exec()) check_abi(pla_b200_prefill_recurrent(&g, stream_of(q)), "prefill");
}

void prefill_recurrent(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& gate,
                       const at::Tensor& beta, const Optional& A_log, const Optional& dt_bias, at::Tensor out,
                       const at::Tensor& cu_seqlens, const Optional& state_in, const Optional& in_indices,
                       const Optional& state_out, const Optional& out_indices, bool transposed, bool is_kda,
                       bool normalize_qk, double scale, std::optional<double> lower_bound, bool gate_activated,
                       bool update_in_place, const Optional& status) {
  run_recurrent(q, k, v, gate, beta, A_log, dt_bias, out, cu_seqlens, state_in, in_indices, state_out, out_indices,
                transposed, is_kda, normalize_qk, scale, lower_bound, gate_activated, update_in_place, status,
                c10::nullopt);
}

// Context-parallel prescan with the token recurrence (GDN or KDA): per (sequence, head) the offset B and
// the transition M of the token range, stored to `pairs` [batch, H, 2, 128, 128] fp32; no output rows.
void prefill_recurrent_prescan(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& gate,
                               const at::Tensor& beta, const Optional& A_log, const Optional& dt_bias,
                               const at::Tensor& cu_seqlens, at::Tensor pairs, bool is_kda, bool normalize_qk,
                               double scale, std::optional<double> lower_bound, bool gate_activated,
                               const Optional& status) {
  at::Tensor no_out = at::empty({v.size(0), v.size(1), 128}, v.options().dtype(q.scalar_type()).memory_format(at::MemoryFormat::Contiguous));
  run_recurrent(q, k, v, gate, beta, A_log, dt_bias, no_out, cu_seqlens, c10::nullopt, c10::nullopt, c10::nullopt,
                c10::nullopt, false, is_kda, normalize_qk, scale, lower_bound, gate_activated, false, status, pairs);
}

// Chunked (chunk 64) GDN prefill on the tensor cores. Returns the scratch workspace it allocated
// from the caching allocator (callers normally drop it; tests inspect the operand images).
at::Tensor run_chunked(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& gate,
                       const at::Tensor& beta, const Optional& A_log, const Optional& dt_bias, at::Tensor out,
                       const Optional& g_cum, const at::Tensor& cu_seqlens, const Optional& state_in,
                       const Optional& in_indices, const Optional& state_out, const Optional& out_indices,
                       bool transposed, bool normalize_qk, double scale, bool gate_activated, bool update_in_place,
                       int64_t max_chunks, int64_t stage, const Optional& status, const Optional& workspace_in,
                       bool prescan, bool is_kda = false, std::optional<double> lower_bound = std::nullopt,
                       const Optional& range_mask = std::nullopt) {
  check_cuda(q, "q");
  const int64_t T = q.size(0);
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3, "q, k, v must be [tokens, heads, 128]");
  const int64_t Hg = k.size(1), H = v.size(1);
  rows_ok(q, Hg, "q");
  rows_ok(k, Hg, "k");
  rows_ok(v, H, "v");
  TORCH_CHECK(Hg > 0 && H % Hg == 0, "the value-head count must be a multiple of the q/k head count");
  TORCH_CHECK(k.size(0) == T && v.size(0) == T, "q, k, v token counts must match");
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 || q.scalar_type() == at::kHalf, "q must be fp16 or bf16");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type() &&
                  out.scalar_type() == q.scalar_type(),
              "q, k, v and out must share a dtype");
  TORCH_CHECK(out.is_contiguous() && out.numel() == T * H * 128, "out must be contiguous [tokens, H, 128]");
  TORCH_CHECK(cu_seqlens.scalar_type() == at::kInt && cu_seqlens.dim() == 1 && cu_seqlens.is_contiguous() &&
                  cu_seqlens.numel() >= 2 && cu_seqlens.device() == q.device(),
              "cu_seqlens must be contiguous int32 [batch+1] on q's device");
  const int64_t N = cu_seqlens.numel() - 1;
  TORCH_CHECK(max_chunks >= 0 && max_chunks <= T / 64 + N, "max_chunks out of range");
  if (sanity_check()) {
    std::string bad = sanity_offsets(cu_seqlens, T, 0);
    if (bad.empty() && in_indices.has_value() && state_in.has_value()) bad = sanity_slots(*in_indices, state_in->size(0));
    TORCH_CHECK(bad.empty(), "chunked prefill: sanity check: ", bad);
  }
  c10::cuda::CUDAGuard guard(q.device());

  pla_b200_gdn_chunk_args g{};
  g.q = q.data_ptr();
  g.k = k.data_ptr();
  g.v = v.data_ptr();
  g.o = out.data_ptr();
  g.q_tok_stride = q.stride(0);
  g.k_tok_stride = k.stride(0);
  g.v_tok_stride = v.stride(0);
  g.act_dtype = dtype_tag(q, "q");
  if (is_kda) {
    TORCH_CHECK(Hg == H, "KDA prefill needs as many q/k heads as value heads");
    TORCH_CHECK(!gate_activated, "chunked KDA prefill takes the raw gate input");
    TORCH_CHECK(gate.size(0) == T && gate.numel() == T * H * 128 && gate.stride(-1) == 1 &&
                    (gate.dim() == 2 || (gate.dim() == 3 && gate.stride(1) == 128)),
                "the KDA gate must be [tokens, H, 128] or [tokens, H*128] with contiguous rows");
  } else {
    TORCH_CHECK(gate.dim() == 2 && gate.size(0) == T && gate.size(1) == H && gate.stride(1) == 1,
                "gate must be [tokens, H] with contiguous heads");
  }
  TORCH_CHECK(beta.dim() == 2 && beta.size(0) == T && beta.size(1) == H && beta.stride(1) == 1,
              "beta must be [tokens, H] with contiguous heads");
  if (gate_activated) {
    TORCH_CHECK(gate.scalar_type() == at::kFloat && beta.scalar_type() == at::kFloat,
                "activated gates (log-decay g, beta) must be fp32");
  } else {
    TORCH_CHECK(gate.scalar_type() == q.scalar_type() && beta.scalar_type() == q.scalar_type(),
                "raw gate inputs must share q's dtype");
    TORCH_CHECK(A_log.has_value() && dt_bias.has_value(), "raw gating needs A_log and dt_bias");
    TORCH_CHECK(A_log->scalar_type() == at::kFloat && dt_bias->scalar_type() == at::kFloat && A_log->is_contiguous() &&
                    dt_bias->is_contiguous() && A_log->numel() == H && dt_bias->numel() == (is_kda ? H * 128 : H),
                "A_log [H] and dt_bias [H] (KDA: [H, 128]) must be contiguous fp32");
    g.A_log = A_log->data_ptr<float>();
    g.dt_bias = dt_bias->data_ptr<float>();
  }
  g.gate = gate.data_ptr();
  g.beta = beta.data_ptr();
  g.gate_tok_stride = gate.stride(0);
  g.beta_tok_stride = beta.stride(0);
  g.gate_activated = gate_activated;
  if (g_cum.has_value()) {
    TORCH_CHECK(g_cum->scalar_type() == at::kFloat && g_cum->is_contiguous() && g_cum->numel() == T * H,
                "g_cum must be contiguous fp32 [tokens, H]");
    g.g_cum = g_cum->data_ptr<float>();
  }
  g.state_dtype = PLA_B200_F32;
  if (state_in.has_value()) {
    state_ok(*state_in, H, q, "initial state");
    g.state = state_in->data_ptr();
    g.state_slot_stride = state_in->stride(0);
    g.num_slots = state_in->size(0);
    g.state_dtype = dtype_tag(*state_in, "initial state");
  } else {
    g.state_init_zero = 1;
  }
  if (in_indices.has_value()) {
    TORCH_CHECK(state_in.has_value(), "state indices need a state");
    TORCH_CHECK(in_indices->scalar_type() == at::kInt && in_indices->is_contiguous() && in_indices->dim() == 1 &&
                    in_indices->numel() == N && in_indices->device() == q.device(),
                "state indices must be contiguous int32 [batch] on q's device");
    g.slot_indices = in_indices->data_ptr<int32_t>();
  } else {
    g.state_by_request = 1;
    if (state_in.has_value()) TORCH_CHECK(state_in->size(0) >= N, "the initial state needs one slot per sequence");
  }
  if (prescan) {
    TORCH_CHECK(state_out.has_value() && state_out->scalar_type() == at::kFloat && state_out->is_contiguous() &&
                    state_out->numel() == N * H * 2 * 128 * 128 && state_out->device() == q.device(),
                "a prescan stores contiguous fp32 [batch, H, 2, 128, 128] on q's device");
    g.state_out = state_out->data_ptr();
    g.prescan = 1;
    if (range_mask.has_value()) {   // ranges with a negative entry are skipped by the prescan
      TORCH_CHECK(range_mask->scalar_type() == at::kInt && range_mask->is_contiguous() && range_mask->numel() == N &&
                      range_mask->device() == q.device(),
                  "the range mask must be contiguous int32 [batch] on q's device");
      g.slot_indices = range_mask->data_ptr<int32_t>();
    }
  } else if (state_out.has_value()) {
    state_ok(*state_out, H, q, "final state");
    if (state_in.has_value())
      TORCH_CHECK(state_out->scalar_type() == state_in->scalar_type(), "initial and final state dtypes must match");
    g.state_out = state_out->data_ptr();
    g.state_out_slot_stride = state_out->stride(0);
    g.state_dtype = dtype_tag(*state_out, "final state");
    if (out_indices.has_value()) {
      TORCH_CHECK(out_indices->scalar_type() == at::kInt && out_indices->is_contiguous() && out_indices->numel() == N,
                  "final-state indices must be contiguous int32 [batch]");
      g.state_out_indices = out_indices->data_ptr<int32_t>();
    } else {
      TORCH_CHECK(state_out->size(0) >= N, "the final state needs one slot per sequence");
    }
  }
  TORCH_CHECK(!(update_in_place && state_out.has_value()), "in-place update and a separate final state are exclusive");
  TORCH_CHECK(!update_in_place || state_in.has_value(), "an in-place update needs the state pool");
  g.write_state = state_out.has_value() || update_in_place;
  g.state_transposed = transposed;
  g.cu_seqlens = cu_seqlens.data_ptr<int32_t>();
  g.N = static_cast<int32_t>(N);
  g.T_total = T;
  g.max_chunks = static_cast<int32_t>(max_chunks);
  g.H = static_cast<int32_t>(Hg);
  g.HV = static_cast<int32_t>(H);
  g.scale = static_cast<float>(scale);
  g.normalize_qk = normalize_qk;
  g.stage = static_cast<int32_t>(stage);
  g.gate_kind = lower_bound.has_value() ? PLA_B200_GATE_SAFE : PLA_B200_GATE_SOFTPLUS;
  g.lower_bound = static_cast<float>(lower_bound.value_or(0.0));
  TORCH_CHECK(is_kda || !lower_bound.has_value(), "lower_bound is only supported for KDA");
  const int64_t bytes = is_kda ? pla_b200_kda_chunk_workspace_bytes(g.max_chunks, g.H)
                               : pla_b200_gdn_chunk_workspace_bytes(g.max_chunks, g.H, g.HV);
  at::Tensor workspace;
  if (workspace_in.has_value()) {
    workspace = *workspace_in;
    TORCH_CHECK(workspace.scalar_type() == at::kByte && workspace.is_contiguous() && workspace.numel() >= bytes &&
                    workspace.device() == q.device(),
                "the workspace must be contiguous uint8 of at least ", bytes, " bytes on q's device");
  } else {
    TORCH_CHECK(stage != 2, "stage 2 runs over the workspace of a stage-1 call");
    workspace = at::empty({std::max<int64_t>(bytes, 16)}, q.options().dtype(at::kByte));
  }
  g.workspace = workspace.data_ptr();
  g.workspace_bytes = bytes;
  g.status = status.has_value() ? const_cast<int32_t*>(i32_ptr(status, "status")) : nullptr;
  if (!bypass_exec()) check_abi(is_kda ? pla_b200_kda_prefill_chunked(&g, stream_of(q)) : pla_b200_gdn_prefill_chunked(&g, stream_of(q)),
            is_kda ? "kda chunked prefill" : "gdn chunked prefill");
  return workspace;
}

at::Tensor gdn_prefill_chunked(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& gate,
                               const at::Tensor& beta, const Optional& A_log, const Optional& dt_bias, at::Tensor out,
                               const Optional& g_cum, const at::Tensor& cu_seqlens, const Optional& state_in,
                               const Optional& in_indices, const Optional& state_out, const Optional& out_indices,
                               bool transposed, bool normalize_qk, double scale, bool gate_activated,
                               bool update_in_place, int64_t max_chunks, int64_t stage, const Optional& status) {
  return run_chunked(q, k, v, gate, beta, A_log, dt_bias, out, g_cum, cu_seqlens, state_in, in_indices, state_out,
                     out_indices, transposed, normalize_qk, scale, gate_activated, update_in_place, max_chunks, stage,
                     status, c10::nullopt, false);
}

// The same kernels, one stage at a time, for context parallelism: stage 1 fills `workspace` (or a
// fresh one) from the rank's tokens; stage 2 with prescan stores each (sequence, head)'s offset and
// transition into `state_out` [batch, H, 2, 128, 128]; stage 2 without prescan is the ordinary
// chain from `state_in`. Returns the workspace.
at::Tensor gdn_prefill_chunked_stage(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                     const at::Tensor& gate, const at::Tensor& beta, const Optional& A_log,
                                     const Optional& dt_bias, at::Tensor out, const Optional& g_cum,
                                     const at::Tensor& cu_seqlens, const Optional& state_in, const Optional& state_out,
                                     const Optional& workspace, bool transposed, bool normalize_qk, double scale,
                                     bool gate_activated, int64_t max_chunks, int64_t stage, bool prescan,
                                     const Optional& status, const Optional& range_mask, const Optional& out_indices) {
  // `range_mask`: for a prescan, ranges with a negative entry are skipped; for the segment pass it is the slot of
  // every range inside `state_in` (a negative entry makes the range padding: zero output rows, no state touched)
  return run_chunked(q, k, v, gate, beta, A_log, dt_bias, out, g_cum, cu_seqlens, state_in,
                     prescan ? Optional() : range_mask, state_out, out_indices, transposed, normalize_qk, scale,
                     gate_activated, false, max_chunks, stage, status, workspace, prescan, false, std::nullopt,
                     prescan ? range_mask : Optional());
}

// Incoming state of every token range of every sequence from the prescan pairs (intra-GPU split).
at::Tensor cp_fold_segments(const at::Tensor& pairs, const at::Tensor& seg_first, const Optional& pool,
                            const Optional& slot_indices, const Optional& status) {
  check_cuda(pairs, "pairs");
  TORCH_CHECK(pairs.scalar_type() == at::kFloat && pairs.is_contiguous() && pairs.dim() == 5 && pairs.size(2) == 2 &&
                  pairs.size(3) == 128 && pairs.size(4) == 128,
              "pairs must be contiguous fp32 [ranges, H, 2, 128, 128]");
  const int64_t ranges = pairs.size(0), H = pairs.size(1);
  TORCH_CHECK(seg_first.scalar_type() == at::kInt && seg_first.is_contiguous() && seg_first.dim() == 1 &&
                  seg_first.numel() >= 1 && seg_first.device() == pairs.device(),
              "seg_first must be contiguous int32 [sequences + 1] on the pairs' device");
  const int64_t sequences = seg_first.numel() - 1;
  c10::cuda::CUDAGuard guard(pairs.device());
  at::Tensor out = at::empty({ranges, H, 128, 128}, pairs.options());
  pla_b200_cp_fold_segments_args f{};
  f.pairs = pairs.data_ptr<float>();
  f.seg_first = seg_first.data_ptr<int32_t>();
  if (pool.has_value()) {
    state_ok(*pool, H, pairs, "state pool");
    TORCH_CHECK(pool->scalar_type() == at::kFloat, "the intra-GPU split reads an fp32 pool");
    f.pool = pool->data_ptr<float>();
    f.pool_slot_stride = pool->stride(0);
    f.slots = static_cast<int32_t>(pool->size(0));
  }
  if (slot_indices.has_value()) {
    TORCH_CHECK(slot_indices->scalar_type() == at::kInt && slot_indices->is_contiguous() &&
                    slot_indices->numel() == sequences && slot_indices->device() == pairs.device(),
                "slot indices must be contiguous int32 [sequences] on the pairs' device");
    f.slot_indices = slot_indices->data_ptr<int32_t>();
  }
  f.state_in = out.data_ptr<float>();
  f.HV = static_cast<int32_t>(H);
  f.sequences = static_cast<int32_t>(sequences);
  f.status = status.has_value() ? const_cast<int32_t*>(i32_ptr(status, "status")) : nullptr;
  if (!bypass_exec()) check_abi(pla_b200_cp_fold_segments(&f, stream_of(pairs)), "cp fold segments");
  return out;
}

// The first `count` pairs composed into one (offset, transition) pair: [H, 2, 128, 128].
at::Tensor cp_compose_pairs(const at::Tensor& pairs, int64_t count, const Optional& status) {
  check_cuda(pairs, "pairs");
  TORCH_CHECK(pairs.scalar_type() == at::kFloat && pairs.is_contiguous() && pairs.dim() == 5 && pairs.size(2) == 2 &&
                  pairs.size(3) == 128 && pairs.size(4) == 128,
              "pairs must be contiguous fp32 [n, H, 2, 128, 128]");
  TORCH_CHECK(count >= 0 && count <= pairs.size(0), "count out of range");
  const int64_t H = pairs.size(1);
  c10::cuda::CUDAGuard guard(pairs.device());
  at::Tensor out = at::empty({H, 2, 128, 128}, pairs.options());
  pla_b200_cp_fold_args f{};
  f.pairs = pairs.data_ptr<float>();
  f.state_out = out.data_ptr<float>();
  f.HV = static_cast<int32_t>(H);
  f.rank = static_cast<int32_t>(count);
  f.world = static_cast<int32_t>(pairs.size(0));
  f.compose = 1;
  f.status = status.has_value() ? const_cast<int32_t*>(i32_ptr(status, "status")) : nullptr;
  if (!bypass_exec()) check_abi(pla_b200_cp_fold_prefix(&f, stream_of(pairs)), "cp compose");
  return out;
}

// Fold of the gathered (offset, transition) pairs of the ranks before `rank` into the state entering its range.
at::Tensor cp_fold_prefix(const at::Tensor& pairs, const Optional& initial_state, int64_t rank, const Optional& status) {
  check_cuda(pairs, "pairs");
  TORCH_CHECK(pairs.scalar_type() == at::kFloat && pairs.is_contiguous() && pairs.dim() == 5 && pairs.size(2) == 2 &&
                  pairs.size(3) == 128 && pairs.size(4) == 128,
              "pairs must be contiguous fp32 [world, H, 2, 128, 128]");
  const int64_t world = pairs.size(0), H = pairs.size(1);
  TORCH_CHECK(rank >= 0 && rank < world, "rank out of range");
  if (initial_state.has_value())
    TORCH_CHECK(initial_state->scalar_type() == at::kFloat && initial_state->is_contiguous() &&
                    initial_state->numel() == H * 128 * 128 && initial_state->device() == pairs.device(),
                "the initial state must be contiguous fp32 [H, 128, 128] on the pairs' device");
  c10::cuda::CUDAGuard guard(pairs.device());
  at::Tensor out = at::empty({H, 128, 128}, pairs.options());
  pla_b200_cp_fold_args f{};
  f.pairs = pairs.data_ptr<float>();
  f.initial_state = initial_state.has_value() ? initial_state->data_ptr<float>() : nullptr;
  f.state_out = out.data_ptr<float>();
  f.HV = static_cast<int32_t>(H);
  f.rank = static_cast<int32_t>(rank);
  f.world = static_cast<int32_t>(world);
  f.status = status.has_value() ? const_cast<int32_t*>(i32_ptr(status, "status")) : nullptr;
  if (!bypass_exec()) check_abi(pla_b200_cp_fold_prefix(&f, stream_of(pairs)), "cp fold");
  return out;
}

// Chunked KDA prefill; all the modes of the GDN ops in one signature (stage 0 = both halves with a fresh
// workspace; stage 1 / 2 and prescan for context parallelism).
at::Tensor kda_prefill_chunked(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& gate,
                               const at::Tensor& beta, const at::Tensor& A_log, const at::Tensor& dt_bias,
                               at::Tensor out, const at::Tensor& cu_seqlens, const Optional& state_in,
                               const Optional& in_indices, const Optional& state_out, const Optional& out_indices,
                               const Optional& workspace, bool transposed, bool normalize_qk, double scale,
                               std::optional<double> lower_bound, bool update_in_place, int64_t max_chunks,
                               int64_t stage, bool prescan, const Optional& status, const Optional& range_mask) {
  return run_chunked(q, k, v, gate, beta, A_log, dt_bias, out, c10::nullopt, cu_seqlens, state_in, in_indices,
                     state_out, out_indices, transposed, normalize_qk, scale, false, update_in_place, max_chunks, stage,
                     status, workspace, prescan, true, lower_bound, range_mask);
}

}  // namespace
// Width-4 causal conv (+ SiLU) over packed varlen rows with a 3-tap history per request; returns y.
at::Tensor causal_conv_prefill(const at::Tensor& x, const at::Tensor& weight, const Optional& bias, const Optional& conv_state,
                               const at::Tensor& cu_seqlens, const Optional& state_indices,
                               const Optional& has_initial_state, bool silu, bool vllm_pad, const Optional& out,
                               const Optional& status) {
  check_cuda(x, "x");
  TORCH_CHECK(x.dim() == 2 && (x.size(0) == 0 || x.stride(1) == 1), "x must be [tokens, channels] with contiguous channels");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf, "x must be bf16 or fp16");
  const int64_t T = x.size(0), C = x.size(1);
  TORCH_CHECK(C > 0 && C % 8 == 0, "the channel count must be a multiple of 8");
  TORCH_CHECK(weight.scalar_type() == at::kFloat && weight.is_contiguous() && weight.dim() == 2 && weight.size(0) == C &&
                  weight.size(1) == 4 && weight.device() == x.device(),
              "weight must be contiguous fp32 [channels, 4] on x's device");
  if (bias.has_value())
    TORCH_CHECK(bias->scalar_type() == at::kFloat && bias->is_contiguous() && bias->numel() == C && bias->device() == x.device(),
                "bias must be contiguous fp32 [channels] on x's device");
  TORCH_CHECK(cu_seqlens.scalar_type() == at::kInt && cu_seqlens.is_contiguous() && cu_seqlens.dim() == 1 &&
                  cu_seqlens.numel() >= 1 && cu_seqlens.device() == x.device(),
              "cu_seqlens must be contiguous int32 [N + 1] on x's device");
  const int64_t N = cu_seqlens.numel() - 1;
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = out.has_value() ? *out : at::empty({T, C}, x.options());
  TORCH_CHECK(y.device() == x.device() && y.scalar_type() == x.scalar_type() && y.dim() == 2 && y.size(0) == T &&
                  y.size(1) == C && (T == 0 || y.stride(1) == 1),
              "out must be [tokens, channels] of x's dtype with contiguous channels");
  pla_b200_conv_prefill_args a{};
  a.x = x.data_ptr();
  a.x_row_stride = T > 0 ? x.stride(0) : C;
  a.y = y.data_ptr();
  a.y_row_stride = T > 0 ? y.stride(0) : C;
  a.weight = weight.data_ptr<float>();
  a.bias = bias.has_value() ? bias->data_ptr<float>() : nullptr;
  if (conv_state.has_value()) {
    TORCH_CHECK(conv_state->device() == x.device() && conv_state->scalar_type() == x.scalar_type() &&
                    conv_state->dim() == 3 && conv_state->size(1) == C && conv_state->size(2) == 3,
                "conv_state must be a [slots, channels, 3] view of x's dtype on x's device");
    a.conv_state = conv_state->data_ptr();
    a.conv_strides = {conv_state->stride(0), conv_state->stride(1), conv_state->stride(2)};
    a.slots = static_cast<int32_t>(conv_state->size(0));
  }
  a.cu_seqlens = cu_seqlens.data_ptr<int32_t>();
  if (state_indices.has_value()) {
    TORCH_CHECK(state_indices->is_contiguous() && state_indices->numel() == N && state_indices->device() == x.device(),
                "state_indices must be contiguous int32 [N] on x's device");
    a.state_indices = i32_ptr(state_indices, "state_indices");
  } else {
    TORCH_CHECK(!conv_state.has_value() || conv_state->size(0) >= N, "conv_state has fewer slots than sequences");
  }
  if (has_initial_state.has_value()) {
    TORCH_CHECK((has_initial_state->scalar_type() == at::kBool || has_initial_state->scalar_type() == at::kByte) &&
                    has_initial_state->is_contiguous() && has_initial_state->numel() == N &&
                    has_initial_state->device() == x.device(),
                "has_initial_state must be contiguous bool or uint8 [N] on x's device");
    a.has_initial_state = static_cast<const uint8_t*>(has_initial_state->data_ptr());
  }
  a.N = static_cast<int32_t>(N);
  a.tokens = static_cast<int32_t>(T);
  a.channels = static_cast<int32_t>(C);
  a.act_dtype = dtype_tag(x, "x");
  a.activation = silu ? 1 : 0;
  a.pad = vllm_pad ? PLA_B200_PAD_VLLM : PLA_B200_PAD_SGLANG;
  a.status = status.has_value() ? const_cast<int32_t*>(i32_ptr(status, "status")) : nullptr;
  if (sanity_check()) {
    const std::string why = sanity_offsets(cu_seqlens, T, 0);
    TORCH_CHECK(why.empty(), "causal conv: ", why);
  }
  if (!bypass_exec()) check_abi(pla_b200_causal_conv_prefill(&a, stream_of(x)), "causal conv prefill");
  return y;
}

}  // namespace pla_ops

TORCH_LIBRARY_FRAGMENT(pla_b200, m) {
  m.def(
      "causal_conv_prefill(Tensor x, Tensor weight, Tensor? bias, Tensor(a!)? conv_state, Tensor cu_seqlens, "
      "Tensor? state_indices, Tensor? has_initial_state, bool silu, bool vllm_pad, Tensor(b!)? out, "
      "Tensor(c!)? status) -> Tensor",
      &pla_ops::causal_conv_prefill);
  m.def("cp_fold_prefix(Tensor pairs, Tensor? initial_state, int rank, Tensor(a!)? status) -> Tensor",
        &pla_ops::cp_fold_prefix);
  m.def("cp_compose_pairs(Tensor pairs, int count, Tensor(a!)? status) -> Tensor", &pla_ops::cp_compose_pairs);
  m.def(
      "kda_prefill_chunked(Tensor q, Tensor k, Tensor v, Tensor gate, Tensor beta, Tensor A_log, Tensor dt_bias, "
      "Tensor(a!) out, Tensor cu_seqlens, Tensor(b!)? state_in, Tensor? in_indices, Tensor(c!)? state_out, "
      "Tensor? out_indices, Tensor(w!)? workspace, bool transposed, bool normalize_qk, float scale, "
      "float? lower_bound, bool update_in_place, int max_chunks, int stage, bool prescan, Tensor(d!)? status, Tensor? range_mask=None) -> Tensor",
      &pla_ops::kda_prefill_chunked);
  m.def(
      "gdn_prefill_chunked(Tensor q, Tensor k, Tensor v, Tensor gate, Tensor beta, Tensor? A_log, Tensor? dt_bias, "
      "Tensor(a!) out, Tensor(e!)? g_cum, Tensor cu_seqlens, Tensor(b!)? state_in, Tensor? in_indices, "
      "Tensor(c!)? state_out, Tensor? out_indices, bool transposed, bool normalize_qk, float scale, "
      "bool gate_activated, bool update_in_place, int max_chunks, int stage, Tensor(d!)? status) -> Tensor",
      &pla_ops::gdn_prefill_chunked);
  m.def(
      "gdn_prefill_chunked_stage(Tensor q, Tensor k, Tensor v, Tensor gate, Tensor beta, Tensor? A_log, "
      "Tensor? dt_bias, Tensor(a!) out, Tensor(e!)? g_cum, Tensor cu_seqlens, Tensor? state_in, Tensor(c!)? state_out, "
      "Tensor(w!)? workspace, bool transposed, bool normalize_qk, float scale, bool gate_activated, int max_chunks, "
      "int stage, bool prescan, Tensor(d!)? status, Tensor? range_mask, Tensor? out_indices) -> Tensor",
      &pla_ops::gdn_prefill_chunked_stage);
  m.def("cp_fold_segments(Tensor pairs, Tensor seg_first, Tensor? pool, Tensor? slot_indices, Tensor(a!)? status) -> Tensor",
        &pla_ops::cp_fold_segments);
  m.def(
      "prefill_recurrent_prescan(Tensor q, Tensor k, Tensor v, Tensor gate, Tensor beta, Tensor? A_log, "
      "Tensor? dt_bias, Tensor cu_seqlens, Tensor(a!) pairs, bool is_kda, bool normalize_qk, float scale, "
      "float? lower_bound, bool gate_activated, Tensor(b!)? status) -> ()",
      &pla_ops::prefill_recurrent_prescan);
  m.def(
      "prefill_recurrent(Tensor q, Tensor k, Tensor v, Tensor gate, Tensor beta, Tensor? A_log, Tensor? dt_bias, "
      "Tensor(a!) out, Tensor cu_seqlens, Tensor(b!)? state_in, Tensor? in_indices, Tensor(c!)? state_out, "
      "Tensor? out_indices, bool transposed, bool is_kda, bool normalize_qk, float scale, float? lower_bound, "
      "bool gate_activated, bool update_in_place, Tensor(d!)? status) -> ()",
      &pla_ops::prefill_recurrent);
}
