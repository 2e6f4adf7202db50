// Host layer of the vLLM-style KDA ReplaySSM ops: the tensor contracts of
// pla.decode.kda_replayssm_vllm._C.{verify, layer_descriptor, commit}
// (src/decode/kda_replayssm_vllm/kda_replayssm_vllm.cpp:34-350) checked with
// TORCH_CHECK, then one C-ABI call on the current stream. No sync, no D2H.
#include <cmath>
#include <string>
#include <vector>

#include "ops_common.h"

namespace pla_ops {
namespace {

constexpr int64_t D = 128;
using Optional = std::optional<at::Tensor>;

void tensor(const at::Tensor& t, const at::Tensor& ref) {
  TORCH_CHECK(t.defined() && t.layout() == at::kStrided && t.is_cuda() && t.device() == ref.device(),
              "replay tensors must share a CUDA device");
  for (auto size : t.sizes()) TORCH_CHECK(size <= INT32_MAX, "tensor dimension exceeds the native int32 ABI");
  for (auto stride : t.strides()) TORCH_CHECK(stride > 0, "strides must be positive");
}
void dense(const at::Tensor& t, at::ScalarType dtype, at::IntArrayRef shape) {
  TORCH_CHECK(t.scalar_type() == dtype && t.sizes() == shape && t.is_contiguous(),
              "invalid replay tensor shape/dtype/contiguity");
}
void indices(const at::Tensor& t, const at::Tensor& ref) {
  tensor(t, ref);
  TORCH_CHECK(t.dim() == 1 && (t.scalar_type() == at::kInt || t.scalar_type() == at::kLong),
              "indices must be int32/int64 vectors");
}
pla_b200_index index(const at::Tensor& t) { return {t.data_ptr(), t.scalar_type() == at::kLong, t.stride(0)}; }
pla_b200_index index(const Optional& t) { return t ? index(*t) : pla_b200_index{nullptr, 0, 1}; }
void null_id(int64_t v) { TORCH_CHECK(v == -1 || v == 0, "null_block_id must be -1 or 0"); }

// Validates the paged cache pair and returns the conv history viewed [slots, channels, history].
at::Tensor cache(const at::Tensor& conv, const at::Tensor& state, const std::string& layout, int64_t H,
                 int64_t slots) {
  TORCH_CHECK(state.is_cuda() && H > 0 && H <= INT32_MAX / (D * D) && slots > 0,
              "paged state requires CUDA, H > 0, slots > 0");
  tensor(state, state);
  tensor(conv, state);
  TORCH_CHECK(state.scalar_type() == at::kFloat && state.sizes() == at::IntArrayRef({slots, H, D, D}) &&
                  state.stride(3) == 1 && state.stride(2) == D && state.stride(1) == D * D &&
                  state.stride(0) >= H * D * D && state.stride(0) % 4 == 0 &&
                  reinterpret_cast<uintptr_t>(state.data_ptr()) % 16 == 0,
              "state must be float4-aligned fp32 [slots,H,128,128] with contiguous pages");
  TORCH_CHECK(layout == "DS" || layout == "SD", "conv_state_layout must be DS or SD");
  TORCH_CHECK(conv.dim() == 3 && conv.size(0) == slots && conv.scalar_type() == at::kBFloat16,
              "conv must be bf16 with three dimensions");
  at::Tensor ds = layout == "DS" ? conv : conv.transpose(1, 2);
  TORCH_CHECK(ds.size(1) == 3 * H * D && ds.size(2) >= 3,
              "conv must contain 3*H*128 channels and at least three history items");
  TORCH_CHECK((ds.stride(2) == 1 && ds.stride(1) >= ds.size(2)) || (ds.stride(1) == 1 && ds.stride(2) >= ds.size(1)),
              "conv channel/history dimensions must not overlap");
  TORCH_CHECK(ds.stride(0) >= (ds.size(1) - 1) * ds.stride(1) + (ds.size(2) - 1) * ds.stride(2) + 1,
              "conv pages must not overlap");
  return ds;
}

void records(const at::Tensor& rv, const at::Tensor& rk, const at::Tensor& g, const at::Tensor& b,
             const at::Tensor& windows, const at::Tensor& ref, int64_t H, int64_t Q, int64_t R) {
  TORCH_CHECK(Q >= 1 && Q <= 32 && R >= 0, "records require Q in [1,32] and R >= 0");
  for (const at::Tensor* t : {&rv, &rk, &g, &b, &windows}) tensor(*t, ref);
  dense(rv, at::kBFloat16, {R, H, Q, D});
  dense(rk, at::kBFloat16, {R, H, Q, D});
  dense(g, at::kFloat, {R, H, Q, D});
  dense(b, at::kFloat, {R, H, Q});
  dense(windows, at::kBFloat16, {R, Q, 3 * H * D, 3});
  for (const at::Tensor* t : {&rv, &rk, &g, &b})
    TORCH_CHECK(reinterpret_cast<uintptr_t>(t->data_ptr()) % 16 == 0, "replay records must be 16-byte aligned");
}

// Conservative byte-span overlap test between writable outputs and everything that is read.
std::pair<uintptr_t, uintptr_t> span(const at::Tensor& t) {
  const auto begin = reinterpret_cast<uintptr_t>(t.data_ptr());
  if (!t.numel()) return {begin, begin};
  int64_t extent = 1;
  for (int64_t d = 0; d < t.dim(); ++d) extent += (t.size(d) - 1) * t.stride(d);
  return {begin, begin + extent * t.element_size()};
}
void disjoint(const std::vector<at::Tensor>& writes, const std::vector<at::Tensor>& reads) {
  auto overlap = [](const at::Tensor& a, const at::Tensor& b) {
    const auto x = span(a), y = span(b);
    return x.first < y.second && y.first < x.second;
  };
  for (size_t i = 0; i < writes.size(); ++i) {
    for (size_t j = 0; j < i; ++j) TORCH_CHECK(!overlap(writes[i], writes[j]), "replay writes must not alias");
    for (const auto& read : reads) TORCH_CHECK(!overlap(writes[i], read), "replay writes must not alias inputs/cache");
  }
}

std::vector<int64_t> layer_descriptor(const at::Tensor& conv, const at::Tensor& state, const at::Tensor& rv,
                                      const at::Tensor& rk, const at::Tensor& gate, const at::Tensor& beta,
                                      const at::Tensor& windows, std::string layout, int64_t H, int64_t slots,
                                      int64_t Q, int64_t R) {
  at::Tensor ds = cache(conv, state, layout, H, slots);
  records(rv, rk, gate, beta, windows, state, H, Q, R);
  disjoint({rv, rk, gate, beta, windows}, {conv, state});
  auto ptr = [](const at::Tensor& t) { return reinterpret_cast<int64_t>(t.data_ptr()); };
  return {ptr(state), state.stride(0), ptr(conv), ds.stride(0), ds.stride(1), ds.stride(2),
          ptr(rv),    ptr(rk),         ptr(gate), ptr(beta),    ptr(windows)};
}

void verify(const at::Tensor& x, const at::Tensor& g, const at::Tensor& beta, const at::Tensor& weight,
            const at::Tensor& conv, const at::Tensor& state, const at::Tensor& a, const at::Tensor& dt,
            at::Tensor out, at::Tensor rv, at::Tensor rk, at::Tensor gate, at::Tensor rb, at::Tensor windows,
            const at::Tensor& cu, const at::Tensor& source, std::string layout, double scale,
            std::optional<double> lower_bound, int64_t null, const Optional& status) {
  null_id(null);
  TORCH_CHECK(state.dim() == 4 && rv.dim() == 4, "invalid state/records rank");
  const int64_t H = state.size(1), slots = state.size(0), Q = rv.size(2), R = rv.size(0);
  at::Tensor cs = cache(conv, state, layout, H, slots);
  const c10::cuda::CUDAGuard guard(state.device());
  records(rv, rk, gate, rb, windows, state, H, Q, R);
  for (const at::Tensor* t : std::initializer_list<const at::Tensor*>{&x, &g, &beta, &weight, &a, &dt, &out, &cu, &source})
    tensor(*t, state);
  TORCH_CHECK(x.dim() == 2 && x.size(0) <= INT32_MAX && x.size(1) == 3 * H * D && x.stride(1) == 1 &&
                  x.stride(0) >= 3 * H * D && x.scalar_type() == at::kBFloat16,
              "mixed_qkv must be bf16 [T,3*H*128] with contiguous channels and T <= INT32_MAX");
  const int64_t T = x.size(0);
  auto projection = [&](const at::Tensor& t, int64_t channels) {
    TORCH_CHECK(t.sizes() == at::IntArrayRef({T, channels}) && t.stride(1) == 1 && t.stride(0) >= channels &&
                    t.scalar_type() == at::kBFloat16,
                "gate/beta must be bf16 projection views");
  };
  projection(g, H * D);
  projection(beta, H);
  dense(weight, at::kFloat, {3 * H * D, 4});
  TORCH_CHECK(a.numel() == H && dt.numel() == H * D && a.is_contiguous() && dt.is_contiguous() &&
                  a.scalar_type() == at::kFloat && dt.scalar_type() == at::kFloat,
              "gate weights must be contiguous fp32");
  dense(out, at::kBFloat16, {T, H * D});
  TORCH_CHECK(std::isfinite(scale) && std::isfinite(static_cast<float>(scale)), "scale must be finite fp32");
  if (lower_bound.has_value())
    TORCH_CHECK(std::isfinite(*lower_bound) && static_cast<float>(*lower_bound) < 0 &&
                    std::isfinite(static_cast<float>(*lower_bound)),
                "scale/lower_bound must be finite fp32; bound < 0");
  indices(cu, state);
  indices(source, state);
  const int64_t N = source.numel();
  TORCH_CHECK(cu.numel() == N + 1 && N <= R, "query index count exceeds record capacity");
  disjoint({out, rv, rk, gate, rb, windows}, {x, g, beta, weight, conv, state, a, dt, cu, source});

  pla_b200_kda_verify_args v{};
  const int64_t C = H * D;
  const auto* xp = static_cast<const char*>(x.data_ptr());
  v.x_q = xp;
  v.x_k = xp + C * 2;
  v.x_v = xp + 2 * C * 2;
  v.xq_tok_stride = v.xk_tok_stride = v.xv_tok_stride = x.stride(0);
  v.raw_g = g.data_ptr();
  v.raw_beta = beta.data_ptr();
  v.g_tok_stride = g.stride(0);
  v.beta_tok_stride = beta.stride(0);
  v.w_q = weight.data_ptr<float>();
  v.w_k = v.w_q + C * 4;
  v.w_v = v.w_q + 2 * C * 4;
  const auto* cp = static_cast<const char*>(conv.data_ptr());
  const pla_b200_conv_strides cstr{cs.stride(0), cs.stride(1), cs.stride(2)};
  v.cs_q = cp;
  v.cs_k = cp + C * cs.stride(1) * 2;
  v.cs_v = cp + 2 * C * cs.stride(1) * 2;
  v.cs_q_strides = v.cs_k_strides = v.cs_v_strides = cstr;
  v.A_log = a.data_ptr<float>();
  v.dt_bias = dt.data_ptr<float>();
  v.state = state.data_ptr<float>();
  v.state_slot_stride = state.stride(0);
  v.slots = static_cast<int32_t>(slots);
  v.out = out.data_ptr();
  v.rec_rawv = rv.data_ptr();
  v.rec_rawk = rk.data_ptr();
  v.rec_g = gate.data_ptr<float>();
  v.rec_beta = rb.data_ptr<float>();
  auto* wp = static_cast<char*>(windows.data_ptr());
  const pla_b200_window_strides wstr{windows.stride(0), windows.stride(1), windows.stride(2), windows.stride(3)};
  v.win_q = wp;
  v.win_k = wp + C * windows.stride(2) * 2;
  v.win_v = wp + 2 * C * windows.stride(2) * 2;
  v.win_q_strides = v.win_k_strides = v.win_v_strides = wstr;
  v.slot_idx = index(source);
  v.cu = index(cu);
  v.scratch_idx = pla_b200_index{nullptr, 0, 1};
  v.H = static_cast<int32_t>(H);
  v.N = static_cast<int32_t>(N);
  v.Q = static_cast<int32_t>(Q);
  v.T = static_cast<int32_t>(T);
  v.null_block_id = static_cast<int32_t>(null);
  v.row_by_slot = 0;
  v.gate = lower_bound.has_value() ? PLA_B200_GATE_SAFE : PLA_B200_GATE_SOFTPLUS;
  v.scale = static_cast<float>(scale);
  v.lower_bound = static_cast<float>(lower_bound.value_or(0.0));
  v.softplus_beta = 1.0f;
  v.softplus_threshold = 20.0f;
  v.status = status.has_value() ? const_cast<int32_t*>(i32_ptr(status, "status")) : nullptr;
  check_abi(pla_b200_kda_replay_verify(&v, stream_of(state)), "kda_replay_verify");
}

void commit(const at::Tensor& table, at::Tensor candidate, at::Tensor plan, const at::Tensor& sampled,
            const at::Tensor& source, const at::Tensor& cu, const Optional& mapping, const Optional& blocks,
            const Optional& computed, int64_t block_size, int64_t H, int64_t slots, int64_t Q, int64_t null,
            int64_t token_capacity, bool plan_only, const Optional& status) {
  null_id(null);
  TORCH_CHECK(token_capacity >= 0 && token_capacity <= INT32_MAX, "token_capacity must be between 0 and INT32_MAX");
  TORCH_CHECK(table.is_cuda() && table.dim() == 2 && table.size(0) > 0 && table.size(1) == PLA_B200_REPLAY_COLUMNS &&
                  table.is_contiguous() && table.scalar_type() == at::kLong,
              "invalid layer pointer table");
  const c10::cuda::CUDAGuard guard(table.device());
  TORCH_CHECK(plan.dim() == 2 && plan.size(0) == 4 && Q >= 1 && Q <= 32 && H > 0 && slots > 0 &&
                  table.size(0) * H <= INT32_MAX,
              "invalid commit plan dimensions");
  const int64_t R = plan.size(1), N = source.numel();
  for (const at::Tensor* t : std::initializer_list<const at::Tensor*>{&table, &candidate, &plan}) tensor(*t, table);
  dense(plan, at::kInt, {4, R});
  dense(candidate, at::kInt, {4, R});
  for (const at::Tensor* t : {&sampled, &source, &cu}) indices(*t, table);
  TORCH_CHECK(N <= R && cu.numel() == N + 1, "commit query count exceeds capacity");
  if (mapping) {
    indices(*mapping, table);
    TORCH_CHECK(mapping->numel() == N, "mapping must have N rows");
  } else {
    TORCH_CHECK(sampled.numel() >= N, "sampler count must cover query rows");
  }
  TORCH_CHECK(bool(blocks) == bool(computed) && bool(blocks) == (block_size != 0),
              "align arguments must be supplied together");
  if (blocks) {
    tensor(*blocks, table);
    indices(*computed, table);
    TORCH_CHECK(block_size >= Q && blocks->dim() == 2 && blocks->size(1) > 0 &&
                    (blocks->scalar_type() == at::kInt || blocks->scalar_type() == at::kLong) &&
                    computed->numel() >= sampled.numel(),
                "invalid align table/count/block size");
  }
  disjoint({candidate, plan}, {table, sampled, source, cu});
  if (mapping) disjoint({candidate, plan}, {*mapping});
  if (blocks) disjoint({candidate, plan}, {*blocks, *computed});

  pla_b200_kda_commit_args c{};
  c.layers = table.data_ptr<int64_t>();
  c.n_layers = static_cast<int32_t>(table.size(0));
  c.candidate = candidate.data_ptr<int32_t>();
  c.plan = plan.data_ptr<int32_t>();
  c.sampled = index(sampled);
  c.source = index(source);
  c.cu = index(cu);
  c.mapping = index(mapping);
  c.computed = index(computed);
  c.blocks = blocks ? pla_b200_index{blocks->data_ptr(), blocks->scalar_type() == at::kLong, 1}
                    : pla_b200_index{nullptr, 0, 1};
  c.block_row_stride = blocks ? blocks->stride(0) : 0;
  c.block_col_stride = blocks ? blocks->stride(1) : 0;
  c.block_size = block_size;
  c.block_rows = blocks ? static_cast<int32_t>(blocks->size(0)) : 0;
  c.block_cols = blocks ? static_cast<int32_t>(blocks->size(1)) : 0;
  c.N = static_cast<int32_t>(N);
  c.capacity = static_cast<int32_t>(R);
  c.sampler_rows = static_cast<int32_t>(sampled.numel());
  c.H = static_cast<int32_t>(H);
  c.slots = static_cast<int32_t>(slots);
  c.Q = static_cast<int32_t>(Q);
  c.null_block_id = static_cast<int32_t>(null);
  c.token_capacity = token_capacity;
  c.status = status.has_value() ? const_cast<int32_t*>(i32_ptr(status, "status")) : nullptr;
  void* stream = static_cast<void*>(c10::cuda::getCurrentCUDAStream(table.device().index()).stream());
  check_abi(plan_only ? pla_b200_kda_replay_plan(&c, stream) : pla_b200_kda_replay_commit(&c, stream),
            "kda_replay_commit");
}

}  // namespace
}  // namespace pla_ops

TORCH_LIBRARY_FRAGMENT(pla_b200, m) {
  m.def(
      "kda_replay_verify(Tensor mixed_qkv, Tensor raw_g, Tensor raw_beta, Tensor conv_weight, Tensor conv_state, "
      "Tensor checkpoint_state, Tensor A_log, Tensor dt_bias, Tensor(a!) out, Tensor(b!) rawv, Tensor(c!) rawk, "
      "Tensor(d!) g, Tensor(e!) beta, Tensor(f!) conv, Tensor query_start_loc, Tensor state_indices, "
      "str conv_state_layout, float scale, float? lower_bound, int null_block_id, Tensor(g!)? status) -> ()",
      &pla_ops::verify);
  m.def(
      "kda_replay_layer_descriptor(Tensor conv, Tensor state, Tensor rawv, Tensor rawk, Tensor g, Tensor beta, "
      "Tensor windows, str conv_state_layout, int heads, int slots, int spec_query_len, int max_num_reqs) -> int[]",
      &pla_ops::layer_descriptor);
  m.def(
      "kda_replay_commit(Tensor table, Tensor(a!) candidate, Tensor(b!) plan, Tensor num_sampled, "
      "Tensor state_indices, Tensor query_start_loc, Tensor? request_indices, Tensor? block_table, "
      "Tensor? num_computed_tokens, int mamba_block_size, int heads, int slots, int spec_query_len, "
      "int null_block_id, int token_capacity, bool plan_only, Tensor(c!)? status) -> ()",
      &pla_ops::commit);
}
