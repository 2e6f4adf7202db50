// Host layer of the vLLM-style KDA ReplaySSM ops: the tensor contracts of
// pla.decode.kda_replayssm_vllm._C.{verify, layer_descriptor, commit}
// (src/decode/kda_replayssm_vllm/kda_replayssm_vllm.cpp:34-350) checked with
// TORCH_CHECK, then one C-ABI call on the current stream. No sync, no D2H.
#include <algorithm>
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
  if (!bypass_exec()) check_abi(pla_b200_kda_replay_verify(&v, stream_of(state)), "kda_replay_verify");
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
  if (!bypass_exec()) check_abi(plan_only ? pla_b200_kda_replay_plan(&c, stream) : pla_b200_kda_replay_commit(&c, stream),
            "kda_replay_commit");
}


// ---- SGLang contract (src/decode/kda_replayssm_sglang/kda_mtp_verify_host.cpp, kda_mtp_fold_host.cpp) ----
// verify_dspark: separate q/k/v activations, conv weights and conv states; rings addressed by state
// slot; conv windows addressed by scratch row; optional fused gated output RMSNorm.
void ring_verify(const at::Tensor& x_q, const at::Tensor& x_k, const at::Tensor& x_v, const at::Tensor& g_in,
                 const at::Tensor& beta_in, const at::Tensor& w_q, const at::Tensor& w_k, const at::Tensor& w_v,
                 const at::Tensor& cs_q, const at::Tensor& cs_k, const at::Tensor& cs_v, const at::Tensor& A_log,
                 const at::Tensor& dt_bias, const at::Tensor& h0, at::Tensor out, at::Tensor ic_q, at::Tensor ic_k,
                 at::Tensor ic_v, at::Tensor ring_rawv, at::Tensor ring_rawk, at::Tensor ring_g, at::Tensor ring_beta,
                 const at::Tensor& slot_idx, const at::Tensor& scratch_idx, const at::Tensor& cu_seqlens, double scale,
                 std::optional<double> lower_bound, const Optional& onorm_gate, const Optional& onorm_weight,
                 std::optional<double> onorm_eps, const Optional& status) {
  const bool apply_onorm = onorm_gate.has_value();
  TORCH_CHECK(onorm_weight.has_value() == apply_onorm && onorm_eps.has_value() == apply_onorm,
              "fused output norm requires onorm_gate, onorm_weight and onorm_eps");
  constexpr int64_t CONV_W = 4, CONV_WIN = 3;
  TORCH_CHECK(x_q.dim() == 4 && x_q.size(0) == 1, "x_q must be [1, T, H, 128]");
  TORCH_CHECK(x_q.is_cuda(), "verify requires CUDA tensors");
  const c10::cuda::CUDAGuard guard(x_q.device());
  const int64_t T = x_q.size(1), H = x_q.size(2);
  TORCH_CHECK(x_q.size(3) == D, "specialised for head_dim 128");
  const int64_t N = cu_seqlens.numel() - 1;
  TORCH_CHECK(N > 0 && T > 0 && H > 0 && T % N == 0, "dense 1 + num_spec tokens per request");
  const int64_t T_LOOP = T / N;
  TORCH_CHECK(ring_rawv.dim() == 4, "rawv ring must be [slot, H, L, 128]");
  const int64_t L = ring_rawv.size(2), slots = ring_rawv.size(0);
  TORCH_CHECK(L >= T_LOOP && L <= 32, "ring shorter than the draft window (or longer than 32)");
  TORCH_CHECK(h0.scalar_type() == at::kFloat, "recurrent state must be fp32");
  TORCH_CHECK(x_q.scalar_type() == at::kBFloat16, "inputs must be bf16");
  TORCH_CHECK(h0.sizes() == at::IntArrayRef({slots, H, D, D}), "state must be [slot, H, 128, 128]");
  for (const at::Tensor* t : std::initializer_list<const at::Tensor*>{
           &x_k, &x_v, &g_in, &beta_in, &w_q, &w_k, &w_v, &cs_q, &cs_k, &cs_v, &A_log, &dt_bias, &h0, &out, &ic_q,
           &ic_k, &ic_v, &ring_rawv, &ring_rawk, &ring_g, &ring_beta, &slot_idx, &scratch_idx, &cu_seqlens})
    TORCH_CHECK(t->device() == x_q.device(), "verify tensors must share one device");
  for (const at::Tensor* t : std::initializer_list<const at::Tensor*>{&ring_rawv, &ring_rawk, &ring_g})
    TORCH_CHECK(t->sizes() == at::IntArrayRef({slots, H, L, D}), "invalid verify ring shape");
  TORCH_CHECK(ring_beta.sizes() == at::IntArrayRef({slots, H, L}) && ring_rawv.scalar_type() == at::kBFloat16 &&
                  ring_rawk.scalar_type() == at::kBFloat16 && ring_g.scalar_type() == at::kFloat &&
                  ring_beta.scalar_type() == at::kFloat,
              "invalid verify ring dtype/shape");
  for (const at::Tensor* t : std::initializer_list<const at::Tensor*>{&w_q, &w_k, &w_v})
    TORCH_CHECK(t->sizes() == at::IntArrayRef({H * D, CONV_W}) && t->is_contiguous() && t->scalar_type() == at::kFloat,
                "conv weights must be contiguous fp32 [H*128, 4]");
  TORCH_CHECK(A_log.numel() == H && dt_bias.numel() == H * D && A_log.is_contiguous() && dt_bias.is_contiguous() &&
                  A_log.scalar_type() == at::kFloat && dt_bias.scalar_type() == at::kFloat,
              "invalid gate weights");
  TORCH_CHECK(h0.storage_offset() % 4 == 0, "recurrent state must be 16-byte aligned for float4 loads");
  for (const at::Tensor* t : std::initializer_list<const at::Tensor*>{&slot_idx, &scratch_idx, &cu_seqlens})
    TORCH_CHECK(t->dim() == 1 && (t->scalar_type() == at::kInt || t->scalar_type() == at::kLong),
                "verify indices must be int32/int64 vectors");
  TORCH_CHECK(slot_idx.numel() == N && scratch_idx.numel() >= N, "verify index count mismatch");
  auto input_stride = [&](const at::Tensor& x) -> int64_t {
    TORCH_CHECK(x.sizes() == x_q.sizes() && x.scalar_type() == at::kBFloat16, "Q/K/V and g must be bf16 [1, T, H, 128]");
    TORCH_CHECK(x.stride(3) == 1 && x.stride(2) == D && x.stride(1) >= H * D,
                "Q/K/V and g must have contiguous head/channel dimensions");
    return x.stride(1);
  };
  auto conv_strides = [&](const at::Tensor& x) -> pla_b200_conv_strides {
    TORCH_CHECK(x.dim() == 3 && x.size(0) == slots && x.size(1) == H * D && x.size(2) == CONV_WIN &&
                    x.scalar_type() == at::kBFloat16,
                "conv states must be bf16 [slot, H*128, 3]");
    TORCH_CHECK(x.stride(0) > 0 && x.stride(1) > 0 && x.stride(2) > 0, "conv state strides must be positive");
    return {x.stride(0), x.stride(1), x.stride(2)};
  };
  auto window_strides = [&](const at::Tensor& x) -> pla_b200_window_strides {
    TORCH_CHECK(x.dim() == 4 && x.size(1) >= T_LOOP && x.size(2) == H * D && x.size(3) == CONV_WIN &&
                    x.scalar_type() == at::kBFloat16,
                "conv windows must be bf16 [scratch, step, H*128, 3]");
    TORCH_CHECK(x.stride(0) > 0 && x.stride(1) > 0 && x.stride(2) > 0 && x.stride(3) > 0,
                "conv window strides must be positive");
    return {x.stride(0), x.stride(1), x.stride(2), x.stride(3)};
  };
  TORCH_CHECK(beta_in.dim() == 3 && beta_in.size(0) == 1 && beta_in.size(1) == T && beta_in.size(2) == H &&
                  beta_in.scalar_type() == at::kBFloat16 && beta_in.stride(2) == 1 && beta_in.stride(1) >= H,
              "beta must be bf16 [1, T, H] with contiguous heads");
  TORCH_CHECK(out.sizes() == x_q.sizes() && out.is_contiguous() && out.scalar_type() == at::kBFloat16 &&
                  h0.is_contiguous() && ring_rawv.is_contiguous() && ring_rawk.is_contiguous() &&
                  ring_g.is_contiguous() && ring_beta.is_contiguous(),
              "output, recurrent state and rings must be contiguous");
  TORCH_CHECK(std::isfinite(scale), "scale must be finite");
  if (lower_bound.has_value()) TORCH_CHECK(std::isfinite(*lower_bound) && *lower_bound < 0, "lower_bound must be finite and negative");

  pla_b200_kda_verify_args v{};
  v.x_q = x_q.data_ptr();
  v.x_k = x_k.data_ptr();
  v.x_v = x_v.data_ptr();
  v.xq_tok_stride = input_stride(x_q);
  v.xk_tok_stride = input_stride(x_k);
  v.xv_tok_stride = input_stride(x_v);
  v.raw_g = g_in.data_ptr();
  v.g_tok_stride = input_stride(g_in);
  v.raw_beta = beta_in.data_ptr();
  v.beta_tok_stride = beta_in.stride(1);
  v.w_q = w_q.data_ptr<float>();
  v.w_k = w_k.data_ptr<float>();
  v.w_v = w_v.data_ptr<float>();
  v.cs_q = cs_q.data_ptr();
  v.cs_k = cs_k.data_ptr();
  v.cs_v = cs_v.data_ptr();
  v.cs_q_strides = conv_strides(cs_q);
  v.cs_k_strides = conv_strides(cs_k);
  v.cs_v_strides = conv_strides(cs_v);
  v.A_log = A_log.data_ptr<float>();
  v.dt_bias = dt_bias.data_ptr<float>();
  v.state = h0.data_ptr<float>();
  v.state_slot_stride = h0.stride(0);
  v.slots = static_cast<int32_t>(slots);
  v.out = out.data_ptr();
  v.rec_rawv = ring_rawv.data_ptr();
  v.rec_rawk = ring_rawk.data_ptr();
  v.rec_g = ring_g.data_ptr<float>();
  v.rec_beta = ring_beta.data_ptr<float>();
  v.win_q = ic_q.data_ptr();
  v.win_k = ic_k.data_ptr();
  v.win_v = ic_v.data_ptr();
  v.win_q_strides = window_strides(ic_q);
  v.win_k_strides = window_strides(ic_k);
  v.win_v_strides = window_strides(ic_v);
  v.slot_idx = index(slot_idx);
  v.scratch_idx = index(scratch_idx);
  v.cu = index(cu_seqlens);
  v.H = static_cast<int32_t>(H);
  v.N = static_cast<int32_t>(N);
  v.Q = static_cast<int32_t>(L);
  v.T = static_cast<int32_t>(T);
  v.null_block_id = -1;
  v.row_by_slot = 1;
  v.win_steps = static_cast<int32_t>(std::min({ic_q.size(1), ic_k.size(1), ic_v.size(1)}));
  v.gate = lower_bound.has_value() ? PLA_B200_GATE_SAFE : PLA_B200_GATE_SOFTPLUS;
  v.scale = static_cast<float>(scale);
  v.lower_bound = static_cast<float>(lower_bound.value_or(0.0));
  v.softplus_beta = 1.0f;
  v.softplus_threshold = 20.0f;
  v.status = status.has_value() ? const_cast<int32_t*>(i32_ptr(status, "status")) : nullptr;
  at::Tensor staging;
  if (apply_onorm) {
    const at::Tensor& gate = *onorm_gate;
    const at::Tensor& weight = *onorm_weight;
    TORCH_CHECK(gate.device() == x_q.device() && weight.device() == x_q.device(),
                "output-norm tensors must share the verify device");
    TORCH_CHECK(gate.sizes() == x_q.sizes() && gate.scalar_type() == at::kBFloat16 && gate.stride(3) == 1 &&
                    gate.stride(2) == D && gate.stride(1) >= H * D,
                "output-norm gate must be bf16 [1, T, H, 128] with contiguous head/channel dimensions");
    TORCH_CHECK(weight.dim() == 1 && weight.size(0) == D && weight.is_contiguous() && weight.scalar_type() == at::kFloat,
                "output-norm weight must be contiguous fp32 [128]");
    TORCH_CHECK(std::isfinite(*onorm_eps) && *onorm_eps >= 0.0, "output-norm eps must be finite and non-negative");
    staging = at::empty({T, H, D}, x_q.options().dtype(at::kFloat));   // caching allocator: safe under graph capture
    v.onorm_gate = gate.data_ptr();
    v.onorm_gate_tok_stride = gate.stride(1);
    v.onorm_weight = weight.data_ptr<float>();
    v.onorm_eps = static_cast<float>(*onorm_eps);
    v.out_f32 = staging.data_ptr<float>();
  }
  if (!bypass_exec()) check_abi(pla_b200_kda_ring_verify(&v, stream_of(x_q)), "verify_dspark");
}

void fold_all_layers(at::Tensor h0, const at::Tensor& rawv, const at::Tensor& rawk, const at::Tensor& gk,
                     const at::Tensor& beta, const at::Tensor& slot_idx, const at::Tensor& accept_lens,
                     const Optional& track_idx, const Optional& track_step, int64_t num_k_heads, int64_t null_block_id,
                     const Optional& status) {
  auto rank = [](const at::Tensor& t, const char* nm, int64_t dim) {
    TORCH_CHECK(t.is_cuda(), nm, " must be CUDA");
    TORCH_CHECK(t.dim() == dim, nm, " expected ", dim, " dims, got ", t.dim());
  };
  rank(h0, "h0", 5);
  const c10::cuda::CUDAGuard guard(h0.device());
  rank(rawv, "rawv", 5);
  rank(rawk, "rawk", 5);
  rank(gk, "gk", 5);
  rank(beta, "beta", 4);
  TORCH_CHECK(h0.scalar_type() == at::kFloat, "h0 must be fp32");
  TORCH_CHECK(rawv.scalar_type() == at::kBFloat16 && rawk.scalar_type() == at::kBFloat16, "rawv/rawk must be bf16");
  TORCH_CHECK(gk.scalar_type() == at::kFloat && beta.scalar_type() == at::kFloat, "gk/beta must be fp32");
  const int64_t layers = h0.size(0), slots = h0.size(1), HV = h0.size(2), V = h0.size(3), K = h0.size(4);
  TORCH_CHECK(K == 128 && V == 128, "this kernel is specialised for K = V = 128, got K=", K, ", V=", V);
  const int64_t B = slot_idx.size(0), L = rawv.size(3);
  TORCH_CHECK(num_k_heads > 0 && HV % num_k_heads == 0 && layers > 0 && HV > 0 && L >= 1 && L <= 32,
              "fold requires grouped heads, positive dimensions, and ring length 1..32");
  TORCH_CHECK(h0.storage_offset() % 4 == 0, "recurrent state must be 16-byte aligned for float4 loads/stores");
  TORCH_CHECK(track_idx.has_value() == track_step.has_value(), "tracking indices and steps must be supplied together");
  TORCH_CHECK(rawv.sizes() == at::IntArrayRef({layers, slots, HV, L, V}) &&
                  rawk.sizes() == at::IntArrayRef({layers, slots, num_k_heads, L, K}) &&
                  gk.sizes() == at::IntArrayRef({layers, slots, HV, L, K}) &&
                  beta.sizes() == at::IntArrayRef({layers, slots, HV, L}),
              "fold state/ring shape mismatch");
  for (const at::Tensor* t : std::initializer_list<const at::Tensor*>{&h0, &rawv, &rawk, &gk, &beta})
    TORCH_CHECK(t->device() == h0.device() && t->is_contiguous(), "fold state/rings must be contiguous on the same device");
  auto check_index = [&](const at::Tensor& t) {
    TORCH_CHECK(t.device() == h0.device() && t.dim() == 1 && t.numel() == B &&
                    (t.scalar_type() == at::kInt || t.scalar_type() == at::kLong),
                "fold indices must be int32/int64 [B] on the state device");
  };
  check_index(slot_idx);
  check_index(accept_lens);
  if (track_idx.has_value()) {
    check_index(*track_idx);
    check_index(*track_step);
  }
  if (B == 0) return;
  pla_b200_kda_fold_args f{};
  f.state = h0.data_ptr<float>();
  f.state_layer_stride = h0.stride(0);
  f.state_slot_stride = h0.stride(1);
  f.rawv = rawv.data_ptr();
  f.rawv_layer_stride = rawv.stride(0);
  f.rawv_slot_stride = rawv.stride(1);
  f.rawk = rawk.data_ptr();
  f.rawk_layer_stride = rawk.stride(0);
  f.rawk_slot_stride = rawk.stride(1);
  f.gate = gk.data_ptr<float>();
  f.gate_layer_stride = gk.stride(0);
  f.gate_slot_stride = gk.stride(1);
  f.beta = beta.data_ptr<float>();
  f.beta_layer_stride = beta.stride(0);
  f.beta_slot_stride = beta.stride(1);
  f.slot_idx = index(slot_idx);
  f.accept_lens = index(accept_lens);
  f.track_idx = index(track_idx);
  f.track_step = index(track_step);
  f.layers = static_cast<int32_t>(layers);
  f.B = static_cast<int32_t>(B);
  f.H = static_cast<int32_t>(num_k_heads);
  f.HV = static_cast<int32_t>(HV);
  f.L = static_cast<int32_t>(L);
  f.slots = static_cast<int32_t>(slots);
  f.null_block_id = static_cast<int32_t>(null_block_id);
  f.status = status.has_value() ? const_cast<int32_t*>(i32_ptr(status, "status")) : nullptr;
  if (!bypass_exec()) check_abi(pla_b200_kda_fold_layers(&f, stream_of(h0)), "fold_all_layers");
}

void conv_window_scatter(at::Tensor dst, const at::Tensor& src, const at::Tensor& dst_idx, const at::Tensor& step_idx) {
  TORCH_CHECK(dst.dim() == 4 && src.dim() == 5, "ranks: dst 4, src 5");
  TORCH_CHECK(dst.is_cuda() && src.device() == dst.device() && dst.scalar_type() == src.scalar_type(),
              "conv source and destination must have the same CUDA device and dtype");
  const c10::cuda::CUDAGuard guard(dst.device());
  TORCH_CHECK(src.size(0) == dst.size(0) && src.size(3) == dst.size(2) && src.size(4) == dst.size(3),
              "conv source/destination shape mismatch");
  TORCH_CHECK(dst.is_contiguous() || dst.transpose(-1, -2).is_contiguous(),
              "conv destination must be contiguous in dim_width or width_dim layout");
  TORCH_CHECK(dst_idx.device() == dst.device() && step_idx.device() == dst.device() && dst_idx.dim() == 1 &&
                  step_idx.dim() == 1 && dst_idx.numel() == step_idx.numel(),
              "invalid conv scatter indices");
  for (const at::Tensor* t : {&dst_idx, &step_idx})
    TORCH_CHECK(t->scalar_type() == at::kInt || t->scalar_type() == at::kLong, "conv scatter indices must be int32/int64");
  const int64_t reqs = step_idx.size(0), km1 = dst.size(3);
  if (reqs == 0) return;
  TORCH_CHECK(km1 >= 1 && km1 <= 4, "conv scatter: unsupported conv window ", km1);
  TORCH_CHECK(dst.scalar_type() == at::kBFloat16 || dst.scalar_type() == at::kFloat,
              "conv scatter: unsupported dtype ", dst.scalar_type());
  pla_b200_kda_conv_scatter_args c{};
  c.dst = dst.data_ptr();
  c.src = src.data_ptr();
  c.dst_layer = dst.stride(0);
  c.dst_slot = dst.stride(1);
  c.dst_channel = dst.stride(2);
  c.dst_tap = dst.stride(3);
  c.src_layer = src.stride(0);
  c.src_row = src.stride(1);
  c.src_step = src.stride(2);
  c.src_channel = src.stride(3);
  c.src_tap = src.stride(4);
  c.dst_idx = index(dst_idx);
  c.step_idx = index(step_idx);
  c.elem_size = dst.scalar_type() == at::kBFloat16 ? 2 : 4;
  c.layers = static_cast<int32_t>(dst.size(0));
  c.reqs = static_cast<int32_t>(reqs);
  c.dim = static_cast<int32_t>(dst.size(2));
  c.taps = static_cast<int32_t>(km1);
  c.src_rows = static_cast<int32_t>(src.size(1));
  c.src_steps = static_cast<int32_t>(src.size(2));
  c.dst_slots = static_cast<int32_t>(dst.size(1));
  if (!bypass_exec()) check_abi(pla_b200_kda_conv_scatter(&c, stream_of(dst)), "conv_window_scatter");
}

}  // namespace
}  // namespace pla_ops

TORCH_LIBRARY_FRAGMENT(pla_b200, m) {
  m.def(
      "kda_ring_verify(Tensor x_q, Tensor x_k, Tensor x_v, Tensor g, Tensor beta, Tensor w_q, Tensor w_k, Tensor w_v, "
      "Tensor cs_q, Tensor cs_k, Tensor cs_v, Tensor A_log, Tensor dt_bias, Tensor h0, Tensor(a!) out, "
      "Tensor(b!) ic_q, Tensor(c!) ic_k, Tensor(d!) ic_v, Tensor(e!) ring_rawv, Tensor(f!) ring_rawk, "
      "Tensor(g!) ring_g, Tensor(h!) ring_beta, Tensor slot_idx, Tensor scratch_idx, Tensor cu_seqlens, float scale, "
      "float? lower_bound, Tensor? onorm_gate, Tensor? onorm_weight, float? onorm_eps, Tensor(i!)? status) -> ()",
      &pla_ops::ring_verify);
  m.def(
      "kda_fold_all_layers(Tensor(a!) h0, Tensor rawv, Tensor rawk, Tensor gk, Tensor beta, Tensor slot_idx, "
      "Tensor accept_lens, Tensor? track_idx, Tensor? track_step, int num_k_heads, int null_block_id, "
      "Tensor(b!)? status) -> ()",
      &pla_ops::fold_all_layers);
  m.def("kda_conv_window_scatter(Tensor(a!) dst, Tensor src, Tensor dst_idx, Tensor step_idx) -> ()",
        &pla_ops::conv_window_scatter);
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
