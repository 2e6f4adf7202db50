// Fused KDA decode step: conv + SiLU with in-place conv-state shift, then the single-token KDA recurrence
// of the streaming k-last kernel on the packed conv outputs, then the optional gated output RMSNorm
// (src/decode/k-last/fused_kda_decode_mega_kernel.cuh:36-79; reference math
// scripts/decode/kda_fusion/compare_kda_decode_fusion.py:252-308).
// Three launches on one stream: the state traffic (128 KiB per request and head) is all in the second one.
#include "common.cuh"
#include "decode_klast.h"

namespace pla {
namespace {

constexpr int D = 128;

__device__ __forceinline__ float silu_f(float x) { return x * sigmoidf_fast(x); }

// One thread per (request, channel): y = silu(w . [t0, t1, t2, x] + bias) -> mixed; conv state <- [t1, t2, x].
template <typename act_t>
__global__ void __launch_bounds__(256) kda_mega_conv_kernel(const pla_b200_kda_mega_args p) {
  const int b = blockIdx.y;
  const int dim = p.H * D;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;   // channel in [0, 3*dim)
  if (c >= 3 * dim) return;
  const int slot = p.state_indices[b];
  if (slot < 0) return;                                  // padding row: the decode kernel zeroes its output
  if (slot >= p.slots) {
    if (p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_BAD_SLOT);
    return;
  }
  const int seg = c / dim, ch = c - seg * dim;
  act_t* cs = static_cast<act_t*>(p.conv_state) + static_cast<int64_t>(slot) * p.conv_strides.slot +
              static_cast<int64_t>(c) * p.conv_strides.channel;
  const act_t t0 = cs[0], t1 = cs[p.conv_strides.tap], t2 = cs[2 * p.conv_strides.tap];
  const act_t xn = static_cast<const act_t*>(p.x)[static_cast<int64_t>(b) * p.x_row_stride + c];
  const float* w = p.weight + static_cast<int64_t>(seg) * 4 * dim + ch;
  float acc = p.bias != nullptr ? p.bias[c] : 0.0f;
  acc = fmaf(w[0], to_f32(t0), acc);
  acc = fmaf(w[dim], to_f32(t1), acc);
  acc = fmaf(w[2 * dim], to_f32(t2), acc);
  acc = fmaf(w[3 * dim], to_f32(xn), acc);
  static_cast<act_t*>(p.mixed)[static_cast<int64_t>(b) * 3 * dim + c] = from_f32<act_t>(silu_f(acc));
  cs[0] = t1;                                            // bit-exact shift of the history
  cs[p.conv_strides.tap] = t2;
  cs[2 * p.conv_strides.tap] = xn;
}

// Gated RMSNorm of the staged fp32 outputs: one warp per (request, head), four channels per lane.
template <typename act_t>
__global__ void __launch_bounds__(128) kda_mega_norm_kernel(const pla_b200_kda_mega_args p) {
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= p.B * p.H) return;
  const int b = item / p.H, h = item % p.H;
  const int slot = p.state_indices[b];
  if (slot < 0 || slot >= p.slots) return;               // output row already zero
  const int64_t e = (static_cast<int64_t>(b) * p.H + h) * D + lane * 4;
  const float4 o = *reinterpret_cast<const float4*>(p.out_f32 + e);
  const float r = rsqrtf(warp_sum(o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w) * (1.0f / D) + p.norm_eps);
  const float4 w = reinterpret_cast<const float4*>(p.norm_weight)[lane];
  const act_t* g = static_cast<const act_t*>(p.output_gate) + static_cast<int64_t>(b) * p.gate_row_stride + h * D + lane * 4;
  act_t* dst = static_cast<act_t*>(p.out) + e;
  dst[0] = from_f32<act_t>(o.x * r * w.x * sigmoidf_fast(to_f32(g[0])));
  dst[1] = from_f32<act_t>(o.y * r * w.y * sigmoidf_fast(to_f32(g[1])));
  dst[2] = from_f32<act_t>(o.z * r * w.z * sigmoidf_fast(to_f32(g[2])));
  dst[3] = from_f32<act_t>(o.w * r * w.w * sigmoidf_fast(to_f32(g[3])));
}

template <typename act_t>
int launch_mega(const pla_b200_kda_mega_args& a, cudaStream_t s) {
  const int dim = a.H * D;
  kda_mega_conv_kernel<act_t><<<dim3((3 * dim + 255) / 256, a.B), 256, 0, s>>>(a);
  PLA_CUDA_OK(cudaGetLastError());

  pla_b200_klast_args k{};
  const act_t* mixed = static_cast<const act_t*>(a.mixed);
  k.q = mixed;
  k.k = mixed + dim;
  k.v = mixed + 2 * dim;
  k.q_tok_stride = k.k_tok_stride = k.v_tok_stride = 3 * static_cast<int64_t>(dim);
  k.a = a.raw_g;
  k.a_tok_stride = dim;
  k.b = a.raw_beta;
  k.b_tok_stride = a.beta_row_stride;
  k.A_log = a.A_log;
  k.A_log_dtype = PLA_B200_F32;
  k.dt_bias = a.dt_bias;
  k.dt_bias_dtype = PLA_B200_F32;
  k.act_dtype = a.act_dtype;
  k.state = a.state;
  k.state_slot_stride = a.state_slot_stride;
  k.num_slots = a.slots;
  k.state_dtype = PLA_B200_F32;
  k.slot_indices = a.state_indices;
  k.o = a.out;
  k.o_f32 = a.output_gate != nullptr ? a.out_f32 : nullptr;
  k.B = a.B;
  k.t_max = 1;
  k.H = a.H;
  k.HV = a.H;
  k.scale = a.scale;
  k.softplus_beta = 1.0f;
  k.softplus_threshold = 20.0f;
  k.lower_bound = a.lower_bound;
  k.gate = a.gate;
  k.is_kda = 1;
  k.use_qk_l2norm = 1;
  k.pad = PLA_B200_PAD_SGLANG;                           // slot < 0 is padding, slot 0 is real
  k.rows_per_cta = 16;                                   // the streaming kernel
  k.status = a.status;
  PLA_REQUIRE(klast_stream_eligible(k), PLA_B200_E_ALIGN,
              "fused KDA decode needs 8-byte aligned raw_g rows and 4-byte aligned out");
  const int rc = launch_klast_stream(k, s);
  if (rc != PLA_B200_OK) return rc;
  if (a.output_gate != nullptr) {
    kda_mega_norm_kernel<act_t><<<(a.B * a.H + 3) / 4, 128, 0, s>>>(a);
    PLA_CUDA_OK(cudaGetLastError());
  }
  return PLA_B200_OK;
}

}  // namespace
}  // namespace pla

extern "C" int pla_b200_kda_decode_mega(const pla_b200_kda_mega_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  const pla_b200_kda_mega_args& a = *args;
  PLA_REQUIRE(a.B >= 0 && a.H > 0 && a.slots > 0, PLA_B200_E_INVALID, "B >= 0, H > 0, slots > 0 required");
  if (a.B == 0) return PLA_B200_OK;
  PLA_REQUIRE(a.x && a.weight && a.conv_state && a.raw_g && a.raw_beta && a.A_log && a.dt_bias && a.state_indices &&
                  a.state && a.out && a.mixed,
              PLA_B200_E_INVALID, "fused KDA decode: a required pointer is NULL");
  PLA_REQUIRE(a.act_dtype == PLA_B200_BF16 || a.act_dtype == PLA_B200_F16, PLA_B200_E_INVALID,
              "activation dtype must be bf16 or fp16");
  PLA_REQUIRE((a.output_gate != nullptr) == (a.norm_weight != nullptr), PLA_B200_E_INVALID,
              "output_gate and norm_weight must be supplied together");
  PLA_REQUIRE(a.output_gate == nullptr || (a.out_f32 != nullptr && aligned16(a.out_f32) && aligned16(a.norm_weight) &&
                                           a.norm_eps >= 0.0f),
              PLA_B200_E_INVALID, "the output norm needs eps >= 0 and 16-byte aligned staging and weight");
  PLA_REQUIRE(aligned16(a.mixed) && aligned16(a.state) && a.state_slot_stride % 4 == 0 &&
                  a.state_slot_stride >= static_cast<int64_t>(a.H) * 16384,
              PLA_B200_E_ALIGN, "scratch and state must be 16-byte aligned; slot pitch must cover H*128*128");
  PLA_REQUIRE(a.gate == PLA_B200_GATE_SOFTPLUS || (a.gate == PLA_B200_GATE_SAFE && a.lower_bound < 0.0f),
              PLA_B200_E_INVALID, "the safe gate needs lower_bound < 0");
  PLA_REQUIRE(a.B <= 65535, PLA_B200_E_TOO_LARGE, "batch exceeds the grid limit");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return a.act_dtype == PLA_B200_BF16 ? launch_mega<__nv_bfloat16>(a, s) : launch_mega<__half>(a, s);
}
