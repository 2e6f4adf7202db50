// Fused KDA decode step in ONE kernel: causal conv (width 4) + SiLU with the in-place shift of the 3-tap conv
// state, L2 norms, per-channel gate, the single-token KDA recurrence on the fp32 k-last state in place, and the
// optional gated output RMSNorm (src/decode/k-last/fused_kda_decode_mega_kernel.cuh:148-732, grid (1, H, B) at
// :58-72; reference math scripts/decode/kda_fusion/compare_kda_decode_fusion.py:252-308).
//
// One CTA per (request, head), 256 threads. The first state rows are requested before anything else; threads
// 0..127 then form the head's q and k channels (conv + SiLU, history shifted), the decay and the norm sums,
// threads 128..255 the v channels; nothing of that leaves the SM. The 64 KiB state tile is streamed through
// registers, never shared memory: warp w owns rows 16 w .. 16 w + 15, eight lanes per row, four rows at a time
// with the next four in flight; each row is decayed, corrected and written back where it came from, and its
// output value stays in shared memory for the norm over the head's 128 values. No scratch buffers.
#include "common.cuh"

namespace pla {
namespace {

constexpr int D = 128;
constexpr int TILE = D * D;
constexpr int MT = 256;

__device__ __forceinline__ float silu_f(float x) { return x * sigmoidf_fast(x); }

struct MegaSmem {
  alignas(16) float q[D];
  alignas(16) float k[D];
  alignas(16) float gam[D];
  float v[D];
  float o[D];
  float part[3][4];
  float beta;
};

template <typename act_t>
__global__ void __launch_bounds__(MT, 3) kda_mega_fused_kernel(const pla_b200_kda_mega_args p) {
  __shared__ MegaSmem sh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x % p.H, b = blockIdx.x / p.H;
  const int dim = p.H * D;
  const int slot = p.state_indices[b];
  act_t* outp = static_cast<act_t*>(p.out) + (static_cast<int64_t>(b) * p.H + h) * D;
  if (slot < 0 || slot >= p.slots) {       // padding row (or a slot outside the pool): zero output, nothing else
    if (slot >= p.slots && tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_BAD_SLOT);
    if (tid < D / 2) reinterpret_cast<uint32_t*>(outp)[tid] = 0u;
    return;
  }

  // ---- the first four state rows of this warp, requested before the conv work
  const int j8 = lane & 7;
  float4* srow0 = reinterpret_cast<float4*>(p.state + static_cast<int64_t>(slot) * p.state_slot_stride +
                                            static_cast<int64_t>(h) * TILE) +
                  (warp * 16 + (lane >> 3)) * (D / 4) + j8;   // row pass ps: + ps * 4 rows; piece i: + i * 8
  float4 st[2][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) st[0][i] = srow0[i * 8];
  // the other twelve (row pass, 128-byte line) pairs of these rows go to L2 meanwhile, one per lane of the row's eight
  for (int idx = j8; idx < 12; idx += 8) prefetch_l2(srow0 - j8 + (1 + idx / 4) * 4 * (D / 4) + (idx % 4) * 8);

  // ---- conv + SiLU of one channel, history shifted in place (bit-exact copies)
  const int c = tid & (D - 1);
  const int ch = h * D + c;
  auto conv = [&](int seg) -> float {
    const int cc = seg * dim + ch;
    act_t* cs = static_cast<act_t*>(p.conv_state) + static_cast<int64_t>(slot) * p.conv_strides.slot +
                static_cast<int64_t>(cc) * p.conv_strides.channel;
    const act_t t0 = cs[0], t1 = cs[p.conv_strides.tap], t2 = cs[2 * p.conv_strides.tap];
    const act_t xn = static_cast<const act_t*>(p.x)[static_cast<int64_t>(b) * p.x_row_stride + cc];
    const float* w = p.weight + static_cast<int64_t>(seg) * 4 * dim + ch;
    float acc = p.bias != nullptr ? p.bias[cc] : 0.0f;
    acc = fmaf(w[0], to_f32(t0), acc);
    acc = fmaf(w[dim], to_f32(t1), acc);
    acc = fmaf(w[2 * dim], to_f32(t2), acc);
    acc = fmaf(w[3 * dim], to_f32(xn), acc);
    cs[0] = t1;
    cs[p.conv_strides.tap] = t2;
    cs[2 * p.conv_strides.tap] = xn;
    return silu_f(acc);
  };
  if (tid < D) {
    const float q = conv(0), k = conv(1);
    const float x = to_f32(static_cast<const act_t*>(p.raw_g)[static_cast<int64_t>(b) * dim + ch]) + p.dt_bias[ch];
    sh.gam[c] = fast_exp(log_decay(x, p.A_log[h], p.gate, 1.0f, 20.0f, p.lower_bound));
    sh.q[c] = q;
    sh.k[c] = k;
    const float sq = warp_sum(q * q), sk = warp_sum(k * k);
    if (lane == 0) {
      sh.part[0][warp] = sq;
      sh.part[1][warp] = sk;
    }
  } else {
    sh.v[c] = conv(2);
    if (c == 0) sh.beta = sigmoidf_fast(to_f32(static_cast<const act_t*>(p.raw_beta)[static_cast<int64_t>(b) * p.beta_row_stride + h]));
  }
  __syncthreads();
  if (tid < D) {   // normalised q (times the scale) and k, in place
    sh.q[c] *= rsqrtf((sh.part[0][0] + sh.part[0][1]) + (sh.part[0][2] + sh.part[0][3]) + 1e-6f) * p.scale;
    sh.k[c] *= rsqrtf((sh.part[1][0] + sh.part[1][1]) + (sh.part[1][2] + sh.part[1][3]) + 1e-6f);
  }
  __syncthreads();
  const float beta = sh.beta;

  // ---- the recurrence, four rows per warp at a time
#pragma unroll
  for (int ps = 0; ps < 4; ++ps) {
    if (ps + 1 < 4) {
#pragma unroll
      for (int i = 0; i < 4; ++i) st[(ps + 1) & 1][i] = srow0[(ps + 1) * 4 * (D / 4) + i * 8];
    }
    const int row = warp * 16 + ps * 4 + (lane >> 3);
    float4 kk[4];
    float d = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 g = reinterpret_cast<const float4*>(sh.gam)[i * 8 + j8];
      kk[i] = reinterpret_cast<const float4*>(sh.k)[i * 8 + j8];
      float4& s4 = st[ps & 1][i];
      s4.x *= g.x; s4.y *= g.y; s4.z *= g.z; s4.w *= g.w;
      d += dot4(s4, kk[i]);
    }
    d += __shfl_xor_sync(0xffffffffu, d, 1);
    d += __shfl_xor_sync(0xffffffffu, d, 2);
    d += __shfl_xor_sync(0xffffffffu, d, 4);
    const float vn = (sh.v[row] - d) * beta;
    float o = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 q4 = reinterpret_cast<const float4*>(sh.q)[i * 8 + j8];
      float4& s4 = st[ps & 1][i];
      s4.x = fmaf(vn, kk[i].x, s4.x);
      s4.y = fmaf(vn, kk[i].y, s4.y);
      s4.z = fmaf(vn, kk[i].z, s4.z);
      s4.w = fmaf(vn, kk[i].w, s4.w);
      o += dot4(s4, q4);
      srow0[ps * 4 * (D / 4) + i * 8] = s4;
    }
    o += __shfl_xor_sync(0xffffffffu, o, 1);
    o += __shfl_xor_sync(0xffffffffu, o, 2);
    o += __shfl_xor_sync(0xffffffffu, o, 4);
    if (j8 == 0) sh.o[row] = o;
  }
  __syncthreads();

  // ---- output row, with the gated RMSNorm over the head's 128 values when asked for
  if (tid < D) {
    float o = sh.o[c];
    if (p.output_gate != nullptr) {
      const float ss = warp_sum(o * o);
      if (lane == 0) sh.part[2][warp] = ss;
    }
    if (p.output_gate != nullptr) {
      asm volatile("bar.sync 1, 128;" ::: "memory");   // threads 0..127 only
      const float r = rsqrtf(((sh.part[2][0] + sh.part[2][1]) + (sh.part[2][2] + sh.part[2][3])) * (1.0f / D) + p.norm_eps);
      const float gate = to_f32(static_cast<const act_t*>(p.output_gate)[static_cast<int64_t>(b) * p.gate_row_stride + ch]);
      o = o * r * p.norm_weight[c] * sigmoidf_fast(gate);
    }
    outp[c] = from_f32<act_t>(o);
  }
}

template <typename act_t>
int launch_mega(const pla_b200_kda_mega_args& a, cudaStream_t s) {
  const int64_t ctas = static_cast<int64_t>(a.B) * a.H;
  PLA_REQUIRE(ctas < (1ll << 31), PLA_B200_E_TOO_LARGE, "B*H exceeds the grid limit");
  kda_mega_fused_kernel<act_t><<<static_cast<unsigned>(ctas), MT, 0, s>>>(a);
  PLA_CUDA_OK(cudaGetLastError());
  return PLA_B200_OK;
}

}  // namespace
}  // namespace pla

extern "C" int pla_b200_kda_decode_mega(const pla_b200_kda_mega_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  pla_b200_kda_mega_args a = *args;
  default_status(a);
  PLA_REQUIRE(a.B >= 0 && a.H > 0 && a.slots > 0, PLA_B200_E_INVALID, "B >= 0, H > 0, slots > 0 required");
  if (a.B == 0) return PLA_B200_OK;
  PLA_REQUIRE(a.x && a.weight && a.conv_state && a.raw_g && a.raw_beta && a.A_log && a.dt_bias && a.state_indices &&
                  a.state && a.out,
              PLA_B200_E_INVALID, "fused KDA decode: a required pointer is NULL");
  PLA_REQUIRE(a.act_dtype == PLA_B200_BF16 || a.act_dtype == PLA_B200_F16, PLA_B200_E_INVALID,
              "activation dtype must be bf16 or fp16");
  PLA_REQUIRE((a.output_gate != nullptr) == (a.norm_weight != nullptr), PLA_B200_E_INVALID,
              "output_gate and norm_weight must be supplied together");
  PLA_REQUIRE(a.output_gate == nullptr || a.norm_eps >= 0.0f, PLA_B200_E_INVALID, "the output norm needs eps >= 0");
  PLA_REQUIRE(aligned16(a.state) && a.state_slot_stride % 4 == 0 &&
                  a.state_slot_stride >= static_cast<int64_t>(a.H) * 16384,
              PLA_B200_E_ALIGN, "state must be 16-byte aligned; slot pitch must cover H*128*128");
  PLA_REQUIRE((reinterpret_cast<uintptr_t>(a.out) & 3) == 0, PLA_B200_E_ALIGN, "out must be 4-byte aligned");
  PLA_REQUIRE(a.gate == PLA_B200_GATE_SOFTPLUS || (a.gate == PLA_B200_GATE_SAFE && a.lower_bound < 0.0f),
              PLA_B200_E_INVALID, "the safe gate needs lower_bound < 0");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return a.act_dtype == PLA_B200_BF16 ? launch_mega<__nv_bfloat16>(a, s) : launch_mega<__half>(a, s);
}
