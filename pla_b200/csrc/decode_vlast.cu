// v-last GDN decode (one token per request) for sm_100a.
//
// State S in R^{K x V}, V contiguous (src/decode/v-last/fused_sigmoid_gating_bigbatch_kernel.cuh:592-857):
//   S <- S * gamma;  delta[v] = sum_k S[k][v] kn[k];  v' = (v - delta) * beta
//   S[k][v] += kn[k] v'[v];  o[v] = sum_k S[k][v] qn[k]
// The reduction runs over rows, so a CTA owns one whole (slot, hv) tile
// (64 KiB, contiguous): four 16 KiB bulk copies land it in shared memory, each
// on its own mbarrier so the first pass starts as soon as the first quarter
// is in. Thread (warp w, lane l) owns rows [16w, 16w+16) x columns [4l, 4l+4):
// column sums are accumulated in registers, combined across the 8 warps
// through shared memory (no shuffles), and the tile is written back with bulk
// stores, again per quarter.
#include "common.cuh"

namespace pla {
namespace {

constexpr int D = 128;
constexpr int TILE = D * D;
constexpr int NT = 256;
constexpr int NW = NT / 32;
constexpr int ROWS_PER_WARP = D / NW;  // 16
constexpr int QUARTERS = 4;            // tile quarters, 32 rows each = 2 warps
constexpr uint32_t kQuarterBytes = TILE * 4 / QUARTERS;

struct VlastSmem {
  static constexpr int kState = 0;
  static constexpr int kQ = kState + TILE * 4;
  static constexpr int kK = kQ + D * 4;
  static constexpr int kRed = kK + D * 4;            // [NW][128] partial sums
  static constexpr int kBar = kRed + NW * D * 4;
  static constexpr int kBytes = kBar + 8 * QUARTERS;
};

template <typename act_t>
__global__ void __launch_bounds__(NT) vlast_kernel(const pla_b200_vlast_args p) {
  extern __shared__ __align__(128) unsigned char smem[];
  float* s_state = reinterpret_cast<float*>(smem + VlastSmem::kState);
  float* s_q = reinterpret_cast<float*>(smem + VlastSmem::kQ);
  float* s_k = reinterpret_cast<float*>(smem + VlastSmem::kK);
  float* s_red = reinterpret_cast<float*>(smem + VlastSmem::kRed);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + VlastSmem::kBar);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int HV = p.HV, H = p.H;
  const int hv = blockIdx.x % HV;
  const int n = blockIdx.x / HV;
  const int h = hv / (HV / H);

  int64_t tok = n;
  if (p.cu_seqlens != nullptr) {
    const int bos = p.cu_seqlens[n], eos = p.cu_seqlens[n + 1];
    if (eos - bos != 1) {  // the op handles exactly one token per request
      if (bos < 0 || eos < bos || eos - bos > 1) {
        if (tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_BAD_INTERVAL);
      }
      return;
    }
    tok = bos;
  }
  const int slot = p.slot_indices[n];
  if (slot < 0) return;  // padded request: output row left as the caller had it
  if (p.num_slots > 0 && slot >= p.num_slots) {
    if (tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_BAD_SLOT);
    return;
  }
  float* g_tile = p.state + (static_cast<int64_t>(slot) * HV + hv) * TILE;

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < QUARTERS; ++i) mbar_init(&bars[i], 1);
    fence_mbar_init();
#pragma unroll
    for (int i = 0; i < QUARTERS; ++i) {
      mbar_expect_tx(&bars[i], kQuarterBytes);
      bulk_load(s_state + i * (TILE / QUARTERS), g_tile + i * (TILE / QUARTERS), kQuarterBytes, &bars[i]);
    }
  }

  // ---- token parameters ----
  const act_t* gq = static_cast<const act_t*>(p.q) + (tok * H + h) * D;
  const act_t* gk = static_cast<const act_t*>(p.k) + (tok * H + h) * D;
  if (warp < 2) {
    float4 x = load4((warp == 0 ? gq : gk) + lane * 4);
    float r = (warp == 0) ? p.scale : 1.0f;
    if (p.use_qk_l2norm) r *= rsqrtf(warp_sum(dot4(x, x)) + 1e-6f);
    reinterpret_cast<float4*>(warp == 0 ? s_q : s_k)[lane] = make_float4(x.x * r, x.y * r, x.z * r, x.w * r);
  }
  const float A_log = load_any(p.A_log, p.A_log_dtype, hv);
  const float xg = to_f32(static_cast<const act_t*>(p.a)[tok * HV + hv]) +
                   to_f32(static_cast<const act_t*>(p.dt_bias)[hv]);
  const float gamma = fast_exp(log_decay(xg, A_log, PLA_B200_GATE_SOFTPLUS, p.softplus_beta, p.softplus_threshold, 0.0f));
  const float beta = sigmoidf_fast(to_f32(static_cast<const act_t*>(p.b)[tok * HV + hv]));
  const float4 vv = load4(static_cast<const act_t*>(p.v) + (tok * HV + hv) * D + lane * 4);
  __syncthreads();  // s_q / s_k ready, mbarriers initialised for everyone

  // Each warp waits (bounded) only for the quarter holding its rows. A timeout
  // is made CTA-uniform at the next barrier so nobody is left behind at it.
  const int q_idx = warp / (NW / QUARTERS);
  const bool landed = mbar_wait(&bars[q_idx], 0);

  // ---- pass 1: decay + column sums of S*k over this warp's 16 rows ----
  float4 st[ROWS_PER_WARP];
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const int krow0 = warp * ROWS_PER_WARP;
#pragma unroll
  for (int r = 0; r < ROWS_PER_WARP; ++r) {
    float4 s = landed ? reinterpret_cast<const float4*>(s_state + (krow0 + r) * D)[lane]
                      : make_float4(0.f, 0.f, 0.f, 0.f);
    s.x *= gamma; s.y *= gamma; s.z *= gamma; s.w *= gamma;
    const float kk = s_k[krow0 + r];
    acc.x += s.x * kk; acc.y += s.y * kk; acc.z += s.z * kk; acc.w += s.w * kk;
    st[r] = s;
  }
  reinterpret_cast<float4*>(s_red + warp * D)[lane] = acc;
  if (__syncthreads_or(!landed)) {
    if (tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_WAIT_TIMEOUT);
    // let every copy land (bounded) before shared memory is released; nothing is stored
    for (int i = 0; i < QUARTERS; ++i) (void)mbar_wait(&bars[i], 0);
    return;
  }
  float4 delta = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int w = 0; w < NW; ++w) {
    const float4 x = reinterpret_cast<const float4*>(s_red + w * D)[lane];
    delta.x += x.x; delta.y += x.y; delta.z += x.z; delta.w += x.w;
  }
  const float4 vn = make_float4((vv.x - delta.x) * beta, (vv.y - delta.y) * beta, (vv.z - delta.z) * beta,
                                (vv.w - delta.w) * beta);
  __syncthreads();  // s_red is reused below

  // ---- pass 2: rank-1 update, column sums of S*q, write the tile back in place ----
  acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int r = 0; r < ROWS_PER_WARP; ++r) {
    const float kk = s_k[krow0 + r], qq = s_q[krow0 + r];
    float4 s = st[r];
    s.x += kk * vn.x; s.y += kk * vn.y; s.z += kk * vn.z; s.w += kk * vn.w;
    acc.x += s.x * qq; acc.y += s.y * qq; acc.z += s.z * qq; acc.w += s.w * qq;
    reinterpret_cast<float4*>(s_state + (krow0 + r) * D)[lane] = s;
  }
  reinterpret_cast<float4*>(s_red + warp * D)[lane] = acc;
  fence_async_smem();
  __syncthreads();
  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < QUARTERS; ++i)
      bulk_store(g_tile + i * (TILE / QUARTERS), s_state + i * (TILE / QUARTERS), kQuarterBytes);
    bulk_commit();
  }
  if (tid < D) {
    float o = 0.0f;
#pragma unroll
    for (int w = 0; w < NW; ++w) o += s_red[w * D + tid];
    static_cast<act_t*>(p.o)[(tok * HV + hv) * D + tid] = from_f32<act_t>(o);
  }
  if (tid == 0) bulk_wait_read<0>();
}

template <typename act_t>
int launch(const pla_b200_vlast_args& a, cudaStream_t stream) {
  auto kern = vlast_kernel<act_t>;
  static DeviceOnce configured;
  int dev = 0;
  PLA_CUDA_OK(cudaGetDevice(&dev));
  if (configured.needed(dev)) {
    PLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, VlastSmem::kBytes));
    configured.mark(dev);
  }
  const int64_t ctas = static_cast<int64_t>(a.B) * a.HV;
  PLA_REQUIRE(ctas < (1ll << 31), PLA_B200_E_TOO_LARGE, "B*HV exceeds the grid limit");
  kern<<<static_cast<unsigned>(ctas), NT, VlastSmem::kBytes, stream>>>(a);
  PLA_CUDA_OK(cudaGetLastError());
  return PLA_B200_OK;
}

}  // namespace
}  // namespace pla

extern "C" int pla_b200_decode_vlast(const pla_b200_vlast_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  pla_b200_vlast_args a = *args;
  default_status(a);
  PLA_REQUIRE(a.B >= 0, PLA_B200_E_INVALID, "B must be non-negative");
  if (a.B == 0) return PLA_B200_OK;
  PLA_REQUIRE(a.H > 0 && a.HV >= a.H && a.HV % a.H == 0, PLA_B200_E_INVALID,
              "HV must be a positive multiple of H, got H=%d, HV=%d", a.H, a.HV);
  PLA_REQUIRE(a.q && a.k && a.v && a.a && a.b && a.o && a.A_log && a.dt_bias && a.state && a.slot_indices,
              PLA_B200_E_INVALID, "q, k, v, a, b, o, A_log, dt_bias, state and slot indices are required");
  PLA_REQUIRE(a.act_dtype == PLA_B200_BF16 || a.act_dtype == PLA_B200_F16, PLA_B200_E_INVALID,
              "activation dtype must be bf16 or fp16");
  PLA_REQUIRE(aligned16(a.state), PLA_B200_E_ALIGN, "state pool must be 16-byte aligned");
  PLA_REQUIRE((reinterpret_cast<uintptr_t>(a.q) & 7) == 0 && (reinterpret_cast<uintptr_t>(a.k) & 7) == 0 &&
                  (reinterpret_cast<uintptr_t>(a.v) & 7) == 0,
              PLA_B200_E_ALIGN, "q/k/v must be 8-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return a.act_dtype == PLA_B200_BF16 ? launch<__nv_bfloat16>(a, s) : launch<__half>(a, s);
}
