// Whole-tile kernel for single-token k-last decode.
//
// One CTA per (request, value head), 256 threads, the 64 KiB tile S[v][k] in shared memory: four 16 KiB bulk
// copies, each on its own mbarrier, so the first warps start as soon as the first quarter is in. Thread
// (warp w, lane l) owns rows 16w + 4(l / 8) .. +3 and the 16 key channels 16 (l % 8) .. +15 of them, 64
// state values that stay in registers across both passes, next to the matching 16 channels of the token's
// k, q and decay. Row sums therefore start as in-register sums over 16 channels; the eight partial sums
// of a row are combined through shared memory (no shuffles). The four 16-byte granules of a row strip are
// visited in an order rotated by (l % 8) / 2, which puts the eight lanes of a quarter warp on eight
// different banks. The tile is written back in place, per quarter, with bulk stores.
//
// Math: src/decode/k-last/fused_sigmoid_gating_k_last_kernel.cuh:396-473, :561-605.
#include "common.cuh"
#include "decode_klast.h"

namespace pla {
namespace {

constexpr int D = 128;
constexpr int TILE = D * D;
constexpr int NT = 256;
constexpr int NW = NT / 32;
constexpr int QUARTERS = 4;
constexpr uint32_t kQuarterBytes = TILE * 4 / QUARTERS;

struct RowsSmem {
  alignas(128) float tile[TILE];
  alignas(16) float q[D];
  alignas(16) float k[D];
  alignas(16) float gam[D];
  alignas(16) float red[D][8];          // [row][column strip] partial row sums
  alignas(8) uint64_t bar[QUARTERS];
};

template <typename act_t, bool IS_KDA>
__global__ void __launch_bounds__(NT, 2) klast_rows_kernel(const pla_b200_klast_args p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  RowsSmem& sh = *reinterpret_cast<RowsSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hv = blockIdx.x % p.HV;
  const int n = blockIdx.x / p.HV;
  const int h = hv / (p.HV / p.H);

  // the slot index and the interval are independent loads: issue both before either is looked at
  const int slot = p.slot_indices[n];
  int64_t tok = n;
  if (p.cu_seqlens != nullptr) {
    const int64_t bos = p.cu_seqlens[n], eos = p.cu_seqlens[n + 1];
    if (eos == bos) return;  // empty request
    if (bos < 0 || eos < bos || eos - bos > 1) {
      if (tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_BAD_INTERVAL);
      return;
    }
    tok = bos;
  }
  act_t* orow = static_cast<act_t*>(p.o) + (tok * p.HV + hv) * D;
  const bool pad = (p.pad == PLA_B200_PAD_SGLANG) ? (slot < 0) : (slot <= 0);
  const bool oob = !pad && p.num_slots > 0 && slot >= p.num_slots;
  if (pad || oob) {
    if (oob && tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_BAD_SLOT);
    if (tid < D) orow[tid] = from_f32<act_t>(0.0f);
    return;
  }
  float* g_tile = static_cast<float*>(p.state) + static_cast<int64_t>(slot) * p.state_slot_stride +
                  static_cast<int64_t>(hv) * TILE;

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < QUARTERS; ++i) mbar_init(&sh.bar[i], 1);
    fence_mbar_init();
#pragma unroll
    for (int i = 0; i < QUARTERS; ++i) {
      mbar_expect_tx(&sh.bar[i], kQuarterBytes);
      bulk_load(sh.tile + i * (TILE / QUARTERS), g_tile + i * (TILE / QUARTERS), kQuarterBytes, &sh.bar[i]);
    }
  }

  // ---- the token's vectors: warp 0 forms q, warp 1 k, warp 2 the per-channel decay; four channels per lane ----
  if (warp < 2) {
    const act_t* src = static_cast<const act_t*>(warp == 0 ? p.q : p.k) + tok * (warp == 0 ? p.q_tok_stride : p.k_tok_stride) +
                       h * D + lane * 4;
    const float4 x = load4(src);
    float r = warp == 0 ? p.scale : 1.0f;
    if (p.use_qk_l2norm) r *= rsqrtf(warp_sum(dot4(x, x)) + 1e-6f);
    reinterpret_cast<float4*>(warp == 0 ? sh.q : sh.k)[lane] = make_float4(x.x * r, x.y * r, x.z * r, x.w * r);
  } else if (IS_KDA && warp == 2) {
    const float4 x = load4(static_cast<const act_t*>(p.a) + tok * p.a_tok_stride + hv * D + lane * 4);
    const float A_log = load_any(p.A_log, p.A_log_dtype, hv);
    const int64_t c = static_cast<int64_t>(hv) * D + lane * 4;
    float4 g;
    g.x = fast_exp(log_decay(x.x + load_any(p.dt_bias, p.dt_bias_dtype, c + 0), A_log, p.gate, p.softplus_beta,
                           p.softplus_threshold, p.lower_bound));
    g.y = fast_exp(log_decay(x.y + load_any(p.dt_bias, p.dt_bias_dtype, c + 1), A_log, p.gate, p.softplus_beta,
                           p.softplus_threshold, p.lower_bound));
    g.z = fast_exp(log_decay(x.z + load_any(p.dt_bias, p.dt_bias_dtype, c + 2), A_log, p.gate, p.softplus_beta,
                           p.softplus_threshold, p.lower_bound));
    g.w = fast_exp(log_decay(x.w + load_any(p.dt_bias, p.dt_bias_dtype, c + 3), A_log, p.gate, p.softplus_beta,
                           p.softplus_threshold, p.lower_bound));
    reinterpret_cast<float4*>(sh.gam)[lane] = g;
  }
  float gs = 1.0f;
  if constexpr (!IS_KDA) {
    const float x = to_f32(static_cast<const act_t*>(p.a)[tok * p.a_tok_stride + hv]) +
                    load_any(p.dt_bias, p.dt_bias_dtype, hv);
    gs = fast_exp(log_decay(x, load_any(p.A_log, p.A_log_dtype, hv), p.gate, p.softplus_beta, p.softplus_threshold,
                          p.lower_bound));
  }
  const float beta = sigmoidf_fast(to_f32(static_cast<const act_t*>(p.b)[tok * p.b_tok_stride + hv]));
  __syncthreads();  // q / k / decay vectors complete, mbarriers initialised for everyone

  // ---- this thread's strip: rows row0 .. row0+3, channels 16 b .. 16 b + 15 ----
  const int b = lane & 7;
  const int row0 = warp * 16 + (lane >> 3) * 4;
  const int rot = b >> 1;
  float4 k4[4], q4[4], g4[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int gj = 4 * b + ((j + rot) & 3);     // granule visited j-th
    k4[j] = reinterpret_cast<const float4*>(sh.k)[gj];
    q4[j] = reinterpret_cast<const float4*>(sh.q)[gj];
    if constexpr (IS_KDA) g4[j] = reinterpret_cast<const float4*>(sh.gam)[gj];
  }
  const float4 v4 = load4(static_cast<const act_t*>(p.v) + tok * p.v_tok_stride + hv * D + row0);

  // Each warp waits (bounded) only for the quarter holding its rows; a timeout is made CTA-uniform at the
  // next barrier so nobody is left behind at it.
  const bool landed = mbar_wait(&sh.bar[warp / (NW / QUARTERS)], 0);

  // ---- pass 1: decay, partial sums of S k over the strip ----
  float4 st[4][4];
  float pr[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    pr[r] = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gj = 4 * b + ((j + rot) & 3);
      float4 s = landed ? reinterpret_cast<const float4*>(sh.tile + (row0 + r) * D)[gj] : make_float4(0.f, 0.f, 0.f, 0.f);
      if constexpr (IS_KDA) {
        s.x *= g4[j].x; s.y *= g4[j].y; s.z *= g4[j].z; s.w *= g4[j].w;
      } else {
        s.x *= gs; s.y *= gs; s.z *= gs; s.w *= gs;
      }
      pr[r] += dot4(s, k4[j]);
      st[r][j] = s;
    }
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) sh.red[row0 + r][b] = pr[r];
  if (__syncthreads_or(!landed)) {
    if (tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_WAIT_TIMEOUT);
    // let every copy land (bounded) before shared memory is released; nothing is stored
    for (int i = 0; i < QUARTERS; ++i) (void)mbar_wait(&sh.bar[i], 0);
    return;
  }
  float dsum[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const float4 x0 = *reinterpret_cast<const float4*>(&sh.red[row0 + r][0]);
    const float4 x1 = *reinterpret_cast<const float4*>(&sh.red[row0 + r][4]);
    dsum[r] = ((x0.x + x0.y) + (x0.z + x0.w)) + ((x1.x + x1.y) + (x1.z + x1.w));
  }
  const float vn[4] = {(v4.x - dsum[0]) * beta, (v4.y - dsum[1]) * beta, (v4.z - dsum[2]) * beta,
                       (v4.w - dsum[3]) * beta};
  __syncthreads();  // red is reused below

  // ---- pass 2: rank-1 update, partial sums of S q, the strip back to shared memory ----
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    pr[r] = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gj = 4 * b + ((j + rot) & 3);
      float4 s = st[r][j];
      s.x = fmaf(k4[j].x, vn[r], s.x);
      s.y = fmaf(k4[j].y, vn[r], s.y);
      s.z = fmaf(k4[j].z, vn[r], s.z);
      s.w = fmaf(k4[j].w, vn[r], s.w);
      pr[r] += dot4(s, q4[j]);
      reinterpret_cast<float4*>(sh.tile + (row0 + r) * D)[gj] = s;
    }
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) sh.red[row0 + r][b] = pr[r];
  fence_async_smem();   // in-place updates -> visible to the bulk-copy engine
  __syncthreads();
  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < QUARTERS; ++i)
      bulk_store(g_tile + i * (TILE / QUARTERS), sh.tile + i * (TILE / QUARTERS), kQuarterBytes);
    bulk_commit();
  }
  if (tid < D) {
    const float4 x0 = *reinterpret_cast<const float4*>(&sh.red[tid][0]);
    const float4 x1 = *reinterpret_cast<const float4*>(&sh.red[tid][4]);
    const float o = ((x0.x + x0.y) + (x0.z + x0.w)) + ((x1.x + x1.y) + (x1.z + x1.w));
    if (p.o_f32 != nullptr) p.o_f32[(tok * p.HV + hv) * D + tid] = o;
    else orow[tid] = from_f32<act_t>(o);
  }
  if (tid == 0) bulk_wait_read<0>();
}

template <typename act_t, bool IS_KDA>
int launch_rows(const pla_b200_klast_args& a, cudaStream_t stream) {
  auto kern = klast_rows_kernel<act_t, IS_KDA>;
  static DeviceOnce configured;
  int dev = 0;
  PLA_CUDA_OK(cudaGetDevice(&dev));
  if (configured.needed(dev)) {
    PLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, sizeof(RowsSmem)));
    configured.mark(dev);
  }
  const int64_t ctas = static_cast<int64_t>(a.B) * a.HV;
  PLA_REQUIRE(ctas < (1ll << 31), PLA_B200_E_TOO_LARGE, "B*HV exceeds the grid limit");
  kern<<<static_cast<unsigned>(ctas), NT, sizeof(RowsSmem), stream>>>(a);
  PLA_CUDA_OK(cudaGetLastError());
  return PLA_B200_OK;
}

}  // namespace

int launch_klast_rows(const pla_b200_klast_args& a, cudaStream_t stream) {
  if (a.act_dtype == PLA_B200_BF16)
    return a.is_kda ? launch_rows<__nv_bfloat16, true>(a, stream) : launch_rows<__nv_bfloat16, false>(a, stream);
  return a.is_kda ? launch_rows<__half, true>(a, stream) : launch_rows<__half, false>(a, stream);
}

}  // namespace pla
