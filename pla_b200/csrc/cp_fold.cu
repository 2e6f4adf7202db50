// Context parallelism, fold step: the state entering a rank's token range from the (offset, transition)
// pairs of the ranks before it,  S <- S M_j + B_j  for j = 0 .. rank-1, row by row of the k-last state
// S[v, k] (the composition the reference applies to its intra-card segments,
// src/prefill/flashqla/kernels/prepare_h_cute.cu:59-67). Exact fp32 FMAs: the products are tiny
// (rank-1 steps of 128^3 per head) and the result seeds a whole token range.
#include "common.cuh"

namespace pla {
namespace {

constexpr int D = 128;
constexpr int TILE = D * D;
constexpr int ROWS = 16;                   // state rows per CTA
constexpr int FOLD_THREADS = 256;
constexpr uint32_t kTileBytes = TILE * 4;

struct FoldSmem {
  alignas(128) float m[TILE];              // transition of the current step, [k][k']
  alignas(16) float s[ROWS * D];           // this CTA's rows of the state
  alignas(8) uint64_t bar;
};

__global__ void __launch_bounds__(FOLD_THREADS) cp_fold_kernel(const pla_b200_cp_fold_args p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  FoldSmem& sh = *reinterpret_cast<FoldSmem*>(smem_raw);
  const int tid = threadIdx.x;
  const int rs = blockIdx.x % (D / ROWS);
  const int hv = (blockIdx.x / (D / ROWS)) % p.HV;
  // compose mode: the second half of the grid carries the transition (rows of the identity through the M_j
  // alone), the first half the offset (zero rows through the full pairs)
  const bool transition = p.compose != 0 && blockIdx.x >= static_cast<unsigned>(p.HV) * (D / ROWS);
  const int row0 = rs * ROWS;
  const int col = tid & 127, rg = tid >> 7;   // this thread: column `col` of rows rg*8 .. rg*8+7

  for (int i = tid; i < ROWS * D; i += FOLD_THREADS) {
    float x = 0.0f;
    if (transition) x = (row0 + i / D == i % D) ? 1.0f : 0.0f;
    else if (p.compose == 0 && p.initial_state != nullptr) x = p.initial_state[static_cast<int64_t>(hv) * TILE + row0 * D + i];
    sh.s[i] = x;
  }
  if (tid == 0) {
    mbar_init(&sh.bar, 1);
    fence_mbar_init();
  }
  __syncthreads();

  for (int j = 0; j < p.rank; ++j) {
    const float* pair = p.pairs + (static_cast<int64_t>(j) * p.HV + hv) * 2 * TILE;   // [offset B | transition M]
    if (tid == 0) {
      mbar_expect_tx(&sh.bar, kTileBytes);
      bulk_load(sh.m, pair + TILE, kTileBytes, &sh.bar);
    }
    float acc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[r] = transition ? 0.0f : pair[(row0 + rg * 8 + r) * D + col];   // B rows
    const bool ok = mbar_wait(&sh.bar, j & 1);
    if (__syncthreads_or(!ok)) {
      if (tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_WAIT_TIMEOUT);
      (void)mbar_wait(&sh.bar, j & 1);
      return;
    }
#pragma unroll 4
    for (int k4 = 0; k4 < D / 4; ++k4) {
      const float m0 = sh.m[(4 * k4 + 0) * D + col], m1 = sh.m[(4 * k4 + 1) * D + col];
      const float m2 = sh.m[(4 * k4 + 2) * D + col], m3 = sh.m[(4 * k4 + 3) * D + col];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float4 sv = *reinterpret_cast<const float4*>(&sh.s[(rg * 8 + r) * D + 4 * k4]);   // broadcast
        acc[r] = fmaf(sv.x, m0, fmaf(sv.y, m1, fmaf(sv.z, m2, fmaf(sv.w, m3, acc[r]))));
      }
    }
    __syncthreads();   // every thread has read the old rows and the transition
#pragma unroll
    for (int r = 0; r < 8; ++r) sh.s[(rg * 8 + r) * D + col] = acc[r];
    __syncthreads();
  }
  // plain fold: [HV, 128, 128]; compose: [HV, 2, 128, 128]
  float* dst = p.state_out + (p.compose != 0 ? (static_cast<int64_t>(hv) * 2 + (transition ? 1 : 0)) * TILE
                                             : static_cast<int64_t>(hv) * TILE) + row0 * D;
  for (int i = tid; i < ROWS * D; i += FOLD_THREADS) dst[i] = sh.s[i];
}

// Ranges of one sequence inside one GPU: every range's incoming state, in order.
__global__ void __launch_bounds__(FOLD_THREADS) cp_fold_segments_kernel(const pla_b200_cp_fold_segments_args p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  FoldSmem& sh = *reinterpret_cast<FoldSmem*>(smem_raw);
  const int tid = threadIdx.x;
  const int rs = blockIdx.x % (D / ROWS);
  const int hv = (blockIdx.x / (D / ROWS)) % p.HV;
  const int seq = blockIdx.x / ((D / ROWS) * p.HV);
  const int row0 = rs * ROWS;
  const int col = tid & 127, rg = tid >> 7;
  const int first = p.seg_first[seq], last = p.seg_first[seq + 1];   // ranges [first, last)
  if (last <= first) return;
  int slot = p.slot_indices != nullptr ? p.slot_indices[seq] : seq;
  if (slot >= p.slots && p.pool != nullptr) {
    if (tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_BAD_SLOT);
    slot = -1;
  }
  const float* init = (p.pool != nullptr && slot >= 0)
                          ? p.pool + static_cast<int64_t>(slot) * p.pool_slot_stride + static_cast<int64_t>(hv) * TILE + row0 * D
                          : nullptr;
  for (int i = tid; i < ROWS * D; i += FOLD_THREADS) sh.s[i] = init != nullptr ? init[i] : 0.0f;
  if (tid == 0) {
    mbar_init(&sh.bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  for (int j = first; j < last; ++j) {
    float* dst = p.state_in + (static_cast<int64_t>(j) * p.HV + hv) * TILE + row0 * D;
    for (int i = tid; i < ROWS * D; i += FOLD_THREADS) dst[i] = sh.s[i];
    if (j + 1 == last) break;
    const float* pair = p.pairs + (static_cast<int64_t>(j) * p.HV + hv) * 2 * TILE;   // [offset B | transition M]
    if (tid == 0) {
      mbar_expect_tx(&sh.bar, kTileBytes);
      bulk_load(sh.m, pair + TILE, kTileBytes, &sh.bar);
    }
    float acc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[r] = pair[(row0 + rg * 8 + r) * D + col];
    const bool ok = mbar_wait(&sh.bar, (j - first) & 1);
    if (__syncthreads_or(!ok)) {
      if (tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_WAIT_TIMEOUT);
      (void)mbar_wait(&sh.bar, (j - first) & 1);
      return;
    }
#pragma unroll 4
    for (int k4 = 0; k4 < D / 4; ++k4) {
      const float m0 = sh.m[(4 * k4 + 0) * D + col], m1 = sh.m[(4 * k4 + 1) * D + col];
      const float m2 = sh.m[(4 * k4 + 2) * D + col], m3 = sh.m[(4 * k4 + 3) * D + col];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float4 sv = *reinterpret_cast<const float4*>(&sh.s[(rg * 8 + r) * D + 4 * k4]);
        acc[r] = fmaf(sv.x, m0, fmaf(sv.y, m1, fmaf(sv.z, m2, fmaf(sv.w, m3, acc[r]))));
      }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 8; ++r) sh.s[(rg * 8 + r) * D + col] = acc[r];
    __syncthreads();
  }
}

}  // namespace
}  // namespace pla

extern "C" int pla_b200_cp_fold_segments(const pla_b200_cp_fold_segments_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  pla_b200_cp_fold_segments_args a = *args;
  default_status(a);
  PLA_REQUIRE(a.HV > 0 && a.sequences >= 0, PLA_B200_E_INVALID, "fold needs HV > 0 and sequences >= 0");
  if (a.sequences == 0) return PLA_B200_OK;
  PLA_REQUIRE(a.pairs && a.seg_first && a.state_in && aligned16(a.pairs), PLA_B200_E_INVALID,
              "pairs (16-byte aligned), seg_first and state_in are required");
  PLA_REQUIRE(a.pool == nullptr || (a.slots > 0 && a.pool_slot_stride >= static_cast<int64_t>(a.HV) * TILE),
              PLA_B200_E_INVALID, "the pool needs slots > 0 and a slot pitch that covers HV*128*128");
  static DeviceOnce configured;
  int dev = 0;
  PLA_CUDA_OK(cudaGetDevice(&dev));
  if (configured.needed(dev)) {
    PLA_CUDA_OK(cudaFuncSetAttribute(cp_fold_segments_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sizeof(FoldSmem)));
    configured.mark(dev);
  }
  const int64_t ctas = static_cast<int64_t>(a.sequences) * a.HV * (D / ROWS);
  PLA_REQUIRE(ctas < (1ll << 31), PLA_B200_E_TOO_LARGE, "fold grid too large");
  cp_fold_segments_kernel<<<static_cast<unsigned>(ctas), FOLD_THREADS, sizeof(FoldSmem), static_cast<cudaStream_t>(stream)>>>(a);
  PLA_CUDA_OK(cudaGetLastError());
  return PLA_B200_OK;
}

extern "C" int pla_b200_cp_fold_prefix(const pla_b200_cp_fold_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  pla_b200_cp_fold_args a = *args;
  default_status(a);
  PLA_REQUIRE(a.HV > 0 && a.rank >= 0 && a.world > 0 && (a.compose != 0 ? a.rank <= a.world : a.rank < a.world),
              PLA_B200_E_INVALID, "fold needs HV > 0 and 0 <= rank < world (<= world when composing)");
  PLA_REQUIRE(a.state_out != nullptr && (a.rank == 0 || a.pairs != nullptr), PLA_B200_E_INVALID,
              "pairs and state_out are required");
  PLA_REQUIRE(a.rank == 0 || aligned16(a.pairs), PLA_B200_E_ALIGN, "pairs must be 16-byte aligned");
  static DeviceOnce configured;
  int dev = 0;
  PLA_CUDA_OK(cudaGetDevice(&dev));
  if (configured.needed(dev)) {
    PLA_CUDA_OK(cudaFuncSetAttribute(cp_fold_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sizeof(FoldSmem)));
    configured.mark(dev);
  }
  cp_fold_kernel<<<static_cast<unsigned>(a.HV) * (D / ROWS) * (a.compose != 0 ? 2u : 1u), FOLD_THREADS, sizeof(FoldSmem),
                   static_cast<cudaStream_t>(stream)>>>(a);
  PLA_CUDA_OK(cudaGetLastError());
  return PLA_B200_OK;
}
