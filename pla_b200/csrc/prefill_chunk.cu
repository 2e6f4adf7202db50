// Chunked GDN prefill (chunk C = 64) on the tcgen05 tensor cores.
//
// Per chunk of one sequence and one value head (rows i = tokens of the chunk, G = chunk-local
// cumulative log decay, Gamma_ij = exp(G_i - G_j), S0 = state entering the chunk, [K x V]):
//     L  = tril(diag(beta) (Kn Kn^T .* Gamma), -1)          T = (I + L)^-1
//     W  = diag(beta) (V - diag(e^G) Kn S0)                  V' = T W
//     O  = diag(e^G) Qn S0 + tril((Qn Kn^T) .* Gamma) V'     S1 = e^{G_C} S0 + Kn^T diag(e^{G_C - G}) V'
// (scripts/prefill/flashqla/e2e_acc_full.py:301-352 states the same algebra; six-GEMM schedule at
//  src/prefill/flashqla/kernels/fused_fwd_cute.cu:52-59).
//
// Launch 1, `prepare` (one CTA per chunk and q/k head): L2-normalises the chunk's k and q rows,
// rounds them to tf32 into the tensor-core operand layout, forms Kn Kn^T and Qn Kn^T with ONE
// 128x64x128 tcgen05 MMA chain ([Kn; Qn] against Kn), and per value head of that q/k head builds
// the gate cumsum, P = tril(Qn Kn^T .* Gamma) and T by fp32 forward substitution (one thread per
// column, the reference found low-precision inverses unstable: docs/prefill_readme.md:162-166).
// Everything the chain needs is written to the workspace as ready-made operand images, so the
// chain fetches them with plain 1-D bulk copies.
//
// Launch 2, `chain` (one CTA per sequence and value head): see the second half of this file.
//
// Precision: all contractions run as kind::tf32 with fp32 accumulation. The operands written by
// this code are rounded to nearest; a bf16 pipeline misses the 1e-3 state bar (measured on a CPU
// emulation: 2-3e-3), tf32 gives 3-4e-4.
#include "common.cuh"
#include "tc05.cuh"

namespace pla {
namespace {

constexpr int C = 64;    // tokens per chunk
constexpr int D = 128;   // head dim (K = V)
constexpr int TILE = D * D;

// Operand images (bytes). A tf32 operand tile [R rows x K] is stored chunk-major:
// byte(r, k) = (k/4) * (R*16) + r*16 + (k%4)*4.
constexpr int KQ_BYTES = 128 * D * 4;   // rows 0-63 Kn, rows 64-127 Qn*scale; K = 128 (feature)
constexpr int KNT_BYTES = D * C * 4;    // rows = feature k (128), K = token (64)
constexpr int TM_BYTES = C * C * 4;     // T: rows = token i, K = token j
constexpr int PM_BYTES = C * C * 4;     // P: rows = token i, K = token j
constexpr int VEC_BYTES = 2 * C * 4;    // G[64] then beta[64]
constexpr int HBLOB = KQ_BYTES + KNT_BYTES;            // per (chunk, q/k head)
constexpr int VBLOB = TM_BYTES + PM_BYTES + VEC_BYTES;  // per (chunk, value head)

__host__ __device__ inline int64_t ws_hblob(int64_t gc, int h, int H) { return (gc * H + h) * HBLOB; }
__host__ __device__ inline int64_t ws_vblob(int64_t max_chunks, int H, int HV, int64_t gc, int hv) {
  return max_chunks * H * static_cast<int64_t>(HBLOB) + (gc * HV + hv) * VBLOB;
}

// Global chunk id -> (sequence, chunk inside it). Chunks restart at every sequence start.
struct ChunkPos {
  int seq, ci, n;   // n = valid tokens in the chunk (1..64)
  int64_t tok0;     // first token row
};
__device__ __forceinline__ bool locate_chunk(const int32_t* cu, int N, int gc, ChunkPos& pos) {
  int acc = 0;
  for (int s = 0; s < N; ++s) {
    const int b = cu[s], e = cu[s + 1];
    const int len = e > b ? e - b : 0;
    const int nc = (len + C - 1) / C;
    if (gc < acc + nc) {
      pos.seq = s;
      pos.ci = gc - acc;
      pos.tok0 = static_cast<int64_t>(b) + static_cast<int64_t>(pos.ci) * C;
      pos.n = min(C, len - pos.ci * C);
      return true;
    }
    acc += nc;
  }
  return false;
}
__device__ __forceinline__ int first_chunk_of(const int32_t* cu, int seq) {
  int acc = 0;
  for (int s = 0; s < seq; ++s) {
    const int len = cu[s + 1] - cu[s];
    acc += (max(len, 0) + C - 1) / C;
  }
  return acc;
}

// ================================================================================================
// prepare
// ================================================================================================
constexpr int L_STRIDE = 68;  // padded row of the fp32 L matrix (floats); rows stay 16-byte aligned

struct PrepSmem {
  alignas(1024) float kq[KQ_BYTES / 4];
  alignas(1024) float knt[KNT_BYTES / 4];
  alignas(16) float L[2][C * L_STRIDE];
  float G[2][C];
  float beta[2][C];
  alignas(8) uint64_t bar;
  uint32_t tmem_base;
};

template <typename act_t>
__device__ __forceinline__ float row_sumsq(const act_t* row, bool vec) {
  float ss = 0.f;
  if (vec) {
#pragma unroll 4
    for (int i = 0; i < D / 8; ++i) {
      const uint4 raw = reinterpret_cast<const uint4*>(row)[i];
      const act_t* e = reinterpret_cast<const act_t*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float x = to_f32(e[j]);
        ss += x * x;
      }
    }
  } else {
#pragma unroll 8
    for (int i = 0; i < D; ++i) {
      const float x = to_f32(row[i]);
      ss += x * x;
    }
  }
  return ss;
}

template <typename act_t>
__global__ void __launch_bounds__(128) gdn_chunk_prepare_kernel(const pla_b200_gdn_chunk_args p) {
  extern __shared__ unsigned char smem_dyn[];
  // the launch reserves 1 KiB of slack so that the operand images can be aligned by hand
  unsigned char* smem_raw = smem_dyn + ((1024u - (smem_addr(smem_dyn) & 1023u)) & 1023u);
  PrepSmem& sh = *reinterpret_cast<PrepSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x % p.H;
  const int gc = blockIdx.x / p.H;
  ChunkPos pos;
  if (!locate_chunk(p.cu_seqlens, p.N, gc, pos)) return;
  const int R = p.HV / p.H;

  if (warp == 0) tc05::tmem_alloc(&sh.tmem_base, 64);
  if (tid == 0) {
    mbar_init(&sh.bar, 1);
    fence_mbar_init();
  }

  // ---- phase A: normalised rows -> tf32 operand images ----
  {
    const int c = tid & 63;
    const bool is_q = tid >= 64;
    float4* kq4 = reinterpret_cast<float4*>(sh.kq);
    if (c < pos.n) {
      const act_t* base = static_cast<const act_t*>(is_q ? p.q : p.k);
      const int64_t stride = is_q ? p.q_tok_stride : p.k_tok_stride;
      const act_t* row = base + (pos.tok0 + c) * stride + h * D;
      const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
      float r = is_q ? p.scale : 1.0f;
      if (p.normalize_qk) r *= rsqrtf(row_sumsq(row, vec) + 1e-6f);
#pragma unroll 2
      for (int i = 0; i < D / 8; ++i) {
        float x[8];
        if (vec) {
          const uint4 raw = reinterpret_cast<const uint4*>(row)[i];
          const act_t* e = reinterpret_cast<const act_t*>(&raw);
#pragma unroll
          for (int j = 0; j < 8; ++j) x[j] = tc05::to_tf32(to_f32(e[j]) * r);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) x[j] = tc05::to_tf32(to_f32(row[i * 8 + j]) * r);
        }
        kq4[(2 * i) * 128 + tid] = make_float4(x[0], x[1], x[2], x[3]);
        kq4[(2 * i + 1) * 128 + tid] = make_float4(x[4], x[5], x[6], x[7]);
        if (!is_q) {
          // transposed copy: rows = feature, K = token
#pragma unroll
          for (int j = 0; j < 8; ++j) sh.knt[(c >> 2) * (D * 4) + (i * 8 + j) * 4 + (c & 3)] = x[j];
        }
      }
    } else {
      for (int i = 0; i < D / 4; ++i) kq4[i * 128 + tid] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (!is_q)
        for (int kk = 0; kk < D; ++kk) sh.knt[(c >> 2) * (D * 4) + kk * 4 + (c & 3)] = 0.f;
    }
  }
  fence_async_smem();   // the images are read by the tensor core and by bulk stores (async proxy)
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tbase = sh.tmem_base;

  // ---- phase B: one MMA chain  D0[128 x 64] = [Kn; Qn] (128 x 128) * Kn^T ----
  if (tid == 0) {
    const uint64_t a_desc = tc05::smem_desc(sh.kq, 128 * 16, 128);
    constexpr uint32_t idesc = tc05::idesc_tf32(128, 64);
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      const uint64_t d = tc05::desc_advance(a_desc, j * 2 * 128 * 16);
      tc05::mma_tf32_ss(tbase, d, d, idesc, j > 0);  // B = the first 64 rows of the same image
    }
    tc05::mma_commit(&sh.bar);
  }
  {
    const bool ok = mbar_wait(&sh.bar, 0, 1u << 20);
    if (__syncthreads_or(!ok)) {
      if (tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_WAIT_TIMEOUT);
      __syncthreads();
      if (warp == 0) tc05::tmem_dealloc(tbase, 64);
      return;
    }
  }
  tc05::fence_after_sync();

  // this thread's row of D0: row i = tid % 64 of Kn Kn^T (tid < 64) or of Qn Kn^T (tid >= 64)
  float d0[C];
  {
    float t0[32], t1[32];
    tc05::tmem_ld32(tc05::taddr(tbase, warp * 32, 0), t0);
    tc05::tmem_ld32(tc05::taddr(tbase, warp * 32, 32), t1);
    tc05::wait_ld();
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      d0[j] = t0[j];
      d0[32 + j] = t1[j];
    }
  }

  unsigned char* ws = static_cast<unsigned char*>(p.workspace);
  const int i_row = tid & 63;
  const bool p_row = tid >= 64;

  for (int r0 = 0; r0 < R; r0 += 2) {
    const int heads_now = min(2, R - r0);
    // ---- gates of up to two value heads: warp s computes head s ----
    if (warp < heads_now) {
      const int hv = h * R + r0 + warp;
      float g2[2], b2[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int c = lane + 32 * u;
        float g = 0.f, b = 0.f;
        if (c < pos.n) {
          const int64_t tok = pos.tok0 + c;
          if (p.gate_activated) {
            g = static_cast<const float*>(p.gate)[tok * p.gate_tok_stride + hv];
            b = static_cast<const float*>(p.beta)[tok * p.beta_tok_stride + hv];
          } else {
            const float x = to_f32(static_cast<const act_t*>(p.gate)[tok * p.gate_tok_stride + hv]) + p.dt_bias[hv];
            g = log_decay(x, p.A_log[hv], PLA_B200_GATE_SOFTPLUS, 1.0f, 20.0f, 0.0f);
            b = sigmoidf_fast(to_f32(static_cast<const act_t*>(p.beta)[tok * p.beta_tok_stride + hv]));
          }
        }
        g2[u] = g;
        b2[u] = b;
      }
      // inclusive scan over 64 tokens: lanes hold tokens (lane, lane + 32)
      float s0 = g2[0], s1 = g2[1];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float t0 = __shfl_up_sync(0xffffffffu, s0, o);
        const float t1 = __shfl_up_sync(0xffffffffu, s1, o);
        if (lane >= o) {
          s0 += t0;
          s1 += t1;
        }
      }
      s1 += __shfl_sync(0xffffffffu, s0, 31);
      sh.G[warp][lane] = s0;
      sh.G[warp][lane + 32] = s1;
      sh.beta[warp][lane] = b2[0];
      sh.beta[warp][lane + 32] = b2[1];
      if (p.g_cum != nullptr) {
        if (lane < pos.n) p.g_cum[(pos.tok0 + lane) * p.HV + hv] = s0;
        if (lane + 32 < pos.n) p.g_cum[(pos.tok0 + lane + 32) * p.HV + hv] = s1;
      }
    }
    __syncthreads();

    // ---- L (strictly lower, fp32, shared) and P (lower incl. diagonal, tf32 image, global) ----
    for (int s = 0; s < heads_now; ++s) {
      const int hv = h * R + r0 + s;
      const float gi = sh.G[s][i_row];
      if (!p_row) {
        const float bi = sh.beta[s][i_row];
        float* Lrow = sh.L[s] + i_row * L_STRIDE;
#pragma unroll
        for (int j = 0; j < C; ++j)
          Lrow[j] = (j < i_row) ? bi * d0[j] * __expf(gi - sh.G[s][j]) : 0.0f;
      } else {
        float4* Pimg = reinterpret_cast<float4*>(ws + ws_vblob(p.max_chunks, p.H, p.HV, gc, hv) + TM_BYTES);
#pragma unroll
        for (int jc = 0; jc < C / 4; ++jc) {
          float x[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int j = jc * 4 + u;
            x[u] = (j <= i_row && i_row < pos.n) ? tc05::to_tf32(d0[j] * __expf(gi - sh.G[s][j])) : 0.0f;
          }
          Pimg[jc * C + i_row] = make_float4(x[0], x[1], x[2], x[3]);
        }
      }
    }
    __syncthreads();

    // ---- T = (I + L)^-1: thread = one column, rows by forward substitution, all in registers ----
    {
      const int s = tid >> 6, col = tid & 63;
      if (s < heads_now) {
        const int hv = h * R + r0 + s;
        float Tcol[C];
#pragma unroll
        for (int i = 0; i < C; ++i) Tcol[i] = 0.0f;
#pragma unroll
        for (int i = 0; i < C; ++i) {
          const float4* Lrow = reinterpret_cast<const float4*>(sh.L[s] + i * L_STRIDE);
          float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
          for (int j4 = 0; j4 < (i + 3) / 4; ++j4) {
            const float4 l = Lrow[j4];  // entries at j >= i are zero
            a0 = fmaf(l.x, Tcol[4 * j4 + 0], a0);
            a1 = fmaf(l.y, Tcol[4 * j4 + 1], a1);
            a2 = fmaf(l.z, Tcol[4 * j4 + 2], a2);
            a3 = fmaf(l.w, Tcol[4 * j4 + 3], a3);
          }
          Tcol[i] = ((i == col) ? 1.0f : 0.0f) - ((a0 + a1) + (a2 + a3));
        }
        float* Timg = reinterpret_cast<float*>(ws + ws_vblob(p.max_chunks, p.H, p.HV, gc, hv));
#pragma unroll
        for (int i = 0; i < C; ++i) Timg[(col >> 2) * (C * 4) + i * 4 + (col & 3)] = tc05::to_tf32(Tcol[i]);
        float* vec = reinterpret_cast<float*>(ws + ws_vblob(p.max_chunks, p.H, p.HV, gc, hv) + TM_BYTES + PM_BYTES);
        vec[col] = sh.G[s][col];
        vec[C + col] = sh.beta[s][col];
      }
    }
    __syncthreads();  // L / G / beta are rewritten by the next pair of heads
  }

  // ---- Kn|Qn and Kn^T images -> workspace (bulk stores straight from shared memory) ----
  if (tid == 0) {
    unsigned char* dst = ws + ws_hblob(gc, h, p.H);
    bulk_store(dst, sh.kq, KQ_BYTES);
    bulk_store(dst + KQ_BYTES, sh.knt, KNT_BYTES);
    bulk_commit();
    bulk_wait_read<0>();
  }
  tc05::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc05::tmem_dealloc(tbase, 64);
}

}  // namespace
}  // namespace pla

extern "C" int64_t pla_b200_gdn_chunk_workspace_bytes(int32_t max_chunks, int32_t H, int32_t HV) {
  if (max_chunks < 0 || H <= 0 || HV <= 0) return 0;
  return static_cast<int64_t>(max_chunks) * (static_cast<int64_t>(H) * pla::HBLOB + static_cast<int64_t>(HV) * pla::VBLOB);
}

extern "C" int pla_b200_gdn_prefill_chunked(const pla_b200_gdn_chunk_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  const pla_b200_gdn_chunk_args& a = *args;
  PLA_REQUIRE(a.N > 0 && a.T_total >= 0 && a.max_chunks >= 0, PLA_B200_E_INVALID, "N, T_total, max_chunks out of range");
  PLA_REQUIRE(a.H > 0 && a.HV >= a.H && a.HV % a.H == 0, PLA_B200_E_INVALID,
              "HV must be a positive multiple of H, got H=%d, HV=%d", a.H, a.HV);
  PLA_REQUIRE(a.q && a.k && a.v && a.gate && a.beta && a.o && a.cu_seqlens, PLA_B200_E_INVALID,
              "q, k, v, gate, beta, o and cu_seqlens are required");
  PLA_REQUIRE(a.gate_activated || (a.A_log && a.dt_bias), PLA_B200_E_INVALID, "raw gating needs A_log and dt_bias");
  PLA_REQUIRE(a.act_dtype == PLA_B200_BF16 || a.act_dtype == PLA_B200_F16, PLA_B200_E_INVALID,
              "activation dtype must be bf16 or fp16");
  PLA_REQUIRE(a.workspace != nullptr && (reinterpret_cast<uintptr_t>(a.workspace) & 127) == 0 &&
                  a.workspace_bytes >= pla_b200_gdn_chunk_workspace_bytes(a.max_chunks, a.H, a.HV),
              PLA_B200_E_INVALID, "workspace missing, not 128-byte aligned or too small");
  if (a.max_chunks == 0) return PLA_B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t items = static_cast<int64_t>(a.max_chunks) * a.H;
  PLA_REQUIRE(items < (1ll << 31), PLA_B200_E_TOO_LARGE, "too many chunks");
  auto launch_prepare = [&](auto kern) -> int {
    static bool configured[64] = {};
    int dev = 0;
    PLA_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
      PLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(PrepSmem) + 1024)));
      configured[dev] = true;
    }
    kern<<<static_cast<unsigned>(items), 128, sizeof(PrepSmem) + 1024, s>>>(a);
    PLA_CUDA_OK(cudaGetLastError());
    return PLA_B200_OK;
  };
  int rc = a.act_dtype == PLA_B200_BF16 ? launch_prepare(gdn_chunk_prepare_kernel<__nv_bfloat16>)
                                        : launch_prepare(gdn_chunk_prepare_kernel<__half>);
  if (rc != PLA_B200_OK || a.stage == 1) return rc;
  PLA_REQUIRE(false, PLA_B200_E_UNSUPPORTED, "the chain stage is not built yet");
}
