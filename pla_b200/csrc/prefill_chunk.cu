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
// the gate cumsum, L (fp32) and P = tril(Qn Kn^T .* Gamma).
// Launch 2, `inverse` (64 threads per chunk and value head): T = (I + L)^-1 by fp32 forward
// substitution, one thread per column (the reference found low-precision inverses unstable:
// docs/prefill_readme.md:162-166).
// Everything the chain needs is written to the workspace as ready-made operand images, so the
// chain fetches them with plain 1-D bulk copies.
//
// Launch 3, `chain` (one CTA per sequence and value head): see the second half of this file.
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
constexpr int VEC_BYTES = 4 * C * 4;    // beta exp(G)[64], beta[64], exp(G)[64], exp(G_last - G)[64]
constexpr int HBLOB = KQ_BYTES + KNT_BYTES;            // per (chunk, q/k head)
constexpr int VBLOB = TM_BYTES + PM_BYTES + VEC_BYTES;  // per (chunk, value head)
// T and P are lower triangular (diagonal included). In their images ([K / 4 = column group jg][row i][4 columns])
// the rows i < 4 jg of column group jg are all zero: they are neither written to the workspace nor copied back.
// Column group jg is one contiguous piece, rows 4 jg .. 63.
__host__ __device__ constexpr int tri_piece_offset(int jg) { return (jg * C + 4 * jg) * 16; }
__host__ __device__ constexpr int tri_piece_bytes(int jg) { return (C - 4 * jg) * 16; }
constexpr int TRI_BYTES = 16 * (C / 4 * C - 4 * (C / 4) * (C / 4 - 1) / 2);   // 8704: all sixteen pieces

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

// T = (I + L)^-1, one column per thread, rows by forward substitution, all in registers.
// A column of the 16-wide column block cb is zero above row 16 cb and only needs rows / terms from its own block
// on. L: strictly lower triangle, fp32, in the workspace's own layout [column group of 4][row][4] (every read
// below is a broadcast to the lanes of an item, so the layout costs no bank conflicts).
__device__ __forceinline__ float4 l_piece(const float* L, int row, int jg) {
  return reinterpret_cast<const float4*>(L)[jg * C + row];
}
__device__ __forceinline__ void invert_column(const float* __restrict__ L, int cb, int col, float (&Tcol)[C]) {
  // Rows go in blocks of four. The part of a row's sum over the columns before its block does not depend on the
  // other rows of the block, so the four rows run side by side (sixteen independent multiply-add chains); only
  // the block's own 4 x 4 triangle is sequential. That cuts the dependent steps from 64 rows to 16 blocks.
#pragma unroll
  for (int i = 0; i < C; ++i) Tcol[i] = 0.0f;
#pragma unroll
  for (int rb = 0; rb < C / 4; ++rb) {
    if (cb <= (rb >> 2)) {
      float acc[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[u][k] = 0.0f;
#pragma unroll
      for (int jq = 0; jq < C / 16; ++jq) {   // 16-column groups from the thread's column block on
        if (cb <= jq) {
#pragma unroll
          for (int jb = jq * 4; jb < jq * 4 + 4 && jb < rb; ++jb) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float4 l = l_piece(L, 4 * rb + u, jb);
              acc[u][0] = fmaf(l.x, Tcol[4 * jb + 0], acc[u][0]);
              acc[u][1] = fmaf(l.y, Tcol[4 * jb + 1], acc[u][1]);
              acc[u][2] = fmaf(l.z, Tcol[4 * jb + 2], acc[u][2]);
              acc[u][3] = fmaf(l.w, Tcol[4 * jb + 3], acc[u][3]);
            }
          }
        }
      }
      // the block's own triangle (the piece of row 4 rb is not staged and not needed: nothing left of its diagonal)
      const int r0 = 4 * rb;
      const float4 l1 = l_piece(L, r0 + 1, rb);
      const float4 l2 = l_piece(L, r0 + 2, rb);
      const float4 l3 = l_piece(L, r0 + 3, rb);
      const float t0 = ((r0 == col) ? 1.0f : 0.0f) - ((acc[0][0] + acc[0][1]) + (acc[0][2] + acc[0][3]));
      const float t1 = ((r0 + 1 == col) ? 1.0f : 0.0f) -
                       (((acc[1][0] + acc[1][1]) + (acc[1][2] + acc[1][3])) + l1.x * t0);
      const float t2 = ((r0 + 2 == col) ? 1.0f : 0.0f) -
                       (((acc[2][0] + acc[2][1]) + (acc[2][2] + acc[2][3])) + fmaf(l2.y, t1, l2.x * t0));
      const float t3 = ((r0 + 3 == col) ? 1.0f : 0.0f) -
                       (((acc[3][0] + acc[3][1]) + (acc[3][2] + acc[3][3])) + fmaf(l3.z, t2, fmaf(l3.y, t1, l3.x * t0)));
      Tcol[r0] = t0;
      Tcol[r0 + 1] = t1;
      Tcol[r0 + 2] = t2;
      Tcol[r0 + 3] = t3;
    }
  }
}

// 4 x 4 transpose across the four lanes of a group (lane % 4 = token inside a token group): in = this lane's four
// values (features f .. f + 3 of its token), out = feature f + lane % 4 of the group's four tokens. Two exchange
// steps. The transposed operand images [token group][feature][4 tokens] are written with it: lane r stores 16
// bytes, the four lanes of a group 64 contiguous bytes (scalar stores touched eight lines per instruction).
__device__ __forceinline__ float4 lane_transpose4(float4 x, bool b0, bool b1) {
  // step 1: even lanes collect the even features of the lane pair, odd lanes the odd ones
  const float r0 = __shfl_xor_sync(0xffffffffu, b0 ? x.x : x.y, 1);
  const float r1 = __shfl_xor_sync(0xffffffffu, b0 ? x.z : x.w, 1);
  const float w00 = b0 ? r0 : x.x, w01 = b0 ? x.y : r0;    // [feature pair][token of the lane pair]
  const float w10 = b0 ? r1 : x.z, w11 = b0 ? x.w : r1;
  // step 2: lanes 0, 1 of the group collect features 0, 1; lanes 2, 3 features 2, 3
  const float s0 = __shfl_xor_sync(0xffffffffu, b1 ? w00 : w10, 2);
  const float s1 = __shfl_xor_sync(0xffffffffu, b1 ? w01 : w11, 2);
  const float t0 = b1 ? w10 : w00, t1 = b1 ? w11 : w01;
  return b1 ? make_float4(s0, s1, t0, t1) : make_float4(t0, t1, s0, s1);
}

constexpr int PREP_THREADS = 256;
constexpr int PREP_HEADS = 4;   // value heads of one q/k head handled per pass
constexpr int L_BYTES = C * C * 4;
// fp32 L matrices [chunk][value head][column group of 4][row][4] behind the operand images (the layout of the T and
// P images, so that a warp that holds 32 rows of one column group stores 512 contiguous bytes)
__host__ __device__ inline int64_t ws_lmat(int64_t max_chunks, int H, int HV, int64_t gc, int hv) {
  return max_chunks * (H * static_cast<int64_t>(HBLOB) + HV * static_cast<int64_t>(VBLOB)) +
         (gc * HV + hv) * static_cast<int64_t>(L_BYTES);
}

constexpr int PREP_PARTS = 8;                      // the [Kn; Qn] image is built in this many slices of the features
constexpr int KQ_PART = KQ_BYTES / PREP_PARTS;     // bytes of one slice: 16 features = 4 feature groups x 128 rows x 16 B
struct PrepSmem {
  alignas(1024) float kq[2][KQ_PART / 4];      // two slices of the [Kn; Qn] image in flight
  alignas(16) uint32_t stg[128 * 68];    // staged raw k rows (0..63) and q rows (64..127)
  float G[PREP_HEADS][C];
  float beta[PREP_HEADS][C];
  float rnorm[128];
  alignas(8) uint64_t bar[2];            // MMAs that read quarter buffer b have finished
  uint32_t tmem_base;
};

// Launch 1 of the GDN prepare: operand images, Kn Kn^T | Qn Kn^T on the tensor core, gates, L (fp32, to the
// workspace) and the P image. 256 threads, 54 KiB of shared memory and 64 registers, so four CTAs share an SM and
// cover each other's phases: the [Kn; Qn] image never exists as a whole in shared memory -- it is built 16 features
// at a time into two 8 KiB buffers, each slice feeding two MMA steps of the one accumulator and one bulk store to
// the workspace while the next slice is built into the other buffer.
// Launch 2 (`chunk_inverse_kernel`) inverts I + L.
template <typename act_t>
__global__ void __launch_bounds__(PREP_THREADS, 4) gdn_chunk_prepare_kernel(const pla_b200_gdn_chunk_args p) {
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
    mbar_init(&sh.bar[0], 1);
    mbar_init(&sh.bar[1], 1);
    fence_mbar_init();
  }
  constexpr int STG = 68;  // staged row pitch in 32-bit words = 17 x 16 bytes
  const act_t* kbase = static_cast<const act_t*>(p.k) + pos.tok0 * p.k_tok_stride + h * D;
  const act_t* qbase = static_cast<const act_t*>(p.q) + pos.tok0 * p.q_tok_stride + h * D;

  // ---- stage the chunk's 64 k rows and 64 q rows. A row of any 2-byte alignment is fetched as the 16 or
  // 17 aligned 16-byte pieces that overlap it (up to 14 bytes before and after it come along, always
  // from a 16-byte granule that the row itself occupies, hence from mapped memory) and starts
  // (address % 16) / 2 halfwords into its staged copy. ----
  for (int r = warp; r < 128; r += PREP_THREADS / 32) {
    const int c = r & 63;
    if (c >= pos.n || lane >= 17) continue;
    const act_t* row = r >= 64 ? qbase + c * p.q_tok_stride : kbase + c * p.k_tok_stride;
    const char* src = reinterpret_cast<const char*>(reinterpret_cast<uintptr_t>(row) & ~uintptr_t(15));
    // an aligned row ends with its 16th piece: the 17th would lie wholly outside it (and, for the
    // buffer's last row, outside the allocation)
    if (lane == 16 && src == reinterpret_cast<const char*>(row)) continue;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(sh.stg + r * STG) + lane * 16),
                 "l"(src + lane * 16)
                 : "memory");
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
  __syncthreads();

  // ---- L2 norms: two threads per row (adjacent lanes), 32 words each ----
  {
    const int r = tid >> 1, half = tid & 1, c = r & 63;
    const bool is_q = r >= 64, live = c < pos.n;
    float ss = 0.f;
    if (live && p.normalize_qk) {
      const act_t* row = is_q ? qbase + c * p.q_tok_stride : kbase + c * p.k_tok_stride;
      const int sh_half = static_cast<int>((reinterpret_cast<uintptr_t>(row) & 15) >> 1);
      const uint32_t* srow = sh.stg + r * STG + (sh_half >> 1) + 32 * half;
      const bool odd = sh_half & 1;
      // rows 8 apart and the two halves of a row start on the same bank: rotate the word order per lane
      const int rot = half | ((lane >> 4) << 1);
#pragma unroll 8
      for (int i0 = 0; i0 < 32; ++i0) {
        const int i = (i0 + rot) & 31;
        const uint32_t w = odd ? __funnelshift_r(srow[i], srow[i + 1], 16) : srow[i];
        const act_t* e = reinterpret_cast<const act_t*>(&w);
        const float x0 = to_f32(e[0]), x1 = to_f32(e[1]);
        ss = fmaf(x0, x0, fmaf(x1, x1, ss));
      }
    }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);   // outside every branch: all lanes take part
    float rn = 0.f;
    if (live) rn = (is_q ? p.scale : 1.0f) * (p.normalize_qk ? rsqrtf(ss + 1e-6f) : 1.0f);
    if (half == 0) sh.rnorm[r] = rn;
  }
  __syncthreads();

  // ---- operand images and the MMA chain  D0[128 x 64] = [Kn; Qn] (128 x 128) * Kn^T, one slice of the features
  // at a time. Thread = (token c, one of the slice's four feature groups) for the k row AND the q row. ----
  unsigned char* ws = static_cast<unsigned char*>(p.workspace);
  uint32_t tbase = 0;
  // gives up on a wait that ran out: status bit, drain the bulk stores, free the tensor memory
  auto bail = [&]() {
    if (tid == 0) {
      if (p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_WAIT_TIMEOUT);
      bulk_wait_read<0>();
    }
    __syncthreads();
    if (warp == 0) tc05::tmem_dealloc(sh.tmem_base, 64);
  };
  {
    const int c = tid & 63, qq = tid >> 6;
    const bool live = c < pos.n;
    const float rnk = sh.rnorm[c], rnq = sh.rnorm[64 + c];
    const int shk = static_cast<int>((reinterpret_cast<uintptr_t>(kbase + c * p.k_tok_stride) & 15) >> 1);
    const int shq = static_cast<int>((reinterpret_cast<uintptr_t>(qbase + c * p.q_tok_stride) & 15) >> 1);
    const uint32_t* __restrict__ krow = sh.stg + c * STG + (shk >> 1);
    const uint32_t* __restrict__ qrow = sh.stg + (64 + c) * STG + (shq >> 1);
    const bool oddk = shk & 1, oddq = shq & 1;
    // transposed image [token group][feature][4 tokens], through 4 x 4 lane transposes
    float4* __restrict__ knt4 = reinterpret_cast<float4*>(ws + ws_hblob(gc, h, p.H) + KQ_BYTES) + (c >> 2) * D + (lane & 3);
    const bool b0 = lane & 1, b1 = lane & 2;
#pragma unroll 1
    for (int q = 0; q < PREP_PARTS; ++q) {
      const int b = q & 1;
      if (q >= 2) {   // buffer b again: the MMAs of slice q - 2 are done with it and its bulk store has read it
        bool ok = true;
        if (tid == 0) {
          bulk_wait_read<1>();
          ok = mbar_wait(&sh.bar[b], ((q >> 1) - 1) & 1, 1u << 20);
        }
        if (__syncthreads_or(!ok)) {
          bail();
          return;
        }
      }
      // restrict: the staged rows (read), the operand image and the workspace (written) never overlap;
      // without it every load waits for the previous store
      float4* __restrict__ kq4 = reinterpret_cast<float4*>(sh.kq[b]);
      {
        const int kl = qq, kc = 4 * q + kl;   // feature group inside the slice / inside the row
        float4 xk = make_float4(0.f, 0.f, 0.f, 0.f), xq = xk;
        if (live) {
          const uint32_t k0 = oddk ? __funnelshift_r(krow[2 * kc], krow[2 * kc + 1], 16) : krow[2 * kc];
          const uint32_t k1 = oddk ? __funnelshift_r(krow[2 * kc + 1], krow[2 * kc + 2], 16) : krow[2 * kc + 1];
          const uint32_t q0 = oddq ? __funnelshift_r(qrow[2 * kc], qrow[2 * kc + 1], 16) : qrow[2 * kc];
          const uint32_t q1 = oddq ? __funnelshift_r(qrow[2 * kc + 1], qrow[2 * kc + 2], 16) : qrow[2 * kc + 1];
          const act_t* a0 = reinterpret_cast<const act_t*>(&k0);
          const act_t* a1 = reinterpret_cast<const act_t*>(&k1);
          const act_t* e0 = reinterpret_cast<const act_t*>(&q0);
          const act_t* e1 = reinterpret_cast<const act_t*>(&q1);
          xk = make_float4(tc05::to_tf32(to_f32(a0[0]) * rnk), tc05::to_tf32(to_f32(a0[1]) * rnk),
                           tc05::to_tf32(to_f32(a1[0]) * rnk), tc05::to_tf32(to_f32(a1[1]) * rnk));
          xq = make_float4(tc05::to_tf32(to_f32(e0[0]) * rnq), tc05::to_tf32(to_f32(e0[1]) * rnq),
                           tc05::to_tf32(to_f32(e1[0]) * rnq), tc05::to_tf32(to_f32(e1[1]) * rnq));
        }
        kq4[kl * 128 + c] = xk;
        kq4[kl * 128 + 64 + c] = xq;
        knt4[kc * 4] = lane_transpose4(xk, b0, b1);
      }
      fence_async_smem();   // the image is read by the tensor core and by a bulk store (async proxy)
      tc05::fence_before_sync();
      __syncthreads();
      tc05::fence_after_sync();
      tbase = sh.tmem_base;
      if (tid == 0) {
        const uint64_t a_desc = tc05::smem_desc(sh.kq[b], 128 * 16, 128);
        constexpr uint32_t idesc = tc05::idesc_tf32(128, 64);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const uint64_t d = tc05::desc_advance(a_desc, j * 2 * 128 * 16);
          tc05::mma_tf32_ss(tbase, d, d, idesc, q > 0 || j > 0);  // B = the first 64 rows of the same image
        }
        tc05::mma_commit(&sh.bar[b]);
        bulk_store(ws + ws_hblob(gc, h, p.H) + q * KQ_PART, sh.kq[b], KQ_PART);
        bulk_commit();
      }
    }
  }

  const int quad = warp & 3, ch = warp >> 2;   // TMEM lane quadrant, column half
  const int i_row = (quad * 32 + lane) & 63;
  const bool p_row = quad >= 2;
  float d0[32];
  bool have_d0 = false;
  for (int r0 = 0; r0 < R; r0 += PREP_HEADS) {
    const int heads_now = min(PREP_HEADS, R - r0);
    if (r0 > 0) __syncthreads();  // G / beta of the previous pass fully consumed
    // ---- gates of up to eight value heads: warp s computes head s (while the tensor core works) ----
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
      // in base-2 units: the L / P epilogue takes differences of these and raises 2 to them (one multiply per
      // element less than through the natural exponential)
      sh.G[warp][lane] = s0 * 1.4426950408889634f;
      sh.G[warp][lane + 32] = s1 * 1.4426950408889634f;
      sh.beta[warp][lane] = b2[0];
      sh.beta[warp][lane + 32] = b2[1];
      if (p.g_cum != nullptr) {
        if (lane < pos.n) p.g_cum[(pos.tok0 + lane) * p.HV + hv] = s0;
        if (lane + 32 < pos.n) p.g_cum[(pos.tok0 + lane + 32) * p.HV + hv] = s1;
      }
      // vectors for the chain
      float* vec = reinterpret_cast<float*>(ws + ws_vblob(p.max_chunks, p.H, p.HV, gc, hv) + TM_BYTES + PM_BYTES);
      const float g_last = __shfl_sync(0xffffffffu, s1, 31);
      const float e0 = fast_exp(s0), e1 = fast_exp(s1);
      vec[lane] = b2[0] * e0;            // W = beta V - (beta e^G) (Kn S): one multiply-add per element in the chain
      vec[lane + 32] = b2[1] * e1;
      vec[C + lane] = b2[0];
      vec[C + lane + 32] = b2[1];
      vec[2 * C + lane] = e0;
      vec[2 * C + lane + 32] = e1;
      vec[3 * C + lane] = fast_exp(g_last - s0);
      vec[3 * C + lane + 32] = fast_exp(g_last - s1);
    }
    if (!have_d0) {
      const bool ok = mbar_wait(&sh.bar[1], ((PREP_PARTS - 1) >> 1) & 1, 1u << 20);   // the last slice's MMAs (and, in order, all before)
      if (__syncthreads_or(!ok)) {
        bail();
        return;
      }
      tc05::fence_after_sync();
      // this thread's half row of D0: row i of Kn Kn^T (lane quadrants 0, 1) or of Qn Kn^T (2, 3)
      tc05::tmem_ld32(tc05::taddr(tbase, quad * 32, 32 * ch), d0);
      tc05::wait_ld();
      have_d0 = true;
    } else {
      __syncthreads();
    }

    // ---- L (strictly lower, fp32) and P (lower incl. diagonal, tf32 image), both to the workspace ----
    for (int s = 0; s < heads_now; ++s) {
      const int hv = h * R + r0 + s;
      const float gi = sh.G[s][i_row];
      const float* __restrict__ Gs = sh.G[s] + 32 * ch;
      if (!p_row) {
        const float bi = sh.beta[s][i_row];
        float4* __restrict__ Lg =
            reinterpret_cast<float4*>(ws + ws_lmat(p.max_chunks, p.H, p.HV, gc, hv)) + ch * 8 * C + i_row;
#pragma unroll
        for (int jc = 0; jc < 8; ++jc) {
          if (32 * ch + 4 * jc >= i_row) continue;   // a piece at or beyond the diagonal: all zero, never read
          float x[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int j = jc * 4 + u;
            x[u] = (32 * ch + j < i_row) ? bi * d0[j] * fast_exp2(gi - Gs[j]) : 0.0f;
          }
          Lg[jc * C] = make_float4(x[0], x[1], x[2], x[3]);   // a warp's 32 rows: 512 contiguous bytes
        }
      } else {
        float4* __restrict__ Pimg = reinterpret_cast<float4*>(ws + ws_vblob(p.max_chunks, p.H, p.HV, gc, hv) + TM_BYTES);
#pragma unroll
        for (int jc = 0; jc < 8; ++jc) {
          if (32 * ch + 4 * jc > i_row) continue;    // rows above a column group's piece (tri_piece_offset)
          float x[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int j = jc * 4 + u;
            x[u] = (32 * ch + j <= i_row && i_row < pos.n) ? tc05::to_tf32(d0[j] * fast_exp2(gi - Gs[j])) : 0.0f;
          }
          Pimg[(ch * 8 + jc) * C + i_row] = make_float4(x[0], x[1], x[2], x[3]);
        }
      }
    }
  }

  if (tid == 0) bulk_wait_read<0>();   // the image store must have read shared memory before the CTA leaves
  tc05::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc05::tmem_dealloc(tbase, 64);
}

// L (fp32, strictly lower) -> T = (I + L)^-1 as a tf32 operand image. Two (chunk, value head) items per CTA.
__global__ void __launch_bounds__(128) chunk_inverse_kernel(const pla_b200_gdn_chunk_args p, int items) {
  __shared__ __align__(16) float Ls[2][C * C];
  // Warp w works on column block w of BOTH items (lanes 0..15 item 0, lanes 16..31 item 1): every lane of a warp
  // then walks the same rows and terms (a column of block cb starts at row 16 cb), where a warp that mixed two
  // column blocks of one item executed the longer walk with half of its lanes idle -- 41 % fewer instructions.
  const int tid = threadIdx.x, s = (tid >> 4) & 1, cb = tid >> 5;
  const int t6 = cb * 16 + (tid & 15);   // this thread's column of T, and the row of L it stages
  const int item = blockIdx.x * 2 + s;
  const bool live = item < items;
  unsigned char* ws = static_cast<unsigned char*>(p.workspace);
  const int hv = live ? item % p.HV : 0;
  const int gc = live ? item / p.HV : 0;
  ChunkPos pos;
  const bool found = live && locate_chunk(p.cu_seqlens, p.N, gc, pos);
  if (found) {
    // 16 asynchronous 16-byte copies per thread, all in flight at once (a load / store loop through registers
    // pays the DRAM latency once per iteration)
    const float4* Lg = reinterpret_cast<const float4*>(ws + ws_lmat(p.max_chunks, p.H, p.HV, gc, hv));
#pragma unroll
    for (int jg = 0; jg < C / 4; ++jg)
      if (4 * jg < t6)   // row t6, columns 4 jg ..: pieces at or beyond the diagonal are never read (nor written)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(&Ls[s][(jg * C + t6) * 4])),
                     "l"(Lg + jg * C + t6)
                     : "memory");
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
  __syncthreads();
  if (!found) return;
  const int col = t6;
  float Tcol[C];
  invert_column(Ls[s], cb, col, Tcol);
  float* Timg = reinterpret_cast<float*>(ws + ws_vblob(p.max_chunks, p.H, p.HV, gc, hv));
  // only the rows of the column group's piece (tri_piece_offset); the rows above it are zero and are not stored
#pragma unroll
  for (int i = 0; i < C; ++i)
    if (i >= (col & ~3)) Timg[(col >> 2) * (C * 4) + i * 4 + (col & 3)] = tc05::to_tf32(Tcol[i]);
}

// ================================================================================================
// KDA (per-channel decay): prepare in two launches
// ================================================================================================
// With a decay per key channel the factor e^{G_i[c] - G_j[c]} sits inside the contraction over c, so
// it is folded into the operands. To keep every factor representable the chunk is cut into four
// sub-blocks of 16 tokens with reference points R_a = cumulative log decay before sub-block a:
//     L[i, j] = beta_i sum_c (k_i e^{G_i - R_a})[c] (k_j e^{R_a - G_j})[c],   i in sub-block a, j < i
// The first factor is <= 1; the second is <= 1 for j in an earlier sub-block and at most the inverse
// decay of one sub-block for j in the same one (bounded by 16 |lower_bound| <= 80 nats for the safe
// gate; an unbounded softplus gate that decays by more than 80 nats inside 16 tokens sets
// PLA_B200_DEV_DECAY_RANGE). One B image per reference a (rows j < 16 (a + 1)), one A image
// [K e^{G-R}; Q e^{G-R}], four MMA chains; row block a of chain a is the wanted block row.
// The chain kernel gets  [K e^{G}; Q e^{G}]  (decay from the chunk start folded in),
// (K e^{G_C - G})^T  for the state update, beta and e^{G_C} per channel.
// Launch 1 (`kda_chunk_prepare_kernel`, 512 threads, one CTA per SM) builds everything except T and
// leaves L (fp32) in the workspace; launch 2 (`chunk_inverse_kernel`, light, many CTAs per SM)
// turns L into the T image.
constexpr int DM_PITCH = 132;  // floats per row of the decay-factor matrix: float4 rows, conflict-free per quarter warp
constexpr int KM_BYTES = 81920;  // four B images of 16, 32, 48, 64 rows x 512 bytes, back to back
__host__ __device__ constexpr int km_offset(int a) { return a * (a + 1) / 2 * 8192; }

constexpr int KDA_PREP_THREADS = 512;
constexpr int SB = 16;  // tokens per sub-block (decay reference points)

struct KdaPrepSmem {
  alignas(1024) float kq[KQ_BYTES / 4];
  alignas(1024) unsigned char km[KM_BYTES];  // first the staged gate rows, then the four B images
  alignas(16) float dm[C * DM_PITCH];        // e^{G - R_block} per (token, channel)
  alignas(16) uint32_t stg[128 * 68];        // staged raw k rows (0..63) and q rows (64..127)
  alignas(16) float part[4][D];              // log decay of each sub-block, per channel
  alignas(16) float erb[4][D];               // e^{R_a}
  alignas(16) float egc[4][D];               // e^{G_C - R_a}
  alignas(16) float fab[6][D];               // e^{R_a - R_b}, a > b, at index a (a - 1) / 2 + b
  float gc[D];
  float beta[C];
  float rnorm[128];
  alignas(8) uint64_t bar;
  uint32_t tmem_base;
};

template <typename act_t>
__global__ void __launch_bounds__(KDA_PREP_THREADS, 1) kda_chunk_prepare_kernel(const pla_b200_gdn_chunk_args p) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem_raw = smem_dyn + ((1024u - (smem_addr(smem_dyn) & 1023u)) & 1023u);
  KdaPrepSmem& sh = *reinterpret_cast<KdaPrepSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x % p.H;
  const int gc = blockIdx.x / p.H;
  ChunkPos pos;
  if (!locate_chunk(p.cu_seqlens, p.N, gc, pos)) return;

  if (warp == 0) tc05::tmem_alloc(&sh.tmem_base, 256);
  if (tid == 0) {
    mbar_init(&sh.bar, 1);
    fence_mbar_init();
  }
  constexpr int STG = 68;  // staged row pitch in 32-bit words = 17 x 16 bytes
  uint32_t* gstg = reinterpret_cast<uint32_t*>(sh.km);
  const act_t* kbase = static_cast<const act_t*>(p.k) + pos.tok0 * p.k_tok_stride + h * D;
  const act_t* qbase = static_cast<const act_t*>(p.q) + pos.tok0 * p.q_tok_stride + h * D;

  // ---- stage the chunk's k, q and gate rows (16 or 17 aligned 16-byte pieces per 256-byte row) ----
  for (int r = warp; r < 192; r += KDA_PREP_THREADS / 32) {
    const int c = r & 63, which = r >> 6;
    if (c >= pos.n || lane >= 17) continue;
    const act_t* row = which == 0   ? kbase + c * p.k_tok_stride
                       : which == 1 ? qbase + c * p.q_tok_stride
                                    : static_cast<const act_t*>(p.gate) + (pos.tok0 + c) * p.gate_tok_stride + h * D;
    const char* src = reinterpret_cast<const char*>(reinterpret_cast<uintptr_t>(row) & ~uintptr_t(15));
    if (lane == 16 && src == reinterpret_cast<const char*>(row)) continue;
    uint32_t* dst = which < 2 ? sh.stg + r * STG : gstg + c * STG;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst) + lane * 16), "l"(src + lane * 16)
                 : "memory");
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
  __syncthreads();

  // ---- L2 norms: four threads per row (adjacent lanes), 16 words each ----
  {
    const int r = tid >> 2, qt = tid & 3, c = r & 63;
    const bool is_q = r >= 64;
    const bool live = c < pos.n;
    float ss = 0.f;
    if (live && p.normalize_qk) {
      const act_t* row = is_q ? qbase + c * p.q_tok_stride : kbase + c * p.k_tok_stride;
      const int sh_half = static_cast<int>((reinterpret_cast<uintptr_t>(row) & 15) >> 1);
      const uint32_t* srow = sh.stg + r * STG + (sh_half >> 1) + 16 * qt;
      const bool odd = sh_half & 1;
      // the eight rows of a warp start 4 banks apart and the quarters 16: a per-lane rotation of the
      // word order gives every lane its own bank
      const int rot = (qt & 2) | ((lane >> 4) & 1);
#pragma unroll 8
      for (int i0 = 0; i0 < 16; ++i0) {
        const int i = (i0 + rot) & 15;
        const uint32_t w = odd ? __funnelshift_r(srow[i], srow[i + 1], 16) : srow[i];
        const act_t* e = reinterpret_cast<const act_t*>(&w);
        const float x0 = to_f32(e[0]), x1 = to_f32(e[1]);
        ss = fmaf(x0, x0, fmaf(x1, x1, ss));
      }
    }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);   // outside every branch: all lanes take part
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    float rn = 0.f;
    if (live) rn = (is_q ? p.scale : 1.0f) * (p.normalize_qk ? rsqrtf(ss + 1e-6f) : 1.0f);
    if (qt == 0) sh.rnorm[r] = rn;
    if (qt == 1 && !is_q)
      sh.beta[c] = live ? sigmoidf_fast(to_f32(static_cast<const act_t*>(p.beta)[(pos.tok0 + c) * p.beta_tok_stride + h]))
                        : 0.f;
  }

  // ---- one thread per (channel, sub-block): log decay, its running sum inside the sub-block, decay
  // factors e^{G - R}; the sub-blocks are independent because R is the sum up to the sub-block start ----
  {
    const int c = tid & 127, blk = tid >> 7;
    const float A_log = p.A_log[h];
    const float dtb = p.dt_bias[h * D + c];
    const unsigned short* gs = reinterpret_cast<const unsigned short*>(gstg);
    const int64_t e0 = static_cast<int64_t>(reinterpret_cast<uintptr_t>(p.gate) >> 1) + pos.tok0 * p.gate_tok_stride + h * D;
    float G = 0.f;
#pragma unroll 4
    for (int tt = 0; tt < SB; ++tt) {
      const int t = blk * SB + tt;
      if (t < pos.n) {
        const int shf = static_cast<int>((e0 + t * p.gate_tok_stride) & 7);
        act_t raw;
        *reinterpret_cast<unsigned short*>(&raw) = gs[t * (STG * 2) + shf + c];
        G += log_decay(to_f32(raw) + dtb, A_log, p.gate_kind, 1.0f, 20.0f, p.lower_bound);
      }
      sh.dm[t * DM_PITCH + c] = fast_exp(G);
    }
    sh.part[blk][c] = G;
    if (G < -80.0f && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_DECAY_RANGE);
  }
  __syncthreads();
  // ---- per-channel tables from the sub-block sums ----
  for (int i = tid; i < 14 * D; i += KDA_PREP_THREADS) {
    const int which = i / D, c = i % D;
    const float b0 = sh.part[0][c], b1 = sh.part[1][c], b2 = sh.part[2][c], b3 = sh.part[3][c];
    // R_a = log decay before sub-block a
    auto ref = [&](int a) { return (a > 0 ? b0 : 0.f) + (a > 1 ? b1 : 0.f) + (a > 2 ? b2 : 0.f); };
    const float total = b0 + b1 + b2 + b3;
    if (which < 4) {
      sh.erb[which][c] = fast_exp(ref(which));
      if (which == 0) sh.gc[c] = total;
    } else if (which < 8) {
      sh.egc[which - 4][c] = fast_exp(total - ref(which - 4));
    } else {
      const int f = which - 8;                       // (a, b): (1,0) (2,0) (2,1) (3,0) (3,1) (3,2)
      const int a = f < 1 ? 1 : f < 3 ? 2 : 3, b = f - a * (a - 1) / 2;
      sh.fab[f][c] = fast_exp(ref(a) - ref(b));
    }
  }
  __syncthreads();  // also: the staged gate rows (aliased with the B images) are fully consumed

  // ---- operand images: thread = (token c, eighth of the channels), for the k row AND the q row of the
  // token (same decay factors, same work for every thread) ----
  unsigned char* ws = static_cast<unsigned char*>(p.workspace);
  {
    const int c = tid & 63, e8 = tid >> 6, blk = c >> 4;
    const bool live = c < pos.n;
    const float rnk = sh.rnorm[c], rnq = sh.rnorm[64 + c];
    const int shk = static_cast<int>((reinterpret_cast<uintptr_t>(kbase + c * p.k_tok_stride) & 15) >> 1);
    const int shq = static_cast<int>((reinterpret_cast<uintptr_t>(qbase + c * p.q_tok_stride) & 15) >> 1);
    const uint32_t* __restrict__ krow = sh.stg + c * STG + (shk >> 1);
    const uint32_t* __restrict__ qrow = sh.stg + (64 + c) * STG + (shq >> 1);
    const bool oddk = shk & 1, oddq = shq & 1;
    float4* __restrict__ kq4 = reinterpret_cast<float4*>(sh.kq);
    float4* __restrict__ kqs_g = reinterpret_cast<float4*>(ws + ws_hblob(gc, h, p.H));
    // transposed image [token group][channel][4 tokens], through 4 x 4 lane transposes
    float4* __restrict__ ke4 = reinterpret_cast<float4*>(ws + ws_hblob(gc, h, p.H) + KQ_BYTES) + (c >> 2) * D + (lane & 3);
    const bool tb0 = lane & 1, tb1 = lane & 2;
    const float4* __restrict__ dmrow = reinterpret_cast<const float4*>(sh.dm + c * DM_PITCH);
    auto tf4 = [](float4 v) {
      return make_float4(tc05::to_tf32(v.x), tc05::to_tf32(v.y), tc05::to_tf32(v.z), tc05::to_tf32(v.w));
    };
    auto mul4 = [](float4 a, float4 b) { return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); };
#pragma unroll
    for (int kc = e8 * 4; kc < e8 * 4 + 4; ++kc) {
      float4 xk = make_float4(0.f, 0.f, 0.f, 0.f), xq = xk;
      if (live) {
        const uint32_t k0 = oddk ? __funnelshift_r(krow[2 * kc], krow[2 * kc + 1], 16) : krow[2 * kc];
        const uint32_t k1 = oddk ? __funnelshift_r(krow[2 * kc + 1], krow[2 * kc + 2], 16) : krow[2 * kc + 1];
        const uint32_t q0 = oddq ? __funnelshift_r(qrow[2 * kc], qrow[2 * kc + 1], 16) : qrow[2 * kc];
        const uint32_t q1 = oddq ? __funnelshift_r(qrow[2 * kc + 1], qrow[2 * kc + 2], 16) : qrow[2 * kc + 1];
        const act_t* a0 = reinterpret_cast<const act_t*>(&k0);
        const act_t* a1 = reinterpret_cast<const act_t*>(&k1);
        const act_t* b0 = reinterpret_cast<const act_t*>(&q0);
        const act_t* b1 = reinterpret_cast<const act_t*>(&q1);
        xk = make_float4(to_f32(a0[0]) * rnk, to_f32(a0[1]) * rnk, to_f32(a1[0]) * rnk, to_f32(a1[1]) * rnk);
        xq = make_float4(to_f32(b0[0]) * rnq, to_f32(b0[1]) * rnq, to_f32(b1[0]) * rnq, to_f32(b1[1]) * rnq);
      }
      const float4 dv = dmrow[kc];
      const float4 er = reinterpret_cast<const float4*>(sh.erb[blk])[kc];
      const float4 kp = mul4(xk, dv), qp = mul4(xq, dv);
      kq4[kc * 128 + c] = tf4(kp);
      kq4[kc * 128 + 64 + c] = tf4(qp);
      kqs_g[kc * 128 + c] = tf4(mul4(kp, er));
      kqs_g[kc * 128 + 64 + c] = tf4(mul4(qp, er));
      const float4 bs = make_float4(__fdividef(xk.x, fmaxf(dv.x, 1e-37f)), __fdividef(xk.y, fmaxf(dv.y, 1e-37f)),
                                    __fdividef(xk.z, fmaxf(dv.z, 1e-37f)), __fdividef(xk.w, fmaxf(dv.w, 1e-37f)));
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        if (a < blk) continue;
        float4 f = make_float4(1.f, 1.f, 1.f, 1.f);
        if (a > blk) f = reinterpret_cast<const float4*>(sh.fab[a * (a - 1) / 2 + blk])[kc];
        reinterpret_cast<float4*>(sh.km + km_offset(a))[kc * (16 * (a + 1)) + c] = tf4(mul4(bs, f));
      }
      const float4 ke = tf4(mul4(bs, reinterpret_cast<const float4*>(sh.egc[blk])[kc]));
      ke4[kc * 4] = lane_transpose4(ke, tb0, tb1);
    }
  }
  fence_async_smem();
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tbase = sh.tmem_base;

  // ---- four MMA chains: D_a[128 x 16(a+1)] = [K+; Q+] (128 x 128) * (K-(a))^T ----
  if (tid == 0) {
    const uint64_t a_desc = tc05::smem_desc(sh.kq, 128 * 16, 128);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int rows = 16 * (a + 1);
      const uint64_t b_desc = tc05::smem_desc(sh.km + km_offset(a), rows * 16, 128);
      const uint32_t idesc = tc05::idesc_tf32(128, rows);
      const uint32_t col = 8 * a * (a + 1);   // 0, 16, 48, 96
#pragma unroll
      for (int j = 0; j < D / 8; ++j)
        tc05::mma_tf32_ss(tbase + col, tc05::desc_advance(a_desc, j * 2 * 128 * 16),
                          tc05::desc_advance(b_desc, j * 2 * rows * 16), idesc, j > 0);
    }
    tc05::mma_commit(&sh.bar);
  }
  // vectors for the chain while the tensor core works: beta per token, e^{G_C} per channel
  if (tid >= 128 && tid < 256) {
    float* vec = reinterpret_cast<float*>(ws + ws_vblob(p.max_chunks, p.H, p.HV, gc, h) + TM_BYTES + PM_BYTES);
    const int c = tid - 128;
    vec[2 * C + c] = fast_exp(sh.gc[c]);
    if (c < C) {
      vec[c] = sh.beta[c];               // the decay is folded into the operands: W = beta V - beta (K+ S)
      vec[C + c] = sh.beta[c];
    }
  }
  {
    const bool ok = mbar_wait(&sh.bar, 0, 1u << 20);
    if (__syncthreads_or(!ok)) {
      if (tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_WAIT_TIMEOUT);
      __syncthreads();
      if (warp == 0) tc05::tmem_dealloc(tbase, 256);
      return;
    }
  }
  tc05::fence_after_sync();

  // ---- rows of L and P: TMEM lane = row (0..63 K+ rows, 64..127 Q+ rows); the four warps that may touch a
  // lane quadrant split the 64 columns; lanes 0-15 of a warp sit in sub-block a0 = 2 (quadrant % 2),
  // lanes 16-31 in a0 + 1 ----
  {
    const int quad = warp & 3, cs = warp >> 2;        // column slice: j in [16 cs, 16 cs + 16)
    const int row = quad * 32 + lane;                 // TMEM lane
    const int i_row = row & 63;
    const bool p_row = row >= 64;
    const int a0 = 2 * (quad & 1);
    float d0[16];
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      const int a = a0 + pass;
      float t0[32];
      tc05::tmem_ld32(tc05::taddr(tbase, quad * 32, 8 * a * (a + 1) + 16 * cs), t0);   // 16 of the 32 are used
      tc05::wait_ld();
      if ((lane >> 4) == pass) {
#pragma unroll
        for (int j = 0; j < 16; ++j) d0[j] = t0[j];
      }
    }
    // columns at or beyond 16 (a + 1) of chain a hold other chains' data: never selected below (j <= i_row)
    if (!p_row) {
      const float bi = sh.beta[i_row];
      float4* __restrict__ Lg = reinterpret_cast<float4*>(ws + ws_lmat(p.max_chunks, p.H, p.HV, gc, h)) + cs * 4 * C + i_row;
#pragma unroll
      for (int jc = 0; jc < 4; ++jc) {
        if (cs * 16 + jc * 4 >= i_row) continue;     // a piece at or beyond the diagonal: all zero, never read
        float x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) x[u] = (cs * 16 + jc * 4 + u < i_row) ? bi * d0[jc * 4 + u] : 0.0f;
        Lg[jc * C] = make_float4(x[0], x[1], x[2], x[3]);
      }
    } else {
      float4* __restrict__ Pimg = reinterpret_cast<float4*>(ws + ws_vblob(p.max_chunks, p.H, p.HV, gc, h) + TM_BYTES);
#pragma unroll
      for (int jc = 0; jc < 4; ++jc) {
        if (cs * 16 + jc * 4 > i_row) continue;      // rows above a column group's piece (tri_piece_offset)
        float x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int j = cs * 16 + jc * 4 + u;
          x[u] = (j <= i_row && i_row < pos.n) ? tc05::to_tf32(d0[jc * 4 + u]) : 0.0f;
        }
        Pimg[(cs * 4 + jc) * C + i_row] = make_float4(x[0], x[1], x[2], x[3]);
      }
    }
  }
  tc05::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc05::tmem_dealloc(tbase, 256);
}

// ================================================================================================
// chain: one CTA per (sequence, value head), chunks in order, state resident in tensor memory
// ================================================================================================
// Orientation: every accumulator is [128 lanes = value index v] x [columns = token or key index],
// i.e. the transposes of the matrices in the header comment, so that a thread of the epilogue
// group owns one v row and writes the next A operand straight back into TMEM:
//   MMA1  D1[v, 0:64 | 64:128] = S^T(TMEM, fp32 read as tf32) x [Kn; Qn]^T       -> (Kn S)^T | (Qn S)^T
//   E1    W^T[v, c] = beta_c (V[c, v] - e^{G_c} (Kn S)^T[v, c])                   -> over D1[:, 0:64]
//         O_inter[v, i] = e^{G_i} (Qn S)^T[v, i]                                  -> D3 (MMA3 accumulates onto it)
//   MMA2  D2[v, 0:64 | 64:128] = W^T(TMEM) x [T; T']^T,  T' = diag(e^{G_C - G}) T  -> V'^T | (decayed V')^T
//   MMA4  S[v, k]  += D2[:, 64:128](TMEM, as MMA2 left it) x Kn^T-image           -> state update
//   MMA3  D3[v, i] += D2[:, 0:64](TMEM, as MMA2 left it) x P^T                    -> + intra-chunk output
//   E3    O[i, v]   = D3[v, i] to 16 bits
// The only epilogue between MMA1 and the state update is E1: the decay of the update rides on the B operand of
// MMA2 (the scaler warps form T' from T in shared memory while MMA1 and E1 run), so MMA2's two results feed MMA3
// and MMA4 directly. MMA3 of chunk c is issued behind MMA1 of chunk c + 1 (D3 is double-buffered for that), so
// the serial path per chunk is MMA1 -> E1 -> MMA2 -> MMA4. Operands read straight from an accumulator are
// truncated to tf32 by the tensor core (3 to 4e-4 -> 5 to 6e-4 state error on 4K-token sequences; bar 1e-3).
// KDA has no scalar decay to fold (its images carry the decays): MMA2 is [128 x 64], the epilogue rounds V'^T to
// nearest in place (E2) and MMA4 reads that.
// TMEM columns: S 0..127, D1 128..255, D2 256..383, D3[0] 384..447, D3[1] 448..511.
//
// Warps: 0 = bulk-copy producer, 1 = MMA issuer (and TMEM owner), 2..9 = two epilogue warpgroups that
// split the columns of every accumulator between them (a warp may only touch TMEM lanes 32*(warp%4)..+31),
// 10 = V loader (global rows of any alignment -> shared memory, one chunk ahead), 11 = output storer
// (bulk stores of the chunk's output rows from shared memory), 12..15 = scalers: they form T' from T in shared
// memory (GDN) and rescale the state between MMA1 and MMA4 of a chunk when that is due (KDA: every chunk, per key
// channel; GDN: only when the lazy scale runs out of range), off the epilogue warps' timeline.
constexpr uint32_t COL_S = 0, COL_D1 = 128, COL_D2 = 256, COL_D3 = 384;
constexpr uint32_t kWaitLimit = 1u << 20;

// Optional phase timestamps of chain CTA 0 (development builds only: -DPLA_B200_DEBUG_CLOCKS).
#ifdef PLA_B200_DEBUG_CLOCKS
__device__ long long g_dbg_clock[2][16][16];
#define DBG_CLOCK(role, c, k) \
  do { if (blockIdx.x == 0 && (c) < 16) g_dbg_clock[role][c][k] = clock64(); } while (0)
#else
#define DBG_CLOCK(role, c, k) do {} while (0)
#endif
constexpr int CHAIN_THREADS = 512;
constexpr int E_THREADS = 256;
constexpr int V_PITCH = 136;  // halfwords per staged V row: 128 + room for one leading / trailing halfword, 16-byte multiple

struct ChainSmem {
  alignas(1024) float kq[KQ_BYTES / 4];
  alignas(1024) float knt[KNT_BYTES / 4];
  alignas(1024) float tm[2 * TM_BYTES / 4];   // [column group][128 rows][4]: rows 0..63 T, rows 64..127 T'
  alignas(1024) float pm[PM_BYTES / 4];
  alignas(16) float vec[2][VEC_BYTES / 4];
  alignas(128) unsigned short v[2][C * V_PITCH];   // raw 16-bit V rows of a chunk, double-buffered
  alignas(128) unsigned short o[C * D];      // output rows of a chunk, 16-bit
  alignas(8) uint64_t full_kq, full_t, full_p, full_k, full_vec[2];
  uint64_t v_full[2], v_free[2], o_full, o_free;
  uint64_t mma1_done, mma2_done, mma3_done, mma4_done;
  uint64_t s_ready, a2_ready, a4_ready, tprime_ready, s_scaled;
  uint32_t tmem_base;
  volatile int abort;
};

// Lazy state scaling (GDN, scalar decay per chunk). Tensor-memory loads and stores are the scarce resource of
// this kernel (about 100 bytes per cycle and SM), and multiplying the whole 64 KiB state by e^{G_C} every chunk
// was 40 % of that traffic. Instead the accumulator holds S / sigma for a scalar sigma that every role tracks
// from the chunk vectors: reads of the state (MMA1's results) are multiplied by sigma in the epilogues that
// touch them anyway, the update operand A4 is divided by the new sigma, and the stored state is only touched
// when sigma would leave [2^-40, 1] -- or not at all when the chunk's own decay is below 2^-40, where the
// update simply overwrites the state (the dropped term is below fp32 resolution).
constexpr float kSigmaFloor = 9.094947e-13f;   // 2^-40
enum : int { kLazy = 0, kOverwrite = 1, kRescale = 2 };
struct LazyScale {
  float sigma = 1.0f;     // true state = sigma * accumulator
  // One chunk with total decay `gamma`: returns the mode; `read` scales this chunk's reads of the state, `a4` its
  // update operand, `factor` is what a kRescale pass multiplies the accumulator by before the update.
  __device__ __forceinline__ int step(float gamma, float& read, float& a4, float& factor) {
    read = sigma;
    a4 = 1.0f;
    factor = 1.0f;
    if (!(gamma >= kSigmaFloor)) {   // also catches a decay that underflowed to zero
      sigma = 1.0f;
      return kOverwrite;
    }
    const float next = sigma * gamma;
    if (next < kSigmaFloor) {
      factor = next;
      sigma = 1.0f;
      return kRescale;
    }
    sigma = next;
    a4 = __fdividef(1.0f, next);
    return kLazy;
  }
};

// Bounded wait that also gives up when another role has already given up.
__device__ __forceinline__ bool chain_wait(ChainSmem& sh, uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u && sh.abort) return false;
  }
  sh.abort = 1;
  return false;
}

template <typename act_t>
__global__ void __launch_bounds__(CHAIN_THREADS, 1) gdn_chunk_chain_kernel(const pla_b200_gdn_chunk_args p) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem_raw = smem_dyn + ((1024u - (smem_addr(smem_dyn) & 1023u)) & 1023u);
  ChainSmem& sh = *reinterpret_cast<ChainSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // Prescan mode (context parallelism): every (sequence, value head) runs two chains that store no
  // output, kind 0 from a zero state over the real V (the segment's offset B) and kind 1 from the
  // identity over V = 0 (the segment's transition M), so that  S_out = S_in M + B  row by row.
  const bool prescan = p.prescan != 0;
  const unsigned chains = static_cast<unsigned>(p.N) * p.HV * (prescan ? 2u : 1u);
  if (blockIdx.x >= chains) {
    if (prescan) return;
    // trailing CTAs: physical token rows past the last sequence get zero output
    const int64_t first = p.cu_seqlens[p.N];
    const int64_t words = (p.T_total - first) * p.HV * (D / 2);
    if (first < 0 || words <= 0) return;
    uint32_t* dst = reinterpret_cast<uint32_t*>(static_cast<act_t*>(p.o) + first * p.HV * D);
    for (int64_t i = static_cast<int64_t>(blockIdx.x - chains) * CHAIN_THREADS + tid; i < words;
         i += static_cast<int64_t>(gridDim.x - chains) * CHAIN_THREADS)
      dst[i] = 0u;
    return;
  }
  const int kind = prescan ? static_cast<int>(blockIdx.x & 1u) : 0;
  const unsigned chain = prescan ? blockIdx.x >> 1 : blockIdx.x;
  int seq = chain / p.HV;
  const int hv = chain % p.HV;
  // Longest sequences first: CTAs start roughly in block order and a chain's run time is its chunk
  // count, so the block index is mapped through the sequences sorted by descending length (for
  // batches small enough to rank in place).
  if (p.N > 1 && p.N <= CHAIN_THREADS) {
    __shared__ int picked;
    if (tid < p.N) {
      const int mine = max(p.cu_seqlens[tid + 1] - p.cu_seqlens[tid], 0);
      int rank = 0;
      for (int s = 0; s < p.N; ++s) {
        const int other = max(p.cu_seqlens[s + 1] - p.cu_seqlens[s], 0);
        rank += (other > mine) || (other == mine && s < tid);
      }
      if (rank == seq) picked = tid;
    }
    __syncthreads();
    seq = picked;
  }
  const int h = hv / (p.HV / p.H);
  const int64_t bos = p.cu_seqlens[seq];
  const int len = p.cu_seqlens[seq + 1] - static_cast<int>(bos);
  if (bos < 0 || len <= 0) return;
  const int nch = (len + C - 1) / C;
  const int gc0 = first_chunk_of(p.cu_seqlens, seq);

  int slot = seq;
  if (p.slot_indices != nullptr && !prescan) slot = p.slot_indices[seq];
  if (prescan && p.slot_indices != nullptr && p.slot_indices[seq] < 0) return;   // pair of this range not wanted
  act_t* o_col = static_cast<act_t*>(p.o) + static_cast<int64_t>(hv) * D;  // + tok*HV*D + v
  if (!prescan && p.slot_indices != nullptr && (slot < 0 || (p.num_slots > 0 && slot >= p.num_slots))) {
    if (slot >= 0 && tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_BAD_SLOT);
    for (int i = tid; i < len * D; i += CHAIN_THREADS) o_col[(bos + i / D) * p.HV * D + (i % D)] = from_f32<act_t>(0.f);
    return;
  }

  if (tid == 0) {
    mbar_init(&sh.full_kq, 1);
    mbar_init(&sh.full_t, 1);
    mbar_init(&sh.full_p, 1);
    mbar_init(&sh.full_k, 1);
    mbar_init(&sh.full_vec[0], 1);
    mbar_init(&sh.full_vec[1], 1);
    mbar_init(&sh.mma1_done, 1);
    mbar_init(&sh.mma2_done, 1);
    mbar_init(&sh.mma3_done, 1);
    mbar_init(&sh.mma4_done, 1);
    mbar_init(&sh.s_ready, E_THREADS);
    mbar_init(&sh.a2_ready, E_THREADS);
    mbar_init(&sh.tprime_ready, 128);
    mbar_init(&sh.a4_ready, E_THREADS);
    mbar_init(&sh.s_scaled, 128);
    mbar_init(&sh.v_full[0], 32);
    mbar_init(&sh.v_full[1], 32);
    mbar_init(&sh.v_free[0], E_THREADS);
    mbar_init(&sh.v_free[1], E_THREADS);
    mbar_init(&sh.o_full, E_THREADS);
    mbar_init(&sh.o_free, 1);
    sh.abort = 0;
    fence_mbar_init();
  }
  // rows of the T, T' and P images above their triangular pieces: zero for the whole run (nothing ever writes them)
  for (int i = tid; i < (2 * TM_BYTES + PM_BYTES) / 16; i += CHAIN_THREADS)
    (i < 2 * TM_BYTES / 16 ? reinterpret_cast<uint4*>(sh.tm)[i] : reinterpret_cast<uint4*>(sh.pm)[i - 2 * TM_BYTES / 16]) =
        make_uint4(0u, 0u, 0u, 0u);
  fence_async_smem();
  if (warp == 1) tc05::tmem_alloc(&sh.tmem_base, 512);
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tb = sh.tmem_base;
  const unsigned char* ws = static_cast<const unsigned char*>(p.workspace);

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      auto load_kq = [&](int c) {
        mbar_expect_tx(&sh.full_kq, KQ_BYTES);
        bulk_load(sh.kq, ws + ws_hblob(gc0 + c, h, p.H), KQ_BYTES, &sh.full_kq);
      };
      // T (and, for GDN, P) come back as the sixteen pieces of their lower triangles; the rows above the pieces
      // were zeroed once when the CTA started. `rows` = rows per column group of the image in shared memory.
      auto load_tri = [&](float* dst, int rows, const unsigned char* src, uint64_t* bar) {
#pragma unroll 1
        for (int jg = 0; jg < C / 4; ++jg)
          bulk_load(reinterpret_cast<unsigned char*>(dst) + (jg * rows + 4 * jg) * 16, src + tri_piece_offset(jg),
                    tri_piece_bytes(jg), bar);
      };
      auto load_t = [&](int c) {
        mbar_expect_tx(&sh.full_t, TRI_BYTES);
        load_tri(sh.tm, 2 * C, ws + ws_vblob(p.max_chunks, p.H, p.HV, gc0 + c, hv), &sh.full_t);
      };
      auto load_p = [&](int c) {
        mbar_expect_tx(&sh.full_p, TRI_BYTES);
        load_tri(sh.pm, C, ws + ws_vblob(p.max_chunks, p.H, p.HV, gc0 + c, hv) + TM_BYTES, &sh.full_p);
      };
      auto load_k = [&](int c) {
        mbar_expect_tx(&sh.full_k, KNT_BYTES);
        bulk_load(sh.knt, ws + ws_hblob(gc0 + c, h, p.H) + KQ_BYTES, KNT_BYTES, &sh.full_k);
      };
      auto load_vec = [&](int c) {
        mbar_expect_tx(&sh.full_vec[c & 1], VEC_BYTES);
        bulk_load(sh.vec[c & 1], ws + ws_vblob(p.max_chunks, p.H, p.HV, gc0 + c, hv) + TM_BYTES + PM_BYTES, VEC_BYTES,
                  &sh.full_vec[c & 1]);
      };
      load_vec(0);
      load_kq(0);
      load_t(0);
      load_k(0);
      load_p(0);
      if (nch > 1) load_vec(1);

      // every buffer is refilled as soon as the last MMA that reads it has finished; the events of a chunk come in
      // the order MMA1(c), MMA3(c - 1), MMA2(c), MMA4(c)
      for (int c = 0; c < nch; ++c) {
        const uint32_t ph = c & 1;
        if (!chain_wait(sh, &sh.mma1_done, ph)) break;
        if (c + 1 < nch) load_kq(c + 1);
        if (c >= 1) {
          if (!chain_wait(sh, &sh.mma3_done, ph ^ 1)) break;
          load_p(c);
        }
        if (!chain_wait(sh, &sh.mma2_done, ph)) break;   // T, T' and this chunk's vectors have been consumed
        if (c + 1 < nch) load_t(c + 1);
        if (c + 2 < nch) load_vec(c + 2);
        if (!chain_wait(sh, &sh.mma4_done, ph)) break;
        if (c + 1 < nch) load_k(c + 1);
      }
      if (sh.abort) {
        // copies may still be in flight into this CTA's shared memory: bounded wait for each
        (void)mbar_wait(&sh.full_kq, 0, 1u << 16);
        (void)mbar_wait(&sh.full_kq, 1, 1u << 16);
        (void)mbar_wait(&sh.full_k, 0, 1u << 16);
        (void)mbar_wait(&sh.full_k, 1, 1u << 16);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint64_t kq_desc = tc05::smem_desc(sh.kq, 128 * 16, 128);
      const uint64_t t_desc = tc05::smem_desc(sh.tm, 128 * 16, 128);    // [T; T']: 128 rows per column group
      const uint64_t p_desc = tc05::smem_desc(sh.pm, 64 * 16, 128);
      const uint64_t knt_desc = tc05::smem_desc(sh.knt, 128 * 16, 128);
      constexpr uint32_t i128 = tc05::idesc_tf32(128, 128), i64 = tc05::idesc_tf32(128, 64);
      const uint32_t d1 = tb + COL_D1, d2 = tb + COL_D2;
      bool ok = chain_wait(sh, &sh.s_ready, 0);
      LazyScale lazy;
      const bool kda_m = p.is_kda != 0;
      // intra-chunk output of chunk c: D3[c & 1] += V'^T x P^T, on the accumulator half that E1 seeded
      auto mma3 = [&](int c) {
#pragma unroll
        for (int j = 0; j < C / 8; ++j)
          tc05::mma_tf32_ts(tb + COL_D3 + (c & 1) * 64, d2 + j * 8, tc05::desc_advance(p_desc, j * 2 * 64 * 16), i64, true);
        tc05::mma_commit(&sh.mma3_done);
      };
      for (int c = 0; c < nch && ok; ++c) {
        const uint32_t ph = c & 1;
        if (!(ok = chain_wait(sh, &sh.full_vec[ph], (c >> 1) & 1))) break;
        float rd, a4s, fac;
        const int mode = kda_m ? kRescale : lazy.step(sh.vec[ph][2 * C + C - 1], rd, a4s, fac);
        if (!(ok = chain_wait(sh, &sh.full_kq, ph))) break;
        tc05::fence_after_sync();
        DBG_CLOCK(0, c, 0);
#pragma unroll
        for (int j = 0; j < D / 8; ++j)
          tc05::mma_tf32_ts(d1, tb + COL_S + j * 8, tc05::desc_advance(kq_desc, j * 2 * 128 * 16), i128, j > 0);
        tc05::mma_commit(&sh.mma1_done);
        DBG_CLOCK(0, c, 1);
        // the previous chunk's MMA3 runs under this chunk's E1 (its operands: D2 as MMA2 left it, P still in place)
        if (c >= 1) {
          if (!(ok = chain_wait(sh, &sh.full_p, ph ^ 1))) break;
          mma3(c - 1);
        }
        if (!(ok = chain_wait(sh, &sh.a2_ready, ph) && chain_wait(sh, kda_m ? &sh.full_t : &sh.tprime_ready, ph))) break;
        tc05::fence_after_sync();
        DBG_CLOCK(0, c, 2);
        // D2 = W^T x [T; T']^T: V'^T in columns 0..63 and, for GDN, the decayed V'^T in 64..127
#pragma unroll
        for (int j = 0; j < C / 8; ++j)
          tc05::mma_tf32_ts(d2, d1 + j * 8, tc05::desc_advance(t_desc, j * 2 * 128 * 16), kda_m ? i64 : i128, j > 0);
        tc05::mma_commit(&sh.mma2_done);
        DBG_CLOCK(0, c, 3);
        if (!(ok = chain_wait(sh, &sh.full_k, ph) && chain_wait(sh, &sh.s_scaled, ph))) break;
        if (kda_m && !(ok = chain_wait(sh, &sh.a4_ready, ph))) break;   // V'^T rounded in place (below)
        tc05::fence_after_sync();
        DBG_CLOCK(0, c, 4);
#pragma unroll
        for (int j = 0; j < C / 8; ++j)
          tc05::mma_tf32_ts(tb + COL_S, d2 + (kda_m ? 0 : C) + j * 8, tc05::desc_advance(knt_desc, j * 2 * 128 * 16), i128,
                            mode != kOverwrite || j > 0);
        tc05::mma_commit(&sh.mma4_done);
        DBG_CLOCK(0, c, 5);
      }
      if (ok && chain_wait(sh, &sh.full_p, (nch - 1) & 1)) mma3(nch - 1);
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------------ V loader
    // Asynchronous copies (no register staging) of the chunk's 64 V rows, one chunk ahead. A row
    // of any 2-byte alignment is fetched as the 16 or 17 aligned 16-byte pieces that overlap it; it
    // then starts (address % 16) / 2 halfwords into its staged copy (the epilogue adds the same
    // shift). Up to 14 bytes before and after the row are read as well, always from a 16-byte
    // granule that the row itself occupies.
    const unsigned short* vbase = reinterpret_cast<const unsigned short*>(p.v) + static_cast<int64_t>(hv) * D;
    for (int c = 0; c < nch; ++c) {
      const int b = c & 1;
      if (c >= 2 && !chain_wait(sh, &sh.v_free[b], ((c >> 1) - 1) & 1)) break;
      if (lane == 0) DBG_CLOCK(0, c, 6);
      const int n = kind == 1 ? 0 : min(C, len - c * C);
      unsigned short* dst = sh.v[b];
      // lane l copies rows l and l + 32: 17 aligned 16-byte pieces that cover each 256-byte row
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int r = lane + 32 * k;
        const unsigned short* row = vbase + (bos + static_cast<int64_t>(c) * C + r) * p.v_tok_stride;
        const uint32_t d = smem_addr(dst + r * V_PITCH);
        if (r >= n) {
          uint4* z = reinterpret_cast<uint4*>(dst + r * V_PITCH);
#pragma unroll
          for (int i = 0; i < 17; ++i) z[i] = make_uint4(0u, 0u, 0u, 0u);
        } else {
          const char* src = reinterpret_cast<const char*>(reinterpret_cast<uintptr_t>(row) & ~uintptr_t(15));
          // an aligned row ends with its 16th piece; the 17th would lie wholly outside the row
          const int pieces = src == reinterpret_cast<const char*>(row) ? 16 : 17;
#pragma unroll
          for (int i = 0; i < 17; ++i)
            if (i < pieces)
              asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d + i * 16), "l"(src + i * 16) : "memory");
        }
      }
      if (n < C) __threadfence_block();  // the zero rows above are plain stores
      // counts as this lane's arrival once all of its copies above have landed
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(&sh.v_full[b])) : "memory");
      if (lane == 0) DBG_CLOCK(0, c, 7);
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (warp == 11) {
    // ------------------------------------------------------------------ output storer
    // 256-byte output rows from shared memory, two rows per warp instruction (16 bytes per lane).
    for (int c = 0; c < nch; ++c) {
      if (!chain_wait(sh, &sh.o_full, c & 1)) break;
      const int n = prescan ? 0 : min(C, len - c * C);
      act_t* orow = o_col + (bos + static_cast<int64_t>(c) * C) * p.HV * D;
      const uint4* src = reinterpret_cast<const uint4*>(sh.o);
#pragma unroll 8
      for (int r2 = 0; r2 < C / 2; ++r2) {
        const int r = r2 * 2 + (lane >> 4);
        if (r < n) reinterpret_cast<uint4*>(orow + static_cast<int64_t>(r) * p.HV * D)[lane & 15] = src[r * 16 + (lane & 15)];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.o_free);
    }
  } else if (warp >= 12) {
    // ------------------------------------------------------------------ scalers (128 threads)
    // GDN: T' = diag(e^{G_C - G} / sigma_new) T into rows 64..127 of the [T; T'] image (thread = (row, half of the
    // column groups); rounded to nearest, since T' carries the state update); then, when the lazy scale is due,
    // S *= factor once MMA1 of the chunk has read S. KDA: S *= e^{G_C}[k] per key channel (vec[128 + k]) every
    // chunk. MMA2 waits for T', MMA4 for the rescaled state.
    const uint32_t tS = tb + (static_cast<uint32_t>((warp & 3) * 32) << 16) + COL_S;
    const bool kda = p.is_kda != 0;
    const int t7 = tid - 12 * 32, trow = t7 & 63, thalf = t7 >> 6;
    LazyScale lazy;
    for (int c = 0; c < nch; ++c) {
      const uint32_t ph = c & 1;
      const float* vec = sh.vec[ph];
      if (!chain_wait(sh, &sh.full_vec[ph], (c >> 1) & 1)) break;
      float rd, a4s = 1.0f, fac = 1.0f;
      const int mode = kda ? kRescale : lazy.step(vec[2 * C + C - 1], rd, a4s, fac);
      if (!kda) {
        if (!chain_wait(sh, &sh.full_t, ph)) break;
        const float d = vec[3 * C + trow] * a4s;
        float4* t4 = reinterpret_cast<float4*>(sh.tm);
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const int jg = thalf * 8 + jj;
          if (4 * jg > trow) continue;          // above the column group's piece: zero in both images
          float4 x = t4[jg * 2 * C + trow];
          x.x = tc05::to_tf32(x.x * d); x.y = tc05::to_tf32(x.y * d); x.z = tc05::to_tf32(x.z * d); x.w = tc05::to_tf32(x.w * d);
          t4[jg * 2 * C + C + trow] = x;
        }
        fence_async_smem();                     // read by the tensor core (async proxy)
        mbar_arrive(&sh.tprime_ready);
      }
      if (!chain_wait(sh, &sh.mma1_done, ph)) break;
      tc05::fence_after_sync();
      if (mode == kRescale) {       // KDA: every chunk, per key channel; GDN: only when sigma runs out of range
#pragma unroll 1
        for (int q4 = 0; q4 < 4; ++q4) {
          float s[32];
          tc05::tmem_ld32(tS + q4 * 32, s);
          tc05::wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) s[j] *= kda ? vec[2 * C + q4 * 32 + j] : fac;
          tc05::tmem_st32(tS + q4 * 32, s);
        }
        tc05::wait_st();
      }
      tc05::fence_before_sync();
      mbar_arrive(&sh.s_scaled);
    }
  } else {
    // ------------------------------------------------------------------ epilogue warpgroups (2 x 128 threads)
    const int quad = warp & 3;
    const int m = quad * 32 + lane;               // value index v owned by this thread
    const int wg = (warp - 2) >> 2;               // 0: token columns 0..31 and key columns 0..63; 1: the rest
    const int cg = wg * 32;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tS = tb + lane_base + COL_S, tD2 = tb + lane_base + COL_D2, tD3 = tb + lane_base + COL_D3;
    const bool f32_state = p.state_dtype == PLA_B200_F32;
    // KDA: the decay factors are folded into the operand images, so E1 / E2 / E3 apply none and the
    // state is rescaled per key channel (vec[128 + k] = e^{G_C}[k]).
    const bool kda = p.is_kda != 0;

    // initial state row v = m -> TMEM (fp32)
    {
      const int64_t in_base = static_cast<int64_t>(slot) * p.state_slot_stride + static_cast<int64_t>(hv) * TILE;
#pragma unroll 1
      // fp32 k-last tiles (the usual case): this thread's row is contiguous, eight 16-byte loads per 32 columns
      // instead of 32 scalar ones (a warp instruction touches 32 lines either way)
      const bool vec_state = f32_state && !p.state_transposed && !prescan && !p.state_init_zero &&
                             ((reinterpret_cast<uintptr_t>(p.state) | static_cast<uintptr_t>(p.state_slot_stride * 4)) & 15) == 0;
      for (int q4 = 2 * wg; q4 < 2 * wg + 2; ++q4) {
        float s[32];
        if (vec_state) {
          const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(p.state) + in_base +
                                                              static_cast<int64_t>(m) * D + q4 * 32);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 x = __ldg(src + j);
            s[4 * j] = x.x; s[4 * j + 1] = x.y; s[4 * j + 2] = x.z; s[4 * j + 3] = x.w;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int kx = q4 * 32 + j;
            s[j] = prescan ? (kind == 1 && kx == m ? 1.0f : 0.0f)
                   : p.state_init_zero
                       ? 0.0f
                       : load_any(p.state, p.state_dtype,
                                                in_base + (p.state_transposed ? static_cast<int64_t>(kx) * D + m
                                                                              : static_cast<int64_t>(m) * D + kx));
          }
        }
        tc05::tmem_st32(tS + q4 * 32, s);
      }
      tc05::wait_st();
      tc05::fence_before_sync();
      mbar_arrive(&sh.s_ready);
    }

    bool ok = true;
    LazyScale lazy;
    const uint32_t tD1 = tb + lane_base + COL_D1;
    // E3: output rows of chunk c, once its MMA3 has added the intra-chunk part to what E1 left in D3[c & 1]
    auto e3 = [&](int c) -> bool {
      if (!chain_wait(sh, &sh.mma3_done, c & 1)) return false;
      tc05::fence_after_sync();
      if (m == 0 && wg == 0) DBG_CLOCK(1, c, 6);
      float d3[32];
      tc05::tmem_ld32(tD3 + (c & 1) * 64 + cg, d3);
      if (c >= 1 && !chain_wait(sh, &sh.o_free, (c - 1) & 1)) return false;  // previous rows stored
      tc05::wait_ld();
      act_t* so = reinterpret_cast<act_t*>(sh.o);
#pragma unroll
      for (int j = 0; j < 32; ++j) so[(cg + j) * D + m] = from_f32<act_t>(d3[j]);
      mbar_arrive(&sh.o_full);  // the storer reads with ordinary loads: no proxy fence needed
      if (m == 0 && wg == 0) DBG_CLOCK(1, c, 7);
      return true;
    };
    for (int c = 0; c < nch && ok; ++c) {
      const uint32_t ph = c & 1;
      const int n = min(C, len - c * C);
      const float* vec = sh.vec[ph];
      if (!(ok = chain_wait(sh, &sh.full_vec[ph], (c >> 1) & 1))) break;
      float rd = 1.0f, a4s = 1.0f, fac;
      if (!kda) (void)lazy.step(vec[2 * C + C - 1], rd, a4s, fac);
      if (m == 0 && wg == 0) DBG_CLOCK(1, c, 3);
      if (!(ok = chain_wait(sh, &sh.v_full[ph], (c >> 1) & 1))) break;
      const act_t* vrows = reinterpret_cast<const act_t*>(sh.v[ph]);
      // halfword shift of token (cg + j)'s staged row = (element address of the row) mod 8
      const int64_t v_e0 = static_cast<int64_t>(reinterpret_cast<uintptr_t>(p.v) >> 1) + static_cast<int64_t>(hv) * D +
                           (bos + static_cast<int64_t>(c) * C + cg) * p.v_tok_stride;
      const int v_sh0 = static_cast<int>(v_e0 & 7), v_shs = static_cast<int>(p.v_tok_stride & 7);
      // this thread's V elements of the chunk, fetched while MMA1 still runs
      float w[32];
      if (v_shs == 0) {
        const act_t* vcol = vrows + cg * V_PITCH + v_sh0 + m;
#pragma unroll
        for (int j = 0; j < 32; ++j) w[j] = to_f32(vcol[j * V_PITCH]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) w[j] = to_f32(vrows[(cg + j) * V_PITCH + ((v_sh0 + j * v_shs) & 7) + m]);
      }
      if (!(ok = chain_wait(sh, &sh.mma1_done, ph))) break;
      tc05::fence_after_sync();
      if (m == 0 && wg == 0) DBG_CLOCK(1, c, 1);
      // ---- E1: W^T = beta V^T - (beta e^G) (Kn S)^T over (Kn S)^T. This code is bound by instruction issue
      // (two epilogue warps per scheduler): coefficients come as 128-bit broadcast loads, the V element needs no
      // address arithmetic when every row of the chunk has the same alignment shift (token stride a multiple
      // of 16 bytes) and is fetched before MMA1 is waited for; then one multiply, one multiply-add and one integer
      // add (rounding) per element. ----
      {
        float x[32];
        tc05::tmem_ld32(tD1 + cg, x);
        const float4* be4 = reinterpret_cast<const float4*>(vec + cg);        // beta e^G (KDA: beta)
        const float4* b4 = reinterpret_cast<const float4*>(vec + C + cg);     // beta
        tc05::wait_ld();
        if (m == 0 && wg == 0) DBG_CLOCK(1, c, 8);
#pragma unroll
        for (int j4 = 0; j4 < 8; ++j4) {
          float4 be = be4[j4];
          const float4 b = b4[j4];
          be.x *= rd; be.y *= rd; be.z *= rd; be.w *= rd;     // the accumulator holds S / sigma
          x[4 * j4 + 0] = tc05::pre_round_tf32(fmaf(-be.x, x[4 * j4 + 0], b.x * w[4 * j4 + 0]));
          x[4 * j4 + 1] = tc05::pre_round_tf32(fmaf(-be.y, x[4 * j4 + 1], b.y * w[4 * j4 + 1]));
          x[4 * j4 + 2] = tc05::pre_round_tf32(fmaf(-be.z, x[4 * j4 + 2], b.z * w[4 * j4 + 2]));
          x[4 * j4 + 3] = tc05::pre_round_tf32(fmaf(-be.w, x[4 * j4 + 3], b.w * w[4 * j4 + 3]));
        }
        if (m == 0 && wg == 0) DBG_CLOCK(1, c, 9);
        tc05::tmem_st32(tD1 + cg, x);
      }
      // ---- ... and the part of the output rows that comes from the incoming state, e^G (Qn S)^T, into the
      // accumulator that MMA3 adds the intra-chunk part to. (KDA: the decay is in the operand images.) ----
      {
        float qs[32];
        tc05::tmem_ld32(tD1 + 64 + cg, qs);
        tc05::wait_ld();
        if (!kda) {
          const float4* e4 = reinterpret_cast<const float4*>(vec + 2 * C + cg);   // e^G
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            float4 e = e4[j4];
            e.x *= rd; e.y *= rd; e.z *= rd; e.w *= rd;
            qs[4 * j4 + 0] *= e.x;
            qs[4 * j4 + 1] *= e.y;
            qs[4 * j4 + 2] *= e.z;
            qs[4 * j4 + 3] *= e.w;
          }
        }
        tc05::tmem_st32(tD3 + ph * 64 + cg, qs);
      }
      tc05::wait_st();
      if (m == 0 && wg == 0) DBG_CLOCK(1, c, 10);
      tc05::fence_before_sync();
      mbar_arrive(&sh.a2_ready);
      if (m == 0 && wg == 0) DBG_CLOCK(1, c, 2);
      mbar_arrive(&sh.v_free[ph]);
      // ---- E2, KDA only: V'^T is rounded to nearest where MMA2 left it before MMA4 reads it. Its update operand
      // carries per-channel decays of up to e^80 in the images, and the products of hundreds of such transitions
      // (the context-parallel pairs) feel the tensor core's truncation; GDN's scalar-decay update does not. ----
      if (kda) {
        if (!(ok = chain_wait(sh, &sh.mma2_done, ph))) break;
        tc05::fence_after_sync();
        float x[32];
        tc05::tmem_ld32(tD2 + cg, x);
        tc05::wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) x[j] = tc05::pre_round_tf32(x[j]);
        tc05::tmem_st32(tD2 + cg, x);
        tc05::wait_st();
        tc05::fence_before_sync();
        mbar_arrive(&sh.a4_ready);
      }
      // the previous chunk's output rows: its MMA3 was issued behind this chunk's MMA1
      if (c >= 1 && !(ok = e3(c - 1))) break;
    }
    if (ok) ok = e3(nch - 1);
    // the state is final once the last MMA4 has landed
    if (ok) ok = chain_wait(sh, &sh.mma4_done, (nch - 1) & 1);
    tc05::fence_after_sync();

    // ---- final state ----
    if (ok && prescan) {
      // [sequence][value head][offset, transition][v][k] fp32
      float* dst = static_cast<float*>(p.state_out) + ((static_cast<int64_t>(seq) * p.HV + hv) * 2 + kind) * TILE +
                   static_cast<int64_t>(m) * D;
#pragma unroll 1
      for (int q4 = 2 * wg; q4 < 2 * wg + 2; ++q4) {
        float s[32];
        tc05::tmem_ld32(tS + q4 * 32, s);
        tc05::wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) s[j] *= lazy.sigma;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + q4 * 32 + j) = make_float4(s[j], s[j + 1], s[j + 2], s[j + 3]);
      }
    } else if (ok && p.write_state) {
      void* dst = p.state;
      int64_t base = static_cast<int64_t>(slot) * p.state_slot_stride;
      bool store = true;
      if (p.state_out != nullptr) {
        const int64_t oslot = p.state_out_indices != nullptr ? p.state_out_indices[seq] : seq;
        store = oslot >= 0;                  // a negative destination: this chain's final state is not wanted
        dst = p.state_out;
        base = oslot * p.state_out_slot_stride;
      }
      base += static_cast<int64_t>(hv) * TILE;
#pragma unroll 1
      for (int q4 = 2 * wg; store && q4 < 2 * wg + 2; ++q4) {
        float s[32];
        tc05::tmem_ld32(tS + q4 * 32, s);
        tc05::wait_ld();
        if (f32_state && !p.state_transposed && (reinterpret_cast<uintptr_t>(static_cast<float*>(dst) + base) & 15) == 0) {
          float4* out4 = reinterpret_cast<float4*>(static_cast<float*>(dst) + base + static_cast<int64_t>(m) * D + q4 * 32);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            out4[j] = make_float4(s[4 * j] * lazy.sigma, s[4 * j + 1] * lazy.sigma, s[4 * j + 2] * lazy.sigma,
                                  s[4 * j + 3] * lazy.sigma);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int kx = q4 * 32 + j;
            const int64_t e = base + (p.state_transposed ? static_cast<int64_t>(kx) * D + m : static_cast<int64_t>(m) * D + kx);
            if (f32_state) static_cast<float*>(dst)[e] = s[j] * lazy.sigma;
            else static_cast<__nv_bfloat16*>(dst)[e] = __float2bfloat16_rn(s[j] * lazy.sigma);
          }
        }
      }
    }
  }

  if (sh.abort && tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_WAIT_TIMEOUT);
  tc05::fence_before_sync();
  __syncthreads();
  if (warp == 1) tc05::tmem_dealloc(tb, 512);
}

}  // namespace
}  // namespace pla

extern "C" int64_t pla_b200_gdn_chunk_workspace_bytes(int32_t max_chunks, int32_t H, int32_t HV) {
  if (max_chunks < 0 || H <= 0 || HV <= 0) return 0;
  return static_cast<int64_t>(max_chunks) *
         (static_cast<int64_t>(H) * pla::HBLOB + static_cast<int64_t>(HV) * (pla::VBLOB + pla::L_BYTES));
}

namespace pla {
namespace {

int check_chunk_args(const pla_b200_gdn_chunk_args& a, int64_t need_bytes) {
  PLA_REQUIRE(a.N > 0 && a.T_total >= 0 && a.max_chunks >= 0, PLA_B200_E_INVALID, "N, T_total, max_chunks out of range");
  PLA_REQUIRE(a.H > 0 && a.HV >= a.H && a.HV % a.H == 0, PLA_B200_E_INVALID,
              "HV must be a positive multiple of H, got H=%d, HV=%d", a.H, a.HV);
  PLA_REQUIRE(a.q && a.k && a.v && a.gate && a.beta && a.o && a.cu_seqlens, PLA_B200_E_INVALID,
              "q, k, v, gate, beta, o and cu_seqlens are required");
  PLA_REQUIRE(a.gate_activated || (a.A_log && a.dt_bias), PLA_B200_E_INVALID, "raw gating needs A_log and dt_bias");
  PLA_REQUIRE(a.act_dtype == PLA_B200_BF16 || a.act_dtype == PLA_B200_F16, PLA_B200_E_INVALID,
              "activation dtype must be bf16 or fp16");
  PLA_REQUIRE(a.workspace != nullptr && (reinterpret_cast<uintptr_t>(a.workspace) & 127) == 0 &&
                  a.workspace_bytes >= need_bytes,
              PLA_B200_E_INVALID, "workspace missing, not 128-byte aligned or too small");
  PLA_REQUIRE(a.stage >= 0 && a.stage <= 2, PLA_B200_E_INVALID, "stage must be 0, 1 or 2");
  PLA_REQUIRE(static_cast<int64_t>(a.max_chunks) * a.H < (1ll << 31), PLA_B200_E_TOO_LARGE, "too many chunks");
  return PLA_B200_OK;
}

int launch_chain_stage(const pla_b200_gdn_chunk_args& a, cudaStream_t s) {
  if (a.prescan) {
    PLA_REQUIRE(a.state_out != nullptr && aligned16(a.state_out), PLA_B200_E_INVALID,
                "prescan needs a 16-byte aligned state_out of [N, HV, 2, 128, 128] fp32");
  } else {
    PLA_REQUIRE(a.state_init_zero || a.state != nullptr, PLA_B200_E_INVALID,
                "an initial state or state_init_zero is required");
    PLA_REQUIRE(a.slot_indices != nullptr || a.state_by_request, PLA_B200_E_INVALID, "slot indices are required");
    PLA_REQUIRE(!a.write_state || a.state_out != nullptr || a.state != nullptr, PLA_B200_E_INVALID,
                "a final state needs somewhere to go");
  }
  PLA_REQUIRE(aligned16(a.o), PLA_B200_E_ALIGN, "o must be 16-byte aligned");
  auto launch_chain = [&](auto kern) -> int {
    // one flag per kernel instantiation: both dtypes share this lambda's body (same function-pointer type)
    static DeviceOnce configured_by_dtype[2];
    DeviceOnce& configured = configured_by_dtype[a.act_dtype == PLA_B200_BF16 ? 0 : 1];
    int dev = 0;
    PLA_CUDA_OK(cudaGetDevice(&dev));
    if (configured.needed(dev)) {
      PLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(ChainSmem) + 1024)));
      configured.mark(dev);
    }
    const int64_t ctas = a.prescan ? static_cast<int64_t>(a.N) * a.HV * 2 : static_cast<int64_t>(a.N) * a.HV + 32;
    PLA_REQUIRE(ctas < (1ll << 31), PLA_B200_E_TOO_LARGE, "N*HV exceeds the grid limit");
    kern<<<static_cast<unsigned>(ctas), CHAIN_THREADS, sizeof(ChainSmem) + 1024, s>>>(a);
    PLA_CUDA_OK(cudaGetLastError());
    return PLA_B200_OK;
  };
  return a.act_dtype == PLA_B200_BF16 ? launch_chain(gdn_chunk_chain_kernel<__nv_bfloat16>)
                                      : launch_chain(gdn_chunk_chain_kernel<__half>);
}

}  // namespace
}  // namespace pla

extern "C" int pla_b200_gdn_prefill_chunked(const pla_b200_gdn_chunk_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  pla_b200_gdn_chunk_args a = *args;
  default_status(a);
  a.is_kda = 0;
  const int rc0 = check_chunk_args(a, pla_b200_gdn_chunk_workspace_bytes(a.max_chunks, a.H, a.HV));
  if (rc0 != PLA_B200_OK) return rc0;
  if (a.max_chunks == 0) return PLA_B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t items = static_cast<int64_t>(a.max_chunks) * a.H;
  auto launch_prepare = [&](auto kern) -> int {
    // one flag per kernel instantiation: both dtypes share this lambda's body (same function-pointer type)
    static DeviceOnce configured_by_dtype[2];
    DeviceOnce& configured = configured_by_dtype[a.act_dtype == PLA_B200_BF16 ? 0 : 1];
    int dev = 0;
    PLA_CUDA_OK(cudaGetDevice(&dev));
    if (configured.needed(dev)) {
      PLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(PrepSmem) + 1024)));
      configured.mark(dev);
    }
    kern<<<static_cast<unsigned>(items), PREP_THREADS, sizeof(PrepSmem) + 1024, s>>>(a);
    PLA_CUDA_OK(cudaGetLastError());
    const int64_t inv_items = static_cast<int64_t>(a.max_chunks) * a.HV;
    PLA_REQUIRE(inv_items < (1ll << 31), PLA_B200_E_TOO_LARGE, "too many chunks");
    chunk_inverse_kernel<<<static_cast<unsigned>((inv_items + 1) / 2), 128, 0, s>>>(a, static_cast<int>(inv_items));
    PLA_CUDA_OK(cudaGetLastError());
    return PLA_B200_OK;
  };
  int rc = PLA_B200_OK;
  if (a.stage != 2)
    rc = a.act_dtype == PLA_B200_BF16 ? launch_prepare(gdn_chunk_prepare_kernel<__nv_bfloat16>)
                                      : launch_prepare(gdn_chunk_prepare_kernel<__half>);
  if (rc != PLA_B200_OK || a.stage == 1) return rc;
  return launch_chain_stage(a, s);
}

extern "C" int64_t pla_b200_kda_chunk_workspace_bytes(int32_t max_chunks, int32_t H) {
  if (max_chunks < 0 || H <= 0) return 0;
  return static_cast<int64_t>(max_chunks) * H * (pla::HBLOB + pla::VBLOB + pla::L_BYTES);
}

extern "C" int pla_b200_kda_prefill_chunked(const pla_b200_gdn_chunk_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  pla_b200_gdn_chunk_args a = *args;
  default_status(a);
  a.is_kda = 1;
  const int rc0 = check_chunk_args(a, pla_b200_kda_chunk_workspace_bytes(a.max_chunks, a.H));
  if (rc0 != PLA_B200_OK) return rc0;
  PLA_REQUIRE(a.H == a.HV, PLA_B200_E_INVALID, "KDA prefill needs as many q/k heads as value heads");
  PLA_REQUIRE(!a.gate_activated, PLA_B200_E_INVALID, "chunked KDA prefill takes the raw gate input");
  PLA_REQUIRE(a.gate_kind == PLA_B200_GATE_SOFTPLUS || (a.gate_kind == PLA_B200_GATE_SAFE && a.lower_bound < 0.0f &&
                                                        a.lower_bound >= -5.0f),
              PLA_B200_E_INVALID, "the safe gate needs -5 <= lower_bound < 0");
  if (a.max_chunks == 0) return PLA_B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t items = static_cast<int64_t>(a.max_chunks) * a.H;
  auto launch_prepare = [&](auto kern) -> int {
    // one flag per kernel instantiation: both dtypes share this lambda's body (same function-pointer type)
    static DeviceOnce configured_by_dtype[2];
    DeviceOnce& configured = configured_by_dtype[a.act_dtype == PLA_B200_BF16 ? 0 : 1];
    int dev = 0;
    PLA_CUDA_OK(cudaGetDevice(&dev));
    if (configured.needed(dev)) {
      PLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(KdaPrepSmem) + 1024)));
      configured.mark(dev);
    }
    kern<<<static_cast<unsigned>(items), KDA_PREP_THREADS, sizeof(KdaPrepSmem) + 1024, s>>>(a);
    PLA_CUDA_OK(cudaGetLastError());
    chunk_inverse_kernel<<<static_cast<unsigned>((items + 1) / 2), 128, 0, s>>>(a, static_cast<int>(items));
    PLA_CUDA_OK(cudaGetLastError());
    return PLA_B200_OK;
  };
  int rc = PLA_B200_OK;
  if (a.stage != 2)
    rc = a.act_dtype == PLA_B200_BF16 ? launch_prepare(kda_chunk_prepare_kernel<__nv_bfloat16>)
                                      : launch_prepare(kda_chunk_prepare_kernel<__half>);
  if (rc != PLA_B200_OK || a.stage == 1) return rc;
  return launch_chain_stage(a, s);
}

#ifdef PLA_B200_DEBUG_CLOCKS
extern "C" int pla_b200_debug_chain_clocks(long long* out) {
  return cudaMemcpyFromSymbol(out, pla::g_dbg_clock, sizeof(pla::g_dbg_clock)) == cudaSuccess ? 0 : -4;
}
#endif
