// KDA ReplaySSM for sm_100a: verify, commit plan, exact fold + conv scatter.
//
// verify  (src/decode/kda_replayssm/kda_mtp_verify.cu:235-583): per request row and head, for
//   every token of the window: causal conv (4 taps) + SiLU on q/k/v, gate, records (post-conv
//   pre-norm k and v in bf16, log-decay and beta in fp32, the 3-tap window after the token),
//   L2-norm q (times scale) and k, one delta-rule step on a PRIVATE copy of the checkpoint.
//   The checkpoint is read once (one bulk copy per CTA) and never written.
// plan    (src/decode/kda_replayssm_vllm/commit_plan.cu:18-115): integer, bit-exact.
// fold    (src/decode/kda_replayssm/kda_mtp_fold.cu:254-529): replay the accepted prefix from the
//   records (division-form norm of the recorded k), store to the final slot and, when the
//   prefix crosses a block boundary, to the boundary slot after `bc` steps.
// scatter (kda_mtp_fold.cu:828-894): conv_state[final, :, 0:3] <- records.conv[row, n-1], exact.
//
// CTA layout for verify and fold: one (row, head, 32-row slice of the 128x128 state); 128
// threads; the slice (16 KiB, contiguous) lives in shared memory, is fetched with one bulk copy
// and (fold) written back with one bulk store. Window steps are staged four at a time.
#include <limits.h>

#include "common.cuh"

namespace pla {
namespace {

constexpr int D = 128;
constexpr int TILE = D * D;
constexpr int BV = 32;            // state rows per CTA
constexpr int NVS = D / BV;
constexpr int NT = 128;
constexpr int NW = NT / 32;
constexpr int TS = 4;             // steps staged per chunk
constexpr uint32_t kSliceBytes = BV * D * 4;

struct Smem {
  float state[BV * D];
  float q[TS][D];
  float k[TS][D];
  float gam[TS][D];
  float v[TS][BV];
  float o[TS][BV];
  float part[TS][2][NW];
  float beta[TS];
  uint64_t bar;
};

__device__ __forceinline__ int64_t idx_at(const pla_b200_index& a, int64_t i) {
  return a.wide ? static_cast<const int64_t*>(a.data)[i * a.stride]
                : static_cast<const int32_t*>(a.data)[i * a.stride];
}

__device__ __forceinline__ float silu(float x) { return x * sigmoidf_fast(x); }

// One delta-rule step on 8 * NPASS state rows (row_base ..) held in shared memory, one warp, 8 lanes per
// row. The norm factors stay scalars: d = kr (S k), S += (vn kr) k, o = qr (S q) with k, q as staged.
// WITH_OUT: also form o = S q. `snap` (optional) receives the updated rows.
template <bool WITH_OUT, int NPASS = 1>
__device__ __forceinline__ void kda_step(float* s_state, const float* sk, const float* sq, const float* sgam,
                                         const float* sv, float kr, float qr, float beta, float* so,
                                         float* snap, int row_base, int lane) {
  const int j = lane & 7;
  float4 kk[4], qq[4], gg[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    kk[i] = reinterpret_cast<const float4*>(sk)[i * 8 + j];
    gg[i] = reinterpret_cast<const float4*>(sgam)[i * 8 + j];
    if constexpr (WITH_OUT) qq[i] = reinterpret_cast<const float4*>(sq)[i * 8 + j];
  }
  const float bk = beta * kr;
#pragma unroll
  for (int ps = 0; ps < NPASS; ++ps) {
    const int row = row_base + ps * 8 + (lane >> 3) * 2;  // two consecutive rows per lane group
#pragma unroll
    for (int pp = 0; pp < 2; ++pp) {
      float4* srow = reinterpret_cast<float4*>(s_state + (row + pp) * D);
      float4 st[4];
      float d = 0.0f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        st[i] = srow[i * 8 + j];
        st[i].x *= gg[i].x; st[i].y *= gg[i].y; st[i].z *= gg[i].z; st[i].w *= gg[i].w;
        d += dot4(st[i], kk[i]);
      }
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      d += __shfl_xor_sync(0xffffffffu, d, 4);
      const float vn = (sv[row + pp] * beta - d * bk) * kr;   // (v - kr d) beta, times kr for the update
      float oacc = 0.0f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        st[i].x = fmaf(vn, kk[i].x, st[i].x);
        st[i].y = fmaf(vn, kk[i].y, st[i].y);
        st[i].z = fmaf(vn, kk[i].z, st[i].z);
        st[i].w = fmaf(vn, kk[i].w, st[i].w);
        if constexpr (WITH_OUT) oacc += dot4(st[i], qq[i]);
        srow[i * 8 + j] = st[i];
        if (snap != nullptr) *reinterpret_cast<float4*>(snap + (row + pp) * D + (i * 8 + j) * 4) = st[i];
      }
      if constexpr (WITH_OUT) {
        oacc += __shfl_xor_sync(0xffffffffu, oacc, 1);
        oacc += __shfl_xor_sync(0xffffffffu, oacc, 2);
        oacc += __shfl_xor_sync(0xffffffffu, oacc, 4);
        if (j == 0) so[row + pp] = oacc * qr;
      }
    }
  }
}

// ------------------------------------------------------------------ verify
// Longest window a request may have: the record steps, or the conv-window steps when fewer.
__device__ __forceinline__ int window_capacity(const pla_b200_kda_verify_args& p) {
  return p.win_steps > 0 ? min(p.Q, p.win_steps) : p.Q;
}
// One CTA per (request, head), 256 threads, the whole 128 x 128 state in shared memory (read once,
// never written back). Threads 0..127 own a q / k / gate channel, threads 128..255 a v channel; conv +
// SiLU, gate and records are formed once per (token, channel); the recurrence runs over the staged
// tokens with warp w on state rows 16w .. 16w + 15.
constexpr int VNT = 256;
constexpr int VTS = 4;             // tokens staged per pass of the verify kernel
struct VerifySmem {
  alignas(128) float state[D * D];
  float q[VTS][D];
  float k[VTS][D];
  float gam[VTS][D];
  float v[VTS][D];
  float o[VTS][D];
  float part[VTS][2][4];
  float beta[VTS];
  alignas(8) uint64_t bar;
};

__global__ void __launch_bounds__(VNT, 2) kda_verify_kernel(const pla_b200_kda_verify_args p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  VerifySmem& sh = *reinterpret_cast<VerifySmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x % p.H;
  const int n = blockIdx.x / p.H;

  const int64_t begin = idx_at(p.cu, n), end = idx_at(p.cu, n + 1);
  const int64_t slot = idx_at(p.slot_idx, n);
  // rows whose metadata is unusable are left completely alone
  if (idx_at(p.cu, 0) != 0 || begin < 0 || end < begin || end > p.T || end - begin > window_capacity(p) || slot >= p.slots ||
      begin == end)
    return;
  const int n_tok = static_cast<int>(end - begin);
  const int64_t out_stride = static_cast<int64_t>(p.H) * D;
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(h) * D;
  if (slot <= p.null_block_id) {  // padding row: zero its output interval, touch nothing else
    for (int i = tid; i < n_tok * D; i += VNT) out[(begin + i / D) * out_stride + (i % D)] = __float2bfloat16(0.0f);
    return;
  }

  if (tid == 0) {
    mbar_init(&sh.bar, 1);
    fence_mbar_init();
    mbar_expect_tx(&sh.bar, D * D * 4);
    const float* src = p.state + slot * p.state_slot_stride + static_cast<int64_t>(h) * TILE;
#pragma unroll
    for (int i = 0; i < 4; ++i) bulk_load(sh.state + i * (TILE / 4), src + i * (TILE / 4), TILE, &sh.bar);
  }

  const int64_t rec_row = p.row_by_slot ? slot : n;
  const int64_t win_row = (p.row_by_slot && p.scratch_idx.data != nullptr) ? idx_at(p.scratch_idx, n) : n;
  const bool is_v = tid >= D;
  const int c = tid & (D - 1);
  const int ch = h * D + c;             // channel of this thread inside its q / k / gate or v tensor
  const __nv_bfloat16* gin = static_cast<const __nv_bfloat16*>(p.raw_g) + begin * p.g_tok_stride + ch;
  const __nv_bfloat16* bin = static_cast<const __nv_bfloat16*>(p.raw_beta) + begin * p.beta_tok_stride + h;

  // conv taps and the sliding 3-tap history in registers: (q, k) for the first half, v for the second
  float wa[4], wb[4], ha[3], hb[3];
  const __nv_bfloat16 *xa, *xb = nullptr;
  int64_t xa_stride, xb_stride = 0;
  __nv_bfloat16 *wina, *winb = nullptr;
  int64_t wina_step, wina_tap, winb_step = 0, winb_tap = 0;
  {
    const float* w0 = is_v ? p.w_v : p.w_q;
    const __nv_bfloat16* cs0 = static_cast<const __nv_bfloat16*>(is_v ? p.cs_v : p.cs_q);
    const pla_b200_conv_strides& st0 = is_v ? p.cs_v_strides : p.cs_q_strides;
    const pla_b200_window_strides& ws0 = is_v ? p.win_v_strides : p.win_q_strides;
#pragma unroll
    for (int w = 0; w < 4; ++w) wa[w] = w0[ch * 4 + w];
#pragma unroll
    for (int w = 0; w < 3; ++w) ha[w] = __bfloat162float(cs0[slot * st0.slot + ch * st0.channel + w * st0.tap]);
    xa = static_cast<const __nv_bfloat16*>(is_v ? p.x_v : p.x_q) + begin * (is_v ? p.xv_tok_stride : p.xq_tok_stride) + ch;
    xa_stride = is_v ? p.xv_tok_stride : p.xq_tok_stride;
    wina = static_cast<__nv_bfloat16*>(is_v ? p.win_v : p.win_q) + win_row * ws0.row + ch * ws0.channel;
    wina_step = ws0.step;
    wina_tap = ws0.tap;
    if (!is_v) {
      const __nv_bfloat16* cs1 = static_cast<const __nv_bfloat16*>(p.cs_k);
#pragma unroll
      for (int w = 0; w < 4; ++w) wb[w] = p.w_k[ch * 4 + w];
#pragma unroll
      for (int w = 0; w < 3; ++w)
        hb[w] = __bfloat162float(cs1[slot * p.cs_k_strides.slot + ch * p.cs_k_strides.channel + w * p.cs_k_strides.tap]);
      xb = static_cast<const __nv_bfloat16*>(p.x_k) + begin * p.xk_tok_stride + ch;
      xb_stride = p.xk_tok_stride;
      winb = static_cast<__nv_bfloat16*>(p.win_k) + win_row * p.win_k_strides.row + ch * p.win_k_strides.channel;
      winb_step = p.win_k_strides.step;
      winb_tap = p.win_k_strides.tap;
    }
  }
  const float A_log = p.A_log[h];
  const float dtb = is_v ? 0.f : p.dt_bias[ch];
  const int64_t rec0 = (rec_row * p.H + h) * p.Q;       // record row of step 0, in 128-element rows
  __nv_bfloat16* rra = static_cast<__nv_bfloat16*>(is_v ? p.rec_rawv : p.rec_rawk) + rec0 * D + c;
  float* rg = p.rec_g + rec0 * D + c;

  bool loaded = false;
  for (int t0 = 0; t0 < n_tok; t0 += VTS) {
    const int nt = min(VTS, n_tok - t0);
    if (t0 > 0) __syncthreads();
    // all of this pass's inputs first: the record / window stores below would otherwise keep each
    // token's loads behind the previous token's stores
    float in_a[VTS], in_b[VTS], in_g[VTS], in_beta[VTS];
#pragma unroll
    for (int s = 0; s < VTS; ++s) {
      in_a[s] = in_b[s] = in_g[s] = in_beta[s] = 0.f;
      if (s < nt) {
        const int t = t0 + s;
        in_a[s] = __bfloat162float(xa[t * xa_stride]);
        if (!is_v) {
          in_b[s] = __bfloat162float(xb[t * xb_stride]);
          in_g[s] = __bfloat162float(gin[t * p.g_tok_stride]);
        } else if (c == 0) {
          in_beta[s] = __bfloat162float(bin[t * p.beta_tok_stride]);
        }
      }
    }
#pragma unroll
    for (int s = 0; s < VTS; ++s) {
      if (s >= nt) break;
      const int t = t0 + s;
      const float fa = in_a[s];
      float ca = fa * wa[3];
#pragma unroll
      for (int w = 0; w < 3; ++w) ca += ha[w] * wa[w];
      ca = silu(ca);
      ha[0] = ha[1]; ha[1] = ha[2]; ha[2] = fa;
#pragma unroll
      for (int w = 0; w < 3; ++w) wina[t * wina_step + w * wina_tap] = __float2bfloat16(ha[w]);  // exact: values came from bf16
      if (is_v) {
        sh.v[s][c] = ca;
        rra[static_cast<int64_t>(t) * D] = __float2bfloat16(ca);
        if (c == 0) {
          const float beta = sigmoidf_fast(in_beta[s]);
          sh.beta[s] = beta;
          p.rec_beta[rec0 + t] = beta;
        }
      } else {
        const float fb = in_b[s];
        float cb = fb * wb[3];
#pragma unroll
        for (int w = 0; w < 3; ++w) cb += hb[w] * wb[w];
        cb = silu(cb);
        hb[0] = hb[1]; hb[1] = hb[2]; hb[2] = fb;
#pragma unroll
        for (int w = 0; w < 3; ++w) winb[t * winb_step + w * winb_tap] = __float2bfloat16(hb[w]);
        const float gk = log_decay(in_g[s] + dtb, A_log, p.gate, p.softplus_beta, p.softplus_threshold, p.lower_bound);
        rra[static_cast<int64_t>(t) * D] = __float2bfloat16(cb);
        rg[static_cast<int64_t>(t) * D] = gk;
        sh.q[s][c] = ca;
        sh.k[s][c] = cb;
        sh.gam[s][c] = fast_exp(gk);
        const float sq = warp_sum(ca * ca), sk = warp_sum(cb * cb);
        if (lane == 0) {
          sh.part[s][0][warp] = sq;
          sh.part[s][1][warp] = sk;
        }
      }
    }
    __syncthreads();
    if (!loaded) {
      const bool ok = mbar_wait(&sh.bar, 0);
      if (__syncthreads_or(!ok)) {
        if (tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_WAIT_TIMEOUT);
        (void)mbar_wait(&sh.bar, 0);
        return;
      }
      loaded = true;
    }
    for (int s = 0; s < nt; ++s) {
      const float sq = (sh.part[s][0][0] + sh.part[s][0][1]) + (sh.part[s][0][2] + sh.part[s][0][3]);
      const float sk = (sh.part[s][1][0] + sh.part[s][1][1]) + (sh.part[s][1][2] + sh.part[s][1][3]);
      const float qr = rsqrtf(sq + 1e-6f) * p.scale, kr = rsqrtf(sk + 1e-6f);
      kda_step<true, 2>(sh.state, sh.k[s], sh.q[s], sh.gam[s], sh.v[s], kr, qr, sh.beta[s], sh.o[s], nullptr,
                        warp * 16, lane);
    }
    __syncthreads();
    if (p.out_f32 != nullptr) {
      float* of = p.out_f32 + static_cast<int64_t>(h) * D;
      for (int i = tid; i < nt * D; i += VNT) of[(begin + t0 + i / D) * out_stride + (i % D)] = sh.o[i / D][i % D];
    } else {
      for (int i = tid; i < nt * D; i += VNT)
        out[(begin + t0 + i / D) * out_stride + (i % D)] = __float2bfloat16(sh.o[i / D][i % D]);
    }
  }
}

// ------------------------------------------------------------------ verify, closed-form window (Q <= 8)
// Verify never writes the checkpoint, so the window's outputs are linear in it. Row by row of the state
// (s_t = the row after token t, A_t = diag(gamma_t) (I - beta_t k_t k_t^T), k_t normalised):
//     s_t = s_{t-1} A_t + beta_t v_t[row] k_t^T          =>
//     o_t[row] = s_t . q_t = s_0 . Qeff_t + sum_{j <= t} c_{j,t} v_j[row],
//     Qeff_t = A_1 ... A_t q_t,      c_{j,t} = beta_j k_j^T (A_{j+1} ... A_t q_t)
// (the reference forms the same window in closed form, src/decode/kda_replayssm/kda_mtp_verify.cu:630-653).
// Qeff_t and c_{.,t} come from one backward sweep per token over k, gamma, beta (warp t: x = q_t; for j = t..1:
// d = k_j . x, c_{j,t} = beta_j d, x = gamma_j (x - beta_j d k_j)) -- O(Q^2) vectors of 128, no state involved.
// The 64 KiB state is then read ONCE, straight from global memory into registers, four rows per warp at a time
// with the next four already requested, and each row gives its Q dot products (lane j of a row's eight lanes
// also carries the c_{j,t} v_j term into the reduction). No shared-memory copy of the state, no dependent
// per-token sweeps over it; 85 registers, so three CTAs share an SM and cover each other's set-up.
constexpr int CQ = 8;   // longest window of the closed-form kernel
struct WindowSmem {
  float q[CQ][D];      // conv + SiLU outputs (unnormalised), then Qeff
  float k[CQ][D];      // conv + SiLU outputs (unnormalised), then normalised
  float gam[CQ][D];
  float v[CQ][D];
  float o[CQ][D];
  float c[CQ][CQ];     // c[j][t]
  float part[CQ][2][4];
  float beta[CQ];
};

__global__ void __launch_bounds__(VNT, 3) kda_verify_window_kernel(const pla_b200_kda_verify_args p) {
  __shared__ __align__(16) WindowSmem sh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x % p.H;
  const int n = blockIdx.x / p.H;

  const int64_t begin = idx_at(p.cu, n), end = idx_at(p.cu, n + 1);
  const int64_t slot = idx_at(p.slot_idx, n);
  // rows whose metadata is unusable are left completely alone
  if (idx_at(p.cu, 0) != 0 || begin < 0 || end < begin || end > p.T || end - begin > window_capacity(p) || slot >= p.slots ||
      begin == end)
    return;
  const int n_tok = static_cast<int>(end - begin);   // <= CQ: the host only picks this kernel for Q <= CQ
  const int64_t out_stride = static_cast<int64_t>(p.H) * D;
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(h) * D;
  if (slot <= p.null_block_id) {  // padding row: zero its output interval, touch nothing else
    for (int i = tid; i < n_tok * D; i += VNT) out[(begin + i / D) * out_stride + (i % D)] = __float2bfloat16(0.0f);
    return;
  }

  // ---- this thread's share of the checkpoint, requested first: warp w owns rows 16 w .. 16 w + 15, eight lanes per
  // row, lane j of a row the columns (i * 8 + j) * 4 .. + 3
  const int j8 = lane & 7;
  const float4* srow0 = reinterpret_cast<const float4*>(p.state + slot * p.state_slot_stride + static_cast<int64_t>(h) * TILE) +
                        (warp * 16 + (lane >> 3)) * (D / 4) + j8;   // row pass ps: + ps * 4 rows; piece i: + i * 8
  float4 st[2][4];   // [buffer][piece]: the row pass being worked on and the next one
#pragma unroll
  for (int i = 0; i < 4; ++i) st[0][i] = __ldg(srow0 + i * 8);

  const int64_t rec_row = p.row_by_slot ? slot : n;
  const int64_t win_row = (p.row_by_slot && p.scratch_idx.data != nullptr) ? idx_at(p.scratch_idx, n) : n;
  const bool is_v = tid >= D;
  const int c = tid & (D - 1);
  const int ch = h * D + c;             // channel of this thread inside its q / k / gate or v tensor
  const __nv_bfloat16* gin = static_cast<const __nv_bfloat16*>(p.raw_g) + begin * p.g_tok_stride + ch;
  const __nv_bfloat16* bin = static_cast<const __nv_bfloat16*>(p.raw_beta) + begin * p.beta_tok_stride + h;

  // conv taps and the sliding 3-tap history in registers: (q, k) for the first half, v for the second
  float wa[4], wb[4], ha[3], hb[3];
  const __nv_bfloat16 *xa, *xb = nullptr;
  int64_t xa_stride, xb_stride = 0;
  __nv_bfloat16 *wina, *winb = nullptr;
  int64_t wina_step, wina_tap, winb_step = 0, winb_tap = 0;
  {
    const float* w0 = is_v ? p.w_v : p.w_q;
    const __nv_bfloat16* cs0 = static_cast<const __nv_bfloat16*>(is_v ? p.cs_v : p.cs_q);
    const pla_b200_conv_strides& st0 = is_v ? p.cs_v_strides : p.cs_q_strides;
    const pla_b200_window_strides& ws0 = is_v ? p.win_v_strides : p.win_q_strides;
#pragma unroll
    for (int w = 0; w < 4; ++w) wa[w] = w0[ch * 4 + w];
#pragma unroll
    for (int w = 0; w < 3; ++w) ha[w] = __bfloat162float(cs0[slot * st0.slot + ch * st0.channel + w * st0.tap]);
    xa = static_cast<const __nv_bfloat16*>(is_v ? p.x_v : p.x_q) + begin * (is_v ? p.xv_tok_stride : p.xq_tok_stride) + ch;
    xa_stride = is_v ? p.xv_tok_stride : p.xq_tok_stride;
    wina = static_cast<__nv_bfloat16*>(is_v ? p.win_v : p.win_q) + win_row * ws0.row + ch * ws0.channel;
    wina_step = ws0.step;
    wina_tap = ws0.tap;
    if (!is_v) {
      const __nv_bfloat16* cs1 = static_cast<const __nv_bfloat16*>(p.cs_k);
#pragma unroll
      for (int w = 0; w < 4; ++w) wb[w] = p.w_k[ch * 4 + w];
#pragma unroll
      for (int w = 0; w < 3; ++w)
        hb[w] = __bfloat162float(cs1[slot * p.cs_k_strides.slot + ch * p.cs_k_strides.channel + w * p.cs_k_strides.tap]);
      xb = static_cast<const __nv_bfloat16*>(p.x_k) + begin * p.xk_tok_stride + ch;
      xb_stride = p.xk_tok_stride;
      winb = static_cast<__nv_bfloat16*>(p.win_k) + win_row * p.win_k_strides.row + ch * p.win_k_strides.channel;
      winb_step = p.win_k_strides.step;
      winb_tap = p.win_k_strides.tap;
    }
  }
  const float A_log = p.A_log[h];
  const float dtb = is_v ? 0.f : p.dt_bias[ch];
  const int64_t rec0 = (rec_row * p.H + h) * p.Q;       // record row of step 0, in 128-element rows
  __nv_bfloat16* rra = static_cast<__nv_bfloat16*>(is_v ? p.rec_rawv : p.rec_rawk) + rec0 * D + c;
  float* rg = p.rec_g + rec0 * D + c;

  // ---- per (token, channel): conv + SiLU, gate, records; four tokens' inputs are fetched ahead of their stores
  for (int t0 = 0; t0 < n_tok; t0 += VTS) {
    const int nt = min(VTS, n_tok - t0);
    float in_a[VTS], in_b[VTS], in_g[VTS], in_beta[VTS];
#pragma unroll
    for (int s = 0; s < VTS; ++s) {
      in_a[s] = in_b[s] = in_g[s] = in_beta[s] = 0.f;
      if (s < nt) {
        const int t = t0 + s;
        in_a[s] = __bfloat162float(xa[t * xa_stride]);
        if (!is_v) {
          in_b[s] = __bfloat162float(xb[t * xb_stride]);
          in_g[s] = __bfloat162float(gin[t * p.g_tok_stride]);
        } else if (c == 0) {
          in_beta[s] = __bfloat162float(bin[t * p.beta_tok_stride]);
        }
      }
    }
#pragma unroll
    for (int s = 0; s < VTS; ++s) {
      if (s >= nt) break;
      const int t = t0 + s;
      const float fa = in_a[s];
      float ca = fa * wa[3];
#pragma unroll
      for (int w = 0; w < 3; ++w) ca += ha[w] * wa[w];
      ca = silu(ca);
      ha[0] = ha[1]; ha[1] = ha[2]; ha[2] = fa;
#pragma unroll
      for (int w = 0; w < 3; ++w) wina[t * wina_step + w * wina_tap] = __float2bfloat16(ha[w]);  // exact: values came from bf16
      if (is_v) {
        sh.v[t][c] = ca;
        rra[static_cast<int64_t>(t) * D] = __float2bfloat16(ca);
        if (c == 0) {
          const float beta = sigmoidf_fast(in_beta[s]);
          sh.beta[t] = beta;
          p.rec_beta[rec0 + t] = beta;
        }
      } else {
        const float fb = in_b[s];
        float cb = fb * wb[3];
#pragma unroll
        for (int w = 0; w < 3; ++w) cb += hb[w] * wb[w];
        cb = silu(cb);
        hb[0] = hb[1]; hb[1] = hb[2]; hb[2] = fb;
#pragma unroll
        for (int w = 0; w < 3; ++w) winb[t * winb_step + w * winb_tap] = __float2bfloat16(hb[w]);
        const float gk = log_decay(in_g[s] + dtb, A_log, p.gate, p.softplus_beta, p.softplus_threshold, p.lower_bound);
        rra[static_cast<int64_t>(t) * D] = __float2bfloat16(cb);
        rg[static_cast<int64_t>(t) * D] = gk;
        sh.q[t][c] = ca;
        sh.k[t][c] = cb;
        sh.gam[t][c] = fast_exp(gk);
        const float sq = warp_sum(ca * ca), sk = warp_sum(cb * cb);
        if (lane == 0) {
          sh.part[t][0][warp] = sq;
          sh.part[t][1][warp] = sk;
        }
      }
    }
  }
  __syncthreads();

  // ---- normalise k in place (all warps), then warp t sweeps back from token t: Qeff_t over q[t], c[.][t]
  for (int i = tid; i < n_tok * D; i += VNT) {
    const int t = i / D;
    const float sk = (sh.part[t][1][0] + sh.part[t][1][1]) + (sh.part[t][1][2] + sh.part[t][1][3]);
    sh.k[t][i % D] *= rsqrtf(sk + 1e-6f);
  }
  __syncthreads();
  if (warp < n_tok) {
    const int t = warp;
    const float sq = (sh.part[t][0][0] + sh.part[t][0][1]) + (sh.part[t][0][2] + sh.part[t][0][3]);
    const float qr = rsqrtf(sq + 1e-6f) * p.scale;
    float4 x = reinterpret_cast<const float4*>(sh.q[t])[lane];
    x.x *= qr; x.y *= qr; x.z *= qr; x.w *= qr;
    for (int jt = t; jt >= 0; --jt) {
      const float4 kk = reinterpret_cast<const float4*>(sh.k[jt])[lane];
      const float4 gg = reinterpret_cast<const float4*>(sh.gam[jt])[lane];
      const float d = warp_sum(dot4(kk, x));
      const float bd = sh.beta[jt] * d;
      if (lane == 0) sh.c[jt][t] = bd;
      x.x = gg.x * fmaf(-bd, kk.x, x.x);
      x.y = gg.y * fmaf(-bd, kk.y, x.y);
      x.z = gg.z * fmaf(-bd, kk.z, x.z);
      x.w = gg.w * fmaf(-bd, kk.w, x.w);
    }
    __syncwarp();
    reinterpret_cast<float4*>(sh.q[t])[lane] = x;   // q[t] is only read by this warp before this point
  }
  __syncthreads();

  // ---- one pass over the state: four rows per warp at a time, the next four in flight
#pragma unroll
  for (int ps = 0; ps < 4; ++ps) {
    if (ps + 1 < 4) {
#pragma unroll
      for (int i = 0; i < 4; ++i) st[(ps + 1) & 1][i] = __ldg(srow0 + (ps + 1) * 4 * (D / 4) + i * 8);
    }
    const int row = warp * 16 + ps * 4 + (lane >> 3);
    for (int t = 0; t < n_tok; ++t) {
      // lane j of the row's eight lanes brings c[j][t] v_j[row] (j <= t) into the sum: CQ = 8 terms at most
      float acc = (j8 <= t) ? sh.c[j8][t] * sh.v[j8][row] : 0.0f;
#pragma unroll
      for (int i = 0; i < 4; ++i) acc += dot4(st[ps & 1][i], reinterpret_cast<const float4*>(sh.q[t])[i * 8 + j8]);
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (j8 == 0) sh.o[t][row] = acc;
    }
  }
  __syncthreads();
  if (p.out_f32 != nullptr) {
    float* of = p.out_f32 + static_cast<int64_t>(h) * D;
    for (int i = tid; i < n_tok * D; i += VNT) of[(begin + i / D) * out_stride + (i % D)] = sh.o[i / D][i % D];
  } else {
    for (int i = tid; i < n_tok * D; i += VNT)
      out[(begin + i / D) * out_stride + (i % D)] = __float2bfloat16(sh.o[i / D][i % D]);
  }
}

// Gated RMSNorm of the staged fp32 outputs: one CTA per (request, head), one warp per token,
// four channels per lane. Rows that verify left alone (unusable metadata, padding) stay as they are.
__global__ void __launch_bounds__(NT) kda_onorm_kernel(const pla_b200_kda_verify_args p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x % p.H, n = blockIdx.x / p.H;
  const int64_t begin = idx_at(p.cu, n), end = idx_at(p.cu, n + 1);
  const int64_t slot = idx_at(p.slot_idx, n);
  if (idx_at(p.cu, 0) != 0 || begin < 0 || end < begin || end > p.T || end - begin > window_capacity(p) || slot >= p.slots ||
      begin == end || slot <= p.null_block_id)
    return;
  const __nv_bfloat16* gate = static_cast<const __nv_bfloat16*>(p.onorm_gate);
  const float4 w = reinterpret_cast<const float4*>(p.onorm_weight)[lane];
  const int64_t row_elems = static_cast<int64_t>(p.H) * D;
  for (int64_t tok = begin + warp; tok < end; tok += NW) {
    const float4 o = *reinterpret_cast<const float4*>(p.out_f32 + tok * row_elems + h * D + lane * 4);
    const float r = rsqrtf(warp_sum(o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w) * (1.0f / D) + p.onorm_eps);
    const __nv_bfloat16* gp = gate + tok * p.onorm_gate_tok_stride + h * D + lane * 4;
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + tok * row_elems + h * D + lane * 4;
    dst[0] = __float2bfloat16(o.x * r * w.x * sigmoidf_fast(__bfloat162float(gp[0])));
    dst[1] = __float2bfloat16(o.y * r * w.y * sigmoidf_fast(__bfloat162float(gp[1])));
    dst[2] = __float2bfloat16(o.z * r * w.z * sigmoidf_fast(__bfloat162float(gp[2])));
    dst[3] = __float2bfloat16(o.w * r * w.w * sigmoidf_fast(__bfloat162float(gp[3])));
  }
}

// -------------------------------------------------------------------- plan
__device__ __forceinline__ bool valid_slot(int64_t slot, const pla_b200_kda_commit_args& p) {
  return slot > p.null_block_id && slot >= 0 && slot < p.slots;
}
__device__ __forceinline__ bool valid_interval(int64_t b, int64_t e, const pla_b200_kda_commit_args& p) {
  return b >= 0 && e > b && e <= p.token_capacity && e - b <= p.Q;
}

// Candidate plan of row b: (count, final, boundary, boundary_len); zeros when the row commits nothing.
__device__ void plan_row(const pla_b200_kda_commit_args& p, int b, int* cand) {
  int64_t count = 0, final_slot = 0, boundary = 0, bc = 0;
  if (b < p.N) {
    const int64_t row = p.mapping.data != nullptr ? idx_at(p.mapping, b) : b;
    const int64_t source = idx_at(p.source, b);
    const int64_t begin = idx_at(p.cu, b), end = idx_at(p.cu, b + 1);
    if (idx_at(p.cu, 0) == 0 && row >= 0 && row < p.sampler_rows && valid_slot(source, p) &&
        valid_interval(begin, end, p)) {
      const int64_t sampled = idx_at(p.sampled, row);
      const int64_t len = end - begin;
      count = sampled <= 0 ? 0 : (sampled > len ? len : sampled);
      final_slot = source;
      if (count != 0 && p.block_size != 0) {
        if (row >= p.block_rows) {
          count = 0;
        } else {
          const int64_t pos = idx_at(p.computed, row);
          if (pos < 0 || pos > LLONG_MAX - p.Q) {
            count = 0;
          } else {
            int64_t col = (pos + count - 1) / p.block_size;
            if (col >= p.block_cols) col = p.block_cols - 1;
            const int64_t f = idx_at(p.blocks, row * p.block_row_stride + col * p.block_col_stride);
            if (!valid_slot(f, p)) count = 0;
            else final_slot = f;
            const int64_t distance = p.block_size - pos % p.block_size;  // tokens left in the current block
            if (count != 0 && count >= distance) {
              const int64_t bcol = pos / p.block_size;
              if (bcol >= p.block_cols) {
                count = 0;
              } else {
                const int64_t dest = idx_at(p.blocks, row * p.block_row_stride + bcol * p.block_col_stride);
                if (!valid_slot(dest, p) || (dest == final_slot && distance != count)) {
                  count = 0;
                } else {
                  boundary = dest;
                  bc = distance;
                }
              }
            }
          }
        }
      }
    }
  }
  const int R = p.capacity;
  cand[b] = static_cast<int>(count);
  cand[R + b] = count ? static_cast<int>(final_slot) : 0;
  cand[2 * R + b] = count ? static_cast<int>(boundary) : 0;
  cand[3 * R + b] = count ? static_cast<int>(bc) : 0;
}

// One warp per row: a row is dropped when one of its destinations is another row's source,
// final or boundary slot, or its source is another row's destination. Symmetric by construction.
__device__ void protect_row(const pla_b200_kda_commit_args& p, int b, int lane, const int* cand, int* plan) {
  const int R = p.capacity;
  bool conflict = false;
  if (cand[b] != 0) {
    const int64_t source = idx_at(p.source, b);
    const int f = cand[R + b], d = cand[2 * R + b];
    const bool has_d = cand[3 * R + b] > 0;
    for (int other = lane; other < p.N; other += 32) {
      if (other == b) continue;
      const int64_t os = idx_at(p.source, other);
      const int64_t ob = idx_at(p.cu, other), oe = idx_at(p.cu, other + 1);
      // a real query that commits nothing still owns its source checkpoint
      if (valid_slot(os, p) && valid_interval(ob, oe, p)) conflict |= (f == os) || (has_d && d == os);
      if (cand[other] == 0) continue;
      const int of = cand[R + other], od = cand[2 * R + other];
      const bool has_od = cand[3 * R + other] > 0;
      conflict |= (f == os) || (f == of) || (has_od && f == od) ||
                  (has_d && (d == os || d == of || (has_od && d == od))) || (source == of) ||
                  (has_od && source == od);
    }
  }
  conflict = __any_sync(0xffffffffu, conflict);
  if (lane == 0) {
#pragma unroll
    for (int c = 0; c < 4; ++c) plan[c * R + b] = conflict ? 0 : cand[c * R + b];
  }
}

__global__ void plan_build_kernel(const pla_b200_kda_commit_args p) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < p.capacity) plan_row(p, b, p.candidate);
}
__global__ void plan_protect_kernel(const pla_b200_kda_commit_args p) {
  const int b = blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
  if (b < p.capacity) protect_row(p, b, threadIdx.x & 31, p.candidate, p.plan);
}
// Small batches: both phases in one CTA.
__global__ void __launch_bounds__(1024) plan_fused_kernel(const pla_b200_kda_commit_args p) {
  for (int b = threadIdx.x; b < p.capacity; b += blockDim.x) plan_row(p, b, p.candidate);
  __threadfence_block();
  __syncthreads();
  for (int b = threadIdx.x >> 5; b < p.capacity; b += blockDim.x / 32)
    protect_row(p, b, threadIdx.x & 31, p.candidate, p.plan);
}

// ----------------------------------------------------------- fold + scatter
struct FoldGrid {
  int fold_ctas;     // N * layers * H * NVS
  int conv_tiles;    // CTAs per (row, layer) of the scatter part
};

__device__ void fold_cta(const pla_b200_kda_commit_args& p, int cta, Smem& sh) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int vs = cta % NVS;
  const int hl = (cta / NVS) % (p.n_layers * p.H);
  const int b = cta / (NVS * p.n_layers * p.H);
  const int layer = hl / p.H, h = hl % p.H;
  const int R = p.capacity;
  const int n_commit = p.plan[b];
  if (n_commit <= 0) return;
  const int64_t slot = idx_at(p.source, b);
  if (slot <= p.null_block_id || slot >= p.slots) return;
  const int final_slot = p.plan[R + b], boundary = p.plan[2 * R + b], bc = p.plan[3 * R + b];
  const int64_t* L = p.layers + static_cast<int64_t>(layer) * PLA_B200_REPLAY_COLUMNS;
  float* pool = reinterpret_cast<float*>(L[PLA_B200_COL_STATE]);
  const int64_t slot_stride = L[PLA_B200_COL_STATE_STRIDE];
  const __nv_bfloat16* rawv = reinterpret_cast<const __nv_bfloat16*>(L[PLA_B200_COL_RAWV]);
  const __nv_bfloat16* rawk = reinterpret_cast<const __nv_bfloat16*>(L[PLA_B200_COL_RAWK]);
  const float* gate = reinterpret_cast<const float*>(L[PLA_B200_COL_GATE]);
  const float* beta = reinterpret_cast<const float*>(L[PLA_B200_COL_BETA]);
  const int row0 = vs * BV;
  const int64_t tile_off = static_cast<int64_t>(h) * TILE + row0 * D;

  if (tid == 0) {
    mbar_init(&sh.bar, 1);
    fence_mbar_init();
    mbar_expect_tx(&sh.bar, kSliceBytes);
    bulk_load(sh.state, pool + slot * slot_stride + tile_off, kSliceBytes, &sh.bar);
  }
  bool loaded = false;
  const int64_t rec0 = (static_cast<int64_t>(b) * p.H + h) * p.Q;
  for (int t0 = 0; t0 < n_commit; t0 += TS) {
    const int nt = min(TS, n_commit - t0);
    if (t0 > 0) __syncthreads();
    for (int s = 0; s < nt; ++s) {
      const int64_t rec = (rec0 + t0 + s) * D;
      const float kf = __bfloat162float(rawk[rec + tid]);
      sh.k[s][tid] = kf;
      sh.gam[s][tid] = fast_exp(gate[rec + tid]);
      const float sk = warp_sum(kf * kf);
      if (lane == 0) sh.part[s][1][warp] = sk;
      if (tid < BV) sh.v[s][tid] = __bfloat162float(rawv[rec + row0 + tid]);
      if (tid == 0) sh.beta[s] = beta[rec0 + t0 + s];
    }
    __syncthreads();
    if (!loaded) {
      const bool ok = mbar_wait(&sh.bar, 0);
      if (__syncthreads_or(!ok)) {
        if (tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_WAIT_TIMEOUT);
        (void)mbar_wait(&sh.bar, 0);
        return;
      }
      loaded = true;
    }
    for (int s = 0; s < nt; ++s) {
      float sk = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) sk += sh.part[s][1][w];
      const float kinv = 1.0f / sqrtf(sk + 1e-6f);  // division form, as the records are replayed
      float* snap = nullptr;
      if (bc > 0 && t0 + s == bc - 1 && boundary > p.null_block_id && boundary < p.slots)
        snap = pool + static_cast<int64_t>(boundary) * slot_stride + tile_off;
      kda_step<false>(sh.state, sh.k[s], nullptr, sh.gam[s], sh.v[s], kinv, 0.f, sh.beta[s], nullptr, snap, warp * 8,
                      lane);
    }
  }
  if (final_slot > p.null_block_id && final_slot < p.slots) {
    fence_async_smem();
    __syncthreads();
    if (tid == 0) {
      bulk_store(pool + static_cast<int64_t>(final_slot) * slot_stride + tile_off, sh.state, kSliceBytes);
      bulk_commit();
      bulk_wait_read<0>();
    }
  }
}

__device__ void scatter_cta(const pla_b200_kda_commit_args& p, int cta, int tiles) {
  const int tile = cta % tiles;
  const int layer = (cta / tiles) % p.n_layers;
  const int b = cta / (tiles * p.n_layers);
  const int R = p.capacity;
  const int count = p.plan[b];
  if (count <= 0) return;
  const int final_slot = p.plan[R + b], boundary = p.plan[2 * R + b], bc = p.plan[3 * R + b];
  const int64_t* L = p.layers + static_cast<int64_t>(layer) * PLA_B200_REPLAY_COLUMNS;
  uint16_t* dst = reinterpret_cast<uint16_t*>(L[PLA_B200_COL_CONV]);
  const uint16_t* src = reinterpret_cast<const uint16_t*>(L[PLA_B200_COL_WINDOWS]);
  const int64_t s_slot = L[PLA_B200_COL_CONV_SLOT], s_ch = L[PLA_B200_COL_CONV_CHANNEL], s_tap = L[PLA_B200_COL_CONV_TAP];
  const int dim = 3 * p.H * D;
  const bool final_ok = final_slot > p.null_block_id && final_slot < p.slots;
  const bool bound_ok = bc > 0 && boundary > p.null_block_id && boundary < p.slots;
  const int64_t fsrc = (static_cast<int64_t>(b) * p.Q + count - 1) * dim * 3;
  const int64_t bsrc = (static_cast<int64_t>(b) * p.Q + bc - 1) * dim * 3;
  for (int i = tile * blockDim.x + threadIdx.x; i < dim * 3; i += tiles * blockDim.x) {
    const int c = i / 3, w = i % 3;
    const int64_t off = static_cast<int64_t>(c) * s_ch + w * s_tap;
    if (bound_ok) dst[static_cast<int64_t>(boundary) * s_slot + off] = src[bsrc + i];
    if (final_ok) dst[static_cast<int64_t>(final_slot) * s_slot + off] = src[fsrc + i];
  }
}

// Fold for windows of at most CQ tokens (the usual case), one CTA per (row, layer, head): the whole 64 KiB
// checkpoint goes global -> registers -> global once, with no shared-memory copy. Warp w owns rows 16 w .. 16 w + 15
// (eight lanes per row), four rows at a time with the next four already requested; the remaining rows are asked
// into L2 (`prefetch.global.L2`) at the start, so that their DRAM fetch runs under the staging of the records.
// The committed tokens' k, decay and v records sit in shared memory (12 KiB for eight tokens) and every row takes
// all of them in turn before it is written to the final slot (and, after token `bc`, to the boundary slot).
// Same arithmetic as `kda_step`, term by term.
constexpr int FT = 256;
struct TileSmem {
  alignas(16) float k[CQ][D];
  alignas(16) float gam[CQ][D];
  float v[CQ][D];
  float part[CQ][4];
  float kinv[CQ];
  float beta[CQ];
};

// What one whole-tile fold needs: where the tile is, where it goes, and the records of the tokens to apply
// (k, gate and v records: 128 values per token, tokens 128 apart; beta: one value per token).
struct TileFold {
  const float* src;             // the 128 x 128 tile to fold
  float* dst;                   // where the folded tile goes (may be `src`; nullptr: nowhere)
  float* snap;                  // receives the tile as it is after token `snap_t` (nullptr: no snapshot)
  int snap_t;
  int n;                        // tokens to apply, at most CQ
  const __nv_bfloat16 *rawk, *rawv;
  const float *gate, *beta;
};

__device__ void fold_tile(const TileFold& f, TileSmem& sh) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, j8 = lane & 7;
  // this thread's pieces: row pass ps -> row 16 warp + 4 ps + lane / 8, piece i -> columns (i * 8 + j8) * 4 ..
  const int64_t my_off = (warp * 16 + (lane >> 3)) * (D / 4) + j8;   // in 16-byte pieces
  const float4* src0 = reinterpret_cast<const float4*>(f.src) + my_off;
  float4 st[2][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) st[0][i] = src0[i * 8];
  for (int idx = j8; idx < 12; idx += 8) prefetch_l2(src0 - j8 + (1 + idx / 4) * 4 * (D / 4) + (idx % 4) * 8);

  for (int s = 0; s < f.n; ++s) {
    if (tid < D) {
      const float kf = __bfloat162float(f.rawk[s * D + tid]);
      sh.k[s][tid] = kf;
      sh.gam[s][tid] = fast_exp(f.gate[s * D + tid]);
      const float sk = warp_sum(kf * kf);
      if (lane == 0) sh.part[s][warp] = sk;
    } else {
      sh.v[s][tid - D] = __bfloat162float(f.rawv[s * D + tid - D]);
      if (tid == D) sh.beta[s] = f.beta[s];
    }
  }
  __syncthreads();
  if (tid < f.n) {
    float sk = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) sk += sh.part[tid][w];
    sh.kinv[tid] = 1.0f / sqrtf(sk + 1e-6f);  // division form, as the records are replayed
  }
  __syncthreads();

  float4* dst = f.dst == nullptr ? nullptr : reinterpret_cast<float4*>(f.dst) + my_off;
  float4* snap = f.snap == nullptr ? nullptr : reinterpret_cast<float4*>(f.snap) + my_off;
#pragma unroll
  for (int ps = 0; ps < 4; ++ps) {
    if (ps + 1 < 4) {
#pragma unroll
      for (int i = 0; i < 4; ++i) st[(ps + 1) & 1][i] = src0[(ps + 1) * 4 * (D / 4) + i * 8];
    }
    const int row = warp * 16 + ps * 4 + (lane >> 3);
    float4(&s4)[4] = st[ps & 1];
    for (int t = 0; t < f.n; ++t) {
      const float kr = sh.kinv[t], bt = sh.beta[t], bk = bt * kr;
      float4 kk[4];
      float d = 0.0f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 g = reinterpret_cast<const float4*>(sh.gam[t])[i * 8 + j8];
        kk[i] = reinterpret_cast<const float4*>(sh.k[t])[i * 8 + j8];
        s4[i].x *= g.x; s4[i].y *= g.y; s4[i].z *= g.z; s4[i].w *= g.w;
        d += dot4(s4[i], kk[i]);
      }
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      d += __shfl_xor_sync(0xffffffffu, d, 4);
      const float vn = (sh.v[t][row] * bt - d * bk) * kr;   // (v - kr d) beta, times kr for the update
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s4[i].x = fmaf(vn, kk[i].x, s4[i].x);
        s4[i].y = fmaf(vn, kk[i].y, s4[i].y);
        s4[i].z = fmaf(vn, kk[i].z, s4[i].z);
        s4[i].w = fmaf(vn, kk[i].w, s4[i].w);
      }
      if (snap != nullptr && t == f.snap_t) {
#pragma unroll
        for (int i = 0; i < 4; ++i) snap[ps * 4 * (D / 4) + i * 8] = s4[i];
      }
    }
    if (dst != nullptr) {
#pragma unroll
      for (int i = 0; i < 4; ++i) dst[ps * 4 * (D / 4) + i * 8] = s4[i];
    }
  }
}

__device__ void fold_tile_cta(const pla_b200_kda_commit_args& p, int cta, TileSmem& sh) {
  const int hl = cta % (p.n_layers * p.H);
  const int b = cta / (p.n_layers * p.H);
  const int layer = hl / p.H, h = hl % p.H;
  const int R = p.capacity;
  const int n_commit = min(p.plan[b], CQ);   // the plan never commits more than Q <= CQ tokens
  if (n_commit <= 0) return;
  const int64_t slot = idx_at(p.source, b);
  if (slot <= p.null_block_id || slot >= p.slots) return;
  const int final_slot = p.plan[R + b], boundary = p.plan[2 * R + b], bc = p.plan[3 * R + b];
  const int64_t* L = p.layers + static_cast<int64_t>(layer) * PLA_B200_REPLAY_COLUMNS;
  float* pool = reinterpret_cast<float*>(L[PLA_B200_COL_STATE]);
  const int64_t slot_stride = L[PLA_B200_COL_STATE_STRIDE];
  const int64_t tile_off = static_cast<int64_t>(h) * TILE;
  const int64_t rec0 = (static_cast<int64_t>(b) * p.H + h) * p.Q;
  const bool final_ok = final_slot > p.null_block_id && final_slot < p.slots;
  const bool bound_ok = bc > 0 && boundary > p.null_block_id && boundary < p.slots;
  TileFold f;
  f.src = pool + slot * slot_stride + tile_off;
  f.dst = final_ok ? pool + static_cast<int64_t>(final_slot) * slot_stride + tile_off : nullptr;
  f.snap = bound_ok ? pool + static_cast<int64_t>(boundary) * slot_stride + tile_off : nullptr;
  f.snap_t = bc - 1;
  f.n = n_commit;
  f.rawk = reinterpret_cast<const __nv_bfloat16*>(L[PLA_B200_COL_RAWK]) + rec0 * D;
  f.rawv = reinterpret_cast<const __nv_bfloat16*>(L[PLA_B200_COL_RAWV]) + rec0 * D;
  f.gate = reinterpret_cast<const float*>(L[PLA_B200_COL_GATE]) + rec0 * D;
  f.beta = reinterpret_cast<const float*>(L[PLA_B200_COL_BETA]) + rec0;
  fold_tile(f, sh);
}

__global__ void __launch_bounds__(FT, 3) fold_tile_scatter_kernel(const pla_b200_kda_commit_args p, const FoldGrid g) {
  __shared__ TileSmem sh;
  if (static_cast<int>(blockIdx.x) < g.fold_ctas)
    fold_tile_cta(p, blockIdx.x, sh);
  else
    scatter_cta(p, blockIdx.x - g.fold_ctas, g.conv_tiles);
}

__global__ void __launch_bounds__(NT) fold_scatter_kernel(const pla_b200_kda_commit_args p, const FoldGrid g) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  if (static_cast<int>(blockIdx.x) < g.fold_ctas)
    fold_cta(p, blockIdx.x, *reinterpret_cast<Smem*>(smem_raw));
  else
    scatter_cta(p, blockIdx.x - g.fold_ctas, g.conv_tiles);
}

// SGLang contract: rings and state of all layers in single tensors, ring row = state slot.
__global__ void __launch_bounds__(NT) fold_layers_kernel(const pla_b200_kda_fold_args p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  Smem& sh = *reinterpret_cast<Smem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int vs = blockIdx.x % NVS;
  const int hvl = (blockIdx.x / NVS) % (p.layers * p.HV);
  const int b = blockIdx.x / (NVS * p.layers * p.HV);
  const int64_t layer = hvl / p.HV;
  const int hv = hvl % p.HV, h = hv / (p.HV / p.H);
  const int64_t slot = idx_at(p.slot_idx, b);
  const int64_t n_commit = idx_at(p.accept_lens, b);
  if (slot <= p.null_block_id || n_commit <= 0) return;
  if (slot < 0 || slot >= p.slots || n_commit > p.L) {
    if (tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_BAD_SLOT);
    return;
  }
  const bool has_track = p.track_idx.data != nullptr;
  const int64_t t_track = has_track ? idx_at(p.track_step, b) : -1;
  const int64_t slot_track = has_track ? idx_at(p.track_idx, b) : p.null_block_id;
  const int row0 = vs * BV;
  const int64_t tile_off = static_cast<int64_t>(hv) * TILE + row0 * D;
  float* pool = p.state + layer * p.state_layer_stride;
  const __nv_bfloat16* rawv = static_cast<const __nv_bfloat16*>(p.rawv) + layer * p.rawv_layer_stride +
                              slot * p.rawv_slot_stride + static_cast<int64_t>(hv) * p.L * D;
  const __nv_bfloat16* rawk = static_cast<const __nv_bfloat16*>(p.rawk) + layer * p.rawk_layer_stride +
                              slot * p.rawk_slot_stride + static_cast<int64_t>(h) * p.L * D;
  const float* gate = p.gate + layer * p.gate_layer_stride + slot * p.gate_slot_stride + static_cast<int64_t>(hv) * p.L * D;
  const float* beta = p.beta + layer * p.beta_layer_stride + slot * p.beta_slot_stride + static_cast<int64_t>(hv) * p.L;

  if (tid == 0) {
    mbar_init(&sh.bar, 1);
    fence_mbar_init();
    mbar_expect_tx(&sh.bar, kSliceBytes);
    bulk_load(sh.state, pool + slot * p.state_slot_stride + tile_off, kSliceBytes, &sh.bar);
  }
  bool loaded = false;
  const int n = static_cast<int>(n_commit);
  for (int t0 = 0; t0 < n; t0 += TS) {
    const int nt = min(TS, n - t0);
    if (t0 > 0) __syncthreads();
    for (int s = 0; s < nt; ++s) {
      const int64_t rec = static_cast<int64_t>(t0 + s) * D;
      const float kf = __bfloat162float(rawk[rec + tid]);
      sh.k[s][tid] = kf;
      sh.gam[s][tid] = fast_exp(gate[rec + tid]);
      const float sk = warp_sum(kf * kf);
      if (lane == 0) sh.part[s][1][warp] = sk;
      if (tid < BV) sh.v[s][tid] = __bfloat162float(rawv[rec + row0 + tid]);
      if (tid == 0) sh.beta[s] = beta[t0 + s];
    }
    __syncthreads();
    if (!loaded) {
      const bool ok = mbar_wait(&sh.bar, 0);
      if (__syncthreads_or(!ok)) {
        if (tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_WAIT_TIMEOUT);
        (void)mbar_wait(&sh.bar, 0);
        return;
      }
      loaded = true;
    }
    for (int s = 0; s < nt; ++s) {
      float sk = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) sk += sh.part[s][1][w];
      const float kinv = 1.0f / sqrtf(sk + 1e-6f);  // division form, as the records are replayed
      float* snap = nullptr;
      if (has_track && t0 + s == t_track && slot_track > p.null_block_id && slot_track >= 0 && slot_track < p.slots)
        snap = pool + slot_track * p.state_slot_stride + tile_off;
      kda_step<false>(sh.state, sh.k[s], nullptr, sh.gam[s], sh.v[s], kinv, 0.f, sh.beta[s], nullptr, snap, warp * 8,
                      lane);
    }
  }
  fence_async_smem();
  __syncthreads();
  if (tid == 0) {
    bulk_store(pool + slot * p.state_slot_stride + tile_off, sh.state, kSliceBytes);
    bulk_commit();
    bulk_wait_read<0>();
  }
}

// The same fold for rings of at most CQ steps, one CTA per (request, layer, value head) on the whole tile (see
// `fold_tile`): the state is folded in place, the tracked snapshot taken after step `track_step`.
__global__ void __launch_bounds__(FT, 3) fold_layers_tile_kernel(const pla_b200_kda_fold_args p) {
  __shared__ TileSmem sh;
  const int hvl = blockIdx.x % (p.layers * p.HV);
  const int b = blockIdx.x / (p.layers * p.HV);
  const int64_t layer = hvl / p.HV;
  const int hv = hvl % p.HV, h = hv / (p.HV / p.H);
  const int64_t slot = idx_at(p.slot_idx, b);
  const int64_t n_commit = idx_at(p.accept_lens, b);
  if (slot <= p.null_block_id || n_commit <= 0) return;
  if (slot < 0 || slot >= p.slots || n_commit > p.L) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_BAD_SLOT);
    return;
  }
  const bool has_track = p.track_idx.data != nullptr;
  const int64_t t_track = has_track ? idx_at(p.track_step, b) : -1;
  const int64_t slot_track = has_track ? idx_at(p.track_idx, b) : p.null_block_id;
  const int64_t tile_off = static_cast<int64_t>(hv) * TILE;
  float* pool = p.state + layer * p.state_layer_stride;
  TileFold f;
  f.src = pool + slot * p.state_slot_stride + tile_off;
  f.dst = pool + slot * p.state_slot_stride + tile_off;
  const bool track_ok = has_track && t_track >= 0 && t_track < n_commit && slot_track > p.null_block_id && slot_track >= 0 &&
                        slot_track < p.slots;
  f.snap = track_ok ? pool + slot_track * p.state_slot_stride + tile_off : nullptr;
  f.snap_t = static_cast<int>(t_track);
  f.n = static_cast<int>(n_commit);
  f.rawv = static_cast<const __nv_bfloat16*>(p.rawv) + layer * p.rawv_layer_stride + slot * p.rawv_slot_stride +
           static_cast<int64_t>(hv) * p.L * D;
  f.rawk = static_cast<const __nv_bfloat16*>(p.rawk) + layer * p.rawk_layer_stride + slot * p.rawk_slot_stride +
           static_cast<int64_t>(h) * p.L * D;
  f.gate = p.gate + layer * p.gate_layer_stride + slot * p.gate_slot_stride + static_cast<int64_t>(hv) * p.L * D;
  f.beta = p.beta + layer * p.beta_layer_stride + slot * p.beta_slot_stride + static_cast<int64_t>(hv) * p.L;
  fold_tile(f, sh);
}

template <typename T>
__global__ void conv_scatter_kernel(const pla_b200_kda_conv_scatter_args p) {
  const int req = blockIdx.x;
  const int64_t layer = blockIdx.y;
  const int64_t step = idx_at(p.step_idx, req), d = idx_at(p.dst_idx, req);
  if (step < 0 || d < 0 || d >= p.dst_slots || req >= p.src_rows || step >= p.src_steps) return;
  const T* src = static_cast<const T*>(p.src) + layer * p.src_layer + req * p.src_row + step * p.src_step;
  T* dst = static_cast<T*>(p.dst) + layer * p.dst_layer + d * p.dst_slot;
  const int total = p.dim * p.taps;
  for (int i = blockIdx.z * blockDim.x + threadIdx.x; i < total; i += gridDim.z * blockDim.x) {
    const int c = i / p.taps, w = i % p.taps;
    dst[c * p.dst_channel + w * p.dst_tap] = src[c * p.src_channel + w * p.src_tap];
  }
}

int check_commit(const pla_b200_kda_commit_args& a) {
  PLA_REQUIRE(a.null_block_id == -1 || a.null_block_id == 0, PLA_B200_E_INVALID, "null_block_id must be -1 or 0");
  PLA_REQUIRE(a.capacity >= 0 && a.N >= 0 && a.N <= a.capacity, PLA_B200_E_INVALID,
              "commit query count exceeds capacity");
  PLA_REQUIRE(a.Q >= 1 && a.Q <= 32 && a.H > 0 && a.slots > 0, PLA_B200_E_INVALID, "invalid commit plan dimensions");
  PLA_REQUIRE(a.token_capacity >= 0 && a.token_capacity <= INT_MAX, PLA_B200_E_INVALID,
              "token_capacity must be between 0 and INT32_MAX");
  if (a.capacity == 0) return PLA_B200_OK;
  PLA_REQUIRE(a.candidate && a.plan && a.sampled.data && a.source.data && a.cu.data, PLA_B200_E_INVALID,
              "plan buffers and index vectors are required");
  PLA_REQUIRE((a.block_size != 0) == (a.blocks.data != nullptr) && (a.block_size != 0) == (a.computed.data != nullptr),
              PLA_B200_E_INVALID, "align arguments must be supplied together");
  PLA_REQUIRE(a.block_size == 0 || (a.block_size >= a.Q && a.block_cols > 0), PLA_B200_E_INVALID,
              "invalid align table/count/block size");
  return PLA_B200_OK;
}

int launch_plan(const pla_b200_kda_commit_args& a, cudaStream_t s) {
  if (a.capacity == 0) return PLA_B200_OK;
  if (a.capacity <= 256) {
    plan_fused_kernel<<<1, 1024, 0, s>>>(a);
  } else {
    plan_build_kernel<<<(a.capacity + 127) / 128, 128, 0, s>>>(a);
    plan_protect_kernel<<<(a.capacity + 3) / 4, 128, 0, s>>>(a);
  }
  PLA_CUDA_OK(cudaGetLastError());
  return PLA_B200_OK;
}

}  // namespace
}  // namespace pla

extern "C" int pla_b200_kda_replay_verify(const pla_b200_kda_verify_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  pla_b200_kda_verify_args a = *args;
  default_status(a);
  PLA_REQUIRE(a.null_block_id == -1 || a.null_block_id == 0 || a.row_by_slot, PLA_B200_E_INVALID,
              "null_block_id must be -1 or 0");
  PLA_REQUIRE(a.H > 0 && a.N >= 0 && a.Q >= 1 && a.Q <= 32 && a.T >= 0 && a.slots > 0, PLA_B200_E_INVALID,
              "verify requires H > 0, N >= 0, Q in [1, 32], slots > 0");
  if (a.N == 0) return PLA_B200_OK;
  PLA_REQUIRE(a.x_q && a.x_k && a.x_v && a.raw_g && a.raw_beta && a.w_q && a.w_k && a.w_v && a.cs_q && a.cs_k &&
                  a.cs_v && a.A_log && a.dt_bias && a.state && a.out && a.rec_rawv && a.rec_rawk && a.rec_g &&
                  a.rec_beta && a.win_q && a.win_k && a.win_v && a.slot_idx.data && a.cu.data,
              PLA_B200_E_INVALID, "verify: a required pointer is NULL");
  PLA_REQUIRE(aligned16(a.state) && a.state_slot_stride % 4 == 0 &&
                  a.state_slot_stride >= static_cast<int64_t>(a.H) * 16384,
              PLA_B200_E_ALIGN, "state must be float4-aligned fp32 [slots,H,128,128] with contiguous pages");
  PLA_REQUIRE(a.gate == PLA_B200_GATE_SOFTPLUS || a.lower_bound < 0.0f, PLA_B200_E_INVALID,
              "scale/lower_bound must be finite fp32; bound < 0");
  static DeviceOnce configured;
  int dev = 0;
  PLA_CUDA_OK(cudaGetDevice(&dev));
  if (configured.needed(dev)) {
    PLA_CUDA_OK(cudaFuncSetAttribute(kda_verify_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sizeof(VerifySmem)));
    configured.mark(dev);
  }
  const int64_t ctas = static_cast<int64_t>(a.N) * a.H;
  PLA_REQUIRE(ctas < (1ll << 31), PLA_B200_E_TOO_LARGE, "N*H exceeds the grid limit");
  const bool onorm = a.onorm_gate != nullptr || a.onorm_weight != nullptr || a.out_f32 != nullptr;
  PLA_REQUIRE(!onorm || (a.onorm_gate && a.onorm_weight && a.out_f32 && aligned16(a.out_f32) &&
                         aligned16(a.onorm_weight) && a.onorm_eps >= 0.0f),
              PLA_B200_E_INVALID, "the fused output norm needs gate, weight, eps >= 0 and a 16-byte aligned fp32 staging buffer");
  // windows of up to eight tokens: closed form, the state streamed once into registers; longer ones: the
  // token-by-token kernel on a shared-memory copy of the state
  const int window = a.win_steps > 0 && a.win_steps < a.Q ? a.win_steps : a.Q;
  if (window <= CQ)
    kda_verify_window_kernel<<<static_cast<unsigned>(ctas), VNT, 0, static_cast<cudaStream_t>(stream)>>>(a);
  else
    kda_verify_kernel<<<static_cast<unsigned>(ctas), VNT, sizeof(VerifySmem), static_cast<cudaStream_t>(stream)>>>(a);
  PLA_CUDA_OK(cudaGetLastError());
  if (onorm) {
    kda_onorm_kernel<<<static_cast<unsigned>(a.N) * a.H, NT, 0, static_cast<cudaStream_t>(stream)>>>(a);
    PLA_CUDA_OK(cudaGetLastError());
  }
  return PLA_B200_OK;
}

extern "C" int pla_b200_kda_ring_verify(const pla_b200_kda_verify_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  PLA_REQUIRE(args->row_by_slot == 1, PLA_B200_E_INVALID, "ring verify addresses records by state slot (row_by_slot = 1)");
  return pla_b200_kda_replay_verify(args, stream);
}

extern "C" int pla_b200_kda_fold_layers(const pla_b200_kda_fold_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  pla_b200_kda_fold_args a = *args;
  default_status(a);
  PLA_REQUIRE(a.layers > 0 && a.B >= 0 && a.H > 0 && a.HV >= a.H && a.HV % a.H == 0 && a.L >= 1 && a.L <= 32 &&
                  a.slots > 0,
              PLA_B200_E_INVALID, "fold requires grouped heads, positive dimensions, and ring length 1..32");
  if (a.B == 0) return PLA_B200_OK;
  PLA_REQUIRE(a.state && a.rawv && a.rawk && a.gate && a.beta && a.slot_idx.data && a.accept_lens.data,
              PLA_B200_E_INVALID, "fold: a required pointer is NULL");
  PLA_REQUIRE((a.track_idx.data != nullptr) == (a.track_step.data != nullptr), PLA_B200_E_INVALID,
              "tracking indices and steps must be supplied together");
  PLA_REQUIRE(aligned16(a.state) && a.state_slot_stride % 4 == 0 && a.state_layer_stride % 4 == 0, PLA_B200_E_ALIGN,
              "recurrent state must be 16-byte aligned");
  static DeviceOnce configured;
  int dev = 0;
  PLA_CUDA_OK(cudaGetDevice(&dev));
  if (configured.needed(dev)) {
    PLA_CUDA_OK(cudaFuncSetAttribute(fold_layers_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sizeof(Smem)));
    configured.mark(dev);
  }
  const bool whole_tiles = a.L <= CQ;   // short rings: one CTA streams the whole tile through registers
  const int64_t ctas = static_cast<int64_t>(a.B) * a.layers * a.HV * (whole_tiles ? 1 : NVS);
  PLA_REQUIRE(ctas < (1ll << 31), PLA_B200_E_TOO_LARGE, "fold grid too large");
  if (whole_tiles) fold_layers_tile_kernel<<<static_cast<unsigned>(ctas), FT, 0, static_cast<cudaStream_t>(stream)>>>(a);
  else fold_layers_kernel<<<static_cast<unsigned>(ctas), NT, sizeof(Smem), static_cast<cudaStream_t>(stream)>>>(a);
  PLA_CUDA_OK(cudaGetLastError());
  return PLA_B200_OK;
}

extern "C" int pla_b200_kda_conv_scatter(const pla_b200_kda_conv_scatter_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  const pla_b200_kda_conv_scatter_args& a = *args;
  PLA_REQUIRE(a.layers >= 0 && a.reqs >= 0 && a.dim >= 0 && a.taps >= 1 && a.taps <= 4, PLA_B200_E_INVALID,
              "conv scatter: unsupported conv window");
  PLA_REQUIRE(a.elem_size == 2 || a.elem_size == 4, PLA_B200_E_INVALID, "conv scatter: unsupported dtype");
  if (a.reqs == 0 || a.layers == 0 || a.dim == 0) return PLA_B200_OK;
  PLA_REQUIRE(a.dst && a.src && a.dst_idx.data && a.step_idx.data, PLA_B200_E_INVALID,
              "conv scatter: a required pointer is NULL");
  PLA_REQUIRE(a.layers <= 65535, PLA_B200_E_TOO_LARGE, "too many layers");
  const int tiles = min(64, (a.dim * a.taps + 255) / 256);
  const dim3 grid(a.reqs, a.layers, tiles);
  if (a.elem_size == 2) conv_scatter_kernel<uint16_t><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  else conv_scatter_kernel<uint32_t><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  PLA_CUDA_OK(cudaGetLastError());
  return PLA_B200_OK;
}

extern "C" int pla_b200_kda_replay_plan(const pla_b200_kda_commit_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  pla_b200_kda_commit_args a = *args;
  default_status(a);
  const int rc = check_commit(a);
  if (rc != PLA_B200_OK) return rc;
  return launch_plan(a, static_cast<cudaStream_t>(stream));
}

extern "C" int pla_b200_kda_replay_commit(const pla_b200_kda_commit_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  pla_b200_kda_commit_args a = *args;
  default_status(a);
  int rc = check_commit(a);
  if (rc != PLA_B200_OK) return rc;
  PLA_REQUIRE(a.layers != nullptr && a.n_layers > 0, PLA_B200_E_INVALID, "invalid layer pointer table");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  rc = launch_plan(a, s);
  if (rc != PLA_B200_OK || a.N == 0) return rc;
  static DeviceOnce configured;
  int dev = 0;
  PLA_CUDA_OK(cudaGetDevice(&dev));
  if (configured.needed(dev)) {
    PLA_CUDA_OK(cudaFuncSetAttribute(fold_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sizeof(Smem)));
    configured.mark(dev);
  }
  FoldGrid g;
  const bool whole_tiles = a.Q <= CQ;   // at most CQ committed tokens per row: one CTA streams the whole tile
  const int cta_threads = whole_tiles ? FT : NT;
  const int64_t fold = static_cast<int64_t>(a.N) * a.n_layers * a.H * (whole_tiles ? 1 : NVS);
  g.conv_tiles = (3 * a.H * D * 3 + cta_threads * 8 - 1) / (cta_threads * 8);
  const int64_t total = fold + static_cast<int64_t>(a.N) * a.n_layers * g.conv_tiles;
  PLA_REQUIRE(total < (1ll << 31), PLA_B200_E_TOO_LARGE, "commit grid too large");
  g.fold_ctas = static_cast<int>(fold);
  if (whole_tiles) fold_tile_scatter_kernel<<<static_cast<unsigned>(total), FT, 0, s>>>(a, g);
  else fold_scatter_kernel<<<static_cast<unsigned>(total), NT, sizeof(Smem), s>>>(a, g);
  PLA_CUDA_OK(cudaGetLastError());
  return PLA_B200_OK;
}

// ------------------------------------------------------------------------------------------------
// Commit plan for callers that must not allocate.
//
// The plan is built in two phases (candidates, then conflict masking) and the phases talk through a
// [4, capacity] int32 candidate buffer that a KDAReplayCommitContext normally allocates when it is
// created. A runner that builds its context late -- after it has handed every free byte of the
// device to its cache pools, or inside a region where its allocator is frozen -- has nowhere to get
// that buffer from. For it the library carries the buffer itself: a fixed array in device memory
// that exists on every GPU that loads the library, for as long as the process lives.
//
// Limit: kStaticPlanRows request rows (64 KiB per GPU). Larger capacities are refused.
// Sharing: every call on a device uses the SAME array. Calls are safe back to back on one stream;
// two calls that overlap on the GPU (different streams, no dependency) race on it. Nothing has to be
// cleared between calls: the first phase rewrites all 4 * capacity entries it later reads.
// First call per device: looks up the array's device address (no allocation, but a runtime call
// that is not a stream operation), so make that call before any stream capture begins.
namespace pla {
namespace {
constexpr int kStaticPlanRows = 4096;
static __device__ __align__(256) int32_t g_plan_candidates[4 * kStaticPlanRows];
}  // namespace
}  // namespace pla

extern "C" int pla_b200_kda_replay_plan_static(const pla_b200_kda_commit_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  PLA_REQUIRE(args->capacity <= kStaticPlanRows, PLA_B200_E_TOO_LARGE,
              "plan capacity %d exceeds the %d rows of the built-in candidate buffer; use "
              "pla_b200_kda_replay_plan with a caller-provided buffer",
              args->capacity, kStaticPlanRows);
  // In host code the array's name is only a handle; the kernel needs the address the symbol has on
  // the CURRENT device, looked up once per device.
  static int32_t* device_address[64] = {};
  int dev = 0;
  PLA_CUDA_OK(cudaGetDevice(&dev));
  PLA_REQUIRE(dev >= 0 && dev < 64, PLA_B200_E_INVALID, "device ordinal %d out of range", dev);
  if (device_address[dev] == nullptr) {
    void* ptr = nullptr;
    PLA_CUDA_OK(cudaGetSymbolAddress(&ptr, g_plan_candidates));
    PLA_REQUIRE(ptr != nullptr, PLA_B200_E_CUDA, "the built-in candidate buffer has no device address");
    device_address[dev] = static_cast<int32_t*>(ptr);
  }
  pla_b200_kda_commit_args a = *args;
  a.candidate = device_address[dev];
  const int rc = check_commit(a);
  if (rc != PLA_B200_OK) return rc;
  return launch_plan(a, static_cast<cudaStream_t>(stream));
}
