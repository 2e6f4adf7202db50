// k-last GDN / KDA decode and MTP verify for sm_100a.
//
// Math per (request n, value head hv), h = hv / (HV/H), state S in R^{V x K}
// (src/decode/k-last/fused_sigmoid_gating_k_last_kernel.cuh:396-473, :561-605):
//   beta = sigmoid(b);  gamma = exp(log_decay(a + dt_bias))      (scalar for GDN, per K column for KDA)
//   qn = q * rsqrt(sum q^2 + 1e-6) * scale;  kn = k * rsqrt(sum k^2 + 1e-6)
//   S <- S * gamma;  delta = S kn;  v' = (v - delta) * beta;  S <- S + v' kn^T;  o = S qn
// Every V row of S evolves independently, so a CTA owns `BV` consecutive rows
// of one (slot, hv) tile: one contiguous BV*512-byte block of the pool.
//
// Data movement: the block is fetched with ONE 1-D bulk copy (TMA engine) into
// shared memory, updated in place by 128-bit shared-memory accesses (8 lanes
// per row, 3-step shuffle reductions), and written back with ONE bulk store.
// For a multi-token window the block stays in shared memory across the steps;
// per-step snapshots (SGLang cache rows or vLLM per-token slots) are written
// straight from registers with 128-bit stores.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"
#include "decode_klast.h"

namespace pla {

namespace {

constexpr int D = 128;          // K = V = 128
constexpr int TILE = D * D;     // elements of one (slot, hv) state

template <int BV, int TS, bool IS_KDA>
struct KlastSmem {
  // state first: bulk copies need 16-byte alignment, the dynamic smem base has it.
  static constexpr int kState = 0;
  static constexpr int kQ = kState + BV * D * 4;
  static constexpr int kK = kQ + TS * D * 4;
  static constexpr int kGam = kK + TS * D * 4;
  static constexpr int kBeta = kGam + (IS_KDA ? TS * D * 4 : TS * 4);
  static constexpr int kV = kBeta + TS * 4;
  static constexpr int kO = kV + TS * BV * 4;
  static constexpr int kBar = (kO + TS * BV * 4 + 7) & ~7;
  static constexpr int kBytes = kBar + 8;
};

// 4 consecutive state elements of a pool that is fp32 or bf16.
__device__ __forceinline__ float4 load_state4(const void* base, int64_t off, bool f32) {
  if (f32) return *reinterpret_cast<const float4*>(static_cast<const float*>(base) + off);
  const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(base) + off);
  const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
  return make_float4(__bfloat162float(e[0]), __bfloat162float(e[1]), __bfloat162float(e[2]), __bfloat162float(e[3]));
}
__device__ __forceinline__ void store_state4(void* base, int64_t off, const float4& v, bool f32) {
  if (f32) {
    *reinterpret_cast<float4*>(static_cast<float*>(base) + off) = v;
  } else {
    __nv_bfloat16 e[4] = {__float2bfloat16_rn(v.x), __float2bfloat16_rn(v.y), __float2bfloat16_rn(v.z),
                          __float2bfloat16_rn(v.w)};
    *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(base) + off) = *reinterpret_cast<const uint2*>(e);
  }
}
template <typename T>
__device__ __forceinline__ float4 load4_scalar(const T* p) {
  return make_float4(to_f32(p[0]), to_f32(p[1]), to_f32(p[2]), to_f32(p[3]));
}

template <typename act_t, int BV, int NT, int TS, bool IS_KDA>
__global__ void __launch_bounds__(NT) klast_kernel(const pla_b200_klast_args p) {
  using L = KlastSmem<BV, TS, IS_KDA>;
  constexpr int NVS = D / BV;      // row slices per tile
  constexpr int NW = NT / 32;      // warps
  constexpr int RP = NT / 8;       // rows per pass (8 lanes per row)
  constexpr int PASSES = BV / RP;
  static_assert(BV % RP == 0 && PASSES >= 1, "rows per CTA must be a multiple of rows per pass");

  extern __shared__ __align__(128) unsigned char smem[];
  float* s_state = reinterpret_cast<float*>(smem + L::kState);
  float* s_q = reinterpret_cast<float*>(smem + L::kQ);
  float* s_k = reinterpret_cast<float*>(smem + L::kK);
  float* s_gam = reinterpret_cast<float*>(smem + L::kGam);
  float* s_beta = reinterpret_cast<float*>(smem + L::kBeta);
  float* s_v = reinterpret_cast<float*>(smem + L::kV);
  float* s_o = reinterpret_cast<float*>(smem + L::kO);
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + L::kBar);

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int HV = p.HV, H = p.H;

  const unsigned bid = blockIdx.x;
  const unsigned work_ctas = static_cast<unsigned>(p.B) * HV * NVS;
  if (bid >= work_ctas) {
    // Trailing CTAs: physical token rows past the last sequence get zero output.
    const int64_t first = p.cu_seqlens != nullptr ? p.cu_seqlens[p.B] : static_cast<int64_t>(p.B) * p.t_max;
    const int64_t words = (p.o_total_rows - first) * HV * (D / 2);  // 16-bit outputs, two per word
    if (first < 0 || words <= 0) return;
    uint32_t* dst = reinterpret_cast<uint32_t*>(static_cast<act_t*>(p.o) + first * HV * D);
    for (int64_t i = static_cast<int64_t>(bid - work_ctas) * NT + tid; i < words;
         i += static_cast<int64_t>(gridDim.x - work_ctas) * NT)
      dst[i] = 0u;
    return;
  }
  const int vs = bid % NVS;
  const int hv = (bid / NVS) % HV;
  const int n = bid / (NVS * HV);
  const int h = hv / (HV / H);
  const int row0 = vs * BV;

  int64_t bos, eos;
  if (p.cu_seqlens != nullptr) {
    bos = p.cu_seqlens[n];
    eos = p.cu_seqlens[n + 1];
  } else {
    bos = static_cast<int64_t>(n) * p.t_max;
    eos = bos + p.t_max;
  }
  if (bos < 0 || eos < bos || eos - bos > p.t_max) {
    if (tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_BAD_INTERVAL);
    return;
  }
  const int T = static_cast<int>(eos - bos);
  if (T == 0) return;  // empty request: nothing read, nothing written

  // ---- slot lookup ----
  const bool table2d = p.slot_row_stride > 0;
  int slot;
  if (table2d) {
    const int acc = (p.num_accepted != nullptr) ? p.num_accepted[n] : 1;
    int col = acc > 0 ? acc - 1 : 0;
    if (col >= p.slot_cols) col = p.slot_cols - 1;
    slot = p.slot_indices[static_cast<int64_t>(n) * p.slot_row_stride + col];
  } else if (p.slot_indices != nullptr) {
    slot = p.slot_indices[n];
  } else {
    slot = n;  // state_by_request
  }
  // Prescan (context parallelism): blockIdx.y = 0 runs the range from a zero state (offset B), 1 from the
  // identity with V = 0 (transition M); no output rows, no slot pool, results to state_out
  // [request][HV][2][V][K] fp32.
  const bool prescan = p.prescan != 0;
  const int kind = prescan ? static_cast<int>(blockIdx.y) : 0;
  if (prescan) slot = 0;
  const bool is_pad = !prescan && p.slot_indices != nullptr && ((p.pad == PLA_B200_PAD_SGLANG) ? (slot < 0) : (slot <= 0));
  const bool oob = !is_pad && p.num_slots > 0 && slot >= p.num_slots;
  act_t* o_base = static_cast<act_t*>(p.o) + hv * D + row0;
  if (is_pad || oob) {
    if (oob && tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_BAD_SLOT);
    for (int i = tid; i < T * BV; i += NT) {
      const int t = i / BV, r = i % BV;
      o_base[(bos + t) * static_cast<int64_t>(HV) * D + r] = from_f32<act_t>(0.0f);
    }
    return;
  }

  // Element offset of this CTA's rows inside a slot: contiguous for [V,K] slots; for
  // transposed [K,V] slots the rows are columns and are gathered by hand.
  const int64_t tile_off = static_cast<int64_t>(hv) * TILE + (p.state_transposed ? row0 : row0 * D);
  const int64_t in_off = static_cast<int64_t>(slot) * p.state_slot_stride + tile_off;
  const bool f32_state = p.state_dtype == PLA_B200_F32;
  const bool bulk_io = f32_state && !p.state_transposed;
  float* g_tile = static_cast<float*>(p.state) + in_off;  // only dereferenced when bulk_io
  constexpr uint32_t kBlockBytes = BV * D * 4;
  const bool bulk_in = bulk_io && !p.state_init_zero && !prescan;

  if (bulk_in) {
    if (tid == 0) {
      mbar_init(bar, 1);
      fence_mbar_init();
      mbar_expect_tx(bar, kBlockBytes);
      bulk_load(s_state, g_tile, kBlockBytes, bar);
    }
  } else {
    // zero start, 16-bit pool or transposed slots: fill shared memory by hand (once per sequence)
    for (int i = tid; i < BV * D; i += NT) {
      float x = 0.0f;
      if (prescan) {
        s_state[i] = (kind == 1 && row0 + i / D == i % D) ? 1.0f : 0.0f;
      } else if (!p.state_init_zero) {
        const int r = p.state_transposed ? (i % BV) : (i / D);
        const int c = p.state_transposed ? (i / BV) : (i % D);
        const int64_t e = in_off + (p.state_transposed ? static_cast<int64_t>(c) * D + r : static_cast<int64_t>(r) * D + c);
        x = load_any(p.state, p.state_dtype, e);
        s_state[r * D + c] = x;
      } else {
        s_state[i] = 0.0f;
      }
    }
  }

  // ---- snapshot destinations ----
  int cache_idx = -1;
  if (p.cache != nullptr && p.cache_indices != nullptr && p.pad == PLA_B200_PAD_SGLANG)
    cache_idx = p.cache_indices[n];
  // element offset of this CTA's rows in step 0 of the request's snapshot row, or -1
  const int64_t cache_off = (cache_idx >= 0) ? static_cast<int64_t>(cache_idx) * p.cache_steps * HV * TILE +
                                                   static_cast<int64_t>(hv) * TILE + row0 * D
                                             : -1;

  const act_t* gq = static_cast<const act_t*>(p.q) + h * D;
  const act_t* gk = static_cast<const act_t*>(p.k) + h * D;
  const act_t* gv = static_cast<const act_t*>(p.v) + hv * D + row0;
  const act_t* ga = static_cast<const act_t*>(p.a);
  const act_t* gb = static_cast<const act_t*>(p.b);
  const float A_log = load_any(p.A_log, p.A_log_dtype, hv);

  const int r_in_pass = warp * 4 + (lane >> 3);  // row inside a pass
  const int j = lane & 7;                        // lane inside the row
  bool loaded = false;
  // 8-byte vector loads of q/k/gate rows need aligned rows; sliced projection
  // buffers may be only 2-byte aligned and then take element loads.
  const auto al8 = [](const void* ptr, int64_t stride) {
    return ((reinterpret_cast<uintptr_t>(ptr) & 7) == 0) && (stride % 4 == 0);
  };
  const bool io_vec = al8(p.q, p.q_tok_stride) && al8(p.k, p.k_tok_stride) &&
                      (!IS_KDA || p.gate_activated || al8(p.a, p.a_tok_stride));

  for (int t0 = 0; t0 < T; t0 += TS) {
    const int nt = min(TS, T - t0);
    if (t0 > 0) __syncthreads();  // previous chunk's parameters and outputs fully consumed

    // ---- per-step parameters, one warp per step ----
    for (int s = warp; s < nt; s += NW) {
      const int64_t tok = bos + t0 + s;
      float4 qv = io_vec ? load4(gq + tok * p.q_tok_stride + lane * 4) : load4_scalar(gq + tok * p.q_tok_stride + lane * 4);
      float4 kv = io_vec ? load4(gk + tok * p.k_tok_stride + lane * 4) : load4_scalar(gk + tok * p.k_tok_stride + lane * 4);
      float qr = p.scale, kr = 1.0f;
      if (p.use_qk_l2norm) {
        const float qs = warp_sum(dot4(qv, qv));
        const float ks = warp_sum(dot4(kv, kv));
        qr = rsqrtf(qs + 1e-6f) * p.scale;
        kr = rsqrtf(ks + 1e-6f);
      }
      reinterpret_cast<float4*>(s_q + s * D)[lane] = make_float4(qv.x * qr, qv.y * qr, qv.z * qr, qv.w * qr);
      reinterpret_cast<float4*>(s_k + s * D)[lane] = make_float4(kv.x * kr, kv.y * kr, kv.z * kr, kv.w * kr);
      if (p.gate_activated) {
        // a holds fp32 log-decays, b fp32 betas: nothing left to activate
        const float* fa = static_cast<const float*>(p.a);
        if constexpr (IS_KDA) {
          const float* row = fa + tok * p.a_tok_stride + hv * D + lane * 4;
          reinterpret_cast<float4*>(s_gam + s * D)[lane] =
              make_float4(fast_exp(row[0]), fast_exp(row[1]), fast_exp(row[2]), fast_exp(row[3]));
        } else if (lane == 0) {
          s_gam[s] = fast_exp(fa[tok * p.a_tok_stride + hv]);
        }
        if (lane == 0) s_beta[s] = static_cast<const float*>(p.b)[tok * p.b_tok_stride + hv];
        for (int i = lane; i < BV; i += 32) s_v[s * BV + i] = kind == 1 ? 0.0f : to_f32(gv[tok * p.v_tok_stride + i]);
        continue;
      }
      if constexpr (IS_KDA) {
        const float4 av = io_vec ? load4(ga + tok * p.a_tok_stride + hv * D + lane * 4)
                                 : load4_scalar(ga + tok * p.a_tok_stride + hv * D + lane * 4);
        const int64_t c = static_cast<int64_t>(hv) * D + lane * 4;
        float4 g;
        g.x = fast_exp(log_decay(av.x + load_any(p.dt_bias, p.dt_bias_dtype, c + 0), A_log, p.gate,
                               p.softplus_beta, p.softplus_threshold, p.lower_bound));
        g.y = fast_exp(log_decay(av.y + load_any(p.dt_bias, p.dt_bias_dtype, c + 1), A_log, p.gate,
                               p.softplus_beta, p.softplus_threshold, p.lower_bound));
        g.z = fast_exp(log_decay(av.z + load_any(p.dt_bias, p.dt_bias_dtype, c + 2), A_log, p.gate,
                               p.softplus_beta, p.softplus_threshold, p.lower_bound));
        g.w = fast_exp(log_decay(av.w + load_any(p.dt_bias, p.dt_bias_dtype, c + 3), A_log, p.gate,
                               p.softplus_beta, p.softplus_threshold, p.lower_bound));
        reinterpret_cast<float4*>(s_gam + s * D)[lane] = g;
      } else if (lane == 0) {
        const float x = to_f32(ga[tok * p.a_tok_stride + hv]) + load_any(p.dt_bias, p.dt_bias_dtype, hv);
        s_gam[s] = fast_exp(log_decay(x, A_log, p.gate, p.softplus_beta, p.softplus_threshold, p.lower_bound));
      }
      if (lane == 0) s_beta[s] = sigmoidf_fast(to_f32(gb[tok * p.b_tok_stride + hv]));
      for (int i = lane; i < BV; i += 32) s_v[s * BV + i] = kind == 1 ? 0.0f : to_f32(gv[tok * p.v_tok_stride + i]);
    }

    // Step parameters visible to all; also orders the mbarrier initialisation
    // by thread 0 before anybody polls it.
    __syncthreads();

    if (!loaded && bulk_in) {
      // Bounded wait for the state block; on timeout flag it, give the copy a
      // second bounded chance to land (shared memory must not be released
      // under it) and leave without touching global memory.
      const bool ok = mbar_wait(bar, 0);
      if (__syncthreads_or(!ok)) {  // CTA-uniform decision
        if (tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_WAIT_TIMEOUT);
        (void)mbar_wait(bar, 0);
        return;
      }
      loaded = true;
    }

    for (int s = 0; s < nt; ++s) {
      const int t = t0 + s;
      float4 kk[4], qq[4], gg[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        kk[i] = reinterpret_cast<const float4*>(s_k + s * D)[i * 8 + j];
        qq[i] = reinterpret_cast<const float4*>(s_q + s * D)[i * 8 + j];
        if constexpr (IS_KDA) gg[i] = reinterpret_cast<const float4*>(s_gam + s * D)[i * 8 + j];
      }
      float gs = 1.0f;
      if constexpr (!IS_KDA) gs = s_gam[s];
      const float beta = s_beta[s];

      // where this step's state snapshot goes (NULL: nowhere)
      void* snap_base = nullptr;
      int64_t snap_off = 0;
      if (cache_off >= 0) {
        if (t < p.cache_steps) {
          snap_base = p.cache;
          snap_off = cache_off + static_cast<int64_t>(t) * HV * TILE;
        }
      } else if (table2d && p.pad == PLA_B200_PAD_VLLM && t < p.slot_cols) {
        const int step_slot = p.slot_indices[static_cast<int64_t>(n) * p.slot_row_stride + t];
        if (step_slot > 0 && (p.num_slots <= 0 || step_slot < p.num_slots)) {
          snap_base = p.state;
          snap_off = static_cast<int64_t>(step_slot) * p.state_slot_stride + static_cast<int64_t>(hv) * TILE + row0 * D;
        }
      }

      // EAGLE tree: continue from the parent's snapshot instead of step t-1.
      // The snapshot rows were written by these same threads earlier in this
      // launch, so plain loads observe them without a fence.
      int64_t reload_off = -1;
      if (p.parents != nullptr && t != 0 && cache_off >= 0) {
        const int64_t pi = static_cast<int64_t>(n) * p.parents_seq_stride + static_cast<int64_t>(t) * p.parents_tok_stride;
        const int64_t parent = p.parents_wide ? static_cast<const int64_t*>(p.parents)[pi]
                                              : static_cast<const int32_t*>(p.parents)[pi];
        if (parent >= t) {
          if (tid == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_BAD_PARENT);
          return;
        }
        if (parent >= 0 && parent != t - 1) reload_off = cache_off + parent * static_cast<int64_t>(HV) * TILE;
      }

#pragma unroll
      for (int ps = 0; ps < PASSES; ++ps) {
        const int row = ps * RP + r_in_pass;
        float4* srow = reinterpret_cast<float4*>(s_state + row * D);
        float4 st[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (reload_off >= 0)
            st[i] = load_state4(p.cache, reload_off + row * D + (i * 8 + j) * 4, f32_state);
          else
            st[i] = srow[i * 8 + j];
        }
        float d = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if constexpr (IS_KDA) {
            st[i].x *= gg[i].x; st[i].y *= gg[i].y; st[i].z *= gg[i].z; st[i].w *= gg[i].w;
          } else {
            st[i].x *= gs; st[i].y *= gs; st[i].z *= gs; st[i].w *= gs;
          }
          d += dot4(st[i], kk[i]);
        }
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        d += __shfl_xor_sync(0xffffffffu, d, 2);
        d += __shfl_xor_sync(0xffffffffu, d, 4);
        const float vn = (s_v[s * BV + row] - d) * beta;
        float oacc = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          st[i].x += kk[i].x * vn; st[i].y += kk[i].y * vn; st[i].z += kk[i].z * vn; st[i].w += kk[i].w * vn;
          oacc += dot4(st[i], qq[i]);
          srow[i * 8 + j] = st[i];
          if (snap_base != nullptr) store_state4(snap_base, snap_off + row * D + (i * 8 + j) * 4, st[i], f32_state);
        }
        oacc += __shfl_xor_sync(0xffffffffu, oacc, 1);
        oacc += __shfl_xor_sync(0xffffffffu, oacc, 2);
        oacc += __shfl_xor_sync(0xffffffffu, oacc, 4);
        if (j == 0) s_o[s * BV + row] = oacc;
      }
    }
    __syncthreads();
    if (!prescan) {
      for (int i = tid; i < nt * BV; i += NT) {
        const int s = i / BV, r = i % BV;
        o_base[(bos + t0 + s) * static_cast<int64_t>(HV) * D + r] = from_f32<act_t>(s_o[i]);
      }
    }
  }

  if (prescan) {
    float* dst = static_cast<float*>(p.state_out) + ((static_cast<int64_t>(n) * HV + hv) * 2 + kind) * TILE + row0 * D;
    fence_async_smem();
    __syncthreads();
    if (tid == 0) {
      bulk_store(dst, s_state, kBlockBytes);
      bulk_commit();
      bulk_wait_read<0>();
    }
    return;
  }

  if (!p.disable_state_update) {
    void* dst_base = p.state;
    int64_t dst_off = in_off;
    if (p.state_out != nullptr) {
      const int64_t oslot = p.state_out_indices != nullptr ? p.state_out_indices[n] : n;
      dst_base = p.state_out;
      dst_off = oslot * p.state_out_slot_stride + tile_off;
    }
    if (bulk_io) {
      // generic-proxy writes to s_state -> visible to the bulk-copy engine
      fence_async_smem();
      __syncthreads();
      if (tid == 0) {
        bulk_store(static_cast<float*>(dst_base) + dst_off, s_state, kBlockBytes);
        bulk_commit();
        bulk_wait_read<0>();  // shared memory must stay valid until the engine has read it
      }
    } else {
      __syncthreads();
      for (int i = tid; i < BV * D; i += NT) {
        const int r = p.state_transposed ? (i % BV) : (i / D);
        const int c = p.state_transposed ? (i / BV) : (i % D);
        const int64_t e = dst_off + (p.state_transposed ? static_cast<int64_t>(c) * D + r : static_cast<int64_t>(r) * D + c);
        if (f32_state) static_cast<float*>(dst_base)[e] = s_state[r * D + c];
        else static_cast<__nv_bfloat16*>(dst_base)[e] = __float2bfloat16_rn(s_state[r * D + c]);
      }
    }
  }
}

template <typename act_t, int BV, int NT, int TS, bool IS_KDA>
int launch_one(const pla_b200_klast_args& a, cudaStream_t stream) {
  using L = KlastSmem<BV, TS, IS_KDA>;
  auto kern = klast_kernel<act_t, BV, NT, TS, IS_KDA>;
  static DeviceOnce configured;
  int dev = 0;
  PLA_CUDA_OK(cudaGetDevice(&dev));
  if (configured.needed(dev)) {
    PLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes));
    configured.mark(dev);
  }
  int64_t ctas = static_cast<int64_t>(a.B) * a.HV * (D / BV);
  if (a.o_total_rows > 0 && !a.prescan) ctas += 64;  // CTAs that zero the padded output suffix
  PLA_REQUIRE(ctas < (1ll << 31), PLA_B200_E_TOO_LARGE, "B*HV*(128/rows_per_cta) exceeds the grid limit");
  kern<<<dim3(static_cast<unsigned>(ctas), a.prescan ? 2 : 1), NT, L::kBytes, stream>>>(a);
  PLA_CUDA_OK(cudaGetLastError());
  return PLA_B200_OK;
}

template <typename act_t, bool IS_KDA>
int launch_shape(const pla_b200_klast_args& a, cudaStream_t stream) {
  const bool multi = a.t_max > 1;
  int rows = a.rows_per_cta;
  if (rows == 0) {
    // Enough CTAs to cover the machine several times over -> larger blocks.
    const int64_t tiles = static_cast<int64_t>(a.B) * a.HV;
    rows = (tiles >= 16 * sm_count()) ? 64 : 32;
  }
  if (multi) {
    switch (rows) {
      case 32: return launch_one<act_t, 32, 128, 4, IS_KDA>(a, stream);
      case 64: return launch_one<act_t, 64, 256, 4, IS_KDA>(a, stream);
      case 128: return launch_one<act_t, 128, 256, 4, IS_KDA>(a, stream);
    }
  } else {
    switch (rows) {
      case 32: return launch_one<act_t, 32, 128, 1, IS_KDA>(a, stream);
      case 64: return launch_one<act_t, 64, 256, 1, IS_KDA>(a, stream);
      case 128: return launch_one<act_t, 128, 256, 1, IS_KDA>(a, stream);
    }
  }
  PLA_REQUIRE(false, PLA_B200_E_INVALID, "rows_per_cta must be 0, 1, 16, 32, 64 or 128 (got %d)", rows);
}

}  // namespace

}  // namespace pla

extern "C" int pla_b200_decode_klast(const pla_b200_klast_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  pla_b200_klast_args a = *args;
  default_status(a);
  PLA_REQUIRE(a.B >= 0 && a.t_max >= 0, PLA_B200_E_INVALID, "B and t_max must be non-negative");
  if (a.B == 0 || a.t_max == 0) return PLA_B200_OK;
  PLA_REQUIRE(a.H > 0 && a.HV >= a.H && a.HV % a.H == 0, PLA_B200_E_INVALID,
              "HV must be a positive multiple of H, got H=%d, HV=%d", a.H, a.HV);
  PLA_REQUIRE(a.q && a.k && a.v && a.a && a.b && (a.o || a.prescan) && a.A_log && a.dt_bias, PLA_B200_E_INVALID,
              "q, k, v, a, b, o, A_log and dt_bias are required");
  PLA_REQUIRE(a.prescan || ((a.state != nullptr || a.state_init_zero) && (a.slot_indices != nullptr || a.state_by_request)),
              PLA_B200_E_INVALID, "the state pool and its slot indices are required");
  PLA_REQUIRE(!a.prescan || (a.state_out != nullptr && a.cu_seqlens != nullptr && a.slot_row_stride == 0 &&
                             a.cache == nullptr),
              PLA_B200_E_INVALID, "a prescan needs cu_seqlens and state_out [B, HV, 2, 128, 128] fp32, and no cache or slot table");
  PLA_REQUIRE(a.state != nullptr || a.state_out != nullptr || a.disable_state_update, PLA_B200_E_INVALID,
              "a final state needs somewhere to go");
  PLA_REQUIRE(a.act_dtype == PLA_B200_BF16 || a.act_dtype == PLA_B200_F16, PLA_B200_E_INVALID,
              "activation dtype must be bf16 or fp16");
  PLA_REQUIRE(a.state_dtype == PLA_B200_F32 || a.state_dtype == PLA_B200_BF16, PLA_B200_E_INVALID,
              "state dtype must be fp32 or bf16");
  PLA_REQUIRE(a.state == nullptr || a.state_slot_stride >= static_cast<int64_t>(a.HV) * 16384, PLA_B200_E_INVALID,
              "state slot pitch must cover HV*128*128 elements");
  PLA_REQUIRE(a.state == nullptr ||
                  (aligned16(a.state) && a.state_slot_stride % (a.state_dtype == PLA_B200_F32 ? 4 : 8) == 0),
              PLA_B200_E_ALIGN,
              "state pool base and slot pitch must be 16-byte aligned");
  PLA_REQUIRE(a.state_out == nullptr || (aligned16(a.state_out) && (a.prescan || (a.state_out_slot_stride % 4 == 0 &&
                                         a.state_out_slot_stride >= static_cast<int64_t>(a.HV) * 16384))),
              PLA_B200_E_ALIGN, "final-state base and slot pitch must be 16-byte aligned and cover HV*128*128");
  PLA_REQUIRE(a.cache == nullptr || aligned16(a.cache), PLA_B200_E_ALIGN, "snapshot cache must be 16-byte aligned");
  PLA_REQUIRE(a.o_total_rows == 0 || (reinterpret_cast<uintptr_t>(a.o) & 3) == 0, PLA_B200_E_ALIGN,
              "o must be 4-byte aligned");
  PLA_REQUIRE(a.gate == PLA_B200_GATE_SOFTPLUS || (a.gate == PLA_B200_GATE_SAFE && a.is_kda), PLA_B200_E_INVALID,
              "lower_bound is only supported for KDA");
  PLA_REQUIRE(a.slot_row_stride == 0 || a.pad == PLA_B200_PAD_VLLM, PLA_B200_E_INVALID,
              "a 2-D slot table is the vLLM layout; pass the vLLM padding convention");
  PLA_REQUIRE(a.slot_row_stride == 0 || a.slot_cols > 0, PLA_B200_E_INVALID, "2-D slot table needs slot_cols > 0");
  PLA_REQUIRE(a.parents == nullptr || a.cache != nullptr, PLA_B200_E_INVALID,
              "a parent table needs the snapshot cache");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // rows_per_cta: 0 = pick (streaming kernel when the call qualifies), 16 = streaming kernel or error,
  // 32/64/128 = the one-block-per-CTA kernel.
  if (a.rows_per_cta == 16 || a.rows_per_cta == 17 || a.rows_per_cta == 1)
    PLA_REQUIRE(klast_stream_eligible(a), PLA_B200_E_INVALID,
                "rows_per_cta=16 / 1 select the single-token decode kernels, which need a plain single-token call");
  if (a.rows_per_cta == 1) {
    PLA_REQUIRE(a.state_dtype == PLA_B200_F32, PLA_B200_E_INVALID, "rows_per_cta=1 needs an fp32 pool");
    return launch_klast_rows(a, s);
  }
  if ((a.rows_per_cta == 0 || a.rows_per_cta == 16 || a.rows_per_cta == 17) && klast_stream_eligible(a))
    return launch_klast_stream(a, s);
  if (a.act_dtype == PLA_B200_BF16)
    return a.is_kda ? launch_shape<__nv_bfloat16, true>(a, s) : launch_shape<__nv_bfloat16, false>(a, s);
  return a.is_kda ? launch_shape<__half, true>(a, s) : launch_shape<__half, false>(a, s);
}

extern "C" int pla_b200_prefill_recurrent(const pla_b200_klast_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  PLA_REQUIRE(args->cu_seqlens != nullptr, PLA_B200_E_INVALID, "prefill needs cu_seqlens");
  PLA_REQUIRE(args->slot_row_stride == 0 && args->cache == nullptr && args->parents == nullptr,
              PLA_B200_E_INVALID, "prefill takes no snapshot cache, parent table or 2-D slot table");
  pla_b200_klast_args a = *args;
  if (a.rows_per_cta == 0 || a.rows_per_cta == 16 || a.rows_per_cta == 17) a.rows_per_cta = 32;  // most CTAs per sequence
  if (a.t_max < 2) a.t_max = 2;                                         // always the multi-step kernel
  return pla_b200_decode_klast(&a, stream);
}
