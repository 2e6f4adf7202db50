// Persistent streaming kernel for single-token k-last decode (the production
// decode step): every (request, value head) 128x128 fp32 state is read once
// and written once, in place.
//
// One CTA per SM and every WARP is its own pipeline. A warp takes TASKS of 64
// consecutive V rows (half of one (slot, hv) tile, 32 KiB contiguous in the
// pool) and streams each task as 8 UNITS of 8 rows (4 KiB): lane 0 keeps NS-1
// bulk loads (TMA engine, mbarrier completion) in flight into the warp's
// private shared-memory ring, the warp updates the landed unit in place with
// 128-bit shared-memory accesses (8 lanes per row, 3-step shuffle reductions)
// and lane 0 writes it back with a bulk store. There is no CTA-wide barrier,
// so nothing waits for the slowest warp. The token's normalised q/k, gate and
// beta are formed once per task; the raw inputs of the NEXT task are
// prefetched into registers half a task ahead.
//
// Math: src/decode/k-last/fused_sigmoid_gating_k_last_kernel.cuh:396-473, :561-605.
#include "common.cuh"
#include "decode_klast.h"

namespace pla {
namespace {

constexpr int D = 128;
constexpr int TILE = D * D;
constexpr int RU = 8;                       // state rows per unit
constexpr int UNIT_FLOATS = RU * D;         // 1024
constexpr uint32_t UNIT_BYTES = UNIT_FLOATS * 4;
constexpr int UPT = 8;                      // units per task
constexpr int TASK_ROWS = RU * UPT;         // 64
constexpr int TASKS_PER_TILE = D / TASK_ROWS;

enum : int { kSkip = 0, kActive = 1, kZero = 2 };

struct Task {
  int kind;     // kSkip: nothing; kActive: stream the rows; kZero: padded request, zero its output rows
  int hv;
  int row0;     // first V row of the task inside the tile
  int64_t tok;  // token row of the request
  float* gptr;  // first unit of the task in the pool (kActive only)
};

template <typename act_t, bool IS_KDA>
struct Raw {    // 16-bit inputs of one task, in the lane layout the compute uses
  uint2 q[4], k[4];
  uint32_t v[UPT];             // rows 2r, 2r+1 of every unit
  uint2 a4[IS_KDA ? 4 : 1];
  act_t a, b;
};

__device__ __forceinline__ Task describe(const pla_b200_klast_args& p, int task, int n_tasks) {
  Task x;
  x.kind = kSkip;
  x.hv = 0;
  x.row0 = 0;
  x.tok = 0;
  x.gptr = nullptr;
  if (task >= n_tasks) return x;
  const int part = task % TASKS_PER_TILE;
  const int t = task / TASKS_PER_TILE;
  x.hv = t % p.HV;
  x.row0 = part * TASK_ROWS;
  const int n = t / p.HV;
  int64_t bos = n, eos = n + 1;
  if (p.cu_seqlens != nullptr) {
    bos = p.cu_seqlens[n];
    eos = p.cu_seqlens[n + 1];
  }
  if (eos == bos) return x;  // empty request
  if (bos < 0 || eos < bos || eos - bos > 1) {
    if (p.status != nullptr && (threadIdx.x & 31) == 0) atomicOr(p.status, PLA_B200_DEV_BAD_INTERVAL);
    return x;
  }
  x.tok = bos;
  const int slot = p.slot_indices[n];
  const bool pad = (p.pad == PLA_B200_PAD_SGLANG) ? (slot < 0) : (slot <= 0);
  if (pad) {
    x.kind = kZero;
    return x;
  }
  if (p.num_slots > 0 && slot >= p.num_slots) {
    if (p.status != nullptr && (threadIdx.x & 31) == 0) atomicOr(p.status, PLA_B200_DEV_BAD_SLOT);
    x.kind = kZero;
    return x;
  }
  x.kind = kActive;
  x.gptr = static_cast<float*>(p.state) + static_cast<int64_t>(slot) * p.state_slot_stride +
           static_cast<int64_t>(x.hv) * TILE + x.row0 * D;
  return x;
}

template <typename act_t, bool IS_KDA>
__device__ __forceinline__ void prefetch(const pla_b200_klast_args& p, const Task& x, int r, int j,
                                         Raw<act_t, IS_KDA>& raw) {
  if (x.kind != kActive) return;
  const int h = x.hv / (p.HV / p.H);
  const act_t* gq = static_cast<const act_t*>(p.q) + x.tok * p.q_tok_stride + h * D;
  const act_t* gk = static_cast<const act_t*>(p.k) + x.tok * p.k_tok_stride + h * D;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    raw.q[i] = *reinterpret_cast<const uint2*>(gq + (i * 8 + j) * 4);
    raw.k[i] = *reinterpret_cast<const uint2*>(gk + (i * 8 + j) * 4);
  }
  const act_t* gv = static_cast<const act_t*>(p.v) + x.tok * p.v_tok_stride + x.hv * D + x.row0 + r * 2;
#pragma unroll
  for (int s = 0; s < UPT; ++s) raw.v[s] = *reinterpret_cast<const uint32_t*>(gv + s * RU);
  if constexpr (IS_KDA) {
    const act_t* ga = static_cast<const act_t*>(p.a) + x.tok * p.a_tok_stride + x.hv * D;
#pragma unroll
    for (int i = 0; i < 4; ++i) raw.a4[i] = *reinterpret_cast<const uint2*>(ga + (i * 8 + j) * 4);
  } else {
    raw.a = static_cast<const act_t*>(p.a)[x.tok * p.a_tok_stride + x.hv];
  }
  raw.b = static_cast<const act_t*>(p.b)[x.tok * p.b_tok_stride + x.hv];
}

template <typename act_t>
__device__ __forceinline__ float4 cvt4(const uint2& raw) {
  const act_t* e = reinterpret_cast<const act_t*>(&raw);
  return make_float4(to_f32(e[0]), to_f32(e[1]), to_f32(e[2]), to_f32(e[3]));
}

__device__ __forceinline__ float group8_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  return x;
}

template <typename act_t, bool IS_KDA, int NWARP, int NS>
__global__ void __launch_bounds__(NWARP * 32, 1) klast_stream_kernel(const pla_b200_klast_args p,
                                                                     const int n_tasks) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 3;  // row pair: rows 2r, 2r+1 of a unit
  const int j = lane & 7;   // position inside a row: columns (i*8+j)*4..+3, i = 0..3
  float* ring = reinterpret_cast<float*>(smem) + warp * (NS * UNIT_FLOATS);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + NWARP * NS * UNIT_BYTES) + warp * NS;

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < NS; ++s) mbar_init(&bars[s], 1);
    fence_mbar_init();
  }
  __syncwarp();

  const int gw = blockIdx.x * NWARP + warp;
  const int GW = gridDim.x * NWARP;

  Task cur = describe(p, gw, n_tasks);
  Raw<act_t, IS_KDA> raw;
  prefetch<act_t, IS_KDA>(p, cur, r, j, raw);
  if (lane == 0 && cur.kind == kActive) {
#pragma unroll
    for (int d = 0; d < NS - 1; ++d) {
      mbar_expect_tx(&bars[d], UNIT_BYTES);
      bulk_load(ring + d * UNIT_FLOATS, cur.gptr + d * UNIT_FLOATS, UNIT_BYTES, &bars[d]);
    }
  }

  // Ring position of the unit being computed and of the next load; both only
  // advance on active units so that they stay in step across padded tasks.
  int stage = 0;
  uint32_t parity = 0;  // bit s = phase of ring slot s
  bool failed = false;

  for (int task = gw; task < n_tasks && !failed; task += GW) {
    const Task nxt = describe(p, task + GW, n_tasks);  // consumed half a task later

    if (cur.kind == kActive) {
      // ---- fp32 parameters of this task's token ----
      float4 kk[4], qq[4], gg[4];
      float gs = 1.0f;
      {
        float qs = 0.f, ks = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          qq[i] = cvt4<act_t>(raw.q[i]);
          kk[i] = cvt4<act_t>(raw.k[i]);
          qs += dot4(qq[i], qq[i]);
          ks += dot4(kk[i], kk[i]);
        }
        float qr = p.scale, kr = 1.0f;
        if (p.use_qk_l2norm) {
          qr = rsqrtf(group8_sum(qs) + 1e-6f) * p.scale;
          kr = rsqrtf(group8_sum(ks) + 1e-6f);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          qq[i].x *= qr; qq[i].y *= qr; qq[i].z *= qr; qq[i].w *= qr;
          kk[i].x *= kr; kk[i].y *= kr; kk[i].z *= kr; kk[i].w *= kr;
        }
      }
      const float A_log = load_any(p.A_log, p.A_log_dtype, cur.hv);
      if constexpr (IS_KDA) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 av = cvt4<act_t>(raw.a4[i]);
          const int64_t c = static_cast<int64_t>(cur.hv) * D + (i * 8 + j) * 4;
          gg[i].x = __expf(log_decay(av.x + load_any(p.dt_bias, p.dt_bias_dtype, c + 0), A_log, p.gate,
                                     p.softplus_beta, p.softplus_threshold, p.lower_bound));
          gg[i].y = __expf(log_decay(av.y + load_any(p.dt_bias, p.dt_bias_dtype, c + 1), A_log, p.gate,
                                     p.softplus_beta, p.softplus_threshold, p.lower_bound));
          gg[i].z = __expf(log_decay(av.z + load_any(p.dt_bias, p.dt_bias_dtype, c + 2), A_log, p.gate,
                                     p.softplus_beta, p.softplus_threshold, p.lower_bound));
          gg[i].w = __expf(log_decay(av.w + load_any(p.dt_bias, p.dt_bias_dtype, c + 3), A_log, p.gate,
                                     p.softplus_beta, p.softplus_threshold, p.lower_bound));
        }
      } else {
        const float x = to_f32(raw.a) + load_any(p.dt_bias, p.dt_bias_dtype, cur.hv);
        gs = __expf(log_decay(x, A_log, p.gate, p.softplus_beta, p.softplus_threshold, p.lower_bound));
      }
      const float beta = sigmoidf_fast(to_f32(raw.b));
      uint32_t vcur[UPT];  // this task's v rows, still 16-bit (raw is refilled half way through)
#pragma unroll
      for (int s = 0; s < UPT; ++s) vcur[s] = raw.v[s];
      act_t* orow = static_cast<act_t*>(p.o) + (cur.tok * p.HV + cur.hv) * D + cur.row0 + r * 2;

#pragma unroll
      for (int sub = 0; sub < UPT; ++sub) {
        if (sub == UPT / 2) prefetch<act_t, IS_KDA>(p, nxt, r, j, raw);  // `raw` of this task is fully consumed
        float* blk = ring + stage * UNIT_FLOATS;
        // warp-uniform verdict, so that no lane is left alone at a later __syncwarp
        if (!__all_sync(0xffffffffu, mbar_wait(&bars[stage], (parity >> stage) & 1u))) {
          failed = true;
          break;
        }
        parity ^= (1u << stage);
        float ov[2];
        const act_t* vpair = reinterpret_cast<const act_t*>(&vcur[sub]);
#pragma unroll
        for (int pp = 0; pp < 2; ++pp) {
          float4* srow = reinterpret_cast<float4*>(blk + (r * 2 + pp) * D);
          float4 st[4];
          float d = 0.0f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            st[i] = srow[i * 8 + j];
            if constexpr (IS_KDA) {
              st[i].x *= gg[i].x; st[i].y *= gg[i].y; st[i].z *= gg[i].z; st[i].w *= gg[i].w;
            }
            d += dot4(st[i], kk[i]);
          }
          d = group8_sum(d);
          if constexpr (!IS_KDA) d *= gs;  // scalar decay folded: (g S) k = g (S k)
          const float vn = (to_f32(vpair[pp]) - d) * beta;
          float oacc = 0.0f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if constexpr (!IS_KDA) {
              st[i].x *= gs; st[i].y *= gs; st[i].z *= gs; st[i].w *= gs;
            }
            st[i].x = fmaf(kk[i].x, vn, st[i].x);
            st[i].y = fmaf(kk[i].y, vn, st[i].y);
            st[i].z = fmaf(kk[i].z, vn, st[i].z);
            st[i].w = fmaf(kk[i].w, vn, st[i].w);
            oacc += dot4(st[i], qq[i]);
            srow[i * 8 + j] = st[i];
          }
          ov[pp] = group8_sum(oacc);
        }
        if (j == 0) {
          if (p.o_f32 != nullptr) {
            *reinterpret_cast<float2*>(p.o_f32 + (cur.tok * p.HV + cur.hv) * D + cur.row0 + r * 2 + sub * RU) =
                make_float2(ov[0], ov[1]);
          } else {
            act_t packed[2] = {from_f32<act_t>(ov[0]), from_f32<act_t>(ov[1])};
            *reinterpret_cast<uint32_t*>(orow + sub * RU) = *reinterpret_cast<const uint32_t*>(packed);
          }
        }
        fence_async_smem();  // in-place updates -> visible to the bulk-copy engine
        __syncwarp();
        if (lane == 0) {
          // The ring slot refilled now held the unit stored one iteration ago:
          // its bulk store must have finished READING shared memory.
          bulk_wait_read<0>();
          const int refill = (stage + NS - 1) % NS;
          const int ahead = sub + NS - 1;
          const float* src = nullptr;
          if (ahead < UPT) {
            src = cur.gptr + ahead * UNIT_FLOATS;
          } else if (nxt.kind == kActive) {
            src = nxt.gptr + (ahead - UPT) * UNIT_FLOATS;
          }
          if (src != nullptr) {
            mbar_expect_tx(&bars[refill], UNIT_BYTES);
            bulk_load(ring + refill * UNIT_FLOATS, src, UNIT_BYTES, &bars[refill]);
          }
          bulk_store(cur.gptr + sub * UNIT_FLOATS, blk, UNIT_BYTES);
          bulk_commit();
        }
        stage = (stage + 1) % NS;
      }
      // A padded / empty next task got no look-ahead loads; the ring restarts at
      // the task after it (see below), so skip the slots its units would have used.
    } else {
      if (cur.kind == kZero) {
        act_t* orow = static_cast<act_t*>(p.o) + (cur.tok * p.HV + cur.hv) * D + cur.row0;
        reinterpret_cast<uint32_t*>(orow)[lane] = 0u;  // 64 rows of 16-bit zeros = 32 words
      }
      prefetch<act_t, IS_KDA>(p, nxt, r, j, raw);
      // Nothing was in flight for `cur`; start the ring for the next task.
      if (lane == 0 && nxt.kind == kActive) {
        bulk_wait_read<0>();
#pragma unroll
        for (int d = 0; d < NS - 1; ++d) {
          const int s = (stage + d) % NS;
          mbar_expect_tx(&bars[s], UNIT_BYTES);
          bulk_load(ring + s * UNIT_FLOATS, nxt.gptr + d * UNIT_FLOATS, UNIT_BYTES, &bars[s]);
        }
      }
      __syncwarp();
    }
    cur = nxt;
  }

  if (failed) {
    if (lane == 0 && p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_WAIT_TIMEOUT);
    // Up to NS-2 further loads may still target this warp's ring: give them a
    // bounded chance to land before shared memory is released. Nothing more is stored.
    for (int d = 1; d < NS - 1; ++d) {
      const int s = (stage + d) % NS;
      (void)mbar_wait(&bars[s], (parity >> s) & 1u, 1u << 16);
    }
  }
  if (lane == 0) bulk_wait_read<0>();
}

template <typename act_t, bool IS_KDA, int NWARP, int NS>
int launch_cfg(const pla_b200_klast_args& a, cudaStream_t stream) {
  constexpr int kSmem = NWARP * NS * UNIT_BYTES + NWARP * NS * 8;
  auto kern = klast_stream_kernel<act_t, IS_KDA, NWARP, NS>;
  static bool configured[64] = {};
  int dev = 0;
  PLA_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    PLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    configured[dev] = true;
  }
  const int64_t n_tasks = static_cast<int64_t>(a.B) * a.HV * TASKS_PER_TILE;
  PLA_REQUIRE(n_tasks < (1ll << 30), PLA_B200_E_TOO_LARGE, "B*HV too large for the streaming decode kernel");
  const int64_t want = (n_tasks + NWARP - 1) / NWARP;
  const int grid = static_cast<int>(want < sm_count() ? want : sm_count());
  kern<<<grid, NWARP * 32, kSmem, stream>>>(a, static_cast<int>(n_tasks));
  PLA_CUDA_OK(cudaGetLastError());
  return PLA_B200_OK;
}

template <typename act_t, bool IS_KDA>
int launch(const pla_b200_klast_args& a, cudaStream_t stream) {
  return launch_cfg<act_t, IS_KDA, 16, 3>(a, stream);
}

}  // namespace

bool klast_stream_eligible(const pla_b200_klast_args& a) {
  const auto al4 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3) == 0; };
  return a.t_max == 1 && a.slot_row_stride == 0 && a.cache == nullptr && a.parents == nullptr &&
         !a.disable_state_update && a.state_dtype == PLA_B200_F32 && al4(a.v) && a.v_tok_stride % 2 == 0 &&
         al4(a.o) && a.slot_indices != nullptr && a.state_out == nullptr && !a.state_init_zero &&
         !a.state_transposed && !a.gate_activated && a.o_total_rows == 0 &&
         (reinterpret_cast<uintptr_t>(a.q) & 7) == 0 && (reinterpret_cast<uintptr_t>(a.k) & 7) == 0 &&
         a.q_tok_stride % 4 == 0 && a.k_tok_stride % 4 == 0 &&
         (!a.is_kda || ((reinterpret_cast<uintptr_t>(a.a) & 7) == 0 && a.a_tok_stride % 4 == 0));
}

int launch_klast_stream(const pla_b200_klast_args& a, cudaStream_t stream) {
  if (a.act_dtype == PLA_B200_BF16)
    return a.is_kda ? launch<__nv_bfloat16, true>(a, stream) : launch<__nv_bfloat16, false>(a, stream);
  return a.is_kda ? launch<__half, true>(a, stream) : launch<__half, false>(a, stream);
}

}  // namespace pla
