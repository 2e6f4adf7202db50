// Persistent streaming kernel for single-token k-last decode (the production
// decode step): every (request, value head) 128x128 state is read once and
// written once, in place. The pool holds fp32 or bf16; the arithmetic is fp32.
//
// At most one CTA per SM and every WARP is its own pipeline. The state of the
// whole call is a sequence of UNITS of 8 consecutive V rows (4 KiB fp32, 2 KiB
// bf16; 16 units per (slot, hv) tile), cut into PIECES of 8, 4, 2 or 1 units;
// warp w of W owns the contiguous piece range [w N / W, (w + 1) N / W). The
// host picks the piece size and the grid so that ranges start and end on half
// tiles whenever the call is large enough (a warp pays one set-up of the
// token's q / k / gate per half tile it touches, and measured on B200 that
// alignment is worth more than the last SMs: 128 CTAs with eight whole half
// tiles per warp beat 148 CTAs with ragged ranges by 6 %), and smaller pieces
// only spread a small batch over more warps. A warp walks its range TASK by task
// (a task = the units of its range inside one half tile of 64 rows): lane 0
// keeps NS-1 bulk loads (TMA engine, mbarrier completion) in flight into the
// warp's private shared-memory ring, the warp updates the landed unit in place
// with 128-bit shared-memory accesses (8 lanes per row, 3-step shuffle
// reductions) and lane 0 writes it back with a bulk store. There is no CTA-wide
// barrier, so nothing waits for the slowest warp. The token's normalised q/k,
// gate and beta are formed once per task; the raw inputs of the NEXT task are
// prefetched into registers while the current one is streamed.
//
// Math: src/decode/k-last/fused_sigmoid_gating_k_last_kernel.cuh:396-473, :561-605;
// bf16 pools as k_last_load_state4 / k_last_store_state4 (:81-112): widened on load,
// rounded to nearest on store, outputs formed from the unrounded fp32 state.
#include <atomic>

#include "common.cuh"
#include "decode_klast.h"

namespace pla {
namespace {

constexpr int D = 128;
constexpr int TILE = D * D;
constexpr int RU = 8;                       // state rows per unit
constexpr int UPT = 8;                      // units per task (half a tile)
constexpr int TASK_ROWS = RU * UPT;         // 64
constexpr int TASKS_PER_TILE = D / TASK_ROWS;
constexpr int UNITS_PER_TILE = D / RU;      // 16

// A lane owns 16 columns of every row it works on, as 16-byte pieces of the stored row:
// piece i of lane j (j = lane % 8) holds columns (i * 8 + j) * CPL .. + CPL - 1.
template <typename state_t>
struct Layout {
  static constexpr int CPL = 16 / static_cast<int>(sizeof(state_t));  // columns per 16-byte piece: 4 or 8
  static constexpr int NI = 16 / CPL;                                 // pieces per lane and row: 4 or 2
  static constexpr uint32_t UNIT_BYTES = RU * D * sizeof(state_t);
  // first column of the e-th group of four columns (e = 0..3) of lane j
  __device__ static __forceinline__ int col4(int e, int j) {
    if constexpr (CPL == 4) return (e * 8 + j) * 4;
    else return ((e >> 1) * 8 + j) * 8 + (e & 1) * 4;
  }
};

enum : int { kSkip = 0, kActive = 1, kZero = 2 };

struct Task {
  int kind;     // kSkip: nothing; kActive: stream the units; kZero: padded request, zero its output rows
  int hv;
  int row0;     // first V row of the half tile
  int sb, se;   // units [sb, se) of the half tile belong to this warp
  int tok;      // token row of the request
  char* gptr;   // first unit of the half tile in the pool (kActive only)
};

template <typename act_t, bool IS_KDA>
struct Raw {    // 16-bit inputs of one task, in the lane layout the compute uses
  uint2 q[4], k[4];
  uint32_t v[UPT];             // rows 2r, 2r+1 of every unit
  uint2 a4[IS_KDA ? 4 : 1];
  act_t a, b;
};

// Half tile `task` clipped to the warp's unit range [g0, g1).
template <typename state_t>
__device__ __forceinline__ Task describe(const pla_b200_klast_args& p, int task, int g0, int g1) {
  Task x;
  x.kind = kSkip;
  x.hv = 0;
  x.row0 = 0;
  x.sb = x.se = 0;
  x.tok = 0;
  x.gptr = nullptr;
  const int u0 = task * UPT;
  if (u0 >= g1) return x;
  x.sb = g0 > u0 ? g0 - u0 : 0;
  x.se = g1 - u0 < UPT ? g1 - u0 : UPT;
  const int part = task % TASKS_PER_TILE;
  const int t = task / TASKS_PER_TILE;
  x.hv = t % p.HV;
  x.row0 = part * TASK_ROWS;
  const int n = t / p.HV;
  int bos = n, eos = n + 1;
  const int slot = p.slot_indices[n];   // issued together with the offsets: one memory round trip, not two
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
  x.gptr = static_cast<char*>(p.state) +
           (static_cast<int64_t>(slot) * p.state_slot_stride + static_cast<int64_t>(x.hv) * TILE + x.row0 * D) *
               static_cast<int64_t>(sizeof(state_t));
  return x;
}

// Address of the unit `pos` places after the first unit of `cur` in the warp's stream of active units
// (continuing into `nxt`), or NULL when the stream has no such unit yet.
template <typename state_t>
__device__ __forceinline__ const char* unit_at(const Task& cur, const Task& nxt, int pos) {
  const int u = cur.sb + pos;
  if (u < cur.se) return cur.gptr + static_cast<int64_t>(u) * Layout<state_t>::UNIT_BYTES;
  const int w = nxt.sb + (u - cur.se);
  if (nxt.kind == kActive && w < nxt.se) return nxt.gptr + static_cast<int64_t>(w) * Layout<state_t>::UNIT_BYTES;
  return nullptr;
}

template <typename act_t, bool IS_KDA, typename state_t>
__device__ __forceinline__ void prefetch(const pla_b200_klast_args& p, const Task& x, int r, int j,
                                         Raw<act_t, IS_KDA>& raw) {
  using L = Layout<state_t>;
  if (x.kind != kActive) return;
  const int h = x.hv / (p.HV / p.H);
  const int64_t tok = x.tok;
  const act_t* gq = static_cast<const act_t*>(p.q) + tok * p.q_tok_stride + h * D;
  const act_t* gk = static_cast<const act_t*>(p.k) + tok * p.k_tok_stride + h * D;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    raw.q[e] = *reinterpret_cast<const uint2*>(gq + L::col4(e, j));
    raw.k[e] = *reinterpret_cast<const uint2*>(gk + L::col4(e, j));
  }
  const act_t* gv = static_cast<const act_t*>(p.v) + tok * p.v_tok_stride + x.hv * D + x.row0 + r * 2;
#pragma unroll
  for (int s = 0; s < UPT; ++s) raw.v[s] = *reinterpret_cast<const uint32_t*>(gv + s * RU);
  if constexpr (IS_KDA) {
    const act_t* ga = static_cast<const act_t*>(p.a) + tok * p.a_tok_stride + x.hv * D;
#pragma unroll
    for (int e = 0; e < 4; ++e) raw.a4[e] = *reinterpret_cast<const uint2*>(ga + L::col4(e, j));
  } else {
    raw.a = static_cast<const act_t*>(p.a)[tok * p.a_tok_stride + x.hv];
  }
  raw.b = static_cast<const act_t*>(p.b)[tok * p.b_tok_stride + x.hv];
}

template <typename act_t>
__device__ __forceinline__ void cvt4(const uint2& raw, float* out) {
  const act_t* e = reinterpret_cast<const act_t*>(&raw);
  out[0] = to_f32(e[0]);
  out[1] = to_f32(e[1]);
  out[2] = to_f32(e[2]);
  out[3] = to_f32(e[3]);
}

// One 16-byte piece of a stored row <-> CPL fp32 values.
template <typename state_t>
__device__ __forceinline__ void widen(const uint4& raw, float* out) {
  if constexpr (sizeof(state_t) == 4) {
    out[0] = __uint_as_float(raw.x);
    out[1] = __uint_as_float(raw.y);
    out[2] = __uint_as_float(raw.z);
    out[3] = __uint_as_float(raw.w);
  } else {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {   // a bf16 is the upper half of the fp32 with the same value
      out[2 * i] = __uint_as_float(w[i] << 16);
      out[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
}
template <typename state_t>
__device__ __forceinline__ uint4 narrow(const float* in) {
  if constexpr (sizeof(state_t) == 4) {
    return make_uint4(__float_as_uint(in[0]), __float_as_uint(in[1]), __float_as_uint(in[2]), __float_as_uint(in[3]));
  } else {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 pr = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&pr);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
}

__device__ __forceinline__ float group8_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  return x;
}

template <typename act_t, bool IS_KDA, typename state_t, int NWARP, int NS>
__global__ void __launch_bounds__(NWARP * 32, 1) klast_stream_kernel(const pla_b200_klast_args p,
                                                                     const int n_pieces, const int piece) {
  using L = Layout<state_t>;
  constexpr uint32_t UNIT_BYTES = L::UNIT_BYTES;
  constexpr int CPL = L::CPL, NI = L::NI;
  extern __shared__ __align__(128) unsigned char smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 3;  // row pair: rows 2r, 2r+1 of a unit
  const int j = lane & 7;   // position inside a row, see Layout
  unsigned char* ring = smem + static_cast<size_t>(warp) * (NS * UNIT_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(NWARP) * NS * UNIT_BYTES) + warp * NS;

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < NS; ++s) mbar_init(&bars[s], 1);
    fence_mbar_init();
  }
  __syncwarp();

  const int64_t gw = static_cast<int64_t>(blockIdx.x) * NWARP + warp;
  const int64_t GW = static_cast<int64_t>(gridDim.x) * NWARP;
  const int g0 = static_cast<int>(n_pieces * gw / GW) * piece, g1 = static_cast<int>(n_pieces * (gw + 1) / GW) * piece;
  if (g0 >= g1) return;
  const int t_first = g0 / UPT, t_end = (g1 + UPT - 1) / UPT;

  Task cur = describe<state_t>(p, t_first, g0, g1);
  // The first loads only need the next task when the first one is too short to fill the ring; otherwise the
  // next task's metadata (dependent global loads) is fetched behind them.
  const bool short_first = cur.kind != kActive || cur.se - cur.sb < NS - 1;
  Task nxt;
  nxt.kind = kSkip;
  nxt.sb = nxt.se = 0;
  nxt.gptr = nullptr;
  if (short_first) nxt = describe<state_t>(p, t_first + 1, g0, g1);
  Raw<act_t, IS_KDA> raw;
  prefetch<act_t, IS_KDA, state_t>(p, cur, r, j, raw);
  if (lane == 0 && cur.kind == kActive) {
#pragma unroll
    for (int d = 0; d < NS - 1; ++d) {
      const char* src = unit_at<state_t>(cur, nxt, d);
      if (src != nullptr) {
        mbar_expect_tx(&bars[d], UNIT_BYTES);
        bulk_load(ring + d * UNIT_BYTES, src, UNIT_BYTES, &bars[d]);
      }
    }
  }

  if (!short_first) nxt = describe<state_t>(p, t_first + 1, g0, g1);

  // Ring position of the unit being computed and of the next load; both only
  // advance on active units so that they stay in step across padded tasks.
  int stage = 0;
  uint32_t parity = 0;  // bit s = phase of ring slot s
  bool failed = false;

  for (int task = t_first; task < t_end && !failed; ++task) {
    if (task > t_first) nxt = describe<state_t>(p, task + 1, g0, g1);  // inputs consumed part of a task later

    if (cur.kind == kActive) {
      // ---- fp32 parameters of this task's token ----
      float kk[16], qq[16], gg[IS_KDA ? 16 : 1];
      float gs = 1.0f;
      {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          cvt4<act_t>(raw.q[e], qq + 4 * e);
          cvt4<act_t>(raw.k[e], kk + 4 * e);
        }
        float qp[4] = {0.f, 0.f, 0.f, 0.f}, kp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          qp[c >> 2] = fmaf(qq[c], qq[c], qp[c >> 2]);
          kp[c >> 2] = fmaf(kk[c], kk[c], kp[c >> 2]);
        }
        const float qs = (qp[0] + qp[1]) + (qp[2] + qp[3]), ks = (kp[0] + kp[1]) + (kp[2] + kp[3]);
        float qr = p.scale, kr = 1.0f;
        if (p.use_qk_l2norm) {
          qr = rsqrtf(group8_sum(qs) + 1e-6f) * p.scale;
          kr = rsqrtf(group8_sum(ks) + 1e-6f);
        }
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          qq[c] *= qr;
          kk[c] *= kr;
        }
      }
      const float A_log = load_any(p.A_log, p.A_log_dtype, cur.hv);
      if constexpr (IS_KDA) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float av[4];
          cvt4<act_t>(raw.a4[e], av);
          const int64_t c0 = static_cast<int64_t>(cur.hv) * D + L::col4(e, j);
#pragma unroll
          for (int c = 0; c < 4; ++c)
            gg[4 * e + c] = fast_exp(log_decay(av[c] + load_any(p.dt_bias, p.dt_bias_dtype, c0 + c), A_log, p.gate,
                                             p.softplus_beta, p.softplus_threshold, p.lower_bound));
        }
      } else {
        const float x = to_f32(raw.a) + load_any(p.dt_bias, p.dt_bias_dtype, cur.hv);
        gs = fast_exp(log_decay(x, A_log, p.gate, p.softplus_beta, p.softplus_threshold, p.lower_bound));
      }
      const float beta = sigmoidf_fast(to_f32(raw.b));
      uint32_t vcur[UPT];  // this task's v rows, still 16-bit (raw is refilled part way through)
#pragma unroll
      for (int s = 0; s < UPT; ++s) vcur[s] = raw.v[s];
      act_t* orow = static_cast<act_t*>(p.o) + (static_cast<int64_t>(cur.tok) * p.HV + cur.hv) * D + cur.row0 + r * 2;
      // The next task's inputs are requested half way through a whole task (`raw` of this task is fully
      // consumed by then), or right away when this warp's part of the task does not reach that unit.
      const bool pf_mid = cur.sb <= UPT / 2 && UPT / 2 < cur.se;
      if (!pf_mid) prefetch<act_t, IS_KDA, state_t>(p, nxt, r, j, raw);

#pragma unroll
      for (int sub = 0; sub < UPT; ++sub) {
        if (sub < cur.sb || sub >= cur.se) continue;             // warp-uniform: another warp's units
        if (sub == UPT / 2) prefetch<act_t, IS_KDA, state_t>(p, nxt, r, j, raw);   // pf_mid holds here
        unsigned char* blk = ring + stage * UNIT_BYTES;
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
          uint4* srow = reinterpret_cast<uint4*>(blk + (r * 2 + pp) * (D * sizeof(state_t)));
          float st[16];
          float dp[4] = {0.f, 0.f, 0.f, 0.f};   // four short dependency chains instead of one of sixteen
#pragma unroll
          for (int i = 0; i < NI; ++i) {
            widen<state_t>(srow[i * 8 + j], st + i * CPL);
#pragma unroll
            for (int c = 0; c < CPL; ++c) {
              const int e = i * CPL + c;
              if constexpr (IS_KDA) st[e] *= gg[e];
              dp[e >> 2] = fmaf(st[e], kk[e], dp[e >> 2]);
            }
          }
          float d = group8_sum((dp[0] + dp[1]) + (dp[2] + dp[3]));
          if constexpr (!IS_KDA) d *= gs;  // scalar decay folded: (g S) k = g (S k)
          const float vn = (to_f32(vpair[pp]) - d) * beta;
          float op[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int i = 0; i < NI; ++i) {
#pragma unroll
            for (int c = 0; c < CPL; ++c) {
              const int e = i * CPL + c;
              float s_ = st[e];
              if constexpr (!IS_KDA) s_ *= gs;
              s_ = fmaf(kk[e], vn, s_);
              op[e >> 2] = fmaf(s_, qq[e], op[e >> 2]);
              st[e] = s_;
            }
            srow[i * 8 + j] = narrow<state_t>(st + i * CPL);
          }
          ov[pp] = group8_sum((op[0] + op[1]) + (op[2] + op[3]));
        }
        if (j == 0) {
          if (p.o_f32 != nullptr) {
            *reinterpret_cast<float2*>(p.o_f32 + (static_cast<int64_t>(cur.tok) * p.HV + cur.hv) * D + cur.row0 + r * 2 + sub * RU) =
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
          const char* src = unit_at<state_t>(cur, nxt, sub - cur.sb + NS - 1);
          if (src != nullptr) {
            mbar_expect_tx(&bars[refill], UNIT_BYTES);
            bulk_load(ring + refill * UNIT_BYTES, src, UNIT_BYTES, &bars[refill]);
          }
          bulk_store(cur.gptr + static_cast<int64_t>(sub) * UNIT_BYTES, blk, UNIT_BYTES);
          bulk_commit();
        }
        stage = (stage + 1) % NS;
      }
      // A padded / empty next task got no look-ahead loads; the ring restarts at
      // the task after it (see below).
    } else {
      if (cur.kind == kZero) {
        // this warp's rows of the half tile: RU rows of 16 bits = 4 words per unit
        act_t* orow = static_cast<act_t*>(p.o) + (static_cast<int64_t>(cur.tok) * p.HV + cur.hv) * D + cur.row0;
        if (lane >= cur.sb * (RU / 2) && lane < cur.se * (RU / 2)) reinterpret_cast<uint32_t*>(orow)[lane] = 0u;
      }
      prefetch<act_t, IS_KDA, state_t>(p, nxt, r, j, raw);
      // Nothing was in flight for `cur`; start the ring for the next task. A task in the middle of
      // the range is whole, so NS-1 <= UPT units never reach past it; the last one may be shorter.
      if (lane == 0 && nxt.kind == kActive) {
        bulk_wait_read<0>();
        Task none;
        none.kind = kSkip;
        none.sb = none.se = 0;
        none.gptr = nullptr;
#pragma unroll
        for (int d = 0; d < NS - 1; ++d) {
          const int s = (stage + d) % NS;
          const char* src = unit_at<state_t>(nxt, none, d);
          if (src != nullptr) {
            mbar_expect_tx(&bars[s], UNIT_BYTES);
            bulk_load(ring + s * UNIT_BYTES, src, UNIT_BYTES, &bars[s]);
          }
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

// Piece size (units) and grid for a call of `n_units` units. Largest piece (8 = a half tile, then 4, 2, 1) that
// still gives two thirds of the SMs a piece per warp; then the grid in [2/3 of the SMs, all SMs] with the least
// idle warp-time, ceil(pieces / warps) * warps / pieces, ties going to the larger grid.
void plan_stream_grid(int64_t n_units, int nwarp, int sms, int* piece_out, int* grid_out) {
  const int lo = (2 * sms + 2) / 3;
  int piece = UPT;
  while (piece > 1 && n_units / piece < static_cast<int64_t>(lo) * nwarp) piece >>= 1;
  const int64_t n_pieces = n_units / piece;       // n_units is a multiple of 16
  int grid = static_cast<int>((n_pieces + nwarp - 1) / nwarp);
  if (grid > lo) {
    double best = 1e30;
    for (int g = lo; g <= sms; ++g) {
      const int64_t warps = static_cast<int64_t>(g) * nwarp;
      const double waste = static_cast<double>((n_pieces + warps - 1) / warps * warps) / static_cast<double>(n_pieces);
      if (waste <= best + 1e-12) {
        best = waste;
        grid = g;
      }
    }
  }
  *piece_out = piece;
  *grid_out = grid < 1 ? 1 : grid;
}

template <typename act_t, bool IS_KDA, typename state_t, int NWARP, int NS>
int launch_cfg(const pla_b200_klast_args& a, cudaStream_t stream) {
  constexpr int kSmem = NWARP * NS * static_cast<int>(Layout<state_t>::UNIT_BYTES) + NWARP * NS * 8;
  auto kern = klast_stream_kernel<act_t, IS_KDA, state_t, NWARP, NS>;
  static DeviceOnce configured;   // per instantiation
  int dev = 0;
  PLA_CUDA_OK(cudaGetDevice(&dev));
  if (configured.needed(dev)) {
    PLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    configured.mark(dev);
  }
  const int64_t n_units = static_cast<int64_t>(a.B) * a.HV * UNITS_PER_TILE;
  PLA_REQUIRE(n_units < (1ll << 31), PLA_B200_E_TOO_LARGE, "B*HV too large for the streaming decode kernel");
  int piece = 0, grid = 0;
  plan_stream_grid(n_units, NWARP, sm_count(), &piece, &grid);
  kern<<<grid, NWARP * 32, kSmem, stream>>>(a, static_cast<int>(n_units / piece), piece);
  PLA_CUDA_OK(cudaGetLastError());
  return PLA_B200_OK;
}

template <typename act_t, bool IS_KDA>
int launch(const pla_b200_klast_args& a, cudaStream_t stream) {
  // bf16 units are half the bytes: a deeper ring keeps the same number of bytes in flight per warp
  if (a.state_dtype == PLA_B200_BF16) return launch_cfg<act_t, IS_KDA, __nv_bfloat16, 16, 5>(a, stream);
  // rows_per_cta = 17: twelve warps (170 registers each instead of 128) with a ring of four units
  if (a.rows_per_cta == 17) return launch_cfg<act_t, IS_KDA, float, 12, 4>(a, stream);
  return launch_cfg<act_t, IS_KDA, float, 16, 3>(a, stream);
}

}  // namespace

bool klast_stream_eligible(const pla_b200_klast_args& a) {
  const auto al4 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3) == 0; };
  const bool state_ok = a.state_dtype == PLA_B200_F32 || (a.state_dtype == PLA_B200_BF16 && a.state_slot_stride % 8 == 0);
  return a.t_max == 1 && a.slot_row_stride == 0 && a.cache == nullptr && a.parents == nullptr &&
         !a.disable_state_update && state_ok && al4(a.v) && a.v_tok_stride % 2 == 0 &&
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
