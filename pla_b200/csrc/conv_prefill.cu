// Caller-side step in front of the prefill ops: width-4 causal conv (+ SiLU) over packed varlen token rows with
// a per-request 3-tap history, the prefill counterpart of the conv inside the fused decode step
// (src/decode/k-last/fused_kda_decode_mega_kernel.cuh:36-79) and of the verify kernels' conv
// (src/decode/kda_replayssm/kda_mtp_verify.cu:356-402):  y_t = act(b + h0 w0 + h1 w1 + h2 w2 + x_t w3),
// (h0,h1,h2) <- (h1,h2,x_t); after a sequence its history holds its last three inputs (shifted in behind the
// old ones when it is shorter; written by a second small launch). The output row is the packed q|k|v row the prefill ops read in place.
//
// HBM-bound streaming: a thread owns 8 adjacent channels (one 16-byte vector per token row) and walks a tile
// of consecutive token rows with the window in registers (rows staged through shared memory by asynchronous copies), so a row is read once (plus a 3-row halo per tile)
// and written once: 2 * 2 bytes per (token, channel).
#include "common.cuh"

namespace pla {
namespace {

constexpr int CONV_THREADS = 128;
constexpr int VEC = 8;          // channels per thread
constexpr int BATCH = 4;        // token rows per asynchronous copy group
constexpr int GROUPS = 4;       // copy groups in flight per thread: 16 rows

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(smem_dst)), "l"(gmem_src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <typename act_t>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[VEC]);
template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& v, float (&f)[VEC]) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(u[i] << 16);
    f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void unpack8<__half>(const uint4& v, float (&f)[VEC]) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 p = __half22float2(h[i]);
    f[2 * i] = p.x, f[2 * i + 1] = p.y;
  }
}

__device__ __forceinline__ uint32_t pack2(float a, float b, __nv_bfloat16) {
  const __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t pack2(float a, float b, __half) {
  const __half2 r = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&r);
}

// SiLU as h + h tanh(h), h = x/2, with the hardware tanh: one special-function operation per element instead of
// the two of x / (1 + e^-x), which at HBM speed would take most of the special-function rate. Absolute error
// at most |x| 2^-12 (the approximation's relative error is 2^-11), below one bf16 / fp16 rounding of x.
__device__ __forceinline__ float silu_tanh(float x) {
  const float h = 0.5f * x;
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
  return fmaf(h, t, h);
}

// History of `slot` for 8 channels starting at c0, tap by tap (zero when there is none).
template <typename act_t>
__device__ __forceinline__ uint4 load_tap(const pla_b200_conv_prefill_args& p, int slot, int c0, int tap) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (slot < 0) return v;
  const act_t* base = static_cast<const act_t*>(p.conv_state) + static_cast<int64_t>(slot) * p.conv_strides.slot +
                      static_cast<int64_t>(tap) * p.conv_strides.tap + static_cast<int64_t>(c0) * p.conv_strides.channel;
  if (p.conv_strides.channel == 1 && (reinterpret_cast<uintptr_t>(base) & 15u) == 0) return *reinterpret_cast<const uint4*>(base);
  act_t* e = reinterpret_cast<act_t*>(&v);
#pragma unroll
  for (int i = 0; i < VEC; ++i) e[i] = base[static_cast<int64_t>(i) * p.conv_strides.channel];
  return v;
}

template <typename act_t>
__device__ __forceinline__ void store_tap(const pla_b200_conv_prefill_args& p, int slot, int c0, int tap, const uint4& v) {
  act_t* base = static_cast<act_t*>(p.conv_state) + static_cast<int64_t>(slot) * p.conv_strides.slot +
                static_cast<int64_t>(tap) * p.conv_strides.tap + static_cast<int64_t>(c0) * p.conv_strides.channel;
  if (p.conv_strides.channel == 1 && (reinterpret_cast<uintptr_t>(base) & 15u) == 0) {
    *reinterpret_cast<uint4*>(base) = v;
    return;
  }
  const act_t* e = reinterpret_cast<const act_t*>(&v);
#pragma unroll
  for (int i = 0; i < VEC; ++i) base[static_cast<int64_t>(i) * p.conv_strides.channel] = e[i];
}

// Slot whose history sequence `seq` reads (reads < 0: none) and writes (writes < 0: none).
__device__ __forceinline__ void slots_of(const pla_b200_conv_prefill_args& p, int seq, int& reads, int& writes) {
  int slot = p.state_indices != nullptr ? p.state_indices[seq] : seq;
  const bool pad = p.pad == PLA_B200_PAD_VLLM ? slot <= 0 : slot < 0;
  if (!pad && slot >= p.slots) {
    if (p.status != nullptr) atomicOr(p.status, PLA_B200_DEV_BAD_SLOT);
    slot = -1;
  }
  if (pad || p.conv_state == nullptr) slot = -1;
  writes = slot;
  reads = (p.has_initial_state == nullptr || p.has_initial_state[seq] != 0) ? slot : -1;
}

template <typename act_t, bool SILU>
__global__ void __launch_bounds__(CONV_THREADS, 5) conv_prefill_kernel(const pla_b200_conv_prefill_args p, const int tile) {
  __shared__ uint4 ring[GROUPS * BATCH][CONV_THREADS];
  const int c0 = (blockIdx.x * CONV_THREADS + threadIdx.x) * VEC;
  if (c0 >= p.channels) return;
  const int t0 = blockIdx.y * tile;
  const int t1 = min(t0 + tile, p.tokens);
  const int total = min(p.cu_seqlens[p.N], p.tokens);
  const act_t* x = static_cast<const act_t*>(p.x) + c0;
  act_t* y = static_cast<act_t*>(p.y) + c0;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

  float w[4][VEC], bias[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const float4 wi = *reinterpret_cast<const float4*>(p.weight + static_cast<int64_t>(c0 + i) * 4);
    w[0][i] = wi.x, w[1][i] = wi.y, w[2][i] = wi.z, w[3][i] = wi.w;
    bias[i] = p.bias != nullptr ? p.bias[c0 + i] : 0.0f;
  }

  // sequence holding row t0: the last one that starts at or before it (empty ones are stepped over below)
  int seq = 0, seq_beg = 0, seq_end = 0, reads = -1, writes = -1;
  float h0[VEC], h1[VEC], h2[VEC];          // the three previous inputs of the sequence, oldest first
#pragma unroll
  for (int i = 0; i < VEC; ++i) h0[i] = h1[i] = h2[i] = 0.0f;
  if (t0 < total) {
    int lo = 0, hi = p.N - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (p.cu_seqlens[mid] <= t0) lo = mid; else hi = mid - 1;
    }
    seq = lo;
    seq_beg = p.cu_seqlens[seq];
    seq_end = p.cu_seqlens[seq + 1];
    slots_of(p, seq, reads, writes);
    const int done = t0 - seq_beg;          // rows of this sequence before the tile; 0 = the start-of-sequence path below
    if (done > 0) {
      // window before row t0 = sequence positions done-3 .. done-1: rows of x, or history tap 3 + position when negative
      unpack8<act_t>(*reinterpret_cast<const uint4*>(x + static_cast<int64_t>(t0 - 1) * p.x_row_stride), h2);
      unpack8<act_t>(done >= 2 ? *reinterpret_cast<const uint4*>(x + static_cast<int64_t>(t0 - 2) * p.x_row_stride)
                               : load_tap<act_t>(p, reads, c0, 2), h1);
      unpack8<act_t>(done >= 3 ? *reinterpret_cast<const uint4*>(x + static_cast<int64_t>(t0 - 3) * p.x_row_stride)
                               : load_tap<act_t>(p, reads, c0, done == 2 ? 2 : 1), h0);
    }
  }

  // One conv step of this thread's 8 channels; shifts the window.
  auto step = [&](const uint4& xv) -> uint4 {
    float fx[VEC], r[VEC];
    unpack8<act_t>(xv, fx);
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      float acc = bias[c];
      acc = fmaf(w[0][c], h0[c], acc);
      acc = fmaf(w[1][c], h1[c], acc);
      acc = fmaf(w[2][c], h2[c], acc);
      acc = fmaf(w[3][c], fx[c], acc);
      r[c] = SILU ? silu_tanh(acc) : acc;
      h0[c] = h1[c], h1[c] = h2[c], h2[c] = fx[c];
    }
    return make_uint4(pack2(r[0], r[1], act_t()), pack2(r[2], r[3], act_t()), pack2(r[4], r[5], act_t()),
                      pack2(r[6], r[7], act_t()));
  };
  // Rows arrive through a thread-private ring in shared memory filled by asynchronous 16-byte copies, GROUPS
  // batches of BATCH rows in flight per thread: the depth does not cost registers. Rows outside the sequences
  // are filled with zeros (source size 0).
  const int tid = threadIdx.x;
  auto issue = [&](int batch) {
    const int tb = t0 + batch * BATCH;
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      const int t = tb + i;
      const bool live = t < t1 && t < total;
      cp_async16(&ring[(batch % GROUPS) * BATCH + i][tid], x + static_cast<int64_t>(live ? t : t0) * p.x_row_stride, live ? 16u : 0u);
    }
  };
  const int batches = (t1 - t0 + BATCH - 1) / BATCH;
#pragma unroll
  for (int b = 0; b < GROUPS; ++b) {
    if (b < batches) issue(b);
    cp_async_commit();
  }
  for (int b = 0; b < batches; ++b) {
    cp_async_wait<GROUPS - 1>();
    const int tb = t0 + b * BATCH;
    const uint4* rows = &ring[(b % GROUPS) * BATCH][tid];
    if (tb > seq_beg && tb + BATCH <= min(seq_end, min(total, t1))) {      // inside one sequence: no per-row checks
#pragma unroll
      for (int i = 0; i < BATCH; ++i)
        *reinterpret_cast<uint4*>(y + static_cast<int64_t>(tb + i) * p.y_row_stride) = step(rows[i * CONV_THREADS]);
    } else {
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const int t = tb + i;
        if (t >= t1) break;
        uint4 out = zero;
        if (t < total) {
          if (t >= seq_end) {
            while (t >= seq_end && seq + 1 < p.N) {   // next sequence (empty ones have seq_end == seq_beg)
              ++seq;
              seq_beg = seq_end;
              seq_end = p.cu_seqlens[seq + 1];
            }
            slots_of(p, seq, reads, writes);
          }
          if (t == seq_beg) {
            unpack8<act_t>(load_tap<act_t>(p, reads, c0, 0), h0);
            unpack8<act_t>(load_tap<act_t>(p, reads, c0, 1), h1);
            unpack8<act_t>(load_tap<act_t>(p, reads, c0, 2), h2);
          }
          out = step(rows[i * CONV_THREADS]);
        }
        *reinterpret_cast<uint4*>(y + static_cast<int64_t>(t) * p.y_row_stride) = out;
      }
    }
    if (b + GROUPS < batches) issue(b + GROUPS);   // refill the slot just consumed (this thread's own 16-byte cells)
    cp_async_commit();
  }
  cp_async_wait<0>();
}

// History after the call, one thread per (sequence, 8 channels): its last three inputs, the old taps shifted in
// behind them when it is shorter. A launch of its own behind the conv: tiles of the conv read the old history
// of sequences whose last row belongs to another tile, so nothing may be written while they run.
template <typename act_t>
__global__ void __launch_bounds__(CONV_THREADS) conv_history_kernel(const pla_b200_conv_prefill_args p) {
  const int c0 = (blockIdx.x * CONV_THREADS + threadIdx.x) * VEC;
  const int seq = blockIdx.y;
  if (c0 >= p.channels) return;
  const int beg = p.cu_seqlens[seq], end = min(p.cu_seqlens[seq + 1], p.tokens);
  const int len = end - beg;
  int reads, writes;
  slots_of(p, seq, reads, writes);
  if (len <= 0 || writes < 0) return;
  const act_t* x = static_cast<const act_t*>(p.x) + c0;
  uint4 taps[3];
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const int pos = len - 3 + j;             // sequence position that ends up in tap j
    taps[j] = pos >= 0 ? *reinterpret_cast<const uint4*>(x + static_cast<int64_t>(beg + pos) * p.x_row_stride)
                       : load_tap<act_t>(p, reads, c0, 3 + pos);
  }
#pragma unroll
  for (int j = 0; j < 3; ++j) store_tap<act_t>(p, writes, c0, j, taps[j]);
}

}  // namespace
}  // namespace pla

extern "C" int pla_b200_causal_conv_prefill(const pla_b200_conv_prefill_args* args, void* stream) {
  using namespace pla;
  PLA_REQUIRE(args != nullptr, PLA_B200_E_INVALID, "args is NULL");
  pla_b200_conv_prefill_args a = *args;
  default_status(a);
  PLA_REQUIRE(a.N >= 0 && a.tokens >= 0 && a.channels > 0 && a.channels % VEC == 0, PLA_B200_E_INVALID,
              "conv needs N >= 0, tokens >= 0 and a channel count that is a multiple of 8");
  PLA_REQUIRE(a.act_dtype == PLA_B200_BF16 || a.act_dtype == PLA_B200_F16, PLA_B200_E_INVALID,
              "conv activations must be bf16 or fp16");
  PLA_REQUIRE(a.pad == PLA_B200_PAD_SGLANG || a.pad == PLA_B200_PAD_VLLM, PLA_B200_E_INVALID, "bad pad convention");
  if (a.tokens == 0) return PLA_B200_OK;
  PLA_REQUIRE(a.x && a.y && a.weight && a.cu_seqlens, PLA_B200_E_INVALID, "x, y, weight and cu_seqlens are required");
  PLA_REQUIRE(a.x != a.y, PLA_B200_E_INVALID, "conv cannot run in place: a tile reads the three rows before it");
  PLA_REQUIRE(aligned16(a.x) && aligned16(a.y) && aligned16(a.weight) && a.x_row_stride % VEC == 0 &&
                  a.y_row_stride % VEC == 0 && a.x_row_stride >= a.channels && a.y_row_stride >= a.channels,
              PLA_B200_E_ALIGN, "x, y rows and weight must be 16-byte aligned with pitches that cover the channels");
  PLA_REQUIRE(a.conv_state == nullptr || a.slots > 0, PLA_B200_E_INVALID, "a conv history needs slots > 0");
  const unsigned gx = static_cast<unsigned>((a.channels / VEC + CONV_THREADS - 1) / CONV_THREADS);
  int tile = 64;                                      // rows per CTA: halo re-read 3/64; smaller for short inputs
  while (tile > 8 && static_cast<int64_t>(gx) * ((a.tokens + tile - 1) / tile) < 8 * 148) tile >>= 1;
  const dim3 grid(gx, static_cast<unsigned>((a.tokens + tile - 1) / tile));
  PLA_REQUIRE(grid.y <= 65535u, PLA_B200_E_TOO_LARGE, "more than 65535 token tiles");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a.act_dtype == PLA_B200_BF16) {
    if (a.activation) conv_prefill_kernel<__nv_bfloat16, true><<<grid, CONV_THREADS, 0, s>>>(a, tile);
    else conv_prefill_kernel<__nv_bfloat16, false><<<grid, CONV_THREADS, 0, s>>>(a, tile);
  } else {
    if (a.activation) conv_prefill_kernel<__half, true><<<grid, CONV_THREADS, 0, s>>>(a, tile);
    else conv_prefill_kernel<__half, false><<<grid, CONV_THREADS, 0, s>>>(a, tile);
  }
  PLA_CUDA_OK(cudaGetLastError());
  if (a.conv_state != nullptr && a.N > 0) {
    PLA_REQUIRE(a.N <= 65535, PLA_B200_E_TOO_LARGE, "more than 65535 sequences");
    const dim3 hgrid(gx, static_cast<unsigned>(a.N));
    if (a.act_dtype == PLA_B200_BF16)
      conv_history_kernel<__nv_bfloat16><<<hgrid, CONV_THREADS, 0, s>>>(a);
    else
      conv_history_kernel<__half><<<hgrid, CONV_THREADS, 0, s>>>(a);
    PLA_CUDA_OK(cudaGetLastError());
  }
  return PLA_B200_OK;
}
