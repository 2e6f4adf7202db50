// tcgen05 (5th-generation tensor core) helpers for sm_100a: tensor-memory allocation, shared-memory
// matrix descriptors, instruction descriptors, MMA issue / commit, TMEM loads and stores.
//
// Conventions used by the kernels in this directory:
//  * one CTA per cluster (cta_group::1), D accumulators [128 lanes (M) x N columns] fp32, row m of D
//    lives in TMEM lane m; warp w of a 4-warp group may only touch lanes [32*(w%4), 32*(w%4)+32).
//  * operands are K-major without swizzle. A shared-memory operand tile [R rows x K] of 32-bit
//    (tf32) elements is stored "chunk-major": 16-byte chunks of 4 consecutive K elements, all R rows
//    of a chunk contiguous:  byte(r, k) = (k/4) * (R*16) + r*16 + (k%4)*4.
//    8 rows x 16 bytes form one core matrix (128 contiguous bytes); the descriptor's leading byte
//    offset is the distance between K-adjacent core matrices (R*16), the stride byte offset the
//    distance between M/N-adjacent ones (128).
//  * an A operand may instead come from TMEM: row m in lane m, one 32-bit K element per column.
#pragma once

#include <stdint.h>

#include "common.cuh"

namespace pla {
namespace tc05 {

// ---- tensor memory -----------------------------------------------------------------------------
// Allocates `cols` (power of two, 32..512) TMEM columns; the base address is written to *smem_out.
// Must be executed by one full warp.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_out, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(smem_out)),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// TMEM address = lane in bits [31:16], column in bits [15:0], relative to the allocation base.
__device__ __forceinline__ uint32_t taddr(uint32_t base, uint32_t lane, uint32_t col) {
  return base + (lane << 16) + col;
}

// 32 consecutive columns of this thread's lane (lane = 32*(warp%4) + laneid) -> 32 registers.
__device__ __forceinline__ void tmem_ld32(uint32_t ta, float (&v)[32]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(ta)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t ta, const float (&v)[32]) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,"
      "%31,%32};" ::"r"(ta),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// ---- descriptors --------------------------------------------------------------------------------
// Shared-memory matrix descriptor, K-major, no swizzle. Byte offsets must be multiples of 16.
__device__ __forceinline__ uint64_t smem_desc(const void* smem_ptr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr(smem_ptr) & 0x3FFFFu) >> 4);   // start address, bits [0,14)
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;       // leading byte offset, bits [16,30)
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;       // stride byte offset, bits [32,46)
  d |= static_cast<uint64_t>(1) << 46;                                 // descriptor version for sm_100
  return d;                                                            // base offset 0, swizzle none (bits 61-63 = 0)
}
// Moves a descriptor's start address by `bytes` (multiple of 16, no carry out of the 14-bit field).
__device__ __forceinline__ uint64_t desc_advance(uint64_t d, uint32_t bytes) { return d + (bytes >> 4); }

// Instruction descriptor for kind::tf32, fp32 accumulate, A and B K-major, M x N tile.
__host__ __device__ constexpr uint32_t idesc_tf32(int M, int N) {
  return (1u << 4)      // D format: f32
         | (2u << 7)    // A format: tf32
         | (2u << 10)   // B format: tf32
         | (0u << 15)   // A major: K
         | (0u << 16)   // B major: K
         | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

// ---- MMA issue (one thread) ----------------------------------------------------------------------
// D[M x N] (+)= A[M x 8] * B[N x 8]^T, A and B from shared memory.
__device__ __forceinline__ void mma_tf32_ss(uint32_t d_taddr, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_taddr),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate))
      : "memory");
}
// Same with A read from tensor memory (row m in lane m, K element k in column a_taddr.col + k).
__device__ __forceinline__ void mma_tf32_ts(uint32_t d_taddr, uint32_t a_taddr, uint64_t b_desc, uint32_t idesc,
                                            bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_taddr),
      "r"(a_taddr), "l"(b_desc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate))
      : "memory");
}
// Arrive on `bar` once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
               : "memory");
}

// fp32 -> tf32 with round-to-nearest, ties away from zero (what cvt.rna.tf32.f32 computes; the tensor
// core itself only truncates). Done on the integer pipe: the conversion instruction shares the
// transcendental unit, which the operand builders already keep busy.
__device__ __forceinline__ float to_tf32(float x) {
  return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
}
// Half of that rounding, for a value that only the tensor core will read (a TMEM A operand): after adding half
// a tf32 unit to the bit pattern, the tensor core's own truncation of the low 13 bits completes the round to
// nearest. One integer add per element (cvt.rna.tf32.f32 was measured at 8 cycles per warp instruction, which
// made the chain kernel's epilogue conversion-bound).
__device__ __forceinline__ float pre_round_tf32(float x) { return __uint_as_float(__float_as_uint(x) + 0x1000u); }

}  // namespace tc05
}  // namespace pla
