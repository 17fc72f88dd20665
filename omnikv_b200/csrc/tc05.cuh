// tcgen05 (5th-generation tensor core) wrappers shared by the kernels that keep their accumulators in tensor memory:
// allocation, MMA issue by one thread, completion through an mbarrier, reads of a TMEM lane, and the shared-memory
// matrix descriptors of operands stored with the 128-byte swizzle.  cta_group::1 only (one SM per tile).
#pragma once
#include <type_traits>

#include "common.cuh"

namespace omnikv {

// ---- tcgen05 wrappers (cta_group::1) ---------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(unsigned* smem_dst, unsigned ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// D[tmem] (+)= A[smem desc] * B[smem desc]; both operands K-major, fp32 accumulate
__device__ __forceinline__ void tc_mma(unsigned d_tmem, uint64_t a_desc, uint64_t b_desc, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// the mbarrier gets one arrival when every MMA issued so far by this thread has completed
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// 16 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld16(unsigned taddr, float (&v)[16]) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// D[tmem] (+)= A[tmem] * B[smem desc]: the A operand lies in tensor memory (row = TMEM lane, two 16-bit elements of
// the contraction per 32-bit column, the lower index in the low half)
__device__ __forceinline__ void tc_mma_ts(unsigned d_tmem, unsigned a_tmem, uint64_t b_desc, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 16 consecutive 32-bit columns of this thread's TMEM lane <- registers
__device__ __forceinline__ void tmem_st16(unsigned taddr, const unsigned (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major operand stored as rows of 128 bytes with the 128-byte swizzle
// (what a TMA box of 64 16-bit elements x rows leaves, and what the query block is written as): 8-row groups
// are 1024 bytes apart (stride byte offset), version 1 (Blackwell), layout type 2 = SWIZZLE_128B.  `addr` is
// the byte address of the first element of this K step inside its 1024-byte-aligned box.
__device__ __forceinline__ uint64_t smem_desc_sw128(unsigned addr) {
  uint64_t d = (uint64_t)((addr & 0x3ffffu) >> 4);
  d |= (uint64_t)1 << 16;            // leading byte offset (unused with a swizzled K-major operand)
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset
  d |= (uint64_t)1 << 46;            // descriptor version
  d |= (uint64_t)2 << 61;            // SWIZZLE_128B
  return d;
}
// Shared-memory matrix descriptor of an MN-major operand with the 128-byte swizzle: what TMA boxes of
// [64 elements along M/N (128 bytes) x rows along K] leave.  The 8 rows (K) of a swizzle pattern are 128 bytes
// apart, groups of 8 rows `sbo_bytes` apart (1024 for a dense box), the next 64 elements along M/N start
// `lbo_bytes` further on (the size of a box).  `addr` = first row of this K step, on a 1024-byte boundary.
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(unsigned addr, unsigned lbo_bytes, unsigned sbo_bytes) {
  uint64_t d = (uint64_t)((addr & 0x3ffffu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor (kind::f16): fp32 accumulator, A and B of the same 16-bit format, M x N tile; a_mn / b_mn
// say that the operand is stored MN-major (rows of shared memory run along K) instead of K-major.
template <typename T>
__device__ __forceinline__ unsigned tc_instr_desc(int M, int N, bool a_mn, bool b_mn) {
  constexpr unsigned fmt = std::is_same<T, __half>::value ? 0u : 1u;  // F16 = 0, BF16 = 1
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((unsigned)(N >> 3) << 17) | ((unsigned)(M >> 4) << 24);
}

// 2^x on the special-function unit (x <= 16 here, -inf gives 0; relative error about 2^-22)
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}


}  // namespace omnikv
