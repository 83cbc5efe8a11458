// tcgen05 (5th-generation tensor core) and tensor-memory helpers for sm_100a:
// shared-memory matrix descriptors, instruction descriptors, MMA issue, commit,
// TMEM allocation and TMEM -> register loads.
#pragma once

#include <stdint.h>

namespace ib200 {

#ifdef __CUDACC__

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of
// 128 bytes with the 128-byte swizzle (16-byte chunk index XOR row % 8), 8-row
// groups `sbo_bytes` apart.  The tile base must be 1024-byte aligned; advancing
// along K inside the 128-byte row is done by adding (bytes >> 4) to the low word.
__device__ __forceinline__ uint64_t umma_desc_k_major_sw128(uint32_t smem_addr, uint32_t sbo_bytes = 1024) {
  uint64_t desc = 0;
  desc |= uint64_t((smem_addr & 0x3FFFFu) >> 4);   // start address, bits [0,14)
  desc |= uint64_t(1) << 16;                       // leading byte offset (unused with swizzle), bits [16,30)
  desc |= uint64_t(sbo_bytes >> 4) << 32;          // stride byte offset, bits [32,46)
  desc |= uint64_t(1) << 46;                       // descriptor version of sm_100
  desc |= uint64_t(2) << 61;                       // layout type: SWIZZLE_128B
  return desc;
}

// Shared-memory matrix descriptor for an MN-major operand tile (the M or N index is
// contiguous) with the 128-byte swizzle: rows are k, each 128 bytes of contiguous MN
// elements; 8-row (k) groups are `sbo_bytes` apart, consecutive 128-byte MN spans are
// `lbo_bytes` apart.
__device__ __forceinline__ uint64_t umma_desc_mn_major_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                            uint32_t sbo_bytes = 1024) {
  uint64_t desc = 0;
  desc |= uint64_t((smem_addr & 0x3FFFFu) >> 4);
  desc |= uint64_t(lbo_bytes >> 4) << 16;
  desc |= uint64_t(sbo_bytes >> 4) << 32;
  desc |= uint64_t(1) << 46;
  desc |= uint64_t(2) << 61;
  return desc;
}

// Instruction descriptor (32 bit) of tcgen05.mma kind::f16 / kind::i8, dense, no negation.
//   c_format: 0 = f16, 1 = f32, 2 = s32;  ab_format: kind::f16 0 = f16, 1 = bf16; kind::i8 0 = u8, 1 = s8
//   a_mn_major / b_mn_major: 0 = K-major operand, 1 = MN-major operand
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t c_format, uint32_t a_format, uint32_t b_format,
                                                  uint32_t a_mn_major, uint32_t b_mn_major, uint32_t m, uint32_t n) {
  return (c_format << 4) | (a_format << 7) | (b_format << 10) | (a_mn_major << 15) | (b_mn_major << 16) |
         ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread on behalf of the CTA.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u, zero = 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc), "r"(zero)
      : "memory");
}

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u, zero = 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc), "r"(zero)
      : "memory");
}

// Arrives once on the mbarrier when every MMA issued so far by this thread has completed
// (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// TMEM allocation: executed by one whole warp; the base address is written to `smem_dst`.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t tmem_base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(columns) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane (base lane + i).
__device__ __forceinline__ void tmem_load_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

#endif  // __CUDACC__

}  // namespace ib200
