// tcgen05 (5th-generation tensor core) building blocks for the widened configuration: shared-memory
// matrix descriptors for the un-swizzled ("interleaved") canonical layouts, the tf32 instruction
// descriptor, TMEM allocation and loads, and the commit -> mbarrier hand-over.  One CTA per MMA
// (cta_group::1), operands in shared memory, fp32 accumulators in tensor memory.
#pragma once

#include "net.cuh"

namespace cnn {
namespace tc {

// Canonical un-swizzled layout, in bytes, of a tile whose rows are grouped by 8 and whose 16-byte
// chunks (4 tf32 values) along the contiguous direction are grouped into "core matrices" of
// 8 rows x 16 B = 128 B:
//     offset(row, chunk) = (row / 8) * kGroupStride(chunks) + chunk * 128 + (row % 8) * 16
// Read as a K-major operand (rows = M or N, chunks along K): LBO = 128 (next chunk along K),
// SBO = group stride.  Read as an MN-major operand (rows = K, chunks along M or N): SBO = 128 (next
// chunk along MN), LBO = group stride (next 8 values of K).
__host__ __device__ constexpr unsigned tile_group_stride(int chunks) { return (unsigned)chunks * 128u; }
__host__ __device__ constexpr unsigned tile_offset(int row, int chunk, int chunks) {
  return (unsigned)(row >> 3) * tile_group_stride(chunks) + (unsigned)chunk * 128u + (unsigned)(row & 7) * 16u;
}

// 64-bit shared-memory matrix descriptor: start address, leading / stride byte offsets (all in units
// of 16 B), descriptor version 1, no swizzle.
__device__ __forceinline__ unsigned long long smem_desc(unsigned smem_addr, unsigned lbo_bytes, unsigned sbo_bytes) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);
  d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (unsigned long long)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  return d;
}

// Instruction descriptor for kind::tf32 with fp32 accumulation: D format f32 (bits 4-5 = 1), A and B
// formats tf32 (bits 7-9 and 10-12 = 2), majors (bit 15 / 16: 0 = K-major, 1 = MN-major), N >> 3 at
// bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr unsigned idesc_tf32(int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)a_mn_major << 15) | ((unsigned)b_mn_major << 16) |
         ((unsigned)(N >> 3) << 17) | ((unsigned)(M >> 4) << 24);
}

__device__ __forceinline__ void tmem_alloc(unsigned* smem_dst, unsigned cols) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned cols) {     // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Generic-proxy shared-memory writes -> visible to the async proxy (the tensor core's operand reads).
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; one thread issues.
__device__ __forceinline__ void mma_tf32(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc,
                                         unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same, called by a WHOLE converged warp: the operands are warp-uniform and one elected lane
// issues.  Measured on B200: a tcgen05.mma issued from inside a divergent branch ("if (tid == 0)")
// costs the issuing thread about 146 cycles whatever its shape; issued this way a 128 x 80 x 8 tf32
// MMA costs 58 cycles, which is its operand traffic (6.5 KB of shared memory at 128 B/cycle).
__device__ __forceinline__ void mma_tf32_elect(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc,
                                               unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Whole converged warp: the lane that elect.sync picks (the same one every time for a full mask)
// arrives on the mbarrier when every MMA it has issued so far has completed.
__device__ __forceinline__ void mma_commit_elect(unsigned long long* bar) {
  asm volatile(
      "{\n\t.reg .pred q;\n\telect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(smem_u32(bar))
      : "memory");
}
// Arrive on an mbarrier when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// 16 consecutive fp32 columns of this warp's 32 TMEM lanes: thread l gets lane (32 * (warp % 4) + l).
__device__ __forceinline__ void tmem_ld16(unsigned taddr, float (&v)[16]) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  // the registers are only valid after the wait; listing them as in/out operands keeps the compiler
  // from scheduling their uses above it
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Split an fp32 value into a tf32-exact high part and the remainder (for the three-pass product
// hi*hi + lo*hi + hi*lo, which restores fp32-level accuracy on tf32 tensor cores).
__device__ __forceinline__ void split_tf32(float v, float& hi, float& lo) {
  hi = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
  lo = v - hi;
}

}  // namespace tc
}  // namespace cnn
