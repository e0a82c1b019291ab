// Building blocks of the per-sample cluster kernels: addresses in another CTA's shared memory,
// one-way stores counted on the receiver's mbarrier, bounded waits on such an mbarrier, and the
// warp-wide reduce-scatter of up to 32 per-lane terms.
#pragma once

#include "net.cuh"

namespace cnn {

constexpr int kClCtas = kF;                                             // one CTA per feature map
constexpr unsigned kWsExchangeBytes = kClCtas * 17 * sizeof(float);     // 408 per receiver and sample

// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ unsigned cluster_addr(const void* local, unsigned rank) {
  unsigned remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  return remote;
}
// One-way store of a float into another CTA's shared memory; its four bytes are counted on that
// CTA's mbarrier when they have landed.
__device__ __forceinline__ void st_async_f32(unsigned remote_addr, float v, unsigned remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(remote_addr),
               "r"(__float_as_uint(v)), "r"(remote_bar)
               : "memory");
}
// The same for four consecutive floats (16-byte aligned): one transaction on the receiver's mbarrier
// instead of four.
__device__ __forceinline__ void st_async_f32x4(unsigned remote_addr, float a, float b, float c, float d,
                                               unsigned remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(
                   remote_addr),
               "r"(__float_as_uint(a)), "r"(__float_as_uint(b)), "r"(__float_as_uint(c)), "r"(__float_as_uint(d)),
               "r"(remote_bar)
               : "memory");
}
// Non-blocking test (test_wait, not try_wait): the exchange waits sit on the critical path of every
// sample and a suspended try_wait was seen to resume late.
__device__ __forceinline__ bool mbar_try_wait_cluster(unsigned long long* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded like mbar_wait_bounded: about two seconds of SM clocks, then the status word is set and
// this thread skips every later wait; the other threads of the launch see the word and stop waiting
// too, so the kernel always ends within seconds.
__device__ __forceinline__ void mbar_wait_cluster_bounded(unsigned long long* bar, unsigned parity, int* status,
                                                          bool& gave_up) {
  if (gave_up) return;
  if (mbar_try_wait_cluster(bar, parity)) return;
  const long long t0 = clock64();
  unsigned spins = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    // a wait that ran out anywhere ends every other wait of the launch soon after
    const bool other_gave_up = status && ((++spins & 1023u) == 0) && *reinterpret_cast<volatile int*>(status) != 0;
    if (other_gave_up || clock64() - t0 > 4000000000LL) {
      gave_up = true;
      if (status) atomicExch(status, 1);
      return;
    }
  }
}

// After the call lane l holds the sum over the warp's lanes of v[l] (unused entries zero-filled).
__device__ __forceinline__ float warp_reduce_scatter32(float (&v)[32], int lane) {
#pragma unroll
  for (int half = 16; half >= 1; half >>= 1) {
    const bool upper = (lane & half) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      const float send = upper ? v[i] : v[i + half];
      const float keep = upper ? v[i + half] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, half);
    }
  }
  return v[0];
}

}  // namespace cnn
