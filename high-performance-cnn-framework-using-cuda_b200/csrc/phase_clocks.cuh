// Optional phase timing of a persistent kernel, for tuning.  Compiled in only with
// -DCNN_PHASE_CLOCKS; otherwise every macro expands to nothing and the kernels carry no trace of it.
//
// Lane 0 of every warp of the CTA for which `owner` is true sums, over the loop iterations, the SM
// clock at each stamp relative to the clock at kernel start; the means per stamp and warp put all
// warps of that CTA on one time axis.  A kernel uses
//   CNN_PHASE_TABLE(name, warps)            at namespace scope: the device table [warps][16]
//   CNN_PHASE_BEGIN(owner, smem_clock_slot) once, after set-up (contains a block barrier)
//   CNN_PHASE(i)                            at stamp i < 16
//   CNN_PHASE_END(name)                     before the kernel returns
// and a host-side reader copies the table out with cudaMemcpyFromSymbol.
#pragma once

#ifdef CNN_PHASE_CLOCKS
#define CNN_PHASE_TABLE(name, warps) __device__ long long name[warps][16];
#define CNN_PHASE_BEGIN(owner, slot)                                                  \
  long long ph_[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};               \
  const bool ph_on_ = (owner) && (threadIdx.x & 31) == 0;                             \
  if (threadIdx.x == 0) (slot) = clock64();                                           \
  __syncthreads();                                                                    \
  const long long ph_base_ = (slot);
#define CNN_PHASE(i)                                                                  \
  do {                                                                                \
    if (ph_on_) {                                                                     \
      long long now_;                                                                 \
      asm volatile("mov.u64 %0, %%clock64;" : "=l"(now_)::"memory");                  \
      ph_[i] += now_ - ph_base_;                                                      \
    }                                                                                 \
  } while (0)
#define CNN_PHASE_END(name)                                                           \
  do {                                                                                \
    if (ph_on_)                                                                       \
      for (int i_ = 0; i_ < 16; ++i_) name[threadIdx.x >> 5][i_] = ph_[i_];           \
  } while (0)
#else
#define CNN_PHASE_TABLE(name, warps)
#define CNN_PHASE_BEGIN(owner, slot)
#define CNN_PHASE(i) do { } while (0)
#define CNN_PHASE_END(name) do { } while (0)
#endif
