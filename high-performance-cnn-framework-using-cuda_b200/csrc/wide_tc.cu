// Convolution of the widened configuration on the 5th-generation tensor cores (tcgen05).
//
// The conv is the implicit GEMM  D[m][f] = sum_t A[m][t] * W[f][t]  with m = (image, output
// position) flattened, t = filter tap (25, padded to K = 32) and f = feature map (N = F).  One CTA
// of 128 threads owns tiles of 128 consecutive rows m:
//   1. every thread gathers the 25 taps of its row straight from the image (L1/L2-resident) and
//      writes them, split into a tf32-exact high part and the remainder, into the two A tiles in
//      shared memory in the canonical un-swizzled K-major layout;
//   2. one elected lane of warp 0 issues 4 (one pass) or 12 (three passes: hi*hi + lo*hi + hi*lo, fp32-level
//      accuracy) tcgen05.mma of shape 128 x F x 8 with the accumulator in tensor memory, and commits
//      to an mbarrier;
//   3. after the (bounded) wait each warp reads its 32 accumulator lanes back with tcgen05.ld, adds
//      the bias, applies the sigmoid and stores the activations, coalesced over positions.
// Several CTAs per SM (48 KB of shared memory and F TMEM columns each) overlap one CTA's gather
// with another's MMA and epilogue, so there is no pipeline inside a CTA.
#include "wide.cuh"
#include "wide_tc.cuh"

namespace cnn {

constexpr int kTcRows = 128;   // M of one MMA = rows per tile = threads per CTA
constexpr int kTcChunks = 8;   // 16-byte chunks along K = 32 tf32 values

bool wide_conv_tc_supported(const WideDims& d) { return d.F % 16 == 0 && d.F >= 16 && d.F <= 256; }

template <int FLAVOR>
__global__ void __launch_bounds__(kTcRows)
k_wide_conv_fwd_tc(WideDims d, const float* __restrict__ images, long n, const float* __restrict__ params,
                   float* __restrict__ ac, int passes, unsigned tmem_cols, int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem[];
  // A hi | A lo (16 KB each) | B hi | B lo (F * 128 B each) | bias (F floats) | mbarrier | tmem address
  unsigned char* a_hi = smem;
  unsigned char* a_lo = a_hi + kTcRows * 128;
  unsigned char* b_hi = a_lo + kTcRows * 128;
  unsigned char* b_lo = b_hi + d.F * 128;
  float* bias = reinterpret_cast<float*>(b_lo + d.F * 128);
  unsigned long long* bar = reinterpret_cast<unsigned long long*>(bias + d.F);
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bar + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int CC = d.C * d.C;
  const long m_total = n * CC;
  const long n_tiles = (m_total + kTcRows - 1) / kTcRows;

  // weights: rows f, 8 chunks of 4 taps; taps >= 25 are zero
  for (int f = tid; f < d.F; f += kTcRows) {
#pragma unroll
    for (int c = 0; c < kTcChunks; ++c) {
      float4 hi, lo;
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = (4 * c + e < 25) ? params[d.o_wc + f * 25 + 4 * c + e] : 0.f;
      tc::split_tf32(v[0], hi.x, lo.x); tc::split_tf32(v[1], hi.y, lo.y);
      tc::split_tf32(v[2], hi.z, lo.z); tc::split_tf32(v[3], hi.w, lo.w);
      const unsigned off = tc::tile_offset(f, c, kTcChunks);
      *reinterpret_cast<float4*>(b_hi + off) = hi;
      *reinterpret_cast<float4*>(b_lo + off) = lo;
    }
    bias[f] = params[d.o_bc + f];
  }
  if (tid == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  if (warp == 0) tc::tmem_alloc(tmem_slot, tmem_cols);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const unsigned tmem_d = *tmem_slot;

  const unsigned idesc = tc::idesc_tf32(kTcRows, d.F, 0, 0);
  const unsigned group = tc::tile_group_stride(kTcChunks);   // 1,024 B between 8-row groups
  const unsigned a_hi_s = smem_u32(a_hi), a_lo_s = smem_u32(a_lo), b_hi_s = smem_u32(b_hi), b_lo_s = smem_u32(b_lo);

  bool gave_up = false;
  unsigned phase = 0;
  for (long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const long m = tile * kTcRows + tid;
    const bool live = m < m_total;
    long b = 0;
    int pos = 0;
    // ---- 1. gather this row's taps --------------------------------------------------------------
    {
      float v[32];
#pragma unroll
      for (int t = 0; t < 32; ++t) v[t] = 0.f;
      if (live) {
        b = m / CC;
        pos = (int)(m - b * CC);
        const int y = pos / d.C, x = pos - y * d.C;
        const float* src = images + (size_t)b * d.H * d.H + y * d.H + x;
#pragma unroll
        for (int i = 0; i < 5; ++i)
#pragma unroll
          for (int j = 0; j < 5; ++j) v[i * 5 + j] = __ldg(src + i * d.H + j);
      }
#pragma unroll
      for (int c = 0; c < kTcChunks; ++c) {
        float4 hi, lo;
        tc::split_tf32(v[4 * c], hi.x, lo.x); tc::split_tf32(v[4 * c + 1], hi.y, lo.y);
        tc::split_tf32(v[4 * c + 2], hi.z, lo.z); tc::split_tf32(v[4 * c + 3], hi.w, lo.w);
        const unsigned off = tc::tile_offset(tid, c, kTcChunks);
        *reinterpret_cast<float4*>(a_hi + off) = hi;
        *reinterpret_cast<float4*>(a_lo + off) = lo;
      }
    }
    tc::fence_async_smem();     // the tiles were written through the generic proxy
    tc::fence_before_sync();    // this thread's TMEM loads of the previous tile are complete
    __syncthreads();
    // ---- 2. MMAs ----------------------------------------------------------------------------------
    if (warp == 0) {   // the whole warp runs the loop, an elected lane issues (see wide_tc.cuh)
      tc::fence_after_sync();
      unsigned accumulate = 0;
      for (int pass = 0; pass < passes; ++pass) {
        const unsigned a_s = (pass == 1) ? a_lo_s : a_hi_s;
        const unsigned b_s = (pass == 2) ? b_lo_s : b_hi_s;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {    // K = 8 per MMA = two 16-byte chunks
          const unsigned long long ad = tc::smem_desc(a_s + ks * 256, 128, group);
          const unsigned long long bd = tc::smem_desc(b_s + ks * 256, 128, group);
          tc::mma_tf32_elect(tmem_d, ad, bd, idesc, accumulate);
          accumulate = 1;
        }
      }
      tc::mma_commit_elect(bar);
    }
    mbar_wait_bounded(bar, phase, status, gave_up);
    phase ^= 1u;
    tc::fence_after_sync();
    // ---- 3. epilogue: lane (32 * warp + l) of TMEM is row tid of the tile --------------------------
    const unsigned lane_base = tmem_d + ((unsigned)(warp * 32) << 16);
    for (int f0 = 0; f0 < d.F; f0 += 16) {
      float acc[16];
      tc::tmem_ld16(lane_base + (unsigned)f0, acc);
      if (live) {
        float* dst = ac + ((size_t)b * d.F + f0) * CC + pos;
#pragma unroll
        for (int e = 0; e < 16; ++e) dst[(size_t)e * CC] = sigmoidf<FLAVOR>(acc[e] + bias[f0 + e]);
      }
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_d, tmem_cols);
}

int wide_conv_fwd_tc(cnn_wide* w, const float* d_images, long n, cudaStream_t st) {
  const WideDims& d = w->d;
  unsigned cols = 32;
  while ((int)cols < d.F) cols <<= 1;
  const size_t smem = 2 * kTcRows * 128 + 2 * (size_t)d.F * 128 + sizeof(float) * d.F + 16;
  const long n_tiles = (n * (long)d.C * d.C + kTcRows - 1) / kTcRows;
  // CTAs per SM: limited by shared memory (227 KB) and by the 512 TMEM columns
  int per_sm = (int)(220 * 1024 / smem);
  if (per_sm > (int)(512 / cols)) per_sm = 512 / cols;
  if (per_sm > 8) per_sm = 8;
  if (per_sm < 1) per_sm = 1;
  long grid = (long)sm_count() * per_sm;
  if (grid > n_tiles) grid = n_tiles;
  const int passes = (w->conv_mode == 2) ? 3 : 1;
#define CNN_LAUNCH_TC(FL)                                                                              \
  do {                                                                                                 \
    CNN_CUDA(cudaFuncSetAttribute(k_wide_conv_fwd_tc<FL>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                  (int)smem));                                                         \
    k_wide_conv_fwd_tc<FL><<<(unsigned)grid, kTcRows, smem, st>>>(d, d_images, n, w->d_params, w->ac,  \
                                                                  passes, cols, w->d_status);          \
  } while (0)
  if (w->flavour == 1) CNN_LAUNCH_TC(1);
  else if (w->flavour == 2) CNN_LAUNCH_TC(2);
  else CNN_LAUNCH_TC(0);
#undef CNN_LAUNCH_TC
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "k_wide_conv_fwd_tc launch");
  return CNN_OK;
}


// ------------------------------------------------------------------------------------------------
// Conv weight gradient on the tensor cores:  G[f][t] = sum_m dc[m][f] * A[m][t]  with the same
// im2col rows A as the forward (m = image x position, t = tap) and dc the conv deltas (already
// divided by C*C).  As an MMA: D[M = F][N = 32] += dcT[F][K = 128 rows] * A[K = 128 rows][32]:
//   * the A operand is dc transposed, K-major (positions contiguous, as dc is stored per map);
//   * the B operand is the im2col tile transposed (rows = taps, positions contiguous), K-major as
//     well; tap 25, unused by the filter, is set to 1 so that column 25 of D is the conv-bias
//     gradient.  (Reading the forward's tile in place as an MN-major operand produced an all-zero
//     accumulator on the B200 and was dropped.);
//   * the accumulator stays in tensor memory over all the tiles of a CTA; at the end every CTA
//     writes one partial [F][26], and the partials are added in CTA order by k_wide_reduce.
// ------------------------------------------------------------------------------------------------
constexpr int kWgChunks = kTcRows / 4;   // 16-byte chunks along K = 128 positions

constexpr int kWgThreads = 256;   // threads 0..127 gather the im2col rows; all eight warps load deltas

__global__ void __launch_bounds__(kWgThreads)
k_wide_grad_c1_tc(WideDims d, const float* __restrict__ images, const float* __restrict__ dc, long n,
                  float* __restrict__ part, int passes, unsigned tmem_cols, int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem[];
  // dcT hi | dcT lo (F * 512 B each) | im2colT hi | im2colT lo (32 rows * 512 B each) | mbarrier | tmem address
  const unsigned a_bytes = (unsigned)d.F * kWgChunks * 16;
  unsigned char* a_hi = smem;
  unsigned char* a_lo = a_hi + a_bytes;
  unsigned char* b_hi = a_lo + a_bytes;
  unsigned char* b_lo = b_hi + kTcRows * 128;
  unsigned long long* bar = reinterpret_cast<unsigned long long*>(b_lo + kTcRows * 128);
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bar + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int CC = d.C * d.C;
  const long m_total = n * CC;
  const long n_tiles = (m_total + kTcRows - 1) / kTcRows;

  if (tid == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  if (warp == 0) tc::tmem_alloc(tmem_slot, tmem_cols);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const unsigned tmem_d = *tmem_slot;

  const unsigned idesc = tc::idesc_tf32(d.F, 32, 0, 0);   // both operands K-major
  const unsigned a_group = tc::tile_group_stride(kWgChunks);         // 4,096 B between 8-map groups
  const unsigned a_hi_s = smem_u32(a_hi), a_lo_s = smem_u32(a_lo), b_hi_s = smem_u32(b_hi), b_lo_s = smem_u32(b_lo);

  bool gave_up = false;
  unsigned phase = 0, accumulate = 0;
  constexpr int kWgFlush = 2;
  int since_flush = 0;
  float racc[32];
#pragma unroll
  for (int c = 0; c < 32; ++c) racc[c] = 0.f;
  const unsigned lane_base = tmem_d + ((unsigned)((warp & 3) * 32) << 16);
  for (long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const long m0 = tile * kTcRows;
    // ---- dcT tile: rows = maps, 32 chunks of 4 positions.  A warp-wide step covers 8 maps x 4
    // chunks: 64 contiguous bytes per map in global memory, 128 contiguous bytes per chunk in
    // shared memory (conflict-free).  All loads of a thread are issued before the first store.
    {
      constexpr int kSteps = 8;                      // per warp and round: 8 warps x 8 steps = 64 units
      const int units = (d.F / 8) * (kWgChunks / 4); // 64 for F = 64, 128 for F = 128
      for (int u0 = 0; u0 < units; u0 += (kWgThreads / 32) * kSteps) {
        float4 v[kSteps];
#pragma unroll
        for (int i = 0; i < kSteps; ++i) {
          const int u = u0 + i * (kWgThreads / 32) + warp;
          const int f = (u % (d.F / 8)) * 8 + (lane & 7);
          const int chunk = (u / (d.F / 8)) * 4 + (lane >> 3);
          const long m = m0 + 4 * chunk;   // CC and the tile size are multiples of 4: one image per chunk
          v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (u < units && m < m_total) {
            const long b = m / CC;
            const int pos = (int)(m - b * CC);
            v[i] = __ldg(reinterpret_cast<const float4*>(dc + ((size_t)b * d.F + f) * CC + pos));
          }
        }
#pragma unroll
        for (int i = 0; i < kSteps; ++i) {
          const int u = u0 + i * (kWgThreads / 32) + warp;
          if (u < units) {
            const int f = (u % (d.F / 8)) * 8 + (lane & 7);
            const int chunk = (u / (d.F / 8)) * 4 + (lane >> 3);
            float4 hi, lo;
            tc::split_tf32(v[i].x, hi.x, lo.x); tc::split_tf32(v[i].y, hi.y, lo.y);
            tc::split_tf32(v[i].z, hi.z, lo.z); tc::split_tf32(v[i].w, hi.w, lo.w);
            const unsigned off = tc::tile_offset(f, chunk, kWgChunks);
            *reinterpret_cast<float4*>(a_hi + off) = hi;
            *reinterpret_cast<float4*>(a_lo + off) = lo;
          }
        }
      }
    }
    // ---- im2col tile, transposed: thread r < 128 owns position m0 + r (one column of every tap row)
    if (tid < kTcRows) {
      const long m = m0 + tid;
      float v[32];
#pragma unroll
      for (int t = 0; t < 32; ++t) v[t] = 0.f;
      if (m < m_total) {
        const long b = m / CC;
        const int pos = (int)(m - b * CC);
        const int y = pos / d.C, x = pos - y * d.C;
        const float* src = images + (size_t)b * d.H * d.H + y * d.H + x;
#pragma unroll
        for (int i = 0; i < 5; ++i)
#pragma unroll
          for (int j = 0; j < 5; ++j) v[i * 5 + j] = __ldg(src + i * d.H + j);
        v[25] = 1.0f;   // bias column
      }
#pragma unroll
      for (int t = 0; t < 32; ++t) {
        float hi, lo;
        tc::split_tf32(v[t], hi, lo);
        const unsigned off = tc::tile_offset(t, tid >> 2, kWgChunks) + (unsigned)(tid & 3) * 4u;
        *reinterpret_cast<float*>(b_hi + off) = hi;
        *reinterpret_cast<float*>(b_lo + off) = lo;
      }
    }
    tc::fence_async_smem();
    __syncthreads();
    if (warp == 0) {   // the whole warp runs the loop, an elected lane issues (see wide_tc.cuh)
      tc::fence_after_sync();
      for (int pass = 0; pass < passes; ++pass) {
        const unsigned a_s = (pass == 1) ? a_lo_s : a_hi_s;
        const unsigned b_s = (pass == 2) ? b_lo_s : b_hi_s;
#pragma unroll 4
        for (int ks = 0; ks < kTcRows / 8; ++ks) {   // 8 positions per MMA
          const unsigned long long ad = tc::smem_desc(a_s + ks * 256, 128, a_group);
          const unsigned long long bd = tc::smem_desc(b_s + ks * 256, 128, a_group);
          tc::mma_tf32_elect(tmem_d, ad, bd, idesc, accumulate);
          accumulate = 1;
        }
      }
      tc::mma_commit_elect(bar);
    }
    mbar_wait_bounded(bar, phase, status, gave_up);   // the tiles may be overwritten
    phase ^= 1u;
    // Every kWgFlush tiles the accumulator moves into registers and starts again from zero: the tensor
    // core adds into its fp32 accumulator with truncation, about one ulp of the running sum per MMA, and
    // 48 MMAs per tile over the ~18 tiles of a CTA at batch 1,024 left the conv-filter gradient 5e-5
    // from the fp64 oracle.  Two tiles per flush keep it at 1e-6; the sums below round to nearest.
    if (++since_flush == kWgFlush) {
      since_flush = 0;
      accumulate = 0;
      tc::fence_after_sync();
      if (warp < 4) {
#pragma unroll
        for (int c0 = 0; c0 < 32; c0 += 16) {
          float acc[16];
          tc::tmem_ld16(lane_base + (unsigned)c0, acc);
#pragma unroll
          for (int e = 0; e < 16; ++e) racc[c0 + e] += acc[e];
        }
      }
      tc::fence_before_sync();   // ordered before the next tile's MMAs by the block barrier that precedes them
    }
  }
  tc::fence_after_sync();
  // ---- epilogue: M = 128: lane l of warp w is map 32w + l; M = 64: lanes 0..15 are maps 16w + l ----
  if (warp < 4) {
    const bool full = d.F == 128;
    const int f = full ? (32 * warp + lane) : (16 * warp + lane);
    const bool owner = full || lane < 16;
    float* dst = part + ((size_t)blockIdx.x * d.F + (owner ? f : 0)) * 26;
#pragma unroll
    for (int c0 = 0; c0 < 32; c0 += 16) {
      float acc[16];
      if (since_flush != 0) tc::tmem_ld16(lane_base + (unsigned)c0, acc);   // what has not been flushed yet
      if (owner) {
#pragma unroll
        for (int e = 0; e < 16; ++e)
          if (c0 + e < 26) dst[c0 + e] = racc[c0 + e] + (since_flush != 0 ? acc[e] : 0.f);
      }
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_d, tmem_cols);
}

bool wide_grad_tc_supported(const WideDims& d) { return (d.F == 64 || d.F == 128) && (d.C * d.C) % 4 == 0; }

int wide_grad_c1_tc(cnn_wide* w, const float* d_images, long n, int* rows_out, cudaStream_t st) {
  const WideDims& d = w->d;
  const size_t smem = 2 * (size_t)d.F * kWgChunks * 16 + 2 * kTcRows * 128 + 16;
  const long n_tiles = (n * (long)d.C * d.C + kTcRows - 1) / kTcRows;
  int per_sm = (int)(220 * 1024 / smem);
  if (per_sm > 16) per_sm = 16;        // 32 TMEM columns per CTA
  if (per_sm < 1) per_sm = 1;
  long grid = (long)sm_count() * per_sm;
  if (grid > n_tiles) grid = n_tiles;
  if (grid > w->part_rows) grid = w->part_rows;
  const int passes = (w->conv_mode == 2) ? 3 : 1;
  CNN_CUDA(cudaFuncSetAttribute(k_wide_grad_c1_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  k_wide_grad_c1_tc<<<(unsigned)grid, kWgThreads, smem, st>>>(d, d_images, w->dc, n, w->part_c, passes, 32u, w->d_status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "k_wide_grad_c1_tc launch");
  *rows_out = (int)grid;
  return CNN_OK;
}

}  // namespace cnn
