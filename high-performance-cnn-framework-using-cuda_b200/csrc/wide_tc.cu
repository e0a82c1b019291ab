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


}  // namespace cnn
