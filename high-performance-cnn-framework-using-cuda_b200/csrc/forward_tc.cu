// Batched forward of the reference's 28x28 net with the convolution (fp_preact_c1, layer.cu:116-133:
// 94 % of the forward MACs) on the 5th-generation tensor cores (tcgen05, accumulators in tensor
// memory), and everything after it -- bias, sigmoid, shared 4x4 subsample, sigmoid, FC 216->10,
// sigmoid, argmax -- done by the epilogue warps straight out of tensor memory.  Selected with the
// option "forward_path" = 1 (three tf32 passes, fp32-level accuracy) or 2 (one tf32 pass and a
// tanh.approx sigmoid: an explicitly reduced-precision inference mode).
//
// The convolution as a GEMM WITHOUT an im2col copy.  A CTA sees its images as one matrix of stacked
// image rows, R[r][c] with r = 28 * image + y (28 floats per row, contiguous in HBM as they are).
// For kernel row i the conv is a product with a banded (Toeplitz) weight matrix,
//     out[r][x][f] = sum_i sum_c R[r + i][c] * T_i[c][x][f],   T_i[c][x][f] = Wc[f][i][c - x] (0 <= c-x < 5),
// so the A operand of kernel row i is the SAME tile of image rows, started i rows further down: in
// the un-swizzled K-major shared-memory layout a row is 16 bytes inside each 16-byte column chunk
// ([chunk][row][4 floats]), and a matrix descriptor may start at any row.  The band is cut into two
// blocks of 12 output columns (16 input columns, K = 16 per kernel row), and because the weights are
// shift-invariant both blocks use the same B operand: 5 x [80 x 16] tf32 values, 25 KB.  One tile of
// 128 stacked rows (4.57 images) costs 2 blocks x 5 kernel rows x 2 K-steps = 20 MMAs of
// 128 x 80 x 8 per pass.  Rows y = 24..27 of every image produce junk (they run into the next image)
// and are discarded: 24 of 28 tensor-memory lanes carry results.
//
// Accuracy.  Path 1 splits both operands into a tf32-exact high part and the remainder and issues
// hi*hi + lo*hi + hi*lo (three passes, fp32 accumulation): pre-activations agree with the fp32 SIMT
// kernel to a few 1e-7, the 1e-5 parity bar holds.  Path 2 feeds the fp32 bit patterns as they are
// (the tensor core reads 19 of the 32 bits) and evaluates sigmoid(v) = 0.5 + 0.5 * tanh.approx(v / 2):
// outputs within about 1e-3, argmax equal wherever the top-two margin is clear of that.
//
// Pipeline (one CTA per SM, 16 warps, everything handed over through mbarriers with bounded waits):
//   warp 0      bulk copies (cp.async.bulk, no multicast) of 136 stacked rows = 15,232 contiguous
//               bytes per tile into a raw staging buffer, three stages;
//   warps 2-3   rearrange a raw tile into the operand layout (and split it, path 1);
//   warp 1      issues the tile's MMAs into one of three 160-column accumulators and commits to an
//               mbarrier (the whole warp runs the loop, an elected lane issues: see wide_tc.cuh);
//   warps 4-15  three epilogue groups of four warps (one per 32-lane quarter of tensor memory), one
//               tile each: tcgen05.ld of 24 columns (one window column, six maps) at a time, bias,
//               sigmoid, the window row's four subsample taps; the four rows of a window are four
//               adjacent lanes (reduce-scatter by shuffles); subsample sigmoid; FC partial sums of a
//               window row into shared memory; the group that completes an image's sixth window row
//               adds them, applies the output sigmoid, takes the argmax and writes 44 bytes.
#include "net.cuh"
#include "wide_tc.cuh"

namespace cnn {

constexpr int kTfThreads = 512;
constexpr int kTfStages = 3;                 // raw buffers = operand slabs = accumulators
constexpr int kTfRows = 128;                 // stacked rows per tile = tensor-memory lanes
constexpr int kTfSlabRows = 136;             // + the 4 rows the last kernel row reaches, padded to 8
constexpr int kTfChunks = 7;                 // 16-byte chunks of a 28-float image row
constexpr int kTfTileBytes = kTfSlabRows * kH * 4;              // 15,232: raw tile and operand slab alike
constexpr unsigned kTfChunkStride = kTfSlabRows * 16;           // 2,176 B between column chunks of a slab
constexpr int kTfBN = 80;                    // MMA N of one 12-column block: 72 used, padded to 16n
constexpr int kTfBlockCols = 12;             // output columns per block
constexpr unsigned kTfBChunk = kTfBN * 16;   // 1,280 B between the K chunks of a B block
constexpr unsigned kTfBRow = 4 * kTfBChunk;  // 5,120 B per kernel row (K = 16)
constexpr int kTfBBytes = 5 * kTfBRow;       // 25,600
constexpr int kTfDCols = 2 * kTfBN;          // 160 accumulator columns per tile
constexpr int kTfSlots = 32;                 // images in flight (FC partial sums), ring
constexpr int kTfConvWarps = 2;
constexpr int kTfEpiWarp0 = 4;

struct TfSmem {
  alignas(128) unsigned char raw[kTfStages][kTfTileBytes];
  alignas(128) unsigned char a_hi[kTfStages][kTfTileBytes + 128];
  alignas(128) unsigned char a_lo[kTfStages][kTfTileBytes + 128];   // path 1 only
  alignas(128) unsigned char b_hi[kTfBBytes];
  alignas(128) unsigned char b_lo[kTfBBytes];                        // path 1 only
  alignas(16) float wf[7][36][12];          // [window row p][6 * q + f][k], p = 6 is the junk row (zeros)
  float wf_tail[12];                        // a lane's empty fifth slot may read one entry past the last row
  alignas(16) float part[kTfSlots][6][12];  // FC partial sums of (image slot, window row)
  int done[kTfSlots];                       // window rows of the slot's image that have arrived
  float bc[8], ws[16], bs[4], bf[12];
  unsigned long long raw_full[kTfStages], raw_free[kTfStages], a_full[kTfStages], d_full[kTfStages],
      d_free[kTfStages];
  unsigned tmem_base;
};

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Eight consecutive fp32 columns of this warp's 32 tensor-memory lanes; not waited for.
__device__ __forceinline__ void tmem_ld8_nowait(unsigned taddr, unsigned (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
}
// Wait for this warp's outstanding tensor-memory loads; the 24 registers of one window column are
// listed as in/out operands so that their uses cannot be scheduled above the wait.
__device__ __forceinline__ void tmem_wait24(unsigned (&a)[8], unsigned (&b)[8], unsigned (&c)[8]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]),
                 "+r"(b[0]), "+r"(b[1]), "+r"(b[2]), "+r"(b[3]), "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7]),
                 "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]), "+r"(c[4]), "+r"(c[5]), "+r"(c[6]), "+r"(c[7])
               :: "memory");
}

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// PATH 1: three tf32 passes, sigmoid flavour SIG (0 or 2).  PATH 2: one pass, tanh sigmoid.
template <int PATH, int SIG>
__global__ void __launch_bounds__(kTfThreads, 1)
k_forward_tc(const float* __restrict__ images, long n, long imgs_per_cta, const float* __restrict__ params,
             float* __restrict__ out, int* __restrict__ argmax, int* __restrict__ status) {
  extern __shared__ unsigned char smem_raw[];
  TfSmem& sm = *reinterpret_cast<TfSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr bool kPrecise = (PATH == 1);
  constexpr float kPre = kPrecise ? 1.0f : 0.5f;   // path 2 computes tanh(v / 2): weights and bias are halved

  const long img0 = (long)blockIdx.x * imgs_per_cta;
  const long imgs_here_l = (n - img0) < imgs_per_cta ? (n - img0) : imgs_per_cta;
  const int imgs_here = imgs_here_l > 0 ? (int)imgs_here_l : 0;
  const int rows_here = imgs_here * kH;
  const int n_tiles = (rows_here + kTfRows - 1) / kTfRows;
  const long rows_total = n * kH;
  const long row0 = img0 * kH;

  // ---- set-up: B operand (banded weights), FC table, small parameters, barriers, tensor memory -----
  for (int e = tid; e < 5 * kTfBN * 16; e += kTfThreads) {
    const int i = e / (kTfBN * 16), rem = e % (kTfBN * 16);
    const int nn = rem / 16, c = rem % 16;
    float v = 0.f;
    if (nn < 72) {
      const int qq = nn / 24, f = (nn % 24) / 4, j = nn % 4;
      const int d = c - (4 * qq + j);
      if (d >= 0 && d < 5) v = kPre * params[kOffWc + f * 25 + i * 5 + d];
    }
    float hi, lo;
    tc::split_tf32(v, hi, lo);
    const unsigned off = (unsigned)i * kTfBRow + (unsigned)(c >> 2) * kTfBChunk + (unsigned)nn * 16u + (unsigned)(c & 3) * 4u;
    *reinterpret_cast<float*>(sm.b_hi + off) = hi;
    if (kPrecise) *reinterpret_cast<float*>(sm.b_lo + off) = lo;
  }
  for (int e = tid; e < 7 * 36 * 12; e += kTfThreads) {
    const int p = e / (36 * 12), idx = (e / 12) % 36, k = e % 12;
    const int q = idx / 6, f = idx % 6;
    sm.wf[p][idx][k] = (p < 6 && k < kOut) ? params[kOffWf + k * kS + f * 36 + p * 6 + q] : 0.f;
  }
  if (tid < kF) sm.bc[tid] = kPre * params[kOffBc + tid];
  if (tid < 16) sm.ws[tid] = params[kOffWs + tid];
  if (tid == 0) sm.bs[0] = params[kOffBs];
  if (tid < 12) sm.bf[tid] = (tid < kOut) ? params[kOffBf + tid] : 0.f;
  if (tid < kTfSlots) sm.done[tid] = 0;
  if (tid == 0) {
    for (int s = 0; s < kTfStages; ++s) {
      mbar_init(&sm.raw_full[s], 1);
      mbar_init(&sm.raw_free[s], kTfConvWarps);
      mbar_init(&sm.a_full[s], kTfConvWarps);
      mbar_init(&sm.d_full[s], 1);
      mbar_init(&sm.d_free[s], 4);
    }
    mbar_fence_init();
  }
  if (warp == 1) tc::tmem_alloc(&sm.tmem_base, 512);
  tc::fence_async_smem();      // the B operand was written through the generic proxy
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const unsigned tmem_base = sm.tmem_base;

  bool gave_up = false;

  if (warp == 0) {
    // ================= producer: raw tiles by bulk copy ==========================================
    if (lane == 0) {
      for (int k = 0; k < n_tiles; ++k) {
        const int s = k % kTfStages;
        const unsigned par = (unsigned)(k / kTfStages) & 1u;
        mbar_wait_bounded(&sm.raw_free[s], par ^ 1u, status, gave_up);
        const long r_first = row0 + (long)k * kTfRows;
        long rows = rows_total - r_first;
        if (rows > kTfSlabRows) rows = kTfSlabRows;
        const unsigned bytes = (unsigned)rows * (kH * 4);
        mbar_expect_tx(&sm.raw_full[s], bytes);
        bulk_g2s(sm.raw[s], images + r_first * kH, bytes, &sm.raw_full[s]);
      }
    }
  } else if (warp == 1) {
    // ================= MMA issue: the whole warp runs the loop, one elected lane issues ============
    const unsigned idesc = tc::idesc_tf32(kTfRows, kTfBN, 0, 0);
    const unsigned b_hi_s = smem_u32(sm.b_hi), b_lo_s = smem_u32(sm.b_lo);
    for (int k = 0; k < n_tiles; ++k) {
      const int s = k % kTfStages;
      const unsigned par = (unsigned)(k / kTfStages) & 1u;
      mbar_wait_bounded(&sm.a_full[s], par, status, gave_up);
      mbar_wait_bounded(&sm.d_free[s], par ^ 1u, status, gave_up);
      __syncwarp();
      tc::fence_after_sync();
      const unsigned a_hi_s = smem_u32(sm.a_hi[s]), a_lo_s = smem_u32(sm.a_lo[s]);
      const unsigned d_tile = tmem_base + (unsigned)(s * kTfDCols);
      constexpr int kPasses = kPrecise ? 3 : 1;
#pragma unroll
      for (int xb = 0; xb < 2; ++xb) {
        unsigned accumulate = 0;
#pragma unroll
        for (int pass = 0; pass < kPasses; ++pass) {
          const unsigned a_s = (pass == 1) ? a_lo_s : a_hi_s;
          const unsigned b_s = (pass == 2) ? b_lo_s : b_hi_s;
#pragma unroll
          for (int i = 0; i < 5; ++i) {
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
              const unsigned long long ad =
                  tc::smem_desc(a_s + (unsigned)(3 * xb + 2 * ks) * kTfChunkStride + (unsigned)i * 16u, kTfChunkStride, 128);
              const unsigned long long bd = tc::smem_desc(b_s + (unsigned)i * kTfBRow + (unsigned)(2 * ks) * kTfBChunk, kTfBChunk, 128);
              tc::mma_tf32_elect(d_tile + (unsigned)(xb * kTfBN), ad, bd, idesc, accumulate);
              accumulate = 1;
            }
          }
        }
      }
      tc::mma_commit_elect(&sm.d_full[s]);
    }
  } else if (warp < kTfEpiWarp0) {
    // ================= converters: raw tile -> operand slab(s) ====================================
    const int ct = tid - 64;                       // 0..63
    for (int k = 0; k < n_tiles; ++k) {
      const int s = k % kTfStages;
      const unsigned par = (unsigned)(k / kTfStages) & 1u;
      mbar_wait_bounded(&sm.raw_full[s], par, status, gave_up);
      mbar_wait_bounded(&sm.d_full[s], par ^ 1u, status, gave_up);   // the slab's previous MMAs are done
      const unsigned char* src = sm.raw[s];
      unsigned char* dhi = sm.a_hi[s];
      unsigned char* dlo = sm.a_lo[s];
#pragma unroll 5
      for (int t = ct; t < kTfChunks * kTfSlabRows; t += 32 * kTfConvWarps) {
        const int chunk = t / kTfSlabRows, row = t - chunk * kTfSlabRows;
        const float4 v = *reinterpret_cast<const float4*>(src + row * (kH * 4) + chunk * 16);
        const unsigned off = (unsigned)chunk * kTfChunkStride + (unsigned)row * 16u;
        if (kPrecise) {
          float4 hi, lo;
          tc::split_tf32(v.x, hi.x, lo.x); tc::split_tf32(v.y, hi.y, lo.y);
          tc::split_tf32(v.z, hi.z, lo.z); tc::split_tf32(v.w, hi.w, lo.w);
          *reinterpret_cast<float4*>(dhi + off) = hi;
          *reinterpret_cast<float4*>(dlo + off) = lo;
        } else {
          *reinterpret_cast<float4*>(dhi + off) = v;
        }
      }
      tc::fence_async_smem();    // generic-proxy writes -> visible to the tensor core's operand reads
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&sm.a_full[s]);
        mbar_arrive(&sm.raw_free[s]);
      }
    }
  } else {
    // ================= epilogue ====================================================================
    const int group = (warp - kTfEpiWarp0) >> 2;   // accumulator / tile residue this group owns
    const int quarter = warp & 3;                  // tensor-memory lanes 32 * quarter ..
    const int rsub = lane & 3;                     // row of the 4x4 window (28, 32 and 128 are multiples of 4)
    float wsr[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) wsr[j] = (kPrecise ? 1.0f : 0.5f) * sm.ws[rsub * 4 + j];
    float bcr[kF];
#pragma unroll
    for (int f = 0; f < kF; ++f) bcr[f] = sm.bc[f];
    // path 2: sum_j ws * (0.5 + 0.5 t) = sum_j (0.5 ws) t + 0.5 * sum(ws); the constant goes into the bias
    float bs_eff = sm.bs[0];
    if (!kPrecise) {
      float sw = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) sw += sm.ws[j];
      bs_eff = fmaf(0.5f, sw, bs_eff);
    }

    for (int k = group; k < n_tiles; k += kTfStages) {
      const unsigned par = (unsigned)(k / kTfStages) & 1u;
      mbar_wait_bounded(&sm.d_full[group], par, status, gave_up);
      tc::fence_after_sync();
      const int R = k * kTfRows + quarter * 32 + lane;     // stacked row of this lane inside the CTA
      const int img_l = R / kH;
      const int y = R - img_l * kH;
      const int p = y >> 2;
      const bool valid = (img_l < imgs_here) && (p < 6);
      const unsigned t0 = tmem_base + (unsigned)(group * kTfDCols) + ((unsigned)(quarter * 32) << 16);

      float fc[kOut];
#pragma unroll
      for (int kk = 0; kk < kOut; ++kk) fc[kk] = 0.f;
      const bool b0 = (lane & 1) != 0, b1 = (lane & 2) != 0;
      const int pw = p < 6 ? p : 6;                 // the junk window row reads the table's zero row

      unsigned ra[8], rb[8], rc[8], na[8], nb[8], nc[8];
      tmem_ld8_nowait(t0 + 0, ra);
      tmem_ld8_nowait(t0 + 8, rb);
      tmem_ld8_nowait(t0 + 16, rc);
      tmem_wait24(ra, rb, rc);
#pragma unroll
      for (int xb = 0; xb < 2; ++xb) {              // one 12-column block = three window columns
        float z[18];
#pragma unroll
        for (int wq = 0; wq < 3; ++wq) {            // window column q = 3 * xb + wq: 24 accumulator columns
          const int nxt = 3 * xb + wq + 1;
          if (nxt < 6) {
            const unsigned c0 = (unsigned)((nxt / 3) * kTfBN + (nxt % 3) * 24);
            tmem_ld8_nowait(t0 + c0, na);
            tmem_ld8_nowait(t0 + c0 + 8, nb);
            tmem_ld8_nowait(t0 + c0 + 16, nc);
          } else {
            // the last columns of this accumulator are in registers: hand it back to the MMA warp
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.d_free[group]);
          }
          // 24 independent activations, written in stages so that their chains interleave
          float av[24];
#pragma unroll
          for (int c = 0; c < 24; ++c) {
            const unsigned bits = (c < 8) ? ra[c] : (c < 16) ? rb[c - 8] : rc[c - 16];
            av[c] = __uint_as_float(bits) + bcr[c >> 2];
          }
#pragma unroll
          for (int c = 0; c < 24; ++c) av[c] = kPrecise ? sigmoidf<SIG>(av[c]) : tanh_approx(av[c]);
#pragma unroll
          for (int f = 0; f < kF; ++f)
            z[wq * 6 + f] = fmaf(wsr[3], av[f * 4 + 3], fmaf(wsr[2], av[f * 4 + 2], fmaf(wsr[1], av[f * 4 + 1], wsr[0] * av[f * 4])));
          if (nxt < 6) {
            tmem_wait24(na, nb, nc);
#pragma unroll
            for (int e = 0; e < 8; ++e) { ra[e] = na[e]; rb[e] = nb[e]; rc[e] = nc[e]; }
          }
        }
        // ---- the window's four rows are lanes 4g..4g+3: reduce-scatter the block's 18 sums -----------
        // step 1 (lane bit 0): 9 each; step 2 (lane bit 1): 5 / 4 (+ one empty slot)
        float w9[9];
#pragma unroll
        for (int i = 0; i < 9; ++i) {
          const float send = b0 ? z[i] : z[i + 9];
          const float keep = b0 ? z[i + 9] : z[i];
          w9[i] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
        }
        float u[5];
#pragma unroll
        for (int i = 0; i < 5; ++i) {
          const float hi9 = (i < 4) ? w9[i + 5] : 0.f;
          const float send = b1 ? w9[i] : hi9;
          const float keep = b1 ? hi9 : w9[i];
          u[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
        }
        // this lane holds the sums e = e0 .. e0+4 of the block (e = 6 * window column + map); for lanes
        // with bit 1 set the fifth slot is empty
        const int e0 = (b0 ? 9 : 0) + (b1 ? 5 : 0);
        const float* wrow = &sm.wf[pw][18 * xb + e0][0];
#pragma unroll
        for (int i = 0; i < 5; ++i) {
          const float zs = u[i] + bs_eff;
          float as = kPrecise ? sigmoidf<SIG>(zs) : fmaf(0.5f, tanh_approx(0.5f * zs), 0.5f);
          if (i == 4 && b1) as = 0.f;
          const float4 w0 = *reinterpret_cast<const float4*>(wrow + i * 12);
          const float4 w1 = *reinterpret_cast<const float4*>(wrow + i * 12 + 4);
          const float2 w2 = *reinterpret_cast<const float2*>(wrow + i * 12 + 8);
          fc[0] = fmaf(w0.x, as, fc[0]); fc[1] = fmaf(w0.y, as, fc[1]); fc[2] = fmaf(w0.z, as, fc[2]);
          fc[3] = fmaf(w0.w, as, fc[3]); fc[4] = fmaf(w1.x, as, fc[4]); fc[5] = fmaf(w1.y, as, fc[5]);
          fc[6] = fmaf(w1.z, as, fc[6]); fc[7] = fmaf(w1.w, as, fc[7]); fc[8] = fmaf(w2.x, as, fc[8]);
          fc[9] = fmaf(w2.y, as, fc[9]);
        }
      }
#pragma unroll
      for (int kk = 0; kk < kOut; ++kk) {
        fc[kk] += __shfl_xor_sync(0xffffffffu, fc[kk], 1);
        fc[kk] += __shfl_xor_sync(0xffffffffu, fc[kk], 2);
      }
      // ---- hand the window row's ten sums to the image; the sixth arrival finishes the image ---------
      const int slot = img_l & (kTfSlots - 1);
      int arrived = 0;
      if (valid && rsub == 0) {
        float* dst = &sm.part[slot][p][0];
        *reinterpret_cast<float4*>(dst) = make_float4(fc[0], fc[1], fc[2], fc[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(fc[4], fc[5], fc[6], fc[7]);
        *reinterpret_cast<float2*>(dst + 8) = make_float2(fc[8], fc[9]);
        __threadfence_block();
        arrived = atomicAdd(&sm.done[slot], 1) + 1;
      }
      arrived = __shfl_sync(0xffffffffu, arrived, lane & ~3);
      if (valid && arrived == 6) {
        __threadfence_block();
        // lane rsub of the window takes outputs k = rsub, rsub + 4, rsub + 8 (< 10)
        float best = -1.f;
        int best_k = 0;
#pragma unroll
        for (int t = 0; t < 3; ++t) {
          const int kk = rsub + 4 * t;
          if (kk < kOut) {
            float zf = 0.f;
#pragma unroll
            for (int pp = 0; pp < 6; ++pp) zf += *reinterpret_cast<volatile float*>(&sm.part[slot][pp][kk]);
            zf += sm.bf[kk];
            const float o = kPrecise ? sigmoidf<SIG>(zf) : fmaf(0.5f, tanh_approx(0.5f * zf), 0.5f);
            if (out) out[(img0 + img_l) * kOut + kk] = o;
            if (best < o) { best = o; best_k = kk; }     // ascending k: the lowest index wins ties
          }
        }
        // classify(): strict '<' scan from index 0 -- the greatest value, the lowest index among equals
#pragma unroll
        for (int m = 1; m <= 2; m <<= 1) {
          const float ov = __shfl_xor_sync(0xfu << (lane & ~3), best, m);
          const int ok = __shfl_xor_sync(0xfu << (lane & ~3), best_k, m);
          if (ov > best || (ov == best && ok < best_k)) { best = ov; best_k = ok; }
        }
        if (rsub == 0) {
          if (argmax) argmax[img0 + img_l] = best_k;
          sm.done[slot] = 0;
        }
      }
    }
  }

  tc::fence_before_sync();
  __syncthreads();
  if (warp == 1) tc::tmem_dealloc(tmem_base, 512);
}

template <int PATH, int SIG>
static int launch_forward_tc(cnn_net* net, const float* d_images, long n, float* d_out, int* d_argmax,
                             cudaStream_t stream) {
  // Every CTA owns a contiguous range of whole images (an image's window rows meet in shared memory).
  long grid = sm_count();
  const long min_imgs = 16;
  if (grid * min_imgs > n) grid = (n + min_imgs - 1) / min_imgs;
  const long per_cta = (n + grid - 1) / grid;
  grid = (n + per_cta - 1) / per_cta;
  const size_t smem = sizeof(TfSmem) + 128;
  CNN_CUDA(cudaFuncSetAttribute(k_forward_tc<PATH, SIG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  k_forward_tc<PATH, SIG><<<(unsigned)grid, kTfThreads, smem, stream>>>(d_images, n, per_cta, net->d_params, d_out,
                                                                       d_argmax, net->d_status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "k_forward_tc launch");
  return CNN_OK;
}

int forward_device_tc(cnn_net* net, const float* d_images, long n, float* d_out, int* d_argmax,
                      cudaStream_t stream) {
  if (net->forward_path == 2) return launch_forward_tc<2, 2>(net, d_images, n, d_out, d_argmax, stream);
  return net->fast_sigmoid ? launch_forward_tc<1, 2>(net, d_images, n, d_out, d_argmax, stream)
                           : launch_forward_tc<1, 0>(net, d_images, n, d_out, d_argmax, stream);
}

}  // namespace cnn
