// Conv deltas and conv weight gradient of the widened configuration in one kernel: a tcgen05 pipeline
// fed by TMA.
//
//   dc[m][f] = Ws[y % 4][x % 4] * ds[window of m][f] * a (1 - a) / (C*C)      (bp_output_s1 + bp_preact_c1)
//   G[f][t]  = sum_m dc[m][f] * A[m][t]      m = (image, output position), t = filter tap
//   Gs[r][c] = sum over windows and maps of ds * a[4 wy + r][4 wx + c]           (bp_weight_s1)
//
// with A the im2col rows of the forward convolution, a the conv activations and ds the subsample
// deltas.  The conv deltas never exist in HBM: the activations of a tile come in by TMA, eight warps
// turn them into deltas in shared memory (and add up the subsample-filter gradient on the way), and
// the tensor core consumes them from there.
// As an MMA:  D[M = F = 64][N = 32] += dcT[64][K = TP positions] * im2colT[32][K = TP positions], both
// operands K-major (dcT with the 128-byte swizzle, im2colT in the canonical un-swizzled layout); tap
// 25, unused by the filter, is a row of ones so that column 25 of D is the conv-bias gradient (taps
// 26..31 are rows of zeros).  A tile is TP consecutive positions of ONE image (the last tile of an
// image is ragged: the positions past the image read as zeros).
//
// One CTA per SM, sixteen warps (128 registers each), four stages of 48 KB in shared memory:
//   * the activation tile (64 maps x TP positions, 32 KB at TP = 128) comes in by TMA: activations
//     are stored per (image, map) with positions contiguous, a 3-D tensor map (position, map,
//     image) with a box of 32 positions x 64 maps and the 128-byte swizzle writes one K-block of the operand (64 rows of
//     128 bytes) per cp.async.bulk.tensor, and the MMA reads it through a SWIZZLE_128B descriptor.
//     (Copying the tile with per-thread cp.async stalled at 2 TB/s: the copies of one tile took
//     4,000 cycles to get into the load/store pipeline.)  No multicast; positions past the image
//     are filled with zeros;
//   * warps 1-3 copy the im2colT tile with 16-byte cp.async.  A tap's window of four
//     consecutive positions starts at column x + j of an image row, 16-byte aligned only for j = 0
//     and 4; a small kernel therefore first writes every image shifted left by 0..3 columns, and
//     tap (i, j) reads the copy shifted by j % 4 at column x + 4 (j / 4).  A warp instruction covers
//     8 taps x 4 chunks (conflict-free in shared memory, 64 contiguous bytes per tap in global
//     memory).  (With 4-byte copies straight from the image the 104 gathers of a tile took 3,000
//     cycles to issue and bound the kernel);
//   * warps 8-15 turn the landed activations into deltas in place (one 16-byte piece = four positions
//     of one window row of one map: one ds value, four filter taps; a warp instruction covers 32 maps
//     of one chunk, conflict-free thanks to the swizzle) and, in the three-pass mode (hi*hi + lo*hi +
//     hi*lo, fp32-level accuracy), split them into a tf32-exact high tile and a remainder tile; the
//     im2col warps split what they copied; in the one-pass mode the tensor core reads the fp32
//     values as they are;
//   * warp 0 issues the MMAs (an elected lane of the converged warp) and commits to mbarriers;
//   * warps 4-7 (one per 32-lane quarter of tensor memory) move the accumulator into registers every
//     256 positions and add it there: the tensor core adds into its fp32 accumulator with truncation,
//     about one ulp of the running sum per MMA, which over the ~150 tiles of a CTA at batch 1,024
//     would leave the gradient 5e-5 from the fp64 oracle.  Two accumulators alternate, so the MMA
//     warp never waits for a flush.
// Every wait is bounded; a wait that runs out sets the status word and lets the kernel finish.
// At the end every CTA writes one partial [F][26] and one partial [17] of the subsample-filter
// gradient; k_wide_reduce adds the partials.
#include <cuda.h>

#include "wide.cuh"
#include "wide_tc.cuh"
#include "phase_clocks.cuh"

namespace cnn {

constexpr int kGtRingBytes = 192 * 1024;     // operand stages of one CTA
constexpr int kGtMaxStages = 8;
constexpr int kGtThreads = 16 * 32;
constexpr int kGtDeltaWarps = 8;
constexpr int kGtIm2colWarps = 3;
constexpr int kGtF = 64;

struct GtBarriers {
  unsigned long long landed[kGtMaxStages], full[kGtMaxStages], free[kGtMaxStages], acc_full[2], acc_free[2];
  unsigned tmem_base;
  long long clock_base;    // phase clocks only
  float ws[16];            // subsample filter
  float red[kGtDeltaWarps][17];   // subsample-filter gradient partials of the delta warps
};

CNN_PHASE_TABLE(g_phase_clocks_wg, 16)

// One 3-D box of the tensor behind `map` into shared memory; completes its bytes on the mbarrier.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(c0), "r"(c1), "r"(c2),
        "r"(smem_u32(bar))
      : "memory");
}

// Shared-memory descriptor of a K-major operand stored with the 128-byte swizzle: rows of 128 bytes (32 tf32
// values of K), eight rows per 1,024-byte atom (SBO), the 16-byte chunks of a row XOR-ed with the row number
// -- what a TMA box with CU_TENSOR_MAP_SWIZZLE_128B writes.  Layout type 2 in bits 61-63, version 1.
__device__ __forceinline__ unsigned long long smem_desc_sw128(unsigned smem_addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);
  d |= 1ull << 16;                        // leading byte offset: not used by swizzled K-major operands
  d |= (unsigned long long)(1024u >> 4) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

constexpr unsigned kGtKBlock = 64 * 128;   // bytes of one K-block of the dcT operand: 64 maps x 32 positions

// TP = positions per tile (K of one tile): 128 with one pass, 64 with three (the stage then holds a high and
// a low tile of each operand).
template <int TP, int PASSES>
__global__ void __launch_bounds__(kGtThreads, 1)
k_wide_grad_c1_pipe(WideDims d, const __grid_constant__ CUtensorMap ac_map, const float* __restrict__ shifted,
                    const float* __restrict__ ds, const float* __restrict__ params, long n,
                    float* __restrict__ part, float* __restrict__ part_s, int* __restrict__ status) {
  constexpr int CH = TP / 4;                          // 16-byte chunks along K
  constexpr unsigned kGroup = tc::tile_group_stride(CH);
  constexpr unsigned kABytes = (kGtF / 8) * kGroup;   // TP * 256
  constexpr unsigned kBBytes = 4 * kGroup;            // 32 tap rows: TP * 128
  // Stage layout: [delta tile | its low part (three passes) | im2col tile | its low part].  With three passes
  // the two im2col tiles lie back to back and are read as ONE operand of 64 rows: the high delta tile times
  // [hi taps | lo taps] fills 64 accumulator columns in one MMA per K step (hi*hi in columns 0..31, hi*lo in
  // 32..63), the low delta tile times the hi taps adds lo*hi to columns 0..31 -- two MMAs per K step instead
  // of three; the flush adds the two column groups.
  constexpr unsigned kALoOff = kABytes;                                  // low delta tile
  constexpr unsigned kBOff = (PASSES == 3 ? 2u : 1u) * kABytes;           // im2col tile (high part)
  constexpr unsigned kBLoOff = kBBytes;                                  // its low part, relative to the high part
  constexpr unsigned kAccCols = (PASSES == 3) ? 64u : 32u;                // TMEM columns per accumulator
  constexpr int kGtStageBytes = (PASSES == 3 ? 2 : 1) * (int)(kABytes + kBBytes);   // 48 KB at TP = 128 (64 with three passes)
  constexpr int kGtStages = kGtRingBytes / kGtStageBytes;
  static_assert(kGtStages >= 3 && kGtStages <= kGtMaxStages && kGtStageBytes % 1024 == 0, "stage ring");
  constexpr int kAhead = kGtStages - 1;               // tiles in flight beyond the one being handed over
  constexpr int kFlushTiles = 256 / TP;               // tiles per accumulator hand-over

  extern __shared__ unsigned char smem_raw[];
  unsigned char* stage0 = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  GtBarriers& bars = *reinterpret_cast<GtBarriers*>(stage0 + kGtStages * kGtStageBytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int CC = d.C * d.C;
  const int tiles_per_image = (CC + TP - 1) / TP;
  const long n_tiles = n * tiles_per_image;
  const int my_tiles = (blockIdx.x < n_tiles) ? (int)((n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;

  // ---- set-up: all stages zero (stale operand bytes must at least be finite), the row of ones, barriers ----
  for (int i = tid; i < kGtStages * kGtStageBytes / 16; i += kGtThreads)
    reinterpret_cast<float4*>(stage0)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  __syncthreads();
  for (int i = tid; i < kGtStages * TP; i += kGtThreads) {
    const int s = i / TP, p = i % TP;
    *reinterpret_cast<float*>(stage0 + s * kGtStageBytes + kBOff + tc::tile_offset(25, p >> 2, CH) + (p & 3) * 4) = 1.0f;
  }
  if (tid < 16) bars.ws[tid] = params[d.o_ws + tid];
  if (tid == 0) {
    for (int s = 0; s < kGtStages; ++s) {
      mbar_init(&bars.landed[s], 1);      // the producer's arrive.expect_tx; the TMA completes the bytes
      mbar_init(&bars.full[s], kGtDeltaWarps + kGtIm2colWarps);   // one arrival per delta warp and per im2col warp
      mbar_init(&bars.free[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars.acc_full[a], 1);
      mbar_init(&bars.acc_free[a], 4);
    }
    mbar_fence_init();
  }
  if (warp == 0) tc::tmem_alloc(&bars.tmem_base, 2 * kAccCols);
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const unsigned tmem_d = bars.tmem_base;

  bool gave_up = false;
  CNN_PHASE_BEGIN(blockIdx.x == 0, bars.clock_base)
  const int n_groups = (my_tiles + kFlushTiles - 1) / kFlushTiles;

  // tile kk of this CTA: image and first position in it
  auto tile_origin = [&](int kk, long& b, int& pos0) {
    const long t = (long)blockIdx.x + (long)kk * gridDim.x;
    b = t / tiles_per_image;
    pos0 = (int)(t - b * tiles_per_image) * TP;
  };

  if (warp == 0) {
    // ================= MMA issue ====================================================================
    const unsigned idesc32 = tc::idesc_tf32(kGtF, 32, 0, 0), idesc64 = tc::idesc_tf32(kGtF, 64, 0, 0);
    for (int k = 0; k < my_tiles; ++k) {
      const int s = k % kGtStages;
      const int grp = k / kFlushTiles, acc = grp & 1;
      const bool first = (k % kFlushTiles) == 0;
      CNN_PHASE(0);
      if (first) mbar_wait_bounded(&bars.acc_free[acc], ((unsigned)(grp >> 1) & 1u) ^ 1u, status, gave_up);
      CNN_PHASE(1);
      mbar_wait_bounded(&bars.full[s], (unsigned)(k / kGtStages) & 1u, status, gave_up);
      CNN_PHASE(2);
      __syncwarp();
      tc::fence_after_sync();
      const unsigned base = smem_u32(stage0 + s * kGtStageBytes);
      const unsigned d_acc = tmem_d + (unsigned)acc * kAccCols;
      unsigned accumulate = first ? 0u : 1u;
      // pass 0: high delta tile x (all im2col rows: 32, or 64 = [hi | lo]); pass 1 (three-pass mode): low delta
      // tile x hi taps, into the first 32 columns
#pragma unroll 1
      for (int pass = 0; pass < (PASSES == 3 ? 2 : 1); ++pass) {
        const unsigned a_s = base + ((pass == 1) ? kALoOff : 0u);
        const unsigned b_s = base + kBOff;
        const unsigned idesc = (PASSES == 3 && pass == 0) ? idesc64 : idesc32;
#pragma unroll
        for (int ks = 0; ks < TP / 8; ++ks) {          // 8 positions per MMA = two 16-byte chunks
          const unsigned long long ad = smem_desc_sw128(a_s + (unsigned)(ks >> 2) * kGtKBlock + (unsigned)(ks & 3) * 32u);
          const unsigned long long bd = tc::smem_desc(b_s + ks * 256, 128, kGroup);
          tc::mma_tf32_elect(d_acc, ad, bd, idesc, accumulate);
          accumulate = 1;
        }
      }
      tc::mma_commit_elect(&bars.free[s]);
      if ((k % kFlushTiles) == kFlushTiles - 1 || k == my_tiles - 1) tc::mma_commit_elect(&bars.acc_full[acc]);
      CNN_PHASE(3);
    }
  } else if (warp >= 4 && warp < 8) {
    // ================= accumulator flush and the CTA's partial ======================================
    float racc[32];
#pragma unroll
    for (int c = 0; c < 32; ++c) racc[c] = 0.f;
    const unsigned lane_base = tmem_d + ((unsigned)((warp & 3) * 32) << 16);
    for (int g = 0; g < n_groups; ++g) {
      const int acc = g & 1;
      CNN_PHASE(0);
      mbar_wait_bounded(&bars.acc_full[acc], (unsigned)(g >> 1) & 1u, status, gave_up);
      CNN_PHASE(1);
      tc::fence_after_sync();
#pragma unroll
      for (int c0 = 0; c0 < (int)kAccCols; c0 += 16) {     // columns 32..63 (three passes) hold hi*lo of the same taps
        float v[16];
        tc::tmem_ld16(lane_base + (unsigned)acc * kAccCols + (unsigned)c0, v);
#pragma unroll
        for (int e = 0; e < 16; ++e) racc[(c0 & 31) + e] += v[e];
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.acc_free[acc]);
      CNN_PHASE(2);
    }
    // M = 64: lanes 0..15 of quarter w hold maps 16 w + lane
    if (lane < 16) {
      float* dst = part + ((size_t)blockIdx.x * kGtF + 16 * (warp & 3) + lane) * 26;
#pragma unroll
      for (int c = 0; c < 26; ++c) dst[c] = racc[c];
    }
  } else if (warp >= 8 && warp < 8 + kGtDeltaWarps) {
    // ================= delta side: TMA producer (lane 0 of warp 8), activations -> deltas ============
    const int lw = warp - 8;
    const float inv_c = 1.0f / (float)CC, inv_s = 1.0f / (float)d.S;
    const int PP = d.P * d.P;
    float gs[17];
#pragma unroll
    for (int t = 0; t < 17; ++t) gs[t] = 0.f;
    constexpr int kMine = 2 * CH / kGtDeltaWarps;           // 8 or 4 items per warp and tile
    // The ds value and the window row of every item of a tile, fetched one tile ahead: ds comes from L2 or
    // DRAM (the activations stream through L2 and push it out), and a gather in the path of every tile
    // cost 4,000 cycles per tile.
    float dl[kMine], dl_next[kMine];
    int rr[kMine], rr_next[kMine];
    auto fetch_ds = [&](int kk, float (&out)[kMine], int (&rows)[kMine]) {
      long b;
      int pos0;
      tile_origin(kk, b, pos0);
      const int y0 = pos0 / d.C, x0 = pos0 - y0 * d.C;        // a tile spans at most TP / C + 1 rows
      const float* ds_b = ds + (size_t)b * d.S + lane * PP;
#pragma unroll
      for (int i = 0; i < kMine; ++i) {
        const int u = lw + kGtDeltaWarps * i;
        const int c = u >> 1;
        int x = x0 + 4 * c, y = y0;
#pragma unroll
        for (int w = 0; w < TP / 32 + 1; ++w)        // rows are at least 32 positions long (checked on the host)
          if (x >= d.C) { x -= d.C; ++y; }
        rows[i] = y & 3;
        out[i] = (pos0 + 4 * c < CC) ? __ldg(ds_b + (u & 1) * 32 * PP + (y >> 2) * d.P + (x >> 2)) : 0.f;
      }
    };
#pragma unroll
    for (int i = 0; i < kMine; ++i) { dl_next[i] = 0.f; rr_next[i] = 0; }
    if (my_tiles > 0) fetch_ds(0, dl_next, rr_next);
    for (int k = 0; k < my_tiles + kAhead; ++k) {
      CNN_PHASE(0);
      if (k >= kAhead) {
        const int kk = k - kAhead, s = kk % kGtStages;
#pragma unroll
        for (int i = 0; i < kMine; ++i) { dl[i] = dl_next[i]; rr[i] = rr_next[i]; }
        if (kk + 1 < my_tiles) fetch_ds(kk + 1, dl_next, rr_next);     // in flight while this tile lands and is turned
        mbar_wait_bounded(&bars.landed[s], (unsigned)(kk / kGtStages) & 1u, status, gave_up);
        CNN_PHASE(1);
        {
          // item u = (chunk c, half h): this lane owns map 32 h + lane, positions pos0 + 4 c .. + 3 (one row
          // of one window).  The piece sits at row * 128 + ((c % 8) ^ (row % 8)) * 16 of K-block c / 8.
          unsigned char* st = stage0 + s * kGtStageBytes;
          float4 v[kMine];
#pragma unroll
          for (int i = 0; i < kMine; ++i) {
            const int u = lw + kGtDeltaWarps * i;
            const int c = u >> 1, row = 32 * (u & 1) + lane;
            v[i] = *reinterpret_cast<const float4*>(st + (unsigned)(c >> 3) * kGtKBlock + (unsigned)row * 128u +
                                                    (unsigned)(((c & 7) ^ (row & 7)) * 16));
          }
#pragma unroll
          for (int i = 0; i < kMine; ++i) {
            const int u = lw + kGtDeltaWarps * i;
            const int c = u >> 1, row = 32 * (u & 1) + lane;
            unsigned char* p = st + (unsigned)(c >> 3) * kGtKBlock + (unsigned)row * 128u + (unsigned)(((c & 7) ^ (row & 7)) * 16);
            const int r = rr[i];                                    // window row: the same for the whole warp
            const float4 w4 = *reinterpret_cast<const float4*>(&bars.ws[4 * r]);
            const float dlt = dl[i];
            float4 dv;
            dv.x = (w4.x * dlt) * v[i].x * (1.f - v[i].x) * inv_c;
            dv.y = (w4.y * dlt) * v[i].y * (1.f - v[i].y) * inv_c;
            dv.z = (w4.z * dlt) * v[i].z * (1.f - v[i].z) * inv_c;
            dv.w = (w4.w * dlt) * v[i].w * (1.f - v[i].w) * inv_c;
            // subsample-filter gradient: taps of window row r; the bias term once per window (its first row)
            if (r == 0) {
              gs[0] = fmaf(dlt, v[i].x, gs[0]); gs[1] = fmaf(dlt, v[i].y, gs[1]);
              gs[2] = fmaf(dlt, v[i].z, gs[2]); gs[3] = fmaf(dlt, v[i].w, gs[3]);
              gs[16] += dlt * inv_s;
            } else if (r == 1) {
              gs[4] = fmaf(dlt, v[i].x, gs[4]); gs[5] = fmaf(dlt, v[i].y, gs[5]);
              gs[6] = fmaf(dlt, v[i].z, gs[6]); gs[7] = fmaf(dlt, v[i].w, gs[7]);
            } else if (r == 2) {
              gs[8] = fmaf(dlt, v[i].x, gs[8]); gs[9] = fmaf(dlt, v[i].y, gs[9]);
              gs[10] = fmaf(dlt, v[i].z, gs[10]); gs[11] = fmaf(dlt, v[i].w, gs[11]);
            } else {
              gs[12] = fmaf(dlt, v[i].x, gs[12]); gs[13] = fmaf(dlt, v[i].y, gs[13]);
              gs[14] = fmaf(dlt, v[i].z, gs[14]); gs[15] = fmaf(dlt, v[i].w, gs[15]);
            }
            if (PASSES == 3) {
              float4 hi, lo;
              tc::split_tf32(dv.x, hi.x, lo.x); tc::split_tf32(dv.y, hi.y, lo.y);
              tc::split_tf32(dv.z, hi.z, lo.z); tc::split_tf32(dv.w, hi.w, lo.w);
              *reinterpret_cast<float4*>(p) = hi;
              *reinterpret_cast<float4*>(p + kALoOff) = lo;
            } else {
              *reinterpret_cast<float4*>(p) = dv;
            }
          }
          tc::fence_async_smem();    // generic-proxy writes -> visible to the tensor core's operand reads
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.full[s]);
        CNN_PHASE(2);
      }
      if (k < my_tiles && warp == 8) {
        const int s = k % kGtStages;
        mbar_wait_bounded(&bars.free[s], ((unsigned)(k / kGtStages) & 1u) ^ 1u, status, gave_up);
        CNN_PHASE(3);
        if (lane == 0) {
          long b;
          int pos0;
          tile_origin(k, b, pos0);
          // the stage's previous readers were the tensor core (async proxy) and, in the three-pass mode,
          // generic-proxy splits that completed before its MMAs: nothing else to order here
          mbar_expect_tx(&bars.landed[s], kABytes);
#pragma unroll
          for (int kb = 0; kb < TP / 32; ++kb)
            tma_load_3d(stage0 + s * kGtStageBytes + kb * kGtKBlock, &ac_map, pos0 + 32 * kb, 0, (int)b, &bars.landed[s]);
        }
        __syncwarp();
      }
      CNN_PHASE(4);
    }
    // this warp's share of the subsample-filter gradient (fixed shuffle tree), then one row per warp
#pragma unroll
    for (int m = 16; m > 0; m >>= 1)
#pragma unroll
      for (int t = 0; t < 17; ++t) gs[t] += __shfl_xor_sync(0xffffffffu, gs[t], m);
    if (lane == 0) {
#pragma unroll
      for (int t = 0; t < 17; ++t) bars.red[lw][t] = gs[t];
    }
  } else {
    // ================= im2colT side: warps 1-3 =======================================================
    const int lw = warp - 1;
    // lane = (tap within its group of 8) + 8 * (chunk within its quad)
    const int HH = d.H * d.H;
    int tap_off[4];
    bool tap_live[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int t = 8 * g + (lane & 7);
      tap_live[g] = t < 25;
      const int ti = t / 5, tj = t % 5;
      tap_off[g] = tap_live[g] ? (tj & 3) * HH + ti * d.H + 4 * (tj >> 2) : 0;   // copy shifted by j % 4, row + i, column + 4 (j / 4)
    }
    constexpr int kBAhead = kGtStages - 2;
    constexpr int kQuads = CH / 4;                     // chunk quads of a tile; warp lw takes quads lw, lw + 3, ...
    constexpr int kMine = (kQuads + kGtIm2colWarps - 1) / kGtIm2colWarps;
    for (int k = 0; k < my_tiles + kBAhead; ++k) {
      CNN_PHASE(0);
      if (k >= kBAhead) {
        const int kk = k - kBAhead, s = kk % kGtStages;
        cp_async_wait<kBAhead - 1>();
        CNN_PHASE(1);
        if (PASSES == 3) {
          // split what this lane copied, in place: the high part stays, the remainder goes to the low tile
          unsigned char* st = stage0 + s * kGtStageBytes + kBOff;
          long b;
          int pos0;
          tile_origin(kk, b, pos0);
          float4 v[kMine][4];
#pragma unroll
          for (int q = 0; q < kMine; ++q)
#pragma unroll
            for (int g = 0; g < 4; ++g)
              v[q][g] = *reinterpret_cast<const float4*>(st + g * kGroup + (unsigned)(4 * (lw + kGtIm2colWarps * q) + (lane >> 3)) * 128u +
                                                         (unsigned)(lane & 7) * 16u);
#pragma unroll
          for (int q = 0; q < kMine; ++q) {
            const int c = 4 * (lw + kGtIm2colWarps * q) + (lane >> 3);
            if (lw + kGtIm2colWarps * q < kQuads && pos0 + 4 * c < CC) {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                if (tap_live[g]) {
                  unsigned char* p = st + g * kGroup + (unsigned)c * 128u + (unsigned)(lane & 7) * 16u;
                  float4 hi, lo;
                  tc::split_tf32(v[q][g].x, hi.x, lo.x); tc::split_tf32(v[q][g].y, hi.y, lo.y);
                  tc::split_tf32(v[q][g].z, hi.z, lo.z); tc::split_tf32(v[q][g].w, hi.w, lo.w);
                  *reinterpret_cast<float4*>(p) = hi;
                  *reinterpret_cast<float4*>(p + kBLoOff) = lo;
                }
              }
            }
          }
        }
        tc::fence_async_smem();    // generic-proxy writes -> visible to the tensor core's operand reads
        __syncwarp();              // ... every lane's, before the warp's one arrival
        if (lane == 0) mbar_arrive(&bars.full[s]);
        CNN_PHASE(2);
      }
      if (k < my_tiles) {
        const int s = k % kGtStages;
        mbar_wait_bounded(&bars.free[s], ((unsigned)(k / kGtStages) & 1u) ^ 1u, status, gave_up);
        CNN_PHASE(3);
        unsigned char* st = stage0 + s * kGtStageBytes + kBOff;
        long b;
        int pos0;
        tile_origin(k, b, pos0);
        const float* img = shifted + (size_t)b * 4 * HH;
        // Chunks past the image keep what the stage held (finite; their dc is zero).
#pragma unroll
        for (int q = 0; q < kMine; ++q) {
          const int c = 4 * (lw + kGtIm2colWarps * q) + (lane >> 3);
          const int pos = pos0 + 4 * c;
          if (lw + kGtIm2colWarps * q < kQuads && pos < CC) {
            const int y = pos / d.C, x = pos - y * d.C;
            const float* src = img + y * d.H + x;
            unsigned char* dst = st + (unsigned)c * 128u + (unsigned)(lane & 7) * 16u;
#pragma unroll
            for (int g = 0; g < 4; ++g)
              if (tap_live[g]) cp_async16(dst + g * kGroup, src + tap_off[g]);
          }
        }
      }
      cp_async_commit();       // (an empty group past the last tile keeps the count uniform)
      CNN_PHASE(4);
    }
  }

  CNN_PHASE_END(g_phase_clocks_wg);
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_d, 2 * kAccCols);
  if (tid < 17) {
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kGtDeltaWarps; ++w) sum += bars.red[w][tid];
    part_s[(size_t)blockIdx.x * 17 + tid] = sum;
  }
}

// shifted[b][s][y][x] = image[b][y][x + s] (zero past the row's end), s = 0..3.  One thread per four
// consecutive output columns.
__global__ void __launch_bounds__(256)
k_wide_shift_images(int H, const float* __restrict__ images, long n, float* __restrict__ shifted) {
  const int q = H >> 2;                                   // float4 groups per row
  const long total = n * 4 * H * q;
  const long o = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= total) return;
  const int x = 4 * (int)(o % q);
  const long r = o / q;                                   // (b * 4 + s) * H + y
  const int y = (int)(r % H);
  const long bs = r / H;
  const int s = (int)(bs & 3);
  const float* src = images + ((bs >> 2) * H + y) * H;
  float4 v;
  v.x = (x + s < H) ? src[x + s] : 0.f;
  v.y = (x + 1 + s < H) ? src[x + 1 + s] : 0.f;
  v.z = (x + 2 + s < H) ? src[x + 2 + s] : 0.f;
  v.w = (x + 3 + s < H) ? src[x + 3 + s] : 0.f;
  reinterpret_cast<float4*>(shifted)[o] = v;
}

// The tensor map over the conv activations [cap images][F maps][CC positions] as (position, map, image);
// box = 32 positions x 64 maps with the 128-byte swizzle = one K-block of the delta operand.
static int encode_ac_map(cnn_wide* w) {
  if (w->ac_map_ptr == w->ac && w->ac_map_cap == w->cap) return CNN_OK;
  typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static encode_fn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    CNN_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || !fn) {
      set_error("cuTensorMapEncodeTiled is not available from this driver");
      return CNN_ERR_CUDA;
    }
    encode = reinterpret_cast<encode_fn>(fn);
  }
  const WideDims& d = w->d;
  const cuuint64_t CC = (cuuint64_t)d.C * d.C;
  const cuuint64_t dims[3] = {CC, (cuuint64_t)kGtF, (cuuint64_t)w->cap};
  const cuuint64_t strides[2] = {CC * 4, (cuuint64_t)kGtF * CC * 4};     // bytes, for dimensions 1 and 2
  const cuuint32_t box[3] = {32, (cuuint32_t)kGtF, 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  CUresult r = encode(reinterpret_cast<CUtensorMap*>(w->ac_map), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, w->ac, dims, strides,
                      box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with %d", (int)r);
    return CNN_ERR_CUDA;
  }
  w->ac_map_ptr = w->ac;
  w->ac_map_cap = w->cap;
  return CNN_OK;
}

bool wide_grad_tc_supported(const WideDims& d) { return d.F == kGtF && d.C % 4 == 0 && d.H % 4 == 0 && d.C >= 32; }

int wide_grad_c1_tc(cnn_wide* w, const float* d_images, long n, int* rows_out, cudaStream_t st) {
  const WideDims& d = w->d;
  const size_t smem = (size_t)kGtRingBytes + sizeof(GtBarriers) + 1024;
  const bool three = (w->conv_mode == 2);
  // Positions per tile: 128 with one pass, 64 with three (48 KB stages, four of them, either way).  Half-size
  // tiles in twice as many stages were measured slower (1.00 against 0.94 ms and 1.28 against 1.06 ms per step).
  const int tp = three ? 64 : 128;
  const long n_tiles = n * ((d.C * d.C + tp - 1) / tp);
  long grid = sm_count();
  if (grid > n_tiles) grid = n_tiles;
  if (grid > w->part_rows) grid = w->part_rows;
  int rc = encode_ac_map(w);
  if (rc != CNN_OK) return rc;
  const CUtensorMap& map = *reinterpret_cast<const CUtensorMap*>(w->ac_map);
  k_wide_shift_images<<<(unsigned)((n * d.H * d.H + 255) / 256), 256, 0, st>>>(d.H, d_images, n, w->img_shift);
#define CNN_LAUNCH_PIPE(TPV, PV)                                                                                     \
  do {                                                                                                               \
    CNN_CUDA(cudaFuncSetAttribute(k_wide_grad_c1_pipe<TPV, PV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    k_wide_grad_c1_pipe<TPV, PV><<<(unsigned)grid, kGtThreads, smem, st>>>(d, map, w->img_shift, w->ds, w->d_params, n, \
                                                                          w->part_c, w->part_s, w->d_status);        \
  } while (0)
  if (three) CNN_LAUNCH_PIPE(64, 3);
  else CNN_LAUNCH_PIPE(128, 1);
#undef CNN_LAUNCH_PIPE
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "k_wide_grad_c1_pipe launch");
  *rows_out = (int)grid;
  return CNN_OK;
}

}  // namespace cnn

#ifdef CNN_PHASE_CLOCKS
// Sums of the SM clock at each stamp for the 16 warps of CTA 0 of the last launch (tuning builds only).
extern "C" int cnn_debug_phase_clocks_wg(long long* out /* [16][16] */) {
  return cudaMemcpyFromSymbol(out, cnn::g_phase_clocks_wg, sizeof(cnn::g_phase_clocks_wg)) == cudaSuccess ? 0 : 2;
}
#endif
