// Fused batched forward, experimental variants (selectable with the "fw_variant" option; the default
// is the scalar kernel of fused_forward.cu, which measured faster): packed-FMA version and a scalar
// version with constant-bank weights.
//
// Same fusion and data movement as fused_forward.cu (bulk-copied image tiles in shared memory, one
// thread per 4x4 subsample window, nothing but 44 B of results per image written back), with three
// changes that cut issue slots, which is what bounds this kernel (58 FLOP/B: the fp32 FMA pipe
// and the special-function pipe are the limits, not HBM):
//   * the conv runs mostly on packed fp32 FMAs (fma.rn.f32x2 through __ffma2_rn): an accumulator
//     pair is two x-adjacent outputs, the input operand is an ALIGNED register pair
//     (p[r][c], p[r][c+1]), c even, exactly as the 128-bit shared loads deliver it, and the weight
//     operand is the pair (w, w) read as one 64-bit broadcast load.  Even filter columns pair
//     outputs (0,1) and (2,3); odd filter columns pair outputs (1,2) and finish outputs 0 and 3 with
//     scalar FMAs, so no shifted copy of the patch is needed (it would not fit in 128 registers);
//   * no __syncthreads in the tile loop: the image stages and the FC partial sums are handed over
//     through mbarriers (full/empty pairs), so a warp never waits for the slowest warp of the block;
//   * 256-thread blocks (7 images, 252 live threads) at two blocks per SM: 16 warps per SM is four
//     per scheduler, which is what lets each thread have 128 registers.
#include "net.cuh"

namespace cnn {

constexpr int kXImgs = 7;                 // images per tile
constexpr int kXThreads = 256;            // 8 warps, 252 live threads
constexpr int kXWarps = kXThreads / 32;
constexpr int kXStages = 2;
constexpr int kXPartStride = 37;
constexpr int kXFinalizers = 3;           // warps 0..2 finish 3 + 3 + 1 images

struct XSmem {
  float img[kXStages][kXImgs][kImg];      // bulk-copy destinations (16-byte aligned, 21,952 B each)
  float2 wc2[kF][26];                     // (w, w) per tap
  float bc[8];
  float2 ws2[8];                          // natural pairs (ws[i][2j], ws[i][2j+1])
  float bs[4];
  float2 wf2[kOut / 2][kS];               // (wf[2kp][s], wf[2kp+1][s])
  float bf[12];
  float part[2][kXImgs][kOut][kXPartStride];
  unsigned long long full[kXStages];      // image stage filled (tx bytes)
  unsigned long long empty[kXStages];     // every warp has taken its patches
  unsigned long long parts_full[2];       // every warp has stored its partial sums
  unsigned long long parts_empty[2];      // the finalizer warps have consumed them
};

// Conv / subsample parameters in the constant bank (scalar kernel variant): an FFMA can take its
// weight operand straight from there, so the weights cost neither registers nor load instructions.
// Slots are filled by a stream-ordered device-to-device copy from the net's arena before a launch
// whenever the net's parameter version differs from what the slot holds.
struct ConvConsts {
  float wc[kF * 25];
  float bc[kF];
  float ws[16];
  float bs;
  float pad;
};
static_assert(sizeof(ConvConsts) == sizeof(float) * 174, "ConvConsts mirrors arena floats 0..172 + pad");
constexpr int kConstSlots = 8;
__constant__ ConvConsts c_conv[kConstSlots];

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <int FLAVOR>
__device__ __forceinline__ void finalize_tile(XSmem& sm, int buf, long first, int imgs_here, int warp,
                                              int lane, float* __restrict__ out, int* __restrict__ argmax) {
  const int li = lane / 10, k = lane % 10;
  const int im = warp * 3 + li;
  const bool valid = (lane < 30) && (im < imgs_here);
  float z = 0.f;
  if (valid) {
#pragma unroll 4
    for (int ww = 0; ww < 36; ++ww) z += sm.part[buf][im][k][ww];
    z += sm.bf[k];
  }
  const float o = sigmoidf<FLAVOR>(z);
  // classify(): strict '<' scan from index 0, so the lowest index wins ties.
  float bv = __shfl_sync(0xffffffffu, o, li * 10);
  int best = 0;
#pragma unroll
  for (int kk = 1; kk < kOut; ++kk) {
    const float v = __shfl_sync(0xffffffffu, o, li * 10 + kk);
    if (bv < v) { bv = v; best = kk; }
  }
  if (valid) {
    const long gi = first + im;
    if (out) out[gi * kOut + k] = o;
    if (argmax && k == 0) argmax[gi] = best;
  }
}

template <int FLAVOR, bool PACKED>
__global__ void __launch_bounds__(kXThreads, 2)
k_fused_forward_x2(const float* __restrict__ images, long n, const float* __restrict__ params,
                   float* __restrict__ out, int* __restrict__ argmax, int* __restrict__ status, int slot) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  XSmem& sm = *reinterpret_cast<XSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long n_tiles = (n + kXImgs - 1) / kXImgs;

  for (int i = tid; i < kF * 26; i += kXThreads) {
    const int f = i / 26, t = i % 26;
    const float w = (t < 25) ? params[kOffWc + f * 25 + t] : 0.f;
    sm.wc2[f][t] = make_float2(w, w);
  }
  if (tid < kF) sm.bc[tid] = params[kOffBc + tid];
  if (tid < 8) sm.ws2[tid] = make_float2(params[kOffWs + 2 * tid], params[kOffWs + 2 * tid + 1]);
  if (tid == 0) sm.bs[0] = params[kOffBs];
  for (int i = tid; i < (kOut / 2) * kS; i += kXThreads) {
    const int kp = i / kS, s = i % kS;
    sm.wf2[kp][s] = make_float2(params[kOffWf + (2 * kp) * kS + s], params[kOffWf + (2 * kp + 1) * kS + s]);
  }
  if (tid < kOut) sm.bf[tid] = params[kOffBf + tid];
  if (tid == 0) {
    for (int s = 0; s < kXStages; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], kXWarps);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.parts_full[b], kXWarps);
      mbar_init(&sm.parts_empty[b], kXFinalizers);
    }
    mbar_fence_init();
  }
  __syncthreads();

  auto issue = [&](int stage, long tile) {
    const long first = tile * kXImgs;
    const long left = n - first;
    const unsigned cnt = (unsigned)(left < kXImgs ? left : kXImgs);
    const unsigned bytes = cnt * (unsigned)(kImg * sizeof(float));
    mbar_expect_tx(&sm.full[stage], bytes);
    bulk_g2s(&sm.img[stage][0][0], images + first * kImg, bytes, &sm.full[stage]);
  };
  if (tid == 0) {
    for (int s = 0; s < kXStages; ++s) {
      const long t = (long)blockIdx.x + (long)s * gridDim.x;
      if (t < n_tiles) issue(s, t);
    }
  }

  const int img = tid / 36, w = tid % 36;   // threads 252..255: img == 7, never live
  const int p = w / 6, q = w % 6;
  bool gave_up = false;

  int it = 0;
  long prev_first = 0;
  int prev_imgs = 0;
  for (long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
    const int stage = it & 1, buf = it & 1;
    const unsigned par = (unsigned)(it >> 1) & 1u;
    mbar_wait_bounded(&sm.full[stage], par, status, gave_up);

    const long first = tile * kXImgs;
    const int imgs_here = (int)((n - first) < kXImgs ? (n - first) : kXImgs);
    const bool live = img < imgs_here;

    // Patch rows 4p..4p+7, columns 4q..4q+7 as the aligned register pairs E[r][c/2] = (p[r][c], p[r][c+1]).
    float2 E[8][4];
    if (live) {
      const float* base = &sm.img[stage][img][(4 * p) * kH + 4 * q];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float4 lo = *reinterpret_cast<const float4*>(base + r * kH);
        const float4 hi = *reinterpret_cast<const float4*>(base + r * kH + 4);
        E[r][0] = make_float2(lo.x, lo.y); E[r][1] = make_float2(lo.z, lo.w);
        E[r][2] = make_float2(hi.x, hi.y); E[r][3] = make_float2(hi.z, hi.w);
      }
    } else {
#pragma unroll
      for (int r = 0; r < 8; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) E[r][c] = make_float2(0.f, 0.f);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm.empty[stage]);

    float2 part2[kOut / 2];
#pragma unroll
    for (int k = 0; k < kOut / 2; ++k) part2[k] = make_float2(0.f, 0.f);

#pragma unroll 1
    for (int f = 0; f < kF; ++f) {
      float2 acc[4][2];
      if constexpr (PACKED) {
      // Even taps (j = 0, 2, 4): outputs (0,1) and (2,3) pair with the aligned inputs.  Odd taps
        // (j = 1, 3): outputs (1,2) pair with an aligned input; outputs 0 and 3 take scalar FMAs.
        float2 e01[4], e23[4], o12[4];
        float o0[4], o3[4];
#pragma unroll
        for (int y = 0; y < 4; ++y) {
          e01[y] = e23[y] = o12[y] = make_float2(0.f, 0.f);
          o0[y] = o3[y] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 5; ++j)
#pragma unroll
          for (int i = 0; i < 5; ++i) {
            const float2 w2 = sm.wc2[f][i * 5 + j];
#pragma unroll
            for (int y = 0; y < 4; ++y) {
              if ((j & 1) == 0) {
                e01[y] = __ffma2_rn(w2, E[y + i][j >> 1], e01[y]);
                e23[y] = __ffma2_rn(w2, E[y + i][(j >> 1) + 1], e23[y]);
              } else {
                o12[y] = __ffma2_rn(w2, E[y + i][(j + 1) >> 1], o12[y]);
                o0[y] = fmaf(w2.x, E[y + i][(j - 1) >> 1].y, o0[y]);
                o3[y] = fmaf(w2.x, E[y + i][(j + 3) >> 1].x, o3[y]);
              }
            }
          }
#pragma unroll
        for (int y = 0; y < 4; ++y) {
          acc[y][0] = make_float2(e01[y].x + o0[y], e01[y].y + o12[y].x);
          acc[y][1] = make_float2(e23[y].x + o12[y].y, e23[y].y + o3[y]);
        }
      } else {
        // Scalar FMAs with the weight as a constant-bank operand.
        const ConvConsts& cw = c_conv[slot];
#pragma unroll
        for (int y = 0; y < 4; ++y) acc[y][0] = acc[y][1] = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 5; ++j)
#pragma unroll
          for (int i = 0; i < 5; ++i) {
            const float wv = cw.wc[f * 25 + i * 5 + j];
#pragma unroll
            for (int y = 0; y < 4; ++y)
#pragma unroll
              for (int x = 0; x < 4; ++x) {
                const int c = x + j;
                const float in = (c & 1) ? E[y + i][c >> 1].y : E[y + i][c >> 1].x;
                float& dst = (x & 1) ? acc[y][x >> 1].y : acc[y][x >> 1].x;
                dst = fmaf(wv, in, dst);
              }
          }
      }
      const float b = sm.bc[f];
      float2 zs2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int y = 0; y < 4; ++y)
#pragma unroll
        for (int xp = 0; xp < 2; ++xp) {
          float2 a;
          a.x = sigmoidf<FLAVOR>(acc[y][xp].x + b);
          a.y = sigmoidf<FLAVOR>(acc[y][xp].y + b);
          zs2 = __ffma2_rn(sm.ws2[y * 2 + xp], a, zs2);
        }
      const float as = sigmoidf<FLAVOR>((zs2.x + zs2.y) + sm.bs[0]);
      const float2 as2 = make_float2(as, as);
#pragma unroll
      for (int k = 0; k < kOut / 2; ++k) part2[k] = __ffma2_rn(sm.wf2[k][f * 36 + w], as2, part2[k]);
    }

    // Producer: refill this stage for the tile after next once every warp has taken its patches.
    if (tid == 0) {
      const long t2 = tile + (long)kXStages * gridDim.x;
      if (t2 < n_tiles) {
        mbar_wait_bounded(&sm.empty[stage], par, status, gave_up);
        issue(stage, t2);
      }
    }
    // Finalizers: finish the previous tile (its partial sums were completed a whole tile ago).
    if (warp < kXFinalizers && it > 0) {
      const int pb = buf ^ 1;
      mbar_wait_bounded(&sm.parts_full[pb], (unsigned)((it - 1) >> 1) & 1u, status, gave_up);
      finalize_tile<FLAVOR>(sm, pb, prev_first, prev_imgs, warp, lane, out, argmax);
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.parts_empty[pb]);
    }
    // Store this tile's partial sums once the finalizers are done with the buffer (tile it-2).
    if (it >= 2) mbar_wait_bounded(&sm.parts_empty[buf], (unsigned)((it - 2) >> 1) & 1u, status, gave_up);
    if (live) {
#pragma unroll
      for (int k = 0; k < kOut / 2; ++k) {
        sm.part[buf][img][2 * k][w] = part2[k].x;
        sm.part[buf][img][2 * k + 1][w] = part2[k].y;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm.parts_full[buf]);
    prev_first = first;
    prev_imgs = imgs_here;
  }
  // drain: the last tile of this block
  if (warp < kXFinalizers && it > 0) {
    const int pb = (it - 1) & 1;
    mbar_wait_bounded(&sm.parts_full[pb], (unsigned)((it - 1) >> 1) & 1u, status, gave_up);
    finalize_tile<FLAVOR>(sm, pb, prev_first, prev_imgs, warp, lane, out, argmax);
  }
}

template <int FLAVOR, bool PACKED>
static int launch_x2_flavor(cnn_net* net, const float* d_images, long n, float* d_out, int* d_argmax,
                            cudaStream_t stream) {
  const long n_tiles = (n + kXImgs - 1) / kXImgs;
  const long max_blocks = 2L * sm_count();
  const int grid = (int)(n_tiles < max_blocks ? n_tiles : max_blocks);
  const size_t smem = sizeof(XSmem);
  CNN_CUDA(cudaFuncSetAttribute(k_fused_forward_x2<FLAVOR, PACKED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)smem));
  int slot = 0;
  if (!PACKED) {
    // One slot per net (round-robin over kConstSlots); refreshed when the parameters have changed.
    static int slot_owner[kConstSlots] = {0};
    static long slot_version[kConstSlots] = {0};
    slot = net->const_slot;
    if (slot_owner[slot] != net->id || slot_version[slot] != net->params_version) {
      CNN_CUDA(cudaMemcpyToSymbolAsync(c_conv, net->d_params, sizeof(ConvConsts), sizeof(ConvConsts) * slot,
                                       cudaMemcpyDeviceToDevice, stream));
      slot_owner[slot] = net->id;
      slot_version[slot] = net->params_version;
    }
  }
  k_fused_forward_x2<FLAVOR, PACKED><<<grid, kXThreads, smem, stream>>>(d_images, n, net->d_params, d_out,
                                                                      d_argmax, net->d_status, slot);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "k_fused_forward_x2 launch");
  return CNN_OK;
}

int launch_forward_x2(cnn_net* net, const float* d_images, long n, float* d_out, int* d_argmax,
                      cudaStream_t stream) {
  const bool packed = net->fw_variant != 3;
  switch (net->fast_sigmoid) {
    case 1: return packed ? launch_x2_flavor<1, true>(net, d_images, n, d_out, d_argmax, stream)
                          : launch_x2_flavor<1, false>(net, d_images, n, d_out, d_argmax, stream);
    case 2: return packed ? launch_x2_flavor<2, true>(net, d_images, n, d_out, d_argmax, stream)
                          : launch_x2_flavor<2, false>(net, d_images, n, d_out, d_argmax, stream);
    default: return packed ? launch_x2_flavor<0, true>(net, d_images, n, d_out, d_argmax, stream)
                           : launch_x2_flavor<0, false>(net, d_images, n, d_out, d_argmax, stream);
  }
}

}  // namespace cnn
