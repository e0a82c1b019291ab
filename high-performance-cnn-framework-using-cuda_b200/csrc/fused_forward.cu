// Fused batched forward: conv 6x5x5 + bias + sigmoid, shared 4x4/stride-4 subsample + bias +
// sigmoid, FC 216->10 + bias + sigmoid and argmax in ONE kernel.  Replaces, for n images at once,
// the reference's forward_pass launch sequence (main.cu:67-88: 8 memsets, one H2D copy and nine
// <<<64,64>>> launches per image) and classify's D2H + host argmax (main.cu:181-189).
//
// Data movement: images are contiguous 3,136-byte records, so a tile of 7 images is one 22 KB
// 1-D bulk copy (cp.async.bulk, no multicast) into shared memory, double-buffered behind
// mbarriers; the only other HBM traffic is the 44 bytes of results per image.
//
// Work decomposition: one thread owns one 4x4 subsample window (36 per image) for all six maps.
// It keeps its 8x8 input patch in registers, so the 96 conv outputs, their sigmoids and the six
// subsample outputs of the window never touch memory; only the 10 partial FC sums per window go
// through shared memory, where 30 lanes per warp finish them and take the argmax by shuffles.
#include "net.cuh"

namespace cnn {

// Seven images per tile: 252 of a block's 256 threads own a window, and two 8-warp blocks per SM may use
// 128 registers per thread.  (Eight images = 288 threads are allocated as ten warps, which caps two
// blocks per SM at 96 registers: 0.387 ms per 65,536 images against 0.333 ms with this shape, 0.321 ms
// with the sigmoid's factor folded into the conv weights.)
constexpr int kFwImgs = 7;                                    // images per tile
constexpr int kFwThreads = (kFwImgs * 36 + 31) / 32 * 32;    // 256 = 8 warps
constexpr int kFwStages = 2;
constexpr int kPartStride = 37;             // 36 windows + 1 pad: conflict-free column reads

struct FwSmem {
  float img[kFwStages][kFwImgs][kImg];      // 2 x 21,952 B, filled by bulk copies
  float wc[kF][28];                         // 25 taps padded to 28 for 128-bit loads
  float bc[8];
  float ws[16];
  float bs[4];
  float wf[kOut][kS];                       // [k][f*36 + window]
  float bf[12];
  float part[kFwImgs][kOut][kPartStride];
  float lut[256];                           // uint8 pixel -> float(pixel / 255.0), uint8 input only
  unsigned long long full[kFwStages];
};

// U8 = false: images are fp32 [n][28][28].  U8 = true: `images` points at uint8 pixels [n][28][28]
// (the storage of the IDX files the reference reads) and the kernel applies the reference's ingest,
// float(pixel / 255.0) (mnist.h:145 then main.cu:57-65), through a 256-entry table.
template <int FAST, int MINB, bool U8, int UNROLL>
__global__ void __launch_bounds__(kFwThreads, MINB)
k_fused_forward(const float* __restrict__ images, long n, const float* __restrict__ params,
                float* __restrict__ out, int* __restrict__ argmax, int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  FwSmem& sm = *reinterpret_cast<FwSmem*>(smem_raw);
  const int tid = threadIdx.x;
  const long n_tiles = (n + kFwImgs - 1) / kFwImgs;
  // With the short sigmoid form its multiplication by -log2(e) is folded into the conv weights and bias.
  constexpr float kPre = (FAST == 1) ? -1.4426950408889634f : 1.0f;

  // Parameters: 9.4 KB from global (L2-resident after the first block) into shared memory.
  for (int i = tid; i < kF * 28; i += kFwThreads) {
    const int f = i / 28, t = i % 28;
    sm.wc[f][t] = (t < 25) ? kPre * params[kOffWc + f * 25 + t] : 0.f;
  }
  if (tid < kF) sm.bc[tid] = kPre * params[kOffBc + tid];
  if (tid < 16) sm.ws[tid] = params[kOffWs + tid];
  if (tid == 0) sm.bs[0] = params[kOffBs];
  for (int i = tid; i < kOut * kS; i += kFwThreads) sm.wf[i / kS][i % kS] = params[kOffWf + i];
  if (tid < kOut) sm.bf[tid] = params[kOffBf + tid];
  if (U8 && tid < 256) sm.lut[tid] = (float)((double)tid / 255.0);

  if (tid == 0) {
    for (int s = 0; s < kFwStages; ++s) mbar_init(&sm.full[s], 1);
    mbar_fence_init();
  }
  __syncthreads();

  auto issue = [&](int stage, long tile) {
    const long first = tile * kFwImgs;
    const long left = n - first;
    const unsigned cnt = (unsigned)(left < kFwImgs ? left : kFwImgs);
    constexpr unsigned kPixelBytes = U8 ? 1u : (unsigned)sizeof(float);
    const unsigned bytes = cnt * (unsigned)kImg * kPixelBytes;
    const unsigned char* src = reinterpret_cast<const unsigned char*>(images) + (size_t)first * kImg * kPixelBytes;
    mbar_expect_tx(&sm.full[stage], bytes);
    bulk_g2s(&sm.img[stage][0][0], src, bytes, &sm.full[stage]);
  };

  if (tid == 0) {
    for (int s = 0; s < kFwStages; ++s) {
      const long t = (long)blockIdx.x + (long)s * gridDim.x;
      if (t < n_tiles) issue(s, t);
    }
  }

  const int img = tid / 36, w = tid % 36;
  const int p = w / 6, q = w % 6;
  const int warp = tid >> 5, lane = tid & 31;
  bool gave_up = false;

  int it = 0;
  for (long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
    const int stage = it % kFwStages;
    const unsigned parity = (unsigned)(it / kFwStages) & 1u;
    mbar_wait_bounded(&sm.full[stage], parity, status, gave_up);

    const long first = tile * kFwImgs;
    const int imgs_here = (int)((n - first) < kFwImgs ? (n - first) : kFwImgs);
    const bool live = img < imgs_here;

    // 8x8 input patch of this thread's window: rows 4p..4p+7, columns 4q..4q+7.
    float patch[8][8];
    if (live && U8) {
      const unsigned char* bytes0 = reinterpret_cast<const unsigned char*>(&sm.img[stage][0][0]);
      const unsigned char* base = bytes0 + img * kImg + (4 * p) * kH + 4 * q;  // 4-byte aligned
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const unsigned lo = *reinterpret_cast<const unsigned*>(base + r * kH);
        const unsigned hi = *reinterpret_cast<const unsigned*>(base + r * kH + 4);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          patch[r][c] = sm.lut[(lo >> (8 * c)) & 0xFFu];
          patch[r][4 + c] = sm.lut[(hi >> (8 * c)) & 0xFFu];
        }
      }
    } else if (live) {
      const float* base = &sm.img[stage][img][(4 * p) * kH + 4 * q];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float4 lo = *reinterpret_cast<const float4*>(base + r * kH);
        const float4 hi = *reinterpret_cast<const float4*>(base + r * kH + 4);
        patch[r][0] = lo.x; patch[r][1] = lo.y; patch[r][2] = lo.z; patch[r][3] = lo.w;
        patch[r][4] = hi.x; patch[r][5] = hi.y; patch[r][6] = hi.z; patch[r][7] = hi.w;
      }
    } else {
#pragma unroll
      for (int r = 0; r < 8; ++r)
#pragma unroll
        for (int c = 0; c < 8; ++c) patch[r][c] = 0.f;
    }
    __syncthreads();  // every thread has taken its patch: the stage may be refilled
    if (tid == 0) {
      const long t2 = tile + (long)kFwStages * gridDim.x;
      if (t2 < n_tiles) issue(stage, t2);
    }

    float part[kOut];
#pragma unroll
    for (int k = 0; k < kOut; ++k) part[k] = 0.f;

#pragma unroll UNROLL
    for (int f = 0; f < kF; ++f) {
      float wr[28];
#pragma unroll
      for (int t = 0; t < 7; ++t) {
        const float4 v = *reinterpret_cast<const float4*>(&sm.wc[f][4 * t]);
        wr[4 * t] = v.x; wr[4 * t + 1] = v.y; wr[4 * t + 2] = v.z; wr[4 * t + 3] = v.w;
      }
      const float b = sm.bc[f];
      float a[4][4];
#pragma unroll
      for (int y = 0; y < 4; ++y)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          float acc = 0.f;
#pragma unroll
          for (int j = 0; j < 5; ++j)
#pragma unroll
            for (int i = 0; i < 5; ++i) acc = fmaf(wr[i * 5 + j], patch[y + i][x + j], acc);
          if (FAST == 1) {
            // conv weights and bias carry the short form's factor -log2(e): the activation is 1 / (1 + 2^t)
            const float dd = 1.0f + exp2f_approx(acc + b);
            float qq;
            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(qq) : "f"(dd));
            a[y][x] = qq;
          } else {
            a[y][x] = sigmoidf<FAST>(acc + b);
          }
        }
      float zs = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) zs = fmaf(sm.ws[i * 4 + j], a[i][j], zs);
      const float as = sigmoidf<FAST>(zs + sm.bs[0]);
#pragma unroll
      for (int k = 0; k < kOut; ++k) part[k] = fmaf(sm.wf[k][f * 36 + w], as, part[k]);
    }

    if (live) {
#pragma unroll
      for (int k = 0; k < kOut; ++k) sm.part[img][k][w] = part[k];
    }
    __syncthreads();

    // Three images per warp on lanes 0..29: lane = 10*local_image + k.
    if (warp < (kFwImgs + 2) / 3) {
      const int li = lane / 10, k = lane % 10;
      const int im = warp * 3 + li;
      const bool valid = (lane < 30) && (im < imgs_here);
      float z = 0.f;
      if (valid) {
#pragma unroll 4
        for (int ww = 0; ww < 36; ++ww) z += sm.part[im][k][ww];
        z += sm.bf[k];
      }
      const float o = sigmoidf<FAST>(z);
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
  }
}

template <int FAST, bool U8, int UNROLL>
static int launch_variant(cnn_net* net, const void* d_images, long n, float* d_out, int* d_argmax,
                          cudaStream_t stream) {
  constexpr int kMinBlocks = 2;   // two 8-warp blocks per SM: 128 registers per thread
  const long n_tiles = (n + kFwImgs - 1) / kFwImgs;
  const long max_blocks = (long)kMinBlocks * sm_count();
  const int grid = (int)(n_tiles < max_blocks ? n_tiles : max_blocks);
  const size_t smem = sizeof(FwSmem);
  CNN_CUDA(cudaFuncSetAttribute(k_fused_forward<FAST, kMinBlocks, U8, UNROLL>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  k_fused_forward<FAST, kMinBlocks, U8, UNROLL><<<grid, kFwThreads, smem, stream>>>(
      static_cast<const float*>(d_images), n, net->d_params, d_out, d_argmax, net->d_status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "k_fused_forward launch");
  return CNN_OK;
}

// fast_sigmoid set (the default): the short sigmoid form, 0.321 ms per 65,536 images; over that batch it
// is as close to the fp64 oracle as the reference expression (2.1e-6; the fp32 oracle itself is 4.0e-6 away).
// The kernel a call over n_total images uses (0 = this file's, 1 / 2 = forward_tc.cu).  Default (-1): the
// three-pass tensor-core kernel from the batch size at which it overtakes this one (measured on a B200:
// 22 us for anything up to 2,368 images against 10-20 us here, 41 against 47 us at 8,192 images, 203 against
// 333 us at 65,536).  Both keep the 1e-5 parity bar.  With the reference's sigmoid expression asked for
// (fast_sigmoid = 0) the default stays on this kernel.
int forward_kernel_for(const cnn_net* net, long n_total) {
  constexpr long kTcMinBatch = 6144;
  if (net->forward_path >= 0) return net->forward_path;
  return (net->fast_sigmoid && n_total >= kTcMinBatch) ? 1 : 0;
}

// `path` as returned by forward_kernel_for: callers that cut a request into chunks decide once for the
// whole request, so that every image of it goes through the same kernel.
int forward_device(cnn_net* net, int path, const float* d_images, long n, float* d_out, int* d_argmax,
                   cudaStream_t stream) {
  if (path != 0) return forward_device_tc(net, path, d_images, n, d_out, d_argmax, stream);
  return net->fast_sigmoid ? launch_variant<1, false, 1>(net, d_images, n, d_out, d_argmax, stream)
                           : launch_variant<0, false, 1>(net, d_images, n, d_out, d_argmax, stream);
}

int forward_device_u8(cnn_net* net, const unsigned char* d_pixels, long n, float* d_out, int* d_argmax,
                      cudaStream_t stream) {
  return net->fast_sigmoid ? launch_variant<1, true, 1>(net, d_pixels, n, d_out, d_argmax, stream)
                           : launch_variant<0, true, 1>(net, d_pixels, n, d_out, d_argmax, stream);
}

}  // namespace cnn

extern "C" int cnn_forward_batched(cnn_net* net, const float* d_images, long n, float* d_out,
                                   int* d_argmax, void* stream) {
  CNN_REQUIRE(net != nullptr, "cnn_forward_batched: NULL net");
  CNN_REQUIRE(n >= 0, "cnn_forward_batched: negative image count");
  if (n == 0) return CNN_OK;
  CNN_REQUIRE(d_images != nullptr, "cnn_forward_batched: NULL images");
  CNN_REQUIRE((reinterpret_cast<uintptr_t>(d_images) & 15u) == 0,
              "cnn_forward_batched: image batch must start on a 16-byte boundary");
  return cnn::forward_device(net, cnn::forward_kernel_for(net, n), d_images, n, d_out, d_argmax, cnn::as_stream(stream));
}

extern "C" int cnn_forward_batched_u8(cnn_net* net, const unsigned char* d_pixels, long n, float* d_out,
                                      int* d_argmax, void* stream) {
  CNN_REQUIRE(net != nullptr, "cnn_forward_batched_u8: NULL net");
  CNN_REQUIRE(n >= 0, "cnn_forward_batched_u8: negative image count");
  if (n == 0) return CNN_OK;
  CNN_REQUIRE(d_pixels != nullptr, "cnn_forward_batched_u8: NULL pixels");
  CNN_REQUIRE((reinterpret_cast<uintptr_t>(d_pixels) & 15u) == 0,
              "cnn_forward_batched_u8: pixel batch must start on a 16-byte boundary");
  return cnn::forward_device_u8(net, d_pixels, n, d_out, d_argmax, cnn::as_stream(stream));
}
