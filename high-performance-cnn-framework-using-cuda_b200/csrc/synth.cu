// Device-side synthetic image generator.  The reference reads the MNIST IDX files
// (main.cu:30-33, mnist.h:79-160); no such files exist offline, so seeded synthetic images with the
// same shape (28x28), storage (uint8 pixel / 255 -> float, mnist.h:145) and label range stand in.
//
// The generator is counter-based and integer-only, so the numpy implementation in the Python
// package (synth.py) produces bit-identical images on the host:
//   base     = mix(mix(seed + G) + index)                      G = 0x9E3779B97F4A7C15
//   label    = mix(base + 0) % 10
//   strokes  = 5 + mix(base + 1) % 3
//   stroke s : r = mix(base + 2 + s);  start (4 + r[0:8] % 20, 4 + r[8:16] % 20), length
//              10 + r[16:24] % 13, direction r[24:28] of 16, optional bend at half length to
//              direction + (r[32:40] % 5) - 2; each step stamps a 2x2 block
//   pixel i  : covered ? 128 + (mix(base + 64 + i) & 127) : 0      (uint8), stored as v / 255
#include "net.cuh"

namespace cnn {

__host__ __device__ inline unsigned long long mix64(unsigned long long z) {
  z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ULL;
  z ^= z >> 27; z *= 0x94D049BB133111EBULL;
  z ^= z >> 31;
  return z;
}

__constant__ int c_dx[16] = {8, 7, 6, 3, 0, -3, -6, -7, -8, -7, -6, -3, 0, 3, 6, 7};
__constant__ int c_dy[16] = {0, 3, 6, 7, 8, 7, 6, 3, 0, -3, -6, -7, -8, -7, -6, -3};

constexpr int kSynthWarps = 8;

__global__ void __launch_bounds__(kSynthWarps * 32)
k_synth(unsigned long long seed, long first_index, long n, float* __restrict__ images,
        unsigned* __restrict__ labels) {
  __shared__ float lut[256];
  __shared__ unsigned canvas[kSynthWarps][kImg / 4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int v = threadIdx.x; v < 256; v += blockDim.x) lut[v] = (float)((double)v / 255.0);
  __syncthreads();
  unsigned char* cv = reinterpret_cast<unsigned char*>(canvas[warp]);
  const unsigned long long seed_mix = mix64(seed + 0x9E3779B97F4A7C15ULL);

  for (long li = (long)blockIdx.x * kSynthWarps + warp; li < n; li += (long)gridDim.x * kSynthWarps) {
    for (int i = lane; i < kImg / 4; i += 32) canvas[warp][i] = 0u;
    __syncwarp();
    const unsigned long long base = mix64(seed_mix + (unsigned long long)(first_index + li));
    const int n_strokes = 5 + (int)(mix64(base + 1) % 3ULL);
    for (int s = 0; s < n_strokes; ++s) {
      const unsigned long long r = mix64(base + 2 + (unsigned long long)s);
      const int x0 = 4 + (int)((r & 0xFF) % 20), y0 = 4 + (int)(((r >> 8) & 0xFF) % 20);
      const int len = 10 + (int)(((r >> 16) & 0xFF) % 13);
      const int d1 = (int)((r >> 24) & 15);
      const int bend = (int)((r >> 28) & 1);
      const int d2 = bend ? ((d1 + (int)(((r >> 32) & 0xFF) % 5) + 14) & 15) : d1;
      const int half = len / 2;
      const int t = lane;
      if (t < len) {
        const int t1 = t < half ? t : half, t2 = t < half ? 0 : t - half;
        const int X = x0 * 8 + t1 * c_dx[d1] + t2 * c_dx[d2];
        const int Y = y0 * 8 + t1 * c_dy[d1] + t2 * c_dy[d2];
        const int px = X >> 3, py = Y >> 3;
#pragma unroll
        for (int b = 0; b < 2; ++b)
#pragma unroll
          for (int a = 0; a < 2; ++a) {
            const int xx = px + a, yy = py + b;
            if (xx >= 0 && xx < kH && yy >= 0 && yy < kH) cv[yy * kH + xx] = 1;
          }
      }
      __syncwarp();
    }
    float* dst = images + li * kImg;
    for (int i = lane; i < kImg; i += 32) {
      const unsigned v = cv[i] ? (128u + (unsigned)(mix64(base + 64 + (unsigned long long)i) & 127ULL)) : 0u;
      dst[i] = lut[v];
    }
    if (labels && lane == 0) labels[li] = (unsigned)(mix64(base) % 10ULL);
    __syncwarp();
  }
}

}  // namespace cnn

extern "C" int cnn_synth_images(unsigned long long seed, long first_index, long n, float* d_images,
                                unsigned int* d_labels, void* stream) {
  using namespace cnn;
  CNN_REQUIRE(n >= 0 && first_index >= 0, "cnn_synth_images: negative count or index");
  if (n == 0) return CNN_OK;
  CNN_REQUIRE(d_images != nullptr, "cnn_synth_images: NULL images");
  long blocks = (n + kSynthWarps - 1) / kSynthWarps;
  const long cap = 32L * sm_count();
  if (blocks > cap) blocks = cap;
  k_synth<<<(int)blocks, kSynthWarps * 32, 0, as_stream(stream)>>>(seed, first_index, n, d_images, d_labels);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "k_synth launch");
  return CNN_OK;
}
