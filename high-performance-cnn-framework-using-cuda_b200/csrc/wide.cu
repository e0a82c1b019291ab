// Widened variant of the same topology (benchmark configuration 5): input HxH, F maps of 5x5 (valid) ->
// sigmoid -> ONE shared 4x4/stride-4 filter -> sigmoid -> FC F*P*P -> 10 -> sigmoid, with the
// reference's update rule generalised as in the oracle: divisors (H-4)^2 for the conv gradient and
// bias, F*P*P for the subsample bias (layer.cu:369, 389, 312 with 24 -> H-4 and 6*6*6 -> F*P*P).
// The reference's own kernels cannot run this shape (fixed array types; N * thread_index overflows
// int), so its check is the generalised oracle.
//
// This file is the fp32 SIMT path: batch-level kernels with the conv activations and conv deltas
// kept in HBM between them (at 56x56 / 64 maps one image's activations are 692 KB, more than an
// SM's shared memory).  All reductions are fixed-order (no atomics).
#include <cstring>
#include <new>
#include <vector>

#include "wide.cuh"

namespace cnn {

constexpr int kWideFg = 8;       // filters per block in the forward conv
constexpr int kWideGg = 4;       // filters per block in the conv weight gradient

// ---- forward ---------------------------------------------------------------------------------
// Block (image b, group of 8 maps): image in shared memory, thread = output position, 8 maps per
// patch read.  Writes the conv ACTIVATIONS (sigmoid applied); pre-activations are never needed again
// because sigmoid' = a (1 - a).
template <int FLAVOR>
__global__ void __launch_bounds__(256)
k_wide_conv_fwd(WideDims d, const float* __restrict__ images, const float* __restrict__ params,
                float* __restrict__ ac) {
  extern __shared__ float sh[];
  float* img = sh;                       // H*H
  float* w = sh + d.H * d.H;             // 8 * 25
  float* bias = w + kWideFg * 25;        // 8
  const int b = blockIdx.x, f0 = blockIdx.y * kWideFg;
  for (int i = threadIdx.x; i < d.H * d.H; i += blockDim.x) img[i] = images[(size_t)b * d.H * d.H + i];
  for (int i = threadIdx.x; i < kWideFg * 25; i += blockDim.x)
    w[i] = (f0 + i / 25 < d.F) ? params[d.o_wc + f0 * 25 + i] : 0.f;
  if (threadIdx.x < kWideFg) bias[threadIdx.x] = (f0 + threadIdx.x < d.F) ? params[d.o_bc + f0 + threadIdx.x] : 0.f;
  __syncthreads();
  const int CC = d.C * d.C;
  for (int o = threadIdx.x; o < CC; o += blockDim.x) {
    const int y = o / d.C, x = o % d.C;
    float acc[kWideFg];
#pragma unroll
    for (int g = 0; g < kWideFg; ++g) acc[g] = 0.f;
#pragma unroll
    for (int j = 0; j < 5; ++j)
#pragma unroll
      for (int i = 0; i < 5; ++i) {
        const float v = img[(y + i) * d.H + x + j];
#pragma unroll
        for (int g = 0; g < kWideFg; ++g) acc[g] = fmaf(w[g * 25 + i * 5 + j], v, acc[g]);
      }
#pragma unroll
    for (int g = 0; g < kWideFg; ++g)
      if (f0 + g < d.F) ac[((size_t)b * d.F + f0 + g) * CC + o] = sigmoidf<FLAVOR>(acc[g] + bias[g]);
  }
}

// Thread = one subsample output (b, f, p, q).
template <int FLAVOR>
__global__ void k_wide_s1_fwd(WideDims d, long n, const float* __restrict__ ac,
                              const float* __restrict__ params, float* __restrict__ as) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n * d.S) return;
  const int q = (int)(idx % d.P), p = (int)((idx / d.P) % d.P);
  const long bf = idx / (d.P * d.P);
  const float* src = ac + (size_t)bf * d.C * d.C + (4 * p) * d.C + 4 * q;
  float z = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) z = fmaf(params[d.o_ws + i * 4 + j], src[i * d.C + j], z);
  as[idx] = sigmoidf<FLAVOR>(z + params[d.o_bs]);
}

// Block = kWideFcImgs images: FC, sigmoid, argmax, makeError, error norm.  (One image per block read the
// 433 KB of FC weights from L2 once per image: 62 us for 1,024 images; four images share them.)
constexpr int kWideFcImgs = 4;

template <int FLAVOR>
__global__ void __launch_bounds__(256)
k_wide_fc_fwd(WideDims d, long n, const float* __restrict__ as, const float* __restrict__ params,
              const unsigned* __restrict__ labels, float* __restrict__ out, int* __restrict__ argmax,
              float* __restrict__ delta_f, float* __restrict__ err) {
  __shared__ float red[8][kWideFcImgs][kOut];
  __shared__ float o_s[kWideFcImgs][kOut];
  const long b0 = (long)blockIdx.x * kWideFcImgs;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int imgs = (int)((n - b0) < kWideFcImgs ? (n - b0) : kWideFcImgs);
  float acc[kWideFcImgs][kOut];
#pragma unroll
  for (int g = 0; g < kWideFcImgs; ++g)
#pragma unroll
    for (int k = 0; k < kOut; ++k) acc[g][k] = 0.f;
  for (int s = threadIdx.x; s < d.S; s += blockDim.x) {
    float wv[kOut];
#pragma unroll
    for (int k = 0; k < kOut; ++k) wv[k] = params[d.o_wf + (size_t)k * d.S + s];
#pragma unroll
    for (int g = 0; g < kWideFcImgs; ++g) {
      const float v = (g < imgs) ? as[(size_t)(b0 + g) * d.S + s] : 0.f;
#pragma unroll
      for (int k = 0; k < kOut; ++k) acc[g][k] = fmaf(wv[k], v, acc[g][k]);
    }
  }
#pragma unroll
  for (int m = 16; m > 0; m >>= 1)
#pragma unroll
    for (int g = 0; g < kWideFcImgs; ++g)
#pragma unroll
      for (int k = 0; k < kOut; ++k) acc[g][k] += __shfl_xor_sync(0xffffffffu, acc[g][k], m);
  if (lane == 0) {
#pragma unroll
    for (int g = 0; g < kWideFcImgs; ++g)
#pragma unroll
      for (int k = 0; k < kOut; ++k) red[warp][g][k] = acc[g][k];
  }
  __syncthreads();
  if (threadIdx.x < kWideFcImgs * kOut) {
    const int g = threadIdx.x / kOut, k = threadIdx.x % kOut;
    float z = 0.f;
    for (int ww = 0; ww < 8; ++ww) z += red[ww][g][k];
    const float o = sigmoidf<FLAVOR>(z + params[d.o_bf + k]);
    o_s[g][k] = o;
    if (g < imgs) {
      const long b = b0 + g;
      if (out) out[(size_t)b * kOut + k] = o;
      if (delta_f) delta_f[(size_t)b * kOut + k] = ((labels[b] == (unsigned)k) ? 1.0f : 0.0f) - o;
    }
  }
  __syncthreads();
  if (threadIdx.x < imgs) {
    const int g = threadIdx.x;
    const long b = b0 + g;
    int best = 0;
    for (int k = 1; k < kOut; ++k)
      if (o_s[g][best] < o_s[g][k]) best = k;
    if (argmax) argmax[b] = best;
    if (err) {
      float ss = 0.f;
      for (int k = 0; k < kOut; ++k) {
        const float dlt = ((labels[b] == (unsigned)k) ? 1.0f : 0.0f) - o_s[g][k];
        ss += dlt * dlt;
      }
      err[b] = sqrtf(ss);
    }
  }
}

// ---- backward --------------------------------------------------------------------------------
// delta_s[b][s] = (sum_k Wf[k][s] delta_f[b][k]) * as (1 - as).  Thread = one s for kWideBpImgs images: the ten
// weights of s stay in registers, the images' output deltas come from shared memory.
constexpr int kWideBpImgs = 8;

__global__ void __launch_bounds__(256)
k_wide_bp_s1(WideDims d, long n, const float* __restrict__ as, const float* __restrict__ delta_f,
             const float* __restrict__ params, float* __restrict__ ds) {
  __shared__ float dlt[kWideBpImgs][kOut];
  const long b0 = (long)blockIdx.x * kWideBpImgs;     // images along x (no 65,535 limit), the S range along y
  const int imgs = (int)((n - b0) < kWideBpImgs ? (n - b0) : kWideBpImgs);
  if (threadIdx.x < kWideBpImgs * kOut) {
    const int g = threadIdx.x / kOut, k = threadIdx.x % kOut;
    dlt[g][k] = (g < imgs) ? delta_f[(b0 + g) * kOut + k] : 0.f;
  }
  __syncthreads();
  const int s = blockIdx.y * blockDim.x + threadIdx.x;
  if (s >= d.S) return;
  float wv[kOut];
#pragma unroll
  for (int k = 0; k < kOut; ++k) wv[k] = params[d.o_wf + (size_t)k * d.S + s];
#pragma unroll
  for (int g = 0; g < kWideBpImgs; ++g) {
    if (g < imgs) {
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < kOut; ++k) acc = fmaf(wv[k], dlt[g][k], acc);
      const size_t idx = (size_t)(b0 + g) * d.S + s;
      const float a = as[idx];
      ds[idx] = acc * a * (1.f - a);
    }
  }
}

// G_wf[k][s] = sum_b delta_f[b][k] as[b][s].  The batch is cut into kWideFcSplit contiguous slices
// (blockIdx.y); each thread owns one s for one slice and writes a partial, and k_wide_grad_fc_sum adds
// the slices in order, so the result does not depend on scheduling.  Also G_bf.
constexpr int kWideFcSplit = 16;

__global__ void k_wide_grad_fc(WideDims d, long n, const float* __restrict__ as, const float* __restrict__ delta_f,
                               float* __restrict__ part_f) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  const long b0 = (n * blockIdx.y) / kWideFcSplit, b1 = (n * (blockIdx.y + 1)) / kWideFcSplit;
  if (s >= d.S) return;
  float acc[kOut];
#pragma unroll
  for (int k = 0; k < kOut; ++k) acc[k] = 0.f;
  for (long b = b0; b < b1; ++b) {
    const float v = as[b * d.S + s];
#pragma unroll
    for (int k = 0; k < kOut; ++k) acc[k] = fmaf(delta_f[b * kOut + k], v, acc[k]);
  }
#pragma unroll
  for (int k = 0; k < kOut; ++k) part_f[((size_t)blockIdx.y * kOut + k) * d.S + s] = acc[k];
}

__global__ void k_wide_grad_fc_sum(WideDims d, long n, const float* __restrict__ part_f,
                                   const float* __restrict__ delta_f, float* __restrict__ G) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;   // over kOut * S
  if (i < (long)kOut * d.S) {
    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < kWideFcSplit; ++c) sum += part_f[(size_t)c * kOut * d.S + i];
    G[d.o_wf + i] = sum;
  }
  // G_bf: the warps of the last block add delta_f[.][k] for k = warp, warp + warps, ... (lane l takes images
  // l, l + 32, ...; fixed shuffle tree)
  if (blockIdx.x == gridDim.x - 1) {
    const int lane = threadIdx.x & 31;
    for (int k = threadIdx.x >> 5; k < kOut; k += (int)(blockDim.x >> 5)) {
      float acc = 0.f;
      for (long b = lane; b < n; b += 32) acc += delta_f[b * kOut + k];
#pragma unroll
      for (int m = 16; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
      if (lane == 0) G[d.o_bf + k] = acc;
    }
  }
}

// Per image: 16 subsample-filter gradient partials + bias partial -> part[b][17]; also writes the
// conv deltas dc = Ws[i][j] * delta_s * a (1 - a) / (C*C).  Block = one image, thread strides over
// (f, p, q).
__global__ void __launch_bounds__(256)
k_wide_bp_c1(WideDims d, const float* __restrict__ ac, const float* __restrict__ ds,
             const float* __restrict__ params, float* __restrict__ dc, float* __restrict__ part) {
  __shared__ float red[8][17];
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float inv_c = 1.0f / (float)(d.C * d.C), inv_s = 1.0f / (float)d.S;
  float ws[16];
#pragma unroll
  for (int t = 0; t < 16; ++t) ws[t] = params[d.o_ws + t];
  float acc[17];
#pragma unroll
  for (int t = 0; t < 17; ++t) acc[t] = 0.f;
  for (int s = threadIdx.x; s < d.S; s += blockDim.x) {
    const int q = s % d.P, p = (s / d.P) % d.P, f = s / (d.P * d.P);
    const float dlt = ds[(size_t)b * d.S + s];
    const size_t base = ((size_t)b * d.F + f) * d.C * d.C + (4 * p) * d.C + 4 * q;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = ac[base + i * d.C + j];
        acc[i * 4 + j] = fmaf(dlt, a, acc[i * 4 + j]);
        dc[base + i * d.C + j] = (ws[i * 4 + j] * dlt) * a * (1.f - a) * inv_c;
      }
    acc[16] += dlt * inv_s;
  }
#pragma unroll
  for (int m = 16; m > 0; m >>= 1)
#pragma unroll
    for (int t = 0; t < 17; ++t) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], m);
  if (lane == 0) {
#pragma unroll
    for (int t = 0; t < 17; ++t) red[warp][t] = acc[t];
  }
  __syncthreads();
  if (threadIdx.x < 17) {
    float sum = 0.f;
    for (int ww = 0; ww < 8; ++ww) sum += red[ww][threadIdx.x];
    part[(size_t)b * 17 + threadIdx.x] = sum;
  }
  // positions outside the 4P x 4P area (only when C is not a multiple of 4) get no delta
  if (4 * d.P != d.C) {
    for (int o = threadIdx.x; o < d.F * d.C * d.C; o += blockDim.x) {
      const int x = o % d.C, y = (o / d.C) % d.C;
      if (y >= 4 * d.P || x >= 4 * d.P) dc[(size_t)b * d.F * d.C * d.C + o] = 0.f;
    }
  }
}

// Conv weight gradient partial of one image for 4 maps: part[b][f][26] (25 taps + bias term).
__global__ void __launch_bounds__(256)
k_wide_grad_c1(WideDims d, const float* __restrict__ images, const float* __restrict__ dc,
               float* __restrict__ part) {
  extern __shared__ float sh[];
  float* img = sh;                                  // H*H
  float* red = sh + d.H * d.H;                      // 8 warps * 4 maps * 26
  const int b = blockIdx.x, f0 = blockIdx.y * kWideGg;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < d.H * d.H; i += blockDim.x) img[i] = images[(size_t)b * d.H * d.H + i];
  __syncthreads();
  const int CC = d.C * d.C;
  float acc[kWideGg][26];
#pragma unroll
  for (int g = 0; g < kWideGg; ++g)
#pragma unroll
    for (int t = 0; t < 26; ++t) acc[g][t] = 0.f;
  for (int o = threadIdx.x; o < CC; o += blockDim.x) {
    const int y = o / d.C, x = o % d.C;
    float dv[kWideGg];
#pragma unroll
    for (int g = 0; g < kWideGg; ++g) {
      dv[g] = (f0 + g < d.F) ? dc[((size_t)b * d.F + f0 + g) * CC + o] : 0.f;
      acc[g][25] += dv[g];
    }
#pragma unroll
    for (int i = 0; i < 5; ++i)
#pragma unroll
      for (int j = 0; j < 5; ++j) {
        const float v = img[(y + i) * d.H + x + j];
#pragma unroll
        for (int g = 0; g < kWideGg; ++g) acc[g][i * 5 + j] = fmaf(dv[g], v, acc[g][i * 5 + j]);
      }
  }
#pragma unroll
  for (int g = 0; g < kWideGg; ++g)
#pragma unroll
    for (int t = 0; t < 26; ++t) {
      float v = acc[g][t];
#pragma unroll
      for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
      if (lane == 0) red[(warp * kWideGg + g) * 26 + t] = v;
    }
  __syncthreads();
  if (threadIdx.x < kWideGg * 26) {
    const int g = threadIdx.x / 26, t = threadIdx.x % 26;
    float sum = 0.f;
    for (int ww = 0; ww < 8; ++ww) sum += red[(ww * kWideGg + g) * 26 + t];
    if (f0 + g < d.F) part[((size_t)b * d.F + f0 + g) * 26 + t] = sum;
  }
}

// Sum the partials into the arena-ordered gradient; G[n_params+1] = sum of the per-image error norms;
// padding zeroed.  One warp per output value: lane l adds rows l, l + 32, ... in order, then the lanes
// are combined by a fixed shuffle tree (the same order every run).  (One thread per value walking up
// to 1,024 rows took 79 us of a 1.3 ms step.)
__global__ void __launch_bounds__(256)
k_wide_reduce(WideDims d, long n, long rows_c, long rows_s, const float* __restrict__ part_c,
              const float* __restrict__ part_s, const float* __restrict__ err, float* __restrict__ G) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int n_c = d.F * 26;
  if (t > n_c + 17) return;
  const float* src;
  long rows, stride;
  if (t < n_c) { src = part_c + t; rows = rows_c; stride = n_c; }
  else if (t < n_c + 17) { src = part_s + (t - n_c); rows = rows_s; stride = 17; }
  else { src = err; rows = n; stride = 1; }
  float sum = 0.f;
  for (long b = lane; b < rows; b += 32) sum += src[(size_t)b * stride];
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
  if (lane != 0) return;
  if (t < n_c) {
    const int f = t / 26, k = t % 26;
    if (k < 25) G[d.o_wc + f * 25 + k] = sum; else G[d.o_bc + f] = sum;
  } else if (t < n_c + 17) {
    const int k = t - n_c;
    if (k < 16) G[d.o_ws + k] = sum; else G[d.o_bs] = sum;
  } else {
    G[d.n_params + 1] = sum;
    G[d.n_params] = 0.f;
    for (int i = d.n_params + 2; i < d.n_padded; ++i) G[i] = 0.f;
  }
}

__global__ void k_wide_update(int n_params, float* __restrict__ params, const float* __restrict__ G, float scale) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_params) params[i] = fmaf(scale, G[i], params[i]);
}

}  // namespace cnn

using namespace cnn;

static int wide_reserve(cnn_wide* w, long n) {
  if (n <= w->cap) return CNN_OK;
  float** bufs[] = {&w->ac, &w->dc, &w->as, &w->ds, &w->delta_f, &w->err, &w->part_c, &w->part_s, &w->img_shift};
  for (float** p : bufs) { cudaFree(*p); *p = nullptr; }
  w->cap = 0;
  const WideDims& d = w->d;
  const size_t fcc = (size_t)d.F * d.C * d.C;
  CNN_CUDA(cudaMalloc(&w->ac, sizeof(float) * fcc * n));
  CNN_CUDA(cudaMalloc(&w->dc, sizeof(float) * fcc * n));
  CNN_CUDA(cudaMalloc(&w->as, sizeof(float) * (size_t)d.S * n));
  CNN_CUDA(cudaMalloc(&w->ds, sizeof(float) * (size_t)d.S * n));
  CNN_CUDA(cudaMalloc(&w->delta_f, sizeof(float) * kOut * n));
  CNN_CUDA(cudaMalloc(&w->err, sizeof(float) * n));
  w->part_rows = n > 4096 ? n : 4096;
  CNN_CUDA(cudaMalloc(&w->part_c, sizeof(float) * (size_t)d.F * 26 * w->part_rows));
  CNN_CUDA(cudaMalloc(&w->part_s, sizeof(float) * 17 * w->part_rows));   // one row per image, or per CTA of the fused kernel
  if (wide_grad_tc_supported(d)) CNN_CUDA(cudaMalloc(&w->img_shift, sizeof(float) * 4 * (size_t)d.H * d.H * n));
  if (!w->part_f) CNN_CUDA(cudaMalloc(&w->part_f, sizeof(float) * (size_t)kWideFcSplit * kOut * d.S));
  w->cap = n;
  return CNN_OK;
}

template <int FL>
static int wide_forward_impl(cnn_wide* w, const float* d_images, const unsigned* d_labels, long n, float* d_out,
                             int* d_argmax, bool training, cudaStream_t st) {
  const WideDims& d = w->d;
  const size_t smem = sizeof(float) * ((size_t)d.H * d.H + kWideFg * 25 + kWideFg);
  CNN_CUDA(cudaFuncSetAttribute(k_wide_conv_fwd<FL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  if (w->conv_mode > 0 && wide_conv_tc_supported(d)) {
    const int rc = wide_conv_fwd_tc(w, d_images, n, st);
    if (rc != CNN_OK) return rc;
  } else {
    k_wide_conv_fwd<FL><<<dim3((unsigned)n, (d.F + kWideFg - 1) / kWideFg), 256, smem, st>>>(d, d_images, w->d_params, w->ac);
  }
  const long ns = n * d.S;
  k_wide_s1_fwd<FL><<<(unsigned)((ns + 255) / 256), 256, 0, st>>>(d, n, w->ac, w->d_params, w->as);
  k_wide_fc_fwd<FL><<<(unsigned)((n + kWideFcImgs - 1) / kWideFcImgs), 256, 0, st>>>(d, n, w->as, w->d_params, d_labels, d_out, d_argmax,
                                                 training ? w->delta_f : nullptr, training ? w->err : nullptr);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "wide forward launch");
  return CNN_OK;
}

static int wide_forward_dispatch(cnn_wide* w, const float* d_images, const unsigned* d_labels, long n, float* d_out,
                                 int* d_argmax, bool training, cudaStream_t st) {
  switch (w->flavour) {
    case 1: return wide_forward_impl<1>(w, d_images, d_labels, n, d_out, d_argmax, training, st);
    case 2: return wide_forward_impl<2>(w, d_images, d_labels, n, d_out, d_argmax, training, st);
    default: return wide_forward_impl<0>(w, d_images, d_labels, n, d_out, d_argmax, training, st);
  }
}

extern "C" {

int cnn_wide_param_count(int H, int F) {
  if (H < 8 || F < 1) return -1;
  return make_wide_dims(H, F).n_params;
}

int cnn_wide_create(int H, int F, cnn_wide** out) {
  CNN_REQUIRE(out != nullptr, "cnn_wide_create: out is NULL");
  *out = nullptr;
  CNN_REQUIRE(H >= 8 && H <= 128 && F >= 1 && F <= 1024, "cnn_wide_create: unsupported shape");
  cnn_wide* w = new (std::nothrow) cnn_wide();
  CNN_REQUIRE(w != nullptr, "cnn_wide_create: out of host memory");
  w->d = make_wide_dims(H, F);
  cudaError_t e = cudaMalloc(&w->d_params, sizeof(float) * w->d.n_padded);
  if (e == cudaSuccess) e = cudaMemset(w->d_params, 0, sizeof(float) * w->d.n_padded);
  if (e == cudaSuccess) e = cudaMalloc(&w->d_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(w->d_status, 0, sizeof(int));
  if (e == cudaSuccess) e = cudaDeviceSynchronize();  // memsets are asynchronous to the host
  if (e != cudaSuccess) { delete w; return cuda_fail(e, "cnn_wide_create"); }
  *out = w;
  return CNN_OK;
}

int cnn_wide_destroy(cnn_wide* w) {
  if (!w) return CNN_OK;
  float* bufs[] = {w->d_params, w->ac, w->dc, w->as, w->ds, w->delta_f, w->err, w->part_c, w->part_s, w->img_shift};
  for (float* p : bufs) cudaFree(p);
  cudaFree(w->d_status);
  cudaFree(w->part_f);
  delete w;
  return CNN_OK;
}

int cnn_wide_set_params(cnn_wide* w, const float* h_params) {
  CNN_REQUIRE(w && h_params, "cnn_wide_set_params: NULL argument");
  // same ordering as cnn_net_set_params: nothing in flight reads the old values, and the upload
  // has landed before a launch on a non-blocking stream
  CNN_CUDA(cudaDeviceSynchronize());
  CNN_CUDA(cudaMemcpy(w->d_params, h_params, sizeof(float) * w->d.n_params, cudaMemcpyHostToDevice));
  CNN_CUDA(cudaDeviceSynchronize());
  return CNN_OK;
}

int cnn_wide_get_params(cnn_wide* w, float* h_params) {
  CNN_REQUIRE(w && h_params, "cnn_wide_get_params: NULL argument");
  CNN_CUDA(cudaMemcpy(h_params, w->d_params, sizeof(float) * w->d.n_params, cudaMemcpyDeviceToHost));
  return CNN_OK;
}

int cnn_wide_set_option(cnn_wide* w, const char* key, int value) {
  CNN_REQUIRE(w && key, "cnn_wide_set_option: NULL argument");
  if (std::strcmp(key, "fast_sigmoid") == 0) { w->flavour = (value == 2) ? 2 : (value ? 1 : 0); return CNN_OK; }
  if (std::strcmp(key, "conv") == 0) {
    CNN_REQUIRE(value >= 0 && value <= 2, "cnn_wide_set_option: conv is 0 (fp32 SIMT), 1 (tf32 tensor cores) or 2 (3 x tf32)");
    w->conv_mode = value;
    return CNN_OK;
  }
  set_error("cnn_wide_set_option: unknown option '%s'", key);
  return CNN_ERR_INVALID;
}

int cnn_wide_status(cnn_wide* w, int* status) {
  CNN_REQUIRE(w && status, "cnn_wide_status: NULL argument");
  CNN_CUDA(cudaDeviceSynchronize());
  CNN_CUDA(cudaMemcpy(status, w->d_status, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status != 0) {
    set_error("a bounded device-side wait ran out (status %d)", *status);
    int zero = 0;
    CNN_CUDA(cudaMemcpy(w->d_status, &zero, sizeof(int), cudaMemcpyHostToDevice));
    return CNN_ERR_TIMEOUT;
  }
  return CNN_OK;
}

int cnn_wide_forward(cnn_wide* w, const float* d_images, long n, float* d_out, int* d_argmax, void* stream) {
  CNN_REQUIRE(w != nullptr, "cnn_wide_forward: NULL handle");
  CNN_REQUIRE(n >= 0 && n <= 65535L * 32, "cnn_wide_forward: bad image count");
  if (n == 0) return CNN_OK;
  CNN_REQUIRE(d_images != nullptr, "cnn_wide_forward: NULL images");
  int rc = wide_reserve(w, n);
  if (rc != CNN_OK) return rc;
  return wide_forward_dispatch(w, d_images, nullptr, n, d_out, d_argmax, false, as_stream(stream));
}

int cnn_wide_grad_batch(cnn_wide* w, const float* d_images, const unsigned int* d_labels, long n, float* d_grad,
                        void* stream) {
  CNN_REQUIRE(w && d_grad, "cnn_wide_grad_batch: NULL argument");
  CNN_REQUIRE(n >= 0 && n <= 65535L * 32, "cnn_wide_grad_batch: bad image count");
  cudaStream_t st = as_stream(stream);
  const WideDims& d = w->d;
  if (n == 0) {
    CNN_CUDA(cudaMemsetAsync(d_grad, 0, sizeof(float) * d.n_padded, st));
    return CNN_OK;
  }
  CNN_REQUIRE(d_images && d_labels, "cnn_wide_grad_batch: NULL images or labels");
  int rc = wide_reserve(w, n);
  if (rc != CNN_OK) return rc;
  if ((rc = wide_forward_dispatch(w, d_images, d_labels, n, nullptr, nullptr, true, st)) != CNN_OK) return rc;
  k_wide_bp_s1<<<dim3((unsigned)((n + kWideBpImgs - 1) / kWideBpImgs), (unsigned)((d.S + 255) / 256)), 256, 0, st>>>(
      d, n, w->as, w->delta_f, w->d_params, w->ds);
  k_wide_grad_fc<<<dim3((d.S + 127) / 128, kWideFcSplit), 128, 0, st>>>(d, n, w->as, w->delta_f, w->part_f);
  k_wide_grad_fc_sum<<<(unsigned)(((long)kOut * d.S + 255) / 256), 256, 0, st>>>(d, n, w->part_f, w->delta_f, d_grad);
  long rows_c = n, rows_s = n;
  if (w->conv_mode > 0 && wide_grad_tc_supported(d)) {
    // conv deltas, conv weight gradient and subsample-filter gradient in one kernel; the deltas stay on chip
    int rows = 0;
    if ((rc = wide_grad_c1_tc(w, d_images, n, &rows, st)) != CNN_OK) return rc;
    rows_c = rows_s = rows;
  } else {
    k_wide_bp_c1<<<(unsigned)n, 256, 0, st>>>(d, w->ac, w->ds, w->d_params, w->dc, w->part_s);
    const size_t smem = sizeof(float) * ((size_t)d.H * d.H + 8 * kWideGg * 26);
    CNN_CUDA(cudaFuncSetAttribute(k_wide_grad_c1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_wide_grad_c1<<<dim3((unsigned)n, (d.F + kWideGg - 1) / kWideGg), 256, smem, st>>>(d, d_images, w->dc, w->part_c);
  }
  const int n_red = d.F * 26 + 18;       // one warp each
  k_wide_reduce<<<(n_red + 7) / 8, 256, 0, st>>>(d, n, rows_c, rows_s, w->part_c, w->part_s, w->err, d_grad);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "wide backward launch");
  return CNN_OK;
}

int cnn_wide_apply_update(cnn_wide* w, const float* d_grad, float scale, void* stream) {
  CNN_REQUIRE(w && d_grad, "cnn_wide_apply_update: NULL argument");
  k_wide_update<<<(w->d.n_params + 255) / 256, 256, 0, as_stream(stream)>>>(w->d.n_params, w->d_params, d_grad, scale);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "k_wide_update launch");
  return CNN_OK;
}

}  // extern "C"
