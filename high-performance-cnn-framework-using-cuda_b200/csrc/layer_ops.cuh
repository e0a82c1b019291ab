// Device bodies of the per-operator kernels (the reference's layer.cu:86-399 operator surface),
// written owner-computes: every output element is produced by exactly one thread, or by one full
// warp that combines its lanes with shuffles, so there is no atomicAdd anywhere and results do
// not depend on scheduling.  Each body works for any 1-D launch shape, like the reference's
// "split N items over all threads" idiom; the warp-cooperative path is used only when the block
// size is a multiple of 32 (otherwise one thread walks all terms of an output).
//
// The contract of each operator is the reference's: operators that the reference implements with
// atomicAdd accumulate INTO the existing contents of their destination (the caller zeroes it with
// Layer::clear / Layer::bp_clear first), bias operators and apply_grad update in place.
#pragma once

#include "cnn_common.cuh"

namespace cnn {
namespace ops {

__device__ __forceinline__ int global_thread() { return blockIdx.x * blockDim.x + threadIdx.x; }
__device__ __forceinline__ int total_threads() { return gridDim.x * blockDim.x; }

// Elementwise helper: f(i) for every i in [0, n), grid-stride.
template <class Fn>
__device__ __forceinline__ void for_each(int n, Fn fn) {
  for (int i = global_thread(); i < n; i += total_threads()) fn(i);
}

// Reduction helper: for each output o in [0, n_out), dst(o, sum_{t<n_terms} term(o, t)).
// Full warps split the terms over lanes and combine with a butterfly (fixed order for a given
// launch shape); otherwise one thread per output.
template <class Term, class Sink>
__device__ __forceinline__ void reduce_terms(int n_out, int n_terms, Term term, Sink sink) {
  if ((blockDim.x & 31) == 0) {
    const int lane = threadIdx.x & 31;
    const int warp = global_thread() >> 5;
    const int n_warps = total_threads() >> 5;
    for (int o = warp; o < n_out; o += n_warps) {
      float acc = 0.f;
      for (int t = lane; t < n_terms; t += 32) acc += term(o, t);
#pragma unroll
      for (int m = 16; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
      if (lane == 0) sink(o, acc);
    }
  } else {
    for (int o = global_thread(); o < n_out; o += total_threads()) {
      float acc = 0.f;
      for (int t = 0; t < n_terms; ++t) acc += term(o, t);
      sink(o, acc);
    }
  }
}

// ---- utility operators --------------------------------------------------------------------
__device__ __forceinline__ void apply_step_function(const float* in, float* out, int n) {
  for_each(n, [&](int i) { out[i] = sigmoidf<false>(in[i]); });
}

__device__ __forceinline__ void make_error(float* err, const float* out, unsigned label, int n) {
  for_each(n, [&](int i) { err[i] = ((label == (unsigned)i) ? 1.0f : 0.0f) - out[i]; });
}

__device__ __forceinline__ void apply_grad(float* w, const float* g, int n) {
  for_each(n, [&](int i) { w[i] += kDt * g[i]; });
}

// ---- forward ------------------------------------------------------------------------------
// preact[f][y][x] += sum_{i,j} W[f][i][j] * in[y+i][x+j]
__device__ __forceinline__ void fp_preact_c1(const float* in, float* pre, const float* W) {
  for_each(kF * kC * kC, [&](int o) {
    const int x = o % kC, y = (o / kC) % kC, f = o / (kC * kC);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 5; ++j)
#pragma unroll
      for (int i = 0; i < 5; ++i) acc += W[f * 25 + i * 5 + j] * in[(y + i) * kH + x + j];
    pre[o] += acc;
  });
}

__device__ __forceinline__ void fp_bias_c1(float* pre, const float* b) {
  for_each(kF * kC * kC, [&](int o) { pre[o] += b[o / (kC * kC)]; });
}

// preact[f][p][q] += sum_{i,j} W[0][i][j] * in[f][4p+i][4q+j]
__device__ __forceinline__ void fp_preact_s1(const float* in, float* pre, const float* W) {
  for_each(kS, [&](int o) {
    const int q = o % kP, p = (o / kP) % kP, f = o / (kP * kP);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc += W[i * 4 + j] * in[(f * kC + 4 * p + i) * kC + 4 * q + j];
    pre[o] += acc;
  });
}

__device__ __forceinline__ void fp_bias_s1(float* pre, const float* b) {
  for_each(kS, [&](int o) { pre[o] += b[0]; });
}

// preact[k] += sum_s W[k][s] * in[s]
__device__ __forceinline__ void fp_preact_f(const float* in, float* pre, const float* W) {
  reduce_terms(
      kOut, kS, [&](int k, int s) { return W[k * kS + s] * in[s]; },
      [&](int k, float v) { pre[k] += v; });
}

__device__ __forceinline__ void fp_bias_f(float* pre, const float* b) {
  for_each(kOut, [&](int k) { pre[k] += b[k]; });
}

// ---- backward -----------------------------------------------------------------------------
__device__ __forceinline__ void bp_weight_f(float* dW, const float* d_pre, const float* p_out) {
  for_each(kOut * kS, [&](int o) { dW[o] = d_pre[o / kS] * p_out[o % kS]; });
}

__device__ __forceinline__ void bp_bias_f(float* b, const float* d_pre) {
  for_each(kOut, [&](int k) { b[k] += kDt * d_pre[k]; });
}

// d_output[s] += sum_k W[k][s] * delta[k]
__device__ __forceinline__ void bp_output_s1(float* d_out, const float* W, const float* nd_pre) {
  for_each(kS, [&](int s) {
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < kOut; ++k) acc += W[k * kS + s] * nd_pre[k];
    d_out[s] += acc;
  });
}

__device__ __forceinline__ void bp_preact_generic(float* d_pre, const float* d_out,
                                                  const float* pre, int n) {
  for_each(n, [&](int i) {
    const float o = sigmoidf<false>(pre[i]);
    d_pre[i] = d_out[i] * o * (1 - o);
  });
}

// d_weight[i][j] += sum_{f,p,q} d_pre[f][p][q] * p_out[f][4p+i][4q+j]   (no normalisation)
__device__ __forceinline__ void bp_weight_s1(float* dW, const float* d_pre, const float* p_out) {
  reduce_terms(
      16, kS,
      [&](int o, int s) {
        const int i = o / 4, j = o % 4;
        const int q = s % kP, p = (s / kP) % kP, f = s / (kP * kP);
        return d_pre[s] * p_out[(f * kC + 4 * p + i) * kC + 4 * q + j];
      },
      [&](int o, float v) { dW[o] += v; });
}

// bias[0] += sum_s (dt * d_pre[s]) / 216
__device__ __forceinline__ void bp_bias_s1(float* b, const float* d_pre) {
  const float d = (float)kS;
  reduce_terms(
      1, kS, [&](int, int s) { return kDt * d_pre[s] / d; }, [&](int, float v) { b[0] += v; });
}

// d_output[f][4p+i][4q+j] += W[0][i][j] * nd_pre[f][p][q]
__device__ __forceinline__ void bp_output_c1(float* d_out, const float* W, const float* nd_pre) {
  for_each(kF * kC * kC, [&](int o) {
    const int x = o % kC, y = (o / kC) % kC, f = o / (kC * kC);
    d_out[o] += W[(y & 3) * 4 + (x & 3)] * nd_pre[(f * kP + (y >> 2)) * kP + (x >> 2)];
  });
}

// d_weight[f][i][j] += sum_{y,x} d_pre[f][y][x] * p_out[y+i][x+j] / 576
__device__ __forceinline__ void bp_weight_c1(float* dW, const float* d_pre, const float* p_out) {
  const float d = (float)(kC * kC);
  reduce_terms(
      kF * 25, kC * kC,
      [&](int o, int t) {
        const int f = o / 25, i = (o / 5) % 5, j = o % 5;
        const int y = t / kC, x = t % kC;
        return d_pre[(f * kC + y) * kC + x] * p_out[(y + i) * kH + x + j] / d;
      },
      [&](int o, float v) { dW[o] += v; });
}

// bias[f] += sum_{y,x} (dt * d_pre[f][y][x]) / 576
__device__ __forceinline__ void bp_bias_c1(float* b, const float* d_pre) {
  const float d = (float)(kC * kC);
  reduce_terms(
      kF, kC * kC, [&](int f, int t) { return kDt * d_pre[f * kC * kC + t] / d; },
      [&](int f, float v) { b[f] += v; });
}

}  // namespace ops
}  // namespace cnn
