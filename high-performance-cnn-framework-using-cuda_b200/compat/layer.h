// Source-level drop-in for the reference's operator header.
//
// A program written against the reference's layer.h (its main.cu: four `Layer` objects, kernels
// launched by the caller as `name<<<grid, block>>>(...)` on the default stream) compiles unchanged
// against this header plus compat/layer.cu.  What is kept: the class name and its public members,
// the three methods, every kernel name with its parameter list, `dt` and `threshold`.  What
// changes underneath: no kernel uses atomicAdd (each output element has one owner, full warps
// combine by shuffles), so results are bit-reproducible; kernels are correct for any 1-D launch
// shape; CUDA return codes are recorded (Layer::last_error()) instead of ignored; Layer is
// non-copyable (the reference's implicit copy would double-free).
#pragma once
#ifndef CNN_B200_COMPAT_LAYER_H
#define CNN_B200_COMPAT_LAYER_H

#include <cublas_v2.h>  // callers of the reference header get cuBLAS types through it
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <memory>
#include <vector>

// Learning rate used by apply_grad and the bias operators; early-stop bound of the training loop.
__device__ const static float dt = 1.0E-01f;
const static float threshold = 1.0E-02f;

class Layer {
 public:
  int M, N, O;  // fan-in per unit, units, output elements

  float* output;
  float* preact;

  float* bias;    // [N]
  float* weight;  // [N][M]

  float* d_output;
  float* d_preact;
  float* d_weight;

  // Draws bias[i] then weight[i][0..M) for each unit from rand(), 0.5f - rand()/RAND_MAX.
  Layer(int M, int N, int O);
  ~Layer();
  Layer(const Layer&) = delete;
  Layer& operator=(const Layer&) = delete;

  void setOutput(float* data);  // blocking host -> device copy of O floats into `output`
  void clear();                 // zero output, preact
  void bp_clear();              // zero d_output, d_preact, d_weight

  // First CUDA error seen by any Layer method in this process (cudaSuccess if none).
  static cudaError_t last_error();
};

// ---- operators -----------------------------------------------------------------------------
// Launch them exactly as before (any 1-D grid/block works).  "+=" marks operators that accumulate
// into what their destination already holds, which is why callers clear() / bp_clear() first.

__device__ float step_function(float v);                                             // 1 / (1 + exp(-v))
__global__ void apply_step_function(float* z, float* a, const int count);            // a = sigmoid(z)
__global__ void makeError(float* delta, float* a, unsigned int label, const int count);  // delta = onehot - a
__global__ void apply_grad(float* params, float* gradient, const int count);         // params += dt * gradient

// forward: conv 6 x 5x5 (valid), shared 4x4 / stride-4 subsample, fully connected 216 -> 10
__global__ void fp_preact_c1(float image[28][28], float z[6][24][24], float filters[6][5][5]);       // z += filters (x) image
__global__ void fp_bias_c1(float z[6][24][24], float b[6]);                                          // z += b[map]
__global__ void fp_preact_s1(float a_c1[6][24][24], float z[6][6][6], float filter[1][4][4]);        // z += filter . window
__global__ void fp_bias_s1(float z[6][6][6], float b[1]);                                            // z += b[0]
__global__ void fp_preact_f(float a_s1[6][6][6], float z[10], float w[10][6][6][6]);                 // z += w . a_s1
__global__ void fp_bias_f(float z[10], float b[10]);                                                 // z += b

// backward, in the order the training loop launches them
__global__ void bp_weight_f(float g_w[10][6][6][6], float delta_f[10], float a_s1[6][6][6]);         // g_w = delta_f (x) a_s1
__global__ void bp_bias_f(float b[10], float delta_f[10]);                                           // b += dt * delta_f
__global__ void bp_output_s1(float g_a[6][6][6], float w[10][6][6][6], float delta_f[10]);           // g_a += w^T delta_f
__global__ void bp_preact_s1(float delta_s[6][6][6], float g_a[6][6][6], float z[6][6][6]);          // delta_s = g_a * sigmoid'(z)
__global__ void bp_weight_s1(float g_w[1][4][4], float delta_s[6][6][6], float a_c1[6][24][24]);     // g_w += delta_s . windows
__global__ void bp_bias_s1(float b[1], float delta_s[6][6][6]);                                      // b += dt * mean(delta_s)
__global__ void bp_output_c1(float g_a[6][24][24], float filter[1][4][4], float delta_s[6][6][6]);   // g_a += filter * delta_s
__global__ void bp_preact_c1(float delta_c[6][24][24], float g_a[6][24][24], float z[6][24][24]);    // delta_c = g_a * sigmoid'(z)
__global__ void bp_weight_c1(float g_w[6][5][5], float delta_c[6][24][24], float image[28][28]);     // g_w += delta_c (x) image / 576
__global__ void bp_bias_c1(float b[6], float delta_c[6][24][24]);                                    // b += dt * mean(delta_c)

#endif  // CNN_B200_COMPAT_LAYER_H
