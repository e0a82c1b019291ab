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

// Utility operators
__device__ float step_function(float v);
__global__ void apply_step_function(float* input, float* output, const int N);
__global__ void makeError(float* err, float* output, unsigned int Y, const int N);
__global__ void apply_grad(float* output, float* grad, const int N);

// Forward operators
__global__ void fp_preact_c1(float input[28][28], float preact[6][24][24], float weight[6][5][5]);
__global__ void fp_bias_c1(float preact[6][24][24], float bias[6]);
__global__ void fp_preact_s1(float input[6][24][24], float preact[6][6][6], float weight[1][4][4]);
__global__ void fp_bias_s1(float preact[6][6][6], float bias[1]);
__global__ void fp_preact_f(float input[6][6][6], float preact[10], float weight[10][6][6][6]);
__global__ void fp_bias_f(float preact[10], float bias[10]);

// Backward operators
__global__ void bp_weight_f(float d_weight[10][6][6][6], float d_preact[10], float p_output[6][6][6]);
__global__ void bp_bias_f(float bias[10], float d_preact[10]);
__global__ void bp_output_s1(float d_output[6][6][6], float n_weight[10][6][6][6], float nd_preact[10]);
__global__ void bp_preact_s1(float d_preact[6][6][6], float d_output[6][6][6], float preact[6][6][6]);
__global__ void bp_weight_s1(float d_weight[1][4][4], float d_preact[6][6][6], float p_output[6][24][24]);
__global__ void bp_bias_s1(float bias[1], float d_preact[6][6][6]);
__global__ void bp_output_c1(float d_output[6][24][24], float n_weight[1][4][4], float nd_preact[6][6][6]);
__global__ void bp_preact_c1(float d_preact[6][24][24], float d_output[6][24][24], float preact[6][24][24]);
__global__ void bp_weight_c1(float d_weight[6][5][5], float d_preact[6][24][24], float p_output[28][28]);
__global__ void bp_bias_c1(float bias[6], float d_preact[6][24][24]);

#endif  // CNN_B200_COMPAT_LAYER_H
