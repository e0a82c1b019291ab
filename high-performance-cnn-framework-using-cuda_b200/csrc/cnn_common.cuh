// Shared definitions for the sm_100a CNN kernels: network dimensions, the parameter arena,
// the sigmoid, and host-side error plumbing.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/cnn_b200.h"

namespace cnn {

// Reference net (main.cu:17-20): input 28x28, 6 maps of 5x5, conv output 24x24, 4x4/stride-4
// subsample to 6x6, FC 216 -> 10.
constexpr int kH = 28;
constexpr int kF = 6;
constexpr int kC = 24;
constexpr int kP = 6;
constexpr int kS = kF * kP * kP;  // 216
constexpr int kOut = 10;
constexpr int kImg = kH * kH;     // 784

// Parameter arena offsets.
constexpr int kOffWc = 0;
constexpr int kOffBc = 150;
constexpr int kOffWs = 156;
constexpr int kOffBs = 172;
constexpr int kOffWf = 173;
constexpr int kOffBf = 2333;
constexpr int kNParams = 2343;
constexpr int kNParamsPadded = 2368;  // multiple of 32 floats

constexpr float kDt = 1.0e-1f;  // layer.h:11

// step_function, layer.cu:81-84.  The exact flavour is the reference's own expression, compiled
// without fast-math, so equal pre-activations give bit-equal activations.
template <bool FAST>
__device__ __forceinline__ float sigmoidf(float v) {
  if constexpr (FAST) {
    return __fdividef(1.0f, 1.0f + __expf(-v));
  } else {
    return 1.0f / (1.0f + expf(-v));
  }
}

// ---- host-side error plumbing ---------------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define CNN_CUDA(call)                                         \
  do {                                                         \
    cudaError_t e__ = (call);                                  \
    if (e__ != cudaSuccess) return ::cnn::cuda_fail(e__, #call); \
  } while (0)

#define CNN_REQUIRE(cond, msg)        \
  do {                                \
    if (!(cond)) {                    \
      ::cnn::set_error("%s", msg);    \
      return CNN_ERR_INVALID;         \
    }                                 \
  } while (0)

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// Number of SMs of the current device (cached per device).
int sm_count();

}  // namespace cnn
