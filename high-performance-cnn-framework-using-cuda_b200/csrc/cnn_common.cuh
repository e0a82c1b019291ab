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

__device__ __forceinline__ float exp2f_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// step_function, layer.cu:81-84.  Three flavours, selected at compile time:
//   0  the reference's own expression, compiled without fast-math (libdevice expf, IEEE divide):
//      equal pre-activations give bit-equal activations; about 21 instructions;
//   1  the short form: one multiply, ex2.approx.ftz, one add, rcp.approx.ftz -- four dependent
//      instructions, written with the flush-to-zero forms explicitly (the non-ftz forms that
//      __expf / __fdividef compile to without fast-math carry range checks and rescaling around
//      each special-function instruction); a flushed subnormal only ever turns an activation of
//      ~1e-38 into 0.  About 1e-6 relative from flavour 0 per evaluation for |v| <= 16 (the
//      multiplication by log2e is rounded before the exponential).  What the fused kernels of the 28x28 net use when
//      fast_sigmoid is set: on the network's outputs it is as close to the fp64 oracle as flavour 0
//      (2.1e-6 over 65,536 images);
//   2  the same two special-function instructions with the argument reduced in two FMA steps
//      (n = round(-v*log2e), r = -v - n*ln2 exactly) and one Newton step on the reciprocal: about 12
//      instructions, a few 1e-7 from flavour 0 per evaluation (selectable for the widened net).
template <int FLAVOR>
__device__ __forceinline__ float sigmoidf(float v) {
  if constexpr (FLAVOR == 1) {
    const float d = 1.0f + exp2f_approx(v * -1.4426950408889634f);
    float q;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(q) : "f"(d));
    return q;
  } else if constexpr (FLAVOR == 2) {
    const float x = fminf(fmaxf(-v, -87.0f), 87.0f);
    const float magic = 12582912.0f;                       // 1.5 * 2^23: adding it rounds to integer
    const float t = fmaf(x, 1.4426950408889634f, magic);
    const float n = t - magic;                              // round(x * log2e)
    float r = fmaf(n, -0.693145751953125f, x);              // x - n*ln2_hi (exact)
    r = fmaf(n, -1.4286068203094173e-6f, r);                // ... - n*ln2_lo
    const float m = exp2f_approx(r * 1.4426950408889634f);  // 2^(r*log2e), |r| <= 0.35
    const float e = __int_as_float(__float_as_int(m) + (__float_as_int(t) << 23));  // * 2^n
    const float d = 1.0f + e;
    float q;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(q) : "f"(d));
    const float err = fmaf(-d, q, 1.0f);
    return fmaf(q, err, q);
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

// Launch with programmatic stream serialization allowed: the kernel may begin (up to its pdl_wait()) while
// the kernel before it in the stream is still running.  Also valid under stream capture.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Number of SMs of the current device (cached per device).
int sm_count();

}  // namespace cnn
