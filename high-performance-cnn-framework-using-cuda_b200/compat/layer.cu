// Definitions behind compat/layer.h: the Layer object and the nineteen operator kernels, each a
// thin __global__ wrapper around the atomic-free device bodies in csrc/layer_ops.cuh (the same
// bodies the C ABI launchers use).  Compile this file together with the caller's sources, as the
// reference compiles its own operator file with its driver.
#include "layer.h"

#include "../csrc/layer_ops.cuh"

namespace cnn {
// The shared header declares these for the C ABI library; the source-level drop-in is
// self-contained, so it carries its own minimal copies.
void set_error(const char*, ...) {}
int cuda_fail(cudaError_t, const char*) { return -2; }
int sm_count() { return 148; }
}  // namespace cnn

namespace {
cudaError_t g_first_error = cudaSuccess;
inline void note(cudaError_t e) {
  if (e != cudaSuccess && g_first_error == cudaSuccess) g_first_error = e;
}
__host__ __device__ inline const float* flat(const void* p) { return static_cast<const float*>(p); }
__host__ __device__ inline float* flat(void* p) { return static_cast<float*>(p); }
}  // namespace

cudaError_t Layer::last_error() { return g_first_error; }

Layer::Layer(int M_, int N_, int O_)
    : M(M_), N(N_), O(O_), output(nullptr), preact(nullptr), bias(nullptr), weight(nullptr),
      d_output(nullptr), d_preact(nullptr), d_weight(nullptr) {
  std::vector<float> hb((size_t)N), hw((size_t)M * (size_t)N);
  for (int unit = 0; unit < N; ++unit) {
    hb[unit] = 0.5f - float(rand()) / float(RAND_MAX);
    for (int k = 0; k < M; ++k) hw[(size_t)unit * M + k] = 0.5f - float(rand()) / float(RAND_MAX);
  }
  const size_t so = sizeof(float) * (size_t)O, sn = sizeof(float) * (size_t)N,
               sw = sizeof(float) * (size_t)M * (size_t)N;
  float** const o_sized[] = {&output, &preact, &d_output, &d_preact};
  for (float** p : o_sized) note(cudaMalloc(p, so));
  note(cudaMalloc(&bias, sn));
  note(cudaMalloc(&weight, sw));
  note(cudaMalloc(&d_weight, sw));
  if (sn) note(cudaMemcpy(bias, hb.data(), sn, cudaMemcpyHostToDevice));
  if (sw) note(cudaMemcpy(weight, hw.data(), sw, cudaMemcpyHostToDevice));
}

Layer::~Layer() {
  float* const all[] = {output, preact, bias, weight, d_output, d_preact, d_weight};
  for (float* p : all) cudaFree(p);
}

void Layer::setOutput(float* data) {
  note(cudaMemcpy(output, data, sizeof(float) * (size_t)O, cudaMemcpyHostToDevice));
}

void Layer::clear() {
  const size_t so = sizeof(float) * (size_t)O;
  note(cudaMemset(output, 0, so));
  note(cudaMemset(preact, 0, so));
}

void Layer::bp_clear() {
  const size_t so = sizeof(float) * (size_t)O;
  note(cudaMemset(d_output, 0, so));
  note(cudaMemset(d_preact, 0, so));
  note(cudaMemset(d_weight, 0, sizeof(float) * (size_t)M * (size_t)N));
}

namespace ops = cnn::ops;

__device__ float step_function(float v) { return cnn::sigmoidf<false>(v); }

__global__ void apply_step_function(float* input, float* output, const int N) { ops::apply_step_function(input, output, N); }
__global__ void makeError(float* err, float* output, unsigned int Y, const int N) { ops::make_error(err, output, Y, N); }
__global__ void apply_grad(float* output, float* grad, const int N) { ops::apply_grad(output, grad, N); }

__global__ void fp_preact_c1(float input[28][28], float preact[6][24][24], float weight[6][5][5]) {
  ops::fp_preact_c1(flat(input), flat(preact), flat(weight));
}
__global__ void fp_bias_c1(float preact[6][24][24], float bias[6]) { ops::fp_bias_c1(flat(preact), bias); }
__global__ void fp_preact_s1(float input[6][24][24], float preact[6][6][6], float weight[1][4][4]) {
  ops::fp_preact_s1(flat(input), flat(preact), flat(weight));
}
__global__ void fp_bias_s1(float preact[6][6][6], float bias[1]) { ops::fp_bias_s1(flat(preact), bias); }
__global__ void fp_preact_f(float input[6][6][6], float preact[10], float weight[10][6][6][6]) {
  ops::fp_preact_f(flat(input), preact, flat(weight));
}
__global__ void fp_bias_f(float preact[10], float bias[10]) { ops::fp_bias_f(preact, bias); }

__global__ void bp_weight_f(float d_weight[10][6][6][6], float d_preact[10], float p_output[6][6][6]) {
  ops::bp_weight_f(flat(d_weight), d_preact, flat(p_output));
}
__global__ void bp_bias_f(float bias[10], float d_preact[10]) { ops::bp_bias_f(bias, d_preact); }
__global__ void bp_output_s1(float d_output[6][6][6], float n_weight[10][6][6][6], float nd_preact[10]) {
  ops::bp_output_s1(flat(d_output), flat(n_weight), nd_preact);
}
__global__ void bp_preact_s1(float d_preact[6][6][6], float d_output[6][6][6], float preact[6][6][6]) {
  ops::bp_preact_generic(flat(d_preact), flat(d_output), flat(preact), cnn::kS);
}
__global__ void bp_weight_s1(float d_weight[1][4][4], float d_preact[6][6][6], float p_output[6][24][24]) {
  ops::bp_weight_s1(flat(d_weight), flat(d_preact), flat(p_output));
}
__global__ void bp_bias_s1(float bias[1], float d_preact[6][6][6]) { ops::bp_bias_s1(bias, flat(d_preact)); }
__global__ void bp_output_c1(float d_output[6][24][24], float n_weight[1][4][4], float nd_preact[6][6][6]) {
  ops::bp_output_c1(flat(d_output), flat(n_weight), flat(nd_preact));
}
__global__ void bp_preact_c1(float d_preact[6][24][24], float d_output[6][24][24], float preact[6][24][24]) {
  ops::bp_preact_generic(flat(d_preact), flat(d_output), flat(preact), cnn::kF * cnn::kC * cnn::kC);
}
__global__ void bp_weight_c1(float d_weight[6][5][5], float d_preact[6][24][24], float p_output[28][28]) {
  ops::bp_weight_c1(flat(d_weight), flat(d_preact), flat(p_output));
}
__global__ void bp_bias_c1(float bias[6], float d_preact[6][24][24]) { ops::bp_bias_c1(bias, flat(d_preact)); }
