// C ABI for the Layer object and the per-operator launchers (see include/cnn_b200.h).
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "layer_ops.cuh"

namespace cnn {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
  return CNN_ERR_CUDA;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// The reference launches every operator as <<<64,64>>>; these launchers size the grid for the
// operator instead (enough 128-thread blocks to give every output one thread or one warp).
static inline int blocks_for(int work_items, int threads = 128) {
  int b = (work_items + threads - 1) / threads;
  return b < 1 ? 1 : b;
}

namespace {
__global__ void k_apply_step_function(const float* in, float* out, int n) { ops::apply_step_function(in, out, n); }
__global__ void k_make_error(float* err, const float* out, unsigned y, int n) { ops::make_error(err, out, y, n); }
__global__ void k_apply_grad(float* w, const float* g, int n) { ops::apply_grad(w, g, n); }
__global__ void k_fp_preact_c1(const float* in, float* pre, const float* w) { ops::fp_preact_c1(in, pre, w); }
__global__ void k_fp_bias_c1(float* pre, const float* b) { ops::fp_bias_c1(pre, b); }
__global__ void k_fp_preact_s1(const float* in, float* pre, const float* w) { ops::fp_preact_s1(in, pre, w); }
__global__ void k_fp_bias_s1(float* pre, const float* b) { ops::fp_bias_s1(pre, b); }
__global__ void k_fp_preact_f(const float* in, float* pre, const float* w) { ops::fp_preact_f(in, pre, w); }
__global__ void k_fp_bias_f(float* pre, const float* b) { ops::fp_bias_f(pre, b); }
__global__ void k_bp_weight_f(float* dw, const float* dp, const float* po) { ops::bp_weight_f(dw, dp, po); }
__global__ void k_bp_bias_f(float* b, const float* dp) { ops::bp_bias_f(b, dp); }
__global__ void k_bp_output_s1(float* dout, const float* w, const float* ndp) { ops::bp_output_s1(dout, w, ndp); }
__global__ void k_bp_preact(float* dp, const float* dout, const float* pre, int n) { ops::bp_preact_generic(dp, dout, pre, n); }
__global__ void k_bp_weight_s1(float* dw, const float* dp, const float* po) { ops::bp_weight_s1(dw, dp, po); }
__global__ void k_bp_bias_s1(float* b, const float* dp) { ops::bp_bias_s1(b, dp); }
__global__ void k_bp_output_c1(float* dout, const float* w, const float* ndp) { ops::bp_output_c1(dout, w, ndp); }
__global__ void k_bp_weight_c1(float* dw, const float* dp, const float* po) { ops::bp_weight_c1(dw, dp, po); }
__global__ void k_bp_bias_c1(float* b, const float* dp) { ops::bp_bias_c1(b, dp); }
}  // namespace

static int finish_launch(const char* name) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("launch of %s failed: %d (%s)", name, (int)e, cudaGetErrorString(e));
    return CNN_ERR_CUDA;
  }
  return CNN_OK;
}

}  // namespace cnn

using namespace cnn;

struct cnn_layer {
  cnn_layer_view v;
};

extern "C" {

const char* cnn_last_error(void) { return cnn::g_err; }

const char* cnn_build_info(void) { return "cnn_b200 0.1 (sm_100a)"; }

int cnn_layer_create(int M, int N, int O, cnn_layer** out) {
  CNN_REQUIRE(out != nullptr, "cnn_layer_create: out is NULL");
  CNN_REQUIRE(M >= 0 && N >= 0 && O >= 0, "cnn_layer_create: negative dimension");
  *out = nullptr;
  cnn_layer* l = new (std::nothrow) cnn_layer();
  CNN_REQUIRE(l != nullptr, "cnn_layer_create: out of host memory");
  std::memset(&l->v, 0, sizeof(l->v));
  l->v.M = M; l->v.N = N; l->v.O = O;
  // Same draw order as Layer::Layer (layer.cu:19-27): bias[i], then the M weights of unit i.
  std::vector<float> hb((size_t)N), hw((size_t)M * (size_t)N);
  for (int i = 0; i < N; ++i) {
    hb[i] = 0.5f - float(rand()) / float(RAND_MAX);
    for (int j = 0; j < M; ++j) hw[(size_t)i * M + j] = 0.5f - float(rand()) / float(RAND_MAX);
  }
  const size_t so = sizeof(float) * (size_t)O, sn = sizeof(float) * (size_t)N,
               sw = sizeof(float) * (size_t)M * (size_t)N;
  cudaError_t e = cudaSuccess;
  auto alloc = [&](float** p, size_t bytes) {
    if (e == cudaSuccess && bytes) e = cudaMalloc(p, bytes);
  };
  alloc(&l->v.output, so); alloc(&l->v.preact, so);
  alloc(&l->v.bias, sn);   alloc(&l->v.weight, sw);
  alloc(&l->v.d_output, so); alloc(&l->v.d_preact, so); alloc(&l->v.d_weight, sw);
  if (e == cudaSuccess && sn) e = cudaMemcpy(l->v.bias, hb.data(), sn, cudaMemcpyHostToDevice);
  if (e == cudaSuccess && sw) e = cudaMemcpy(l->v.weight, hw.data(), sw, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    cnn_layer_destroy(l);
    return cuda_fail(e, "cnn_layer_create");
  }
  *out = l;
  return CNN_OK;
}

int cnn_layer_destroy(cnn_layer* l) {
  if (!l) return CNN_OK;
  cudaFree(l->v.output); cudaFree(l->v.preact); cudaFree(l->v.bias); cudaFree(l->v.weight);
  cudaFree(l->v.d_output); cudaFree(l->v.d_preact); cudaFree(l->v.d_weight);
  delete l;
  return CNN_OK;
}

int cnn_layer_set_output(cnn_layer* l, const float* h_data) {
  CNN_REQUIRE(l && h_data, "cnn_layer_set_output: NULL argument");
  if (l->v.O) CNN_CUDA(cudaMemcpy(l->v.output, h_data, sizeof(float) * (size_t)l->v.O, cudaMemcpyHostToDevice));
  return CNN_OK;
}

int cnn_layer_clear(cnn_layer* l) {
  CNN_REQUIRE(l, "cnn_layer_clear: NULL layer");
  const size_t so = sizeof(float) * (size_t)l->v.O;
  if (so) {
    CNN_CUDA(cudaMemsetAsync(l->v.output, 0, so, 0));
    CNN_CUDA(cudaMemsetAsync(l->v.preact, 0, so, 0));
  }
  return CNN_OK;
}

int cnn_layer_bp_clear(cnn_layer* l) {
  CNN_REQUIRE(l, "cnn_layer_bp_clear: NULL layer");
  const size_t so = sizeof(float) * (size_t)l->v.O;
  const size_t sw = sizeof(float) * (size_t)l->v.M * (size_t)l->v.N;
  if (so) {
    CNN_CUDA(cudaMemsetAsync(l->v.d_output, 0, so, 0));
    CNN_CUDA(cudaMemsetAsync(l->v.d_preact, 0, so, 0));
  }
  if (sw) CNN_CUDA(cudaMemsetAsync(l->v.d_weight, 0, sw, 0));
  return CNN_OK;
}

int cnn_layer_view_get(const cnn_layer* l, cnn_layer_view* out) {
  CNN_REQUIRE(l && out, "cnn_layer_view_get: NULL argument");
  *out = l->v;
  return CNN_OK;
}

#define REQ3(a, b, c, name) CNN_REQUIRE((a) && (b) && (c), name ": NULL device pointer")
#define REQ2(a, b, name) CNN_REQUIRE((a) && (b), name ": NULL device pointer")

int cnn_apply_step_function(const float* in, float* out, int n, void* s) {
  REQ2(in, out, "cnn_apply_step_function");
  CNN_REQUIRE(n >= 0, "cnn_apply_step_function: negative n");
  if (n == 0) return CNN_OK;
  k_apply_step_function<<<blocks_for(n), 128, 0, as_stream(s)>>>(in, out, n);
  return finish_launch("apply_step_function");
}

int cnn_make_error(float* err, const float* out, unsigned int label, int n, void* s) {
  REQ2(err, out, "cnn_make_error");
  CNN_REQUIRE(n >= 0, "cnn_make_error: negative n");
  if (n == 0) return CNN_OK;
  k_make_error<<<1, 32, 0, as_stream(s)>>>(err, out, label, n);
  return finish_launch("make_error");
}

int cnn_apply_grad(float* out, const float* grad, int n, void* s) {
  REQ2(out, grad, "cnn_apply_grad");
  CNN_REQUIRE(n >= 0, "cnn_apply_grad: negative n");
  if (n == 0) return CNN_OK;
  k_apply_grad<<<blocks_for(n), 128, 0, as_stream(s)>>>(out, grad, n);
  return finish_launch("apply_grad");
}

int cnn_fp_preact_c1(const float* in, float* pre, const float* w, void* s) {
  REQ3(in, pre, w, "cnn_fp_preact_c1");
  k_fp_preact_c1<<<blocks_for(kF * kC * kC), 128, 0, as_stream(s)>>>(in, pre, w);
  return finish_launch("fp_preact_c1");
}
int cnn_fp_bias_c1(float* pre, const float* b, void* s) {
  REQ2(pre, b, "cnn_fp_bias_c1");
  k_fp_bias_c1<<<blocks_for(kF * kC * kC), 128, 0, as_stream(s)>>>(pre, b);
  return finish_launch("fp_bias_c1");
}
int cnn_fp_preact_s1(const float* in, float* pre, const float* w, void* s) {
  REQ3(in, pre, w, "cnn_fp_preact_s1");
  k_fp_preact_s1<<<blocks_for(kS), 128, 0, as_stream(s)>>>(in, pre, w);
  return finish_launch("fp_preact_s1");
}
int cnn_fp_bias_s1(float* pre, const float* b, void* s) {
  REQ2(pre, b, "cnn_fp_bias_s1");
  k_fp_bias_s1<<<blocks_for(kS), 128, 0, as_stream(s)>>>(pre, b);
  return finish_launch("fp_bias_s1");
}
int cnn_fp_preact_f(const float* in, float* pre, const float* w, void* s) {
  REQ3(in, pre, w, "cnn_fp_preact_f");
  k_fp_preact_f<<<blocks_for(kOut * 32), 128, 0, as_stream(s)>>>(in, pre, w);
  return finish_launch("fp_preact_f");
}
int cnn_fp_bias_f(float* pre, const float* b, void* s) {
  REQ2(pre, b, "cnn_fp_bias_f");
  k_fp_bias_f<<<1, 32, 0, as_stream(s)>>>(pre, b);
  return finish_launch("fp_bias_f");
}

int cnn_bp_weight_f(float* dw, const float* dp, const float* po, void* s) {
  REQ3(dw, dp, po, "cnn_bp_weight_f");
  k_bp_weight_f<<<blocks_for(kOut * kS), 128, 0, as_stream(s)>>>(dw, dp, po);
  return finish_launch("bp_weight_f");
}
int cnn_bp_bias_f(float* b, const float* dp, void* s) {
  REQ2(b, dp, "cnn_bp_bias_f");
  k_bp_bias_f<<<1, 32, 0, as_stream(s)>>>(b, dp);
  return finish_launch("bp_bias_f");
}
int cnn_bp_output_s1(float* dout, const float* w, const float* ndp, void* s) {
  REQ3(dout, w, ndp, "cnn_bp_output_s1");
  k_bp_output_s1<<<blocks_for(kS), 128, 0, as_stream(s)>>>(dout, w, ndp);
  return finish_launch("bp_output_s1");
}
int cnn_bp_preact_s1(float* dp, const float* dout, const float* pre, void* s) {
  REQ3(dp, dout, pre, "cnn_bp_preact_s1");
  k_bp_preact<<<blocks_for(kS), 128, 0, as_stream(s)>>>(dp, dout, pre, kS);
  return finish_launch("bp_preact_s1");
}
int cnn_bp_weight_s1(float* dw, const float* dp, const float* po, void* s) {
  REQ3(dw, dp, po, "cnn_bp_weight_s1");
  k_bp_weight_s1<<<blocks_for(16 * 32), 128, 0, as_stream(s)>>>(dw, dp, po);
  return finish_launch("bp_weight_s1");
}
int cnn_bp_bias_s1(float* b, const float* dp, void* s) {
  REQ2(b, dp, "cnn_bp_bias_s1");
  k_bp_bias_s1<<<1, 32, 0, as_stream(s)>>>(b, dp);
  return finish_launch("bp_bias_s1");
}
int cnn_bp_output_c1(float* dout, const float* w, const float* ndp, void* s) {
  REQ3(dout, w, ndp, "cnn_bp_output_c1");
  k_bp_output_c1<<<blocks_for(kF * kC * kC), 128, 0, as_stream(s)>>>(dout, w, ndp);
  return finish_launch("bp_output_c1");
}
int cnn_bp_preact_c1(float* dp, const float* dout, const float* pre, void* s) {
  REQ3(dp, dout, pre, "cnn_bp_preact_c1");
  k_bp_preact<<<blocks_for(kF * kC * kC), 128, 0, as_stream(s)>>>(dp, dout, pre, kF * kC * kC);
  return finish_launch("bp_preact_c1");
}
int cnn_bp_weight_c1(float* dw, const float* dp, const float* po, void* s) {
  REQ3(dw, dp, po, "cnn_bp_weight_c1");
  k_bp_weight_c1<<<blocks_for(kF * 25 * 32), 128, 0, as_stream(s)>>>(dw, dp, po);
  return finish_launch("bp_weight_c1");
}
int cnn_bp_bias_c1(float* b, const float* dp, void* s) {
  REQ2(b, dp, "cnn_bp_bias_c1");
  k_bp_bias_c1<<<blocks_for(kF * 32), 128, 0, as_stream(s)>>>(b, dp);
  return finish_launch("bp_bias_c1");
}

}  // extern "C"
