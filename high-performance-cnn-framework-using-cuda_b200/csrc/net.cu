// Fused-network handle: parameter arena, status word, and the host-buffer forward pipeline.
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "net.cuh"

namespace cnn {
int forward_kernel_for(const cnn_net* net, long n_total);
int forward_device(cnn_net* net, int path, const float* d_images, long n, float* d_out, int* d_argmax,
                   cudaStream_t stream);
int forward_device_u8(cnn_net* net, const unsigned char* d_pixels, long n, float* d_out, int* d_argmax,
                      cudaStream_t stream);

int ensure_train_scratch(cnn_net* net, int rows) {
  if (!net->d_grad) CNN_CUDA(cudaMalloc(&net->d_grad, sizeof(float) * (kNParamsPadded + 8)));
  if (rows > net->partial_rows) {
    if (net->d_partials) CNN_CUDA(cudaFree(net->d_partials));
    net->d_partials = nullptr;
    net->partial_rows = 0;
    CNN_CUDA(cudaMalloc(&net->d_partials, sizeof(float) * (size_t)rows * (kNParamsPadded + 8)));
    net->partial_rows = rows;
  }
  return CNN_OK;
}

// Host pipeline: images per chunk.  8,192 images = 25.7 MB per copy, large enough to run the
// copy engine at full rate, small enough that the first kernel starts early.
constexpr long kStageImages = 8192;

static int ensure_stage(cnn_net* net) {
  if (net->stage_images) return CNN_OK;
  for (int s = 0; s < 2; ++s) {
    CNN_CUDA(cudaMalloc(&net->d_stage_img[s], sizeof(float) * kStageImages * kImg));
    CNN_CUDA(cudaMalloc(&net->d_stage_out[s], sizeof(float) * kStageImages * kOut));
    CNN_CUDA(cudaMalloc(&net->d_stage_arg[s], sizeof(int) * kStageImages));
    CNN_CUDA(cudaStreamCreateWithFlags(&net->copy_stream[s], cudaStreamNonBlocking));
  }
  CNN_CUDA(cudaEventCreateWithFlags(&net->order_event, cudaEventDisableTiming));
  net->stage_images = kStageImages;
  return CNN_OK;
}
}  // namespace cnn

using namespace cnn;

extern "C" {

int cnn_net_create(unsigned int seed, cnn_net** out) {
  CNN_REQUIRE(out != nullptr, "cnn_net_create: out is NULL");
  *out = nullptr;
  cnn_net* net = new (std::nothrow) cnn_net();
  CNN_REQUIRE(net != nullptr, "cnn_net_create: out of host memory");
  net->seed = seed;
  cudaError_t e = cudaGetDevice(&net->device);
  if (e == cudaSuccess) e = cudaMalloc(&net->d_params, sizeof(float) * kNParamsPadded);
  if (e == cudaSuccess) e = cudaMalloc(&net->d_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(net->d_status, 0, sizeof(int));
  if (e != cudaSuccess) {
    cnn_net_destroy(net);
    return cuda_fail(e, "cnn_net_create");
  }
  // Draw order of the reference's static Layer objects (main.cu:18-20 through layer.cu:19-27):
  // c1 (6 units: bias, 25 weights), s1 (1 unit: bias, 16 weights), f (10 units: bias, 216 weights).
  std::vector<float> h(kNParamsPadded, 0.f);
  srand(seed);
  auto draw = [] { return 0.5f - float(rand()) / float(RAND_MAX); };
  for (int i = 0; i < kF; ++i) {
    h[kOffBc + i] = draw();
    for (int j = 0; j < 25; ++j) h[kOffWc + i * 25 + j] = draw();
  }
  h[kOffBs] = draw();
  for (int j = 0; j < 16; ++j) h[kOffWs + j] = draw();
  for (int i = 0; i < kOut; ++i) {
    h[kOffBf + i] = draw();
    for (int j = 0; j < kS; ++j) h[kOffWf + i * kS + j] = draw();
  }
  e = cudaMemcpy(net->d_params, h.data(), sizeof(float) * kNParamsPadded, cudaMemcpyHostToDevice);
  // the upload and the status memset must have landed before a launch on a non-blocking stream
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cnn_net_destroy(net);
    return cuda_fail(e, "cnn_net_create: parameter upload");
  }
  *out = net;
  return CNN_OK;
}

int cnn_net_destroy(cnn_net* net) {
  if (!net) return CNN_OK;
  cudaFree(net->d_params);
  cudaFree(net->d_status);
  cudaFree(net->d_partials);
  cudaFree(net->d_grad);
  for (int s = 0; s < 2; ++s) {
    cudaFree(net->d_stage_img[s]);
    cudaFree(net->d_stage_out[s]);
    cudaFree(net->d_stage_arg[s]);
    if (net->copy_stream[s]) cudaStreamDestroy(net->copy_stream[s]);
  }
  if (net->order_event) cudaEventDestroy(net->order_event);
  delete net;
  return CNN_OK;
}

int cnn_net_set_params(cnn_net* net, const float* h_params) {
  CNN_REQUIRE(net && h_params, "cnn_net_set_params: NULL argument");
  // Wait for work in flight that may still read the old values, upload, and wait again: a copy from
  // pageable memory may return while its DMA is pending, and a launch on a non-blocking stream (the
  // host pipeline's, or the caller's) is not ordered behind it.
  CNN_CUDA(cudaDeviceSynchronize());
  CNN_CUDA(cudaMemcpy(net->d_params, h_params, sizeof(float) * kNParams, cudaMemcpyHostToDevice));
  CNN_CUDA(cudaDeviceSynchronize());
  return CNN_OK;
}

int cnn_net_get_params(cnn_net* net, float* h_params) {
  CNN_REQUIRE(net && h_params, "cnn_net_get_params: NULL argument");
  CNN_CUDA(cudaMemcpy(h_params, net->d_params, sizeof(float) * kNParams, cudaMemcpyDeviceToHost));
  return CNN_OK;
}

int cnn_net_params_device(cnn_net* net, float** d_params) {
  CNN_REQUIRE(net && d_params, "cnn_net_params_device: NULL argument");
  *d_params = net->d_params;
  return CNN_OK;
}

int cnn_net_set_fast_sigmoid(cnn_net* net, int enable) {
  CNN_REQUIRE(net, "cnn_net_set_fast_sigmoid: NULL net");
  net->fast_sigmoid = enable ? 1 : 0;
  return CNN_OK;
}

int cnn_net_set_option(cnn_net* net, const char* key, int value) {
  CNN_REQUIRE(net && key, "cnn_net_set_option: NULL argument");
  if (std::strcmp(key, "persample_kernel") == 0) {
    CNN_REQUIRE(value == 0 || value == 1, "cnn_net_set_option: persample_kernel takes 0 or 1");
    net->ps_kernel = value;
    return CNN_OK;
  }
  if (std::strcmp(key, "forward_path") == 0) {
    CNN_REQUIRE(value >= -1 && value <= 2, "cnn_net_set_option: forward_path takes -1 (by batch size), 0, 1 or 2");
    net->forward_path = value;
    return CNN_OK;
  }
  if (std::strcmp(key, "fast_sigmoid") == 0) {
    net->fast_sigmoid = value ? 1 : 0;
    return CNN_OK;
  }
  set_error("cnn_net_set_option: unknown option '%s'", key);
  return CNN_ERR_INVALID;
}

int cnn_net_status(cnn_net* net, int* status) {
  CNN_REQUIRE(net && status, "cnn_net_status: NULL argument");
  CNN_CUDA(cudaDeviceSynchronize());
  CNN_CUDA(cudaMemcpy(status, net->d_status, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status != 0) {
    set_error("a bounded device-side wait ran out (status %d)", *status);
    int zero = 0;
    CNN_CUDA(cudaMemcpy(net->d_status, &zero, sizeof(int), cudaMemcpyHostToDevice));
    return CNN_ERR_TIMEOUT;
  }
  return CNN_OK;
}

}  // extern "C"

static int forward_host_impl(cnn_net* net, const void* h_images, bool u8, long n, float* h_out,
                             int* h_argmax) {
  CNN_REQUIRE(net != nullptr, "cnn_forward_batched_host: NULL net");
  CNN_REQUIRE(n >= 0, "cnn_forward_batched_host: negative image count");
  if (n == 0) return CNN_OK;
  CNN_REQUIRE(h_images != nullptr, "cnn_forward_batched_host: NULL images");
  const size_t image_bytes = u8 ? (size_t)kImg : sizeof(float) * kImg;
  int rc = ensure_stage(net);
  if (rc != CNN_OK) return rc;
  // The pipeline runs on two private non-blocking streams.  Both are first put behind everything
  // queued so far on the legacy default stream (a parameter update, a training call), so that a
  // forward issued right after such work sees its result; work on a caller's own non-blocking
  // stream is NOT waited for (the caller synchronises that stream first).
  CNN_CUDA(cudaEventRecord(net->order_event, cudaStreamLegacy));
  CNN_CUDA(cudaStreamWaitEvent(net->copy_stream[0], net->order_event, 0));
  CNN_CUDA(cudaStreamWaitEvent(net->copy_stream[1], net->order_event, 0));
  // Two staging slots, one stream each: within a slot the copy-in, the kernel and the copy-out
  // are stream-ordered; the two slots overlap each other (H2D of chunk c+1 under the kernel and
  // D2H of chunk c).
  long done = 0;
  int slot = 0;
  const int path = forward_kernel_for(net, n);     // one kernel for the whole request, whatever the chunking
  while (done < n) {
    const long cnt = (n - done) < net->stage_images ? (n - done) : net->stage_images;
    cudaStream_t st = net->copy_stream[slot];
    CNN_CUDA(cudaMemcpyAsync(net->d_stage_img[slot],
                             static_cast<const unsigned char*>(h_images) + (size_t)done * image_bytes,
                             (size_t)cnt * image_bytes, cudaMemcpyHostToDevice, st));
    rc = u8 ? forward_device_u8(net, reinterpret_cast<const unsigned char*>(net->d_stage_img[slot]), cnt,
                                net->d_stage_out[slot], net->d_stage_arg[slot], st)
            : forward_device(net, path, net->d_stage_img[slot], cnt, net->d_stage_out[slot],
                             net->d_stage_arg[slot], st);
    if (rc != CNN_OK) return rc;
    if (h_out)
      CNN_CUDA(cudaMemcpyAsync(h_out + done * kOut, net->d_stage_out[slot],
                               sizeof(float) * (size_t)cnt * kOut, cudaMemcpyDeviceToHost, st));
    if (h_argmax)
      CNN_CUDA(cudaMemcpyAsync(h_argmax + done, net->d_stage_arg[slot], sizeof(int) * (size_t)cnt,
                               cudaMemcpyDeviceToHost, st));
    done += cnt;
    slot ^= 1;
  }
  CNN_CUDA(cudaStreamSynchronize(net->copy_stream[0]));
  CNN_CUDA(cudaStreamSynchronize(net->copy_stream[1]));
  int status = 0;
  CNN_CUDA(cudaMemcpy(&status, net->d_status, sizeof(int), cudaMemcpyDeviceToHost));
  if (status != 0) {
    set_error("cnn_forward_batched_host: a bounded device-side wait ran out");
    int zero = 0;
    cudaMemcpy(net->d_status, &zero, sizeof(int), cudaMemcpyHostToDevice);
    return CNN_ERR_TIMEOUT;
  }
  return CNN_OK;
}

int cnn_forward_batched_host(cnn_net* net, const float* h_images, long n, float* h_out, int* h_argmax) {
  return forward_host_impl(net, h_images, false, n, h_out, h_argmax);
}

int cnn_forward_batched_u8_host(cnn_net* net, const unsigned char* h_pixels, long n, float* h_out,
                                int* h_argmax) {
  return forward_host_impl(net, h_pixels, true, n, h_out, h_argmax);
}

