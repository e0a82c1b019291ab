// The fused-network handle shared by the forward, training and host-pipeline translation units.
#pragma once

#include "cnn_common.cuh"

struct cnn_net {
  int device = 0;
  unsigned seed = 0;               // what cnn_net_create drew the initial parameters from (kept for checkpoints)
  int ps_kernel = 1;               // per-sample SGD: 1 = six-CTA cluster kernel (default), 0 = single persistent block
  int forward_path = -1;           // batched forward: 0 = exact fp32 SIMT kernel, 1 = tensor cores in three tf32 passes
                                   // (fp32-level accuracy), 2 = tensor cores, one tf32 pass + tanh sigmoid,
                                   // -1 (default) = 1 for batches of kTcMinBatch images or more, else 0
  float* d_params = nullptr;       // kNParamsPadded floats
  int* d_status = nullptr;         // device status word: 0 ok, non-zero = a bounded wait ran out
  int fast_sigmoid = 1;            // sigmoid of the fused kernels: 0 = reference expression, 1 = short form (default)

  // Training scratch (allocated on first use): per-block partial gradients and the reduced vector.
  float* d_partials = nullptr;     // [partial_rows][kNParamsPadded]
  int partial_rows = 0;
  float* d_grad = nullptr;         // kNParamsPadded floats + 8 floats of statistics
  // Host pipeline staging (allocated on first use).
  float* d_stage_img[2] = {nullptr, nullptr};
  float* d_stage_out[2] = {nullptr, nullptr};
  int* d_stage_arg[2] = {nullptr, nullptr};
  long stage_images = 0;
  cudaStream_t copy_stream[2] = {nullptr, nullptr};
  cudaEvent_t order_event = nullptr;   // host pipeline: ties the two copy streams behind the legacy stream
};

namespace cnn {

// ---- mbarrier / bulk-copy primitives (sm_90+ PTX, used in their non-multicast form only) ----
__device__ __forceinline__ unsigned smem_u32(const void* p) {
  return static_cast<unsigned>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// One arrival on an mbarrier of this CTA (release at CTA scope).
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 1-D bulk copy global -> this CTA's shared memory, completion signalled on an mbarrier.
// Both addresses must be 16-byte aligned and bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes,
                                         unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// Programmatic dependent launch: a kernel launched with launch_pdl() may start while its predecessor in the
// stream is still running, once every block of the predecessor has called pdl_launch_dependents() (or
// exited); whatever it reads of the predecessor's results must come after pdl_wait(), which returns when
// the predecessor has completed and its writes are visible.  Both are no-ops in an ordinary launch.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Per-thread asynchronous copies global -> shared (LDGSTS), 16 bytes (L2 only) or 4 bytes, and their groups.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after about two seconds of SM clocks, records it in *status and lets the
// caller carry on (with whatever the buffer holds) so that control flow stays uniform and the
// kernel always terminates.  Returns false once a wait has run out.
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, unsigned parity,
                                                  int* status, bool& gave_up) {
  if (gave_up) return false;
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > 4000000000LL) {
      gave_up = true;
      if (status) atomicExch(status, 1);
      return false;
    }
  }
  return true;
}

// Partial-gradient rows of the minibatch kernels: arena-ordered gradient [0, 2343), zero padding,
// and at kRowErr the sum over the row's images of ||delta_f||_2.
constexpr int kRowStride = kNParamsPadded + 8;
constexpr int kRowErr = kNParams + 1;  // 2344

// Batched forward with the convolution on the tensor cores (forward_tc.cu): net->forward_path 1 or 2.
int forward_device_tc(cnn_net* net, int path, const float* d_images, long n, float* d_out, int* d_argmax,
                      cudaStream_t stream);
int ensure_train_scratch(cnn_net* net, int rows);
// Blocks of the minibatch gradient kernel for a batch of n images (one partial row per block).
int grid_for_batch(long n);
// Fused forward + backward of n images at fixed parameters: `grid` partial rows into net->d_partials.
// `chained`: the kernel before this one on the stream is this library's reduce + update kernel of the previous
// step of the same call (then, and only then, the gradient kernel may fetch its first images before waiting
// for that kernel: see k_grad_partials).
int launch_grad_partials(cnn_net* net, const float* d_images, const unsigned* d_labels, long n, int grid,
                         cudaStream_t st, bool chained = false);
int launch_persample_cluster8(cnn_net* net, const float* d_images, const unsigned* d_labels, long n, int epochs,
                              float dt, float threshold, float* d_mean, int* d_ran, cudaStream_t st);

}  // namespace cnn
