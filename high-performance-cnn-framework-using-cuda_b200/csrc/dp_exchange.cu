// Data-parallel minibatch SGD over the GPUs of one box: the gradient exchange fused into the kernel
// that reduces a GPU's partial-gradient rows and applies the update.
//
// The reference trains on one GPU (main.cu:125-170 is the whole loop; there is no collective
// anywhere in layer.cu / main.cu).  Here every rank computes the summed gradient of its slice of a
// global batch (k_grad_partials), and ONE kernel per step then
//   1. adds the rank's partial rows in fixed order (what k_reduce_rows does),
//   2. stores the resulting 2,368-float vector into a per-source slot of EVERY rank's exchange
//      buffer through peer-mapped memory (NVLink).  Every element travels as ONE naturally aligned
//      64-bit store carrying the value in its low half and the step number in its high half, so a
//      word is its own arrival flag: no fence, no separate flag store, no second round trip,
//   3. polls -- bounded -- its OWN buffer until every rank's word of this step has landed,
//   4. adds the values in rank order (so every rank computes bit-identical sums) and applies
//      params += scale * sum.
// No TMA, no multicast, no load from a peer's memory: remote data always lands in the local buffer
// first and is read from there.  A 9.5 KB all-reduce is pure latency; this replaces NCCL's launch,
// protocol and second kernel by one one-way trip over NVLink inside a kernel that has to run anyway.
//
// Granularity: the kernel's blocks own 32 columns each and never talk to each other; a lane only
// waits for its own column of the other ranks.  Step numbers live in device memory (one counter per block,
// advanced by the block itself), so a captured CUDA graph of steps can be replayed.  Slots alternate
// with the step's parity: a rank can only be one step ahead of the slowest rank (it needs that
// rank's data to finish a step), and its stores of step s+1 go to the other parity while a slow
// rank may still be reading step s.
#include <cstring>
#include <new>

#include "net.cuh"

namespace cnn {

constexpr int kDpMaxRanks = 8;
constexpr int kDpBlocks = (kNParamsPadded + 31) / 32;   // 74 blocks of 32 columns
constexpr int kDpRedGroups = 32;   // row groups per column: 1,024 threads per block, at most ~10 dependent adds per thread

// Exchange buffer of one rank (device memory of that rank; every rank maps all of them).
struct DpBuffer {
  // [step parity][source rank][column]: value bits | step number << 32 (zero = nothing yet; steps count from 1)
  unsigned long long slot[2][kDpMaxRanks][kRowStride];
  unsigned step[kDpBlocks];                    // local only: steps completed by block b of this rank
};

struct DpPeers {
  DpBuffer* buf[kDpMaxRanks];
};

// A naturally aligned 64-bit scalar access is single-copy atomic: a reader sees the whole word of
// one store or none of it, never the step number of one store with the value of another.
__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// rows [n_rows][kRowStride] -> this rank's vector -> all ranks -> sum over ranks -> update.
// send == 0 is host-side fault injection for the tests: the rank keeps its vector to itself (its own
// slot included), so that every rank's bounded wait runs out.
__global__ void __launch_bounds__(32 * kDpRedGroups)
k_reduce_exchange_update(const float* __restrict__ rows, int n_rows, DpPeers peers, DpBuffer* mine, int rank, int world,
                         float* __restrict__ params, float scale, float* __restrict__ G,
                         float* __restrict__ mean_err, float err_scale, long long wait_clocks, int send,
                         int* __restrict__ status) {
  __shared__ float part[kDpRedGroups][33];
  const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int b = blockIdx.x;
  const int col = b * 32 + lane;
  // (`mine` is this rank's own buffer, peers.buf[rank], passed separately: the pointer table is a kernel
  // parameter and only compile-time indices keep it out of local memory -- with a 64-byte stack frame
  // for it this kernel took 12 us instead of 6)
  pdl_launch_dependents();   // the next step's gradient kernel may set itself up now
  pdl_wait();                // this step's rows are complete
  unsigned seq = 0;
  if (world > 1 && g == 0) seq = mine->step[b] + 1u;   // written only by this block, one launch ago; in flight under the row sums
  float acc = 0.f;
  if (col < kRowStride) {
#pragma unroll 4
    for (int r = g; r < n_rows; r += kDpRedGroups) acc += rows[(size_t)r * kRowStride + col];
  }
  part[g][lane] = acc;
  __syncthreads();
  if (g != 0) return;

  float total;
  {
    float q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      q[i] = (part[4 * i][lane] + part[4 * i + 1][lane]) + (part[4 * i + 2][lane] + part[4 * i + 3][lane]);
    total = ((q[0] + q[1]) + (q[2] + q[3])) + ((q[4] + q[5]) + (q[6] + q[7]));
  }
  if (world == 1) {
    // a single rank has nobody to exchange with: reduce + update, no flags, no system-scope fences
    if (col < kRowStride) {
      if (G) G[col] = total;
      if (col < kNParams) params[col] = fmaf(scale, total, params[col]);
      if (mean_err && col == kRowErr) *mean_err += err_scale * total;
    }
    return;
  }
  const int parity = (int)(seq & 1u);
  if (send && col < kRowStride) {
    const unsigned long long word = (unsigned long long)__float_as_uint(total) | ((unsigned long long)seq << 32);
#pragma unroll
    for (int r = 0; r < kDpMaxRanks; ++r)
      if (r < world) st_relaxed_sys_u64(&peers.buf[r]->slot[parity][rank][col], word);
  }
  // ---- collect every rank's word of this step for this lane's column (own buffer only), bounded ----
  bool ok = true;
  float sum = 0.f;
  if (col < kRowStride) {
    long long t0 = 0;
    unsigned spins = 0;
    for (int r = 0; r < world && ok; ++r) {
      const unsigned long long* w = &mine->slot[parity][r][col];
      unsigned long long v = ld_relaxed_sys_u64(w);
      while ((unsigned)(v >> 32) != seq) {
        if (t0 == 0) t0 = clock64();
        // a wait that ran out anywhere on this GPU ends the others soon after
        const bool other = ((++spins & 255u) == 0) && *reinterpret_cast<volatile int*>(status) != 0;
        if (other || clock64() - t0 > wait_clocks) {
          ok = false;
          break;
        }
        v = ld_relaxed_sys_u64(w);
      }
      sum += __uint_as_float((unsigned)v);     // rank order: every rank adds the same values in the same order
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  if (!ok) {
    if (lane == 0) {
      atomicExch(status, 2);
      mine->step[b] = seq;
    }
    return;   // parameters are left as they are: the step is reported as failed, not half applied
  }
  if (col < kRowStride) {
    if (G) G[col] = sum;
    if (col < kNParams) params[col] = fmaf(scale, sum, params[col]);
    if (mean_err && col == kRowErr) *mean_err += err_scale * sum;
  }
  __syncwarp();
  if (lane == 0) mine->step[b] = seq;
}

}  // namespace cnn

struct cnn_dp {
  cnn_net* net = nullptr;
  int rank = 0, world = 1;
  cnn::DpBuffer* local = nullptr;
  cnn::DpPeers peers = {};
  bool ipc_opened[cnn::kDpMaxRanks] = {};
  bool connected = false;
  int wait_limit_ms = 2000;
  int drop_next_send = 0;
  int clock_khz = 1965000;
};

using namespace cnn;

extern "C" {

int cnn_dp_create(cnn_net* net, int rank, int world, cnn_dp** out) {
  CNN_REQUIRE(out != nullptr, "cnn_dp_create: out is NULL");
  *out = nullptr;
  CNN_REQUIRE(net != nullptr, "cnn_dp_create: NULL net");
  CNN_REQUIRE(world >= 1 && world <= kDpMaxRanks, "cnn_dp_create: world must be 1..8 (the GPUs of one box)");
  CNN_REQUIRE(rank >= 0 && rank < world, "cnn_dp_create: rank out of range");
  cnn_dp* dp = new (std::nothrow) cnn_dp();
  CNN_REQUIRE(dp != nullptr, "cnn_dp_create: out of host memory");
  dp->net = net;
  dp->rank = rank;
  dp->world = world;
  cudaError_t e = cudaMalloc(&dp->local, sizeof(DpBuffer));
  if (e == cudaSuccess) e = cudaMemset(dp->local, 0, sizeof(DpBuffer));
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&dp->clock_khz, cudaDevAttrClockRate, net->device);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cudaFree(dp->local);
    delete dp;
    return cuda_fail(e, "cnn_dp_create");
  }
  dp->peers.buf[rank] = dp->local;
  dp->connected = (world == 1);
  *out = dp;
  return CNN_OK;
}

int cnn_dp_destroy(cnn_dp* dp) {
  if (!dp) return CNN_OK;
  cudaDeviceSynchronize();
  for (int r = 0; r < dp->world; ++r)
    if (dp->ipc_opened[r]) cudaIpcCloseMemHandle(dp->peers.buf[r]);
  cudaFree(dp->local);
  delete dp;
  return CNN_OK;
}

int cnn_dp_export_handle(cnn_dp* dp, void* handle) {
  CNN_REQUIRE(dp && handle, "cnn_dp_export_handle: NULL argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == CNN_DP_HANDLE_BYTES, "IPC handle size");
  cudaIpcMemHandle_t h;
  CNN_CUDA(cudaIpcGetMemHandle(&h, dp->local));
  std::memcpy(handle, &h, sizeof(h));
  return CNN_OK;
}

int cnn_dp_connect(cnn_dp* dp, const void* handles) {
  CNN_REQUIRE(dp && (handles || dp->world == 1), "cnn_dp_connect: NULL argument");
  for (int r = 0; r < dp->world; ++r) {
    if (r == dp->rank || dp->peers.buf[r]) continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, static_cast<const unsigned char*>(handles) + (size_t)r * CNN_DP_HANDLE_BYTES, sizeof(h));
    void* p = nullptr;
    CNN_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    dp->peers.buf[r] = static_cast<DpBuffer*>(p);
    dp->ipc_opened[r] = true;
  }
  dp->connected = true;
  return CNN_OK;
}

int cnn_dp_local_buffer(cnn_dp* dp, void** d_buffer) {
  CNN_REQUIRE(dp && d_buffer, "cnn_dp_local_buffer: NULL argument");
  *d_buffer = dp->local;
  return CNN_OK;
}

int cnn_dp_connect_pointers(cnn_dp* dp, void* const* d_buffers) {
  CNN_REQUIRE(dp && (d_buffers || dp->world == 1), "cnn_dp_connect_pointers: NULL argument");
  for (int r = 0; r < dp->world; ++r) {
    if (r == dp->rank) continue;
    CNN_REQUIRE(d_buffers[r] != nullptr, "cnn_dp_connect_pointers: NULL peer buffer");
    dp->peers.buf[r] = static_cast<DpBuffer*>(d_buffers[r]);
  }
  dp->connected = true;
  return CNN_OK;
}

int cnn_dp_set_option(cnn_dp* dp, const char* key, int value) {
  CNN_REQUIRE(dp && key, "cnn_dp_set_option: NULL argument");
  if (std::strcmp(key, "wait_limit_ms") == 0) {
    CNN_REQUIRE(value >= 1 && value <= 60000, "cnn_dp_set_option: wait_limit_ms takes 1..60000");
    dp->wait_limit_ms = value;
    return CNN_OK;
  }
  if (std::strcmp(key, "drop_next_send") == 0) {
    dp->drop_next_send = value ? 1 : 0;
    return CNN_OK;
  }
  set_error("cnn_dp_set_option: unknown option '%s'", key);
  return CNN_ERR_INVALID;
}

static int dp_step(cnn_dp* dp, const float* d_images, const unsigned int* d_labels, long n_local, float scale,
                   float* d_grad_sum, float* d_mean_err, float err_scale, void* stream, bool chained) {
  CNN_REQUIRE(dp != nullptr, "cnn_dp_step: NULL handle");
  CNN_REQUIRE(dp->connected, "cnn_dp_step: cnn_dp_connect has not been called");
  CNN_REQUIRE(n_local >= 0, "cnn_dp_step: negative image count");
  cnn_net* net = dp->net;
  cudaStream_t st = as_stream(stream);
  int rc = ensure_train_scratch(net, 2 * sm_count());
  if (rc != CNN_OK) return rc;
  int grid = 0;
  if (n_local > 0) {
    CNN_REQUIRE(d_images && d_labels, "cnn_dp_step: NULL images or labels");
    CNN_REQUIRE((reinterpret_cast<uintptr_t>(d_images) & 15u) == 0,
                "cnn_dp_step: image batch must start on a 16-byte boundary");
    grid = grid_for_batch(n_local);
    if ((rc = launch_grad_partials(net, d_images, d_labels, n_local, grid, st, chained)) != CNN_OK) return rc;
  }
  const long long wait_clocks = (long long)dp->wait_limit_ms * dp->clock_khz;
  const int send = dp->drop_next_send ? 0 : 1;
  dp->drop_next_send = 0;
  cudaError_t e = launch_pdl(k_reduce_exchange_update, dim3(kDpBlocks), dim3(32 * kDpRedGroups), 0, st,
                             (const float*)net->d_partials, grid, dp->peers, dp->local, dp->rank, dp->world, net->d_params,
                             scale, d_grad_sum, d_mean_err, err_scale, wait_clocks, send, net->d_status);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "k_reduce_exchange_update launch");
  return CNN_OK;
}

int cnn_dp_step(cnn_dp* dp, const float* d_images, const unsigned int* d_labels, long n_local, float scale,
                float* d_grad_sum, float* d_mean_err, float err_scale, void* stream) {
  return dp_step(dp, d_images, d_labels, n_local, scale, d_grad_sum, d_mean_err, err_scale, stream, false);
}

int cnn_train_minibatch_dp(cnn_dp* dp, const float* d_images, const unsigned int* d_labels, long n,
                           long global_batch, int epochs, float dt, float* d_mean_err, void* stream) {
  CNN_REQUIRE(dp != nullptr, "cnn_train_minibatch_dp: NULL handle");
  CNN_REQUIRE(n >= 0 && global_batch > 0 && epochs >= 0, "cnn_train_minibatch_dp: bad sizes");
  if (n == 0 || epochs == 0) return CNN_OK;
  CNN_REQUIRE(d_images && d_labels, "cnn_train_minibatch_dp: NULL images or labels");
  cudaStream_t st = as_stream(stream);
  if (d_mean_err) CNN_CUDA(cudaMemsetAsync(d_mean_err, 0, sizeof(float) * (size_t)epochs, st));
  for (int e = 0; e < epochs; ++e) {
    for (long first = 0; first < n; first += global_batch) {
      const long size = (n - first) < global_batch ? (n - first) : global_batch;
      // this rank's contiguous slice of the global batch (sizes differ by at most one image)
      const long lo = size * dp->rank / dp->world, hi = size * (dp->rank + 1) / dp->world;
      int rc = dp_step(dp, d_images + (first + lo) * kImg, d_labels + first + lo, hi - lo, dt / (float)size,
                       nullptr, d_mean_err ? d_mean_err + e : nullptr, 1.0f / (float)n, stream, first > 0 || e > 0);
      if (rc != CNN_OK) return rc;
    }
  }
  return CNN_OK;
}

}  // extern "C"
