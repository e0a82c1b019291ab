// Per-sample SGD (the reference's learn(), main.cu:125-170) on a thread-block cluster.
//
// One SGD step depends on the previous step's parameters, so throughput is 1 / latency of a step.
// A single SM cannot finish a step (190 k FMAs, 7.4 k sigmoids) in much less than 5 us; this kernel
// spreads the step over a cluster of six CTAs -- one feature map each -- that exchange only what the
// maps share: the ten FC partial sums (before the output layer) and the 17 partial sums of the
// shared subsample filter's gradient, through distributed shared memory.  Everything else (the
// map's conv filter and bias, its slice of the FC weights) is private to a CTA.  The replicated
// parameters (subsample filter and bias, FC bias) are updated identically in every CTA (same
// values, same order), so they stay bit-identical.
//
// Two exchanges per sample.  With hardware cluster barriers (EXCHANGE = 1) the second barrier is
// split into arrive / wait around the next sample's convolution, which needs none of the exchanged
// values, so only the first is exposed.  With one-way stores (EXCHANGE = 2) every value travels as
// an st.async that counts its bytes on an mbarrier of the receiving CTA; receivers wait on their
// own mbarrier only, there is no barrier round trip and no release fence, and the buffers alternate
// with the sample's parity.  The data dependencies alone order the reuse of a buffer: a CTA cannot
// send the FC partials of sample i+1 before it has every CTA's subsample partials of sample i, which
// a CTA sends only after it has read the FC partials of sample i (and likewise the other way).
//
// Thread (window, row): four x-adjacent conv outputs of one row of a 4x4 subsample window,
// t = 4 * window + row, 144 live threads in a 160-thread CTA.  Four outputs per thread keep the
// warp-shuffle traffic (one shuffle per cycle per SM) low: the 26 conv-gradient partials of a thread
// are accumulated over its four outputs in registers before the warp-wide reduce-scatter.
#include <cooperative_groups.h>

#include "cluster_exchange.cuh"
#include "net.cuh"

namespace cg = cooperative_groups;

namespace cnn {

constexpr int kClThreads = 160;
constexpr int kClLive = 144;
constexpr int kClWarps = kClThreads / 32;    // 5

struct ClSmem {
  float img[2][kImg];
  float wc[28];                 // this map's 25 taps (padded for 128-bit loads)
  float bc[4];
  float ws[16];
  float bs[4];
  float wf[kOut][36];           // Wf[k][this map][window]
  float bf[12];
  float fc_part[kClWarps][12];  // per-warp FC partial sums
  float xfc[2][kClCtas][12];    // FC partial sums of every CTA (written remotely), by sample parity
  float c_part[kClWarps][28];   // per-warp conv-filter gradient partials (25) + conv-bias partial
  float s_part[kClWarps][20];   // per-warp subsample-filter gradient partials (16) + bias partial
  float xws[2][kClCtas][20];    // subsample gradient partials of every CTA (written remotely)
  unsigned label[2];
  unsigned long long full[2];
  unsigned long long fc_bar[2]; // one-way exchange: bytes of xfc[parity] that have landed
  unsigned long long ws_bar[2]; // one-way exchange: bytes of xws[parity] that have landed
  int flag[2];
  long long clock_base;         // phase timing only
};

constexpr unsigned kFcExchangeBytes = kClCtas * kOut * sizeof(float);   // 240 per receiver and sample

// Optional phase timing for tuning (off unless the file is compiled with -DCNN_PHASE_CLOCKS): lane 0
// of every warp of CTA 0 sums, over the samples, the SM clock at each stamp (relative to the clock at
// kernel start, one counter per SM); means per stamp and warp put all warps on one time axis.
#ifdef CNN_PHASE_CLOCKS
__device__ long long g_phase_clocks[kClWarps][16];
#define CNN_PHASE(i)                                                     \
  do {                                                                   \
    if (f == 0 && lane == 0) {                                           \
      long long now_;                                                    \
      asm volatile("mov.u64 %0, %%clock64;" : "=l"(now_)::"memory");     \
      ph_[i] += now_ - base_;                                            \
    }                                                                    \
  } while (0)
#else
#define CNN_PHASE(i) do { } while (0)
#endif

template <int FLAVOR, int EXCHANGE>
__global__ void __launch_bounds__(kClThreads, 1)
k_train_persample_cluster(const float* __restrict__ images, const unsigned* __restrict__ labels, long n,
                          int epochs, float dt, float threshold, float* __restrict__ params,
                          float* __restrict__ mean_err, int* __restrict__ epochs_run,
                          int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  ClSmem& sm = *reinterpret_cast<ClSmem*>(smem_raw);
  cg::cluster_group cluster = cg::this_cluster();
  const int f = (int)cluster.block_rank();   // this CTA's feature map
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool live = tid < kClLive;
  const int win = live ? (tid >> 2) : 35;
  const int r = tid & 3;
  const int p = win / 6, q = win % 6;
  const int y = 4 * p + r, x0 = 4 * q;
  constexpr bool kOneWay = (EXCHANGE == 2);

  if (tid < 28) sm.wc[tid] = (tid < 25) ? params[kOffWc + f * 25 + tid] : 0.f;
  if (tid == 0) { sm.bc[0] = params[kOffBc + f]; sm.bs[0] = params[kOffBs]; sm.flag[0] = 0; }
  if (tid < 16) sm.ws[tid] = params[kOffWs + tid];
  for (int i = tid; i < kOut * 36; i += kClThreads)
    sm.wf[i / 36][i % 36] = params[kOffWf + (i / 36) * kS + f * 36 + (i % 36)];
  if (tid < kOut) sm.bf[tid] = params[kOffBf + tid];
  if (tid == 0) {
    mbar_init(&sm.full[0], 1);
    mbar_init(&sm.full[1], 1);
    mbar_init(&sm.fc_bar[0], 1);
    mbar_init(&sm.fc_bar[1], 1);
    mbar_init(&sm.ws_bar[0], 1);
    mbar_init(&sm.ws_bar[1], 1);
    mbar_fence_init();
  }
  __syncthreads();

  const long total = (long)epochs * n;
  auto issue = [&](int stage, long im, unsigned lab) {
    mbar_expect_tx(&sm.full[stage], kImg * sizeof(float));
    bulk_g2s(&sm.img[stage][0], images + im * kImg, kImg * sizeof(float), &sm.full[stage]);
    sm.label[stage] = lab;
  };
  if (tid == 0) {
    if (total > 0) issue(0, 0, labels[0]);
    if (total > 1) issue(1, 1 % n, labels[1 % n]);
    if (kOneWay && total > 0) {   // the first sample's exchanges are expected before anyone can send
      mbar_expect_tx(&sm.fc_bar[0], kFcExchangeBytes);
      mbar_expect_tx(&sm.ws_bar[0], kWsExchangeBytes);
    }
  }
  cluster.sync();  // every CTA's shared memory is initialised before anyone writes into it remotely

#ifdef CNN_PHASE_CLOCKS
  long long ph_[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
  if (tid == 0) sm.clock_base = clock64();
  __syncthreads();
  const long long base_ = sm.clock_base;
#endif
  bool gave_up = false;
  bool pending = false;    // a split cluster barrier has been arrived at and not yet waited for
  float err = 0.f;         // CTA 0, warp 3, lane 0: running sum of the epoch (a float, like main.cu:130)
  int done_epochs = 0;
  long step = 0;
  const float inv_c = 1.0f / (float)(kC * kC);
  const float inv_s = 1.0f / (float)kS;

  // Second half of a step: wait for the subsample-gradient partials of all CTAs, apply the update.
  // `step` is one past the sample whose exchange is pending at both call sites.
  auto finish_update = [&]() {
    if (!pending) return;   // uniform across the cluster
    const int par = (int)((step - 1) & 1);
    if (kOneWay) {
      // only the readers wait; the others are held by the block / cluster barrier that follows
      if (warp == 1) mbar_wait_cluster_bounded(&sm.ws_bar[par], (unsigned)((step - 1) >> 1) & 1u, status, gave_up);
    } else {
      cluster.barrier_wait();
    }
    // warp 1 has its scheduler to itself (warps 0 and 4 share one and finish the convolution later)
    if (tid >= 32 && tid < 32 + 17) {
      const int t = tid - 32;
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < kClCtas; ++c) sum += sm.xws[par][c][t];
      if (t < 16) sm.ws[t] = fmaf(dt, sum, sm.ws[t]);                 // apply_grad (s1)
      else sm.bs[0] = fmaf(dt, sum, sm.bs[0]);                        // bp_bias_s1
    }
    pending = false;
  };

  if (total > 0) mbar_wait_bounded(&sm.full[0], 0u, status, gave_up);   // the first image
  for (int e = 0; e < epochs; ++e) {
    for (long it = 0; it < n; ++it, ++step) {
      const int stage = (int)(step & 1);   // also the parity of the exchange buffers
      // thread 0 fetches the label of the sample after next now; the load is long done when the
      // stage is re-issued below
      long next_im = 0;
      unsigned next_label = 0;
      if (tid == 0 && step + 2 < total) {
        next_im = it + 2;
        while (next_im >= n) next_im -= n;
        next_label = labels[next_im];
      }
      CNN_PHASE(0);   // loop top; the image is there (first sample: waited for before the loop,
                      // later ones: by warp 4 ahead of the previous sample's last barrier)
      const unsigned label = sm.label[stage];
      CNN_PHASE(1);

      // ---- forward: four conv outputs (y, x0..x0+3) of map f -----------------------------------
      float pt[5][8];
      {
        const float* src = &sm.img[stage][y * kH + x0];
#pragma unroll
        for (int ii = 0; ii < 5; ++ii) {
          const float4 lo = *reinterpret_cast<const float4*>(src + ii * kH);
          const float4 hi = *reinterpret_cast<const float4*>(src + ii * kH + 4);
          pt[ii][0] = lo.x; pt[ii][1] = lo.y; pt[ii][2] = lo.z; pt[ii][3] = lo.w;
          pt[ii][4] = hi.x; pt[ii][5] = hi.y; pt[ii][6] = hi.z; pt[ii][7] = hi.w;
        }
      }
      float a[4];
      {
        float w[28];
#pragma unroll
        for (int t = 0; t < 7; ++t) {
          const float4 v = *reinterpret_cast<const float4*>(&sm.wc[4 * t]);
          w[4 * t] = v.x; w[4 * t + 1] = v.y; w[4 * t + 2] = v.z; w[4 * t + 3] = v.w;
        }
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int jj = 0; jj < 5; ++jj)
#pragma unroll
          for (int ii = 0; ii < 5; ++ii)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[c] = fmaf(w[ii * 5 + jj], pt[ii][c + jj], acc[c]);
        const float b = sm.bc[0];
#pragma unroll
        for (int c = 0; c < 4; ++c) a[c] = sigmoidf<FLAVOR>(acc[c] + b);
      }
      CNN_PHASE(2);      // patch loads, convolution, four sigmoids
      finish_update();   // previous sample's subsample-filter update (its barrier was split)
      CNN_PHASE(3);
      __syncthreads();   // that update is visible; every thread has taken its patch and the label
      CNN_PHASE(4);
      if (tid == 0 && step + 2 < total) issue(stage, next_im, next_label);

      // subsample: row r of the window, then the window's four rows
      const float4 wsr = *reinterpret_cast<const float4*>(&sm.ws[4 * r]);
      float zs = wsr.x * a[0];
      zs = fmaf(wsr.y, a[1], zs); zs = fmaf(wsr.z, a[2], zs); zs = fmaf(wsr.w, a[3], zs);
      zs += __shfl_xor_sync(0xffffffffu, zs, 1);
      zs += __shfl_xor_sync(0xffffffffu, zs, 2);
      const float as = sigmoidf<FLAVOR>(zs + sm.bs[0]);
      // FC: lane r of a window handles outputs k = r, r+4, r+8 (< 10); then the warp's 8 windows
      float wfk[3], pk[3];
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        const int k = r + 4 * j;
        wfk[j] = (live && k < kOut) ? sm.wf[k][win] : 0.f;
        pk[j] = wfk[j] * as;
      }
#pragma unroll
      for (int m = 4; m <= 16; m <<= 1)
#pragma unroll
        for (int j = 0; j < 3; ++j) pk[j] += __shfl_xor_sync(0xffffffffu, pk[j], m);
      if (lane < 4) {
#pragma unroll
        for (int j = 0; j < 3; ++j)
          if (lane + 4 * j < kOut) sm.fc_part[warp][lane + 4 * j] = pk[j];
      }
      CNN_PHASE(5);     // subsample, sigmoid, FC partials
      __syncthreads();  // (B1)
      CNN_PHASE(6);

      // ---- CTA partial of the output layer, sent to every CTA --------------------------------
      if (warp == 0) {
        float zc = 0.f;
        if (lane < kOut) {
#pragma unroll
          for (int ww = 0; ww < kClWarps; ++ww) zc += sm.fc_part[ww][lane];
        }
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          const int idx = lane + 32 * rr;         // (destination CTA, k)
          const float v = __shfl_sync(0xffffffffu, zc, idx % kOut);
          if (idx < kClCtas * kOut) {
            float* slot = &sm.xfc[stage][f][idx % kOut];
            if (kOneWay)
              st_async_f32(cluster_addr(slot, idx / kOut), v, cluster_addr(&sm.fc_bar[stage], idx / kOut));
            else
              *cluster.map_shared_rank(slot, idx / kOut) = v;
          }
        }
      }
      // (C1) all six partials have landed everywhere / here
      CNN_PHASE(7);     // CTA partial and its sends
      if (kOneWay) {
        mbar_wait_cluster_bounded(&sm.fc_bar[stage], (unsigned)(step >> 1) & 1u, status, gave_up);
        CNN_PHASE(8);   // exposed exchange
        // Expect the next sample's exchanges now: the other barrier pair's previous phases are
        // complete (waited for one sample ago and earlier in this one), and nobody can send
        // for the next sample before this CTA's subsample partials of this one, sent further down.
        if (tid == 0 && step + 1 < total) {
          mbar_expect_tx(&sm.fc_bar[stage ^ 1], kFcExchangeBytes);
          mbar_expect_tx(&sm.ws_bar[stage ^ 1], kWsExchangeBytes);
        }
      } else {
        cluster.sync();
      }

      // ---- output layer on lanes 0..9 of every warp --------------------------------------------
      float delta = 0.f;
      if (lane < kOut) {
        float z = 0.f;
#pragma unroll
        for (int c = 0; c < kClCtas; ++c) z += sm.xfc[stage][c][lane];
        z += sm.bf[lane];
        const float o = sigmoidf<FLAVOR>(z);
        delta = ((label == (unsigned)lane) ? 1.0f : 0.0f) - o;   // makeError
      }
      float d[3];
#pragma unroll
      for (int j = 0; j < 3; ++j) d[j] = __shfl_sync(0xffffffffu, delta, r + 4 * j);  // lanes 10, 11 hold 0

      CNN_PHASE(9);     // output layer
      // ---- backward --------------------------------------------------------------------------
      float das = wfk[0] * d[0];
      das = fmaf(wfk[1], d[1], das); das = fmaf(wfk[2], d[2], das);
      das += __shfl_xor_sync(0xffffffffu, das, 1);
      das += __shfl_xor_sync(0xffffffffu, das, 2);
      const float delta_s = live ? das * as * (1.f - as) : 0.f;
      if (live) {
#pragma unroll
        for (int j = 0; j < 3; ++j)
          if (r + 4 * j < kOut) sm.wf[r + 4 * j][win] = fmaf(dt, d[j] * as, wfk[j]);  // bp_weight_f + apply_grad
      }
      // subsample filter gradient: row r of the filter, summed over the warp's 8 windows; bias term
      float gs[5];
#pragma unroll
      for (int c = 0; c < 4; ++c) gs[c] = delta_s * a[c];
      gs[4] = (r == 0) ? delta_s * inv_s : 0.f;
#pragma unroll
      for (int m = 4; m <= 16; m <<= 1)
#pragma unroll
        for (int c = 0; c < 5; ++c) gs[c] += __shfl_xor_sync(0xffffffffu, gs[c], m);
      if (lane < 4) {
#pragma unroll
        for (int c = 0; c < 4; ++c) sm.s_part[warp][4 * lane + c] = gs[c];
        if (lane == 0) sm.s_part[warp][16] = gs[4];
      }
      // conv deltas of the four outputs and the thread's 25 filter-gradient terms (+ bias term)
      const float wsv[4] = {wsr.x, wsr.y, wsr.z, wsr.w};
      float dc[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) dc[c] = (wsv[c] * delta_s) * a[c] * (1.f - a[c]) * inv_c;
      float g[32];
#pragma unroll
      for (int ii = 0; ii < 5; ++ii)
#pragma unroll
        for (int jj = 0; jj < 5; ++jj) {
          float s = dc[0] * pt[ii][jj];
#pragma unroll
          for (int c = 1; c < 4; ++c) s = fmaf(dc[c], pt[ii][c + jj], s);
          g[ii * 5 + jj] = s;
        }
      g[25] = (dc[0] + dc[1]) + (dc[2] + dc[3]);
#pragma unroll
      for (int t = 26; t < 32; ++t) g[t] = 0.f;
      CNN_PHASE(10);    // deltas and the thread's gradient terms
      const float mine = warp_reduce_scatter32(g, lane);
      if (lane < 26) sm.c_part[warp][lane] = mine;
      if (warp == 3) {
        // warp 3 reaches the barrier well before warps 0 and 4 (which share a scheduler): the
        // sample's error norm costs nothing here (every warp holds delta_f on its lanes 0..9)
        float sq = delta * delta;   // zero on lanes >= 10
#pragma unroll
        for (int m = 8; m > 0; m >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, m);
        if (lane == 0) err += sqrtf(sq);
      }
      CNN_PHASE(11);    // reduce-scatter
      __syncthreads();  // (B2)
      CNN_PHASE(12);

      if (tid < 26) {
        float sum = 0.f;
#pragma unroll
        for (int ww = 0; ww < kClWarps; ++ww) sum += sm.c_part[ww][tid];
        if (tid < 25) sm.wc[tid] = fmaf(dt, sum, sm.wc[tid]);          // apply_grad (c1)
        else sm.bc[0] = fmaf(dt, sum, sm.bc[0]);                        // bp_bias_c1
      } else if (warp == 3) {
        if (lane < kOut) sm.bf[lane] = fmaf(dt, delta, sm.bf[lane]);    // bp_bias_f
      } else if (warp == 4) {
        // the next sample's image: one idle warp observes its arrival, the barrier below hands
        // that on to the others, and nobody waits for it at the top of the loop
        if (step + 1 < total)
          mbar_wait_bounded(&sm.full[stage ^ 1], (unsigned)((step + 1) >> 1) & 1u, status, gave_up);
      } else if (tid >= 32 && tid < 32 + 17) {
        const int t = tid - 32;
        float sum = 0.f;
#pragma unroll
        for (int ww = 0; ww < kClWarps; ++ww) sum += sm.s_part[ww][t];
#pragma unroll
        for (int c = 0; c < kClCtas; ++c) {
          float* slot = &sm.xws[stage][f][t];
          if (kOneWay) st_async_f32(cluster_addr(slot, c), sum, cluster_addr(&sm.ws_bar[stage], c));
          else *cluster.map_shared_rank(slot, c) = sum;
        }
      }
      // (C2, split) arrive now; the wait sits after the next sample's convolution.  This CTA's own
      // updates of wc / bc / bf are ordered before its next convolution by the __syncthreads.
      CNN_PHASE(13);    // conv-filter update / subsample partial sends
      __syncthreads();
      CNN_PHASE(14);
      if (!kOneWay) cluster.barrier_arrive();
      pending = true;
    }
    // epoch end, main.cu:159-166: every CTA must take the same branch
    finish_update();
    if (f == 0 && tid == 96) {
      const float m = err / (float)n;
      if (mean_err) mean_err[e] = m;
      err = 0.f;
      const int stop = (m < threshold) ? 1 : 0;
      for (int c = 0; c < kClCtas; ++c) *cluster.map_shared_rank(&sm.flag[0], c) = stop;
    }
    done_epochs = e + 1;
    cluster.sync();
    const int stop = sm.flag[0];
    cluster.sync();  // everyone has read the flag before CTA 0 may overwrite it next epoch
    if (stop) break;
  }

  // After an early stop up to two prefetched images are still on their way into this CTA's shared
  // memory: the CTA does not exit under them.
  if (tid == 0) {
    for (long s2 = step; s2 < total && s2 < step + 2; ++s2)
      mbar_wait_bounded(&sm.full[s2 & 1], (unsigned)(s2 >> 1) & 1u, status, gave_up);
  }
  __syncthreads();
  if (tid < 25) params[kOffWc + f * 25 + tid] = sm.wc[tid];
  if (tid == 0) params[kOffBc + f] = sm.bc[0];
  for (int i = tid; i < kOut * 36; i += kClThreads)
    params[kOffWf + (i / 36) * kS + f * 36 + (i % 36)] = sm.wf[i / 36][i % 36];
  if (f == 0) {
    if (tid < 16) params[kOffWs + tid] = sm.ws[tid];
    if (tid == 0) params[kOffBs] = sm.bs[0];
    if (tid < kOut) params[kOffBf + tid] = sm.bf[tid];
    if (tid == 0 && epochs_run) *epochs_run = done_epochs;
  }
#ifdef CNN_PHASE_CLOCKS
  if (f == 0 && lane == 0)
    for (int i = 0; i < 16; ++i) g_phase_clocks[warp][i] = ph_[i];
#endif
}

template <int FLAVOR, int EXCHANGE>
static int launch_cluster_flavor(const float* d_images, const unsigned* d_labels, long n, int epochs,
                                 float dt, float threshold, float* d_params, float* d_mean, int* d_ran,
                                 int* d_status, cudaStream_t st) {
  auto kernel = k_train_persample_cluster<FLAVOR, EXCHANGE>;
  CNN_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(ClSmem)));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kClCtas, 1, 1);
  cfg.blockDim = dim3(kClThreads, 1, 1);
  cfg.dynamicSmemBytes = sizeof(ClSmem);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kClCtas;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CNN_CUDA(cudaLaunchKernelEx(&cfg, kernel, d_images, d_labels, n, epochs, dt, threshold, d_params, d_mean,
                              d_ran, d_status));
  return CNN_OK;
}

int launch_persample_cluster(cnn_net* net, const float* d_images, const unsigned* d_labels, long n, int epochs,
                             float dt, float threshold, float* d_mean, int* d_ran, cudaStream_t st) {
#define CNN_CLUSTER_CASE(FL, EX)                                                                              \
  return launch_cluster_flavor<FL, EX>(d_images, d_labels, n, epochs, dt, threshold, net->d_params, d_mean, \
                                       d_ran, net->d_status, st)
  if (net->ps_cluster == 2) {
    switch (net->fast_sigmoid) {
      case 1: CNN_CLUSTER_CASE(1, 2);
      case 2: CNN_CLUSTER_CASE(2, 2);
      default: CNN_CLUSTER_CASE(0, 2);
    }
  }
  switch (net->fast_sigmoid) {
    case 1: CNN_CLUSTER_CASE(1, 1);
    case 2: CNN_CLUSTER_CASE(2, 1);
    default: CNN_CLUSTER_CASE(0, 1);
  }
#undef CNN_CLUSTER_CASE
}

}  // namespace cnn

#ifdef CNN_PHASE_CLOCKS
extern "C" int cnn_debug_phase_clocks(long long* out32 /* [5][16] */) {
  return cudaMemcpyFromSymbol(out32, cnn::g_phase_clocks, sizeof(cnn::g_phase_clocks)) == cudaSuccess ? 0 : 2;
}
#endif
