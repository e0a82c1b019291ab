// Per-sample SGD (the reference's learn(), main.cu:125-170) on a thread-block cluster: the default
// kernel of cnn_train_sgd_persample.
//
// One SGD step depends on the previous step's parameters, so throughput is 1 / latency of a step.
// The step is spread over a cluster of six CTAs -- one feature map each -- that exchange only what
// the maps share: the FC partial sums (before the output layer) and the 17 partial sums of the
// shared subsample filter's gradient.  Both cross the cluster as one-way st.async stores into the
// receivers' shared memory, counted on the receivers' mbarriers: no cluster barrier, no release
// fence; exchange buffers and mbarriers alternate with the sample's parity and the data
// dependencies alone order buffer reuse.  Everything else (the map's conv filter and bias, its
// slice of the FC weights) is private to a CTA; the replicated parameters (subsample filter and
// bias, FC bias) are updated identically in every CTA, so they stay bit-identical.
//
// The CTA has four warps, one per scheduler of the SM:
//   warps 0..2  compute: thread (window, half) owns two rows of a 4x4 subsample window, i.e. eight
//               conv outputs on a 6x8 patch; 12 windows = 24 live lanes per warp;
//   warp 3      service: everything serial that is not arithmetic on the patch -- the previous
//               sample's subsample-filter update (it waits for the other CTAs' partials while the
//               compute warps convolve), issuing the bulk copy of the image after next and
//               observing the next image's arrival, the error norm, the conv-filter, conv-bias and
//               FC-bias steps.
// No warp shares a scheduler with another, each patch row is loaded half as often as with four
// outputs per thread, a window's rows are summed with one shuffle instead of two, and the compute
// warps send their FC partial sums themselves (no block barrier and no CTA-level sum before the
// exchange).  Three block barriers per sample (A: subsample filter updated, patch taken; B2: gradient
// partials in shared memory; E: conv filter updated).  While the FC partial sums are in flight the
// compute warps form their conv-filter gradient terms per unit of their window's delta (a thread's
// eight outputs share that delta), so only a scaling remains behind the output layer: measured on a
// B200, 1.49 us per sample against 1.58-1.62 with the terms computed after it.
#include <cooperative_groups.h>

#include "cluster_exchange.cuh"
#include "net.cuh"
#include "phase_clocks.cuh"

namespace cg = cooperative_groups;

namespace cnn {

// Sigmoid behind fast_sigmoid != 0: the short form (cnn_common.cuh).  This kernel is a chain of
// dependent latencies with three sigmoids in sequence per sample: 1.646 us per sample with it against
// 1.714 us with the refined twelve-instruction form, and the same distance from the oracle after 2,000
// steps (1.2e-5 of the largest parameter, set by summation order).
constexpr int kC8FastFlavor = 1;
constexpr int kC8Threads = 128;
constexpr int kC8Compute = 3;                 // compute warps
constexpr int kC8WinPerWarp = 12;
constexpr unsigned kC8FcBytes = kClCtas * kC8Compute * kOut * sizeof(float);   // 720 per receiver and sample

struct C8Smem {
  float img[2][kImg];
  float wc[28];                 // this map's 25 taps (padded for 128-bit loads)
  float bc[4];
  float ws[16];
  float bs[4];
  float wf[kOut][36];           // Wf[k][this map][window]
  float bf[12];
  float xfc[2][kClCtas][kC8Compute][16];   // FC partial sums of every compute warp of every CTA: outputs 0..4 at
                                           // [0..4], outputs 5..9 at [8..12] (two 16-byte aligned halves)
  float c_part[kC8Compute][28]; // per-warp conv-filter gradient partials (25) + conv-bias partial
  float s_part[kC8Compute][20]; // per-warp subsample-filter gradient partials (16) + bias partial
  float xws[2][kClCtas][20];    // subsample gradient partials of every CTA
  unsigned label[2];
  unsigned long long full[2];
  unsigned long long fc_bar[2];
  unsigned long long ws_bar[2];
  int flag[2];
  long long clock_base;         // phase timing only
};

CNN_PHASE_TABLE(g_phase_clocks8, 4)

template <int FLAVOR>
__global__ void __launch_bounds__(kC8Threads, 1)
k_train_persample_cluster8(const float* __restrict__ images, const unsigned* __restrict__ labels, long n,
                           int epochs, float dt, float threshold, float* __restrict__ params,
                           float* __restrict__ mean_err, int* __restrict__ epochs_run,
                           int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  C8Smem& sm = *reinterpret_cast<C8Smem*>(smem_raw);
  cg::cluster_group cluster = cg::this_cluster();
  const int f = (int)cluster.block_rank();   // this CTA's feature map
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool service = (warp == kC8Compute);
  const int slot = lane >> 1, half = lane & 1;
  const bool live = !service && slot < kC8WinPerWarp;
  const int win = live ? kC8WinPerWarp * warp + slot : 35;
  const int p = win / 6, q = win % 6;
  const int y0 = 4 * p + 2 * half, x0 = 4 * q;
  const int svc0 = kC8Compute * 32;          // first thread of the service warp

  if (tid < 28) sm.wc[tid] = (tid < 25) ? params[kOffWc + f * 25 + tid] : 0.f;
  if (tid == 0) { sm.bc[0] = params[kOffBc + f]; sm.bs[0] = params[kOffBs]; sm.flag[0] = 0; }
  if (tid < 16) sm.ws[tid] = params[kOffWs + tid];
  for (int i = tid; i < kOut * 36; i += kC8Threads)
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
  if (tid == svc0) {
    if (total > 0) issue(0, 0, labels[0]);
    if (total > 1) issue(1, 1 % n, labels[1 % n]);
    if (total > 0) {   // the first sample's exchanges are expected before anyone can send
      mbar_expect_tx(&sm.fc_bar[0], kC8FcBytes);
      mbar_expect_tx(&sm.ws_bar[0], kWsExchangeBytes);
    }
  }
  cluster.sync();  // every CTA's shared memory and mbarriers are initialised before anyone sends

  CNN_PHASE_BEGIN(f == 0, sm.clock_base)
  bool gave_up = false;
  bool pending = false;    // the previous sample's subsample-gradient exchange has not been consumed yet
  float err = 0.f;         // CTA 0, service lane 0: running sum of the epoch (a float, like main.cu:130)
  int done_epochs = 0;
  long step = 0;
  const float inv_c = 1.0f / (float)(kC * kC);
  const float inv_s = 1.0f / (float)kS;

  // Service warp: wait for the subsample-gradient partials of all CTAs of the sample before `step`,
  // apply the update.  Every CTA adds the same six values in the same order.
  auto finish_update = [&]() {
    if (!pending) return;   // uniform across the cluster
    if (service) {
      const int par = (int)((step - 1) & 1);
      mbar_wait_cluster_bounded(&sm.ws_bar[par], (unsigned)((step - 1) >> 1) & 1u, status, gave_up);
      if (lane < 17) {
        float sum = 0.f;
#pragma unroll
        for (int c = 0; c < kClCtas; ++c) sum += sm.xws[par][c][lane];
        if (lane < 16) sm.ws[lane] = fmaf(dt, sum, sm.ws[lane]);        // apply_grad (s1)
        else sm.bs[0] = fmaf(dt, sum, sm.bs[0]);                        // bp_bias_s1
      }
    }
    pending = false;
  };

  if (total > 0) mbar_wait_bounded(&sm.full[0], 0u, status, gave_up);   // the first image
  for (int e = 0; e < epochs; ++e) {
    for (long it = 0; it < n; ++it, ++step) {
      const int stage = (int)(step & 1);   // image buffer and parity of the exchange buffers
      long next_im = 0;
      unsigned next_label = 0;
      if (tid == svc0 && step + 2 < total) {
        next_im = it + 2;
        while (next_im >= n) next_im -= n;
        next_label = labels[next_im];
      }
      const unsigned label = sm.label[stage];
      CNN_PHASE(0);     // top of the loop

      // ---- forward: eight conv outputs (rows y0, y0+1; columns x0..x0+3) of map f ------------------
      float pt[6][8];
      float a[2][4];
      if (!service) {
        const float* src = &sm.img[stage][y0 * kH + x0];
#pragma unroll
        for (int ii = 0; ii < 6; ++ii) {
          const float4 lo = *reinterpret_cast<const float4*>(src + ii * kH);
          const float4 hi = *reinterpret_cast<const float4*>(src + ii * kH + 4);
          pt[ii][0] = lo.x; pt[ii][1] = lo.y; pt[ii][2] = lo.z; pt[ii][3] = lo.w;
          pt[ii][4] = hi.x; pt[ii][5] = hi.y; pt[ii][6] = hi.z; pt[ii][7] = hi.w;
        }
        float w[28];
#pragma unroll
        for (int t = 0; t < 7; ++t) {
          const float4 v = *reinterpret_cast<const float4*>(&sm.wc[4 * t]);
          w[4 * t] = v.x; w[4 * t + 1] = v.y; w[4 * t + 2] = v.z; w[4 * t + 3] = v.w;
        }
        float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int jj = 0; jj < 5; ++jj)
#pragma unroll
          for (int ii = 0; ii < 5; ++ii)
#pragma unroll
            for (int rr = 0; rr < 2; ++rr)
#pragma unroll
              for (int c = 0; c < 4; ++c) acc[rr][c] = fmaf(w[ii * 5 + jj], pt[rr + ii][c + jj], acc[rr][c]);
        const float b = sm.bc[0];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr)
#pragma unroll
          for (int c = 0; c < 4; ++c) a[rr][c] = sigmoidf<FLAVOR>(acc[rr][c] + b);
      } else {
#pragma unroll
        for (int ii = 0; ii < 6; ++ii)
#pragma unroll
          for (int c = 0; c < 8; ++c) pt[ii][c] = 0.f;
#pragma unroll
        for (int rr = 0; rr < 2; ++rr)
#pragma unroll
          for (int c = 0; c < 4; ++c) a[rr][c] = 0.f;
      }
      CNN_PHASE(1);     // compute: patch loads, convolution, eight sigmoids
      finish_update();   // service warp, under the compute warps' convolution
      CNN_PHASE(2);     // at barrier A
      __syncthreads();   // (A) that update is visible; every thread has taken its patch and the label

      float wsv[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      float wfk[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
      float as = 0.f;
      float h[26];       // the thread's conv-filter gradient terms per unit of its window's subsample delta
#pragma unroll
      for (int t = 0; t < 26; ++t) h[t] = 0.f;
      if (service) {
        if (lane == 0 && step + 2 < total) issue(stage, next_im, next_label);
        // the next sample's image: this warp observes its arrival, the block barriers below hand that
        // on to the compute warps, and nobody waits for it at the top of the loop
        if (step + 1 < total)
          mbar_wait_bounded(&sm.full[stage ^ 1], (unsigned)((step + 1) >> 1) & 1u, status, gave_up);
      } else {
        // subsample: rows 2*half and 2*half+1 of the window, then the other half's two rows
        float zs = 0.f;
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          const float4 v = *reinterpret_cast<const float4*>(&sm.ws[4 * (2 * half + rr)]);
          wsv[rr][0] = v.x; wsv[rr][1] = v.y; wsv[rr][2] = v.z; wsv[rr][3] = v.w;
          float zr = wsv[rr][0] * a[rr][0];
          zr = fmaf(wsv[rr][1], a[rr][1], zr); zr = fmaf(wsv[rr][2], a[rr][2], zr); zr = fmaf(wsv[rr][3], a[rr][3], zr);
          zs = (rr == 0) ? zr : zs + zr;
        }
        zs += __shfl_xor_sync(0xffffffffu, zs, 1);
        as = sigmoidf<FLAVOR>(zs + sm.bs[0]);
        // FC: the window's two lanes split the outputs, k = 5 * half + j; then the warp's windows
        float pk[5];
#pragma unroll
        for (int j = 0; j < 5; ++j) {
          wfk[j] = live ? sm.wf[5 * half + j][win] : 0.f;
          pk[j] = wfk[j] * as;
        }
#pragma unroll
        for (int m = 2; m <= 16; m <<= 1)
#pragma unroll
          for (int j = 0; j < 5; ++j) pk[j] += __shfl_xor_sync(0xffffffffu, pk[j], m);
        // every lane now holds the warp's sums for its five outputs: lane 2c + half sends them to CTA c
        // as one 16-byte store and one 4-byte store (two transactions on the receiver's mbarrier)
        if (lane < 2 * kClCtas) {
          const unsigned dst = (unsigned)(lane >> 1);
          const unsigned bar = cluster_addr(&sm.fc_bar[stage], dst);
          const unsigned to = cluster_addr(&sm.xfc[stage][f][warp][8 * half], dst);
          st_async_f32x4(to, pk[0], pk[1], pk[2], pk[3], bar);
          st_async_f32(to + 16u, pk[4], bar);
        }
        // While the partial sums are in flight: everything of the conv-filter gradient that does not need the
        // output layer.  The thread's eight outputs belong to one window, so their conv deltas are that
        // window's subsample delta times cf = Ws * a (1 - a) / 576, and the thread's gradient terms are the
        // delta times h = sum cf * patch: 200 of the backward pass's FMAs leave the dependent chain.
        float cf[2][4];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr)
#pragma unroll
          for (int c = 0; c < 4; ++c) cf[rr][c] = wsv[rr][c] * a[rr][c] * (1.f - a[rr][c]) * inv_c;
#pragma unroll
        for (int ii = 0; ii < 5; ++ii)
#pragma unroll
          for (int jj = 0; jj < 5; ++jj) {
            float s = cf[0][0] * pt[ii][jj];
#pragma unroll
            for (int c = 1; c < 4; ++c) s = fmaf(cf[0][c], pt[ii][c + jj], s);
#pragma unroll
            for (int c = 0; c < 4; ++c) s = fmaf(cf[1][c], pt[1 + ii][c + jj], s);
            h[ii * 5 + jj] = s;
          }
        h[25] = ((cf[0][0] + cf[0][1]) + (cf[0][2] + cf[0][3])) + ((cf[1][0] + cf[1][1]) + (cf[1][2] + cf[1][3]));
      }

      // ---- (C1) the partial sums of all 18 compute warps have landed here ---------------------------
      CNN_PHASE(3);     // compute: subsample, sigmoid, FC partials sent; service: image issued / observed
      mbar_wait_cluster_bounded(&sm.fc_bar[stage], (unsigned)(step >> 1) & 1u, status, gave_up);
      CNN_PHASE(4);     // exchange complete
      // Expect the next sample's exchanges now: the other barrier pair's previous phases are complete
      // (waited for one sample ago and at the top of this one), and nobody can send for the next
      // sample before this CTA's subsample partials of this one, which go out after barrier B2.
      if (tid == svc0 && step + 1 < total) {
        mbar_expect_tx(&sm.fc_bar[stage ^ 1], kC8FcBytes);
        mbar_expect_tx(&sm.ws_bar[stage ^ 1], kWsExchangeBytes);
      }

      // ---- output layer on lanes 0..9 of every warp ------------------------------------------------
      float delta = 0.f;
      if (lane < kOut) {
        float z = 0.f;
#pragma unroll
        for (int c = 0; c < kClCtas; ++c) {
          float zc = 0.f;
#pragma unroll
          for (int ww = 0; ww < kC8Compute; ++ww) zc += sm.xfc[stage][c][ww][lane < 5 ? lane : lane + 3];
          z += zc;
        }
        z += sm.bf[lane];
        const float o = sigmoidf<FLAVOR>(z);
        delta = ((label == (unsigned)lane) ? 1.0f : 0.0f) - o;   // makeError
      }

      CNN_PHASE(5);     // output layer
      if (service) {
        // the sample's error norm, while the compute warps run the backward pass
        float sq = delta * delta;   // zero on lanes >= 10
#pragma unroll
        for (int m = 8; m > 0; m >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, m);
        if (lane == 0) err += sqrtf(sq);
      } else {
        // ---- backward ----------------------------------------------------------------------------
        float d[5];
#pragma unroll
        for (int j = 0; j < 5; ++j) d[j] = __shfl_sync(0xffffffffu, delta, 5 * half + j);
        float das = wfk[0] * d[0];
#pragma unroll
        for (int j = 1; j < 5; ++j) das = fmaf(wfk[j], d[j], das);
        das += __shfl_xor_sync(0xffffffffu, das, 1);
        const float delta_s = live ? das * as * (1.f - as) : 0.f;
        if (live) {
#pragma unroll
          for (int j = 0; j < 5; ++j) sm.wf[5 * half + j][win] = fmaf(dt, d[j] * as, wfk[j]);  // bp_weight_f + apply_grad
        }
        // subsample filter gradient: this thread's two filter rows, reduce-scattered over the warp's
        // 16 window slots (lane bits 4, 3, 2 pick the element, bit 1 is summed last); bias term
        float gs[8];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr)
#pragma unroll
          for (int c = 0; c < 4; ++c) gs[rr * 4 + c] = delta_s * a[rr][c];
        float gb = (half == 0) ? delta_s * inv_s : 0.f;
#pragma unroll
        for (int keep_n = 4; keep_n >= 1; keep_n >>= 1) {
          const int mask = keep_n << 2;   // 16, 8, 4
          const bool upper = (lane & mask) != 0;
#pragma unroll
          for (int i = 0; i < keep_n; ++i) {
            const float send = upper ? gs[i] : gs[i + keep_n];
            const float keep = upper ? gs[i + keep_n] : gs[i];
            gs[i] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
          }
        }
        gs[0] += __shfl_xor_sync(0xffffffffu, gs[0], 2);
#pragma unroll
        for (int m = 2; m <= 16; m <<= 1) gb += __shfl_xor_sync(0xffffffffu, gb, m);
        if ((lane & 2) == 0) {
          const int idx = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);   // rr * 4 + c
          sm.s_part[warp][(2 * half + (idx >> 2)) * 4 + (idx & 3)] = gs[0];
        }
        if (lane == 0) sm.s_part[warp][16] = gb;
        // the thread's 25 filter-gradient terms and its bias term: the window's delta times what was
        // prepared under the exchange
        float g[32];
#pragma unroll
        for (int t = 0; t < 26; ++t) g[t] = delta_s * h[t];
        CNN_PHASE(6);   // deltas, subsample gradient, the thread's gradient terms
#pragma unroll
        for (int t = 26; t < 32; ++t) g[t] = 0.f;
        const float mine = warp_reduce_scatter32(g, lane);
        if (lane < 26) sm.c_part[warp][lane] = mine;
      }
      // (the service warp is the last to leave the stretch between B2 and E: what it can read or
      // compute before B2 it does here, while it waits for the compute warps anyway)
      float w_old = 0.f, bf_new = 0.f;
      if (service) {
        w_old = (lane < 25) ? sm.wc[lane] : sm.bc[0];
        if (lane < kOut) bf_new = fmaf(dt, delta, sm.bf[lane]);          // bp_bias_f, stored after B2: a compute
      }                                                                  // warp may still be reading bf before it
      CNN_PHASE(7);     // at barrier B2 (compute: reduce-scatter done; service: error norm done)
      __syncthreads();  // (B2)

      if (service) {
        if (lane < 26) {
          const float sum = (sm.c_part[0][lane] + sm.c_part[1][lane]) + sm.c_part[2][lane];
          if (lane < 25) sm.wc[lane] = fmaf(dt, sum, w_old);             // apply_grad (c1)
          else sm.bc[0] = fmaf(dt, sum, w_old);                          // bp_bias_c1
        }
        if (lane < kOut) sm.bf[lane] = bf_new;
      } else if (warp == 0 && lane < 17) {
        float sum = 0.f;
#pragma unroll
        for (int ww = 0; ww < kC8Compute; ++ww) sum += sm.s_part[ww][lane];
#pragma unroll
        for (int c = 0; c < kClCtas; ++c)
          st_async_f32(cluster_addr(&sm.xws[stage][f][lane], c), sum, cluster_addr(&sm.ws_bar[stage], c));
      }
      CNN_PHASE(8);     // at barrier E
      __syncthreads();  // (E) this CTA's updates of wc / bc / bf are ordered before its next convolution
      pending = true;
    }
    // epoch end, main.cu:159-166: every CTA must take the same branch
    finish_update();
    if (f == 0 && tid == svc0) {
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
  if (tid == svc0) {
    for (long s2 = step; s2 < total && s2 < step + 2; ++s2)
      mbar_wait_bounded(&sm.full[s2 & 1], (unsigned)(s2 >> 1) & 1u, status, gave_up);
  }
  __syncthreads();
  if (tid < 25) params[kOffWc + f * 25 + tid] = sm.wc[tid];
  if (tid == 0) params[kOffBc + f] = sm.bc[0];
  for (int i = tid; i < kOut * 36; i += kC8Threads)
    params[kOffWf + (i / 36) * kS + f * 36 + (i % 36)] = sm.wf[i / 36][i % 36];
  if (f == 0) {
    if (tid < 16) params[kOffWs + tid] = sm.ws[tid];
    if (tid == 0) params[kOffBs] = sm.bs[0];
    if (tid < kOut) params[kOffBf + tid] = sm.bf[tid];
    if (tid == 0 && epochs_run) *epochs_run = done_epochs;
  }
  CNN_PHASE_END(g_phase_clocks8);
}

template <int FLAVOR>
static int launch_cluster8_flavor(const float* d_images, const unsigned* d_labels, long n, int epochs, float dt,
                                  float threshold, float* d_params, float* d_mean, int* d_ran, int* d_status,
                                  cudaStream_t st) {
  auto kernel = k_train_persample_cluster8<FLAVOR>;
  CNN_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(C8Smem)));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kClCtas, 1, 1);
  cfg.blockDim = dim3(kC8Threads, 1, 1);
  cfg.dynamicSmemBytes = sizeof(C8Smem);
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

int launch_persample_cluster8(cnn_net* net, const float* d_images, const unsigned* d_labels, long n, int epochs,
                              float dt, float threshold, float* d_mean, int* d_ran, cudaStream_t st) {
  if (net->fast_sigmoid)
    return launch_cluster8_flavor<kC8FastFlavor>(d_images, d_labels, n, epochs, dt, threshold, net->d_params, d_mean, d_ran, net->d_status, st);
  return launch_cluster8_flavor<0>(d_images, d_labels, n, epochs, dt, threshold, net->d_params, d_mean, d_ran, net->d_status, st);
}

}  // namespace cnn

#ifdef CNN_PHASE_CLOCKS
extern "C" int cnn_debug_phase_clocks8(long long* out /* [4][16] */) {
  return cudaMemcpyFromSymbol(out, cnn::g_phase_clocks8, sizeof(cnn::g_phase_clocks8)) == cudaSuccess ? 0 : 2;
}
#endif
