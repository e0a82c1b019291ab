// Fused forward + backward kernels.
//
//  * k_grad_partials  -- minibatch mode: every block walks a strided subset of the batch, keeps the
//    gradient of its images in registers, reduces it inside the block with warp shuffles / shared
//    memory (no atomics) and writes one partial row; k_reduce_rows adds the rows in fixed order and
//    optionally applies the update.  Replaces, per image, forward_pass + makeError + back_pass
//    (main.cu:67-88, 147-153, 99-119: 17 memsets, 23 launches, one blocking norm).
//  * k_train_persample -- the reference's learn() loop (main.cu:125-170) as ONE persistent block
//    (the fallback; the default is the six-CTA cluster kernel of persample_cluster8.cu, this one
//    is selected with the "persample_kernel" option set to 0 and needs no cluster launch):
//    parameters live in shared memory, one SGD step per image in file order, same update
//    semantics (output delta without sigmoid derivative, every backward product from pre-update
//    weights, biases and weights stepped by dt), per-epoch mean of ||delta_f||_2, early stop.
//
// Decomposition (both kernels): thread (f, window) owns one 4x4 subsample window of one feature
// map: 16 conv outputs (400 FMA forward, 400 FMA for the conv weight gradient), so conv
// activations, their deltas and the 25 weight-gradient partials stay in registers.  216 threads
// are live in a 224-thread block.
//
// Arithmetic notes (all within fp32 rounding of the reference, which itself sums with atomics in
// a run-dependent order): sums use FMA; the per-term divisions by 576 / 216 of layer.cu:379, 397,
// 320 become one multiplication of the delta by the reciprocal constant.
#include "net.cuh"

namespace cnn {

constexpr int kTrThreads = 224;  // 7 warps; threads 216..223 carry zeros
constexpr int kTrWarps = kTrThreads / 32;
constexpr int kRedStride = 27;   // 25 conv-weight partials + 1 conv-bias partial + pad (odd stride)

struct TrSmem {
  float img[2][kImg];
  float wc[kF][28];
  float bc[8];
  float ws[16];
  float bs[4];
  float wf[kOut][kS];
  float bf[12];
  float fc_part[kTrWarps][12];
  float delta_f[12];
  float red_c[kS][kRedStride];
  float red_s[kTrWarps][20];
  unsigned long long full[2];
  int flag[4];
};

__device__ __forceinline__ void load_params_to_smem(TrSmem& sm, const float* __restrict__ params, int tid) {
  for (int i = tid; i < kF * 28; i += kTrThreads) {
    const int f = i / 28, t = i % 28;
    sm.wc[f][t] = (t < 25) ? params[kOffWc + f * 25 + t] : 0.f;
  }
  if (tid < kF) sm.bc[tid] = params[kOffBc + tid];
  if (tid < 16) sm.ws[tid] = params[kOffWs + tid];
  if (tid == 0) sm.bs[0] = params[kOffBs];
  for (int i = tid; i < kOut * kS; i += kTrThreads) sm.wf[i / kS][i % kS] = params[kOffWf + i];
  if (tid < kOut) sm.bf[tid] = params[kOffBf + tid];
}

// Per-thread state of one image's forward pass.
struct FwdRegs {
  float patch[8][8];
  float a[4][4];   // conv activations of the window
  float as;        // subsample activation
  float wfv[kOut]; // this thread's column of the FC weights
};

template <int FAST>
__device__ __forceinline__ void thread_forward(const TrSmem& sm, const float* img, int f, int p, int q,
                                               int s, bool live, FwdRegs& r, float (&pk)[kOut]) {
  if (live) {
    const float* base = img + (4 * p) * kH + 4 * q;
#pragma unroll
    for (int y = 0; y < 8; ++y) {
      const float4 lo = *reinterpret_cast<const float4*>(base + y * kH);
      const float4 hi = *reinterpret_cast<const float4*>(base + y * kH + 4);
      r.patch[y][0] = lo.x; r.patch[y][1] = lo.y; r.patch[y][2] = lo.z; r.patch[y][3] = lo.w;
      r.patch[y][4] = hi.x; r.patch[y][5] = hi.y; r.patch[y][6] = hi.z; r.patch[y][7] = hi.w;
    }
  } else {
#pragma unroll
    for (int y = 0; y < 8; ++y)
#pragma unroll
      for (int x = 0; x < 8; ++x) r.patch[y][x] = 0.f;
  }
  float wr[28];
#pragma unroll
  for (int t = 0; t < 7; ++t) {
    const float4 v = *reinterpret_cast<const float4*>(&sm.wc[f][4 * t]);
    wr[4 * t] = v.x; wr[4 * t + 1] = v.y; wr[4 * t + 2] = v.z; wr[4 * t + 3] = v.w;
  }
  const float b = sm.bc[f];
#pragma unroll
  for (int y = 0; y < 4; ++y)
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 5; ++j)
#pragma unroll
        for (int i = 0; i < 5; ++i) acc = fmaf(wr[i * 5 + j], r.patch[y + i][x + j], acc);
      r.a[y][x] = sigmoidf<FAST>(acc + b);
    }
  float zs = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) zs = fmaf(sm.ws[i * 4 + j], r.a[i][j], zs);
  r.as = sigmoidf<FAST>(zs + sm.bs[0]);
#pragma unroll
  for (int k = 0; k < kOut; ++k) {
    r.wfv[k] = sm.wf[k][s];
    pk[k] = live ? r.wfv[k] * r.as : 0.f;
  }
}

// Sum each of n values over the 32 lanes (butterfly); every lane ends with the total.
template <int N>
__device__ __forceinline__ void warp_sum(float (&v)[N]) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1)
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] += __shfl_xor_sync(0xffffffffu, v[i], m);
}

// Backward of one image for this thread, given delta_f in shared memory.  Produces the thread's
// contributions: gws[16] (subsample weight), gbs (subsample bias term), gwc[25] (conv weight, already
// divided by 576), gbc (conv bias term, divided by 576), and das-derived delta_s.
__device__ __forceinline__ void thread_backward(const TrSmem& sm, const FwdRegs& r, bool live,
                                                const float (&df)[kOut], float& delta_s,
                                                float (&gws)[16], float (&gwc)[25], float& gbc) {
  float das = 0.f;
#pragma unroll
  for (int k = 0; k < kOut; ++k) das = fmaf(r.wfv[k], df[k], das);
  delta_s = live ? das * r.as * (1.f - r.as) : 0.f;
  float dc[4][4];
  const float inv_c = 1.0f / (float)(kC * kC);
  gbc = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      gws[i * 4 + j] = delta_s * r.a[i][j];
      const float dac = sm.ws[i * 4 + j] * delta_s;
      const float d = dac * r.a[i][j] * (1.f - r.a[i][j]);
      dc[i][j] = d * inv_c;
      gbc += dc[i][j];
    }
#pragma unroll
  for (int u = 0; u < 5; ++u)
#pragma unroll
    for (int v = 0; v < 5; ++v) {
      float acc = 0.f;
#pragma unroll
      for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) acc = fmaf(dc[y][x], r.patch[y + u][x + v], acc);
      gwc[u * 5 + v] = acc;
    }
}

// ----------------------------------------------------------------------------------------------
// Minibatch gradient: one partial row per block.
// Row layout (kRowStride floats): arena-ordered gradient [0, 2343), zero padding, and at
// kRowErr the sum over the block's images of ||delta_f||_2.
// ----------------------------------------------------------------------------------------------

// MINB = 1: one block per SM, no register cap -- lowest latency, used for small batches.
// MINB = 2: two blocks per SM at 128 registers -- higher throughput on large batches.
// EARLY = true (used when every block has one image -- a training step of a few hundred images -- and the
// predecessor on the stream is this library's own reduce + update kernel of the previous step, which does
// not touch the images): the first image copies are issued before the wait for the predecessor kernel.  With many images per block that order
// of the prologue compiles to a slower loop (1.06 against 0.985 ms for 57,344 images), so it is a variant.
template <int FAST, int MINB, bool EARLY>
__global__ void __launch_bounds__(kTrThreads, MINB)
k_grad_partials(const float* __restrict__ images, const unsigned* __restrict__ labels, long n,
                const float* __restrict__ params, float* __restrict__ rows, int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  TrSmem& sm = *reinterpret_cast<TrSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool live = tid < kS;
  const int s = live ? tid : kS - 1;
  const int f = s / 36, w = s % 36, p = w / 6, q = w % 6;

  // In a training loop this kernel follows the previous step's reduce + update kernel.  Launched with
  // launch_pdl() it starts while that kernel still runs: the barriers and the first two image copies (the
  // images are nobody's output) are under way when the parameters become readable.
  auto issue = [&](int stage, long img) {
    mbar_expect_tx(&sm.full[stage], kImg * sizeof(float));
    bulk_g2s(&sm.img[stage][0], images + img * kImg, kImg * sizeof(float), &sm.full[stage]);
  };
  if (EARLY) {
    pdl_launch_dependents();   // one short-lived block per image: the reduce kernel's blocks may come on board at once
    if (tid == 0) {
      mbar_init(&sm.full[0], 1);
      mbar_init(&sm.full[1], 1);
      mbar_fence_init();
      for (int st = 0; st < 2; ++st) {
        const long im = (long)blockIdx.x + (long)st * gridDim.x;
        if (im < n) issue(st, im);
      }
    }
    pdl_wait();      // the parameters (and the row buffer this kernel writes at its end) belong to the predecessor until here
    load_params_to_smem(sm, params, tid);
    __syncthreads();
  } else {
    pdl_wait();
    load_params_to_smem(sm, params, tid);
    if (tid == 0) {
      mbar_init(&sm.full[0], 1);
      mbar_init(&sm.full[1], 1);
      mbar_fence_init();
    }
    __syncthreads();
    if (tid == 0) {
      for (int st = 0; st < 2; ++st) {
        const long im = (long)blockIdx.x + (long)st * gridDim.x;
        if (im < n) issue(st, im);
      }
    }
  }

  float acc_wc[25], acc_ws[16], acc_wf[kOut];
  float acc_bc = 0.f, acc_bs = 0.f, acc_bf = 0.f, acc_err = 0.f;
#pragma unroll
  for (int i = 0; i < 25; ++i) acc_wc[i] = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) acc_ws[i] = 0.f;
#pragma unroll
  for (int i = 0; i < kOut; ++i) acc_wf[i] = 0.f;

  bool gave_up = false;
  int it = 0;
  for (long im = blockIdx.x; im < n; im += gridDim.x, ++it) {
    const int stage = it & 1;
    mbar_wait_bounded(&sm.full[stage], (unsigned)(it >> 1) & 1u, status, gave_up);
    unsigned label = 0;
    if (warp == 0 && lane < kOut) label = labels[im];

    FwdRegs r;
    float pk[kOut];
    thread_forward<FAST>(sm, &sm.img[stage][0], f, p, q, s, live, r, pk);
    warp_sum(pk);
    if (lane == 0) {
#pragma unroll
      for (int k = 0; k < kOut; ++k) sm.fc_part[warp][k] = pk[k];
    }
    __syncthreads();  // (A) FC partials visible; every thread has taken its patch
    if (tid == 0) {
      const long nx = im + 2L * gridDim.x;
      if (nx < n) issue(stage, nx);
    }
    if (warp == 0) {
      float d = 0.f;
      if (lane < kOut) {
        float z = 0.f;
#pragma unroll
        for (int ww = 0; ww < kTrWarps; ++ww) z += sm.fc_part[ww][lane];
        z += sm.bf[lane];
        const float o = sigmoidf<FAST>(z);
        d = ((label == (unsigned)lane) ? 1.0f : 0.0f) - o;
        sm.delta_f[lane] = d;
        acc_bf += d;
      }
      float sq = d * d;
#pragma unroll
      for (int m = 8; m > 0; m >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, m);
      // lanes 0..15 hold the sum over lanes 0..15 (lanes 10..15 contributed zero)
      if (lane == 0) acc_err += sqrtf(sq);
    }
    __syncthreads();  // (B) delta_f visible
    float df[kOut];
#pragma unroll
    for (int k = 0; k < kOut; ++k) df[k] = sm.delta_f[k];
    float delta_s, gws[16], gwc[25], gbc;
    thread_backward(sm, r, live, df, delta_s, gws, gwc, gbc);
#pragma unroll
    for (int k = 0; k < kOut; ++k) acc_wf[k] = fmaf(df[k], live ? r.as : 0.f, acc_wf[k]);
#pragma unroll
    for (int i = 0; i < 16; ++i) acc_ws[i] += gws[i];
#pragma unroll
    for (int i = 0; i < 25; ++i) acc_wc[i] += gwc[i];
    acc_bc += gbc;
    acc_bs += delta_s * (1.0f / (float)kS);
    // No barrier needed here: the next iteration writes fc_part only after its own forward, and
    // delta_f only after barrier (A) of the next iteration, which every thread reaches after this
    // point.
  }
  // With many images per block the reduce kernel is only brought onto the SMs from here on: its blocks wait
  // for this grid to finish, and while they wait they hold registers that a second gradient block per SM needs.
  if (!EARLY) pdl_launch_dependents();

  // ---- block-level reduction, fixed order ----------------------------------------------------
  float* row = rows + (size_t)blockIdx.x * kRowStride;
  if (live) {
#pragma unroll
    for (int k = 0; k < kOut; ++k) row[kOffWf + k * kS + s] = acc_wf[k];
#pragma unroll
    for (int i = 0; i < 25; ++i) sm.red_c[s][i] = acc_wc[i];
    sm.red_c[s][25] = acc_bc;
  }
  {
    float v[17];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = live ? acc_ws[i] : 0.f;
    v[16] = live ? acc_bs : 0.f;
    warp_sum(v);
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < 17; ++i) sm.red_s[warp][i] = v[i];
    }
  }
  if (warp == 0 && lane < kOut) row[kOffBf + lane] = acc_bf;
  if (tid == 0) row[kRowErr] = acc_err;
  __syncthreads();
  if (tid < kF * 26) {
    const int ff = tid / 26, t = tid % 26;
    float sum = 0.f;
    for (int ww = 0; ww < 36; ++ww) sum += sm.red_c[ff * 36 + ww][t];
    if (t < 25) row[kOffWc + ff * 25 + t] = sum;
    else row[kOffBc + ff] = sum;
  } else if (tid >= 192 && tid < 192 + 17) {
    const int t = tid - 192;
    float sum = 0.f;
#pragma unroll
    for (int ww = 0; ww < kTrWarps; ++ww) sum += sm.red_s[ww][t];
    if (t < 16) row[kOffWs + t] = sum;
    else row[kOffBs] = sum;
  }
  // zero the padding so that reductions and collectives over the padded row stay finite
  if (tid < kRowStride - kNParams && kNParams + tid != kRowErr) row[kNParams + tid] = 0.f;
}

// G[i] = sum over rows (fixed order: thirty-two interleaved row groups, then a fixed tree over the
// groups) and, if params is given, params[i] += scale * G[i].  Element kRowErr carries the error sum;
// if mean_err is given, *mean_err += err_scale * that sum.  Block: 1,024 threads = 32 columns x 32 groups.
// (The data-parallel exchange kernel adds a rank's rows in exactly this order.)
constexpr int kRedGroups = 32;

__global__ void __launch_bounds__(32 * kRedGroups)
k_reduce_rows(const float* __restrict__ rows, int n_rows, float* __restrict__ G,
              float* __restrict__ params, float scale, float* __restrict__ mean_err, float err_scale) {
  __shared__ float part[kRedGroups][33];
  const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + lane;
  pdl_launch_dependents();   // the next step's gradient kernel may set itself up now
  pdl_wait();                // the rows are complete
  float acc = 0.f;
  if (col < kRowStride) {
#pragma unroll 4
    for (int r = g; r < n_rows; r += kRedGroups) acc += rows[(size_t)r * kRowStride + col];
  }
  part[g][lane] = acc;
  __syncthreads();
  if (g == 0 && col < kRowStride) {
    float q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      q[i] = (part[4 * i][lane] + part[4 * i + 1][lane]) + (part[4 * i + 2][lane] + part[4 * i + 3][lane]);
    const float total = ((q[0] + q[1]) + (q[2] + q[3])) + ((q[4] + q[5]) + (q[6] + q[7]));
    if (G) G[col] = total;
    if (params && col < kNParams) params[col] = fmaf(scale, total, params[col]);
    if (mean_err && col == kRowErr) *mean_err += err_scale * total;
  }
}

__global__ void k_apply_update(float* __restrict__ params, const float* __restrict__ G, float scale) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < kNParams) params[i] = fmaf(scale, G[i], params[i]);
}

// ----------------------------------------------------------------------------------------------
// Per-sample SGD, one persistent block.
// ----------------------------------------------------------------------------------------------
template <int FAST>
__global__ void __launch_bounds__(kTrThreads, 1)
k_train_persample(const float* __restrict__ images, const unsigned* __restrict__ labels, long n,
                  int epochs, float dt, float threshold, float* __restrict__ params,
                  float* __restrict__ mean_err, int* __restrict__ epochs_run, int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  TrSmem& sm = *reinterpret_cast<TrSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool live = tid < kS;
  const int s = live ? tid : kS - 1;
  const int f = s / 36, w = s % 36, p = w / 6, q = w % 6;

  load_params_to_smem(sm, params, tid);
  if (tid == 0) {
    mbar_init(&sm.full[0], 1);
    mbar_init(&sm.full[1], 1);
    mbar_fence_init();
    sm.flag[0] = 0;
  }
  __syncthreads();

  const long total = (long)epochs * n;
  auto issue = [&](int stage, long step) {
    mbar_expect_tx(&sm.full[stage], kImg * sizeof(float));
    bulk_g2s(&sm.img[stage][0], images + (step % n) * kImg, kImg * sizeof(float), &sm.full[stage]);
  };
  if (tid == 0) {
    if (total > 0) issue(0, 0);
    if (total > 1) issue(1, 1);
  }

  bool gave_up = false;
  float err = 0.f;  // thread 0: running sum of the epoch, a float like main.cu:130
  int done_epochs = 0;
  unsigned next_label = 0;
  if (warp == 0 && lane < kOut && total > 0) next_label = labels[0];

  long step = 0;
  for (int e = 0; e < epochs; ++e) {
    for (long i = 0; i < n; ++i, ++step) {
      const int stage = (int)(step & 1);
      mbar_wait_bounded(&sm.full[stage], (unsigned)(step >> 1) & 1u, status, gave_up);
      const unsigned label = next_label;
      if (warp == 0 && lane < kOut && step + 1 < total) next_label = labels[(step + 1) % n];

      FwdRegs r;
      float pk[kOut];
      thread_forward<FAST>(sm, &sm.img[stage][0], f, p, q, s, live, r, pk);
      warp_sum(pk);
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < kOut; ++k) sm.fc_part[warp][k] = pk[k];
      }
      __syncthreads();  // (A)
      if (tid == 0 && step + 2 < total) issue(stage, step + 2);
      if (warp == 0) {
        float d = 0.f;
        if (lane < kOut) {
          float z = 0.f;
#pragma unroll
          for (int ww = 0; ww < kTrWarps; ++ww) z += sm.fc_part[ww][lane];
          z += sm.bf[lane];
          const float o = sigmoidf<FAST>(z);
          d = ((label == (unsigned)lane) ? 1.0f : 0.0f) - o;  // makeError
          sm.delta_f[lane] = d;
          sm.bf[lane] = fmaf(dt, d, sm.bf[lane]);              // bp_bias_f
        }
        float sq = d * d;
#pragma unroll
        for (int m = 8; m > 0; m >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, m);
        if (lane == 0) err += sqrtf(sq);                        // the norm of main.cu:153-154
      }
      __syncthreads();  // (B)
      float df[kOut];
#pragma unroll
      for (int k = 0; k < kOut; ++k) df[k] = sm.delta_f[k];
      float delta_s, gws[16], gwc[25], gbc;
      thread_backward(sm, r, live, df, delta_s, gws, gwc, gbc);
      if (live) {
        // bp_weight_f then apply_grad on this thread's own column of the FC weights.
#pragma unroll
        for (int k = 0; k < kOut; ++k) sm.wf[k][s] = fmaf(dt, df[k] * r.as, r.wfv[k]);
#pragma unroll
        for (int i = 0; i < 25; ++i) sm.red_c[s][i] = gwc[i];
        sm.red_c[s][25] = gbc;
      }
      {
        float v[17];
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = gws[i];
        v[16] = delta_s * (1.0f / (float)kS);
        warp_sum(v);
        if (lane == 0) {
#pragma unroll
          for (int i = 0; i < 17; ++i) sm.red_s[warp][i] = v[i];
        }
      }
      __syncthreads();  // (C) all backward reads of ws / wc are done; partials visible
      if (tid < kF * 26) {
        const int ff = tid / 26, t = tid % 26;
        float sum = 0.f;
#pragma unroll 6
        for (int ww = 0; ww < 36; ++ww) sum += sm.red_c[ff * 36 + ww][t];
        if (t < 25) sm.wc[ff][t] = fmaf(dt, sum, sm.wc[ff][t]);  // apply_grad (c1)
        else sm.bc[ff] = fmaf(dt, sum, sm.bc[ff]);               // bp_bias_c1
      } else if (tid >= 192 && tid < 192 + 17) {
        const int t = tid - 192;
        float sum = 0.f;
#pragma unroll
        for (int ww = 0; ww < kTrWarps; ++ww) sum += sm.red_s[ww][t];
        if (t < 16) sm.ws[t] = fmaf(dt, sum, sm.ws[t]);          // apply_grad (s1)
        else sm.bs[0] = fmaf(dt, sum, sm.bs[0]);                 // bp_bias_s1
      }
      __syncthreads();  // (D) updated parameters visible to the next forward
    }
    // epoch end, main.cu:159-166
    if (tid == 0) {
      const float m = err / (float)n;
      if (mean_err) mean_err[e] = m;
      err = 0.f;
      sm.flag[0] = (m < threshold) ? 1 : 0;
    }
    done_epochs = e + 1;
    __syncthreads();
    if (sm.flag[0]) break;
  }
  // After an early stop up to two prefetched images are still on their way into shared memory:
  // the block does not exit under them.
  if (tid == 0) {
    for (long s2 = step; s2 < total && s2 < step + 2; ++s2)
      mbar_wait_bounded(&sm.full[s2 & 1], (unsigned)(s2 >> 1) & 1u, status, gave_up);
  }

  // write the parameters back
  for (int i = tid; i < kF * 25; i += kTrThreads) params[kOffWc + i] = sm.wc[i / 25][i % 25];
  if (tid < kF) params[kOffBc + tid] = sm.bc[tid];
  if (tid < 16) params[kOffWs + tid] = sm.ws[tid];
  if (tid == 0) params[kOffBs] = sm.bs[0];
  for (int i = tid; i < kOut * kS; i += kTrThreads) params[kOffWf + i] = sm.wf[i / kS][i % kS];
  if (tid < kOut) params[kOffBf + tid] = sm.bf[tid];
  if (tid == 0 && epochs_run) *epochs_run = done_epochs;
}

template <class K>
static int set_smem_attr(K kernel, size_t bytes) {
  CNN_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return CNN_OK;
}

int launch_grad_partials(cnn_net* net, const float* d_images, const unsigned* d_labels, long n,
                                int grid, cudaStream_t st, bool chained) {
  const size_t smem = sizeof(TrSmem);
  int rc;
  cudaError_t le = cudaSuccess;
#define CNN_LAUNCH_GRAD3(FL, MB, EA)                                                                          \
  do {                                                                                                       \
    if ((rc = set_smem_attr(k_grad_partials<FL, MB, EA>, smem)) != CNN_OK) return rc;                        \
    le = launch_pdl(k_grad_partials<FL, MB, EA>, dim3(grid), dim3(kTrThreads), smem, st, d_images, d_labels, n, \
                    (const float*)net->d_params, net->d_partials, net->d_status);                            \
  } while (0)
#define CNN_LAUNCH_GRAD(FL)                                   \
  do {                                                        \
    const bool early = chained && ((long)grid == n);          \
    if (grid > sm_count()) {                                  \
      if (early) CNN_LAUNCH_GRAD3(FL, 2, true);               \
      else CNN_LAUNCH_GRAD3(FL, 2, false);                    \
    } else {                                                  \
      if (early) CNN_LAUNCH_GRAD3(FL, 1, true);               \
      else CNN_LAUNCH_GRAD3(FL, 1, false);                    \
    }                                                         \
  } while (0)
  if (net->fast_sigmoid) CNN_LAUNCH_GRAD(1);
  else CNN_LAUNCH_GRAD(0);
#undef CNN_LAUNCH_GRAD
#undef CNN_LAUNCH_GRAD3
  if (le != cudaSuccess) return cuda_fail(le, "k_grad_partials launch");
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "k_grad_partials launch");
  return CNN_OK;
}

// Blocks of the gradient kernel.  Up to two blocks per SM there is one image per block (a training
// step of a few hundred images is pure latency: one image per block halves it against two images
// in sequence on half as many blocks); from 8 images per SM on, two blocks per SM walk the batch.
int grid_for_batch(long n) {
  const long sms = sm_count();
  if (n <= 2 * sms) return (int)n;
  const long cap = (n >= 8 * sms) ? 2 * sms : sms;
  return (int)cap;
}

}  // namespace cnn

using namespace cnn;

extern "C" {

int cnn_grad_batch(cnn_net* net, const float* d_images, const unsigned int* d_labels, long n,
                   float* d_grad, void* stream) {
  CNN_REQUIRE(net && d_grad, "cnn_grad_batch: NULL argument");
  CNN_REQUIRE(n >= 0, "cnn_grad_batch: negative image count");
  cudaStream_t st = as_stream(stream);
  if (n == 0) {
    CNN_CUDA(cudaMemsetAsync(d_grad, 0, sizeof(float) * kNParamsPadded, st));
    return CNN_OK;
  }
  CNN_REQUIRE(d_images && d_labels, "cnn_grad_batch: NULL images or labels");
  CNN_REQUIRE((reinterpret_cast<uintptr_t>(d_images) & 15u) == 0,
              "cnn_grad_batch: image batch must start on a 16-byte boundary");
  const int grid = grid_for_batch(n);
  int rc = ensure_train_scratch(net, 2 * sm_count());
  if (rc != CNN_OK) return rc;
  if ((rc = launch_grad_partials(net, d_images, d_labels, n, grid, st)) != CNN_OK) return rc;
  k_reduce_rows<<<(kNParamsPadded + 31) / 32, 32 * kRedGroups, 0, st>>>(net->d_partials, grid, d_grad, nullptr, 0.f,
                                                           nullptr, 0.f);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "k_reduce_rows launch");
  return CNN_OK;
}

int cnn_apply_update(cnn_net* net, const float* d_grad, float scale, void* stream) {
  CNN_REQUIRE(net && d_grad, "cnn_apply_update: NULL argument");
  k_apply_update<<<(kNParams + 255) / 256, 256, 0, as_stream(stream)>>>(net->d_params, d_grad, scale);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "k_apply_update launch");
  return CNN_OK;
}

int cnn_train_minibatch(cnn_net* net, const float* d_images, const unsigned int* d_labels, long n,
                        int batch, int epochs, float dt, float* d_mean_err, void* stream) {
  CNN_REQUIRE(net != nullptr, "cnn_train_minibatch: NULL net");
  CNN_REQUIRE(n >= 0 && batch > 0 && epochs >= 0, "cnn_train_minibatch: bad sizes");
  if (n == 0 || epochs == 0) return CNN_OK;
  CNN_REQUIRE(d_images && d_labels, "cnn_train_minibatch: NULL images or labels");
  CNN_REQUIRE((reinterpret_cast<uintptr_t>(d_images) & 15u) == 0,
              "cnn_train_minibatch: image batch must start on a 16-byte boundary");
  cudaStream_t st = as_stream(stream);
  int rc = ensure_train_scratch(net, 2 * sm_count());
  if (rc != CNN_OK) return rc;
  if (d_mean_err) CNN_CUDA(cudaMemsetAsync(d_mean_err, 0, sizeof(float) * (size_t)epochs, st));
  for (int e = 0; e < epochs; ++e) {
    for (long first = 0; first < n; first += batch) {
      const long b = (n - first) < batch ? (n - first) : batch;
      const int grid = grid_for_batch(b);
      if ((rc = launch_grad_partials(net, d_images + first * kImg, d_labels + first, b, grid, st, first > 0 || e > 0)) != CNN_OK)
        return rc;
      cudaError_t err = launch_pdl(k_reduce_rows, dim3((kNParamsPadded + 31) / 32), dim3(32 * kRedGroups), 0, st,
                                   (const float*)net->d_partials, grid, net->d_grad, net->d_params, dt / (float)b,
                                   d_mean_err ? d_mean_err + e : nullptr, 1.0f / (float)n);
      if (err == cudaSuccess) err = cudaGetLastError();
      if (err != cudaSuccess) return cuda_fail(err, "k_reduce_rows launch");
    }
  }
  return CNN_OK;
}

int cnn_train_sgd_persample(cnn_net* net, const float* d_images, const unsigned int* d_labels, long n,
                            int epochs, float dt, float threshold, float* h_mean_err, int* h_epochs_run,
                            void* stream) {
  CNN_REQUIRE(net != nullptr, "cnn_train_sgd_persample: NULL net");
  CNN_REQUIRE(n >= 0 && epochs >= 0, "cnn_train_sgd_persample: bad sizes");
  if (h_epochs_run) *h_epochs_run = 0;
  if (n == 0 || epochs == 0) return CNN_OK;
  CNN_REQUIRE(d_images && d_labels, "cnn_train_sgd_persample: NULL images or labels");
  CNN_REQUIRE((reinterpret_cast<uintptr_t>(d_images) & 15u) == 0,
              "cnn_train_sgd_persample: image batch must start on a 16-byte boundary");
  cudaStream_t st = as_stream(stream);
  int rc = ensure_train_scratch(net, 2 * sm_count());
  if (rc != CNN_OK) return rc;
  // Scratch reuse: d_grad holds the per-epoch means (epochs <= kNParamsPadded) and the epoch count.
  CNN_REQUIRE(epochs <= kNParamsPadded, "cnn_train_sgd_persample: too many epochs");
  float* d_mean = net->d_grad;
  int* d_ran = reinterpret_cast<int*>(net->d_grad + kNParamsPadded);
  const size_t smem = sizeof(TrSmem);
  if (net->ps_kernel) {
    if ((rc = launch_persample_cluster8(net, d_images, d_labels, n, epochs, dt, threshold, d_mean, d_ran, st)) != CNN_OK)
      return rc;
  } else {
#define CNN_LAUNCH_PS(FL)                                                                          \
  do {                                                                                             \
    if ((rc = set_smem_attr(k_train_persample<FL>, smem)) != CNN_OK) return rc;                    \
    k_train_persample<FL><<<1, kTrThreads, smem, st>>>(d_images, d_labels, n, epochs, dt, threshold, \
                                                       net->d_params, d_mean, d_ran, net->d_status); \
  } while (0)
  if (net->fast_sigmoid) CNN_LAUNCH_PS(1);
  else CNN_LAUNCH_PS(0);
#undef CNN_LAUNCH_PS
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "k_train_persample launch");
  CNN_CUDA(cudaStreamSynchronize(st));
  int ran = 0;
  CNN_CUDA(cudaMemcpy(&ran, d_ran, sizeof(int), cudaMemcpyDeviceToHost));
  if (h_epochs_run) *h_epochs_run = ran;
  if (h_mean_err && ran > 0)
    CNN_CUDA(cudaMemcpy(h_mean_err, d_mean, sizeof(float) * (size_t)ran, cudaMemcpyDeviceToHost));
  int status = 0;
  CNN_CUDA(cudaMemcpy(&status, net->d_status, sizeof(int), cudaMemcpyDeviceToHost));
  if (status != 0) {
    set_error("cnn_train_sgd_persample: a bounded device-side wait ran out");
    int zero = 0;
    cudaMemcpy(net->d_status, &zero, sizeof(int), cudaMemcpyHostToDevice);
    return CNN_ERR_TIMEOUT;
  }
  return CNN_OK;
}

// ----------------------------------------------------------------------------------------------
// Gradient of a batch without any allocation.
//
// Some callers may not allocate device memory at the point where they need a gradient: code that
// runs inside a memory-budgeted service whose pools are carved up at start-up, plug-ins that are
// handed device buffers by a host application and are forbidden to call cudaMalloc themselves,
// and real-time loops where an allocation (a device-wide synchronisation) is not acceptable.
// cnn_grad_batch needs a cnn_net, and creating one allocates; this entry point takes raw device
// pointers instead and keeps the partial-gradient rows of k_grad_partials in a fixed array that is
// part of the library image.
// ----------------------------------------------------------------------------------------------
namespace cnn {
constexpr int kNoAllocMaxRows = 160;          // one row per block, at most this many blocks
constexpr long kNoAllocMaxImages = 65536;     // largest batch the entry point accepts
// rows | status word (+ padding to keep the array a multiple of 256 bytes)
constexpr size_t kNoAllocFloats = (size_t)kNoAllocMaxRows * kRowStride + 64;
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocFloats];

// Set-up, once per device, with that device current: in host code the array's name is only a
// handle, its device address has to be asked for.  Also raises the kernel's shared-memory limit.
static int noalloc_scratch(float** rows) {
  static float* scratch_of_device[64] = {nullptr};
  int dev = -1;
  CNN_CUDA(cudaGetDevice(&dev));
  CNN_REQUIRE(dev >= 0 && dev < 64, "cnn_grad_batch_noalloc: device ordinal out of range");
  if (scratch_of_device[dev] == nullptr) {
    float* ptr = nullptr;
    CNN_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch));
    CNN_REQUIRE(ptr != nullptr, "cnn_grad_batch_noalloc: no device address for the scratch array");
    CNN_CUDA(cudaFuncSetAttribute(k_grad_partials<0, 1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)sizeof(TrSmem)));
    scratch_of_device[dev] = ptr;
  }
  *rows = scratch_of_device[dev];
  return CNN_OK;
}
}  // namespace cnn

int cnn_grad_batch_noalloc(const float* d_params, const float* d_images, const unsigned int* d_labels,
                           long n, float* d_grad, void* stream) {
  CNN_REQUIRE(d_params && d_grad, "cnn_grad_batch_noalloc: NULL params or gradient buffer");
  CNN_REQUIRE(n >= 0, "cnn_grad_batch_noalloc: negative image count");
  if (n > kNoAllocMaxImages) {
    set_error("cnn_grad_batch_noalloc: %ld images exceed the fixed-scratch limit of %ld per call; "
              "split the batch (gradients add) or use cnn_grad_batch", n, kNoAllocMaxImages);
    return CNN_ERR_INVALID;
  }
  cudaStream_t st = as_stream(stream);
  if (n == 0) {
    CNN_CUDA(cudaMemsetAsync(d_grad, 0, sizeof(float) * kNParamsPadded, st));
    return CNN_OK;
  }
  CNN_REQUIRE(d_images && d_labels, "cnn_grad_batch_noalloc: NULL images or labels");
  CNN_REQUIRE((reinterpret_cast<uintptr_t>(d_images) & 15u) == 0,
              "cnn_grad_batch_noalloc: image batch must start on a 16-byte boundary");
  float* rows = nullptr;
  int rc = noalloc_scratch(&rows);
  if (rc != CNN_OK) return rc;
  int* status = reinterpret_cast<int*>(rows + (size_t)kNoAllocMaxRows * kRowStride);

  long grid_l = sm_count();
  if (grid_l > kNoAllocMaxRows) grid_l = kNoAllocMaxRows;
  if (grid_l > n) grid_l = n;
  const int grid = (int)grid_l;
  // The array keeps what the previous call left.  Every row that is read below is rewritten in full
  // by its block, padding included, so no row needs clearing.  The status word starts at zero when
  // the library is loaded, is only ever set by a wait that ran out, and stays set until
  // cnn_grad_batch_noalloc_status reads and clears it.
  k_grad_partials<0, 1, false><<<grid, kTrThreads, sizeof(TrSmem), st>>>(d_images, d_labels, n, d_params, rows, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "k_grad_partials launch (no-alloc)");
  k_reduce_rows<<<(kNParamsPadded + 31) / 32, 32 * kRedGroups, 0, st>>>(rows, grid, d_grad, nullptr, 0.f, nullptr, 0.f);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "k_reduce_rows launch (no-alloc)");
  return CNN_OK;
}

int cnn_grad_batch_noalloc_status(void* stream) {
  float* rows = nullptr;
  int rc = noalloc_scratch(&rows);
  if (rc != CNN_OK) return rc;
  int* d_status = reinterpret_cast<int*>(rows + (size_t)kNoAllocMaxRows * kRowStride);
  cudaStream_t st = as_stream(stream);
  CNN_CUDA(cudaStreamSynchronize(st));
  int status = 0;
  CNN_CUDA(cudaMemcpyAsync(&status, d_status, sizeof(int), cudaMemcpyDeviceToHost, st));
  CNN_CUDA(cudaStreamSynchronize(st));
  if (status != 0) {
    CNN_CUDA(cudaMemsetAsync(d_status, 0, sizeof(int), st));
    CNN_CUDA(cudaStreamSynchronize(st));
    set_error("cnn_grad_batch_noalloc: a bounded device-side wait ran out; the gradient of that call is not valid");
    return CNN_ERR_TIMEOUT;
  }
  return CNN_OK;
}

int cnn_copy_to_host(void* h_dst, const void* d_src, size_t bytes) {
  CNN_REQUIRE(h_dst && d_src, "cnn_copy_to_host: NULL argument");
  CNN_CUDA(cudaMemcpy(h_dst, d_src, bytes, cudaMemcpyDeviceToHost));
  return CNN_OK;
}

int cnn_copy_to_device(void* d_dst, const void* h_src, size_t bytes) {
  CNN_REQUIRE(d_dst && h_src, "cnn_copy_to_device: NULL argument");
  CNN_CUDA(cudaMemcpy(d_dst, h_src, bytes, cudaMemcpyHostToDevice));
  CNN_CUDA(cudaStreamSynchronize(cudaStreamLegacy));  // a pageable source may still be in DMA on return
  return CNN_OK;
}

}  // extern "C"
