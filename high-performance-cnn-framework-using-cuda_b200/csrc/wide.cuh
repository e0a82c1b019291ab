// Shared definitions of the widened configuration (wide.cu: fp32 SIMT kernels and the C ABI;
// wide_tc.cu: tcgen05 tensor-core convolution).
#pragma once

#include "net.cuh"

namespace cnn {

struct WideDims {
  int H, F, C, P, S;        // C = H-4, P = C/4, S = F*P*P
  int o_wc, o_bc, o_ws, o_bs, o_wf, o_bf, n_params, n_padded;
};

inline WideDims make_wide_dims(int H, int F) {
  WideDims d;
  d.H = H; d.F = F; d.C = H - 4; d.P = d.C / 4; d.S = F * d.P * d.P;
  d.o_wc = 0; d.o_bc = d.o_wc + F * 25; d.o_ws = d.o_bc + F; d.o_bs = d.o_ws + 16;
  d.o_wf = d.o_bs + 1; d.o_bf = d.o_wf + kOut * d.S; d.n_params = d.o_bf + kOut;
  d.n_padded = ((d.n_params + 2 + 31) / 32) * 32;
  return d;
}

}  // namespace cnn

struct cnn_wide {
  cnn::WideDims d;
  float* d_params = nullptr;
  long cap = 0;                 // images the workspace holds
  float *ac = nullptr, *dc = nullptr, *as = nullptr, *ds = nullptr, *delta_f = nullptr, *err = nullptr;
  float *part_c = nullptr, *part_s = nullptr;
  float* img_shift = nullptr;   // [cap][4][H][H]: every image shifted left by 0..3 columns (16-byte aligned tap windows)
  float* part_f = nullptr;      // FC weight-gradient partials of the batch slices
  int flavour = 1;              // sigmoid flavour (cnn_common.cuh): 1 = the short form (default, as cnn_net), 2 = refined, 0 = reference expression
  int conv_mode = 0;            // 0 fp32 SIMT, 1 tf32 tcgen05 (one pass), 2 tf32 tcgen05 (three passes)
  int* d_status = nullptr;      // bounded-wait status word
  long part_rows = 0;           // rows of [F][26] that part_c holds
  // Tensor map (a CUtensorMap, kept opaque here) through which the fused delta + weight-gradient kernel reads the
  // conv activations, and what it was encoded for.
  alignas(64) unsigned char ac_map[128] = {};
  const float* ac_map_ptr = nullptr;
  long ac_map_cap = 0;
};


namespace cnn {
bool wide_conv_tc_supported(const WideDims& d);
// Conv + bias + sigmoid on the tensor cores: writes w->ac for n images.
int wide_conv_fwd_tc(cnn_wide* w, const float* d_images, long n, cudaStream_t st);
bool wide_grad_tc_supported(const WideDims& d);
// Conv deltas, conv weight + bias gradient partials and subsample-filter gradient partials on the tensor cores,
// from w->ac and w->ds: fills w->part_c with *rows_out rows of [F][26] and w->part_s with as many rows of [17].
int wide_grad_c1_tc(cnn_wide* w, const float* d_images, long n, int* rows_out, cudaStream_t st);
}  // namespace cnn
