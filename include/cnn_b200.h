/*
 * C ABI of the B200 (sm_100a) implementation of the reference CNN hot path:
 *   28x28 input -> conv 6x5x5 (valid) -> sigmoid -> one shared 4x4/stride-4 weighted subsample
 *   -> sigmoid -> fully connected 216->10 -> sigmoid, with the reference's per-sample SGD rule.
 *
 * The reference has no FFI layer: its boundary is the C++/CUDA header layer.h (class Layer plus
 * 19 __global__ kernels launched by the caller).  This header is what a binding for that path
 * would import instead; every entry point names the reference interface it replaces.  A C++
 * source-level drop-in with the reference's own names (class Layer, fp_*, bp_*, ...) lives in
 * the package's compat/layer.h.
 *
 * Conventions
 *   - every function returns 0 on success or a negative cnn_status; nothing throws or aborts;
 *     cnn_last_error() returns a thread-local description of the most recent failure;
 *   - pointers named d_* are device pointers, h_* are host pointers; "stream" is a cudaStream_t
 *     passed as void* (NULL = the legacy default stream, as the reference uses);
 *   - all tensors are fp32, row-major, contiguous; image batches are [n][28][28] and must start
 *     on a 16-byte boundary;
 *   - parameter arena order (2343 floats): [Wc 150 | bc 6 | Ws 16 | bs 1 | Wf 2160 | bf 10], each
 *     block in the reference's Layer::weight / Layer::bias layout (layer.cu:19-27);
 *   - there is no CPU fallback: without a usable CUDA device every compute call fails.
 */
#ifndef CNN_B200_H
#define CNN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum cnn_status {
  CNN_OK = 0,
  CNN_ERR_INVALID = -1,   /* bad argument (NULL pointer, negative size, misaligned batch) */
  CNN_ERR_CUDA = -2,      /* a CUDA runtime call or launch failed; see cnn_last_error() */
  CNN_ERR_TIMEOUT = -3,   /* a bounded device-side wait ran out (reported, never hangs) */
  CNN_ERR_UNSUPPORTED = -4/* shape or mode this build does not implement */
} cnn_status;

#define CNN_N_PARAMS 2343
#define CNN_IMAGE_ELEMS 784
#define CNN_N_OUT 10

const char* cnn_last_error(void);
/* Library version and the -gencode target it was compiled for, e.g. "sm_100a". */
const char* cnn_build_info(void);

/* ------------------------------------------------------------------------------------------
 * Layer object -- replaces class Layer (layer.h:14-35).
 * ---------------------------------------------------------------------------------------- */
typedef struct cnn_layer cnn_layer;

/* Device buffers of a layer, same names as the reference's public members (layer.h:18-26). */
typedef struct cnn_layer_view {
  int M, N, O;
  float* output;   /* [O]   */
  float* preact;   /* [O]   */
  float* bias;     /* [N]   */
  float* weight;   /* [N*M] */
  float* d_output; /* [O]   */
  float* d_preact; /* [O]   */
  float* d_weight; /* [N*M] */
} cnn_layer_view;

/* Layer::Layer(M,N,O), layer.cu:5-43: allocates the seven buffers and fills bias[i], then
 * weight[i*M..] for each unit i with 0.5f - rand()/RAND_MAX from the C library's rand(), in the
 * reference's draw order. */
int cnn_layer_create(int M, int N, int O, cnn_layer** out);
/* Layer::~Layer, layer.cu:46-58. */
int cnn_layer_destroy(cnn_layer* l);
/* Layer::setOutput, layer.cu:61-64: blocking copy of O host floats into output. */
int cnn_layer_set_output(cnn_layer* l, const float* h_data);
/* Layer::clear, layer.cu:67-71: zero output and preact. */
int cnn_layer_clear(cnn_layer* l);
/* Layer::bp_clear, layer.cu:73-78: zero d_output, d_preact, d_weight. */
int cnn_layer_bp_clear(cnn_layer* l);
/* Exposes the public data members of layer.h:16-26. */
int cnn_layer_view_get(const cnn_layer* l, cnn_layer_view* out);

/* ------------------------------------------------------------------------------------------
 * Per-operator launchers -- one per reference kernel, same argument order as layer.h:40-62.
 * Each keeps the reference's contract: accumulate-into-existing-contents where the reference
 * uses atomicAdd, in-place "+=" for the bias kernels and apply_grad, plain stores elsewhere.
 * None uses atomics: every output element is owned by one thread (or one warp), so results are
 * bit-reproducible run to run.
 * ---------------------------------------------------------------------------------------- */
int cnn_apply_step_function(const float* d_input, float* d_output, int n, void* stream); /* layer.cu:86-94 */
int cnn_make_error(float* d_err, const float* d_output, unsigned int label, int n, void* stream); /* layer.cu:96-104 */
int cnn_apply_grad(float* d_output, const float* d_grad, int n, void* stream);           /* layer.cu:106-114 */

int cnn_fp_preact_c1(const float* d_input, float* d_preact, const float* d_weight, void* stream); /* layer.cu:116-133 */
int cnn_fp_bias_c1(float* d_preact, const float* d_bias, void* stream);                           /* layer.cu:135-150 */
int cnn_fp_preact_s1(const float* d_input, float* d_preact, const float* d_weight, void* stream); /* layer.cu:152-169 */
int cnn_fp_bias_s1(float* d_preact, const float* d_bias, void* stream);                           /* layer.cu:171-186 */
int cnn_fp_preact_f(const float* d_input, float* d_preact, const float* d_weight, void* stream);  /* layer.cu:188-204 */
int cnn_fp_bias_f(float* d_preact, const float* d_bias, void* stream);                            /* layer.cu:206-216 */

int cnn_bp_weight_f(float* d_d_weight, const float* d_d_preact, const float* d_p_output, void* stream);  /* layer.cu:218-234 */
int cnn_bp_bias_f(float* d_bias, const float* d_d_preact, void* stream);                                 /* layer.cu:236-246 */
int cnn_bp_output_s1(float* d_d_output, const float* d_n_weight, const float* d_nd_preact, void* stream);/* layer.cu:248-264 */
int cnn_bp_preact_s1(float* d_d_preact, const float* d_d_output, const float* d_preact, void* stream);   /* layer.cu:266-283 */
int cnn_bp_weight_s1(float* d_d_weight, const float* d_d_preact, const float* d_p_output, void* stream); /* layer.cu:285-304 */
int cnn_bp_bias_s1(float* d_bias, const float* d_d_preact, void* stream);                                /* layer.cu:306-322 */
int cnn_bp_output_c1(float* d_d_output, const float* d_n_weight, const float* d_nd_preact, void* stream);/* layer.cu:324-342 */
int cnn_bp_preact_c1(float* d_d_preact, const float* d_d_output, const float* d_preact, void* stream);   /* layer.cu:344-361 */
int cnn_bp_weight_c1(float* d_d_weight, const float* d_d_preact, const float* d_p_output, void* stream); /* layer.cu:363-381 */
int cnn_bp_bias_c1(float* d_bias, const float* d_d_preact, void* stream);                                /* layer.cu:383-399 */

/* ------------------------------------------------------------------------------------------
 * Fused network -- replaces the launch sequences that ARE the reference's model:
 * forward_pass (main.cu:55-92), back_pass (main.cu:95-123), learn (125-170), classify/test
 * (173-208), with the four Layer globals of main.cu:17-20 as one parameter arena.
 * ---------------------------------------------------------------------------------------- */
typedef struct cnn_net cnn_net;

/* Creates the net on the current CUDA device.  Parameters are drawn like the reference's static
 * Layer objects would draw them after srand(seed) (c1, s1, f in that order; main.cu:17-20), so
 * seed 0 or 1 gives the reference binary's own initial parameters.  The draw goes through the C
 * library's srand / rand, like the reference's: it reseeds the process-wide generator and must not
 * run concurrently with other users of rand(). */
int cnn_net_create(unsigned int seed, cnn_net** out);
int cnn_net_destroy(cnn_net* net);
/* Blocking copies of the 2343-float arena from / to host memory.  cnn_net_set_params waits for all
 * work on the device before and after its upload, so a launch on any stream (non-blocking ones
 * included) that follows it sees the new values, and none in flight sees a mixture. */
int cnn_net_set_params(cnn_net* net, const float* h_params);
int cnn_net_get_params(cnn_net* net, float* h_params);
/* Device pointer of the arena (CNN_N_PARAMS floats, padded to 2368), for collectives. */
int cnn_net_params_device(cnn_net* net, float** d_params);

/* Sigmoid of the fused kernels (the per-operator kernels always use the reference's expression):
 *   0 = the reference's own expression 1/(1+expf(-v)) with IEEE division (layer.cu:81-84): equal
 *       pre-activations give bit-equal activations, about 21 instructions per evaluation;
 *   non-zero (default) = the short form, ex2.approx and rcp.approx (the special-function instructions
 *       expf and the division are themselves built on), four instructions, about 1e-6 relative per
 *       evaluation.  On the network's outputs the two are equally close to an fp64 evaluation: 2.1e-6
 *       over the 65,536 images of benchmark configuration 2, where the fp32 oracle itself is 4.0e-6 away
 *       (tests/test_gpu_forward.py prints both).
 * Both meet the 1e-5 parity bar in every test. */
int cnn_net_set_fast_sigmoid(cnn_net* net, int enable);

/* Synchronises the device and reports whether any kernel of this net gave up a bounded wait since
 * the last call (CNN_ERR_TIMEOUT, *status non-zero); the status word is cleared. */
int cnn_net_status(cnn_net* net, int* status);

/* Batched forward (forward_pass + classify for n images at once): d_images [n][28][28] ->
 * d_out [n][10] sigmoids and d_argmax [n] (lowest index wins ties, main.cu:183-189).  Either
 * output may be NULL.  One fused kernel; activations never leave the chip. */
int cnn_forward_batched(cnn_net* net, const float* d_images, long n, float* d_out, int* d_argmax,
                        void* stream);

/* Same through host buffers: pipelined pinned-or-pageable H2D of the images in chunks, the fused
 * kernel per chunk, D2H of the results; returns after everything has landed.  The pipeline runs on
 * two private streams which are first ordered behind all work queued so far on the legacy default
 * stream (stream NULL: a cnn_apply_update, cnn_train_minibatch or cnn_grad_batch issued there is
 * seen).  Work that updates the parameters on a caller's own non-blocking stream is not waited for:
 * synchronise that stream before this call. */
int cnn_forward_batched_host(cnn_net* net, const float* h_images, long n, float* h_out,
                             int* h_argmax);

/* The same two calls for uint8 pixels [n][28][28] -- the storage of the IDX files the reference's
 * loader reads (mnist.h:79-160).  The kernel applies the reference's ingest, float(pixel / 255.0)
 * (mnist.h:145, main.cu:57-65), on the fly, so results are bit-identical to the fp32 calls on the
 * converted images while a quarter of the bytes cross PCIe and HBM. */
int cnn_forward_batched_u8(cnn_net* net, const unsigned char* d_pixels, long n, float* d_out,
                           int* d_argmax, void* stream);
int cnn_forward_batched_u8_host(cnn_net* net, const unsigned char* h_pixels, long n, float* h_out,
                                int* h_argmax);

/* Device-side synthetic data (stands in for the MNIST files the reference reads, main.cu:30-33):
 * image i of the set 'seed' = strokes of uint8 values 128..255 on a zero canvas, stored as
 * float(uint8)/255 like mnist.h:145; label = hash % 10.  Bit-identical to the host generator in
 * the Python package.  d_labels may be NULL. */
int cnn_synth_images(unsigned long long seed, long first_index, long n, float* d_images,
                     unsigned int* d_labels, void* stream);

/* Options, by name:
 *   "forward_path"     kernel behind cnn_forward_batched (fp32 images): 0 = exact fp32 on the CUDA
 *                      cores; 1 = the convolution on the tensor cores (tcgen05) in three tf32 passes,
 *                      fp32-level accuracy, same 1e-5 parity bar; -1 (default) = 1 for batches of 6,144
 *                      images or more (where it is the faster one) and 0 below, or always 0 when the
 *                      reference's sigmoid expression is selected; 2 = one tf32 pass and a tanh.approx
 *                      sigmoid: about 1e-4 on the outputs, argmax equal wherever the top-two margin is
 *                      clear of that -- an explicitly reduced-precision inference mode, never chosen
 *                      unless asked for;
 *   "persample_kernel" kernel of cnn_train_sgd_persample: 1 (default) = a cluster of six CTAs, one per
 *                      feature map, exchanging partial sums by one-way stores counted on mbarriers;
 *                      0 = one persistent block (no cluster launch needed), about half the speed;
 *   "fast_sigmoid"     as cnn_net_set_fast_sigmoid. */
int cnn_net_set_option(cnn_net* net, const char* key, int value);

/* ------------------------------------------------------------------------------------------
 * Training.  The "gradient" of one image is what one reference step would add to each parameter,
 * divided by dt: the d_weight buffers for weights (bp_weight_f / bp_weight_s1 / bp_weight_c1,
 * layer.cu:218-234, 285-304, 363-381), and for biases delta_f[k], sum(delta_s)/216 and
 * sum(delta_c[f])/576 (bp_bias_f / bp_bias_s1 / bp_bias_c1, layer.cu:236-246, 306-322, 383-399).
 * With a batch of one, params += dt * gradient is the reference's step.
 * ---------------------------------------------------------------------------------------- */

/* forward_pass + makeError + back_pass (main.cu:55-123, 147-153) for n images at FIXED parameters:
 * d_grad[0..2342] = sum of the per-image gradients (arena order), d_grad[2344] = sum of the
 * per-image error norms ||delta_f||_2 (what cublasSnrm2 returns at main.cu:153); the rest of the
 * 2368 floats is zero.  Uses the net's scratch rows; deterministic (no atomics). */
int cnn_grad_batch(cnn_net* net, const float* d_images, const unsigned int* d_labels, long n,
                   float* d_grad, void* stream);
/* apply_grad for the whole arena (layer.cu:106-114 with a caller-chosen step):
 * params[i] += scale * d_grad[i], i < 2343. */
int cnn_apply_update(cnn_net* net, const float* d_grad, float scale, void* stream);

/* Minibatch SGD over n images in index order: for each batch of `batch` images (the last one may
 * be smaller) params += (dt / batch_size) * sum of gradients.  d_mean_err (device, `epochs`
 * floats, may be NULL) receives the per-epoch mean error norm.  Asynchronous on `stream`. */
int cnn_train_minibatch(cnn_net* net, const float* d_images, const unsigned int* d_labels, long n,
                        int batch, int epochs, float dt, float* d_mean_err, void* stream);

/* learn() (main.cu:125-170): per-sample SGD in index order, one step per image, in one persistent
 * kernel; after each epoch the mean error norm goes to h_mean_err[epoch] and training stops early
 * when it is below `threshold` (the reference uses 0.01; pass a negative value to disable).
 * Blocking; *h_epochs_run receives the number of epochs run. */
int cnn_train_sgd_persample(cnn_net* net, const float* d_images, const unsigned int* d_labels, long n,
                            int epochs, float dt, float threshold, float* h_mean_err, int* h_epochs_run,
                            void* stream);

/* No counterpart in the reference.  The same computation as cnn_grad_batch for callers that must
 * not allocate device memory: no cnn_net is needed (creating one allocates), only raw device
 * pointers -- d_params (2343 floats, arena order), the images and labels, and d_grad (2368 floats,
 * same layout as cnn_grad_batch).  Nothing in this call allocates or frees, on the device or through
 * any library: the per-block partial rows live in a 1.5 MB array inside the library image
 * (160 rows; every GPU that loads the library holds that memory until the process exits).
 *   - at most 65,536 images per call; larger batches are rejected with CNN_ERR_INVALID (split them:
 *     gradients of sub-batches add);
 *   - the first call on each device looks up the array's device address and raises the kernel's
 *     shared-memory limit; make that first call outside any stream capture;
 *   - all calls on one device share the one array (it still holds the previous call's rows), so two
 *     calls whose kernels can overlap on the GPU -- different streams, or different host threads --
 *     race; serialise them on one stream or with events;
 *   - the reference sigmoid (flavour 0) is used;
 *   - a bounded device-side wait that runs out (never seen in practice: it would mean a bulk copy
 *     that did not land within seconds) cannot be reported by this asynchronous call; it sets a
 *     word in the array that cnn_grad_batch_noalloc_status reads. */
int cnn_grad_batch_noalloc(const float* d_params, const float* d_images, const unsigned int* d_labels,
                           long n, float* d_grad, void* stream);
/* No counterpart in the reference.  Waits for `stream`, then reports whether any
 * cnn_grad_batch_noalloc call on the current device gave up a bounded wait since the last query
 * (CNN_ERR_TIMEOUT: the gradient of that call is not valid; the word is cleared), else CNN_OK.
 * Allocates nothing. */
int cnn_grad_batch_noalloc_status(void* stream);

/* ------------------------------------------------------------------------------------------
 * Data-parallel minibatch SGD over the GPUs of one box (one host thread or process per GPU).  No
 * counterpart in the reference, which trains on a single GPU (main.cu:125-170 is its whole loop and
 * there is no collective in layer.cu / main.cu); the per-step arithmetic is cnn_train_minibatch's.
 * Every rank computes the summed gradient of its slice of a global batch; one kernel per step then
 * reduces the rank's partial rows, stores the 2368-float vector into a per-source slot of every
 * rank's exchange buffer (through peer-mapped memory over NVLink; every element travels as one
 * 64-bit word holding the value and the step number, so a word is its own arrival flag), polls --
 * bounded -- its own buffer for all ranks' words of the step, adds the values in rank order
 * and applies params += (dt / global_batch) * sum.  All ranks add the same values in the same order,
 * so their parameters stay bit-identical.  A wait that runs out (a rank that never sent) leaves the
 * parameters of that step untouched and is reported by cnn_net_status as CNN_ERR_TIMEOUT.
 *
 * Set-up: cnn_dp_create on every rank (allocates the rank's exchange buffer on the current device),
 * then either exchange the 64-byte handles of cnn_dp_export_handle between PROCESSES by any host
 * channel and pass all of them, in rank order, to cnn_dp_connect (CUDA IPC), or, for ranks that are
 * THREADS of one process, pass the pointers of cnn_dp_local_buffer to cnn_dp_connect_pointers (peer
 * access between the devices must be enabled by the caller).  world <= 8.
 * ---------------------------------------------------------------------------------------- */
typedef struct cnn_dp cnn_dp;
#define CNN_DP_HANDLE_BYTES 64
int cnn_dp_create(cnn_net* net, int rank, int world, cnn_dp** out);
int cnn_dp_destroy(cnn_dp* dp);
int cnn_dp_export_handle(cnn_dp* dp, void* handle /* CNN_DP_HANDLE_BYTES */);
int cnn_dp_connect(cnn_dp* dp, const void* handles /* world * CNN_DP_HANDLE_BYTES, rank order */);
int cnn_dp_local_buffer(cnn_dp* dp, void** d_buffer);
int cnn_dp_connect_pointers(cnn_dp* dp, void* const* d_buffers /* world device pointers, rank order */);
/* "wait_limit_ms" (default 2000): bound of the device-side waits for the other ranks.
 * "drop_next_send" = 1: host-side fault injection for tests -- the next step of this rank sends
 * nothing, so every rank's wait runs out and reports CNN_ERR_TIMEOUT. */
int cnn_dp_set_option(cnn_dp* dp, const char* key, int value);
/* One step: gradient of this rank's n_local images (may be 0), exchange, params += scale * sum over
 * all ranks.  d_grad_sum (2368 floats, may be NULL) receives the all-rank sum; if d_mean_err is given,
 * *d_mean_err += err_scale * (all-rank sum of the error norms).  Asynchronous on `stream`; every rank
 * must call it the same number of times. */
int cnn_dp_step(cnn_dp* dp, const float* d_images, const unsigned int* d_labels, long n_local, float scale,
                float* d_grad_sum, float* d_mean_err, float err_scale, void* stream);
/* cnn_train_minibatch across the ranks: d_images / d_labels hold ALL n images on every rank; of each
 * global batch of `global_batch` images (the last may be smaller) rank r takes the contiguous slice
 * [size*r/world, size*(r+1)/world).  d_mean_err (device, `epochs` floats, may be NULL) receives the
 * per-epoch mean error norm over all n images, identical on every rank.  Asynchronous on `stream`. */
int cnn_train_minibatch_dp(cnn_dp* dp, const float* d_images, const unsigned int* d_labels, long n,
                           long global_batch, int epochs, float dt, float* d_mean_err, void* stream);

/* ------------------------------------------------------------------------------------------
 * Widened variant of the same topology: input HxH, F maps of 5x5 -> sigmoid -> one shared 4x4 /
 * stride-4 filter -> sigmoid -> FC F*P*P -> 10 -> sigmoid (C = H-4, P = C/4).  The reference's
 * kernels are fixed to 28x28 / 6 maps (layer.h:45-62); this is the same operator sequence
 * (layer.cu:116-399 in main.cu's order) with its literals generalised: divisors (H-4)^2 for the conv
 * gradient and conv bias, F*P*P for the subsample bias.  Parameter arena:
 * [Wc F*25 | bc F | Ws 16 | bs 1 | Wf 10*F*P*P | bf 10]; gradient vectors hold the arena, then 0, then
 * the sum of error norms, zero-padded to a multiple of 32 floats.
 * ---------------------------------------------------------------------------------------- */
typedef struct cnn_wide cnn_wide;
int cnn_wide_param_count(int H, int F);
int cnn_wide_create(int H, int F, cnn_wide** out);       /* parameters start at zero */
int cnn_wide_destroy(cnn_wide* w);
int cnn_wide_set_params(cnn_wide* w, const float* h_params);
int cnn_wide_get_params(cnn_wide* w, float* h_params);
/* "fast_sigmoid": 0 = the reference's expression, 1 = the short form (default, as for cnn_net), 2 = a
 * refined form (two-step argument reduction, Newton-refined reciprocal); "conv": 0 = fp32 SIMT
 * convolution, 1 = implicit GEMM on the tf32 tensor cores (tcgen05, about 1e-3 relative), 2 = the same
 * in three tf32 passes (hi*hi + lo*hi + hi*lo, fp32-level accuracy).  The tensor-core forward needs F to
 * be a multiple of 16, at most 256; the fused tensor-core backward (conv deltas + weight gradients in one
 * TMA-fed kernel) needs F = 64 and H a multiple of 4, otherwise the fp32 SIMT backward runs. */
int cnn_wide_set_option(cnn_wide* w, const char* key, int value);
/* As cnn_net_status. */
int cnn_wide_status(cnn_wide* w, int* status);
/* forward_pass + classify for n images [n][H][H] -> d_out [n][10], d_argmax [n] (either may be NULL). */
int cnn_wide_forward(cnn_wide* w, const float* d_images, long n, float* d_out, int* d_argmax, void* stream);
/* forward + makeError + back_pass for n images at fixed parameters: summed gradient as for
 * cnn_grad_batch. */
int cnn_wide_grad_batch(cnn_wide* w, const float* d_images, const unsigned int* d_labels, long n,
                        float* d_grad, void* stream);
int cnn_wide_apply_update(cnn_wide* w, const float* d_grad, float scale, void* stream);

/* ------------------------------------------------------------------------------------------
 * Parameter checkpoints.  The reference keeps its parameters only in the device buffers of its
 * four static Layer objects (main.cu:17-20, filled at layer.cu:19-27) and loses them at exit; these
 * calls write / read them as a file: little-endian, 32-byte header {magic "CNNB200P", version 1,
 * kind (0 = 28x28 net, 1 = widened), H, F, parameter count, seed}, the arena as fp32, and a 64-bit
 * FNV-1a checksum of header + arena.  Loading checks magic, version, shape and checksum and leaves
 * the net untouched on any mismatch (CNN_ERR_INVALID).  Both calls block.
 * ---------------------------------------------------------------------------------------- */
int cnn_net_save(cnn_net* net, const char* path);
int cnn_net_load(cnn_net* net, const char* path);
int cnn_wide_save(cnn_wide* w, const char* path);
int cnn_wide_load(cnn_wide* w, const char* path);

/* Blocking copies between host and device memory (for bindings without a CUDA runtime of their own). */
int cnn_copy_to_host(void* h_dst, const void* d_src, size_t bytes);
int cnn_copy_to_device(void* d_dst, const void* h_src, size_t bytes);

#ifdef __cplusplus
}
#endif
#endif /* CNN_B200_H */
