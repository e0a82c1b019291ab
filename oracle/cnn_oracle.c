/*
 * CPU oracle for the conv -> sigmoid -> shared-weight subsample -> sigmoid -> FC -> sigmoid
 * network.  TEST INFRASTRUCTURE ONLY: this file is the checker that the CUDA path is compared
 * against (and the timed host-CPU baseline of the benchmark); nothing in the shipped library
 * links, imports or calls it.
 *
 * It restates, as plain owner-computes loops, the arithmetic of the reference's per-sample CUDA
 * kernels (layer.cu:81-399) in the launch order of main.cu:55-123, 137-167, 173-192.  Each
 * accumulating reference kernel adds its terms with float atomicAdd in an order that varies from
 * run to run; here every output adds its terms in ascending order of the reference's flat work
 * index n (one legal ordering of those atomics).  Products that the reference hands to atomicAdd
 * are rounded before the add (no FMA contraction is possible there), so this file must be built
 * with -ffp-contract=off; the two places where nvcc does contract (apply_grad, bp_bias_f:
 * "x += dt * g") call fma() explicitly.
 *
 * Parity status: pinned.  The reference ships no tests, fixtures or recorded outputs, so the pin is
 * the reference's own kernels: compiled unmodified into oracle/_ref/libref_cnn.so (ref_harness.cu,
 * build_oracle.py) they are run next to this restatement by the -m gpu tests, and their outputs on
 * seeded inputs, recorded on a B200 (tests/golden/make_golden.py), are committed under tests/golden/
 * and checked against this file by the CPU tests.
 *
 * The same source is compiled twice: REAL=float (symbols *_f32, the oracle proper) and REAL=double
 * (symbols *_f64, used to bound fp32 rounding).
 *
 * Shapes are generalised over H (input side) and F (feature maps): C = H-4 conv output side,
 * P = C/4 subsample side, FC fan-in F*P*P, 10 outputs.  H=28,F=6 is the reference net.
 * Parameter arena order: [Wc F*25 | bc F | Ws 16 | bs 1 | Wf 10*F*P*P | bf 10], each block laid
 * out exactly as the reference's Layer::weight / Layer::bias (unit-major, layer.cu:19-27).
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#ifndef REAL
#define REAL float
#endif
#ifndef SUFFIX
#define SUFFIX _f32
#endif
#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUFFIX)

typedef REAL real;

#define N_OUT 10

typedef struct {
  int H, F, C, P, S; /* S = F*P*P, FC fan-in */
  int o_wc, o_bc, o_ws, o_bs, o_wf, o_bf, n_params;
} dims_t;

static dims_t make_dims(int H, int F) {
  dims_t d;
  d.H = H; d.F = F; d.C = H - 4; d.P = d.C / 4; d.S = F * d.P * d.P;
  d.o_wc = 0;
  d.o_bc = d.o_wc + F * 25;
  d.o_ws = d.o_bc + F;
  d.o_bs = d.o_ws + 16;
  d.o_wf = d.o_bs + 1;
  d.o_bf = d.o_wf + N_OUT * d.S;
  d.n_params = d.o_bf + N_OUT;
  return d;
}

int FN(oracle_param_count)(int H, int F) { return make_dims(H, F).n_params; }

/* step_function, layer.cu:81-84: 1/(1+exp(-v)) in the working precision. */
static inline real sigmoid(real v) {
#if defined(REAL_IS_DOUBLE)
  return 1.0 / (1.0 + exp(-v));
#else
  return 1.0f / (1.0f + expf(-v));
#endif
}

static inline real fma_r(real a, real b, real c) {
#if defined(REAL_IS_DOUBLE)
  return fma(a, b, c);
#else
  return fmaf(a, b, c);
#endif
}

/* Pointers to every intermediate the reference keeps in its Layer buffers.  Any may be NULL
 * except where noted; sizes in elements. */
typedef struct {
  real *c1_preact;  /* [F][C][C]   l_c1.preact   */
  real *c1_output;  /* [F][C][C]   l_c1.output   */
  real *s1_preact;  /* [F][P][P]   l_s1.preact   */
  real *s1_output;  /* [F][P][P]   l_s1.output   */
  real *f_preact;   /* [10]        l_f.preact    */
  real *f_output;   /* [10]        l_f.output    */
  real *f_d_preact; /* [10]        l_f.d_preact (makeError) */
  real *f_d_weight; /* [10][S]     l_f.d_weight  */
  real *s1_d_output;/* [F][P][P]   l_s1.d_output */
  real *s1_d_preact;/* [F][P][P]   l_s1.d_preact */
  real *s1_d_weight;/* [16]        l_s1.d_weight */
  real *c1_d_output;/* [F][C][C]   l_c1.d_output */
  real *c1_d_preact;/* [F][C][C]   l_c1.d_preact */
  real *c1_d_weight;/* [F][25]     l_c1.d_weight */
} FN(oracle_trace);

/* ------------------------------------------------------------------------------------------
 * Forward, one image.  Follows fp_preact_c1 / fp_bias_c1 / apply_step_function / fp_preact_s1 /
 * fp_bias_s1 / fp_preact_f / fp_bias_f (layer.cu:116-216) in the order of main.cu:76-88.
 * All six output arrays are required.
 * ---------------------------------------------------------------------------------------- */
static void forward_one(const dims_t *d, const real *prm, const real *x, real *zc, real *ac,
                        real *zs, real *as, real *zf, real *af) {
  const int H = d->H, F = d->F, C = d->C, P = d->P, S = d->S;
  const real *Wc = prm + d->o_wc, *bc = prm + d->o_bc, *Ws = prm + d->o_ws;
  const real *bs = prm + d->o_bs, *Wf = prm + d->o_wf, *bf = prm + d->o_bf;

  /* c1: zc[f][y][x] = sum W[f][i][j]*in[y+i][x+j]; the reference's n has the row offset i
   * fastest, then j (layer.cu:124-131), so per output: j outer, i inner; bias added afterwards
   * (fp_bias_c1, layer.cu:135-150). */
  for (int f = 0; f < F; ++f)
    for (int y = 0; y < C; ++y)
      for (int xx = 0; xx < C; ++xx) {
        real acc = 0;
        for (int j = 0; j < 5; ++j)
          for (int i = 0; i < 5; ++i) acc += Wc[f * 25 + i * 5 + j] * x[(y + i) * H + (xx + j)];
        acc += bc[f];
        zc[(f * C + y) * C + xx] = acc;
        ac[(f * C + y) * C + xx] = sigmoid(acc);
      }

  /* s1: one 4x4 filter shared by all maps, stride 4 (fp_preact_s1, layer.cu:152-169);
   * per output: j outer, i inner; then + bs[0] (layer.cu:171-186). */
  for (int f = 0; f < F; ++f)
    for (int p = 0; p < P; ++p)
      for (int q = 0; q < P; ++q) {
        real acc = 0;
        for (int j = 0; j < 4; ++j)
          for (int i = 0; i < 4; ++i)
            acc += Ws[i * 4 + j] * ac[(f * C + (4 * p + i)) * C + (4 * q + j)];
        acc += bs[0];
        zs[(f * P + p) * P + q] = acc;
        as[(f * P + p) * P + q] = sigmoid(acc);
      }

  /* f: zf[k] = sum Wf[k][f][p][q]*as[f][p][q] (fp_preact_f, layer.cu:188-204); for a fixed k
   * the reference's n runs f fastest, then p, then q; then + bf[k] (layer.cu:206-216). */
  for (int k = 0; k < N_OUT; ++k) {
    real acc = 0;
    for (int q = 0; q < P; ++q)
      for (int p = 0; p < P; ++p)
        for (int f = 0; f < F; ++f) {
          const int s = (f * P + p) * P + q;
          acc += Wf[k * S + s] * as[s];
        }
    acc += bf[k];
    zf[k] = acc;
    af[k] = sigmoid(acc);
  }
}

/* classify, main.cu:183-189: strict '<', so the lowest index wins ties. */
static int argmax10(const real *v) {
  int m = 0;
  for (int i = 1; i < N_OUT; ++i)
    if (v[m] < v[i]) m = i;
  return m;
}

typedef struct {
  real *zc, *ac, *zs, *as, *zf, *af;      /* forward */
  real *df, *das, *ds, *dac, *dc;          /* backward deltas */
  real *gwf, *gws, *gwc;                   /* weight gradients (reference d_weight buffers) */
} scratch_t;

static size_t scratch_elems(const dims_t *d) {
  const size_t FCC = (size_t)d->F * d->C * d->C, S = (size_t)d->S;
  return 2 * FCC + 2 * S + 2 * N_OUT + N_OUT + 2 * S + 2 * FCC + (size_t)N_OUT * S + 16 +
         (size_t)d->F * 25;
}

static void carve(const dims_t *d, real *buf, scratch_t *s) {
  const size_t FCC = (size_t)d->F * d->C * d->C, S = (size_t)d->S;
  s->zc = buf; buf += FCC;  s->ac = buf; buf += FCC;
  s->zs = buf; buf += S;    s->as = buf; buf += S;
  s->zf = buf; buf += N_OUT; s->af = buf; buf += N_OUT;
  s->df = buf; buf += N_OUT;
  s->das = buf; buf += S;   s->ds = buf; buf += S;
  s->dac = buf; buf += FCC; s->dc = buf; buf += FCC;
  s->gwf = buf; buf += (size_t)N_OUT * S;
  s->gws = buf; buf += 16;
  s->gwc = buf; buf += (size_t)d->F * 25;
}

/* ------------------------------------------------------------------------------------------
 * Backward quantities that depend only on pre-update parameters: makeError (layer.cu:96-104),
 * bp_weight_f (218-234), bp_output_s1 (248-264), bp_preact_s1 (266-283), bp_weight_s1 (285-304),
 * bp_output_c1 (324-342), bp_preact_c1 (344-361), bp_weight_c1 (363-381).  The three in-place
 * bias kernels and apply_grad are applied by the callers, because per-sample SGD and the
 * minibatch rule use them differently.
 * ---------------------------------------------------------------------------------------- */
static void backward_deltas(const dims_t *d, const real *prm, const real *x, unsigned label,
                            scratch_t *s) {
  const int H = d->H, F = d->F, C = d->C, P = d->P, S = d->S;
  const real *Ws = prm + d->o_ws, *Wf = prm + d->o_wf;
  const real dc1 = (real)(C * C); /* pow(24,2) at layer.cu:369 */

  /* makeError: delta_f[k] = [k==label] - a_f[k]; there is no sigmoid-derivative factor. */
  for (int k = 0; k < N_OUT; ++k) s->df[k] = ((label == (unsigned)k) ? (real)1 : (real)0) - s->af[k];

  /* bp_weight_f: plain assignment. */
  for (int k = 0; k < N_OUT; ++k)
    for (int i = 0; i < S; ++i) s->gwf[k * S + i] = s->df[k] * s->as[i];

  /* bp_output_s1: per output the reference's n runs k ascending. */
  for (int i = 0; i < S; ++i) {
    real acc = 0;
    for (int k = 0; k < N_OUT; ++k) acc += Wf[k * S + i] * s->df[k];
    s->das[i] = acc;
  }
  /* bp_preact_s1: sigmoid recomputed from the pre-activation. */
  for (int i = 0; i < S; ++i) {
    const real o = sigmoid(s->zs[i]);
    s->ds[i] = s->das[i] * o * (1 - o);
  }
  /* bp_weight_s1: no normalisation (the 'd' of layer.cu:291 is unused).  n has the filter taps
   * fastest and then f, p, q, so per tap: q outer, p, f inner. */
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j) {
      real acc = 0;
      for (int q = 0; q < P; ++q)
        for (int p = 0; p < P; ++p)
          for (int f = 0; f < F; ++f)
            acc += s->ds[(f * P + p) * P + q] * s->ac[(f * C + (4 * p + i)) * C + (4 * q + j)];
      s->gws[i * 4 + j] = acc;
    }
  /* bp_output_c1: windows do not overlap, exactly one term per address. */
  for (int f = 0; f < F; ++f)
    for (int p = 0; p < P; ++p)
      for (int q = 0; q < P; ++q)
        for (int i = 0; i < 4; ++i)
          for (int j = 0; j < 4; ++j)
            s->dac[(f * C + (4 * p + i)) * C + (4 * q + j)] =
                (real)0 + Ws[i * 4 + j] * s->ds[(f * P + p) * P + q];
  /* rows/cols beyond 4*P (only when C is not a multiple of 4) receive nothing. */
  if (4 * P != C)
    for (int f = 0; f < F; ++f)
      for (int y = 0; y < C; ++y)
        for (int xx = 0; xx < C; ++xx)
          if (y >= 4 * P || xx >= 4 * P) s->dac[(f * C + y) * C + xx] = 0;
  /* bp_preact_c1. */
  for (int i = 0; i < F * C * C; ++i) {
    const real o = sigmoid(s->zc[i]);
    s->dc[i] = s->dac[i] * o * (1 - o);
  }
  /* bp_weight_c1: every term divided by C*C before the add (layer.cu:379); per output the
   * reference's n runs y fastest, then x. */
  for (int f = 0; f < F; ++f)
    for (int i = 0; i < 5; ++i)
      for (int j = 0; j < 5; ++j) {
        real acc = 0;
        for (int xx = 0; xx < C; ++xx)
          for (int y = 0; y < C; ++y)
            acc += s->dc[(f * C + y) * C + xx] * x[(y + i) * H + (xx + j)] / dc1;
        s->gwc[f * 25 + i * 5 + j] = acc;
      }
}

static void export_trace(const dims_t *d, const scratch_t *s, const FN(oracle_trace) * t) {
  const size_t FCC = (size_t)d->F * d->C * d->C, S = (size_t)d->S;
  if (!t) return;
#define CP(dst, src, n) if (t->dst) memcpy(t->dst, s->src, (n) * sizeof(real))
  CP(c1_preact, zc, FCC); CP(c1_output, ac, FCC);
  CP(s1_preact, zs, S);   CP(s1_output, as, S);
  CP(f_preact, zf, N_OUT); CP(f_output, af, N_OUT);
  CP(f_d_preact, df, N_OUT); CP(f_d_weight, gwf, (size_t)N_OUT * S);
  CP(s1_d_output, das, S); CP(s1_d_preact, ds, S); CP(s1_d_weight, gws, 16);
  CP(c1_d_output, dac, FCC); CP(c1_d_preact, dc, FCC); CP(c1_d_weight, gwc, (size_t)d->F * 25);
#undef CP
}

/* One per-sample SGD step with the reference's exact update semantics (main.cu:141-156,
 * 95-123): biases are incremented in place, term by term, during the backward sweep
 * (bp_bias_f 236-246, bp_bias_s1 306-322, bp_bias_c1 383-399: each term is (dt*delta)/count
 * and is added straight into the bias), weights wait for apply_grad (106-114) in the order f, s1,
 * c1.  Returns ||delta_f||_2 (cublasSnrm2 at main.cu:153) through *err_norm. */
static void sgd_step(const dims_t *d, real *prm, const real *x, unsigned label, real dt,
                     scratch_t *s, real *err_norm) {
  const int F = d->F, C = d->C, P = d->P, S = d->S;
  forward_one(d, prm, x, s->zc, s->ac, s->zs, s->as, s->zf, s->af);
  backward_deltas(d, prm, x, label, s);
  if (err_norm) {
    real ss = 0;
    for (int k = 0; k < N_OUT; ++k) ss += s->df[k] * s->df[k];
#if defined(REAL_IS_DOUBLE)
    *err_norm = sqrt(ss);
#else
    *err_norm = sqrtf(ss);
#endif
  }
  real *bc = prm + d->o_bc, *bs = prm + d->o_bs, *bf = prm + d->o_bf;
  real *Wc = prm + d->o_wc, *Ws = prm + d->o_ws, *Wf = prm + d->o_wf;
  /* bp_bias_f: bias += dt*delta, contracted to one fma by nvcc. */
  for (int k = 0; k < N_OUT; ++k) bf[k] = fma_r(dt, s->df[k], bf[k]);
  /* bp_bias_s1: n = f + F*(p + P*q) ascending; divisor is the s1 element count (pow(6,3)). */
  {
    const real ds1 = (real)S;
    for (int q = 0; q < P; ++q)
      for (int p = 0; p < P; ++p)
        for (int f = 0; f < F; ++f) bs[0] += dt * s->ds[(f * P + p) * P + q] / ds1;
  }
  /* bp_bias_c1: n = f + F*(y + C*x) ascending; divisor C*C. */
  {
    const real dc1 = (real)(C * C);
    for (int xx = 0; xx < C; ++xx)
      for (int y = 0; y < C; ++y)
        for (int f = 0; f < F; ++f) bc[f] += dt * s->dc[(f * C + y) * C + xx] / dc1;
  }
  /* apply_grad x3. */
  for (int i = 0; i < N_OUT * S; ++i) Wf[i] = fma_r(dt, s->gwf[i], Wf[i]);
  for (int i = 0; i < 16; ++i) Ws[i] = fma_r(dt, s->gws[i], Ws[i]);
  for (int i = 0; i < F * 25; ++i) Wc[i] = fma_r(dt, s->gwc[i], Wc[i]);
}

/* Per-sample "gradient" in arena order: what one reference step would add to each parameter,
 * divided by dt.  Weights: the d_weight buffers.  Biases: sum of delta/count terms. */
static void grad_one(const dims_t *d, const real *prm, const real *x, unsigned label, scratch_t *s,
                     real *G, real *err_norm) {
  const int F = d->F, C = d->C, P = d->P, S = d->S;
  forward_one(d, prm, x, s->zc, s->ac, s->zs, s->as, s->zf, s->af);
  backward_deltas(d, prm, x, label, s);
  if (err_norm) {
    real ss = 0;
    for (int k = 0; k < N_OUT; ++k) ss += s->df[k] * s->df[k];
#if defined(REAL_IS_DOUBLE)
    *err_norm = sqrt(ss);
#else
    *err_norm = sqrtf(ss);
#endif
  }
  memcpy(G + d->o_wc, s->gwc, sizeof(real) * F * 25);
  memcpy(G + d->o_ws, s->gws, sizeof(real) * 16);
  memcpy(G + d->o_wf, s->gwf, sizeof(real) * N_OUT * S);
  for (int k = 0; k < N_OUT; ++k) G[d->o_bf + k] = s->df[k];
  {
    real acc = 0;
    const real ds1 = (real)S;
    for (int q = 0; q < P; ++q)
      for (int p = 0; p < P; ++p)
        for (int f = 0; f < F; ++f) acc += s->ds[(f * P + p) * P + q] / ds1;
    G[d->o_bs] = acc;
  }
  {
    const real dc1 = (real)(C * C);
    for (int f = 0; f < F; ++f) {
      real acc = 0;
      for (int xx = 0; xx < C; ++xx)
        for (int y = 0; y < C; ++y) acc += s->dc[(f * C + y) * C + xx] / dc1;
      G[d->o_bc + f] = acc;
    }
  }
}

/* ============================== exported entry points ================================== */

/* Forward of one image with every intermediate exported (any trace pointer may be NULL). */
void FN(oracle_forward)(int H, int F, const real *params, const real *x,
                        const FN(oracle_trace) * trace) {
  dims_t d = make_dims(H, F);
  real *buf = (real *)calloc(scratch_elems(&d), sizeof(real));
  scratch_t s;
  carve(&d, buf, &s);
  forward_one(&d, params, x, s.zc, s.ac, s.zs, s.as, s.zf, s.af);
  if (trace) {
    FN(oracle_trace) t = *trace;
    t.f_d_preact = t.f_d_weight = t.s1_d_output = t.s1_d_preact = t.s1_d_weight = NULL;
    t.c1_d_output = t.c1_d_preact = t.c1_d_weight = NULL;
    export_trace(&d, &s, &t);
  }
  free(buf);
}

/* Batched forward: out[n][10] sigmoids and argmax[n] (either may be NULL).  OpenMP over
 * images with 'threads' threads (<=0: the OpenMP default). */
void FN(oracle_forward_batch)(int H, int F, const real *params, const real *x, long n, real *out,
                              int *argmax, int threads) {
  dims_t d = make_dims(H, F);
  const size_t img = (size_t)H * H;
#ifdef _OPENMP
  if (threads <= 0) threads = omp_get_max_threads();
#else
  threads = 1;
#endif
#pragma omp parallel num_threads(threads)
  {
    real *buf = (real *)calloc(scratch_elems(&d), sizeof(real));
    scratch_t s;
    carve(&d, buf, &s);
#pragma omp for schedule(static)
    for (long b = 0; b < n; ++b) {
      forward_one(&d, params, x + b * img, s.zc, s.ac, s.zs, s.as, s.zf, s.af);
      if (out) memcpy(out + b * N_OUT, s.af, sizeof(real) * N_OUT);
      if (argmax) argmax[b] = argmax10(s.af);
    }
    free(buf);
  }
}

/* One reference SGD step on one image; params updated in place. */
void FN(oracle_sgd_step)(int H, int F, real *params, const real *x, unsigned label, real dt,
                         real *err_norm, const FN(oracle_trace) * trace) {
  dims_t d = make_dims(H, F);
  real *buf = (real *)calloc(scratch_elems(&d), sizeof(real));
  scratch_t s;
  carve(&d, buf, &s);
  sgd_step(&d, params, x, label, dt, &s, err_norm);
  export_trace(&d, &s, trace);
  free(buf);
}

/* learn(), main.cu:125-170: up to 'epochs' passes in index order, one step per sample; the mean
 * of ||delta_f||_2 over each epoch goes to mean_err[epoch]; stops early after an epoch whose mean
 * is below 'threshold' (pass a negative threshold to disable).  Returns epochs run. */
int FN(oracle_train_persample)(int H, int F, real *params, const real *x, const unsigned *labels,
                               long n, int epochs, real dt, real threshold, real *mean_err) {
  dims_t d = make_dims(H, F);
  const size_t img = (size_t)H * H;
  real *buf = (real *)calloc(scratch_elems(&d), sizeof(real));
  scratch_t s;
  carve(&d, buf, &s);
  int e = 0;
  for (; e < epochs; ++e) {
    float err = 0.0f; /* the reference accumulates in a host float (main.cu:130, 154) */
    for (long i = 0; i < n; ++i) {
      real en;
      sgd_step(&d, params, x + i * img, labels[i], dt, &s, &en);
      err += (float)en;
    }
    err /= (float)n;
    if (mean_err) mean_err[e] = (real)err;
    if (err < (float)threshold) { ++e; break; }
  }
  free(buf);
  return e;
}

/* Summed per-sample gradients of a batch at fixed parameters: G[n_params] = sum_b G_b, images
 * added in index order (deterministic for any thread count: per-image vectors are computed in
 * parallel and then added serially).  err_sum receives sum_b ||delta_f||_2. */
void FN(oracle_grad_batch)(int H, int F, const real *params, const real *x, const unsigned *labels,
                           long n, real *G, real *err_sum, int threads) {
  dims_t d = make_dims(H, F);
  const size_t img = (size_t)H * H;
  const int np = d.n_params;
  real *all = (real *)malloc(sizeof(real) * (size_t)np * (size_t)(n > 0 ? n : 1));
  real *errs = (real *)malloc(sizeof(real) * (size_t)(n > 0 ? n : 1));
#ifdef _OPENMP
  if (threads <= 0) threads = omp_get_max_threads();
#else
  threads = 1;
#endif
#pragma omp parallel num_threads(threads)
  {
    real *buf = (real *)calloc(scratch_elems(&d), sizeof(real));
    scratch_t s;
    carve(&d, buf, &s);
#pragma omp for schedule(static)
    for (long b = 0; b < n; ++b)
      grad_one(&d, params, x + b * img, labels[b], &s, all + (size_t)b * np, errs + b);
    free(buf);
  }
  for (int i = 0; i < np; ++i) G[i] = 0;
  real es = 0;
  for (long b = 0; b < n; ++b) {
    for (int i = 0; i < np; ++i) G[i] += all[(size_t)b * np + i];
    es += errs[b];
  }
  if (err_sum) *err_sum = es;
  free(all);
  free(errs);
}

/* Minibatch rule used by the library: params += (dt / global_batch) * G for every parameter. */
void FN(oracle_apply_update)(int n_params, real *params, const real *G, real dt, real global_batch) {
  const real s = dt / global_batch;
  for (int i = 0; i < n_params; ++i) params[i] = fma_r(s, G[i], params[i]);
}

int FN(oracle_argmax10)(const real *v) { return argmax10(v); }
