/*
 * CPU oracle for the flutter_ml hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * A float64, scalar-loop restatement of the reference's pure-Dart eager engine:
 * same formulas, same loop order, same accumulate-into-grad (`+=`) semantics.
 * Only tests, the smoke check and the benchmark's CPU-baseline leg may load this
 * library; the product never does.
 *
 * Pinning status: the reference ships one known-answer check for this path
 * (all-ones 1024x1024x1024 matmul => every element equals k,
 * lib/gpu_benching.dart:34-37,60) and one fixed-input demo whose outputs follow
 * by hand (lib/autogradEngine/tensor.dart:1359-1376).  Both are tests here.
 * Everything else is PARITY UNPINNED: the reference holds no golden vectors and
 * its Dart code cannot be executed in this environment (no Dart SDK), so the
 * restatement is guarded by finite differences and an independent torch-float64
 * autograd model instead.
 *
 * Items marked EXTENSION do not exist in the reference and are defined here.
 *
 * Build: see oracle/Makefile (plain gcc, -O2, no -ffast-math; -fopenmp variant
 * parallelises only loops whose iterations are independent, so results are
 * bit-identical to the single-thread build).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#define ORC_PAR_FOR _Pragma("omp parallel for schedule(static)")
#else
#define ORC_PAR_FOR
#endif

/* Number of OpenMP threads to use from now on (ignored by the single-thread build). */
void orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int orc_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ---------------------------------------------------------------- matMul --- */

/* C[MxP] = A[MxN] . B[NxP].  lib/autogradEngine/tensor.dart:867-899: the
 * reference first materialises B^T (:877-884) and then takes row dot products
 * (:887-899); the summation order over k is ascending. */
void orc_matmul_fwd(const double* A, const double* B, double* C, int M, int N, int P) {
  double* bT = (double*)malloc(sizeof(double) * (size_t)N * P);
  for (int i = 0; i < P; i++)
    for (int j = 0; j < N; j++) bT[(size_t)i * N + j] = B[(size_t)j * P + i];
  ORC_PAR_FOR
  for (int i = 0; i < M; i++) {
    const double* rowA = A + (size_t)i * N;
    for (int j = 0; j < P; j++) {
      const double* rowBT = bT + (size_t)j * N;
      double sum = 0;
      for (int k = 0; k < N; k++) sum += rowA[k] * rowBT[k];
      C[(size_t)i * P + j] = sum;
    }
  }
  free(bT);
}

/* dA += dC . B^T (tensor.dart:918-924), dB += A^T . dC (:935-941); both
 * accumulate into the existing gradient.  Loop nests follow the reference. */
void orc_matmul_bwd(const double* A, const double* B, const double* dC, double* dA, double* dB,
                    int M, int N, int P) {
  if (dA) {
    ORC_PAR_FOR
    for (int i = 0; i < M; i++)
      for (int k = 0; k < N; k++) {
        double acc = dA[(size_t)i * N + k];
        for (int j = 0; j < P; j++) acc += dC[(size_t)i * P + j] * B[(size_t)k * P + j];
        dA[(size_t)i * N + k] = acc;
      }
  }
  if (dB) {
    ORC_PAR_FOR
    for (int k = 0; k < N; k++)
      for (int j = 0; j < P; j++) {
        double acc = dB[(size_t)k * P + j];
        for (int i = 0; i < M; i++) acc += A[(size_t)i * N + k] * dC[(size_t)i * P + j];
        dB[(size_t)k * P + j] = acc;
      }
  }
}

/* y[R] = M[RxC] . v[C]; tensor.dart:949-963.  Backward :965-974:
 * dM[i][j] += dy[i]*v[j]; dv[j] += M[i][j]*dy[i]. */
void orc_matvec_fwd(const double* Mx, const double* v, double* y, int R, int C) {
  for (int i = 0; i < R; i++) {
    double sum = 0;
    for (int j = 0; j < C; j++) sum += Mx[(size_t)i * C + j] * v[j];
    y[i] = sum;
  }
}
void orc_matvec_bwd(const double* Mx, const double* v, const double* dy, double* dM, double* dv,
                    int R, int C) {
  for (int i = 0; i < R; i++)
    for (int j = 0; j < C; j++) {
      if (dM) dM[(size_t)i * C + j] += dy[i] * v[j];
      if (dv) dv[j] += Mx[(size_t)i * C + j] * dy[i];
    }
}

/* ------------------------------------------------- bias add / elementwise --- */

/* Y = M + 1.b^T; tensor.dart:679-709.  Backward: dM += dY, db[j] += sum_i dY[i][j]. */
void orc_add_matrix_vector_fwd(const double* Mx, const double* b, double* Y, int R, int C) {
  for (int i = 0; i < R; i++)
    for (int j = 0; j < C; j++) Y[(size_t)i * C + j] = Mx[(size_t)i * C + j] + b[j];
}
void orc_add_matrix_vector_bwd(const double* dY, double* dM, double* db, int R, int C) {
  for (int i = 0; i < R; i++)
    for (int j = 0; j < C; j++) {
      if (dM) dM[(size_t)i * C + j] += dY[(size_t)i * C + j];
      if (db) db[j] += dY[(size_t)i * C + j];
    }
}

/* addMatrix tensor.dart:651-677 / addVector :395-414 (same arithmetic). */
void orc_add_fwd(const double* a, const double* b, double* y, int64_t n) {
  for (int64_t i = 0; i < n; i++) y[i] = a[i] + b[i];
}
void orc_add_bwd(const double* dy, double* da, double* db, int64_t n) {
  for (int64_t i = 0; i < n; i++) {
    if (da) da[i] += dy[i];
    if (db) db[i] += dy[i];
  }
}

/* elementWiseMultiply tensor.dart:478-497: da += dy*b, db += dy*a. */
void orc_mul_fwd(const double* a, const double* b, double* y, int64_t n) {
  for (int64_t i = 0; i < n; i++) y[i] = a[i] * b[i];
}
void orc_mul_bwd(const double* a, const double* b, const double* dy, double* da, double* db,
                 int64_t n) {
  for (int64_t i = 0; i < n; i++) {
    if (da) da[i] += dy[i] * b[i];
    if (db) db[i] += dy[i] * a[i];
  }
}

/* scaleMatrix tensor.dart:1075-1101. */
void orc_scale_fwd(const double* x, double s, double* y, int64_t n) {
  for (int64_t i = 0; i < n; i++) y[i] = x[i] * s;
}
void orc_scale_bwd(const double* dy, double s, double* dx, int64_t n) {
  for (int64_t i = 0; i < n; i++) dx[i] += dy[i] * s;
}

/* transpose tensor.dart:1211-1236 (backward adds the transposed gradient). */
void orc_transpose(const double* x, double* y, int R, int C) {
  for (int i = 0; i < R; i++)
    for (int j = 0; j < C; j++) y[(size_t)j * R + i] = x[(size_t)i * C + j];
}
void orc_transpose_bwd(const double* dy, double* dx, int R, int C) {
  for (int i = 0; i < R; i++)
    for (int j = 0; j < C; j++) dx[(size_t)i * C + j] += dy[(size_t)j * R + i];
}

/* ------------------------------------------------------------ activations --- */

/* reluMatrix tensor.dart:1013-1038; the gradient gate tests the PRE-activation
 * (`m.value > 0`, :1030). */
void orc_relu_fwd(const double* x, double* y, int64_t n) {
  for (int64_t i = 0; i < n; i++) y[i] = x[i] > 0 ? x[i] : 0.0;
}
void orc_relu_bwd(const double* x, const double* dy, double* dx, int64_t n) {
  for (int64_t i = 0; i < n; i++) dx[i] += dy[i] * (x[i] > 0 ? 1.0 : 0.0);
}

/* sigmoid tensor.dart:541-559 (matrix form :1123-1151): grad from the OUTPUT y(1-y). */
void orc_sigmoid_fwd(const double* x, double* y, int64_t n) {
  for (int64_t i = 0; i < n; i++) y[i] = 1.0 / (1.0 + exp(-x[i]));
}
void orc_sigmoid_bwd(const double* y, const double* dy, double* dx, int64_t n) {
  for (int64_t i = 0; i < n; i++) dx[i] += dy[i] * (y[i] * (1 - y[i]));
}

/* vectorTanh tensor.dart:581-605 (matrix form :1178-1209): (e^{2x}-1)/(e^{2x}+1),
 * returning exactly 1.0 when e^{2x} overflows (:582-586); grad 1 - y^2 (:598). */
void orc_tanh_fwd(const double* x, double* y, int64_t n) {
  for (int64_t i = 0; i < n; i++) {
    double e2x = exp(2 * x[i]);
    y[i] = isinf(e2x) ? 1.0 : (e2x - 1) / (e2x + 1);
  }
}
void orc_tanh_bwd(const double* y, const double* dy, double* dx, int64_t n) {
  for (int64_t i = 0; i < n; i++) dx[i] += dy[i] * (1 - y[i] * y[i]);
}

/* EXTENSION (no GELU in the reference): exact GELU 0.5*x*(1+erf(x/sqrt2));
 * derivative Phi(x) + x*phi(x). */
void orc_gelu_fwd(const double* x, double* y, int64_t n) {
  for (int64_t i = 0; i < n; i++) y[i] = 0.5 * x[i] * (1.0 + erf(x[i] * 0.70710678118654752440));
}
void orc_gelu_bwd(const double* x, const double* dy, double* dx, int64_t n) {
  for (int64_t i = 0; i < n; i++) {
    double cdf = 0.5 * (1.0 + erf(x[i] * 0.70710678118654752440));
    double pdf = 0.39894228040143267794 * exp(-0.5 * x[i] * x[i]);
    dx[i] += dy[i] * (cdf + x[i] * pdf);
  }
}

/* ---------------------------------------------------------------- softmax --- */

/* softmaxMatrix lib/activationFunctions/softmax.dart:68-96: per row, subtract
 * the max (:75-80), exponentiate, normalise (:82-93).
 * EXTENSION: causal_period > 0 masks column j > (r mod causal_period) to -inf
 * before the max; masked probabilities are exactly 0. */
void orc_softmax_rows_fwd(const double* x, double* y, int R, int C, int causal_period) {
  ORC_PAR_FOR
  for (int r = 0; r < R; r++) {
    const double* row = x + (size_t)r * C;
    double* out = y + (size_t)r * C;
    int lim = causal_period > 0 ? (r % causal_period) + 1 : C;
    if (lim > C) lim = C;
    double maxVal = -INFINITY;
    for (int j = 0; j < lim; j++)
      if (row[j] > maxVal) maxVal = row[j];
    double sumExps = 0.0;
    for (int j = 0; j < lim; j++) {
      out[j] = exp(row[j] - maxVal);
      sumExps += out[j];
    }
    for (int j = 0; j < lim; j++) out[j] = out[j] / sumExps;
    for (int j = lim; j < C; j++) out[j] = 0.0;
  }
}
/* softmax.dart:98-112: dx = y * (dy - sum_i dy_i y_i), accumulated. */
void orc_softmax_rows_bwd(const double* y, const double* dy, double* dx, int R, int C) {
  ORC_PAR_FOR
  for (int r = 0; r < R; r++) {
    const double* s = y + (size_t)r * C;
    const double* g = dy + (size_t)r * C;
    double dot = 0;
    for (int i = 0; i < C; i++) dot += g[i] * s[i];
    for (int j = 0; j < C; j++) dx[(size_t)r * C + j] += s[j] * (g[j] - dot);
  }
}

/* -------------------------------------------------------------- layerNorm --- */

/* layerNorm lib/transformer/layerNormalization.dart:137-169: per-row mean,
 * BIASED variance (:153-156), xhat=(x-mean)/sqrt(var+eps), y=gamma*xhat+beta. */
void orc_layernorm_fwd(const double* x, const double* gamma, const double* beta, double* y,
                       double* xhat, double* var, int R, int C, double eps) {
  ORC_PAR_FOR
  for (int r = 0; r < R; r++) {
    const double* row = x + (size_t)r * C;
    double mean = 0;
    for (int c = 0; c < C; c++) mean += row[c];
    mean /= C;
    double variance = 0;
    for (int c = 0; c < C; c++) variance += (row[c] - mean) * (row[c] - mean);
    variance /= C;
    var[r] = variance;
    for (int c = 0; c < C; c++) {
      double n = (row[c] - mean) / sqrt(variance + eps);
      xhat[(size_t)r * C + c] = n;
      y[(size_t)r * C + c] = gamma[c] * n + beta[c];
    }
  }
}
/* layerNormalization.dart:174-200. */
void orc_layernorm_bwd(const double* dy, const double* gamma, const double* xhat,
                       const double* var, double* dx, double* dgamma, double* dbeta, int R, int C,
                       double eps) {
  for (int r = 0; r < R; r++) {
    double sum_g = 0, dot = 0;
    for (int c = 0; c < C; c++) {
      double g = dy[(size_t)r * C + c] * gamma[c];
      if (dgamma) dgamma[c] += dy[(size_t)r * C + c] * xhat[(size_t)r * C + c];
      if (dbeta) dbeta[c] += dy[(size_t)r * C + c];
      sum_g += g;
    }
    for (int c = 0; c < C; c++) dot += dy[(size_t)r * C + c] * gamma[c] * xhat[(size_t)r * C + c];
    if (dx)
      for (int c = 0; c < C; c++) {
        double g = dy[(size_t)r * C + c] * gamma[c];
        double term1 = C * g, term2 = sum_g, term3 = xhat[(size_t)r * C + c] * dot;
        dx[(size_t)r * C + c] += (1.0 / (C * sqrt(var[r] + eps))) * (term1 - term2 - term3);
      }
  }
}

/* ------------------------------------------------------------------ losses --- */

/* mseMatrix tensor.dart:982-1011 (mse :499-519 is the same over a vector):
 * mean over all n elements; grad upstream*2(p-t)/n accumulated. */
double orc_mse_fwd(const double* p, const double* t, int64_t n) {
  double s = 0.0;
  for (int64_t i = 0; i < n; i++) {
    double e = p[i] - t[i];
    s += e * e;
  }
  return s / (double)n;
}
void orc_mse_bwd(const double* p, const double* t, double* dp, int64_t n, double upstream) {
  for (int64_t i = 0; i < n; i++) dp[i] += upstream * 2 * (p[i] - t[i]) / (double)n;
}

/* EXTENSION (the reference has no softmax cross-entropy): returns
 * sum_r -log softmax(z_r)[label_r] * inv_count and accumulates
 * dz += (softmax(z) - onehot) * inv_count.  inv_count = 1/(rows of the GLOBAL
 * batch) so that shards of a data-parallel step add up to the full-batch value. */
double orc_softmax_xent(const double* z, const int32_t* labels, double* dz, int R, int C,
                        double inv_count) {
  double loss = 0;
  for (int r = 0; r < R; r++) {
    const double* row = z + (size_t)r * C;
    double mx = -INFINITY;
    for (int j = 0; j < C; j++)
      if (row[j] > mx) mx = row[j];
    double se = 0;
    for (int j = 0; j < C; j++) se += exp(row[j] - mx);
    loss += -(row[labels[r]] - mx - log(se)) * inv_count;
    if (dz)
      for (int j = 0; j < C; j++)
        dz[(size_t)r * C + j] += (exp(row[j] - mx) / se - (j == labels[r] ? 1.0 : 0.0)) * inv_count;
  }
  return loss;
}

/* -------------------------------------------------------------- optimizers --- */

/* SGD.step lib/optimizers/sgd.dart:24-42. */
void orc_sgd_step(double* w, const double* g, int64_t n, double lr) {
  for (int64_t i = 0; i < n; i++) w[i] -= lr * g[i];
}
/* Adam.step lib/optimizers/adam.dart:44-77; t is the value of _t AFTER the
 * increment at :46; pow(beta,t) is evaluated per element as in :57-58. */
void orc_adam_step(double* w, const double* g, double* m, double* v, int64_t n, double lr,
                   double b1, double b2, double eps, int t) {
  for (int64_t i = 0; i < n; i++) {
    m[i] = b1 * m[i] + (1 - b1) * g[i];
    v[i] = b2 * v[i] + (1 - b2) * (g[i] * g[i]);
    double mHat = m[i] / (1 - pow(b1, t));
    double vHat = v[i] / (1 - pow(b2, t));
    w[i] -= lr * mHat / (sqrt(vHat) + eps);
  }
}

/* The other optimizers of lib/optimizers (same per-element loops; state arrays start at zero):
 *   1 Momentum  sgdmomentum.dart:56-57   v = mu v + lr g;  w -= v
 *   2 NAG       nag.dart:58-60           v = mu v + g;     w -= lr (g + mu v)
 *   3 RMSprop   rmsprop.dart:57-58       s = b s + (1-b) g^2;  w -= lr g / (sqrt(s) + eps)
 *   4 Adagrad   adagrad.dart:54-55       G += g^2;             w -= lr g / (sqrt(G) + eps)
 *   6 AdamW     adamw.dart:82-89         Adam step, then w -= lr wd w
 *   7 AMSGrad   amsgrad.dart:80-86       m, v as Adam; vhat = max(vhat, v); w -= lr mHat / (sqrt(vhat) + eps)
 * h1..h4: (mu) | (mu) | (b, eps) | (-, eps) | (b1, b2, eps, wd) | (b1, b2, eps). */
void orc_optimizer_step(int kind, double* w, const double* g, double* s1, double* s2, double* s3, int64_t n,
                        double lr, double h1, double h2, double h3, double h4, int t) {
  for (int64_t i = 0; i < n; i++) {
    switch (kind) {
      case 1: s1[i] = h1 * s1[i] + lr * g[i]; w[i] -= s1[i]; break;
      case 2: { double vNew = h1 * s1[i] + g[i]; s1[i] = vNew; w[i] -= lr * (g[i] + h1 * vNew); break; }
      case 3: s1[i] = h1 * s1[i] + (1 - h1) * (g[i] * g[i]); w[i] -= lr * g[i] / (sqrt(s1[i]) + h2); break;
      case 4: s1[i] += g[i] * g[i]; w[i] -= lr * g[i] / (sqrt(s1[i]) + h2); break;
      case 6: {
        s1[i] = h1 * s1[i] + (1 - h1) * g[i];
        s2[i] = h2 * s2[i] + (1 - h2) * (g[i] * g[i]);
        double mHat = s1[i] / (1 - pow(h1, t)), vHat = s2[i] / (1 - pow(h2, t));
        w[i] -= lr * mHat / (sqrt(vHat) + h3);
        w[i] -= lr * h4 * w[i];
        break;
      }
      case 7: {
        s1[i] = h1 * s1[i] + (1 - h1) * g[i];
        s2[i] = h2 * s2[i] + (1 - h2) * (g[i] * g[i]);
        s3[i] = s3[i] > s2[i] ? s3[i] : s2[i];
        double mHat = s1[i] / (1 - pow(h1, t));
        w[i] -= lr * mHat / (sqrt(s3[i]) + h3);
        break;
      }
      default: break;
    }
  }
}

/* LeakyReLU lib/activationFunctions/leakyRelu.dart:35-48, ELU elu.dart:27-41 (grad out + alpha for x <= 0),
 * Swish silu.dart:29-49, Mish mish.dart:29-31 = x * tanh(log(exp(x) + 1)) composed from tape ops. */
void orc_act2_fwd(int kind, double alpha, const double* x, double* y, int64_t n) {
  for (int64_t i = 0; i < n; i++) {
    double v = x[i];
    switch (kind) {
      case 5: y[i] = v > 0 ? v : alpha * v; break;
      case 6: y[i] = v > 0 ? v : alpha * (exp(v) - 1); break;
      case 7: y[i] = v * (1.0 / (1.0 + exp(-v))); break;
      case 8: { double sp = log(exp(v) + 1.0); double e2 = exp(2 * sp); y[i] = v * (isinf(e2) ? 1.0 : (e2 - 1) / (e2 + 1)); break; }
      default: y[i] = v;
    }
  }
}
void orc_act2_bwd(int kind, double alpha, const double* x, const double* dy, double* dx, int64_t n) {
  for (int64_t i = 0; i < n; i++) {
    double v = x[i], d = 1.0;
    switch (kind) {
      case 5: d = v > 0 ? 1.0 : alpha; break;
      case 6: d = v > 0 ? 1.0 : (alpha * (exp(v) - 1)) + alpha; break;
      case 7: { double sg = 1.0 / (1.0 + exp(-v)); d = sg * (1 + v * (1 - sg)); break; }
      case 8: {
        /* chain rule through multiply, tanh (1 - y^2), log (1/u), exp: as the tape would */
        double ex = exp(v), sp = log(ex + 1.0), e2 = exp(2 * sp), th = isinf(e2) ? 1.0 : (e2 - 1) / (e2 + 1);
        d = th + v * (1 - th * th) * (ex / (ex + 1.0));
        break;
      }
      default: break;
    }
    dx[i] += dy[i] * d;
  }
}

/* ------------------------------------------------- embedding / positional --- */

/* EmbeddingLayer.forward lib/transformer/embeddingLayer.dart:47-56: ids arrive
 * as doubles and are truncated with toInt(); backward :58-65 scatter-adds. */
void orc_embedding_fwd(const double* table, const double* ids, double* out, int n, int dim) {
  for (int i = 0; i < n; i++)
    memcpy(out + (size_t)i * dim, table + (size_t)((int64_t)ids[i]) * dim, sizeof(double) * dim);
}
void orc_embedding_bwd(const double* dout, const double* ids, double* dtable, int n, int dim) {
  for (int i = 0; i < n; i++) {
    int64_t idx = (int64_t)ids[i];
    for (int j = 0; j < dim; j++) dtable[(size_t)idx * dim + j] += dout[(size_t)i * dim + j];
  }
}
/* PositionalEncoding.build lib/transformer/positionalEncodingLayer.dart:39-48:
 * angle = pos / 10000^(2i/dModel) for EVERY column i (not i/2); sin for even i,
 * cos for odd i. */
void orc_positional_table(double* pe, int max_len, int d_model) {
  for (int pos = 0; pos < max_len; pos++)
    for (int i = 0; i < d_model; i++) {
      double angle = pos / pow(10000, (2.0 * i) / d_model);
      pe[(size_t)pos * d_model + i] = (i % 2 == 0) ? sin(angle) : cos(angle);
    }
}

/* -------------------------------------------------------------------- LSTM --- */

/* LSTMLayer.forward lib/layertypes/lstmLayer.dart:112-150 for a batch of
 * independent sequences, followed by the loss mse(h_T, target) per sequence
 * (tensor.dart:499-519) summed over the batch, and the backward pass the tape
 * would run (BPTT through matVecMul :965-974, addVector, sigmoid :552,
 * vectorTanh :598, elementWiseMultiply :487-490, concatenate :446-451).
 *
 * W: 4 gate matrices [H x (H+I)] in order f,i,c~,o (lstmLayer.dart:64), columns
 * [h_{t-1} | x_t] (:119).  b: 4 x H.  x: [B][T][I].  target: [B][H].
 * Outputs: h_last [B][H]; loss_out; dW [4][H][H+I], db [4][H] (accumulated,
 * caller zeroes).  Weight gradients are reduced over the batch in ascending
 * sample order, which is the order successive backward() calls would add them.
 */
static double orc_sig(double x) { return 1.0 / (1.0 + exp(-x)); }
static double orc_tanh1(double x) {
  double e2x = exp(2 * x);
  return isinf(e2x) ? 1.0 : (e2x - 1) / (e2x + 1);
}
void orc_lstm_fwd_bwd(const double* W, const double* b, const double* x, const double* target,
                      double* h_last, double* loss_out, double* dW, double* db, int B, int T, int I,
                      int H, int do_backward) {
  const int Z = H + I;
  double loss = 0;
  /* per-sample work is independent; gradients are reduced afterwards in sample order */
  double* dW_s = do_backward ? (double*)calloc((size_t)B * 4 * H * Z, sizeof(double)) : NULL;
  double* db_s = do_backward ? (double*)calloc((size_t)B * 4 * H, sizeof(double)) : NULL;
  double* losses = (double*)calloc(B, sizeof(double));
  ORC_PAR_FOR
  for (int s = 0; s < B; s++) {
    /* saved activations per step: z[T][Z], gates[T][4][H], c[T+1][H], tanh_c[T][H] */
    double* zs = (double*)calloc((size_t)T * Z, sizeof(double));
    double* gs = (double*)calloc((size_t)T * 4 * H, sizeof(double));
    double* cs = (double*)calloc((size_t)(T + 1) * H, sizeof(double));
    double* tc = (double*)calloc((size_t)T * H, sizeof(double));
    double* h = (double*)calloc(H, sizeof(double));
    for (int t = 0; t < T; t++) {
      double* z = zs + (size_t)t * Z;
      memcpy(z, h, sizeof(double) * H);
      memcpy(z + H, x + ((size_t)s * T + t) * I, sizeof(double) * I);
      double* g = gs + (size_t)t * 4 * H;
      for (int q = 0; q < 4; q++)
        for (int r = 0; r < H; r++) {
          const double* wr = W + ((size_t)q * H + r) * Z;
          double sum = 0;
          for (int j = 0; j < Z; j++) sum += wr[j] * z[j];
          sum = sum + b[q * H + r];
          g[q * H + r] = (q == 2) ? orc_tanh1(sum) : orc_sig(sum);
        }
      const double* cp = cs + (size_t)t * H;
      double* cn = cs + (size_t)(t + 1) * H;
      for (int r = 0; r < H; r++) {
        cn[r] = g[0 * H + r] * cp[r] + g[1 * H + r] * g[2 * H + r];
        tc[(size_t)t * H + r] = orc_tanh1(cn[r]);
        h[r] = g[3 * H + r] * tc[(size_t)t * H + r];
      }
    }
    memcpy(h_last + (size_t)s * H, h, sizeof(double) * H);
    double se = 0;
    for (int r = 0; r < H; r++) {
      double e = h[r] - target[(size_t)s * H + r];
      se += e * e;
    }
    losses[s] = se / H;
    if (do_backward) {
      double* dWs = dW_s + (size_t)s * 4 * H * Z;
      double* dbs = db_s + (size_t)s * 4 * H;
      double* dh = (double*)calloc(H, sizeof(double));
      double* dc = (double*)calloc(H, sizeof(double));
      double* dz = (double*)calloc(Z, sizeof(double));
      double* dpre = (double*)calloc((size_t)4 * H, sizeof(double));
      for (int r = 0; r < H; r++) dh[r] = 2 * (h[r] - target[(size_t)s * H + r]) / H;
      for (int t = T - 1; t >= 0; t--) {
        const double* g = gs + (size_t)t * 4 * H;
        const double* z = zs + (size_t)t * Z;
        const double* cp = cs + (size_t)t * H;
        for (int r = 0; r < H; r++) {
          double tcr = tc[(size_t)t * H + r];
          double d_o = dh[r] * tcr;                    /* h = o * tanh(c) */
          double d_tc = dh[r] * g[3 * H + r];
          double dct = dc[r] + d_tc * (1 - tcr * tcr); /* c feeds tanh(c) and c_{t+1} */
          double d_f = dct * cp[r];
          double d_i = dct * g[2 * H + r];
          double d_g = dct * g[1 * H + r];
          dc[r] = dct * g[0 * H + r];
          dpre[0 * H + r] = d_f * (g[0 * H + r] * (1 - g[0 * H + r]));
          dpre[1 * H + r] = d_i * (g[1 * H + r] * (1 - g[1 * H + r]));
          dpre[2 * H + r] = d_g * (1 - g[2 * H + r] * g[2 * H + r]);
          dpre[3 * H + r] = d_o * (g[3 * H + r] * (1 - g[3 * H + r]));
        }
        memset(dz, 0, sizeof(double) * Z);
        for (int q = 0; q < 4; q++)
          for (int r = 0; r < H; r++) {
            double d = dpre[q * H + r];
            dbs[q * H + r] += d;
            double* dwr = dWs + ((size_t)q * H + r) * Z;
            const double* wr = W + ((size_t)q * H + r) * Z;
            for (int j = 0; j < Z; j++) {
              dwr[j] += d * z[j];
              dz[j] += wr[j] * d;
            }
          }
        memcpy(dh, dz, sizeof(double) * H); /* concatenate backward: first H entries go to h_{t-1} */
      }
      free(dh); free(dc); free(dz); free(dpre);
    }
    free(zs); free(gs); free(cs); free(tc); free(h);
  }
  for (int s = 0; s < B; s++) loss += losses[s];
  if (do_backward) {
    for (int s = 0; s < B; s++) {
      for (size_t i = 0; i < (size_t)4 * H * Z; i++) dW[i] += dW_s[(size_t)s * 4 * H * Z + i];
      for (int i = 0; i < 4 * H; i++) db[i] += db_s[(size_t)s * 4 * H + i];
    }
    free(dW_s); free(db_s);
  }
  free(losses);
  *loss_out = loss;
}

/* conv2d lib/autogradEngine/tensor.dart:765-833: one input matrix [H x W], one kernel [kh x kw], cross-correlation
 * (no kernel flip); padding 'same' pads (kh - 1) / 2 zeros on every side (:773-776, integer division), so the
 * output is [H + 2p - kh + 1] x [W + 2p - kw + 1].  Loop order y, x, ky, kx as the reference. */
void orc_conv2d_fwd(const double* in, const double* k, double* out, int H, int W, int kh, int kw, int pad) {
  const int OH = H + 2 * pad - kh + 1, OW = W + 2 * pad - kw + 1;
  for (int y = 0; y < OH; y++)
    for (int x = 0; x < OW; x++) {
      double sum = 0;
      for (int ky = 0; ky < kh; ky++)
        for (int kx = 0; kx < kw; kx++) {
          const int iy = y + ky - pad, ix = x + kx - pad;
          const double v = (iy < 0 || iy >= H || ix < 0 || ix >= W) ? 0.0 : in[(size_t)iy * W + ix];
          sum += v * k[ky * kw + kx];
        }
      out[(size_t)y * OW + x] = sum;
    }
}
/* closure :808-826: input.grad += kernel * out.grad, kernel.grad += padded input * out.grad; positions in the
 * padding are skipped for BOTH gradients (the `continue` at :813-818). */
void orc_conv2d_bwd(const double* in, const double* k, const double* dout, double* din, double* dk, int H, int W,
                    int kh, int kw, int pad) {
  const int OH = H + 2 * pad - kh + 1, OW = W + 2 * pad - kw + 1;
  for (int y = 0; y < OH; y++)
    for (int x = 0; x < OW; x++)
      for (int ky = 0; ky < kh; ky++)
        for (int kx = 0; kx < kw; kx++) {
          const int iy = y + ky - pad, ix = x + kx - pad;
          if (iy < 0 || iy >= H || ix < 0 || ix >= W) continue;
          din[(size_t)iy * W + ix] += k[ky * kw + kx] * dout[(size_t)y * OW + x];
          dk[ky * kw + kx] += in[(size_t)iy * W + ix] * dout[(size_t)y * OW + x];
        }
}
