/*
 * TEST INFRASTRUCTURE — NOT PART OF THE PRODUCT.
 *
 * CPU restatement of the arithmetic of vnnm404/gpt2.cu's three linear-layer GEMMs
 * (include/gpt2/layers/mlp.h). Only tests/, __graft_entry__.smoke() and bench.py's CPU
 * baseline legs may load this file's library; the CUDA library never does.
 *
 * Parity pin: these functions are checked (tests/test_oracle.py) against fixtures under
 * tests/golden/ that were produced by running the reference's own PyTorch model
 * (scripts/llm.py: nn.Linear forward/backward inside GPT) in fp32, and — on a GPU box —
 * against the reference's own CUDA kernels compiled unmodified from its header
 * (oracle/_ref, see oracle/Makefile and tests/test_reference_kernels.py).
 *
 * Two flavours per GEMM:
 *   *_f32 : the reference's own order of operations — one fp32 accumulator per output,
 *           reduction index ascending, one fused multiply-add per step (the reference is
 *           built with --use_fast_math, which contracts `acc += a * b` into an FMA;
 *           mlp.h:282-294, 611-623, 929-941), bias added once at the end (mlp.h:305-333),
 *           bias gradient as a plain ascending sum over rows (mlp.h:970-995).
 *   *_f64 : the same sums with double accumulators and double output: the ground truth
 *           that error metrics are measured against.
 *
 * Conventions (as in the reference): in[M][K], w[K][N], out[M][N], all row-major fp32,
 * M = B*S; K and N describe the forward weight in all three calls; outputs are
 * overwritten; b / g_b may be NULL.
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static int g_threads = 0;

void oracle_set_threads(int n) { g_threads = n; }

int oracle_get_threads(void) {
#ifdef _OPENMP
  return g_threads > 0 ? g_threads : omp_get_max_threads();
#else
  return 1;
#endif
}

#ifdef _OPENMP
#define NT() (g_threads > 0 ? g_threads : omp_get_max_threads())
#else
#define NT() 1
#endif

/* ---- forward: out[m][n] = sum_k in[m][k] * w[k][n] + b[n]   (mlp.h:282-333) ---- */
int oracle_linear_forward_f32(float *out, const float *in, const float *w, const float *b, int B, int S, int K,
                              int N) {
  const long M = (long)B * S;
  if (M <= 0 || K <= 0 || N <= 0) return -2;
#pragma omp parallel for schedule(static) num_threads(NT())
  for (long m = 0; m < M; ++m) {
    float *acc = out + m * N;
    for (int n = 0; n < N; ++n) acc[n] = 0.0f;
    for (int k = 0; k < K; ++k) {
      const float a = in[m * K + k];
      const float *wr = w + (long)k * N;
      for (int n = 0; n < N; ++n) acc[n] = fmaf(a, wr[n], acc[n]);
    }
    if (b)
      for (int n = 0; n < N; ++n) acc[n] = acc[n] + b[n];
  }
  return 0;
}

int oracle_linear_forward_f64(double *out, const float *in, const float *w, const float *b, int B, int S, int K,
                              int N) {
  const long M = (long)B * S;
  if (M <= 0 || K <= 0 || N <= 0) return -2;
#pragma omp parallel for schedule(static) num_threads(NT())
  for (long m = 0; m < M; ++m) {
    double *acc = out + m * N;
    for (int n = 0; n < N; ++n) acc[n] = 0.0;
    for (int k = 0; k < K; ++k) {
      const double a = in[m * K + k];
      const float *wr = w + (long)k * N;
      for (int n = 0; n < N; ++n) acc[n] += a * (double)wr[n];
    }
    if (b)
      for (int n = 0; n < N; ++n) acc[n] += (double)b[n];
  }
  return 0;
}

/* ---- backward_input: g_in[m][k] = sum_n g_out[m][n] * w[k][n]   (mlp.h:463-467, 611-650)
 * The weight is walked transposed; a transposed copy keeps the ascending-n order while the
 * inner loop runs over contiguous k. */
static float *transpose_kn(const float *w, int K, int N) {
  float *wt = (float *)malloc((size_t)K * N * sizeof(float));
  if (!wt) return NULL;
#pragma omp parallel for schedule(static) num_threads(NT())
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) wt[(long)n * K + k] = w[(long)k * N + n];
  return wt;
}

int oracle_linear_backward_input_f32(float *g_in, const float *g_out, const float *w, int B, int S, int K, int N) {
  const long M = (long)B * S;
  if (M <= 0 || K <= 0 || N <= 0) return -2;
  float *wt = transpose_kn(w, K, N);
  if (!wt) return -3;
#pragma omp parallel for schedule(static) num_threads(NT())
  for (long m = 0; m < M; ++m) {
    float *acc = g_in + m * K;
    for (int k = 0; k < K; ++k) acc[k] = 0.0f;
    for (int n = 0; n < N; ++n) {
      const float g = g_out[m * N + n];
      const float *wr = wt + (long)n * K;
      for (int k = 0; k < K; ++k) acc[k] = fmaf(g, wr[k], acc[k]);
    }
  }
  free(wt);
  return 0;
}

int oracle_linear_backward_input_f64(double *g_in, const float *g_out, const float *w, int B, int S, int K,
                                     int N) {
  const long M = (long)B * S;
  if (M <= 0 || K <= 0 || N <= 0) return -2;
  float *wt = transpose_kn(w, K, N);
  if (!wt) return -3;
#pragma omp parallel for schedule(static) num_threads(NT())
  for (long m = 0; m < M; ++m) {
    double *acc = g_in + m * K;
    for (int k = 0; k < K; ++k) acc[k] = 0.0;
    for (int n = 0; n < N; ++n) {
      const double g = g_out[m * N + n];
      const float *wr = wt + (long)n * K;
      for (int k = 0; k < K; ++k) acc[k] += g * (double)wr[k];
    }
  }
  free(wt);
  return 0;
}

/* ---- backward_weight: g_w[k][n] = sum_m in[m][k] * g_out[m][n]   (mlp.h:738-742, 929-968)
 *      g_b[n] = sum_m g_out[m][n], ascending m, plain adds          (mlp.h:970-995) ---- */
int oracle_linear_backward_weight_f32(float *g_w, float *g_b, const float *g_out, const float *in, int B, int S,
                                      int K, int N) {
  const long M = (long)B * S;
  if (M <= 0 || K <= 0 || N <= 0) return -2;
#pragma omp parallel for schedule(static) num_threads(NT())
  for (int k = 0; k < K; ++k) {
    float *acc = g_w + (long)k * N;
    for (int n = 0; n < N; ++n) acc[n] = 0.0f;
    for (long m = 0; m < M; ++m) {
      const float a = in[m * K + k];
      const float *gr = g_out + m * N;
      for (int n = 0; n < N; ++n) acc[n] = fmaf(a, gr[n], acc[n]);
    }
  }
  if (g_b) {
#pragma omp parallel for schedule(static) num_threads(NT())
    for (int n = 0; n < N; ++n) {
      float s = 0.0f;
      for (long m = 0; m < M; ++m) s += g_out[m * N + n];
      g_b[n] = s;
    }
  }
  return 0;
}

int oracle_linear_backward_weight_f64(double *g_w, double *g_b, const float *g_out, const float *in, int B, int S,
                                      int K, int N) {
  const long M = (long)B * S;
  if (M <= 0 || K <= 0 || N <= 0) return -2;
#pragma omp parallel for schedule(static) num_threads(NT())
  for (int k = 0; k < K; ++k) {
    double *acc = g_w + (long)k * N;
    for (int n = 0; n < N; ++n) acc[n] = 0.0;
    for (long m = 0; m < M; ++m) {
      const double a = in[m * K + k];
      const float *gr = g_out + m * N;
      for (int n = 0; n < N; ++n) acc[n] += a * (double)gr[n];
    }
  }
  if (g_b) {
#pragma omp parallel for schedule(static) num_threads(NT())
    for (int n = 0; n < N; ++n) {
      double s = 0.0;
      for (long m = 0; m < M; ++m) s += (double)g_out[m * N + n];
      g_b[n] = s;
    }
  }
  return 0;
}

/* tanh GELU of the reference model (scripts/llm.py:22-25; src/layers/gelu.cu:20-29), used to
 * check the optional dual-store epilogue. */
void oracle_gelu_f32(float *out, const float *x, long n) {
  const float k = 0.7978845608028654f;
  for (long i = 0; i < n; ++i) {
    const float v = x[i];
    out[i] = 0.5f * v * (1.0f + tanhf(k * (v + 0.044715f * v * v * v)));
  }
}

/* Local gradient of the tanh GELU as the reference's backward kernel computes it
 * (src/layers/gelu.cu:49-63: 0.5(1+tanh u) + x/2 * sech^2(u) * s * (1 + 3*0.044715 x^2), u = s(x + 0.044715 x^3)),
 * in double, times the incoming gradient: out[i] = g[i] * gelu'(x[i]). Checks the fused GELU-backward epilogue. */
void oracle_gelu_grad_mul_f64(double *out, const float *x, const double *g, long n) {
  const double s = sqrt(2.0 / M_PI);
  for (long i = 0; i < n; ++i) {
    const double v = x[i];
    const double u = s * (v + 0.044715 * v * v * v);
    const double th = tanh(u);
    const double ch = cosh(u);
    const double sech2 = 1.0 / (ch * ch);
    out[i] = g[i] * (0.5 * (1.0 + th) + v * 0.5 * sech2 * s * (1.0 + 3.0 * 0.044715 * v * v));
  }
}
