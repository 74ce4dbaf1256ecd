// Test program for include/compat/gpt2/layers/mlp.h: calls the three linear-layer names with the
// reference's argument order (src/train.cu:356-376, 404-442 of the reference are the call sites this
// stands in for), on seeded data, and checks every output against plain double-precision loops written
// here. Prints "compat ok" and exits 0, or a diagnostic and 1. Built and run by tests/test_compat_header.py.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "gpt2/layers/mlp.h"

static float lcg(unsigned &s) {
  s = s * 1664525u + 1013904223u;
  return ((s >> 8) & 0xffff) / 65536.0f - 0.5f;
}

static double max_rel(const std::vector<float> &got, const std::vector<double> &want) {
  double num = 0, den = 0;
  for (size_t i = 0; i < got.size(); ++i) {
    num = fmax(num, fabs((double)got[i] - want[i]));
    den = fmax(den, fabs(want[i]));
  }
  return num / den;
}

int main() {
  const int B = 2, S = 75, K = 96, N = 160, M = B * S;  // ragged rows on purpose
  if (gpt2_linear_init(0) != 0) { printf("init failed\n"); return 1; }
  unsigned seed = 7;
  std::vector<float> x(M * K), w(K * N), b(N), dy(M * N);
  for (auto &v : x) v = lcg(seed);
  for (auto &v : w) v = 0.1f * lcg(seed);
  for (auto &v : b) v = 0.1f * lcg(seed);
  for (auto &v : dy) v = 0.05f * lcg(seed);
  float *dx_, *dw_, *db_, *dx, *dwt, *dbias, *dy_, *dout;
  cudaMalloc(&dx_, x.size() * 4); cudaMalloc(&dw_, w.size() * 4); cudaMalloc(&db_, b.size() * 4);
  cudaMalloc(&dy_, dy.size() * 4); cudaMalloc(&dout, dy.size() * 4); cudaMalloc(&dx, x.size() * 4);
  cudaMalloc(&dwt, w.size() * 4); cudaMalloc(&dbias, b.size() * 4);
  cudaMemcpy(dx_, x.data(), x.size() * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(dw_, w.data(), w.size() * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(db_, b.data(), b.size() * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(dy_, dy.data(), dy.size() * 4, cudaMemcpyHostToDevice);

  // the geometry macros still evaluate (the reference's scheduler counts tiles with them)
  const dim3 g = MLP_FORWARD_GRID(N, B, S);
  if (g.x != 5 || g.y != 5 || MLP_BLOCK_DIM.x != 256 || MLP_SHARED_MEM_SIZE != 16384) { printf("macros\n"); return 1; }

  int rc = 0;
  rc |= mlp_forward<TILE_SIZE>(dout, dx_, dw_, db_, B, S, K, N);
  rc |= mlp_backward_input<TILE_SIZE>(dx, dy_, dw_, B, S, K, N);
  rc |= mlp_backward_weight<TILE_SIZE>(dwt, dbias, dy_, dx_, B, S, K, N);
  if (rc != 0 || cudaDeviceSynchronize() != cudaSuccess) { printf("launch rc=%d\n", rc); return 1; }

  std::vector<float> out(M * N), gx(M * K), gw(K * N), gb(N);
  cudaMemcpy(out.data(), dout, out.size() * 4, cudaMemcpyDeviceToHost);
  cudaMemcpy(gx.data(), dx, gx.size() * 4, cudaMemcpyDeviceToHost);
  cudaMemcpy(gw.data(), dwt, gw.size() * 4, cudaMemcpyDeviceToHost);
  cudaMemcpy(gb.data(), dbias, gb.size() * 4, cudaMemcpyDeviceToHost);

  std::vector<double> t_out(M * N), t_gx(M * K), t_gw(K * N), t_gb(N);
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      double s = b[j];
      for (int k = 0; k < K; ++k) s += (double)x[i * K + k] * w[k * N + j];
      t_out[i * N + j] = s;
    }
  for (int i = 0; i < M; ++i)
    for (int k = 0; k < K; ++k) {
      double s = 0;
      for (int j = 0; j < N; ++j) s += (double)dy[i * N + j] * w[k * N + j];
      t_gx[i * K + k] = s;
    }
  for (int k = 0; k < K; ++k)
    for (int j = 0; j < N; ++j) {
      double s = 0;
      for (int i = 0; i < M; ++i) s += (double)x[i * K + k] * dy[i * N + j];
      t_gw[k * N + j] = s;
    }
  for (int j = 0; j < N; ++j) {
    double s = 0;
    for (int i = 0; i < M; ++i) s += dy[i * N + j];
    t_gb[j] = s;
  }
  const double e[4] = {max_rel(out, t_out), max_rel(gx, t_gx), max_rel(gw, t_gw), max_rel(gb, t_gb)};
  printf("errors %.3g %.3g %.3g %.3g\n", e[0], e[1], e[2], e[3]);
  for (double v : e)
    if (!(v <= 2e-5)) { printf("compat mismatch\n"); return 1; }  // 3xTF32: fp32-faithful
  gpt2_linear_shutdown();
  printf("compat ok\n");
  return 0;
}
