// CUDA-core kernels that sit beside the tcgen05 path:
//   * a strided fp32 GEMM for shapes TMA cannot address (row strides or pointers that are not
//     16-byte multiples, e.g. the unpadded vocabulary 50257) — still GPU code, never a CPU path;
//   * a deterministic column sum (the bias gradient when a fixed summation order is asked for).
#include <cuda_runtime.h>

#include "linear_internal.h"

namespace g2l {

constexpr int ST = 64;   // output tile edge
constexpr int SK = 16;   // reduction slab
// C[i][j] = sum_k A(i,k) * B(k,j) (+ bias[j]);  A(i,k) = a[i*ai + k*ak], B(k,j) = b[k*bk + j*bj]
__global__ void __launch_bounds__(256)
gpt2_linear_simt_kernel(float *__restrict__ c, const float *__restrict__ a, const float *__restrict__ b,
                        const float *__restrict__ bias, int Mc, int Nc, int Kc, long long ai, long long ak,
                        long long bk, long long bj, long long ldc) {
  __shared__ float sa[SK][ST + 1];
  __shared__ float sb[SK][ST + 1];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int i0 = blockIdx.y * ST, j0 = blockIdx.x * ST;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < Kc; k0 += SK) {
    for (int e = threadIdx.x; e < ST * SK; e += 256) {
      const int kk = e % SK, ii = e / SK;
      const int gi = i0 + ii, gk = k0 + kk;
      sa[kk][ii] = (gi < Mc && gk < Kc) ? a[gi * ai + gk * ak] : 0.f;
      const int jj = e % ST, kb = e / ST;
      const int gj = j0 + jj, gk2 = k0 + kb;
      sb[kb][jj] = (gj < Nc && gk2 < Kc) ? b[gk2 * bk + gj * bj] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) { av[u] = sa[kk][ty * 4 + u]; bv[u] = sb[kk][tx * 4 + u]; }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int v = 0; v < 4; ++v) acc[u][v] = fmaf(av[u], bv[v], acc[u][v]);
    }
    __syncthreads();
  }
  for (int u = 0; u < 4; ++u) {
    const int gi = i0 + ty * 4 + u;
    if (gi >= Mc) continue;
    for (int v = 0; v < 4; ++v) {
      const int gj = j0 + tx * 4 + v;
      if (gj < Nc) c[gi * ldc + gj] = acc[u][v] + (bias ? bias[gj] : 0.f);
    }
  }
}

// out[j] = sum_i x[i][j], fixed order: each block owns 32 columns, 8 row lanes add strided
// rows, then a fixed tree combines them.
__global__ void __launch_bounds__(256)
gpt2_linear_colsum_kernel(float *__restrict__ out, const float *__restrict__ x, int rows, int cols) {
  __shared__ float part[8][33];
  const int cx = threadIdx.x % 32, ry = threadIdx.x / 32;
  const int j = blockIdx.x * 32 + cx;
  float s = 0.f;
  if (j < cols)
    for (int i = ry; i < rows; i += 8) s += x[(long long)i * cols + j];
  part[ry][cx] = s;
  __syncthreads();
  if (ry == 0 && j < cols) {
    float t = 0.f;
    for (int r = 0; r < 8; ++r) t += part[r][cx];
    out[j] = t;
  }
}

// dst[c][r] = src[r][c] for src[rows][cols]; 32 x 32 tiles through shared memory, both sides coalesced.
__global__ void __launch_bounds__(256)
gpt2_linear_transpose_kernel(float *__restrict__ dst, const float *__restrict__ src, int rows, int cols) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int i = ty; i < 32; i += 8) {
    const int r = r0 + i, c = c0 + tx;
    tile[i][tx] = (r < rows && c < cols) ? src[(long long)r * cols + c] : 0.f;
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    const int c = c0 + i, r = r0 + tx;
    if (c < cols && r < rows) dst[(long long)c * rows + r] = tile[tx][i];
  }
}

int launch_transpose(float *dst, const float *src, int rows, int cols, cudaStream_t stream) {
  dim3 grid((cols + 31) / 32, (rows + 31) / 32);
  gpt2_linear_transpose_kernel<<<grid, 256, 0, stream>>>(dst, src, rows, cols);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? GPT2L_OK : GPT2L_ERR_CUDA;
}

int launch_simt(const GemmDesc &d, cudaStream_t stream) {
  int Mc, Nc, Kc;
  long long ai, ak, bk, bj;
  const float *bias = nullptr;
  switch (d.kind) {
    case GPT2L_OP_FORWARD:
      Mc = d.M; Nc = d.N; Kc = d.K; ai = d.K; ak = 1; bk = d.N; bj = 1; bias = d.bias; break;
    case GPT2L_OP_BACKWARD_INPUT:
      Mc = d.M; Nc = d.K; Kc = d.N; ai = d.N; ak = 1; bk = 1; bj = d.N; break;
    case GPT2L_OP_BACKWARD_WEIGHT:
      Mc = d.K; Nc = d.N; Kc = d.M; ai = 1; ak = d.K; bk = d.N; bj = 1; break;
    default:
      return GPT2L_ERR_BAD_ARG;
  }
  dim3 grid((Nc + ST - 1) / ST, (Mc + ST - 1) / ST);
  gpt2_linear_simt_kernel<<<grid, 256, 0, stream>>>(d.out, d.a, d.b, bias, Mc, Nc, Kc, ai, ak, bk, bj, Nc);
  count_launch();
  if (cudaGetLastError() != cudaSuccess) return GPT2L_ERR_CUDA;
  if (d.kind == GPT2L_OP_BACKWARD_WEIGHT && d.out_bias) return launch_colsum(d.out_bias, d.b, d.M, d.N, stream);
  return GPT2L_OK;
}

int launch_colsum(float *out, const float *x, int rows, int cols, cudaStream_t stream) {
  gpt2_linear_colsum_kernel<<<(cols + 31) / 32, 256, 0, stream>>>(out, x, rows, cols);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? GPT2L_OK : GPT2L_ERR_CUDA;
}

}  // namespace g2l
