// Causal self-attention on the tensor cores, built from the batched form of the GEMM kernel:
//
//   forward    S_bh = Q K^T         (tiles above the diagonal are skipped)
//              P    = softmax(S / 8) row-wise, causal, in place (P is kept for the backward pass)
//              O_bh = P V           (reduction stops at the tile's last row: P is lower-triangular)
//   backward   delta = rowsum(dO o O)   ( = rowsum(P o dP) )
//              dS   = P o (dO V^T - delta) / 8     (one GEMM; the softmax gradient is its epilogue;
//                                                   tiles above the diagonal skipped)
//              dQ   = dS K          (reduction stops at the diagonal)
//              dK   = dS^T Q,  dV = P^T dO    (reduction starts at the diagonal)
//
// Q, K, V are the head slices of qkv[B*T][3C] (row pitch 3C), O / dO those of [B*T][C]; nothing is
// copied or transposed: the batched tensor maps address the slices in place (two batch dimensions:
// head and sequence). This replaces the reference's one-CTA-per-query-row kernel
// (src/layers/attention.cu:43-363) and, like it, materialises the T x T probabilities.
#include <cuda_runtime.h>
#include <math.h>

#include "layers.h"
#include "linear_internal.h"

namespace g2l {

constexpr int AHS = 64;

// one warp per row (b, h, i): P[i][j] = softmax_j(S[i][j] * scale) for j <= i; zeros up to the end of
// the row's 128-column block (what the P.V and P^T.dO reductions read past the diagonal).
__global__ void __launch_bounds__(256)
attn_softmax_kernel(float *S, int T, long long rows, float scale) {
  const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const int i = (int)(r % T);
  float *row = S + r * T;
  float mx = -INFINITY;
  for (int j = lane; j <= i; j += 32) mx = fmaxf(mx, row[j]);
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int j = lane; j <= i; j += 32) sum += __expf((row[j] - mx) * scale);
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
  for (int j = lane; j <= i; j += 32) row[j] = __expf((row[j] - mx) * scale) * inv;
  const int end = min(T, (i | 127) + 1);
  for (int j = i + 1 + lane; j < end; j += 32) row[j] = 0.f;
}

// delta[b][h][i] = sum_d dO[b,i,h,d] * O[b,i,h,d]  ( = sum_j P[i][j] dP[i][j], without touching the
// T x T tensors): one warp per (b, i, h), two of the 64 head values per lane.
__global__ void __launch_bounds__(256)
attn_delta_kernel(float *delta, const float *dout, const float *out, int T, int C, int NH, long long rows) {
  const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);  // (b*T + i)*NH + h
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const int h = (int)(r % NH);
  const long long bt = r / NH;
  const float2 a = *reinterpret_cast<const float2 *>(dout + bt * C + h * AHS + 2 * lane);
  const float2 b = *reinterpret_cast<const float2 *>(out + bt * C + h * AHS + 2 * lane);
  float s = a.x * b.x + a.y * b.y;
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) delta[((bt / T) * NH + h) * T + bt % T] = s;
}

// delta[B][NH][T] = rowsum(dout o out) per head
int attention_row_dot(float *delta, const float *dout, const float *out, int B, int T, int C, int NH, cudaStream_t st) {
  const long long rows = (long long)B * NH * T;
  attn_delta_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(delta, dout, out, T, C, NH, rows);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? GPT2L_OK : GPT2L_ERR_CUDA;
}

static int run(DeviceCtx *ctx, const BatchedDesc &d, cudaStream_t st) {
  GemmOp op;
  int e = build_batched_op(d, ctx->num_sms, &op);
  if (e) return e;
  return launch_single(ctx, op, st);
}

bool attention_gemm_supported(int T, int C, int NH) { return C == NH * AHS && (T & 31) == 0; }

// out[B*T][C], P[B][NH][T][T] (kept for the backward pass)
int attention_forward_gemm(float *out, float *P, const float *qkv, int B, int T, int C, int NH, int mode,
                           cudaStream_t st) {
  int err;
  DeviceCtx *ctx = ctx_current(&err);
  if (!ctx) return err;
  if (!attention_gemm_supported(T, C, NH)) return GPT2L_ERR_BAD_ARG;
  const long long TT = (long long)T * T;
  BatchedDesc d;
  // S = Q K^T
  d.Mc = T; d.Nc = T; d.Kc = AHS; d.a_mn = 0; d.b_mn = 0;
  d.a = qkv; d.b = qkv + C; d.c = P;
  d.lda = d.ldb = 3 * C; d.ldc = T;
  d.batch_outer = B; d.batch_inner = NH;
  d.a_bs_outer = d.b_bs_outer = (long long)T * 3 * C; d.a_bs_inner = d.b_bs_inner = AHS;
  d.c_bs_outer = NH * TT; d.c_bs_inner = TT;
  d.causal = 1; d.mode = mode;
  if ((err = run(ctx, d, st))) return err;
  const long long rows = (long long)B * NH * T;
  attn_softmax_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(P, T, rows, 0.125f);
  count_launch();
  if (cudaGetLastError() != cudaSuccess) return GPT2L_ERR_CUDA;
  // O = P V
  d.Mc = T; d.Nc = AHS; d.Kc = T; d.a_mn = 0; d.b_mn = 1;
  d.a = P; d.b = qkv + 2 * C; d.c = out;
  d.lda = T; d.ldb = 3 * C; d.ldc = C;
  d.a_bs_outer = NH * TT; d.a_bs_inner = TT;
  d.b_bs_outer = (long long)T * 3 * C; d.b_bs_inner = AHS;
  d.c_bs_outer = (long long)T * C; d.c_bs_inner = AHS;
  d.causal = 2;
  return run(ctx, d, st);
}

// dqkv[B*T][3C] from dout[B*T][C]; dP is scratch of the size of P, delta scratch of [B][NH][T]; out is
// the forward result (the softmax gradient's row term comes from dout . out, so that dS is formed in
// the epilogue of the dP GEMM and never needs a pass of its own)
int attention_backward_gemm(float *dqkv, float *dP, float *delta, const float *dout, const float *out, const float *P,
                            const float *qkv, int B, int T, int C, int NH, int mode, cudaStream_t st) {
  int err;
  DeviceCtx *ctx = ctx_current(&err);
  if (!ctx) return err;
  if (!attention_gemm_supported(T, C, NH)) return GPT2L_ERR_BAD_ARG;
  const long long TT = (long long)T * T;
  const long long qs = (long long)T * 3 * C, os = (long long)T * C;
  BatchedDesc d;
  d.batch_outer = B; d.batch_inner = NH; d.mode = mode;
  if ((err = attention_row_dot(delta, dout, out, B, T, C, NH, st))) return err;
  // dS = P o (dO V^T - delta) / 8   (P is zero past the diagonal inside the diagonal tiles, so dS is too)
  d.aux = P; d.aux_row = delta; d.aux_scale = 0.125f; d.aux_op = AUX_SOFTMAX_GRAD;
  d.Mc = T; d.Nc = T; d.Kc = AHS; d.a_mn = 0; d.b_mn = 0;
  d.a = dout; d.b = qkv + 2 * C; d.c = dP;
  d.lda = C; d.ldb = 3 * C; d.ldc = T;
  d.a_bs_outer = os; d.a_bs_inner = AHS; d.b_bs_outer = qs; d.b_bs_inner = AHS;
  d.c_bs_outer = NH * TT; d.c_bs_inner = TT;
  d.causal = 1;
  if ((err = run(ctx, d, st))) return err;
  d.aux = nullptr; d.aux_row = nullptr; d.aux_op = 0;
  // dQ = dS K   (K stored [T][64], its rows are the reduction index)
  d.Mc = T; d.Nc = AHS; d.Kc = T; d.a_mn = 0; d.b_mn = 1;
  d.a = dP; d.b = qkv + C; d.c = dqkv;
  d.lda = T; d.ldb = 3 * C; d.ldc = 3 * C;
  d.a_bs_outer = NH * TT; d.a_bs_inner = TT; d.b_bs_outer = qs; d.b_bs_inner = AHS;
  d.c_bs_outer = qs; d.c_bs_inner = AHS;
  d.causal = 2;
  if ((err = run(ctx, d, st))) return err;
  // dK = dS^T Q   (A = dS read transposed: its rows are the reduction index)
  d.a_mn = 1; d.b_mn = 1;
  d.a = dP; d.b = qkv; d.c = dqkv + C;
  d.causal = 3;
  if ((err = run(ctx, d, st))) return err;
  // dV = P^T dO
  d.a = P; d.b = dout; d.c = dqkv + 2 * C;
  d.ldb = C; d.b_bs_outer = os; d.b_bs_inner = AHS;
  return run(ctx, d, st);
}

}  // namespace g2l
