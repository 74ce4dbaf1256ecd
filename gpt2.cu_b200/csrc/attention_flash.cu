// Causal self-attention without the T x T tensors: one tcgen05 kernel in three modes.
//
// A CTA owns 128 rows (the 128 TMEM lanes) of one (sequence, head) and walks 64-wide column blocks:
//
//   FWD    rows = queries i, columns = keys j <= i
//          S = Q_i K_j^T -> online softmax (running max m, sum l) -> P_j -> O += P_j V_j
//          out = O / l, lse = m + log2(l) (base-2 domain, kept for the backward pass)
//   BWD_Q  rows = queries i, columns = keys j <= i
//          S = Q_i K_j^T, dP = dO_i V_j^T -> dS = P o (dP - delta) / 8 -> dQ += dS K_j
//   BWD_KV rows = keys j, columns = queries i >= j
//          S^T = K_j Q_i^T, dP^T = V_j dO_i^T -> P^T, dS^T -> dV += P^T dO_i, dK += dS^T Q_i
//
// with P = 2^(S * log2(e)/8 - lse) recomputed in the backward modes and delta = rowsum(dO o O).
// All three are "score MMAs into TMEM -> the row-work threads read their TMEM row, turn it into P / dS
// and write it back over the scores (tcgen05.st) -> accumulate MMAs that take that tile as their A
// operand straight from TMEM", so they share one skeleton; P and dS never touch shared memory, which
// saves the 32 KiB tile per step, its stores and the proxy fence they would need, and leaves the room
// for double-buffered operand stages (measured: a 128 x 64 x 8 TF32 MMA costs about 75 ns from one CTA
// wherever its A operand lives; two resident CTAs overlap to about 38 ns each): warp 0 loads operands with TMA straight out of qkv[B*T][3C] / dout[B*T][C] (batched
// tensor maps, nothing is copied or transposed), warp 1 issues the MMAs (BWD_KV: warp 1 the score MMAs,
// warp 2 the accumulate MMAs), the remaining 4 (BWD_KV: 8) warps do the row work.
// In FWD and BWD_KV score buffers rotate through three TMEM slots (the score MMAs of block t+1 run while
// the row work of block t is in progress and the accumulate MMAs of block t-1 may still be reading their
// slot) and operand stages are double-buffered. FWD and BWD_Q run two CTAs per SM (BWD_Q with one stage
// and one slot, so that it fits twice); BWD_KV, one CTA per SM, splits a step's columns between two sets
// of row-work warps and issues its MMAs from two warps.
//
// Operands are fp32 read as TF32 by the tensor core; P and dS are rounded to TF32 (to nearest) before
// they are written back, so the second contraction carries no truncation bias. The reference computes the
// same attention with one CTA per query row and materialised T x T tensors
// (src/layers/attention.cu:43-363); buffers and layouts (qkv in, atty out) are the same.
#include <cuda_runtime.h>
#include <math.h>

#include "attention_flash.cuh"
#include "layers.h"

namespace g2l {

using namespace flash;

namespace {

// one status word per device, shared by the three modes (0, or the site of a wait that gave up)
constexpr int F_MAX_DEVICES = 16;
int current_device() {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= F_MAX_DEVICES) return -1;
  return d;
}

int *flash_status_ptr() {
  static int *p[F_MAX_DEVICES] = {};
  const int d = current_device();
  if (d < 0) return nullptr;
  if (!p[d]) {
    if (cudaMalloc(&p[d], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p[d], 0, sizeof(int));
  }
  return p[d];
}

int build_maps(FlashMaps *m, const float *qkv, const float *dout, int B, int T, int C, int NH, int box_rows) {
  const float *src[4] = {qkv, qkv + C, qkv + 2 * C, dout};
  const long long ld[4] = {3LL * C, 3LL * C, 3LL * C, (long long)C};
  for (int x = 0; x < 4; ++x) {
    if (!src[x]) continue;
    int e = encode_map_batched_k(&m->k_major[x], src[x], FHS, T, ld[x], NH, FHS, B, (long long)T * ld[x], (uint32_t)box_rows);
    if (e) return e;
    e = encode_map_batched_mn(&m->mn_major[x], src[x], FHS, T, ld[x], NH, FHS, B, (long long)T * ld[x], 2);
    if (e) return e;
  }
  return GPT2L_OK;
}

template <int MODE>
int launch(const FlashMaps &maps, const FlashArgs &args, cudaStream_t st) {
  static bool attr_set_on[F_MAX_DEVICES] = {};  // the attribute is per device
  const int dev = current_device();
  if (dev < 0) return GPT2L_ERR_CUDA;
  bool &attr_set = attr_set_on[dev];
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_flash_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<MODE>::SMEM) !=
        cudaSuccess)
      return GPT2L_ERR_CUDA;
    attr_set = true;
  }
  const int grid = args.B * args.NH * (args.T / FROWS);
  attn_flash_kernel<MODE><<<grid, Cfg<MODE>::THREADS, Cfg<MODE>::SMEM, st>>>(maps, args);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? GPT2L_OK : GPT2L_ERR_CUDA;
}

}  // namespace

int attention_flash_build_maps(FlashMaps *maps, const float *qkv, const float *dout, int B, int T, int C, int NH) {
  return build_maps(maps, qkv, dout, B, T, C, NH, 64);  // every mode steps by 64 columns
}

bool attention_flash_supported(int T, int C, int NH) { return C == NH * FHS && T % FROWS == 0 && (C & 3) == 0; }

int attention_flash_status() {
  int *p = flash_status_ptr();
  int v = -1;
  if (!p || cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return v;
}

int attention_flash_forward(float *out, float *lse, const float *qkv, int B, int T, int C, int NH, cudaStream_t st) {
  if (!attention_flash_supported(T, C, NH)) return GPT2L_ERR_BAD_ARG;
  FlashMaps maps;
  int e = build_maps(&maps, qkv, nullptr, B, T, C, NH, Cfg<F_FWD>::FC);
  if (e) return e;
  FlashArgs a = {};
  a.B = B; a.T = T; a.C = C; a.NH = NH;
  a.out = out; a.lse = lse;
  a.status = flash_status_ptr();
  a.wait_limit_ns = 2000000000LL;
  if (!a.status) return GPT2L_ERR_CUDA;
  return launch<F_FWD>(maps, a, st);
}

// dqkv[B*T][3C] from dout[B*T][C]; out and lse are the forward pass's; delta is scratch of [B][NH][T]
int attention_flash_backward(float *dqkv, float *delta, const float *dout, const float *out, const float *qkv,
                             const float *lse, int B, int T, int C, int NH, cudaStream_t st) {
  if (!attention_flash_supported(T, C, NH)) return GPT2L_ERR_BAD_ARG;
  int e = attention_row_dot(delta, dout, out, B, T, C, NH, st);
  if (e) return e;
  return attention_flash_backward_core(dqkv, delta, dout, qkv, lse, B, T, C, NH, st);
}

// the two backward kernels alone: delta[b][h][t] = rowsum(dout o out) has been computed by the caller
int attention_flash_backward_core(float *dqkv, const float *delta, const float *dout, const float *qkv,
                                  const float *lse, int B, int T, int C, int NH, cudaStream_t st) {
  if (!attention_flash_supported(T, C, NH)) return GPT2L_ERR_BAD_ARG;
  FlashMaps maps, maps_kv;  // the two kernels step by different widths: different K-major boxes
  int e = build_maps(&maps, qkv, dout, B, T, C, NH, Cfg<F_BWD_Q>::FC);
  if (e) return e;
  e = build_maps(&maps_kv, qkv, dout, B, T, C, NH, Cfg<F_BWD_KV>::FC);
  if (e) return e;
  FlashArgs a = {};
  a.B = B; a.T = T; a.C = C; a.NH = NH;
  a.lse = const_cast<float *>(lse); a.delta = delta; a.dqkv = dqkv;
  a.status = flash_status_ptr();
  a.wait_limit_ns = 2000000000LL;
  if (!a.status) return GPT2L_ERR_CUDA;
  e = launch<F_BWD_KV>(maps_kv, a, st);
  if (e) return e;
  return launch<F_BWD_Q>(maps, a, st);
}

}  // namespace g2l
