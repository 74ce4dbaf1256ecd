// The non-GEMM layers of the GPT-2 training step (embedding, layernorm, attention, GELU backward,
// residual, softmax + cross-entropy, AdamW), written for the model driver in model.cu. They keep the
// reference's tensor layouts (src/layers/*.cu of vnnm404/gpt2.cu: activations [B*T][C], qkv
// [B*T][3C] with q | k | v side by side, wte stored [C][V]) but not its kernels: attention is
// flash-style (no [B,NH,T,T] tensors; only the log-sum-exp per row is kept for the backward pass),
// softmax and cross-entropy are one pass that leaves dlogits in place of the logits, and layernorm
// works a row per warp. All fp32 CUDA-core code; the GEMMs around them are the tcgen05 path.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

#include "layers.h"
#include "linear_internal.h"

namespace g2l {

static inline int cdiv(long long a, int b) { return (int)((a + b - 1) / b); }

// ------------------------------------------------------------------------------------
// embedding: out[m][c] = wte[c][tok[m]] + wpe[t][c]     (reference: embedding.cu:11-27; wte is [C][V])
// ------------------------------------------------------------------------------------
__global__ void embedding_forward_kernel(float *out, const int *tokens, const float *wte, const float *wpe, int M,
                                         int T, int C, int Vp) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)M * C) return;
  const int m = (int)(i / C), c = (int)(i % C);
  const int tok = tokens[m], t = m % T;
  out[i] = wte[(long long)c * Vp + tok] + wpe[(long long)t * C + c];
}

// g_wte[c][tok] += g[m][c]; g_wpe[t][c] += g[m][c]. (The reference indexes g_wte as [V][C] here,
// embedding.cu:93, which does not match its own forward; the PyTorch model is the semantics kept.)
__global__ void embedding_backward_kernel(float *g_wte, float *g_wpe, const float *g, const int *tokens, int M, int T,
                                          int C, int Vp) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)M * C) return;
  const int m = (int)(i / C), c = (int)(i % C);
  const int tok = tokens[m], t = m % T;
  const float v = g[i];
  atomicAdd(g_wte + (long long)c * Vp + tok, v);
  atomicAdd(g_wpe + (long long)t * C + c, v);
}

// ------------------------------------------------------------------------------------
// layernorm, one warp per row (eps 1e-5 as layernorm.cu:54-116)
// ------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(256)
layernorm_forward_kernel(float *out, float *mean, float *rstd, const float *in, const float *w, const float *b,
                         int M, int C) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const float *x = in + (long long)row * C;
  float s = 0.f;
  for (int c = lane; c < C; c += 32) s += x[c];
  const float mu = warp_sum(s) / C;
  float v = 0.f;
  for (int c = lane; c < C; c += 32) { const float d = x[c] - mu; v += d * d; }
  const float rs = rsqrtf(warp_sum(v) / C + 1e-5f);
  float *o = out + (long long)row * C;
  for (int c = lane; c < C; c += 32) o[c] = (x[c] - mu) * rs * w[c] + b[c];
  if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
}

// the same with the row held in registers (K4 float4 per lane): one read of x, one write of out
template <int K4>  // C <= 128 * K4, C a multiple of 4
__global__ void __launch_bounds__(256)
layernorm_forward_vec_kernel(float *out, float *mean, float *rstd, const float *in, const float *w, const float *b,
                             int M, int C) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const float *x = in + (long long)row * C;
  float4 v[K4];
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < K4; ++k) {
    const int c = 4 * (lane + 32 * k);
    v[k] = c < C ? *reinterpret_cast<const float4 *>(x + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    s += v[k].x + v[k].y + v[k].z + v[k].w;
  }
  const float mu = warp_sum(s) / C;
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < K4; ++k) {
    const int c = 4 * (lane + 32 * k);
    if (c < C) {
      const float dx = v[k].x - mu, dy = v[k].y - mu, dz = v[k].z - mu, dw = v[k].w - mu;
      q += dx * dx + dy * dy + dz * dz + dw * dw;
    }
  }
  const float rs = rsqrtf(warp_sum(q) / C + 1e-5f);
  float *o = out + (long long)row * C;
#pragma unroll
  for (int k = 0; k < K4; ++k) {
    const int c = 4 * (lane + 32 * k);
    if (c < C) {
      const float4 wv = __ldg(reinterpret_cast<const float4 *>(w + c));
      const float4 bv = __ldg(reinterpret_cast<const float4 *>(b + c));
      *reinterpret_cast<float4 *>(o + c) =
          make_float4((v[k].x - mu) * rs * wv.x + bv.x, (v[k].y - mu) * rs * wv.y + bv.y,
                      (v[k].z - mu) * rs * wv.z + bv.z, (v[k].w - mu) * rs * wv.w + bv.w);
    }
  }
  if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
}

// g_in[row] += layernorm backward of g_out[row]; g_w / g_b accumulate over rows. A warp owns a row at a
// time and lane l always owns columns l, l+32, ...: the column sums for g_w / g_b stay in registers
// across the rows of the block and are combined once (shared memory, then one atomicAdd per column
// per block).
template <int K4>  // float4 columns per lane: C <= 128 * K4 (C is a multiple of 4)
__global__ void __launch_bounds__(256, (K4 <= 6 ? 2 : 1))
layernorm_backward_kernel(float *g_in, float *g_w, float *g_b, const float *g_out, const float *in, const float *w,
                          const float *mean, const float *rstd, int M, int C, int rows_per_block) {
  extern __shared__ float sm[];  // [2][C] column sums of this block
  float *sw = sm, *sb = sm + C;
  for (int c = threadIdx.x; c < 2 * C; c += blockDim.x) sm[c] = 0.f;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  float4 aw[K4], ab[K4];
#pragma unroll
  for (int k = 0; k < K4; ++k) {
    aw[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    ab[k] = aw[k];
  }
  const int r0 = blockIdx.x * rows_per_block;
  const int r1 = min(M, r0 + rows_per_block);
  for (int row = r0 + warp; row < r1; row += nwarps) {
    const float *x = in + (long long)row * C;
    const float *go = g_out + (long long)row * C;
    const float mu = mean[row], rs = rstd[row];
    float4 nh[K4], g[K4];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < K4; ++k) {
      const int c = 4 * (lane + 32 * k);
      const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
      const float4 xv = c < C ? *reinterpret_cast<const float4 *>(x + c) : make_float4(mu, mu, mu, mu);
      g[k] = c < C ? *reinterpret_cast<const float4 *>(go + c) : zero;
      nh[k] = make_float4((xv.x - mu) * rs, (xv.y - mu) * rs, (xv.z - mu) * rs, (xv.w - mu) * rs);
      const float4 wv = c < C ? __ldg(reinterpret_cast<const float4 *>(w + c)) : zero;
      const float4 dn = make_float4(g[k].x * wv.x, g[k].y * wv.y, g[k].z * wv.z, g[k].w * wv.w);
      s1 += dn.x + dn.y + dn.z + dn.w;
      s2 += dn.x * nh[k].x + dn.y * nh[k].y + dn.z * nh[k].z + dn.w * nh[k].w;
    }
    s1 = warp_sum(s1) / C;
    s2 = warp_sum(s2) / C;
    float *gi = g_in + (long long)row * C;
#pragma unroll
    for (int k = 0; k < K4; ++k) {
      const int c = 4 * (lane + 32 * k);
      if (c < C) {
        float4 o = *reinterpret_cast<float4 *>(gi + c);
        const float4 wv = __ldg(reinterpret_cast<const float4 *>(w + c));
        o.x += (g[k].x * wv.x - s1 - nh[k].x * s2) * rs;
        o.y += (g[k].y * wv.y - s1 - nh[k].y * s2) * rs;
        o.z += (g[k].z * wv.z - s1 - nh[k].z * s2) * rs;
        o.w += (g[k].w * wv.w - s1 - nh[k].w * s2) * rs;
        *reinterpret_cast<float4 *>(gi + c) = o;
      }
      aw[k].x += g[k].x * nh[k].x; aw[k].y += g[k].y * nh[k].y; aw[k].z += g[k].z * nh[k].z; aw[k].w += g[k].w * nh[k].w;
      ab[k].x += g[k].x; ab[k].y += g[k].y; ab[k].z += g[k].z; ab[k].w += g[k].w;
    }
  }
#pragma unroll
  for (int k = 0; k < K4; ++k) {
    const int c = 4 * (lane + 32 * k);
    if (c < C) {
      atomicAdd(sw + c, aw[k].x); atomicAdd(sw + c + 1, aw[k].y); atomicAdd(sw + c + 2, aw[k].z); atomicAdd(sw + c + 3, aw[k].w);
      atomicAdd(sb + c, ab[k].x); atomicAdd(sb + c + 1, ab[k].y); atomicAdd(sb + c + 2, ab[k].z); atomicAdd(sb + c + 3, ab[k].w);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    atomicAdd(g_w + c, sw[c]);
    atomicAdd(g_b + c, sb[c]);
  }
}

// ------------------------------------------------------------------------------------
// elementwise
// ------------------------------------------------------------------------------------
__global__ void add_kernel(float *out, const float *a, const float *b, long long n) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n) {
    const float4 x = *reinterpret_cast<const float4 *>(a + i), y = *reinterpret_cast<const float4 *>(b + i);
    *reinterpret_cast<float4 *>(out + i) = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
  } else {
    for (long long j = i; j < n; ++j) out[j] = a[j] + b[j];
  }
}

__device__ __forceinline__ float gelu_grad(float x) {
  const float k = 0.7978845608028654f;
  const float cube = 0.044715f * x * x * x;
  const float th = tanhf(k * (x + cube));
  const float sech2 = 1.f - th * th;
  return 0.5f * (1.f + th) + x * 0.5f * sech2 * k * (1.f + 3.f * 0.044715f * x * x);
}
// g[i] = g[i] * gelu'(pre[i])     (gelu.cu:49-63 computes the same derivative, accumulating)
__global__ void gelu_backward_kernel(float *g, const float *pre, long long n) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n) {
    float4 gv = *reinterpret_cast<float4 *>(g + i);
    const float4 p = *reinterpret_cast<const float4 *>(pre + i);
    gv.x *= gelu_grad(p.x); gv.y *= gelu_grad(p.y); gv.z *= gelu_grad(p.z); gv.w *= gelu_grad(p.w);
    *reinterpret_cast<float4 *>(g + i) = gv;
  } else {
    for (long long j = i; j < n; ++j) g[j] *= gelu_grad(pre[j]);
  }
}

// ------------------------------------------------------------------------------------
// softmax + cross-entropy, one block per row: loss[row] = -log softmax(logits[row])[target], and the
// logits row is overwritten with dlogits = (p - onehot) * scale (pad columns V..Vp-1 get 0).
// (reference: softmax.cu, cross_entropy.cu:24-93; scale = 1 / (B*T).)
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
softmax_xent_kernel(float *logits, float *losses, const int *targets, int V, int Vp, float scale) {
  // the row (V floats, 196 KiB for GPT-2) is read from HBM once and kept in shared memory
  extern __shared__ float srow[];
  __shared__ float red[32];
  float *row = logits + (long long)blockIdx.x * Vp;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
  float mx = -INFINITY;
  const int V4 = V & ~3;
  for (int c = tid * 4; c < V4; c += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4 *>(row + c);
    *reinterpret_cast<float4 *>(srow + c) = v;
    mx = fmaxf(fmaxf(mx, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
  }
  for (int c = V4 + tid; c < V; c += blockDim.x) { const float v = row[c]; srow[c] = v; mx = fmaxf(mx, v); }
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
  for (int i = 1; i < nw; ++i) mx = fmaxf(mx, red[i]);
  __syncthreads();
  float s = 0.f;
  for (int c = tid; c < V; c += blockDim.x) { const float e = __expf(srow[c] - mx); srow[c] = e; s += e; }
  s = warp_sum(s);
  if (lane == 0) red[warp] = s;
  __syncthreads();
  s = 0.f;
  for (int i = 0; i < nw; ++i) s += red[i];
  const int tgt = targets[blockIdx.x];
  const float inv = 1.f / s;
  if (tid == 0) losses[blockIdx.x] = -logf(srow[tgt] * inv);
  const float k = inv * scale;
  for (int c = tid * 4; c < Vp; c += blockDim.x * 4) {  // Vp is a multiple of 4
    float4 g;
    g.x = c + 0 < V ? srow[c + 0] * k - (c + 0 == tgt ? scale : 0.f) : 0.f;
    g.y = c + 1 < V ? srow[c + 1] * k - (c + 1 == tgt ? scale : 0.f) : 0.f;
    g.z = c + 2 < V ? srow[c + 2] * k - (c + 2 == tgt ? scale : 0.f) : 0.f;
    g.w = c + 3 < V ? srow[c + 3] * k - (c + 3 == tgt ? scale : 0.f) : 0.f;
    *reinterpret_cast<float4 *>(row + c) = g;
  }
}

// The same without shared-memory staging: pass 1 streams the row from HBM once and keeps a running
// (max, sum) pair per thread; pass 2 reads the row again (from L2: the rows in flight on all SMs are a few
// tens of MB) and writes dlogits. No large shared-memory footprint, so several blocks share an SM and
// the loads of one row overlap the stores of another.
__global__ void __launch_bounds__(512, 3)
softmax_xent_online_kernel(float *logits, float *losses, const int *targets, int V, int Vp, float scale) {
  __shared__ float red_m[16], red_s[16];
  float *row = logits + (long long)blockIdx.x * Vp;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float L2E = 1.4426950408889634f;
  float m = -INFINITY, s = 0.f;  // base-2 domain: m = max(x * log2e), s = sum 2^(x*log2e - m)
  const int V4 = V & ~3;
  for (int c = tid * 4; c < V4; c += 512 * 4) {
    float4 v = *reinterpret_cast<const float4 *>(row + c);
    v.x *= L2E; v.y *= L2E; v.z *= L2E; v.w *= L2E;
    const float mn = fmaxf(fmaxf(m, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
    s = s * exp2f(m - mn) + exp2f(v.x - mn) + exp2f(v.y - mn) + exp2f(v.z - mn) + exp2f(v.w - mn);
    m = mn;
  }
  for (int c = V4 + tid; c < V; c += 512) {
    const float v = row[c] * L2E;
    const float mn = fmaxf(m, v);
    s = s * exp2f(m - mn) + exp2f(v - mn);
    m = mn;
  }
  // combine (m, s) pairs: warp, then block. A thread that saw no element holds (-inf, 0); guard the
  // -inf - -inf case.
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const float mn = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * exp2f(m - mn)) + (m2 == -INFINITY ? 0.f : s2 * exp2f(m2 - mn));
    m = mn;
  }
  if (lane == 0) { red_m[warp] = m; red_s[warp] = s; }
  __syncthreads();
  m = red_m[0]; s = red_s[0];
  for (int i = 1; i < 16; ++i) {
    const float m2 = red_m[i], s2 = red_s[i];
    const float mn = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * exp2f(m - mn)) + (m2 == -INFINITY ? 0.f : s2 * exp2f(m2 - mn));
    m = mn;
  }
  const int tgt = targets[blockIdx.x];
  // loss = -(x_t - max - ln(sum)) in natural units
  if (tid == 0) losses[blockIdx.x] = -((row[tgt] * L2E - m) - log2f(s)) * 0.6931471805599453f;
  __syncthreads();  // the target logit is read before anyone overwrites it
  const float k = scale / s;
  for (int c = tid * 4; c < Vp; c += 512 * 4) {  // Vp is a multiple of 4
    float4 g = *reinterpret_cast<const float4 *>(row + c);
    g.x = c + 0 < V ? exp2f(g.x * L2E - m) * k - (c + 0 == tgt ? scale : 0.f) : 0.f;
    g.y = c + 1 < V ? exp2f(g.y * L2E - m) * k - (c + 1 == tgt ? scale : 0.f) : 0.f;
    g.z = c + 2 < V ? exp2f(g.z * L2E - m) * k - (c + 2 == tgt ? scale : 0.f) : 0.f;
    g.w = c + 3 < V ? exp2f(g.w * L2E - m) * k - (c + 3 == tgt ? scale : 0.f) : 0.f;
    *reinterpret_cast<float4 *>(row + c) = g;
  }
}

// the same in three passes over global memory, for vocabularies that do not fit in shared memory
__global__ void __launch_bounds__(512)
softmax_xent_large_kernel(float *logits, float *losses, const int *targets, int V, int Vp, float scale) {
  __shared__ float red[32];
  float *row = logits + (long long)blockIdx.x * Vp;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
  float mx = -INFINITY;
  for (int c = tid; c < V; c += blockDim.x) mx = fmaxf(mx, row[c]);
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
  for (int i = 1; i < nw; ++i) mx = fmaxf(mx, red[i]);
  __syncthreads();
  float s = 0.f;
  for (int c = tid; c < V; c += blockDim.x) s += expf(row[c] - mx);
  s = warp_sum(s);
  if (lane == 0) red[warp] = s;
  __syncthreads();
  s = 0.f;
  for (int i = 0; i < nw; ++i) s += red[i];
  const int tgt = targets[blockIdx.x];
  const float inv = 1.f / s;
  if (tid == 0) losses[blockIdx.x] = -(row[tgt] - mx - logf(s));
  __syncthreads();
  for (int c = tid; c < Vp; c += blockDim.x) {
    float g = 0.f;
    if (c < V) g = (expf(row[c] - mx) * inv - (c == tgt ? 1.f : 0.f)) * scale;
    row[c] = g;
  }
}

// ------------------------------------------------------------------------------------
// second half of the fused lm_head + softmax + cross-entropy: the GEMM epilogue left, per row and per
// column tile, (max, sum of 2^(x - max)) in the base-2 domain; a warp per row folds the `stride` pairs into
// lse[m] = max + log2(sum) and losses[m] = (lse[m] - logit[m][target] * log2 e) * ln 2.
// ------------------------------------------------------------------------------------
__global__ void xent_combine_kernel(float *lse, float *losses, const float2 *stats, int stride, const float *logits,
                                    long long ld, const int *targets, int M) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const float2 *s = stats + (size_t)row * stride;
  float m = -INFINITY, sum = 0.f;
  for (int i = lane; i < stride; i += 32) {
    const float2 v = s[i];
    const float mn = fmaxf(m, v.x);
    if (mn > -INFINITY) sum = (m == -INFINITY ? 0.f : sum * exp2f(m - mn)) + (v.x == -INFINITY ? 0.f : v.y * exp2f(v.x - mn));
    m = mn;
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, sum, o);
    const float mn = fmaxf(m, m2);
    sum = (m == -INFINITY ? 0.f : sum * exp2f(m - mn)) + (m2 == -INFINITY ? 0.f : s2 * exp2f(m2 - mn));
    m = mn;
  }
  if (lane == 0) {
    const float l2 = m + log2f(sum);
    lse[row] = l2;
    losses[row] = (l2 - logits[(long long)row * ld + targets[row]] * 1.4426950408889634f) * 0.6931471805599453f;
  }
}

// logits[m][c] <- (2^(logits[m][c] log2 e - lse[m]) - [c == target[m]]) * scale for c < V, 0 for the pad columns:
// the gradient of the mean cross-entropy, in place, one read and one write of the tensor (the row maxima and
// sums are known already, so nothing is reduced here). A block per row.
__global__ void __launch_bounds__(512)
xent_grad_inplace_kernel(float *logits, const float *lse, const int *targets, int V, int Vp, float scale) {
  float *row = logits + (long long)blockIdx.x * Vp;
  const float l2 = lse[blockIdx.x];
  const int tgt = targets[blockIdx.x];
  const float L2E = 1.4426950408889634f;
  for (int c = threadIdx.x * 4; c < Vp; c += 512 * 4) {  // Vp is a multiple of 4
    float4 g = *reinterpret_cast<const float4 *>(row + c);
    g.x = c + 0 < V ? (exp2f(g.x * L2E - l2) - (c + 0 == tgt ? 1.f : 0.f)) * scale : 0.f;
    g.y = c + 1 < V ? (exp2f(g.y * L2E - l2) - (c + 1 == tgt ? 1.f : 0.f)) * scale : 0.f;
    g.z = c + 2 < V ? (exp2f(g.z * L2E - l2) - (c + 2 == tgt ? 1.f : 0.f)) * scale : 0.f;
    g.w = c + 3 < V ? (exp2f(g.w * L2E - l2) - (c + 3 == tgt ? 1.f : 0.f)) * scale : 0.f;
    *reinterpret_cast<float4 *>(row + c) = g;
  }
}

// ------------------------------------------------------------------------------------
// causal self-attention, flash style, head size 64. qkv[m][3C] = q | k | v, head h at columns h*64.
// forward: out[m][h*64 + d], lse[b][h][t] = log sum_j exp(q_t.k_j / 8)
// One thread per query row, 128 rows per block; keys / values stream through shared memory in
// blocks of 32 and are read as broadcasts.
// ------------------------------------------------------------------------------------
constexpr int HS = 64;
constexpr int ATT_ROWS = 128;
constexpr int ATT_KB = 32;

__global__ void __launch_bounds__(ATT_ROWS)
attention_forward_kernel(float *out, float *lse, const float *qkv, int T, int C, int NH) {
  __shared__ float4 sk[ATT_KB][HS / 4];
  __shared__ float4 sv[ATT_KB][HS / 4];
  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * ATT_ROWS;
  const int t = q0 + threadIdx.x;
  const bool live = t < T;
  const float scale = 0.125f;  // 1 / sqrt(64)
  const long long base = (long long)b * T * 3 * C;
  float q[HS], acc[HS];
  if (live) {
    const float4 *qp = reinterpret_cast<const float4 *>(qkv + base + (long long)t * 3 * C + h * HS);
#pragma unroll
    for (int d = 0; d < HS / 4; ++d) {
      const float4 v = qp[d];
      q[4 * d] = v.x * scale; q[4 * d + 1] = v.y * scale; q[4 * d + 2] = v.z * scale; q[4 * d + 3] = v.w * scale;
    }
  }
#pragma unroll
  for (int d = 0; d < HS; ++d) acc[d] = 0.f;
  float m = -INFINITY, l = 0.f;
  const int kend = min(T, q0 + ATT_ROWS);  // causal: no key beyond the block's last query
  for (int k0 = 0; k0 < kend; k0 += ATT_KB) {
    __syncthreads();
    for (int i = threadIdx.x; i < ATT_KB * (HS / 4); i += ATT_ROWS) {
      const int j = i / (HS / 4), d = i % (HS / 4);
      const int kt = k0 + j;
      float4 kk = make_float4(0.f, 0.f, 0.f, 0.f), vv = kk;
      if (kt < T) {
        const float *rowp = qkv + base + (long long)kt * 3 * C + h * HS;
        kk = reinterpret_cast<const float4 *>(rowp + C)[d];
        vv = reinterpret_cast<const float4 *>(rowp + 2 * C)[d];
      }
      sk[j][d] = kk;
      sv[j][d] = vv;
    }
    __syncthreads();
    if (!live) continue;
    const int jmax = min(ATT_KB, t - k0 + 1);  // keys k0 .. t
    for (int j = 0; j < jmax; ++j) {
      float s = 0.f;
#pragma unroll
      for (int d = 0; d < HS / 4; ++d) {
        const float4 kk = sk[j][d];
        s += q[4 * d] * kk.x + q[4 * d + 1] * kk.y + q[4 * d + 2] * kk.z + q[4 * d + 3] * kk.w;
      }
      const float mn = fmaxf(m, s);
      const float corr = __expf(m - mn), p = __expf(s - mn);
      l = l * corr + p;
#pragma unroll
      for (int d = 0; d < HS / 4; ++d) {
        const float4 vv = sv[j][d];
        acc[4 * d] = acc[4 * d] * corr + p * vv.x;
        acc[4 * d + 1] = acc[4 * d + 1] * corr + p * vv.y;
        acc[4 * d + 2] = acc[4 * d + 2] * corr + p * vv.z;
        acc[4 * d + 3] = acc[4 * d + 3] * corr + p * vv.w;
      }
      m = mn;
    }
  }
  if (live) {
    const float inv = 1.f / l;
    float4 *op = reinterpret_cast<float4 *>(out + ((long long)b * T + t) * C + h * HS);
#pragma unroll
    for (int d = 0; d < HS / 4; ++d)
      op[d] = make_float4(acc[4 * d] * inv, acc[4 * d + 1] * inv, acc[4 * d + 2] * inv, acc[4 * d + 3] * inv);
    lse[((long long)b * NH + h) * T + t] = m + logf(l);
  }
}

// delta[b][h][t] = sum_d dout[m][h*64+d] * out[m][h*64+d]
__global__ void attention_delta_kernel(float *delta, const float *dout, const float *out, int T, int C, int NH,
                                       long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // over B*NH*T
  if (i >= total) return;
  const int t = (int)(i % T);
  const int h = (int)((i / T) % NH);
  const int b = (int)(i / ((long long)T * NH));
  const float4 *a = reinterpret_cast<const float4 *>(dout + ((long long)b * T + t) * C + h * HS);
  const float4 *o = reinterpret_cast<const float4 *>(out + ((long long)b * T + t) * C + h * HS);
  float s = 0.f;
#pragma unroll
  for (int d = 0; d < HS / 4; ++d) {
    const float4 x = a[d], y = o[d];
    s += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
  }
  delta[i] = s;
}

// dq: one thread per query row, streaming keys/values (same structure as the forward pass).
// dS_ij = p_ij (dO_i.V_j - delta_i), dQ_i = sum_j dS_ij K_j / 8
__global__ void __launch_bounds__(ATT_ROWS)
attention_backward_dq_kernel(float *dqkv, const float *dout, const float *qkv, const float *lse, const float *delta,
                             int T, int C, int NH) {
  __shared__ float4 sk[ATT_KB][HS / 4];
  __shared__ float4 sv[ATT_KB][HS / 4];
  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * ATT_ROWS;
  const int t = q0 + threadIdx.x;
  const bool live = t < T;
  const float scale = 0.125f;
  const long long base = (long long)b * T * 3 * C;
  float q[HS], go[HS], acc[HS];
  float L = 0.f, D = 0.f;
  if (live) {
    const float4 *qp = reinterpret_cast<const float4 *>(qkv + base + (long long)t * 3 * C + h * HS);
    const float4 *gp = reinterpret_cast<const float4 *>(dout + ((long long)b * T + t) * C + h * HS);
#pragma unroll
    for (int d = 0; d < HS / 4; ++d) {
      const float4 v = qp[d], g = gp[d];
      q[4 * d] = v.x * scale; q[4 * d + 1] = v.y * scale; q[4 * d + 2] = v.z * scale; q[4 * d + 3] = v.w * scale;
      go[4 * d] = g.x; go[4 * d + 1] = g.y; go[4 * d + 2] = g.z; go[4 * d + 3] = g.w;
    }
    L = lse[((long long)b * NH + h) * T + t];
    D = delta[((long long)b * NH + h) * T + t];
  }
#pragma unroll
  for (int d = 0; d < HS; ++d) acc[d] = 0.f;
  const int kend = min(T, q0 + ATT_ROWS);
  for (int k0 = 0; k0 < kend; k0 += ATT_KB) {
    __syncthreads();
    for (int i = threadIdx.x; i < ATT_KB * (HS / 4); i += ATT_ROWS) {
      const int j = i / (HS / 4), d = i % (HS / 4);
      const int kt = k0 + j;
      float4 kk = make_float4(0.f, 0.f, 0.f, 0.f), vv = kk;
      if (kt < T) {
        const float *rowp = qkv + base + (long long)kt * 3 * C + h * HS;
        kk = reinterpret_cast<const float4 *>(rowp + C)[d];
        vv = reinterpret_cast<const float4 *>(rowp + 2 * C)[d];
      }
      sk[j][d] = kk;
      sv[j][d] = vv;
    }
    __syncthreads();
    if (!live) continue;
    const int jmax = min(ATT_KB, t - k0 + 1);
    for (int j = 0; j < jmax; ++j) {
      float s = 0.f, dp = 0.f;
#pragma unroll
      for (int d = 0; d < HS / 4; ++d) {
        const float4 kk = sk[j][d], vv = sv[j][d];
        s += q[4 * d] * kk.x + q[4 * d + 1] * kk.y + q[4 * d + 2] * kk.z + q[4 * d + 3] * kk.w;
        dp += go[4 * d] * vv.x + go[4 * d + 1] * vv.y + go[4 * d + 2] * vv.z + go[4 * d + 3] * vv.w;
      }
      const float ds = __expf(s - L) * (dp - D) * scale;
#pragma unroll
      for (int d = 0; d < HS / 4; ++d) {
        const float4 kk = sk[j][d];
        acc[4 * d] += ds * kk.x; acc[4 * d + 1] += ds * kk.y; acc[4 * d + 2] += ds * kk.z; acc[4 * d + 3] += ds * kk.w;
      }
    }
  }
  if (live) {
    float4 *op = reinterpret_cast<float4 *>(dqkv + base + (long long)t * 3 * C + h * HS);
#pragma unroll
    for (int d = 0; d < HS / 4; ++d) op[d] = make_float4(acc[4 * d], acc[4 * d + 1], acc[4 * d + 2], acc[4 * d + 3]);
  }
}

// dk, dv: TWO threads per key row (each owns half of the head dimension, the two dot products are
// completed with one shuffle), streaming the queries at or after the key.
// dV_j = sum_i p_ij dO_i;  dK_j = sum_i dS_ij Q_i / 8
constexpr int HH = HS / 2;
__global__ void __launch_bounds__(2 * ATT_ROWS)
attention_backward_dkv_kernel(float *dqkv, const float *dout, const float *qkv, const float *lse, const float *delta,
                              int T, int C, int NH) {
  __shared__ float4 sq[ATT_KB][HS / 4];
  __shared__ float4 sg[ATT_KB][HS / 4];
  __shared__ float sl[ATT_KB], sd[ATT_KB];
  const int b = blockIdx.z, h = blockIdx.y, k0 = blockIdx.x * ATT_ROWS;
  const int j = k0 + (threadIdx.x >> 1);
  const int half = threadIdx.x & 1;  // which 32 of the 64 head columns
  const bool live = j < T;
  const float scale = 0.125f;
  const long long base = (long long)b * T * 3 * C;
  float k[HH], v[HH], dk[HH], dv[HH];
  if (live) {
    const float *rowp = qkv + base + (long long)j * 3 * C + h * HS + half * HH;
    const float4 *kp = reinterpret_cast<const float4 *>(rowp + C);
    const float4 *vp = reinterpret_cast<const float4 *>(rowp + 2 * C);
#pragma unroll
    for (int d = 0; d < HH / 4; ++d) {
      const float4 a = kp[d], c = vp[d];
      k[4 * d] = a.x; k[4 * d + 1] = a.y; k[4 * d + 2] = a.z; k[4 * d + 3] = a.w;
      v[4 * d] = c.x; v[4 * d + 1] = c.y; v[4 * d + 2] = c.z; v[4 * d + 3] = c.w;
    }
  } else {
#pragma unroll
    for (int d = 0; d < HH; ++d) { k[d] = 0.f; v[d] = 0.f; }
  }
#pragma unroll
  for (int d = 0; d < HH; ++d) { dk[d] = 0.f; dv[d] = 0.f; }
  for (int i0 = k0; i0 < T; i0 += ATT_KB) {  // queries from the block's first key on
    __syncthreads();
    for (int i = threadIdx.x; i < ATT_KB * (HS / 4); i += 2 * ATT_ROWS) {
      const int r = i / (HS / 4), d = i % (HS / 4);
      const int qt = i0 + r;
      float4 qq = make_float4(0.f, 0.f, 0.f, 0.f), gg = qq;
      if (qt < T) {
        qq = reinterpret_cast<const float4 *>(qkv + base + (long long)qt * 3 * C + h * HS)[d];
        gg = reinterpret_cast<const float4 *>(dout + ((long long)b * T + qt) * C + h * HS)[d];
      }
      sq[r][d] = qq;
      sg[r][d] = gg;
    }
    if (threadIdx.x < ATT_KB) {
      const int qt = i0 + threadIdx.x;
      sl[threadIdx.x] = qt < T ? lse[((long long)b * NH + h) * T + qt] : 0.f;
      sd[threadIdx.x] = qt < T ? delta[((long long)b * NH + h) * T + qt] : 0.f;
    }
    __syncthreads();
    // The two threads of a pair share j and therefore the trip count of this loop; other pairs of
    // the warp run a different number of iterations, so the shuffles name only the pair's two lanes.
    const unsigned pair_mask = 3u << (threadIdx.x & 30);
    const int rmin = live ? max(0, j - i0) : ATT_KB;  // queries i >= j only
    const int rmax = min(ATT_KB, T - i0);
    for (int r = rmin; r < rmax; ++r) {
      float s = 0.f, dp = 0.f;
#pragma unroll
      for (int d = 0; d < HH / 4; ++d) {
        const float4 qq = sq[r][half * (HH / 4) + d], gg = sg[r][half * (HH / 4) + d];
        s += k[4 * d] * qq.x + k[4 * d + 1] * qq.y + k[4 * d + 2] * qq.z + k[4 * d + 3] * qq.w;
        dp += v[4 * d] * gg.x + v[4 * d + 1] * gg.y + v[4 * d + 2] * gg.z + v[4 * d + 3] * gg.w;
      }
      s += __shfl_xor_sync(pair_mask, s, 1);
      dp += __shfl_xor_sync(pair_mask, dp, 1);
      const float p = __expf(s * scale - sl[r]);
      const float ds = p * (dp - sd[r]) * scale;
#pragma unroll
      for (int d = 0; d < HH / 4; ++d) {
        const float4 qq = sq[r][half * (HH / 4) + d], gg = sg[r][half * (HH / 4) + d];
        dv[4 * d] += p * gg.x; dv[4 * d + 1] += p * gg.y; dv[4 * d + 2] += p * gg.z; dv[4 * d + 3] += p * gg.w;
        dk[4 * d] += ds * qq.x; dk[4 * d + 1] += ds * qq.y; dk[4 * d + 2] += ds * qq.z; dk[4 * d + 3] += ds * qq.w;
      }
    }
  }
  if (live) {
    float *rowp = dqkv + base + (long long)j * 3 * C + h * HS + half * HH;
    float4 *kp = reinterpret_cast<float4 *>(rowp + C);
    float4 *vp = reinterpret_cast<float4 *>(rowp + 2 * C);
#pragma unroll
    for (int d = 0; d < HH / 4; ++d) {
      kp[d] = make_float4(dk[4 * d], dk[4 * d + 1], dk[4 * d + 2], dk[4 * d + 3]);
      vp[d] = make_float4(dv[4 * d], dv[4 * d + 1], dv[4 * d + 2], dv[4 * d + 3]);
    }
  }
}

// ------------------------------------------------------------------------------------
// AdamW over the flat parameter buffer; decay on every element, bias-corrected (adamw.cu:11-48)
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void adamw_one(float &p, float &m, float &v, float gi, float lr, float b1, float b2, float eps,
                                          float wd, float bc1, float bc2) {
  const float mi = b1 * m + (1.f - b1) * gi;
  const float vi = b2 * v + (1.f - b2) * gi * gi;
  m = mi;
  v = vi;
  const float mh = mi / bc1, vh = vi / bc2;
  p -= lr * (mh / (sqrtf(vh) + eps) + wd * p);
}

// `head` scalar elements bring the pointers to a 16-byte boundary, then float4 elements, then a scalar
// tail (a range of the flat buffer may start anywhere); every element sees the same arithmetic.
__global__ void adamw_kernel(float *p, float *m, float *v, const float *g, long long n, long long head, long long n4,
                             float lr, float b1, float b2, float eps, float wd, float bc1, float bc2) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n4) {
    const long long o = head + 4 * i;
    float4 pp = *reinterpret_cast<float4 *>(p + o), mm = *reinterpret_cast<float4 *>(m + o),
           vv = *reinterpret_cast<float4 *>(v + o);
    const float4 gg = *reinterpret_cast<const float4 *>(g + o);
    adamw_one(pp.x, mm.x, vv.x, gg.x, lr, b1, b2, eps, wd, bc1, bc2);
    adamw_one(pp.y, mm.y, vv.y, gg.y, lr, b1, b2, eps, wd, bc1, bc2);
    adamw_one(pp.z, mm.z, vv.z, gg.z, lr, b1, b2, eps, wd, bc1, bc2);
    adamw_one(pp.w, mm.w, vv.w, gg.w, lr, b1, b2, eps, wd, bc1, bc2);
    *reinterpret_cast<float4 *>(p + o) = pp;
    *reinterpret_cast<float4 *>(m + o) = mm;
    *reinterpret_cast<float4 *>(v + o) = vv;
  } else {
    // the few elements before and after the aligned body
    const long long j = i - n4;
    const long long tail0 = head + 4 * n4;
    const long long o = j < head ? j : tail0 + (j - head);
    if (o < n) adamw_one(p[o], m[o], v[o], g[o], lr, b1, b2, eps, wd, bc1, bc2);
  }
}

// ------------------------------------------------------------------------------------
// launchers
// ------------------------------------------------------------------------------------
#define LAUNCH_OK() (count_launch(), cudaGetLastError() == cudaSuccess ? GPT2L_OK : GPT2L_ERR_CUDA)

int embedding_forward(float *out, const int *tokens, const float *wte, const float *wpe, int B, int T, int C, int Vp,
                      cudaStream_t s) {
  const long long n = (long long)B * T * C;
  embedding_forward_kernel<<<cdiv(n, 256), 256, 0, s>>>(out, tokens, wte, wpe, B * T, T, C, Vp);
  return LAUNCH_OK();
}
int embedding_backward(float *g_wte, float *g_wpe, const float *g, const int *tokens, int B, int T, int C, int Vp,
                       cudaStream_t s) {
  const long long n = (long long)B * T * C;
  embedding_backward_kernel<<<cdiv(n, 256), 256, 0, s>>>(g_wte, g_wpe, g, tokens, B * T, T, C, Vp);
  return LAUNCH_OK();
}
int layernorm_forward(float *out, float *mean, float *rstd, const float *in, const float *w, const float *b, int M,
                      int C, cudaStream_t s) {
#define LN_FWD(K4) layernorm_forward_vec_kernel<K4><<<cdiv(M, 8), 256, 0, s>>>(out, mean, rstd, in, w, b, M, C)
  if (C & 3) layernorm_forward_kernel<<<cdiv(M, 8), 256, 0, s>>>(out, mean, rstd, in, w, b, M, C);
  else if (C <= 128) LN_FWD(1);
  else if (C <= 256) LN_FWD(2);
  else if (C <= 512) LN_FWD(4);
  else if (C <= 768) LN_FWD(6);
  else if (C <= 1024) LN_FWD(8);
  else if (C <= 1280) LN_FWD(10);
  else if (C <= 2048) LN_FWD(16);
  else layernorm_forward_kernel<<<cdiv(M, 8), 256, 0, s>>>(out, mean, rstd, in, w, b, M, C);
#undef LN_FWD
  return LAUNCH_OK();
}
int layernorm_backward(float *g_in, float *g_w, float *g_b, const float *g_out, const float *in, const float *w,
                       const float *mean, const float *rstd, int M, int C, cudaStream_t s) {
  // one block per resident slot (two per SM) where there are rows enough: every block then ends at about
  // the same time, and the column sums meet in global memory only ~300 times instead of M / 32 times
  static const int slots = [] {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
    return 2 * sms;
  }();
  int rows_per_block = cdiv(M, slots);
  if (rows_per_block < 32) rows_per_block = 32;
  const int blocks = cdiv(M, rows_per_block);
  const size_t smem = 2 * C * sizeof(float);
  if (C & 3) return GPT2L_ERR_BAD_ARG;
#define LN_BWD(K4) layernorm_backward_kernel<K4><<<blocks, 256, smem, s>>>(g_in, g_w, g_b, g_out, in, w, mean, rstd, M, C, rows_per_block)
  if (C <= 128) LN_BWD(1);
  else if (C <= 256) LN_BWD(2);
  else if (C <= 512) LN_BWD(4);
  else if (C <= 768) LN_BWD(6);
  else if (C <= 1024) LN_BWD(8);
  else if (C <= 1280) LN_BWD(10);
  else if (C <= 2048) LN_BWD(16);
  else return GPT2L_ERR_TOO_LARGE;
#undef LN_BWD
  return LAUNCH_OK();
}
int add_forward(float *out, const float *a, const float *b, long long n, cudaStream_t s) {
  add_kernel<<<cdiv((n + 3) / 4, 256), 256, 0, s>>>(out, a, b, n);
  return LAUNCH_OK();
}
int gelu_backward(float *g, const float *pre, long long n, cudaStream_t s) {
  gelu_backward_kernel<<<cdiv((n + 3) / 4, 256), 256, 0, s>>>(g, pre, n);
  return LAUNCH_OK();
}
int softmax_xent(float *logits, float *losses, const int *targets, int M, int V, int Vp, cudaStream_t s) {
  const size_t row_bytes = (size_t)V * sizeof(float);
  static const bool staged = [] { const char *e = getenv("GPT2_SOFTMAX_XENT"); return e && !strcmp(e, "staged"); }();
  if (!staged && (Vp & 3) == 0) {
    softmax_xent_online_kernel<<<M, 512, 0, s>>>(logits, losses, targets, V, Vp, 1.f / (float)M);
  } else if (row_bytes <= 220 * 1024) {
    // per device and cheap: set every time rather than tracking which devices have seen it
    if (cudaFuncSetAttribute(softmax_xent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) !=
        cudaSuccess)
      return GPT2L_ERR_CUDA;
    softmax_xent_kernel<<<M, 1024, row_bytes, s>>>(logits, losses, targets, V, Vp, 1.f / (float)M);
  } else {
    softmax_xent_large_kernel<<<M, 512, 0, s>>>(logits, losses, targets, V, Vp, 1.f / (float)M);
  }
  return LAUNCH_OK();
}
int launch_xent_combine(float *lse, float *losses, const float *stats, int stride, const float *logits, long long ld,
                        const int *targets, int M, cudaStream_t s) {
  xent_combine_kernel<<<cdiv(M, 8), 256, 0, s>>>(lse, losses, reinterpret_cast<const float2 *>(stats), stride, logits, ld,
                                                  targets, M);
  return LAUNCH_OK();
}
int xent_grad_inplace(float *logits, const float *lse, const int *targets, int M, int V, int Vp, cudaStream_t s) {
  if (Vp & 3) return GPT2L_ERR_BAD_ARG;
  xent_grad_inplace_kernel<<<M, 512, 0, s>>>(logits, lse, targets, V, Vp, 1.f / (float)M);
  return LAUNCH_OK();
}
int attention_forward(float *out, float *lse, const float *qkv, int B, int T, int C, int NH, cudaStream_t s) {
  if (C != NH * HS) return GPT2L_ERR_BAD_ARG;
  dim3 grid(cdiv(T, ATT_ROWS), NH, B);
  attention_forward_kernel<<<grid, ATT_ROWS, 0, s>>>(out, lse, qkv, T, C, NH);
  return LAUNCH_OK();
}
int attention_backward(float *dqkv, float *delta, const float *dout, const float *out, const float *qkv,
                       const float *lse, int B, int T, int C, int NH, cudaStream_t s) {
  if (C != NH * HS) return GPT2L_ERR_BAD_ARG;
  const long long total = (long long)B * NH * T;
  attention_delta_kernel<<<cdiv(total, 256), 256, 0, s>>>(delta, dout, out, T, C, NH, total);
  count_launch();
  dim3 grid(cdiv(T, ATT_ROWS), NH, B);
  attention_backward_dq_kernel<<<grid, ATT_ROWS, 0, s>>>(dqkv, dout, qkv, lse, delta, T, C, NH);
  count_launch();
  attention_backward_dkv_kernel<<<grid, 2 * ATT_ROWS, 0, s>>>(dqkv, dout, qkv, lse, delta, T, C, NH);
  return LAUNCH_OK();
}
int adamw_update(float *p, float *m, float *v, const float *g, long long n, float lr, float b1, float b2, float eps,
                 float wd, int t, cudaStream_t s) {
  const float bc1 = 1.f - powf(b1, (float)t), bc2 = 1.f - powf(b2, (float)t);
  // all four buffers are offset alike from 256-byte aligned allocations, so p decides the alignment
  long long head = (long long)((16 - (reinterpret_cast<uintptr_t>(p) & 15)) & 15) / 4;
  if (head > n) head = n;
  const long long n4 = (n - head) / 4;
  const long long extra = n - 4 * n4;  // head + tail, at most 6
  adamw_kernel<<<cdiv(n4 + extra, 256), 256, 0, s>>>(p, m, v, g, n, head, n4, lr, b1, b2, eps, wd, bc1, bc2);
  return LAUNCH_OK();
}

}  // namespace g2l
