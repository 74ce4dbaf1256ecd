// The row-local layers of a training step as tiles of the persistent step kernel: embedding, layernorm
// (forward / backward), softmax + cross-entropy, the attention row dot, the embedding backward scatter,
// AdamW and an activation transpose. They are the ops the reference's megakernel interprets between its
// GEMM cases (src/mk.cu:1155-1810: embedding :1157, layernorm :1167 / :1252 / :1358, softmax and
// cross-entropy :1384-1412, layernorm backward :1458 / :1623 / :1774, embedding backward :1786, AdamW :1796),
// written here for the eight worker warps (256 threads) of a GEMM CTA instead of a CTA of their own.
//
// A tile is `rows_per_tile` rows (or a chunk of the flat parameter buffer). Warps that only need their
// own rows never meet; ops whose threads share a result (a row maximum, column sums) meet through
// RowSync, an mbarrier rendezvous with the same bounded wait as every other wait of the kernel, so that
// a launch that is being aborted cannot strand a warp.
#pragma once

#include "kernel_common.cuh"

namespace g2l {

struct RowSync {
  uint32_t bar;    // shared-memory address of an mbarrier initialised with NUM_WORKER_WARPS arrivals
  uint32_t phase;  // rendezvous completed so far (every worker warp counts the same sequence)
  Ctrl *ctrl;
  // every lane of every worker warp calls this; false = the launch is being aborted
  __device__ __forceinline__ bool sync(const LaunchParams &p, int op, int lane) {
    __syncwarp();
    int okl = 1;
    if (lane == 0) {
      mbar_arrive(bar);
      okl = wait_bar(bar, phase & 1u, ctrl, p, SITE_ROW_SYNC, op, (int)phase, 20) ? 1 : 0;
    }
    ++phase;
    return __shfl_sync(0xffffffffu, okl, 0) != 0;
  }
};

__device__ __forceinline__ void prefetch_l2(const void *ptr) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr));
}

__device__ __forceinline__ float rw_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- embedding forward: thread per float4 of the tile ---------------------------------------------
__device__ __forceinline__ void row_embed_fwd(const GemmOp *op, int tile, int wtid) {
  const RowArgs &a = op->ra;
  const int M = a.i0, C = a.i1, T = a.i2, Vp = a.i4;
  const int r0 = tile * op->rows_per_tile;
  const int r1 = min(M, r0 + op->rows_per_tile);
  const int c4n = C >> 2;
  const int total = (r1 - r0) * c4n;
#pragma unroll 4
  for (int i = wtid; i < total; i += NUM_WORKER_WARPS * 32) {
    const int m = r0 + i / c4n, c = (i % c4n) * 4;
    const int tok = a.idx0[m], t = m % T;
    const float *w = a.in0 + (long long)c * Vp + tok;  // wte is [C][Vp]: four rows apart
    const float4 pe = *reinterpret_cast<const float4 *>(a.in1 + (long long)t * C + c);
    *reinterpret_cast<float4 *>(a.out0 + (long long)m * C + c) =
        make_float4(w[0] + pe.x, w[Vp] + pe.y, w[2 * (long long)Vp] + pe.z, w[3 * (long long)Vp] + pe.w);
  }
}

// ---- embedding backward: g_wte[c][tok[m]] += g[m][c], g_wpe[t][c] += g[m][c] -------------------------
__device__ __forceinline__ void row_embed_bwd(const GemmOp *op, int tile, int wtid) {
  const RowArgs &a = op->ra;
  const int M = a.i0, C = a.i1, T = a.i2, Vp = a.i4;
  const int r0 = tile * op->rows_per_tile;
  const int r1 = min(M, r0 + op->rows_per_tile);
  const int total = (r1 - r0) * C;
  for (int i = wtid; i < total; i += NUM_WORKER_WARPS * 32) {
    const int m = r0 + i / C, c = i % C;
    const int tok = a.idx0[m], t = m % T;
    const float v = a.in0[(long long)m * C + c];
    atomicAdd(a.out0 + (long long)c * Vp + tok, v);
    atomicAdd(a.out1 + (long long)t * C + c, v);
  }
}

// ---- layernorm forward: a warp takes its rows two at a time, both rows in registers, so that twice as many
// loads are in flight per warp (eight warps per SM have to cover the memory latency alone) ------------------
template <int K4>  // C <= 128 * K4, C % 4 == 0
__device__ __forceinline__ void row_ln_fwd(const GemmOp *op, int tile, int w8, int lane) {
  const RowArgs &a = op->ra;
  const int M = a.i0, C = a.i1;
  const int r0 = tile * op->rows_per_tile;
  const int r1 = min(M, r0 + op->rows_per_tile);
  constexpr int R = K4 <= 6 ? 4 : 2;  // rows in flight per warp (R * K4 float4 registers)
  for (int rowb = r0 + w8; rowb < r1; rowb += R * NUM_WORKER_WARPS) {
    float4 v[R][K4];
    float s[R];
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const int row = rowb + j * NUM_WORKER_WARPS;
      const float *x = a.in0 + (long long)row * C;
      s[j] = 0.f;
#pragma unroll
      for (int k = 0; k < K4; ++k) {
        const int c = 4 * (lane + 32 * k);
        v[j][k] = (c < C && row < r1) ? *reinterpret_cast<const float4 *>(x + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int j = 0; j < R; ++j)
#pragma unroll
      for (int k = 0; k < K4; ++k) s[j] += v[j][k].x + v[j][k].y + v[j][k].z + v[j][k].w;
    float mu[R], rs[R];
#pragma unroll
    for (int j = 0; j < R; ++j) mu[j] = rw_warp_sum(s[j]) / C;
#pragma unroll
    for (int j = 0; j < R; ++j) {
      float q = 0.f;
#pragma unroll
      for (int k = 0; k < K4; ++k) {
        const int c = 4 * (lane + 32 * k);
        if (c < C) {
          const float dx = v[j][k].x - mu[j], dy = v[j][k].y - mu[j], dz = v[j][k].z - mu[j], dw = v[j][k].w - mu[j];
          q += dx * dx + dy * dy + dz * dz + dw * dw;
        }
      }
      rs[j] = rsqrtf(rw_warp_sum(q) / C + 1e-5f);
    }
#pragma unroll
    for (int k = 0; k < K4; ++k) {
      const int c = 4 * (lane + 32 * k);
      if (c < C) {
        const float4 wv = *reinterpret_cast<const float4 *>(a.in1 + c);
        const float4 bv = *reinterpret_cast<const float4 *>(a.in2 + c);
#pragma unroll
        for (int j = 0; j < R; ++j) {
          const int row = rowb + j * NUM_WORKER_WARPS;
          if (row < r1)
            *reinterpret_cast<float4 *>(a.out0 + (long long)row * C + c) =
                make_float4((v[j][k].x - mu[j]) * rs[j] * wv.x + bv.x, (v[j][k].y - mu[j]) * rs[j] * wv.y + bv.y,
                            (v[j][k].z - mu[j]) * rs[j] * wv.z + bv.z, (v[j][k].w - mu[j]) * rs[j] * wv.w + bv.w);
        }
      }
    }
    if (lane == 0) {
#pragma unroll
      for (int j = 0; j < R; ++j) {
        const int row = rowb + j * NUM_WORKER_WARPS;
        if (row < r1) { a.out1[row] = mu[j]; a.out2[row] = rs[j]; }
      }
    }
  }
}

// ---- layernorm backward -------------------------------------------------------------------------------
// g_in[row] += backward of g_out[row]. A warp takes every eighth row of the tile and keeps the column sums
// for g_w / g_b of its rows in registers; after the tile the eight warps' sums meet in shared memory (`acc`,
// 8 x C floats per pass, plain stores) and leave the CTA as one atomicAdd per column per tile. (Shared-memory
// float atomics per row were tried first: they are compare-and-swap loops, and with 48 of them per lane and
// row a 128-row tile took 160 us.)
template <int K4>
__device__ __forceinline__ bool row_ln_bwd(const GemmOp *op, int tile, int w8, int lane, float *acc, RowSync &rs_,
                                           const LaunchParams &p) {
  const RowArgs &a = op->ra;
  const int M = a.i0, C = a.i1;
  const int wtid = w8 * 32 + lane;
  const int r0 = tile * op->rows_per_tile;
  const int r1 = min(M, r0 + op->rows_per_tile);
  float4 dw[K4], db[K4];
#pragma unroll
  for (int k = 0; k < K4; ++k) dw[k] = db[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int row = r0 + w8; row < r1; row += NUM_WORKER_WARPS) {
    float4 nh[K4], g[K4], o[K4];
    const float *x = a.in1 + (long long)row * C;
    const float *go = a.in0 + (long long)row * C;
    float *gi = a.out0 + (long long)row * C;
    const float mu = a.in3[row], rs = a.in4[row];
    // all three rows in one round trip: the residual gradient this row is added to comes with its inputs
#pragma unroll
    for (int k = 0; k < K4; ++k) {
      const int c = 4 * (lane + 32 * k);
      const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
      nh[k] = c < C ? *reinterpret_cast<const float4 *>(x + c) : zero;   // x for now
      g[k] = c < C ? *reinterpret_cast<const float4 *>(go + c) : zero;
      o[k] = c < C ? *reinterpret_cast<const float4 *>(gi + c) : zero;
    }
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < K4; ++k) {
      const int c = 4 * (lane + 32 * k);
      if (c < C) {
        const float4 xv = nh[k];
        nh[k] = make_float4((xv.x - mu) * rs, (xv.y - mu) * rs, (xv.z - mu) * rs, (xv.w - mu) * rs);
        const float4 wv = *reinterpret_cast<const float4 *>(a.in2 + c);
        const float4 dn = make_float4(g[k].x * wv.x, g[k].y * wv.y, g[k].z * wv.z, g[k].w * wv.w);
        s1 += dn.x + dn.y + dn.z + dn.w;
        s2 += dn.x * nh[k].x + dn.y * nh[k].y + dn.z * nh[k].z + dn.w * nh[k].w;
      }
    }
    s1 = rw_warp_sum(s1) / C;
    s2 = rw_warp_sum(s2) / C;
#pragma unroll
    for (int k = 0; k < K4; ++k) {
      const int c = 4 * (lane + 32 * k);
      if (c < C) {
        const float4 wv = *reinterpret_cast<const float4 *>(a.in2 + c);
        o[k].x += (g[k].x * wv.x - s1 - nh[k].x * s2) * rs;
        o[k].y += (g[k].y * wv.y - s1 - nh[k].y * s2) * rs;
        o[k].z += (g[k].z * wv.z - s1 - nh[k].z * s2) * rs;
        o[k].w += (g[k].w * wv.w - s1 - nh[k].w * s2) * rs;
        *reinterpret_cast<float4 *>(gi + c) = o[k];
        dw[k].x += g[k].x * nh[k].x; dw[k].y += g[k].y * nh[k].y; dw[k].z += g[k].z * nh[k].z; dw[k].w += g[k].w * nh[k].w;
        db[k].x += g[k].x; db[k].y += g[k].y; db[k].z += g[k].z; db[k].w += g[k].w;
      }
    }
  }
  // Two passes (weight, bias) through the 32 KiB of scratch: warp w parks its C sums at acc + slot * C, the 256
  // threads add the copies of their columns and send one atomic per column. As many warps per round as fit
  // (all eight up to C = 1024, four at 1280 and 1600).
  const int per_round = C <= 1024 ? NUM_WORKER_WARPS : (C <= 2048 ? 4 : (C <= 4096 ? 2 : 1));
  for (int pass = 0; pass < 2; ++pass) {
    float *dst = pass == 0 ? a.out1 : a.out2;
    for (int first = 0; first < NUM_WORKER_WARPS; first += per_round) {
      if (!rs_.sync(p, op->op_index, lane)) return false;  // the scratch is free (everybody has read the last round)
      if (w8 >= first && w8 < first + per_round) {
        float4 *mine = reinterpret_cast<float4 *>(acc + (size_t)(w8 - first) * C);
#pragma unroll
        for (int k = 0; k < K4; ++k) {
          const int q = lane + 32 * k;
          if (4 * q < C) mine[q] = pass == 0 ? dw[k] : db[k];
        }
      }
      if (!rs_.sync(p, op->op_index, lane)) return false;
      for (int c = wtid; c < C; c += NUM_WORKER_WARPS * 32) {
        float v = 0.f;
        for (int w = 0; w < per_round; ++w) v += acc[(size_t)w * C + c];
        atomicAdd(dst + c, v);
      }
    }
  }
  // the scratch doubles as the warps' GEMM epilogue boxes: nobody may move on to a GEMM tile before every
  // warp has read its share
  return rs_.sync(p, op->op_index, lane);
}

// ---- softmax + cross-entropy of one row by all 256 worker threads -----------------------------------
// loss[row] = -log softmax(logits[row])[target]; the row is overwritten with (p - onehot) * scale, pad
// columns V..Vp-1 with 0. Pass 1 streams the row once (running max / sum per thread), pass 2 reads it again
// (from L2: one row per CTA is in flight, ~30 MB over the whole GPU) and writes the gradient. Only 256
// threads per SM work on this, so each keeps XU independent 16-byte loads in flight before it touches the
// first value: with one load per trip the row took ~50 us, all of it memory latency.
__device__ __forceinline__ bool row_xent(const GemmOp *op, int tile, int w8, int lane, float *red, RowSync &rs_,
                                         const LaunchParams &p) {
  const RowArgs &a = op->ra;
  const int M = a.i0, V = a.i3, Vp = a.i4;
  const float scale = a.f0;
  const int wtid = w8 * 32 + lane;
  constexpr int NT = NUM_WORKER_WARPS * 32;
  const float L2E = 1.4426950408889634f;
  const int r0 = tile * op->rows_per_tile;
  const int r1 = min(M, r0 + op->rows_per_tile);
  for (int rowi = r0; rowi < r1; ++rowi) {
    float *row = a.out0 + (long long)rowi * Vp;
    float m = -INFINITY, s = 0.f;
    const int V4 = V & ~3;
    constexpr int XU = 16;
    for (int c0 = wtid * 4; c0 < V4; c0 += NT * 4 * XU) {
      float4 v[XU];
#pragma unroll
      for (int u = 0; u < XU; ++u) {
        const int c = c0 + u * NT * 4;
        v[u] = c < V4 ? *reinterpret_cast<const float4 *>(row + c) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
      float mn = m;
#pragma unroll
      for (int u = 0; u < XU; ++u) {
        v[u].x *= L2E; v[u].y *= L2E; v[u].z *= L2E; v[u].w *= L2E;
        mn = fmaxf(fmaxf(mn, fmaxf(v[u].x, v[u].y)), fmaxf(v[u].z, v[u].w));
      }
      float add = 0.f;
#pragma unroll
      for (int u = 0; u < XU; ++u) add += exp2f(v[u].x - mn) + exp2f(v[u].y - mn) + exp2f(v[u].z - mn) + exp2f(v[u].w - mn);
      s = (m == -INFINITY ? 0.f : s * exp2f(m - mn)) + add;  // c0 < V4: the first chunk is real, so mn is finite
      m = mn;
    }
    for (int c = V4 + wtid; c < V; c += NT) {
      const float v = row[c] * L2E;
      const float mn = fmaxf(m, v);
      s = s * exp2f(m - mn) + exp2f(v - mn);
      m = mn;
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      const float mn = fmaxf(m, m2);
      s = (m == -INFINITY ? 0.f : s * exp2f(m - mn)) + (m2 == -INFINITY ? 0.f : s2 * exp2f(m2 - mn));
      m = mn;
    }
    if (lane == 0) { red[w8] = m; red[8 + w8] = s; }
    const float tlogit = row[a.idx1[rowi]];  // read before anyone overwrites the row
    if (!rs_.sync(p, op->op_index, lane)) return false;
    m = red[0]; s = red[8];
#pragma unroll
    for (int i = 1; i < NUM_WORKER_WARPS; ++i) {
      const float m2 = red[i], s2 = red[8 + i];
      const float mn = fmaxf(m, m2);
      s = (m == -INFINITY ? 0.f : s * exp2f(m - mn)) + (m2 == -INFINITY ? 0.f : s2 * exp2f(m2 - mn));
      m = mn;
    }
    const int tgt = a.idx1[rowi];
    if (wtid == 0) a.out1[rowi] = -((tlogit * L2E - m) - log2f(s)) * 0.6931471805599453f;
    // `red` is rewritten by the next row only after this rendezvous; it also orders the target-logit
    // read of every thread before the first overwrite of the row
    if (!rs_.sync(p, op->op_index, lane)) return false;
    const float k = scale / s;
    for (int c0 = wtid * 4; c0 < Vp; c0 += NT * 4 * XU) {
      float4 gv[XU];
#pragma unroll
      for (int u = 0; u < XU; ++u) {
        const int c = c0 + u * NT * 4;
        gv[u] = c < Vp ? *reinterpret_cast<const float4 *>(row + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < XU; ++u) {
        const int c = c0 + u * NT * 4;
        if (c < Vp) {
          float4 g = gv[u];
          g.x = c + 0 < V ? exp2f(g.x * L2E - m) * k - (c + 0 == tgt ? scale : 0.f) : 0.f;
          g.y = c + 1 < V ? exp2f(g.y * L2E - m) * k - (c + 1 == tgt ? scale : 0.f) : 0.f;
          g.z = c + 2 < V ? exp2f(g.z * L2E - m) * k - (c + 2 == tgt ? scale : 0.f) : 0.f;
          g.w = c + 3 < V ? exp2f(g.w * L2E - m) * k - (c + 3 == tgt ? scale : 0.f) : 0.f;
          *reinterpret_cast<float4 *>(row + c) = g;
        }
      }
    }
  }
  // `red` lives in a GEMM epilogue box as well
  return rs_.sync(p, op->op_index, lane);
}

// ---- lse[m], losses[m] from the softmax statistics the lm_head epilogue left (a warp per row; see
// xent_combine_kernel in layers.cu for the stand-alone form) ----------------------------------------------
__device__ __forceinline__ void row_xent_combine(const GemmOp *op, int tile, int w8, int lane) {
  const RowArgs &a = op->ra;
  const int M = a.i0, stride = a.i1, Vp = a.i4;
  const int r0 = tile * op->rows_per_tile;
  const int r1 = min(M, r0 + op->rows_per_tile);
  for (int row = r0 + w8; row < r1; row += NUM_WORKER_WARPS) {
    const float2 *s = reinterpret_cast<const float2 *>(a.in0) + (size_t)row * stride;
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
      a.out0[row] = l2;
      a.out1[row] = (l2 - a.in1[(long long)row * Vp + a.idx1[row]] * 1.4426950408889634f) * 0.6931471805599453f;
    }
  }
}

// ---- logits[m][:] <- (softmax - onehot) * scale from the rows' log-sum-exp: elementwise, every thread keeps
// XG independent 16-byte loads in flight; no thread needs another's result ------------------------------------
__device__ __forceinline__ void row_xent_grad(const GemmOp *op, int tile, int wtid) {
  const RowArgs &a = op->ra;
  const int M = a.i0, V = a.i3, Vp = a.i4;
  const float scale = a.f0;
  constexpr int NT = NUM_WORKER_WARPS * 32, XG = 8;
  const int r0 = tile * op->rows_per_tile;
  const int r1 = min(M, r0 + op->rows_per_tile);
  for (int rowi = r0; rowi < r1; ++rowi) {
    float *row = a.out0 + (long long)rowi * Vp;
    const float l2 = a.in0[rowi];
    const int tgt = a.idx1[rowi];
    for (int c0 = wtid * 4; c0 < Vp; c0 += NT * 4 * XG) {
      float4 gv[XG];
#pragma unroll
      for (int u = 0; u < XG; ++u) {
        const int c = c0 + u * NT * 4;
        gv[u] = c < Vp ? *reinterpret_cast<const float4 *>(row + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < XG; ++u) {
        const int c = c0 + u * NT * 4;
        if (c < Vp) {
          float4 g = gv[u];
          g.x = xent_grad(g.x, l2, c, tgt, V, scale);
          g.y = xent_grad(g.y, l2, c + 1, tgt, V, scale);
          g.z = xent_grad(g.z, l2, c + 2, tgt, V, scale);
          g.w = xent_grad(g.w, l2, c + 3, tgt, V, scale);
          *reinterpret_cast<float4 *>(row + c) = g;
        }
      }
    }
  }
}

// ---- delta[b][h][t] = sum_d dout[m][h*64+d] * out[m][h*64+d]: a thread per (row, head) ----------------
__device__ __forceinline__ void row_rowdot(const GemmOp *op, int tile, int wtid) {
  const RowArgs &a = op->ra;
  const int M = a.i0, C = a.i1, T = a.i2, NH = a.i3;
  const int r0 = tile * op->rows_per_tile;
  const int r1 = min(M, r0 + op->rows_per_tile);
  const int total = (r1 - r0) * NH;
  for (int i = wtid; i < total; i += NUM_WORKER_WARPS * 32) {
    const int m = r0 + i / NH, h = i % NH;
    const float4 *x = reinterpret_cast<const float4 *>(a.in0 + (long long)m * C + h * 64);
    const float4 *y = reinterpret_cast<const float4 *>(a.in1 + (long long)m * C + h * 64);
    float s = 0.f;
#pragma unroll
    for (int d = 0; d < 16; ++d) {
      const float4 u = x[d], v = y[d];
      s += u.x * v.x + u.y * v.y + u.z * v.z + u.w * v.w;
    }
    const int b = m / T, t = m % T;
    a.out0[((long long)b * NH + h) * T + t] = s;
  }
}

// ---- AdamW over [n0 + tile * chunk, ...) of the flat buffers (src/layers/adamw.cu:11-48 of the reference:
// decay on every element, bias-corrected moments). chunk = rows_per_tile * 1024 elements. --------------
__device__ __forceinline__ void row_adamw(const GemmOp *op, int tile, int wtid, const LaunchParams &p) {
  const RowArgs &a = op->ra;
  const long long chunk = (long long)op->rows_per_tile * 1024;
  const long long lo = a.n0 + (long long)tile * chunk;
  long long hi = lo + chunk;
  const long long end = a.n0 + a.n1;
  if (hi > end) hi = end;
  const float lr = p.adam[0], b1 = p.adam[1], b2 = p.adam[2], eps = p.adam[3], wd = p.adam[4], bc1 = p.adam[5],
              bc2 = p.adam[6];
  float *P = a.out0, *Mo = a.out1, *Vo = a.out2;
  const float *G = a.in0;
  // the flat buffers are 16-byte aligned and every op range starts at a multiple of four floats
  const long long n4 = (hi - lo) >> 2;
#pragma unroll 4
  for (long long i = wtid; i < n4; i += NUM_WORKER_WARPS * 32) {
    const long long o = lo + 4 * i;
    float4 pp = *reinterpret_cast<float4 *>(P + o), mm = *reinterpret_cast<float4 *>(Mo + o),
           vv = *reinterpret_cast<float4 *>(Vo + o);
    const float4 gg = *reinterpret_cast<const float4 *>(G + o);
#define G2L_ADAM1(pc, mc, vc, gc)                                  \
    {                                                              \
      const float mi = b1 * mc + (1.f - b1) * gc;                  \
      const float vi = b2 * vc + (1.f - b2) * gc * gc;             \
      mc = mi; vc = vi;                                            \
      pc -= lr * ((mi / bc1) / (sqrtf(vi / bc2) + eps) + wd * pc); \
    }
    G2L_ADAM1(pp.x, mm.x, vv.x, gg.x) G2L_ADAM1(pp.y, mm.y, vv.y, gg.y)
    G2L_ADAM1(pp.z, mm.z, vv.z, gg.z) G2L_ADAM1(pp.w, mm.w, vv.w, gg.w)
    *reinterpret_cast<float4 *>(P + o) = pp;
    *reinterpret_cast<float4 *>(Mo + o) = mm;
    *reinterpret_cast<float4 *>(Vo + o) = vv;
  }
  for (long long o = lo + 4 * n4 + wtid; o < hi; o += NUM_WORKER_WARPS * 32) {
    float pc = P[o], mc = Mo[o], vc = Vo[o];
    const float gc = G[o];
    G2L_ADAM1(pc, mc, vc, gc)
    P[o] = pc; Mo[o] = mc; Vo[o] = vc;
  }
#undef G2L_ADAM1
}

// ---- out[c][m] = in[m][c] for the tile's rows: 32 x 32 blocks through a padded shared-memory box per warp ---
__device__ __forceinline__ void row_transpose(const GemmOp *op, int tile, int w8, int lane, float *box /* 32 x 32 */) {
  const RowArgs &a = op->ra;
  const int M = a.i0, C = a.i1;
  const int r0 = tile * op->rows_per_tile;
  const int nrb = op->rows_per_tile / 32, ncb = (C + 31) / 32;
  for (int blk = w8; blk < nrb * ncb; blk += NUM_WORKER_WARPS) {
    const int rb = blk / ncb, cb = blk % ncb;
    const int m0 = r0 + rb * 32, c0 = cb * 32;
    __syncwarp();
    float v[32];
#pragma unroll
    for (int r = 0; r < 32; ++r) {  // 32 independent loads in flight, then the box
      const int m = m0 + r, c = c0 + lane;
      v[r] = (m < M && c < C) ? a.in0[(long long)m * C + c] : 0.f;
    }
#pragma unroll
    for (int r = 0; r < 32; ++r) box[r * 32 + (lane ^ r)] = v[r];
    __syncwarp();
#pragma unroll
    for (int r = 0; r < 32; ++r) {
      const int c = c0 + r, m = m0 + lane;
      if (c < C && m < M) a.out0[(long long)c * M + m] = box[lane * 32 + (r ^ lane)];
    }
  }
}

}  // namespace g2l
