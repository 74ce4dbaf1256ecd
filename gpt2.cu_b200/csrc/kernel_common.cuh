// Device-side helpers shared by the one-CTA and the CTA-pair GEMM kernels: the shared-memory
// control block, tile decoding, and the bounded waits.
#pragma once

#include "linear_internal.h"
#include "ptx_sm100.cuh"

namespace g2l {

using namespace ptx;

constexpr int MAX_STAGES = 6;

// ------------------------------------------------------------------------------------
// shared-memory control block
// ------------------------------------------------------------------------------------
struct Ctrl {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t ready[MAX_STAGES];
  uint64_t tmem_full[NUM_ACC];
  uint64_t tmem_empty[NUM_ACC];
  uint64_t row_bar;  // step kernel: rendezvous of the eight worker warps
  uint64_t cta_bar;  // step kernel: rendezvous of every warp of the CTA (attention tiles)
  uint32_t tmem_base;
  int abort;
};
constexpr int CTRL_MAIN_BYTES = 256;  // the attention tiles' three barrier sets follow at this offset
static_assert(sizeof(Ctrl) <= CTRL_MAIN_BYTES, "control block too large");

struct Tile {
  int m_tile, n_tile, split;
  int kb0, kb1;
  int bh, bb;  // inner / outer batch index (batched GEMMs)
  int skip;    // nothing to compute: above the causal diagonal, or an empty reduction range
};

// Advances `cursor` to the op that owns global tile `t` and decodes the tile.
// Order inside an op: splits outermost (tiles that run together share a k-range); inside a
// split the output tiles are walked in bands of `band_m` tile rows, row index fastest inside a
// band. The ~148 tiles in flight then cover band_m rows x a few columns of tiles: the A rows of
// the band stay in L2 for the whole sweep and every B column block is fetched from HBM once
// per band instead of once per tile row.
__device__ __forceinline__ const GemmOp *decode_tile(const GemmOp *ops, int n_ops, int t, int &cursor,
                                                     Tile &tc) {
  while (cursor + 1 < n_ops && t >= ops[cursor].tile_base + ops[cursor].n_tiles) ++cursor;
  const GemmOp *op = ops + cursor;
  int local = t - op->tile_base;
  tc.bh = 0;
  tc.bb = 0;
  if (op->op_kind != OPK_GEMM) {  // row-local op or attention: tiles are numbered linearly
    tc.m_tile = local;
    tc.n_tile = 0;
    tc.split = 0;
    tc.kb0 = tc.kb1 = 0;
    tc.skip = 0;
    return op;
  }
  if (op->batch > 1) {
    const int bi = local / op->tiles_per_batch;
    local -= bi * op->tiles_per_batch;
    tc.bh = bi % op->batch_inner;
    tc.bb = bi / op->batch_inner;
  }
  decode_local(local, op->tiles_dec, op->tiles_n, op->band_m, tc.m_tile, tc.n_tile, tc.split);
  tc.kb0 = tc.split * op->kb_per_split;
  int kb1 = tc.kb0 + op->kb_per_split;
  tc.kb1 = kb1 < op->kb_total ? kb1 : op->kb_total;
  tc.skip = 0;
  if (op->causal) {
    const int m0 = tc.m_tile * BM;
    if (op->causal == 1) {
      tc.skip = (tc.n_tile * op->bn >= m0 + BM) ? 1 : 0;
    } else if (op->causal == 2) {
      const int lim = (m0 + BM + BK - 1) / BK;
      if (tc.kb1 > lim) tc.kb1 = lim;
    } else {
      const int lo = m0 / BK;
      if (tc.kb0 < lo) tc.kb0 = lo;
    }
    if (tc.kb0 >= tc.kb1) tc.skip = 1;
  }
  return op;
}

static __device__ __noinline__ void raise_timeout(Ctrl *ctrl, const LaunchParams &p, int site, int op, int idx,
                                           int seen, int expected) {
  *reinterpret_cast<volatile int *>(&ctrl->abort) = 1;
  if (atomicCAS(&p.status->status, 0, GPT2L_DEV_TIMEOUT) == 0) {
    p.status->op = op;
    p.status->counter = idx;
    p.status->seen = seen;
    p.status->expected = expected;
    p.status->where = site;
    __threadfence();
    if (p.sticky && atomicCAS(&p.sticky->status, 0, GPT2L_DEV_TIMEOUT) == 0) {
      p.sticky->op = op;
      p.sticky->counter = idx;
      p.sticky->seen = seen;
      p.sticky->expected = expected;
      p.sticky->where = site;
      __threadfence();
    }
    if (p.host_flag) {
      *reinterpret_cast<volatile int *>(p.host_flag) = GPT2L_DEV_TIMEOUT;
      __threadfence_system();
    }
  }
}

// true = the phase completed; false = abort (ours or another CTA's) or the limit ran out.
// `backoff_ns` > 0 parks the polling lane between probes (waits that last microseconds and are not
// on the critical path: epilogue, producer), so that spinning does not eat the issue slots the
// MMA and epilogue warps need.
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, Ctrl *ctrl, const LaunchParams &p,
                                         int site, int op, int idx, unsigned backoff_ns = 0) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    if (backoff_ns) __nanosleep(backoff_ns);
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 127u) == 0) {
      if (*reinterpret_cast<volatile int *>(&ctrl->abort)) return false;
      if (*reinterpret_cast<volatile int *>(&p.status->status) != 0) {
        *reinterpret_cast<volatile int *>(&ctrl->abort) = 1;
        return false;
      }
      if (globaltimer_ns() - t0 > p.wait_limit_ns) {
        raise_timeout(ctrl, p, site, op, idx, -1, (int)parity);
        return false;
      }
    }
  }
}

// Bounded acquire-poll on a dependency counter.
__device__ __forceinline__ bool wait_counter(const unsigned *ctr, unsigned expected, Ctrl *ctrl,
                                             const LaunchParams &p, int op, int idx) {
  unsigned v = ld_acquire(ctr);
  if (v >= expected) return true;
  const long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    __nanosleep(64);
    v = ld_acquire(ctr);
    if (v >= expected) return true;
    if ((++spins & 15u) == 0) {
      if (*reinterpret_cast<volatile int *>(&ctrl->abort)) return false;
      if (*reinterpret_cast<volatile int *>(&p.status->status) != 0) {
        *reinterpret_cast<volatile int *>(&ctrl->abort) = 1;
        return false;
      }
      if (globaltimer_ns() - t0 > p.wait_limit_ns) {
        raise_timeout(ctrl, p, SITE_DEP_COUNTER, op, idx, (int)v, (int)expected);
        return false;
      }
    }
  }
}

// Every dependency of a tile at once (one lane calls this): the counters are probed with independent
// relaxed loads, so a tile whose producers are done pays one round trip to L2 however many
// dependencies it has, and one acquire fence orders the tile's reads behind them. Only a counter that
// is still short is polled (bounded). `rb` is the consumer's 128-row block. `done` remembers, per role and
// op, which producers have been seen complete as a whole (bit w = dependency w): those are skipped from then
// on, so the tiles of a long op stop paying for dependencies that were settled during its first wave.
__device__ __forceinline__ bool wait_deps(const GemmOp *op, int rb, Ctrl *ctrl, const LaunchParams &p, unsigned &done) {
  bool all = true, looked = false;
  unsigned newly = 0u;
#pragma unroll
  for (int w = 0; w < MAX_WAITS; ++w) {
    const int base = op->wait_ctr[w];
    if (base < 0 || ((done >> w) & 1u)) continue;
    looked = true;
    const unsigned need = (unsigned)op->wait_expected[w];
    const bool whole = ld_relaxed(p.counters + op->wait_op_ctr[w]) >= (unsigned)op->wait_op_expected[w];
    bool ok;
    if (op->wait_kind[w] == DEP_SEQUENCE) {
      const int n = op->rb_per_seq, first = base + (rb / n) * n;
      ok = true;
      for (int i = 0; i < n; ++i) ok &= ld_relaxed(p.counters + first + i) >= need;
    } else {
      ok = ld_relaxed(p.counters + base + (op->wait_kind[w] == GPT2L_DEP_ROWBLOCK ? rb : 0)) >= need;
    }
    if (whole) newly |= 1u << w;
    all &= (ok || whole);
  }
  if (!looked) return true;
  if (!all) {
    for (int w = 0; w < MAX_WAITS; ++w) {
      const int base = op->wait_ctr[w];
      if (base < 0 || (((done | newly) >> w) & 1u)) continue;
      const unsigned need = (unsigned)op->wait_expected[w];
      if (op->wait_kind[w] == DEP_SEQUENCE) {
        const int n = op->rb_per_seq, first = base + (rb / n) * n;
        for (int i = 0; i < n; ++i)
          if (!wait_counter(p.counters + first + i, need, ctrl, p, op->op_index, first + i)) return false;
      } else {
        const int idx = base + (op->wait_kind[w] == GPT2L_DEP_ROWBLOCK ? rb : 0);
        if (!wait_counter(p.counters + idx, need, ctrl, p, op->op_index, idx)) return false;
      }
    }
  }
  fence_acq_rel_gpu();
  done |= newly;
  return true;
}

// tanh(u) = 1 - 2 / (1 + e^{2u}) on the special-function unit (ex2.approx, rcp.approx): absolute error
// about 2e-7, which is what GELU needs (it uses 1 + tanh and 1 - tanh^2, never tanh alone); tanhf
// costs several times as many instructions, and the epilogue warps evaluate 32K of these per tile.
__device__ __forceinline__ float tanh_sfu(float u) { return 1.f - __fdividef(2.f, 1.f + __expf(2.f * u)); }

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k = 0.7978845608028654f;  // sqrt(2/pi)
  float u = k * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanh_sfu(u));
}

__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float k = 0.7978845608028654f;
  const float th = tanh_sfu(k * (x + 0.044715f * x * x * x));
  return 0.5f * (1.f + th) + x * 0.5f * (1.f - th * th) * k * (1.f + 3.f * 0.044715f * x * x);
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr float LOG2E_F = 1.4426950408889634f;

// dlogit of one element: logits -> (softmax - onehot) * scale, columns at or past the true vocabulary -> 0
__device__ __forceinline__ float xent_grad(float logit, float lse2, int col, int tgt, int vocab, float scale) {
  const float p = ex2_approx(fmaf(logit, LOG2E_F, -lse2));
  return col < vocab ? (p - (col == tgt ? 1.f : 0.f)) * scale : 0.f;
}

__device__ __forceinline__ float tf32_round(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}



// Epilogue store of one 32-row x 32-column chunk held as "thread = row, 32 consecutive columns"
// (the tcgen05.ld 32x32b layout). Written straight from registers each thread would touch 32
// different 128-byte lines per instruction; instead the chunk goes through a swizzled 4 KiB box in
// shared memory and comes back as "instruction = 4 rows x 128 bytes", so that every global store (or
// split-K reduction) instruction covers four whole lines. Only the warp's own lanes are involved:
// __syncwarp is the only synchronisation, and no asynchronous-proxy fence is needed.
// The epilogue operand `e.aux` (same indexing as C) is read in the coalesced phase, so it costs one
// more fully coalesced 16-byte load per lane: GPT2L_AUX_ADD adds it, GPT2L_AUX_GELU_GRAD multiplies by
// gelu'(aux), AUX_SOFTMAX_GRAD computes aux * (acc - e.row[r]) * e.scale.
struct EpiAux {
  const float *aux = nullptr;
  const float *row = nullptr;  // one value per output row (AUX_SOFTMAX_GRAD)
  float scale = 1.f;
  int op = 0;
};

// The operand values a chunk needs, fetched ahead of the accumulator read so that their latency
// overlaps it (issued inside the store loop they would serialise behind each store).
struct AuxRegs {
  float4 a[8];
  float drow = 0.f;  // AUX_SOFTMAX_GRAD: lane l holds the row term of row l of the warp's 32 rows
};

__device__ __forceinline__ void load_aux(AuxRegs &r, const EpiAux &e, long long ldc, int row0, int nb, int Mc, int Nc,
                                         int lane) {
  if (!e.op) return;
  const int rr = lane >> 3, cc = lane & 7;
  const int col = nb + cc * 4;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int grow = row0 + 4 * i + rr;
    r.a[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    // a plain load: inside a schedule the operand may have been written earlier in the same launch
    if (grow < Mc && col < Nc) r.a[i] = *reinterpret_cast<const float4 *>(e.aux + (long long)grow * ldc + col);
  }
}

__device__ __forceinline__ void store_chunk(const float (&v)[32], uint32_t sbuf, float *C, long long ldc,
                                            int row0, int nb, int Mc, int Nc, int lane, bool atomic,
                                            const EpiAux &e, const AuxRegs &r) {
  __syncwarp();  // the previous chunk's reads of this box are done
#pragma unroll
  for (int j = 0; j < 8; ++j)
    st_shared_v4(sbuf + lane * 128 + ((j ^ (lane & 7)) << 4), v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  __syncwarp();
  const int rr = lane >> 3, cc = lane & 7;
  const int col = nb + cc * 4;
  float4 x[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rl = 4 * i + rr;
    x[i] = ld_shared_v4(sbuf + rl * 128 + ((cc ^ (rl & 7)) << 4));
  }
  if (e.op == GPT2L_AUX_ADD) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      x[i].x += r.a[i].x; x[i].y += r.a[i].y; x[i].z += r.a[i].z; x[i].w += r.a[i].w;
    }
  } else if (e.op == GPT2L_AUX_GELU_GRAD) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      x[i].x *= gelu_tanh_grad(r.a[i].x); x[i].y *= gelu_tanh_grad(r.a[i].y);
      x[i].z *= gelu_tanh_grad(r.a[i].z); x[i].w *= gelu_tanh_grad(r.a[i].w);
    }
  } else if (e.op != 0) {  // AUX_SOFTMAX_GRAD
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float d = __shfl_sync(0xffffffffu, r.drow, 4 * i + rr);
      x[i].x = r.a[i].x * (x[i].x - d) * e.scale; x[i].y = r.a[i].y * (x[i].y - d) * e.scale;
      x[i].z = r.a[i].z * (x[i].z - d) * e.scale; x[i].w = r.a[i].w * (x[i].w - d) * e.scale;
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int grow = row0 + 4 * i + rr;
    if (grow < Mc && col < Nc) {
      float *dst = C + (long long)grow * ldc + col;
      if (atomic) red_add_v4(dst, x[i].x, x[i].y, x[i].z, x[i].w);
      else *reinterpret_cast<float4 *>(dst) = x[i];
    }
  }
}

}  // namespace g2l
