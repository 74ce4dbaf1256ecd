// Per-tile bodies shared by the GEMM kernel, the step kernel and the CTA-pair kernel: the epilogue of one
// tile by one warp, and the TF32-mode bias gradient read beside the ring.
#pragma once
#ifndef G2L_TMEM_FULL_BACKOFF
#define G2L_TMEM_FULL_BACKOFF 128
#endif

#include "kernel_common.cuh"

namespace g2l {

using namespace ptx;

// wait on a local barrier whose arrivals may come from the peer CTA (cluster-scope acquire)
__device__ __forceinline__ bool wait_bar_cluster(uint32_t bar, uint32_t parity, Ctrl *ctrl, const LaunchParams &p,
                                                 int site, int op, int idx, unsigned backoff_ns = 0) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    if (backoff_ns) __nanosleep(backoff_ns);
    if (mbar_try_wait_cluster(bar, parity)) return true;
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

// TF32-mode bias gradient of one weight-gradient tile: this tile row's share of the k-blocks
// (kb % tiles_m == m_tile) of the B operand, summed over the reduction and added into the zeroed g_b. The 128
// calling threads (x = 0..127) read the rows from global memory, not from the ring: shared-memory loads crawl
// while the tensor core and the copy engine keep the banks busy, and a stage held for them stalls a ring that
// is only four deep; the copy engine has just brought the same rows into L2.
__device__ __forceinline__ bool colsum_global_tile(const GemmOp *op, const Tile &tc, int m_tile, int x, int lane,
                                                   Ctrl *ctrl, const LaunchParams &p) {
  if (op->wait_ctr[0] >= 0) {  // step kernel: the operand's producers are done before it is read
    unsigned seen = 0u;
    int okl = 1;
    if (lane == 0) okl = wait_deps(op, m_tile, ctrl, p, seen) ? 1 : 0;
    if (__shfl_sync(0xffffffffu, okl, 0) == 0) return false;
  }
  const int bn = op->bn;
  const int g_groups = bn >> 2;          // float4 column groups of the tile: 16, 32 or 64
  const int g_parts = 128 / g_groups;    // threads that share a group, each with 32 / g_parts rows of a block
  const int g_rows = 32 / g_parts;
  const int g_grp = x % g_groups, g_part = x / g_groups;
  const int col = tc.n_tile * bn + g_grp * 4;
  if (col >= op->Nc) return true;
  float4 csum = make_float4(0.f, 0.f, 0.f, 0.f);
  const int tm = op->tiles_m;
  int kb = tc.kb0 + ((m_tile - tc.kb0 % tm) % tm + tm) % tm;
  for (; kb < tc.kb1; kb += tm) {
    const int r0 = kb * BK + g_part * g_rows;
    const float *src = op->cs_src + (long long)r0 * op->Nc + col;
#pragma unroll 8
    for (int i = 0; i < g_rows; ++i) {
      if (r0 + i < op->Kc) {
        // plain loads: in a schedule the operand may have been written earlier in the same launch
        const float4 v = *reinterpret_cast<const float4 *>(src + (long long)i * op->Nc);
        csum.x += v.x; csum.y += v.y; csum.z += v.z; csum.w += v.w;
      }
    }
  }
  // Nc is a multiple of four (TMA row pitch), so the group is inside the matrix as a whole
  atomicAdd(op->colsum + col, csum.x);
  atomicAdd(op->colsum + col + 1, csum.y);
  atomicAdd(op->colsum + col + 2, csum.z);
  atomicAdd(op->colsum + col + 3, csum.w);
  return true;
}

// Epilogue of one tile by one warp: waits for the accumulator `tcount & 1`, drains the 32-column chunks
// c_first, c_first + n_epi, ... of its TMEM lane quarter, hands the accumulator back (`arrive` arrivals: a
// warp that works without its helper twin arrives for both) and publishes the tile on the dependency
// counters (`pub` arrivals). PAIR: a CTA of a cluster of two, draining its own 128 rows (tile row `m_tile`) of a
// 256-row tile; the accumulator barriers are the leader's.
template <bool PAIR>
__device__ __forceinline__ bool epilogue_tile(const GemmOp *op, const Tile &tc, int m_tile, uint32_t tcount, bool helper,
                                              int n_epi, int c_first, unsigned arrive, unsigned pub, uint32_t sbuf,
                                              uint32_t sbuf_alt, uint32_t tmem_base, Ctrl *ctrl, const LaunchParams &p, int warp, int lane) {
  const int q = warp & 3;  // TMEM lane quarter this warp may read
  const uint32_t as = tcount & 1u;
  const uint32_t aph = (tcount >> 1) & 1u;
  int okl = 1;
  if (lane == 0)
    okl = PAIR ? wait_bar_cluster(smem_u32(&ctrl->tmem_full[as]), aph, ctrl, p, SITE_TMEM_FULL, op->op_index, as, G2L_TMEM_FULL_BACKOFF)
               : wait_bar(smem_u32(&ctrl->tmem_full[as]), aph, ctrl, p, SITE_TMEM_FULL, op->op_index, as, G2L_TMEM_FULL_BACKOFF);
  if (__shfl_sync(0xffffffffu, okl, 0) == 0) return false;
  tc_fence_after();

  const int bn = op->bn;
  const int Mc = op->Mc, Nc = op->Nc;
  const long long ldc = op->ldc;
  const int row = m_tile * BM + q * 32 + lane;
  const int n0 = tc.n_tile * bn;
  const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + as * MAX_BN;
  const bool det_split = (op->splits > 1) && !op->atomic_out;
  const bool add_bias = (op->bias != nullptr) && (tc.split == 0 || det_split);
  const bool dual = (op->flags & GPT2L_EPI_GELU_DUAL) && op->C2 != nullptr;
  const int out_tile = m_tile * op->tiles_n + tc.n_tile;
  // one CTA of a pair may hold rows below the matrix: it waits and hands back like the other, and drains nothing
  const bool live = !PAIR || m_tile < op->tiles_m;

  bool tma_used = false;
  if (live && !det_split) {
    // ---- registers -> swizzled 32x32 box in shared memory -> coalesced stores (or vector
    // reductions for split-K partials); see store_chunk
    const int row0 = m_tile * BM + q * 32;
    EpiAux ea;
    if (op->aux_op && tc.split == 0) {
      ea.aux = op->aux + tc.bb * op->c_bs_outer + tc.bh * op->c_bs_inner;
      ea.op = op->aux_op;
      ea.scale = op->aux_scale;
      if (op->aux_row) ea.row = op->aux_row + ((long long)tc.bb * op->batch_inner + tc.bh) * Mc;
    }
    const EpiAux none;
    const bool use_tma = op->epi_tma && ea.op == 0 && op->batch <= 1;
    tma_used = use_tma;
    const float drow = (ea.row && row0 + lane < Mc) ? __ldg(ea.row + row0 + lane) : 0.f;
    // softmax statistics of this thread's row over the columns this warp drains (base-2 domain)
    const bool stats = op->xent_mode == 1;
    float st_m = -INFINITY, st_s = 0.f;
    uint32_t box = 0u;
    for (int c = c_first; c < bn / 32; c += n_epi) {
      const int nb = n0 + c * 32;
      if (nb >= Nc || row0 >= Mc) break;  // warp-uniform
      AuxRegs ar;
      ar.drow = drow;
      load_aux(ar, ea, ldc, row0, nb, Mc, Nc, lane);  // in flight while the accumulator is read
      uint32_t r[32];
      tmem_ld_32x32(taddr + c * 32, r);
      tmem_ld_wait();
      float v[32];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (add_bias && nb + 4 * j < Nc) bv = __ldg(reinterpret_cast<const float4 *>(op->bias + nb) + j);
        v[4 * j + 0] = __uint_as_float(r[4 * j + 0]) + bv.x;
        v[4 * j + 1] = __uint_as_float(r[4 * j + 1]) + bv.y;
        v[4 * j + 2] = __uint_as_float(r[4 * j + 2]) + bv.z;
        v[4 * j + 3] = __uint_as_float(r[4 * j + 3]) + bv.w;
      }
      if (stats) {
        float cm = -INFINITY;
#pragma unroll
        for (int j = 0; j < 32; ++j) cm = fmaxf(cm, nb + j < op->xent_vocab ? v[j] : -INFINITY);
        if (cm > -INFINITY) {
          const float mn = fmaxf(st_m, cm * LOG2E_F);
          float add = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) add += nb + j < op->xent_vocab ? ex2_approx(fmaf(v[j], LOG2E_F, -mn)) : 0.f;
          st_s = (st_m == -INFINITY ? 0.f : st_s * ex2_approx(st_m - mn)) + add;
          st_m = mn;
        }
      }
      for (int pass = 0; pass < (dual ? 2 : 1); ++pass) {
        if (pass == 1) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
        }
        float *cbase = (pass == 0 ? op->C : op->C2) + tc.bb * op->c_bs_outer + tc.bh * op->c_bs_inner;
        // the epilogue operand applies to the first output only, and once per element: with
        // split-K reduce-adds the split that also adds the bias carries it
        // (a warp with two boxes alternates between them, so a chunk's stores are not held up by the previous
        // chunk's reads of the same box)
        const uint32_t bx = (box++ & 1u) ? sbuf_alt : sbuf;
        if (use_tma) {
          // the copy engine takes the box from here: no read-back through the load/store unit and no store
          // instructions, which is what the tensor core's own operand fetches compete with
          if (lane == 0) {  // the bulk group that read this box last is done reading
            if (sbuf_alt != sbuf) bulk_wait_read<1>();
            else bulk_wait_read<0>();
          }
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            st_shared_v4(bx + lane * 128 + ((j ^ (lane & 7)) << 4), v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const CUtensorMap *map = pass == 0 ? &op->tmC : &op->tmC2;
            if (op->atomic_out) tma_reduce_add_2d(map, bx, nb, row0);
            else tma_store_2d(map, bx, nb, row0);
            bulk_commit();
          }
        } else {
          store_chunk(v, bx, cbase, ldc, row0, nb, Mc, Nc, lane, op->atomic_out != 0, pass == 0 ? ea : none, ar);
        }
      }
    }
    if (stats && row < Mc) {
      float2 *dst = reinterpret_cast<float2 *>(op->xent_stats) + (size_t)row * op->xent_stride + 2 * tc.n_tile;
      dst[helper ? 1 : 0] = make_float2(st_m, st_s);
      if (n_epi == 1) dst[1] = make_float2(-INFINITY, 0.f);  // no helper twin in this launch / op
    }
  } else if (live && !helper) {
    // fixed-order split-K: the quarter's own warp parks its 32 rows of the partial tile in the workspace,
    // through the staging box so that the stores are whole 128-byte lines (store_chunk)
    float *ws_rows = op->ws + ((size_t)(tc.split * op->tiles_m * op->tiles_n + out_tile)) * (size_t)(BM * bn);
    const EpiAux none;
    AuxRegs ar;
    uint32_t box = 0u;
    for (int c = 0; c < bn / 32; ++c) {
      const int nb = n0 + c * 32;
      if (nb >= Nc) break;  // warp-uniform
      uint32_t r[32];
      tmem_ld_32x32(taddr + c * 32, r);
      tmem_ld_wait();
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
      store_chunk(v, (box++ & 1u) ? sbuf_alt : sbuf, ws_rows, bn, q * 32, c * 32, BM, bn, lane, false, none, ar);
    }
  }
  // the accumulator is in registers / memory now: hand the TMEM buffer back
  tc_fence_before();
  __syncwarp();
  if (lane == 0) {
    // a pair's accumulators are handed back on the leader's barrier, which counts the warps of both CTAs
    if (PAIR) mbar_arrive_cluster_cnt(mapa_cluster(smem_u32(&ctrl->tmem_empty[as]), 0), arrive);
    else mbar_arrive_cnt(smem_u32(&ctrl->tmem_empty[as]), arrive);
  }

  if (live && det_split && !helper) {
    // Deterministic split-K: every split parks its partial rows in the workspace; the
    // warp that arrives last for this (output tile, lane quarter) adds the partials in
    // split order and writes C. No ordering between splits is ever waited for.
    __threadfence();
    __syncwarp();
    unsigned old = 0;
    unsigned *sem = op->ws_sem + (size_t)out_tile * 4 + q;
    if (lane == 0) old = atom_acq_rel_add(sem, 1u);
    old = __shfl_sync(0xffffffffu, old, 0);
    if (old == (unsigned)(op->splits - 1)) {
      __threadfence();
      if (lane == 0) *sem = 0;  // ready for the next launch
      const size_t split_stride = (size_t)op->tiles_m * op->tiles_n * (size_t)(BM * bn);
      // split 0's copy of this quarter's rows; a lane owns four columns, the warp walks the rows four at a time
      // (whole lines in, whole lines out, 4 x splits loads in flight: read one row per thread, as the partials
      // are drained, this took one L2 round trip per 16 bytes and 50 - 100 us per tile)
      const float *t0 = op->ws + (size_t)out_tile * (size_t)(BM * bn) + (size_t)(q * 32) * bn;
      const int row0q = m_tile * BM + q * 32;
      for (int cb = 0; cb < bn; cb += 128) {
        const int lc = cb + lane * 4;
        const int col = n0 + lc;
        if (lc >= bn || col >= Nc) continue;  // (Nc is a multiple of four: the four columns are inside together)
        float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (add_bias) bv = __ldg(reinterpret_cast<const float4 *>(op->bias + col));
        for (int r = 0; r < 32; r += 4) {
          float4 acc[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)  // L2 reads: the partials were written by other SMs during this launch
            acc[i] = __ldcg(reinterpret_cast<const float4 *>(t0 + (size_t)(r + i) * bn + lc));
          for (int sp = 1; sp < op->splits; ++sp) {
            float4 v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
              v[i] = __ldcg(reinterpret_cast<const float4 *>(t0 + sp * split_stride + (size_t)(r + i) * bn + lc));
#pragma unroll
            for (int i = 0; i < 4; ++i) { acc[i].x += v[i].x; acc[i].y += v[i].y; acc[i].z += v[i].z; acc[i].w += v[i].w; }
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int grow = row0q + r + i;
            if (grow >= Mc) continue;
            const float4 o = make_float4(acc[i].x + bv.x, acc[i].y + bv.y, acc[i].z + bv.z, acc[i].w + bv.w);
            *reinterpret_cast<float4 *>(op->C + (long long)grow * ldc + col) = o;
            if (dual)
              *reinterpret_cast<float4 *>(op->C2 + (long long)grow * ldc + col) =
                  make_float4(gelu_tanh(o.x), gelu_tanh(o.y), gelu_tanh(o.z), gelu_tanh(o.w));
          }
        }
      }
    }
  }

  if (tma_used && lane == 0) {
    // the boxes may be rewritten (or the CTA may exit) only after the copy engine has read them; a published
    // tile must also have landed in global memory
    if (live && pub != 0u && (op->pub_rb_base >= 0 || op->pub_op_ctr >= 0)) {
      bulk_wait_all();
      fence_proxy_async_all();
    } else {
      bulk_wait_read<0>();
    }
  }
  __syncwarp();
  // ---- publish: everything this warp stored is visible before the counters move (helpers
  // publish too, so a tile counts NUM_EPI_WARPS or 2 * NUM_EPI_WARPS arrivals: epi_arrivals())
  if (live && pub != 0u && (op->pub_rb_base >= 0 || op->pub_op_ctr >= 0)) {
    __threadfence();
    __syncwarp();
    if (lane == 0) {
      if (op->pub_rb_base >= 0) red_release_add(p.counters + op->pub_rb_base + m_tile, pub);
      if (op->pub_op_ctr >= 0) red_release_add(p.counters + op->pub_op_ctr, pub);
    }
  }
  return true;
}


}  // namespace g2l
