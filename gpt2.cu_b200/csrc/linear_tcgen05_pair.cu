// The CTA-pair variant of the GEMM kernel: a cluster of two CTAs computes one 256 x bn tile with
// tcgen05.mma.cta_group::2.
//
// Why: in a pair each CTA stages its own 128 rows of A and only HALF of B (bn/2 columns), 32 KiB per
// k-block instead of 48 KiB for the same 2.1 MFLOP per CTA; the tensor cores of both SMs read both halves
// of B through the pair's shared memory. Operand traffic per flop drops by a third, the ring is six
// stages deep instead of four, and the epilogue that runs beside the main loop disturbs it less. That
// pays on the vocabulary-wide GEMMs; short tiles lose more to the cluster's hand-shakes than they gain.
//
// Protocol (rank 0 = leader, the only CTA that issues MMAs):
//   * no load is multicast: CTA r loads A rows [256*mp + 128*r, +128) and B columns [n0 + r*bn/2, +bn/2)
//     into its own ring;
//   * TF32 mode: the loads of BOTH CTAs are issued in the .cta_group::2 form and complete on ONE barrier,
//     the leader's full[s], which the leader arms for the bytes of both (the peer's bytes may land first:
//     the transaction count may run negative inside a phase, which cannot complete before the leader's
//     arrival). The leader issues a k-block when that barrier flips;
//   * 3xTF32 mode: each CTA's loads complete on its own full[s]; the transform warps of both CTAs split
//     their stage into hi + lo and arrive on the leader's ready[s] (eight arrivals), which the leader
//     waits for instead;
//   * tcgen05.commit (cta_group::2) then arrives on empty[s] of BOTH CTAs (two commits, one per
//     CTA, each to a plain cluster address) and, after the last k-block, on tmem_full[acc] of both;
//   * each CTA's epilogue drains its own 128 x bn accumulator and arrives on the LEADER's
//     tmem_empty[acc] (eight arrivals free the accumulator pair);
//   * tensor memory is allocated and freed with the cta_group::2 forms by warp 1 of both CTAs;
//     a cluster barrier after barrier initialisation and one before the free keep the two CTAs
//     from touching each other's barriers or memory outside that window.
// All waits are bounded exactly as in the one-CTA kernel.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "kernel_common.cuh"
#include "epilogue.cuh"

namespace g2l {

using namespace ptx;

constexpr int P_B_TILE_BYTES = (MAX_BN / 2) * BK * 4;             // 16 KiB: half of B per CTA
constexpr int P_STAGE_BYTES = A_TILE_BYTES + P_B_TILE_BYTES;      // 32 KiB
constexpr int P_STAGES_1X = RING_BYTES / P_STAGE_BYTES;           // 6
constexpr int P_STAGES_3X = RING_BYTES / (2 * P_STAGE_BYTES);     // 3
static_assert(P_STAGES_1X <= MAX_STAGES, "control block too small");

template <bool X3>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gpt2_linear_tcgen05_pair_kernel(const __grid_constant__ GemmOp op0, const LaunchParams p) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int NST = X3 ? P_STAGES_3X : P_STAGES_1X;
  constexpr int STAGE_STRIDE = X3 ? 2 * P_STAGE_BYTES : P_STAGE_BYTES;
  constexpr int LO_OFFSET = P_STAGE_BYTES;

  const GemmOp *ops = p.ops ? p.ops : &op0;
  const int n_ops = p.ops ? p.n_ops : 1;

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t ring = (raw + 1023u) & ~1023u;
  uint8_t *ring_ptr = smem_raw + (ring - raw);
  Ctrl *ctrl = reinterpret_cast<Ctrl *>(ring_ptr + RING_BYTES + EPI_BYTES);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t rank = cluster_ctarank();       // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;
  const bool xform = X3 && p.xform_active != 0;  // the transform warps only work in 3xTF32 mode
  // TF32 launches: no warp looks at its own CTA's ring (the transform warps only work in 3xTF32 mode), so the
  // loads of both CTAs complete directly on the leader's full[s]
  const bool direct = !X3;

  if (tid == 0) {
    for (int s = 0; s < MAX_STAGES; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1 + (xform ? NUM_XFORM_WARPS : 0));
      // leader only, 3xTF32 mode: the transform warps of both CTAs
      mbar_init(smem_u32(&ctrl->ready[s]), 2 * NUM_XFORM_WARPS);
    }
    for (int a = 0; a < NUM_ACC; ++a) {
      mbar_init(smem_u32(&ctrl->tmem_full[a]), 1);
      mbar_init(smem_u32(&ctrl->tmem_empty[a]), 2 * NUM_EPI_WARPS);  // leader only: both epilogues
    }
    ctrl->abort = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&ctrl->tmem_base), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anyone arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(&ctrl->tmem_base);

  if (warp == 0) {
    // =============================== TMA producer (both CTAs) ===============================
    int cursor = 0;
    uint32_t it = 0;
    bool ok = true;
    for (int t = pair_id; t < p.total_tiles && ok; t += n_pairs) {
      Tile tc;
      const GemmOp *op = decode_tile(ops, n_ops, t, cursor, tc);
      const int m_tile = 2 * tc.m_tile + (int)rank;  // this CTA's 128-row block
      bool waited = false;
#pragma unroll
      for (int w = 0; w < MAX_WAITS; ++w) {
        const int base = op->wait_ctr[w];
        if (base < 0) continue;
        const bool rowblock = op->wait_kind[w] == GPT2L_DEP_ROWBLOCK;
        // a row-block dependency guards this CTA's A rows; if those lie outside the matrix there
        // is nothing to wait for (its half of B is still loaded, and whole-op waits still apply)
        if (rowblock && m_tile >= op->tiles_m) continue;
        const int idx = base + (rowblock ? m_tile : 0);
        int okl = 1;
        if (lane == 0)
          okl = wait_counter(p.counters + idx, (unsigned)op->wait_expected[w], ctrl, p, op->op_index, idx);
        ok = __shfl_sync(0xffffffffu, okl, 0) != 0;
        waited = true;
        if (!ok) break;
      }
      if (!ok) break;
      if (waited) fence_proxy_async_all();

      const int bh = op->bn >> 1;  // B columns this CTA stages
      const int m0 = m_tile * BM;
      const int n0 = tc.n_tile * op->bn + (int)rank * bh;
      const int a_mn = op->a_mn, b_mn = op->b_mn;
      const uint32_t tx_bytes = (uint32_t)(A_TILE_BYTES + bh * BK * 4);
      for (int kb = tc.kb0; kb < tc.kb1; ++kb, ++it) {
        const int s = it % NST;
        const uint32_t ph = (it / NST) & 1u;
        int okl = 1;
        if (lane == 0)
          okl = wait_bar(smem_u32(&ctrl->empty[s]), ph ^ 1u, ctrl, p, SITE_SMEM_EMPTY, op->op_index, s, 32);
        ok = __shfl_sync(0xffffffffu, okl, 0) != 0;
        if (!ok) break;
        if (lane == 0) {
          const uint32_t a_dst = ring + s * STAGE_STRIDE;
          const uint32_t b_dst = a_dst + A_TILE_BYTES;
          const int k0 = kb * BK;
          if (direct) {
            // both CTAs' loads of this k-block complete on the leader's full[s]: the leader arms it for
            // the bytes of both (the peer's bytes may land first: the transaction count may run negative
            // inside a phase, which cannot complete before the leader's arrival)
            const uint32_t bar = mapa_cluster(smem_u32(&ctrl->full[s]), 0);
            if (rank == 0) mbar_arrive_expect_tx(smem_u32(&ctrl->full[s]), 2u * tx_bytes);
            if (!a_mn) {
              tma_load_2d_pair(a_dst, &op->tmA, bar, k0, m0);
            } else if (op->a_3d) {
              tma_load_3d_pair(a_dst, &op->tmA, bar, 0, k0, m0 >> 5);
            } else {
#pragma unroll
              for (int c = 0; c < BM / 32; ++c) tma_load_2d_pair(a_dst + c * 4096, &op->tmA, bar, m0 + c * 32, k0);
            }
            if (!b_mn) {
              tma_load_2d_pair(b_dst, &op->tmB, bar, k0, n0);
            } else if (op->b_3d) {
              tma_load_3d_pair(b_dst, &op->tmB, bar, 0, k0, n0 >> 5);
            } else {
              for (int c = 0; c < bh / 32; ++c) tma_load_2d_pair(b_dst + c * 4096, &op->tmB, bar, n0 + c * 32, k0);
            }
          } else {
            const uint32_t bar = smem_u32(&ctrl->full[s]);
            mbar_arrive_expect_tx(bar, tx_bytes);
            if (!a_mn) {
              tma_load_2d(a_dst, &op->tmA, bar, k0, m0);
            } else if (op->a_3d) {
              tma_load_3d(a_dst, &op->tmA, bar, 0, k0, m0 >> 5);
            } else {
#pragma unroll
              for (int c = 0; c < BM / 32; ++c) tma_load_2d(a_dst + c * 4096, &op->tmA, bar, m0 + c * 32, k0);
            }
            if (!b_mn) {
              tma_load_2d(b_dst, &op->tmB, bar, k0, n0);
            } else if (op->b_3d) {
              tma_load_3d(b_dst, &op->tmB, bar, 0, k0, n0 >> 5);
            } else {
              for (int c = 0; c < bh / 32; ++c) tma_load_2d(b_dst + c * 4096, &op->tmB, bar, n0 + c * 32, k0);
            }
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == 1 && rank == 0) {
    // =============================== MMA issuer (leader) ===============================
    int cursor = 0;
    uint32_t it = 0, tcount = 0;
    bool ok = true;
    // the same barrier offsets in the peer CTA, as cluster addresses
    for (int t = pair_id; t < p.total_tiles && ok; t += n_pairs, ++tcount) {
      Tile tc;
      const GemmOp *op = decode_tile(ops, n_ops, t, cursor, tc);
      const uint32_t as = tcount & 1u;
      const uint32_t aph = (tcount >> 1) & 1u;
      int okl = 1;
      if (lane == 0)
        okl = wait_bar_cluster(smem_u32(&ctrl->tmem_empty[as]), aph ^ 1u, ctrl, p, SITE_TMEM_EMPTY, op->op_index,
                               as, 32);
      ok = __shfl_sync(0xffffffffu, okl, 0) != 0;
      if (!ok) break;
      tc_fence_after();

      const uint32_t d_tmem = tmem_base + as * MAX_BN;
      const uint32_t idesc = op->idesc;
      const uint64_t hiA = op->a_mn ? smem_desc_hi(4096, 512, 1) : smem_desc_hi(16, 1024, 2);
      const uint64_t hiB = op->b_mn ? smem_desc_hi(4096, 512, 1) : smem_desc_hi(16, 1024, 2);
      const uint32_t stepA = op->a_mn ? 1024u : 32u;
      const uint32_t stepB = op->b_mn ? 1024u : 32u;

      for (int kb = tc.kb0; kb < tc.kb1; ++kb, ++it) {
        const int s = it % NST;
        const uint32_t ph = (it / NST) & 1u;
        okl = 1;
        if (lane == 0) {
          // TF32: full[s] counts the bytes of both CTAs.
          // 3xTF32: ready counts the transform warps of both CTAs, which implies both rings landed and were split.
          if (!X3) okl = wait_bar(smem_u32(&ctrl->full[s]), ph, ctrl, p, SITE_SMEM_FULL, op->op_index, s);
          if (okl && !direct)
            okl = wait_bar_cluster(smem_u32(&ctrl->ready[s]), ph, ctrl, p, SITE_SMEM_READY, op->op_index, s);
        }
        ok = __shfl_sync(0xffffffffu, okl, 0) != 0;
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_addr = ring + s * STAGE_STRIDE;
          const uint32_t b_addr = a_addr + A_TILE_BYTES;
#pragma unroll
          for (int ks = 0; ks < BK / UMMA_K; ++ks) {
            const uint32_t acc = (kb > tc.kb0 || ks > 0) ? 1u : 0u;
            const uint64_t da = smem_desc(hiA, a_addr + ks * stepA);
            const uint64_t db = smem_desc(hiB, b_addr + ks * stepB);
            if (X3) {
              const uint64_t da_lo = smem_desc(hiA, a_addr + LO_OFFSET + ks * stepA);
              const uint64_t db_lo = smem_desc(hiB, b_addr + LO_OFFSET + ks * stepB);
              mma_tf32_pair(d_tmem, da_lo, db, idesc, acc);
              mma_tf32_pair(d_tmem, da, db_lo, idesc, 1u);
              mma_tf32_pair(d_tmem, da, db, idesc, 1u);
            } else {
              mma_tf32_pair(d_tmem, da, db, idesc, acc);
            }
          }
          // the stage is free in BOTH CTAs once these MMAs have read it
          const uint32_t e = smem_u32(&ctrl->empty[s]);
          mma_commit_pair(mapa_cluster(e, 0));
          mma_commit_pair(mapa_cluster(e, 1));
        }
        __syncwarp();
      }
      if (!ok) break;
      if (lane == 0) {
        const uint32_t f = smem_u32(&ctrl->tmem_full[as]);
        mma_commit_pair(mapa_cluster(f, 0));
        mma_commit_pair(mapa_cluster(f, 1));
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // (the peer CTA issues no MMAs: its warp 1 only allocates and frees tensor memory)
  } else if (warp < EPI_WARP0 && xform) {
    // =============================== operand transform (both CTAs) ===============================
    {
      const int x = tid - XFORM_WARP0 * 32;  // 0..127
      int cursor = 0;
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair_id; t < p.total_tiles && ok; t += n_pairs) {
        Tile tc;
        const GemmOp *op = decode_tile(ops, n_ops, t, cursor, tc);
        const int bh = op->bn >> 1;
        // the bias gradient belongs to tile row 0 (both CTAs of that pair: each sums its half of
        // the columns)
        const bool do_colsum = (op->colsum != nullptr) && tc.m_tile == 0 && op->b_mn;
        const int groups = bh >> 2;
        const int parts = 128 / groups;
        const int rows_per_part = 32 / parts;
        const int grp = x / parts, part = x % parts;
        const int chunk = grp >> 3, q16 = grp & 7;
        float4 csum = make_float4(0.f, 0.f, 0.f, 0.f);
        const int stage_f4 = (A_TILE_BYTES + bh * BK * 4) >> 4;

        for (int kb = tc.kb0; kb < tc.kb1; ++kb, ++it) {
          const int s = it % NST;
          const uint32_t ph = (it / NST) & 1u;
          int okl = 1;
          if (lane == 0)
            okl = wait_bar(smem_u32(&ctrl->full[s]), ph, ctrl, p, SITE_SMEM_FULL, op->op_index, s, X3 ? 0 : 64);
          ok = __shfl_sync(0xffffffffu, okl, 0) != 0;
          if (!ok) break;
          uint8_t *stage = ring_ptr + s * STAGE_STRIDE;
          const bool walk_b = op->b_mn && (X3 || do_colsum);
          if (walk_b) {
            uint8_t *bchunk = stage + A_TILE_BYTES + chunk * 4096;
#pragma unroll 4
            for (int r = part * rows_per_part; r < (part + 1) * rows_per_part; ++r) {
              const int phys32 = (q16 >> 1) ^ (r & 3);
              float4 *ptr = reinterpret_cast<float4 *>(bchunk + r * 128 + phys32 * 32 + (q16 & 1) * 16);
              const float4 v = *ptr;
              csum.x += v.x; csum.y += v.y; csum.z += v.z; csum.w += v.w;
              if (X3) {
                float4 h, l;
                h.x = tf32_round(v.x); h.y = tf32_round(v.y); h.z = tf32_round(v.z); h.w = tf32_round(v.w);
                l.x = v.x - h.x; l.y = v.y - h.y; l.z = v.z - h.z; l.w = v.w - h.w;
                *ptr = h;
                *reinterpret_cast<float4 *>(reinterpret_cast<uint8_t *>(ptr) + LO_OFFSET) = l;
              }
            }
          }
          if (X3) {
            float4 *hi = reinterpret_cast<float4 *>(stage);
            float4 *lo = reinterpret_cast<float4 *>(stage + LO_OFFSET);
            const int lin_f4 = walk_b ? (A_TILE_BYTES >> 4) : stage_f4;
            for (int i = x; i < lin_f4; i += NUM_XFORM_WARPS * 32) {
              const float4 v = hi[i];
              float4 h, l;
              h.x = tf32_round(v.x); h.y = tf32_round(v.y); h.z = tf32_round(v.z); h.w = tf32_round(v.w);
              l.x = v.x - h.x; l.y = v.y - h.y; l.z = v.z - h.z; l.w = v.w - h.w;
              hi[i] = h;
              lo[i] = l;
            }
            fence_proxy_async_smem();
          }
          __syncwarp();
          if (lane == 0) {
            if (X3) mbar_arrive_cluster(mapa_cluster(smem_u32(&ctrl->ready[s]), 0));
            mbar_arrive(smem_u32(&ctrl->empty[s]));
          }
        }
        if (!ok) break;
        if (do_colsum) {
          for (int o = 1; o < parts; o <<= 1) {
            csum.x += __shfl_xor_sync(0xffffffffu, csum.x, o);
            csum.y += __shfl_xor_sync(0xffffffffu, csum.y, o);
            csum.z += __shfl_xor_sync(0xffffffffu, csum.z, o);
            csum.w += __shfl_xor_sync(0xffffffffu, csum.w, o);
          }
          if (part == 0) {
            const int col = tc.n_tile * op->bn + (int)rank * bh + grp * 4;
            const float v[4] = {csum.x, csum.y, csum.z, csum.w};
            for (int j = 0; j < 4; ++j) {
              if (col + j < op->Nc) {
                if (op->splits > 1) atomicAdd(op->colsum + col + j, v[j]);
                else op->colsum[col + j] = v[j];
              }
            }
          }
        }
      }
    }
  } else {
    // =============================== epilogue (both CTAs) ===============================
    // Warps 6-9 drain the accumulator, each CTA its own 128 rows of the pair's tile, every warp with two
    // staging boxes (eight warps on it measured slower here than four: lm_head forward 1186 against 1125 us).
    // Warps 2-5, when there is nothing to transform, sum their tile's share of the bias gradient beside the ring.
    const bool helper = warp < EPI_WARP0;
    const uint32_t sbuf = ring + RING_BYTES + (uint32_t)(warp - EPI_WARP0) * 2u * EPI_BUF_BYTES;
    int cursor = 0;
    uint32_t tcount = 0;
    bool ok = true;
    for (int t = pair_id; t < p.total_tiles && ok; t += n_pairs, ++tcount) {
      Tile tc;
      const GemmOp *op = decode_tile(ops, n_ops, t, cursor, tc);
      const int m_tile = 2 * tc.m_tile + (int)rank;
      if (helper) {
        if (!X3 && op->colsum != nullptr && op->colsum_spread && m_tile < op->tiles_m)
          ok = colsum_global_tile(op, tc, m_tile, tid - XFORM_WARP0 * 32, lane, ctrl, p);
      } else {
        ok = epilogue_tile<true>(op, tc, m_tile, tcount, false, 1, 0, 1u, 1u, sbuf, sbuf + EPI_BUF_BYTES, tmem_base, ctrl,
                                 p, warp, lane);
      }
    }
  }

  // =============================== teardown ===============================
  if (*reinterpret_cast<volatile int *>(&ctrl->abort)) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees tensor memory or exits while the other may still use it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------
int pair_set_kernel_attributes() {
  cudaError_t e = cudaFuncSetAttribute(gpt2_linear_tcgen05_pair_kernel<false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return GPT2L_ERR_CUDA;
  e = cudaFuncSetAttribute(gpt2_linear_tcgen05_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           SMEM_BYTES);
  return e == cudaSuccess ? GPT2L_OK : GPT2L_ERR_CUDA;
}

static void fill_config(cudaLaunchConfig_t *cfg, cudaLaunchAttribute *attr, int n_pairs, cudaStream_t stream) {
  memset(cfg, 0, sizeof(*cfg));
  cfg->gridDim = dim3(2 * n_pairs, 1, 1);
  cfg->blockDim = dim3(NUM_THREADS, 1, 1);
  cfg->dynamicSmemBytes = SMEM_BYTES;
  cfg->stream = stream;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg->attrs = attr;
  cfg->numAttrs = 1;
}

int pair_max_pairs(int num_sms) {
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  fill_config(&cfg, attr, num_sms / 2, nullptr);
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, gpt2_linear_tcgen05_pair_kernel<false>, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  const int cap = num_sms / 2;
  return clusters < cap ? clusters : cap;
}

int pair_launch(const GemmOp *op_by_value, const LaunchParams &p, int n_pairs, bool x3, cudaStream_t stream) {
  static GemmOp dummy;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  fill_config(&cfg, attr, n_pairs, stream);
  const GemmOp &op = op_by_value ? *op_by_value : dummy;
  cudaError_t e;
  if (x3) e = cudaLaunchKernelEx(&cfg, gpt2_linear_tcgen05_pair_kernel<true>, op, p);
  else e = cudaLaunchKernelEx(&cfg, gpt2_linear_tcgen05_pair_kernel<false>, op, p);
  count_launch();
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return GPT2L_ERR_CUDA;
  }
  return GPT2L_OK;
}

}  // namespace g2l
