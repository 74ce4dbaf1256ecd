// The sm_100a GEMM kernel behind all three linear-layer calls and the megakernel.
//
// One persistent, warp-specialised kernel:  C[Mc][Nc] = A . B (+ bias), fp32 in HBM,
// TF32 (or 3xTF32) on the tcgen05 tensor cores, fp32 accumulators in tensor memory.
//
//   warp 0      TMA producer: waits for the tile's dependency counters, then streams
//               128 x 32 (A) and bn x 32 (B) fp32 blocks into a shared-memory ring with
//               cp.async.bulk.tensor (no multicast), signalling `full[s]`.
//   warp 1      allocates the 512 TMEM columns; one lane issues tcgen05.mma.kind::tf32
//               (128 x bn x 8 per instruction, 4 per k-block), commits to `empty[s]`, and
//               after the last k-block commits to `tmem_full[acc]`.
//   warps 2-5   operand transform: in 3xTF32 mode split each landed stage into hi + lo
//               copies; in backward_weight they also add up the columns of the B block
//               (the bias gradient) for the tile row that owns it.
//   warps 6-9   epilogue: tcgen05.ld the accumulator (warp w reads TMEM lanes 32*(w%4)..),
//               add bias / GELU dual store / split-K combine, store fp32, then publish the
//               tile on the dependency counters with a release reduction.
//
// Operand layouts. A k-block is 32 fp32 = 128 bytes wide. An operand whose reduction index
// is contiguous in HBM ("K-major") lands as rows of 128 bytes with the 128-byte swizzle
// (16-byte chunk index XOR row%8). An operand whose output index is contiguous ("MN-major":
// W in forward, both operands in backward_weight) lands as 32 x 32 boxes with the 128-byte
// swizzle on 32-byte atoms (32-byte chunk index XOR row%4) — the only shared-memory layout
// tcgen05 accepts for MN-major 32-bit operands.
//
// Every wait in here is bounded: on expiry the CTA records where it gave up in the status
// record, raises an abort flag that every other loop polls, and the kernel unwinds (TMEM
// is freed) instead of hanging.
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>

#include "linear_internal.h"
#include "ptx_sm100.cuh"
#include "kernel_common.cuh"
#include "epilogue.cuh"
#include "step_rowops.cuh"
#include "attention_flash.cuh"

namespace g2l {

using namespace ptx;

// ------------------------------------------------------------------------------------
// per-tile bodies of the operand-transform and epilogue roles (shared by the GEMM kernel and the
// step kernel, which runs them for GEMM tiles between its other ops)
// ------------------------------------------------------------------------------------
template <bool X3>
struct RingCfg {
  static constexpr int NST = X3 ? STAGES_3X : STAGES_1X;
  static constexpr int STAGE_STRIDE = X3 ? 2 * STAGE_BYTES : STAGE_BYTES;
  static constexpr int LO_OFFSET = STAGE_BYTES;  // 3x: lo copies sit behind the hi copies of a stage
};

// Operand transform of one tile: 3xTF32 hi/lo split of every landed stage and / or the bias-gradient
// column sums of the B blocks. `x` = thread index among the 128 transform threads. Advances `it`.
template <bool X3>
__device__ __forceinline__ bool xform_tile(const GemmOp *op, const Tile &tc, uint8_t *ring_ptr, Ctrl *ctrl,
                                           const LaunchParams &p, uint32_t &it, int x, int lane) {
  using R = RingCfg<X3>;
  bool ok = true;
  const int bn = op->bn;
  // softmax / cross-entropy backward folded into the operand: the logits become dlogits in shared memory
  const int xmode = op->xent_mode;
  const bool rewrites = X3 || xmode >= 2;
  float x_lse = 0.f;  // xmode 2 (A operand, K-major): this thread owns row x of the tile for the whole tile
  int x_tgt = -1;
  // bias gradient = column sums of the B blocks. Spread over the tile rows (row m takes the
  // k-blocks with kb % tiles_m == m) so that no CTA carries the whole extra pass: with tile row 0
  // doing all of it those CTAs ran ~30 % longer than the rest and the launch waited for them.
  const bool has_cs = (op->colsum != nullptr) && op->b_mn;
  const bool spread = has_cs && op->colsum_spread != 0;
  const bool do_colsum = has_cs && (spread || tc.m_tile == 0);
  // column-sum mapping: `groups` float4 column groups, `parts` threads share a group and
  // split the 32 k-rows of a block between them.
  const int groups = bn >> 2;
  const int parts = 128 / groups;
  const int rows_per_part = 32 / parts;
  const int grp = x / parts, part = x % parts;
  const int chunk = grp >> 3, q16 = grp & 7;
  float4 csum = make_float4(0.f, 0.f, 0.f, 0.f);
  const int stage_f4 = (A_TILE_BYTES + bn * BK * 4) >> 4;

  if (!rewrites) {
    // TF32 mode: the stages need nothing from these warps (the MMA lane arrives on empty[s] in their place);
    // the column sums, if any, do not go through the ring (colsum_global_tile; every weight gradient is planned
    // with its column sums spread over the tile rows)
    it += (uint32_t)(tc.kb1 - tc.kb0);
    return has_cs ? colsum_global_tile(op, tc, tc.m_tile, x, lane, ctrl, p) : true;
  }

  for (int kb = tc.kb0; kb < tc.kb1; ++kb, ++it) {
    const int s = it % R::NST;
    const uint32_t ph = (it / R::NST) & 1u;
    int okl = 1;
    const bool cs_kb = do_colsum && (!spread || (kb % op->tiles_m) == tc.m_tile);
    // (these warps rewrite or sum every stage here, so each is on the ring's critical path: no back-off)
    if (lane == 0) okl = wait_bar(smem_u32(&ctrl->full[s]), ph, ctrl, p, SITE_SMEM_FULL, op->op_index, s);
    ok = __shfl_sync(0xffffffffu, okl, 0) != 0;
    if (!ok) break;
    uint8_t *stage = ring_ptr + s * R::STAGE_STRIDE;
    if (xmode == 2 && kb == tc.kb0) {
      // only now: the tile's first block has landed, so the producer has seen the tile's dependencies
      // (the row statistics among them) complete
      const int grow = tc.m_tile * BM + x;
      if (grow < op->Mc) {
        x_lse = op->xent_lse[grow];
        x_tgt = op->xent_tgt[grow];
      }
    }
    // An MN-major B block is walked by (column group, k-row) so that the thread that sums a
    // column is also the one that rewrites it in 3xTF32 mode (no cross-thread hazard).
    // TMA zero-fills rows and columns outside the matrix, so no guards are needed.
    const bool walk_b = op->b_mn && (X3 || cs_kb || xmode == 3);
    if (xmode == 2) {
      // row x of the A block: eight 16-byte chunks, chunk j at physical position j ^ (x & 7)
      uint8_t *arow = stage + x * 128;
      const int k0 = kb * BK;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 *ptr = reinterpret_cast<float4 *>(arow + ((j ^ (x & 7)) << 4));
        float4 v = *ptr;
        const int col = k0 + 4 * j;
        v.x = xent_grad(v.x, x_lse, col, x_tgt, op->xent_vocab, op->xent_scale);
        v.y = xent_grad(v.y, x_lse, col + 1, x_tgt, op->xent_vocab, op->xent_scale);
        v.z = xent_grad(v.z, x_lse, col + 2, x_tgt, op->xent_vocab, op->xent_scale);
        v.w = xent_grad(v.w, x_lse, col + 3, x_tgt, op->xent_vocab, op->xent_scale);
        if (X3) {
          float4 h, l;
          h.x = tf32_round(v.x); h.y = tf32_round(v.y); h.z = tf32_round(v.z); h.w = tf32_round(v.w);
          l.x = v.x - h.x; l.y = v.y - h.y; l.z = v.z - h.z; l.w = v.w - h.w;
          *ptr = h;
          *reinterpret_cast<float4 *>(reinterpret_cast<uint8_t *>(ptr) + R::LO_OFFSET) = l;
        } else {
          *ptr = v;
        }
      }
    }
    if (walk_b) {
      uint8_t *bchunk = stage + A_TILE_BYTES + chunk * 4096;
#pragma unroll 4
      for (int r = part * rows_per_part; r < (part + 1) * rows_per_part; ++r) {
        const int phys32 = (q16 >> 1) ^ (r & 3);
        float4 *ptr = reinterpret_cast<float4 *>(bchunk + r * 128 + phys32 * 32 + (q16 & 1) * 16);
        float4 v = *ptr;
        if (xmode == 3) {
          // k-row r of this block is token kb * 32 + r; the columns are vocabulary entries
          const int tokn = kb * BK + r;
          const bool live = tokn < op->Kc;
          const float lse2 = live ? op->xent_lse[tokn] : 0.f;
          const int tg = live ? op->xent_tgt[tokn] : -1;
          const int col = tc.n_tile * bn + grp * 4;
          const float sc = live ? op->xent_scale : 0.f;
          v.x = xent_grad(v.x, lse2, col, tg, op->xent_vocab, sc);
          v.y = xent_grad(v.y, lse2, col + 1, tg, op->xent_vocab, sc);
          v.z = xent_grad(v.z, lse2, col + 2, tg, op->xent_vocab, sc);
          v.w = xent_grad(v.w, lse2, col + 3, tg, op->xent_vocab, sc);
          if (!X3) *ptr = v;
        }
        if (cs_kb) { csum.x += v.x; csum.y += v.y; csum.z += v.z; csum.w += v.w; }
        if (X3) {
          float4 h, l;
          h.x = tf32_round(v.x); h.y = tf32_round(v.y); h.z = tf32_round(v.z); h.w = tf32_round(v.w);
          l.x = v.x - h.x; l.y = v.y - h.y; l.z = v.z - h.z; l.w = v.w - h.w;
          *ptr = h;
          *reinterpret_cast<float4 *>(reinterpret_cast<uint8_t *>(ptr) + R::LO_OFFSET) = l;
        }
      }
    }
    if (X3) {
      float4 *hi = reinterpret_cast<float4 *>(stage);
      float4 *lo = reinterpret_cast<float4 *>(stage + R::LO_OFFSET);
      // what is left to split linearly: A (unless its rows were rewritten above) and a K-major B
      const int lin_lo = xmode == 2 ? (A_TILE_BYTES >> 4) : 0;
      const int lin_f4 = walk_b ? (A_TILE_BYTES >> 4) : stage_f4;
      for (int i = lin_lo + x; i < lin_f4; i += NUM_XFORM_WARPS * 32) {
        const float4 v = hi[i];
        float4 h, l;
        h.x = tf32_round(v.x); h.y = tf32_round(v.y); h.z = tf32_round(v.z); h.w = tf32_round(v.w);
        l.x = v.x - h.x; l.y = v.y - h.y; l.z = v.z - h.z; l.w = v.w - h.w;
        hi[i] = h;
        lo[i] = l;
      }
    }
    if (rewrites) fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      if (rewrites) mbar_arrive(smem_u32(&ctrl->ready[s]));
      mbar_arrive(smem_u32(&ctrl->empty[s]));
    }
  }
  if (!ok) return false;
  if (do_colsum) {
    for (int o = 1; o < parts; o <<= 1) {
      csum.x += __shfl_xor_sync(0xffffffffu, csum.x, o);
      csum.y += __shfl_xor_sync(0xffffffffu, csum.y, o);
      csum.z += __shfl_xor_sync(0xffffffffu, csum.z, o);
      csum.w += __shfl_xor_sync(0xffffffffu, csum.w, o);
    }
    if (part == 0) {
      const int col = tc.n_tile * bn + grp * 4;
      const float v[4] = {csum.x, csum.y, csum.z, csum.w};
      for (int j = 0; j < 4; ++j) {
        if (col + j < op->Nc) {
          if (op->splits > 1 || spread) atomicAdd(op->colsum + col + j, v[j]);
          else op->colsum[col + j] = v[j];
        }
      }
    }
  }
  return true;
}

// A non-GEMM tile of the step kernel, executed by one of the eight worker warps (w8 = 0..7). `scratch` is
// the 32 KiB of epilogue boxes, free while all eight warps are inside the same tile.
__device__ __noinline__ bool row_op_tile(const GemmOp *op, const Tile &tc, int w8, int lane, float *scratch,
                                            RowSync &rs, Ctrl *ctrl, const LaunchParams &p, unsigned &deps_done) {
  const int tile = tc.m_tile;
  const int rpt = op->rows_per_tile;
  // dependencies are counted per 128-row block; every warp makes its own acquire before it reads
  const int rb = op->op_kind == OPK_ADAMW ? 0 : (int)(((long long)tile * rpt) >> 7);
  int okl = 1;
  if (lane == 0) okl = wait_deps(op, rb, ctrl, p, deps_done) ? 1 : 0;
  if (__shfl_sync(0xffffffffu, okl, 0) == 0) return false;
  const int wtid = w8 * 32 + lane;
  bool ok = true;
  switch (op->op_kind) {
    case OPK_EMBED_FWD: row_embed_fwd(op, tile, wtid); break;
    case OPK_EMBED_BWD: row_embed_bwd(op, tile, wtid); break;
    case OPK_LN_FWD:
      if (op->ra.i1 <= 256) row_ln_fwd<2>(op, tile, w8, lane);
      else if (op->ra.i1 <= 768) row_ln_fwd<6>(op, tile, w8, lane);
      else row_ln_fwd<10>(op, tile, w8, lane);
      break;
    case OPK_LN_BWD:
      if (op->ra.i1 <= 256) ok = row_ln_bwd<2>(op, tile, w8, lane, scratch, rs, p);
      else if (op->ra.i1 <= 768) ok = row_ln_bwd<6>(op, tile, w8, lane, scratch, rs, p);
      else ok = row_ln_bwd<10>(op, tile, w8, lane, scratch, rs, p);
      break;
    case OPK_XENT: ok = row_xent(op, tile, w8, lane, scratch, rs, p); break;
    case OPK_ROWDOT: row_rowdot(op, tile, wtid); break;
    case OPK_ADAMW: row_adamw(op, tile, wtid, p); break;
    case OPK_TRANSPOSE: row_transpose(op, tile, w8, lane, scratch + w8 * 1024); break;
    case OPK_XENT_COMBINE: row_xent_combine(op, tile, w8, lane); break;
    case OPK_XENT_GRAD: row_xent_grad(op, tile, wtid); break;
    default: break;
  }
  if (!ok) return false;
  // publish: one arrival per worker warp and tile
  if (op->pub_rb_base >= 0 || op->pub_op_ctr >= 0) {
    __threadfence();
    __syncwarp();
    if (lane == 0) {
      if (op->pub_rb_base >= 0) red_release_add(p.counters + op->pub_rb_base + rb, 1u);
      if (op->pub_op_ctr >= 0) red_release_add(p.counters + op->pub_op_ctr, 1u);
    }
  }
  return true;
}

// ------------------------------------------------------------------------------------
// attention tiles inside the step kernel
// ------------------------------------------------------------------------------------
static_assert(CTRL_MAIN_BYTES + 3 * sizeof(flash::FlashCtrl) <= SMEM_CTRL_BYTES, "control region too small");
static_assert(flash::Cfg<flash::F_BWD_KV>::OFF_CTRL <= RING_BYTES + EPI_BYTES, "attention tile does not fit");
static_assert(flash::Cfg<flash::F_BWD_KV>::THREADS <= STEP_THREADS, "attention tile needs more warps");

// Every warp's view of how far the CTA's attention barriers have been driven (see attn_tile_body): steps and
// tiles per mode, and the number of CTA rendezvous so far. All warps run the same tiles, so all count alike.
struct AttnProgress {
  uint32_t steps[3] = {0u, 0u, 0u};
  uint32_t tiles[3] = {0u, 0u, 0u};
  uint32_t cta_phase = 0u;
  int dep_op = -1;          // warp 0: the attention op `deps_done` belongs to
  unsigned deps_done = 0u;  //         its dependencies already seen complete (see wait_deps)
};

// rendezvous of all STEP_THREADS / 32 warps (bounded like every other wait)
__device__ __forceinline__ bool cta_sync(Ctrl *ctrl, const LaunchParams &p, AttnProgress &ap, int op, int lane) {
  __syncwarp();
  int okl = 1;
  if (lane == 0) {
    const uint32_t bar = smem_u32(&ctrl->cta_bar);
    mbar_arrive(bar);
    okl = wait_bar(bar, ap.cta_phase & 1u, ctrl, p, SITE_CTA_SYNC, op, (int)ap.cta_phase, 20) ? 1 : 0;
  }
  ++ap.cta_phase;
  return __shfl_sync(0xffffffffu, okl, 0) != 0;
}

// One attention tile (128 rows of one head of one sequence) run by the whole CTA between two GEMM tiles:
// everybody meets (the ring, the epilogue boxes and the tensor memory are idle then), the fused attention
// code runs with its own barriers in the same shared memory and tensor memory, everybody meets again and
// the worker warps publish the tile. Tile order inside the op: sequence, then row block (heavy ones first),
// then head.
// (not inlined: the attention code gets a register allocation of its own instead of sharing one with the
// GEMM roles, whose state is dead while it runs)
template <int MODE>
__device__ __noinline__ bool attention_tile_mode(const GemmOp *op, int grb, int rb, int bh, uint8_t *ring_ptr, uint32_t ring,
                                                    Ctrl *ctrl, uint32_t tmem_base, const LaunchParams &p, AttnProgress &ap,
                                                    int warp, int lane) {
  using namespace flash;
  if (warp == 0) {
    int okl = 1;
    if (ap.dep_op != op->op_index) {
      ap.dep_op = op->op_index;
      ap.deps_done = 0u;
    }
    if (lane == 0) okl = wait_deps(op, grb, ctrl, p, ap.deps_done) ? 1 : 0;
    if (__shfl_sync(0xffffffffu, okl, 0) == 0) return false;
    fence_proxy_async_all();  // the operands were written with plain stores; TMA reads them next
  }
  if (!cta_sync(ctrl, p, ap, op->op_index, lane)) return false;
  FlashCtrl *fc = reinterpret_cast<FlashCtrl *>(reinterpret_cast<uint8_t *>(ctrl) + CTRL_MAIN_BYTES) + MODE;
  const RowArgs &ra = op->ra;
  FlashArgs a;
  a.B = ra.i0; a.C = ra.i1; a.T = ra.i2; a.NH = ra.i3;
  a.out = ra.out0;
  a.lse = MODE == F_FWD ? ra.out1 : const_cast<float *>(ra.in2);
  a.delta = ra.in3;
  a.dqkv = ra.out0;
  a.status = nullptr;
  a.wait_limit_ns = p.wait_limit_ns;
  a.cta_abort = &ctrl->abort;
  a.step_status = p.status;
  a.host_flag = p.host_flag;
  a.op_index = op->op_index;
  attn_tile_body<MODE>(p.fmaps[ra.i4], a, ring_ptr, ring, fc, tmem_base, warp, lane, rb, bh, ap.steps[MODE], ap.tiles[MODE]);
  ap.steps[MODE] += (uint32_t)attn_tile_steps<MODE>(rb, a.T);
  ap.tiles[MODE] += 1u;
  if (*reinterpret_cast<volatile int *>(&fc->abort)) return false;
  tc_fence_before();
  // the row-work warps' stores, before the rendezvous the publishing warps leave through (the loader and the
  // MMA issuers stored nothing)
  if (warp >= XFORM_WARP0) __threadfence();
  if (!cta_sync(ctrl, p, ap, op->op_index, lane)) return false;
  tc_fence_after();
  if (warp >= XFORM_WARP0 && warp < EPI_WARP0 + NUM_EPI_WARPS && lane == 0) {
    if (op->pub_rb_base >= 0) red_release_add(p.counters + op->pub_rb_base + grb, 1u);
    if (op->pub_op_ctr >= 0) red_release_add(p.counters + op->pub_op_ctr, 1u);
  }
  return true;
}

__device__ __forceinline__ bool attention_tile(const GemmOp *op, const Tile &tc, uint8_t *ring_ptr, uint32_t ring, Ctrl *ctrl,
                                               uint32_t tmem_base, const LaunchParams &p, AttnProgress &ap, int warp, int lane) {
  const int per_seq = op->rb_per_seq, heads = op->ra.i3;
  const int local = tc.m_tile;
  const int seq = local / (per_seq * heads);
  const int i = (local % (per_seq * heads)) / heads;
  const int h = local % heads;
  const int rb = op->op_kind == OPK_ATTN_BWD_KV ? i : per_seq - 1 - i;
  const int grb = seq * per_seq + rb;
  const int bh = seq * heads + h;
  if (op->op_kind == OPK_ATTN_FWD)
    return attention_tile_mode<flash::F_FWD>(op, grb, rb, bh, ring_ptr, ring, ctrl, tmem_base, p, ap, warp, lane);
  if (op->op_kind == OPK_ATTN_BWD_KV)
    return attention_tile_mode<flash::F_BWD_KV>(op, grb, rb, bh, ring_ptr, ring, ctrl, tmem_base, p, ap, warp, lane);
  return attention_tile_mode<flash::F_BWD_Q>(op, grb, rb, bh, ring_ptr, ring, ctrl, tmem_base, p, ap, warp, lane);
}

__device__ __forceinline__ bool is_attention(const GemmOp *op) {
  return op->op_kind >= OPK_ATTN_FWD && op->op_kind <= OPK_ATTN_BWD_Q;
}

// ------------------------------------------------------------------------------------
// the kernel. MEGA = false: one GEMM (or a list of GEMMs whose transform needs are the same for the
// whole launch). MEGA = true: the step kernel: GEMM ops with a per-op decision on the transform warps,
// row-local ops on the worker warps, one more warp, profile stamps.
// ------------------------------------------------------------------------------------
template <bool X3, bool MEGA>
__global__ void __launch_bounds__(MEGA ? STEP_THREADS : NUM_THREADS, 1)
gpt2_linear_tcgen05_kernel(const __grid_constant__ GemmOp op0, const LaunchParams p) {
  extern __shared__ uint8_t smem_raw[];
  using R = RingCfg<X3>;
  constexpr int NST = R::NST;
  constexpr int STAGE_STRIDE = R::STAGE_STRIDE;
  constexpr int LO_OFFSET = R::LO_OFFSET;

  const GemmOp *ops = p.ops ? p.ops : &op0;
  const int n_ops = p.ops ? p.n_ops : 1;

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t ring = (raw + 1023u) & ~1023u;
  uint8_t *ring_ptr = smem_raw + (ring - raw);
  Ctrl *ctrl = reinterpret_cast<Ctrl *>(ring_ptr + RING_BYTES + EPI_BYTES);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  // MEGA: barrier counts are fixed at their maximum; a party with nothing to do in an op is stood in for
  const bool xf_all = MEGA ? true : (p.xform_active != 0);

  if (tid == 0) {
    for (int s = 0; s < STAGES_1X; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1 + (xf_all ? NUM_XFORM_WARPS : 0));
      mbar_init(smem_u32(&ctrl->ready[s]), NUM_XFORM_WARPS);
    }
    for (int a = 0; a < NUM_ACC; ++a) {
      mbar_init(smem_u32(&ctrl->tmem_full[a]), 1);
      mbar_init(smem_u32(&ctrl->tmem_empty[a]), NUM_EPI_WARPS * ((MEGA || !p.xform_active) ? 2 : 1));
    }
    mbar_init(smem_u32(&ctrl->row_bar), NUM_WORKER_WARPS);
    mbar_init(smem_u32(&ctrl->cta_bar), STEP_THREADS / 32);
    if (MEGA) {
      flash::FlashCtrl *fc = reinterpret_cast<flash::FlashCtrl *>(reinterpret_cast<uint8_t *>(ctrl) + CTRL_MAIN_BYTES);
      flash::attn_init_barriers(fc + flash::F_FWD, flash::Cfg<flash::F_FWD>::NCW);
      flash::attn_init_barriers(fc + flash::F_BWD_Q, flash::Cfg<flash::F_BWD_Q>::NCW);
      flash::attn_init_barriers(fc + flash::F_BWD_KV, flash::Cfg<flash::F_BWD_KV>::NCW);
    }
    ctrl->abort = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(&ctrl->tmem_base);

  if (warp == 0) {
    // =============================== TMA producer ===============================
    int cursor = 0;
    uint32_t it = 0;
    bool ok = true;
    AttnProgress ap;
    int dep_op = -1;
    unsigned deps_done = 0u;
    for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
      Tile tc;
      const GemmOp *op = decode_tile(ops, n_ops, t, cursor, tc);
      if (MEGA && op->op_kind != OPK_GEMM) {
        // attention tiles take the whole CTA; the row-local ops are the worker warps' alone
        if (is_attention(op)) ok = attention_tile(op, tc, ring_ptr, ring, ctrl, tmem_base, p, ap, warp, lane);
        continue;
      }
      if (tc.skip) continue;  // every role skips the same tiles, so no barrier phase is consumed
      // ---- dependency counters: do not touch the operands before their producers are done
      if (op->wait_ctr[0] >= 0) {  // dependencies fill the slots from 0 up
        if (dep_op != op->op_index) {
          dep_op = op->op_index;
          deps_done = 0u;
        }
        int okl = 1;
        if (lane == 0) okl = wait_deps(op, tc.m_tile, ctrl, p, deps_done) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, okl, 0) != 0;
        if (!ok) break;
        fence_proxy_async_all();  // producers wrote with plain stores; TMA reads next
      }

      const int m0 = tc.m_tile * BM;
      const int n0 = tc.n_tile * op->bn;
      const int a_mn = op->a_mn, b_mn = op->b_mn, bn = op->bn;
      const uint32_t tx_bytes = (uint32_t)(A_TILE_BYTES + bn * BK * 4);
      for (int kb = tc.kb0; kb < tc.kb1; ++kb, ++it) {
        const int s = it % NST;
        const uint32_t ph = (it / NST) & 1u;
        int okl = 1;
        if (lane == 0)
          okl = wait_bar(smem_u32(&ctrl->empty[s]), ph ^ 1u, ctrl, p, SITE_SMEM_EMPTY, op->op_index, s, 32);
        ok = __shfl_sync(0xffffffffu, okl, 0) != 0;
        if (!ok) break;
        if (lane == 0) {
          const uint32_t bar = smem_u32(&ctrl->full[s]);
          const uint32_t a_dst = ring + s * STAGE_STRIDE;
          const uint32_t b_dst = a_dst + A_TILE_BYTES;
          mbar_arrive_expect_tx(bar, tx_bytes);
          const int k0 = kb * BK;
          if (op->batch > 1) {
            // batched operands: two trailing coordinates select the head and the sequence
            if (!a_mn) tma_load_4d(a_dst, &op->tmA, bar, k0, m0, tc.bh, tc.bb);
            else tma_load_5d(a_dst, &op->tmA, bar, 0, k0, m0 >> 5, tc.bh, tc.bb);
            if (!b_mn) tma_load_4d(b_dst, &op->tmB, bar, k0, n0, tc.bh, tc.bb);
            else tma_load_5d(b_dst, &op->tmB, bar, 0, k0, n0 >> 5, tc.bh, tc.bb);
          } else {
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
            for (int c = 0; c < bn / 32; ++c) tma_load_2d(b_dst + c * 4096, &op->tmB, bar, n0 + c * 32, k0);
          }
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // =============================== MMA issuer ===============================
    // The next tile is decoded while the current one is being issued: at a tile boundary the
    // tensor pipe holds less than a k-block of queued work, so nothing slow may sit there.
    int cursor = 0;
    uint32_t it = 0, tcount = 0;
    // one parity bit per stage for the `ready` barriers: only k-blocks whose stage is rewritten (3xTF32
    // split, logits -> dlogits) go through them, so their phases do not follow the ring position
    uint32_t rdy_par = 0u;
    bool ok = true;
    AttnProgress ap;
    int t = blockIdx.x;
    Tile tc;
    const GemmOp *op = nullptr;
    bool have = t < p.total_tiles;
    if (have) op = decode_tile(ops, n_ops, t, cursor, tc);
    while (have && ok) {
      const int t_next = t + (int)gridDim.x;
      const bool have_next = t_next < p.total_tiles;
      Tile tc_next = tc;
      const GemmOp *op_next = op;
      if (have_next) op_next = decode_tile(ops, n_ops, t_next, cursor, tc_next);
      if (tc.skip || (MEGA && op->op_kind != OPK_GEMM)) {
        if (MEGA && is_attention(op)) ok = attention_tile(op, tc, ring_ptr, ring, ctrl, tmem_base, p, ap, warp, lane);
        t = t_next; tc = tc_next; op = op_next; have = have_next;
        continue;
      }

      const uint32_t as = tcount & 1u;
      const uint32_t aph = (tcount >> 1) & 1u;
      int okl = 1;
      if (lane == 0)
        okl = wait_bar(smem_u32(&ctrl->tmem_empty[as]), aph ^ 1u, ctrl, p, SITE_TMEM_EMPTY, op->op_index, as, 32);
      ok = __shfl_sync(0xffffffffu, okl, 0) != 0;
      if (!ok) break;
      tc_fence_after();

      const uint32_t d_tmem = tmem_base + as * MAX_BN;
      const uint32_t idesc = op->idesc;
      // K-major: 8-row groups 1024 B apart, 128B swizzle; k-step = 32 B inside the row.
      // MN-major: 32-column chunks 4096 B apart (LBO), 4-row k-groups 512 B apart (SBO),
      //           128B swizzle on 32-byte atoms; k-step = 8 rows = 1024 B.
      const uint64_t hiA = op->a_mn ? smem_desc_hi(4096, 512, 1) : smem_desc_hi(16, 1024, 2);
      const uint64_t hiB = op->b_mn ? smem_desc_hi(4096, 512, 1) : smem_desc_hi(16, 1024, 2);
      const uint32_t stepA = op->a_mn ? 1024u : 32u;
      const uint32_t stepB = op->b_mn ? 1024u : 32u;
      // The transform warps' share of empty[s] is left to us wherever they do not touch the stages: in the step
      // kernel for every op that needs no operand transform, and in any TF32 launch whose barriers count them
      // (they rewrite stages only in 3xTF32 mode and for the fused cross-entropy; the bias gradient is read
      // beside the ring).
      const bool via_ready = X3 || op->xent_mode >= 2;  // the transform warps hand the stage over
      const bool xf_counted = MEGA || p.xform_active != 0;
      const bool stand_in = xf_counted && !((MEGA ? (op->xform != 0) : (p.xform_active != 0)) && via_ready);

      for (int kb = tc.kb0; kb < tc.kb1; ++kb, ++it) {
        const int s = it % NST;
        const uint32_t ph = (it / NST) & 1u;
        okl = 1;
        if (lane == 0) {
          const uint32_t bar = via_ready ? smem_u32(&ctrl->ready[s]) : smem_u32(&ctrl->full[s]);
          okl = wait_bar(bar, via_ready ? ((rdy_par >> s) & 1u) : ph, ctrl, p, via_ready ? SITE_SMEM_READY : SITE_SMEM_FULL,
                         op->op_index, s);
        }
        if (via_ready) rdy_par ^= 1u << s;
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
              mma_tf32(d_tmem, da_lo, db, idesc, acc);  // small terms first
              mma_tf32(d_tmem, da, db_lo, idesc, 1u);
              mma_tf32(d_tmem, da, db, idesc, 1u);
            } else {
              mma_tf32(d_tmem, da, db, idesc, acc);
            }
          }
          mma_commit(smem_u32(&ctrl->empty[s]));  // frees the stage once these MMAs have read it
          if (stand_in) mbar_arrive_cnt(smem_u32(&ctrl->empty[s]), NUM_XFORM_WARPS);
        }
        __syncwarp();
      }
      if (!ok) break;
      if (lane == 0) mma_commit(smem_u32(&ctrl->tmem_full[as]));
      __syncwarp();
      t = t_next;
      tc = tc_next;
      op = op_next;
      have = have_next;
      ++tcount;
    }
  } else if (!MEGA && warp < EPI_WARP0 && p.xform_active) {
    // =============================== operand transform ===============================
    // (in launches where no op needs a split or a column sum these warps join the epilogue instead)
    const int x = tid - XFORM_WARP0 * 32;  // 0..127
    int cursor = 0;
    uint32_t it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
      Tile tc;
      const GemmOp *op = decode_tile(ops, n_ops, t, cursor, tc);
      if (tc.skip) continue;
      ok = xform_tile<X3>(op, tc, ring_ptr, ctrl, p, it, x, lane);
    }
  } else if (!MEGA) {
    // =============================== epilogue ===============================
    // Warps 6-9 always work here. When the transform warps 2-5 have nothing to transform they
    // help: warp w and warp w + 4 read the same TMEM lane quarter and take alternate 32-column
    // chunks of every tile, which halves the time a tile spends in the epilogue (what bounds
    // short reductions such as the attention score GEMMs, and every CTA's last tile).
    const bool helper = warp < EPI_WARP0;
    const int n_epi = p.xform_active ? 1 : 2;
    const int c_first = helper ? 1 : 0;
    const uint32_t sbuf = ring + RING_BYTES +
                          (uint32_t)(helper ? (warp - XFORM_WARP0) * 2 + 1 : (warp - EPI_WARP0) * 2) * EPI_BUF_BYTES;
    int cursor = 0;
    uint32_t tcount = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
      Tile tc;
      const GemmOp *op = decode_tile(ops, n_ops, t, cursor, tc);
      if (tc.skip) continue;
      // TF32 bias gradient: the helper warps sum their tile's share of g_out while its main loop runs
      if (!X3 && helper && op->colsum != nullptr && op->colsum_spread)
        ok = colsum_global_tile(op, tc, tc.m_tile, tid - XFORM_WARP0 * 32, lane, ctrl, p);
      if (ok) ok = epilogue_tile<false>(op, tc, tc.m_tile, tcount, helper, n_epi, c_first, 1u, 1u, sbuf,
                                        n_epi == 1 ? sbuf + EPI_BUF_BYTES : sbuf, tmem_base, ctrl, p, warp, lane);
      ++tcount;
    }
  } else if (warp < EPI_WARP0 + NUM_EPI_WARPS) {
    // =============================== step kernel: worker warps 2-9 ===============================
    // GEMM tile of an op that needs the transform: warps 2-5 transform, warps 6-9 drain the accumulator
    // alone (and arrive twice). GEMM tile of any other op: all eight drain it, alternate chunks. Any other
    // tile: all eight run the row-local op.
    const bool helper = warp < EPI_WARP0;
    const int w8 = warp - XFORM_WARP0;
    const int x = tid - XFORM_WARP0 * 32;
    const uint32_t sbuf = ring + RING_BYTES +
                          (uint32_t)(helper ? (warp - XFORM_WARP0) * 2 + 1 : (warp - EPI_WARP0) * 2) * EPI_BUF_BYTES;
    float *scratch = reinterpret_cast<float *>(ring_ptr + RING_BYTES);
    RowSync rs = {smem_u32(&ctrl->row_bar), 0u, ctrl};
    AttnProgress ap;
    int cursor = 0;
    uint32_t it = 0, tcount = 0;
    bool ok = true;
    int dep_op = -1;
    unsigned deps_done = 0u;
    for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
      Tile tc;
      const GemmOp *op = decode_tile(ops, n_ops, t, cursor, tc);
      if (dep_op != op->op_index) {
        dep_op = op->op_index;
        deps_done = 0u;
      }
      long long t0 = 0;
      if (p.prof && tid == EPI_WARP0 * 32) t0 = globaltimer_ns();
      if (op->op_kind != OPK_GEMM) {
        if (is_attention(op)) ok = attention_tile(op, tc, ring_ptr, ring, ctrl, tmem_base, p, ap, warp, lane);
        else ok = row_op_tile(op, tc, w8, lane, scratch, rs, ctrl, p, deps_done);
      } else if (tc.skip) {
        continue;
      } else if (op->xform) {
        if (helper) ok = xform_tile<X3>(op, tc, ring_ptr, ctrl, p, it, x, lane);
        else ok = epilogue_tile<false>(op, tc, tc.m_tile, tcount, false, 1, 0, 2u, 2u, sbuf, sbuf + EPI_BUF_BYTES, tmem_base, ctrl, p, warp, lane);
        if (!helper) it += (uint32_t)(tc.kb1 - tc.kb0);
        ++tcount;
      } else {
        if (!X3 && helper && op->colsum != nullptr && op->colsum_spread) ok = colsum_global_tile(op, tc, tc.m_tile, x, lane, ctrl, p);
        if (ok) ok = epilogue_tile<false>(op, tc, tc.m_tile, tcount, helper, 2, helper ? 1 : 0, 1u, 1u, sbuf, sbuf, tmem_base, ctrl, p, warp, lane);
        it += (uint32_t)(tc.kb1 - tc.kb0);
        ++tcount;
      }
      if (p.prof && tid == EPI_WARP0 * 32) {
        // per-tile profile stamp (the reference keeps such arrays per instruction, src/mk.cu:966-971):
        // start time, and SM id with the time this warp spent in the tile
        const long long t1 = globaltimer_ns();
        p.prof[2 * (size_t)t] = (unsigned long long)t0;
        p.prof[2 * (size_t)t + 1] = ((unsigned long long)smid() << 48) | (unsigned long long)(t1 - t0);
      }
    }
  }

  else if (MEGA) {
    // =============================== step kernel: warp 10 ===============================
    // only the key/value pass of the attention backward has work for an eleventh warp
    AttnProgress ap;
    int cursor = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
      Tile tc;
      const GemmOp *op = decode_tile(ops, n_ops, t, cursor, tc);
      if (is_attention(op)) ok = attention_tile(op, tc, ring_ptr, ring, ctrl, tmem_base, p, ap, warp, lane);
    }
  }

  // =============================== teardown ===============================
  if (*reinterpret_cast<volatile int *>(&ctrl->abort)) {
    // give copies and MMAs that are still in flight time to land before smem/TMEM go away
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------
static std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n); }
long long launch_count_value() { return g_launches.load(); }

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(sym);
    else (void)cudaGetLastError();
  }
  return fn;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

bool tma_eligible(const GemmDesc &d) {
  // row strides of every tensor involved are K or N floats; TMA needs 16-byte multiples
  if ((d.K & 3) || (d.N & 3)) return false;
  if (!aligned16(d.out) || !aligned16(d.a) || !aligned16(d.b)) return false;
  if (d.bias && !aligned16(d.bias)) return false;
  if (d.opts.out2 && !aligned16(d.opts.out2)) return false;
  if (d.opts.aux_op && !aligned16(d.opts.aux)) return false;
  return true;
}

// 2-D fp32 tensor map: `inner` contiguous elements per row, `outer` rows, row pitch = inner.
static int encode_map(CUtensorMap *map, const float *base, uint64_t inner, uint64_t outer, uint32_t box_inner,
                      uint32_t box_outer, bool mn_major) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return GPT2L_ERR_CUDA;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {inner * sizeof(float)};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? GPT2L_OK : GPT2L_ERR_CUDA;
}

// MN-major operand whose contiguous extent is a multiple of 32: viewed as [inner/32][outer][32]
// so that ONE copy lands every 32-column chunk of a tile (chunk c at offset c * 4096 bytes).
static int encode_map_chunked(CUtensorMap *map, const float *base, uint64_t inner, uint64_t outer,
                              uint32_t chunks) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return GPT2L_ERR_CUDA;
  cuuint64_t dims[3] = {32, outer, inner / 32};
  cuuint64_t strides[2] = {inner * sizeof(float), 32 * sizeof(float)};
  cuuint32_t box[3] = {32, 32, chunks};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? GPT2L_OK : GPT2L_ERR_CUDA;
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Picks the tile width and the number of reduction splits: the pair that needs the fewest
// (waves x per-tile work), where a tile's cost follows the bytes it pulls per k-block.
static void choose_tiling(int Mc, int Nc, int kb_total, int num_sms, int forced_splits, bool pair, int *bn_out,
                          int *splits_out) {
  // scheduling units: SMs with 128-row tiles, or CTA pairs with 256-row tiles
  const int tile_rows = pair ? 2 * BM : BM;
  if (pair) num_sms = num_sms / 2 > 0 ? num_sms / 2 : 1;
  const int tiles_m = ceil_div(Mc, tile_rows);
  double best = 1e300;
  int best_bn = 128, best_s = 1;
  const int cand[3] = {256, 128, 64};
  for (int ci = 0; ci < 3; ++ci) {
    const int bn = cand[ci];
    if (pair && bn < 128) continue;         // each CTA of a pair holds bn / 2 >= 64 columns of B
    if (bn > 64 && bn / 2 >= Nc) continue;  // tile twice as wide as the matrix
    const int tiles = tiles_m * ceil_div(Nc, bn);
    const int smax = forced_splits > 0 ? forced_splits : (kb_total < 32 ? kb_total : 32);
    const int smin = forced_splits > 0 ? forced_splits : 1;
    for (int s = smin; s <= smax; ++s) {
      if (s > kb_total) break;
      const int per = ceil_div(kb_total, s);
      if (forced_splits == 0 && s > 1 && (s - 1) * per >= kb_total) continue;  // an empty split
      const double waves = (double)ceil_div(tiles * s, num_sms);
      // + 6 k-blocks of fixed per-tile overhead (pipeline fill, epilogue); splits pay an extra pass over the
      // output (two k-blocks' worth since the partials go out as reduce-adds of the copy engine; measured on the
      // qkv weight gradient at M = 16384: 8 splits 153 us, 5 splits 163 us)
      const double cost = waves * (per + 6.0 + (s > 1 ? 2.0 : 0.0)) * (double)(tile_rows + bn);
      if (cost < best - 1e-9) {
        best = cost;
        best_bn = bn;
        best_s = s;
      }
    }
  }
  *bn_out = best_bn;
  *splits_out = best_s;
}

// Host-only part of build_op: shapes, majorness, tiling, descriptor bits. No CUDA calls.
int plan_op(const GemmDesc &d, int num_sms, GemmOp *op) {
  memset(op, 0, sizeof(*op));
  if (d.M <= 0 || d.K <= 0 || d.N <= 0) return GPT2L_ERR_BAD_ARG;
  switch (d.kind) {
    case GPT2L_OP_FORWARD:  // out[M][N] = in[M][K] . w[K][N]
      op->Mc = d.M; op->Nc = d.N; op->Kc = d.K; op->a_mn = 0; op->b_mn = 1;
      op->bias = d.bias;
      break;
    case GPT2L_OP_BACKWARD_INPUT:  // g_in[M][K] = g_out[M][N] . w[K][N]^T
      op->Mc = d.M; op->Nc = d.K; op->Kc = d.N; op->a_mn = 0; op->b_mn = 0;
      break;
    case GPT2L_OP_BACKWARD_WEIGHT:  // g_w[K][N] = in[M][K]^T . g_out[M][N]
      op->Mc = d.K; op->Nc = d.N; op->Kc = d.M; op->a_mn = 1; op->b_mn = 1;
      op->colsum = d.out_bias;
      op->colsum_spread = d.out_bias ? 1 : 0;
      op->cs_src = d.b;
      break;
    default:
      return GPT2L_ERR_BAD_ARG;
  }
  if (d.opts.mode != GPT2L_MODE_TF32 && d.opts.mode != GPT2L_MODE_TF32X3) return GPT2L_ERR_BAD_ARG;
  if (d.opts.split_k < 0 || d.opts.cta_pair < 0 || d.opts.cta_pair > 2) return GPT2L_ERR_BAD_ARG;
  op->C = d.out;
  op->ldc = op->Nc;
  op->mode = d.opts.mode;
  op->flags = (d.kind == GPT2L_OP_FORWARD) ? d.opts.flags : 0u;
  op->C2 = (op->flags & GPT2L_EPI_GELU_DUAL) ? d.opts.out2 : nullptr;
  if ((op->flags & GPT2L_EPI_GELU_DUAL) && !op->C2) return GPT2L_ERR_BAD_ARG;
  // epilogue operand: a product with gelu' cannot be applied to partial sums, and the fixed-order
  // combine does not carry it, so those cases run unsplit
  op->aux = d.opts.aux_op ? d.opts.aux : nullptr;
  op->aux_op = op->aux ? d.opts.aux_op : 0;
  op->aux_row = nullptr;
  op->aux_scale = 1.f;
  if (d.opts.aux_op && !d.opts.aux) return GPT2L_ERR_BAD_ARG;
  if (d.opts.aux_op < 0 || d.opts.aux_op > GPT2L_AUX_GELU_GRAD) return GPT2L_ERR_BAD_ARG;
  if (op->aux_op && d.kind == GPT2L_OP_BACKWARD_WEIGHT) return GPT2L_ERR_BAD_ARG;
  // softmax / cross-entropy around the lm_head: statistics in the forward epilogue, logits -> dlogits in
  // the operand transform of the two backward GEMMs (whichever form they are given in)
  if (d.xent_stats) {
    if (d.kind != GPT2L_OP_FORWARD || d.xent_vocab <= 0 || d.xent_vocab > d.N) return GPT2L_ERR_BAD_ARG;
    op->xent_mode = 1;
    op->xent_stats = d.xent_stats;
    op->xent_vocab = d.xent_vocab;
  } else if (d.opts.xent_lse) {
    if (!d.opts.xent_targets || d.opts.xent_vocab <= 0 || d.opts.aux_op) return GPT2L_ERR_BAD_ARG;
    // the logits are the reduction-side operand: A for backward_input, B for backward_weight and for its
    // forward form over a transposed activation copy
    op->xent_mode = d.kind == GPT2L_OP_BACKWARD_INPUT ? 2 : 3;
    op->xent_lse = d.opts.xent_lse;
    op->xent_tgt = d.opts.xent_targets;
    op->xent_vocab = d.opts.xent_vocab;
    op->xent_scale = d.opts.xent_scale;
  }
  op->kb_total = ceil_div(op->Kc, BK);
  int bn, splits;
  int forced = d.opts.split_k;
  if (op->xent_mode == 1) forced = 1;  // statistics of partial sums would be meaningless
  if (op->aux_op == GPT2L_AUX_GELU_GRAD || (op->aux_op && d.opts.deterministic) || (op->aux_op && op->C2)) forced = 1;
  if (forced > op->kb_total) forced = op->kb_total;
  // CTA pairs (256-row tiles, B split between the two CTAs) cut operand traffic per flop by a third; whether
  // that pays depends on the shape, so the choice is the caller's (the public entry points pick for cta_pair = 0)
  op->pair = (d.opts.cta_pair == 2) ? 1 : 0;
  choose_tiling(op->Mc, op->Nc, op->kb_total, num_sms > 0 ? num_sms : 148, forced, op->pair != 0, &bn, &splits);
  op->bn = bn;
  op->kb_per_split = ceil_div(op->kb_total, splits);
  op->splits = ceil_div(op->kb_total, op->kb_per_split);  // no empty trailing split
  op->tiles_m = ceil_div(op->Mc, BM);
  op->tiles_n = ceil_div(op->Nc, bn);
  op->tiles_dec = op->pair ? ceil_div(op->tiles_m, 2) : op->tiles_m;
  op->n_tiles = op->tiles_dec * op->tiles_n * op->splits;
  {
    // band height: as many tile rows as keep the band's A rows (of one split) within ~48 MB of L2
    const double a_bytes_per_tile_row = (double)(op->pair ? 2 * BM : BM) * (double)op->kb_per_split * BK * 4.0;
    int g = (int)(48.0 * 1024 * 1024 / a_bytes_per_tile_row);
    if (g < 1) g = 1;
    if (g > op->tiles_dec) g = op->tiles_dec;
    const int bands = ceil_div(op->tiles_dec, g);
    op->band_m = ceil_div(op->tiles_dec, bands);  // balanced bands
    // A B operand that stays in L2 anyway (the layers' weights: 2 - 9 MB) needs no bands: its tiles are walked
    // one tile row after the other, so that row blocks complete in order from the first wave on. Inside a
    // schedule a consumer's first tiles then find their row blocks done long before the producer's last wave;
    // with the row index fastest a row block is complete only when nearly the whole op is.
    static const int env_rows = [] { const char *e = getenv("GPT2L_ROW_MAJOR_TILES"); return e ? atoi(e) : 1; }();
    if (env_rows && op->splits == 1 && (double)op->Kc * (double)op->Nc * 4.0 <= 24.0 * 1024 * 1024) op->band_m = 1;
  }
  op->atomic_out = (op->splits > 1 && !d.opts.deterministic && !op->C2) ? 1 : 0;
  op->xent_stride = 2 * op->tiles_n;
  {
    // (GPT2L_EPI_TMA=0 keeps the boxes on the load/store path: read back and stored by the warps themselves)
    static const int env_tma = [] { const char *e = getenv("GPT2L_EPI_TMA"); return e ? atoi(e) : 1; }();
    op->epi_tma = env_tma;
  }
  if (op->xent_mode >= 2 && op->pair) return GPT2L_ERR_BAD_ARG;  // the pair kernel's transform warps only split
  op->idesc = make_idesc_tf32(op->pair ? 2 * BM : BM, bn, op->a_mn, op->b_mn);
  for (int w = 0; w < MAX_WAITS; ++w) { op->wait_ctr[w] = -1; op->wait_kind[w] = 0; op->wait_expected[w] = 0; }
  op->pub_rb_base = -1;
  op->pub_op_ctr = -1;
  return GPT2L_OK;
}

int build_op(const GemmDesc &d, int num_sms, GemmOp *op) {
  if (!d.out || !d.a || !d.b) return GPT2L_ERR_BAD_ARG;
  int e = plan_op(d, num_sms, op);
  if (e) return e;
  uint64_t a_inner, a_outer, b_inner, b_outer;
  switch (d.kind) {
    case GPT2L_OP_FORWARD: a_inner = d.K; a_outer = d.M; b_inner = d.N; b_outer = d.K; break;
    case GPT2L_OP_BACKWARD_INPUT: a_inner = d.N; a_outer = d.M; b_inner = d.N; b_outer = d.K; break;
    default: a_inner = d.K; a_outer = d.M; b_inner = d.N; b_outer = d.M; break;
  }
  op->a_3d = (op->a_mn && a_inner % 32 == 0) ? 1 : 0;
  op->b_3d = (op->b_mn && b_inner % 32 == 0) ? 1 : 0;
  if (op->a_3d) e = encode_map_chunked(&op->tmA, d.a, a_inner, a_outer, BM / 32);
  else e = encode_map(&op->tmA, d.a, a_inner, a_outer, 32, op->a_mn ? 32 : BM, op->a_mn);
  if (e) return e;
  const int bn_cta = op->pair ? op->bn / 2 : op->bn;  // B columns one CTA stages
  if (op->b_3d) e = encode_map_chunked(&op->tmB, d.b, b_inner, b_outer, bn_cta / 32);
  else e = encode_map(&op->tmB, d.b, b_inner, b_outer, 32, op->b_mn ? 32 : bn_cta, op->b_mn);
  if (e) return e;
  e = encode_map(&op->tmC, op->C, (uint64_t)op->Nc, (uint64_t)op->Mc, 32, 32, false);
  if (e) return e;
  if (op->C2) e = encode_map(&op->tmC2, op->C2, (uint64_t)op->Nc, (uint64_t)op->Mc, 32, 32, false);
  return e;
}

// K-major batched operand: [outer][inner][rows][red] -> dims {red, rows, inner batches, outer batches}
int encode_map_batched_k(CUtensorMap *map, const float *base, uint64_t red, uint64_t rows, uint64_t ld,
                                uint64_t nb_inner, uint64_t bs_inner, uint64_t nb_outer, uint64_t bs_outer,
                                uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return GPT2L_ERR_CUDA;
  cuuint64_t dims[4] = {red, rows, nb_inner, nb_outer};
  cuuint64_t strides[3] = {ld * 4, (bs_inner ? bs_inner : rows * ld) * 4, (bs_outer ? bs_outer : rows * ld) * 4};
  cuuint32_t box[4] = {32, box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? GPT2L_OK : GPT2L_ERR_CUDA;
}
// MN-major batched operand stored [red rows][mn] (mn a multiple of 32), viewed in 32-column chunks:
// dims {32, red rows, mn / 32, inner batches, outer batches}
int encode_map_batched_mn(CUtensorMap *map, const float *base, uint64_t mn, uint64_t red_rows, uint64_t ld,
                                 uint64_t nb_inner, uint64_t bs_inner, uint64_t nb_outer, uint64_t bs_outer,
                                 uint32_t chunks) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return GPT2L_ERR_CUDA;
  cuuint64_t dims[5] = {32, red_rows, mn / 32, nb_inner, nb_outer};
  cuuint64_t strides[4] = {ld * 4, 128, (bs_inner ? bs_inner : red_rows * ld) * 4,
                           (bs_outer ? bs_outer : red_rows * ld) * 4};
  cuuint32_t box[5] = {32, 32, chunks, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? GPT2L_OK : GPT2L_ERR_CUDA;
}

int build_batched_op(const BatchedDesc &d, int num_sms, GemmOp *op) {
  (void)num_sms;
  memset(op, 0, sizeof(*op));
  if (d.Mc <= 0 || d.Nc <= 0 || d.Kc <= 0 || !d.a || !d.b || !d.c || d.batch_outer <= 0 || d.batch_inner <= 0)
    return GPT2L_ERR_BAD_ARG;
  if ((d.lda & 3) || (d.ldb & 3) || (d.ldc & 3) || !aligned16(d.a) || !aligned16(d.b) || !aligned16(d.c))
    return GPT2L_ERR_BAD_ARG;
  if ((d.a_mn && (d.Mc & 31)) || (d.b_mn && (d.Nc & 31))) return GPT2L_ERR_BAD_ARG;
  op->Mc = d.Mc; op->Nc = d.Nc; op->Kc = d.Kc;
  op->a_mn = d.a_mn; op->b_mn = d.b_mn;
  op->C = d.c;
  op->ldc = d.ldc;
  op->mode = d.mode;
  op->kb_total = ceil_div(d.Kc, BK);
  op->bn = d.Nc <= 64 ? 64 : (d.Nc <= 128 ? 128 : 256);
  op->splits = 1;
  op->kb_per_split = op->kb_total;
  op->tiles_m = ceil_div(d.Mc, BM);
  op->tiles_n = ceil_div(d.Nc, op->bn);
  op->tiles_dec = op->tiles_m;
  op->band_m = op->tiles_m;
  op->batch = d.batch_outer * d.batch_inner;
  op->batch_inner = d.batch_inner;
  op->tiles_per_batch = op->tiles_m * op->tiles_n;
  op->n_tiles = op->batch * op->tiles_per_batch;
  op->c_bs_outer = d.c_bs_outer;
  op->c_bs_inner = d.c_bs_inner;
  op->causal = d.causal;
  op->aux = d.aux_op ? d.aux : nullptr;
  op->aux_op = op->aux ? d.aux_op : 0;
  op->aux_row = d.aux_row;
  op->aux_scale = d.aux_scale;
  if (op->aux_op == AUX_SOFTMAX_GRAD && !op->aux_row) return GPT2L_ERR_BAD_ARG;
  op->idesc = make_idesc_tf32(BM, op->bn, op->a_mn, op->b_mn);
  for (int w = 0; w < MAX_WAITS; ++w) op->wait_ctr[w] = -1;
  op->pub_rb_base = -1;
  op->pub_op_ctr = -1;
  if (op->batch < 2) op->batch = 2;  // the batched load path is keyed on batch > 1
  int e;
  if (!d.a_mn)
    e = encode_map_batched_k(&op->tmA, d.a, d.Kc, d.Mc, d.lda, d.batch_inner, d.a_bs_inner, d.batch_outer,
                             d.a_bs_outer, BM);
  else
    e = encode_map_batched_mn(&op->tmA, d.a, d.Mc, d.Kc, d.lda, d.batch_inner, d.a_bs_inner, d.batch_outer,
                              d.a_bs_outer, BM / 32);
  if (e) return e;
  if (!d.b_mn)
    e = encode_map_batched_k(&op->tmB, d.b, d.Kc, d.Nc, d.ldb, d.batch_inner, d.b_bs_inner, d.batch_outer,
                             d.b_bs_outer, op->bn);
  else
    e = encode_map_batched_mn(&op->tmB, d.b, d.Nc, d.Kc, d.ldb, d.batch_inner, d.b_bs_inner, d.batch_outer,
                              d.b_bs_outer, op->bn / 32);
  return e;
}

size_t xent_stats_floats(const GemmOp &op) { return (size_t)op.Mc * op.xent_stride * 2; }

size_t op_workspace_bytes(const GemmOp &op) {
  if (op.splits <= 1 || op.atomic_out) return 0;
  return (size_t)op.tiles_m * op.tiles_n * op.splits * BM * op.bn * sizeof(float);
}

int set_kernel_attributes() {
  cudaError_t e = cudaFuncSetAttribute(gpt2_linear_tcgen05_kernel<false, false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return GPT2L_ERR_CUDA;
  e = cudaFuncSetAttribute(gpt2_linear_tcgen05_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           SMEM_BYTES);
  if (e != cudaSuccess) return GPT2L_ERR_CUDA;
  e = cudaFuncSetAttribute(gpt2_linear_tcgen05_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           SMEM_BYTES);
  if (e != cudaSuccess) return GPT2L_ERR_CUDA;
  e = cudaFuncSetAttribute(gpt2_linear_tcgen05_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           SMEM_BYTES);
  return e == cudaSuccess ? GPT2L_OK : GPT2L_ERR_CUDA;
}

static long long default_wait_limit_ns() { return 4000000000ll; }  // 4 s

int launch_single(DeviceCtx *ctx, GemmOp &op, cudaStream_t stream) {
  op.tile_base = 0;
  op.op_index = 0;
  LaunchParams p;
  p.ops = nullptr;
  p.n_ops = 1;
  p.total_tiles = op.n_tiles;
  p.status = ctx->d_status;
  p.sticky = ctx->sticky;
  p.host_flag = ctx->d_flag;
  p.counters = nullptr;
  p.fmaps = nullptr;
  p.prof = nullptr;
  for (float &f : p.adam) f = 0.f;
  p.wait_limit_ns = default_wait_limit_ns();
  // (a TF32 bias gradient summed beside the ring needs no transform warps: the helpers do it, see the kernel)
  p.xform_active = (op.mode == GPT2L_MODE_TF32X3 || (op.colsum != nullptr && !op.colsum_spread) || op.xent_mode >= 2) ? 1 : 0;
  if (op.pair) {
    const int pairs = op.n_tiles < ctx->max_pairs ? op.n_tiles : ctx->max_pairs;
    if (pairs <= 0) return GPT2L_ERR_CUDA;
    return pair_launch(&op, p, pairs, op.mode == GPT2L_MODE_TF32X3, stream);
  }
  const int grid = op.n_tiles < ctx->num_sms ? op.n_tiles : ctx->num_sms;
  if (op.mode == GPT2L_MODE_TF32X3)
    gpt2_linear_tcgen05_kernel<true, false><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(op, p);
  else
    gpt2_linear_tcgen05_kernel<false, false><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(op, p);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? GPT2L_OK : GPT2L_ERR_CUDA;
}

// One launch over a device array of ops. GEMM-only lists on CTA pairs keep the pair kernel; everything
// else runs the step kernel (per-op transform decision, row-local ops, STEP_THREADS threads).
int launch_list(DeviceCtx *ctx, const GemmOp *d_ops, int n_ops, int total_tiles, int grid, bool any_3x, bool any_colsum,
                bool pair, Status *d_status, unsigned *d_counters, long long wait_limit_ns, const float *adam,
                const FlashMaps *fmaps, unsigned long long *prof, cudaStream_t stream) {
  static GemmOp dummy;  // the by-value slot is unused when a list is given
  LaunchParams p;
  p.ops = d_ops;
  p.n_ops = n_ops;
  p.total_tiles = total_tiles;
  p.status = d_status;
  p.sticky = nullptr;
  p.host_flag = ctx ? ctx->d_flag : nullptr;
  p.counters = d_counters;
  p.wait_limit_ns = wait_limit_ns > 0 ? wait_limit_ns : default_wait_limit_ns();
  p.xform_active = any_3x ? 1 : 0;  // (read by the pair kernel only; TF32 column sums are read beside the ring)
  (void)any_colsum;
  for (int i = 0; i < 7; ++i) p.adam[i] = adam ? adam[i] : 0.f;
  p.fmaps = fmaps;
  p.prof = prof;
  if (pair) return pair_launch(nullptr, p, grid, any_3x, stream);
  if (any_3x)
    gpt2_linear_tcgen05_kernel<true, true><<<grid, STEP_THREADS, SMEM_BYTES, stream>>>(dummy, p);
  else
    gpt2_linear_tcgen05_kernel<false, true><<<grid, STEP_THREADS, SMEM_BYTES, stream>>>(dummy, p);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? GPT2L_OK : GPT2L_ERR_CUDA;
}

}  // namespace g2l
