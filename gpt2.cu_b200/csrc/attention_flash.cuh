// Device side of the fused causal attention (see attention_flash.cu for the algorithm): configuration,
// the per-tile body shared by the stand-alone kernels and the step kernel, and the stand-alone kernel.
#pragma once

#include <cuda_runtime.h>
#include <math.h>

#include "linear_internal.h"
#include "ptx_sm100.cuh"

namespace g2l {

using namespace ptx;

namespace flash {

constexpr int FHS = 64;        // head size
constexpr int FROWS = 128;     // rows per CTA (TMEM lanes)

enum { F_FWD = 0, F_BWD_Q = 1, F_BWD_KV = 2 };

constexpr int TILE_A = FROWS * FHS * 4;   // 32 KiB: [128][64] K-major, two 16 KiB k-blocks

enum { X_Q = 0, X_K = 1, X_V = 2, X_DO = 3 };

struct FlashArgs {
  int B, T, C, NH;
  float *out;          // FWD: [B*T][C]
  float *lse;          // [B][NH][T], base-2 log-sum-exp of the scaled scores
  const float *delta;  // [B][NH][T]
  float *dqkv;         // BWD: [B*T][3C]
  int *status;         // 0, or the site of a wait that gave up
  long long wait_limit_ns;
  // inside the step kernel: the launch's own abort flag and status record (null in the stand-alone kernels)
  int *cta_abort;
  Status *step_status;
  int *host_flag;
  int op_index;
};

struct FlashCtrl {
  unsigned long long fixed_full, sc_full[2], sc_empty[2], ac_full[2], ac_empty[2], s_full[3], p_ready[3], slot_free[3], acc_done[2];
  uint32_t tmem_base;
  int abort;
};

template <int MODE>
struct Cfg {
  static constexpr int FC = 64;                         // columns per step
  static constexpr int NA = MODE == F_FWD ? 1 : 2;      // fixed A tiles; also score MMAs per step
  static constexpr int NP = MODE == F_BWD_KV ? 2 : 1;   // accumulators (and A tiles written back per step)
  // BWD_Q trades its double buffers for a second resident CTA per SM (two CTAs overlap each other's MMA
  // latency, which is what bounds these kernels): one operand stage, one score slot, 113 KiB, 256 TMEM columns
  static constexpr int NST = MODE == F_BWD_Q ? 1 : 2;   // operand stages
  static constexpr int NSB = MODE == F_BWD_Q ? 1 : 3;   // score slots in TMEM
  // sets of four row-work warps; the backward modes split a step's columns between two sets
  static constexpr int NCW = MODE == F_BWD_KV ? 2 : 1;
  static constexpr int MINB = MODE == F_BWD_KV ? 1 : 2;  // CTAs per SM
  static constexpr int NMW = MODE == F_BWD_KV ? 2 : 1;  // MMA-issuing warps
  static constexpr int THREADS = 32 * (1 + NMW) + 128 * NCW;  // producer, MMA issuers, row-work warps
  static constexpr int TILE_B = FC * FHS * 4;           // [FC][64] K-major (two k-blocks) or MN-major (FC/32 k-blocks)
  static constexpr int OFF_A = 0;
  static constexpr int OFF_SB = OFF_A + NA * TILE_A;          // score-stage B operands (K-major)
  static constexpr int OFF_AB = OFF_SB + NST * NA * TILE_B;   // accumulate-stage B operands (MN-major)
  static constexpr int OFF_VEC = OFF_AB + NST * NP * TILE_B;  // BWD_KV: lse and delta of the step's queries
  static constexpr int OFF_CTRL = OFF_VEC + (MODE == F_BWD_KV ? 8 * 2 * 64 * 4 : 0);  // per row-work warp, two buffers of 64 floats
  // the control block (barriers) sits in whichever end of the allocation the 1024-byte alignment of the
  // tiles leaves free, so the request is tiles + 1024 bytes and not a byte more
  static constexpr int CTRL_BYTES = 256;
  static constexpr int SMEM = 1024 + OFF_CTRL;
  // TMEM columns: NSB score slots of NA x FC columns, then the accumulators (NP x 64)
  static constexpr int COL_ACC = NSB * NA * FC;
  static constexpr int TMEM_COLS = COL_ACC + NP * FHS <= 256 ? 256 : 512;
};

__device__ __forceinline__ bool f_wait(uint32_t bar, uint32_t parity, FlashCtrl *ctrl, const FlashArgs &a, int site) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0) {
      if (*reinterpret_cast<volatile int *>(&ctrl->abort)) return false;
      if (a.cta_abort && *reinterpret_cast<volatile int *>(a.cta_abort)) {
        *reinterpret_cast<volatile int *>(&ctrl->abort) = 1;
        return false;
      }
      if (globaltimer_ns() - t0 > a.wait_limit_ns) {
        *reinterpret_cast<volatile int *>(&ctrl->abort) = 1;
        if (a.status) atomicCAS(a.status, 0, site);
        if (a.cta_abort) *reinterpret_cast<volatile int *>(a.cta_abort) = 1;
        if (a.step_status && atomicCAS(&a.step_status->status, 0, GPT2L_DEV_TIMEOUT) == 0) {
          a.step_status->op = a.op_index;
          a.step_status->counter = site;
          a.step_status->seen = -1;
          a.step_status->expected = (int)parity;
          a.step_status->where = SITE_ATTENTION + site;
          __threadfence();
          if (a.host_flag) {
            *reinterpret_cast<volatile int *>(a.host_flag) = GPT2L_DEV_TIMEOUT;
            __threadfence_system();
          }
        }
        return false;
      }
    }
  }
}

// Row-work warps wait as a warp: lane 0 polls and every lane takes its verdict, so a wait that
// gives up can never split a warp (or leave part of it behind at a later warp-level sync).
__device__ __forceinline__ bool w_wait(uint32_t bar, uint32_t parity, FlashCtrl *ctrl, const FlashArgs &a, int site,
                                       int lane) {
  int okl = 1;
  if (lane == 0) okl = f_wait(bar, parity, ctrl, a, site) ? 1 : 0;
  return __shfl_sync(0xffffffffu, okl, 0) != 0;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float f_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// N consecutive TMEM columns of this thread's lane, written back (the A tile of the accumulate MMAs)
template <int N>
__device__ __forceinline__ void store_cols(uint32_t taddr, const float (&v)[N]) {
#pragma unroll
  for (int hf = 0; hf < N / 32; ++hf) {
    uint32_t r[32];
#pragma unroll
    for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(v[hf * 32 + c]);
    tmem_st_32x32(taddr + hf * 32, r);
  }
}

// FC consecutive TMEM columns of this thread's lane (all loads in flight before the one wait)
template <int FC>
__device__ __forceinline__ void load_cols(uint32_t taddr, float (&v)[FC]) {
  uint32_t r[FC / 32][32];
#pragma unroll
  for (int hf = 0; hf < FC / 32; ++hf) tmem_ld_32x32(taddr + hf * 32, r[hf]);
  tmem_ld_wait();
#pragma unroll
  for (int hf = 0; hf < FC / 32; ++hf)
#pragma unroll
    for (int c = 0; c < 32; ++c) v[hf * 32 + c] = __uint_as_float(r[hf][c]);
}

// two column ranges (score and its partner), one wait
template <int FC>
__device__ __forceinline__ void load_cols2(uint32_t t0, uint32_t t1, float (&v0)[FC], float (&v1)[FC]) {
  uint32_t r0[FC / 32][32], r1[FC / 32][32];
#pragma unroll
  for (int hf = 0; hf < FC / 32; ++hf) {
    tmem_ld_32x32(t0 + hf * 32, r0[hf]);
    tmem_ld_32x32(t1 + hf * 32, r1[hf]);
  }
  tmem_ld_wait();
#pragma unroll
  for (int hf = 0; hf < FC / 32; ++hf)
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      v0[hf * 32 + c] = __uint_as_float(r0[hf][c]);
      v1[hf * 32 + c] = __uint_as_float(r1[hf][c]);
    }
}

// One tile — 128 rows of one (sequence, head) — from the first operand load to the last store, for every warp
// of the CTA: warp 0 loads, warps 1..NMW issue the MMAs, the next 4 * NCW warps do the row work, any further
// warp has nothing to do. Barriers and tensor memory exist already. The stand-alone kernels run one tile per
// CTA (g0 = tcnt = 0); the step kernel runs many through the same barriers, so steps (g0 = steps this CTA
// has run in this mode before) and tiles (tcnt) are numbered through and every parity follows from them.
template <int MODE>
__device__ __forceinline__ void attn_tile_body(const FlashMaps &maps, const FlashArgs &a, uint8_t *base_ptr,
                                               uint32_t base, FlashCtrl *ctrl, uint32_t tmem, int warp, int lane,
                                               int rb, int bh, uint32_t g0, uint32_t tcnt) {
  using K = Cfg<MODE>;
  constexpr int FC = K::FC;
  constexpr int TILE_B = K::TILE_B;
  float *vec = reinterpret_cast<float *>(base_ptr + K::OFF_VEC);
  const int b = bh / a.NH, h = bh % a.NH;
  const int row0 = rb * FROWS;
  // column blocks [cb0, cb1)
  const int cb0 = MODE == F_BWD_KV ? row0 / FC : 0;
  const int cb1 = MODE == F_BWD_KV ? a.T / FC : (row0 + FROWS) / FC;
  const int n_it = cb1 - cb0;

  // which tensors play which part
  //              fixed A0, A1        score B0, B1      accumulate B (MN-major) 0, 1
  //   FWD        Q                   K                 V
  //   BWD_Q      Q, dO               K, V              K
  //   BWD_KV     K, V                Q, dO             dO (with P^T), Q (with dS^T)
  constexpr int A0 = MODE == F_BWD_KV ? X_K : X_Q;
  constexpr int A1 = MODE == F_BWD_KV ? X_V : X_DO;
  constexpr int SB0 = MODE == F_BWD_KV ? X_Q : X_K;
  constexpr int SB1 = MODE == F_BWD_KV ? X_DO : X_V;
  constexpr int AB0 = MODE == F_FWD ? X_V : (MODE == F_BWD_Q ? X_K : X_DO);
  constexpr int AB1 = X_Q;

  if (warp == 0) {
    // =============================== TMA producer ===============================
    if (lane == 0) {
      const uint32_t bar = smem_u32(&ctrl->fixed_full);
      mbar_arrive_expect_tx(bar, K::NA * TILE_A);  // (waited for with the parity of the tile count)
#pragma unroll
      for (int x = 0; x < K::NA; ++x) {
        const CUtensorMap *m = &maps.k_major[x == 0 ? A0 : A1];
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int piece = 0; piece < FROWS / FC; ++piece)
            tma_load_4d(base + K::OFF_A + x * TILE_A + kb * 16384 + piece * FC * 128, m, bar, kb * 32, row0 + piece * FC,
                        h, b);
      }
      bool ok = true;
      for (int it = 0; it < n_it && ok; ++it) {
        const int c0 = (cb0 + it) * FC;
        const uint32_t G = g0 + (uint32_t)it;  // steps are numbered through all tiles this CTA has run in this mode
        const int st = (int)(G % K::NST);
        const uint32_t par = (G / K::NST) & 1u;
        ok = f_wait(smem_u32(&ctrl->sc_empty[st]), par ^ 1u, ctrl, a, 1);
        if (!ok) break;
        {
          const uint32_t sb = smem_u32(&ctrl->sc_full[st]);
          mbar_arrive_expect_tx(sb, K::NA * TILE_B);
#pragma unroll
          for (int x = 0; x < K::NA; ++x) {
            const CUtensorMap *m = &maps.k_major[x == 0 ? SB0 : SB1];
#pragma unroll
            for (int kb = 0; kb < 2; ++kb)
              tma_load_4d(base + K::OFF_SB + (st * K::NA + x) * TILE_B + kb * FC * 128, m, sb, kb * 32, c0, h, b);
          }
        }
        ok = f_wait(smem_u32(&ctrl->ac_empty[st]), par ^ 1u, ctrl, a, 2);
        if (!ok) break;
        {
          const uint32_t ab = smem_u32(&ctrl->ac_full[st]);
          mbar_arrive_expect_tx(ab, K::NP * TILE_B);
#pragma unroll
          for (int y = 0; y < K::NP; ++y) {
            const CUtensorMap *m = &maps.mn_major[y == 0 ? AB0 : AB1];
#pragma unroll
            for (int kb = 0; kb < FC / 32; ++kb)
              tma_load_5d(base + K::OFF_AB + (st * K::NP + y) * TILE_B + kb * 8192, m, ab, 0, c0 + kb * 32, 0, h, b);
          }
        }
      }
    }
  } else if (warp <= K::NMW) {
    // =============================== MMA issuers ===============================
    // One thread issuing all of a step's 16-32 small MMAs needs ~35-45 ns per instruction (measured
    // with %globaltimer) and was what the row work waited for, so the backward modes use two issuing
    // warps: warp 1 the score products, warp 2 the accumulate products. FWD (16 MMAs per step, two CTAs
    // per SM, register-bound) keeps both in warp 1.
    if (lane == 0) {
      const uint64_t hiK = smem_desc_hi(16, 1024, 2);     // K-major, 128-byte swizzle
      const uint64_t hiMN = smem_desc_hi(4096, 512, 1);   // MN-major, 32-byte swizzle atoms
      const uint32_t idesc_sc = make_idesc_tf32(FROWS, FC, 0, 0);
      const uint32_t idesc_ac = make_idesc_tf32(FROWS, FHS, 0, 1);
      // score MMAs of step k into TMEM slot k % NSB
      auto issue_score = [&](int k_local) -> bool {
        const uint32_t k = g0 + (uint32_t)k_local;
        const int st = (int)(k % K::NST);
        if (!f_wait(smem_u32(&ctrl->sc_full[st]), (k / K::NST) & 1u, ctrl, a, 4)) return false;
        if (k >= (uint32_t)K::NSB) {
          // the slot still holds the A tile of step k - NSB: its accumulate MMAs must have retired
          if (!f_wait(smem_u32(&ctrl->slot_free[k % K::NSB]), (k / K::NSB - 1) & 1u, ctrl, a, 16)) return false;
        }
        tc_fence_after();
#pragma unroll
        for (int x = 0; x < K::NA; ++x) {
          const uint32_t d = tmem + (uint32_t)((k % K::NSB) * K::NA + x) * FC;
          const uint32_t a_addr = base + K::OFF_A + x * TILE_A;
          const uint32_t b_addr = base + K::OFF_SB + (st * K::NA + x) * TILE_B;
#pragma unroll
          for (int kb = 0; kb < 2; ++kb)
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              mma_tf32(d, smem_desc(hiK, a_addr + kb * 16384 + ks * 32), smem_desc(hiK, b_addr + kb * FC * 128 + ks * 32),
                       idesc_sc, (kb | ks) ? 1u : 0u);
        }
        mma_commit(smem_u32(&ctrl->s_full[k % K::NSB]));
        mma_commit(smem_u32(&ctrl->sc_empty[st]));
        return true;
      };
      // accumulate MMAs of step it: A = the tile the row work wrote back into slot it % NSB
      auto issue_acc = [&](int it) -> bool {
        const uint32_t I = g0 + (uint32_t)it;
        if (!f_wait(smem_u32(&ctrl->p_ready[I % K::NSB]), (I / K::NSB) & 1u, ctrl, a, 5)) return false;
        const int st = (int)(I % K::NST);
        if (!f_wait(smem_u32(&ctrl->ac_full[st]), (I / K::NST) & 1u, ctrl, a, 6)) return false;
        tc_fence_after();
#pragma unroll
        for (int y = 0; y < K::NP; ++y) {
          const uint32_t d = tmem + K::COL_ACC + y * FHS;
          // the tile sits over S (FWD), over dP (BWD_Q), over S^T for dV and over dP^T for dK (BWD_KV)
          const int slot_x = MODE == F_FWD ? 0 : (MODE == F_BWD_Q ? 1 : y);
          const uint32_t a_tmem = tmem + (uint32_t)((I % K::NSB) * K::NA + slot_x) * FC;
          const uint32_t b_addr = base + K::OFF_AB + (st * K::NP + y) * TILE_B;
#pragma unroll
          for (int kb = 0; kb < FC / 32; ++kb)
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              // FWD reads every step's product on its own (the rescaling happens in registers)
              const uint32_t acc = (MODE == F_FWD ? 0u : (it > 0 ? 1u : 0u)) | ((kb | ks) ? 1u : 0u);
              mma_tf32_tmem_a(d, a_tmem + kb * 32 + ks * 8, smem_desc(hiMN, b_addr + kb * 8192 + ks * 1024), idesc_ac, acc);
            }
        }
        mma_commit(smem_u32(&ctrl->acc_done[I & 1u]));
        mma_commit(smem_u32(&ctrl->ac_empty[st]));
        mma_commit(smem_u32(&ctrl->slot_free[I % K::NSB]));
        return true;
      };
      bool ok = true;
      if (warp == 1) {
        ok = f_wait(smem_u32(&ctrl->fixed_full), tcnt & 1u, ctrl, a, 3);
        tc_fence_after();
      }
      if (K::NMW == 1 && K::NSB == 1) {
        // one slot: the scores of step it + 1 can only follow the accumulate MMAs of step it
        for (int it = 0; it < n_it && ok; ++it) {
          ok = issue_score(it);
          if (ok) ok = issue_acc(it);
        }
      } else if (K::NMW == 1) {
        if (ok && n_it > 0) ok = issue_score(0);
        for (int it = 0; it < n_it && ok; ++it) {
          if (it + 1 < n_it) ok = issue_score(it + 1);
          if (ok) ok = issue_acc(it);
        }
      } else if (warp == 1) {
        for (int k = 0; k < n_it && ok; ++k) ok = issue_score(k);
      } else {
        for (int it = 0; it < n_it && ok; ++it) ok = issue_acc(it);
      }
    }
  } else if (warp < 1 + K::NMW + 4 * K::NCW) {
    // =============================== row work ===============================
    const int q4 = warp & 3;                  // TMEM lane quarter of this warp
    const int cset = (warp - 1 - K::NMW) >> 2;  // which set of four row-work warps
    const int r = q4 * 32 + lane;             // row inside the block
    const int grow = row0 + r;                // position in the sequence
    const uint32_t tlane = tmem + ((uint32_t)(q4 * 32) << 16);
    const float cs = 0.125f * 1.4426950408889634f;  // 1/sqrt(64) * log2(e)
    const long long vbase = ((long long)b * a.NH + h) * a.T;
    bool ok = true;

    if (MODE == F_FWD) {
      float o[FHS];
#pragma unroll
      for (int c = 0; c < FHS; ++c) o[c] = 0.f;
      float m_run = -INFINITY, l_run = 0.f, alpha_prev = 0.f;
      for (int it = 0; it < n_it && ok; ++it) {
        ok = w_wait(smem_u32(&ctrl->s_full[(g0 + it) % K::NSB]), ((g0 + it) / K::NSB) & 1u, ctrl, a, 7, lane);
        if (!ok) break;
        tc_fence_after();
        float s[FC];
        const uint32_t slot = tlane + (uint32_t)(((g0 + it) % K::NSB) * K::NA) * FC;
        load_cols(slot, s);
        const int c0 = (cb0 + it) * FC;
        // raw scores: max first (scale > 0 commutes with max), then p = 2^(s * scale - max) in one FMA
        if (c0 + FC - 1 > row0) {  // the block reaches past the diagonal for some row: mask
#pragma unroll
          for (int c = 0; c < FC; ++c) s[c] = (c0 + c > grow) ? -INFINITY : s[c];
        }
        float mraw = -INFINITY;
#pragma unroll
        for (int c = 0; c < FC; ++c) mraw = fmaxf(mraw, s[c]);
        const float mx = fmaxf(m_run, mraw * cs);
        const float alpha = ex2(m_run - mx);  // first step: 2^(-inf) = 0; mx is finite from step 0 on (key 0 <= any query)
        float sum = 0.f;
#pragma unroll
        for (int c = 0; c < FC; ++c) {
          s[c] = f_tf32(ex2(fmaf(s[c], cs, -mx)));
          sum += s[c];
        }
        l_run = l_run * alpha + sum;
        m_run = mx;
        if (it > 0) {
          // the previous product is complete: fold it in (it was formed with the previous maximum),
          // and its operands in shared memory are free again
          ok = w_wait(smem_u32(&ctrl->acc_done[(g0 + it - 1) & 1u]), ((g0 + it - 1) >> 1) & 1u, ctrl, a, 8, lane);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            uint32_t pv[32];
            tmem_ld_32x32(tlane + K::COL_ACC + hf * 32, pv);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) o[hf * 32 + c] = o[hf * 32 + c] * alpha_prev + __uint_as_float(pv[c]);
          }
        }
        alpha_prev = alpha;
        store_cols(slot, s);  // P over S: the A tile of this step's P.V
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(smem_u32(&ctrl->p_ready[(g0 + it) % K::NSB]));
      }
      if (ok && n_it > 0) {
        ok = w_wait(smem_u32(&ctrl->acc_done[(g0 + n_it - 1) & 1u]), ((g0 + n_it - 1) >> 1) & 1u, ctrl, a, 9, lane);
        if (ok) {
          tc_fence_after();
          float pv[FHS];
          load_cols(tlane + K::COL_ACC, pv);
          const float inv = 1.f / l_run;
          float *dst = a.out + ((long long)b * a.T + grow) * a.C + h * FHS;
#pragma unroll
          for (int c = 0; c < FHS; c += 4)
            *reinterpret_cast<float4 *>(dst + c) =
                make_float4((o[c] * alpha_prev + pv[c]) * inv, (o[c + 1] * alpha_prev + pv[c + 1]) * inv,
                            (o[c + 2] * alpha_prev + pv[c + 2]) * inv, (o[c + 3] * alpha_prev + pv[c + 3]) * inv);
          a.lse[vbase + grow] = m_run + log2f(l_run);
        }
      }
    } else if (MODE == F_BWD_Q) {
      // NCW warp sets share the rows: set k handles columns [HC k, HC k + HC) of every step and of dQ at the end
      constexpr int HC = FC / K::NCW;
      const float lse = a.lse[vbase + grow];
      const float dlt8 = a.delta[vbase + grow] * 0.125f;
      for (int it = 0; it < n_it && ok; ++it) {
        ok = w_wait(smem_u32(&ctrl->s_full[(g0 + it) % K::NSB]), ((g0 + it) / K::NSB) & 1u, ctrl, a, 10, lane);
        if (!ok) break;
        tc_fence_after();
        float s[HC], dp[HC];
        const uint32_t slot = tlane + (uint32_t)(((g0 + it) % K::NSB) * K::NA) * FC + cset * HC;
        load_cols2(slot, slot + FC, s, dp);
        const int c0 = (cb0 + it) * FC + cset * HC;
        if (c0 + HC - 1 > row0) {  // the block reaches past the diagonal for some row: mask
#pragma unroll
          for (int c = 0; c < HC; ++c) {
            const float p = (c0 + c > grow) ? 0.f : ex2(fmaf(s[c], cs, -lse));
            s[c] = f_tf32(p * fmaf(dp[c], 0.125f, -dlt8));
          }
        } else {
#pragma unroll
          for (int c = 0; c < HC; ++c) s[c] = f_tf32(ex2(fmaf(s[c], cs, -lse)) * fmaf(dp[c], 0.125f, -dlt8));
        }
        store_cols(slot + FC, s);  // dS over dP: the A tile of this step's dS.K
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(smem_u32(&ctrl->p_ready[(g0 + it) % K::NSB]));
      }
      if (ok && n_it > 0) {
        ok = w_wait(smem_u32(&ctrl->acc_done[(g0 + n_it - 1) & 1u]), ((g0 + n_it - 1) >> 1) & 1u, ctrl, a, 12, lane);
        if (ok) {
          tc_fence_after();
          float dq[HC];
          load_cols(tlane + K::COL_ACC + cset * HC, dq);
          float *dst = a.dqkv + ((long long)b * a.T + grow) * 3 * a.C + h * FHS + cset * HC;
#pragma unroll
          for (int c = 0; c < HC; c += 4)
            *reinterpret_cast<float4 *>(dst + c) = make_float4(dq[c], dq[c + 1], dq[c + 2], dq[c + 3]);
        }
      }
    } else {
      constexpr int HC = FC / K::NCW;
      // lse and delta of the warp's 32 queries of a step are fetched one step ahead (their latency would
      // otherwise sit at the head of every step) and shared through a per-warp copy in shared memory,
      // double-buffered by step parity: only warp-level synchronisation is involved
      float nl = a.lse[vbase + cb0 * FC + cset * HC + lane];
      float nd = a.delta[vbase + cb0 * FC + cset * HC + lane];
      for (int it = 0; it < n_it && ok; ++it) {
        const int c0 = (cb0 + it) * FC + cset * HC;
        float *vv = vec + ((warp - 1 - K::NMW) * 2 + (it & 1)) * 64;
        vv[lane] = nl;
        vv[32 + lane] = nd * 0.125f;
        if (it + 1 < n_it) {
          nl = a.lse[vbase + c0 + FC + lane];
          nd = a.delta[vbase + c0 + FC + lane];
        }
        __syncwarp();
        ok = w_wait(smem_u32(&ctrl->s_full[(g0 + it) % K::NSB]), ((g0 + it) / K::NSB) & 1u, ctrl, a, 13, lane);
        if (!ok) break;
        tc_fence_after();
        float s[HC], dp[HC];
        const uint32_t slot = tlane + (uint32_t)(((g0 + it) % K::NSB) * K::NA) * FC + cset * HC;
        load_cols2(slot, slot + FC, s, dp);
        if (row0 + FROWS - 1 > c0) {  // some key of the block comes after some query of the step: mask
#pragma unroll
          for (int c = 0; c < HC; ++c) {
            const float p = (grow > c0 + c) ? 0.f : ex2(fmaf(s[c], cs, -vv[c]));
            s[c] = f_tf32(p);
            dp[c] = f_tf32(p * fmaf(dp[c], 0.125f, -vv[32 + c]));
          }
        } else {
#pragma unroll
          for (int c = 0; c < HC; ++c) {
            const float p = ex2(fmaf(s[c], cs, -vv[c]));
            s[c] = f_tf32(p);
            dp[c] = f_tf32(p * fmaf(dp[c], 0.125f, -vv[32 + c]));
          }
        }
        store_cols(slot, s);        // P^T over S^T: A tile of dV += P^T dO
        store_cols(slot + FC, dp);  // dS^T over dP^T: A tile of dK += dS^T Q
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(smem_u32(&ctrl->p_ready[(g0 + it) % K::NSB]));
      }
      if (ok && n_it > 0) {
        ok = w_wait(smem_u32(&ctrl->acc_done[(g0 + n_it - 1) & 1u]), ((g0 + n_it - 1) >> 1) & 1u, ctrl, a, 15, lane);
        if (ok) {
          tc_fence_after();
          // set 0 stores dV (accumulated with P^T), set 1 stores dK (with dS^T)
          float g[FHS];
          load_cols(tlane + K::COL_ACC + cset * FHS, g);
          float *dst = a.dqkv + ((long long)b * a.T + grow) * 3 * a.C + h * FHS + (cset == 0 ? 2 * a.C : a.C);
#pragma unroll
          for (int c = 0; c < FHS; c += 4)
            *reinterpret_cast<float4 *>(dst + c) = make_float4(g[c], g[c + 1], g[c + 2], g[c + 3]);
        }
      }
    }
  }

}

// column steps a tile of row block `rb` takes (what advances g0)
template <int MODE>
__host__ __device__ __forceinline__ int attn_tile_steps(int rb, int T) {
  constexpr int FC = Cfg<MODE>::FC;
  const int row0 = rb * FROWS;
  return MODE == F_BWD_KV ? T / FC - row0 / FC : (row0 + FROWS) / FC;
}

__device__ __forceinline__ void attn_init_barriers(FlashCtrl *ctrl, int ncw) {
  mbar_init(smem_u32(&ctrl->fixed_full), 1);
  for (int i = 0; i < 2; ++i) {
    mbar_init(smem_u32(&ctrl->sc_full[i]), 1);
    mbar_init(smem_u32(&ctrl->sc_empty[i]), 1);
    mbar_init(smem_u32(&ctrl->ac_full[i]), 1);
    mbar_init(smem_u32(&ctrl->ac_empty[i]), 1);
  }
  // one barrier per TMEM score slot for each hand-over (scores ready, tile written back, tile
  // consumed): with two independent MMA issuers a single barrier could run two phases ahead of a
  // waiter, which a parity wait cannot tell from zero
  for (int i = 0; i < 3; ++i) {
    mbar_init(smem_u32(&ctrl->s_full[i]), 1);
    mbar_init(smem_u32(&ctrl->p_ready[i]), 128 * ncw);
    mbar_init(smem_u32(&ctrl->slot_free[i]), 1);
  }
  mbar_init(smem_u32(&ctrl->acc_done[0]), 1);
  mbar_init(smem_u32(&ctrl->acc_done[1]), 1);
  ctrl->abort = 0;
}

template <int MODE>
__global__ void __launch_bounds__(Cfg<MODE>::THREADS, Cfg<MODE>::MINB)  // FWD: 97 KiB, 256 TMEM columns: two CTAs per SM
attn_flash_kernel(const __grid_constant__ FlashMaps maps, const FlashArgs a) {
  using K = Cfg<MODE>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - raw);
  FlashCtrl *ctrl = reinterpret_cast<FlashCtrl *>((base - raw) >= (uint32_t)K::CTRL_BYTES ? smem_raw
                                                                                          : base_ptr + K::OFF_CTRL);
  static_assert(sizeof(FlashCtrl) <= K::CTRL_BYTES, "control block");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_rb = a.T / FROWS;
  // heavy row blocks first: FWD / BWD_Q rows near the end of the sequence see the most keys,
  // BWD_KV rows near the start see the most queries
  const int bh_count = a.B * a.NH;
  const int order = blockIdx.x / bh_count;
  const int rb = MODE == F_BWD_KV ? order : n_rb - 1 - order;
  const int bh = blockIdx.x % bh_count;

  if (threadIdx.x == 0) {
    attn_init_barriers(ctrl, K::NCW);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), K::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t *>(&ctrl->tmem_base);

  attn_tile_body<MODE>(maps, a, base_ptr, base, ctrl, tmem, warp, lane, rb, bh, 0u, 0u);

  // =============================== teardown ===============================
  if (*reinterpret_cast<volatile int *>(&ctrl->abort)) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let copies and MMAs in flight land
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, K::TMEM_COLS);
  }
}

}  // namespace flash
}  // namespace g2l
