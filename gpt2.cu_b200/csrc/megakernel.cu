// Host side of the persistent multi-GEMM launch ("megakernel" path): turns a list of GEMM
// ops with dependencies into tile ranges, dependency counters and a device op array, checks
// the schedule by replaying it on the host, and launches the kernel once per run.
//
// Counter layout: op i owns tiles_m(i) row-block counters followed by one op-level counter.
// A finished tile publishes A arrivals to the row-block counter of its rows and A to the op counter
// (A = 8, the worker warps of a CTA; 4 in the CTA-pair kernel), so a complete row block of a GEMM shows
// A * tiles_n * splits arrivals and a complete op A * n_tiles.
#include <cuda_runtime.h>
#include <string.h>

#include <vector>

#include "linear_internal.h"
#include "schedule_internal.h"

namespace g2l {

static GemmDesc desc_from(const gpt2l_op &o) {
  GemmDesc d;
  d.kind = o.kind;
  d.M = (o.B > 0 && o.S > 0 && (long long)o.B * o.S <= 0x7fffffffll) ? o.B * o.S : 0;
  d.K = o.K;
  d.N = o.N;
  d.out = o.out;
  d.out_bias = o.out_bias;
  d.a = o.a;
  d.b = o.b;
  d.bias = o.bias;
  d.opts = o.opts;
  return d;
}

OpSpec spec_from(const gpt2l_op &o) {
  OpSpec s;
  s.kind = OPK_GEMM;
  s.gemm = desc_from(o);
  s.layer = o.layer;
  for (int w = 0; w < GPT2L_MAX_DEPS; ++w)
    if (o.deps[w].kind != GPT2L_DEP_NONE) s.deps.push_back({o.deps[w].producer, o.deps[w].kind});
  return s;
}

// Shapes, tiling, counters and dependency wiring. No CUDA calls (used by the CPU tests).
// Counter arrivals: in the step kernel every finished tile, of whatever op, counts NUM_WORKER_WARPS
// arrivals (a GEMM tile whose transform warps are busy has its four epilogue warps arrive twice); in the
// pair kernel the four epilogue warps of each CTA arrive once.
int make_plan(const std::vector<OpSpec> &specs, int num_sms, Plan *plan) {
  const int n_ops = (int)specs.size();
  if (n_ops <= 0) return GPT2L_ERR_BAD_ARG;
  plan->ops.resize(n_ops);
  int tile_base = 0, ctr = 0;
  // one kernel runs the whole list, so all ops use the same CTA arrangement: pairs only when
  // every op is a GEMM that asks for them (cta_pair == 2)
  bool pair = true;
  for (const auto &s : specs)
    if (s.kind != OPK_GEMM || s.gemm.opts.cta_pair != 2) pair = false;
  plan->pair = pair;
  for (int i = 0; i < n_ops; ++i) {
    const OpSpec &s = specs[i];
    GemmOp &g = plan->ops[i];
    if (s.kind == OPK_GEMM) {
      GemmDesc d = s.gemm;
      d.opts.cta_pair = pair ? 2 : 1;
      // bias gradient inside a schedule is always the fused column sum
      int e = plan_op(d, num_sms, &g);
      if (e) return e;
      if (g.mode != plan->ops[0].mode && plan->ops[0].op_kind == OPK_GEMM) return GPT2L_ERR_SCHEDULE;  // one mode per launch
      if (g.mode == GPT2L_MODE_TF32X3) plan->any_3x = true;
      if (g.colsum) plan->any_colsum = true;
      g.rows_per_tile = BM;
    } else {
      if (s.rows <= 0 || s.rows_per_tile <= 0) return GPT2L_ERR_BAD_ARG;
      memset(&g, 0, sizeof(g));
      g.op_kind = s.kind;
      g.ra = s.ra;
      g.rows_per_tile = s.rows_per_tile;
      g.rb_per_seq = s.rb_per_seq;
      if (s.kind == OPK_ADAMW) {
        g.tiles_m = 1;  // one counter block: consumers (none today) would wait for the whole op
        g.n_tiles = (int)((s.ra.n1 + (long long)s.rows_per_tile * 1024 - 1) / ((long long)s.rows_per_tile * 1024));
      } else if (s.kind >= OPK_ATTN_FWD && s.kind <= OPK_ATTN_BWD_Q) {
        // tile = (sequence * heads + head, 128-row block of the sequence); row blocks are numbered over all rows
        g.tiles_m = s.rows / BM;
        g.n_tiles = g.tiles_m * s.ra.i3;  // i3 = heads
      } else {
        // whole 128-row blocks: tiles past the last row do nothing but still count, so that every block
        // shows the same number of arrivals
        if (BM % s.rows_per_tile != 0) return GPT2L_ERR_BAD_ARG;
        g.tiles_m = (s.rows + BM - 1) / BM;
        g.n_tiles = g.tiles_m * (BM / s.rows_per_tile);
      }
      g.Mc = s.rows;
      g.tiles_n = 1;
      g.splits = 1;
      g.tiles_dec = g.tiles_m;
      for (int w = 0; w < MAX_WAITS; ++w) g.wait_ctr[w] = -1;
    }
    g.op_index = i;
    g.layer = s.layer;
    g.tile_base = tile_base;
    tile_base += g.n_tiles;
    g.pub_rb_base = ctr;
    g.pub_op_ctr = ctr + g.tiles_m;
    ctr += g.tiles_m + 1;
  }
  // transform warps: per op in the step kernel, per launch in the pair kernel
  for (auto &g : plan->ops)
    g.xform = (g.op_kind == OPK_GEMM && (plan->any_3x || (g.colsum != nullptr && g.b_mn && !g.colsum_spread) || g.xent_mode >= 2)) ? 1 : 0;
  plan->arrivals = plan->pair ? NUM_EPI_WARPS : NUM_WORKER_WARPS;
  const unsigned A = (unsigned)plan->arrivals;
  std::vector<char> waited_for(n_ops, 0);
  for (int i = 0; i < n_ops; ++i) {
    GemmOp &g = plan->ops[i];
    if ((int)specs[i].deps.size() > MAX_WAITS) return GPT2L_ERR_SCHEDULE;
    int w = 0;
    for (const auto &dep : specs[i].deps) {
      if (dep.kind == GPT2L_DEP_NONE) continue;
      if (dep.producer < 0 || dep.producer >= i) return GPT2L_ERR_SCHEDULE;  // must point backwards
      waited_for[dep.producer] = 1;
      const GemmOp &pr = plan->ops[dep.producer];
      // arrivals a complete 128-row block / the complete op shows
      unsigned per_block, whole;
      if (pr.op_kind == OPK_GEMM) {
        per_block = A * pr.tiles_n * pr.splits;
        whole = A * pr.tiles_m * pr.tiles_n * pr.splits;
      } else if (pr.op_kind >= OPK_ATTN_FWD && pr.op_kind <= OPK_ATTN_BWD_Q) {
        per_block = A * pr.ra.i3;
        whole = A * pr.n_tiles;
      } else if (pr.op_kind == OPK_ADAMW) {
        per_block = whole = A * pr.n_tiles;
      } else {
        per_block = A * (BM / pr.rows_per_tile);
        whole = A * pr.n_tiles;
      }
      if (dep.kind == GPT2L_DEP_ROWBLOCK || dep.kind == DEP_SEQUENCE) {
        // row block r of the consumer reads rows [128r, 128r+128) of the producer's output
        if (g.op_kind == OPK_GEMM && (pr.Mc != g.Mc || g.a_mn)) return GPT2L_ERR_SCHEDULE;
        if (pr.tiles_m != g.tiles_m && g.op_kind != OPK_ADAMW) return GPT2L_ERR_SCHEDULE;
        if (dep.kind == DEP_SEQUENCE && (g.rb_per_seq <= 0 || pr.tiles_m % g.rb_per_seq != 0)) return GPT2L_ERR_SCHEDULE;
        g.wait_ctr[w] = pr.pub_rb_base;
        g.wait_kind[w] = dep.kind;
        g.wait_expected[w] = (int)per_block;
        g.wait_op_ctr[w] = pr.pub_op_ctr;
        g.wait_op_expected[w] = (int)whole;
      } else if (dep.kind == GPT2L_DEP_WHOLE_OP) {
        g.wait_ctr[w] = pr.pub_op_ctr;
        g.wait_kind[w] = GPT2L_DEP_WHOLE_OP;
        g.wait_expected[w] = (int)whole;
        g.wait_op_ctr[w] = pr.pub_op_ctr;
        g.wait_op_expected[w] = (int)whole;
      } else {
        return GPT2L_ERR_SCHEDULE;
      }
      ++w;
    }
  }
  // an op nobody waits for publishes nothing: its tiles skip the fence, the wait for their stores to land and
  // the counter updates (the launch's end makes its results visible)
  for (int i = 0; i < n_ops; ++i)
    if (!waited_for[i]) plan->ops[i].pub_rb_base = plan->ops[i].pub_op_ctr = -1;
  plan->total_tiles = tile_base;
  plan->n_counters = ctr;
  return GPT2L_OK;
}

// 128-row blocks a tile of op g touches as a consumer / publishes as a producer
static void tile_blocks(const GemmOp &g, int local, bool pair, int *rb, int *n_rb) {
  if (g.op_kind == OPK_GEMM) {
    int m_dec, n_tile, split;
    decode_local(local, g.tiles_dec, g.tiles_n, g.band_m, m_dec, n_tile, split);
    *rb = pair ? 2 * m_dec : m_dec;
    *n_rb = pair ? ((2 * m_dec + 1 < g.tiles_m) ? 2 : 1) : 1;
  } else if (g.op_kind == OPK_ADAMW) {
    *rb = 0;
    *n_rb = 1;
  } else if (g.op_kind >= OPK_ATTN_FWD && g.op_kind <= OPK_ATTN_BWD_Q) {
    // tile order: see attention_tile_coords()
    const int per_seq = g.rb_per_seq, heads = g.ra.i3;
    const int seq = local / (per_seq * heads), i = (local % (per_seq * heads)) / heads;
    const int blk = g.op_kind == OPK_ATTN_BWD_KV ? i : per_seq - 1 - i;
    *rb = seq * per_seq + blk;
    *n_rb = 1;
  } else {
    *rb = (int)(((long long)local * g.rows_per_tile) / BM);
    *n_rb = 1;
  }
}

// Replays the schedule: CTA c owns tiles c, c+grid, ... and runs them in order; a tile may
// run when its counters have reached the expected values. Returns OK when every tile ran.
int replay(const Plan &plan, int grid) {
  if (grid <= 0) return GPT2L_ERR_BAD_ARG;
  std::vector<long long> counters(plan.n_counters, 0);
  std::vector<int> next(grid);
  for (int c = 0; c < grid; ++c) next[c] = c;
  int remaining = plan.total_tiles;
  std::vector<int> cursor(grid, 0);
  const int A = plan.arrivals;
  while (remaining > 0) {
    bool progress = false;
    for (int c = 0; c < grid; ++c) {
      while (next[c] < plan.total_tiles) {
        const int t = next[c];
        int &cur = cursor[c];
        while (cur + 1 < (int)plan.ops.size() && t >= plan.ops[cur].tile_base + plan.ops[cur].n_tiles) ++cur;
        const GemmOp &g = plan.ops[cur];
        int rb0, n_rb;
        tile_blocks(g, t - g.tile_base, plan.pair, &rb0, &n_rb);
        bool ready = true;
        for (int h = 0; h < n_rb; ++h) {
          const int rb = rb0 + h;
          for (int w = 0; w < MAX_WAITS; ++w) {
            if (g.wait_ctr[w] < 0) continue;
            int first = g.wait_ctr[w], count = 1;
            if (g.wait_kind[w] == GPT2L_DEP_ROWBLOCK) first += rb;
            else if (g.wait_kind[w] == DEP_SEQUENCE) { first += (rb / g.rb_per_seq) * g.rb_per_seq; count = g.rb_per_seq; }
            for (int i = 0; i < count; ++i) {
              if (first + i < 0 || first + i >= plan.n_counters) return GPT2L_ERR_SCHEDULE;
              if (counters[first + i] < g.wait_expected[w]) ready = false;
            }
          }
        }
        if (!ready) break;
        for (int h = 0; h < n_rb && g.pub_rb_base >= 0; ++h) {
          counters[g.pub_rb_base + rb0 + h] += A;
          counters[g.pub_op_ctr] += A;
        }
        next[c] += grid;
        --remaining;
        progress = true;
      }
    }
    if (!progress) return GPT2L_ERR_SCHEDULE;  // every CTA is blocked: the schedule would time out
  }
  return GPT2L_OK;
}

}  // namespace g2l

using namespace g2l;

namespace g2l {

gpt2l_schedule *schedule_build(const std::vector<OpSpec> &specs, int grid_limit, int *err) {
  int e = GPT2L_OK;
  DeviceCtx *ctx = ctx_current(&e);
  if (!ctx) { *err = e; return nullptr; }
  gpt2l_schedule *s = new gpt2l_schedule();
  s->ctx = ctx;
  s->specs = specs;
  e = make_plan(specs, ctx->num_sms, &s->plan);
  if (e) { *err = e; delete s; return nullptr; }
  const int n_ops = (int)specs.size();
  {
    int units = s->plan.pair ? ctx->max_pairs : ctx->num_sms;  // CTA pairs or CTAs
    if (grid_limit > 0 && grid_limit < units) units = grid_limit;
    s->grid = units < s->plan.total_tiles ? units : s->plan.total_tiles;
    if (s->grid <= 0) { *err = GPT2L_ERR_CUDA; delete s; return nullptr; }
  }
  e = replay(s->plan, s->grid);
  if (e) { *err = e; delete s; return nullptr; }
  // tensor maps + workspace
  size_t ws_bytes = 0, sem_count = 0;
  for (int i = 0; i < n_ops; ++i) {
    if (specs[i].kind != OPK_GEMM) continue;
    GemmDesc d = specs[i].gemm;
    d.opts.cta_pair = s->plan.pair ? 2 : 1;
    if (!d.out || !d.a || !d.b || !tma_eligible(d)) { *err = GPT2L_ERR_BAD_ARG; delete s; return nullptr; }
    GemmOp full;
    e = build_op(d, ctx->num_sms, &full);
    if (e) { *err = e; delete s; return nullptr; }
    GemmOp &g = s->plan.ops[i];
    g.tmA = full.tmA;
    g.tmB = full.tmB;
    g.tmC = full.tmC;
    g.tmC2 = full.tmC2;
    g.a_3d = full.a_3d;
    g.b_3d = full.b_3d;
    if (specs[i].transposed_a) {
      // the forward form of a weight gradient: the B operand is still g_out, its column sums are g_b
      g.colsum = specs[i].gemm.out_bias;
      g.colsum_spread = g.colsum ? 1 : 0;
      g.cs_src = specs[i].gemm.b;
      g.xform = (s->plan.any_3x || g.xent_mode >= 2) ? 1 : 0;  // (the column sums are read beside the ring)
    }
    ws_bytes += op_workspace_bytes(g);
    if (g.splits > 1 && !g.atomic_out) sem_count += (size_t)g.tiles_m * g.tiles_n * 4;
    // accumulated outputs start from zero at every launch
    if (g.splits > 1 && g.atomic_out) s->zero.push_back({g.C, (size_t)g.Mc * g.Nc * sizeof(float)});
    if (g.colsum && (g.splits > 1 || g.colsum_spread)) s->zero.push_back({g.colsum, (size_t)g.Nc * sizeof(float)});
  }
  // attention ops: one set of tensor maps each, in a device array the kernel indexes with ra.i4
  std::vector<FlashMaps> fmaps;
  for (int i = 0; i < n_ops; ++i) {
    const int k = specs[i].kind;
    if (k < OPK_ATTN_FWD || k > OPK_ATTN_BWD_Q) continue;
    const RowArgs &ra = specs[i].ra;
    FlashMaps fm;
    memset(&fm, 0, sizeof(fm));
    e = attention_flash_build_maps(&fm, ra.in0, k == OPK_ATTN_FWD ? nullptr : ra.in1, ra.i0, ra.i2, ra.i1, ra.i3);
    if (e) { *err = e; delete s; return nullptr; }
    s->plan.ops[i].ra.i4 = (int)fmaps.size();
    fmaps.push_back(fm);
  }
  bool ok = true;
  if (!fmaps.empty()) {
    ok = ok && cudaMalloc(reinterpret_cast<void **>(&s->d_fmaps), sizeof(FlashMaps) * fmaps.size()) == cudaSuccess;
    ok = ok && cudaMemcpy(s->d_fmaps, fmaps.data(), sizeof(FlashMaps) * fmaps.size(), cudaMemcpyHostToDevice) == cudaSuccess;
  }
  if (ws_bytes) {
    ok = ok && cudaMalloc(reinterpret_cast<void **>(&s->ws), ws_bytes) == cudaSuccess;
    ok = ok && cudaMalloc(reinterpret_cast<void **>(&s->ws_sem), sem_count * sizeof(unsigned)) == cudaSuccess;
    ok = ok && cudaMemset(s->ws_sem, 0, sem_count * sizeof(unsigned)) == cudaSuccess;
    size_t off = 0, soff = 0;
    for (auto &g : s->plan.ops) {
      if (g.op_kind == OPK_GEMM && g.splits > 1 && !g.atomic_out) {
        g.ws = s->ws + off / sizeof(float);
        g.ws_sem = s->ws_sem + soff;
        off += op_workspace_bytes(g);
        soff += (size_t)g.tiles_m * g.tiles_n * 4;
      }
    }
  }
  ok = ok && cudaMalloc(reinterpret_cast<void **>(&s->d_ops), sizeof(GemmOp) * n_ops) == cudaSuccess;
  ok = ok && cudaMalloc(reinterpret_cast<void **>(&s->d_counters), sizeof(unsigned) * s->plan.n_counters) == cudaSuccess;
  ok = ok && cudaMalloc(reinterpret_cast<void **>(&s->d_status), sizeof(Status)) == cudaSuccess;
  ok = ok && cudaMemcpy(s->d_ops, s->plan.ops.data(), sizeof(GemmOp) * n_ops, cudaMemcpyHostToDevice) == cudaSuccess;
  ok = ok && cudaMemset(s->d_status, 0, sizeof(Status)) == cudaSuccess;
  if (!ok) {
    (void)cudaGetLastError();
    *err = GPT2L_ERR_CUDA;
    gpt2_schedule_destroy(s);
    return nullptr;
  }
  *err = GPT2L_OK;
  return s;
}

}  // namespace g2l

static std::vector<OpSpec> specs_from(const gpt2l_op *ops, int n_ops) {
  std::vector<OpSpec> v;
  if (ops)
    for (int i = 0; i < n_ops; ++i) v.push_back(spec_from(ops[i]));
  return v;
}

extern "C" {

int gpt2_schedule_validate(const gpt2l_op *ops, int n_ops, int grid) {
  Plan plan;
  int e = make_plan(specs_from(ops, n_ops), grid, &plan);
  if (e) return e;
  int units = plan.pair ? (grid / 2 > 0 ? grid / 2 : 1) : grid;  // CTAs, or CTA pairs
  if (units > plan.total_tiles) units = plan.total_tiles;
  return replay(plan, units);
}

int gpt2_schedule_describe(const gpt2l_op *ops, int n_ops, int num_sms, int counts[3]) {
  Plan plan;
  int e = make_plan(specs_from(ops, n_ops), num_sms, &plan);
  if (e) return e;
  if (counts) {
    counts[0] = plan.total_tiles;
    counts[1] = plan.n_counters;
    const int units = plan.pair ? (num_sms / 2 > 0 ? num_sms / 2 : 1) : num_sms;
    counts[2] = units < plan.total_tiles ? units : plan.total_tiles;  // CTAs, or CTA pairs
  }
  return GPT2L_OK;
}

gpt2l_schedule *gpt2_schedule_create(const gpt2l_op *ops, int n_ops, int *err) {
  int dummy;
  if (!err) err = &dummy;
  if (!ops || n_ops <= 0) { *err = GPT2L_ERR_BAD_ARG; return nullptr; }
  std::vector<OpSpec> in = specs_from(ops, n_ops);
  // Wide weight gradients (lm_head: N >= 8192 and N >= 8 K) run faster from a K-major copy of the
  // activations, as in the single-call entry point: a transpose op in front, then the product in the
  // forward form. Ops move down the list, so the callers' producer indices are translated.
  bool pairs = true;
  for (const auto &s : in) pairs = pairs && s.gemm.opts.cta_pair == 2;
  size_t xt_floats = 0;
  for (const auto &s : in) {
    const GemmDesc &d = s.gemm;
    if (!pairs && d.kind == GPT2L_OP_BACKWARD_WEIGHT && d.N >= 8192 && d.N >= 8 * d.K && d.M % 32 == 0 && d.M > 0)
      xt_floats += (size_t)d.M * d.K;
  }
  float *xt = nullptr;
  if (xt_floats && cudaMalloc(reinterpret_cast<void **>(&xt), xt_floats * sizeof(float)) != cudaSuccess) {
    (void)cudaGetLastError();
    *err = GPT2L_ERR_CUDA;
    return nullptr;
  }
  // A transpose goes as far up the list as its own producers allow (right behind the last of them, or to
  // the front): placed directly before its weight gradient it ran when that op's tiles were already
  // waiting for it, behind whatever long op happened to precede them.
  auto wide = [&](const GemmDesc &d) {
    return xt && d.kind == GPT2L_OP_BACKWARD_WEIGHT && d.N >= 8192 && d.N >= 8 * d.K && d.M % 32 == 0;
  };
  std::vector<std::vector<size_t>> hoisted(in.size() + 1);  // original position -> wide gradients whose transpose goes there
  for (size_t i = 0; i < in.size(); ++i) {
    if (!wide(in[i].gemm)) continue;
    int last = -1;
    for (const auto &d : in[i].deps)
      if (d.producer >= 0 && d.producer < (int)i && d.producer > last) last = d.producer;
    hoisted[(size_t)(last + 1)].push_back(i);
  }
  std::vector<OpSpec> out;
  std::vector<int> where(in.size()), t_where(in.size(), -1);
  std::vector<size_t> t_off(in.size(), 0);
  size_t used = 0;
  for (size_t i = 0; i < in.size(); ++i) {
    for (size_t w : hoisted[i]) {
      const GemmDesc d = in[w].gemm;
      OpSpec t;
      t.kind = OPK_TRANSPOSE;
      t.rows = d.M;
      t.rows_per_tile = BM;
      t.layer = in[w].layer;
      memset(&t.ra, 0, sizeof(t.ra));
      t.ra.in0 = d.a; t.ra.out0 = xt + used; t.ra.i0 = d.M; t.ra.i1 = d.K;
      t.deps = in[w].deps;  // the activations' producers, all above this position
      for (auto &dd : t.deps) {
        dd.producer = (dd.producer >= 0 && dd.producer < (int)w) ? where[dd.producer] : -1;
        dd.kind = GPT2L_DEP_WHOLE_OP;
      }
      t_where[w] = (int)out.size();
      t_off[w] = used;
      used += (size_t)d.M * d.K;
      out.push_back(t);
    }
    OpSpec s = in[i];
    for (auto &d : s.deps) d.producer = (d.producer >= 0 && d.producer < (int)i) ? where[d.producer] : -1;
    const GemmDesc d = s.gemm;
    if (wide(d)) {
      s.gemm.kind = GPT2L_OP_FORWARD;
      s.gemm.M = d.K;  // output rows
      s.gemm.K = d.M;  // reduction
      s.gemm.a = xt + t_off[i];
      s.gemm.bias = nullptr;
      s.gemm.opts.flags = 0;
      s.transposed_a = true;
      s.deps.push_back({t_where[i], GPT2L_DEP_WHOLE_OP});
    }
    where[i] = (int)out.size();
    out.push_back(s);
  }
  gpt2l_schedule *sch = schedule_build(out, 0, err);
  if (!sch) {
    if (xt) cudaFree(xt);
    return nullptr;
  }
  sch->xt = xt;
  return sch;
}

void gpt2_schedule_destroy(gpt2l_schedule *s) {
  if (!s) return;
  if (s->d_ops) cudaFree(s->d_ops);
  if (s->d_counters) cudaFree(s->d_counters);
  if (s->d_status) cudaFree(s->d_status);
  if (s->ws) cudaFree(s->ws);
  if (s->ws_sem) cudaFree(s->ws_sem);
  if (s->d_fmaps) cudaFree(s->d_fmaps);
  if (s->xt) cudaFree(s->xt);
  if (s->d_prof) cudaFree(s->d_prof);
  delete s;
}

int gpt2_megakernel_run(gpt2l_schedule *s, gpt2l_stream_t stream) {
  if (!s) return GPT2L_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (*reinterpret_cast<volatile int *>(s->ctx->h_flag) != 0) return GPT2L_DEV_TIMEOUT;  // see gpt2_linear_last_status
  // the reference zeroes bar[] before every launch (tests/test_train_mk.cu:285); so do we
  if (cudaMemsetAsync(s->d_counters, 0, sizeof(unsigned) * s->plan.n_counters, st) != cudaSuccess)
    return GPT2L_ERR_CUDA;
  if (cudaMemsetAsync(s->d_status, 0, sizeof(Status), st) != cudaSuccess) return GPT2L_ERR_CUDA;
  for (const auto &z : s->zero)
    if (cudaMemsetAsync(z.ptr, 0, z.bytes, st) != cudaSuccess) return GPT2L_ERR_CUDA;
  return launch_list(s->ctx, s->d_ops, (int)s->plan.ops.size(), s->plan.total_tiles, s->grid, s->plan.any_3x,
                     s->plan.any_colsum, s->plan.pair, s->d_status, s->d_counters, s->wait_limit_ns, s->adam, s->d_fmaps,
                     s->d_prof, st);
}

int gpt2_megakernel_status(gpt2l_schedule *s) {
  if (!s) return GPT2L_ERR_BAD_ARG;
  Status h;
  if (cudaMemcpy(&h, s->d_status, sizeof(Status), cudaMemcpyDeviceToHost) != cudaSuccess) return GPT2L_ERR_CUDA;
  return h.status;
}

int gpt2_schedule_debug_set_expected(gpt2l_schedule *s, int op, int dep, int expected, int wait_limit_ms) {
  if (!s || op < 0 || op >= (int)s->plan.ops.size() || dep < 0 || dep >= MAX_WAITS) return GPT2L_ERR_BAD_ARG;
  s->plan.ops[op].wait_expected[dep] = expected;
  s->plan.ops[op].wait_op_expected[dep] = expected;
  if (wait_limit_ms > 0) s->wait_limit_ns = (long long)wait_limit_ms * 1000000ll;
  if (cudaMemcpy(s->d_ops + op, &s->plan.ops[op], sizeof(GemmOp), cudaMemcpyHostToDevice) != cudaSuccess)
    return GPT2L_ERR_CUDA;
  return GPT2L_OK;
}

// Per-tile profile of the next runs: {start (%globaltimer ns), SM id << 48 | ns spent} per tile, in the
// global tile order (the reference keeps per-instruction %globaltimer arrays, src/mk.cu:966-971,
// 1117-1138, 1814-1819). enable = 0 stops recording.
int gpt2_schedule_profile(gpt2l_schedule *s, int enable) {
  if (!s) return GPT2L_ERR_BAD_ARG;
  if (enable && !s->d_prof) {
    if (cudaMalloc(reinterpret_cast<void **>(&s->d_prof), sizeof(unsigned long long) * 2 * (size_t)s->plan.total_tiles) !=
        cudaSuccess) {
      (void)cudaGetLastError();
      return GPT2L_ERR_CUDA;
    }
    cudaMemset(s->d_prof, 0, sizeof(unsigned long long) * 2 * (size_t)s->plan.total_tiles);
  } else if (!enable && s->d_prof) {
    cudaFree(s->d_prof);
    s->d_prof = nullptr;
  }
  return GPT2L_OK;
}

// Copies the profile of the last run to the host: for tile i, out[4*i .. 4*i+3] = {op index, start ns,
// duration ns, SM id}. Returns the number of tiles, or a negative error. `max_tiles` bounds the copy.
long long gpt2_schedule_read_profile(gpt2l_schedule *s, long long *out, long long max_tiles) {
  if (!s || !out || !s->d_prof) return GPT2L_ERR_BAD_ARG;
  const long long n = s->plan.total_tiles < max_tiles ? s->plan.total_tiles : max_tiles;
  std::vector<unsigned long long> h(2 * (size_t)n);
  if (cudaMemcpy(h.data(), s->d_prof, h.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost) != cudaSuccess)
    return GPT2L_ERR_CUDA;
  size_t cur = 0;
  for (long long i = 0; i < n; ++i) {
    while (cur + 1 < s->plan.ops.size() && i >= s->plan.ops[cur].tile_base + s->plan.ops[cur].n_tiles) ++cur;
    out[4 * i] = (long long)cur;
    out[4 * i + 1] = (long long)h[2 * i];
    out[4 * i + 2] = (long long)(h[2 * i + 1] & 0xffffffffffffull);
    out[4 * i + 3] = (long long)(h[2 * i + 1] >> 48);
  }
  return n;
}

}  // extern "C"
