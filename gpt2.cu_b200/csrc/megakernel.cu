// Host side of the persistent multi-GEMM launch ("megakernel" path): turns a list of GEMM
// ops with dependencies into tile ranges, dependency counters and a device op array, checks
// the schedule by replaying it on the host, and launches the kernel once per run.
//
// Counter layout: op i owns tiles_m(i) row-block counters followed by one op-level counter.
// Each epilogue warp of a tile publishes once to the row-block counter of its tile row and once
// to the op counter, so with A arrivals per tile (4 epilogue warps; 8 in one-CTA launches whose
// transform warps help in the epilogue) a complete row block shows A * tiles_n * splits arrivals
// and a complete op A * n_tiles.
#include <cuda_runtime.h>
#include <string.h>

#include <vector>

#include "linear_internal.h"

namespace g2l {

struct Plan {
  std::vector<GemmOp> ops;
  int total_tiles = 0;
  int n_counters = 0;
  bool any_3x = false;
  bool any_colsum = false;
  bool pair = false;  // every op runs on CTA pairs (256-row tiles)
  int arrivals = NUM_EPI_WARPS;  // counter arrivals per finished 128-row tile (see epi_arrivals)
};

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

// Shapes, tiling, counters and dependency wiring. No CUDA calls (used by the CPU tests).
static int make_plan(const gpt2l_op *ops, int n_ops, int num_sms, Plan *plan) {
  if (!ops || n_ops <= 0) return GPT2L_ERR_BAD_ARG;
  plan->ops.resize(n_ops);
  int tile_base = 0, ctr = 0;
  // one kernel runs the whole list, so all ops use the same CTA arrangement: pairs only when
  // every op asks for them (cta_pair == 2)
  bool pair = true;
  for (int i = 0; i < n_ops; ++i)
    if (ops[i].opts.cta_pair != 2) pair = false;
  plan->pair = pair;
  for (int i = 0; i < n_ops; ++i) {
    GemmDesc d = desc_from(ops[i]);
    d.opts.cta_pair = pair ? 2 : 1;
    // bias gradient inside a schedule is always the fused column sum
    int e = plan_op(d, num_sms, &plan->ops[i]);
    if (e) return e;
    GemmOp &g = plan->ops[i];
    if (i > 0 && g.mode != plan->ops[0].mode) return GPT2L_ERR_SCHEDULE;  // one mode per launch
    g.op_index = i;
    g.layer = ops[i].layer;
    g.tile_base = tile_base;
    tile_base += g.n_tiles;
    g.pub_rb_base = ctr;
    g.pub_op_ctr = ctr + g.tiles_m;
    ctr += g.tiles_m + 1;
    if (g.mode == GPT2L_MODE_TF32X3) plan->any_3x = true;
    if (g.colsum) plan->any_colsum = true;
  }
  // the pair kernel always publishes from its four epilogue warps per CTA
  plan->arrivals = plan->pair ? NUM_EPI_WARPS : epi_arrivals(plan->any_3x || plan->any_colsum);
  const unsigned ARRIVALS_PER_TILE = (unsigned)plan->arrivals;
  for (int i = 0; i < n_ops; ++i) {
    GemmOp &g = plan->ops[i];
    for (int w = 0; w < GPT2L_MAX_DEPS; ++w) {
      const gpt2l_dep &dep = ops[i].deps[w];
      if (dep.kind == GPT2L_DEP_NONE) continue;
      if (dep.producer < 0 || dep.producer >= i) return GPT2L_ERR_SCHEDULE;  // must point backwards
      const GemmOp &pr = plan->ops[dep.producer];
      if (dep.kind == GPT2L_DEP_ROWBLOCK) {
        // row block r of the consumer reads rows [128r, 128r+128) of the producer's output
        if (pr.Mc != g.Mc || g.a_mn) return GPT2L_ERR_SCHEDULE;
        g.wait_ctr[w] = pr.pub_rb_base;
        g.wait_kind[w] = GPT2L_DEP_ROWBLOCK;
        g.wait_expected[w] = (int)(ARRIVALS_PER_TILE * pr.tiles_n * pr.splits);
      } else if (dep.kind == GPT2L_DEP_WHOLE_OP) {
        g.wait_ctr[w] = pr.pub_op_ctr;
        g.wait_kind[w] = GPT2L_DEP_WHOLE_OP;
        g.wait_expected[w] = (int)(ARRIVALS_PER_TILE * pr.tiles_m * pr.tiles_n * pr.splits);
      } else {
        return GPT2L_ERR_SCHEDULE;
      }
    }
  }
  plan->total_tiles = tile_base;
  plan->n_counters = ctr;
  return GPT2L_OK;
}

// Replays the schedule: CTA c owns tiles c, c+grid, ... and runs them in order; a tile may
// run when its counters have reached the expected values. Returns OK when every tile ran.
static int replay(const Plan &plan, int grid) {
  if (grid <= 0) return GPT2L_ERR_BAD_ARG;
  std::vector<long long> counters(plan.n_counters, 0);
  std::vector<int> next(grid);
  for (int c = 0; c < grid; ++c) next[c] = c;
  int remaining = plan.total_tiles;
  std::vector<int> cursor(grid, 0);
  const int ARRIVALS_PER_TILE = plan.arrivals;
  while (remaining > 0) {
    bool progress = false;
    for (int c = 0; c < grid; ++c) {
      while (next[c] < plan.total_tiles) {
        const int t = next[c];
        int &cur = cursor[c];
        while (cur + 1 < (int)plan.ops.size() && t >= plan.ops[cur].tile_base + plan.ops[cur].n_tiles) ++cur;
        const GemmOp &g = plan.ops[cur];
        int m_dec, n_tile, split;
        decode_local(t - g.tile_base, g.tiles_dec, g.tiles_n, g.band_m, m_dec, n_tile, split);
        // a pair tile covers two 128-row blocks, one per CTA
        const int halves = g.pair ? 2 : 1;
        bool ready = true;
        for (int h = 0; h < halves; ++h) {
          const int m_tile = g.pair ? 2 * m_dec + h : m_dec;
          if (m_tile >= g.tiles_m) continue;
          for (int w = 0; w < MAX_WAITS; ++w) {
            if (g.wait_ctr[w] < 0) continue;
            const int idx = g.wait_ctr[w] + (g.wait_kind[w] == GPT2L_DEP_ROWBLOCK ? m_tile : 0);
            if (idx < 0 || idx >= plan.n_counters) return GPT2L_ERR_SCHEDULE;
            if (counters[idx] < g.wait_expected[w]) ready = false;
          }
        }
        if (!ready) break;
        for (int h = 0; h < halves; ++h) {
          const int m_tile = g.pair ? 2 * m_dec + h : m_dec;
          if (m_tile >= g.tiles_m) continue;
          counters[g.pub_rb_base + m_tile] += ARRIVALS_PER_TILE;
          counters[g.pub_op_ctr] += ARRIVALS_PER_TILE;
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

struct gpt2l_schedule {
  Plan plan;
  std::vector<gpt2l_op> user_ops;
  GemmOp *d_ops = nullptr;
  unsigned *d_counters = nullptr;
  Status *d_status = nullptr;
  float *ws = nullptr;
  unsigned *ws_sem = nullptr;
  int grid = 0;
  long long wait_limit_ns = 0;
  DeviceCtx *ctx = nullptr;
};

extern "C" {

int gpt2_schedule_validate(const gpt2l_op *ops, int n_ops, int grid) {
  Plan plan;
  int e = make_plan(ops, n_ops, grid, &plan);
  if (e) return e;
  int units = plan.pair ? (grid / 2 > 0 ? grid / 2 : 1) : grid;  // CTAs, or CTA pairs
  if (units > plan.total_tiles) units = plan.total_tiles;
  return replay(plan, units);
}

int gpt2_schedule_describe(const gpt2l_op *ops, int n_ops, int num_sms, int counts[3]) {
  Plan plan;
  int e = make_plan(ops, n_ops, num_sms, &plan);
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
  int e = GPT2L_OK;
  int dummy;
  if (!err) err = &dummy;
  DeviceCtx *ctx = ctx_current(&e);
  if (!ctx) { *err = e; return nullptr; }
  gpt2l_schedule *s = new gpt2l_schedule();
  s->ctx = ctx;
  e = make_plan(ops, n_ops, ctx->num_sms, &s->plan);
  if (e) { *err = e; delete s; return nullptr; }
  s->user_ops.assign(ops, ops + n_ops);
  {
    const int units = s->plan.pair ? ctx->max_pairs : ctx->num_sms;  // CTA pairs or CTAs
    s->grid = units < s->plan.total_tiles ? units : s->plan.total_tiles;
    if (s->grid <= 0) { *err = GPT2L_ERR_CUDA; delete s; return nullptr; }
  }
  e = replay(s->plan, s->grid);
  if (e) { *err = e; delete s; return nullptr; }
  // tensor maps + workspace
  size_t ws_bytes = 0, sem_count = 0;
  for (int i = 0; i < n_ops; ++i) {
    GemmDesc d = desc_from(ops[i]);
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
    ws_bytes += op_workspace_bytes(g);
    if (g.splits > 1 && !g.atomic_out) sem_count += (size_t)g.tiles_m * g.tiles_n * 4;
  }
  bool ok = true;
  if (ws_bytes) {
    ok = ok && cudaMalloc(reinterpret_cast<void **>(&s->ws), ws_bytes) == cudaSuccess;
    ok = ok && cudaMalloc(reinterpret_cast<void **>(&s->ws_sem), sem_count * sizeof(unsigned)) == cudaSuccess;
    ok = ok && cudaMemset(s->ws_sem, 0, sem_count * sizeof(unsigned)) == cudaSuccess;
    size_t off = 0, soff = 0;
    for (auto &g : s->plan.ops) {
      if (g.splits > 1 && !g.atomic_out) {
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

void gpt2_schedule_destroy(gpt2l_schedule *s) {
  if (!s) return;
  if (s->d_ops) cudaFree(s->d_ops);
  if (s->d_counters) cudaFree(s->d_counters);
  if (s->d_status) cudaFree(s->d_status);
  if (s->ws) cudaFree(s->ws);
  if (s->ws_sem) cudaFree(s->ws_sem);
  delete s;
}

int gpt2_megakernel_run(gpt2l_schedule *s, gpt2l_stream_t stream) {
  if (!s) return GPT2L_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the reference zeroes bar[] before every launch (tests/test_train_mk.cu:285); so do we
  if (cudaMemsetAsync(s->d_counters, 0, sizeof(unsigned) * s->plan.n_counters, st) != cudaSuccess)
    return GPT2L_ERR_CUDA;
  if (cudaMemsetAsync(s->d_status, 0, sizeof(Status), st) != cudaSuccess) return GPT2L_ERR_CUDA;
  for (const auto &g : s->plan.ops) {
    if (g.splits > 1) {
      if (g.atomic_out &&
          cudaMemsetAsync(g.C, 0, (size_t)g.Mc * g.Nc * sizeof(float), st) != cudaSuccess)
        return GPT2L_ERR_CUDA;
      if (g.colsum && cudaMemsetAsync(g.colsum, 0, (size_t)g.Nc * sizeof(float), st) != cudaSuccess)
        return GPT2L_ERR_CUDA;
    } else if (g.colsum && g.colsum_spread) {
      if (cudaMemsetAsync(g.colsum, 0, (size_t)g.Nc * sizeof(float), st) != cudaSuccess) return GPT2L_ERR_CUDA;
    }
  }
  return launch_list(s->ctx, s->d_ops, (int)s->plan.ops.size(), s->plan.total_tiles, s->grid, s->plan.any_3x, s->plan.any_colsum, s->plan.pair,
                     s->d_status, s->d_counters, s->wait_limit_ns, st);
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
  if (wait_limit_ms > 0) s->wait_limit_ns = (long long)wait_limit_ms * 1000000ll;
  if (cudaMemcpy(s->d_ops + op, &s->plan.ops[op], sizeof(GemmOp), cudaMemcpyHostToDevice) != cudaSuccess)
    return GPT2L_ERR_CUDA;
  return GPT2L_OK;
}

}  // extern "C"
