// A whole training step as a schedule of the persistent step kernel — the role of schedule_instructions
// (src/mk.cu:281-942 of vnnm404/gpt2.cu) and of the launch around megakernel (tests/test_train_mk.cu:292-314).
//
// The builder walks the step in the order the reference's interpreter lists its ops (src/mk.cu:1155-1810):
// embedding, per block layernorm -> QKV -> attention -> projection (+ residual) -> layernorm -> fc (+ GELU)
// -> fc-proj (+ residual), final layernorm, lm_head, softmax / cross-entropy, then the backward ops in
// reverse with every weight gradient right behind its input gradient, the embedding backward and AdamW.
// The residual adds and the GELU backward ride in GEMM epilogues, so the list is shorter than the
// reference's 35 ops per block.
//
// Dependencies are not written by hand: every op declares which buffers it reads and writes and at what
// granularity (its own 128-row block, its whole sequence, everything), and the builder derives
// read-after-write, write-after-read and write-after-write edges from that, then drops the edges another
// edge already implies. A consumer tile therefore starts when the row block (or sequence) it reads is
// complete — not when the producing op is — and buffers that the step reuses from block to block
// (the residual gradient, the GEMM gradient scratch) are protected without extra barriers.
//
// Where attention runs: `attention_in_kernel` puts the fused attention tiles inside the same launch;
// otherwise the list is cut at every attention op and the attention kernels are launched between the
// pieces (stream order replaces the cross-piece dependencies).
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <set>
#include <vector>

#include "layers.h"
#include "linear_internal.h"
#include "model_internal.h"
#include "schedule_internal.h"

using namespace g2l;

namespace {

enum Gran { ROW = 0, SEQ = 1, WHOLE = 2 };

struct Access {
  const void *buf;
  int gran;
  bool partial;  // write that covers only a part of the buffer another op completes (attention dq | dk, dv)
};

struct BufState {
  std::vector<std::pair<int, int>> writers;  // (op, granularity)
  std::vector<std::pair<int, int>> readers;
};

int combine(int producer_gran, int consumer_gran) {
  if (producer_gran == ROW && consumer_gran == ROW) return GPT2L_DEP_ROWBLOCK;
  if (producer_gran == ROW && consumer_gran == SEQ) return DEP_SEQUENCE;
  return GPT2L_DEP_WHOLE_OP;
}
int strength(int kind) { return kind == GPT2L_DEP_WHOLE_OP ? 3 : (kind == DEP_SEQUENCE ? 2 : 1); }

struct Builder {
  std::vector<OpSpec> ops;
  std::map<const void *, BufState> bufs;
  std::vector<std::set<int>> closure;  // ops complete (at least for the same rows) once op i is

  void add_dep(std::map<int, int> &deps, int producer, int kind, int self) {
    if (producer == self) return;
    auto it = deps.find(producer);
    if (it == deps.end() || strength(kind) > strength(it->second)) deps[producer] = kind;
  }

  int emit(OpSpec s, const std::vector<Access> &reads, const std::vector<Access> &writes,
           const std::vector<DepSpec> &extra = {}) {
    const int self = (int)ops.size();
    std::map<int, int> deps;
    for (const auto &e : extra) add_dep(deps, e.producer, e.kind, self);
    for (const auto &r : reads)
      for (const auto &w : bufs[r.buf].writers) add_dep(deps, w.first, combine(w.second, r.gran), self);
    for (const auto &w : writes) {
      BufState &b = bufs[w.buf];
      for (const auto &r : b.readers) add_dep(deps, r.first, combine(r.second, w.gran), self);   // write after read
      for (const auto &p : b.writers) add_dep(deps, p.first, combine(p.second, w.gran), self);   // write after write
      if (!w.partial) {
        b.writers.clear();
        b.readers.clear();
      }
      b.writers.push_back({self, w.gran});
    }
    for (const auto &r : reads) {
      bool also_written = false;
      for (const auto &w : writes) also_written |= (w.buf == r.buf);
      if (!also_written) bufs[r.buf].readers.push_back({self, r.gran});
    }
    // drop what another edge implies. An edge to Q makes everything Q waited for (transitively) complete for
    // at least the same rows; a whole-op edge to Q makes all of it complete entirely.
    std::vector<DepSpec> kept;
    for (const auto &d : deps) {
      bool implied = false;
      for (const auto &q : deps) {
        if (q.first == d.first) continue;
        if (strength(q.second) < strength(d.second)) continue;
        if (closure[q.first].count(d.first)) { implied = true; break; }
      }
      if (!implied) kept.push_back({d.first, d.second});
    }
    std::set<int> cl;
    for (const auto &d : kept) {
      cl.insert(d.producer);
      cl.insert(closure[d.producer].begin(), closure[d.producer].end());
    }
    closure.push_back(cl);
    s.deps = kept;
    ops.push_back(s);
    return self;
  }
};

OpSpec gemm_spec(int kind, int M, int K, int N, float *out, float *out_bias, const float *a, const float *b,
                 const float *bias, const gpt2_linear_opts &o, int layer) {
  OpSpec s;
  s.kind = OPK_GEMM;
  s.gemm.kind = kind;
  s.gemm.M = M; s.gemm.K = K; s.gemm.N = N;
  s.gemm.out = out; s.gemm.out_bias = out_bias; s.gemm.a = a; s.gemm.b = b; s.gemm.bias = bias;
  s.gemm.opts = o;
  s.layer = layer;
  return s;
}

OpSpec row_spec(int kind, int rows, int rows_per_tile, int layer) {
  OpSpec s;
  s.kind = kind;
  s.rows = rows;
  s.rows_per_tile = rows_per_tile;
  s.layer = layer;
  memset(&s.ra, 0, sizeof(s.ra));
  return s;
}

}  // namespace

// One piece of a step: a persistent launch, or an attention pass launched on its own between two pieces.
struct StepItem {
  gpt2l_schedule *sched = nullptr;
  int attn = 0;  // 0 none, 1 forward, 2 backward
  int layer = 0;
};

struct gpt2l_step {
  gpt2_model *m = nullptr;
  std::vector<StepItem> items;
  float *scratch = nullptr;  // d_ln, d_atty, dqkv, xt of this step object
  float *d_ln = nullptr, *d_atty = nullptr, *dqkv = nullptr, *xt = nullptr;
  float *xstats = nullptr;   // per-tile softmax statistics of the lm_head (fused cross-entropy)
  int with_update = 0;
  int n_ops = 0;
  int launches = 0;
};

extern "C" {

void gpt2_free_schedule(gpt2l_step *s) {
  if (!s) return;
  for (auto &it : s->items)
    if (it.sched) gpt2_schedule_destroy(it.sched);
  if (s->scratch) cudaFree(s->scratch);
  if (s->xstats) cudaFree(s->xstats);
  delete s;
}

gpt2l_step *gpt2_schedule_instructions(gpt2_model *m, const int *tokens, const int *targets, unsigned flags, int *err) {
  int dummy;
  if (!err) err = &dummy;
  *err = GPT2L_ERR_BAD_ARG;
  if (!m || !tokens || !targets) return nullptr;
  const int B = m->B, T = m->T, C = m->cfg.n_embd, L = m->cfg.n_layer, NH = m->cfg.n_head;
  const int V = m->cfg.vocab_size, Vp = m->cfg.padded_vocab_size;
  const int M = B * T;
  // the row-local ops of the step kernel hold a layernorm row in registers up to this width; attention
  // tiles inside the launch are the fused kernels' (whole 128-row blocks per sequence)
  const bool in_kernel = (flags & GPT2_STEP_ATTENTION_IN_KERNEL) != 0;
  if (C > 1280 || (C & 3) || (in_kernel && !m->attn_flash)) { *err = GPT2L_ERR_TOO_LARGE; return nullptr; }
  int e = GPT2L_OK;
  DeviceCtx *ctx = ctx_current(&e);
  if (!ctx) { *err = e; return nullptr; }

  gpt2l_step *st = new gpt2l_step();
  st->m = m;
  st->with_update = (flags & GPT2_STEP_WITH_UPDATE) ? 1 : 0;
  const bool wide_head = (Vp >= 8192 && Vp >= 8 * C && (M & 3) == 0 && M % 32 == 0);
  // Rows per layernorm tile. A GEMM's first wave waits for the layernorm tiles of its first row blocks, which
  // were all handed out at the same moment: short tiles keep that wait short.
  int ln_rows = 64;
  if (const char *e = getenv("GPT2_STEP_LN_ROWS")) {
    const int v = atoi(e);
    if (v == 8 || v == 16 || v == 32 || v == 64 || v == 128) ln_rows = v;
  }
  {
    const size_t floats = (size_t)M * C * 2 + (size_t)M * 3 * C + (wide_head ? (size_t)M * C : 0);
    if (cudaMalloc(reinterpret_cast<void **>(&st->scratch), floats * sizeof(float)) != cudaSuccess) {
      (void)cudaGetLastError();
      *err = GPT2L_ERR_CUDA;
      delete st;
      return nullptr;
    }
    st->d_ln = st->scratch;
    st->d_atty = st->d_ln + (size_t)M * C;
    st->dqkv = st->d_atty + (size_t)M * C;
    st->xt = wide_head ? st->dqkv + (size_t)M * 3 * C : nullptr;
  }

  float *P = m->params, *G = m->grads;
  gpt2_linear_opts o;   // forward and input-gradient GEMMs
  memset(&o, 0, sizeof(o));
  o.mode = m->mode;
  // Their outputs are activation buffers, some of them reused several times inside one step, so a split
  // reduction must not need a zeroed output: partial tiles go through the workspace and are combined by the
  // last split to arrive. Weight gradients (`ow`) land in the gradient buffer, which the step zeroes whole,
  // and keep the cheaper reduce-adds.
  o.deterministic = 1;
  gpt2_linear_opts ow = o;
  ow.deterministic = 0;
  Builder b;
  const int rb_per_seq = T / BM;

  // ---------------- forward ----------------
  {
    OpSpec s = row_spec(OPK_EMBED_FWD, M, 32, -1);
    s.ra.in0 = P + m->off_wte; s.ra.in1 = P + m->off_wpe; s.ra.out0 = m->encoded; s.ra.idx0 = tokens;
    s.ra.i0 = M; s.ra.i1 = C; s.ra.i2 = T; s.ra.i3 = V; s.ra.i4 = Vp;
    b.emit(s, {}, {{m->encoded, ROW, false}});
  }
  const float *res = m->encoded;
  for (int l = 0; l < L; ++l) {
    const LayerParams &p = m->lp[l];
    LayerActs &a = m->la[l];
    {
      OpSpec s = row_spec(OPK_LN_FWD, M, ln_rows, l);
      s.ra.in0 = res; s.ra.in1 = P + p.ln1_w; s.ra.in2 = P + p.ln1_b;
      s.ra.out0 = a.ln1; s.ra.out1 = a.ln1_mean; s.ra.out2 = a.ln1_rstd; s.ra.i0 = M; s.ra.i1 = C;
      b.emit(s, {{res, ROW, false}}, {{a.ln1, ROW, false}});
    }
    b.emit(gemm_spec(GPT2L_OP_FORWARD, M, C, 3 * C, a.qkv, nullptr, a.ln1, P + p.qkv_w, P + p.qkv_b, o, l),
           {{a.ln1, ROW, false}}, {{a.qkv, ROW, false}});
    {
      OpSpec s = row_spec(OPK_ATTN_FWD, M, BM, l);
      s.rb_per_seq = rb_per_seq;
      s.ra.in0 = a.qkv; s.ra.out0 = a.atty; s.ra.out1 = a.lse;
      s.ra.i0 = B; s.ra.i1 = C; s.ra.i2 = T; s.ra.i3 = NH;
      b.emit(s, {{a.qkv, SEQ, false}}, {{a.atty, ROW, false}});
    }
    gpt2_linear_opts orr = o;  // both projections add the residual stream in their epilogue
    orr.aux_op = GPT2L_AUX_ADD;
    orr.aux = res;
    b.emit(gemm_spec(GPT2L_OP_FORWARD, M, C, C, a.res2, nullptr, a.atty, P + p.proj_w, P + p.proj_b, orr, l),
           {{a.atty, ROW, false}, {res, ROW, false}}, {{a.res2, ROW, false}});
    {
      OpSpec s = row_spec(OPK_LN_FWD, M, ln_rows, l);
      s.ra.in0 = a.res2; s.ra.in1 = P + p.ln2_w; s.ra.in2 = P + p.ln2_b;
      s.ra.out0 = a.ln2; s.ra.out1 = a.ln2_mean; s.ra.out2 = a.ln2_rstd; s.ra.i0 = M; s.ra.i1 = C;
      b.emit(s, {{a.res2, ROW, false}}, {{a.ln2, ROW, false}});
    }
    gpt2_linear_opts og = o;  // fc: the epilogue stores the pre-activation and its GELU
    og.flags = GPT2L_EPI_GELU_DUAL;
    og.out2 = a.fc_gelu;
    b.emit(gemm_spec(GPT2L_OP_FORWARD, M, C, 4 * C, a.fc, nullptr, a.ln2, P + p.fc_w, P + p.fc_b, og, l),
           {{a.ln2, ROW, false}}, {{a.fc, ROW, false}, {a.fc_gelu, ROW, false}});
    orr.aux = a.res2;
    b.emit(gemm_spec(GPT2L_OP_FORWARD, M, 4 * C, C, a.res3, nullptr, a.fc_gelu, P + p.fcproj_w, P + p.fcproj_b, orr, l),
           {{a.fc_gelu, ROW, false}, {a.res2, ROW, false}}, {{a.res3, ROW, false}});
    res = a.res3;
  }
  {
    OpSpec s = row_spec(OPK_LN_FWD, M, ln_rows, L);
    s.ra.in0 = res; s.ra.in1 = P + m->off_lnf_w; s.ra.in2 = P + m->off_lnf_b;
    s.ra.out0 = m->lnf; s.ra.out1 = m->lnf_mean; s.ra.out2 = m->lnf_rstd; s.ra.i0 = M; s.ra.i1 = C;
    b.emit(s, {{res, ROW, false}}, {{m->lnf, ROW, false}});
    if (wide_head) {
      // the lm_head's weight gradient reads these activations K-major: the transposed copy is made here, long
      // before that op's tiles come up, so that they never wait for it
      OpSpec t = row_spec(OPK_TRANSPOSE, M, BM, L);
      t.ra.in0 = m->lnf; t.ra.out0 = st->xt; t.ra.i0 = M; t.ra.i1 = C;
      b.emit(t, {{m->lnf, ROW, false}}, {{st->xt, WHOLE, false}});
    }
  }
  gpt2_linear_opts oh = o, ohw = ow;  // the lm_head's backward GEMMs
  if (m->xent_path) {
    // softmax statistics in the lm_head's epilogue and a small combine per row; then either one elementwise
    // pass that turns the logits into their gradient, or the gradient formed from the stored logits inside the
    // two backward GEMMs
    OpSpec g = gemm_spec(GPT2L_OP_FORWARD, M, C, Vp, m->logits, nullptr, m->lnf, P + m->off_wte, nullptr, o, L);
    g.gemm.opts.deterministic = 0;
    g.gemm.xent_vocab = V;
    g.gemm.xent_stats = reinterpret_cast<float *>(16);  // placeholder while the tiling is planned
    GemmOp probe;
    e = plan_op(g.gemm, ctx->num_sms, &probe);
    if (!e && cudaMalloc(reinterpret_cast<void **>(&st->xstats), xent_stats_floats(probe) * sizeof(float)) != cudaSuccess) {
      (void)cudaGetLastError();
      e = GPT2L_ERR_CUDA;
    }
    if (e) {
      *err = e;
      gpt2_free_schedule(st);
      return nullptr;
    }
    g.gemm.xent_stats = st->xstats;
    b.emit(g, {{m->lnf, ROW, false}}, {{m->logits, ROW, false}, {st->xstats, ROW, false}});
    OpSpec s = row_spec(OPK_XENT_COMBINE, M, BM, L);
    s.ra.in0 = st->xstats; s.ra.in1 = m->logits; s.ra.out0 = m->xlse; s.ra.out1 = m->losses; s.ra.idx1 = targets;
    s.ra.i0 = M; s.ra.i1 = probe.xent_stride; s.ra.i3 = V; s.ra.i4 = Vp;
    b.emit(s, {{st->xstats, ROW, false}, {m->logits, ROW, false}}, {{m->xlse, ROW, false}, {m->losses, ROW, false}});
    if (m->xent_path == 2) {
      for (gpt2_linear_opts *x : {&oh, &ohw}) {
        x->xent_lse = m->xlse;
        x->xent_targets = targets;
        x->xent_vocab = V;
        x->xent_scale = 1.f / (float)M;
      }
    } else {
      OpSpec d = row_spec(OPK_XENT_GRAD, M, 8, L);
      d.ra.in0 = m->xlse; d.ra.out0 = m->logits; d.ra.idx1 = targets;
      d.ra.i0 = M; d.ra.i3 = V; d.ra.i4 = Vp; d.ra.f0 = 1.f / (float)M;
      b.emit(d, {{m->logits, ROW, false}, {m->xlse, ROW, false}}, {{m->logits, ROW, false}});
    }
  } else {
    b.emit(gemm_spec(GPT2L_OP_FORWARD, M, C, Vp, m->logits, nullptr, m->lnf, P + m->off_wte, nullptr, o, L),
           {{m->lnf, ROW, false}}, {{m->logits, ROW, false}});
    OpSpec s = row_spec(OPK_XENT, M, 8, L);
    s.ra.out0 = m->logits; s.ra.out1 = m->losses; s.ra.idx1 = targets;
    s.ra.i0 = M; s.ra.i3 = V; s.ra.i4 = Vp; s.ra.f0 = 1.f / (float)M;
    b.emit(s, {{m->logits, ROW, false}}, {{m->logits, ROW, false}, {m->losses, ROW, false}});
  }

  // ---------------- backward ----------------
  // lm_head: the logits buffer holds dlogits now (or still the logits, with the fused cross-entropy)
  b.emit(gemm_spec(GPT2L_OP_BACKWARD_INPUT, M, C, Vp, st->d_ln, nullptr, m->logits, P + m->off_wte, nullptr, oh, L),
         {{m->logits, ROW, false}, {m->xlse, ROW, false}}, {{st->d_ln, ROW, false}});
  if (wide_head) {
    // the weight gradient of the lm_head reads its activations K-major: one transposed copy, then the
    // product in the forward form g_wte[C][Vp] = lnf^T[C][M] . dlogits[M][Vp]
    // (the transposed copy was made right behind the final layernorm, see above)
    OpSpec g = gemm_spec(GPT2L_OP_FORWARD, C, M, Vp, G + m->off_wte, nullptr, st->xt, m->logits, nullptr, ohw, L);
    g.transposed_a = true;
    b.emit(g, {{st->xt, WHOLE, false}, {m->logits, WHOLE, false}, {m->xlse, WHOLE, false}}, {{G + m->off_wte, WHOLE, false}});
  } else {
    b.emit(gemm_spec(GPT2L_OP_BACKWARD_WEIGHT, M, C, Vp, G + m->off_wte, nullptr, m->lnf, m->logits, nullptr, ohw, L),
           {{m->lnf, WHOLE, false}, {m->logits, WHOLE, false}, {m->xlse, WHOLE, false}}, {{G + m->off_wte, WHOLE, false}});
  }
  const float *res_last = L > 0 ? m->la[L - 1].res3 : m->encoded;
  std::vector<int> adam_after(L + 2, -1);  // op whose completion makes bucket i's gradients final
  std::vector<std::vector<int>> wgrads(L);
  {
    OpSpec s = row_spec(OPK_LN_BWD, M, ln_rows, L);
    s.ra.in0 = st->d_ln; s.ra.in1 = res_last; s.ra.in2 = P + m->off_lnf_w; s.ra.in3 = m->lnf_mean; s.ra.in4 = m->lnf_rstd;
    s.ra.out0 = m->dresid; s.ra.out1 = G + m->off_lnf_w; s.ra.out2 = G + m->off_lnf_b; s.ra.i0 = M; s.ra.i1 = C;
    adam_after[L] = b.emit(s, {{st->d_ln, ROW, false}, {res_last, ROW, false}}, {{m->dresid, ROW, false}});
  }
  for (int l = L - 1; l >= 0; --l) {
    const LayerParams &p = m->lp[l];
    LayerActs &a = m->la[l];
    const float *res_in = l > 0 ? m->la[l - 1].res3 : m->encoded;
    // MLP: res3 = res2 + fcproj(gelu(fc(ln2(res2))))
    gpt2_linear_opts ogb = o;  // the GELU backward rides in the epilogue: dbig = (dresid . W^T) * gelu'(fc)
    ogb.aux_op = GPT2L_AUX_GELU_GRAD;
    ogb.aux = a.fc;
    b.emit(gemm_spec(GPT2L_OP_BACKWARD_INPUT, M, 4 * C, C, m->dbig, nullptr, m->dresid, P + p.fcproj_w, nullptr, ogb, l),
           {{m->dresid, ROW, false}, {a.fc, ROW, false}}, {{m->dbig, ROW, false}});
    wgrads[l].push_back(b.emit(
        gemm_spec(GPT2L_OP_BACKWARD_WEIGHT, M, 4 * C, C, G + p.fcproj_w, G + p.fcproj_b, a.fc_gelu, m->dresid, nullptr, ow, l),
        {{m->dresid, WHOLE, false}, {a.fc_gelu, WHOLE, false}}, {{G + p.fcproj_w, WHOLE, false}}));
    b.emit(gemm_spec(GPT2L_OP_BACKWARD_INPUT, M, C, 4 * C, st->d_ln, nullptr, m->dbig, P + p.fc_w, nullptr, o, l),
           {{m->dbig, ROW, false}}, {{st->d_ln, ROW, false}});
    wgrads[l].push_back(b.emit(
        gemm_spec(GPT2L_OP_BACKWARD_WEIGHT, M, C, 4 * C, G + p.fc_w, G + p.fc_b, a.ln2, m->dbig, nullptr, ow, l),
        {{m->dbig, WHOLE, false}, {a.ln2, WHOLE, false}}, {{G + p.fc_w, WHOLE, false}}));
    {
      OpSpec s = row_spec(OPK_LN_BWD, M, ln_rows, l);
      s.ra.in0 = st->d_ln; s.ra.in1 = a.res2; s.ra.in2 = P + p.ln2_w; s.ra.in3 = a.ln2_mean; s.ra.in4 = a.ln2_rstd;
      s.ra.out0 = m->dresid; s.ra.out1 = G + p.ln2_w; s.ra.out2 = G + p.ln2_b; s.ra.i0 = M; s.ra.i1 = C;
      b.emit(s, {{st->d_ln, ROW, false}, {a.res2, ROW, false}}, {{m->dresid, ROW, false}});
    }
    // attention: res2 = res_in + proj(attention(qkv(ln1(res_in))))
    b.emit(gemm_spec(GPT2L_OP_BACKWARD_INPUT, M, C, C, st->d_atty, nullptr, m->dresid, P + p.proj_w, nullptr, o, l),
           {{m->dresid, ROW, false}}, {{st->d_atty, ROW, false}});
    wgrads[l].push_back(b.emit(
        gemm_spec(GPT2L_OP_BACKWARD_WEIGHT, M, C, C, G + p.proj_w, G + p.proj_b, a.atty, m->dresid, nullptr, ow, l),
        {{m->dresid, WHOLE, false}, {a.atty, WHOLE, false}}, {{G + p.proj_w, WHOLE, false}}));
    if (m->attn_flash) {  // the other attention implementations compute their row terms themselves
      OpSpec s = row_spec(OPK_ROWDOT, M, BM, l);
      s.ra.in0 = st->d_atty; s.ra.in1 = a.atty; s.ra.out0 = m->delta; s.ra.i0 = M; s.ra.i1 = C; s.ra.i2 = T; s.ra.i3 = NH;
      b.emit(s, {{st->d_atty, ROW, false}, {a.atty, ROW, false}}, {{m->delta, ROW, false}});
    }
    for (int pass = 0; pass < 2; ++pass) {
      OpSpec s = row_spec(pass == 0 ? OPK_ATTN_BWD_KV : OPK_ATTN_BWD_Q, M, BM, l);
      s.rb_per_seq = rb_per_seq;
      s.ra.in0 = a.qkv; s.ra.in1 = st->d_atty; s.ra.in2 = a.lse; s.ra.in3 = m->delta; s.ra.out0 = st->dqkv;
      s.ra.i0 = B; s.ra.i1 = C; s.ra.i2 = T; s.ra.i3 = NH;
      b.emit(s, {{a.qkv, SEQ, false}, {st->d_atty, SEQ, false}, {m->delta, SEQ, false}}, {{st->dqkv, ROW, pass == 1}});
    }
    b.emit(gemm_spec(GPT2L_OP_BACKWARD_INPUT, M, C, 3 * C, st->d_ln, nullptr, st->dqkv, P + p.qkv_w, nullptr, o, l),
           {{st->dqkv, ROW, false}}, {{st->d_ln, ROW, false}});
    wgrads[l].push_back(b.emit(
        gemm_spec(GPT2L_OP_BACKWARD_WEIGHT, M, C, 3 * C, G + p.qkv_w, G + p.qkv_b, a.ln1, st->dqkv, nullptr, ow, l),
        {{st->dqkv, WHOLE, false}, {a.ln1, WHOLE, false}}, {{G + p.qkv_w, WHOLE, false}}));
    {
      OpSpec s = row_spec(OPK_LN_BWD, M, ln_rows, l);
      s.ra.in0 = st->d_ln; s.ra.in1 = res_in; s.ra.in2 = P + p.ln1_w; s.ra.in3 = a.ln1_mean; s.ra.in4 = a.ln1_rstd;
      s.ra.out0 = m->dresid; s.ra.out1 = G + p.ln1_w; s.ra.out2 = G + p.ln1_b; s.ra.i0 = M; s.ra.i1 = C;
      adam_after[l] = b.emit(s, {{st->d_ln, ROW, false}, {res_in, ROW, false}}, {{m->dresid, ROW, false}});
    }
  }
  {
    OpSpec s = row_spec(OPK_EMBED_BWD, M, 32, -1);
    s.ra.in0 = m->dresid; s.ra.out0 = G + m->off_wte; s.ra.out1 = G + m->off_wpe; s.ra.idx0 = tokens;
    s.ra.i0 = M; s.ra.i1 = C; s.ra.i2 = T; s.ra.i3 = V; s.ra.i4 = Vp;
    adam_after[L + 1] = b.emit(s, {{m->dresid, ROW, false}}, {{G + m->off_wte, WHOLE, true}});
  }
  if (st->with_update) {
    // AdamW per bucket. Completion of the last layernorm backward of a block implies (through the row-block
    // chain) that every input-gradient GEMM, attention pass and layernorm of the block is complete, i.e. that
    // nobody reads the block's parameters any more and its layernorm gradients are final; the four weight
    // gradients are named explicitly. The embedding bucket waits for the embedding backward, which ends the
    // whole chain; ln_f for its own layernorm backward.
    auto adam = [&](long long first, long long count, const std::vector<int> &after, int layer) {
      OpSpec s = row_spec(OPK_ADAMW, 1, 64, layer);
      s.ra.in0 = G; s.ra.out0 = P; s.ra.out1 = m->m1; s.ra.out2 = m->m2; s.ra.n0 = first; s.ra.n1 = count;
      std::vector<DepSpec> deps;
      for (int a : after) deps.push_back({a, GPT2L_DEP_WHOLE_OP});
      b.emit(s, {}, {}, deps);
    };
    for (int l = L - 1; l >= 0; --l) {
      std::vector<int> after = wgrads[l];
      after.push_back(adam_after[l]);
      const long long first = m->lp[l].ln1_w;
      const long long end = l + 1 < L ? m->lp[l + 1].ln1_w : m->off_lnf_w;
      adam(first, end - first, after, l);
    }
    adam(m->off_lnf_w, m->n_params - m->off_lnf_w, {adam_after[L], adam_after[L + 1]}, L);
    adam(0, m->lp.empty() ? m->off_lnf_w : m->lp[0].ln1_w, {adam_after[L + 1]}, -1);
  }
  st->n_ops = (int)b.ops.size();

  // ---------------- pieces ----------------
  std::vector<std::vector<int>> pieces(1);
  std::vector<StepItem> order;
  for (int i = 0; i < (int)b.ops.size(); ++i) {
    const int k = b.ops[i].kind;
    const bool attn = k >= OPK_ATTN_FWD && k <= OPK_ATTN_BWD_Q;
    if (attn && !in_kernel) {
      if (k == OPK_ATTN_BWD_Q) continue;  // launched together with the key/value pass
      StepItem piece;
      piece.layer = (int)pieces.size() - 1;  // index into `pieces`, resolved below
      order.push_back(piece);
      StepItem at;
      at.attn = k == OPK_ATTN_FWD ? 1 : 2;
      at.layer = b.ops[i].layer;
      order.push_back(at);
      pieces.emplace_back();
    } else {
      pieces.back().push_back(i);
    }
  }
  {
    StepItem piece;
    piece.layer = (int)pieces.size() - 1;
    order.push_back(piece);
  }
  for (auto &it : order) {
    if (it.attn) {
      st->items.push_back(it);
      ++st->launches;
      if (it.attn == 2) st->launches += 1;  // key/value pass + query pass
      continue;
    }
    const std::vector<int> &idx = pieces[it.layer];
    if (idx.empty()) continue;
    std::map<int, int> local;
    for (int j = 0; j < (int)idx.size(); ++j) local[idx[j]] = j;
    std::vector<OpSpec> specs;
    for (int j : idx) {
      OpSpec s = b.ops[j];
      std::vector<DepSpec> deps;
      for (const auto &d : s.deps) {
        auto f = local.find(d.producer);
        if (f != local.end()) deps.push_back({f->second, d.kind});  // an earlier piece is complete by stream order
      }
      s.deps = deps;
      specs.push_back(s);
    }
    StepItem piece;
    piece.sched = schedule_build(specs, 0, &e);
    if (!piece.sched) {
      *err = e;
      gpt2_free_schedule(st);
      return nullptr;
    }
    if (getenv("GPT2_STEP_DUMP")) {  // debugging aid: the piece as the kernel will see it
      static const char *names[] = {"gemm", "embed_fwd", "ln_fwd", "xent", "ln_bwd", "rowdot", "embed_bwd", "adamw",
                                    "attn_fwd", "attn_bwd_kv", "attn_bwd_q", "transpose", "xent_combine", "xent_grad"};
      fprintf(stderr, "piece %d: %d ops, %d tiles, grid %d\n", (int)st->items.size(), (int)specs.size(),
              piece.sched->plan.total_tiles, piece.sched->grid);
      for (size_t j = 0; j < specs.size(); ++j) {
        const GemmOp &g = piece.sched->plan.ops[j];
        fprintf(stderr, "  op %3d %-11s layer %2d tiles %5d", (int)j, names[g.op_kind], g.layer, g.n_tiles);
        if (g.op_kind == OPK_GEMM)
          fprintf(stderr, " [%d x %d x %d] bn %d splits %d xform %d", g.Mc, g.Nc, g.Kc, g.bn, g.splits, g.xform);
        for (int w = 0; w < MAX_WAITS; ++w)
          if (g.wait_ctr[w] >= 0)
            fprintf(stderr, " | dep %d kind %d need %d", specs[j].deps[w].producer, g.wait_kind[w], g.wait_expected[w]);
        fprintf(stderr, "\n");
      }
    }
    piece.sched->zero.clear();  // every accumulated output lies in the gradient buffer, which the step zeroes whole
    st->items.push_back(piece);
    ++st->launches;
  }
  *err = GPT2L_OK;
  return st;
}

int gpt2_megakernel_step(gpt2l_step *s, float lr, float beta1, float beta2, float eps, float weight_decay, int t,
                         gpt2l_stream_t stream) {
  if (!s || (s->with_update && t < 1)) return GPT2L_ERR_BAD_ARG;
  gpt2_model *m = s->m;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int B = m->B, T = m->T, C = m->cfg.n_embd, NH = m->cfg.n_head;
  const size_t M = (size_t)B * T;
  // gradients are accumulated into (split-K reduce-adds, column sums, the layernorm and embedding
  // scatters), and so is the residual gradient: both start from zero, as gpt2_zero_grad and
  // zero_activation_grads do in the reference's loop (tests/test_train_mk.cu:280-290)
  if (cudaMemsetAsync(m->grads, 0, (size_t)m->n_params * sizeof(float), st) != cudaSuccess) return GPT2L_ERR_CUDA;
  if (cudaMemsetAsync(m->dresid, 0, M * C * sizeof(float), st) != cudaSuccess) return GPT2L_ERR_CUDA;
  const float adam[7] = {lr, beta1, beta2, eps, weight_decay, 1.f - powf(beta1, (float)t), 1.f - powf(beta2, (float)t)};
  for (auto &it : s->items) {
    int e = GPT2L_OK;
    if (it.sched) {
      for (int i = 0; i < 7; ++i) it.sched->adam[i] = adam[i];
      e = gpt2_megakernel_run(it.sched, stream);
    } else if (it.attn == 1) {
      const LayerActs &a = m->la[it.layer];
      if (m->attn_flash) e = attention_flash_forward(a.atty, a.lse, a.qkv, B, T, C, NH, st);
      else if (m->attn_gemm) e = attention_forward_gemm(a.atty, a.att, a.qkv, B, T, C, NH, m->mode, st);
      else e = attention_forward(a.atty, a.lse, a.qkv, B, T, C, NH, st);
    } else {
      const LayerActs &a = m->la[it.layer];
      if (m->attn_flash) e = attention_flash_backward_core(s->dqkv, m->delta, s->d_atty, a.qkv, a.lse, B, T, C, NH, st);
      else if (m->attn_gemm)
        e = attention_backward_gemm(s->dqkv, m->datt, m->delta, s->d_atty, a.atty, a.att, a.qkv, B, T, C, NH, m->mode, st);
      else e = attention_backward(s->dqkv, m->delta, s->d_atty, a.atty, a.qkv, a.lse, B, T, C, NH, st);
    }
    if (e) return e;
  }
  m->tokens = nullptr;  // the separate-launch backward entry points need a forward of their own
  return GPT2L_OK;
}

int gpt2_megakernel_step_status(gpt2l_step *s) {
  if (!s) return GPT2L_ERR_BAD_ARG;
  for (auto &it : s->items)
    if (it.sched) {
      const int v = gpt2_megakernel_status(it.sched);
      if (v) return v;
    }
  return attention_flash_status() != 0 ? GPT2L_DEV_TIMEOUT : 0;
}

// Test hook for the bounded-wait path of a step (host-side fault injection, no device fault is provoked):
// overrides the expected count of dependency `dep` of op `op` of persistent piece `piece`, and the wait
// limit of that piece in milliseconds.
int gpt2_megakernel_step_debug_set_expected(gpt2l_step *s, int piece, int op, int dep, int expected, int wait_limit_ms) {
  if (!s) return GPT2L_ERR_BAD_ARG;
  int k = 0;
  for (auto &it : s->items)
    if (it.sched && k++ == piece) return gpt2_schedule_debug_set_expected(it.sched, op, dep, expected, wait_limit_ms);
  return GPT2L_ERR_BAD_ARG;
}

// Per-tile profile of the persistent pieces (see gpt2_schedule_profile): enable / disable for all pieces, and
// read piece `piece` of the last step. Rows as in gpt2_schedule_read_profile, with the op's kind in the
// upper half of the first value: out[4i] = op index | kind << 32.
int gpt2_megakernel_step_profile(gpt2l_step *s, int enable) {
  if (!s) return GPT2L_ERR_BAD_ARG;
  for (auto &it : s->items)
    if (it.sched) {
      const int e = gpt2_schedule_profile(it.sched, enable);
      if (e) return e;
    }
  return GPT2L_OK;
}

long long gpt2_megakernel_step_read_profile(gpt2l_step *s, int piece, long long *out, long long max_tiles) {
  if (!s) return GPT2L_ERR_BAD_ARG;
  int k = 0;
  for (auto &it : s->items)
    if (it.sched && k++ == piece) {
      const long long n = gpt2_schedule_read_profile(it.sched, out, max_tiles);
      for (long long i = 0; i < n; ++i) out[4 * i] |= (long long)it.sched->plan.ops[out[4 * i]].op_kind << 32;
      return n;
    }
  return GPT2L_ERR_BAD_ARG;
}

int gpt2_megakernel_step_info(const gpt2l_step *s, int out[3]) {
  if (!s || !out) return GPT2L_ERR_BAD_ARG;
  out[0] = s->n_ops;
  out[1] = s->launches;
  int tiles = 0;
  for (const auto &it : s->items)
    if (it.sched) tiles += it.sched->plan.total_tiles;
  out[2] = tiles;
  return GPT2L_OK;
}

}  // extern "C"
