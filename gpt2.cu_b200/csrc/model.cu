// GPT-2 training step around the linear-layer GEMM path: buffers, forward, backward, AdamW.
// C ABI in include/gpt2_model.h; the reference counterpart is src/train.cu + src/gpt2.cu of
// vnnm404/gpt2.cu (same parameter order and tensor layouts, new kernels).
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "gpt2_model.h"
#include "layers.h"
#include "linear_internal.h"
#include "model_internal.h"

using namespace g2l;

#define CK(call)                      \
  do {                                \
    int _e = (call);                  \
    if (_e != GPT2L_OK) return _e;    \
  } while (0)

static gpt2_linear_opts opts_for(const gpt2_model *m) {
  gpt2_linear_opts o;
  memset(&o, 0, sizeof(o));
  o.mode = m->mode;
  return o;
}

extern "C" {

gpt2_model *gpt2_model_create(const gpt2_model_config *cfg, int B, int T, int mode, int *err) {
  int dummy;
  if (!err) err = &dummy;
  *err = GPT2L_ERR_BAD_ARG;
  if (!cfg || B <= 0 || T <= 0) return nullptr;
  const int C = cfg->n_embd, L = cfg->n_layer, V = cfg->vocab_size, Vp = cfg->padded_vocab_size;
  if (C <= 0 || L <= 0 || cfg->n_head <= 0 || C != cfg->n_head * 64 || V <= 0 || Vp < V || (Vp & 3) || (C & 3) ||
      T > cfg->n_positions)
    return nullptr;
  if (mode != GPT2L_MODE_TF32 && mode != GPT2L_MODE_TF32X3) return nullptr;
  int e;
  if (!ctx_current(&e)) { *err = e; return nullptr; }

  gpt2_model *m = new gpt2_model();
  m->cfg = *cfg;
  m->B = B; m->T = T; m->mode = mode;
  // ---- parameter layout (reference order) ----
  long long off = 0;
  auto take = [&](long long n) { long long o = off; m->tensor_offsets.push_back(o); off += n; return o; };
  m->off_wte = take((long long)C * Vp);
  m->off_wpe = take((long long)cfg->n_positions * C);
  m->lp.resize(L);
  for (int l = 0; l < L; ++l) {
    LayerParams &p = m->lp[l];
    p.ln1_w = take(C); p.ln1_b = take(C);
    p.qkv_w = take((long long)C * 3 * C); p.qkv_b = take(3 * C);
    p.proj_w = take((long long)C * C); p.proj_b = take(C);
    p.ln2_w = take(C); p.ln2_b = take(C);
    p.fc_w = take((long long)C * 4 * C); p.fc_b = take(4 * C);
    p.fcproj_w = take((long long)4 * C * C); p.fcproj_b = take(C);
  }
  m->off_lnf_w = take(C);
  m->off_lnf_b = take(C);
  m->n_params = off;

  // ---- activations ----
  const long long M = (long long)B * T;
  const int NH = cfg->n_head;
  long long a = 0;
  auto act = [&](long long n) { long long o = a; a += (n + 3) / 4 * 4; return o; };
  // Attention: the fused tensor-core kernel (no T x T tensors; T % 128 == 0) in TF32 mode, batched
  // GEMMs on the linear-layer kernel (T % 32 == 0; they follow the 3xTF32 mode) otherwise, CUDA-core
  // kernels for everything else. GPT2_ATTENTION = flash | gemm | simt overrides the choice.
  m->attn_gemm = attention_gemm_supported(T, C, NH);
  m->attn_flash = attention_flash_supported(T, C, NH) && mode == GPT2L_MODE_TF32;
  if (const char *env = getenv("GPT2_ATTENTION")) {
    if (!strcmp(env, "simt")) m->attn_gemm = m->attn_flash = false;
    else if (!strcmp(env, "gemm")) m->attn_flash = false;
    else if (!strcmp(env, "flash")) m->attn_flash = attention_flash_supported(T, C, NH);
  }
  if (m->attn_flash) m->attn_gemm = false;
  const long long att_floats = m->attn_gemm ? (long long)B * NH * T * T : 0;
  std::vector<long long> o_layer(L * 14);
  const long long o_encoded = act(M * C);
  for (int l = 0; l < L; ++l) {
    long long *o = &o_layer[l * 14];
    o[13] = act(att_floats);
    o[0] = act(M * C); o[1] = act(M); o[2] = act(M);          // ln1, mean, rstd
    o[3] = act(M * 3 * C);                                    // qkv
    o[4] = act(M * C);                                        // atty
    o[5] = act((long long)B * NH * T);                        // lse
    o[6] = act(M * C);                                        // res2
    o[7] = act(M * C); o[8] = act(M); o[9] = act(M);          // ln2, mean, rstd
    o[10] = act(M * 4 * C); o[11] = act(M * 4 * C);           // fc, fc_gelu
    o[12] = act(M * C);                                       // res3
  }
  const long long o_lnf = act(M * C), o_lnf_mean = act(M), o_lnf_rstd = act(M);
  const long long o_logits = act(M * Vp), o_losses = act(M), o_xlse = act(M);
  const long long o_tmp = act(M * C), o_dres = act(M * C), o_dbig = act(M * 4 * C);
  const long long o_delta = act((long long)B * NH * T);
  const long long o_datt = act(att_floats);
  m->acts_floats = a;

  bool ok = true;
  const size_t pbytes = (size_t)m->n_params * sizeof(float);
  ok = ok && cudaMalloc(reinterpret_cast<void **>(&m->params), pbytes) == cudaSuccess;
  ok = ok && cudaMalloc(reinterpret_cast<void **>(&m->grads), pbytes) == cudaSuccess;
  ok = ok && cudaMalloc(reinterpret_cast<void **>(&m->m1), pbytes) == cudaSuccess;
  ok = ok && cudaMalloc(reinterpret_cast<void **>(&m->m2), pbytes) == cudaSuccess;
  ok = ok && cudaMalloc(reinterpret_cast<void **>(&m->acts), (size_t)a * sizeof(float)) == cudaSuccess;
  ok = ok && cudaMallocHost(reinterpret_cast<void **>(&m->h_losses), (size_t)M * sizeof(float)) == cudaSuccess;
  if (!ok) {
    (void)cudaGetLastError();
    *err = GPT2L_ERR_CUDA;
    gpt2_model_destroy(m);
    return nullptr;
  }
  cudaMemset(m->params, 0, pbytes);
  cudaMemset(m->grads, 0, pbytes);
  cudaMemset(m->m1, 0, pbytes);
  cudaMemset(m->m2, 0, pbytes);
  m->device_bytes = 4ll * (long long)pbytes + a * (long long)sizeof(float);
  float *A = m->acts;
  m->encoded = A + o_encoded;
  m->la.resize(L);
  for (int l = 0; l < L; ++l) {
    const long long *o = &o_layer[l * 14];
    LayerActs &x = m->la[l];
    x.att = A + o[13];
    x.ln1 = A + o[0]; x.ln1_mean = A + o[1]; x.ln1_rstd = A + o[2]; x.qkv = A + o[3]; x.atty = A + o[4];
    x.lse = A + o[5]; x.res2 = A + o[6]; x.ln2 = A + o[7]; x.ln2_mean = A + o[8]; x.ln2_rstd = A + o[9];
    x.fc = A + o[10]; x.fc_gelu = A + o[11]; x.res3 = A + o[12];
  }
  m->lnf = A + o_lnf; m->lnf_mean = A + o_lnf_mean; m->lnf_rstd = A + o_lnf_rstd;
  m->logits = A + o_logits; m->losses = A + o_losses; m->xlse = A + o_xlse;
  // where softmax / cross-entropy run (see model_internal.h): GPT2_XENT = separate | stats | fused
  {
    const char *env = getenv("GPT2_XENT");
    m->xent_path = 1;
    if (env && !strcmp(env, "separate")) m->xent_path = 0;
    if (env && !strcmp(env, "fused")) m->xent_path = 2;
  }
  m->tmp_c = A + o_tmp; m->dresid = A + o_dres; m->dbig = A + o_dbig; m->delta = A + o_delta; m->datt = A + o_datt;
  *err = GPT2L_OK;
  return m;
}

void gpt2_model_destroy(gpt2_model *m) {
  if (!m) return;
  if (m->params) cudaFree(m->params);
  if (m->grads) cudaFree(m->grads);
  if (m->m1) cudaFree(m->m1);
  if (m->m2) cudaFree(m->m2);
  if (m->acts) cudaFree(m->acts);
  if (m->h_losses) cudaFreeHost(m->h_losses);
  if (m->graph_exec) cudaGraphExecDestroy(m->graph_exec);
  if (m->graph) cudaGraphDestroy(m->graph);
  if (m->cap_stream) cudaStreamDestroy(m->cap_stream);
  delete m;
}

long long gpt2_model_num_params(const gpt2_model *m) { return m ? m->n_params : 0; }
float *gpt2_model_params(gpt2_model *m) { return m ? m->params : nullptr; }
float *gpt2_model_grads(gpt2_model *m) { return m ? m->grads : nullptr; }
long long gpt2_model_device_bytes(const gpt2_model *m) { return m ? m->device_bytes : 0; }

int gpt2_model_param_offsets(const gpt2_model *m, long long *offsets, int max) {
  if (!m || !offsets) return GPT2L_ERR_BAD_ARG;
  const int n = (int)m->tensor_offsets.size();
  if (max < n) return GPT2L_ERR_TOO_LARGE;
  for (int i = 0; i < n; ++i) offsets[i] = m->tensor_offsets[i];
  return n;
}

int gpt2_model_set_params(gpt2_model *m, const float *host, long long count) {
  if (!m || !host || count != m->n_params) return GPT2L_ERR_BAD_ARG;
  return cudaMemcpy(m->params, host, (size_t)count * sizeof(float), cudaMemcpyHostToDevice) == cudaSuccess
             ? GPT2L_OK : GPT2L_ERR_CUDA;
}
int gpt2_model_get_params(gpt2_model *m, float *host, long long count) {
  if (!m || !host || count != m->n_params) return GPT2L_ERR_BAD_ARG;
  return cudaMemcpy(host, m->params, (size_t)count * sizeof(float), cudaMemcpyDeviceToHost) == cudaSuccess
             ? GPT2L_OK : GPT2L_ERR_CUDA;
}
int gpt2_model_get_grads(gpt2_model *m, float *host, long long count) {
  if (!m || !host || count != m->n_params) return GPT2L_ERR_BAD_ARG;
  return cudaMemcpy(host, m->grads, (size_t)count * sizeof(float), cudaMemcpyDeviceToHost) == cudaSuccess
             ? GPT2L_OK : GPT2L_ERR_CUDA;
}

int gpt2_model_forward(gpt2_model *m, const int *tokens, const int *targets, gpt2l_stream_t stream) {
  if (!m || !tokens || !targets) return GPT2L_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int B = m->B, T = m->T, C = m->cfg.n_embd, L = m->cfg.n_layer, NH = m->cfg.n_head;
  const int V = m->cfg.vocab_size, Vp = m->cfg.padded_vocab_size;
  const int M = B * T;
  float *P = m->params;
  gpt2_linear_opts o = opts_for(m);
  m->tokens = tokens;
  CK(embedding_forward(m->encoded, tokens, P + m->off_wte, P + m->off_wpe, B, T, C, Vp, st));
  const float *res = m->encoded;
  for (int l = 0; l < L; ++l) {
    const LayerParams &p = m->lp[l];
    LayerActs &a = m->la[l];
    CK(layernorm_forward(a.ln1, a.ln1_mean, a.ln1_rstd, res, P + p.ln1_w, P + p.ln1_b, M, C, st));
    CK(gpt2_linear_forward(a.qkv, a.ln1, P + p.qkv_w, P + p.qkv_b, B, T, C, 3 * C, &o, stream));
    if (m->attn_flash) CK(attention_flash_forward(a.atty, a.lse, a.qkv, B, T, C, NH, st));
    else if (m->attn_gemm) CK(attention_forward_gemm(a.atty, a.att, a.qkv, B, T, C, NH, m->mode, st));
    else CK(attention_forward(a.atty, a.lse, a.qkv, B, T, C, NH, st));
    gpt2_linear_opts orr = o;  // both projections add the residual stream in their epilogue
    orr.aux_op = GPT2L_AUX_ADD;
    orr.aux = res;
    CK(gpt2_linear_forward(a.res2, a.atty, P + p.proj_w, P + p.proj_b, B, T, C, C, &orr, stream));
    CK(layernorm_forward(a.ln2, a.ln2_mean, a.ln2_rstd, a.res2, P + p.ln2_w, P + p.ln2_b, M, C, st));
    gpt2_linear_opts og = o;  // fc: the epilogue stores the pre-activation and its GELU in one pass
    og.flags = GPT2L_EPI_GELU_DUAL;
    og.out2 = a.fc_gelu;
    CK(gpt2_linear_forward(a.fc, a.ln2, P + p.fc_w, P + p.fc_b, B, T, C, 4 * C, &og, stream));
    orr.aux = a.res2;
    CK(gpt2_linear_forward(a.res3, a.fc_gelu, P + p.fcproj_w, P + p.fcproj_b, B, T, 4 * C, C, &orr, stream));
    res = a.res3;
  }
  CK(layernorm_forward(m->lnf, m->lnf_mean, m->lnf_rstd, res, P + m->off_lnf_w, P + m->off_lnf_b, M, C, st));
  m->targets = targets;
  if (m->xent_path) {
    // loss and log-sum-exp come out of the lm_head's epilogue
    CK(gpt2_linear_forward_xent(m->logits, m->losses, m->xlse, m->lnf, P + m->off_wte, targets, B, T, C, Vp, V, &o, stream));
    if (m->xent_path == 1) CK(xent_grad_inplace(m->logits, m->xlse, targets, M, V, Vp, st));
  } else {
    CK(gpt2_linear_forward(m->logits, m->lnf, P + m->off_wte, nullptr, B, T, C, Vp, &o, stream));
    CK(softmax_xent(m->logits, m->losses, targets, M, V, Vp, st));
  }
  return GPT2L_OK;
}

// The backward pass in three parts, so that a data-parallel driver can hand each finished slice of
// the gradient buffer to the all-reduce while the next part computes.
int gpt2_model_backward_head(gpt2_model *m, gpt2l_stream_t stream) {
  if (!m || !m->tokens) return GPT2L_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int B = m->B, T = m->T, C = m->cfg.n_embd, L = m->cfg.n_layer;
  const int Vp = m->cfg.padded_vocab_size;
  const int M = B * T;
  float *P = m->params, *G = m->grads;
  gpt2_linear_opts o = opts_for(m);
  if (cudaMemsetAsync(G, 0, (size_t)m->n_params * sizeof(float), st) != cudaSuccess) return GPT2L_ERR_CUDA;
  if (cudaMemsetAsync(m->dresid, 0, (size_t)M * C * sizeof(float), st) != cudaSuccess) return GPT2L_ERR_CUDA;
  // lm_head: the logits buffer holds dlogits since the forward pass — or, with the fused cross-entropy, still
  // the logits, which the two GEMMs turn into dlogits tile by tile as they read them
  gpt2_linear_opts oh = o;
  if (m->xent_path == 2) {
    oh.xent_lse = m->xlse;
    oh.xent_targets = m->targets;
    oh.xent_vocab = m->cfg.vocab_size;
    oh.xent_scale = 1.f / (float)M;
  }
  CK(gpt2_linear_backward_input(m->tmp_c, m->logits, P + m->off_wte, B, T, C, Vp, &oh, stream));
  CK(gpt2_linear_backward_weight(G + m->off_wte, nullptr, m->logits, m->lnf, B, T, C, Vp, &oh, stream));
  const float *res_last = L > 0 ? m->la[L - 1].res3 : m->encoded;
  CK(layernorm_backward(m->dresid, G + m->off_lnf_w, G + m->off_lnf_b, m->tmp_c, res_last, P + m->off_lnf_w,
                        m->lnf_mean, m->lnf_rstd, M, C, st));
  return GPT2L_OK;
}

int gpt2_model_backward_layer(gpt2_model *m, int l, gpt2l_stream_t stream) {
  if (!m || !m->tokens || l < 0 || l >= m->cfg.n_layer) return GPT2L_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int B = m->B, T = m->T, C = m->cfg.n_embd, NH = m->cfg.n_head;
  const int M = B * T;
  float *P = m->params, *G = m->grads;
  gpt2_linear_opts o = opts_for(m);
  const LayerParams &p = m->lp[l];
  LayerActs &a = m->la[l];
  const float *res_in = l > 0 ? m->la[l - 1].res3 : m->encoded;
  // MLP: res3 = res2 + fcproj(gelu(fc(ln2(res2))))
  gpt2_linear_opts ogb = o;  // the GELU backward rides in the epilogue: dbig = (dresid . W^T) * gelu'(fc)
  ogb.aux_op = GPT2L_AUX_GELU_GRAD;
  ogb.aux = a.fc;
  CK(gpt2_linear_backward_input(m->dbig, m->dresid, P + p.fcproj_w, B, T, 4 * C, C, &ogb, stream));
  CK(gpt2_linear_backward_weight(G + p.fcproj_w, G + p.fcproj_b, m->dresid, a.fc_gelu, B, T, 4 * C, C, &o, stream));
  CK(gpt2_linear_backward_input(m->tmp_c, m->dbig, P + p.fc_w, B, T, C, 4 * C, &o, stream));
  CK(gpt2_linear_backward_weight(G + p.fc_w, G + p.fc_b, m->dbig, a.ln2, B, T, C, 4 * C, &o, stream));
  CK(layernorm_backward(m->dresid, G + p.ln2_w, G + p.ln2_b, m->tmp_c, a.res2, P + p.ln2_w, a.ln2_mean, a.ln2_rstd,
                        M, C, st));
  // attention: res2 = res_in + proj(attention(qkv(ln1(res_in))))
  CK(gpt2_linear_backward_input(m->tmp_c, m->dresid, P + p.proj_w, B, T, C, C, &o, stream));
  CK(gpt2_linear_backward_weight(G + p.proj_w, G + p.proj_b, m->dresid, a.atty, B, T, C, C, &o, stream));
  if (m->attn_flash) CK(attention_flash_backward(m->dbig, m->delta, m->tmp_c, a.atty, a.qkv, a.lse, B, T, C, NH, st));
  else if (m->attn_gemm) CK(attention_backward_gemm(m->dbig, m->datt, m->delta, m->tmp_c, a.atty, a.att, a.qkv, B, T, C, NH, m->mode, st));
  else CK(attention_backward(m->dbig, m->delta, m->tmp_c, a.atty, a.qkv, a.lse, B, T, C, NH, st));
  CK(gpt2_linear_backward_input(m->tmp_c, m->dbig, P + p.qkv_w, B, T, C, 3 * C, &o, stream));
  CK(gpt2_linear_backward_weight(G + p.qkv_w, G + p.qkv_b, m->dbig, a.ln1, B, T, C, 3 * C, &o, stream));
  CK(layernorm_backward(m->dresid, G + p.ln1_w, G + p.ln1_b, m->tmp_c, res_in, P + p.ln1_w, a.ln1_mean, a.ln1_rstd,
                        M, C, st));
  return GPT2L_OK;
}

int gpt2_model_backward_embedding(gpt2_model *m, gpt2l_stream_t stream) {
  if (!m || !m->tokens) return GPT2L_ERR_BAD_ARG;
  return embedding_backward(m->grads + m->off_wte, m->grads + m->off_wpe, m->dresid, m->tokens, m->B, m->T,
                            m->cfg.n_embd, m->cfg.padded_vocab_size, static_cast<cudaStream_t>(stream));
}

int gpt2_model_backward(gpt2_model *m, gpt2l_stream_t stream) {
  if (!m) return GPT2L_ERR_BAD_ARG;
  CK(gpt2_model_backward_head(m, stream));
  for (int l = m->cfg.n_layer - 1; l >= 0; --l) CK(gpt2_model_backward_layer(m, l, stream));
  return gpt2_model_backward_embedding(m, stream);
}

// Forward + backward replayed from a CUDA graph: at small shapes (the reference's B=4, T=64) the step is
// ~250 short launches plus the host-side tensor-map encoding of 147 GEMM calls, and the GPU waits for
// the host; a graph replays the whole step with one call. Kernel parameters (tensor maps, pointers,
// tilings) are frozen at capture, so the graph is rebuilt when the token / target pointers change.
int gpt2_model_forward_backward_graph(gpt2_model *m, const int *tokens, const int *targets, gpt2l_stream_t stream) {
  if (!m || !tokens || !targets) return GPT2L_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!m->eager_done) {
    // workspaces, scratch and function attributes are set up lazily by the first calls: not under capture
    CK(gpt2_model_forward(m, tokens, targets, stream));
    CK(gpt2_model_backward(m, stream));
    m->eager_done = true;
    return GPT2L_OK;
  }
  if (!m->graph_exec || tokens != m->g_tokens || targets != m->g_targets) {
    if (m->graph_exec) cudaGraphExecDestroy(m->graph_exec);
    if (m->graph) cudaGraphDestroy(m->graph);
    m->graph_exec = nullptr;
    m->graph = nullptr;
    if (!m->cap_stream && cudaStreamCreateWithFlags(&m->cap_stream, cudaStreamNonBlocking) != cudaSuccess)
      return GPT2L_ERR_CUDA;
    if (cudaStreamBeginCapture(m->cap_stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) return GPT2L_ERR_CUDA;
    int e = gpt2_model_forward(m, tokens, targets, m->cap_stream);
    if (e == GPT2L_OK) e = gpt2_model_backward(m, m->cap_stream);
    const cudaError_t ce = cudaStreamEndCapture(m->cap_stream, &m->graph);
    if (e != GPT2L_OK || ce != cudaSuccess) {
      if (m->graph) cudaGraphDestroy(m->graph);
      m->graph = nullptr;
      (void)cudaGetLastError();
      return e != GPT2L_OK ? e : GPT2L_ERR_CUDA;
    }
    if (cudaGraphInstantiate(&m->graph_exec, m->graph, 0) != cudaSuccess) return GPT2L_ERR_CUDA;
    m->g_tokens = tokens;
    m->g_targets = targets;
  }
  m->tokens = tokens;
  return cudaGraphLaunch(m->graph_exec, st) == cudaSuccess ? GPT2L_OK : GPT2L_ERR_CUDA;
}

int gpt2_model_update(gpt2_model *m, float lr, float beta1, float beta2, float eps, float weight_decay, int t,
                      gpt2l_stream_t stream) {
  if (!m || t < 1) return GPT2L_ERR_BAD_ARG;
  return adamw_update(m->params, m->m1, m->m2, m->grads, m->n_params, lr, beta1, beta2, eps, weight_decay, t,
                      static_cast<cudaStream_t>(stream));
}

int gpt2_model_update_range(gpt2_model *m, long long first, long long count, float lr, float beta1, float beta2,
                            float eps, float weight_decay, int t, gpt2l_stream_t stream) {
  if (!m || t < 1 || first < 0 || count < 0 || first + count > m->n_params) return GPT2L_ERR_BAD_ARG;
  if (count == 0) return GPT2L_OK;
  return adamw_update(m->params + first, m->m1 + first, m->m2 + first, m->grads + first, count, lr, beta1, beta2, eps,
                      weight_decay, t, static_cast<cudaStream_t>(stream));
}

float gpt2_model_mean_loss(gpt2_model *m, gpt2l_stream_t stream) {
  if (!m) return NAN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long M = (long long)m->B * m->T;
  if (cudaMemcpyAsync(m->h_losses, m->losses, (size_t)M * sizeof(float), cudaMemcpyDeviceToHost, st) != cudaSuccess)
    return NAN;
  if (cudaStreamSynchronize(st) != cudaSuccess) return NAN;
  // a bounded wait that gave up inside an attention kernel leaves garbage behind: report it
  if (m->attn_flash && attention_flash_status() != 0) return NAN;
  double s = 0.0;
  for (long long i = 0; i < M; ++i) s += m->h_losses[i];
  return (float)(s / (double)M);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Files. A weight file is the reference's: headerless fp32, tensors in parameter order, wte as
// [C][V] with the true vocabulary (no pad columns). In memory wte rows are padded_vocab_size long,
// so the copy goes row by row through a host image of the flat buffer.
// ---------------------------------------------------------------------------------------------
namespace {

long long file_floats(const gpt2_model *m) {
  return m->n_params - (long long)m->cfg.n_embd * (m->cfg.padded_vocab_size - m->cfg.vocab_size);
}

// one flat device buffer -> file section
int write_section(const gpt2_model *m, const float *dev, FILE *f, std::vector<float> &host) {
  host.resize((size_t)m->n_params);
  if (cudaMemcpy(host.data(), dev, host.size() * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess)
    return GPT2L_ERR_CUDA;
  const int C = m->cfg.n_embd, V = m->cfg.vocab_size, Vp = m->cfg.padded_vocab_size;
  for (int c = 0; c < C; ++c)
    if (fwrite(host.data() + m->off_wte + (size_t)c * Vp, sizeof(float), (size_t)V, f) != (size_t)V) return GPT2M_ERR_IO;
  const size_t rest = (size_t)(m->n_params - m->off_wpe);
  return fwrite(host.data() + m->off_wpe, sizeof(float), rest, f) == rest ? GPT2L_OK : GPT2M_ERR_IO;
}

// file section -> one flat device buffer (pad columns zero)
int read_section(const gpt2_model *m, float *dev, FILE *f, std::vector<float> &host) {
  host.assign((size_t)m->n_params, 0.f);
  const int C = m->cfg.n_embd, V = m->cfg.vocab_size, Vp = m->cfg.padded_vocab_size;
  for (int c = 0; c < C; ++c)
    if (fread(host.data() + m->off_wte + (size_t)c * Vp, sizeof(float), (size_t)V, f) != (size_t)V) return GPT2M_ERR_IO;
  const size_t rest = (size_t)(m->n_params - m->off_wpe);
  if (fread(host.data() + m->off_wpe, sizeof(float), rest, f) != rest) return GPT2M_ERR_IO;
  return cudaMemcpy(dev, host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice) == cudaSuccess
             ? GPT2L_OK : GPT2L_ERR_CUDA;
}

long long size_of_file(FILE *f) {
  if (fseek(f, 0, SEEK_END) != 0) return -1;
  const long long n = ftell(f);
  rewind(f);
  return n;
}

struct CheckpointHeader {  // 64 bytes, little-endian ints
  char magic[8];           // "G2CKPT1\0"
  int vocab_size, n_layer, n_head, n_embd, n_positions;
  int step;                // AdamW steps taken so far: the next update runs with t = step + 1
  long long floats_per_section;
  int reserved[6];
};
static_assert(sizeof(CheckpointHeader) == 64, "header layout");
const char kMagic[8] = {'G', '2', 'C', 'K', 'P', 'T', '1', 0};

}  // namespace

extern "C" {

int gpt2_model_load_weights(gpt2_model *m, const char *path) {
  if (!m || !path) return GPT2L_ERR_BAD_ARG;
  FILE *f = fopen(path, "rb");
  if (!f) return GPT2M_ERR_IO;
  std::vector<float> host;
  int rc = size_of_file(f) == file_floats(m) * (long long)sizeof(float) ? GPT2L_OK : GPT2M_ERR_FORMAT;
  if (rc == GPT2L_OK) rc = read_section(m, m->params, f, host);
  fclose(f);
  return rc;
}

int gpt2_model_dump_weights(gpt2_model *m, const char *path) {
  if (!m || !path) return GPT2L_ERR_BAD_ARG;
  FILE *f = fopen(path, "wb");
  if (!f) return GPT2M_ERR_IO;
  std::vector<float> host;
  int rc = write_section(m, m->params, f, host);
  if (fclose(f) != 0 && rc == GPT2L_OK) rc = GPT2M_ERR_IO;
  return rc;
}

int gpt2_model_save_checkpoint(gpt2_model *m, const char *path, int step) {
  if (!m || !path || step < 0) return GPT2L_ERR_BAD_ARG;
  FILE *f = fopen(path, "wb");
  if (!f) return GPT2M_ERR_IO;
  CheckpointHeader h;
  memset(&h, 0, sizeof(h));
  memcpy(h.magic, kMagic, 8);
  h.vocab_size = m->cfg.vocab_size; h.n_layer = m->cfg.n_layer; h.n_head = m->cfg.n_head;
  h.n_embd = m->cfg.n_embd; h.n_positions = m->cfg.n_positions; h.step = step;
  h.floats_per_section = file_floats(m);
  int rc = fwrite(&h, sizeof(h), 1, f) == 1 ? GPT2L_OK : GPT2M_ERR_IO;
  std::vector<float> host;
  const float *sections[3] = {m->params, m->m1, m->m2};
  for (int i = 0; i < 3 && rc == GPT2L_OK; ++i) rc = write_section(m, sections[i], f, host);
  if (fclose(f) != 0 && rc == GPT2L_OK) rc = GPT2M_ERR_IO;
  return rc;
}

int gpt2_model_load_checkpoint(gpt2_model *m, const char *path, int *step) {
  if (!m || !path) return GPT2L_ERR_BAD_ARG;
  FILE *f = fopen(path, "rb");
  if (!f) return GPT2M_ERR_IO;
  CheckpointHeader h;
  int rc = GPT2L_OK;
  const long long bytes = size_of_file(f);
  if (fread(&h, sizeof(h), 1, f) != 1 || memcmp(h.magic, kMagic, 8) != 0) rc = GPT2M_ERR_FORMAT;
  if (rc == GPT2L_OK &&
      (h.vocab_size != m->cfg.vocab_size || h.n_layer != m->cfg.n_layer || h.n_head != m->cfg.n_head ||
       h.n_embd != m->cfg.n_embd || h.n_positions != m->cfg.n_positions || h.step < 0 ||
       h.floats_per_section != file_floats(m) ||
       bytes != (long long)sizeof(h) + 3 * h.floats_per_section * (long long)sizeof(float)))
    rc = GPT2M_ERR_FORMAT;
  std::vector<float> host;
  float *sections[3] = {m->params, m->m1, m->m2};
  // a file that fails the checks above leaves the model untouched; a read error below does not
  for (int i = 0; i < 3 && rc == GPT2L_OK; ++i) rc = read_section(m, sections[i], f, host);
  fclose(f);
  if (rc == GPT2L_OK && step) *step = h.step;
  return rc;
}

}  // extern "C"
