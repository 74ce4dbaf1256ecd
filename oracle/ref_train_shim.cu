// TEST INFRASTRUCTURE — NOT PART OF THE PRODUCT.
//
// C entry points around the reference's own, unmodified training step ("Path A": separate kernel
// launches): gpt2_initialize, setup_train_buffers, forward, cross_entropy, gpt2_zero_grad,
// zero_activation_grads, backward, gpt2_update, called in the order of tests/test_train.cu:283-301 of
// the reference. This file contains no reference code: it includes the reference's headers from where
// the reference tree is mounted and is linked with the reference's src/*.cu compiled by oracle/Makefile.
// The reference's pretrained weight file is not available, so the parameters are filled with seeded
// values (normal, std 0.02; layernorm weights 1, every bias 0), the same way for any caller.
// The resulting library (oracle/_ref/libref_train.so) gives the step time of the reference on this GPU.
// Compiled a second time with -DREF_TRAIN_B200, against a copy of src/train.cu whose 15 linear-layer
// launch sites call the launchers of include/compat/gpt2/layers/mlp.h, it becomes
// oracle/_ref/libref_train_b200.so: the reference's host code and layer kernels around this library's GEMMs.
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>

#include <random>
#include <vector>

#include "gpt2/gpt2.h"
#include "gpt2/train.h"
#include "gpt2/layers/attention.h"
#ifdef REF_TRAIN_B200
#include "gpt2_linear.h"
#endif

namespace {
config_t g_cfg;
gpt2_t g_model, g_grads;
train_buffers_t g_buf, g_gbuf;
adamw_state_t g_opt;
int g_B = 0, g_S = 0;
bool g_ready = false;

void fill(tensor_t &t, std::mt19937 &rng, float std_, float constant, bool use_constant) {
  const int n = tensor_size(t);
  std::vector<float> h((size_t)n);
  std::normal_distribution<float> d(0.f, std_);
  for (int i = 0; i < n; ++i) h[i] = use_constant ? constant : d(rng);
  cudaMemcpy(t.data, h.data(), (size_t)n * sizeof(float), cudaMemcpyHostToDevice);
}
}  // namespace

extern "C" {

// GPT-2 small with batch B and sequence length S; returns 0 on success
int ref_train_create(int B, int S, unsigned seed) {
  if (g_ready) return -1;
#ifdef REF_TRAIN_B200
  {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || gpt2_linear_init(dev) != 0) return -7;
  }
#endif
  g_cfg.vocab_size = VOCAB_SIZE;
  g_cfg.batch_size = B;
  g_cfg.n_layer = NUM_LAYERS;
  g_cfg.n_head = NUM_HEADS;
  g_cfg.n_embd = EMBEDDING_SIZE;
  g_cfg.n_positions = CONTEXT_SIZE;
  g_cfg.n_ctx = CONTEXT_SIZE;
  if (gpt2_initialize(&g_model, &g_cfg) != 0) return -2;
  if (gpt2_initialize(&g_grads, &g_cfg) != 0) return -3;
  std::mt19937 rng(seed);
  fill(g_model.emb.wte, rng, 0.02f, 0.f, false);
  fill(g_model.emb.wpe, rng, 0.02f, 0.f, false);
  for (int l = 0; l < NUM_LAYERS; ++l) {
    block_t &b = g_model.h[l];
    fill(b.ln_1.w, rng, 0.f, 1.f, true);  fill(b.ln_1.b, rng, 0.f, 0.f, true);
    fill(b.attn.qkv_w, rng, 0.02f, 0.f, false);  fill(b.attn.qkv_b, rng, 0.f, 0.f, true);
    fill(b.attn.proj_w, rng, 0.02f, 0.f, false); fill(b.attn.proj_b, rng, 0.f, 0.f, true);
    fill(b.ln_2.w, rng, 0.f, 1.f, true);  fill(b.ln_2.b, rng, 0.f, 0.f, true);
    fill(b.mlp.fc_w, rng, 0.02f, 0.f, false);    fill(b.mlp.fc_b, rng, 0.f, 0.f, true);
    fill(b.mlp.proj_w, rng, 0.02f, 0.f, false);  fill(b.mlp.proj_b, rng, 0.f, 0.f, true);
  }
  fill(g_model.ln_f.w, rng, 0.f, 1.f, true);
  fill(g_model.ln_f.b, rng, 0.f, 0.f, true);
  if (setup_train_buffers(g_cfg, &g_buf, S) != 0) return -4;
  if (setup_train_buffers(g_cfg, &g_gbuf, S) != 0) return -5;
  g_opt.learning_rate = 1e-4f; g_opt.beta1 = 0.9f; g_opt.beta2 = 0.999f; g_opt.eps = 1e-8f;
  g_opt.weight_decay = 0.01f; g_opt.t = 0; g_opt.m_memory = nullptr; g_opt.v_memory = nullptr;
  g_B = B; g_S = S;
  g_ready = cudaDeviceSynchronize() == cudaSuccess;
  return g_ready ? 0 : -6;
}

long long ref_train_num_params(void) { return g_ready ? (long long)g_model.num_parameters : -1; }

// overwrite all parameters from a host vector in the reference's order (wte as [768][50257])
int ref_train_set_params(const float *host, long long n) {
  if (!g_ready || n != (long long)g_model.num_parameters) return -1;
  return (int)cudaMemcpy(g_model.params_memory, host, (size_t)n * sizeof(float), cudaMemcpyHostToDevice);
}

// one training step on device tokens / targets [B*S]; returns the mean loss of the forward pass
float ref_train_step(const int *d_tokens, const int *d_targets) {
  if (!g_ready) return -1.f;
  forward(g_cfg, g_model, g_buf, d_tokens, g_S);
  cross_entropy(g_cfg, g_buf, d_targets, g_S);
  const float loss = compute_mean_loss(&g_buf.losses, g_B, g_S);
  gpt2_zero_grad(&g_grads);
  zero_activation_grads(g_cfg, &g_gbuf);
  backward(g_cfg, g_model, g_buf, g_grads, g_gbuf, d_tokens, d_targets, g_S);
  gpt2_update(&g_model, &g_grads, &g_opt);
  return loss;
}

int ref_train_sync(void) { return (int)cudaDeviceSynchronize(); }

// forward + loss + backward without the optimizer step; the gradients stay in the gradient model
float ref_train_forward_backward(const int *d_tokens, const int *d_targets) {
  if (!g_ready) return -1.f;
  forward(g_cfg, g_model, g_buf, d_tokens, g_S);
  cross_entropy(g_cfg, g_buf, d_targets, g_S);
  const float loss = compute_mean_loss(&g_buf.losses, g_B, g_S);
  gpt2_zero_grad(&g_grads);
  zero_activation_grads(g_cfg, &g_gbuf);
  backward(g_cfg, g_model, g_buf, g_grads, g_gbuf, d_tokens, d_targets, g_S);
  return cudaDeviceSynchronize() == cudaSuccess ? loss : -2.f;
}

// all parameter gradients to a host vector, in the reference's parameter order
int ref_train_get_grads(float *host, long long n) {
  if (!g_ready || n != (long long)g_grads.num_parameters) return -1;
  return (int)cudaMemcpy(host, g_grads.params_memory, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost);
}

// The reference's attention kernels on caller-owned device buffers, launched the way src/train.cu:358 and
// :439 launch them. out [B*T][C]; preatt, att, g_preatt, g_att [B][NH][T][T]; inp, g_inp [B*T][3C];
// g_out [B*T][C]. The backward kernel accumulates into g_inp, which the reference zeroes once per step
// (zero_activation_grads); it is zeroed here. Both return the CUDA error code after synchronising.
int ref_attention_forward(float *out, float *preatt, float *att, const float *inp, int B, int T, int NH, int C) {
  attention_forward<<<ATTN_FWD_GRID(B, T, NH), ATTN_FWD_BLOCK(), ATTN_FWD_SMEM(T, C / NH)>>>(out, preatt, att, inp, B, T,
                                                                                            NH, C);
  return (int)cudaDeviceSynchronize();
}

int ref_attention_backward(float *g_inp, float *g_preatt, float *g_att, const float *g_out, const float *inp,
                           const float *att, int B, int T, int C, int NH) {
  const size_t tt = (size_t)B * NH * T * T * sizeof(float);
  cudaMemset(g_inp, 0, (size_t)B * T * 3 * C * sizeof(float));
  cudaMemset(g_preatt, 0, tt);
  cudaMemset(g_att, 0, tt);
  attention_backward<<<ATTN_BWD_GRID(B, T, NH), ATTN_BWD_BLOCK(), ATTN_BWD_SMEM(T, C / NH)>>>(g_inp, g_preatt, g_att, g_out,
                                                                                             inp, att, B, T, C, NH);
  return (int)cudaDeviceSynchronize();
}

}  // extern "C"
