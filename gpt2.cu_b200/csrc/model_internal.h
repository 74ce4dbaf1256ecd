// The model object behind include/gpt2_model.h, shared by model.cu (separate launches per layer) and
// step_schedule.cu (the same step as a schedule of the persistent kernel).
#pragma once

#include <cuda_runtime.h>

#include <vector>

#include "gpt2_model.h"

namespace g2l {

struct LayerParams {  // offsets into the flat parameter / gradient buffers
  long long ln1_w, ln1_b, qkv_w, qkv_b, proj_w, proj_b, ln2_w, ln2_b, fc_w, fc_b, fcproj_w, fcproj_b;
};

struct LayerActs {  // device pointers into the activation buffer
  float *ln1, *ln1_mean, *ln1_rstd, *qkv, *atty, *lse, *res2, *ln2, *ln2_mean, *ln2_rstd, *fc, *fc_gelu, *res3;
  float *att;  // [B][NH][T][T] attention probabilities (tensor-core attention only)
};

}  // namespace g2l

struct gpt2_model {
  gpt2_model_config cfg;
  int B = 0, T = 0, mode = 0;
  long long n_params = 0;
  long long off_wte = 0, off_wpe = 0, off_lnf_w = 0, off_lnf_b = 0;
  std::vector<g2l::LayerParams> lp;
  std::vector<long long> tensor_offsets;
  float *params = nullptr, *grads = nullptr, *m1 = nullptr, *m2 = nullptr;
  float *acts = nullptr;
  long long acts_floats = 0;
  float *encoded = nullptr, *lnf = nullptr, *lnf_mean = nullptr, *lnf_rstd = nullptr, *logits = nullptr,
        *losses = nullptr;
  float *xlse = nullptr;     // [M] base-2 log-sum-exp of the logits rows (fused lm_head + cross-entropy)
  // how the loss is computed: 0 = a softmax / cross-entropy kernel over the logits after the lm_head;
  // 1 = statistics in the lm_head's epilogue, then one elementwise pass that turns the logits into their gradient;
  // 2 = statistics in the epilogue and the gradient formed inside the two backward GEMMs (no pass of its own)
  int xent_path = 0;
  const int *targets = nullptr;  // of the last forward
  float *tmp_c = nullptr;    // [M][C]   GEMM output before a residual add / small gradient scratch
  float *dresid = nullptr;   // [M][C]   gradient of the residual stream
  float *dbig = nullptr;     // [M][4C]  gradient scratch (d_fc, d_qkv)
  float *delta = nullptr;    // [B][NH][T]
  float *datt = nullptr;     // [B][NH][T][T] gradient scratch (tensor-core attention only)
  bool attn_gemm = false;    // attention as batched GEMMs on the tensor cores
  bool attn_flash = false;   // attention as one fused tensor-core kernel per pass
  std::vector<g2l::LayerActs> la;
  const int *tokens = nullptr;  // of the last forward
  // forward + backward as a CUDA graph (gpt2_model_forward_backward_graph)
  bool eager_done = false;            // one eager pass has made every lazy allocation
  cudaStream_t cap_stream = nullptr;  // capture happens here (the legacy default stream cannot capture)
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t graph_exec = nullptr;
  const int *g_tokens = nullptr, *g_targets = nullptr;
  float *h_losses = nullptr;    // pinned
  long long device_bytes = 0;
};
