// Launchers of the non-GEMM layers (layers.cu). All take device pointers and a stream and return a
// GPT2L_* code.
#pragma once
#include <cuda_runtime.h>

namespace g2l {

int embedding_forward(float *out, const int *tokens, const float *wte, const float *wpe, int B, int T, int C, int Vp,
                      cudaStream_t s);
int embedding_backward(float *g_wte, float *g_wpe, const float *g, const int *tokens, int B, int T, int C, int Vp,
                       cudaStream_t s);
int layernorm_forward(float *out, float *mean, float *rstd, const float *in, const float *w, const float *b, int M,
                      int C, cudaStream_t s);
int layernorm_backward(float *g_in, float *g_w, float *g_b, const float *g_out, const float *in, const float *w,
                       const float *mean, const float *rstd, int M, int C, cudaStream_t s);
int add_forward(float *out, const float *a, const float *b, long long n, cudaStream_t s);
int gelu_backward(float *g, const float *pre, long long n, cudaStream_t s);
int softmax_xent(float *logits, float *losses, const int *targets, int M, int V, int Vp, cudaStream_t s);
// logits <- gradient of the mean cross-entropy, in place, from the rows' base-2 log-sum-exp (one read, one write)
int xent_grad_inplace(float *logits, const float *lse, const int *targets, int M, int V, int Vp, cudaStream_t s);
int attention_forward(float *out, float *lse, const float *qkv, int B, int T, int C, int NH, cudaStream_t s);
int attention_backward(float *dqkv, float *delta, const float *dout, const float *out, const float *qkv,
                       const float *lse, int B, int T, int C, int NH, cudaStream_t s);
int adamw_update(float *p, float *m, float *v, const float *g, long long n, float lr, float b1, float b2, float eps,
                 float wd, int t, cudaStream_t s);

// attention on the tensor cores (attention_gemm.cu); needs T % 32 == 0 and head size 64
bool attention_gemm_supported(int T, int C, int NH);
int attention_forward_gemm(float *out, float *P, const float *qkv, int B, int T, int C, int NH, int mode,
                           cudaStream_t s);
int attention_backward_gemm(float *dqkv, float *dP, float *delta, const float *dout, const float *out, const float *P,
                            const float *qkv, int B, int T, int C, int NH, int mode, cudaStream_t st);

int attention_row_dot(float *delta, const float *dout, const float *out, int B, int T, int C, int NH, cudaStream_t st);

// attention without T x T tensors (attention_flash.cu); needs T % 128 == 0 and head size 64. lse is
// [B][NH][T] (base-2 log-sum-exp of the scaled scores), written by the forward pass and read by the
// backward pass; delta is scratch of the same size. attention_flash_status() returns 0, or the
// number of the wait that gave up in a kernel (bounded waits), or -1 when it cannot be read.
bool attention_flash_supported(int T, int C, int NH);
int attention_flash_forward(float *out, float *lse, const float *qkv, int B, int T, int C, int NH, cudaStream_t st);
int attention_flash_backward(float *dqkv, float *delta, const float *dout, const float *out, const float *qkv,
                             const float *lse, int B, int T, int C, int NH, cudaStream_t st);
int attention_flash_backward_core(float *dqkv, const float *delta, const float *dout, const float *qkv,
                                  const float *lse, int B, int T, int C, int NH, cudaStream_t st);
int attention_flash_status();

}  // namespace g2l
