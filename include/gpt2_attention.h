/*
 * gpt2_attention.h — C ABI of causal multi-head self-attention (head size 64), the layer between the
 * QKV and the output-projection GEMMs of the path.
 *
 * Replaces attention_forward / attention_backward of vnnm404/gpt2.cu
 * (include/gpt2/layers/attention.h:26-30, src/layers/attention.cu:213-222, 366-375): same input
 * (`inp` = the QKV GEMM's output [B*T][3C], q | k | v, heads side by side) and output ([B*T][C]); the
 * argument order follows the reference (forward ... B, T, NH, C; backward ... B, T, C, NH). The
 * reference's preatt / att / g_preatt / g_att tensors ([B][NH][T][T]) are not part of the contract of
 * the fused implementation, which keeps one value per row (lse) instead.
 *
 * Implementations:
 *   GPT2A_FLASH  one fused tcgen05 kernel per pass, no T x T tensors; TF32; needs T % 128 == 0
 *   GPT2A_GEMM   batched causal GEMMs on the linear-layer kernel with the T x T probabilities kept
 *                (`probs`), TF32 or 3xTF32 (`mode`); needs T % 32 == 0
 *   GPT2A_SIMT   CUDA-core kernels, fp32, any T
 * Returns GPT2L_OK or a negative GPT2L_ERR_* code (GPT2L_ERR_BAD_ARG when the shape does not fit the
 * implementation). Requires gpt2_linear_init() on the device.
 */
#ifndef GPT2_ATTENTION_H
#define GPT2_ATTENTION_H

#include "gpt2_linear.h"

#ifdef __cplusplus
extern "C" {
#endif

enum gpt2a_impl { GPT2A_FLASH = 0, GPT2A_GEMM = 1, GPT2A_SIMT = 2 };

/* 1 when `impl` can run this shape */
int gpt2_attention_supported(int impl, int T, int C, int NH);

/* out[B*T][C]. lse[B][NH][T] is written by FLASH (base-2) and SIMT (natural log); probs[B][NH][T][T]
 * is written by GEMM. The one the implementation does not use may be NULL. */
int gpt2_attention_forward(float *out, float *lse, float *probs, const float *inp, int B, int T, int NH, int C,
                           int impl, int mode, gpt2l_stream_t stream);

/* g_inp[B*T][3C] (overwritten) from g_out[B*T][C]; out / lse / probs are the forward pass's.
 * row_scratch: [B][NH][T] floats (all implementations); tt_scratch: [B][NH][T][T] floats (GEMM only). */
int gpt2_attention_backward(float *g_inp, const float *g_out, const float *inp, const float *out, const float *lse,
                            const float *probs, float *row_scratch, float *tt_scratch, int B, int T, int C, int NH,
                            int impl, int mode, gpt2l_stream_t stream);

/* 0, or the number of the bounded wait that gave up inside a FLASH kernel; -1 if unreadable */
int gpt2_attention_status(void);

#ifdef __cplusplus
}
#endif
#endif /* GPT2_ATTENTION_H */
