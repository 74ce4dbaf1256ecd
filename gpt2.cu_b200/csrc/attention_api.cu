// C ABI of the attention layer (include/gpt2_attention.h): argument checks and dispatch to the
// three implementations.
#include <cuda_runtime.h>

#include "gpt2_attention.h"
#include "layers.h"
#include "linear_internal.h"

using namespace g2l;

extern "C" {

int gpt2_attention_supported(int impl, int T, int C, int NH) {
  if (T <= 0 || C <= 0 || NH <= 0 || C != NH * 64) return 0;
  switch (impl) {
    case GPT2A_FLASH: return attention_flash_supported(T, C, NH) ? 1 : 0;
    case GPT2A_GEMM: return attention_gemm_supported(T, C, NH) ? 1 : 0;
    case GPT2A_SIMT: return 1;
    default: return 0;
  }
}

int gpt2_attention_forward(float *out, float *lse, float *probs, const float *inp, int B, int T, int NH, int C,
                           int impl, int mode, gpt2l_stream_t stream) {
  if (!out || !inp || B <= 0 || !gpt2_attention_supported(impl, T, C, NH)) return GPT2L_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (impl) {
    case GPT2A_FLASH:
      if (!lse) return GPT2L_ERR_BAD_ARG;
      return attention_flash_forward(out, lse, inp, B, T, C, NH, st);
    case GPT2A_GEMM:
      if (!probs) return GPT2L_ERR_BAD_ARG;
      return attention_forward_gemm(out, probs, inp, B, T, C, NH, mode, st);
    default:
      if (!lse) return GPT2L_ERR_BAD_ARG;
      return attention_forward(out, lse, inp, B, T, C, NH, st);
  }
}

int gpt2_attention_backward(float *g_inp, const float *g_out, const float *inp, const float *out, const float *lse,
                            const float *probs, float *row_scratch, float *tt_scratch, int B, int T, int C, int NH,
                            int impl, int mode, gpt2l_stream_t stream) {
  if (!g_inp || !g_out || !inp || !out || !row_scratch || B <= 0 || !gpt2_attention_supported(impl, T, C, NH))
    return GPT2L_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (impl) {
    case GPT2A_FLASH:
      if (!lse) return GPT2L_ERR_BAD_ARG;
      return attention_flash_backward(g_inp, row_scratch, g_out, out, inp, lse, B, T, C, NH, st);
    case GPT2A_GEMM:
      if (!probs || !tt_scratch) return GPT2L_ERR_BAD_ARG;
      return attention_backward_gemm(g_inp, tt_scratch, row_scratch, g_out, out, probs, inp, B, T, C, NH, mode, st);
    default:
      if (!lse) return GPT2L_ERR_BAD_ARG;
      return attention_backward(g_inp, row_scratch, g_out, out, inp, lse, B, T, C, NH, st);
  }
}

int gpt2_attention_status(void) { return attention_flash_status(); }

}  // extern "C"
