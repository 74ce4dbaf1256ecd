// TEST INFRASTRUCTURE — NOT PART OF THE PRODUCT.
//
// C entry points around the reference's own, unmodified GEMM kernels. This file contains no
// reference code: it includes the reference's header from where the reference tree is mounted
// (the include path is given by oracle/Makefile) and launches its three __global__ templates
// with the reference's own launch macros, exactly as src/train.cu:356 / :404 / :405 do.
// The resulting library (oracle/_ref/libref_mlp.so) is the "reference run here": the parity
// tests compare the new kernels, the CPU restatement and these kernels on the same inputs.
#include <cuda_runtime.h>

#include "gpt2/layers/mlp.h"

extern "C" {

int ref_mlp_forward(float *out, const float *in, const float *w, const float *b, int B, int S, int K, int N,
                    void *stream) {
  mlp_forward<TILE_SIZE><<<MLP_FORWARD_GRID(N, B, S), MLP_BLOCK_DIM, MLP_SHARED_MEM_SIZE,
                           static_cast<cudaStream_t>(stream)>>>(out, in, w, b, B, S, K, N);
  return (int)cudaGetLastError();
}

int ref_mlp_backward_input(float *g_in, const float *g_out, const float *w, int B, int S, int K, int N,
                           void *stream) {
  mlp_backward_input<TILE_SIZE><<<MLP_BACKWARD_INPUT_GRID(K, B, S), MLP_BLOCK_DIM, MLP_SHARED_MEM_SIZE,
                                  static_cast<cudaStream_t>(stream)>>>(g_in, g_out, w, B, S, K, N);
  return (int)cudaGetLastError();
}

int ref_mlp_backward_weight(float *g_w, float *g_b, const float *g_out, const float *in, int B, int S, int K,
                            int N, void *stream) {
  mlp_backward_weight<TILE_SIZE><<<MLP_BACKWARD_WEIGHT_GRID(N, K), MLP_BLOCK_DIM, MLP_SHARED_MEM_SIZE,
                                   static_cast<cudaStream_t>(stream)>>>(g_w, g_b, g_out, in, B, S, K, N);
  return (int)cudaGetLastError();
}

int ref_sync(void) { return (int)cudaDeviceSynchronize(); }

}  // extern "C"
