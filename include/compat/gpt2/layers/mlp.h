/*
 * Compatibility header: put this directory ahead of the reference's include/ on the include path and
 * `#include "gpt2/layers/mlp.h"` resolves here (same include guard, so the reference's copy is
 * shadowed even when it is reached through another path).
 *
 * It keeps the names the reference's host code uses for the linear layer (include/gpt2/layers/mlp.h:
 * TILE_SIZE :9, MLP_FORWARD_GRID :12, MLP_BACKWARD_INPUT_GRID :16, MLP_BACKWARD_WEIGHT_GRID :20,
 * MLP_BLOCK_DIM :25, MLP_SHARED_MEM_SIZE :28, mlp_forward :336, mlp_backward_input :653,
 * mlp_backward_weight :998) with the same argument order and meaning, but the three kernel names are
 * host launchers here: a <<<grid, block, smem>>> launch cannot carry TMA descriptors, so a call site
 *
 *     mlp_forward<TILE_SIZE><<<MLP_FORWARD_GRID(N, B, S), MLP_BLOCK_DIM, MLP_SHARED_MEM_SIZE>>>(out, in, w, b, B, S, K, N);
 * becomes
 *     mlp_forward<TILE_SIZE>(out, in, w, b, B, S, K, N);
 *
 * The geometry macros stay defined (the reference's scheduler counts 32 x 32 tiles with them) but no
 * launch consumes them. Work goes to the stream set with gpt2l_compat_set_stream (default: the
 * legacy default stream, as in the reference); the arithmetic mode is GPT2L_COMPAT_MODE. Each
 * launcher returns the library's status code; the reference's kernels return nothing, so existing
 * call sites that ignore it keep compiling. gpt2_linear_init(device) must have run first.
 */
#ifndef GPT2_LAYERS_MLP_H
#define GPT2_LAYERS_MLP_H

#include <cuda_runtime.h>

#include "gpt2_linear.h"

#ifndef GPT2L_COMPAT_MODE
#define GPT2L_COMPAT_MODE GPT2L_MODE_TF32X3 /* closest to the reference's fp32 results */
#endif

#define TILE_SIZE 32

static inline dim3 gpt2l_compat_tiles(int cols, int rows) {
  return dim3((unsigned)((cols + TILE_SIZE - 1) / TILE_SIZE), (unsigned)((rows + TILE_SIZE - 1) / TILE_SIZE));
}
#define MLP_FORWARD_GRID(output_dim, batch_size, seq_len) gpt2l_compat_tiles((output_dim), (batch_size) * (seq_len))
#define MLP_BACKWARD_INPUT_GRID(input_dim, batch_size, seq_len) gpt2l_compat_tiles((input_dim), (batch_size) * (seq_len))
#define MLP_BACKWARD_WEIGHT_GRID(output_dim, input_dim) gpt2l_compat_tiles((output_dim), (input_dim))
#define MLP_BLOCK_DIM dim3(256)
#define MLP_SHARED_MEM_SIZE ((size_t)16384)

static inline cudaStream_t &gpt2l_compat_stream_ref() {
  static cudaStream_t s = nullptr;
  return s;
}
static inline void gpt2l_compat_set_stream(cudaStream_t s) { gpt2l_compat_stream_ref() = s; }

static inline gpt2_linear_opts gpt2l_compat_opts() {
  gpt2_linear_opts o = {};
  o.mode = GPT2L_COMPAT_MODE;
  return o;
}

template <int MLP_TILE>
inline int mlp_forward(float *out, const float *input, const float *w, const float *b, int batch_size, int seq_len,
                       int input_dim, int output_dim) {
  const gpt2_linear_opts o = gpt2l_compat_opts();
  return gpt2_linear_forward(out, input, w, b, batch_size, seq_len, input_dim, output_dim, &o,
                             (gpt2l_stream_t)gpt2l_compat_stream_ref());
}

template <int MLP_TILE>
inline int mlp_backward_input(float *g_input, const float *g_out, const float *weight, int batch_size, int seq_len,
                              int input_dim, int output_dim) {
  const gpt2_linear_opts o = gpt2l_compat_opts();
  return gpt2_linear_backward_input(g_input, g_out, weight, batch_size, seq_len, input_dim, output_dim, &o,
                                    (gpt2l_stream_t)gpt2l_compat_stream_ref());
}

template <int MLP_TILE>
inline int mlp_backward_weight(float *g_weight, float *g_bias, const float *g_out, const float *input, int batch_size,
                               int seq_len, int input_dim, int output_dim) {
  const gpt2_linear_opts o = gpt2l_compat_opts();
  return gpt2_linear_backward_weight(g_weight, g_bias, g_out, input, batch_size, seq_len, input_dim, output_dim, &o,
                                     (gpt2l_stream_t)gpt2l_compat_stream_ref());
}

#endif /* GPT2_LAYERS_MLP_H */
