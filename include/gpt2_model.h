/*
 * gpt2_model.h — C ABI of the GPT-2 training step built around the linear-layer GEMM path.
 *
 * This is the caller side of the hot path: what src/train.cu of vnnm404/gpt2.cu does with
 * setup_train_buffers / forward / cross_entropy / backward / gpt2_update / gpt2_zero_grad /
 * compute_mean_loss (include/gpt2/train.h:49-58), with the reference's parameter order and tensor
 * layouts (src/gpt2.cu:48-198: wte[C][V], wpe[n_positions][C], then per layer ln_1.w, ln_1.b,
 * qkv_w[C][3C], qkv_b, proj_w[C][C], proj_b, ln_2.w, ln_2.b, fc_w[C][4C], fc_b, fcproj_w[4C][C],
 * fcproj_b, then ln_f.w, ln_f.b), every linear weight stored [in][out]. The vocabulary dimension of
 * wte and of the logits is padded (50257 -> 50304) so that the lm_head GEMMs run on the tensor cores;
 * pad columns of wte are kept at zero.
 *
 * All 15 GEMM kinds of a step go through gpt2_linear_forward / _backward_input / _backward_weight;
 * the other layers are CUDA-core kernels of this library (attention is flash-style: no [B,NH,T,T]
 * tensors). Requires gpt2_linear_init() on the device first.
 */
#ifndef GPT2_MODEL_H
#define GPT2_MODEL_H

#include "gpt2_linear.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct gpt2_model_config {
  int vocab_size;        /* 50257                                          */
  int padded_vocab_size; /* row stride of wte / logits, multiple of 4      */
  int n_layer;
  int n_head;            /* n_embd / n_head must be 64                     */
  int n_embd;
  int n_positions;       /* rows of wpe (1024)                             */
} gpt2_model_config;

typedef struct gpt2_model gpt2_model; /* opaque: parameters, gradients, AdamW moments, activations */

/* Allocates everything for batches of B sequences of T tokens. mode = enum gpt2l_mode for every
 * GEMM. Parameters start at zero: fill them with gpt2_model_set_params. */
gpt2_model *gpt2_model_create(const gpt2_model_config *cfg, int B, int T, int mode, int *err);
void gpt2_model_destroy(gpt2_model *m);

long long gpt2_model_num_params(const gpt2_model *m); /* floats, padded vocabulary included */
float *gpt2_model_params(gpt2_model *m);              /* device pointer, flat, order above   */
float *gpt2_model_grads(gpt2_model *m);               /* device pointer, same layout         */
/* Offsets (in floats) of the 4 + 12*n_layer tensors inside the flat buffers, in order; returns
 * the number of tensors, or a negative error when `max` is too small. */
int gpt2_model_param_offsets(const gpt2_model *m, long long *offsets, int max);
int gpt2_model_set_params(gpt2_model *m, const float *host, long long count);
int gpt2_model_get_params(gpt2_model *m, float *host, long long count);
int gpt2_model_get_grads(gpt2_model *m, float *host, long long count);

/* embedding -> blocks -> ln_f -> lm_head -> softmax/cross-entropy. tokens/targets: device int32
 * [B*T]. Leaves the per-token losses and dlogits in the model (forward + cross_entropy of the
 * reference, src/train.cu:334-389). */
int gpt2_model_forward(gpt2_model *m, const int *tokens, const int *targets, gpt2l_stream_t stream);
/* Zeroes the gradients, then the whole backward pass (gpt2_zero_grad + backward, src/train.cu:391-448). */
int gpt2_model_backward(gpt2_model *m, gpt2l_stream_t stream);
/* The same backward pass in parts, for data-parallel drivers that overlap the gradient exchange with
 * the computation: head (zeroes the gradients; lm_head and ln_f), one transformer block (call with
 * l = n_layer-1 ... 0; afterwards the gradients of block l are final), and the embedding (afterwards
 * wte and wpe are final). gpt2_model_backward is exactly head, every layer, embedding. */
int gpt2_model_backward_head(gpt2_model *m, gpt2l_stream_t stream);
int gpt2_model_backward_layer(gpt2_model *m, int l, gpt2l_stream_t stream);
int gpt2_model_backward_embedding(gpt2_model *m, gpt2l_stream_t stream);
/* gpt2_model_forward + gpt2_model_backward of one step replayed from a CUDA graph (the reference
 * launches every kernel of its step separately, src/train.cu:334-448; at its shipped shape B=4, T=64 the
 * launches and the host-side set-up of 147 GEMM calls outweigh the kernels). The first call runs eagerly
 * (lazy allocations), the second captures, later calls replay; the graph is rebuilt when `tokens` or
 * `targets` point elsewhere. Kernel parameters are frozen at capture: buffer contents may change, buffers
 * may not move. */
int gpt2_model_forward_backward_graph(gpt2_model *m, const int *tokens, const int *targets, gpt2l_stream_t stream);
/* AdamW over the flat parameter buffer, step count t >= 1 (gpt2_update, src/train.cu:450-481). */
int gpt2_model_update(gpt2_model *m, float lr, float beta1, float beta2, float eps, float weight_decay, int t,
                      gpt2l_stream_t stream);
/* AdamW over floats [first, first + count) of the flat buffers only: for drivers that shard the
 * optimizer across data-parallel ranks (each rank updates its slice, then the slices are gathered). */
int gpt2_model_update_range(gpt2_model *m, long long first, long long count, float lr, float beta1, float beta2,
                            float eps, float weight_decay, int t, gpt2l_stream_t stream);
/* Synchronises the stream and returns the mean of the per-token losses of the last forward
 * (compute_mean_loss, src/train.cu:36-49). NaN on error. */
float gpt2_model_mean_loss(gpt2_model *m, gpt2l_stream_t stream);
/* Bytes of device memory the model holds. */
long long gpt2_model_device_bytes(const gpt2_model *m);

/* ------------------------------------------------------------------------------------------------
 * The same training step as a schedule of the persistent kernel: what schedule_instructions /
 * free_schedule (include/gpt2/mk.h:34, src/mk.cu:281-942) and the launch of megakernel
 * (tests/test_train_mk.cu:292-314) are in the reference. gpt2_schedule_instructions builds the op list of
 * one step of `m` on fixed token / target buffers — embedding, the blocks, loss, the backward pass with
 * every weight gradient, the embedding backward and (GPT2_STEP_WITH_UPDATE) AdamW — derives the tile
 * dependencies from the buffers each op reads and writes, and uploads it; gpt2_megakernel_step runs it.
 * Where the reference takes a config_t and returns per-SM instruction streams, this takes the model
 * (which owns the buffers the reference passes to the kernel launch) and returns an opaque handle; the
 * dependency counters are per 128-row block, every wait is bounded, and a step that gave up on a wait
 * reports GPT2L_DEV_TIMEOUT through gpt2_megakernel_step_status instead of hanging.
 * Without GPT2_STEP_ATTENTION_IN_KERNEL the attention passes are launched between the persistent pieces
 * (one piece and one attention pass per block and direction instead of a single launch), with whichever
 * attention implementation the model uses. Needs n_embd <= 1280, and for attention inside the launch the
 * fused attention (T % 128 == 0, TF32 mode or GPT2_ATTENTION=flash); otherwise GPT2L_ERR_TOO_LARGE and the
 * caller keeps using gpt2_model_forward / _backward / _update. tokens / targets must stay valid and in place.
 * ------------------------------------------------------------------------------------------------ */
#define GPT2_STEP_WITH_UPDATE 1u         /* AdamW inside the step (single GPU)                          */
#define GPT2_STEP_ATTENTION_IN_KERNEL 2u /* attention tiles inside the persistent launch                */
typedef struct gpt2l_step gpt2l_step;
gpt2l_step *gpt2_schedule_instructions(gpt2_model *m, const int *tokens, const int *targets, unsigned flags, int *err);
void gpt2_free_schedule(gpt2l_step *s);
/* One step. lr ... t are AdamW's (ignored without GPT2_STEP_WITH_UPDATE); the losses of the forward pass
 * are left where gpt2_model_mean_loss reads them. */
int gpt2_megakernel_step(gpt2l_step *s, float lr, float beta1, float beta2, float eps, float weight_decay, int t,
                         gpt2l_stream_t stream);
/* After the stream has been synchronised: 0, or GPT2L_DEV_TIMEOUT when a wait of the last step gave up. */
int gpt2_megakernel_step_status(gpt2l_step *s);
/* out = {ops in the step, kernel launches per step, tiles per step}. */
int gpt2_megakernel_step_info(const gpt2l_step *s, int out[3]);
/* Per-tile profile of the persistent pieces of a step (the reference's megakernel records %globaltimer per
 * instruction, src/mk.cu:966-971, 1117-1138, 1814-1819). enable = 1 records every following step.
 * gpt2_megakernel_step_read_profile copies persistent piece `piece` of the last step: for tile i of that
 * piece, out[4i..4i+3] = {op index | op kind << 32, start in ns, ns spent in the tile, SM id}; returns the
 * number of tiles copied (at most max_tiles), or a negative error (no such piece, profile not enabled). */
int gpt2_megakernel_step_profile(gpt2l_step *s, int enable);
long long gpt2_megakernel_step_read_profile(gpt2l_step *s, int piece, long long *out, long long max_tiles);
/* Test hook for the bounded waits (host-side fault injection; no device fault is provoked): overrides the
 * arrival count dependency `dep` of op `op` of persistent piece `piece` waits for, and that piece's wait
 * limit in milliseconds (0 keeps the default). */
int gpt2_megakernel_step_debug_set_expected(gpt2l_step *s, int piece, int op, int dep, int expected, int wait_limit_ms);

/* ---- files (blocking; they synchronise the device) ---- */
#define GPT2M_ERR_IO (-7)     /* open / read / write failed                                   */
#define GPT2M_ERR_FORMAT (-8) /* size, magic or configuration does not match this model       */
/* The reference's weight file (gpt2_load_weights / gpt2_dump_weights, src/gpt2.cu:206-314, written by
 * scripts/hf_to_bin.py): headerless native-endian fp32, tensors in the parameter order above, wte
 * stored [n_embd][vocab_size] with the true vocabulary. Loading pads wte rows with zeros; dumping
 * drops the pad columns, so files interchange with the reference. The size must match exactly. */
int gpt2_model_load_weights(gpt2_model *m, const char *path);
int gpt2_model_dump_weights(gpt2_model *m, const char *path);
/* Training checkpoint: a 64-byte header ("G2CKPT1", the configuration, the number of AdamW steps
 * taken) followed by three sections in the weight-file layout: parameters, first moments, second
 * moments. The reference has no counterpart (it can only dump weights, so its AdamW state is lost on
 * restart). load returns the step count through *step (may be NULL); resume with t = step + 1. */
int gpt2_model_save_checkpoint(gpt2_model *m, const char *path, int step);
int gpt2_model_load_checkpoint(gpt2_model *m, const char *path, int *step);

#ifdef __cplusplus
}
#endif
#endif /* GPT2_MODEL_H */
