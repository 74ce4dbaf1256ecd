/*
 * gpt2_linear.h — C ABI of the B200 (sm_100a) linear-layer GEMM path.
 *
 * Every entry point replaces one interface of vnnm404/gpt2.cu and keeps its argument
 * order and meaning.  All tensors are fp32, row-major and contiguous; every linear weight
 * is W[K][N] (input_dim x output_dim, the HF Conv1D layout), y = x.W + b.  K and N always
 * describe the FORWARD weight, also for the two backward calls, so the reduction runs over
 * K (forward), N (backward_input) or M = B*S (backward_weight) — the reference's convention
 * (src/train.cu:404-405).
 *
 * Conventions
 *   - return 0 on success; negative = argument / environment error found on the host before
 *     anything was launched; positive = device status word (bounded wait ran out).
 *     Nothing here calls exit() or prints from device code.
 *   - work is enqueued on the caller's stream; the *_host variants synchronise that stream.
 *   - pointers are device pointers unless the function name ends in _host.
 *   - outputs are fully overwritten (the reference's semantics: mlp.h:305-333, 634-650,
 *     952-995); bias / g_bias may be NULL.
 *   - there is no CPU fallback: without a CUDA device every compute entry returns
 *     GPT2L_ERR_NO_DEVICE.
 */
#ifndef GPT2_LINEAR_H
#define GPT2_LINEAR_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* CUDA stream handle (cudaStream_t) passed as an opaque pointer so that C callers and
 * ctypes need no CUDA headers. NULL = the default stream. */
typedef void *gpt2l_stream_t;

/* ---- error codes (negative: host side) ---- */
#define GPT2L_OK 0
#define GPT2L_ERR_NO_DEVICE (-1)   /* no CUDA device / wrong architecture (needs sm_100)   */
#define GPT2L_ERR_BAD_ARG (-2)     /* NULL operand, non-positive dimension, bad option     */
#define GPT2L_ERR_CUDA (-3)        /* a CUDA runtime / driver call failed                  */
#define GPT2L_ERR_NOT_INIT (-4)    /* gpt2_linear_init() has not run on this device        */
#define GPT2L_ERR_TOO_LARGE (-5)   /* size beyond a documented fixed limit                 */
#define GPT2L_ERR_SCHEDULE (-6)    /* megakernel schedule is malformed (see validate)      */
/* positive device status: bit 0 = a bounded wait expired (dependency counter, mbarrier or
 * split-K turnstile); the op index and counter are in gpt2_linear_last_status(). */
#define GPT2L_DEV_TIMEOUT 1

/* ---- options ---- */
enum gpt2l_mode {
  GPT2L_MODE_TF32 = 0,   /* one tcgen05.mma.kind::tf32 per product                          */
  GPT2L_MODE_TF32X3 = 1  /* operands split hi+lo, three MMAs per product (fp32-faithful)    */
};

/* epilogue flags */
#define GPT2L_EPI_GELU_DUAL 1u /* forward only: also store gelu(out) (tanh form) to opts->out2 */
/* epilogue operand (opts->aux, same shape as the output): what the reference does in separate
 * kernels right after the GEMM (src/layers/residual.cu:24-31, src/layers/gelu.cu:49-63), folded
 * into the store. aux must not overlap the output. Forward and backward_input only; the request runs
 * unsplit where a split could not carry it. GPT2L_ERR_BAD_ARG on the CUDA-core path (shapes or
 * pointers the tensor-core path cannot take) */
#define GPT2L_AUX_NONE 0
#define GPT2L_AUX_ADD 1       /* out = gemm (+ bias) + aux            (residual connection)          */
#define GPT2L_AUX_GELU_GRAD 2 /* out = gemm * gelu'(aux)              (GELU backward; aux = fc output) */

typedef struct gpt2_linear_opts {
  int mode;          /* enum gpt2l_mode                                                     */
  unsigned flags;    /* GPT2L_EPI_*                                                         */
  int split_k;       /* backward_weight: number of M-splits; 0 = choose from the SM count   */
  int deterministic; /* backward_weight with split_k>1: combine partials in a fixed order   */
  float *out2;       /* second output for GPT2L_EPI_GELU_DUAL, [B*S][N]                     */
  int force_simt;    /* 1 = run the CUDA-core fallback kernel even where TMA is possible    */
  int cta_pair;      /* 0 = choose; 1 = one CTA per 128-row tile; 2 = CTA pairs, 256-row tiles */
  const float *aux;  /* epilogue operand, [rows][cols] of the output; NULL = none           */
  int aux_op;        /* GPT2L_AUX_*                                                         */
  /* Softmax / cross-entropy folded into the lm_head's backward calls (see gpt2_linear_forward_xent).
   * With xent_lse set, the g_out argument of backward_input / backward_weight holds the LOGITS and the
   * kernels turn them into (softmax - onehot(target)) * xent_scale while the tiles sit in shared memory. */
  const float *xent_lse;   /* [B*S] base-2 log-sum-exp of each row, from gpt2_linear_forward_xent; NULL = off */
  const int *xent_targets; /* [B*S] target column of each row                                                  */
  int xent_vocab;          /* true vocabulary <= N: columns at or past it carry no probability and no gradient  */
  float xent_scale;        /* gradient scale, 1 / (B*S) for the mean loss                                       */
} gpt2_linear_opts;

/* One-time set-up for the current device: checks the architecture, raises the dynamic
 * shared-memory limit of the kernels, allocates the status word, the split-K workspace
 * and (for the *_host entry points) nothing else — staging buffers grow on demand.
 * Must run before the first compute call on that device. Idempotent. */
int gpt2_linear_init(int device);
/* Releases what init allocated on every device. */
void gpt2_linear_shutdown(void);
/* Library version, for the binding's sanity check. */
int gpt2_linear_version(void);
/* Number of kernel launches this library issued since init (all entry points). */
long long gpt2_linear_launch_count(void);
/* Last device status record of the current device: {status, op, counter, seen, expected,
 * where}. Returns the status word and clears a non-zero record. out may be NULL.
 * A kernel that gives up on a wait also raises a flag in host-visible memory: from then on every
 * device-pointer entry point returns GPT2L_DEV_TIMEOUT without launching anything, until this
 * function has been called. (Callers through include/compat ignore return codes, as the
 * reference's kernels have none; they can poll this function instead.) */
int gpt2_linear_last_status(int out[6]);

/*
 * out[M][N] = in[M][K] . w[K][N] + b[N]        (M = B*S; b may be NULL)
 * Replaces mlp_forward<32> (include/gpt2/layers/mlp.h:336-353; call sites
 * src/train.cu:356,360,365,369,376 and megakernel cases 3,5,8,10,13 in src/mk.cu).
 */
int gpt2_linear_forward(float *out, const float *in, const float *w, const float *b,
                        int B, int S, int K, int N,
                        const gpt2_linear_opts *opts, gpt2l_stream_t stream);

/*
 * The lm_head forward with softmax and cross-entropy in its epilogue: logits[M][N] = in[M][K] . w[K][N] as
 * gpt2_linear_forward (no bias), and for every row lse[m] = log2 sum_{c < V} 2^(logits[m][c] log2 e) and
 * losses[m] = -log softmax(logits[m][:V])[targets[m]]. The reference computes the same in three more kernels
 * over the logits (softmax_forward, cross_entropy_forward, cross_entropy_backward: src/train.cu:378, 388, 402;
 * megakernel cases 14-16, src/mk.cu:1384-1412), reading and writing the [M][V] tensor again each time; here
 * the epilogue keeps running (max, sum) pairs per row while it stores the tile, a small second kernel
 * combines them, and the gradient is never stored: pass `lse`, `targets`, V and the scale through
 * opts->xent_* to gpt2_linear_backward_input / _backward_weight, with the logits in place of g_out.
 * V <= N; columns V..N-1 (vocabulary padding) are excluded. Tensor-core path only (GPT2L_ERR_BAD_ARG for
 * shapes it cannot take).
 */
int gpt2_linear_forward_xent(float *logits, float *losses, float *lse, const float *in, const float *w,
                             const int *targets, int B, int S, int K, int N, int V,
                             const gpt2_linear_opts *opts, gpt2l_stream_t stream);

/*
 * g_in[M][K] = g_out[M][N] . w[K][N]^T          (overwrites g_in)
 * Replaces mlp_backward_input<32> (mlp.h:653-670; src/train.cu:404,424,429,436,441;
 * megakernel cases 17,21,24,28,31).
 */
int gpt2_linear_backward_input(float *g_in, const float *g_out, const float *w,
                               int B, int S, int K, int N,
                               const gpt2_linear_opts *opts, gpt2l_stream_t stream);

/*
 * g_w[K][N] = in[M][K]^T . g_out[M][N]          (overwrites g_w)
 * g_b[N]    = sum_m g_out[m][n]                 (overwrites g_b; g_b may be NULL)
 * Replaces mlp_backward_weight<32> (mlp.h:998-1017, bias-grad at :970-995;
 * src/train.cu:405,425,430,437,442; megakernel cases 18,22,25,29,32).
 */
int gpt2_linear_backward_weight(float *g_w, float *g_b, const float *g_out, const float *in,
                                int B, int S, int K, int N,
                                const gpt2_linear_opts *opts, gpt2l_stream_t stream);

/*
 * The same three operations with HOST buffers: inputs are copied to the device, the
 * kernel runs, outputs are copied back, the stream is synchronised. This is the call a
 * host-side plugin user makes when their tensors live in host memory; staging buffers are
 * kept and reused between calls. Pinned host memory makes the copies asynchronous.
 */
int gpt2_linear_forward_host(float *out, const float *in, const float *w, const float *b,
                             int B, int S, int K, int N,
                             const gpt2_linear_opts *opts, gpt2l_stream_t stream);
int gpt2_linear_backward_input_host(float *g_in, const float *g_out, const float *w,
                                    int B, int S, int K, int N,
                                    const gpt2_linear_opts *opts, gpt2l_stream_t stream);
int gpt2_linear_backward_weight_host(float *g_w, float *g_b, const float *g_out,
                                     const float *in, int B, int S, int K, int N,
                                     const gpt2_linear_opts *opts, gpt2l_stream_t stream);

/*
 * Pipelined host-buffer calls, for a sequence of operations on host tensors. Each call only enqueues
 * its work — copies in on one internal stream, the kernel on a second, copies out on a third, two sets
 * of staging buffers in rotation — and returns; the host->device copies of the next call then overlap
 * this call's kernel and its device->host copies (PCIe carries both directions at once). Output
 * buffers hold their results, and input buffers may be changed or freed, only after
 * gpt2_linear_host_synchronize(), which waits for everything enqueued on the current device and
 * returns the device status like the *_host calls. An input buffer handed to several calls between two
 * synchronisations (same address and size: a weight used by forward and backward_input, activations used
 * by forward and backward_weight) is copied to the device once. Use pinned host memory (pageable memory makes the
 * copies synchronous). Epilogue operands (opts->aux, GELU dual store) are device pointers and are
 * not supported here. The reference has no host-buffer path at all.
 */
int gpt2_linear_forward_host_async(float *out, const float *in, const float *w, const float *b,
                                   int B, int S, int K, int N, const gpt2_linear_opts *opts);
int gpt2_linear_backward_input_host_async(float *g_in, const float *g_out, const float *w,
                                          int B, int S, int K, int N, const gpt2_linear_opts *opts);
int gpt2_linear_backward_weight_host_async(float *g_w, float *g_b, const float *g_out,
                                           const float *in, int B, int S, int K, int N,
                                           const gpt2_linear_opts *opts);
int gpt2_linear_host_synchronize(void);

/*
 * Weight gradient for callers that may not allocate device memory. (No counterpart in the
 * reference, which allocates everything up front and has no split-K.)
 *
 * Computes what gpt2_linear_backward_weight computes with opts->deterministic = 1 — the
 * reduction over M split into chunks whose partial tiles are combined in a fixed order — but keeps
 * the partial tiles in a fixed array inside the library image instead of a cudaMalloc'ed
 * workspace. With the same tiling and split count the two results are bit-identical; they differ
 * in the last bits where the regular call picks another arrangement (wide weights, N >= 8192 and
 * N >= 8 K, which it computes from a transposed copy of `in`) or where the split count had to be
 * lowered to fit the array. Use it from code that runs after a server has given the whole GPU to
 * its own memory pool, from loops that cannot afford the device-wide synchronisation cudaMalloc /
 * cudaFree imply, or wherever a driver allocation at call time is simply forbidden. It does not
 * need gpt2_linear_init() and calls no cudaMalloc, cudaFree or other allocating routine.
 * One caveat on "allocates nothing": the array belongs to the library's CUDA module, and with
 * CUDA's default lazy module loading the driver reserves device memory for the module when the
 * first call on a device touches it. Make that first call (or set CUDA_MODULE_LOADING=EAGER)
 * before the application's pool takes what is left of the device; a first call made later fails
 * with GPT2L_ERR_CUDA if the driver cannot place the module.
 *
 * Limits and rules:
 *   - the partial tiles (splits x ceil(K/128) x ceil(N/bn) tiles of 128 x bn floats) must fit in
 *     GPT2L_NOALLOC_MAX_WORKSPACE_BYTES. A split count forced through opts->split_k that does not
 *     fit returns GPT2L_ERR_TOO_LARGE; an automatic one is lowered until it fits (a single split
 *     needs no workspace, so large weight matrices still run, just without the split);
 *   - at most 4096 output tiles when splitting (else GPT2L_ERR_TOO_LARGE);
 *   - the first call on each device resolves the array's device address and configures the
 *     kernels; make that first call outside of any stream capture;
 *   - the array is shared by every call on the device and keeps the previous call's contents;
 *     each call re-zeroes the part that must start at zero, on the caller's stream. Two calls whose
 *     kernels overlap on the GPU (different streams, or different threads) race on it: serialise
 *     them. Every GPU that loads the library holds the array until the process exits;
 *   - opts->flags and opts->out2 are ignored; opts->mode and opts->split_k are honoured;
 *   - the kernels' status record lives in the array too. A wait that gives up (it never should) is
 *     kept there, across later calls, until gpt2_linear_noalloc_last_status() reads it; that call
 *     returns the status word (0 = every call since the last read completed), fills
 *     {status, op, counter, seen, expected, where} and clears a non-zero record. It synchronises
 *     with the device and allocates nothing.
 */
#define GPT2L_NOALLOC_MAX_WORKSPACE_BYTES (32u << 20)
int gpt2_linear_backward_weight_noalloc(float *g_w, float *g_b, const float *g_out, const float *in,
                                        int B, int S, int K, int N,
                                        const gpt2_linear_opts *opts, gpt2l_stream_t stream);
int gpt2_linear_noalloc_last_status(int out[6]);
/* Test hook for the reader above: stores a record in the kept slot from the host (no kernel runs,
 * no device fault is provoked). */
int gpt2_linear_noalloc_debug_set_status(const int rec[6]);

/* ------------------------------------------------------------------------------------
 * Megakernel side: one persistent launch that runs a list of GEMM ops whose tiles are
 * ordered by dependency counters (the role of schedule_instructions / megakernel / bar[]
 * in src/mk.cu:281-942, 974-1028, 1124-1131, 1821-1824 and include/gpt2/mk.h:14-34).
 *
 * Differences from the reference's contract, all deliberate:
 *   - counters are per (op, 128-row block) as well as per op, so a consumer tile starts as
 *     soon as the row block it reads is complete, not when the whole previous op is;
 *   - every wait is bounded; on expiry the launch ends and returns GPT2L_DEV_TIMEOUT;
 *   - tiles are handed to CTAs in one global order (tile t runs on CTA t mod grid), which
 *     with backward-pointing dependencies cannot deadlock while all CTAs are resident.
 * ------------------------------------------------------------------------------------ */

enum gpt2l_op_kind {
  GPT2L_OP_FORWARD = 0,
  GPT2L_OP_BACKWARD_INPUT = 1,
  GPT2L_OP_BACKWARD_WEIGHT = 2
};

#define GPT2L_MAX_DEPS 2
/* what a dependency waits for */
#define GPT2L_DEP_NONE 0
#define GPT2L_DEP_ROWBLOCK 1 /* the producer's 128-row block with the same index as mine */
#define GPT2L_DEP_WHOLE_OP 2 /* every tile of the producer                               */

typedef struct gpt2l_dep {
  int producer; /* index of an EARLIER op in the list                                     */
  int kind;     /* GPT2L_DEP_*                                                             */
} gpt2l_dep;

/* One GEMM of the schedule, in the argument vocabulary of the three calls above. */
typedef struct gpt2l_op {
  int kind;            /* enum gpt2l_op_kind                                               */
  int layer;           /* carried through to profiling records; not interpreted            */
  int B, S, K, N;
  float *out;          /* forward: out; backward_input: g_in; backward_weight: g_w         */
  float *out_bias;     /* backward_weight: g_b or NULL; others: unused                     */
  const float *a;      /* forward: in; backward_input: g_out; backward_weight: in          */
  const float *b;      /* forward: w;  backward_input: w;     backward_weight: g_out       */
  const float *bias;   /* forward: b or NULL                                               */
  gpt2_linear_opts opts;
  gpt2l_dep deps[GPT2L_MAX_DEPS];
} gpt2l_op;

typedef struct gpt2l_schedule gpt2l_schedule; /* opaque; owns device copies */

/* Builds the device-side schedule (tensor maps, tile ranges, counters) for n_ops ops.
 * Returns NULL and sets *err on failure. The op list is copied. */
gpt2l_schedule *gpt2_schedule_create(const gpt2l_op *ops, int n_ops, int *err);
void gpt2_schedule_destroy(gpt2l_schedule *s);
/* Host-only replay of the schedule with `grid` CTAs taking tiles round-robin: returns 0 if
 * every wait is satisfied under the in-order execution model, GPT2L_ERR_SCHEDULE otherwise.
 * Needs no GPU (used by the CPU tests). */
int gpt2_schedule_validate(const gpt2l_op *ops, int n_ops, int grid);
/* Host-only: fills counts[0]=total tiles, [1]=number of counters, [2]=grid the launch
 * would use on a device with `num_sms` SMs. */
int gpt2_schedule_describe(const gpt2l_op *ops, int n_ops, int num_sms, int counts[3]);
/* Zeroes the counters and launches the persistent kernel once on `stream`. */
int gpt2_megakernel_run(gpt2l_schedule *s, gpt2l_stream_t stream);
/* After the stream has been synchronised: returns the device status of the last run. */
int gpt2_megakernel_status(gpt2l_schedule *s);
/* Test hook for the bounded-wait path: overrides the expected count of one dependency of
 * one op in the device copy (host-side fault injection; no device fault is provoked) and
 * the wait limit in milliseconds (0 keeps the default). */
int gpt2_schedule_debug_set_expected(gpt2l_schedule *s, int op, int dep, int expected,
                                     int wait_limit_ms);

/* Per-tile profile of the following runs of `s` (the reference keeps %globaltimer arrays per instruction,
 * src/mk.cu:966-971, 1117-1138, 1814-1819): enable = 1 allocates the record, 0 frees it.
 * gpt2_schedule_read_profile copies the record of the last run: for tile i (global tile order),
 * out[4i..4i+3] = {op index, start in ns (%globaltimer), ns the tile's epilogue / worker warp spent in it,
 * SM id}; returns the number of tiles copied (at most max_tiles) or a negative error. */
int gpt2_schedule_profile(gpt2l_schedule *s, int enable);
long long gpt2_schedule_read_profile(gpt2l_schedule *s, long long *out, long long max_tiles);

#ifdef __cplusplus
}
#endif
#endif /* GPT2_LINEAR_H */
