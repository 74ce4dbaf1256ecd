// Internal declarations shared by the translation units of libgpt2_linear.so.
// Nothing in here is part of the C ABI (see include/gpt2_linear.h for that).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gpt2_linear.h"

namespace g2l {

// ---- tile geometry of the tcgen05 kernel ------------------------------------------
constexpr int BM = 128;      // UMMA M (one TMEM lane per output row)
constexpr int BK = 32;       // fp32 elements per k-block = one 128-byte swizzle row
constexpr int MAX_BN = 256;  // UMMA N upper bound
constexpr int UMMA_K = 8;    // kind::tf32
constexpr int A_TILE_BYTES = BM * BK * 4;      // 16 KiB
constexpr int B_TILE_BYTES = MAX_BN * BK * 4;  // 32 KiB
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int STAGES_1X = 4;  // TF32: 4 x 48 KiB
constexpr int STAGES_3X = 2;  // 3xTF32: 2 x (48 KiB hi + 48 KiB lo)
constexpr int RING_BYTES = STAGES_1X * STAGE_BYTES;  // 192 KiB in both modes
constexpr int NUM_ACC = 2;                           // TMEM accumulator double buffer
constexpr int TMEM_COLS = 512;
constexpr int NUM_THREADS = 320;  // 10 warps: producer, mma, 4 transform, 4 epilogue
constexpr int EPI_WARP0 = 6;
constexpr int XFORM_WARP0 = 2;
constexpr int NUM_XFORM_WARPS = 4;
constexpr int NUM_EPI_WARPS = 4;
// counter arrivals one finished tile produces in the one-CTA kernel: the transform warps double as
// epilogue warps (and publish) in launches that need no transform
constexpr int epi_arrivals(bool xform_active) { return xform_active ? NUM_EPI_WARPS : 2 * NUM_EPI_WARPS; }
constexpr int SMEM_CTRL_BYTES = 1024;  // mbarriers + tmem pointer + abort flag; the attention tiles' barriers behind them
constexpr int EPI_BUF_BYTES = 32 * 32 * 4;                       // one 32 x 32 fp32 store box
constexpr int EPI_BYTES = NUM_EPI_WARPS * 2 * EPI_BUF_BYTES;    // two boxes per epilogue warp
constexpr int SMEM_BYTES = 1024 /*alignment slack*/ + RING_BYTES + EPI_BYTES + SMEM_CTRL_BYTES;

constexpr int MAX_WAITS = 8;  // dependencies per op inside the library (the public gpt2l_op carries GPT2L_MAX_DEPS)
static_assert(MAX_WAITS >= GPT2L_MAX_DEPS, "public dependency count");

// The persistent step kernel (a whole training step in one launch) runs with one more warp than the
// GEMM-only kernel: the key/value pass of the attention backward needs two MMA issuers and eight
// row-work warps besides the producer.
constexpr int STEP_THREADS = 352;
constexpr int NUM_WORKER_WARPS = NUM_XFORM_WARPS + NUM_EPI_WARPS;  // warps 2..9: row-local ops run on these

// What an entry of a schedule is. Everything but OPK_GEMM exists only inside the persistent step kernel:
// the layers between the GEMMs of a training step (src/mk.cu:1155-1810 of the reference lists the same
// ops as cases of its interpreter), executed as tiles of `rows_per_tile` rows by the eight worker warps.
enum OpKind : int {
  OPK_GEMM = 0,
  OPK_EMBED_FWD = 1,    // out[m][:] = wte[:, tok[m]] + wpe[m % T][:]
  OPK_LN_FWD = 2,       // out, mean, rstd = layernorm(in) * w + b
  OPK_XENT = 3,         // losses[m], logits[m][:] <- dlogits (softmax + cross-entropy, in place)
  OPK_LN_BWD = 4,       // g_in[m][:] += layernorm backward; g_w, g_b += column sums
  OPK_ROWDOT = 5,       // delta[b][h][t] = sum_d dout[m][h*64+d] * out[m][h*64+d]
  OPK_EMBED_BWD = 6,    // g_wte[:, tok[m]] += g[m][:]; g_wpe[m % T][:] += g[m][:]
  OPK_ADAMW = 7,        // AdamW over a range of the flat buffers
  OPK_ATTN_FWD = 8,     // fused causal attention, forward (tile = 128 query rows of one head)
  OPK_ATTN_BWD_KV = 9,  //   dK, dV
  OPK_ATTN_BWD_Q = 10,  //   dQ
  OPK_TRANSPOSE = 11,   // out[c][m] = in[m][c] (K-major copy of activations for wide weight gradients)
  OPK_XENT_COMBINE = 12, // lse[m], loss[m] from the per-tile softmax statistics the lm_head epilogue left
  OPK_XENT_GRAD = 13     // logits[m][:] <- gradient of the mean cross-entropy, elementwise from lse[m]
};

// Operands of a non-GEMM op (meaning per kind: see the builder in step_schedule.cu)
struct RowArgs {
  const float *in0, *in1, *in2, *in3, *in4;
  float *out0, *out1, *out2;
  const int *idx0, *idx1;  // tokens / targets
  long long n0, n1;        // AdamW: first element and element count of the range
  int i0, i1, i2, i3, i4;  // M, C, T, V, Vp ... per kind
  float f0;
};

// what a dependency waits for, beyond the two public kinds: every 128-row block of the consumer tile's
// sequence (attention: a query block needs the keys of its whole sequence, a key block every later query)
constexpr int DEP_SEQUENCE = 3;

// where a bounded wait gave up (status record field `where`)
enum WaitSite {
  SITE_NONE = 0,
  SITE_DEP_COUNTER = 1,
  SITE_SMEM_EMPTY = 2,
  SITE_SMEM_FULL = 3,
  SITE_SMEM_READY = 4,
  SITE_TMEM_EMPTY = 5,
  SITE_TMEM_FULL = 6,
  SITE_SPLITK_TURNSTILE = 7,
  SITE_ROW_SYNC = 8,   // rendezvous of the worker warps inside a row-local op
  SITE_CTA_SYNC = 9,   // rendezvous of the whole CTA around an attention tile
  SITE_ATTENTION = 16  // + the wait number inside the attention tile code
};

// Device status record: one per device (single-op calls) or per schedule.
struct Status {
  int status;    // 0 ok, bit0 timeout
  int op;        // op index whose wait expired
  int counter;   // dependency counter index or mbarrier stage
  int seen;      // last value read
  int expected;  // value waited for
  int where;     // WaitSite
};

// One GEMM as the kernel sees it: C[Mc][Nc] = A . B (+ bias), reduction length Kc.
// A is "K-major" when its reduction index is contiguous in memory ([Mc][Kc] row-major) and
// "MN-major" when its Mc index is contiguous ([Kc][Mc] row-major); likewise B with Nc.
struct alignas(64) GemmOp {
  CUtensorMap tmA;  // box {32, 128} (K-major) or {32, 32} (MN-major)
  CUtensorMap tmB;  // box {32, bn}  (K-major) or {32, 32} (MN-major)
  CUtensorMap tmC;  // output, box {32, 32}: epilogue stores / split-K reduce-adds
  CUtensorMap tmC2; // second output of the GELU dual store
  int epi_tma;      // 1: the epilogue hands its staged boxes to the copy engine (TMA stores / reduce-adds)
  float *C;
  float *C2;            // gelu(C) when flags & GPT2L_EPI_GELU_DUAL
  const float *aux;     // epilogue operand shaped like C (residual to add / pre-activation for GELU')
  int aux_op;           // GPT2L_AUX_* or AUX_SOFTMAX_GRAD
  const float *aux_row; // AUX_SOFTMAX_GRAD: one value per (batch, output row), [batch][Mc]
  float aux_scale;
  const float *bias;    // [Nc] or null
  float *colsum;        // wgrad: g_b[Nc] or null (column sums of B over the reduction)
  const float *cs_src;  // the B operand [Kc][Nc] as a plain pointer (row stride Nc): TF32-mode column sums read it
                        // from global memory, beside the ring
  int colsum_spread;     // 1: every tile row sums its share of the k-blocks (kb % tiles_m == m_tile) and adds
                         // it atomically into a zeroed colsum; 0: tile row 0 sums everything
  float *ws;            // deterministic split-K: partial tiles [n_tiles][BM*bn]
  float *ws_colsum;     // deterministic split-K: [splits][Nc]
  unsigned *ws_sem;     // deterministic split-K: per output tile arrival counter
  long long ldc;
  int Mc, Nc, Kc;
  int a_mn, b_mn;       // 1 = MN-major
  int a_3d, b_3d;       // MN-major operand fetched with one chunked 3-D copy per k-block
  int bn;               // 64 / 128 / 256
  int tiles_m, tiles_n, splits, kb_total, kb_per_split;
  int band_m;           // rasterisation: tile rows per band (see decode_local)
  int pair;             // 1: tiles are 256 rows, computed by a CTA pair (cta_group::2)
  // batched GEMMs (attention): `batch` independent products whose operands sit batch_inner (heads)
  // x batch / batch_inner (sequences) apart; the tensor maps carry two extra dimensions for them
  int batch;            // 0 or 1 = plain GEMM
  int batch_inner;
  int tiles_per_batch;
  long long c_bs_outer, c_bs_inner;  // C offset per outer / inner batch index, in floats
  // causal structure of attention: 1 skip output tiles entirely above the diagonal; 2 the reduction
  // ends with the tile's last row (A is lower-triangular); 3 it starts at the tile's first row
  int causal;
  int tiles_dec;        // tile rows in scheduling units: tiles_m, or ceil(tiles_m / 2) for pairs
  int tile_base;        // global index of this op's first tile
  int n_tiles;          // tiles_m * tiles_n * splits
  int mode;             // gpt2l_mode
  unsigned flags;
  int atomic_out;       // split-K partials combined with red.add into a zeroed C
  int wait_ctr[MAX_WAITS];       // first counter index, -1 = none
  int wait_kind[MAX_WAITS];      // GPT2L_DEP_*
  int wait_expected[MAX_WAITS];  // arrivals to wait for
  int wait_op_ctr[MAX_WAITS];       // the producer's op-level counter and the count that means "all of it is
  int wait_op_expected[MAX_WAITS];  // done": once seen, the dependency is never looked at again
  int pub_rb_base;      // counter index of row block 0 (or -1)
  int pub_op_ctr;       // op-level counter index (or -1)
  unsigned idesc;       // tcgen05 instruction descriptor
  int op_index;
  int layer;
  // ---- softmax / cross-entropy fused around the lm_head ----
  // 1: forward, the epilogue also leaves per-row (max, sum of 2^(x - max)) of the tile's columns (base-2
  //    domain, columns >= xent_vocab excluded) in xent_stats[row * xent_stride + 2 * n_tile + (0 | 1)];
  // 2: the A operand is the logits and is turned into dlogits = (2^(x log2e - lse[row]) - [col == target]) *
  //    scale while it sits in shared memory (backward_input: rows = tokens, reduction index = vocabulary);
  // 3: the same for the B operand (backward_weight: reduction index = tokens, columns = vocabulary)
  int xent_mode;
  int xent_stride;
  int xent_vocab;
  float xent_scale;
  float *xent_stats;
  const float *xent_lse;
  const int *xent_tgt;
  // ---- non-GEMM ops of the step kernel ----
  int op_kind;          // OpKind; 0 = GEMM
  int rows_per_tile;    // rows one tile covers (divides 128, or a multiple of it); GEMM: 128
  int rb_per_seq;       // DEP_SEQUENCE: 128-row blocks per sequence (T / 128)
  int xform;            // this op needs the operand-transform warps (3xTF32 split or fused column sums)
  RowArgs ra;
};

// tensor maps of one fused-attention pass (attention_flash.cu): K-major views [T rows][64] of one head
// (box 32 x 64) and MN-major views (box 32 x 32 x 2 chunks) of Q, K, V (inside qkv) and dO
struct FlashMaps {
  CUtensorMap k_major[4];   // Q, K, V, dO
  CUtensorMap mn_major[4];  // Q, K, V, dO
};

struct LaunchParams {
  const GemmOp *ops;  // device array, or nullptr to use the by-value op
  int n_ops;
  int total_tiles;
  Status *status;
  unsigned *counters;
  long long wait_limit_ns;
  int xform_active;  // 0: no op needs the transform warps (TF32 mode, no fused bias gradient)
  // Where a wait that gives up is recorded besides `status`, both optional:
  //   sticky     a second record in device memory that launches never clear (only its reader does), so a
  //              timeout survives the per-call reset of `status`;
  //   host_flag  an int in mapped pinned host memory: the host sees it without a synchronisation and the
  //              next entry-point call returns the status instead of launching.
  Status *sticky;
  int *host_flag;
  // step kernel only: AdamW hyper-parameters of this launch {lr, beta1, beta2, eps, weight_decay,
  // 1 - beta1^t, 1 - beta2^t}, the tensor maps of the attention ops, and the profile buffer
  float adam[7];
  const FlashMaps *fmaps;
  unsigned long long *prof;  // [total_tiles][2] = {%globaltimer at tile start, SM id << 32 | duration} or null
};

// Host-side description of a batched, strided GEMM C_b[Mc][Nc] = A_b . B_b (no bias, no split).
// a_mn / b_mn as in GemmOp; ld* are row pitches in floats of the arrays as stored ([rows][inner]);
// *_bs_outer / *_bs_inner are the offsets in floats between outer / inner batch entries.
// internal epilogue op of the attention backward: out = aux * (acc - aux_row[row]) * aux_scale
constexpr int AUX_SOFTMAX_GRAD = 3;

struct BatchedDesc {
  int Mc, Nc, Kc, a_mn, b_mn;
  const float *a, *b;
  float *c;
  long long lda, ldb, ldc;
  int batch_outer, batch_inner;
  long long a_bs_outer, a_bs_inner, b_bs_outer, b_bs_inner, c_bs_outer, c_bs_inner;
  int causal;
  int mode;
  const float *aux = nullptr;      // epilogue operand shaped and batched like c
  const float *aux_row = nullptr;  // [batch_outer * batch_inner][Mc]
  float aux_scale = 1.f;
  int aux_op = 0;
};
int build_batched_op(const BatchedDesc &d, int num_sms, GemmOp *op);
// Batched tensor maps over [outer][inner] slices of a row-major matrix with row pitch ld (floats):
// K-major view {red, rows, inner, outer} with box 32 x box_rows (128-byte swizzle), and MN-major view
// {32, red_rows, mn / 32, inner, outer} with box 32 x 32 x chunks (32-byte swizzle atoms).
int encode_map_batched_k(CUtensorMap *map, const float *base, uint64_t red, uint64_t rows, uint64_t ld,
                         uint64_t nb_inner, uint64_t bs_inner, uint64_t nb_outer, uint64_t bs_outer, uint32_t box_rows);
int encode_map_batched_mn(CUtensorMap *map, const float *base, uint64_t mn, uint64_t red_rows, uint64_t ld,
                          uint64_t nb_inner, uint64_t bs_inner, uint64_t nb_outer, uint64_t bs_outer, uint32_t chunks);

// host-side description used to build a GemmOp
struct GemmDesc {
  int kind;  // gpt2l_op_kind
  int M, K, N;
  float *xent_stats = nullptr;  // forward: leave per-tile softmax statistics here (see GemmOp::xent_mode)
  int xent_vocab = 0;
  float *out;
  float *out_bias;
  const float *a;
  const float *b;
  const float *bias;
  gpt2_linear_opts opts;
};

struct DeviceCtx {
  bool ready = false;
  int device = -1;
  int num_sms = 0;
  int max_pairs = 0;                // resident CTA pairs (cluster size 2)
  Status *d_status = nullptr;       // device
  Status *h_status = nullptr;       // pinned host mirror
  int *h_flag = nullptr;            // mapped pinned int the kernels raise on a timeout (see LaunchParams)
  int *d_flag = nullptr;            // its device-side address
  Status *sticky = nullptr;         // optional second record (the no-allocation path)
  float *ws = nullptr;              // split-K workspace
  size_t ws_bytes = 0;
  unsigned *ws_sem = nullptr;
  size_t ws_sem_count = 0;
  float *xt = nullptr;              // transposed activations for wide weight gradients
  size_t xt_bytes = 0;
  float *xstats = nullptr;          // per-tile softmax statistics of gpt2_linear_forward_xent
  size_t xstats_bytes = 0;
  // host-call staging
  float *stage[4] = {nullptr, nullptr, nullptr, nullptr};
  size_t stage_bytes[4] = {0, 0, 0, 0};
  struct HostPipe *pipe = nullptr;  // streams, events and staging sets of the *_host_async calls (api.cu)
};

DeviceCtx *ctx_current(int *err);

// --- linear_tcgen05.cu ---
// Can this GEMM go through TMA + tcgen05? (16-byte aligned pointers and row strides)
bool tma_eligible(const GemmDesc &d);
// Fills `op` (tensor maps, tiling, idesc). `num_sms` guides the tile width / split choice.
// Workspace pointers and dependency fields are left for the caller.
int build_op(const GemmDesc &d, int num_sms, GemmOp *op);
// The host-only part of build_op (no tensor maps, no CUDA calls): shapes, tiling, descriptor bits.
int plan_op(const GemmDesc &d, int num_sms, GemmOp *op);
long long launch_count_value();
// tile index inside an op -> (tile row, tile column, split); shared by the kernel and the host replay
__host__ __device__ __forceinline__ void decode_local(int local, int tiles_m, int tiles_n, int band_m,
                                                      int &m_tile, int &n_tile, int &split) {
  const int per_split = tiles_m * tiles_n;
  split = local / per_split;
  const int l = local - split * per_split;
  const int band_size = band_m * tiles_n;
  const int band = l / band_size;
  const int rem = l - band * band_size;
  const int left = tiles_m - band * band_m;
  const int gb = left < band_m ? left : band_m;
  n_tile = rem / gb;
  m_tile = band * band_m + (rem - n_tile * gb);
}

// bytes of deterministic split-K workspace the op needs (0 if none)
size_t op_workspace_bytes(const GemmOp &op);
int launch_single(DeviceCtx *ctx, GemmOp &op, cudaStream_t stream);
// --- linear_tcgen05_pair.cu (CTA-pair kernel) ---
int pair_set_kernel_attributes();
int pair_max_pairs(int num_sms);  // how many CTA pairs can be resident at once
int pair_launch(const GemmOp *op_by_value, const LaunchParams &p, int n_pairs, bool x3, cudaStream_t stream);
int launch_list(DeviceCtx *ctx, const GemmOp *d_ops, int n_ops, int total_tiles, int grid,
                bool any_3x, bool any_colsum, bool pair, Status *d_status, unsigned *d_counters, long long wait_limit_ns,
                const float *adam, const FlashMaps *fmaps, unsigned long long *prof, cudaStream_t stream);
int set_kernel_attributes();
void count_launch(int n = 1);

// --- attention_flash.cu ---
// tensor maps of the fused attention over qkv[B*T][3C] and dout[B*T][C] (dout may be null: forward)
int attention_flash_build_maps(FlashMaps *maps, const float *qkv, const float *dout, int B, int T, int C, int NH);

// --- linear_simt.cu ---
int launch_simt(const GemmDesc &d, cudaStream_t stream);
int launch_colsum(float *out, const float *x, int rows, int cols, cudaStream_t stream);
int launch_transpose(float *dst, const float *src, int rows, int cols, cudaStream_t stream);
// floats of statistics a forward GEMM with xent_stats leaves: rows * stride(op) * 2
size_t xent_stats_floats(const GemmOp &op);
// lse[m], losses[m] from the statistics and the stored logits (layers.cu)
int launch_xent_combine(float *lse, float *losses, const float *stats, int stride, const float *logits, long long ld,
                        const int *targets, int M, cudaStream_t stream);

// --- driver entry point for tensor-map encoding ---
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_fn();

}  // namespace g2l
