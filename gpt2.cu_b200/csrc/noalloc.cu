// gpt2_linear_backward_weight_noalloc: the deterministic split-K weight gradient for callers that
// must not allocate device memory.
//
// Who needs it: code that runs where cudaMalloc is off limits — inside a region whose memory
// budget was fixed up front (an inference or training server that hands the whole device to its
// own pool allocator at start-up and treats any later driver allocation as a bug), inside a
// latency-critical loop where the implicit device synchronisation of cudaMalloc/cudaFree is not
// acceptable, or in a host thread that is not allowed to take the driver's allocation lock.
// The regular entry point, gpt2_linear_backward_weight with opts->deterministic = 1, keeps its
// split-K partial tiles in a workspace that gpt2_linear_init / the first large call obtains with
// cudaMalloc; this variant keeps them in a fixed array that is part of the library image instead.
//
// The price: the array has a fixed size (GPT2L_NOALLOC_MAX_WORKSPACE_BYTES), every GPU that loads
// the library carries it until the process exits, and all calls on one device share it.
#include <cuda_runtime.h>
#include <string.h>

#include <mutex>

#include "linear_internal.h"

namespace g2l {
namespace {

// layout of the array: [status of the call in flight | arrival counters | kept status | partial tiles]
constexpr size_t NA_STATUS_BYTES = 256;   // status record the kernels of the current call poll; zeroed per call
constexpr size_t NA_SEM_COUNT = 16384;    // arrival counters: 4 per output tile
constexpr size_t NA_SEM_BYTES = NA_SEM_COUNT * sizeof(unsigned);
constexpr size_t NA_KEPT_BYTES = 256;     // first timeout record since the last read; calls never clear it
constexpr size_t NA_WS_BYTES = GPT2L_NOALLOC_MAX_WORKSPACE_BYTES;
constexpr size_t NA_WS_OFFSET = NA_STATUS_BYTES + NA_SEM_BYTES + NA_KEPT_BYTES;
constexpr size_t NA_TOTAL_BYTES = NA_WS_OFFSET + NA_WS_BYTES;

// The scratch itself. In HOST code this name is only a handle for cudaGetSymbolAddress — it is not
// a device address and must never be handed to a kernel as one.
static __device__ __align__(256) unsigned char g_noalloc_scratch[NA_TOTAL_BYTES];

struct PerDevice {
  bool ready = false;
  unsigned char *base = nullptr;  // device address of g_noalloc_scratch on this device
  int num_sms = 0;
  int max_pairs = 0;
};
constexpr int NA_MAX_DEVICES = 16;
PerDevice g_dev[NA_MAX_DEVICES];
std::mutex g_na_mu;

// One-time set-up for the CURRENT device: resolves the device address of the scratch array,
// raises the kernels' shared-memory limit, reads the SM count. No allocation of any kind.
int setup_current_device(PerDevice **out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NA_MAX_DEVICES) {
    (void)cudaGetLastError();
    return GPT2L_ERR_NO_DEVICE;
  }
  std::lock_guard<std::mutex> lk(g_na_mu);
  PerDevice &d = g_dev[dev];
  if (!d.ready) {
    int major = 0, sms = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
      (void)cudaGetLastError();
      return GPT2L_ERR_NO_DEVICE;
    }
    if (major != 10) return GPT2L_ERR_NO_DEVICE;
    if (!get_encode_fn()) return GPT2L_ERR_CUDA;
    int e = set_kernel_attributes();
    if (e) return e;
    e = pair_set_kernel_attributes();
    if (e) return e;
    d.max_pairs = pair_max_pairs(sms);
    void *ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || ptr == nullptr) {
      (void)cudaGetLastError();
      return GPT2L_ERR_CUDA;
    }
    d.base = static_cast<unsigned char *>(ptr);
    d.num_sms = sms;
    d.ready = true;
  }
  *out = &d;
  return GPT2L_OK;
}

}  // namespace
}  // namespace g2l

using namespace g2l;

extern "C" int gpt2_linear_backward_weight_noalloc(float *g_w, float *g_b, const float *g_out, const float *in,
                                                   int B, int S, int K, int N, const gpt2_linear_opts *opts,
                                                   gpt2l_stream_t stream) {
  if (!g_w || !g_out || !in || B <= 0 || S <= 0 || K <= 0 || N <= 0) return GPT2L_ERR_BAD_ARG;
  if ((long long)B * S > 0x7fffffffll) return GPT2L_ERR_TOO_LARGE;
  PerDevice *dev = nullptr;
  int err = setup_current_device(&dev);
  if (err) return err;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  GemmDesc d;
  memset(&d, 0, sizeof(d));
  d.kind = GPT2L_OP_BACKWARD_WEIGHT;
  d.M = B * S; d.K = K; d.N = N;
  d.out = g_w; d.out_bias = nullptr;  // bias gradient: the fixed-order column-sum kernel below
  d.a = in; d.b = g_out; d.bias = nullptr;
  if (opts) d.opts = *opts;
  d.opts.deterministic = 1;
  d.opts.flags = 0;
  d.opts.out2 = nullptr;
  if (d.opts.mode != GPT2L_MODE_TF32 && d.opts.mode != GPT2L_MODE_TF32X3) return GPT2L_ERR_BAD_ARG;
  if (d.opts.split_k < 0) return GPT2L_ERR_BAD_ARG;
  const bool forced = d.opts.split_k > 0;

  if (d.opts.force_simt || !tma_eligible(d)) {
    // shapes TMA cannot address run on the CUDA-core kernel, which needs no scratch at all
    d.out_bias = g_b;
    return launch_simt(d, st);
  }

  GemmOp op;
  err = build_op(d, dev->num_sms, &op);
  if (err) return err;
  // the partial tiles must fit the fixed array: a forced split count that does not fit is an
  // error; an automatic one is lowered until it fits (one split needs no workspace)
  while (op.splits > 1 && op_workspace_bytes(op) > NA_WS_BYTES) {
    if (forced) return GPT2L_ERR_TOO_LARGE;
    d.opts.split_k = op.splits - 1;
    err = build_op(d, dev->num_sms, &op);
    if (err) return err;
  }
  if (op.splits > 1 && (size_t)op.tiles_m * op.tiles_n * 4 > NA_SEM_COUNT) return GPT2L_ERR_TOO_LARGE;

  Status *status = reinterpret_cast<Status *>(dev->base);
  unsigned *sem = reinterpret_cast<unsigned *>(dev->base + NA_STATUS_BYTES);
  float *ws = reinterpret_cast<float *>(dev->base + NA_WS_OFFSET);
  // the array keeps whatever the previous call left: the status record and the arrival counters
  // must start at zero (the partial tiles are fully rewritten before they are read). The kept record
  // behind the counters is NOT cleared here: a timeout stays readable through
  // gpt2_linear_noalloc_last_status() however many calls follow it.
  if (cudaMemsetAsync(dev->base, 0, NA_STATUS_BYTES + NA_SEM_BYTES, st) != cudaSuccess) return GPT2L_ERR_CUDA;
  if (op.splits > 1) {
    op.ws = ws;
    op.ws_sem = sem;
  }
  DeviceCtx ctx;  // a view for the shared launcher; nothing in it is owned or allocated
  ctx.ready = true;
  ctx.num_sms = dev->num_sms;
  ctx.max_pairs = dev->max_pairs;
  ctx.d_status = status;
  ctx.sticky = reinterpret_cast<Status *>(dev->base + NA_STATUS_BYTES + NA_SEM_BYTES);
  err = launch_single(&ctx, op, st);
  if (err) return err;
  if (g_b) return launch_colsum(g_b, g_out, d.M, d.N, st);
  return GPT2L_OK;
}

// Reads (and, when it is non-zero, clears) the kept status record of the current device. Synchronises the
// device's work on the array through the copy; allocates nothing.
extern "C" int gpt2_linear_noalloc_last_status(int out[6]) {
  PerDevice *dev = nullptr;
  int err = setup_current_device(&dev);
  if (err) return err;
  Status h;
  unsigned char *kept = dev->base + NA_STATUS_BYTES + NA_SEM_BYTES;
  if (cudaMemcpy(&h, kept, sizeof(Status), cudaMemcpyDeviceToHost) != cudaSuccess) return GPT2L_ERR_CUDA;
  if (h.status != 0 && cudaMemset(kept, 0, sizeof(Status)) != cudaSuccess) return GPT2L_ERR_CUDA;
  if (out) {
    out[0] = h.status; out[1] = h.op; out[2] = h.counter; out[3] = h.seen; out[4] = h.expected; out[5] = h.where;
  }
  return h.status;
}

// Test hook: writes a record into the kept status slot from the host, so that the reader above can be
// exercised without making any kernel give up on a wait.
extern "C" int gpt2_linear_noalloc_debug_set_status(const int rec[6]) {
  if (!rec) return GPT2L_ERR_BAD_ARG;
  PerDevice *dev = nullptr;
  int err = setup_current_device(&dev);
  if (err) return err;
  Status h = {rec[0], rec[1], rec[2], rec[3], rec[4], rec[5]};
  return cudaMemcpy(dev->base + NA_STATUS_BYTES + NA_SEM_BYTES, &h, sizeof(Status), cudaMemcpyHostToDevice) ==
                 cudaSuccess ? GPT2L_OK : GPT2L_ERR_CUDA;
}
