// Host-side schedule of the persistent kernel: a list of ops (GEMMs and, in the step kernel, the
// row-local layers and attention between them) with dependencies, turned into tile ranges and counters.
// Shared by megakernel.cu (the C ABI over GEMM lists) and step_schedule.cu (the training step).
#pragma once

#include <vector>

#include "linear_internal.h"

namespace g2l {

struct DepSpec {
  int producer;  // index of an earlier op
  int kind;      // GPT2L_DEP_ROWBLOCK, GPT2L_DEP_WHOLE_OP or DEP_SEQUENCE
};

struct OpSpec {
  int kind = OPK_GEMM;     // OpKind
  GemmDesc gemm = {};      // OPK_GEMM
  bool transposed_a = false;  // GEMM: backward_weight given as the forward form over a transposed activation copy
  RowArgs ra = {};         // other kinds
  int rows = 0;            // rows the op covers (B*T)
  int rows_per_tile = 0;   // AdamW: units of 1024 elements per tile
  int rb_per_seq = 0;      // DEP_SEQUENCE / attention: 128-row blocks per sequence
  int layer = 0;
  std::vector<DepSpec> deps;
};

struct Plan {
  std::vector<GemmOp> ops;
  int total_tiles = 0;
  int n_counters = 0;
  bool any_3x = false;
  bool any_colsum = false;
  bool pair = false;  // every op runs on CTA pairs (256-row tiles)
  int arrivals = NUM_WORKER_WARPS;  // counter arrivals per finished 128-row tile
};

int make_plan(const std::vector<OpSpec> &specs, int num_sms, Plan *plan);
int replay(const Plan &plan, int grid);
OpSpec spec_from(const gpt2l_op &o);

}  // namespace g2l

// The schedule object behind the C ABI (gpt2l_schedule is opaque to callers).
struct gpt2l_schedule {
  g2l::Plan plan;
  std::vector<g2l::OpSpec> specs;
  g2l::GemmOp *d_ops = nullptr;
  unsigned *d_counters = nullptr;
  g2l::Status *d_status = nullptr;
  float *ws = nullptr;
  unsigned *ws_sem = nullptr;
  g2l::FlashMaps *d_fmaps = nullptr;     // tensor maps of the attention ops (step schedules)
  float *xt = nullptr;                   // transposed activation copies for wide weight gradients
  unsigned long long *d_prof = nullptr;  // [total_tiles][2] profile stamps, allocated on request
  int grid = 0;
  long long wait_limit_ns = 0;
  g2l::DeviceCtx *ctx = nullptr;
  // what must be zero before a launch: outputs that are accumulated into (split-K reduce-adds, spread
  // column sums); filled by the builder
  struct ZeroRange { void *ptr; size_t bytes; };
  std::vector<ZeroRange> zero;
  float adam[7] = {0, 0, 0, 0, 0, 0, 0};
};

namespace g2l {
// Builds the device side of a schedule from op specs on the current device (tensor maps, workspaces,
// counters). Returns nullptr and sets *err on failure.
gpt2l_schedule *schedule_build(const std::vector<OpSpec> &specs, int grid_limit, int *err);
}  // namespace g2l
