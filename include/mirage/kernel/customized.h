// kernel::KNCustomizedOp - a kernel-graph node that owns a threadblock graph
// (reference: include/mirage/kernel/customized.h:28-44).  Construction builds the
// threadblock graph from an ExecutionPlan (or replays a template graph), discovers the
// outputs and allocates them in the device arena; `fingerprint`, `run` and `profile`
// lower the graph to an `mgd_program`, let the kernel selector match it against the
// specialised sm_100a kernels and fall back to the generic interpreters.
#pragma once
#include "mirage/kernel/device_tensor.h"
#include "mirage/kernel/operator.h"
#include "mirage/threadblock/graph.h"
#include <string>
#include <vector>

namespace mirage {
namespace kernel {

class KNCustomizedOp : public KNOperator {
public:
  KNCustomizedOp(std::vector<DTensor> const &inputs, mirage::threadblock::ExecutionPlan const &plan);
  KNCustomizedOp(std::vector<DTensor> const &inputs, mirage::threadblock::Graph const &graph);
  ~KNCustomizedOp() override;
  bool profile(ProfileResult &profile) override;
  void run(void);
  bool fingerprint(void) override;
  int launch_fingerprint(void *stream) override;
  int launch_float(void *stream) override;
  // same as the two above for `num_sets` independent tensor sets (strides in elements)
  int launch_fingerprint_sets(int num_sets, void const *const *in, long long const *in_stride, void *const *out,
                              long long const *out_stride, void *stream);
  int launch_float_sets(int num_sets, void const *const *in, long long const *in_stride, void *const *out,
                        long long const *out_stride, void *stream);
  // The fused pair (this operator + `merge`, see can_fuse_with) for `num_sets` independent tensor sets in one
  // launch: in / out as above (out = this operator's two outputs in operator order), merged_out = the merge
  // operator's output, tickets = heads * num_sets zeroed int32 of device memory.
  int launch_fused_sets(KNCustomizedOp *merge, bool fingerprint_mode, int num_sets, void const *const *in,
                        long long const *in_stride, void *const *out, long long const *out_stride, void *merged_out,
                        long long merged_stride, int *tickets, void *stream, bool partials_are_scratch = false);

  // Non-asserting construction: nullptr plus a message when the plan is invalid for these inputs
  // or the outputs do not fit the arena.
  static KNCustomizedOp *create(std::vector<DTensor> const &inputs, mirage::threadblock::ExecutionPlan const &plan,
                                std::string *error, int *status);

  // which kernel `launch_*` picks: 0 = generic interpreter, >0 = a specialised kernel (see kernel_select.h)
  int selected_kernel(bool fingerprint_mode);
  // True when `next` is the cross-split merge operator consuming exactly this operator's two outputs and
  // both run on the specialised kernels: the pair can then be issued as ONE launch.
  bool can_fuse_with(KNOperator *next, bool fingerprint_mode);
  int launch_fused(KNCustomizedOp *merge, bool fingerprint_mode, void *stream);

  mirage::threadblock::ExecutionPlan plan;
  mirage::threadblock::Graph bgraph;
  // float-mode extension: per-row causal window of the speculative-decode graph (0 = off)
  int causal_window = 0;
  void set_causal_window(int window) {
    causal_window = window;
    lowered_ = false; // kernel choice depends on it
  }

private:
  struct Deferred {};
  KNCustomizedOp(Deferred, std::vector<DTensor> const &inputs, mirage::threadblock::ExecutionPlan const &plan);
  bool build_from_plan(std::string *error, int *status);
  bool lowered_ = false;
  mgd_program program_;
  int kernel_fp_ = -1, kernel_float_ = -1;
  // Operand order of a matched pattern: which of the two outputs is the (un-normalised) attention result, and,
  // for an operator that consumes such a pair, which of its two inputs is.  Hand-written plans give 0; plans
  // found by a search may list the row-sum first.
  int o_output_ = 0, o_input_ = 0;
  bool ensure_lowered();
  void after_build();
  struct FusedMerge { // the merge operator's output riding along with a split-KV launch
    void *out;
    long long set_stride;
    size_t bytes;
    int *tickets;
    bool partials_are_scratch; // nobody reads the split-KV partials after the launch
  };
  int launch_split(bool fingerprint_mode, int num_sets, void const *const *in, long long const *in_stride,
                   void *const *out, long long const *out_stride, FusedMerge const *merge, void *stream);
  int launch_rows(struct mgd_attn_rows const *rows, void const *const *in, void *o_acc, void *r_acc, void *o_div, void *stream);
  int launch_sets(bool fingerprint_mode, int num_sets, void const *const *in, long long const *in_stride,
                  void *const *out, long long const *out_stride, void *stream);
  int *tickets_ = nullptr; // per-head "last block done" counters of the fused launch (arena scratch)
};

} // namespace kernel
} // namespace mirage
