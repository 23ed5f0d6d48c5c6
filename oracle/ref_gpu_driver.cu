// GPU driver around the reference's OWN fingerprint kernel.  TEST INFRASTRUCTURE ONLY.
//
// This file contains no arithmetic and no kernel.  It is compiled for sm_100a together with the reference's
// sources, taken where they lie in the reference checkout (see oracle/Makefile, target `refgpu`):
//   src/kernel/cuda/customized_kernel.cu      compute_customizedop_fingerprint + KNCustomizedOp::fingerprint
//                                             (:307-603, :655-678)
//   src/kernel/device_memory_manager.cu       the 10 GiB arena and the lookup tables (:26-145)
//   src/kernel/cuda/input_kernel.cu           KNInputOp::fingerprint (:56-73)
//   src/kernel/cuda/device_tensor_kernel.cu   DTensor::has_same_fingerprint (:22-53)
//   + the host sources the CPU checker already uses (customized.cc, operator.cc, device_tensor.cc, threadblock/*.cc ...)
// into oracle/_ref/libref_gpu.so, and gives tests and the benchmark a C entry point that builds customized
// operators with the reference's constructors, copies input fingerprints in, calls the reference's
// `fingerprint()` (one launch and one device synchronisation per operator, as the reference does it) and copies
// the results out.  It is the same-box GPU comparator of the verification sweep and a second source of golden
// fingerprints next to the CPU checker.
#include "mirage/kernel/customized.h"
#include "mirage/kernel/device_memory_manager.h"
#include "mirage/kernel/graph.h"
#include "mirage/threadblock/graph.h"
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>
#include <vector>

using namespace mirage;
using namespace mirage::type;
namespace tb = mirage::threadblock;

struct RefGpuOp {
  kernel::KNCustomizedOp *op;
  std::vector<kernel::KNInputOp *> inputs; // empty when the operator consumes another operator's outputs
};

extern "C" {

// Same flat-array protocol as the CPU checker's ref_customized_create.  With `producer` non-null the inputs are
// that operator's output tensors (the way the second customized op of a muGraph consumes the first) and the
// in_* arrays are ignored.  info receives {threadblock operators, parameter ints, shared-memory bytes, outputs}.
void *refgpu_customized_create(int num_inputs, int const *in_ndims, int const *in_dims, int const *in_layouts,
                               int const *in_dtypes, int num_ops, int const *op_types, int const *op_nsrc,
                               int const *op_srcs, int const *input_map, int const *forloop_dim,
                               int const *smem_layouts, int const *output_map, int forloop_range, int reduction_dimx,
                               int const *grid, int const *block, void *producer, int *info) {
  RefGpuOp *r = new RefGpuOp();
  std::vector<kernel::DTensor> ins;
  if (producer != nullptr) {
    ins = static_cast<RefGpuOp *>(producer)->op->output_tensors;
  } else {
    for (int i = 0; i < num_inputs; i++) {
      std::vector<int> dims(in_dims + 4 * i, in_dims + 4 * i + in_ndims[i]);
      auto *iop = new kernel::KNInputOp(dims, (DataType)in_dtypes[i], (layout::DmemLayout)in_layouts[i]);
      r->inputs.push_back(iop);
      ins.push_back(iop->output_tensors[0]);
    }
  }
  tb::ExecutionPlan plan;
  int s = 0;
  for (int j = 0; j < num_ops; j++) {
    std::vector<std::pair<int, int>> srcs;
    for (int t = 0; t < op_nsrc[j]; t++, s++) {
      srcs.push_back({op_srcs[2 * s], op_srcs[2 * s + 1]});
    }
    plan.ops.push_back({(TBOperatorType)op_types[j], srcs});
  }
  for (int i = 0; i < num_inputs; i++) {
    plan.input_map.push_back({input_map[3 * i], input_map[3 * i + 1], input_map[3 * i + 2]});
    plan.forloop_dim.push_back(forloop_dim[i]);
    plan.input_smem_layouts.push_back((layout::SmemLayout)smem_layouts[i]);
  }
  plan.output_map = {output_map[0], output_map[1], output_map[2]};
  plan.forloop_range = forloop_range;
  plan.reduction_dimx = reduction_dimx;
  plan.grid_dim = dim3(grid[0], grid[1], grid[2]);
  plan.block_dim = dim3(block[0], block[1], block[2]);
  r->op = new kernel::KNCustomizedOp(ins, plan);
  tb::NewKernelParams P = r->op->bgraph.get_new_kernel_params(true);
  info[0] = P.num_operators;
  info[1] = P.num_parameters;
  info[2] = (int)r->op->bgraph.smem_offset;
  info[3] = (int)r->op->output_tensors.size();
  return r;
}

void refgpu_customized_output_dims(void *h, int idx, int *ndims, int *dims) {
  kernel::DTensor const &t = static_cast<RefGpuOp *>(h)->op->output_tensors[idx];
  *ndims = t.num_dims;
  for (int i = 0; i < t.num_dims; i++) {
    dims[i] = t.dim[i];
  }
}

// fills input idx with the reference's own input fingerprint kernel (fp[i] = i % 25651)
int refgpu_customized_fill_reference(void *h, int idx) {
  RefGpuOp *r = static_cast<RefGpuOp *>(h);
  if (idx < 0 || idx >= (int)r->inputs.size()) return 1;
  return r->inputs[idx]->fingerprint() ? 0 : 1;
}

int refgpu_customized_set_input(void *h, int idx, uint16_t const *fp) {
  RefGpuOp *r = static_cast<RefGpuOp *>(h);
  if (idx < 0 || idx >= (int)r->inputs.size()) return 1;
  kernel::DTensor const &t = r->inputs[idx]->output_tensors[0];
  return (int)cudaMemcpy(t.fp_ptr, fp, t.fingerprint_size(), cudaMemcpyHostToDevice);
}

// device-to-device: input idx <- `device_fp` (a buffer of the calling process, e.g. a seeded fill of this library)
int refgpu_customized_set_input_from_device(void *h, int idx, void const *device_fp) {
  RefGpuOp *r = static_cast<RefGpuOp *>(h);
  if (idx < 0 || idx >= (int)r->inputs.size()) return 1;
  kernel::DTensor const &t = r->inputs[idx]->output_tensors[0];
  return (int)cudaMemcpy(t.fp_ptr, device_fp, t.fingerprint_size(), cudaMemcpyDeviceToDevice);
}

// the reference's launch wrapper: one kernel, one cudaDeviceSynchronize
int refgpu_customized_fingerprint(void *h) { return static_cast<RefGpuOp *>(h)->op->fingerprint() ? 0 : 1; }

int refgpu_customized_get_output(void *h, int idx, uint16_t *fp) {
  kernel::DTensor const &t = static_cast<RefGpuOp *>(h)->op->output_tensors[idx];
  return (int)cudaMemcpy(fp, t.fp_ptr, t.fingerprint_size(), cudaMemcpyDeviceToHost);
}

// device address of output idx's fingerprints (for a device-side comparison by the caller)
void *refgpu_customized_output_ptr(void *h, int idx) {
  return static_cast<RefGpuOp *>(h)->op->output_tensors[idx].fp_ptr;
}

// DTensor::has_same_fingerprint of the reference between output a_idx of ha and output b_idx of hb
int refgpu_has_same_fingerprint(void *ha, int a_idx, void *hb, int b_idx) {
  kernel::DTensor const &a = static_cast<RefGpuOp *>(ha)->op->output_tensors[a_idx];
  kernel::DTensor const &b = static_cast<RefGpuOp *>(hb)->op->output_tensors[b_idx];
  return a.has_same_fingerprint(b) ? 1 : 0;
}

// `iters` evaluations of a two-operator muGraph with the reference's protocol (`for op: op->fingerprint()`);
// returns wall-clock milliseconds per evaluation.
double refgpu_time_pair(void *h1, void *h2, int iters) {
  RefGpuOp *a = static_cast<RefGpuOp *>(h1), *b = static_cast<RefGpuOp *>(h2);
  cudaDeviceSynchronize();
  auto t0 = std::chrono::steady_clock::now();
  for (int i = 0; i < iters; i++) {
    a->op->fingerprint();
    b->op->fingerprint();
  }
  auto t1 = std::chrono::steady_clock::now();
  return std::chrono::duration<double, std::milli>(t1 - t0).count() / (iters > 0 ? iters : 1);
}

// LIFO arena: destroy in reverse order of creation.
void refgpu_customized_destroy(void *h) {
  RefGpuOp *r = static_cast<RefGpuOp *>(h);
  delete r->op;
  for (int i = (int)r->inputs.size() - 1; i >= 0; i--) {
    delete r->inputs[i];
  }
  delete r;
}

int refgpu_last_cuda_error(void) { return (int)cudaGetLastError(); }
}
