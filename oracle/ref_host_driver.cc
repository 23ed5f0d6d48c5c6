// Host driver around the reference's OWN code.  TEST INFRASTRUCTURE ONLY.
//
// This file contains no arithmetic of its own except the 12-line matmul loop
// noted below.  It is compiled together with the reference's sources, taken
// where they lie in the reference checkout (see oracle/Makefile), into
// oracle/_ref/libref_host.so and gives tests a C entry point that
//   * builds a customized operator with the reference's constructor
//     (src/kernel/customized.cc:65-186) and its threadblock graph builder,
//   * serialises it with threadblock::Graph::get_new_kernel_params
//     (src/threadblock/graph.cc:68-432),
//   * walks blocks x for-loop iterations x operators in the order of
//     compute_customizedop_fingerprint (src/kernel/cuda/customized_kernel.cu:307-603)
//     and runs the reference's fingerprinter classes
//     (include/mirage/threadblock/cuda/*.h) on the CPU with thread_id 0 of 1.
// Those classes are plain loops in `CUTLASS_DEVICE` constructors and that
// macro is `inline` under g++, so they run unchanged on the host.  The one
// header that cannot be host-compiled is threadblock/cuda/matmul.h (it pulls
// in cutlass::arch::LaneId); TBMatmulFingerprinter (matmul.h:773-804) is
// therefore restated in `host_matmul_fingerprint`.
//
// The reference allocates tensors from a cudaMalloc'ed arena
// (src/kernel/device_memory_manager.cu); here DeviceMemoryManager is defined
// over host memory so that the same constructors run without a GPU.
#include <algorithm>
#include <cassert>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <omp.h>
#include <vector>
#include <vector_types.h>
using std::max;
using std::min;
static thread_local dim3 threadIdx, blockIdx, blockDim;
#define __shared__ static
inline unsigned __shfl_sync(unsigned, unsigned v, int) { return v; }
inline float __shfl_xor_sync(unsigned, float v, int) { return v; }
inline void __syncthreads() {}
inline unsigned __byte_perm(unsigned a, unsigned, unsigned) { return a; }
#include "mirage/layout.h"
#include "mirage/type.h"
#include "cutlass/cutlass.h"
#include "cutlass/matrix_coord.h"
#include "mirage/kernel/customized.h"
#include "mirage/kernel/device_memory_manager.h"
#include "mirage/kernel/graph.h"
#include "mirage/threadblock/graph.h"
#include "mirage/threadblock/cuda/concat.h"
#include "mirage/threadblock/cuda/element_binary.h"
#include "mirage/threadblock/cuda/element_unary.h"
#include "mirage/threadblock/cuda/input_loader.h"
#include "mirage/threadblock/cuda/output_saver.h"
#include "mirage/threadblock/cuda/reduction.h"
#include "mirage/threadblock/serializer/concat_serializer.h"
#include "mirage/threadblock/serializer/element_binary_serializer.h"
#include "mirage/threadblock/serializer/element_unary_serializer.h"
#include "mirage/threadblock/serializer/input_loader_serializer.h"
#include "mirage/threadblock/serializer/matmul_serializer.h"
#include "mirage/threadblock/serializer/output_saver_serializer.h"
#include "mirage/threadblock/serializer/reduction_serializer.h"

using namespace mirage;
using namespace mirage::type;
namespace tb = mirage::threadblock;

// ---------------------------------------------------------------------------
// DeviceMemoryManager over host memory: same bump/LIFO discipline and the same
// table construction as src/kernel/device_memory_manager.cu:26-145.
// ---------------------------------------------------------------------------
namespace mirage {
namespace kernel {
DeviceMemoryManager *DeviceMemoryManager::singleton = nullptr;
DeviceMemoryManager::DeviceMemoryManager() {
  total_size = (size_t)1 << 30;
  offset = 0;
  base_ptr = (char *)std::malloc(total_size);
  exp_lookup_table = (FPType *)base_ptr;
  offset += (sizeof(FPType) * FP_Q + 15) / 16 * 16;
  exp_lookup_table[0] = 1;
  for (int i = 1; i < FP_Q; i++) {
    exp_lookup_table[i] = (exp_lookup_table[i - 1] * FP_EXP_BASE) % FP_P;
  }
  div_p_lookup_table = (FPType *)(base_ptr + offset);
  offset += (sizeof(FPType) * FP_P + 15) / 16 * 16;
  for (int i = 0; i < FP_P; i++) {
    div_p_lookup_table[i] = 1;
    for (int j = 1; j < FP_P; j++) {
      if ((i * j) % FP_P == 1) {
        div_p_lookup_table[i] = j;
      }
    }
  }
  div_q_lookup_table = (FPType *)(base_ptr + offset);
  offset += (sizeof(FPType) * FP_Q + 15) / 16 * 16;
  for (int i = 0; i < FP_Q; i++) {
    div_q_lookup_table[i] = 1;
    for (int j = 1; j < FP_Q; j++) {
      if ((i * j) % FP_Q == 1) {
        div_q_lookup_table[i] = j;
      }
    }
  }
}
DeviceMemoryManager::~DeviceMemoryManager() { std::free(base_ptr); }
bool DeviceMemoryManager::allocate(DTensor &tensor, bool allocate_fingerprint) {
  void *ret_ptr = base_ptr + offset;
  size_t sz = (tensor.data_size() + 15) / 16 * 16;
  offset += sz;
  tensor.data_ptr = ret_ptr;
  allocated_tensors.push_back({ret_ptr, sz});
  if (allocate_fingerprint) {
    ret_ptr = base_ptr + offset;
    sz = (tensor.fingerprint_size() + 15) / 16 * 16;
    offset += sz;
    tensor.fp_ptr = (FPType *)ret_ptr;
    allocated_tensors.push_back({ret_ptr, sz});
  }
  assert((size_t)offset <= total_size);
  return true;
}
bool DeviceMemoryManager::free(DTensor &tensor) {
  if (tensor.fp_ptr != nullptr) {
    assert(allocated_tensors.back().first == tensor.fp_ptr);
    offset -= allocated_tensors.back().second;
    allocated_tensors.pop_back();
  }
  assert(allocated_tensors.back().first == tensor.data_ptr);
  offset -= allocated_tensors.back().second;
  allocated_tensors.pop_back();
  return true;
}
DeviceMemoryManager *DeviceMemoryManager::get_instance() {
  if (singleton == nullptr) {
    singleton = new DeviceMemoryManager();
  }
  return singleton;
}

// matmul.h:773-804 restated (the header does not compile for the host).
static void host_matmul_fingerprint(FPType *A, FPType *B, FPType *C, int m, int n, int k) {
  for (int i = 0; i < m * n; i++) {
    uint32_t result = 0;
    int mm = i / n, nn = i % n;
    for (int x = 0; x < k; x++) {
      uint32_t a = A[mm * k + x], b = B[x * n + nn];
      result = (result + a * b) % FP_PQ;
    }
    C[i] = result;
  }
}

// One thread block of compute_customizedop_fingerprint, on the host.
static void run_block(tb::NewKernelParams const &P, int forloop_range, int bx, int by, int bz, char *smem,
                      FPType *exp_tbl, FPType *divp, FPType *divq) {
  int osi = P.num_operators - P.num_dmem_outputs;
  for (int i = 0; i < forloop_range; i++) {
    int pi = 0;
    for (int op = 0; op < P.num_operators; op++) {
      switch (P.operator_types[op]) {
        case TB_INPUT_OP: {
          int3 rs, cs, gs;
          int rf, cf, gf, off;
          int2 dsh, ssh;
          layout::DmemLayout dl;
          layout::SmemLayout sl;
          tb::deserialize_input_loader_parameters(P.parameters, pi, rs, cs, rf, cf, gs, gf, dsh, ssh, dl, sl, off);
          int row = bx * rs.x + by * rs.y + bz * rs.z + i * rf;
          int col = bx * cs.x + by * cs.y + bz * cs.z + i * cf;
          int g = bx * gs.x + by * gs.y + bz * gs.z + i * gf;
          tb::TBInputLoaderFingerprinter fp((FPType *)P.dmem_input_ptrs[op], (FPType *)(smem + off), dsh, ssh, dl, sl,
                                            0, 1, cutlass::MatrixCoord(row, col), g);
          break;
        }
        case TB_OUTPUT_OP: {
          int3 rs, cs, gs;
          int2 dsh, ssh;
          int ioff, aoff;
          layout::DmemLayout dl;
          layout::SmemLayout sl;
          tb::deserialize_output_saver_parameters(P.parameters, pi, rs, cs, gs, dsh, ssh, dl, sl, ioff, aoff);
          tb::TBOutputAccumFingerprinter acc((FPType *)(smem + ioff), (FPType *)(smem + aoff), ssh, i == 0, 0, 1);
          if (i == forloop_range - 1) {
            int row = bx * rs.x + by * rs.y + bz * rs.z;
            int col = bx * cs.x + by * cs.y + bz * cs.z;
            int g = bx * gs.x + by * gs.y + bz * gs.z;
            tb::TBOutputSaverFingerprinter sv((FPType *)P.dmem_output_ptrs[op - osi], (FPType *)(smem + aoff), dsh, ssh,
                                              dl, sl, 0, 1, cutlass::MatrixCoord(row, col), g);
          }
          break;
        }
        case TB_MATMUL_OP: {
          int m, n, k, ao, bo, co;
          tb::deserialize_matmul_op_parameters(P.parameters, pi, m, n, k, ao, bo, co);
          host_matmul_fingerprint((FPType *)(smem + ao), (FPType *)(smem + bo), (FPType *)(smem + co), m, n, k);
          break;
        }
        case TB_EXP_OP: {
          int off, ne;
          tb::deserialize_elementunary_op_parameters(P.parameters, pi, off, ne);
          tb::TBElementUnaryFingerPrinter fp(TB_EXP_OP, exp_tbl, (FPType *)(smem + off), ne, 0, 1);
          break;
        }
        case TB_DIV_OP: {
          int3 s1, s2;
          int o1, o2, oo;
          tb::deserialize_elementbinary_op_parameters(P.parameters, pi, s1, s2, o1, o2, oo);
          tb::TBElementBinaryFingerPrinter fp(TB_DIV_OP, divp, divq, (FPType *)(smem + o1), (FPType *)(smem + o2),
                                              (FPType *)(smem + oo), s1, s2, 0, 1);
          break;
        }
        case TB_REDUCTION_0_OP:
        case TB_REDUCTION_1_OP:
        case TB_REDUCTION_2_OP:
        case TB_REDUCTION_0_TO_DIMX_OP:
        case TB_REDUCTION_1_TO_DIMX_OP:
        case TB_REDUCTION_2_TO_DIMX_OP: {
          int ne, deg, inner, io, oo;
          tb::deserialize_reduction_op_parameters(P.parameters, pi, ne, deg, inner, io, oo);
          tb::TBReductionFingerprinter fp(P.operator_types[op], (FPType *)(smem + io), (FPType *)(smem + oo), ne, deg,
                                          inner, 0, 1);
          break;
        }
        case TB_CONCAT_0_OP:
        case TB_CONCAT_1_OP:
        case TB_CONCAT_2_OP: {
          int ne, ad, bd, inner, ao, bo, oo;
          tb::deserialize_concat_op_parameters(P.parameters, pi, ne, ad, bd, inner, ao, bo, oo);
          tb::TBConcatFingerprinter fp((FPType *)(smem + ao), (FPType *)(smem + bo), (FPType *)(smem + oo), ne, ad, bd,
                                       inner, 0, 1);
          break;
        }
        default:
          assert(false && "Unsupported threadblock operator");
      }
    }
    assert(pi == P.num_parameters);
  }
}

// The three launch wrappers of src/kernel/cuda/customized_kernel.cu:605-678.
bool KNCustomizedOp::fingerprint(void) {
  tb::NewKernelParams P = bgraph.get_new_kernel_params(true);
  DeviceMemoryManager *dmm = DeviceMemoryManager::get_instance();
  int gx = bgraph.grid_dim.x, gy = bgraph.grid_dim.y, gz = bgraph.grid_dim.z;
  int nblocks = gx * gy * gz;
#pragma omp parallel
  {
    std::vector<char> smem(bgraph.smem_offset + 64);
#pragma omp for schedule(static)
    for (int b = 0; b < nblocks; b++) {
      int bx = b % gx, by = (b / gx) % gy, bz = b / (gx * gy);
      blockIdx = dim3(bx, by, bz);
      run_block(P, bgraph.forloop_range, bx, by, bz, smem.data(), dmm->exp_lookup_table, dmm->div_p_lookup_table,
                dmm->div_q_lookup_table);
    }
  }
  return true;
}
bool KNCustomizedOp::profile(ProfileResult &) { return false; }
void KNCustomizedOp::run(void) {}
bool KNInputOp::profile(ProfileResult &) { return false; }
bool KNInputOp::fingerprint(void) { return true; }
} // namespace kernel
} // namespace mirage

// ---------------------------------------------------------------------------
// C entry points (called from Python through ctypes)
// ---------------------------------------------------------------------------
struct RefOp {
  kernel::KNCustomizedOp *op;
  std::vector<kernel::KNInputOp *> inputs;
};

extern "C" {

// Builds KNInputOp tensors + one KNCustomizedOp with the reference's own
// constructors.  All arrays are flat ints:
//   in_dims[4*i..], in_ndims[i], in_layouts[i], in_dtypes[i]
//   op_types[j], op_nsrc[j], op_srcs = (op_idx, ts_idx) pairs, concatenated
//   input_map[3*i..], forloop_dim[i], smem_layouts[i], output_map[3], grid[3], block[3]
// info receives {num tb operators, num serialised parameter ints, smem bytes, num outputs}.
void *ref_customized_create(int num_inputs, int const *in_ndims, int const *in_dims, int const *in_layouts,
                            int const *in_dtypes, int num_ops, int const *op_types, int const *op_nsrc,
                            int const *op_srcs, int const *input_map, int const *forloop_dim, int const *smem_layouts,
                            int const *output_map, int forloop_range, int reduction_dimx, int const *grid,
                            int const *block, int *info) {
  RefOp *r = new RefOp();
  std::vector<kernel::DTensor> ins;
  for (int i = 0; i < num_inputs; i++) {
    std::vector<int> dims(in_dims + 4 * i, in_dims + 4 * i + in_ndims[i]);
    auto *iop = new kernel::KNInputOp(dims, (DataType)in_dtypes[i], (layout::DmemLayout)in_layouts[i]);
    r->inputs.push_back(iop);
    ins.push_back(iop->output_tensors[0]);
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

void ref_customized_output_dims(void *h, int idx, int *ndims, int *dims) {
  RefOp *r = (RefOp *)h;
  kernel::DTensor const &t = r->op->output_tensors[idx];
  *ndims = t.num_dims;
  for (int i = 0; i < t.num_dims; i++) {
    dims[i] = t.dim[i];
  }
}

void ref_customized_set_input(void *h, int idx, uint16_t const *fp) {
  RefOp *r = (RefOp *)h;
  kernel::DTensor const &t = r->inputs[idx]->output_tensors[0];
  std::memcpy(t.fp_ptr, fp, t.fingerprint_size());
}

void ref_customized_fingerprint(void *h) { ((RefOp *)h)->op->fingerprint(); }

// Threads the block loop of fingerprint() uses from now on (<= 0: leave as is); returns the count in effect.
int ref_set_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
}

void ref_customized_get_output(void *h, int idx, uint16_t *fp) {
  RefOp *r = (RefOp *)h;
  kernel::DTensor const &t = r->op->output_tensors[idx];
  std::memcpy(fp, t.fp_ptr, t.fingerprint_size());
}

// LIFO arena: destroy in reverse order of creation.
void ref_customized_destroy(void *h) {
  RefOp *r = (RefOp *)h;
  delete r->op;
  for (int i = (int)r->inputs.size() - 1; i >= 0; i--) {
    delete r->inputs[i];
  }
  delete r;
}

void ref_tables(uint16_t *exp_tbl, uint16_t *divp, uint16_t *divq) {
  kernel::DeviceMemoryManager *dmm = kernel::DeviceMemoryManager::get_instance();
  std::memcpy(exp_tbl, dmm->exp_lookup_table, sizeof(FPType) * FP_Q);
  std::memcpy(divp, dmm->div_p_lookup_table, sizeof(FPType) * FP_P);
  std::memcpy(divq, dmm->div_q_lookup_table, sizeof(FPType) * FP_Q);
}
}
