// threadblock::Graph and ExecutionPlan - the description of what one thread block of a
// customized operator computes (reference: include/mirage/threadblock/graph.h:28-117).
//
// The builder methods come in the reference's two flavours: `create_*_op` returns nullptr
// for an invalid shape or a shared-memory overflow, the value-returning form asserts.
// `lower()` turns the graph into the flat `mgd_program` the CUDA side consumes; it plays
// the part of get_new_kernel_params (src/threadblock/graph.cc:68-432).
#pragma once
#include "mirage/kernel/device_tensor.h"
#include "mirage/threadblock/operator.h"
#include "mirage/threadblock/smem_tensor.h"
#include "mugraph_device.h"
#include <sys/types.h>
#include <utility>
#include <vector>
#include <vector_types.h>

namespace mirage {
namespace threadblock {

class ExecutionPlan {
public:
  // (operator type, [(producer operator index, output index)...]); inputs are operators 0..n-1
  std::vector<std::pair<mirage::type::TBOperatorType, std::vector<std::pair<int, int>>>> ops;
  std::vector<int3> input_map;
  std::vector<int> forloop_dim;
  std::vector<mirage::layout::SmemLayout> input_smem_layouts;
  int3 output_map; // all outputs share one map
  int forloop_range;
  int reduction_dimx = mirage::type::TB_REDUCTION_DIMX;
  dim3 grid_dim, block_dim;
};

class Graph {
public:
  Graph(dim3 grid_dim, dim3 block_dim, int forloop_range, int reduction_dimx);
  Graph(Graph const &) = delete;
  Graph &operator=(Graph const &) = delete;

  STensor new_input(mirage::kernel::DTensor const &dtensor, int3 input_map, int forloop_dim,
                    mirage::layout::SmemLayout layout);
  TBOperator *create_input_op(mirage::kernel::DTensor const &dtensor, int3 input_map, int forloop_dim,
                              mirage::layout::SmemLayout layout);
  mirage::kernel::DTensor new_output(STensor const &stensor, int3 output_map);
  TBOperator *create_output_op(STensor const &stensor, int3 output_map);
  STensor matmul(STensor const &A, STensor const &B);
  TBOperator *create_matmul_op(STensor const &A, STensor const &B);
  STensor exp(STensor const &A);
  TBOperator *create_elementunary_op(STensor const &A, mirage::type::TBOperatorType type);
  STensor add(STensor const &A, STensor const &B);
  STensor mul(STensor const &A, STensor const &B);
  STensor div(STensor const &A, STensor const &B);
  TBOperator *create_elementbinary_op(STensor const &A, STensor const &B, mirage::type::TBOperatorType type);
  STensor reduction(STensor const &A, int dim);
  TBOperator *create_reduction_op(STensor const &A, int dim);
  STensor reduction_to_dimx(STensor const &A, int dim);
  TBOperator *create_reduction_to_dimx_op(STensor const &A, int dim);
  STensor concat(STensor const &A, STensor const &B, int dim);
  TBOperator *create_concat_op(STensor const &A, STensor const &B, int dim);

  // shared-memory plan: 16-byte aligned bump allocation, LIFO release
  off_t allocate(STensor const &tensor);
  void free(STensor const &tensor);
  void free(std::vector<STensor> const &tensors);
  bool fits(size_t extra_bytes, bool strict = false) const;

  // Flatten into the kernel-level program.  Returns false (and leaves `why`) if the graph
  // exceeds the program container or contains an operator no kernel implements.
  bool lower(mgd_program &prog, char const **why = nullptr) const;

  dim3 grid_dim, block_dim;
  int forloop_range;
  int reduction_dimx;
  std::vector<TBOperator *> operators;
  off_t smem_offset;
  size_t max_smem; // budget checked by the builders; defaults to type::MAX_SMEM_SIZE
  std::vector<std::pair<off_t, size_t>> allocated_tensors;
};

} // namespace threadblock
} // namespace mirage
