// Operators of a threadblock graph (reference: include/mirage/threadblock/operator.h and the
// per-op headers matmul.h, element_unary.h, element_binary.h, reduction.h, concat.h).
// Constructing an operator infers its output tile shape and reserves the tile in the owning
// graph's shared-memory plan; destruction releases it (LIFO).
#pragma once
#include "mirage/kernel/device_tensor.h"
#include "mirage/threadblock/smem_tensor.h"
#include <vector>
#include <vector_types.h>

namespace mirage {
namespace threadblock {

class Graph;

class TBOperator {
public:
  TBOperator(Graph *graph, mirage::type::TBOperatorType type);
  TBOperator(Graph *graph, mirage::type::TBOperatorType type, STensor const &in1);
  TBOperator(Graph *graph, mirage::type::TBOperatorType type, STensor const &in1, STensor const &in2);
  virtual ~TBOperator();
  Graph *bgraph;
  mirage::type::TBOperatorType op_type;
  std::vector<STensor> input_tensors;
  std::vector<STensor> output_tensors;
};

class TBInputOp : public TBOperator {
public:
  TBInputOp(Graph *graph, mirage::kernel::DTensor const &dtensor, int3 input_map, int forloop_dim,
            mirage::layout::SmemLayout layout);
  ~TBInputOp() override;
  mirage::kernel::DTensor dtensor;
  int3 input_map;
  int forloop_dim;
};

class TBOutputOp : public TBOperator {
public:
  TBOutputOp(Graph *graph, STensor const &input, int3 output_map);
  ~TBOutputOp() override;
  mirage::kernel::DTensor dtensor;
  int3 output_map;
};

class TBMatmulOp : public TBOperator {
public:
  TBMatmulOp(Graph *graph, STensor const &A, STensor const &B);
  ~TBMatmulOp() override;
};

class TBElementUnaryOp : public TBOperator {
public:
  TBElementUnaryOp(Graph *graph, STensor const &A, mirage::type::TBOperatorType type);
  ~TBElementUnaryOp() override;
};

class TBElementBinaryOp : public TBOperator {
public:
  TBElementBinaryOp(Graph *graph, STensor const &A, STensor const &B, mirage::type::TBOperatorType type);
  ~TBElementBinaryOp() override;
};

class TBReductionOp : public TBOperator {
public:
  TBReductionOp(Graph *graph, STensor const &A, int dim, int size);
  ~TBReductionOp() override;
  int reduce_dim, reduce_size;
};

class TBConcatOp : public TBOperator {
public:
  TBConcatOp(Graph *graph, STensor const &A, STensor const &B, int dim);
  ~TBConcatOp() override;
  int concat_dim;
};

} // namespace threadblock
} // namespace mirage
