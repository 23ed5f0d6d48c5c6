// kernel::Graph - builder of the kernel graph (reference: include/mirage/kernel/graph.h:28-85).
// Same method names and conventions: value-returning builders assert, `create_*_op` return
// nullptr when the result does not fit the device arena or the shapes are invalid.
#pragma once
#include "mirage/kernel/customized.h"
#include "mirage/kernel/device_tensor.h"
#include "mirage/kernel/operator.h"
#include "mirage/threadblock/graph.h"
#include <vector>

namespace mirage {
namespace kernel {

class Graph {
public:
  Graph(void);
  ~Graph(); // deletes the operators in reverse order: arena frees are LIFO
  Graph(Graph const &) = delete;
  Graph &operator=(Graph const &) = delete;

  DTensor new_input(std::vector<int> const &dims, mirage::type::DataType data_type,
                    mirage::layout::DmemLayout layout);
  DTensor *new_input_ptr(std::vector<int> const &dims, mirage::type::DataType data_type,
                         mirage::layout::DmemLayout layout);
  KNOperator *create_input_op(std::vector<int> const &dims, mirage::type::DataType data_type,
                              mirage::layout::DmemLayout layout);
  DTensor matmul(DTensor const &A, DTensor const &B);
  DTensor *matmul(DTensor const *A, DTensor const *B);
  KNOperator *create_matmul_op(DTensor const &A, DTensor const &B);
  DTensor exp(DTensor const &input);
  DTensor *exp(DTensor const *input);
  KNOperator *create_elementunary_op(DTensor const &input, mirage::type::KNOperatorType type);
  DTensor add(DTensor const &a, DTensor const &b);
  DTensor mul(DTensor const &a, DTensor const &b);
  DTensor div(DTensor const &a, DTensor const &b);
  DTensor *add(DTensor const *a, DTensor const *b);
  DTensor *mul(DTensor const *a, DTensor const *b);
  DTensor *div(DTensor const *a, DTensor const *b);
  KNOperator *create_elementbinary_op(DTensor const &a, DTensor const &b, mirage::type::KNOperatorType type);
  DTensor reduction(DTensor const &input, int dim, int size = 1);
  DTensor *reduction(DTensor const *input, int dim, int size = 1);
  KNOperator *create_reduction_op(DTensor const &input, int dim, int factor);
  std::vector<DTensor> customized(std::vector<DTensor> const &inputs,
                                  mirage::threadblock::ExecutionPlan const &plan);
  KNOperator *create_customized_op(std::vector<DTensor> const &inputs,
                                   mirage::threadblock::ExecutionPlan const &plan);
  std::vector<DTensor> customized(std::vector<DTensor> const &inputs, mirage::threadblock::Graph const &graph);
  KNOperator *create_customized_op(std::vector<DTensor> const &inputs, mirage::threadblock::Graph const &graph);

  std::vector<KNOperator *> operators;
};

} // namespace kernel
} // namespace mirage
