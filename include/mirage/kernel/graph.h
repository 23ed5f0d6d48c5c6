// kernel::Graph - builder of the kernel graph (reference: include/mirage/kernel/graph.h:28-85).
// Same method names and conventions: value-returning builders assert, `create_*_op` return
// nullptr when the result does not fit the device arena or the shapes are invalid.
#pragma once
#include "mirage/kernel/customized.h"
#include "mirage/kernel/device_tensor.h"
#include "mirage/kernel/operator.h"
#include "mirage/threadblock/graph.h"
#include <memory>
#include <vector>

namespace mirage {
namespace kernel {

class Graph {
public:
  Graph(void);
  // Copies are shallow, as in the reference (its Graph is a plain struct around `operators`, and callers such as
  // the search keep graphs by value, src/search/search.cc:13-21): the operator list is copied, the operators
  // themselves are shared.  The reference never deletes operators; here the LAST live copy of a graph deletes
  // the operators still in its list, in reverse order (arena frees are LIFO).  A caller that deletes operators
  // itself (the search pops and deletes while backtracking) removes them from the list first, as it does today,
  // or calls release() to take over ownership of everything.
  Graph(Graph const &other);
  Graph &operator=(Graph const &other);
  ~Graph();
  void release(); // this copy, and every copy made from it afterwards, no longer deletes anything

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

private:
  void drop();
  std::shared_ptr<int> owners_; // one count shared by all copies; null after release()
};

} // namespace kernel
} // namespace mirage
