// Compiles against the C++ facade (include/mirage/**) exactly like the reference's
// cpp_examples/group_query_attn_inc_decode.cc uses its own headers: un-fused graph, two customized operators
// built from ExecutionPlans, then shape / plan checks.  Runs on a planning-only device memory manager
// (no GPU): operators can be built and lowered, launching is refused.
#include "mirage/kernel/device_memory_manager.h"
#include "mirage/kernel/graph.h"
#include "mirage/utils/json_utils.h"
#ifdef MG_TEST_NLOHMANN
#include "mirage/utils/json_nlohmann.h"
#endif
#include "mirage/threadblock/graph.h"
#include <cstdio>
#include <cstdlib>

using namespace mirage;

#define CHECK(cond)                                                   \
  do {                                                                \
    if (!(cond)) {                                                    \
      std::fprintf(stderr, "CHECK failed: %s (line %d)\n", #cond, __LINE__); \
      return 1;                                                       \
    }                                                                 \
  } while (0)

int main() {
  char const *err = nullptr;
  CHECK(kernel::DeviceMemoryManager::create(-1, (size_t)1 << 30, &err) == 0);
  {
    kernel::Graph ref_graph;
    kernel::DTensor Q = ref_graph.new_input({2, 8, 64}, type::DT_FLOAT16, layout::DmemRowMajor);
    kernel::DTensor K = ref_graph.new_input({2, 64, 4096}, type::DT_FLOAT16, layout::DmemColumnMajor);
    kernel::DTensor V = ref_graph.new_input({2, 4096, 64}, type::DT_FLOAT16, layout::DmemColumnMajor);
    kernel::DTensor A = ref_graph.matmul(Q, K);
    kernel::DTensor E = ref_graph.exp(A);
    kernel::DTensor S = ref_graph.reduction(E, 2 /*dim*/);
    kernel::DTensor D = ref_graph.div(E, S);
    kernel::DTensor O = ref_graph.matmul(D, V);
    CHECK(A.dim[2] == 4096 && S.dim[2] == 1 && O.dim[1] == 8 && O.dim[2] == 64);
    CHECK(ref_graph.create_matmul_op(Q, V) == nullptr); // inner dimensions differ

    kernel::Graph graph;
    kernel::DTensor q = graph.new_input({2, 8, 64}, type::DT_FLOAT16, layout::DmemRowMajor);
    kernel::DTensor k = graph.new_input({2, 64, 4096}, type::DT_FLOAT16, layout::DmemColumnMajor);
    kernel::DTensor v = graph.new_input({2, 4096, 64}, type::DT_FLOAT16, layout::DmemColumnMajor);
    std::vector<kernel::DTensor> outputs;
    {
      threadblock::ExecutionPlan plan;
      plan.ops.push_back({type::TB_MATMUL_OP, {{0, 0}, {1, 0}}});
      plan.ops.push_back({type::TB_EXP_OP, {{3, 0}}});
      plan.ops.push_back({type::TB_MATMUL_OP, {{4, 0}, {2, 0}}});
      plan.ops.push_back({type::TB_REDUCTION_2_OP, {{4, 0}}});
      plan.input_map = {{0, -1, -1}, {0, 2, -1}, {0, 1, -1}};
      plan.input_smem_layouts = {layout::SmemRowMajorTensorOpMultiplicand_Crosswise64,
                                 layout::SmemColumnMajorTensorOpMultiplicand_Crosswise64,
                                 layout::SmemColumnMajorTensorOpMultiplicand_Crosswise64};
      plan.output_map = {0, 2, -1};
      plan.forloop_dim = {-1, 2, 1};
      plan.grid_dim = {2, 16, 1};
      plan.block_dim = {128, 1, 1};
      plan.forloop_range = 4;
      plan.reduction_dimx = 64;
      outputs = graph.customized({q, k, v}, plan);
      CHECK(outputs.size() == 2);
      CHECK(outputs[0].dim[0] == 2 && outputs[0].dim[1] == 8 && outputs[0].dim[2] == 1024);
      CHECK(outputs[1].dim[2] == 16);
      auto *op = static_cast<kernel::KNCustomizedOp *>(graph.operators.back());
      CHECK(op->bgraph.operators.size() == 9);
      CHECK(op->bgraph.smem_offset == 20512); // same shared-memory plan as the reference's builder
      // an invalid plan yields nullptr instead of an operator
      plan.grid_dim = {2, 3, 1};
      CHECK(graph.create_customized_op({q, k, v}, plan) == nullptr);
    }
    {
      threadblock::ExecutionPlan plan;
      plan.ops.push_back({type::TB_REDUCTION_2_TO_DIMX_OP, {{0, 0}}});
      plan.ops.push_back({type::TB_REDUCTION_2_OP, {{1, 0}}});
      plan.ops.push_back({type::TB_DIV_OP, {{2, 0}, {3, 0}}});
      plan.input_map = {{0, -1, -1}, {0, -1, -1}};
      plan.input_smem_layouts = {layout::SmemRowMajor, layout::SmemRowMajor};
      plan.output_map = {0, -1, -1};
      plan.forloop_dim = {-1, -1};
      plan.grid_dim = {2, 1, 1};
      plan.block_dim = {128, 1, 1};
      plan.forloop_range = 1;
      plan.reduction_dimx = 64;
      outputs = graph.customized({outputs[0], outputs[1]}, plan);
      CHECK(outputs.size() == 1 && outputs[0].dim[2] == 64);
      auto *op = static_cast<kernel::KNCustomizedOp *>(graph.operators.back());
      CHECK(op->bgraph.smem_offset == 19728);
    }
    // the template-graph constructor replays an existing threadblock graph
    {
      auto *first = static_cast<kernel::KNCustomizedOp *>(graph.operators[3]);
      kernel::KNOperator *copy = graph.create_customized_op({q, k, v}, first->bgraph);
      CHECK(copy != nullptr && copy->output_tensors.size() == 2);
      CHECK(static_cast<kernel::KNCustomizedOp *>(copy)->plan.ops.size() == 4);
      delete copy;
    }
    // JSON wire format: dump, rebuild into a second graph, dump again
    {
      std::string doc = kernel::to_json_string(graph);
      CHECK(doc.find("\"kn_customized_op\"") != std::string::npos && doc.find("\"tb_matmul_op\"") != std::string::npos);
      kernel::Graph again;
      std::string err;
      CHECK(kernel::from_json_string(doc, again, &err));
      CHECK(again.operators.size() == graph.operators.size());
      auto *a = static_cast<kernel::KNCustomizedOp *>(again.operators[3]);
      auto *b = static_cast<kernel::KNCustomizedOp *>(graph.operators[3]);
      CHECK(a->bgraph.smem_offset == b->bgraph.smem_offset && a->output_tensors.size() == b->output_tensors.size());
      CHECK(!kernel::from_json_string("[{\"op_type\": \"kn_matmul_op\"}]", again, &err) && !err.empty());
    }
    // copies are shallow and share ownership, as the reference's callers expect: a copy taken by value (the
    // search keeps the computation graph that way) sees the same operators, grows on its own, and going out of
    // scope deletes nothing while the original lives
    {
      size_t before = (size_t)kernel::DeviceMemoryManager::get_instance()->offset;
      {
        kernel::Graph by_value = graph;
        CHECK(by_value.operators.size() == graph.operators.size() && by_value.operators[3] == graph.operators[3]);
        kernel::Graph assigned;
        assigned = by_value;
        CHECK(assigned.operators.back() == graph.operators.back());
      }
      CHECK((size_t)kernel::DeviceMemoryManager::get_instance()->offset == before);
      CHECK(graph.operators.back()->output_tensors.size() == 1);
    }
#ifdef MG_TEST_NLOHMANN
    // the nlohmann::json spellings of the wire format (header-only adapter over the text functions)
    {
      json j = graph;
      CHECK(j.is_array() && j.size() == graph.operators.size() && j[3]["op_type"] == "kn_customized_op");
      CHECK(kernel::operator_json(*graph.operators[0])["op_type"] == "kn_input_op");
      kernel::Graph rebuilt;
      j.get_to(rebuilt);
      CHECK(rebuilt.operators.size() == graph.operators.size());
      CHECK(json(rebuilt).dump().size() == j.dump().size());
    }
#endif
    // no device: nothing can be computed here, and the library says so instead of falling back
    CHECK(graph.operators.back()->fingerprint() == false);
    ProfileResult result;
    CHECK(graph.operators.back()->profile(result) == false);
  }
  kernel::DeviceMemoryManager *dmm = kernel::DeviceMemoryManager::get_instance();
  CHECK((size_t)dmm->offset <= 2048); // everything was released in LIFO order
  kernel::DeviceMemoryManager::destroy();
  std::printf("facade ok\n");
  return 0;
}
