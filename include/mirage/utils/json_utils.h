// Graph JSON wire format (reference: src/kernel/graph.cc:33-159 `to_json` / `from_json`, the `operator json()` of
// every kernel and threadblock operator, NLOHMANN_DEFINE_TYPE_NON_INTRUSIVE of DTensor, STensor and ExecutionPlan,
// the enum name tables of include/mirage/type.h:64-129 and include/mirage/layout.h:28-58, int3/dim3 as {x,y,z}
// objects, src/utils/json_utils.cc).
//
// The reference speaks nlohmann::json values; this library has no third-party JSON dependency, so the same
// documents travel as text.  A caller that has nlohmann/json.hpp on its include path includes
// mirage/utils/json_nlohmann.h and gets the reference's own spellings back: `json j = g;` (to_json by argument
// lookup), `j.get_to(g)` / `from_json(j, g)`, and `mirage::kernel::operator_json(*op)` for `json(*op)`.
// Documents written by the reference (for instance the search checkpoints' "generated_graphs" entries) load
// unchanged, and documents written here load in the reference.
#pragma once
#include "mirage/kernel/graph.h"
#include <string>

namespace mirage {
namespace kernel {

// The graph as a JSON array of operators, keys in alphabetical order as nlohmann's dump() prints them.
std::string to_json_string(Graph const &g);
// One operator: the document the reference's `operator json()` of that operator class builds.
std::string to_json_string(KNOperator const &op);

// Rebuilds the operators described by `text` into `g` (normally an empty graph), following the reference's
// from_json: inputs by shape / data type / layout, matmul / exp / div / add / mul / reduction by the guids of
// their operands, customized operators from their "plan" (the "bgraph" entry only supplies tile layouts).
// Returns false and leaves a message in *error on malformed text, an unknown operator, an operand guid that no
// earlier operator produced, or an operator the builders refuse; operators built before the failure stay in `g`.
bool from_json_string(std::string const &text, Graph &g, std::string *error = nullptr);

} // namespace kernel
} // namespace mirage
