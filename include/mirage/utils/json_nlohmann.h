// nlohmann::json spellings of the graph wire format, for callers that already use that library (the reference's
// search does: src/search/search.cc keeps candidate graphs as `json` values and its checkpoints are read with
// `from_json`, src/kernel/graph.cc:33-159).  Header-only and thin: every function converts through the text
// form of mirage/utils/json_utils.h, so this library itself still needs no third-party JSON code.  Include it
// only where <nlohmann/json.hpp> is available.
#pragma once
#include "mirage/utils/json_utils.h"
#include <nlohmann/json.hpp>
#include <stdexcept>

using json = nlohmann::json;

namespace mirage {
namespace kernel {

// found by argument-dependent lookup: `json j = graph;`, `json(graph)`
inline void to_json(json &j, Graph const &g) { j = json::parse(to_json_string(g)); }

// `from_json(j, graph)` / `j.get_to(graph)`; the reference asserts on malformed documents, this throws
inline void from_json(json const &j, Graph &g) {
  std::string error;
  if (!from_json_string(j.dump(), g, &error)) throw std::invalid_argument("mirage::kernel::from_json: " + error);
}

// the reference's `json(*op)` (KNOperator::operator json())
inline json operator_json(KNOperator const &op) { return json::parse(to_json_string(op)); }

} // namespace kernel
} // namespace mirage
