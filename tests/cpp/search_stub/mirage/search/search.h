// Stand-in for the reference's search header, for compiling its cpp_examples unmodified against this library.
// The superoptimizer search is outside the executor; its public names are declared here so that the tail of every
// example (configure a generator, hand it the computation graph, run it) compiles and links.  The generator keeps
// the computation graph BY VALUE, exactly as the reference's does (include/mirage/search/search.h:81), so the
// examples also exercise kernel::Graph's copy semantics; generate_kernel_graphs() reports that no search is done.
#pragma once
#include "mirage/kernel/graph.h"
#include "mirage/threadblock/graph.h"
#include <cstdio>
#include <string>
#include <vector>

namespace mirage {
namespace search {

struct GeneratorConfig {
  std::vector<type::KNOperatorType> knop_to_explore;
  std::vector<type::TBOperatorType> tbop_to_explore;
  std::vector<int3> imap_to_explore;
  std::vector<std::vector<int3>> imap_comb_to_explore;
  std::vector<int3> omap_to_explore;
  std::vector<dim3> grid_dim_to_explore;
  std::vector<dim3> block_dim_to_explore;
  std::vector<int> fmap_to_explore;
  std::vector<int> frange_to_explore;
  std::vector<layout::SmemLayout> smem_layout_to_explore;
  int reduction_dimx = 64;
  void print_config() const {}
  static GeneratorConfig get_default_config() { return GeneratorConfig(); }
  static GeneratorConfig get_attention_default_config() { return GeneratorConfig(); }
  static GeneratorConfig get_mlp_default_config() { return GeneratorConfig(); }
  static GeneratorConfig get_lora_default_config() { return GeneratorConfig(); }
};

class KernelGraphGenerator {
public:
  KernelGraphGenerator(kernel::Graph const &graph, GeneratorConfig const &cfg, char const *file)
      : computation_graph(graph), config(cfg), filename(file ? file : "") {}
  void generate_kernel_graphs() {
    std::printf("[search stand-in] computation graph of %zu operators received by value; no search is run\n",
                computation_graph.operators.size());
  }
  kernel::Graph computation_graph;
  GeneratorConfig config;
  std::string filename;
};

} // namespace search
} // namespace mirage
