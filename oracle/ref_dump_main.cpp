// TEST INFRASTRUCTURE ONLY.  Driver around the reference's own .param/.bin loader
// (lib/Graph/graph.cpp + lib/Graph/parser.cpp, compiled where they lie, never
// copied): prints Graph::dump() followed by one FNV-1a hash per weight tensor, or
// "ERROR: <message>" when the reference rejects the files.  The output pins the
// product loader and the Python oracle's reader to the reference's behaviour.
#include <cstdint>
#include <cstdio>
#include <string>

#include "ncnn-mlir/Graph/graph.hpp"

int main(int argc, char** argv) {
  if (argc < 2) {
    std::fprintf(stderr, "usage: ref_dump model.param [model.bin]\n");
    return 2;
  }
  auto graph = ncnn_graph::Graph::load(argv[1], argc > 2 ? argv[2] : "");
  if (!graph) {
    std::printf("ERROR: %s\n", graph.error().c_str());
    return 1;
  }
  std::fputs(graph->dump().c_str(), stdout);
  std::printf("weights:\n");
  std::size_t index = 0;
  for (const auto& layer : graph->get_layers()) {
    std::size_t slot = 0;
    for (const auto& weight : layer.get_weights()) {
      std::uint64_t hash = 1469598103934665603ull;
      for (std::byte b : weight.get_data()) {
        hash ^= static_cast<std::uint8_t>(b);
        hash *= 1099511628211ull;
      }
      std::printf("  [%3zu].%zu %016llx\n", index, slot++, static_cast<unsigned long long>(hash));
    }
    ++index;
  }
  return 0;
}
