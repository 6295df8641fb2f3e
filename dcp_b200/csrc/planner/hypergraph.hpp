// Multilevel k-way hypergraph partitioner (connectivity-1 objective, two balance
// constraints) used to place attention work units and their data blocks on devices.
//
// It plays the role KaHyPar / Mt-KaHyPar / PaToH play for the reference planner
// (dcp/graph_partition/graph.py:735-898): vertices carry a (compute, memory) weight pair,
// nets carry the byte volume that crosses a link when the net is cut, and every part has
// its own capacity per weight dimension.  Pipeline: clustering coarsening by heavy-edge
// rating -> greedy growing initial partition (several seeded tries) -> label-propagation
// refinement with exact km1 gains at every level.  Fully deterministic for a given seed.
#pragma once
#include <cstdint>
#include <vector>

namespace dcpp {

struct Hypergraph {
  int n_vertices = 0;
  std::vector<int64_t> vw_comp, vw_mem;      // vertex weights
  std::vector<int64_t> net_weight;           // per net
  std::vector<int> net_offsets, net_pins;    // CSR: pins of net e = net_pins[net_offsets[e]..net_offsets[e+1])
  std::vector<int> vtx_offsets, vtx_nets;    // CSR: nets of vertex v (built by finalize)
  int n_nets() const { return int(net_weight.size()); }
  void finalize();
};

struct PartitionConfig {
  int k = 2;
  std::vector<int64_t> cap_comp, cap_mem;    // per part capacities (size k)
  uint64_t seed = 42;
  int n_tries = 4;
  int max_refine_passes = 12;
  int coarsen_limit_per_part = 48;           // stop coarsening below k * this many vertices
  std::vector<int> fixed;                    // optional: fixed part per vertex (-1 = free)
};

struct PartitionResult {
  std::vector<int> part;
  int64_t km1 = 0;
  std::vector<int64_t> load_comp, load_mem;
  bool balanced = true;
};

int64_t connectivity_minus_one(const Hypergraph& hg, const std::vector<int>& part, int k);
PartitionResult partition(const Hypergraph& hg, const PartitionConfig& cfg);
// refine an existing assignment in place; returns the km1 improvement
int64_t refine(const Hypergraph& hg, const PartitionConfig& cfg, std::vector<int>& part);

}  // namespace dcpp
