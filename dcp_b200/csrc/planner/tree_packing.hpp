// Multicast tree packing: which node sends a block to which node in which stage, so that the
// largest volume any node sends or receives in one stage is minimal.  Greedy longest-first
// packing followed by an exact depth-first branch and bound (optimal when the search finishes
// inside its budget, else the best packing found).  Role of the OR-tools CP-SAT model of the
// reference (dcp/core/steiner_tree_packing.py:14-167).
#pragma once

#include <cstdint>
#include <map>
#include <set>
#include <tuple>
#include <utility>
#include <vector>

namespace dcpp {

struct TreeRequest {
  int block = 0;
  int src = 0;
  std::vector<int> dsts;    // destination nodes (the source itself is ignored)
  double size = 0.0;
  std::vector<int> arrival;  // per destination: the stage it must arrive in, or -1 (free); empty = all free
};

struct TreeEdge {
  int stage, from, to;
};

struct TreePacking {
  std::map<int, std::vector<TreeEdge>> trees;  // block -> edges
  double cost = 0.0;
  double greedy_cost = 0.0;
  bool proven_optimal = false;
};

TreePacking pack_multicast_trees(const std::vector<TreeRequest>& requests, int n_nodes, int n_stages, bool exact,
                                 int64_t search_budget);

}  // namespace dcpp
