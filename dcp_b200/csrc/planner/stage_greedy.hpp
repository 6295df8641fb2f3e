// Greedy per-stage selection of work units and the block transfers that unlock them.
//
// Interface parity with the reference's `dcp_cpp.greedy_selection_per_device`
// (csrc/pipeline_generator/pipeline_generator.hpp:37-50).  Differences by design:
//  * devices, work units and holders are visited in sorted order, so the result is
//    reproducible (the reference iterates unordered containers);
//  * an optional intra-node budget also limits NVLink traffic per stage, because on a
//    single NVSwitch node that is the only traffic there is and the stage split exists to
//    overlap it with the tensor-core work of the previous stage.
#pragma once
#include <cstdint>
#include <map>
#include <set>
#include <string>
#include <tuple>
#include <utility>
#include <vector>

namespace dcpp {

using Device = std::pair<int, int>;  // (node, local device)

struct GreedyResult {
  std::map<Device, std::vector<int>> unlocked;                       // device -> work ids (selection order)
  std::map<Device, std::vector<std::pair<int, Device>>> comm;        // dst -> [(input id, src device)]
  std::map<Device, std::map<int, int>> local_inputs;                 // device -> input id -> stage obtained
};

GreedyResult greedy_selection_per_device(
    const std::vector<Device>& devices, const std::set<int>& scheduled, const std::vector<double>& work_cost,
    const std::vector<double>& input_size, const std::vector<std::vector<int>>& work_inputs,
    const std::vector<std::string>& input_type, const std::map<Device, std::vector<int>>& device_work,
    std::map<Device, std::map<int, int>> local_inputs, const std::map<Device, double>& inter_budget,
    const std::map<Device, double>& intra_budget, bool is_bw, int stage_id);

}  // namespace dcpp
