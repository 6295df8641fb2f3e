#include "stage_greedy.hpp"

#include <algorithm>
#include <limits>

namespace dcpp {

namespace {

struct Loads {
  std::map<Device, double> inter_send, inter_recv, intra_send, intra_recv;
};

struct Fetch {
  int input;
  Device src;
  double size;
  bool inter;
};

double budget_of(const std::map<Device, double>& b, const Device& d) {
  if (b.empty()) return std::numeric_limits<double>::infinity();
  auto it = b.find(d);
  return it == b.end() ? std::numeric_limits<double>::infinity() : it->second;
}

}  // namespace

GreedyResult greedy_selection_per_device(
    const std::vector<Device>& devices_in, const std::set<int>& scheduled, const std::vector<double>& work_cost,
    const std::vector<double>& input_size, const std::vector<std::vector<int>>& work_inputs,
    const std::vector<std::string>& input_type, const std::map<Device, std::vector<int>>& device_work,
    std::map<Device, std::map<int, int>> local_inputs, const std::map<Device, double>& inter_budget,
    const std::map<Device, double>& intra_budget, bool is_bw, int stage_id) {
  std::vector<Device> devices(devices_in);
  std::sort(devices.begin(), devices.end());
  GreedyResult res;
  Loads loads;

  // holders[input] = devices that owned the block before this stage started (sorted)
  std::vector<std::vector<Device>> holders(input_size.size());
  for (const Device& d : devices) {
    auto it = local_inputs.find(d);
    if (it == local_inputs.end()) continue;
    for (const auto& kv : it->second)
      if (kv.second < stage_id && kv.first >= 0 && size_t(kv.first) < holders.size()) holders[kv.first].push_back(d);
  }
  auto eff_size = [&](int input) {
    double s = input_size[input];
    // in backward the output block travels with its gradient: count it twice
    if (is_bw && input_type[input] == "OUT") s *= 2.0;
    return s;
  };

  // pending work per device, most expensive first
  std::map<Device, std::vector<int>> pending;
  for (const Device& d : devices) {
    auto it = device_work.find(d);
    if (it == device_work.end()) continue;
    std::vector<int> w;
    for (int id : it->second)
      if (!scheduled.count(id)) w.push_back(id);
    std::sort(w.begin(), w.end(), [&](int a, int b) {
      return work_cost[a] != work_cost[b] ? work_cost[a] > work_cost[b] : a < b;
    });
    pending[d] = std::move(w);
  }

  // plan the fetches one input needs on device d; returns false if no holder exists
  auto plan_fetch = [&](const Device& d, int input, const Device* preferred, Loads& scratch, Fetch& out) -> bool {
    const auto& hs = holders[input];
    if (hs.empty()) return false;
    const Device* best = nullptr;
    bool best_inter = true;
    double best_load = 0;
    if (preferred)
      for (const Device& h : hs)
        if (h == *preferred) { best = &h; best_inter = h.first != d.first; }
    if (!best) {
      for (const Device& h : hs) {
        const bool inter = h.first != d.first;
        const double load = inter ? scratch.inter_send[h] : scratch.intra_send[h];
        if (!best || (best_inter && !inter) || (best_inter == inter && load < best_load)) {
          best = &h; best_inter = inter; best_load = load;
        }
      }
    }
    out = Fetch{input, *best, eff_size(input), best_inter};
    return true;
  };
  auto within = [&](const Fetch& f, const Device& dst, const Loads& l) {
    auto get = [](const std::map<Device, double>& m, const Device& k) {
      auto it = m.find(k);
      return it == m.end() ? 0.0 : it->second;
    };
    if (f.inter)
      return get(l.inter_send, f.src) + f.size <= budget_of(inter_budget, f.src) &&
             get(l.inter_recv, dst) + f.size <= budget_of(inter_budget, dst);
    return get(l.intra_send, f.src) + f.size <= budget_of(intra_budget, f.src) &&
           get(l.intra_recv, dst) + f.size <= budget_of(intra_budget, dst);
  };
  auto apply = [&](const Fetch& f, const Device& dst, Loads& l) {
    if (f.inter) { l.inter_send[f.src] += f.size; l.inter_recv[dst] += f.size; }
    else { l.intra_send[f.src] += f.size; l.intra_recv[dst] += f.size; }
  };

  std::map<Device, double> ready_time;
  std::set<Device> exhausted;
  for (const Device& d : devices) ready_time[d] = 0.0;
  while (exhausted.size() < devices.size()) {
    // device with the least compute unlocked so far goes next
    const Device* cur = nullptr;
    for (const Device& d : devices) {
      if (exhausted.count(d)) continue;
      if (!cur || ready_time[d] < ready_time[*cur]) cur = &d;
    }
    const Device d = *cur;
    auto& pend = pending[d];
    auto& mine = local_inputs[d];
    bool took = false;
    for (size_t idx = 0; idx < pend.size() && !took; ++idx) {
      const int w = pend[idx];
      Loads scratch = loads;
      std::vector<Fetch> fetches;
      bool feasible = true;
      const Device* preferred = nullptr;
      Device pref_store;
      for (int input : work_inputs[w]) {
        if (mine.count(input)) continue;
        Fetch f;
        if (!plan_fetch(d, input, preferred, scratch, f) || !within(f, d, scratch)) { feasible = false; break; }
        apply(f, d, scratch);
        fetches.push_back(f);
        pref_store = f.src;
        preferred = &pref_store;
      }
      if (!feasible) continue;
      loads = scratch;
      for (const Fetch& f : fetches) {
        res.comm[d].push_back({f.input, f.src});
        mine[f.input] = stage_id;
      }
      res.unlocked[d].push_back(w);
      ready_time[d] += work_cost[w];
      pend.erase(pend.begin() + long(idx));
      took = true;
    }
    if (!took) exhausted.insert(d);
  }

  // squeeze in prefetches for work that stays behind, while budget remains
  for (const Device& d : devices) {
    auto& mine = local_inputs[d];
    for (int w : pending[d]) {
      const Device* preferred = nullptr;
      Device pref_store;
      for (int input : work_inputs[w]) {
        if (mine.count(input)) continue;
        Fetch f;
        if (!plan_fetch(d, input, preferred, loads, f)) continue;
        if (!within(f, d, loads)) continue;
        apply(f, d, loads);
        res.comm[d].push_back({f.input, f.src});
        mine[f.input] = stage_id;
        pref_store = f.src;
        preferred = &pref_store;
      }
    }
  }
  res.local_inputs = std::move(local_inputs);
  return res;
}

}  // namespace dcpp
