#include "tree_packing.hpp"

#include <algorithm>
#include <cmath>
#include <limits>
#include <stdexcept>

namespace dcpp {
namespace {

constexpr double kEps = 1e-9;

struct Req {
  int block, src;
  std::vector<int> dsts;     // without the source, sorted, unique
  std::vector<int> arrival;  // aligned with dsts, -1 = free
  double size;
};

struct Search {
  const std::vector<Req>& reqs;
  int n_nodes, n_stages;
  int64_t budget, visited = 0;
  bool cut = false;
  double lower = 0.0, best_cost;
  std::vector<std::vector<double>> send, recv;  // [stage][node]
  std::vector<std::vector<TreeEdge>> current, best;

  Search(const std::vector<Req>& r, int nn, int ns, int64_t b, double incumbent_cost,
         const std::vector<std::vector<TreeEdge>>& incumbent)
      : reqs(r), n_nodes(nn), n_stages(ns), budget(b), best_cost(incumbent_cost),
        send(ns, std::vector<double>(nn, 0.0)), recv(ns, std::vector<double>(nn, 0.0)), current(r.size()),
        best(incumbent) {}

  // have[node] = stage in which the node obtained the block (-2: not yet; the source holds -1)
  void dfs(size_t ri, std::vector<int>& have, std::vector<char>& remaining, int n_remaining, std::pair<int, int> last,
           double cur_max) {
    if (best_cost <= lower + kEps || cut) return;
    if (++visited > budget) {
      cut = true;
      return;
    }
    const Req& rq = reqs[ri];
    if (n_remaining == 0) {
      if (ri + 1 == reqs.size()) {
        if (cur_max < best_cost - kEps) {
          best_cost = cur_max;
          best = current;
        }
        return;
      }
      start(ri + 1, cur_max);
      return;
    }
    struct Opt {
      double cost;
      int stage, dst_idx, holder;
    };
    std::vector<Opt> options;
    for (size_t di = 0; di < rq.dsts.size(); ++di) {
      if (!remaining[di]) continue;
      const int d = rq.dsts[di], fixed = rq.arrival[di];
      for (int h = 0; h < n_nodes; ++h) {
        if (have[h] < -1) continue;
        const int lo = fixed >= 0 ? fixed : have[h] + 1, hi = fixed >= 0 ? fixed : n_stages - 1;
        for (int st = std::max(lo, have[h] + 1); st <= hi; ++st) {
          if (std::make_pair(st, d) <= last) continue;
          options.push_back({std::max({cur_max, send[st][h] + rq.size, recv[st][d] + rq.size}), st, int(di), h});
        }
      }
    }
    std::sort(options.begin(), options.end(), [&](const Opt& a, const Opt& b) {
      return std::make_tuple(a.cost, a.stage, rq.dsts[a.dst_idx], a.holder) <
             std::make_tuple(b.cost, b.stage, rq.dsts[b.dst_idx], b.holder);
    });
    for (const Opt& o : options) {
      if (o.cost >= best_cost - kEps) break;  // sorted by cost: nothing better follows
      const int d = rq.dsts[o.dst_idx];
      // every other remaining destination must still be reachable later in (stage, destination) order
      bool feasible = true;
      for (size_t oi = 0; oi < rq.dsts.size() && feasible; ++oi) {
        if (!remaining[oi] || int(oi) == o.dst_idx) continue;
        const int latest = rq.arrival[oi] >= 0 ? rq.arrival[oi] : n_stages - 1;
        if (std::make_pair(latest, rq.dsts[oi]) <= std::make_pair(o.stage, d)) feasible = false;
      }
      if (!feasible) continue;
      send[o.stage][o.holder] += rq.size;
      recv[o.stage][d] += rq.size;
      have[d] = o.stage;
      remaining[o.dst_idx] = 0;
      current[ri].push_back({o.stage, o.holder, d});
      dfs(ri, have, remaining, n_remaining - 1, {o.stage, d}, o.cost);
      current[ri].pop_back();
      remaining[o.dst_idx] = 1;
      have[d] = -2;
      send[o.stage][o.holder] -= rq.size;
      recv[o.stage][d] -= rq.size;
      if (cut) return;
    }
  }

  void start(size_t ri, double cur_max) {
    const Req& rq = reqs[ri];
    std::vector<int> have(n_nodes, -2);
    have[rq.src] = -1;
    std::vector<char> remaining(rq.dsts.size(), 1);
    current[ri].clear();
    dfs(ri, have, remaining, int(rq.dsts.size()), {-1, -1}, cur_max);
    current[ri].clear();
  }
};

double cost_of(const std::vector<Req>& reqs, const std::vector<std::vector<TreeEdge>>& trees, int n_nodes, int n_stages) {
  std::vector<std::vector<double>> send(n_stages, std::vector<double>(n_nodes, 0.0)), recv = send;
  for (size_t i = 0; i < reqs.size(); ++i)
    for (const TreeEdge& e : trees[i]) {
      send[e.stage][e.from] += reqs[i].size;
      recv[e.stage][e.to] += reqs[i].size;
    }
  double m = 0.0;
  for (int s = 0; s < n_stages; ++s)
    for (int n = 0; n < n_nodes; ++n) m = std::max({m, send[s][n], recv[s][n]});
  return m;
}

std::vector<std::vector<TreeEdge>> greedy(const std::vector<Req>& reqs, int n_nodes, int n_stages) {
  std::vector<std::vector<double>> send(n_stages, std::vector<double>(n_nodes, 0.0)), recv = send;
  std::vector<std::vector<TreeEdge>> trees(reqs.size());
  for (size_t ri = 0; ri < reqs.size(); ++ri) {
    const Req& rq = reqs[ri];
    std::vector<int> have(n_nodes, -2);
    have[rq.src] = -1;
    std::vector<int> holders{rq.src};  // in the order they obtained the block
    std::vector<char> remaining(rq.dsts.size(), 1);
    for (size_t left = rq.dsts.size(); left > 0; --left) {
      bool found = false;
      std::tuple<double, int, int> best_key;
      int b_stage = 0, b_holder = 0, b_di = 0;
      for (size_t di = 0; di < rq.dsts.size(); ++di) {
        if (!remaining[di]) continue;
        const int d = rq.dsts[di], fixed = rq.arrival[di];
        for (int h : holders) {
          const int st = fixed >= 0 ? fixed : have[h] + 1;  // earliest feasible stage for this holder
          if (st <= have[h] || st >= n_stages) continue;
          auto key = std::make_tuple(std::max(send[st][h], recv[st][d]) + rq.size, st, h);
          if (!found || key < best_key) {
            found = true;
            best_key = key;
            b_stage = st; b_holder = h; b_di = int(di);
          }
        }
      }
      if (!found) throw std::invalid_argument("tree packing: no holder can serve a destination in its stage");
      const int d = rq.dsts[b_di];
      send[b_stage][b_holder] += rq.size;
      recv[b_stage][d] += rq.size;
      have[d] = b_stage;
      holders.push_back(d);
      remaining[b_di] = 0;
      trees[ri].push_back({b_stage, b_holder, d});
    }
  }
  return trees;
}

}  // namespace

TreePacking pack_multicast_trees(const std::vector<TreeRequest>& requests, int n_nodes, int n_stages, bool exact,
                                 int64_t search_budget) {
  std::vector<Req> reqs;
  for (const TreeRequest& r : requests) {
    if (r.src < 0 || r.src >= n_nodes) throw std::invalid_argument("tree packing: source node out of range");
    if (!r.arrival.empty() && r.arrival.size() != r.dsts.size())
      throw std::invalid_argument("tree packing: arrival list must match the destinations");
    std::map<int, int> dst;  // node -> arrival (sorted, unique)
    for (size_t i = 0; i < r.dsts.size(); ++i) {
      if (r.dsts[i] < 0 || r.dsts[i] >= n_nodes) throw std::invalid_argument("tree packing: destination out of range");
      if (r.dsts[i] == r.src) continue;
      const int a = r.arrival.empty() ? -1 : r.arrival[i];
      if (a >= n_stages) throw std::invalid_argument("tree packing: arrival stage out of range");
      dst[r.dsts[i]] = a;
    }
    Req q{r.block, r.src, {}, {}, r.size};
    for (auto& kv : dst) {
      q.dsts.push_back(kv.first);
      q.arrival.push_back(kv.second);
    }
    reqs.push_back(std::move(q));
  }
  // largest total volume first (ties: block id)
  std::stable_sort(reqs.begin(), reqs.end(), [](const Req& a, const Req& b) {
    return std::make_pair(-a.size * double(a.dsts.size()), a.block) < std::make_pair(-b.size * double(b.dsts.size()), b.block);
  });
  TreePacking out;
  auto trees = greedy(reqs, n_nodes, n_stages);
  out.greedy_cost = out.cost = cost_of(reqs, trees, n_nodes, n_stages);
  if (exact && !reqs.empty()) {
    Search s(reqs, n_nodes, n_stages, search_budget, out.cost, trees);
    // lower bounds: the largest block that moves at all; per node the mandatory receive volume of a
    // stage (fixed arrivals) or spread over all stages (free arrivals)
    std::map<std::pair<int, int>, double> fixed_recv;
    std::vector<double> free_recv(n_nodes, 0.0);
    for (const Req& r : reqs) {
      if (!r.dsts.empty()) s.lower = std::max(s.lower, r.size);
      for (size_t i = 0; i < r.dsts.size(); ++i) {
        if (r.arrival[i] >= 0) fixed_recv[{r.arrival[i], r.dsts[i]}] += r.size;
        else free_recv[r.dsts[i]] += r.size;
      }
    }
    for (auto& kv : fixed_recv) s.lower = std::max(s.lower, kv.second);
    for (double v : free_recv) s.lower = std::max(s.lower, v / n_stages);
    s.start(0, 0.0);
    trees = s.best;
    out.cost = s.best_cost;
    out.proven_optimal = !s.cut;
  }
  for (size_t i = 0; i < reqs.size(); ++i) out.trees[reqs[i].block] = trees[i];
  return out;
}

}  // namespace dcpp
