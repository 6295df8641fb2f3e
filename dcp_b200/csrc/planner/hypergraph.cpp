#include "hypergraph.hpp"

#include <algorithm>
#include <cmath>
#include <numeric>
#include <unordered_map>

namespace dcpp {

namespace {

struct Rng {  // splitmix64: small, deterministic, good enough for tie-breaking and shuffles
  uint64_t s;
  explicit Rng(uint64_t seed) : s(seed ? seed : 0x9E3779B97F4A7C15ull) {}
  uint64_t next() {
    uint64_t z = (s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
  template <class T>
  void shuffle(std::vector<T>& v) {
    for (size_t i = v.size(); i > 1; --i) std::swap(v[i - 1], v[next() % i]);
  }
};

struct State {
  const Hypergraph& hg;
  const PartitionConfig& cfg;
  int k;
  std::vector<int>& part;
  std::vector<int> pins;  // [net * k + p]
  std::vector<int64_t> load_comp, load_mem;

  State(const Hypergraph& h, const PartitionConfig& c, std::vector<int>& p)
      : hg(h), cfg(c), k(c.k), part(p), pins(size_t(h.n_nets()) * c.k, 0), load_comp(c.k, 0), load_mem(c.k, 0) {
    for (int e = 0; e < hg.n_nets(); ++e)
      for (int i = hg.net_offsets[e]; i < hg.net_offsets[e + 1]; ++i) ++pins[size_t(e) * k + part[hg.net_pins[i]]];
    for (int v = 0; v < hg.n_vertices; ++v) {
      load_comp[part[v]] += hg.vw_comp[v];
      load_mem[part[v]] += hg.vw_mem[v];
    }
  }
  bool fits(int v, int p) const {
    return load_comp[p] + hg.vw_comp[v] <= cfg.cap_comp[p] && load_mem[p] + hg.vw_mem[v] <= cfg.cap_mem[p];
  }
  bool overloaded(int p) const { return load_comp[p] > cfg.cap_comp[p] || load_mem[p] > cfg.cap_mem[p]; }
  double rel_load(int p) const {
    double a = cfg.cap_comp[p] > 0 ? double(load_comp[p]) / double(cfg.cap_comp[p]) : 0.0;
    double b = cfg.cap_mem[p] > 0 ? double(load_mem[p]) / double(cfg.cap_mem[p]) : 0.0;
    return std::max(a, b);
  }
  void move(int v, int to) {
    const int from = part[v];
    for (int i = hg.vtx_offsets[v]; i < hg.vtx_offsets[v + 1]; ++i) {
      const int e = hg.vtx_nets[i];
      --pins[size_t(e) * k + from];
      ++pins[size_t(e) * k + to];
    }
    load_comp[from] -= hg.vw_comp[v]; load_mem[from] -= hg.vw_mem[v];
    load_comp[to] += hg.vw_comp[v];   load_mem[to] += hg.vw_mem[v];
    part[v] = to;
  }
  // gains[p] = km1 reduction if v moves to p
  void gains(int v, std::vector<int64_t>& conn, int64_t& benefit, int64_t& total_w) const {
    std::fill(conn.begin(), conn.end(), 0);
    benefit = 0; total_w = 0;
    const int from = part[v];
    for (int i = hg.vtx_offsets[v]; i < hg.vtx_offsets[v + 1]; ++i) {
      const int e = hg.vtx_nets[i];
      const int64_t w = hg.net_weight[e];
      const int* pc = &pins[size_t(e) * k];
      total_w += w;
      if (pc[from] == 1) benefit += w;
      for (int p = 0; p < k; ++p)
        if (pc[p] > 0) conn[p] += w;
    }
  }
};

int64_t refine_impl(const Hypergraph& hg, const PartitionConfig& cfg, std::vector<int>& part, Rng& rng) {
  State st(hg, cfg, part);
  const int k = cfg.k;
  std::vector<int> order(hg.n_vertices);
  std::iota(order.begin(), order.end(), 0);
  std::vector<int64_t> conn(k);
  int64_t improved_total = 0;
  const bool has_fixed = !cfg.fixed.empty();
  for (int pass = 0; pass < cfg.max_refine_passes; ++pass) {
    rng.shuffle(order);
    int64_t improved = 0;
    int moves = 0;
    for (int v : order) {
      if (has_fixed && cfg.fixed[v] >= 0) continue;
      const int from = st.part[v];
      int64_t benefit, total_w;
      st.gains(v, conn, benefit, total_w);
      const bool must_leave = st.overloaded(from);
      int best = -1;
      int64_t best_gain = must_leave ? INT64_MIN : 0;
      double best_rel = 0;
      const double from_rel = st.rel_load(from);
      for (int p = 0; p < k; ++p) {
        if (p == from || !st.fits(v, p)) continue;
        const int64_t g = benefit - (total_w - conn[p]);
        const double rel = st.rel_load(p);
        bool take = false;
        if (g > best_gain) take = true;
        else if (g == best_gain && best >= 0 && rel < best_rel) take = true;
        else if (g == best_gain && best < 0 && !must_leave && g == 0) {
          // zero-gain move only when it clearly evens out the load
          take = rel + 0.02 < from_rel;
        }
        if (take) { best = p; best_gain = g; best_rel = rel; }
      }
      if (best >= 0 && (must_leave || best_gain > 0 || st.rel_load(best) + 0.02 < from_rel)) {
        st.move(v, best);
        improved += best_gain;
        ++moves;
      }
    }
    improved_total += improved;
    if (moves == 0 || (improved <= 0 && pass > 1)) break;
  }
  return improved_total;
}

Hypergraph contract(const Hypergraph& hg, const std::vector<int>& cluster, int n_clusters) {
  Hypergraph c;
  c.n_vertices = n_clusters;
  c.vw_comp.assign(n_clusters, 0);
  c.vw_mem.assign(n_clusters, 0);
  for (int v = 0; v < hg.n_vertices; ++v) {
    c.vw_comp[cluster[v]] += hg.vw_comp[v];
    c.vw_mem[cluster[v]] += hg.vw_mem[v];
  }
  c.net_offsets.push_back(0);
  std::vector<int> tmp;
  for (int e = 0; e < hg.n_nets(); ++e) {
    tmp.clear();
    for (int i = hg.net_offsets[e]; i < hg.net_offsets[e + 1]; ++i) tmp.push_back(cluster[hg.net_pins[i]]);
    std::sort(tmp.begin(), tmp.end());
    tmp.erase(std::unique(tmp.begin(), tmp.end()), tmp.end());
    if (tmp.size() < 2) continue;
    c.net_pins.insert(c.net_pins.end(), tmp.begin(), tmp.end());
    c.net_offsets.push_back(int(c.net_pins.size()));
    c.net_weight.push_back(hg.net_weight[e]);
  }
  c.finalize();
  return c;
}

// one level of clustering; returns number of clusters and fills `cluster`
int coarsen_once(const Hypergraph& hg, const PartitionConfig& cfg, const std::vector<int>& fixed,
                 int64_t max_comp, int64_t max_mem, Rng& rng, std::vector<int>& cluster) {
  const int n = hg.n_vertices;
  cluster.assign(n, -1);
  std::vector<int64_t> c_comp, c_mem;
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  rng.shuffle(order);
  std::unordered_map<int, double> rating;
  int n_clusters = 0;
  auto new_cluster = [&](int v) {
    cluster[v] = n_clusters++;
    c_comp.push_back(hg.vw_comp[v]);
    c_mem.push_back(hg.vw_mem[v]);
  };
  for (int u : order) {
    if (cluster[u] >= 0) continue;
    if (!fixed.empty() && fixed[u] >= 0) { new_cluster(u); continue; }
    rating.clear();
    for (int i = hg.vtx_offsets[u]; i < hg.vtx_offsets[u + 1]; ++i) {
      const int e = hg.vtx_nets[i];
      const int sz = hg.net_offsets[e + 1] - hg.net_offsets[e];
      if (sz < 2 || sz > 512) continue;
      const double r = double(hg.net_weight[e]) / double(sz - 1);
      for (int j = hg.net_offsets[e]; j < hg.net_offsets[e + 1]; ++j) {
        const int v = hg.net_pins[j];
        if (v == u || cluster[v] < 0) continue;
        if (!fixed.empty() && fixed[v] >= 0) continue;
        rating[cluster[v]] += r;
      }
    }
    int best = -1;
    double best_r = 0;
    for (auto& kv : rating) {
      const int c = kv.first;
      if (c_comp[c] + hg.vw_comp[u] > max_comp || c_mem[c] + hg.vw_mem[u] > max_mem) continue;
      if (kv.second > best_r || (kv.second == best_r && best >= 0 && c < best)) { best = c; best_r = kv.second; }
    }
    if (best >= 0) {
      cluster[u] = best;
      c_comp[best] += hg.vw_comp[u];
      c_mem[best] += hg.vw_mem[u];
    } else {
      new_cluster(u);
    }
  }
  return n_clusters;
}

void initial_partition(const Hypergraph& hg, const PartitionConfig& cfg, Rng& rng, std::vector<int>& part) {
  const int n = hg.n_vertices, k = cfg.k;
  part.assign(n, -1);
  std::vector<int> pins(size_t(hg.n_nets()) * k, 0);
  std::vector<int64_t> lc(k, 0), lm(k, 0);
  int64_t tot_c = 1, tot_m = 1;
  for (int v = 0; v < n; ++v) { tot_c += hg.vw_comp[v]; tot_m += hg.vw_mem[v]; }
  std::vector<std::pair<double, int>> keyed(n);
  for (int v = 0; v < n; ++v) {
    const double key = std::max(double(hg.vw_comp[v]) / double(tot_c), double(hg.vw_mem[v]) / double(tot_m));
    keyed[v] = {-(key + 1e-12 * double(rng.next() % 1000)), v};
  }
  std::sort(keyed.begin(), keyed.end());
  auto place = [&](int v, int p) {
    part[v] = p;
    lc[p] += hg.vw_comp[v]; lm[p] += hg.vw_mem[v];
    for (int i = hg.vtx_offsets[v]; i < hg.vtx_offsets[v + 1]; ++i) ++pins[size_t(hg.vtx_nets[i]) * k + p];
  };
  if (!cfg.fixed.empty())
    for (int v = 0; v < n; ++v)
      if (cfg.fixed[v] >= 0) place(v, cfg.fixed[v]);
  std::vector<int64_t> conn(k);
  for (auto& kv : keyed) {
    const int v = kv.second;
    if (part[v] >= 0) continue;
    std::fill(conn.begin(), conn.end(), 0);
    for (int i = hg.vtx_offsets[v]; i < hg.vtx_offsets[v + 1]; ++i) {
      const int e = hg.vtx_nets[i];
      for (int p = 0; p < k; ++p)
        if (pins[size_t(e) * k + p] > 0) conn[p] += hg.net_weight[e];
    }
    int best = -1; int64_t best_conn = -1; double best_rel = 0;
    int fallback = 0; double fallback_rel = 1e300;
    for (int p = 0; p < k; ++p) {
      const double rel = std::max(cfg.cap_comp[p] > 0 ? double(lc[p] + hg.vw_comp[v]) / double(cfg.cap_comp[p]) : 0.0,
                                  cfg.cap_mem[p] > 0 ? double(lm[p] + hg.vw_mem[v]) / double(cfg.cap_mem[p]) : 0.0);
      if (rel < fallback_rel) { fallback_rel = rel; fallback = p; }
      if (rel > 1.0) continue;
      if (conn[p] > best_conn || (conn[p] == best_conn && rel < best_rel)) { best = p; best_conn = conn[p]; best_rel = rel; }
    }
    place(v, best >= 0 ? best : fallback);
  }
}

bool is_balanced(const Hypergraph& hg, const PartitionConfig& cfg, const std::vector<int>& part,
                 std::vector<int64_t>& lc, std::vector<int64_t>& lm) {
  lc.assign(cfg.k, 0); lm.assign(cfg.k, 0);
  for (int v = 0; v < hg.n_vertices; ++v) { lc[part[v]] += hg.vw_comp[v]; lm[part[v]] += hg.vw_mem[v]; }
  for (int p = 0; p < cfg.k; ++p)
    if (lc[p] > cfg.cap_comp[p] || lm[p] > cfg.cap_mem[p]) return false;
  return true;
}

}  // namespace

void Hypergraph::finalize() {
  vtx_offsets.assign(n_vertices + 1, 0);
  for (int p : net_pins) ++vtx_offsets[p + 1];
  for (int v = 0; v < n_vertices; ++v) vtx_offsets[v + 1] += vtx_offsets[v];
  vtx_nets.assign(net_pins.size(), 0);
  std::vector<int> cur(vtx_offsets.begin(), vtx_offsets.end() - 1);
  for (int e = 0; e < n_nets(); ++e)
    for (int i = net_offsets[e]; i < net_offsets[e + 1]; ++i) vtx_nets[cur[net_pins[i]]++] = e;
}

int64_t connectivity_minus_one(const Hypergraph& hg, const std::vector<int>& part, int k) {
  int64_t total = 0;
  std::vector<char> seen(k);
  for (int e = 0; e < hg.n_nets(); ++e) {
    std::fill(seen.begin(), seen.end(), 0);
    int lambda = 0;
    for (int i = hg.net_offsets[e]; i < hg.net_offsets[e + 1]; ++i) {
      const int p = part[hg.net_pins[i]];
      if (!seen[p]) { seen[p] = 1; ++lambda; }
    }
    if (lambda > 1) total += int64_t(lambda - 1) * hg.net_weight[e];
  }
  return total;
}

int64_t refine(const Hypergraph& hg, const PartitionConfig& cfg, std::vector<int>& part) {
  Rng rng(cfg.seed);
  return refine_impl(hg, cfg, part, rng);
}

PartitionResult partition(const Hypergraph& hg, const PartitionConfig& cfg) {
  PartitionResult best;
  const int k = cfg.k;
  if (k <= 1 || hg.n_vertices == 0) {
    best.part.assign(hg.n_vertices, 0);
    is_balanced(hg, cfg, best.part, best.load_comp, best.load_mem);
    return best;
  }
  int64_t tot_c = 0, tot_m = 0, max_vc = 0, max_vm = 0;
  for (int v = 0; v < hg.n_vertices; ++v) {
    tot_c += hg.vw_comp[v]; tot_m += hg.vw_mem[v];
    max_vc = std::max(max_vc, hg.vw_comp[v]); max_vm = std::max(max_vm, hg.vw_mem[v]);
  }
  bool have_best = false;
  for (int attempt = 0; attempt < std::max(1, cfg.n_tries); ++attempt) {
    Rng rng(cfg.seed + 7919ull * uint64_t(attempt));
    // ---- coarsening
    std::vector<Hypergraph> levels;
    std::vector<std::vector<int>> maps;     // maps[l][v at level l] = vertex at level l+1
    std::vector<std::vector<int>> fixeds;   // fixed assignment per level
    levels.push_back(hg);
    fixeds.push_back(cfg.fixed);
    const int64_t max_c = std::max<int64_t>(max_vc, tot_c / (int64_t(k) * 12) + 1);
    const int64_t max_m = std::max<int64_t>(max_vm, tot_m / (int64_t(k) * 12) + 1);
    while (int(levels.size()) < 16 && levels.back().n_vertices > k * cfg.coarsen_limit_per_part) {
      std::vector<int> cluster;
      const Hypergraph& cur = levels.back();
      const int nc = coarsen_once(cur, cfg, fixeds.back(), max_c, max_m, rng, cluster);
      if (nc > cur.n_vertices * 0.95) break;
      std::vector<int> cf;
      if (!fixeds.back().empty()) {
        cf.assign(nc, -1);
        for (int v = 0; v < cur.n_vertices; ++v)
          if (fixeds.back()[v] >= 0) cf[cluster[v]] = fixeds.back()[v];
      }
      Hypergraph coarse = contract(cur, cluster, nc);
      maps.push_back(std::move(cluster));
      fixeds.push_back(std::move(cf));
      levels.push_back(std::move(coarse));
    }
    // ---- initial partition on the coarsest level
    PartitionConfig lcfg = cfg;
    lcfg.fixed = fixeds.back();
    std::vector<int> part;
    initial_partition(levels.back(), lcfg, rng, part);
    refine_impl(levels.back(), lcfg, part, rng);
    // ---- uncoarsening
    for (int l = int(levels.size()) - 2; l >= 0; --l) {
      std::vector<int> fine(levels[l].n_vertices);
      for (int v = 0; v < levels[l].n_vertices; ++v) fine[v] = part[maps[l][v]];
      part.swap(fine);
      lcfg.fixed = fixeds[l];
      refine_impl(levels[l], lcfg, part, rng);
    }
    PartitionResult cand;
    cand.part = part;
    cand.balanced = is_balanced(hg, cfg, part, cand.load_comp, cand.load_mem);
    cand.km1 = connectivity_minus_one(hg, part, k);
    if (!have_best || (cand.balanced && !best.balanced) || (cand.balanced == best.balanced && cand.km1 < best.km1)) {
      best = std::move(cand);
      have_best = true;
    }
  }
  return best;
}

}  // namespace dcpp
