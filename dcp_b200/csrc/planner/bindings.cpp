// pybind11 surface of the native planner: hypergraph partitioning and stage selection.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "hypergraph.hpp"
#include "kernel_tables.hpp"
#include "mask_slices.hpp"
#include "stage_greedy.hpp"
#include "tree_packing.hpp"

namespace py = pybind11;
using namespace dcpp;

namespace {

py::tuple py_greedy(const std::set<Device>& devices, const std::set<int>& scheduled,
                    const std::vector<double>& work_cost, const std::vector<double>& input_size,
                    const std::vector<std::vector<int>>& work_inputs, const std::vector<std::string>& input_type,
                    const std::map<Device, std::vector<int>>& device_work,
                    const std::map<Device, std::map<int, int>>& local_inputs,
                    const std::map<Device, double>& inter_budget, bool is_bw, int stage_id, py::object /*logger*/,
                    const std::map<Device, double>& intra_budget) {
  std::vector<Device> devs(devices.begin(), devices.end());
  GreedyResult r;
  {
    py::gil_scoped_release release;
    r = greedy_selection_per_device(devs, scheduled, work_cost, input_size, work_inputs, input_type, device_work,
                                    local_inputs, inter_budget, intra_budget, is_bw, stage_id);
  }
  py::dict unlocked;
  for (auto& kv : r.unlocked) {
    py::set s;
    for (int w : kv.second) s.add(py::int_(w));
    unlocked[py::make_tuple(kv.first.first, kv.first.second)] = s;
  }
  py::dict comm;
  for (auto& kv : r.comm) {
    py::list l;
    for (auto& c : kv.second) l.append(py::make_tuple(c.first, py::make_tuple(c.second.first, c.second.second)));
    comm[py::make_tuple(kv.first.first, kv.first.second)] = l;
  }
  return py::make_tuple(unlocked, comm, r.local_inputs);
}

py::dict py_partition(int n_vertices, const std::vector<int64_t>& vw_comp, const std::vector<int64_t>& vw_mem,
                      const std::vector<int>& net_offsets, const std::vector<int>& net_pins,
                      const std::vector<int64_t>& net_weight, int k, const std::vector<int64_t>& cap_comp,
                      const std::vector<int64_t>& cap_mem, uint64_t seed, int n_tries, const std::vector<int>& fixed,
                      const std::vector<int>& initial) {
  Hypergraph hg;
  hg.n_vertices = n_vertices;
  hg.vw_comp = vw_comp;
  hg.vw_mem = vw_mem;
  hg.net_offsets = net_offsets;
  hg.net_pins = net_pins;
  hg.net_weight = net_weight;
  if (int(vw_comp.size()) != n_vertices || int(vw_mem.size()) != n_vertices ||
      net_offsets.size() != net_weight.size() + 1 || int(cap_comp.size()) != k || int(cap_mem.size()) != k)
    throw std::invalid_argument("inconsistent hypergraph arrays");
  for (int p : net_pins)
    if (p < 0 || p >= n_vertices) throw std::invalid_argument("pin out of range");
  PartitionConfig cfg;
  cfg.k = k;
  cfg.cap_comp = cap_comp;
  cfg.cap_mem = cap_mem;
  cfg.seed = seed;
  cfg.n_tries = n_tries;
  cfg.fixed = fixed;
  PartitionResult r;
  {
    py::gil_scoped_release release;
    hg.finalize();
    if (!initial.empty()) {
      r.part = initial;
      refine(hg, cfg, r.part);
      r.km1 = connectivity_minus_one(hg, r.part, k);
      r.load_comp.assign(k, 0);
      r.load_mem.assign(k, 0);
      for (int v = 0; v < n_vertices; ++v) { r.load_comp[r.part[v]] += vw_comp[v]; r.load_mem[r.part[v]] += vw_mem[v]; }
      r.balanced = true;
      for (int p = 0; p < k; ++p) r.balanced = r.balanced && r.load_comp[p] <= cap_comp[p] && r.load_mem[p] <= cap_mem[p];
    } else {
      r = partition(hg, cfg);
    }
  }
  py::dict out;
  out["part"] = r.part;
  out["km1"] = r.km1;
  out["load_comp"] = r.load_comp;
  out["load_mem"] = r.load_mem;
  out["balanced"] = r.balanced;
  return out;
}

int64_t py_km1(int n_vertices, const std::vector<int>& net_offsets, const std::vector<int>& net_pins,
               const std::vector<int64_t>& net_weight, const std::vector<int>& part, int k) {
  Hypergraph hg;
  hg.n_vertices = n_vertices;
  hg.net_offsets = net_offsets;
  hg.net_pins = net_pins;
  hg.net_weight = net_weight;
  return connectivity_minus_one(hg, part, k);
}

// requests: (block, source node, destination nodes, size, arrival stage per destination or empty)
py::dict py_pack_trees(const std::vector<std::tuple<int, int, std::vector<int>, double, std::vector<int>>>& requests,
                       int n_nodes, int n_stages, bool exact, int64_t search_budget) {
  std::vector<TreeRequest> reqs;
  for (auto& r : requests) {
    TreeRequest t;
    t.block = std::get<0>(r);
    t.src = std::get<1>(r);
    t.dsts = std::get<2>(r);
    t.size = std::get<3>(r);
    t.arrival = std::get<4>(r);
    reqs.push_back(std::move(t));
  }
  TreePacking p;
  {
    py::gil_scoped_release release;
    p = pack_multicast_trees(reqs, n_nodes, n_stages, exact, search_budget);
  }
  py::dict trees;
  for (auto& kv : p.trees) {
    py::list l;
    for (auto& e : kv.second) l.append(py::make_tuple(e.stage, e.from, e.to));
    trees[py::int_(kv.first)] = l;
  }
  py::dict out;
  out["trees"] = trees;
  out["cost"] = p.cost;
  out["greedy_cost"] = p.greedy_cost;
  out["proven_optimal"] = p.proven_optimal;
  return out;
}

// one attention row = (q_row, n_tokens, heads, [(kv row, tokens)], ranges int32 [n_tokens, 4], out_dev, out_row,
// dq_dev, dq_row, [(dkv device, dkv row)])
using PyAttnRow = std::tuple<int64_t, int64_t, std::vector<int>, std::vector<std::pair<int64_t, int64_t>>,
                             py::array_t<int32_t, py::array::c_style | py::array::forcecast>, int64_t, int64_t, int64_t,
                             int64_t, std::vector<std::pair<int64_t, int64_t>>>;

std::vector<AttnRowDesc> to_rows(const std::vector<PyAttnRow>& rows) {
  std::vector<AttnRowDesc> out;
  out.reserve(rows.size());
  for (const PyAttnRow& r : rows) {
    AttnRowDesc d;
    d.q_row = std::get<0>(r);
    d.n_tokens = std::get<1>(r);
    d.heads = std::get<2>(r);
    d.kv = std::get<3>(r);
    const auto& rng = std::get<4>(r);
    if (rng.size() != 4 * d.n_tokens) throw std::invalid_argument("ranges must be [n_tokens, 4]");
    d.ranges = rng.data();
    d.out_dev = std::get<5>(r);
    d.out_row = std::get<6>(r);
    d.dq_dev = std::get<7>(r);
    d.dq_row = std::get<8>(r);
    d.dkv = std::get<9>(r);
    if (!d.dkv.empty() && d.dkv.size() != d.kv.size()) throw std::invalid_argument("dkv must match kv");
    out.push_back(std::move(d));
  }
  return out;
}

py::array_t<int32_t> to_array(const std::vector<int32_t>& v, int width) {
  py::array_t<int32_t> a({py::ssize_t(v.size() / size_t(width)), py::ssize_t(width)});
  std::copy(v.begin(), v.end(), a.mutable_data());
  return a;
}

py::tuple py_build_fwd_tables(const std::vector<PyAttnRow>& rows, int64_t block_size, int tile_m) {
  const auto desc = to_rows(rows);     // `rows` keeps the range arrays alive
  FwdTablesOut t = build_fwd_tables(desc, block_size, tile_m);
  return py::make_tuple(to_array(t.tiles, 8), to_array(t.entries, tile_m == 128 ? 2 : 4), to_array(t.masks, 4), t.pairs);
}

py::tuple py_build_bwd_tables(const std::vector<PyAttnRow>& rows, int64_t block_size, int hq) {
  const auto desc = to_rows(rows);
  BwdTablesOut t = build_bwd_tables(desc, block_size, hq);
  return py::make_tuple(to_array(t.ctas, 8), to_array(t.items, 8), to_array(t.masks, 4), t.pairs);
}

}  // namespace

namespace {

// rng: int64 [T, 2, 2] C-contiguous -> (kv block indices, allowed pair counts, int32 [n, 2, 2, n_q])
py::tuple py_slice_mask_pairs(py::array_t<int64_t, py::array::c_style | py::array::forcecast> rng, int64_t q_lo,
                              int64_t q_hi, int n_blk, int64_t block_size) {
  if (rng.ndim() != 3 || rng.shape(1) != 2 || rng.shape(2) != 2) throw std::invalid_argument("rng must be [T, 2, 2]");
  if (q_lo < 0 || q_hi > rng.shape(0) || q_hi < q_lo) throw std::invalid_argument("query range outside the mask");
  MaskSlices r;
  {
    py::gil_scoped_release release;
    r = slice_mask_pairs(rng.data(), q_lo, q_hi, n_blk, block_size);
  }
  const py::ssize_t n = py::ssize_t(r.kv_blocks.size()), n_q = q_hi - q_lo;
  py::array_t<int32_t> local({n, py::ssize_t(2), py::ssize_t(2), n_q});
  std::copy(r.local.begin(), r.local.end(), local.mutable_data());
  return py::make_tuple(r.kv_blocks, r.allowed, local);
}

}  // namespace

PYBIND11_MODULE(_planner, m) {
  m.doc() = "native planner kernels: k-way hypergraph partitioning and per-stage greedy selection";
  m.def("greedy_selection_per_device", &py_greedy, py::arg("devices"), py::arg("scheduled_workloads"),
        py::arg("workload_costs"), py::arg("input_sizes"), py::arg("workload_input_map"),
        py::arg("input_block_type_map"), py::arg("device_workload_map"), py::arg("device_local_inputs_map"),
        py::arg("target_comm_load_per_node"), py::arg("is_bw"), py::arg("stage_id"), py::arg("py_logger") = py::none(),
        py::arg("intra_node_budget") = std::map<Device, double>());
  m.def("partition_hypergraph", &py_partition, py::arg("n_vertices"), py::arg("vw_comp"), py::arg("vw_mem"),
        py::arg("net_offsets"), py::arg("net_pins"), py::arg("net_weight"), py::arg("k"), py::arg("cap_comp"),
        py::arg("cap_mem"), py::arg("seed") = 42, py::arg("n_tries") = 4, py::arg("fixed") = std::vector<int>(),
        py::arg("initial") = std::vector<int>());
  m.def("connectivity_minus_one", &py_km1);
  m.def("build_fwd_tables", &py_build_fwd_tables, py::arg("rows"), py::arg("block_size"), py::arg("tile_m"));
  m.def("build_bwd_tables", &py_build_bwd_tables, py::arg("rows"), py::arg("block_size"), py::arg("hq"));
  m.def("pack_multicast_trees", &py_pack_trees, py::arg("requests"), py::arg("n_nodes"), py::arg("n_stages"),
        py::arg("exact") = true, py::arg("search_budget") = 50000);
  m.def("slice_mask_pairs", &py_slice_mask_pairs, py::arg("rng"), py::arg("q_lo"), py::arg("q_hi"), py::arg("n_blk"),
        py::arg("block_size"));
}
