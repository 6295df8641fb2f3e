// Work tables of the sm_100a attention kernels, built from the attention rows of one stage of one
// device (a row = one Q block with the KV blocks it attends to and its per-query key ranges).
// Forward: CTA tiles of 256 (two-tile kernel) or 128 query rows, with the walk over 128-key tiles
// each CTA makes; backward: one entry per 128-key tile listing the 64-query tiles that see it.
// The layouts are the ones dcp_b200/ops/attention.py documents (its Python builders are the
// oracle of this file).
#pragma once

#include <cstdint>
#include <utility>
#include <vector>

namespace dcpp {

struct AttnRowDesc {
  int64_t q_row = 0, n_tokens = 0;
  std::vector<int> heads;
  std::vector<std::pair<int64_t, int64_t>> kv;  // (arena row, tokens) per KV block, in concatenation order
  const int32_t* ranges = nullptr;              // [n_tokens, 4] = (s0, e0, s1, e1)
  int64_t out_dev = 0, out_row = 0, dq_dev = 0, dq_row = 0;
  std::vector<std::pair<int64_t, int64_t>> dkv;  // (device, row) per KV block (backward; may be empty)
};

struct FwdTablesOut {
  std::vector<int32_t> tiles;    // [n, 8]
  std::vector<int32_t> entries;  // [m, 2] (tile_m 128) or [m, 4] (tile_m 256)
  std::vector<int32_t> masks;    // [rows, 4]
  double pairs = 0.0;            // allowed (query, key) pairs x heads
};

struct BwdTablesOut {
  std::vector<int32_t> ctas;   // [n, 8]
  std::vector<int32_t> items;  // [m, 8]
  std::vector<int32_t> masks;  // [rows, 4]
  double pairs = 0.0;
};

FwdTablesOut build_fwd_tables(const std::vector<AttnRowDesc>& rows, int64_t block_size, int tile_m);
BwdTablesOut build_bwd_tables(const std::vector<AttnRowDesc>& rows, int64_t block_size, int hq);

}  // namespace dcpp
