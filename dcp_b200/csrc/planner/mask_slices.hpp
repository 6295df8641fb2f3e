// Per query block: clamp every query's (at most two) key intervals to each KV block of its
// sequence, rebase them to the block start and count the allowed (query, key) pairs.
// This is the inner loop of workload generation (one call per query block instead of one
// Python iteration per (query block, KV block) pair); the reference does it pair by pair in
// Python (dcp/data/dataloader.py:1392-1545).
#pragma once
#include <cstdint>
#include <vector>

namespace dcpp {

struct MaskSlices {
  std::vector<int> kv_blocks;        // KV blocks with at least one allowed pair, ascending
  std::vector<int64_t> allowed;      // allowed pairs of each listed block
  std::vector<int32_t> local;        // [listed block][range 2][bound 2][n_q] rebased intervals
};

// rng: [n_tokens][2 ranges][2 bounds] in sequence coordinates (row-major), queries [q_lo, q_hi)
MaskSlices slice_mask_pairs(const int64_t* rng, int64_t q_lo, int64_t q_hi, int n_blk, int64_t block_size);

}  // namespace dcpp
