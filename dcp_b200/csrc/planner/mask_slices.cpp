#include "mask_slices.hpp"

#include <algorithm>

namespace dcpp {

MaskSlices slice_mask_pairs(const int64_t* rng, int64_t q_lo, int64_t q_hi, int n_blk, int64_t block_size) {
  MaskSlices out;
  const int64_t n_q = q_hi - q_lo;
  if (n_q <= 0 || n_blk <= 0) return out;
  // the union of all intervals bounds the KV blocks that can be non-empty
  int64_t lo_all = INT64_MAX, hi_all = INT64_MIN;
  for (int64_t q = q_lo; q < q_hi; ++q) {
    const int64_t* r = rng + q * 4;
    for (int k = 0; k < 2; ++k) {
      if (r[2 * k + 1] > r[2 * k]) {
        lo_all = std::min(lo_all, r[2 * k]);
        hi_all = std::max(hi_all, r[2 * k + 1]);
      }
    }
  }
  if (hi_all <= lo_all) return out;
  const int j0 = int(std::max<int64_t>(0, lo_all / block_size));
  const int j1 = int(std::min<int64_t>(n_blk, (hi_all + block_size - 1) / block_size));
  std::vector<int32_t> tile(size_t(4) * n_q);
  for (int j = j0; j < j1; ++j) {
    const int64_t lo = int64_t(j) * block_size, hi = lo + block_size;
    int64_t count = 0;
    for (int64_t q = 0; q < n_q; ++q) {
      const int64_t* r = rng + (q_lo + q) * 4;
      int64_t s[2], e[2];
      for (int k = 0; k < 2; ++k) {
        s[k] = std::min(std::max(r[2 * k], lo), hi) - lo;
        e[k] = std::min(std::max(r[2 * k + 1], lo), hi) - lo;
        e[k] = std::max(e[k], s[k]);
        if (e[k] - s[k] <= 0) s[k] = e[k] = 0;
      }
      const int64_t overlap = std::max<int64_t>(0, std::min(e[0], e[1]) - std::max(s[0], s[1]));
      count += (e[0] - s[0]) + (e[1] - s[1]) - overlap;
      // layout [range][bound][n_q]
      tile[(0 * 2 + 0) * n_q + q] = int32_t(s[0]);
      tile[(0 * 2 + 1) * n_q + q] = int32_t(e[0]);
      tile[(1 * 2 + 0) * n_q + q] = int32_t(s[1]);
      tile[(1 * 2 + 1) * n_q + q] = int32_t(e[1]);
    }
    if (count > 0) {
      out.kv_blocks.push_back(j);
      out.allowed.push_back(count);
      out.local.insert(out.local.end(), tile.begin(), tile.end());
    }
  }
  return out;
}

}  // namespace dcpp
