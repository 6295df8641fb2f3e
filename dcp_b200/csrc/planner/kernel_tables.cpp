#include "kernel_tables.hpp"

#include <algorithm>
#include <limits>
#include <map>
#include <stdexcept>
#include <tuple>

namespace dcpp {
namespace {

constexpr int64_t kTileN = 128;   // keys per tile
constexpr int64_t kTileM = 128;   // query rows of one forward tile
constexpr int64_t kQTileBwd = 64; // query rows of one backward item

// per query tile: union and intersection of each of the two key ranges over the tile's rows
struct TileBounds {
  std::vector<int64_t> u0s, u0e, u1s, u1e, i0s, i0e, i1s, i1e;
  int64_t n_tiles = 0;
};

TileBounds tile_bounds(const int32_t* rng, int64_t n, int64_t tile) {
  const int64_t big = std::numeric_limits<int32_t>::max(), small = std::numeric_limits<int32_t>::min();
  TileBounds b;
  b.n_tiles = (n + tile - 1) / tile;
  auto init = [&](std::vector<int64_t>& v, int64_t x) { v.assign(size_t(b.n_tiles), x); };
  init(b.u0s, big); init(b.u0e, small); init(b.u1s, big); init(b.u1e, small);
  init(b.i0s, small); init(b.i0e, big); init(b.i1s, small); init(b.i1e, big);
  for (int64_t r = 0; r < n; ++r) {
    const int64_t t = r / tile;
    const int64_t s0 = rng[4 * r], e0 = std::max<int64_t>(rng[4 * r + 1], s0);
    const int64_t s1 = rng[4 * r + 2], e1 = std::max<int64_t>(rng[4 * r + 3], s1);
    if (e0 > s0) { b.u0s[t] = std::min(b.u0s[t], s0); b.u0e[t] = std::max(b.u0e[t], e0); }
    if (e1 > s1) { b.u1s[t] = std::min(b.u1s[t], s1); b.u1e[t] = std::max(b.u1e[t], e1); }
    b.i0s[t] = std::max(b.i0s[t], s0); b.i0e[t] = std::min(b.i0e[t], e0);
    b.i1s[t] = std::max(b.i1s[t], s1); b.i1e[t] = std::min(b.i1e[t], e1);
  }
  return b;
}

inline bool need(const TileBounds& b, int64_t t, int64_t lo, int64_t hi) {
  return (lo < b.u0e[t] && hi > b.u0s[t]) || (lo < b.u1e[t] && hi > b.u1s[t]);
}
inline bool full(const TileBounds& b, int64_t t, int64_t lo, int64_t hi, int64_t nv) {
  return nv == kTileN && ((b.i0s[t] <= lo && b.i0e[t] >= hi) || (b.i1s[t] <= lo && b.i1e[t] >= hi));
}

double pair_count(const int32_t* rng, int64_t n) {
  int64_t s = 0;
  for (int64_t r = 0; r < n; ++r) {
    s += std::max<int64_t>(int64_t(rng[4 * r + 1]) - rng[4 * r], 0);
    s += std::max<int64_t>(int64_t(rng[4 * r + 3]) - rng[4 * r + 2], 0);
  }
  return double(s);
}

}  // namespace

FwdTablesOut build_fwd_tables(const std::vector<AttnRowDesc>& rows, int64_t block_size, int tile_m) {
  if (tile_m != 128 && tile_m != 256) throw std::invalid_argument("tile_m must be 128 or 256");
  FwdTablesOut out;
  struct Tile { int32_t v[8]; };
  std::vector<Tile> tiles;
  int64_t mask_row = 0, n_entries = 0;
  for (const AttnRowDesc& row : rows) {
    out.masks.insert(out.masks.end(), row.ranges, row.ranges + 4 * row.n_tokens);
    out.pairs += pair_count(row.ranges, row.n_tokens) * double(row.heads.size());
    const int64_t n_sub = (row.n_tokens + tile_m - 1) / tile_m;
    std::vector<std::pair<int64_t, int64_t>> per_tile;  // (offset, count) into the entry list
    if (tile_m == 128) {
      for (auto& kv : row.kv) {
        out.entries.push_back(int32_t(kv.first));
        out.entries.push_back(int32_t(kv.second));
      }
      per_tile.assign(size_t(n_sub), {n_entries, int64_t(row.kv.size())});
      n_entries += int64_t(row.kv.size());
    } else {
      const TileBounds b = tile_bounds(row.ranges, row.n_tokens, kTileM);
      const int64_t n_ct = (b.n_tiles + 1) / 2;
      for (int64_t c = 0; c < n_ct; ++c) {
        const int64_t ta = 2 * c, tb = 2 * c + 1;
        const int64_t start = n_entries;
        for (size_t e = 0; e < row.kv.size(); ++e) {
          const int64_t kv_row = row.kv[e].first, n_tok = row.kv[e].second;
          for (int64_t s = 0; s * kTileN < n_tok; ++s) {
            const int64_t pos = int64_t(e) * block_size + s * kTileN, nv = std::min(kTileN, n_tok - s * kTileN);
            const int64_t lo = pos, hi = pos + nv;
            const bool na = need(b, ta, lo, hi), nb = tb < b.n_tiles && need(b, tb, lo, hi);
            if (!na && !nb) continue;
            const bool fa = na && full(b, ta, lo, hi, nv), fb = nb && full(b, tb, lo, hi, nv);
            out.entries.push_back(int32_t(kv_row + s * kTileN));
            out.entries.push_back(int32_t(pos));
            out.entries.push_back(int32_t(nv));
            out.entries.push_back(int32_t(int(na) | (int(nb) << 1) | (int(fa) << 2) | (int(fb) << 3)));
            ++n_entries;
          }
        }
        per_tile.push_back({start, n_entries - start});
      }
    }
    for (int64_t t = 0; t < n_sub; ++t) {
      const int64_t n_rows = std::min<int64_t>(tile_m, row.n_tokens - t * tile_m);
      for (int h : row.heads) {
        Tile x{{int32_t(row.q_row + t * tile_m), int32_t(n_rows), int32_t(h), int32_t(per_tile[size_t(t)].first),
                int32_t(per_tile[size_t(t)].second), int32_t(mask_row + t * tile_m), int32_t(row.out_dev),
                int32_t(row.out_row + t * tile_m)}};
        tiles.push_back(x);
      }
    }
    mask_row += row.n_tokens;
  }
  // longest tiles first: the grid is scheduled in index order, so this is LPT packing
  std::stable_sort(tiles.begin(), tiles.end(), [](const Tile& a, const Tile& b) { return a.v[4] > b.v[4]; });
  out.tiles.reserve(tiles.size() * 8);
  for (const Tile& t : tiles) out.tiles.insert(out.tiles.end(), t.v, t.v + 8);
  return out;
}

BwdTablesOut build_bwd_tables(const std::vector<AttnRowDesc>& rows, int64_t block_size, int hq) {
  BwdTablesOut out;
  using Key = std::tuple<int64_t, int64_t, int64_t, int64_t>;  // (kv row, valid keys, dkv device, dkv row)
  struct Cta { Key key; std::vector<int32_t> items; };
  std::vector<Cta> ctas;               // in order of first appearance
  std::map<Key, size_t> index;
  int64_t mask_row = 0;
  for (const AttnRowDesc& row : rows) {
    if (int(row.heads.size()) != hq) throw std::invalid_argument("the backward kernel visits every query head of a row");
    out.masks.insert(out.masks.end(), row.ranges, row.ranges + 4 * row.n_tokens);
    out.pairs += pair_count(row.ranges, row.n_tokens) * double(row.heads.size());
    const TileBounds b = tile_bounds(row.ranges, row.n_tokens, kQTileBwd);
    for (size_t e = 0; e < row.kv.size(); ++e) {
      const int64_t kv_row = row.kv[e].first, n_tok = row.kv[e].second;
      const int64_t dkv_dev = row.dkv.empty() ? 0 : row.dkv[e].first, dkv_row = row.dkv.empty() ? kv_row : row.dkv[e].second;
      for (int64_t s = 0; s * kTileN < n_tok; ++s) {
        const int64_t p0 = int64_t(e) * block_size + s * kTileN, nv = std::min(kTileN, n_tok - s * kTileN);
        const int64_t lo = p0, hi = p0 + nv;
        Cta* cta = nullptr;
        for (int64_t qt = 0; qt < b.n_tiles; ++qt) {
          if (!need(b, qt, lo, hi)) continue;
          if (cta == nullptr) {
            const Key key{kv_row + s * kTileN, nv, dkv_dev, dkv_row + s * kTileN};
            auto it = index.find(key);
            if (it == index.end()) {
              it = index.emplace(key, ctas.size()).first;
              ctas.push_back(Cta{key, {}});
            }
            cta = &ctas[it->second];
          }
          const int64_t n_rows = std::min(kQTileBwd, row.n_tokens - qt * kQTileBwd);
          const int32_t item[8] = {int32_t(row.q_row + qt * kQTileBwd), int32_t(n_rows), int32_t(p0),
                                   int32_t(mask_row + qt * kQTileBwd), int32_t(row.dq_dev),
                                   int32_t(row.dq_row + qt * kQTileBwd), int32_t(full(b, qt, lo, hi, nv)), 0};
          cta->items.insert(cta->items.end(), item, item + 8);
        }
      }
    }
    mask_row += row.n_tokens;
  }
  // key tiles with the most items first (LPT packing of the grid)
  std::vector<size_t> order(ctas.size());
  for (size_t i = 0; i < order.size(); ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return ctas[a].items.size() > ctas[b].items.size(); });
  int64_t off = 0;
  for (size_t i : order) {
    const Cta& c = ctas[i];
    const int64_t n = int64_t(c.items.size() / 8);
    const int32_t row[8] = {int32_t(std::get<0>(c.key)), int32_t(std::get<1>(c.key)), int32_t(off), int32_t(n),
                            int32_t(std::get<2>(c.key)), int32_t(std::get<3>(c.key)), 0, 0};
    out.ctas.insert(out.ctas.end(), row, row + 8);
    out.items.insert(out.items.end(), c.items.begin(), c.items.end());
    off += n;
  }
  return out;
}

}  // namespace dcpp
