// Shared definitions of the blockwise attention kernels (forward and backward).
//
// Work model.  A plan stage hands a device a list of "q rows": one Q block (up to
// `block_size` tokens of one head block) together with the ordered list of KV blocks
// it attends to in this stage.  KV positions are numbered in the concatenation of
// those KV blocks, each block occupying `block_size` positions whether or not it is
// full (same convention as the plan's AttnInstr: seqlen_kv = block_size * len(row)).
// Every query token carries up to two half-open position ranges [s0,e0) U [s1,e1);
// a (query, key) pair is computed iff the key position lies in one of them.
//
// The host flattens the q rows into 128-token tiles (`AttnTile`).  All operands live
// in row-addressed arenas ([rows, heads, head_dim] bf16) that hold this rank's own
// tokens first and the staging slots for blocks pulled from peers after them, so
// one TMA tensor map per arena reaches everything the kernel reads.
#pragma once
#include <stdint.h>

namespace dcpk {

static constexpr int kTileM = 128;   // query rows per CTA tile
static constexpr int kTileN = 128;   // key rows per inner tile
static constexpr int kHeadDim = 128; // compiled head dimension
static constexpr int kMaxPeers = 16;

struct AttnTile {
  int q_row;        // first arena row of this tile's queries
  int n_rows;       // valid query rows (1..128)
  int head;         // query head index inside the arena
  int kv_off;       // first entry of this tile's KV-block list in `kv_entries`
  int n_kv;         // number of KV blocks
  int mask_row;     // first row of this tile in the range-mask table
  int out_dev;      // index into the output pointer table (0 = this rank)
  int out_row;      // first arena row of the output
};

struct KvEntry {
  int row;          // first arena row of the KV block
  int n_tok;        // valid tokens in the block (<= block_size)
};

struct PeerPtrs {
  void* out[kMaxPeers];   // bf16 [rows, hq, d] per destination
  float* lse[kMaxPeers];  // fp32 [hq, rows] per destination
};

// Union / intersection of the per-row ranges of one 128-row tile; lets every warp role
// enumerate the same list of needed KV tiles without touching the mask table again.
struct TileBounds {
  int u0s, u0e, u1s, u1e;  // union of range 0 / range 1 over valid rows
  int i0s, i0e, i1s, i1e;  // intersection (max start, min end) over valid rows
};

struct KvTileIter {
  // iterates (entry, sub-tile) pairs, skipping sub-tiles no row of the Q tile can see
  const KvEntry* entries;
  int n_kv, block_size;
  TileBounds b;
  int e, t;          // cursor
  int row, pos0, n_valid;  // current tile
  bool full;         // current tile needs no per-element masking

  KvEntry cur, ahead;  // entry under the cursor and the one after it, held in registers

  __device__ __forceinline__ void init(const KvEntry* ents, int n, int bs, const TileBounds& tb) {
    entries = ents; n_kv = n; block_size = bs; b = tb; e = 0; t = -1;
    cur = KvEntry{0, 0};
    if (n > 0) cur = ents[0];
    ahead = cur;
    if (n > 1) ahead = ents[1];
  }
  // The table entry is read one block ahead of its use, so a call never waits on global memory.
  __device__ __forceinline__ bool next() {
    while (e < n_kv) {
      const int n_sub = (cur.n_tok + kTileN - 1) / kTileN;
      ++t;
      if (t >= n_sub) {
        ++e; t = -1;
        cur = ahead;
        if (e + 1 < n_kv) ahead = entries[e + 1];
        continue;
      }
      const int p0 = e * block_size + t * kTileN;
      const int nv = min(kTileN, cur.n_tok - t * kTileN);
      const bool need = (p0 < b.u0e && p0 + nv > b.u0s) || (p0 < b.u1e && p0 + nv > b.u1s);
      if (!need) continue;
      row = cur.row + t * kTileN; pos0 = p0; n_valid = nv;
      full = (nv == kTileN) && ((b.i0s <= p0 && b.i0e >= p0 + nv) || (b.i1s <= p0 && b.i1e >= p0 + nv));
      return true;
    }
    return false;
  }
  // the same two tests for another set of bounds (a sub-tile of the rows `b` covers) on the current tile
  __device__ __forceinline__ bool needed_by(const TileBounds& tb) const {
    return (pos0 < tb.u0e && pos0 + n_valid > tb.u0s) || (pos0 < tb.u1e && pos0 + n_valid > tb.u1s);
  }
  __device__ __forceinline__ bool full_for(const TileBounds& tb) const {
    return (n_valid == kTileN) && ((tb.i0s <= pos0 && tb.i0e >= pos0 + n_valid) || (tb.i1s <= pos0 && tb.i1e >= pos0 + n_valid));
  }
};

}  // namespace dcpk
