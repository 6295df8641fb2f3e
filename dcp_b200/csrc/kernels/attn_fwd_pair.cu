// Blockwise range-masked attention forward for sm_100a, two query tiles per CTA.
//
// One CTA = up to 256 queries (two 128-row tiles A and B of one Q block) of one head.  Warps:
//   0-3  softmax of tile A, 4-7 softmax of tile B (one thread per query row),
//   8    TMA producer (Q of both tiles once, 2-deep rings of K and V tiles),
//   9    UMMA issuer,
//   10-11 fetch the next plan stage's remote operands (copy jobs: peer loads over NVLink into this
//        GPU's staging rows, see copy_jobs.cuh) while the tiles are computed; they also donate
//        registers (setmaxnreg).
// K and V tiles are loaded once and used by both query tiles, and the two softmax warpgroups
// alternate on the tensor core: per KV tile j the issuer emits
//   PV(A, j-1), QK(A, j), PV(B, j-1), QK(B, j)
// so one warpgroup's exp2 / TMEM round trips run while the other's UMMAs execute.  A query tile
// that cannot see a KV tile (from the per-tile union of its rows' ranges) skips it: no UMMA is
// issued for it and its softmax warpgroup does not wait.
// TMEM (512 columns): S_A [0,128) S_B [128,256) O_A [256,384) O_B [384,512); P_X overwrites the
// first 64 columns of S_X as packed bf16 pairs and is the TMEM A operand of O_X += P_X V.
// S_X = Q_X K^T takes both operands from shared memory (no TMEM columns are left to park Q in).
//
// The partial (out, lse) of a tile is stored straight to its destination arena, which may be a
// peer GPU's memory (plain st.global over the NVLink mapping).
//
// Reference behaviour covered: the varlen forward with block tables and per-query KV ranges that
// dcp/runtime/flash_attention/executor.py:884-913 calls.
#include <limits.h>
#include <math.h>

#include "attn_common.cuh"
#include "copy_jobs.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace dcpk {

static constexpr int kPairThreads = 384;  // 8 softmax warps + producer + UMMA issuer + 2 idle warps (register donors)
static constexpr int kHalfBytesP = 128 * 64 * 2;
static constexpr int kTileBytesP = 2 * kHalfBytesP;

struct __align__(1024) PairSmem {
  uint8_t q[2][kTileBytesP];
  uint8_t k[2][kTileBytesP];
  uint8_t v[2][kTileBytesP];
  uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_ready[2], o_done[2];
  uint32_t tmem_base;
  int abort_word;
};

// One 128-key tile of the CTA's KV walk, prepared by the host (build_fwd_tables with tile_m = 256).
struct KvSub {
  int row;       // first arena row of the 128 keys
  int pos0;      // position of the first key in the Q block's concatenated KV
  int n_valid;   // valid keys (1..128)
  int flags;     // bit 0 / 1: query tile A / B sees at least one key; bit 2 / 3: A / B sees every pair
};

// walks the list with the next entry already in registers, so a step never waits on global memory
struct SubIter {
  const int4* p;
  int n, i;
  int4 cur, ahead;
  __device__ __forceinline__ void init(const int4* base, int count) {
    p = base; n = count; i = -1;
    ahead = count > 0 ? base[0] : make_int4(0, 0, 0, 0);
  }
  __device__ __forceinline__ bool next() {
    if (++i >= n) return false;
    cur = ahead;
    if (i + 1 < n) ahead = p[i + 1];
    return true;
  }
};

__global__ void __launch_bounds__(kPairThreads, 1)
attn_fwd_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
                     const AttnTile* __restrict__ tiles, const int4* __restrict__ kv_subs,
                     const int4* __restrict__ masks, PeerPtrs ptrs, int hq, int hkv, int lse_stride_a,
                     int lse_stride_b, int n_dst_a, int n_dst, int q_rows, int block_size, int n_mask_rows,
                     int n_kv_subs, float scale, const CopyJob* __restrict__ jobs, int n_jobs,
                     const __grid_constant__ CopyCtx copy_ctx, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  PairSmem& sm = *reinterpret_cast<PairSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const AttnTile tile = tiles[blockIdx.x];
  const int kv_head = tile.head / (hq / hkv);
  {
    // table sanity before anything is allocated: a tile that would store outside its destination
    // arena, or read a head / row / table entry that does not exist, is reported and skipped
    const int dst_rows = tile.out_dev < n_dst_a ? lse_stride_a : lse_stride_b;
    const bool bad = tile.out_dev < 0 || tile.out_dev >= n_dst || tile.out_row < 0 || tile.n_rows < 0 ||
                     tile.n_rows > 2 * kTileM || tile.out_row + tile.n_rows > dst_rows || tile.head < 0 ||
                     tile.head >= hq || tile.q_row < 0 || tile.q_row + tile.n_rows > q_rows || tile.n_kv < 0 ||
                     tile.mask_row < 0 || tile.mask_row + tile.n_rows > n_mask_rows || tile.kv_off < 0 ||
                     tile.kv_off + tile.n_kv > n_kv_subs;
    if (bad) {
      if (threadIdx.x == 0) atomicExch(status, kStatusBadArgs);
      return;
    }
  }
  if (threadIdx.x == 256) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_kv);
    mbar_init(&sm.q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.k_full[i], 1);  mbar_init(&sm.k_empty[i], 1);
      mbar_init(&sm.v_full[i], 1);  mbar_init(&sm.v_empty[i], 1);
      mbar_init(&sm.s_full[i], 1);  mbar_init(&sm.p_ready[i], 128);
      mbar_init(&sm.o_done[i], 1);
    }
    sm.abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  // this thread's query row (softmax warps): X = which tile, r = row inside it
  const int X = warp >> 2, r = threadIdx.x & 127;
  int s0 = 0, e0 = 0, s1 = 0, e1 = 0;
  if (warp < 8) {
    const bool valid = X * kTileM + r < tile.n_rows;
    if (valid) {
      int4 m = masks[tile.mask_row + X * kTileM + r];
      s0 = m.x; e0 = max(m.y, m.x); s1 = m.z; e1 = max(m.w, m.z);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  volatile int* abort_word = &sm.abort_word;
  SubIter it;
  it.init(kv_subs + tile.kv_off, tile.n_kv);

  // register rebalancing between warpgroups (setmaxnreg inside each role's branch): the four
  // non-softmax warps give registers up, the softmax warps take them
  // (8 x 32 x 208 + 4 x 32 x 72 = 62464 of 65536)
  if (warp >= 8) {
   asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
   if (warp == 8) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(&sm.q_full, 2 * kTileBytesP);
      for (int x = 0; x < 2; ++x) {
        tma_load_3d(sm.q[x], &tm_q, &sm.q_full, 0, tile.head, tile.q_row + x * kTileM);
        tma_load_3d(sm.q[x] + kHalfBytesP, &tm_q, &sm.q_full, 64, tile.head, tile.q_row + x * kTileM);
      }
      int j = 0;
      bool ok = true;
      int k_pending[2] = {-1, -1}, v_pending[2] = {-1, -1};
      while (ok && it.next()) {
        const int st = j & 1, u = j >> 1;
        ok = mbar_wait(&sm.k_empty[st], (u & 1) ^ 1, abort_word);
        if (!ok) break;
        mbar_expect_tx(&sm.k_full[st], kTileBytesP);
        tma_load_3d(sm.k[st], &tm_kv, &sm.k_full[st], 0, kv_head, it.cur.x);
        tma_load_3d(sm.k[st] + kHalfBytesP, &tm_kv, &sm.k_full[st], 64, kv_head, it.cur.x);
        k_pending[st] = u & 1;
        ok = mbar_wait(&sm.v_empty[st], (u & 1) ^ 1, abort_word);
        if (!ok) break;
        mbar_expect_tx(&sm.v_full[st], kTileBytesP);
        tma_load_3d(sm.v[st], &tm_kv, &sm.v_full[st], 0, hkv + kv_head, it.cur.x);
        tma_load_3d(sm.v[st] + kHalfBytesP, &tm_kv, &sm.v_full[st], 64, hkv + kv_head, it.cur.x);
        v_pending[st] = u & 1;
        ++j;
      }
      if (!ok) {
        // give copies already in flight a bounded chance to land before the CTA retires
        for (int st = 0; st < 2; ++st) {
          if (k_pending[st] >= 0)
            for (int spin = 0; spin < 200000 && !mbar_try_wait(&sm.k_full[st], k_pending[st]); ++spin) {}
          if (v_pending[st] >= 0)
            for (int spin = 0; spin < 200000 && !mbar_try_wait(&sm.v_full[st], v_pending[st]); ++spin) {}
        }
      }
    }
   } else if (warp == 9) {
    // ------------------------------------------------------------ UMMA issuer
    constexpr uint32_t idesc_qk = make_idesc_bf16(128, 128, 0, 0);
    constexpr uint32_t idesc_pv = make_idesc_bf16(128, 128, 0, 1);
    bool ok = mbar_wait(&sm.q_full, 0, abort_word);
    int j = 0;
    int cnt[2] = {0, 0};                 // KV tiles issued so far per query tile
    bool need_prev[2] = {false, false};  // did query tile X take part in the previous KV tile
    // O_X += P_X V: P from TMEM (TS), V of ring stage `st` is the MN-major B operand; `i` = index
    // of this KV tile among the ones query tile X takes part in, `jv` = its index in the ring
    auto issue_pv = [&](int x, int i, int jv) -> bool {
      const int st = jv & 1;
      if (!mbar_wait(&sm.p_ready[x], i & 1, abort_word)) return false;
      if (!mbar_wait(&sm.v_full[st], (jv >> 1) & 1, abort_word)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t v_addr = smem_u32(sm.v[st]);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          uint64_t bdesc = make_sdesc_sw128(v_addr + k * 2048, kHalfBytesP, 1024);
          umma_ts(tmem + 256 + x * 128, tmem + x * 128 + k * 8, bdesc, idesc_pv, (i > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&sm.o_done[x]);
      }
      __syncwarp();
      return true;
    };
    // S_X = Q_X K^T, both operands from shared memory
    auto issue_qk = [&](int x, int st) {
      if (lane == 0) {
        const uint32_t q_addr = smem_u32(sm.q[x]), k_addr = smem_u32(sm.k[st]);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          uint64_t adesc = make_sdesc_sw128(q_addr + (k >> 2) * kHalfBytesP + (k & 3) * 32, 16, 1024);
          uint64_t bdesc = make_sdesc_sw128(k_addr + (k >> 2) * kHalfBytesP + (k & 3) * 32, 16, 1024);
          umma_ss(tmem + x * 128, adesc, bdesc, idesc_qk, k > 0 ? 1u : 0u);
        }
        umma_commit(&sm.s_full[x]);
      }
      __syncwarp();
    };
    while (ok && it.next()) {
      const int st = j & 1, u = j >> 1;
      ok = mbar_wait(&sm.k_full[st], u & 1, abort_word);
      if (!ok) break;
      tc_fence_after();
      bool need_cur[2];
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        need_cur[x] = (it.cur.w >> x) & 1;
        // S_X may only be overwritten after P_X of the previous tile was consumed: its PV goes first
        if (need_prev[x]) { ok = issue_pv(x, cnt[x] - 1, j - 1); if (!ok) break; }
        if (need_cur[x]) { issue_qk(x, st); ++cnt[x]; }
      }
      if (!ok) break;
      if (lane == 0) {
        umma_commit(&sm.k_empty[st]);                   // both query tiles are through with K(j)
        if (j > 0) umma_commit(&sm.v_empty[st ^ 1]);    // ... and with V(j-1)
      }
      __syncwarp();
      need_prev[0] = need_cur[0]; need_prev[1] = need_cur[1];
      ++j;
    }
#pragma unroll
    for (int x = 0; x < 2; ++x)
      if (ok && need_prev[x]) ok = issue_pv(x, cnt[x] - 1, j - 1);
    // keep TMEM alive until the last accumulate retired (the epilogues also wait on it)
#pragma unroll
    for (int x = 0; x < 2; ++x)
      if (ok && cnt[x] > 0) ok = mbar_wait(&sm.o_done[x], (cnt[x] - 1) & 1, abort_word);
   } else {
    // ------------------------------------------------------------ operand fetch for the next stage
    run_copy_jobs(jobs, n_jobs, copy_ctx, blockIdx.x, gridDim.x, threadIdx.x - 320, 64);
   }
  } else {
    // ------------------------------------------------------------ softmax + epilogue of tile X
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    const uint32_t s_addr = tmem + lane_base + X * 128, o_addr = tmem + lane_base + 256 + X * 128;
    const float sl2 = scale * 1.4426950408889634f;
    const float rescale_gap = 8.0f / sl2;   // 8 in the base-2 exponent, expressed in raw score units
    const int len0 = e0 - s0, len1 = e1 - s1;
    float m_run = -INFINITY, l_run = 0.f;
    int j = 0;   // KV tiles this query tile took part in
    bool ok = true;
    while (ok && it.next()) {
      if (!((it.cur.w >> X) & 1)) continue;
      ok = mbar_wait(&sm.s_full[X], j & 1, abort_word);
      if (!ok) break;
      tc_fence_after();
      uint32_t sreg[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + c * 32, sreg + c * 32);
      tmem_wait_ld();
      // Row maximum and row sum are reduced through 8 independent partial chains: a single running
      // value would be a 128-long dependent chain with nothing to hide its latency behind.
      float mxp[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mxp[i] = -INFINITY;
      if ((it.cur.w >> (2 + X)) & 1) {
#pragma unroll
        for (int c = 0; c < 64; ++c)
          mxp[c & 7] = fmax3(mxp[c & 7], __uint_as_float(sreg[2 * c]), __uint_as_float(sreg[2 * c + 1]));
      } else {
        const int rel0 = it.cur.y - s0, rel1 = it.cur.y - s1, n_valid = it.cur.z;
#pragma unroll
        for (int c = 0; c < 128; ++c) {
          bool allow = (unsigned(rel0 + c) < unsigned(len0)) || (unsigned(rel1 + c) < unsigned(len1));
          allow = allow && (c < n_valid);
          float sv = allow ? __uint_as_float(sreg[c]) : -INFINITY;
          sreg[c] = __float_as_uint(sv);
          mxp[c & 7] = fmaxf(mxp[c & 7], sv);
        }
      }
      const float mx = fmaxf(fmaxf(fmaxf(mxp[0], mxp[1]), fmaxf(mxp[2], mxp[3])),
                             fmaxf(fmaxf(mxp[4], mxp[5]), fmaxf(mxp[6], mxp[7])));
      // The running maximum only moves when the tile's maximum exceeds it by more than 2^8 in the
      // exponent (or on the first tile): probabilities may then reach 256 instead of 1, which fp32 /
      // bf16 hold without loss, and O has to be rescaled in TMEM only a few times per row instead of
      // in most tiles.  out = O / l and lse = m + ln l are exact for any reference value m.
      const float m_new = (mx > m_run + rescale_gap) ? mx : m_run;
      const float m_sub = (m_new == -INFINITY) ? 0.f : m_new * sl2;
      const float alpha = (m_new == -INFINITY) ? 1.f : fast_exp2(m_run * sl2 - m_sub);
      // packed fp32: one instruction scales two scores, one adds two probabilities to the row sum
      // every probability carries the factor kTruncScale (folded into the exponent), so cutting it to
      // bf16 is unbiased; the row sum carries the same factor, which cancels in O / l and is taken
      // out of the LSE in the epilogue
      const uint64_t sl2_2 = pack_f32x2(sl2, sl2), negm_2 = pack_f32x2(kTruncLog2 - m_sub, kTruncLog2 - m_sub);
      uint64_t ps2[4] = {0ull, 0ull, 0ull, 0ull};
      // P goes back in two 32-column stores so fewer registers stay live
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t preg[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int cc = 32 * h + c;
          const uint64_t x2 = fma_f32x2(pack_f32x2(__uint_as_float(sreg[2 * cc]), __uint_as_float(sreg[2 * cc + 1])), sl2_2, negm_2);
          float x0, x1;
          unpack_f32x2(x2, x0, x1);
          const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
          ps2[c & 3] = add_f32x2(ps2[c & 3], pack_f32x2(p0, p1));
          preg[c] = pack_bf16x2_trunc(p0, p1);
        }
        tmem_st32(s_addr + 32 * h, preg);
      }
      float psp[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) unpack_f32x2(ps2[i], psp[2 * i], psp[2 * i + 1]);
      const float psum = ((psp[0] + psp[1]) + (psp[2] + psp[3])) + ((psp[4] + psp[5]) + (psp[6] + psp[7]));
      l_run = l_run * alpha + psum;
      m_run = m_new;
      if (j > 0) {
        // O_X may only be rescaled once the previous accumulate into it retired
        ok = mbar_wait(&sm.o_done[X], (j - 1) & 1, abort_word);
        if (!ok) break;
        tc_fence_after();
      }
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t oreg[32];
          tmem_ld32(o_addr + c * 32, oreg);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
          tmem_st32(o_addr + c * 32, oreg);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&sm.p_ready[X]);
      ++j;
    }
    if (ok && j > 0) {
      ok = mbar_wait(&sm.o_done[X], (j - 1) & 1, abort_word);
      tc_fence_after();
    }
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      const int row = X * kTileM + r;
      const bool store = row < tile.n_rows;
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(ptrs.out[tile.out_dev]) +
                           (size_t(tile.out_row + row) * hq + tile.head) * kHeadDim;
      if (store)
        ptrs.lse[tile.out_dev][size_t(tile.head) * (tile.out_dev < n_dst_a ? lse_stride_a : lse_stride_b) + tile.out_row + row] =
            l_run > 0.f ? m_run * scale + logf(l_run) - kTruncLn : -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t oreg[32];
        if (j > 0) {  // warp-uniform: the TMEM load is a warp-collective instruction
          tmem_ld32(o_addr + c * 32, oreg);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) oreg[i] = 0;
        }
        if (store) {
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            packed[i] = pack_bf16x2(__uint_as_float(oreg[2 * i]) * inv_l, __uint_as_float(oreg[2 * i + 1]) * inv_l);
          uint4* dst = reinterpret_cast<uint4*>(out + c * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            dst[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  if (threadIdx.x == 0 && sm.abort_word) atomicExch(status, kStatusBarrierTimeout);
}

static int g_pair_attr_set = 0;

}  // namespace dcpk

void dcpk_fill_copy_ctx(dcpk::CopyCtx* ctx, void* const* src_ptrs, void* const* dst_ptrs, int stat_stride);

using namespace dcpk;

// Same contract as dcpk_attn_fwd, for tile tables built with 256-row tiles (AttnTile.n_rows <= 256):
// `kv_entries` is the KvSub list (AttnTile.kv_off / n_kv index it), n_mask_rows / n_kv_entries are the
// lengths of the mask table and of that list (bounds checks).
extern "C" int dcpk_attn_fwd_pair(const void* q_arena, long q_rows, const void* kv_arena, long kv_rows, int hq,
                                  int hkv, const void* tiles, int n_tiles, const void* kv_entries, int n_kv_entries,
                                  const void* masks, int n_mask_rows, void* const* out_ptrs, float* const* lse_ptrs,
                                  int n_dst, int lse_stride_a, int lse_stride_b, int n_dst_a, int block_size,
                                  float scale, const void* jobs, int n_jobs, void* const* job_src_ptrs,
                                  void* const* job_dst_ptrs, int job_stat_stride, int* status, void* stream) {
  if (n_tiles <= 0) return n_jobs > 0 ? -6 : 0;   // copy jobs need a kernel to ride on
  if (n_dst > kMaxPeers || hq % hkv != 0) return -3;
  CUtensorMap tm_q, tm_kv;
  if (encode_arena_map(&tm_q, q_arena, uint64_t(q_rows), uint32_t(hq), kHeadDim, 128)) return -1;
  if (encode_arena_map(&tm_kv, kv_arena, uint64_t(kv_rows), uint32_t(2 * hkv), kHeadDim, 128)) return -1;
  PeerPtrs pp;
  for (int i = 0; i < kMaxPeers; ++i) {
    pp.out[i] = i < n_dst ? out_ptrs[i] : nullptr;
    pp.lse[i] = i < n_dst ? lse_ptrs[i] : nullptr;
  }
  CopyCtx ctx;
  dcpk_fill_copy_ctx(&ctx, n_jobs > 0 ? job_src_ptrs : nullptr, n_jobs > 0 ? job_dst_ptrs : nullptr, job_stat_stride);
  const int smem = int(sizeof(PairSmem)) + 1024;
  if (!g_pair_attr_set) {
    if (cudaFuncSetAttribute(attn_fwd_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return -4;
    g_pair_attr_set = 1;
  }
  attn_fwd_pair_kernel<<<n_tiles, kPairThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      tm_q, tm_kv, static_cast<const AttnTile*>(tiles), static_cast<const int4*>(kv_entries),
      static_cast<const int4*>(masks), pp, hq, hkv, lse_stride_a, lse_stride_b, n_dst_a, n_dst, int(q_rows),
      block_size, n_mask_rows, n_kv_entries, scale, static_cast<const CopyJob*>(jobs), n_jobs, ctx, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
