// Blockwise range-masked attention backward for sm_100a.
//
// One CTA owns one 128-row KV tile of one KV head and walks a host-built list of 64-query
// tiles that attend to it, once per query head of the GQA group.  Everything is computed in
// the transposed orientation (lane = key row):
//   S^T  = K  Q^T          (SS UMMA, M=128 keys, N=64 queries, K=d)        -> TMEM
//   dP^T = V  dO^T         (SS)                                             -> TMEM
//   P^T  = exp2(S^T*c - lse),  dS^T = P^T o (dP^T - delta) * scale          (8 gradient warps)
//   P^T and dS^T are written as bf16 into two swizzled smem tiles, then
//   dV  += P^T  dO         (SS, A = P^T tile K-major, B = dO MN-major, accumulates in TMEM)
//   dK  += dS^T Q          (SS)
//   dQ^T = K^T dS^T        (SS, A = K MN-major, B = the same dS^T bytes MN-major)
// The Q/dO stage is handed back to the TMA producer after dV and dK are issued, so the load of
// the next-but-one item overlaps dQ^T.  dQ^T alternates between two TMEM buffers; while the
// tensor core works on item t the gradient warps transpose dQ^T(t-1) through a per-warp
// [32 q x 32 d] fp32 staging tile and add it to the accumulator with one tiled TMA reduce-add
// (local accumulator) or one 128-byte bulk reduce per query row (peer accumulator).  dK/dV stay
// in TMEM for the CTA's lifetime and are added once with red.global.add.v4.f32.
// TMEM columns: S^T [0,64) dP^T [64,128) dQ^T [128,192) [192,256) dK [256,384) dV [384,512).
// Warps: 0-15 gradient (warp = 32 key rows x 16 query columns), 16 TMA producer, 17 UMMA issuer.
// The first `n_copy_rows` rows of the grid are fetch CTAs: they compute nothing and bring the next plan
// stage's remote operands (Q, dO, KV rows and the lse / delta statistics of the queries) from peer
// GPUs into this GPU's staging rows (copy_jobs.cuh) while the other CTAs of the same launch work
// through the items; they are scheduled first and retire after about a millisecond.
//
// Reference behaviour covered: the varlen backward the executor calls at
// dcp/runtime/flash_attention/executor.py:1058-1115, plus the blockwise partial sums
// that follow it (dcp/ops/fused_ops.py:1087-1360), which the atomics make unnecessary.
#include <limits.h>
#include <math.h>

#include "attn_common.cuh"
#include "copy_jobs.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace dcpk {

static constexpr int kBwdThreads = 576;  // 16 gradient warps + TMA producer + UMMA issuer
static constexpr int kQTile = 64;
static constexpr int kStages = 3;  // depth of the Q / dO / statistics ring
static constexpr int kKvHalf = 128 * 64 * 2;  // [128 x 64] bf16 half tile, 16 KB
static constexpr int kQHalf = 64 * 64 * 2;    // [64 x 64] bf16 half tile, 8 KB

// One item = one 64-query tile that attends to the CTA's key tile; the CTA visits it once per
// query head of its KV head's group, so the table does not grow with the head count.
struct BwdItemDesc {
  int q_row;     // arena row of the 64-query tile (same row addresses Q, dO, lse, delta)
  int n_rows;    // valid queries
  int kv_pos0;   // position of this CTA's first key inside the item's concatenated KV
  int mask_row;  // row in the range table
  int dq_dev;    // destination index of the dQ accumulator
  int dq_row;    // arena row in that accumulator
  int full;      // 1: every (query, key) pair of the tile is allowed
  int pad;
};

struct BwdItem {  // descriptor + the query head of the current visit
  int q_row, n_rows, head, kv_pos0, mask_row, dq_dev, dq_row, full;
};

struct BwdCta {
  int kv_row;    // arena row of the 128-key tile
  int n_valid;   // valid keys
  int item_off, n_items;
  int dkv_dev, dkv_row;
  int pad0, pad1;
};

__device__ __forceinline__ BwdItem load_item(const BwdItemDesc* descs, int visit, int group, int kv_head) {
  const BwdItemDesc d = descs[visit / group];
  BwdItem it;
  it.q_row = d.q_row; it.n_rows = d.n_rows; it.head = kv_head * group + visit % group; it.kv_pos0 = d.kv_pos0;
  it.mask_row = d.mask_row; it.dq_dev = d.dq_dev; it.dq_row = d.dq_row; it.full = d.full;
  return it;
}

struct BwdPtrs {
  float* dq[kMaxPeers];   // fp32 [rows, hq, d]
  float* dkv[kMaxPeers];  // fp32 [rows, 2, hkv, d]
};

struct __align__(1024) BwdSmem {
  uint8_t k[2 * kKvHalf];
  uint8_t v[2 * kKvHalf];
  uint8_t q[kStages][2 * kQHalf];
  uint8_t dout[kStages][2 * kQHalf];
  uint8_t ds[kKvHalf];     // dS^T: [128 keys x 64 queries]
  uint8_t p[kKvHalf];      // P^T:  [128 keys x 64 queries]
  // dQ staging, one private [16 queries x 32 channels] fp32 tile per gradient warp; drained to the
  // fp32 accumulator with bulk reduce-add copies (L2 handles those a line at a time, scalar
  // red.add is limited to one element per L2 slice per clock)
  float dq_stage[16][8 * 32];
  // per-stage item descriptor and per-query statistics, staged by the producer warp next to Q / dO
  // so the gradient warps never touch global memory on their critical path
  BwdItem item[kStages];
  // statistics are staged in the form the packed-fp32 math consumes them (pairs of queries per
  // 64-bit load): -lse * log2(e) (-inf for rows past the tile) and -delta * scale
  alignas(8) float lse2[kStages][kQTile];
  alignas(8) float delta[kStages][kQTile];
  int4 rng[kStages][kQTile];     // normalised ranges (end >= start)
  uint64_t kv_full, qdo_full[kStages], qdo_empty[kStages], stats_full[kStages], sdp_full, s_free, p_ready, dq_full;
  uint32_t tmem_base;
  int abort_word;
};

// Optional per-phase cycle counters of CTA (0,0) (set with dcpk_attn_bwd_set_timeline; null = off).
// Layout: [phase][sum of cycles]; phases 0-7 gradient warp 0, 8-11 UMMA warp.  The counters live in
// a separately instantiated kernel (kTL) so the production kernel carries no probe branches; each
// phase includes the cost of one probe (about 110 cycles).
__device__ long long* g_bwd_timeline = nullptr;
#define TL_ADD(idx, t_prev)                                                        \
  do {                                                                             \
    if constexpr (kTL) if (tl) { long long now_ = clock64(); if (lane == 0) atomicAdd(reinterpret_cast<unsigned long long*>(tl + (idx)), (unsigned long long)(now_ - (t_prev))); (t_prev) = now_; } \
  } while (0)

__device__ __forceinline__ void red_add_f32(float* p, float v) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

template <bool kTL>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_dq,
                const BwdCta* __restrict__ ctas, const BwdItemDesc* __restrict__ items, const int4* __restrict__ masks,
                const float* __restrict__ lse, const float* __restrict__ delta, BwdPtrs ptrs, int hq, int hkv,
                int stat_stride, int n_dst, int q_rows, int kv_rows, int n_mask_rows, int n_items_total, float scale,
                const CopyJob* __restrict__ jobs, int n_jobs, const __grid_constant__ CopyCtx copy_ctx,
                int n_copy_rows, int* __restrict__ status) {
  if (int(blockIdx.y) < n_copy_rows) {
    // ------------------------------------------------------------ operand fetch for the next stage
    run_copy_jobs(jobs, n_jobs, copy_ctx, blockIdx.y * gridDim.x + blockIdx.x, n_copy_rows * gridDim.x, threadIdx.x,
                  kBwdThreads);
    return;
  }
  extern __shared__ uint8_t smem_raw[];
  BwdSmem& sm = *reinterpret_cast<BwdSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid = (kv heads, key tiles): neighbouring CTAs share the item list and the mask rows
  const BwdCta cta = ctas[blockIdx.y - n_copy_rows];
  const int kv_head = blockIdx.x;
  const int group = hq / hkv;
  const BwdItemDesc* my_items = items + cta.item_off;
  const int n_items = cta.n_items * group;  // visits
  {
    // table sanity before anything is allocated: a key tile whose gradient rows would fall outside
    // the accumulator, or whose item list runs past the item table, is reported and skipped (items
    // are checked one by one by the producer warp, mask rows included)
    const bool bad = cta.dkv_dev < 0 || cta.dkv_dev >= n_dst || cta.dkv_row < 0 || cta.n_valid < 0 ||
                     cta.n_valid > 128 || cta.dkv_row + cta.n_valid > kv_rows || cta.kv_row < 0 ||
                     cta.kv_row + cta.n_valid > kv_rows || cta.n_items < 0 || cta.item_off < 0 ||
                     cta.item_off + cta.n_items > n_items_total;
    if (bad) {
      if (threadIdx.x == 0) atomicExch(status, kStatusBadArgs);
      return;
    }
  }

  if (threadIdx.x == 512) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_do);
    tma_prefetch_desc(&tm_kv);
    tma_prefetch_desc(&tm_dq);
    mbar_init(&sm.kv_full, 1);
    for (int i = 0; i < kStages; ++i) { mbar_init(&sm.qdo_full[i], 1); mbar_init(&sm.qdo_empty[i], 1); mbar_init(&sm.stats_full[i], 1); }
    mbar_init(&sm.sdp_full, 1);
    mbar_init(&sm.s_free, 512);
    mbar_init(&sm.p_ready, 512);
    mbar_init(&sm.dq_full, 1);
    sm.abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 17) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  volatile int* abort_word = &sm.abort_word;
  constexpr uint32_t cS = 0, cdP = 64, cdQ = 128 /* two 64-column buffers */, cdK = 256, cdV = 384;

  long long* tl = (kTL && blockIdx.x == 0 && int(blockIdx.y) == n_copy_rows && (warp == 0 || warp == 17)) ? g_bwd_timeline : nullptr;
  long long tl_t = kTL ? clock64() : 0;
  if (warp == 16) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(&sm.kv_full, 4 * kKvHalf);
      tma_load_3d(sm.k, &tm_kv, &sm.kv_full, 0, kv_head, cta.kv_row);
      tma_load_3d(sm.k + kKvHalf, &tm_kv, &sm.kv_full, 64, kv_head, cta.kv_row);
      tma_load_3d(sm.v, &tm_kv, &sm.kv_full, 0, hkv + kv_head, cta.kv_row);
      tma_load_3d(sm.v + kKvHalf, &tm_kv, &sm.kv_full, 64, hkv + kv_head, cta.kv_row);
    }
    bool ok = true;
    int pending[kStages];
#pragma unroll
    for (int i = 0; i < kStages; ++i) pending[i] = -1;
    int st = 0, u = 0;  // ring slot and its use count
    for (int i = 0; i < n_items && ok; ++i, st = (st + 1 == kStages ? 0 : st + 1), u += (st == 0)) {
      const BwdItem itx = load_item(my_items, i, group, kv_head);
      if (itx.n_rows < 0 || itx.n_rows > kQTile || itx.q_row < 0 || itx.q_row + itx.n_rows > q_rows ||
          itx.q_row + itx.n_rows > stat_stride || itx.dq_dev >= n_dst || itx.mask_row < 0 ||
          (!itx.full && itx.mask_row + itx.n_rows > n_mask_rows) ||
          (itx.dq_dev >= 0 && (itx.dq_row < 0 || itx.dq_row + itx.n_rows > q_rows))) {
        sm.abort_word = kStatusBadArgs;  // every waiter unwinds; the code is reported as the status
        ok = false;
        break;
      }
      // the statistics are fetched before the stage is waited for: their latency hides behind the wait
      float l[2], d[2];
      int4 m[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int qi = lane + 32 * h;
        const bool qv = qi < itx.n_rows;
        const size_t si = size_t(itx.head) * stat_stride + itx.q_row + qi;
        l[h] = qv ? lse[si] : INFINITY;
        d[h] = qv ? delta[si] : 0.f;
        m[h] = make_int4(0, 0, 0, 0);
        if (qv && !itx.full) m[h] = masks[itx.mask_row + qi];
      }
      if (lane == 0 && i + kStages < n_items) {
        // the ring holds kStages items; the one after them is pulled into L2 now, so that its TMA load
        // (issued when a slot frees up) finds it there
        const BwdItem nx = load_item(my_items, i + kStages, group, kv_head);
        if (nx.q_row >= 0 && nx.q_row < q_rows && nx.head < hq) {
          tma_prefetch_l2_3d(&tm_q, 0, nx.head, nx.q_row);
          tma_prefetch_l2_3d(&tm_q, 64, nx.head, nx.q_row);
          tma_prefetch_l2_3d(&tm_do, 0, nx.head, nx.q_row);
          tma_prefetch_l2_3d(&tm_do, 64, nx.head, nx.q_row);
        }
      }
      ok = mbar_wait(&sm.qdo_empty[st], (u & 1) ^ 1, abort_word);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(&sm.qdo_full[st], 4 * kQHalf);
        tma_load_3d(sm.q[st], &tm_q, &sm.qdo_full[st], 0, itx.head, itx.q_row);
        tma_load_3d(sm.q[st] + kQHalf, &tm_q, &sm.qdo_full[st], 64, itx.head, itx.q_row);
        tma_load_3d(sm.dout[st], &tm_do, &sm.qdo_full[st], 0, itx.head, itx.q_row);
        tma_load_3d(sm.dout[st] + kQHalf, &tm_do, &sm.qdo_full[st], 64, itx.head, itx.q_row);
        pending[st] = u & 1;
        sm.item[st] = itx;
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int qi = lane + 32 * h;
        sm.lse2[st][qi] = (l[h] == -INFINITY) ? -INFINITY : -(l[h] * 1.4426950408889634f);
        sm.delta[st][qi] = -d[h] * scale;
        int4 mm = m[h];
        mm.y = max(mm.y, mm.x); mm.w = max(mm.w, mm.z);
        sm.rng[st][qi] = mm;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.stats_full[st]);  // release: the stores above are visible to waiters
    }
    if (!ok && lane == 0) {
#pragma unroll
      for (int s2 = 0; s2 < kStages; ++s2)
        if (pending[s2] >= 0)
          for (int spin = 0; spin < 200000 && !mbar_try_wait(&sm.qdo_full[s2], pending[s2]); ++spin) {}
    }
  } else if (warp == 17) {
    // ------------------------------------------------------------ UMMA issuer
    constexpr uint32_t idesc_sdp = make_idesc_bf16(128, 64, 0, 0);
    constexpr uint32_t idesc_acc = make_idesc_bf16(128, 128, 0, 1);
    constexpr uint32_t idesc_dq = make_idesc_bf16(128, 64, 1, 1);
    const uint32_t k_addr = smem_u32(sm.k), v_addr = smem_u32(sm.v), ds_addr = smem_u32(sm.ds), p_addr = smem_u32(sm.p);
    bool ok = mbar_wait(&sm.kv_full, 0, abort_word);
    auto issue_acc = [&](int t) -> bool {
      const int st = t % kStages;
      TL_ADD(8, tl_t);
      if (!mbar_wait(&sm.p_ready, t & 1, abort_word)) return false;
      TL_ADD(9, tl_t);
      tc_fence_after();
      if (lane == 0) {
        const uint32_t q_addr = smem_u32(sm.q[st]), do_addr = smem_u32(sm.dout[st]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {  // 16 queries per step; A = P^T tile, K-major (queries contiguous)
          uint64_t a_p = make_sdesc_sw128(p_addr + k * 32, 16, 1024);
          uint64_t b_do = make_sdesc_sw128(do_addr + k * 2048, kQHalf, 1024);
          umma_ss(tmem + cdV, a_p, b_do, idesc_acc, (t > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          uint64_t a_ds = make_sdesc_sw128(ds_addr + k * 32, 16, 1024);
          uint64_t b_q = make_sdesc_sw128(q_addr + k * 2048, kQHalf, 1024);
          umma_ss(tmem + cdK, a_ds, b_q, idesc_acc, (t > 0 || k > 0) ? 1u : 0u);
        }
        // Q and dO are not read after this point: hand the stage back to the producer now, so the
        // next-but-one item loads while dQ^T is still being computed
        umma_commit(&sm.qdo_empty[st]);
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // 16 keys per step; same dS^T bytes read as the MN-major B operand
          uint64_t a_kt = make_sdesc_sw128(k_addr + k * 2048, kKvHalf, 1024);
          uint64_t b_ds = make_sdesc_sw128(ds_addr + k * 2048, 16, 1024);
          umma_ss(tmem + cdQ + (t & 1) * 64, a_kt, b_ds, idesc_dq, k > 0 ? 1u : 0u);
        }
        umma_commit(&sm.dq_full);
      }
      __syncwarp();
      TL_ADD(10, tl_t);
      return true;
    };
    for (int i = 0; i < n_items && ok; ++i) {
      const int st = i % kStages, u = i / kStages;
      ok = mbar_wait(&sm.qdo_full[st], u & 1, abort_word);
      if (ok && i > 0) ok = mbar_wait(&sm.s_free, (i - 1) & 1, abort_word);
      if (!ok) break;
      TL_ADD(11, tl_t);
      tc_fence_after();
      if (lane == 0) {
        const uint32_t q_addr = smem_u32(sm.q[st]), do_addr = smem_u32(sm.dout[st]);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          uint64_t a = make_sdesc_sw128(k_addr + (k >> 2) * kKvHalf + (k & 3) * 32, 16, 1024);
          uint64_t b = make_sdesc_sw128(q_addr + (k >> 2) * kQHalf + (k & 3) * 32, 16, 1024);
          umma_ss(tmem + cS, a, b, idesc_sdp, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          uint64_t a = make_sdesc_sw128(v_addr + (k >> 2) * kKvHalf + (k & 3) * 32, 16, 1024);
          uint64_t b = make_sdesc_sw128(do_addr + (k >> 2) * kQHalf + (k & 3) * 32, 16, 1024);
          umma_ss(tmem + cdP, a, b, idesc_sdp, k > 0 ? 1u : 0u);
        }
        umma_commit(&sm.sdp_full);
      }
      __syncwarp();
      if (i > 0) ok = issue_acc(i - 1);
    }
    if (ok && n_items > 0) ok = issue_acc(n_items - 1);
    if (ok && n_items > 0) mbar_wait(&sm.dq_full, (n_items - 1) & 1, abort_word);
  } else {
    // ------------------------------------------------------------ softmax-gradient threads
    // 16 warps: warp w works on TMEM lanes 32*(w&3).. (key rows) and on query columns 16*(w>>2)..+15; four
    // warps per scheduler hide each other's TMEM / shared-memory / special-function latencies
    const int quad = warp & 3, hf = warp >> 2;
    const int r = quad * 32 + lane;  // key row inside the tile == TMEM lane
    const uint32_t lane_base = uint32_t(quad * 32) << 16;
    const float sl2 = scale * 1.4426950408889634f;
    const bool key_valid = r < cta.n_valid;
    bool ok = true;
    BwdItem prev{};
    // adds half (8 queries) of this warp's [32 d x 16 q] part of dQ^T of an item into the fp32
    // accumulator: transpose through the warp's staging tile, then one TMA reduce-add of the
    // [8 q x 32 d] tile (local accumulator) or one 128-byte bulk reduce per query row (peer)
    auto flush_dq = [&](const BwdItem& itx, int buf, int half) {
      if (itx.dq_dev < 0) return;  // dQ not wanted (used to measure the cost of the drain)
      float* stage = sm.dq_stage[warp];
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the earlier drain has left smem
      __syncwarp();
      uint32_t reg[8];
      tmem_ld8(tmem + lane_base + cdQ + buf * 64 + hf * 16 + half * 8, reg);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 8; ++i) stage[i * 32 + lane] = __uint_as_float(reg[i]);
      fence_proxy_async_smem();
      __syncwarp();
      const int q0 = hf * 16 + half * 8;
      if (itx.dq_dev == 0) {
        // rows past n_rows hold exact zeros (their probabilities are masked to 0): adding them is harmless
        if (lane == 0) {
          asm volatile(
              "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
              ::"l"(reinterpret_cast<uint64_t>(&tm_dq)), "r"(smem_u32(stage)), "r"(quad * 32), "r"(itx.head),
              "r"(itx.dq_row + q0)
              : "memory");
        }
      } else {
        const int qi = q0 + lane;
        if (lane < 8 && qi < itx.n_rows) {
          float* dq = ptrs.dq[itx.dq_dev] + (size_t(itx.dq_row + qi) * hq + itx.head) * kHeadDim + quad * 32;
          asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;"
                       ::"l"(dq), "r"(smem_u32(stage + lane * 32)), "r"(128)
                       : "memory");
        }
      }
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    };
    // S^T / dP^T of an item are pulled into registers as early as possible (right after the
    // previous item's operands were handed to the tensor core), which frees their TMEM columns for
    // the next-but-one item while this warp still drains dQ and does the math
    uint32_t sreg[16], dreg[16];
    auto load_sdp = [&](int t) -> bool {
      bool k = mbar_wait(&sm.sdp_full, t & 1, abort_word);
      k = __all_sync(0xffffffffu, k);
      if (!k) return false;
      TL_ADD(1, tl_t);
      tc_fence_after();
      tmem_ld16(tmem + lane_base + cS + hf * 16, sreg);
      tmem_ld16(tmem + lane_base + cdP + hf * 16, dreg);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(&sm.s_free);
      TL_ADD(2, tl_t);
      return true;
    };
    if (n_items > 0) ok = load_sdp(0);
    for (int t = 0; t < n_items && ok; ++t) {
      const int st = t % kStages;
      ok = mbar_wait(&sm.stats_full[st], (t / kStages) & 1, abort_word);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const BwdItem itx = sm.item[st];
      TL_ADD(0, tl_t);
      const int kpos = itx.kv_pos0 + r;
      const int n_rows_h = itx.n_rows - hf * 16;  // valid queries inside this warp's column quarter
      uint32_t preg[8], dsreg[8];
      // The tile-level "no masking needed" switch is taken once, outside the element loop: with a
      // branch per element every element becomes its own basic block and the compiler cannot
      // interleave the independent exp / multiply chains.
      const float* lse2_w = sm.lse2[st] + hf * 16;
      const float* delta_w = sm.delta[st] + hf * 16;
      const uint64_t sl2_2 = pack_f32x2(sl2, sl2), scale_2 = pack_f32x2(scale, scale);
      const uint64_t* nlse_w = reinterpret_cast<const uint64_t*>(lse2_w);
      const uint64_t* ndel_w = reinterpret_cast<const uint64_t*>(delta_w);
      if (itx.full) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          // two queries per instruction: exponent argument and (dP - delta) * scale in packed fp32
          const uint64_t x2 = fma_f32x2(pack_f32x2(__uint_as_float(sreg[2 * c]), __uint_as_float(sreg[2 * c + 1])), sl2_2, nlse_w[c]);
          const uint64_t g2 = fma_f32x2(pack_f32x2(__uint_as_float(dreg[2 * c]), __uint_as_float(dreg[2 * c + 1])), scale_2, ndel_w[c]);
          float x0, x1;
          unpack_f32x2(x2, x0, x1);
          const float e0 = fast_exp2(x0), e1 = fast_exp2(x1);
          const float p0 = (key_valid && (2 * c < n_rows_h)) ? e0 : 0.f;
          const float p1 = (key_valid && (2 * c + 1 < n_rows_h)) ? e1 : 0.f;
          float d0, d1;
          unpack_f32x2(mul_f32x2(pack_f32x2(p0, p1), g2), d0, d1);
          preg[c] = pack_bf16x2(p0, p1);
          dsreg[c] = pack_bf16x2(d0, d1);
        }
      } else {
        const int4* rng_w = sm.rng[st] + hf * 16;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint64_t x2 = fma_f32x2(pack_f32x2(__uint_as_float(sreg[2 * c]), __uint_as_float(sreg[2 * c + 1])), sl2_2, nlse_w[c]);
          const uint64_t g2 = fma_f32x2(pack_f32x2(__uint_as_float(dreg[2 * c]), __uint_as_float(dreg[2 * c + 1])), scale_2, ndel_w[c]);
          float x0, x1;
          unpack_f32x2(x2, x0, x1);
          const float e0 = fast_exp2(x0), e1 = fast_exp2(x1);
          const int4 m0 = rng_w[2 * c], m1 = rng_w[2 * c + 1];
          const bool a0 = key_valid && ((unsigned(kpos - m0.x) < unsigned(m0.y - m0.x)) || (unsigned(kpos - m0.z) < unsigned(m0.w - m0.z)));
          const bool a1 = key_valid && ((unsigned(kpos - m1.x) < unsigned(m1.y - m1.x)) || (unsigned(kpos - m1.z) < unsigned(m1.w - m1.z)));
          const float p0 = a0 ? e0 : 0.f, p1 = a1 ? e1 : 0.f;
          float d0, d1;
          unpack_f32x2(mul_f32x2(pack_f32x2(p0, p1), g2), d0, d1);
          preg[c] = pack_bf16x2(p0, p1);
          dsreg[c] = pack_bf16x2(d0, d1);
        }
      }
      TL_ADD(5, tl_t);
      if (t > 0) {
        // the accumulating UMMAs of the previous item must have finished reading the P^T / dS^T tiles
        ok = mbar_wait(&sm.dq_full, (t - 1) & 1, abort_word);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
      }
      TL_ADD(3, tl_t);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int ch = hf * 2 + i;
        const uint32_t off = r * 128 + ((ch ^ (r & 7)) << 4);
        *reinterpret_cast<uint4*>(sm.p + off) = make_uint4(preg[4 * i], preg[4 * i + 1], preg[4 * i + 2], preg[4 * i + 3]);
        *reinterpret_cast<uint4*>(sm.ds + off) = make_uint4(dsreg[4 * i], dsreg[4 * i + 1], dsreg[4 * i + 2], dsreg[4 * i + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&sm.p_ready);
      TL_ADD(6, tl_t);
      // dQ^T of the previous item sits in the other TMEM buffer: drain it, in two halves around the
      // early load of the next S^T / dP^T, while the tensor core already accumulates this item
      if (t > 0) flush_dq(prev, (t - 1) & 1, 0);
      TL_ADD(4, tl_t);
      if (t + 1 < n_items) ok = load_sdp(t + 1);
      if (ok && t > 0) flush_dq(prev, (t - 1) & 1, 1);
      TL_ADD(7, tl_t);
      prev = itx;
    }
    ok = __all_sync(0xffffffffu, ok);
    if (ok && n_items > 0) {
      ok = mbar_wait(&sm.dq_full, (n_items - 1) & 1, abort_word);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        flush_dq(prev, (n_items - 1) & 1, 0);
        flush_dq(prev, (n_items - 1) & 1, 1);
        // dK / dV: lane = key row; this warp adds channels 32*hf .. 32*hf+31 of both
        float* dk = ptrs.dkv[cta.dkv_dev] + ((size_t(cta.dkv_row + r) * 2 + 0) * hkv + kv_head) * kHeadDim + hf * 32;
        float* dv = ptrs.dkv[cta.dkv_dev] + ((size_t(cta.dkv_row + r) * 2 + 1) * hkv + kv_head) * kHeadDim + hf * 32;
        uint32_t reg[32];
        tmem_ld32(tmem + lane_base + cdK + hf * 32, reg);
        tmem_wait_ld();
        if (key_valid) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            red_add_v4(dk + 4 * i, __uint_as_float(reg[4 * i]), __uint_as_float(reg[4 * i + 1]),
                       __uint_as_float(reg[4 * i + 2]), __uint_as_float(reg[4 * i + 3]));
        }
        tmem_ld32(tmem + lane_base + cdV + hf * 32, reg);
        tmem_wait_ld();
        if (key_valid) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            red_add_v4(dv + 4 * i, __uint_as_float(reg[4 * i]), __uint_as_float(reg[4 * i + 1]),
                       __uint_as_float(reg[4 * i + 2]), __uint_as_float(reg[4 * i + 3]));
        }
      }
    }
    // no staged dQ tile may still be in flight when the CTA retires (also on the abort path)
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 17) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  if (threadIdx.x == 0 && sm.abort_word) atomicExch(status, sm.abort_word);  // 1 = wait timeout, 3 = bad table
}

// delta[h][row] = sum_d dO[row][h][d] * O[row][h][d]; one warp per (row, head)
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  float* __restrict__ delta, int n_rows, int hq, int stat_stride, int row0) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (gw >= n_rows * hq) return;
  const int row = gw / hq, h = gw % hq;
  const size_t off = (size_t(row0 + row) * hq + h) * kHeadDim + lane * 4;
  const uint2 a = *reinterpret_cast<const uint2*>(o + off);
  const uint2 b = *reinterpret_cast<const uint2*>(d_o + off);
  const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float2 x = __bfloat1622float2(a2[i]), y = __bfloat1622float2(b2[i]);
    acc += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) delta[size_t(h) * stat_stride + row0 + row] = acc;
}

static int g_bwd_attr_set[2] = {0, 0};
static long long* g_bwd_timeline_host = nullptr;  // non-null selects the instrumented build of the kernel

}  // namespace dcpk

void dcpk_fill_copy_ctx(dcpk::CopyCtx* ctx, void* const* src_ptrs, void* const* dst_ptrs, int stat_stride);

using namespace dcpk;

extern "C" int dcpk_attn_delta(const void* o, const void* d_o, float* delta, int n_rows, int hq, int stat_stride,
                               int row0, void* stream) {
  if (n_rows <= 0) return 0;
  const long warps = long(n_rows) * hq;
  const int threads = 256;
  const long blocks = (warps * 32 + threads - 1) / threads;
  attn_delta_kernel<<<unsigned(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), delta, n_rows, hq, stat_stride,
      row0);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// Points the kernel's cycle-counter timeline at `buf` (>= 16 int64, device memory) or disables it (null).
extern "C" int dcpk_attn_bwd_set_timeline(void* buf) {
  long long* p = static_cast<long long*>(buf);
  g_bwd_timeline_host = p;
  return cudaMemcpyToSymbol(g_bwd_timeline, &p, sizeof(p)) == cudaSuccess ? 0 : -5;
}

// Launches the backward kernel: one CTA per (entry of `ctas`, KV head).  n_items_total / n_mask_rows are the
// lengths of the item and mask tables; entries that point past them are reported (status 3), not read.
extern "C" int dcpk_attn_bwd(const void* q_arena, const void* do_arena, long q_rows, const void* kv_arena,
                             long kv_rows, int hq, int hkv, const void* ctas, int n_ctas, const void* items,
                             int n_items_total, const void* masks, int n_mask_rows, const float* lse, const float* delta,
                             int stat_stride, float* const* dq_ptrs, float* const* dkv_ptrs, int n_dst, float scale,
                             const void* jobs, int n_jobs, void* const* job_src_ptrs, void* const* job_dst_ptrs,
                             int job_stat_stride, int* status, void* stream) {
  if (n_ctas <= 0) return n_jobs > 0 ? -6 : 0;   // copy jobs need a kernel to ride on
  if (n_dst > kMaxPeers || hq % hkv != 0) return -3;
  CUtensorMap tm_q, tm_do, tm_kv, tm_dq;
  if (encode_f32_tile_map(&tm_dq, dq_ptrs[0], uint64_t(q_rows), uint32_t(hq), kHeadDim, 8, 32)) return -1;
  if (encode_arena_map(&tm_q, q_arena, uint64_t(q_rows), uint32_t(hq), kHeadDim, kQTile)) return -1;
  if (encode_arena_map(&tm_do, do_arena, uint64_t(q_rows), uint32_t(hq), kHeadDim, kQTile)) return -1;
  if (encode_arena_map(&tm_kv, kv_arena, uint64_t(kv_rows), uint32_t(2 * hkv), kHeadDim, 128)) return -1;
  BwdPtrs pp;
  for (int i = 0; i < kMaxPeers; ++i) {
    pp.dq[i] = i < n_dst ? dq_ptrs[i] : nullptr;
    pp.dkv[i] = i < n_dst ? dkv_ptrs[i] : nullptr;
  }
  CopyCtx ctx;
  dcpk_fill_copy_ctx(&ctx, n_jobs > 0 ? job_src_ptrs : nullptr, n_jobs > 0 ? job_dst_ptrs : nullptr, job_stat_stride);
  const int smem = int(sizeof(BwdSmem)) + 1024;
  const int v = g_bwd_timeline_host ? 1 : 0;
  auto kernel = v ? attn_bwd_kernel<true> : attn_bwd_kernel<false>;
  if (!g_bwd_attr_set[v]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4;
    g_bwd_attr_set[v] = 1;
  }
  // about 16 fetch CTAs when there is something to fetch
  const int n_copy_rows = n_jobs > 0 ? (16 + hkv - 1) / hkv : 0;
  kernel<<<dim3(hkv, n_ctas + n_copy_rows), kBwdThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      tm_q, tm_do, tm_kv, tm_dq, static_cast<const BwdCta*>(ctas), static_cast<const BwdItemDesc*>(items),
      static_cast<const int4*>(masks), lse, delta, pp, hq, hkv, stat_stride, n_dst, int(q_rows), int(kv_rows),
      n_mask_rows, n_items_total, scale, static_cast<const CopyJob*>(jobs), n_jobs, ctx, n_copy_rows, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
