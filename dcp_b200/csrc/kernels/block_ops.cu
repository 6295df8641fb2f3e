// Data-movement and reduction kernels around the attention kernels.  All of them can read
// or write peer GPU memory through NVLink mappings (plain ld/st/red, never TMA multicast):
//
//  copy_jobs        stand-alone launch of a stage's copy-job list (see copy_jobs.cuh; normally the
//                   attention kernel of the previous stage carries the list).
//  gather_rows      pull token rows of Q/KV/dO (and per-head fp32 statistics) from peers'
//                   arenas into this GPU's staging rows; replaces pack -> all_to_all -> unpack
//                   (dcp/ops/fused_ops.py:290-335 + executor.py:1915-2074 in the reference).
//  merge_out_lse    LSE-weighted merge of partial (out, lse) rows that peers stored into this
//                   GPU's partial arena (dcp/ops/fused_ops.py:15-247).
//  push_add_rows    add fp32 gradient staging rows into the owner's fp32 accumulator with
//                   vector red over NVLink (replaces send + blockwise sum, fused_ops.py:1087-1360).
//  cast_rows        fp32 accumulators -> bf16 gradients.
//  signal_barrier   all-to-all flag barrier with a deadline: a peer that never arrives makes
//                   the kernel record an error code and return instead of spinning forever.
#include "attn_common.cuh"
#include "copy_jobs.cuh"
#include "ptx.cuh"

namespace dcpk {

struct RowCopy {
  int peer;      // index into the pointer table
  int src_row;   // row in the source arena
  int dst_row;   // row in the destination arena
  int n_rows;
};

struct PtrTable {
  void* p[kMaxPeers];
};

// 16-byte vector copy of whole rows; blockIdx.y = entry, blockIdx.x strides the entry's vectors.
__global__ void gather_rows_kernel(const RowCopy* __restrict__ entries, PtrTable srcs, uint8_t* __restrict__ dst,
                                   int row_bytes) {
  const RowCopy e = entries[blockIdx.y];
  const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(srcs.p[e.peer]) +
                                                    size_t(e.src_row) * row_bytes);
  uint4* out = reinterpret_cast<uint4*>(dst + size_t(e.dst_row) * row_bytes);
  const size_t n_vec = size_t(e.n_rows) * row_bytes / 16;
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  // four independent loads in flight per thread to cover NVLink latency
  for (; i + 3 * stride < n_vec; i += 4 * stride) {
    uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    out[i] = a; out[i + stride] = b; out[i + 2 * stride] = c; out[i + 3 * stride] = d;
  }
  for (; i < n_vec; i += stride) out[i] = src[i];
}

// per-head fp32 statistics ([heads, rows] layout): copy n_rows consecutive floats per head
__global__ void gather_stats_kernel(const RowCopy* __restrict__ entries, PtrTable srcs, float* __restrict__ dst,
                                    int n_heads, int src_stride, int dst_stride) {
  const RowCopy e = entries[blockIdx.y];
  const float* src = static_cast<const float*>(srcs.p[e.peer]);
  const int total = n_heads * e.n_rows;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int h = i / e.n_rows, r = i % e.n_rows;
    dst[size_t(h) * dst_stride + e.dst_row + r] = src[size_t(h) * src_stride + e.src_row + r];
  }
}

__global__ void copy_jobs_kernel(const CopyJob* __restrict__ jobs, int n_jobs, CopyCtx ctx) {
  run_copy_jobs(jobs, n_jobs, ctx, blockIdx.x, gridDim.x, threadIdx.x, blockDim.x);
}

struct MergeOp {
  int dst_row;   // first row in the local out / lse buffers
  int n_tok;
  int src_off;   // first entry in src_rows
  int n_src;
};

// sixteen lanes per (token, head), each covering 8 of the 128 channels with 16-byte accesses; the
// loads of all sources of an item are independent, so several rows are in flight per thread
__global__ void merge_out_lse_kernel(const MergeOp* __restrict__ ops, const int* __restrict__ src_rows,
                                     const __nv_bfloat16* __restrict__ part_out, const float* __restrict__ part_lse,
                                     int part_stride, __nv_bfloat16* __restrict__ out, float* __restrict__ lse,
                                     int out_stride, int hq) {
  const MergeOp op = ops[blockIdx.y];
  const int sub = threadIdx.x & 15;
  const int per_block = blockDim.x >> 4;
  const int total = op.n_tok * hq;
  const int* rows = src_rows + op.src_off;
  for (int item = blockIdx.x * per_block + (threadIdx.x >> 4); item < total; item += gridDim.x * per_block) {
    // heads fastest: the 16-lane groups of a block read neighbouring heads of one partial row
    const int t = item / hq, h = item % hq;
    float m = -INFINITY;
#pragma unroll 4
    for (int s = 0; s < op.n_src; ++s) {
      const float l = part_lse[size_t(h) * part_stride + rows[s] + t];
      if (l == l && l != INFINITY) m = fmaxf(m, l);  // skip NaN / +inf partials
    }
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float wsum = 0.f;
    if (m != -INFINITY) {
#pragma unroll 4
      for (int s = 0; s < op.n_src; ++s) {
        const int row = rows[s] + t;
        const float l = part_lse[size_t(h) * part_stride + row];
        const uint4 raw = *reinterpret_cast<const uint4*>(part_out + (size_t(row) * hq + h) * kHeadDim + sub * 8);
        if (!(l == l) || l == INFINITY || l == -INFINITY) continue;
        const float w = __expf(l - m);
        wsum += w;
        const __nv_bfloat162* v = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 a = __bfloat1622float2(v[j]);
          acc[2 * j] += w * a.x; acc[2 * j + 1] += w * a.y;
        }
      }
    }
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
    uint4 packed;
    packed.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
    packed.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
    packed.z = pack_bf16x2(acc[4] * inv, acc[5] * inv);
    packed.w = pack_bf16x2(acc[6] * inv, acc[7] * inv);
    *reinterpret_cast<uint4*>(out + (size_t(op.dst_row + t) * hq + h) * kHeadDim + sub * 8) = packed;
    if (sub == 0) lse[size_t(h) * out_stride + op.dst_row + t] = wsum > 0.f ? m + __logf(wsum) : -INFINITY;
  }
}

// dst[peer][dst_row..] += src[src_row..] (fp32 rows, vector red); peer may be this GPU
__global__ void push_add_rows_kernel(const RowCopy* __restrict__ entries, const float* __restrict__ src,
                                     PtrTable dsts, int row_floats) {
  const RowCopy e = entries[blockIdx.y];
  const float4* s = reinterpret_cast<const float4*>(src + size_t(e.src_row) * row_floats);
  float* d = static_cast<float*>(dsts.p[e.peer]) + size_t(e.dst_row) * row_floats;
  const size_t n_vec = size_t(e.n_rows) * row_floats / 4;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += size_t(gridDim.x) * blockDim.x) {
    const float4 v = s[i];
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d + 4 * i), "f"(v.x), "f"(v.y), "f"(v.z),
                 "f"(v.w)
                 : "memory");
  }
}

__global__ void cast_f32_bf16_kernel(const float4* __restrict__ src, uint2* __restrict__ dst, size_t n_vec) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += size_t(gridDim.x) * blockDim.x) {
    const float4 v = src[i];
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    dst[i] = o;
  }
}

struct FlagTable {
  uint32_t* p[kMaxPeers];  // p[r] = base of rank r's flag array: flags[r][sender]
};

// thread t: tell rank t we reached `epoch`, then wait until rank t told us the same.
__global__ void signal_barrier_kernel(FlagTable flags, int my_rank, int world, uint32_t epoch, uint64_t timeout_ns,
                                      int* __restrict__ status) {
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();  // everything this GPU wrote before the barrier is visible first
  if (t != my_rank) st_release_sys(flags.p[t] + my_rank, epoch);
  if (t == my_rank) return;
  const uint32_t* mine = flags.p[my_rank] + t;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    const uint32_t v = ld_acquire_sys(mine);
    if (int32_t(v - epoch) >= 0) break;
    if ((++spins & 255u) == 0 && global_timer_ns() - t0 > timeout_ns) {
      atomicExch(status, kStatusSignalTimeout);
      break;
    }
    __nanosleep(64);
  }
}

}  // namespace dcpk

using namespace dcpk;

static PtrTable make_ptrs(void* const* ptrs, int n) {
  PtrTable t;
  for (int i = 0; i < kMaxPeers; ++i) t.p[i] = i < n ? ptrs[i] : nullptr;
  return t;
}

// src_ptrs: kCopyKinds x kMaxPeers region bases (row-major, unused entries null), dst_ptrs: kCopyKinds bases
void dcpk_fill_copy_ctx(CopyCtx* ctx, void* const* src_ptrs, void* const* dst_ptrs, int stat_stride) {
  ctx->stat_stride = stat_stride;
  for (int k = 0; k < kCopyKinds; ++k) {
    for (int r = 0; r < kMaxPeers; ++r) ctx->src[k][r] = static_cast<const uint8_t*>(src_ptrs ? src_ptrs[k * kMaxPeers + r] : nullptr);
    ctx->dst[k] = static_cast<uint8_t*>(dst_ptrs ? dst_ptrs[k] : nullptr);
  }
}

extern "C" int dcpk_copy_jobs(const void* jobs, int n_jobs, void* const* src_ptrs, void* const* dst_ptrs, int stat_stride,
                              void* stream) {
  if (n_jobs <= 0) return 0;
  CopyCtx ctx;
  dcpk_fill_copy_ctx(&ctx, src_ptrs, dst_ptrs, stat_stride);
  const int grid = n_jobs < 592 ? n_jobs : 592;
  copy_jobs_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const CopyJob*>(jobs), n_jobs, ctx);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int dcpk_gather_rows(const void* entries, int n_entries, void* const* src_ptrs, int n_src, void* dst,
                                int row_bytes, void* stream) {
  if (n_entries <= 0) return 0;
  if (row_bytes % 16 != 0 || n_src > kMaxPeers) return -3;
  dim3 grid(16, n_entries);
  gather_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const RowCopy*>(entries), make_ptrs(src_ptrs, n_src), static_cast<uint8_t*>(dst), row_bytes);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int dcpk_gather_stats(const void* entries, int n_entries, void* const* src_ptrs, int n_src, float* dst,
                                 int n_heads, int src_stride, int dst_stride, void* stream) {
  if (n_entries <= 0) return 0;
  dim3 grid(4, n_entries);
  gather_stats_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const RowCopy*>(entries), make_ptrs(src_ptrs, n_src), dst, n_heads, src_stride, dst_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int dcpk_merge_out_lse(const void* ops, int n_ops, const void* src_rows, const void* part_out,
                                  const float* part_lse, int part_stride, void* out, float* lse, int out_stride,
                                  int hq, void* stream) {
  if (n_ops <= 0) return 0;
  // enough CTAs to fill the GPU whatever the number of ops (an op is one Q block, up to block_size tokens)
  const int per_op = n_ops >= 592 ? 1 : (592 + n_ops - 1) / n_ops;
  dim3 grid(per_op, n_ops);
  merge_out_lse_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const MergeOp*>(ops), static_cast<const int*>(src_rows),
      static_cast<const __nv_bfloat16*>(part_out), part_lse, part_stride, static_cast<__nv_bfloat16*>(out), lse,
      out_stride, hq);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int dcpk_push_add_rows(const void* entries, int n_entries, const float* src, void* const* dst_ptrs,
                                  int n_dst, int row_floats, void* stream) {
  if (n_entries <= 0) return 0;
  if (row_floats % 4 != 0 || n_dst > kMaxPeers) return -3;
  dim3 grid(16, n_entries);
  push_add_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const RowCopy*>(entries), src, make_ptrs(dst_ptrs, n_dst), row_floats);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int dcpk_cast_f32_bf16(const float* src, void* dst, long n, void* stream) {
  if (n <= 0) return 0;
  if (n % 4 != 0) return -3;
  const size_t n_vec = size_t(n) / 4;
  const int blocks = int(n_vec / 256 + 1 < 2048 ? n_vec / 256 + 1 : 2048);
  cast_f32_bf16_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float4*>(src), static_cast<uint2*>(dst), n_vec);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// flag_ptrs[r] = device address of rank r's flag array (>= world uint32 each, zero-initialised).
extern "C" int dcpk_signal_barrier(void* const* flag_ptrs, int my_rank, int world, unsigned epoch, double timeout_s,
                                   int* status, void* stream) {
  if (world > kMaxPeers) return -3;
  if (world <= 1) return 0;
  FlagTable ft;
  for (int i = 0; i < kMaxPeers; ++i) ft.p[i] = i < world ? static_cast<uint32_t*>(flag_ptrs[i]) : nullptr;
  signal_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      ft, my_rank, world, epoch, uint64_t(timeout_s * 1e9), status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
