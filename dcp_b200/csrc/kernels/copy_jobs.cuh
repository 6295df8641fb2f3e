// Copy jobs: the data movement of a plan stage, executed from inside the compute kernels.
//
// A job moves a contiguous run of 16-byte (row data) or 4-byte (per-head statistics) units from a
// region of a peer GPU's arena into the same kind of region of this GPU's arena with plain loads
// and stores over the NVLink mapping.  The attention kernel of stage s carries the job list of
// stage s + 1: two otherwise idle warps of every CTA work through their share of the list while the
// CTA's tiles are being computed, so the operands of the next stage arrive during this stage's
// math and no separate copy launch, side stream or event is needed.  The same routine backs the
// stand-alone launch used when a stage has operands to fetch but no kernel to ride on.
//
// Takes the role of the reference's pack -> all_to_all -> unpack sequence
// (dcp/runtime/flash_attention/executor.py:1915-2074, dcp/ops/fused_ops.py:290-429).
#pragma once
#include <stdint.h>

#include "attn_common.cuh"

namespace dcpk {

static constexpr int kCopyKinds = 5;   // q, kv, dout (16-byte units); lse, delta (4-byte units)

struct CopyCtx {
  const uint8_t* src[kCopyKinds][kMaxPeers];   // base of the region on every rank (index = rank in the group)
  uint8_t* dst[kCopyKinds];                    // base of the region on this rank
  int stat_stride;                             // rows per head of the [heads, rows] statistics regions (same on all ranks)
};

struct CopyJob {
  int src_off;   // in units from the region base on the source rank
  int dst_off;   // in units from the region base on this rank
  int n;         // units
  int where;     // bits 0-7 source rank, bits 8-15 region kind, bit 16: 4-byte units instead of 16-byte,
                 // bits 24-31: head of a statistics job (its offsets are rows inside that head's row of the region)
};

// `tid` of `n_threads` cooperating threads of worker `worker` (of `n_workers`): the workers take jobs
// round-robin, the threads of a worker stride through a job with four loads in flight each
__device__ __forceinline__ void run_copy_jobs(const CopyJob* __restrict__ jobs, int n_jobs, const CopyCtx& ctx,
                                              int worker, int n_workers, int tid, int n_threads) {
  for (int j = worker; j < n_jobs; j += n_workers) {
    const CopyJob job = jobs[j];
    const int peer = job.where & 0xff, kind = (job.where >> 8) & 0xff;
    if (kind >= kCopyKinds || peer >= kMaxPeers || job.n <= 0 || job.src_off < 0 || job.dst_off < 0) continue;
    if (job.where & (1 << 16)) {
      const size_t head_off = size_t((job.where >> 24) & 0xff) * size_t(ctx.stat_stride);
      if (job.src_off + job.n > ctx.stat_stride || job.dst_off + job.n > ctx.stat_stride) continue;
      const float* s = reinterpret_cast<const float*>(ctx.src[kind][peer]) + head_off + job.src_off;
      float* d = reinterpret_cast<float*>(ctx.dst[kind]) + head_off + job.dst_off;
      for (int i = tid; i < job.n; i += n_threads) d[i] = s[i];
    } else {
      const uint4* s = reinterpret_cast<const uint4*>(ctx.src[kind][peer]) + job.src_off;
      uint4* d = reinterpret_cast<uint4*>(ctx.dst[kind]) + job.dst_off;
      int i = tid;
      for (; i + 3 * n_threads < job.n; i += 4 * n_threads) {
        const uint4 a = s[i], b = s[i + n_threads], c = s[i + 2 * n_threads], e = s[i + 3 * n_threads];
        d[i] = a; d[i + n_threads] = b; d[i + 2 * n_threads] = c; d[i + 3 * n_threads] = e;
      }
      for (; i < job.n; i += n_threads) d[i] = s[i];
    }
  }
}

}  // namespace dcpk
