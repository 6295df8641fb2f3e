// Data-parallel gradient reduction and sharded optimizer step over NVLink peer memory.
//
//  grad_reduce_scatter   rank r reads slice r of every rank's bf16 gradient buffer with 16-byte
//                        peer loads, sums in fp32, applies the loss/DP scale and writes the fp32
//                        main-grad shard; the squared norm of the shard is accumulated on the fly.
//                        One kernel replaces NCCL reduce-scatter + cast + scale + norm
//                        (what Megatron's distributed optimizer does for the reference,
//                        benchmark/mlm/launch_template.txt:78).
//  adamw_all_gather      AdamW on the fp32 master shard; the updated bf16 parameters are stored
//                        straight into every rank's parameter buffer (the all-gather is the
//                        epilogue of the update).
//  cast_all_gather       bf16(master shard) stored into every rank's parameter buffer (resume).
//
// The flat buffers are cut into buckets (one per decoder layer plus the embeddings / head); a
// bucket's reduce-scatter is launched on a side stream as soon as the layer's backward has
// written its gradients, so the reduction overlaps the rest of the backward pass.
//
// Failure containment: every kernel that changes optimizer state or parameters takes the status
// words of the arenas whose barriers guard its inputs; if either is nonzero (a barrier wait ran
// out, a table was bad) the kernel returns without touching master weights, moments, main
// gradients or parameters, so a detected failure never reaches the weights.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dcpk {

static constexpr int kMaxRanks = 16;
struct GradPtrs { const void* p[kMaxRanks]; };
struct ParamPtrs { void* p[kMaxRanks]; };
struct StatusPtrs { const int* a; const int* b; };

__device__ __forceinline__ bool failed(const StatusPtrs& st) {
  return (st.a && *reinterpret_cast<const volatile int*>(st.a) != 0) ||
         (st.b && *reinterpret_cast<const volatile int*>(st.b) != 0);
}

__global__ void grad_reduce_scatter_kernel(GradPtrs grads, int world, size_t shard_off, size_t shard_len, float scale,
                                           float* __restrict__ main_grad, float* __restrict__ sq_norm,
                                           StatusPtrs st) {
  // shard_off / shard_len in elements, both multiples of 8
  if (failed(st)) return;
  const size_t n_vec = shard_len / 8;
  float local_sq = 0.f;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += size_t(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
      const uint4 raw = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(grads.p[r]) + shard_off)[i];
      const __nv_bfloat162* v = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(v[j]);
        acc[2 * j] += f.x; acc[2 * j + 1] += f.y;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) { acc[j] *= scale; local_sq += acc[j] * acc[j]; }
    float4* out = reinterpret_cast<float4*>(main_grad + i * 8);
    out[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    out[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) local_sq += __shfl_xor_sync(0xffffffffu, local_sq, s);
  if ((threadIdx.x & 31) == 0 && sq_norm) atomicAdd(sq_norm, local_sq);
}

__global__ void adamw_all_gather_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                        const float* __restrict__ grad, ParamPtrs params, int world, size_t shard_off,
                                        size_t shard_len, float lr, float beta1, float beta2, float eps, float wd,
                                        float bc1, float bc2, const float* __restrict__ clip_coef, StatusPtrs st) {
  if (failed(st)) return;
  const float clip = clip_coef ? *clip_coef : 1.f;
  const size_t n_vec = shard_len / 8;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += size_t(gridDim.x) * blockDim.x) {
    uint4 packed;
    __nv_bfloat162* pk = reinterpret_cast<__nv_bfloat162*>(&packed);
    float p[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const size_t e = i * 8 + j;
      const float g = grad[e] * clip;
      const float mi = beta1 * m[e] + (1.f - beta1) * g;
      const float vi = beta2 * v[e] + (1.f - beta2) * g * g;
      float w = master[e];
      w -= lr * (mi / bc1 / (sqrtf(vi / bc2) + eps) + wd * w);
      m[e] = mi; v[e] = vi; master[e] = w;
      p[j] = w;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) pk[j] = __floats2bfloat162_rn(p[2 * j], p[2 * j + 1]);
    for (int r = 0; r < world; ++r)
      reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.p[r]) + shard_off)[i] = packed;
  }
}

// squared norm of the scaled, rank-summed gradient slice; nothing is written but the scalar
__global__ void grad_sqnorm_kernel(GradPtrs grads, int world, size_t shard_off, size_t shard_len, float scale,
                                   float* __restrict__ sq_norm) {
  const size_t n_vec = shard_len / 8;
  float local_sq = 0.f;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += size_t(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
      const uint4 raw = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(grads.p[r]) + shard_off)[i];
      const __nv_bfloat162* v = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(v[j]);
        acc[2 * j] += f.x; acc[2 * j + 1] += f.y;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) { acc[j] *= scale; local_sq += acc[j] * acc[j]; }
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) local_sq += __shfl_xor_sync(0xffffffffu, local_sq, s);
  if ((threadIdx.x & 31) == 0) atomicAdd(sq_norm, local_sq);
}

// reduce-scatter + AdamW + all-gather in one pass: the gradient slice is summed from every rank's
// bf16 buffer on the fly (no fp32 gradient copy exists), the fp32 state is updated, and the new
// bf16 parameters are stored into every rank's parameter buffer.
__global__ void fused_rs_adamw_ag_kernel(GradPtrs grads, ParamPtrs params, int world, size_t shard_off,
                                         size_t shard_len, float scale, float* __restrict__ master,
                                         float* __restrict__ m, float* __restrict__ v, float lr, float beta1,
                                         float beta2, float eps, float wd, float bc1, float bc2,
                                         const float* __restrict__ clip_coef, StatusPtrs st) {
  if (failed(st)) return;
  const float gscale = scale * (clip_coef ? *clip_coef : 1.f);
  const size_t n_vec = shard_len / 8;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += size_t(gridDim.x) * blockDim.x) {
    float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
      const uint4 raw = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(grads.p[r]) + shard_off)[i];
      const __nv_bfloat162* gv = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(gv[j]);
        g[2 * j] += f.x; g[2 * j + 1] += f.y;
      }
    }
    float4* mp = reinterpret_cast<float4*>(m + i * 8);
    float4* vp = reinterpret_cast<float4*>(v + i * 8);
    float4* wp = reinterpret_cast<float4*>(master + i * 8);
    float mm[8], vv[8], ww[8];
    *reinterpret_cast<float4*>(mm) = mp[0]; *reinterpret_cast<float4*>(mm + 4) = mp[1];
    *reinterpret_cast<float4*>(vv) = vp[0]; *reinterpret_cast<float4*>(vv + 4) = vp[1];
    *reinterpret_cast<float4*>(ww) = wp[0]; *reinterpret_cast<float4*>(ww + 4) = wp[1];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * gscale;
      mm[j] = beta1 * mm[j] + (1.f - beta1) * gj;
      vv[j] = beta2 * vv[j] + (1.f - beta2) * gj * gj;
      ww[j] -= lr * (mm[j] / bc1 / (sqrtf(vv[j] / bc2) + eps) + wd * ww[j]);
    }
    mp[0] = *reinterpret_cast<float4*>(mm); mp[1] = *reinterpret_cast<float4*>(mm + 4);
    vp[0] = *reinterpret_cast<float4*>(vv); vp[1] = *reinterpret_cast<float4*>(vv + 4);
    wp[0] = *reinterpret_cast<float4*>(ww); wp[1] = *reinterpret_cast<float4*>(ww + 4);
    uint4 packed;
    __nv_bfloat162* pk = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int j = 0; j < 4; ++j) pk[j] = __floats2bfloat162_rn(ww[2 * j], ww[2 * j + 1]);
    for (int r = 0; r < world; ++r)
      reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.p[r]) + shard_off)[i] = packed;
  }
}

// bf16(master) -> every rank's parameter buffer: rebuilds the replicated bf16 parameters from the
// sharded fp32 master weights (after loading a checkpoint)
__global__ void cast_all_gather_kernel(const float* __restrict__ master, ParamPtrs params, int world, size_t shard_off,
                                       size_t shard_len) {
  const size_t n_vec = shard_len / 8;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += size_t(gridDim.x) * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(master + i * 8)[0];
    const float4 b = reinterpret_cast<const float4*>(master + i * 8)[1];
    uint4 packed;
    __nv_bfloat162* pk = reinterpret_cast<__nv_bfloat162*>(&packed);
    pk[0] = __floats2bfloat162_rn(a.x, a.y); pk[1] = __floats2bfloat162_rn(a.z, a.w);
    pk[2] = __floats2bfloat162_rn(b.x, b.y); pk[3] = __floats2bfloat162_rn(b.z, b.w);
    for (int r = 0; r < world; ++r)
      reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.p[r]) + shard_off)[i] = packed;
  }
}

}  // namespace dcpk

using namespace dcpk;

extern "C" int dcpk_grad_sqnorm(const void* const* grad_ptrs, int world, long shard_off, long shard_len, float scale,
                                float* sq_norm, void* stream) {
  if (shard_len <= 0) return 0;
  if (world > kMaxRanks || shard_off % 8 || shard_len % 8) return -3;
  GradPtrs g;
  for (int i = 0; i < kMaxRanks; ++i) g.p[i] = i < world ? grad_ptrs[i] : nullptr;
  grad_sqnorm_kernel<<<148 * 4, 256, 0, static_cast<cudaStream_t>(stream)>>>(g, world, size_t(shard_off),
                                                                             size_t(shard_len), scale, sq_norm);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int dcpk_fused_rs_adamw_ag(const void* const* grad_ptrs, void* const* param_ptrs, int world, long shard_off,
                                      long shard_len, float scale, float* master, float* m, float* v, float lr,
                                      float beta1, float beta2, float eps, float wd, int step, const float* clip_coef,
                                      const int* status_a, const int* status_b, void* stream) {
  if (shard_len <= 0) return 0;
  if (world > kMaxRanks || shard_off % 8 || shard_len % 8) return -3;
  GradPtrs g;
  ParamPtrs p;
  for (int i = 0; i < kMaxRanks; ++i) {
    g.p[i] = i < world ? grad_ptrs[i] : nullptr;
    p.p[i] = i < world ? param_ptrs[i] : nullptr;
  }
  const float bc1 = 1.f - powf(beta1, float(step)), bc2 = 1.f - powf(beta2, float(step));
  fused_rs_adamw_ag_kernel<<<148 * 4, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      g, p, world, size_t(shard_off), size_t(shard_len), scale, master, m, v, lr, beta1, beta2, eps, wd, bc1, bc2,
      clip_coef, StatusPtrs{status_a, status_b});
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// n_ctas: grid size (0 = fill the GPU).  A reduce that overlaps the backward pass is given a small
// grid so it trickles over NVLink next to the GEMMs instead of taking their SMs.
extern "C" int dcpk_grad_reduce_scatter(const void* const* grad_ptrs, int world, long shard_off, long shard_len,
                                        float scale, float* main_grad, float* sq_norm, int n_ctas,
                                        const int* status_a, const int* status_b, void* stream) {
  if (shard_len <= 0) return 0;
  if (world > kMaxRanks || shard_off % 8 || shard_len % 8) return -3;
  GradPtrs g;
  for (int i = 0; i < kMaxRanks; ++i) g.p[i] = i < world ? grad_ptrs[i] : nullptr;
  grad_reduce_scatter_kernel<<<n_ctas > 0 ? n_ctas : 148 * 4, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      g, world, size_t(shard_off), size_t(shard_len), scale, main_grad, sq_norm, StatusPtrs{status_a, status_b});
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int dcpk_adamw_all_gather(float* master, float* m, float* v, const float* grad, void* const* param_ptrs,
                                     int world, long shard_off, long shard_len, float lr, float beta1, float beta2,
                                     float eps, float wd, int step, const float* clip_coef, const int* status_a,
                                     const int* status_b, void* stream) {
  if (shard_len <= 0) return 0;
  if (world > kMaxRanks || shard_off % 8 || shard_len % 8) return -3;
  ParamPtrs p;
  for (int i = 0; i < kMaxRanks; ++i) p.p[i] = i < world ? param_ptrs[i] : nullptr;
  const float bc1 = 1.f - powf(beta1, float(step)), bc2 = 1.f - powf(beta2, float(step));
  adamw_all_gather_kernel<<<148 * 4, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      master, m, v, grad, p, world, size_t(shard_off), size_t(shard_len), lr, beta1, beta2, eps, wd, bc1, bc2,
      clip_coef, StatusPtrs{status_a, status_b});
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int dcpk_cast_all_gather(const float* master, void* const* param_ptrs, int world, long shard_off,
                                    long shard_len, void* stream) {
  if (shard_len <= 0) return 0;
  if (world > kMaxRanks || shard_off % 8 || shard_len % 8) return -3;
  ParamPtrs p;
  for (int i = 0; i < kMaxRanks; ++i) p.p[i] = i < world ? param_ptrs[i] : nullptr;
  cast_all_gather_kernel<<<148 * 4, 256, 0, static_cast<cudaStream_t>(stream)>>>(master, p, world, size_t(shard_off),
                                                                                size_t(shard_len));
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
