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
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dcpk {

static constexpr int kMaxRanks = 16;
struct GradPtrs { const void* p[kMaxRanks]; };
struct ParamPtrs { void* p[kMaxRanks]; };

__global__ void grad_reduce_scatter_kernel(GradPtrs grads, int world, size_t shard_off, size_t shard_len, float scale,
                                           float* __restrict__ main_grad, float* __restrict__ sq_norm) {
  // shard_off / shard_len in elements, both multiples of 8
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
                                        float bc1, float bc2, const float* __restrict__ clip_coef) {
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

}  // namespace dcpk

using namespace dcpk;

extern "C" int dcpk_grad_reduce_scatter(const void* const* grad_ptrs, int world, long shard_off, long shard_len,
                                        float scale, float* main_grad, float* sq_norm, void* stream) {
  if (shard_len <= 0) return 0;
  if (world > kMaxRanks || shard_off % 8 || shard_len % 8) return -3;
  GradPtrs g;
  for (int i = 0; i < kMaxRanks; ++i) g.p[i] = i < world ? grad_ptrs[i] : nullptr;
  grad_reduce_scatter_kernel<<<148 * 4, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      g, world, size_t(shard_off), size_t(shard_len), scale, main_grad, sq_norm);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int dcpk_adamw_all_gather(float* master, float* m, float* v, const float* grad, void* const* param_ptrs,
                                     int world, long shard_off, long shard_len, float lr, float beta1, float beta2,
                                     float eps, float wd, int step, const float* clip_coef, void* stream) {
  if (shard_len <= 0) return 0;
  if (world > kMaxRanks || shard_off % 8 || shard_len % 8) return -3;
  ParamPtrs p;
  for (int i = 0; i < kMaxRanks; ++i) p.p[i] = i < world ? param_ptrs[i] : nullptr;
  const float bc1 = 1.f - powf(beta1, float(step)), bc2 = 1.f - powf(beta2, float(step));
  adamw_all_gather_kernel<<<148 * 4, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      master, m, v, grad, p, world, size_t(shard_off), size_t(shard_len), lr, beta1, beta2, eps, wd, bc1, bc2,
      clip_coef);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
