// Memory-bound transformer ops in bf16 with fp32 math, written for HBM3e: 16-byte vector
// accesses, one pass over the data wherever the math allows, and layout changes fused into
// the op that touches the data anyway.
//
//  rmsnorm_fwd / rmsnorm_bwd      y = x * rsqrt(mean(x^2) + eps) * w
//  qkv_rope_split_fwd             packed QKV projection -> rotary on q,k -> attention arenas
//  qkv_rope_pack_bwd              fp32 dQ / dKV accumulators -> inverse rotary -> packed bf16 dQKV
//  swiglu_fwd / swiglu_bwd        y = silu(gate) * up on a [T, 2F] gate|up tensor
//  cross_entropy_fwd_bwd          per-row loss and in-place dlogits in one kernel
//
// The reference takes these from Megatron-LM / TransformerEngine / apex
// (benchmark/mlm/pretrain_gpt.py:143-167, benchmark/mlm/monkey_patch.py:158-251).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>

namespace dcpk {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
  return v;
}
template <int kWarps>
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = lane < kWarps ? scratch[lane] : 0.f;
  return warp_sum(t);
}
template <int kWarps>
__device__ __forceinline__ float block_max(float v, float* scratch) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = lane < kWarps ? scratch[lane] : -INFINITY;
  return warp_max(t);
}
__device__ __forceinline__ void unpack8(const uint4& raw, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x; f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 raw;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return raw;
}

// ------------------------------------------------------------------ RMSNorm
// one CTA of 128 threads per row; hidden must be a multiple of 1024 (8 per vector x 128 threads)
template <int kVecs>
__global__ void __launch_bounds__(128) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                                          int hidden, float eps) {
  __shared__ float scratch[4];
  const size_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * hidden);
  float v[kVecs][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    unpack8(xr[threadIdx.x + i * 128], v[i]);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
  }
  ss = block_sum<4>(ss, scratch);
  const float r = rsqrtf(ss / hidden + eps);
  if (threadIdx.x == 0) rstd[row] = r;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + row * hidden);
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    float wv[8];
    unpack8(wr[threadIdx.x + i * 128], wv);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[i][j] = v[i][j] * r * wv[j];
    yr[threadIdx.x + i * 128] = pack8(v[i]);
  }
}

// persistent CTAs: each walks rows blockIdx.x, +gridDim.x, ... and keeps its dW slice in registers
template <int kVecs>
__global__ void __launch_bounds__(128) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          const __nv_bfloat16* __restrict__ dy,
                                                          const float* __restrict__ rstd,
                                                          __nv_bfloat16* __restrict__ dx, float* __restrict__ dw,
                                                          int n_rows, int hidden) {
  __shared__ float scratch[4];
  float wv[kVecs][8], dwv[kVecs][8];
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    unpack8(wr[threadIdx.x + i * 128], wv[i]);
#pragma unroll
    for (int j = 0; j < 8; ++j) dwv[i][j] = 0.f;
  }
  for (size_t row = blockIdx.x; row < size_t(n_rows); row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * hidden);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + row * hidden);
    const float r = rstd[row];
    float xh[kVecs][8], g[kVecs][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kVecs; ++i) {
      unpack8(xr[threadIdx.x + i * 128], xh[i]);
      unpack8(gr[threadIdx.x + i * 128], g[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        xh[i][j] *= r;
        dwv[i][j] += g[i][j] * xh[i][j];
        g[i][j] *= wv[i][j];
        dot += g[i][j] * xh[i][j];
      }
    }
    dot = block_sum<4>(dot, scratch) / hidden;
    uint4* dxr = reinterpret_cast<uint4*>(dx + row * hidden);
#pragma unroll
    for (int i = 0; i < kVecs; ++i) {
#pragma unroll
      for (int j = 0; j < 8; ++j) g[i][j] = r * (g[i][j] - xh[i][j] * dot);
      dxr[threadIdx.x + i * 128] = pack8(g[i]);
    }
  }
  // one vector reduction per four channels (a quarter of the scalar atomics, which bound this kernel)
#pragma unroll
  for (int i = 0; i < kVecs; ++i)
#pragma unroll
    for (int j = 0; j < 8; j += 4)
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dw + (threadIdx.x + i * 128) * 8 + j),
                   "f"(dwv[i][j]), "f"(dwv[i][j + 1]), "f"(dwv[i][j + 2]), "f"(dwv[i][j + 3])
                   : "memory");
}

// ------------------------------------------------------------------ QKV split + rotary
// qkv: [T, (hq + 2*hkv) * 128] packed as q heads | k heads | v heads.  cos/sin: [T, 64].
// rotate-half convention: (x1, x2) -> (x1 cos - x2 sin, x2 cos + x1 sin), x1 = x[:64], x2 = x[64:].
// eight lanes per (token, head): lane s of the group owns channels 8s .. 8s+7 of each half, so every
// global access is a 16-byte vector (a warp moves four heads).
__global__ void qkv_rope_split_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ cs,
                                          const float* __restrict__ sn, __nv_bfloat16* __restrict__ q_out,
                                          __nv_bfloat16* __restrict__ kv_out, int n_tok, int hq, int hkv,
                                          int q_row0, int kv_row0) {
  const int heads = hq + 2 * hkv;
  const long item = (long(blockIdx.x) * blockDim.x + threadIdx.x) >> 3;
  const int sub = threadIdx.x & 7;
  if (item >= long(n_tok) * heads) return;
  const int t = int(item / heads), h = int(item % heads);
  const __nv_bfloat16* src = qkv + (size_t(t) * heads + h) * 128;
  __nv_bfloat16* dst;
  if (h < hq) dst = q_out + (size_t(q_row0 + t) * hq + h) * 128;
  else if (h < hq + hkv) dst = kv_out + ((size_t(kv_row0 + t) * 2 + 0) * hkv + (h - hq)) * 128;
  else dst = kv_out + ((size_t(kv_row0 + t) * 2 + 1) * hkv + (h - hq - hkv)) * 128;
  const uint4 a = *reinterpret_cast<const uint4*>(src + 8 * sub);
  const uint4 b = *reinterpret_cast<const uint4*>(src + 64 + 8 * sub);
  if (h < hq + hkv) {
    float x1[8], x2[8], c[8], sv[8], o1[8], o2[8];
    unpack8(a, x1); unpack8(b, x2);
    *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cs + size_t(t) * 64 + 8 * sub);
    *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cs + size_t(t) * 64 + 8 * sub + 4);
    *reinterpret_cast<float4*>(sv) = *reinterpret_cast<const float4*>(sn + size_t(t) * 64 + 8 * sub);
    *reinterpret_cast<float4*>(sv + 4) = *reinterpret_cast<const float4*>(sn + size_t(t) * 64 + 8 * sub + 4);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o1[j] = x1[j] * c[j] - x2[j] * sv[j];
      o2[j] = x2[j] * c[j] + x1[j] * sv[j];
    }
    *reinterpret_cast<uint4*>(dst + 8 * sub) = pack8(o1);
    *reinterpret_cast<uint4*>(dst + 64 + 8 * sub) = pack8(o2);
  } else {
    *reinterpret_cast<uint4*>(dst + 8 * sub) = a;
    *reinterpret_cast<uint4*>(dst + 64 + 8 * sub) = b;
  }
}

// dq: fp32 [rows, hq, 128], dkv: fp32 [rows, 2, hkv, 128] -> dqkv bf16 [T, (hq+2hkv)*128] with the
// rotation transposed (sin negated) on the q and k parts.  Same eight-lanes-per-head layout.
__global__ void qkv_rope_pack_bwd_kernel(const float* __restrict__ dq, const float* __restrict__ dkv,
                                         const float* __restrict__ cs, const float* __restrict__ sn,
                                         __nv_bfloat16* __restrict__ dqkv, int n_tok, int hq, int hkv, int q_row0,
                                         int kv_row0) {
  const int heads = hq + 2 * hkv;
  const long item = (long(blockIdx.x) * blockDim.x + threadIdx.x) >> 3;
  const int sub = threadIdx.x & 7;
  if (item >= long(n_tok) * heads) return;
  const int t = int(item / heads), h = int(item % heads);
  const float* src;
  if (h < hq) src = dq + (size_t(q_row0 + t) * hq + h) * 128;
  else if (h < hq + hkv) src = dkv + ((size_t(kv_row0 + t) * 2 + 0) * hkv + (h - hq)) * 128;
  else src = dkv + ((size_t(kv_row0 + t) * 2 + 1) * hkv + (h - hq - hkv)) * 128;
  __nv_bfloat16* dst = dqkv + (size_t(t) * heads + h) * 128;
  float g1[8], g2[8];
  *reinterpret_cast<float4*>(g1) = *reinterpret_cast<const float4*>(src + 8 * sub);
  *reinterpret_cast<float4*>(g1 + 4) = *reinterpret_cast<const float4*>(src + 8 * sub + 4);
  *reinterpret_cast<float4*>(g2) = *reinterpret_cast<const float4*>(src + 64 + 8 * sub);
  *reinterpret_cast<float4*>(g2 + 4) = *reinterpret_cast<const float4*>(src + 64 + 8 * sub + 4);
  if (h < hq + hkv) {
    float c[8], sv[8], o1[8], o2[8];
    *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cs + size_t(t) * 64 + 8 * sub);
    *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cs + size_t(t) * 64 + 8 * sub + 4);
    *reinterpret_cast<float4*>(sv) = *reinterpret_cast<const float4*>(sn + size_t(t) * 64 + 8 * sub);
    *reinterpret_cast<float4*>(sv + 4) = *reinterpret_cast<const float4*>(sn + size_t(t) * 64 + 8 * sub + 4);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o1[j] = g1[j] * c[j] + g2[j] * sv[j];
      o2[j] = g2[j] * c[j] - g1[j] * sv[j];
    }
    *reinterpret_cast<uint4*>(dst + 8 * sub) = pack8(o1);
    *reinterpret_cast<uint4*>(dst + 64 + 8 * sub) = pack8(o2);
  } else {
    *reinterpret_cast<uint4*>(dst + 8 * sub) = pack8(g1);
    *reinterpret_cast<uint4*>(dst + 64 + 8 * sub) = pack8(g2);
  }
}

// ------------------------------------------------------------------ SwiGLU
__global__ void swiglu_fwd_kernel(const uint4* __restrict__ gu, uint4* __restrict__ y, size_t n_rows, int f_vec) {
  const size_t total = n_rows * f_vec;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const size_t r = i / f_vec, c = i % f_vec;
    float g[8], u[8];
    unpack8(gu[r * 2 * f_vec + c], g);
    unpack8(gu[r * 2 * f_vec + f_vec + c], u);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    y[i] = pack8(g);
  }
}
__global__ void swiglu_bwd_kernel(const uint4* __restrict__ gu, const uint4* __restrict__ dy, uint4* __restrict__ dgu,
                                  size_t n_rows, int f_vec) {
  const size_t total = n_rows * f_vec;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const size_t r = i / f_vec, c = i % f_vec;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(gu[r * 2 * f_vec + c], g);
    unpack8(gu[r * 2 * f_vec + f_vec + c], u);
    unpack8(dy[i], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sg;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * (sg + silu * (1.f - sg));
    }
    dgu[r * 2 * f_vec + c] = pack8(dg);
    dgu[r * 2 * f_vec + f_vec + c] = pack8(du);
  }
}

// ------------------------------------------------------------------ cross entropy (loss + dlogits)
// one CTA of 256 threads per row; vocab must be a multiple of 8.  Rows whose label is < 0 are ignored
// (loss 0, zero gradient).  dlogits overwrite logits: (softmax - onehot) * grad_scale.
__global__ void __launch_bounds__(256) cross_entropy_kernel(__nv_bfloat16* __restrict__ logits,
                                                            const int64_t* __restrict__ labels,
                                                            float* __restrict__ loss, int vocab, float grad_scale) {
  __shared__ float scratch[8];
  const size_t row = blockIdx.x;
  uint4* lr = reinterpret_cast<uint4*>(logits + row * vocab);
  const int n_vec = vocab / 8;
  const long label = labels[row];
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < n_vec; i += 256) {
    float v[8];
    unpack8(lr[i], v);
    float lm = v[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, v[j]);
    const float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __expf(v[j] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  const float gm = block_max<8>(m, scratch);
  s = block_sum<8>(s * __expf(m - gm), scratch);
  const float lse = gm + __logf(s);
  if (threadIdx.x == 0) {
    float l = 0.f;
    if (label >= 0) l = lse - __bfloat162float(logits[row * vocab + label]);
    loss[row] = l;
  }
  __syncthreads();  // the label logit is read before anyone overwrites it
  const float scale = label >= 0 ? grad_scale : 0.f;
  for (int i = threadIdx.x; i < n_vec; i += 256) {
    float v[8];
    unpack8(lr[i], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(v[j] - lse);
      if (long(i) * 8 + j == label) p -= 1.f;
      v[j] = p * scale;
    }
    lr[i] = pack8(v);
  }
}

// ------------------------------------------------------------------ AdamW on a flat shard
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                             const float* __restrict__ grad, __nv_bfloat16* __restrict__ param_bf16, size_t n,
                             float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                             const float* __restrict__ clip_coef) {
  const float clip = clip_coef ? *clip_coef : 1.f;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
    const float g = grad[i] * clip;
    const float mi = beta1 * m[i] + (1.f - beta1) * g;
    const float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    float p = master[i];
    p -= lr * (mi / bc1 / (sqrtf(vi / bc2) + eps) + wd * p);
    m[i] = mi; v[i] = vi; master[i] = p;
    param_bf16[i] = __float2bfloat16(p);
  }
}

}  // namespace dcpk

using namespace dcpk;
#define STREAM static_cast<cudaStream_t>(stream)
#define LAUNCH_OK (cudaGetLastError() == cudaSuccess ? 0 : -5)

extern "C" int dcpk_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int n_rows, int hidden, float eps,
                                void* stream) {
  if (n_rows <= 0) return 0;
  auto X = static_cast<const __nv_bfloat16*>(x); auto W = static_cast<const __nv_bfloat16*>(w);
  auto Y = static_cast<__nv_bfloat16*>(y);
  switch (hidden) {
    case 1024: rmsnorm_fwd_kernel<1><<<n_rows, 128, 0, STREAM>>>(X, W, Y, rstd, hidden, eps); break;
    case 2048: rmsnorm_fwd_kernel<2><<<n_rows, 128, 0, STREAM>>>(X, W, Y, rstd, hidden, eps); break;
    case 4096: rmsnorm_fwd_kernel<4><<<n_rows, 128, 0, STREAM>>>(X, W, Y, rstd, hidden, eps); break;
    case 8192: rmsnorm_fwd_kernel<8><<<n_rows, 128, 0, STREAM>>>(X, W, Y, rstd, hidden, eps); break;
    default: return -3;
  }
  return LAUNCH_OK;
}

extern "C" int dcpk_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, void* dx, float* dw,
                                int n_rows, int hidden, void* stream) {
  if (n_rows <= 0) return 0;
  auto X = static_cast<const __nv_bfloat16*>(x); auto W = static_cast<const __nv_bfloat16*>(w);
  auto G = static_cast<const __nv_bfloat16*>(dy); auto DX = static_cast<__nv_bfloat16*>(dx);
  // persistent CTAs: exactly as many as are resident at once (registers decide), so no CTA waits for a
  // slot while others already finished their share
  auto launch = [&](auto kernel) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 128, 0) != cudaSuccess || per_sm < 1) per_sm = 2;
    const int cap = 148 * per_sm;
    const int grid = n_rows < cap ? n_rows : cap;
    kernel<<<grid, 128, 0, STREAM>>>(X, W, G, rstd, DX, dw, n_rows, hidden);
  };
  switch (hidden) {
    case 1024: launch(rmsnorm_bwd_kernel<1>); break;
    case 2048: launch(rmsnorm_bwd_kernel<2>); break;
    case 4096: launch(rmsnorm_bwd_kernel<4>); break;
    case 8192: launch(rmsnorm_bwd_kernel<8>); break;
    default: return -3;
  }
  return LAUNCH_OK;
}

extern "C" int dcpk_qkv_rope_split_fwd(const void* qkv, const float* cs, const float* sn, void* q_out, void* kv_out,
                                       int n_tok, int hq, int hkv, int q_row0, int kv_row0, void* stream) {
  if (n_tok <= 0) return 0;
  const long items = long(n_tok) * (hq + 2 * hkv);   // eight threads per (token, head)
  const long blocks = (items * 8 + 255) / 256;
  qkv_rope_split_fwd_kernel<<<unsigned(blocks), 256, 0, STREAM>>>(
      static_cast<const __nv_bfloat16*>(qkv), cs, sn, static_cast<__nv_bfloat16*>(q_out),
      static_cast<__nv_bfloat16*>(kv_out), n_tok, hq, hkv, q_row0, kv_row0);
  return LAUNCH_OK;
}

extern "C" int dcpk_qkv_rope_pack_bwd(const float* dq, const float* dkv, const float* cs, const float* sn, void* dqkv,
                                      int n_tok, int hq, int hkv, int q_row0, int kv_row0, void* stream) {
  if (n_tok <= 0) return 0;
  const long items = long(n_tok) * (hq + 2 * hkv);   // eight threads per (token, head)
  const long blocks = (items * 8 + 255) / 256;
  qkv_rope_pack_bwd_kernel<<<unsigned(blocks), 256, 0, STREAM>>>(dq, dkv, cs, sn, static_cast<__nv_bfloat16*>(dqkv),
                                                                  n_tok, hq, hkv, q_row0, kv_row0);
  return LAUNCH_OK;
}

extern "C" int dcpk_swiglu_fwd(const void* gu, void* y, long n_rows, int f, void* stream) {
  if (n_rows <= 0) return 0;
  if (f % 8 != 0) return -3;
  swiglu_fwd_kernel<<<148 * 8, 256, 0, STREAM>>>(static_cast<const uint4*>(gu), static_cast<uint4*>(y), size_t(n_rows), f / 8);
  return LAUNCH_OK;
}

extern "C" int dcpk_swiglu_bwd(const void* gu, const void* dy, void* dgu, long n_rows, int f, void* stream) {
  if (n_rows <= 0) return 0;
  if (f % 8 != 0) return -3;
  swiglu_bwd_kernel<<<148 * 8, 256, 0, STREAM>>>(static_cast<const uint4*>(gu), static_cast<const uint4*>(dy),
                                                  static_cast<uint4*>(dgu), size_t(n_rows), f / 8);
  return LAUNCH_OK;
}

extern "C" int dcpk_cross_entropy(void* logits, const void* labels, float* loss, int n_rows, int vocab, float grad_scale,
                                  void* stream) {
  if (n_rows <= 0) return 0;
  if (vocab % 8 != 0) return -3;
  cross_entropy_kernel<<<n_rows, 256, 0, STREAM>>>(static_cast<__nv_bfloat16*>(logits),
                                                   static_cast<const int64_t*>(labels), loss, vocab, grad_scale);
  return LAUNCH_OK;
}

extern "C" int dcpk_adamw(float* master, float* m, float* v, const float* grad, void* param_bf16, long n, float lr,
                          float beta1, float beta2, float eps, float wd, int step, const float* clip_coef,
                          void* stream) {
  if (n <= 0) return 0;
  const float bc1 = 1.f - powf(beta1, float(step)), bc2 = 1.f - powf(beta2, float(step));
  adamw_kernel<<<148 * 8, 256, 0, STREAM>>>(master, m, v, grad, static_cast<__nv_bfloat16*>(param_bf16), size_t(n), lr,
                                            beta1, beta2, eps, wd, bc1, bc2, clip_coef);
  return LAUNCH_OK;
}

// ------------------------------------------------------------------ allocation-free RMSNorm backward
// See noalloc.h.  The fp32 weight-gradient accumulator the regular entry point takes from its
// caller lives here, in a file-scope device array, so callers that must not allocate can still
// run the backward pass.
#include "noalloc.h"

static __device__ __align__(256) float g_noalloc_dw_accum[DCPK_NOALLOC_MAX_HIDDEN];

namespace dcpk {
static constexpr int kNoallocMaxDevices = 64;
// device address of g_noalloc_dw_accum per device; in host code the array's name is only a
// handle, the address a kernel can use comes from cudaGetSymbolAddress
static float* g_noalloc_accum_ptr[kNoallocMaxDevices] = {nullptr};

__global__ void dw_accum_to_bf16_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dw, int hidden) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < hidden) dw[i] = __float2bfloat16(acc[i]);
}
}  // namespace dcpk

extern "C" int dcpk_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd, void* dx,
                                        void* dw_bf16, int n_rows, int hidden, void* stream) {
  if (hidden > DCPK_NOALLOC_MAX_HIDDEN || (hidden != 1024 && hidden != 2048 && hidden != 4096 && hidden != 8192)) {
    fprintf(stderr, "dcpk_rmsnorm_bwd_noalloc: hidden=%d is not supported (1024, 2048, 4096 or 8192, at most %d)\n",
            hidden, DCPK_NOALLOC_MAX_HIDDEN);
    return -3;
  }
  if (n_rows < 0) return -3;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoallocMaxDevices) return -6;
  if (g_noalloc_accum_ptr[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_dw_accum) != cudaSuccess || p == nullptr) return -6;
    g_noalloc_accum_ptr[dev] = p;
  }
  float* accum = g_noalloc_accum_ptr[dev];
  // the array keeps what the previous call left: clear the part this call accumulates into
  if (cudaMemsetAsync(accum, 0, size_t(hidden) * sizeof(float), STREAM) != cudaSuccess) return -6;
  if (n_rows > 0) {
    const int rc = dcpk_rmsnorm_bwd(x, w, dy, rstd, dx, accum, n_rows, hidden, stream);
    if (rc != 0) return rc;
  }
  dw_accum_to_bf16_kernel<<<(hidden + 255) / 256, 256, 0, STREAM>>>(accum, static_cast<__nv_bfloat16*>(dw_bf16), hidden);
  return LAUNCH_OK;
}
