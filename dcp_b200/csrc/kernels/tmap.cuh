// Host-side helper: encode TMA tensor maps for the row-addressed bf16 arenas
// ([rows, heads, head_dim], 128-byte swizzle, box = 64 x 1 x box_rows).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace dcpk {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// arena: bf16 [rows, heads, d]; tile box: [box_rows, 1, 64]
inline int encode_arena_map(CUtensorMap* out, const void* base, uint64_t rows, uint32_t heads, uint32_t d,
                            uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {d, heads, rows};
  cuuint64_t strides[2] = {uint64_t(d) * 2, uint64_t(d) * heads * 2};
  cuuint32_t box[3] = {64, 1, box_rows};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "dcpk: cuTensorMapEncodeTiled failed (%d) base=%p rows=%llu heads=%u d=%u\n", int(r), base,
            (unsigned long long)rows, heads, d);
    return -2;
  }
  return 0;
}

// fp32 accumulator arena [rows, heads, 128] addressed as [box_rows x 1 x 32 floats] tiles (no swizzle),
// the shape the backward kernel's per-warp dQ staging tiles have
inline int encode_f32_tile_map(CUtensorMap* out, const void* base, uint64_t rows, uint32_t heads, uint32_t d,
                               uint32_t box_rows, uint32_t box_inner) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {d, heads, rows};
  cuuint64_t strides[2] = {uint64_t(d) * 4, uint64_t(d) * heads * 4};
  cuuint32_t box[3] = {box_inner, 1, box_rows};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "dcpk: cuTensorMapEncodeTiled (fp32 tile) failed (%d)\n", int(r));
    return -2;
  }
  return 0;
}

}  // namespace dcpk
