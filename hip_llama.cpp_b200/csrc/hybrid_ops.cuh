// Typed loads and stores of the layer-program kernels (matrices and matrix-product inputs are bf16 or fp32), the scalar
// functions of their gates, and the address of a cache row in the block pool.
#pragma once
#include <cuda_bf16.h>

#include "tha_hybrid.h"

namespace tha {
__device__ __forceinline__ float hyb_load(const float* p) { return *p; }
__device__ __forceinline__ float hyb_load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void hyb_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void hyb_store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float hyb_softcap(float z, float cap) { return cap * tanhf(z / cap); }
__device__ __forceinline__ float hyb_logsigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float hyb_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float hyb_softplus(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// Element d of a vector whose first rot_dims entries are rotated by the row's angles (c, s: cos and sin of its rot_dims / 2
// pairs): the pair (first, second) becomes (first c - second s, second c + first s).  THA_ROT_INTERLEAVED pairs (2i, 2i + 1),
// THA_ROT_HALVES pairs (i, i + rot_dims / 2); entries from rot_dims on pass unchanged.
__device__ __forceinline__ float hyb_rotated(const float* src, int d, int rot_dims, int layout, const float* c, const float* s) {
  if (d >= rot_dims) return src[d];
  const int half = rot_dims >> 1;
  const bool first = layout == THA_ROT_HALVES ? d < half : !(d & 1);
  const int i = layout == THA_ROT_HALVES ? (first ? d : d - half) : d >> 1;
  const int partner = layout == THA_ROT_HALVES ? (first ? d + half : d - half) : d ^ 1;
  const float x = src[d], y = src[partner];
  return first ? x * c[i] - y * s[i] : x * c[i] + y * s[i];
}

// first float of the cache row of (slot, position t) in cache layer `layer` of a pool
__device__ __forceinline__ size_t hyb_kv_row(const tha_kv_t& kv, int slot, int t, int layer) {
  const int blk = kv.table[(size_t)slot * kv.table_stride + t / kv.block_size];
  return ((size_t)blk * kv.n_cache_layers + layer) * kv.block_size * kv.kv_dim + (size_t)(t % kv.block_size) * kv.kv_dim;
}
}  // namespace tha
