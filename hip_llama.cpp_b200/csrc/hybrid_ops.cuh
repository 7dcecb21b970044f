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
// What the attention kernels share beyond the causal block-of-positions rule.
// Visibility of key t for a query at p whose block of positions starts at `first`:
__device__ __forceinline__ bool hyb_attn_sees(const tha_attn_t& a, int t, int p, int first) {
  return t <= p && t >= first && (a.window <= 0 || p - t < a.window || t < a.keep_first);
}
// The key tiles (of 32, aligned to absolute multiples of 32) a block of queries at positions p_first..p_last walks: all from
// the tile of key_lo to the tile of p_last, except, under a window, the run of tiles that lie wholly between the kept first
// keys and the window of the block's first query.  Logical tile i of n: kt = i < n_a ? begin + 32 i : resume + 32 (i - n_a).
struct HybTiles { int begin, n_a, resume, n; };
__device__ __forceinline__ HybTiles hyb_attn_tiles(const tha_attn_t& a, int key_lo, int p_first, int p_last) {
  HybTiles t;
  t.begin = (key_lo / 32) * 32;
  t.n_a = 0;
  t.resume = t.begin;
  if (a.window > 0) {
    const int win_lo = max(key_lo, p_first - a.window + 1);
    const int keep_end = min(a.keep_first, p_last + 1);                                  // kept keys: [key_lo, keep_end)
    const int after_kept = keep_end > key_lo ? ((keep_end - 1) / 32 + 1) * 32 : t.begin;  // first tile past them
    const int wt = (win_lo / 32) * 32;
    if (wt > after_kept) { t.n_a = (after_kept - t.begin) / 32; t.resume = wt; }
  }
  t.n = t.n_a + (p_last - t.resume) / 32 + 1;
  return t;
}
// The end of a (query, head): with m, l the running maximum and sum, the factor the accumulator is multiplied by --
// 1 / (l + exp(sink - m)) in a form that cannot overflow, times the head's output gate.
__device__ __forceinline__ float hyb_attn_final_factor(const tha_attn_t& a, int h, float m, float l, const float* gate_row) {
  float f;
  if (a.sink) {
    const float sk = a.sink[h], M = fmaxf(m, sk), e = expf(m - M);
    f = e / (l * e + expf(sk - M));
  } else {
    f = 1.0f / l;
  }
  if (gate_row) f *= hyb_sigmoid(gate_row[h]);
  return f;
}
}  // namespace tha
