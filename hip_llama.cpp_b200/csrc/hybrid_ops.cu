// The mechanisms of the layer-program path (include/tha_hybrid.h), one kernel family each:
//   rmsnorm with an offset weight, the row-gathering / grouped linear map, rotary tables in float64, attention
//   preparation (rotate, unit-rms, cache write), softmax attention over a paged cache limited to the query's block of
//   positions, the matrix-memory scan, the short convolution with its tail, the gated-delta-rule scan, the top-k router
//   with its counting sort, and the clamped gated activation.
// All of them take ragged rows (tha_rows_t): what a row may see depends only on its own sequence, position, block table
// and state slot, never on where it sits in the batch.  Reductions run in a fixed order, so a position's result does
// not depend on how the prompt was cut or on what else is in the step.
#include <cuda_bf16.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "gemm_tc.h"
#include "hybrid_ops.cuh"
#include "tha_hybrid.h"

namespace tha {

// ------------------------------------------------------------------------------------------------------------------
// rmsnorm: one block per row
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void hyb_rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w, float w_offset,
                                   float eps, int width, const int* __restrict__ rows_idx) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows_idx ? rows_idx[r] : r) * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) { const float v = xr[i]; ss = fmaf(v, v, ss); }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) hyb_store(out + (size_t)r * width + i, xr[i] * inv * (w_offset + (w ? w[i] : 0.f)));
}

// dynamic tanh: tanh(alpha x) w + b, element by element (no mean, no variance)
template <typename T>
__global__ void hyb_dyt_kernel(T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                               float alpha, int width, const int* __restrict__ rows_idx) {
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows_idx ? rows_idx[r] : r) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) hyb_store(out + (size_t)r * width + i, fmaf(tanhf(alpha * xr[i]), w[i], b ? b[i] : 0.f));
}

// two dynamic-tanh norms of the same row in one pass (the two norms of a parallel block)
template <typename T>
__global__ void hyb_dyt2_kernel(T* __restrict__ out1, T* __restrict__ out2, const float* __restrict__ x, tha_norm_t n1, tha_norm_t n2, int width) {
  const int r = blockIdx.x;
  const float* xr = x + (size_t)r * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = xr[i];
    hyb_store(out1 + (size_t)r * width + i, fmaf(tanhf(n1.alpha * v), n1.w[i], n1.b ? n1.b[i] : 0.f));
    hyb_store(out2 + (size_t)r * width + i, fmaf(tanhf(n2.alpha * v), n2.w[i], n2.b ? n2.b[i] : 0.f));
  }
}

// layer norm: (x - mean) / sqrt(variance + eps) * w + b, the variance as the mean of the squared deviations (two passes
// over the row, which the block keeps in registers / L1); one block per row
template <typename T>
__global__ void hyb_layernorm_kernel(T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                     float eps, int width, const int* __restrict__ rows_idx) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows_idx ? rows_idx[r] : r) * width;
  float sum = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) sum += xr[i];
  const float mean = block_sum(sum, red) / (float)width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) { const float d = xr[i] - mean; ss = fmaf(d, d, ss); }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) hyb_store(out + (size_t)r * width + i, fmaf((xr[i] - mean) * inv, w[i], b ? b[i] : 0.f));
}

// ------------------------------------------------------------------------------------------------------------------
// linear: 64 x 64 output tile per block, 16-deep k slices through shared memory, 4 x 4 per thread, fp32 FMA in
// ascending k: the sum of an output element is the same whatever tile or group it lands in.
// ------------------------------------------------------------------------------------------------------------------
constexpr int LT = 64, LK = 16;

template <typename TA, typename TW>
__global__ void __launch_bounds__(256) hyb_linear_kernel(float* __restrict__ C, long long ldc, const TA* __restrict__ A, long long lda,
                                                         const int* __restrict__ a_rows, const TW* __restrict__ W,
                                                         long long w_group_stride, int M, int N, int K,
                                                         const int* __restrict__ group_off, int n_groups, long long a_zs, long long w_zs,
                                                         long long c_zs) {
  __shared__ float As[LK][LT + 4];
  __shared__ float Ws[LK][LT + 4];
  // blockIdx.z: one independent product per head (strides in elements), 0 strides otherwise
  A += (size_t)blockIdx.z * a_zs; W += (size_t)blockIdx.z * w_zs; C += (size_t)blockIdx.z * c_zs;
  // which group and which rows this block covers
  int g = 0, m0 = 0, m_end = M;
  if (group_off) {
    int tile = blockIdx.y, found = 0;
    for (g = 0; g < n_groups; g++) {
      const int lo = group_off[g], hi = group_off[g + 1];
      const int nt = (hi - lo + LT - 1) / LT;
      if (tile < nt) { m0 = lo + tile * LT; m_end = hi; found = 1; break; }
      tile -= nt;
    }
    if (!found) return;
  } else {
    m0 = blockIdx.y * LT;
    if (m0 >= M) return;
  }
  const int n0 = blockIdx.x * LT;
  const TW* Wg = W + (size_t)g * w_group_stride;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // tx: columns, ty: rows
  float acc[4][4] = {};
  // loader mapping: thread loads 4 elements of a row of A and of W per slice
  const int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;
  const int am = m0 + lr;
  const long long arow = am < m_end ? (long long)(a_rows ? a_rows[am] : am) : -1;
  const int wn = n0 + lr;
  for (int k0 = 0; k0 < K; k0 += LK) {
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const int k = k0 + lk + e;
      As[lk + e][lr] = (arow >= 0 && k < K) ? hyb_load(A + arow * lda + k) : 0.f;
      Ws[lk + e][lr] = (wn < N && k < K) ? hyb_load(Wg + (size_t)wn * K + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < LK; k++) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; i++) { a[i] = As[k][ty * 4 + i]; b[i] = Ws[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + ty * 4 + i;
    if (m >= m_end) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// the same map for bf16 x bf16 on the tensor cores, for the products the TMA-fed matmul of the bf16 path cannot take:
// rows gathered through an index list and one matrix per group of rows (the experts of a mixture).  64 x 64 tile, k
// slices of 32 through padded shared memory (global -> registers -> shared, the next slice in flight during the math),
// 4 warps of 32 x 32, mma.sync m16n8k16 with fp32 accumulators; k ascending, so an output element's sum does not depend
// on its tile or group.  Needs K % 8 == 0 and 16-byte aligned rows (128-bit loads).
// ------------------------------------------------------------------------------------------------------------------
constexpr int MK = 32, MKP = MK + 8;   // padded row: 80 bytes, conflict-free fragment reads

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__global__ void __launch_bounds__(128) hyb_linear_mma_kernel(float* __restrict__ C, long long ldc, const __nv_bfloat16* __restrict__ A,
                                                             long long lda, const int* __restrict__ a_rows,
                                                             const __nv_bfloat16* __restrict__ W, long long w_group_stride, int M, int N,
                                                             int K, const int* __restrict__ group_off, int n_groups, long long a_zs,
                                                             long long w_zs, long long c_zs) {
  __shared__ __align__(16) __nv_bfloat16 As[LT][MKP];
  __shared__ __align__(16) __nv_bfloat16 Ws[LT][MKP];
  A += (size_t)blockIdx.z * a_zs; W += (size_t)blockIdx.z * w_zs; C += (size_t)blockIdx.z * c_zs;
  int g = 0, m0 = 0, m_end = M;
  if (group_off) {
    int tile = blockIdx.y, found = 0;
    for (g = 0; g < n_groups; g++) {
      const int lo = group_off[g], hi = group_off[g + 1];
      const int nt = (hi - lo + LT - 1) / LT;
      if (tile < nt) { m0 = lo + tile * LT; m_end = hi; found = 1; break; }
      tile -= nt;
    }
    if (!found) return;
  } else {
    m0 = blockIdx.y * LT;
    if (m0 >= M) return;
  }
  const int n0 = blockIdx.x * LT;
  const __nv_bfloat16* Wg = W + (size_t)g * w_group_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
  // loader: 2 chunks of 8 values per thread and matrix; chunk id = threadIdx.x + 128 * u -> row = id / 4, k chunk = id % 4
  const __nv_bfloat16* a_src[2]; const __nv_bfloat16* w_src[2];
  int l_row[2], l_kc[2];
#pragma unroll
  for (int u = 0; u < 2; u++) {
    const int id = threadIdx.x + 128 * u;
    l_row[u] = id >> 2; l_kc[u] = (id & 3) * 8;
    const int am = m0 + l_row[u];
    a_src[u] = am < m_end ? A + (size_t)(a_rows ? a_rows[am] : am) * lda : nullptr;
    const int wr = n0 + l_row[u];
    w_src[u] = wr < N ? Wg + (size_t)wr * K : nullptr;
  }
  uint4 ra[2], rw[2];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int u = 0; u < 2; u++) {
      const int k = k0 + l_kc[u];
      ra[u] = (a_src[u] && k < K) ? *reinterpret_cast<const uint4*>(a_src[u] + k) : make_uint4(0, 0, 0, 0);
      rw[u] = (w_src[u] && k < K) ? *reinterpret_cast<const uint4*>(w_src[u] + k) : make_uint4(0, 0, 0, 0);
    }
  };
  float acc[2][4][4] = {};
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += MK) {
#pragma unroll
    for (int u = 0; u < 2; u++) {
      *reinterpret_cast<uint4*>(&As[l_row[u]][l_kc[u]]) = ra[u];
      *reinterpret_cast<uint4*>(&Ws[l_row[u]][l_kc[u]]) = rw[u];
    }
    __syncthreads();
    if (k0 + MK < K) fetch(k0 + MK);
#pragma unroll
    for (int kk = 0; kk < MK; kk += 16) {
      uint32_t af[2][4], bf[4][2];
      const int kc = kk + (lane & 3) * 2, rr = lane >> 2;
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const int r = wm + i * 16 + rr;
        af[i][0] = *reinterpret_cast<const uint32_t*>(&As[r][kc]);
        af[i][1] = *reinterpret_cast<const uint32_t*>(&As[r + 8][kc]);
        af[i][2] = *reinterpret_cast<const uint32_t*>(&As[r][kc + 8]);
        af[i][3] = *reinterpret_cast<const uint32_t*>(&As[r + 8][kc + 8]);
      }
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int n = wn + j * 8 + rr;
        bf[j][0] = *reinterpret_cast<const uint32_t*>(&Ws[n][kc]);
        bf[j][1] = *reinterpret_cast<const uint32_t*>(&Ws[n][kc + 8]);
      }
#pragma unroll
      for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) mma_bf16_16816(acc[i][j], af[i], bf[j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; i++)
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
      for (int v = 0; v < 4; v++) {
        const int m = m0 + wm + i * 16 + (lane >> 2) + (v >> 1) * 8;
        const int n = n0 + wn + j * 8 + (lane & 3) * 2 + (v & 1);
        if (m < m_end && n < N) C[(size_t)m * ldc + n] = acc[i][j][v];
      }
}

// ------------------------------------------------------------------------------------------------------------------
// rotary tables: float64 angles so that position * frequency keeps its low bits at long contexts
// ------------------------------------------------------------------------------------------------------------------
__global__ void hyb_rotary_kernel(const double* __restrict__ inv_freq, int half, float mag, const int* __restrict__ pos, int n_rows,
                                  float* __restrict__ cos_out, float* __restrict__ sin_out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_rows * half) return;
  const int r = i / half, c = i % half;
  double s, co;
  sincos((double)pos[r] * inv_freq[c], &s, &co);
  cos_out[i] = (float)(co * (double)mag);
  sin_out[i] = (float)(s * (double)mag);
}

// ------------------------------------------------------------------------------------------------------------------
// attention preparation: one block per row, one warp per head (query heads first, then key heads, then value heads)
// ------------------------------------------------------------------------------------------------------------------

__global__ void hyb_attn_prepare_kernel(tha_attn_t a, tha_rows_t rows, tha_kv_t kv, const float* __restrict__ proj, long long ldp,
                                        const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dims,
                                        float* __restrict__ q_out) {
  const int r = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int slot = rows.seq_slot[rows.row_seq[r]], t = rows.pos[r];
  const float* pr = proj + (size_t)r * ldp;
  const int half = rot_dims / 2;
  const size_t krow = hyb_kv_row(kv, slot, t, a.cache_layer);
  // a layer that reads another layer's cache rows prepares its queries only; key heads that share a value head write it once
  const int n_k = a.kv_shared ? 0 : a.kv_heads, n_v = a.kv_shared ? 0 : a.kv_heads / (a.v_share > 1 ? a.v_share : 1);
  // queries grow with the logarithm of their position, in steps of q_temp_every positions
  const float q_mult = a.q_temp_every > 0 ? 1.0f + a.q_temp_coef * logf((float)((t + 1) / a.q_temp_every + 1)) : 1.0f;
  for (int h = warp; h < a.heads + n_k + n_v; h += nwarps) {
    if (h >= a.heads + n_k) {   // a value head: plain copy
      const int g = h - a.heads - n_k;
      for (int e = lane; e < a.vdim; e += 32) kv.v_pool[krow + (size_t)g * a.vdim + e] = pr[a.o_v + g * a.vdim + e];
      continue;
    }
    const bool is_q = h < a.heads;
    const float* src = pr + (is_q ? a.o_q + h * a.dim : a.o_k + (h - a.heads) * a.dim);
    float* dst = is_q ? q_out + (size_t)r * a.heads * a.dim + (size_t)h * a.dim : kv.k_pool + krow + (size_t)(h - a.heads) * a.dim;
    // the first rot_dims entries rotated (pairs by the layout), the rest passed through
    const float* cr = cos_t + (size_t)r * half;
    const float* sr = sin_t + (size_t)r * half;
    float ss = 0.f;
    if (a.unit_rms) {
      for (int d = lane; d < a.dim; d += 32) { const float v = hyb_rotated(src, d, rot_dims, a.rot_layout, cr, sr); ss = fmaf(v, v, ss); }
      ss = warp_sum(ss);
    }
    const float inv = (a.unit_rms ? 1.0f / sqrtf(ss / (float)a.dim + a.eps) : 1.0f) * (is_q ? q_mult : 1.0f);
    for (int d = lane; d < a.dim; d += 32) dst[d] = hyb_rotated(src, d, rot_dims, a.rot_layout, cr, sr) * inv;
  }
}

// ------------------------------------------------------------------------------------------------------------------
// attention, prompts and decoding alike.  A block takes 16 (position, query head) pairs that share one key/value head:
// AP consecutive positions of one sequence x AG heads of the group (AG = min(group size, 16), AP = 16 / AG), so a key
// tile is read once for all of them.  Keys come in tiles of 32 aligned to absolute multiples of 32: whatever the step's
// cut, a position meets the same tiles in the same order and its running (max, sum, accumulator) takes the same values.
// Per tile: scores (warp = 4 pairs, lane = key), masked to the query's visible range [start of its block of `chunk`
// positions, own position], online softmax per pair, then P.V with lanes over value channels.
// ------------------------------------------------------------------------------------------------------------------
constexpr int ATT_PAIRS = 16, ATT_KEYS = 32, ATT_MAX_VC = 16;   // value channels per lane (template VC: 8 up to vdim 256, else 16)

template <typename T, int VC>
__global__ void __launch_bounds__(128) hyb_attn_kernel(tha_attn_t a, tha_rows_t rows, tha_kv_t kv, const float* __restrict__ q,
                                                       T* __restrict__ out, int AG, int AP, int splits, float* __restrict__ partial,
                                                       const float* __restrict__ gate, long long ldg) {
  extern __shared__ __align__(16) float sm[];
  const int D = a.dim, E = a.vdim, gsize = a.heads / a.kv_heads;
  const bool vec = ((D | E) & 3) == 0;         // 128-bit shared-memory reads: rows padded to keep them aligned and conflict-free
  const int KS = vec ? D + 4 : D + 1;
  float* Qs = sm;                              // [16][D]
  float* Ks = Qs + ATT_PAIRS * D;              // [32][KS]
  float* Vs = Ks + ATT_KEYS * KS;              // [32][E]
  float* Ps = Vs + ATT_KEYS * E;               // [16][32]
  // which sequence and which positions: tiles of AP rows per sequence, found by walking the sequences
  int seq = -1, r0 = 0, r_end = 0;
  {
    // the last tiles of a prompt see the most keys: they start first, so that the grid does not end on its longest blocks
    int tile = (int)(gridDim.x / splits) - 1 - (int)(blockIdx.x / splits);
    for (int s = 0; s < rows.n_seqs; s++) {
      const int lo = rows.seq_first[s], hi = rows.seq_first[s + 1];
      const int nt = (hi - lo + AP - 1) / AP;
      if (tile < nt) { seq = s; r0 = lo + tile * AP; r_end = min(hi, r0 + AP); break; }
      tile -= nt;
    }
    if (seq < 0) return;
  }
  const int g = blockIdx.y, part = blockIdx.z;
  const int gv = a.v_share > 1 ? g / a.v_share : g;   // the value head this key head reads
  const int slot = rows.seq_slot[seq];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int p_first = rows.pos[r0], p_last = p_first + (r_end - r0) - 1;
  // the block's pairs
  for (int i = threadIdx.x; i < ATT_PAIRS * D; i += blockDim.x) {
    const int pr = i / D, d = i - pr * D;
    const int r = r0 + pr / AG, hg = part * AG + pr % AG;
    Qs[i] = (r < r_end && hg < gsize) ? q[(size_t)r * a.heads * D + (size_t)(g * gsize + hg) * D + d] : 0.f;
  }
  int my_pos[4], my_first[4];
  bool my_ok[4];
  float m_run[4], l_run[4], acc[4][VC], my_scale[4];
#pragma unroll
  for (int rr = 0; rr < 4; rr++) {
    const int pr = warp * 4 + rr;
    const int r = r0 + pr / AG, hg = part * AG + pr % AG;
    my_ok[rr] = r < r_end && hg < gsize;
    my_pos[rr] = p_first + pr / AG;
    my_first[rr] = a.chunk > 0 ? (my_pos[rr] / a.chunk) * a.chunk : 0;
    my_scale[rr] = (a.head_scale && my_ok[rr]) ? a.head_scale[g * gsize + hg] : 1.0f;
    m_run[rr] = -INFINITY; l_run[rr] = 0.f;
#pragma unroll
    for (int c = 0; c < VC; c++) acc[rr][c] = 0.f;
  }
  const int key_lo = a.chunk > 0 ? (p_first / a.chunk) * a.chunk : 0;
  // with splits > 1 (few rows, long contexts) the key tiles are dealt to `splits` blocks in contiguous runs; each leaves
  // its running (max, sum, accumulator) in `partial` and hyb_attn_merge_kernel combines them in order
  const HybTiles tiles = hyb_attn_tiles(a, key_lo, p_first, p_last);
  int ti_begin = 0, ti_end = tiles.n;
  if (splits > 1) {
    const int per = (tiles.n + splits - 1) / splits, sp = blockIdx.x % splits;
    ti_begin = sp * per;
    ti_end = min(tiles.n, ti_begin + per);
  }
  for (int ti = ti_begin; ti < ti_end; ti++) {
    const int kt = ti < tiles.n_a ? tiles.begin + ATT_KEYS * ti : tiles.resume + ATT_KEYS * (ti - tiles.n_a);
    __syncthreads();   // the previous tile is consumed (and Qs is written, the first time)
    // a warp fetches 8 keys: all 8 table entries first, then the rows four at a time into registers before any of them
    // goes to shared memory, so that the loads are in flight together (a load followed by its own store waits for it)
    size_t krow[ATT_KEYS / 4];
#pragma unroll
    for (int jj = 0; jj < ATT_KEYS / 4; jj++) {
      const int t = kt + warp + 4 * jj;
      krow[jj] = (t <= p_last && t >= key_lo) ? hyb_kv_row(kv, slot, t, a.cache_layer) : (size_t)-1;
    }
#pragma unroll
    for (int which = 0; which < 2; which++) {
      const float* pool = which ? kv.v_pool : kv.k_pool;
      const int width = which ? E : D, stride = which ? E : KS;
      const int gh = which ? gv : g;
      float* dst = which ? Vs : Ks;
#pragma unroll
      for (int j0 = 0; j0 < ATT_KEYS / 4; j0 += 4) {
        float buf[4][VC];
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
          const bool live = krow[j0 + jj] != (size_t)-1;
          const float* src = pool + (live ? krow[j0 + jj] : 0) + (size_t)gh * width;
#pragma unroll
          for (int c = 0; c < VC; c++) buf[jj][c] = (live && lane + 32 * c < width) ? __ldg(src + lane + 32 * c) : 0.f;
        }
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
          const int j = warp + 4 * (j0 + jj);
#pragma unroll
          for (int c = 0; c < VC; c++)
            if (lane + 32 * c < width) dst[j * stride + lane + 32 * c] = buf[jj][c];
          if (width > 32 * VC) {   // wider key rows than the register buffer: the rest one by one
            const bool live = krow[j0 + jj] != (size_t)-1;
            const float* src = pool + (live ? krow[j0 + jj] : 0) + (size_t)gh * width;
            for (int d = lane + 32 * VC; d < width; d += 32) dst[j * stride + d] = live ? src[d] : 0.f;
          }
        }
      }
    }
    __syncthreads();
    float sc[4] = {0.f, 0.f, 0.f, 0.f};
    const float* kl = Ks + lane * KS;
    const float* q0 = Qs + (warp * 4) * D;
    if (vec) {
      const float4* k4 = reinterpret_cast<const float4*>(kl);
      const float4* qa = reinterpret_cast<const float4*>(q0);
      const int D4 = D >> 2;
      for (int d = 0; d < D4; d++) {
        const float4 kd = k4[d];
        sc[0] = dot4(qa[d], kd, sc[0]);
        sc[1] = dot4(qa[D4 + d], kd, sc[1]);
        sc[2] = dot4(qa[2 * D4 + d], kd, sc[2]);
        sc[3] = dot4(qa[3 * D4 + d], kd, sc[3]);
      }
    } else {
      for (int d = 0; d < D; d++) {
        const float kd = kl[d];
        sc[0] = fmaf(q0[d], kd, sc[0]);
        sc[1] = fmaf(q0[D + d], kd, sc[1]);
        sc[2] = fmaf(q0[2 * D + d], kd, sc[2]);
        sc[3] = fmaf(q0[3 * D + d], kd, sc[3]);
      }
    }
    const int t = kt + lane;
#pragma unroll
    for (int rr = 0; rr < 4; rr++) {
      const bool vis = my_ok[rr] && hyb_attn_sees(a, t, my_pos[rr], my_first[rr]);
      const float sv = vis ? sc[rr] * a.scale * my_scale[rr] : -INFINITY;
      const float m_new = fmaxf(m_run[rr], warp_max(sv));
      float p = 0.f, corr = 1.f;
      if (m_new > -INFINITY) {
        p = vis ? expf(sv - m_new) : 0.f;
        corr = expf(m_run[rr] - m_new);      // 0 when nothing was seen before
      }
      l_run[rr] = l_run[rr] * corr + warp_sum(p);
      m_run[rr] = m_new;
      Ps[(warp * 4 + rr) * ATT_KEYS + lane] = p;
#pragma unroll
      for (int c = 0; c < VC; c++) acc[rr][c] *= corr;
    }
    __syncwarp();
    const float* pw = Ps + (warp * 4) * ATT_KEYS;
    if (vec) {
      const float4* p4 = reinterpret_cast<const float4*>(pw);
      for (int j4 = 0; j4 < ATT_KEYS / 4; j4++) {
        const float4 pa = p4[j4], pb = p4[ATT_KEYS / 4 + j4], pc = p4[2 * (ATT_KEYS / 4) + j4], pd = p4[3 * (ATT_KEYS / 4) + j4];
        const float P0[4] = {pa.x, pa.y, pa.z, pa.w}, P1[4] = {pb.x, pb.y, pb.z, pb.w}, P2[4] = {pc.x, pc.y, pc.z, pc.w},
                    P3[4] = {pd.x, pd.y, pd.z, pd.w};
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
          const float* vrow = Vs + (4 * j4 + jj) * E;
#pragma unroll
          for (int c = 0; c < VC; c++) {
            const int e = lane + 32 * c;
            if (e < E) {
              const float v = vrow[e];
              acc[0][c] = fmaf(P0[jj], v, acc[0][c]);
              acc[1][c] = fmaf(P1[jj], v, acc[1][c]);
              acc[2][c] = fmaf(P2[jj], v, acc[2][c]);
              acc[3][c] = fmaf(P3[jj], v, acc[3][c]);
            }
          }
        }
      }
    } else {
      for (int j = 0; j < ATT_KEYS; j++) {
        const float p0 = pw[j], p1 = pw[ATT_KEYS + j], p2 = pw[2 * ATT_KEYS + j], p3 = pw[3 * ATT_KEYS + j];
#pragma unroll
        for (int c = 0; c < VC; c++) {
          const int e = lane + 32 * c;
          if (e < E) {
            const float v = Vs[j * E + e];
            acc[0][c] = fmaf(p0, v, acc[0][c]);
            acc[1][c] = fmaf(p1, v, acc[1][c]);
            acc[2][c] = fmaf(p2, v, acc[2][c]);
            acc[3][c] = fmaf(p3, v, acc[3][c]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int rr = 0; rr < 4; rr++) {
    if (!my_ok[rr]) continue;
    const int pr = warp * 4 + rr;
    const int r = r0 + pr / AG, h = g * gsize + part * AG + pr % AG;
    if (splits > 1) {
      float* dst = partial + (((size_t)(blockIdx.x % splits) * rows.n_rows + r) * a.heads + h) * (E + 2);
#pragma unroll
      for (int c = 0; c < VC; c++) {
        const int e = lane + 32 * c;
        if (e < E) dst[e] = acc[rr][c];
      }
      if (lane == 0) { dst[E] = m_run[rr]; dst[E + 1] = l_run[rr]; }
      continue;
    }
    const float inv = hyb_attn_final_factor(a, h, m_run[rr], l_run[rr], gate ? gate + (size_t)r * ldg : nullptr);
#pragma unroll
    for (int c = 0; c < VC; c++) {
      const int e = lane + 32 * c;
      if (e < E) {
        const size_t at = (size_t)r * a.heads * E + (size_t)h * E + e;
        if (a.out_f32) reinterpret_cast<float*>(out)[at] = acc[rr][c] * inv;
        else hyb_store(out + at, acc[rr][c] * inv);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// the same attention on the tensor cores, for the bf16 number format and heads of up to 128 channels (multiples of 16 /
// 8): a block takes 64 (position, query head) pairs of one K/V head, each of its 4 warps 16 of them.  Per tile of 32 keys
// (aligned to absolute multiples of 32 as above): K rows and V rows go to shared memory as bf16, both row-major; a warp
// computes its 16 x 32 scores with mma.sync m16n8k16 (q as the A operand from registers), scales and masks them in fp32,
// keeps the online softmax of its rows among the four lanes that share a row, rounds the weights to bf16 (the row sums
// add the rounded weights, so that they still sum to one) and multiplies them with V straight from the score registers:
// two adjacent 8-key score tiles are one 16-deep A operand.  No exchange between warps; accumulators fp32.
// ------------------------------------------------------------------------------------------------------------------
constexpr int AM_PAIRS = 64, AM_MAXD = 128;

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

template <bool EXACT>
__global__ void __launch_bounds__(128, 3) hyb_attn_mma_kernel(tha_attn_t a, tha_rows_t rows, tha_kv_t kv, const float* __restrict__ q,
                                                           __nv_bfloat16* __restrict__ out, int AG, int AP, int splits,
                                                           float* __restrict__ partial, const float* __restrict__ gate, long long ldg) {
  extern __shared__ __align__(16) unsigned char smraw[];
  const int D = a.dim, E = a.vdim, gsize = a.heads / a.kv_heads;
  const int KS = D + 8, VS = E + 8;                      // padded rows: conflict-free fragment and ldmatrix reads
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smraw);   // [32][KS]
  __nv_bfloat16* Vs = Ks + ATT_KEYS * KS;                        // [32][VS], row-major like the cache: transposed on the way out
  const unsigned vs_base = (unsigned)__cvta_generic_to_shared(Vs);
  int seq = -1, r0 = 0, r_end = 0;
  {
    // the last tiles of a prompt see the most keys: they start first, so that the grid does not end on its longest blocks
    int tile = (int)(gridDim.x / splits) - 1 - (int)(blockIdx.x / splits);
    for (int s = 0; s < rows.n_seqs; s++) {
      const int lo = rows.seq_first[s], hi = rows.seq_first[s + 1];
      const int nt = (hi - lo + AP - 1) / AP;
      if (tile < nt) { seq = s; r0 = lo + tile * AP; r_end = min(hi, r0 + AP); break; }
      tile -= nt;
    }
    if (seq < 0) return;
  }
  const int g = blockIdx.y, part = blockIdx.z;
  const int gv = a.v_share > 1 ? g / a.v_share : g;   // the value head this key head reads
  const int slot = rows.seq_slot[seq];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int p_first = rows.pos[r0], p_last = p_first + (r_end - r0) - 1;
  const int lr = lane >> 2, lc = (lane & 3) * 2;
  // this lane's two rows (pairs): A = 16 * warp + lr, B = A + 8
  int row_r[2], row_h[2], row_pos[2], row_first[2];
  bool row_ok[2];
  float row_scale[2];
#pragma unroll
  for (int x = 0; x < 2; x++) {
    const int pr = warp * 16 + lr + 8 * x;
    const int pp = pr / AG, hg = part * AG + pr % AG;
    row_r[x] = r0 + pp;
    row_h[x] = g * gsize + hg;
    row_ok[x] = pp < AP && row_r[x] < r_end && hg < gsize;
    row_pos[x] = p_first + pp;
    row_first[x] = a.chunk > 0 ? (row_pos[x] / a.chunk) * a.chunk : 0;
    row_scale[x] = (a.head_scale && row_ok[x]) ? a.head_scale[row_h[x]] : 1.0f;
  }
  // q fragments: [k step][4]
  uint32_t qf[AM_MAXD / 16][4];
#pragma unroll
  for (int ks = 0; ks < AM_MAXD / 16; ks++) {
#pragma unroll
    for (int x = 0; x < 2; x++) {
      const float* qr = q + (size_t)row_r[x] * a.heads * D + (size_t)row_h[x] * D;
      const bool ok = row_ok[x] && 16 * ks < D;
      qf[ks][x] = ok ? pack_bf16(qr[16 * ks + lc], qr[16 * ks + lc + 1]) : 0u;
      qf[ks][2 + x] = ok ? pack_bf16(qr[16 * ks + 8 + lc], qr[16 * ks + 8 + lc + 1]) : 0u;
    }
  }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float oacc[AM_MAXD / 8][4];
#pragma unroll
  for (int n = 0; n < AM_MAXD / 8; n++)
#pragma unroll
    for (int v = 0; v < 4; v++) oacc[n][v] = 0.f;
  const int key_lo = a.chunk > 0 ? (p_first / a.chunk) * a.chunk : 0;
  const HybTiles tiles = hyb_attn_tiles(a, key_lo, p_first, p_last);
  int ti_begin = 0, ti_end = tiles.n;
  if (splits > 1) {
    const int per = (tiles.n + splits - 1) / splits, sp = blockIdx.x % splits;
    ti_begin = sp * per;
    ti_end = min(tiles.n, ti_begin + per);
  }
  // cache rows start on 16-byte boundaries when the pool's row pitch and the heads' offsets are multiples of four floats
  const bool vec4 = (kv.kv_dim & 3) == 0 && ((D | E) & 3) == 0 && ((reinterpret_cast<size_t>(kv.k_pool) | reinterpret_cast<size_t>(kv.v_pool)) & 15) == 0;
  for (int ti = ti_begin; ti < ti_end; ti++) {
    const int kt = ti < tiles.n_a ? tiles.begin + ATT_KEYS * ti : tiles.resume + ATT_KEYS * (ti - tiles.n_a);
    __syncthreads();
    // stage the tile: a warp takes 8 keys, four at a time through registers
    size_t krow[ATT_KEYS / 4];
#pragma unroll
    for (int jj = 0; jj < ATT_KEYS / 4; jj++) {
      const int t = kt + warp + 4 * jj;
      krow[jj] = (t <= p_last && t >= key_lo) ? hyb_kv_row(kv, slot, t, a.cache_layer) : (size_t)-1;
    }
    if (vec4) {
      // 16-byte aligned cache rows: a lane takes four channels of a row in one 128-bit load (eight rows in flight) and leaves
      // them as four bf16 in one 64-bit store
#pragma unroll
      for (int which = 0; which < 2; which++) {
        const float* pool = which ? kv.v_pool : kv.k_pool;
        const int width4 = (which ? E : D) >> 2;
        float4 buf[ATT_KEYS / 4];
#pragma unroll
        for (int jj = 0; jj < ATT_KEYS / 4; jj++) {
          const bool live = krow[jj] != (size_t)-1 && lane < width4;
          const float4* src = reinterpret_cast<const float4*>(pool + (live ? krow[jj] : 0) + (size_t)(which ? gv : g) * (width4 << 2));
          buf[jj] = live ? __ldg(src + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (lane < width4) {
#pragma unroll
          for (int jj = 0; jj < ATT_KEYS / 4; jj++) {
            const int j = warp + 4 * jj;
            uint2 pk;
            pk.x = pack_bf16(buf[jj].x, buf[jj].y);
            pk.y = pack_bf16(buf[jj].z, buf[jj].w);
            *reinterpret_cast<uint2*>((which ? Vs + j * VS : Ks + j * KS) + 4 * lane) = pk;
          }
        }
      }
    } else {
#pragma unroll
    for (int which = 0; which < 2; which++) {
      const float* pool = which ? kv.v_pool : kv.k_pool;
      const int width = which ? E : D;
      const int gh = which ? gv : g;
#pragma unroll
      for (int j0 = 0; j0 < ATT_KEYS / 4; j0 += 4) {
        float buf[4][AM_MAXD / 32];
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
          const bool live = krow[j0 + jj] != (size_t)-1;
          const float* src = pool + (live ? krow[j0 + jj] : 0) + (size_t)gh * width;
#pragma unroll
          for (int c = 0; c < AM_MAXD / 32; c++) buf[jj][c] = (live && lane + 32 * c < width) ? __ldg(src + lane + 32 * c) : 0.f;
        }
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
          const int j = warp + 4 * (j0 + jj);
#pragma unroll
          for (int c = 0; c < AM_MAXD / 32; c++) {
            const int d = lane + 32 * c;
            if (d < width) {
              if (which) Vs[j * VS + d] = __float2bfloat16_rn(buf[jj][c]);
              else Ks[j * KS + d] = __float2bfloat16_rn(buf[jj][c]);
            }
          }
        }
      }
    }
    }
    __syncthreads();
    // scores of this warp's 16 pairs against the 32 keys
    float sacc[4][4];
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
      for (int v = 0; v < 4; v++) sacc[j][v] = 0.f;
#pragma unroll
    for (int ks = 0; ks < AM_MAXD / 16; ks++) {
      if (16 * ks < D) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
          uint32_t b[2];
          const __nv_bfloat16* kr = Ks + (8 * j + lr) * KS + 16 * ks + lc;
          b[0] = *reinterpret_cast<const uint32_t*>(kr);
          b[1] = *reinterpret_cast<const uint32_t*>(kr + 8);
          mma_bf16_16816(sacc[j], qf[ks], b);
        }
      }
    }
    // scale, mask, online softmax of rows A (values 0, 1 of every score tile) and B (values 2, 3)
    uint32_t pa[2][4], pl[2][4];   // the weights as A operands: rounded to bf16, and (EXACT) what the rounding left over
#pragma unroll
    for (int x = 0; x < 2; x++) {
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; j++)
#pragma unroll
        for (int y = 0; y < 2; y++) {
          const int t = kt + 8 * j + lc + y;
          const bool vis = row_ok[x] && hyb_attn_sees(a, t, row_pos[x], row_first[x]);
          const float sv = vis ? sacc[j][2 * x + y] * a.scale * row_scale[x] : -INFINITY;
          sacc[j][2 * x + y] = sv;
          mx = fmaxf(mx, sv);
        }
      mx = fmaxf(mx, __shfl_xor_sync(THA_FULL_MASK, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(THA_FULL_MASK, mx, 2));
      const float m_new = fmaxf(m_run[x], mx);
      const float corr = m_new > -INFINITY ? expf(m_run[x] - m_new) : 1.f;
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float p0 = 0.f, p1 = 0.f;
        if (m_new > -INFINITY) { p0 = expf(sacc[j][2 * x] - m_new); p1 = expf(sacc[j][2 * x + 1] - m_new); }   // exp(-inf) = 0 for masked keys
        const __nv_bfloat162 pr = __floats2bfloat162_rn(p0, p1);
        if (EXACT) {   // hi + lo carry 16 mantissa bits of the fp32 weight; the sum adds the fp32 weights themselves
          sum += p0 + p1;
          pl[j >> 1][(j & 1) * 2 + x] = pack_bf16(p0 - __low2float(pr), p1 - __high2float(pr));
        } else {
          sum += __low2float(pr) + __high2float(pr);
        }
        pa[j >> 1][(j & 1) * 2 + x] = *reinterpret_cast<const uint32_t*>(&pr);
      }
      sum += __shfl_xor_sync(THA_FULL_MASK, sum, 1);
      sum += __shfl_xor_sync(THA_FULL_MASK, sum, 2);
      l_run[x] = l_run[x] * corr + sum;
      m_run[x] = m_new;
#pragma unroll
      for (int n = 0; n < AM_MAXD / 8; n++) { oacc[n][2 * x] *= corr; oacc[n][2 * x + 1] *= corr; }
    }
    // weights times values: two k steps of 16 keys, two channel tiles per ldmatrix.  Values [key][channel] row-major,
    // transposed on the way: lanes 0..15 name the rows of keys 16 t2 + (lane & 15) at this channel tile, lanes 16..31 the same
    // keys at the next one (an odd last tile reads its own twice)
#pragma unroll
    for (int n = 0; n < AM_MAXD / 8; n += 2) {
      if (8 * n < E) {
        const bool two = 8 * (n + 1) < E;
#pragma unroll
        for (int t2 = 0; t2 < 2; t2++) {
          uint32_t vf[4];
          const int ch = 8 * n + ((two && lane >= 16) ? 8 : 0);
          const unsigned addr = vs_base + (unsigned)(((16 * t2 + (lane & 15)) * VS + ch) * sizeof(__nv_bfloat16));
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                       : "=r"(vf[0]), "=r"(vf[1]), "=r"(vf[2]), "=r"(vf[3]) : "r"(addr));
          const uint32_t v0[2] = {vf[0], vf[1]}, v1[2] = {vf[2], vf[3]};
          mma_bf16_16816(oacc[n], pa[t2], v0);
          if (EXACT) mma_bf16_16816(oacc[n], pl[t2], v0);
          if (two) {
            mma_bf16_16816(oacc[n + 1], pa[t2], v1);
            if (EXACT) mma_bf16_16816(oacc[n + 1], pl[t2], v1);
          }
        }
      }
    }
  }
#pragma unroll
  for (int x = 0; x < 2; x++) {
    if (!row_ok[x]) continue;
    if (splits > 1) {
      float* dst = partial + (((size_t)(blockIdx.x % splits) * rows.n_rows + row_r[x]) * a.heads + row_h[x]) * (E + 2);
#pragma unroll
      for (int n = 0; n < AM_MAXD / 8; n++)
        if (8 * n < E) { dst[8 * n + lc] = oacc[n][2 * x]; dst[8 * n + lc + 1] = oacc[n][2 * x + 1]; }
      if ((lane & 3) == 0) { dst[E] = m_run[x]; dst[E + 1] = l_run[x]; }
      continue;
    }
    const float inv = hyb_attn_final_factor(a, row_h[x], m_run[x], l_run[x], gate ? gate + (size_t)row_r[x] * ldg : nullptr);
    if (a.out_f32) {
      float* dst = reinterpret_cast<float*>(out) + (size_t)row_r[x] * a.heads * E + (size_t)row_h[x] * E;
#pragma unroll
      for (int n = 0; n < AM_MAXD / 8; n++)
        if (8 * n < E) *reinterpret_cast<float2*>(dst + 8 * n + lc) = make_float2(oacc[n][2 * x] * inv, oacc[n][2 * x + 1] * inv);
      continue;
    }
    __nv_bfloat16* dst = out + (size_t)row_r[x] * a.heads * E + (size_t)row_h[x] * E;
#pragma unroll
    for (int n = 0; n < AM_MAXD / 8; n++)
      if (8 * n < E) *reinterpret_cast<__nv_bfloat162*>(dst + 8 * n + lc) = __floats2bfloat162_rn(oacc[n][2 * x] * inv, oacc[n][2 * x + 1] * inv);
  }
}

// the splits of a (row, head) in ascending key order: out = sum_s acc_s e^(m_s - M) / sum_s l_s e^(m_s - M); a warp each
template <typename T>
__global__ void hyb_attn_merge_kernel(T* __restrict__ out, const float* __restrict__ partial, int n_rows, int heads, int E, int splits,
                                      tha_attn_t a, const float* __restrict__ gate, long long ldg) {
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= n_rows * heads) return;
  const size_t stride = (size_t)n_rows * heads * (E + 2);
  const float* p0 = partial + (size_t)idx * (E + 2);
  float M = -INFINITY;
  for (int s = 0; s < splits; s++) M = fmaxf(M, p0[s * stride + E]);
  float L = 0.f;
  for (int s = 0; s < splits; s++) { const float ms = p0[s * stride + E]; if (ms > -INFINITY) L += p0[s * stride + E + 1] * expf(ms - M); }
  // lane s keeps split s's factor (at most 16 splits); splits that saw nothing have factor 0 and are not read
  float w = 0.f;
  if (lane < splits) { const float ms = p0[lane * stride + E]; w = ms > -INFINITY ? expf(ms - M) : 0.f; }
  const int row = idx / heads, head = idx - row * heads;
  const float fin = hyb_attn_final_factor(a, head, M, L, gate ? gate + (size_t)row * ldg : nullptr);
  // every lane walks every group of 32 channels (the shuffles need the whole warp), also where E is not a multiple of 32
  for (int e0 = 0; e0 < E; e0 += 32) {
    const int e = e0 + lane;
    float o = 0.f;
    for (int s = 0; s < splits; s++) { const float ws = __shfl_sync(THA_FULL_MASK, w, s); if (ws > 0.f && e < E) o = fmaf(p0[s * stride + e], ws, o); }
    if (e < E) hyb_store(out + (size_t)idx * E + e, o * fin);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// matrix memory: one block per (sequence, head); S [dim, vdim], n [dim] in shared memory, tokens in order.
// ------------------------------------------------------------------------------------------------------------------


// The scalar arithmetic of the gates does not depend on the state, so it runs for all rows at once before the scans and
// in place: the two gate columns of the stacked projection become the log input gate cap * tanh((z + b) / cap) and the log
// forget gate logsigmoid(cap * tanh((z + b) / cap)); for the delta rule the raw step sizes become the decays
// exp(-exp(A_log) * softplus(z + dt_bias)) and the raw write strength becomes sigmoid(z).
__global__ void hyb_mem_gates_kernel(float* __restrict__ proj, long long ldp, int n_rows, int heads, int o_i, int o_f,
                                     const float* __restrict__ b_i, const float* __restrict__ b_f, float cap) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_rows * heads) return;
  const int r = idx / heads, h = idx - r * heads;
  float* pr = proj + (size_t)r * ldp;
  pr[o_i + h] = hyb_softcap(pr[o_i + h] + b_i[h], cap);
  pr[o_f + h] = hyb_logsigmoid(hyb_softcap(pr[o_f + h] + b_f[h], cap));
}
__global__ void hyb_delta_gates_kernel(float* __restrict__ dt, float* __restrict__ proj, long long ldp, int n_rows, int heads, int D, int o_b,
                                       const float* __restrict__ a_log, const float* __restrict__ dt_bias) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)n_rows * heads * D) return;
  const int hd = (int)(idx % ((size_t)heads * D)), h = hd / D;
  dt[idx] = expf(-expf(a_log[h]) * hyb_softplus(dt[idx] + dt_bias[hd]));
  if (hd % D == 0) { float* b = proj + (idx / ((size_t)heads * D)) * ldp + o_b + h; *b = hyb_sigmoid(*b); }
}

// The state's value columns are independent of each other (column e of S only ever meets v[e]), so a head is cut into
// slices of SC columns, one block each: block (sequence, head, slice) keeps S[:, slice] in shared memory, its own copy of
// n and m, and walks the sequence's rows in order.  Thread (part, e) owns the rows d = part, part + parts, ... of column e:
// it updates them and accumulates its share of S^T q in the same pass.  The inputs of the next token are fetched while
// the current one is computed, and live in alternating buffers: two barriers per token.
// Output: o / max(|n.q|, exp(-m)) per (row, head, column) in fp32; the head norm and the output gate follow in
// hyb_head_gate_kernel, which needs all columns of a head.
constexpr int SCAN_THREADS = 256;

__global__ void __launch_bounds__(SCAN_THREADS) hyb_mem_scan_kernel(tha_mem_t m, tha_rows_t rows, tha_state_store_t st,
                                                                    const float* __restrict__ proj, long long ldp, float* __restrict__ o_raw, int SC) {
  extern __shared__ float sm[];
  const int s = blockIdx.x, h = blockIdx.y, e0 = blockIdx.z * SC;
  const int D = m.dim, E = m.vdim, nt = SCAN_THREADS;
  const int ec = min(SC, E - e0);
  const int parts = nt / SC;
  float* S = sm;                    // [D][SC]
  float* nv = S + D * SC;           // [D]
  float* in = nv + D;               // 2 x (q [D] | k [D] | v [SC] | ig | fg)
  const int in_stride = 2 * D + SC + 2;
  float* part = in + 2 * in_stride; // [parts][SC]
  float* gstate = st.base + (size_t)rows.seq_slot[s] * st.slot_floats + m.state_off + (size_t)h * ((size_t)D * E + D + 1);
  for (int i = threadIdx.x; i < D * SC; i += nt) { const int d = i / SC, e = i - d * SC; S[i] = e < ec ? gstate[(size_t)d * E + e0 + e] : 0.f; }
  for (int i = threadIdx.x; i < D; i += nt) nv[i] = gstate[(size_t)D * E + i];
  float mrun = gstate[(size_t)D * E + D];
  const float qscale = 1.0f / sqrtf((float)D);
  const int r_begin = rows.seq_first[s], r_end = rows.seq_first[s + 1];
  // element i of a token's inputs: q, k, v slice, the two raw gates
  auto fetch = [&](int r, int i) -> float {
    const float* pr = proj + (size_t)r * ldp;
    if (i < D) return pr[m.o_q + h * D + i] * qscale;
    if (i < 2 * D) return pr[m.o_k + h * D + (i - D)];
    if (i < 2 * D + SC) return (i - 2 * D) < ec ? pr[m.o_v + h * E + e0 + (i - 2 * D)] : 0.f;
    return i == 2 * D + SC ? pr[m.o_i + h] : pr[m.o_f + h];   // the log gates (hyb_mem_gates_kernel)
  };
  constexpr int PF = 4;             // prefetch registers per thread: up to 1024 inputs per token
  float pf[PF];
#pragma unroll
  for (int u = 0; u < PF; u++) { const int i = threadIdx.x + u * nt; pf[u] = (i < in_stride && r_begin < r_end) ? fetch(r_begin, i) : 0.f; }
  const int pe = threadIdx.x % SC, pp = threadIdx.x / SC;
  for (int r = r_begin; r < r_end; r++) {
    float* cur = in + ((r - r_begin) & 1) * in_stride;
#pragma unroll
    for (int u = 0; u < PF; u++) { const int i = threadIdx.x + u * nt; if (i < in_stride) cur[i] = pf[u]; }
    for (int i = threadIdx.x + PF * nt; i < in_stride; i += nt) cur[i] = fetch(r, i);   // very wide heads: the rest, unprefetched
    if (r + 1 < r_end) {
#pragma unroll
      for (int u = 0; u < PF; u++) { const int i = threadIdx.x + u * nt; if (i < in_stride) pf[u] = fetch(r + 1, i); }
    }
    __syncthreads();
    const float* sq = cur; const float* sk = cur + D; const float* sv = cur + 2 * D;
    const float ig = cur[2 * D + SC], fg = cur[2 * D + SC + 1];
    const float mnew = fmaxf(fg + mrun, ig);
    const float a = expf(fg + mrun - mnew), b = expf(ig - mnew);
    mrun = mnew;
    if (pp < parts) {
      const float bv = b * sv[pe];
      float acc = 0.f;
      for (int d = pp; d < D; d += parts) { const float v = fmaf(a, S[d * SC + pe], sk[d] * bv); S[d * SC + pe] = v; acc = fmaf(v, sq[d], acc); }
      part[pp * SC + pe] = acc;
    }
    for (int i = threadIdx.x; i < D; i += nt) nv[i] = fmaf(a, nv[i], b * sk[i]);
    __syncthreads();
    if (threadIdx.x < 32) {          // one warp finishes the token: n.q, the column sums, the division
      float nq = 0.f;
      for (int i = threadIdx.x; i < D; i += 32) nq = fmaf(nv[i], sq[i], nq);
      nq = warp_sum(nq);
      const float den = fmaxf(fabsf(nq), expf(-mrun)) + 1e-6f;
      for (int e = threadIdx.x; e < ec; e += 32) {
        float acc = 0.f;
        for (int p = 0; p < parts; p++) acc += part[p * SC + e];
        o_raw[(size_t)r * m.heads * E + (size_t)h * E + e0 + e] = acc / den;
      }
    }
    // no barrier here: the next token writes the other input buffer, and `part` is rewritten only after its barrier
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D * SC; i += nt) { const int d = i / SC, e = i - d * SC; if (e < ec) gstate[(size_t)d * E + e0 + e] = S[i]; }
  if (blockIdx.z == 0) {
    for (int i = threadIdx.x; i < D; i += nt) gstate[(size_t)D * E + i] = nv[i];
    if (threadIdx.x == 0) gstate[(size_t)D * E + D] = mrun;
  }
}

// The same two recurrences with the state in REGISTERS, for head sizes up to 256 key channels: a warp owns SCW value
// columns, lane l the key channels l, l + 32, ... of those columns.  Nothing is shared between warps, so a token costs no
// block barrier: the column sums S^T q (and S^T k) are warp shuffles, the next token's inputs are fetched a token ahead.
constexpr int SCW = 2, SCAN_WARPS = 4, SCAN_AHEAD = 4;

template <int RPL>
__global__ void __launch_bounds__(32 * SCAN_WARPS) hyb_mem_scan_warp_kernel(tha_mem_t m, tha_rows_t rows, tha_state_store_t st,
                                                                            const float* __restrict__ proj, long long ldp,
                                                                            float* __restrict__ o_raw) {
  const int s = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int D = m.dim, E = m.vdim;
  const int e0 = (blockIdx.z * SCAN_WARPS + warp) * SCW;
  if (e0 >= E) return;
  float* gstate = st.base + (size_t)rows.seq_slot[s] * st.slot_floats + m.state_off + (size_t)h * ((size_t)D * E + D + 1);
  float S[RPL][SCW], nv[RPL];
#pragma unroll
  for (int i = 0; i < RPL; i++) {
    const int d = lane + 32 * i;
    nv[i] = d < D ? gstate[(size_t)D * E + d] : 0.f;
#pragma unroll
    for (int c = 0; c < SCW; c++) S[i][c] = (d < D && e0 + c < E) ? gstate[(size_t)d * E + e0 + c] : 0.f;
  }
  float mrun = gstate[(size_t)D * E + D];
  const float qscale = 1.0f / sqrtf((float)D);
  const int r_begin = rows.seq_first[s], r_end = rows.seq_first[s + 1];
  // a token's inputs are loaded SCAN_AHEAD tokens before they are used (a ring of register sets, the loop unrolled over
  // it), so that a load has several tokens' worth of arithmetic to arrive in
  struct In { float q[RPL], k[RPL], v[SCW], gi, gf; };
  In ring[SCAN_AHEAD];
  auto fetch = [&](int r, In& in) {
    const float* pr = proj + (size_t)r * ldp;
#pragma unroll
    for (int i = 0; i < RPL; i++) {
      const int d = lane + 32 * i;
      in.q[i] = d < D ? pr[m.o_q + h * D + d] : 0.f;
      in.k[i] = d < D ? pr[m.o_k + h * D + d] : 0.f;
    }
#pragma unroll
    for (int c = 0; c < SCW; c++) in.v[c] = e0 + c < E ? pr[m.o_v + h * E + e0 + c] : 0.f;
    in.gi = pr[m.o_i + h];
    in.gf = pr[m.o_f + h];
  };
#pragma unroll
  for (int u = 0; u < SCAN_AHEAD; u++)
    if (r_begin + u < r_end) fetch(r_begin + u, ring[u]);
  // one token; `refill` (a row, or -1) is what the token's ring entry is loaded with once its values are taken
  auto token = [&](int r, In& in, int refill) {
    float cq[RPL], ck[RPL], cv[SCW];
#pragma unroll
    for (int i = 0; i < RPL; i++) { cq[i] = in.q[i] * qscale; ck[i] = in.k[i]; }
#pragma unroll
    for (int c = 0; c < SCW; c++) cv[c] = in.v[c];
    const float ig = in.gi, fg = in.gf;   // the log gates (hyb_mem_gates_kernel)
    if (refill >= 0) fetch(refill, in);
    const float mnew = fmaxf(fg + mrun, ig);
    const float a = expf(fg + mrun - mnew), b = expf(ig - mnew);
    mrun = mnew;
    float nq = 0.f, acc[SCW];
#pragma unroll
    for (int c = 0; c < SCW; c++) acc[c] = 0.f;
#pragma unroll
    for (int i = 0; i < RPL; i++) {
      nv[i] = fmaf(a, nv[i], b * ck[i]);
      nq = fmaf(nv[i], cq[i], nq);
#pragma unroll
      for (int c = 0; c < SCW; c++) {
        S[i][c] = fmaf(a, S[i][c], ck[i] * (b * cv[c]));
        acc[c] = fmaf(S[i][c], cq[i], acc[c]);
      }
    }
    nq = warp_sum(nq);
    const float den = fmaxf(fabsf(nq), expf(-mnew)) + 1e-6f;
#pragma unroll
    for (int c = 0; c < SCW; c++) {
      const float o = warp_sum(acc[c]);
      if (lane == c && e0 + c < E) o_raw[(size_t)r * m.heads * E + (size_t)h * E + e0 + c] = o / den;
    }
  };
  // whole groups without a branch between their tokens (the refill row is clamped instead of tested), so that one
  // token's shuffles and stores can be scheduled under the next token's arithmetic; then the ragged end
  int rb = r_begin;
  for (; rb + SCAN_AHEAD <= r_end; rb += SCAN_AHEAD) {
#pragma unroll
    for (int u = 0; u < SCAN_AHEAD; u++) token(rb + u, ring[u], min(rb + u + SCAN_AHEAD, r_end - 1));
  }
#pragma unroll
  for (int u = 0; u < SCAN_AHEAD; u++)
    if (rb + u < r_end) token(rb + u, ring[u], -1);
#pragma unroll
  for (int i = 0; i < RPL; i++) {
    const int d = lane + 32 * i;
    if (d >= D) continue;
#pragma unroll
    for (int c = 0; c < SCW; c++)
      if (e0 + c < E) gstate[(size_t)d * E + e0 + c] = S[i][c];
    if (e0 == 0) gstate[(size_t)D * E + d] = nv[i];
  }
  if (e0 == 0 && lane == 0) gstate[(size_t)D * E + D] = mrun;
}

template <int RPL>
__global__ void __launch_bounds__(32 * SCAN_WARPS) hyb_delta_scan_warp_kernel(tha_delta_t dl, tha_rows_t rows, tha_state_store_t st,
                                                                              const float* __restrict__ qkv, const float* __restrict__ proj,
                                                                              long long ldp, const float* __restrict__ dt_raw,
                                                                              float* __restrict__ o_raw) {
  const int s = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int D = dl.dim, E = dl.vdim;
  const int e0 = (blockIdx.z * SCAN_WARPS + warp) * SCW;
  if (e0 >= E) return;
  const int hk = h / (dl.heads / dl.kv_heads);
  const int C = 2 * dl.kv_heads * D + dl.heads * E;
  float* gstate = st.base + (size_t)rows.seq_slot[s] * st.slot_floats + dl.state_off + (size_t)h * D * E;
  float S[RPL][SCW];
#pragma unroll
  for (int i = 0; i < RPL; i++) {
    const int d = lane + 32 * i;
#pragma unroll
    for (int c = 0; c < SCW; c++) S[i][c] = (d < D && e0 + c < E) ? gstate[(size_t)d * E + e0 + c] : 0.f;
  }
  const float qscale = 1.0f / sqrtf((float)D);
  const int r_begin = rows.seq_first[s], r_end = rows.seq_first[s + 1];
  float q[RPL], k[RPL], dt[RPL], v[SCW], braw = 0.f;
  auto fetch = [&](int r) {
    const float* x = qkv + (size_t)r * C;
#pragma unroll
    for (int i = 0; i < RPL; i++) {
      const int d = lane + 32 * i;
      q[i] = d < D ? x[hk * D + d] : 0.f;
      k[i] = d < D ? x[dl.kv_heads * D + hk * D + d] : 0.f;
      dt[i] = d < D ? dt_raw[(size_t)r * dl.heads * D + h * D + d] : 0.f;
    }
#pragma unroll
    for (int c = 0; c < SCW; c++) v[c] = e0 + c < E ? x[2 * dl.kv_heads * D + h * E + e0 + c] : 0.f;
    braw = proj[(size_t)r * ldp + dl.o_b + h];
  };
  if (r_begin < r_end) fetch(r_begin);
  for (int r = r_begin; r < r_end; r++) {
    float cq[RPL], ck[RPL], cg[RPL], cv[SCW];
    float qq = 0.f, kk = 0.f;
#pragma unroll
    for (int i = 0; i < RPL; i++) {
      cq[i] = q[i]; ck[i] = k[i];
      qq = fmaf(cq[i], cq[i], qq);
      kk = fmaf(ck[i], ck[i], kk);
      cg[i] = dt[i];   // the decay (hyb_delta_gates_kernel); lanes past D hold S = 0 whatever it is
    }
#pragma unroll
    for (int c = 0; c < SCW; c++) cv[c] = v[c];
    const float beta = braw;
    if (r + 1 < r_end) fetch(r + 1);
    qq = warp_sum(qq);
    kk = warp_sum(kk);
    const float qn = qscale / sqrtf(qq + 1e-6f), kn = 1.0f / sqrtf(kk + 1e-6f);
    float kv[SCW], o[SCW];
#pragma unroll
    for (int c = 0; c < SCW; c++) { kv[c] = 0.f; o[c] = 0.f; }
#pragma unroll
    for (int i = 0; i < RPL; i++) {
      ck[i] *= kn;
      cq[i] *= qn;
#pragma unroll
      for (int c = 0; c < SCW; c++) { S[i][c] *= cg[i]; kv[c] = fmaf(S[i][c], ck[i], kv[c]); }
    }
    float u[SCW];
#pragma unroll
    for (int c = 0; c < SCW; c++) u[c] = beta * (cv[c] - warp_sum(kv[c]));
#pragma unroll
    for (int i = 0; i < RPL; i++)
#pragma unroll
      for (int c = 0; c < SCW; c++) { S[i][c] = fmaf(ck[i], u[c], S[i][c]); o[c] = fmaf(S[i][c], cq[i], o[c]); }
#pragma unroll
    for (int c = 0; c < SCW; c++) {
      const float ov = warp_sum(o[c]);
      if (lane == c && e0 + c < E) o_raw[(size_t)r * dl.heads * E + (size_t)h * E + e0 + c] = ov;
    }
  }
#pragma unroll
  for (int i = 0; i < RPL; i++) {
    const int d = lane + 32 * i;
    if (d >= D) continue;
#pragma unroll
    for (int c = 0; c < SCW; c++)
      if (e0 + c < E) gstate[(size_t)d * E + e0 + c] = S[i][c];
  }
}

// out = o / rms(o over the head) * norm * sigmoid(gate), dtype-typed; a warp per (row, head)
template <typename T>
__global__ void hyb_head_gate_kernel(T* __restrict__ out, const float* __restrict__ o_raw, int n_rows, int heads, int E, float eps,
                                     const float* __restrict__ norm, int norm_per_head, const float* __restrict__ gate, long long ldg,
                                     int do_norm, int gate_act) {
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= n_rows * heads) return;
  const int r = idx / heads, h = idx - r * heads;
  const float* o = o_raw + (size_t)r * heads * E + (size_t)h * E;
  float inv = 1.0f;
  if (do_norm) {
    float ss = 0.f;
    for (int e = lane; e < E; e += 32) ss = fmaf(o[e], o[e], ss);
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)E + eps);
  }
  for (int e = lane; e < E; e += 32) {
    const float z = gate ? gate[(size_t)r * ldg + h * E + e] : 0.f;
    const float g = !gate ? 1.0f : gate_act == THA_GATE_SILU ? z * hyb_sigmoid(z) : hyb_sigmoid(z);
    const float v = do_norm ? o[e] * inv * norm[norm_per_head ? h * E + e : e] : o[e];
    hyb_store(out + (size_t)r * heads * E + (size_t)h * E + e, v * g);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// short causal convolution + silu; the slot keeps the last taps-1 inputs of every channel (oldest first)
// ------------------------------------------------------------------------------------------------------------------
// V channels per thread (V = 4: 128-bit reads of the rows; the caller checks the alignment); taps up to CONV_MAX_TAPS keep their
// weights in registers across the rows a thread walks
constexpr int CONV_MAX_TAPS = 8;
template <typename T, int V>
__global__ void hyb_conv_kernel(tha_rows_t rows, tha_state_store_t st, long long conv_state_off, const float* __restrict__ proj,
                                long long ldp, int col0, int channels, int taps, const float* __restrict__ w, int act, int add_input,
                                T* __restrict__ out) {
  const int c = V * (blockIdx.x * blockDim.x + threadIdx.x);
  if (c >= channels) return;
  float wr[CONV_MAX_TAPS][V];
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; j++)
#pragma unroll
    for (int v = 0; v < V; v++) wr[j][v] = j < taps ? w[(size_t)(c + v) * taps + j] : 0.f;
  for (int r = blockIdx.y; r < rows.n_rows; r += gridDim.y) {
    const int s = rows.row_seq[r], first = rows.seq_first[s];
    const float* tail = st.base + (size_t)rows.seq_slot[s] * st.slot_floats + conv_state_off + (size_t)c * (taps - 1);
    float acc[V], x[V], cur[V];
#pragma unroll
    for (int v = 0; v < V; v++) acc[v] = 0.f;
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; j++) {
      if (j >= taps) break;
      const int rr = r - (taps - 1 - j);
      if (rr >= first) {
        if (V == 4) { const float4 t = *reinterpret_cast<const float4*>(proj + (size_t)rr * ldp + col0 + c); x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w; }
        else x[0] = proj[(size_t)rr * ldp + col0 + c];
      } else {
#pragma unroll
        for (int v = 0; v < V; v++) x[v] = tail[(size_t)v * (taps - 1) + (taps - 1) - (first - rr)];
      }
#pragma unroll
      for (int v = 0; v < V; v++) { acc[v] = fmaf(wr[j][v], x[v], acc[v]); cur[v] = x[v]; }
    }
#pragma unroll
    for (int v = 0; v < V; v++) {
      if (act == 1) acc[v] = acc[v] / (1.0f + expf(-acc[v]));
      if (add_input) acc[v] += cur[v];                       // the last tap's input is the row itself
    }
    T* dst = out + (size_t)r * channels + c;
    if (V == 4 && sizeof(T) == 4) {
      *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    } else if (V == 4) {
      uint2 pk;
      const __nv_bfloat162 lo = __floats2bfloat162_rn(acc[0], acc[1]), hi = __floats2bfloat162_rn(acc[2], acc[3]);
      pk.x = *reinterpret_cast<const unsigned*>(&lo); pk.y = *reinterpret_cast<const unsigned*>(&hi);
      *reinterpret_cast<uint2*>(dst) = pk;
    } else {
      hyb_store(dst, acc[0]);
    }
  }
}
// any number of taps, a channel per thread
template <typename T>
__global__ void hyb_conv_long_kernel(tha_rows_t rows, tha_state_store_t st, long long conv_state_off, const float* __restrict__ proj,
                                     long long ldp, int col0, int channels, int taps, const float* __restrict__ w, int act, int add_input,
                                     T* __restrict__ out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  for (int r = blockIdx.y; r < rows.n_rows; r += gridDim.y) {
    const int s = rows.row_seq[r], first = rows.seq_first[s];
    const float* tail = st.base + (size_t)rows.seq_slot[s] * st.slot_floats + conv_state_off + (size_t)c * (taps - 1);
    float acc = 0.f;
    for (int j = 0; j < taps; j++) {
      const int rr = r - (taps - 1 - j);
      const float x = rr >= first ? proj[(size_t)rr * ldp + col0 + c] : tail[(taps - 1) - (first - rr)];
      acc = fmaf(w[(size_t)c * taps + j], x, acc);
    }
    if (act == 1) acc = acc / (1.0f + expf(-acc));
    if (add_input) acc += proj[(size_t)r * ldp + col0 + c];
    hyb_store(out + (size_t)r * channels + c, acc);
  }
}
// after the convolution: tail[i] <- the input (taps-1-i) tokens before the end of what the sequence has seen now
__global__ void hyb_conv_tail_kernel(tha_rows_t rows, tha_state_store_t st, long long conv_state_off, const float* __restrict__ proj,
                                     long long ldp, int col0, int channels, int taps) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
  if (c >= channels) return;
  const int first = rows.seq_first[s], n = rows.seq_first[s + 1] - first;
  float* tail = st.base + (size_t)rows.seq_slot[s] * st.slot_floats + conv_state_off + (size_t)c * (taps - 1);
  for (int i = 0; i < taps - 1; i++) {           // ascending: tail[i + n] is read before it is overwritten
    const int back = (taps - 1) - i;             // this entry is the input `back` tokens before the end
    tail[i] = back <= n ? proj[(size_t)(first + n - back) * ldp + col0 + c] : tail[i + n];
  }
}

// ------------------------------------------------------------------------------------------------------------------
// gated delta rule: block (sequence, value head, column slice) as in the matrix memory.  Per token, thread (part, e):
// decay its rows of column e and sum S^T k; after the column's u = beta (v - S^T k) is known, add k u and sum S^T q.
// Output: S^T q per (row, head, column) in fp32 (norm and gate in hyb_head_gate_kernel).
// ------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(SCAN_THREADS) hyb_delta_scan_kernel(tha_delta_t dl, tha_rows_t rows, tha_state_store_t st,
                                                                      const float* __restrict__ qkv, const float* __restrict__ proj, long long ldp,
                                                                      const float* __restrict__ dt_raw, float* __restrict__ o_raw, int SC) {
  extern __shared__ float sm[];
  const int s = blockIdx.x, h = blockIdx.y, e0 = blockIdx.z * SC;
  const int D = dl.dim, E = dl.vdim, nt = SCAN_THREADS;
  const int ec = min(SC, E - e0);
  const int hk = h / (dl.heads / dl.kv_heads);
  const int C = 2 * dl.kv_heads * D + dl.heads * E;
  const int parts = nt / SC;
  float* S = sm;                     // [D][SC]
  float* in = S + D * SC;            // 2 x (q [D] | k [D] | g [D] | v [SC] | beta)
  const int in_stride = 3 * D + SC + 1;
  float* part = in + 2 * in_stride;  // [parts][SC]
  float* su = part + parts * SC;     // [SC]
  float* gstate = st.base + (size_t)rows.seq_slot[s] * st.slot_floats + dl.state_off + (size_t)h * D * E;
  for (int i = threadIdx.x; i < D * SC; i += nt) { const int d = i / SC, e = i - d * SC; S[i] = e < ec ? gstate[(size_t)d * E + e0 + e] : 0.f; }
  const float qscale = 1.0f / sqrtf((float)D);
  const int r_begin = rows.seq_first[s], r_end = rows.seq_first[s + 1];
  auto fetch = [&](int r, int i) -> float {
    const float* x = qkv + (size_t)r * C;
    if (i < D) return x[hk * D + i];
    if (i < 2 * D) return x[dl.kv_heads * D + hk * D + (i - D)];
    if (i < 3 * D) return dt_raw[(size_t)r * dl.heads * D + h * D + (i - 2 * D)];   // the decays (hyb_delta_gates_kernel)
    if (i < 3 * D + SC) return (i - 3 * D) < ec ? x[2 * dl.kv_heads * D + h * E + e0 + (i - 3 * D)] : 0.f;
    return proj[(size_t)r * ldp + dl.o_b + h];
  };
  constexpr int PF = 4;
  float pf[PF];
#pragma unroll
  for (int u = 0; u < PF; u++) { const int i = threadIdx.x + u * nt; pf[u] = (i < in_stride && r_begin < r_end) ? fetch(r_begin, i) : 0.f; }
  const int pe = threadIdx.x % SC, pp = threadIdx.x / SC, lane = threadIdx.x & 31;
  for (int r = r_begin; r < r_end; r++) {
    float* cur = in + ((r - r_begin) & 1) * in_stride;
#pragma unroll
    for (int u = 0; u < PF; u++) { const int i = threadIdx.x + u * nt; if (i < in_stride) cur[i] = pf[u]; }
    for (int i = threadIdx.x + PF * nt; i < in_stride; i += nt) cur[i] = fetch(r, i);
    if (r + 1 < r_end) {
#pragma unroll
      for (int u = 0; u < PF; u++) { const int i = threadIdx.x + u * nt; if (i < in_stride) pf[u] = fetch(r + 1, i); }
    }
    __syncthreads();
    const float* sq = cur; const float* sk = cur + D; const float* sg = cur + 2 * D; const float* sv = cur + 3 * D;
    // unit vectors: every warp sums the squares itself (the same values in the same order in every warp)
    float qq = 0.f, kk = 0.f;
    for (int i = lane; i < D; i += 32) { qq = fmaf(sq[i], sq[i], qq); kk = fmaf(sk[i], sk[i], kk); }
    qq = warp_sum(qq);
    kk = warp_sum(kk);
    const float qn = qscale / sqrtf(qq + 1e-6f), kn = 1.0f / sqrtf(kk + 1e-6f);
    if (pp < parts) {
      float acc = 0.f;
      for (int d = pp; d < D; d += parts) { const float v = S[d * SC + pe] * sg[d]; S[d * SC + pe] = v; acc = fmaf(v, sk[d] * kn, acc); }
      part[pp * SC + pe] = acc;
    }
    __syncthreads();
    if (threadIdx.x < SC) {
      float acc = 0.f;
      for (int p = 0; p < parts; p++) acc += part[p * SC + threadIdx.x];
      su[threadIdx.x] = cur[3 * D + SC] * (sv[threadIdx.x] - acc);
    }
    __syncthreads();
    if (pp < parts) {
      const float u = su[pe];
      float acc = 0.f;
      for (int d = pp; d < D; d += parts) { const float v = fmaf(sk[d] * kn, u, S[d * SC + pe]); S[d * SC + pe] = v; acc = fmaf(v, sq[d] * qn, acc); }
      part[pp * SC + pe] = acc;
    }
    __syncthreads();
    if (threadIdx.x < ec) {
      float acc = 0.f;
      for (int p = 0; p < parts; p++) acc += part[p * SC + threadIdx.x];
      o_raw[(size_t)r * dl.heads * E + (size_t)h * E + e0 + threadIdx.x] = acc;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D * SC; i += nt) { const int d = i / SC, e = i - d * SC; if (e < ec) gstate[(size_t)d * E + e0 + e] = S[i]; }
}

// ------------------------------------------------------------------------------------------------------------------
// router: a warp per row picks the `top` largest logits (lowest index on ties), softmax over them
// ------------------------------------------------------------------------------------------------------------------
__global__ void hyb_route_kernel(int experts, int top, int o_router, const float* __restrict__ proj, long long ldp, int n_rows,
                                 int* __restrict__ expert_id, float* __restrict__ weight, int* __restrict__ counts) {
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= n_rows) return;
  const float* z = proj + (size_t)r * ldp + o_router;
  float zmax = 0.f, sum = 0.f, mine = 0.f;   // lane j keeps the j-th pick's logit (top <= 32)
  for (int j = 0; j < top; j++) {
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      bool taken = false;
      for (int p = 0; p < j; p++) taken |= expert_id[(size_t)r * top + p] == e;
      const float v = z[e];
      if (!taken && (v > best || (v == best && e < bi))) { best = v; bi = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(THA_FULL_MASK, best, o);
      const int oi = __shfl_xor_sync(THA_FULL_MASK, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) { expert_id[(size_t)r * top + j] = bi; atomicAdd(counts + bi, 1); }
    __syncwarp();
    if (j == 0) zmax = best;
    if (lane == j) mine = best;
    sum += expf(best - zmax);
  }
  if (lane < top) weight[(size_t)r * top + lane] = expf(mine - zmax) / sum;
}
// Router with scores over ALL experts: s = softmax(z); the choice uses s + correction, limited to the `keep` groups (of
// experts / groups neighbours each) whose largest choice score is highest -- experts outside them count as minus infinity,
// whatever the sign of their score; the weights are the chosen s over their sum.  A warp per row; ties go to the lowest
// index; needs top <= 32 and at most 4096 experts (blocks of 128 threads).
__global__ void hyb_route_groups_kernel(int experts, int top, int groups, int keep, int o_router, const float* __restrict__ correction,
                                        const float* __restrict__ proj, long long ldp, int n_rows, int* __restrict__ expert_id,
                                        float* __restrict__ weight, int* __restrict__ counts) {
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= n_rows) return;
  const float* z = proj + (size_t)r * ldp + o_router;
  float zmax = -INFINITY;
  for (int e = lane; e < experts; e += 32) zmax = fmaxf(zmax, z[e]);
  for (int o = 16; o > 0; o >>= 1) zmax = fmaxf(zmax, __shfl_xor_sync(THA_FULL_MASK, zmax, o));
  float den = 0.f;
  for (int e = lane; e < experts; e += 32) den += expf(z[e] - zmax);
  den = warp_sum(den);
  // bit g of the warp's words: group g may be chosen from (shared memory, so that any number of groups up to the experts fits)
  __shared__ unsigned allowed_s[4][128];
  unsigned* allowed = allowed_s[threadIdx.x >> 5];
  const int per = groups > 1 ? experts / groups : experts;
  const bool bound = groups > 1 && keep < groups;
  for (int w = lane; w < 128; w += 32) allowed[w] = bound ? 0u : 0xffffffffu;
  __syncwarp();
  if (bound) {
    auto group_best = [&](int g) {   // the largest choice score of group g
      float b = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; e++) b = fmaxf(b, expf(z[e] - zmax) / den + (correction ? correction[e] : 0.f));
      return b;
    };
    const float gbest = lane < groups ? group_best(lane) : -INFINITY;   // lane g keeps group g's; groups beyond 32 are recomputed
    for (int j = 0; j < keep; j++) {
      float best = -INFINITY; int bi = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        if ((allowed[g >> 5] >> (g & 31)) & 1u) continue;
        const float v = g < 32 ? gbest : group_best(g);
        if (v > best || (v == best && g < bi)) { best = v; bi = g; }
      }
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(THA_FULL_MASK, best, o);
        const int oi = __shfl_xor_sync(THA_FULL_MASK, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      if (lane == 0 && bi < groups) allowed[bi >> 5] |= 1u << (bi & 31);
      __syncwarp();
    }
  }
  float sum = 0.f, mine = 0.f;
  unsigned long long taken_lo = 0ull;   // experts this lane has given away (bit = e / 32 of its own stride), up to 2048 experts
  unsigned long long taken_hi = 0ull;
  for (int j = 0; j < top; j++) {
    float best = -INFINITY, bs = 0.f; int bi = 0x7fffffff;
    for (int e = lane, n = 0; e < experts; e += 32, n++) {
      const bool taken = n < 64 ? (taken_lo >> n) & 1ull : (taken_hi >> (n - 64)) & 1ull;
      const int g = groups > 1 ? e / per : 0;
      if (taken || !((allowed[g >> 5] >> (g & 31)) & 1u)) continue;
      const float sc = expf(z[e] - zmax) / den;
      const float v = sc + (correction ? correction[e] : 0.f);
      if (v > best || (v == best && e < bi)) { best = v; bi = e; bs = sc; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(THA_FULL_MASK, best, o);
      const int oi = __shfl_xor_sync(THA_FULL_MASK, bi, o);
      const float os = __shfl_xor_sync(THA_FULL_MASK, bs, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; bs = os; }
    }
    if (bi >= experts) bi = 0, bs = 0.f;   // fewer allowed experts than picks: cannot happen with a valid config
    if ((bi & 31) == lane) { const int n = bi >> 5; if (n < 64) taken_lo |= 1ull << n; else taken_hi |= 1ull << (n - 64); }
    if (lane == 0) { expert_id[(size_t)r * top + j] = bi; atomicAdd(counts + bi, 1); }
    if (lane == j) mine = bs;
    sum += bs;
  }
  if (lane < top) weight[(size_t)r * top + lane] = mine / (sum + 1e-20f);
}

// any of the feed-forward activations (THA_ACT_*): gated ones read a gate value g and an up value u, ungated ones u only.
// THA_ACT_XIELU arrives with (limit, alpha) = (softplus(p), 1/2 + softplus(q)) of its two stored numbers.
__device__ __forceinline__ float hyb_act_value(int act, float g, float u, float limit, float alpha) {
  if (act == THA_ACT_RELU2) {
    const float p = fmaxf(u, 0.f);
    return p * p;
  }
  if (act == THA_ACT_XIELU) return u > 0.f ? fmaf(limit * u, u, 0.5f * u) : fmaf(alpha, expm1f(u) - u, 0.5f * u);
  if (act == THA_ACT_SILU_GLU) return g * hyb_sigmoid(g) * u;
  if (act == THA_ACT_GELU_TANH_GLU) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
  const float gc = fminf(g, limit);
  return gc * hyb_sigmoid(alpha * gc) * (fminf(fmaxf(u, -limit), limit) + 1.0f);
}
template <typename T>
__global__ void hyb_ff_act_kernel(T* __restrict__ y, const float* __restrict__ gu, long long ldg, int col_g, int col_u, int n, int ff, int act,
                                  float limit, float alpha) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n * ff) return;
  const size_t r = i / ff; const int c = (int)(i - r * ff);
  const bool gated = act != THA_ACT_RELU2 && act != THA_ACT_XIELU;
  hyb_store(y + i, hyb_act_value(act, gated ? gu[r * ldg + col_g + c] : 0.f, gu[r * ldg + col_u + c], limit, alpha));
}
// the same with four columns per thread and a row per blockIdx.y (sizes and offsets that are multiples of four)
template <typename T>
__global__ void hyb_ff_act_vec_kernel(T* __restrict__ y, const float* __restrict__ gu, long long ldg, int col_g, int col_u, int ff, int act,
                                      float limit, float alpha) {
  const int c = 4 * (blockIdx.x * blockDim.x + threadIdx.x);
  if (c >= ff) return;
  const size_t r = blockIdx.y;
  const bool gated = act != THA_ACT_RELU2 && act != THA_ACT_XIELU;
  const float4 u = *reinterpret_cast<const float4*>(gu + r * ldg + col_u + c);
  const float4 g = gated ? *reinterpret_cast<const float4*>(gu + r * ldg + col_g + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  const float v0 = hyb_act_value(act, g.x, u.x, limit, alpha), v1 = hyb_act_value(act, g.y, u.y, limit, alpha);
  const float v2 = hyb_act_value(act, g.z, u.z, limit, alpha), v3 = hyb_act_value(act, g.w, u.w, limit, alpha);
  T* dst = y + r * ff + c;
  hyb_store(dst, v0); hyb_store(dst + 1, v1); hyb_store(dst + 2, v2); hyb_store(dst + 3, v3);
}

// counting sort of the (row, pick) pairs by expert, a block per expert: within an expert the pairs stay in ascending
// (row, pick) order, so the placement is the same on every run.  The block finds its expert's first place from the counts,
// then walks all pairs in chunks of its size: a ballot per warp, the warps' counts through shared memory, a pair's place =
// what the expert has so far + the hits of the warps before + the hits of the lanes before.
__global__ void __launch_bounds__(1024) hyb_route_sort_kernel(int experts, int top, int n_rows, const int* __restrict__ expert_id,
                                                              const int* __restrict__ counts, int* __restrict__ group_off,
                                                              int* __restrict__ sorted_row, int* __restrict__ inv) {
  __shared__ int wcount[32];
  __shared__ int s_start;
  const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (warp == 0) {
    int acc = 0;
    for (int x = lane; x < e; x += 32) acc += counts[x];
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(THA_FULL_MASK, acc, o);
    if (lane == 0) {
      s_start = acc;
      group_off[e] = acc;
      if (e == experts - 1) group_off[experts] = acc + counts[e];
    }
  }
  __syncthreads();
  int at = s_start;
  const int n = n_rows * top;
  for (int i0 = 0; i0 < n; i0 += blockDim.x) {
    const int i = i0 + threadIdx.x;
    const bool hit = i < n && expert_id[i] == e;
    const unsigned m = __ballot_sync(THA_FULL_MASK, hit);
    if (lane == 0) wcount[warp] = __popc(m);
    __syncthreads();
    int before = 0, total = 0;
    for (int w = 0; w < nwarps; w++) { const int c = wcount[w]; total += c; if (w < warp) before += c; }
    if (hit) { const int p = at + before + __popc(m & ((1u << lane) - 1)); sorted_row[p] = i / top; inv[i] = p; }
    at += total;
    __syncthreads();
  }
}

// THA_HYB_TC=0 keeps every product on the plain kernel (A/B aid)
static bool hyb_tc_linear() {
  static int on = -1;
  if (on < 0) { const char* v = getenv("THA_HYB_TC"); on = (v && *v) ? atoi(v) != 0 : 1; }
  return on != 0;
}

static int pick_threads(int want) {   // a multiple of 32 in 64..256
  int t = 64;
  while (t < want && t < 256) t += 32;
  return t;
}

}  // namespace tha

using namespace tha;
typedef __nv_bfloat16 bf16;

extern "C" int tha_hyb_rmsnorm(void* stream, int dtype, void* out, const float* x, const float* w, float w_offset, float eps,
                               int n_rows, int width, const int* rows_idx) {
  if (n_rows < 1) return THA_STATUS_SUCCESS;
  const int nt = pick_threads(width / 4);
  if (dtype == THA_DT_BF16)
    THA_CUDA_OK(launch(hyb_rmsnorm_kernel<bf16>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, (bf16*)out, x, w, w_offset, eps, width, rows_idx));
  else
    THA_CUDA_OK(launch(hyb_rmsnorm_kernel<float>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, (float*)out, x, w, w_offset, eps, width, rows_idx));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_norm(void* stream, int dtype, void* out, const float* x, const tha_norm_t* n, float eps, int n_rows, int width,
                            const int* rows_idx) {
  if (n->kind == THA_NORM_RMS) return tha_hyb_rmsnorm(stream, dtype, out, x, n->w, n->w_offset, eps, n_rows, width, rows_idx);
  if (n->kind == THA_NORM_LAYER) {
    if (!n->w) return THA_STATUS_INVALID_ARG;
    if (n_rows < 1) return THA_STATUS_SUCCESS;
    const int nt = pick_threads(width / 4);
    if (dtype == THA_DT_BF16)
      THA_CUDA_OK(launch(hyb_layernorm_kernel<bf16>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, (bf16*)out, x, n->w, n->b, eps, width, rows_idx));
    else
      THA_CUDA_OK(launch(hyb_layernorm_kernel<float>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, (float*)out, x, n->w, n->b, eps, width, rows_idx));
    return THA_STATUS_SUCCESS;
  }
  if (n->kind != THA_NORM_DYT || !n->w) return THA_STATUS_INVALID_ARG;
  if (n_rows < 1) return THA_STATUS_SUCCESS;
  const int nt = pick_threads(width);
  if (dtype == THA_DT_BF16)
    THA_CUDA_OK(launch(hyb_dyt_kernel<bf16>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, (bf16*)out, x, n->w, n->b, n->alpha, width, rows_idx));
  else
    THA_CUDA_OK(launch(hyb_dyt_kernel<float>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, (float*)out, x, n->w, n->b, n->alpha, width, rows_idx));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_norm_pair(void* stream, int dtype, void* out1, void* out2, const float* x, const tha_norm_t* n1, const tha_norm_t* n2,
                                 float eps, int n_rows, int width) {
  if (n1->kind == THA_NORM_DYT && n2->kind == THA_NORM_DYT && n1->w && n2->w) {
    if (n_rows < 1) return THA_STATUS_SUCCESS;
    const int nt = pick_threads(width);
    if (dtype == THA_DT_BF16)
      THA_CUDA_OK(launch(hyb_dyt2_kernel<bf16>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, (bf16*)out1, (bf16*)out2, x, *n1, *n2, width));
    else
      THA_CUDA_OK(launch(hyb_dyt2_kernel<float>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, (float*)out1, (float*)out2, x, *n1, *n2, width));
    return THA_STATUS_SUCCESS;
  }
  const int st = tha_hyb_norm(stream, dtype, out1, x, n1, eps, n_rows, width, nullptr);
  return st != THA_STATUS_SUCCESS ? st : tha_hyb_norm(stream, dtype, out2, x, n2, eps, n_rows, width, nullptr);
}

extern "C" int tha_hyb_linear_heads(void* stream, int dtype, float* C, long long ldc, long long c_hs, const void* A, long long lda,
                                    long long a_hs, int a_f32, const void* W, long long w_hs, int M, int N, int K, int heads) {
  if (M < 1 || N < 1 || heads < 1) return THA_STATUS_SUCCESS;
  if (K < 1 || !C || !A || !W) return THA_STATUS_INVALID_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 grid(ceil_div(N, LT), ceil_div(M, LT), heads), block(256);
  const int* none = nullptr;
  if (dtype == THA_DT_BF16 && !a_f32 && hyb_tc_linear() && K % 8 == 0 && lda % 8 == 0 && a_hs % 8 == 0 && w_hs % 8 == 0 && aligned16(A) && aligned16(W)) {
    THA_CUDA_OK(launch(hyb_linear_mma_kernel, grid, dim3(128), 0, s, false, C, ldc, (const bf16*)A, lda, none, (const bf16*)W, 0ll, M, N, K, none, 0,
                       a_hs, w_hs, c_hs));
    return THA_STATUS_SUCCESS;
  }
  if (dtype == THA_DT_F32)
    THA_CUDA_OK(launch(hyb_linear_kernel<float, float>, grid, block, 0, s, false, C, ldc, (const float*)A, lda, none, (const float*)W, 0ll, M, N, K,
                       none, 0, a_hs, w_hs, c_hs));
  else if (a_f32)
    THA_CUDA_OK(launch(hyb_linear_kernel<float, bf16>, grid, block, 0, s, false, C, ldc, (const float*)A, lda, none, (const bf16*)W, 0ll, M, N, K,
                       none, 0, a_hs, w_hs, c_hs));
  else
    THA_CUDA_OK(launch(hyb_linear_kernel<bf16, bf16>, grid, block, 0, s, false, C, ldc, (const bf16*)A, lda, none, (const bf16*)W, 0ll, M, N, K,
                       none, 0, a_hs, w_hs, c_hs));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_head_gate(void* stream, int dtype, void* out, const float* o_raw, int n_rows, int heads, int E, int do_norm,
                                 float eps, const float* norm, int norm_per_head, const float* gate, long long ldg, int gate_act) {
  if (n_rows < 1) return THA_STATUS_SUCCESS;
  if (do_norm && !norm) return THA_STATUS_INVALID_ARG;
  const dim3 grid(ceil_div(n_rows * heads, 4));
  if (dtype == THA_DT_BF16)
    THA_CUDA_OK(launch(hyb_head_gate_kernel<bf16>, grid, dim3(128), 0, (cudaStream_t)stream, false, (bf16*)out, o_raw, n_rows, heads, E, eps, norm,
                       norm_per_head, gate, ldg, do_norm, gate_act));
  else
    THA_CUDA_OK(launch(hyb_head_gate_kernel<float>, grid, dim3(128), 0, (cudaStream_t)stream, false, (float*)out, o_raw, n_rows, heads, E, eps, norm,
                       norm_per_head, gate, ldg, do_norm, gate_act));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_linear(void* stream, int dtype, float* C, long long ldc, const void* A, long long lda, int a_f32,
                              const int* a_rows, const void* W, long long w_group_stride, int M, int N, int K,
                              const int* group_off, int n_groups) {
  if (M < 1 || N < 1) return THA_STATUS_SUCCESS;
  if (K < 1 || !C || !A || !W) return THA_STATUS_INVALID_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == THA_DT_BF16 && !a_f32 && !a_rows && !group_off) {
    // a plain bf16 product: the tcgen05 matmul of the bf16 model path (TMA-fed, fp32 accumulators in TMEM) when its
    // alignment rules hold; the rows of this step are its activation columns
    BfArgs b = {};
    b.n_mats = 1; b.W[0] = (const uint16_t*)W; b.M[0] = N; b.out_off[0] = 0; b.K = K;
    b.X = (const uint16_t*)A; b.N = M; b.ldx = lda;
    b.out = C; b.ldo = ldc; b.zstride = 0; b.splits = 1; b.colscale = nullptr;
    if (hyb_tc_linear() && gemm_bf16_ok(b)) return gemm_bf16_launch(s, b, false);
  }
  const int mt = ceil_div(M, LT) + (group_off ? n_groups : 0);
  const dim3 grid(ceil_div(N, LT), mt), block(256);
  if (dtype == THA_DT_BF16 && !a_f32 && hyb_tc_linear() && K % 8 == 0 && lda % 8 == 0 && w_group_stride % 8 == 0 && aligned16(A) && aligned16(W)) {
    THA_CUDA_OK(launch(hyb_linear_mma_kernel, grid, dim3(128), 0, s, false, C, ldc, (const bf16*)A, lda, a_rows, (const bf16*)W, w_group_stride,
                       M, N, K, group_off, n_groups, 0ll, 0ll, 0ll));
    return THA_STATUS_SUCCESS;
  }
  if (dtype == THA_DT_F32)
    THA_CUDA_OK(launch(hyb_linear_kernel<float, float>, grid, block, 0, s, false, C, ldc, (const float*)A, lda, a_rows, (const float*)W,
                       w_group_stride, M, N, K, group_off, n_groups, 0ll, 0ll, 0ll));
  else if (a_f32)
    THA_CUDA_OK(launch(hyb_linear_kernel<float, bf16>, grid, block, 0, s, false, C, ldc, (const float*)A, lda, a_rows, (const bf16*)W,
                       w_group_stride, M, N, K, group_off, n_groups, 0ll, 0ll, 0ll));
  else
    THA_CUDA_OK(launch(hyb_linear_kernel<bf16, bf16>, grid, block, 0, s, false, C, ldc, (const bf16*)A, lda, a_rows, (const bf16*)W,
                       w_group_stride, M, N, K, group_off, n_groups, 0ll, 0ll, 0ll));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_rotary_table(void* stream, const tha_rotary_t* rot, const int* pos, int n_rows, float* cos_out, float* sin_out) {
  const int half = rot->dims / 2;
  if (n_rows < 1 || half < 1) return THA_STATUS_SUCCESS;
  THA_CUDA_OK(launch(hyb_rotary_kernel, dim3(ceil_div(n_rows * half, 128)), dim3(128), 0, (cudaStream_t)stream, false, rot->inv_freq, half,
                     rot->mag, pos, n_rows, cos_out, sin_out));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_attn_prepare(void* stream, const tha_attn_t* a, const tha_rows_t* rows, const tha_kv_t* kv, const float* proj,
                                    long long ldp, const float* cos_t, const float* sin_t, int rot_dims, float* q_out) {
  if (rows->n_rows < 1) return THA_STATUS_SUCCESS;
  if (a->heads % a->kv_heads || rot_dims > a->dim || (rot_dims & 1) || a->kv_heads * a->dim > kv->kv_dim ||
      a->kv_heads / (a->v_share > 1 ? a->v_share : 1) * a->vdim > kv->kv_dim)
    return THA_STATUS_INVALID_ARG;
  const int nt = pick_threads(32 * (a->heads + 2 * a->kv_heads));
  THA_CUDA_OK(launch(hyb_attn_prepare_kernel, dim3(rows->n_rows), dim3(nt), 0, (cudaStream_t)stream, false, *a, *rows, *kv, proj, ldp, cos_t,
                     sin_t, rot_dims, q_out));
  return THA_STATUS_SUCCESS;
}

namespace tha {
// hybrid_latent.cu: tensor-core attention for key rows wider than AM_MAXD whose values lie inside the keys
bool hyb_attn_wide_ok(const tha_attn_t* a);
int hyb_attn_wide_pairs(const tha_attn_t* a, const tha_rows_t* rows);
int hyb_attn_wide_launch(cudaStream_t s, const tha_attn_t* a, const tha_rows_t* rows, const tha_kv_t* kv, const float* q, __nv_bfloat16* out,
                         dim3 grid, int pairs, int AG, int AP, int splits, float* partial);
}  // namespace tha

extern "C" int tha_hyb_attn(void* stream, int dtype, const tha_attn_t* a, const tha_rows_t* rows, const tha_kv_t* kv, const float* q,
                            void* out, float* split_scratch, size_t split_scratch_floats) {
  return tha_hyb_attn_gated(stream, dtype, a, rows, kv, q, out, split_scratch, split_scratch_floats, nullptr, 0);
}

// THA_HYB_ATTN_TC=0 keeps attention on the fp32 cores in the bf16 number format as well (A/B aid)
static bool hyb_tc_attn() {
  static int on = -1;
  if (on < 0) { const char* v = getenv("THA_HYB_ATTN_TC"); on = (v && *v) ? atoi(v) != 0 : 1; }
  return on != 0;
}

extern "C" int tha_hyb_attn_gated(void* stream, int dtype, const tha_attn_t* a, const tha_rows_t* rows, const tha_kv_t* kv, const float* q,
                                  void* out, float* split_scratch, size_t split_scratch_floats, const float* proj, long long ldp) {
  if (rows->n_rows < 1) return THA_STATUS_SUCCESS;
  if (a->window < 0 || a->keep_first < 0) return THA_STATUS_INVALID_ARG;
  const float* gate = (a->head_gate && proj) ? proj + a->o_g : nullptr;
  const long long ldg = ldp;
  if (a->heads % a->kv_heads || a->vdim > 32 * ATT_MAX_VC) return THA_STATUS_NOT_SUPPORTED;
  if (a->v_share > 1 && (a->kv_heads % a->v_share || a->values_in_keys)) return THA_STATUS_INVALID_ARG;
  const int gsize = a->heads / a->kv_heads;
  // bf16 with heads the tensor-core form covers: 64 pairs per block; else 16 pairs on the fp32 cores
  const bool tc = dtype == THA_DT_BF16 && hyb_tc_linear() && hyb_tc_attn() && a->dim % 16 == 0 && a->vdim % 8 == 0 && a->dim <= AM_MAXD && a->vdim <= AM_MAXD &&
                  (a->heads * a->vdim) % 2 == 0;
  const bool wide = !tc && !gate && !a->head_scale && !a->out_f32 && a->v_share <= 1 && dtype == THA_DT_BF16 && hyb_tc_linear() && hyb_tc_attn() && hyb_attn_wide_ok(a);
  const int pairs = wide ? hyb_attn_wide_pairs(a, rows) : tc ? AM_PAIRS : ATT_PAIRS;
  const int AG = gsize < pairs ? gsize : pairs, AP = pairs / AG;
  const size_t smem = tc ? sizeof(__nv_bfloat16) * ((size_t)ATT_KEYS * (a->dim + 8) + (size_t)ATT_KEYS * (a->vdim + 8))
                         : sizeof(float) * ((size_t)ATT_PAIRS * a->dim + (size_t)ATT_KEYS * (a->dim + 4) + (size_t)ATT_KEYS * a->vdim + ATT_PAIRS * ATT_KEYS);
  if (!wide && smem > 227 * 1024) return THA_STATUS_NOT_SUPPORTED;
  // position tiles: at most one ragged tile per sequence beyond rows / AP
  const int tiles = rows->n_rows / AP + rows->n_seqs;
  // few blocks and many keys (decoding at long contexts): deal the key tiles of a block to several
  const int seen = rows->max_pos + 1;
  int max_keys = a->chunk > 0 && a->chunk < seen ? a->chunk : seen;
  if (a->window > 0 && a->window + a->keep_first + 2 * ATT_KEYS < max_keys) max_keys = a->window + a->keep_first + 2 * ATT_KEYS;
  int splits = 1;
  const long long blocks = (long long)tiles * a->kv_heads * ceil_div(gsize, AG);
  if (split_scratch && blocks < 4 * 148 && max_keys >= 4 * ATT_KEYS) {
    splits = (int)((6 * 148 + blocks - 1) / blocks);
    if (splits > max_keys / (2 * ATT_KEYS)) splits = max_keys / (2 * ATT_KEYS);
    if (splits > 16) splits = 16;
    while (splits > 1 && (size_t)splits * rows->n_rows * a->heads * (a->vdim + 2) > split_scratch_floats) splits--;
  }
  const dim3 grid(tiles * splits, a->kv_heads, ceil_div(gsize, AG));
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == THA_DT_BF16) {
    if (wide) {
      const int st = hyb_attn_wide_launch(s, a, rows, kv, q, (bf16*)out, grid, pairs, AG, AP, splits, split_scratch);
      if (st != THA_STATUS_SUCCESS) return st;
    } else if (tc) {
      if (a->fp32_scores)
        THA_CUDA_OK(launch(hyb_attn_mma_kernel<true>, grid, dim3(128), smem, s, false, *a, *rows, *kv, q, (bf16*)out, AG, AP, splits, split_scratch, gate, ldg));
      else
        THA_CUDA_OK(launch(hyb_attn_mma_kernel<false>, grid, dim3(128), smem, s, false, *a, *rows, *kv, q, (bf16*)out, AG, AP, splits, split_scratch, gate, ldg));
    } else {
      if (a->vdim <= 256) {
        if (smem > 48 * 1024) THA_CUDA_OK(cudaFuncSetAttribute(hyb_attn_kernel<bf16, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        THA_CUDA_OK(launch(hyb_attn_kernel<bf16, 8>, grid, dim3(128), smem, s, false, *a, *rows, *kv, q, (bf16*)out, AG, AP, splits, split_scratch, gate, ldg));
      } else {
        if (smem > 48 * 1024) THA_CUDA_OK(cudaFuncSetAttribute(hyb_attn_kernel<bf16, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        THA_CUDA_OK(launch(hyb_attn_kernel<bf16, 16>, grid, dim3(128), smem, s, false, *a, *rows, *kv, q, (bf16*)out, AG, AP, splits, split_scratch, gate, ldg));
      }
    }
    if (splits > 1 && a->out_f32)
      THA_CUDA_OK(launch(hyb_attn_merge_kernel<float>, dim3(ceil_div(rows->n_rows * a->heads, 4)), dim3(128), 0, s, false, (float*)out,
                         (const float*)split_scratch, rows->n_rows, a->heads, a->vdim, splits, *a, gate, ldg));
    else if (splits > 1)
      THA_CUDA_OK(launch(hyb_attn_merge_kernel<bf16>, dim3(ceil_div(rows->n_rows * a->heads, 4)), dim3(128), 0, s, false, (bf16*)out,
                         (const float*)split_scratch, rows->n_rows, a->heads, a->vdim, splits, *a, gate, ldg));
  } else {
    if (a->vdim <= 256) {
      if (smem > 48 * 1024) THA_CUDA_OK(cudaFuncSetAttribute(hyb_attn_kernel<float, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      THA_CUDA_OK(launch(hyb_attn_kernel<float, 8>, grid, dim3(128), smem, s, false, *a, *rows, *kv, q, (float*)out, AG, AP, splits, split_scratch, gate, ldg));
    } else {
      if (smem > 48 * 1024) THA_CUDA_OK(cudaFuncSetAttribute(hyb_attn_kernel<float, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      THA_CUDA_OK(launch(hyb_attn_kernel<float, 16>, grid, dim3(128), smem, s, false, *a, *rows, *kv, q, (float*)out, AG, AP, splits, split_scratch, gate, ldg));
    }
    if (splits > 1)
      THA_CUDA_OK(launch(hyb_attn_merge_kernel<float>, dim3(ceil_div(rows->n_rows * a->heads, 4)), dim3(128), 0, s, false, (float*)out,
                         (const float*)split_scratch, rows->n_rows, a->heads, a->vdim, splits, *a, gate, ldg));
  }
  return THA_STATUS_SUCCESS;
}

// THA_HYB_SCAN=shared keeps the shared-memory scans at every head size (A/B aid and the test of that form)
static bool scan_in_registers() {
  const char* v = getenv("THA_HYB_SCAN");
  return !(v && !strcmp(v, "shared"));
}
// columns per block of the scans: a power of two that divides the thread count
static int scan_slice(int vdim) { int sc = 1; while (sc < vdim && sc < 16) sc <<= 1; return sc; }

template <typename T>
static int head_gate_launch(cudaStream_t s, T* out, const float* o_raw, int n_rows, int heads, int E, float eps, const float* norm,
                            int norm_per_head, const float* gate, long long ldg) {
  THA_CUDA_OK(launch(hyb_head_gate_kernel<T>, dim3(ceil_div(n_rows * heads, 4)), dim3(128), 0, s, false, out, o_raw, n_rows, heads, E, eps, norm,
                     norm_per_head, gate, ldg, 1, (int)THA_GATE_SIGMOID));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_mem_scan(void* stream, int dtype, const tha_mem_t* m, const tha_rows_t* rows, const tha_state_store_t* st,
                                float* proj, long long ldp, float* o_raw, void* out) {
  if (rows->n_seqs < 1) return THA_STATUS_SUCCESS;
  cudaStream_t s = (cudaStream_t)stream;
  THA_CUDA_OK(launch(hyb_mem_gates_kernel, dim3(ceil_div(rows->n_rows * m->heads, 128)), dim3(128), 0, s, false, proj, ldp, rows->n_rows, m->heads,
                     m->o_i, m->o_f, m->b_i, m->b_f, m->gate_cap));
  if (m->dim <= 256 && scan_in_registers()) {
    const dim3 grid(rows->n_seqs, m->heads, ceil_div(m->vdim, SCW * SCAN_WARPS)), block(32 * SCAN_WARPS);
    if (m->dim <= 32) THA_CUDA_OK(launch(hyb_mem_scan_warp_kernel<1>, grid, block, 0, s, false, *m, *rows, *st, proj, ldp, o_raw));
    else if (m->dim <= 64) THA_CUDA_OK(launch(hyb_mem_scan_warp_kernel<2>, grid, block, 0, s, false, *m, *rows, *st, proj, ldp, o_raw));
    else if (m->dim <= 128) THA_CUDA_OK(launch(hyb_mem_scan_warp_kernel<4>, grid, block, 0, s, false, *m, *rows, *st, proj, ldp, o_raw));
    else THA_CUDA_OK(launch(hyb_mem_scan_warp_kernel<8>, grid, block, 0, s, false, *m, *rows, *st, proj, ldp, o_raw));
  } else {
    const int SC = scan_slice(m->vdim), parts = SCAN_THREADS / SC;
    const size_t smem = sizeof(float) * ((size_t)m->dim * SC + m->dim + 2 * (2 * (size_t)m->dim + SC + 2) + (size_t)parts * SC);
    if (smem > 227 * 1024) return THA_STATUS_NOT_SUPPORTED;
    const dim3 grid(rows->n_seqs, m->heads, ceil_div(m->vdim, SC));
    if (smem > 48 * 1024) THA_CUDA_OK(cudaFuncSetAttribute(hyb_mem_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    THA_CUDA_OK(launch(hyb_mem_scan_kernel, grid, dim3(SCAN_THREADS), smem, s, false, *m, *rows, *st, proj, ldp, o_raw, SC));
  }
  const float* gate = proj + m->o_g;
  if (dtype == THA_DT_BF16) return head_gate_launch(s, (bf16*)out, o_raw, rows->n_rows, m->heads, m->vdim, m->eps, m->norm, 1, gate, ldp);
  return head_gate_launch(s, (float*)out, o_raw, rows->n_rows, m->heads, m->vdim, m->eps, m->norm, 1, gate, ldp);
}

extern "C" int tha_hyb_conv(void* stream, int dtype, const tha_rows_t* rows, const tha_state_store_t* st, long long conv_state_off,
                            const float* proj, long long ldp, int col0, int channels, int taps, const float* w, int act, int add_input,
                            int out_f32, void* out) {
  if (rows->n_rows < 1 || channels < 1) return THA_STATUS_SUCCESS;
  if (taps < 1) return THA_STATUS_INVALID_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const bool f32 = out_f32 || dtype == THA_DT_F32;
#define CONV_GO(KF, KB, per)                                                                                                              \
  do {                                                                                                                                    \
    const int gx = ceil_div(ceil_div(channels, per), 128);                                                                               \
    /* about eight blocks per SM: a block walks several rows with its taps in registers */                                               \
    const int gy = min(rows->n_rows, max(1, 148 * 8 / gx));                                                                               \
    const dim3 grid(gx, gy);                                                                                                              \
    if (f32) THA_CUDA_OK(launch(KF, grid, dim3(128), 0, s, false, *rows, *st, conv_state_off, proj, ldp, col0, channels, taps, w, act, add_input, \
                                (float*)out));                                                                                            \
    else THA_CUDA_OK(launch(KB, grid, dim3(128), 0, s, false, *rows, *st, conv_state_off, proj, ldp, col0, channels, taps, w, act, add_input,     \
                            (bf16*)out));                                                                                                 \
  } while (0)
  if (taps > CONV_MAX_TAPS) CONV_GO(hyb_conv_long_kernel<float>, hyb_conv_long_kernel<bf16>, 1);
  else if (channels % 4 == 0 && ldp % 4 == 0 && col0 % 4 == 0 && aligned16(proj) && aligned16(out))
    CONV_GO((hyb_conv_kernel<float, 4>), (hyb_conv_kernel<bf16, 4>), 4);
  else CONV_GO((hyb_conv_kernel<float, 1>), (hyb_conv_kernel<bf16, 1>), 1);
#undef CONV_GO
  return THA_STATUS_SUCCESS;
}
extern "C" int tha_hyb_conv_tail(void* stream, const tha_rows_t* rows, const tha_state_store_t* st, long long conv_state_off,
                                 const float* proj, long long ldp, int col0, int channels, int taps) {
  if (rows->n_rows < 1 || channels < 1 || taps <= 1) return THA_STATUS_SUCCESS;
  THA_CUDA_OK(launch(hyb_conv_tail_kernel, dim3(ceil_div(channels, 128), rows->n_seqs), dim3(128), 0, (cudaStream_t)stream, false, *rows, *st,
                     conv_state_off, proj, ldp, col0, channels, taps));
  return THA_STATUS_SUCCESS;
}
extern "C" int tha_hyb_conv_silu(void* stream, const tha_rows_t* rows, const tha_state_store_t* st, long long conv_state_off,
                                 const float* proj, long long ldp, int col0, int channels, int taps, const float* w, float* out) {
  const int status = tha_hyb_conv(stream, THA_DT_F32, rows, st, conv_state_off, proj, ldp, col0, channels, taps, w, 1, 0, 1, out);
  if (status != THA_STATUS_SUCCESS) return status;
  return tha_hyb_conv_tail(stream, rows, st, conv_state_off, proj, ldp, col0, channels, taps);
}

extern "C" int tha_hyb_delta_scan(void* stream, int dtype, const tha_delta_t* d, const tha_rows_t* rows, const tha_state_store_t* st,
                                  const float* qkv, float* proj, long long ldp, float* dt_raw, const float* gate_raw,
                                  float* o_raw, void* out) {
  if (rows->n_seqs < 1) return THA_STATUS_SUCCESS;
  if (d->heads % d->kv_heads) return THA_STATUS_INVALID_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  {
    const size_t n = (size_t)rows->n_rows * d->heads * d->dim;
    THA_CUDA_OK(launch(hyb_delta_gates_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, false, dt_raw, proj, ldp, rows->n_rows, d->heads,
                       d->dim, d->o_b, d->a_log, d->dt_bias));
  }
  if (d->dim <= 256 && scan_in_registers()) {
    const dim3 grid(rows->n_seqs, d->heads, ceil_div(d->vdim, SCW * SCAN_WARPS)), block(32 * SCAN_WARPS);
    if (d->dim <= 32) THA_CUDA_OK(launch(hyb_delta_scan_warp_kernel<1>, grid, block, 0, s, false, *d, *rows, *st, qkv, proj, ldp, dt_raw, o_raw));
    else if (d->dim <= 64) THA_CUDA_OK(launch(hyb_delta_scan_warp_kernel<2>, grid, block, 0, s, false, *d, *rows, *st, qkv, proj, ldp, dt_raw, o_raw));
    else if (d->dim <= 128) THA_CUDA_OK(launch(hyb_delta_scan_warp_kernel<4>, grid, block, 0, s, false, *d, *rows, *st, qkv, proj, ldp, dt_raw, o_raw));
    else THA_CUDA_OK(launch(hyb_delta_scan_warp_kernel<8>, grid, block, 0, s, false, *d, *rows, *st, qkv, proj, ldp, dt_raw, o_raw));
  } else {
    const int SC = scan_slice(d->vdim), parts = SCAN_THREADS / SC;
    const size_t smem = sizeof(float) * ((size_t)d->dim * SC + 2 * (3 * (size_t)d->dim + SC + 1) + (size_t)parts * SC + SC);
    if (smem > 227 * 1024) return THA_STATUS_NOT_SUPPORTED;
    const dim3 grid(rows->n_seqs, d->heads, ceil_div(d->vdim, SC));
    if (smem > 48 * 1024) THA_CUDA_OK(cudaFuncSetAttribute(hyb_delta_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    THA_CUDA_OK(launch(hyb_delta_scan_kernel, grid, dim3(SCAN_THREADS), smem, s, false, *d, *rows, *st, qkv, proj, ldp, dt_raw, o_raw, SC));
  }
  const long long ldg = (long long)d->heads * d->vdim;
  if (dtype == THA_DT_BF16) return head_gate_launch(s, (bf16*)out, o_raw, rows->n_rows, d->heads, d->vdim, d->eps, d->norm, 0, gate_raw, ldg);
  return head_gate_launch(s, (float*)out, o_raw, rows->n_rows, d->heads, d->vdim, d->eps, d->norm, 0, gate_raw, ldg);
}

extern "C" int tha_hyb_moe_route(void* stream, const tha_moe_t* e, const float* proj, long long ldp, int n_rows, int* expert_id,
                                 float* weight, int* group_off, int* sorted_row, int* inv) {
  if (n_rows < 1) return THA_STATUS_SUCCESS;
  if (e->top < 1 || e->top > 32 || e->top > e->experts) return THA_STATUS_INVALID_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  int* counts = group_off + e->experts + 1;   // the second half of group_off is the routers' counters
  THA_CUDA_OK(cudaMemsetAsync(counts, 0, sizeof(int) * e->experts, s));
  if (e->route == THA_ROUTE_SOFTMAX_GROUPS) {
    const int groups = e->groups > 1 ? e->groups : 1;
    if (e->experts % groups || e->experts > 4096 || e->keep_groups < 1) return THA_STATUS_INVALID_ARG;
    THA_CUDA_OK(launch(hyb_route_groups_kernel, dim3(ceil_div(n_rows, 4)), dim3(128), 0, s, false, e->experts, e->top, groups,
                       e->keep_groups < groups ? e->keep_groups : groups, e->o_router, e->correction, proj, ldp, n_rows, expert_id, weight, counts));
  } else {
    THA_CUDA_OK(launch(hyb_route_kernel, dim3(ceil_div(n_rows, 4)), dim3(128), 0, s, false, e->experts, e->top, e->o_router, proj, ldp, n_rows,
                       expert_id, weight, counts));
  }
  int nt = 64;
  while (nt < 1024 && nt < n_rows * e->top) nt *= 2;
  THA_CUDA_OK(launch(hyb_route_sort_kernel, dim3(e->experts), dim3(nt), 0, s, false, e->experts, e->top, n_rows, (const int*)expert_id,
                     (const int*)counts, group_off, sorted_row, inv));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_ff_act(void* stream, int dtype, int act, void* y, const float* gu, long long ldg, int col_g, int col_u, int n,
                              int ff, float limit, float alpha) {
  if (n < 1 || ff < 1) return THA_STATUS_SUCCESS;
  if (act == THA_ACT_XIELU) {   // the two stored numbers p, q -> the factors the kernel multiplies with
    const float p = limit, q = alpha;
    limit = fmaxf(p, 0.f) + log1pf(expf(-fabsf(p)));
    alpha = 0.5f + fmaxf(q, 0.f) + log1pf(expf(-fabsf(q)));
  }
  cudaStream_t s = (cudaStream_t)stream;
  const bool gated = act != THA_ACT_RELU2 && act != THA_ACT_XIELU;
  if (ff % 4 == 0 && ldg % 4 == 0 && col_u % 4 == 0 && (!gated || col_g % 4 == 0) && aligned16(gu) && n <= 65535) {
    const dim3 grid(ceil_div(ff / 4, 128), n);
    if (dtype == THA_DT_BF16)
      THA_CUDA_OK(launch(hyb_ff_act_vec_kernel<bf16>, grid, dim3(128), 0, s, false, (bf16*)y, gu, ldg, col_g, col_u, ff, act, limit, alpha));
    else
      THA_CUDA_OK(launch(hyb_ff_act_vec_kernel<float>, grid, dim3(128), 0, s, false, (float*)y, gu, ldg, col_g, col_u, ff, act, limit, alpha));
    return THA_STATUS_SUCCESS;
  }
  const dim3 grid((unsigned)(((size_t)n * ff + 255) / 256));
  if (dtype == THA_DT_BF16)
    THA_CUDA_OK(launch(hyb_ff_act_kernel<bf16>, grid, dim3(256), 0, s, false, (bf16*)y, gu, ldg, col_g, col_u, n, ff, act, limit, alpha));
  else
    THA_CUDA_OK(launch(hyb_ff_act_kernel<float>, grid, dim3(256), 0, s, false, (float*)y, gu, ldg, col_g, col_u, n, ff, act, limit, alpha));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_glu_clamped(void* stream, int dtype, void* y, const float* gu, long long ldg, int col_g, int col_u, int n,
                                   int ff, float limit, float alpha) {
  return tha_hyb_ff_act(stream, dtype, THA_ACT_GLU_CLAMPED, y, gu, ldg, col_g, col_u, n, ff, limit, alpha);
}
