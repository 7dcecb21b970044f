// Latent attention (tha_latent_t): what surrounds the products and the attention kernel.
//   hyb_latent_prepare_kernel   per row: the query latent's rms norm (dtype-typed, input of the query expansion); the
//                               key/value latent's rms norm and the rotation of the shared key part, written as ONE cache
//                               row [latent | rotated part] of the K pool
//   hyb_latent_split_q_kernel   per row and head: the plain query part as the input of the per-head product with the
//                               transposed key expansion; the rotated part, rotated, behind it in the absorbed query
// The attention itself is tha_hyb_attn with one key/value head whose values are the first kv_rank channels of its keys.
// Norms, rotation and the cache are fp32 in both number formats.
#include <cuda_bf16.h>
#include <stdlib.h>

#include "common.cuh"
#include "hybrid_ops.cuh"
#include "tha_hybrid.h"

namespace tha {

template <typename T>
__global__ void hyb_latent_prepare_kernel(tha_latent_t a, tha_rows_t rows, tha_kv_t kv, const float* __restrict__ proj, long long ldp,
                                          const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dims, T* __restrict__ cq) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* pr = proj + (size_t)r * ldp;
  // query latent (models whose queries come straight from the stacked projection have none)
  float ss = 0.f, inv = 1.f;
  if (!a.direct_q) {
    for (int i = threadIdx.x; i < a.q_rank; i += blockDim.x) { const float v = pr[a.o_dq + i]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    inv = 1.0f / sqrtf(ss / (float)a.q_rank + a.eps);
    for (int i = threadIdx.x; i < a.q_rank; i += blockDim.x) hyb_store(cq + (size_t)r * a.q_rank + i, pr[a.o_dq + i] * inv * a.q_norm[i]);
  }
  // key/value latent -> cache row
  const int slot = rows.seq_slot[rows.row_seq[r]], t = rows.pos[r];
  float* krow = kv.k_pool + hyb_kv_row(kv, slot, t, a.cache_layer);
  ss = 0.f;
  for (int i = threadIdx.x; i < a.kv_rank; i += blockDim.x) { const float v = pr[a.o_dkv + i]; ss = fmaf(v, v, ss); }
  ss = block_sum(ss, red);
  inv = 1.0f / sqrtf(ss / (float)a.kv_rank + a.eps);
  for (int i = threadIdx.x; i < a.kv_rank; i += blockDim.x) krow[i] = pr[a.o_dkv + i] * inv * a.kv_norm[i];
  // the shared key part: its first rot_dims entries rotated, the rest passed through
  const float* kr = pr + a.o_dkv + a.kv_rank;
  const int half = rot_dims / 2;
  for (int i = threadIdx.x; i < a.rot_dim; i += blockDim.x)
    krow[a.kv_rank + i] = hyb_rotated(kr, i, rot_dims, a.rot_layout, cos_t + (size_t)r * half, sin_t + (size_t)r * half);
}

template <typename T>
__global__ void hyb_latent_split_q_kernel(tha_latent_t a, int n_rows, const float* __restrict__ qfull, long long ldq, const float* __restrict__ cos_t,
                                          const float* __restrict__ sin_t, int rot_dims, T* __restrict__ q_plain, float* __restrict__ q_abs) {
  const int r = blockIdx.x;
  const int per = a.dim + a.rot_dim, DA = a.kv_rank + a.rot_dim, half = rot_dims / 2;
  const float* q = qfull + (size_t)r * ldq;
  for (int i = threadIdx.x; i < a.heads * a.dim; i += blockDim.x) {
    const int h = i / a.dim, d = i - h * a.dim;
    hyb_store(q_plain + (size_t)r * a.heads * a.dim + i, q[h * per + d]);
  }
  for (int i = threadIdx.x; i < a.heads * a.rot_dim; i += blockDim.x) {
    const int h = i / a.rot_dim, d = i - h * a.rot_dim;
    q_abs[(size_t)r * a.heads * DA + (size_t)h * DA + a.kv_rank + d] =
        hyb_rotated(q + h * per + a.dim, d, rot_dims, a.rot_layout, cos_t + (size_t)r * half, sin_t + (size_t)r * half);
  }
}


// ------------------------------------------------------------------------------------------------------------------
// Tensor-core attention for WIDE key rows whose values are their first vdim channels (the absorbed form of latent
// attention: 512 + 64 channels at full size).  Neither a query row nor a row of the output fits a warp's registers at
// that width, so a block shares them: 16 * MT (position, query head) pairs, 4 * MT warps; warp (mi, ei) owns row tile
// mi (16 pairs) and slice ei of four.  Per tile of 32 keys (aligned to absolute multiples of 32, like the other forms):
//   1. the tile's key rows go to shared memory once, as bf16 -- they are also the values;
//   2. warp (mi, ei): scores of its 16 pairs against the 32 keys over a quarter of the channels (mma.sync m16n8k16; the
//      query fragment and the key fragments of two 8-key tiles come from shared memory by ldmatrix.x4), written to shared
//      memory in fp32 as one of four shares;
//   3. a warp takes 4 pairs (lane = key): sum of the shares in a fixed order, scale, mask, running maximum and sum in
//      fp32, weights rounded to bf16 (the sums add the rounded weights), the rescale factor of each pair;
//   4. warp (mi, ei): rescales its accumulators [16 pairs, vdim / 4 channels] and adds weights x values; the value
//      fragments come out of the row-major key tile through ldmatrix.trans.
// Three block barriers per tile.  Splits along the keys and their merge as in the other forms.
// ------------------------------------------------------------------------------------------------------------------
constexpr int WK_KEYS = 32, WK_MAX_SLICE = 128;   // channels of the output per warp: vdim <= 512

__device__ __forceinline__ void mma_bf16_m16n8k16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

template <int MT>
__global__ void __launch_bounds__(128 * MT) hyb_attn_wide_kernel(tha_attn_t a, tha_rows_t rows, tha_kv_t kv, const float* __restrict__ q,
                                                                 __nv_bfloat16* __restrict__ out, int AG, int AP, int splits,
                                                                 float* __restrict__ partial) {
  constexpr int PAIRS = 16 * MT, NW = 4 * MT;
  extern __shared__ __align__(16) unsigned char smraw[];
  const int D = a.dim, E = a.vdim, gsize = a.heads / a.kv_heads, ES = E / 4;
  const int DS = D + 8;                                   // padded rows: conflict-free fragment and ldmatrix reads
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw);          // [PAIRS][DS]
  __nv_bfloat16* Ks = Qs + (size_t)PAIRS * DS;                             // [32][DS]
  __nv_bfloat16* Pb = Ks + (size_t)WK_KEYS * DS;                           // [PAIRS][40] weights
  __nv_bfloat16* Pl = Pb + PAIRS * 40;                                     // [PAIRS][40] what their rounding to bf16 left over
  float* Sf = reinterpret_cast<float*>(Pl + PAIRS * 40);                   // [4][PAIRS][33] partial scores
  float* corr_s = Sf + 4 * PAIRS * 33;                                       // [PAIRS] rescale factors, then 1 / sum
  float* m_s = corr_s + PAIRS;                                             // [PAIRS] running maxima at the end
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
  const int slot = rows.seq_slot[seq];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int mi = warp >> 2, ei = warp & 3;
  const int p_first = rows.pos[r0], p_last = p_first + (r_end - r0) - 1;
  const int lr = lane >> 2, lc = (lane & 3) * 2;
  // pair pr of the block: position r0 + pr / AG, head g * gsize + part * AG + pr % AG
  auto pair_row = [&](int pr) { return r0 + pr / AG; };
  auto pair_head = [&](int pr) { return g * gsize + part * AG + pr % AG; };
  auto pair_ok = [&](int pr) { return pr / AG < AP && r0 + pr / AG < r_end && part * AG + pr % AG < gsize; };
  // queries -> shared memory (bf16), rows of absent pairs zero
  for (int pr = warp; pr < PAIRS; pr += NW) {
    const bool ok = pair_ok(pr);
    const float* qr = q + (size_t)(ok ? pair_row(pr) : 0) * a.heads * D + (size_t)(ok ? pair_head(pr) : 0) * D;
    for (int d = lane; d < D; d += 32) Qs[(size_t)pr * DS + d] = __float2bfloat16_rn(ok ? qr[d] : 0.f);
  }
  // the softmax state of this warp's 4 pairs (identical in every lane)
  float m_run[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY}, l_run[4] = {0.f, 0.f, 0.f, 0.f};
  int s_pos[4];
  bool s_ok[4];
#pragma unroll
  for (int rr = 0; rr < 4; rr++) {
    const int pr = warp * 4 + rr;
    s_ok[rr] = pair_ok(pr);
    s_pos[rr] = p_first + pr / AG;
  }
  float oacc[WK_MAX_SLICE / 8][4];
#pragma unroll
  for (int n = 0; n < WK_MAX_SLICE / 8; n++)
#pragma unroll
    for (int v = 0; v < 4; v++) oacc[n][v] = 0.f;
  const bool exact = a.fp32_scores != 0;
  const HybTiles tiles = hyb_attn_tiles(a, 0, p_first, p_last);
  int ti_begin = 0, ti_end = tiles.n;
  if (splits > 1) {
    const int per = (tiles.n + splits - 1) / splits, sp = blockIdx.x % splits;
    ti_begin = sp * per;
    ti_end = min(tiles.n, ti_begin + per);
  }
  // cache rows start on 16-byte boundaries when the pool's row pitch and the head's offset are multiples of four floats
  const bool vec4 = (kv.kv_dim & 3) == 0 && (D & 3) == 0 && (reinterpret_cast<size_t>(kv.k_pool) & 15) == 0;
  const unsigned ks_base = (unsigned)__cvta_generic_to_shared(Ks), qs_base = (unsigned)__cvta_generic_to_shared(Qs);
  for (int ti = ti_begin; ti < ti_end; ti++) {
    const int kt = ti < tiles.n_a ? tiles.begin + WK_KEYS * ti : tiles.resume + WK_KEYS * (ti - tiles.n_a);
    __syncthreads();   // the previous tile's weights and values have been used (first pass: the queries are in place)
    // 1. the tile's key rows; keys past the last position of the block are zero
    for (int j = warp; j < WK_KEYS; j += NW) {
      const int t = kt + j;
      const bool live = t <= p_last;
      const float* src = kv.k_pool + (live ? hyb_kv_row(kv, slot, t, a.cache_layer) : 0) + (size_t)g * D;
      if (vec4) {   // 16-byte aligned rows: five 128-bit loads per lane in flight, four bf16 per store
        const float4* src4 = reinterpret_cast<const float4*>(src);
        const int D4 = D >> 2;
        for (int i0 = 0; i0 < D4; i0 += 160) {
          float4 buf[5];
#pragma unroll
          for (int c = 0; c < 5; c++) { const int i = i0 + lane + 32 * c; buf[c] = (live && i < D4) ? __ldg(src4 + i) : make_float4(0.f, 0.f, 0.f, 0.f); }
#pragma unroll
          for (int c = 0; c < 5; c++) {
            const int i = i0 + lane + 32 * c;
            if (i < D4) {
              uint2 pk;
              pk.x = pack2_bf16(buf[c].x, buf[c].y);
              pk.y = pack2_bf16(buf[c].z, buf[c].w);
              *reinterpret_cast<uint2*>(Ks + (size_t)j * DS + 4 * i) = pk;
            }
          }
        }
      } else {
        for (int d0 = 0; d0 < D; d0 += 320) {   // ten loads per lane in flight
          float buf[10];
#pragma unroll
          for (int c = 0; c < 10; c++) { const int d = d0 + lane + 32 * c; buf[c] = (live && d < D) ? __ldg(src + d) : 0.f; }
#pragma unroll
          for (int c = 0; c < 10; c++) { const int d = d0 + lane + 32 * c; if (d < D) Ks[(size_t)j * DS + d] = __float2bfloat16_rn(buf[c]); }
        }
      }
    }
    __syncthreads();
    // 2. partial scores of row tile mi against all 32 keys over this warp's share of the channels (k steps ei, ei + 4, ...);
    //    a whole query fragment and the key fragments of two 8-key tiles per ldmatrix
    {
      float sacc[4][4];
#pragma unroll
      for (int j = 0; j < 4; j++)
#pragma unroll
        for (int v = 0; v < 4; v++) sacc[j][v] = 0.f;
      const unsigned a_addr = qs_base + (unsigned)(((size_t)(mi * 16 + (lane & 15)) * DS + (lane >> 4) * 8) * sizeof(__nv_bfloat16));
      const unsigned b_addr = ks_base + (unsigned)(((size_t)((lane & 7) + ((lane >> 4) << 3)) * DS + ((lane >> 3) & 1) * 8) * sizeof(__nv_bfloat16));
      for (int ks = ei; ks < D / 16; ks += 4) {
        uint32_t af[4];
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                     : "=r"(af[0]), "=r"(af[1]), "=r"(af[2]), "=r"(af[3]) : "r"(a_addr + ks * 32));
#pragma unroll
        for (int j2 = 0; j2 < 2; j2++) {
          uint32_t bq[4];
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                       : "=r"(bq[0]), "=r"(bq[1]), "=r"(bq[2]), "=r"(bq[3])
                       : "r"(b_addr + (unsigned)(j2 * 16 * DS * sizeof(__nv_bfloat16)) + ks * 32));
          const uint32_t b0[2] = {bq[0], bq[1]}, b1[2] = {bq[2], bq[3]};
          mma_bf16_m16n8k16(sacc[2 * j2], af, b0);
          mma_bf16_m16n8k16(sacc[2 * j2 + 1], af, b1);
        }
      }
      float* sr = Sf + (size_t)ei * PAIRS * 33 + (mi * 16 + lr) * 33 + lc;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        sr[8 * j] = sacc[j][0]; sr[8 * j + 1] = sacc[j][1];
        sr[8 * 33 + 8 * j] = sacc[j][2]; sr[8 * 33 + 8 * j + 1] = sacc[j][3];
      }
    }
    __syncthreads();
    // 3. online softmax of this warp's 4 pairs, lane = key
#pragma unroll
    for (int rr = 0; rr < 4; rr++) {
      const int pr = warp * 4 + rr, t = kt + lane;
      const bool vis = s_ok[rr] && hyb_attn_sees(a, t, s_pos[rr], 0);
      const float* sp = Sf + pr * 33 + lane;   // the four channel shares, summed in a fixed order
      const float sv = vis ? ((sp[0] + sp[PAIRS * 33]) + (sp[2 * PAIRS * 33] + sp[3 * PAIRS * 33])) * a.scale : -INFINITY;
      const float m_new = fmaxf(m_run[rr], warp_max(sv));
      float p = 0.f, corr = 1.f;
      if (m_new > -INFINITY) {
        p = vis ? expf(sv - m_new) : 0.f;
        corr = expf(m_run[rr] - m_new);      // 0 when nothing was seen before
      }
      const __nv_bfloat16 pb = __float2bfloat16_rn(p);
      // exact: the sum adds the fp32 weights, and hi + lo (16 mantissa bits) meet the values; else the rounded weights do both
      l_run[rr] = l_run[rr] * corr + warp_sum(exact ? p : __bfloat162float(pb));
      m_run[rr] = m_new;
      Pb[pr * 40 + lane] = pb;
      if (exact) Pl[pr * 40 + lane] = __float2bfloat16_rn(p - __bfloat162float(pb));
      if (lane == 0) corr_s[pr] = corr;
    }
    __syncthreads();
    // 4. accumulators of row tile mi, channels ei * ES ..: rescale, then weights x values
    {
      const float ca = corr_s[mi * 16 + lr], cb = corr_s[mi * 16 + lr + 8];
      uint32_t pf[2][4], pg[2][4];
      const __nv_bfloat16* pa = Pb + (mi * 16 + lr) * 40 + lc;
      const __nv_bfloat16* pc = Pl + (mi * 16 + lr) * 40 + lc;
#pragma unroll
      for (int t2 = 0; t2 < 2; t2++) {
        pf[t2][0] = *reinterpret_cast<const uint32_t*>(pa + 16 * t2);
        pf[t2][1] = *reinterpret_cast<const uint32_t*>(pa + 8 * 40 + 16 * t2);
        pf[t2][2] = *reinterpret_cast<const uint32_t*>(pa + 16 * t2 + 8);
        pf[t2][3] = *reinterpret_cast<const uint32_t*>(pa + 8 * 40 + 16 * t2 + 8);
        if (exact) {
          pg[t2][0] = *reinterpret_cast<const uint32_t*>(pc + 16 * t2);
          pg[t2][1] = *reinterpret_cast<const uint32_t*>(pc + 8 * 40 + 16 * t2);
          pg[t2][2] = *reinterpret_cast<const uint32_t*>(pc + 16 * t2 + 8);
          pg[t2][3] = *reinterpret_cast<const uint32_t*>(pc + 8 * 40 + 16 * t2 + 8);
        }
      }
#pragma unroll
      for (int n = 0; n < WK_MAX_SLICE / 8; n += 2) {
        if (8 * n < ES) {
          const bool two = 8 * (n + 1) < ES;
          oacc[n][0] *= ca; oacc[n][1] *= ca; oacc[n][2] *= cb; oacc[n][3] *= cb;
          if (two) { oacc[n + 1][0] *= ca; oacc[n + 1][1] *= ca; oacc[n + 1][2] *= cb; oacc[n + 1][3] *= cb; }
#pragma unroll
          for (int t2 = 0; t2 < 2; t2++) {
            // values [key][channel] row-major, transposed on the way: lanes 0..15 name the rows of keys 16 t2 + (lane & 15) at
            // this channel tile, lanes 16..31 the same keys at the next one (an odd last tile reads its own twice)
            uint32_t vf[4];
            const int ch = ei * ES + 8 * n + ((two && lane >= 16) ? 8 : 0);
            const unsigned addr = ks_base + (unsigned)(((size_t)(16 * t2 + (lane & 15)) * DS + ch) * sizeof(__nv_bfloat16));
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                         : "=r"(vf[0]), "=r"(vf[1]), "=r"(vf[2]), "=r"(vf[3]) : "r"(addr));
            const uint32_t v0[2] = {vf[0], vf[1]}, v1[2] = {vf[2], vf[3]};
            mma_bf16_m16n8k16(oacc[n], pf[t2], v0);
            if (two) mma_bf16_m16n8k16(oacc[n + 1], pf[t2], v1);
            if (exact) {
              mma_bf16_m16n8k16(oacc[n], pg[t2], v0);
              if (two) mma_bf16_m16n8k16(oacc[n + 1], pg[t2], v1);
            }
          }
        }
      }
    }
  }
  // the sums and maxima of the pairs, for the warps that hold their accumulators
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int rr = 0; rr < 4; rr++) { corr_s[warp * 4 + rr] = l_run[rr]; m_s[warp * 4 + rr] = m_run[rr]; }
  }
  __syncthreads();
#pragma unroll
  for (int x = 0; x < 2; x++) {
    const int pr = mi * 16 + lr + 8 * x;
    if (!pair_ok(pr)) continue;
    const int row = pair_row(pr), head = pair_head(pr);
    const float l = corr_s[pr];
    if (splits > 1) {
      float* dst = partial + (((size_t)(blockIdx.x % splits) * rows.n_rows + row) * a.heads + head) * (E + 2);
#pragma unroll
      for (int n = 0; n < WK_MAX_SLICE / 8; n++)
        if (8 * n < ES) { dst[ei * ES + 8 * n + lc] = oacc[n][2 * x]; dst[ei * ES + 8 * n + lc + 1] = oacc[n][2 * x + 1]; }
      if (ei == 0 && (lane & 3) == 0) { dst[E] = m_s[pr]; dst[E + 1] = l; }
      continue;
    }
    const float inv = hyb_attn_final_factor(a, head, m_s[pr], l, nullptr);
    __nv_bfloat16* dst = out + (size_t)row * a.heads * E + (size_t)head * E + ei * ES;
#pragma unroll
    for (int n = 0; n < WK_MAX_SLICE / 8; n++)
      if (8 * n < ES) *reinterpret_cast<__nv_bfloat162*>(dst + 8 * n + lc) = __floats2bfloat162_rn(oacc[n][2 * x] * inv, oacc[n][2 * x + 1] * inv);
  }
}

static size_t wide_smem(const tha_attn_t* a, int pairs) {
  return sizeof(__nv_bfloat16) * ((size_t)(pairs + WK_KEYS) * (a->dim + 8) + (size_t)2 * pairs * 40) + sizeof(float) * ((size_t)4 * pairs * 33 + 2 * pairs);
}

// one key/value head, key rows a multiple of 16 wide, values inside them, four slices of at most 128 channels that are multiples of 8, no
// block-of-positions mask (a window and a sink are served; per-head factors and gates are not), and the larger block must fit shared memory
bool hyb_attn_wide_ok(const tha_attn_t* a) {
  return a->values_in_keys && a->kv_heads == 1 && a->chunk == 0 && a->dim % 16 == 0 && a->vdim % 32 == 0 && a->vdim <= 4 * WK_MAX_SLICE && a->vdim <= a->dim &&
         (a->heads * a->vdim) % 2 == 0 && wide_smem(a, 64) <= 200 * 1024;
}
// 64 pairs per block when the step has prompt portions that fill them, else 16
int hyb_attn_wide_pairs(const tha_attn_t* a, const tha_rows_t* rows) {
  static int forced = -1;   // THA_WIDE_PAIRS=16|32|64 fixes the block size (A/B aid)
  if (forced < 0) { const char* v = getenv("THA_WIDE_PAIRS"); forced = (v && *v) ? atoi(v) : 0; }
  if (forced == 16 || forced == 32 || forced == 64) return forced;
  const long long per_seq = (long long)rows->max_seq_rows * (a->heads / a->kv_heads);
  return per_seq >= 64 ? 64 : 16;
}
int hyb_attn_wide_launch(cudaStream_t s, const tha_attn_t* a, const tha_rows_t* rows, const tha_kv_t* kv, const float* q, __nv_bfloat16* out,
                         dim3 grid, int pairs, int AG, int AP, int splits, float* partial) {
  const size_t smem = wide_smem(a, pairs);
  if (pairs == 64) {
    THA_CUDA_OK(cudaFuncSetAttribute(hyb_attn_wide_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    THA_CUDA_OK(launch(hyb_attn_wide_kernel<4>, grid, dim3(512), smem, s, false, *a, *rows, *kv, q, out, AG, AP, splits, partial));
  } else if (pairs == 32) {
    THA_CUDA_OK(cudaFuncSetAttribute(hyb_attn_wide_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    THA_CUDA_OK(launch(hyb_attn_wide_kernel<2>, grid, dim3(256), smem, s, false, *a, *rows, *kv, q, out, AG, AP, splits, partial));
  } else {
    THA_CUDA_OK(cudaFuncSetAttribute(hyb_attn_wide_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    THA_CUDA_OK(launch(hyb_attn_wide_kernel<1>, grid, dim3(128), smem, s, false, *a, *rows, *kv, q, out, AG, AP, splits, partial));
  }
  return THA_STATUS_SUCCESS;
}

}  // namespace tha

using namespace tha;
typedef __nv_bfloat16 bf16;

extern "C" int tha_hyb_latent_prepare(void* stream, int dtype, const tha_latent_t* a, const tha_rows_t* rows, const tha_kv_t* kv,
                                      const float* proj, long long ldp, const float* cos_t, const float* sin_t, int rot_dims, void* cq) {
  if (rows->n_rows < 1) return THA_STATUS_SUCCESS;
  if (rot_dims > a->rot_dim || (rot_dims & 1) || a->kv_rank + a->rot_dim > kv->kv_dim || (!a->direct_q && a->q_rank < 1) || a->kv_rank < 1 ||
      (rot_dims > 0 && (!cos_t || !sin_t)))
    return THA_STATUS_INVALID_ARG;
  int nt = 64;
  while (nt < a->kv_rank / 2 && nt < 256) nt += 32;
  if (dtype == THA_DT_BF16)
    THA_CUDA_OK(launch(hyb_latent_prepare_kernel<bf16>, dim3(rows->n_rows), dim3(nt), 0, (cudaStream_t)stream, false, *a, *rows, *kv, proj, ldp,
                       cos_t, sin_t, rot_dims, (bf16*)cq));
  else
    THA_CUDA_OK(launch(hyb_latent_prepare_kernel<float>, dim3(rows->n_rows), dim3(nt), 0, (cudaStream_t)stream, false, *a, *rows, *kv, proj, ldp,
                       cos_t, sin_t, rot_dims, (float*)cq));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_latent_split_q(void* stream, int dtype, const tha_latent_t* a, int n_rows, const float* qfull, long long ldq,
                                      const float* cos_t, const float* sin_t, int rot_dims, void* q_plain, float* q_abs) {
  if (n_rows < 1) return THA_STATUS_SUCCESS;
  if (ldq <= 0) ldq = (long long)a->heads * (a->dim + a->rot_dim);
  if (rot_dims > a->rot_dim || (rot_dims & 1) || (rot_dims > 0 && (!cos_t || !sin_t))) return THA_STATUS_INVALID_ARG;
  int nt = 64;
  while (nt < a->heads * a->dim / 2 && nt < 256) nt += 32;
  if (dtype == THA_DT_BF16)
    THA_CUDA_OK(launch(hyb_latent_split_q_kernel<bf16>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, *a, n_rows, qfull, ldq, cos_t, sin_t,
                       rot_dims, (bf16*)q_plain, q_abs));
  else
    THA_CUDA_OK(launch(hyb_latent_split_q_kernel<float>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, *a, n_rows, qfull, ldq, cos_t, sin_t,
                       rot_dims, (float*)q_plain, q_abs));
  return THA_STATUS_SUCCESS;
}
