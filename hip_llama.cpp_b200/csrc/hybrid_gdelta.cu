// Generalized delta rule (tha_gdelta_t): per head, with a decay w and a removal rate a per key channel and the unit key
// u = k / sqrt(sum(k^2) + 1e-6),
//     S' = diag(w) S - (a o u)(u^T S) + k v^T   (S on the right is the state before the token throughout),   o = S'^T r.
//   hyb_tanh_cols_kernel     the low-rank decay input in place: columns of the stacked projection -> their tanh
//   hyb_gdelta_gates_kernel  all rows at once, in place: z_w + w0 -> w = exp(-exp(-1/2) * sigmoid(z_w + w0)) and the removal
//                            columns of the projection z_a + a_b -> a = sigmoid(z_a + a_b)
//   hyb_gdelta_scan_kernel   the recurrence with the state in registers: a warp owns two value columns of one (sequence,
//                            head), lane l the key channels l, l + 32, ...; per token two rounds of column sums by warp
//                            shuffles (k^T S of the old state beside the key's square sum, then S^T r of the new one); a
//                            token's inputs are fetched ahead into a ring of registers; no barrier.  (A lane owning a run of
//                            consecutive channels, fetched by 128-bit loads, measured 10-30 % slower.)
// The state of a head lies in the slot as [column pair][key channel][2] (a warp's share is one contiguous run).  It is read
// from the sequence's slot before its first row of the step and written back after its last, so a prompt cut anywhere continues
// exactly where it stopped.  Decays, rates, unit keys, state and read-out are fp32 in both number formats; the head norm and
// the sigmoid gate follow in tha_hyb_head_gate.
#include <cuda_bf16.h>
#include <stdlib.h>

#include "common.cuh"
#include "hybrid_ops.cuh"
#include "tha_hybrid.h"

namespace tha {

constexpr int GD_WARPS = 4, GD_COLS = 2;

__global__ void hyb_tanh_cols_kernel(float* __restrict__ proj, long long ldp, int col0, int cols, int n_rows) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_rows * cols) return;
  float* p = proj + (size_t)(i / cols) * ldp + col0 + i % cols;
  *p = tanhf(*p);
}

__global__ void hyb_gdelta_gates_kernel(float* __restrict__ w, float* __restrict__ proj, long long ldp, int o_a, size_t n, int hd,
                                        const float* __restrict__ w0, const float* __restrict__ a_b) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int c = (int)(i % hd);
  w[i] = expf(-0.6065306597126334f * hyb_sigmoid(w[i] + w0[c]));   // exp(-1/2)
  float* a = proj + (i / hd) * ldp + o_a + c;
  *a = hyb_sigmoid(*a + a_b[c]);
}

template <int RPL, int AHEAD>
__global__ void __launch_bounds__(32 * GD_WARPS) hyb_gdelta_scan_kernel(tha_gdelta_t g, tha_rows_t rows, tha_state_store_t st,
                                                                        const float* __restrict__ proj, long long ldp,
                                                                        const float* __restrict__ decay, float* __restrict__ o_raw) {
  const int s = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int D = g.dim;
  const int pair = blockIdx.z * GD_WARPS + warp, e0 = pair * GD_COLS;
  if (e0 >= D) return;
  const int EP = (D + GD_COLS - 1) / GD_COLS * GD_COLS;
  float* gstate = st.base + (size_t)rows.seq_slot[s] * st.slot_floats + g.state_off + (size_t)h * D * EP + (size_t)pair * D * GD_COLS;
  float S[RPL][GD_COLS];
#pragma unroll
  for (int i = 0; i < RPL; i++) {
    const int d = lane + 32 * i;
#pragma unroll
    for (int c = 0; c < GD_COLS; c++) S[i][c] = (d < D && e0 + c < D) ? gstate[(size_t)d * GD_COLS + c] : 0.f;
  }
  const int r_begin = rows.seq_first[s], r_end = rows.seq_first[s + 1];
  struct In { float r[RPL], k[RPL], w[RPL], a[RPL], v[GD_COLS]; };
  In ring[AHEAD];
  auto fetch = [&](int row, In& in) {
    const float* x = proj + (size_t)row * ldp;
#pragma unroll
    for (int i = 0; i < RPL; i++) {
      const int d = lane + 32 * i;
      in.r[i] = d < D ? x[g.o_r + h * D + d] : 0.f;
      in.k[i] = d < D ? x[g.o_k + h * D + d] : 0.f;
      in.a[i] = d < D ? x[g.o_a + h * D + d] : 0.f;
      in.w[i] = d < D ? decay[(size_t)row * g.heads * D + h * D + d] : 0.f;
    }
#pragma unroll
    for (int c = 0; c < GD_COLS; c++) in.v[c] = e0 + c < D ? x[g.o_v + h * D + e0 + c] : 0.f;
  };
#pragma unroll
  for (int u = 0; u < AHEAD; u++)
    if (r_begin + u < r_end) fetch(r_begin + u, ring[u]);
  // One token.  With ks = k^T S (per column) and kk = k^T k, both of the old state and summed over the warp side by side,
  // u^T S = ks / sqrt(kk + 1e-6) and the removal term (a * u) (u^T S) = a * k * ks / (kk + 1e-6): the only sums on the path from
  // one token's state to the next are the columns' ks.
  auto token = [&](int row, In& in, int refill) {
    float cr[RPL], ck[RPL], cw[RPL], ca[RPL], cv[GD_COLS], ks[GD_COLS];
    float kk = 0.f;
#pragma unroll
    for (int c = 0; c < GD_COLS; c++) { cv[c] = in.v[c]; ks[c] = 0.f; }
#pragma unroll
    for (int i = 0; i < RPL; i++) {
      cr[i] = in.r[i]; ck[i] = in.k[i]; cw[i] = in.w[i]; ca[i] = in.a[i];
      kk = fmaf(ck[i], ck[i], kk);
#pragma unroll
      for (int c = 0; c < GD_COLS; c++) ks[c] = fmaf(ck[i], S[i][c], ks[c]);
    }
    if (refill >= 0) fetch(refill, in);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      kk += __shfl_xor_sync(THA_FULL_MASK, kk, off);
#pragma unroll
      for (int c = 0; c < GD_COLS; c++) ks[c] += __shfl_xor_sync(THA_FULL_MASK, ks[c], off);
    }
    const float inv2 = 1.0f / (kk + 1e-6f);
    float o[GD_COLS];
#pragma unroll
    for (int c = 0; c < GD_COLS; c++) { ks[c] *= inv2; o[c] = 0.f; }
#pragma unroll
    for (int i = 0; i < RPL; i++)
#pragma unroll
      for (int c = 0; c < GD_COLS; c++) {
        S[i][c] = fmaf(cw[i], S[i][c], ck[i] * fmaf(-ca[i], ks[c], cv[c]));
        o[c] = fmaf(S[i][c], cr[i], o[c]);
      }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
#pragma unroll
      for (int c = 0; c < GD_COLS; c++) o[c] += __shfl_xor_sync(THA_FULL_MASK, o[c], off);
#pragma unroll
    for (int c = 0; c < GD_COLS; c++)
      if (lane == c && e0 + c < D) o_raw[(size_t)row * g.heads * D + (size_t)h * D + e0 + c] = o[c];
  };
  int rb = r_begin;
  for (; rb + AHEAD <= r_end; rb += AHEAD) {
#pragma unroll
    for (int u = 0; u < AHEAD; u++) token(rb + u, ring[u], min(rb + u + AHEAD, r_end - 1));
  }
#pragma unroll
  for (int u = 0; u < AHEAD; u++)
    if (rb + u < r_end) token(rb + u, ring[u], -1);
#pragma unroll
  for (int i = 0; i < RPL; i++) {
    const int d = lane + 32 * i;
    if (d >= D) continue;
#pragma unroll
    for (int c = 0; c < GD_COLS; c++)
      if (e0 + c < D) gstate[(size_t)d * GD_COLS + c] = S[i][c];
  }
}

}  // namespace tha

using namespace tha;

extern "C" long long tha_hyb_gdelta_state_floats(int heads, int dim) {
  return (long long)heads * dim * ((dim + GD_COLS - 1) / GD_COLS * GD_COLS);
}

extern "C" int tha_hyb_gdelta_scan(void* stream, int dtype, const tha_gdelta_t* g, const tha_rows_t* rows, const tha_state_store_t* st,
                                   float* proj, long long ldp, float* w_raw, float* o_raw, void* out) {
  if (rows->n_seqs < 1 || rows->n_rows < 1) return THA_STATUS_SUCCESS;
  if (g->heads < 1 || g->dim < 1 || g->rank < 1) return THA_STATUS_INVALID_ARG;
  if (g->dim > 256) return THA_STATUS_NOT_SUPPORTED;   // 8 key channels per lane is the widest register form
  cudaStream_t s = (cudaStream_t)stream;
  const int R = rows->n_rows, HD = g->heads * g->dim;
  THA_CUDA_OK(launch(hyb_tanh_cols_kernel, dim3(ceil_div(R * g->rank, 256)), dim3(256), 0, s, false, proj, ldp, g->o_w1, g->rank, R));
  const int st1 = tha_hyb_linear(stream, dtype, w_raw, HD, proj + g->o_w1, ldp, 1, nullptr, g->w_w2, 0, R, HD, g->rank, nullptr, 0);
  if (st1 != THA_STATUS_SUCCESS) return st1;
  const size_t n = (size_t)R * HD;
  THA_CUDA_OK(launch(hyb_gdelta_gates_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, false, w_raw, proj, ldp, g->o_a, n, HD, g->w0,
                     g->a_b));
  const dim3 grid(rows->n_seqs, g->heads, ceil_div(g->dim, GD_COLS * GD_WARPS)), block(32 * GD_WARPS);
#define GD_LAUNCH(RPL, A) \
  THA_CUDA_OK(launch(hyb_gdelta_scan_kernel<RPL, A>, grid, block, 0, s, false, *g, *rows, *st, (const float*)proj, ldp, (const float*)w_raw, o_raw))
  // tokens fetched ahead: two at 65 .. 128 key channels (measured: four 4 % slower, eight spill), four below
  if (g->dim <= 32) GD_LAUNCH(1, 4);
  else if (g->dim <= 64) GD_LAUNCH(2, 4);
  else if (g->dim <= 128) GD_LAUNCH(4, 2);
  else GD_LAUNCH(8, 1);
#undef GD_LAUNCH
  return tha_hyb_head_gate(stream, dtype, out, o_raw, R, g->heads, g->dim, 1, g->eps, g->norm, 1, proj + g->o_g, ldp, THA_GATE_SIGMOID);
}
