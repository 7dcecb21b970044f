// Gated linear attention (tha_gla_t): per head S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t / sqrt(dim).
//   hyb_gla_decay_kernel   all rows at once, in place: z + b -> a = sigmoid(z + b)^(1/tau) = exp(-softplus(-(z + b)) / tau)
//   hyb_gla_scan_kernel    the recurrence with the state in registers: a warp owns GLA_COLS value columns of one
//                          (sequence, head), lane l the key channels l, l + 32, ...; the column sums S^T q are warp
//                          shuffles, a token's inputs are fetched several tokens ahead into a ring of registers; no barrier.
//                          The state of a head lies in the slot as [column pair][key channel][2] (a warp's share is one
//                          contiguous run).  It is read from the sequence's slot before its first row of the step and written back
//                          after its last, so a prompt cut anywhere continues exactly where it stopped.
// Decays, state and read-out are fp32 in both number formats; the head norm and the silu gate follow in
// tha_hyb_head_gate.
#include <cuda_bf16.h>
#include <stdlib.h>

#include "common.cuh"
#include "hybrid_ops.cuh"
#include "tha_hybrid.h"

namespace tha {

constexpr int GLA_WARPS = 4, GLA_STATE_PAD = 8;   // a head's value columns are padded to a multiple of 8 in the slot

__global__ void hyb_gla_decay_kernel(float* __restrict__ z, size_t n, int hd, const float* __restrict__ bias, float inv_tau) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = z[i] + (bias ? bias[i % hd] : 0.f);
  z[i] = expf(-hyb_softplus(-v) * inv_tau);
}

__global__ void hyb_hgrn_gates_kernel(float* __restrict__ proj, long long ldp, float* __restrict__ decay, size_t n, int hd, int o_q, int o_f,
                                      const float* __restrict__ f_b, const float* __restrict__ lower) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const size_t r = i / hd;
  const int c = (int)(i - r * hd);
  float* row = proj + r * ldp;
  const float q = row[o_q + c];
  row[o_q + c] = q * hyb_sigmoid(q);
  const float z = row[o_f + c] + f_b[c], lo = lower[c];
  const float open = (1.0f - lo) * hyb_sigmoid(-z);   // 1 - f
  decay[i] = 1.0f - open;
  row[o_f + c] = open;
}

template <int RPL, int AHEAD, int GLA_COLS>
__global__ void __launch_bounds__(32 * GLA_WARPS) hyb_gla_scan_kernel(tha_gla_t g, tha_rows_t rows, tha_state_store_t st,
                                                                      const float* __restrict__ proj, long long ldp,
                                                                      const float* __restrict__ decay, float* __restrict__ o_raw, float qscale) {
  const int s = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int D = g.dim, E = g.vdim;
  const int e0 = (blockIdx.z * GLA_WARPS + warp) * GLA_COLS;
  if (e0 >= E) return;
  // the head's state as [column pair][key channel][2]: a warp's share is one contiguous run, a lane's two columns adjacent
  const int EP = (E + GLA_STATE_PAD - 1) / GLA_STATE_PAD * GLA_STATE_PAD;
  float* gstate = st.base + (size_t)rows.seq_slot[s] * st.slot_floats + g.state_off + (size_t)h * D * EP + (size_t)(e0 / GLA_COLS) * D * GLA_COLS;
  float S[RPL][GLA_COLS];
#pragma unroll
  for (int i = 0; i < RPL; i++) {
    const int d = lane + 32 * i;
#pragma unroll
    for (int c = 0; c < GLA_COLS; c++) S[i][c] = (d < D && e0 + c < E) ? gstate[(size_t)d * GLA_COLS + c] : 0.f;
  }
  const int r_begin = rows.seq_first[s], r_end = rows.seq_first[s + 1];
  // a token's inputs are loaded AHEAD tokens before they are used (a ring of register sets, the loop unrolled over it)
  struct In { float q[RPL], k[RPL], a[RPL], v[GLA_COLS]; };
  In ring[AHEAD];
  auto fetch = [&](int r, In& in) {
    const float* x = proj + (size_t)r * ldp;
#pragma unroll
    for (int i = 0; i < RPL; i++) {
      const int d = lane + 32 * i;
      in.q[i] = d < D ? x[g.o_q + h * D + d] : 0.f;
      in.k[i] = d < D ? x[g.o_k + h * D + d] : 0.f;
      in.a[i] = d < D ? decay[(size_t)r * g.heads * D + h * D + d] : 0.f;
    }
#pragma unroll
    for (int c = 0; c < GLA_COLS; c++) in.v[c] = e0 + c < E ? x[g.o_v + h * E + e0 + c] : 0.f;
  };
#pragma unroll
  for (int u = 0; u < AHEAD; u++)
    if (r_begin + u < r_end) fetch(r_begin + u, ring[u]);
  // one token; `refill` (a row, or -1) is what the token's ring entry is loaded with once its values are taken
  auto token = [&](int r, In& in, int refill) {
    float cq[RPL], ck[RPL], ca[RPL], cv[GLA_COLS], o[GLA_COLS];
#pragma unroll
    for (int i = 0; i < RPL; i++) { cq[i] = in.q[i] * qscale; ck[i] = in.k[i]; ca[i] = in.a[i]; }
#pragma unroll
    for (int c = 0; c < GLA_COLS; c++) { cv[c] = in.v[c]; o[c] = 0.f; }
    if (refill >= 0) fetch(refill, in);
#pragma unroll
    for (int i = 0; i < RPL; i++)
#pragma unroll
      for (int c = 0; c < GLA_COLS; c++) {
        S[i][c] = fmaf(S[i][c], ca[i], ck[i] * cv[c]);
        o[c] = fmaf(S[i][c], cq[i], o[c]);
      }
    // the column sums: halve the columns a lane carries while exchanging across lane bits 4, 3, 2 (a lane ends with ONE
    // column, col = its bits [4 : 4 - log2(COLS)]), then finish over the remaining lane bits
    int width = GLA_COLS;
#pragma unroll
    for (int off = 16; off >= 4; off >>= 1) {
      if (width > 1) {
        const int hw = width / 2;
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int j = 0; j < GLA_COLS / 2; j++) {
          if (j < hw) {
            const float send = upper ? o[j] : o[j + hw];
            const float keep = upper ? o[j + hw] : o[j];
            o[j] = keep + __shfl_xor_sync(THA_FULL_MASK, send, off);
          }
        }
        width = hw;
      } else {
        o[0] += __shfl_xor_sync(THA_FULL_MASK, o[0], off);
      }
    }
    o[0] += __shfl_xor_sync(THA_FULL_MASK, o[0], 2);
    o[0] += __shfl_xor_sync(THA_FULL_MASK, o[0], 1);
    {
      constexpr int LG = GLA_COLS == 8 ? 3 : GLA_COLS == 4 ? 2 : GLA_COLS == 2 ? 1 : 0;
      const int col = LG ? (lane >> (5 - LG)) : 0;                 // the column this lane ended with
      const bool writer = (lane & ((32 >> LG) - 1)) == 0;
      if (writer && e0 + col < E) o_raw[(size_t)r * g.heads * E + (size_t)h * E + e0 + col] = o[0];
    }
  };
  // whole groups without a branch between their tokens (the refill row is clamped instead of tested), then the ragged end
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
    for (int c = 0; c < GLA_COLS; c++)
      if (e0 + c < E) gstate[(size_t)d * GLA_COLS + c] = S[i][c];
  }
}

}  // namespace tha

using namespace tha;

// the scan over decays and inputs that are ready: q at o_q, k at o_k, v at o_v of proj, the read-out times qscale
static int gla_scan_launch(cudaStream_t s, const tha_gla_t* g, const tha_rows_t* rows, const tha_state_store_t* st, const float* proj,
                           long long ldp, const float* dec, float* o_raw, float qscale) {
  static int cols_env = -1;   // THA_GLA_COLS=2|4|8: value columns per warp (A/B aid)
  if (cols_env < 0) { const char* v = getenv("THA_GLA_COLS"); cols_env = (v && *v) ? atoi(v) : 0; }
  const int cols = (cols_env == 2 || cols_env == 4 || cols_env == 8) && g->dim <= 128 ? cols_env : 2;
  const dim3 grid(rows->n_seqs, g->heads, ceil_div(g->vdim, cols * GLA_WARPS)), block(32 * GLA_WARPS);
#define GLA_LAUNCH(R, A, C) THA_CUDA_OK(launch(hyb_gla_scan_kernel<R, A, C>, grid, block, 0, s, false, *g, *rows, *st, proj, ldp, dec, o_raw, qscale))
#define GLA_LAUNCH_COLS(R, A) do { if (cols == 8) GLA_LAUNCH(R, A, 8); else if (cols == 4) GLA_LAUNCH(R, A, 4); else GLA_LAUNCH(R, A, 2); } while (0)
  if (g->dim <= 32) GLA_LAUNCH_COLS(1, 4);
  else if (g->dim <= 64) GLA_LAUNCH_COLS(2, 4);
  else if (g->dim <= 128) GLA_LAUNCH_COLS(4, 4);
  else if (g->dim <= 256) GLA_LAUNCH(8, 2, 2);
  else GLA_LAUNCH(16, 1, 2);
#undef GLA_LAUNCH_COLS
#undef GLA_LAUNCH
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_gla_scan(void* stream, int dtype, const tha_gla_t* g, const tha_rows_t* rows, const tha_state_store_t* st,
                                const float* proj, long long ldp, float* z_raw, float* o_raw, void* out) {
  if (rows->n_seqs < 1 || rows->n_rows < 1) return THA_STATUS_SUCCESS;
  if (g->heads < 1 || g->dim < 1 || g->vdim < 1 || !(g->tau > 0.f)) return THA_STATUS_INVALID_ARG;
  if (g->dim > 512) return THA_STATUS_NOT_SUPPORTED;   // 16 key channels per lane is the widest register form
  cudaStream_t s = (cudaStream_t)stream;
  const size_t n = (size_t)rows->n_rows * g->heads * g->dim;
  THA_CUDA_OK(launch(hyb_gla_decay_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, false, z_raw, n, g->heads * g->dim, g->b_a2,
                     1.0f / g->tau));
  const int status = gla_scan_launch(s, g, rows, st, proj, ldp, z_raw, o_raw, 1.0f / sqrtf((float)g->dim));
  if (status != THA_STATUS_SUCCESS) return status;
  return tha_hyb_head_gate(stream, dtype, out, o_raw, rows->n_rows, g->heads, g->vdim, 1, g->eps, g->norm, 0, proj + g->o_g, ldp, THA_GATE_SILU);
}

// The bounded-forget-gate recurrence (tha_hgrn_t) is the same scan with k = 1 - f and a = f.  Its gate arithmetic runs for all
// rows at once, in place: q -> silu(q), the f columns -> 1 - f (what is written), decay <- f = lower + (1 - lower) sigmoid(z + b).
// 1 - f is formed as (1 - lower) (1 - sigmoid(z + b)) so that a nearly closed gate keeps its relative precision.
extern "C" int tha_hyb_hgrn_scan(void* stream, int dtype, const tha_hgrn_t* g, const tha_rows_t* rows, const tha_state_store_t* st,
                                 float* proj, long long ldp, float* decay, float* o_raw, void* out) {
  if (rows->n_seqs < 1 || rows->n_rows < 1) return THA_STATUS_SUCCESS;
  if (g->heads < 1 || g->dim < 1 || g->vdim < 1) return THA_STATUS_INVALID_ARG;
  if (g->dim > 512) return THA_STATUS_NOT_SUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t n = (size_t)rows->n_rows * g->heads * g->dim;
  THA_CUDA_OK(launch(hyb_hgrn_gates_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, false, proj, ldp, decay, n, g->heads * g->dim,
                     g->o_q, g->o_f, g->f_b, g->lower));
  tha_gla_t a = {};
  a.heads = g->heads; a.dim = g->dim; a.vdim = g->vdim; a.o_q = g->o_q; a.o_k = g->o_f; a.o_v = g->o_v; a.state_off = g->state_off;
  const int status = gla_scan_launch(s, &a, rows, st, proj, ldp, decay, o_raw, 1.0f);
  if (status != THA_STATUS_SUCCESS) return status;
  return tha_hyb_head_gate(stream, dtype, out, o_raw, rows->n_rows, g->heads, g->vdim, 1, g->eps, g->norm, 0, nullptr, 0, THA_GATE_SIGMOID);
}
