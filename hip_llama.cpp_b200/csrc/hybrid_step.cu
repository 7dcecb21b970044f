// tha_hyb_step: one scheduler step of a layer-program model (include/tha_hybrid.h) over ragged rows.
// The layer loop walks the model's layer descriptions and issues the mechanisms of hybrid_ops.cu; every matrix that
// reads a layer's normed input is one stacked product, its columns are handed to the mixers, the router and the shared
// expert by offset.  Scratch is one slab owned by the library, carved per step.
#include <cuda_bf16.h>

#include <stdlib.h>

#include <mutex>

#include "common.cuh"
#include "hybrid_ops.cuh"
#include "tha_hybrid.h"

namespace tha {

// x = embed[token] * scale (+ the learned vector of the row's position when the model has a position table); x0, when given,
// keeps a copy of it for the layers that add the embedding output again
template <typename T>
__global__ void hyb_embed_kernel(float* __restrict__ x, const T* __restrict__ embed, const int* __restrict__ token, int width,
                                 const T* __restrict__ pos_embed, const int* __restrict__ pos, float scale, float* __restrict__ x0) {
  const int r = blockIdx.x;
  const T* e = embed + (size_t)token[r] * width;
  const T* p = pos_embed ? pos_embed + (size_t)pos[r] * width : nullptr;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = hyb_load(e + i) * scale + (p ? hyb_load(p + i) : 0.f);
    x[(size_t)r * width + i] = v;
    if (x0) x0[(size_t)r * width + i] = v;
  }
}

// x += scale_mix * mixer + scale_ff * feed-forward (layer scales optional).  Two-sided mixers: each side's projection is normed over the width with its own weight,
// the mixer is half their sum.  Feed-forward: the chosen experts' outputs by router weight (found through `inv` in the
// expert-sorted buffer), plus the shared expert (times sigmoid of the row's shared_gate entry when given); a dense
// feed-forward arrives as `shared_down` alone.
__global__ void hyb_finish_kernel(float* __restrict__ x, int width, float eps, const float* __restrict__ left, const float* __restrict__ right,
                                  const float* __restrict__ w_left, const float* __restrict__ w_right, int top,
                                  const float* __restrict__ weight, const int* __restrict__ inv, const float* __restrict__ down,
                                  const float* __restrict__ shared_down, const float* __restrict__ shared_gate, long long ld_shared_gate,
                                  const float* __restrict__ scale_mix, const float* __restrict__ scale_ff, float* __restrict__ tap) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* l = left + (size_t)r * width;
  float il = 1.f, ir = 0.f;
  if (right) {
    const float* rr = right + (size_t)r * width;
    float sl = 0.f, sr = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) { sl = fmaf(l[i], l[i], sl); sr = fmaf(rr[i], rr[i], sr); }
    sl = block_sum(sl, red);
    sr = block_sum(sr, red);
    il = 1.0f / sqrtf(sl / (float)width + eps);
    ir = 1.0f / sqrtf(sr / (float)width + eps);
  }
  const float sg = shared_gate ? 1.0f / (1.0f + expf(-shared_gate[(size_t)r * ld_shared_gate])) : 1.0f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float y = right ? 0.5f * (l[i] * il * w_left[i] + right[(size_t)r * width + i] * ir * w_right[i]) : l[i];
    float f = 0.f;
    for (int j = 0; j < top; j++) f = fmaf(weight[(size_t)r * top + j], down[(size_t)inv[(size_t)r * top + j] * width + i], f);
    if (shared_down) f = fmaf(shared_down[(size_t)r * width + i], sg, f);
    if (scale_mix) y *= scale_mix[i];
    if (scale_ff) f *= scale_ff[i];
    const float v = x[(size_t)r * width + i] + (y + f);
    x[(size_t)r * width + i] = v;
    if (tap) tap[(size_t)r * width + i] = v;
  }
}

__global__ void hyb_softcap_kernel(float* __restrict__ z, size_t n, float cap) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) z[i] = cap * tanhf(z[i] / cap);
}

// ---- scratch -------------------------------------------------------------------------------------------------------
struct HybScratch { char* base = nullptr; size_t cap = 0; int* host_ints = nullptr; std::mutex mu; };
constexpr int HYB_HOST_INTS = 1024;

// rows of h in expert-sorted order, so that every expert's rows are one contiguous matrix
template <typename T>
__global__ void hyb_gather_rows_kernel(T* __restrict__ dst, const T* __restrict__ src, const int* __restrict__ rows_idx, int width) {
  const size_t r = blockIdx.x;
  const T* s = src + (size_t)rows_idx[r] * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[r * width + i] = s[i];
}
static HybScratch g_scratch[64];

struct Carver {
  char* base; size_t at = 0;
  template <typename T> T* take(size_t n) {
    at = (at + 255) & ~(size_t)255;
    T* p = base ? reinterpret_cast<T*>(base + at) : nullptr;
    at += n * sizeof(T);
    return p;
  }
};

struct StepBuffers {
  float *x, *proj, *q, *left, *right, *conv, *dt_raw, *gate_raw, *gu, *down, *sdown, *weight, *oraw, *split; size_t split_floats;
  float *proj2, *qfull, *x0, *sgate;
  float *xs, *hf, *att;   // the residual streams [rows, n, width]; a normed input before its convolution; fp32 attention maps
  void* sg;
  void *h, *h2, *cq, *qplain, *abuf, *mbuf, *y, *sy, *hn, *hg;
  int *expert_id, *group_off, *sorted_row, *inv;
  float* cos_t[64]; float* sin_t[64];
};

// Steps of at least this many rows MAY run a mixture's experts as one tensor-core matmul per expert (the group sizes
// come back to the host for that): they do when an expert gets hyb_expert_rows() rows on average, which is where a
// matmul's work outweighs its launch (measured: 4096-token prompts, 16 experts: 512 rows per expert 18.4 ms against 16.6
// with the grouped kernel, 1024 rows per expert 28.8 against 29.9).  THA_HYB_EXPERT_ROWS overrides the average.
constexpr int HYB_EXPERT_LAUNCH_ROWS = 1024;
static long long hyb_expert_rows() {
  const char* v = getenv("THA_HYB_EXPERT_ROWS");
  return (v && *v) ? atoll(v) : 1024;
}

// channels of an attention layer's short convolution: its projected q | k | v columns (q alone when it reads another layer's rows)
static size_t hyb_attn_conv_channels(const tha_attn_t& a) {
  size_t c = (size_t)a.heads * a.dim;
  if (!a.kv_shared) c += (size_t)a.kv_heads * a.dim + (size_t)(a.kv_heads / (a.v_share > 1 ? a.v_share : 1)) * a.vdim;
  return c;
}

static size_t carve(const tha_hyb_model_t* m, int R, int n_want, char* base, StepBuffers* b) {
  Carver c{base};
  const size_t W = m->width, es = m->dtype == THA_DT_BF16 ? 2 : 4;
  size_t n_in = 0, qd = 0, av = 0, mv = 0, cc = 0, dd = 0, dg = 0, gu = 0, ff = 0, sff = 0, top = 0, ne = 0;
  size_t n_in2 = 0, qr = 0, qf = 0, qp = 0;
  bool norm2 = false, keep_embed = false;
  size_t sd = 0, n_str = 0, hfw = 0, attf = 0;
  for (int i = 0; i < m->n_layers; i++) {
    const tha_hyb_layer_t& L = m->layers[i];
    n_in = max(n_in, (size_t)L.n_in);
    if (L.block == THA_BLOCK_STREAMS) n_str = (size_t)(m->n_streams > 0 ? m->n_streams : 1);
    if (L.in_conv_taps > 0) hfw = W;
    if (L.pre_add_embed) keep_embed = true;
    sd = max(sd, (size_t)L.side.dim);
    if (L.mixer == THA_MIX_ATTN || L.mixer == THA_MIX_ATTN_GDELTA) {
      qd = max(qd, (size_t)L.attn.heads * L.attn.dim);
      av = max(av, (size_t)L.attn.heads * L.attn.vdim);
      if (L.attn.diff) attf = max(attf, (size_t)L.attn.heads * L.attn.vdim);
      if (L.attn.conv_taps > 0) cc = max(cc, hyb_attn_conv_channels(L.attn));
    }
    if (L.mixer == THA_MIX_HGRN) {
      dd = max(dd, (size_t)L.hgrn.heads * L.hgrn.dim);
      mv = max(mv, (size_t)L.hgrn.heads * L.hgrn.vdim);
    }
    if (L.mixer == THA_MIX_ATTN_GDELTA) {
      dd = max(dd, (size_t)L.gdelta.heads * L.gdelta.dim);
      mv = max(mv, (size_t)L.gdelta.heads * L.gdelta.dim);
    }
    if (L.mixer == THA_MIX_PARALLEL) {
      qd = max(qd, (size_t)L.attn.heads * L.attn.dim);
      av = max(av, (size_t)L.attn.heads * L.attn.vdim);
      mv = max(mv, (size_t)L.mem.heads * L.mem.vdim);
    } else if (L.mixer == THA_MIX_DELTA) {
      cc = max(cc, (size_t)2 * L.delta.kv_heads * L.delta.dim + (size_t)L.delta.heads * L.delta.vdim);
      dd = max(dd, (size_t)L.delta.heads * L.delta.dim);
      dg = max(dg, (size_t)L.delta.heads * L.delta.vdim);
      mv = max(mv, (size_t)L.delta.heads * L.delta.vdim);
    } else if (L.mixer == THA_MIX_GLA) {
      dd = max(dd, (size_t)L.gla.heads * L.gla.dim);
      mv = max(mv, (size_t)L.gla.heads * L.gla.vdim);
    } else if (L.mixer == THA_MIX_LATENT) {
      const tha_latent_t& a = L.latent;
      qr = max(qr, (size_t)a.q_rank);
      qf = max(qf, (size_t)a.heads * (a.dim + a.rot_dim));
      qp = max(qp, (size_t)a.heads * a.dim);
      qd = max(qd, (size_t)a.heads * (a.kv_rank + a.rot_dim));
      av = max(av, (size_t)a.heads * a.kv_rank);
      mv = max(mv, (size_t)a.heads * a.vdim);
    }
    if (L.has_norm2) { norm2 = true; n_in2 = max(n_in2, (size_t)L.n_in2); }
    if (L.has_ff == THA_FF_MOE) {
      top = max(top, (size_t)L.moe.top);
      ne = max(ne, (size_t)L.moe.experts);
      gu = max(gu, (size_t)L.moe.top * 2 * L.moe.ff);
      ff = max(ff, (size_t)L.moe.top * L.moe.ff);
      sff = max(sff, (size_t)L.moe.shared_ff);
    } else if (L.has_ff == THA_FF_DENSE) {
      sff = max(sff, (size_t)L.dense.ff);
    }
  }
  b->x = c.take<float>(R * W);
  b->x0 = c.take<float>(keep_embed ? R * W : 0);
  if (!keep_embed) b->x0 = nullptr;
  b->xs = c.take<float>(R * n_str * W);
  b->hf = c.take<float>(R * hfw);
  b->att = c.take<float>(R * attf);
  b->h = c.take<char>(R * W * es);
  b->proj = c.take<float>(R * n_in);
  b->h2 = c.take<char>(norm2 ? R * W * es : 0);
  b->proj2 = c.take<float>(R * n_in2);
  b->cq = c.take<char>(R * qr * es);
  b->qfull = c.take<float>(R * qf);
  b->qplain = c.take<char>(R * qp * es);
  b->q = c.take<float>(R * qd);
  b->abuf = c.take<char>(R * av * es);
  b->mbuf = c.take<char>(R * mv * es);
  b->oraw = c.take<float>(R * mv);
  // key splits of the attention in small steps: 16 x rows x heads x (vdim + 2) floats at most (2 * heads <= 2 * heads * dim)
  b->split_floats = R <= 1024 ? (size_t)16 * R * (av + 2 * qd) : 0;
  b->split = c.take<float>(b->split_floats);
  b->left = c.take<float>(R * W);
  b->right = c.take<float>(R * W);
  b->conv = c.take<float>(R * cc);
  b->dt_raw = c.take<float>(R * dd);
  b->gate_raw = c.take<float>(R * dg);
  b->hg = c.take<char>(R >= HYB_EXPERT_LAUNCH_ROWS ? R * top * W * es : 0);
  b->gu = c.take<float>(R * gu);
  b->y = c.take<char>(R * ff * es);
  b->down = c.take<float>(R * top * W);
  b->sy = c.take<char>(R * sff * es);
  b->sdown = c.take<float>(R * W);
  b->weight = c.take<float>(R * top);
  b->expert_id = c.take<int>(R * top);
  b->sorted_row = c.take<int>(R * top);
  b->inv = c.take<int>(R * top);
  b->group_off = c.take<int>(2 * (ne + 1));
  b->sgate = c.take<float>(R * sd);
  b->sg = c.take<char>(R * sd * es);
  b->hn = c.take<char>((size_t)n_want * W * es);
  for (int i = 0; i < m->n_rot && i < 64; i++) {
    b->cos_t[i] = c.take<float>((size_t)R * (m->rot[i].dims / 2));
    b->sin_t[i] = c.take<float>((size_t)R * (m->rot[i].dims / 2));
  }
  return c.at + 256;
}

}  // namespace tha

using namespace tha;
typedef __nv_bfloat16 bf16;

#define HYB_OK(expr)                         \
  do {                                       \
    const int _s = (expr);                   \
    if (_s != THA_STATUS_SUCCESS) return _s; \
  } while (0)

// A mixture's router and chosen experts over R rows of hf (their router logits in fproj): the experts' results land in b.down in
// expert-sorted order, found per (row, pick) through b.inv and weighted by b.weight by whoever adds them to the residual.
static int hyb_run_experts(void* stream, HybScratch& sc, int dt, int R, int W, const tha_moe_t& e, const void* hf, const float* fproj,
                           long long ldf, StepBuffers& b) {
  cudaStream_t s = (cudaStream_t)stream;
  const int top = e.top;
  const bool gated = e.act != THA_ACT_RELU2;
  const int gw = gated ? 2 * e.ff : e.ff, col_u = gated ? e.ff : 0;   // an expert's rows of w_gate_up; where its up rows start
  HYB_OK(tha_hyb_moe_route(stream, &e, fproj, ldf, R, b.expert_id, b.weight, b.group_off, b.sorted_row, b.inv));
  const bool per_expert = dt == THA_DT_BF16 && R >= HYB_EXPERT_LAUNCH_ROWS && (long long)R * top >= hyb_expert_rows() * e.experts &&
                          e.experts < HYB_HOST_INTS && W % 8 == 0 && e.ff % 8 == 0 && W >= 64 && e.ff >= 64;
  if (per_expert) {
    // prompt-sized steps: gather the rows into expert order once, read the group sizes, and give every expert's
    // contiguous rows to the TMA-fed tcgen05 matmul of the bf16 path (two launches per expert that has rows)
    if (!sc.host_ints) THA_CUDA_OK(cudaMallocHost((void**)&sc.host_ints, HYB_HOST_INTS * sizeof(int)));
    THA_CUDA_OK(cudaMemcpyAsync(sc.host_ints, b.group_off, (e.experts + 1) * sizeof(int), cudaMemcpyDeviceToHost, s));
    THA_CUDA_OK(launch(hyb_gather_rows_kernel<bf16>, dim3(R * top), dim3(128), 0, s, false, (bf16*)b.hg, (const bf16*)hf, (const int*)b.sorted_row, W));
    THA_CUDA_OK(cudaStreamSynchronize(s));
    const int* off = sc.host_ints;
    for (int x = 0; x < e.experts; x++) {
      const int n = off[x + 1] - off[x];
      if (n > 0)
        HYB_OK(tha_hyb_linear(stream, dt, b.gu + (size_t)off[x] * gw, gw, (const bf16*)b.hg + (size_t)off[x] * W, W, 0, nullptr,
                              (const bf16*)e.w_gate_up + (size_t)x * gw * W, 0, n, gw, W, nullptr, 0));
    }
    HYB_OK(tha_hyb_ff_act(stream, dt, e.act, b.y, b.gu, gw, 0, col_u, R * top, e.ff, e.limit, e.alpha));
    for (int x = 0; x < e.experts; x++) {
      const int n = off[x + 1] - off[x];
      if (n > 0)
        HYB_OK(tha_hyb_linear(stream, dt, b.down + (size_t)off[x] * W, W, (const bf16*)b.y + (size_t)off[x] * e.ff, e.ff, 0, nullptr,
                              (const bf16*)e.w_down + (size_t)x * W * e.ff, 0, n, W, e.ff, nullptr, 0));
    }
  } else {
    HYB_OK(tha_hyb_linear(stream, dt, b.gu, gw, hf, W, 0, b.sorted_row, e.w_gate_up, (long long)gw * W, R * top, gw, W,
                          b.group_off, e.experts));
    HYB_OK(tha_hyb_ff_act(stream, dt, e.act, b.y, b.gu, gw, 0, col_u, R * top, e.ff, e.limit, e.alpha));
    HYB_OK(tha_hyb_linear(stream, dt, b.down, W, b.y, e.ff, 0, nullptr, e.w_down, (long long)W * e.ff, R * top, W, e.ff, b.group_off, e.experts));
  }
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_step(void* stream, const tha_hyb_model_t* m, const tha_rows_t* rows, const tha_kv_t* kv,
                            const tha_state_store_t* st, int n_want, const int* want_rows, float* logits, float* taps) {
  if (!m || !rows || !kv || !st || m->n_rot > 64) return THA_STATUS_INVALID_ARG;
  const int R = rows->n_rows;
  if (R < 1) return THA_STATUS_SUCCESS;
  cudaStream_t s = (cudaStream_t)stream;
  const int dt = m->dtype, W = m->width;
  int dev = 0;
  THA_CUDA_OK(cudaGetDevice(&dev));
  HybScratch& sc = g_scratch[dev & 63];
  std::lock_guard<std::mutex> lock(sc.mu);
  StepBuffers b;
  const size_t need = carve(m, R, n_want, nullptr, &b);
  if (need > sc.cap) {   // grow: nothing of an earlier step may still be using the old slab
    THA_CUDA_OK(cudaDeviceSynchronize());
    if (sc.base) THA_CUDA_OK(cudaFree(sc.base));
    sc.base = nullptr; sc.cap = 0;
    const size_t want = need + need / 2;
    THA_CUDA_OK(cudaMalloc((void**)&sc.base, want));
    sc.cap = want;
  }
  carve(m, R, n_want, sc.base, &b);

  const float embed_scale = m->embed_scale != 0.f ? m->embed_scale : 1.0f;
  if (dt == THA_DT_BF16)
    THA_CUDA_OK(launch(hyb_embed_kernel<bf16>, dim3(R), dim3(128), 0, s, false, b.x, (const bf16*)m->embed, rows->token, W, (const bf16*)m->pos_embed,
                       rows->pos, embed_scale, b.x0));
  else
    THA_CUDA_OK(launch(hyb_embed_kernel<float>, dim3(R), dim3(128), 0, s, false, b.x, (const float*)m->embed, rows->token, W,
                       (const float*)m->pos_embed, rows->pos, embed_scale, b.x0));
  for (int i = 0; i < m->n_rot; i++) HYB_OK(tha_hyb_rotary_table(stream, &m->rot[i], rows->pos, R, b.cos_t[i], b.sin_t[i]));

  bool h_ready = false;   // the previous block's last pass already left this layer's first norm in b.h
  for (int li = 0; li < m->n_layers; li++) {
    const tha_hyb_layer_t& L = m->layers[li];
    const long long ldp = L.n_in;
    const bool seq = L.block == THA_BLOCK_SEQUENTIAL;
    const bool streams = L.block == THA_BLOCK_STREAMS;
    const int n_str = m->n_streams > 0 ? m->n_streams : 1;
    const bool two_norms = !seq && !streams && L.has_norm2 && L.has_ff != THA_FF_NONE;
    if (streams) {
      // the mixer's input: the first sublayer's read of the streams and its norm (left behind by the previous layer's last
      // pass, or made here from the embedding output), then h + conv(h) continuing from the slot's tail
      const bool conv = L.in_conv_taps > 0;
      if (!h_ready)
        HYB_OK(tha_hyb_streams(stream, dt, b.xs, n_str, (li == 0 || m->layers[li - 1].block != THA_BLOCK_STREAMS) ? b.x : nullptr, nullptr, nullptr, nullptr, 0, nullptr, nullptr, nullptr, nullptr,
                               nullptr, &L.streams1, &L.norm1, m->eps, conv, conv ? (void*)b.hf : b.h, R, W));
      h_ready = false;
      if (conv) {
        HYB_OK(tha_hyb_conv(stream, dt, rows, st, L.in_conv_state_off, b.hf, W, 0, W, L.in_conv_taps, L.in_conv_w, 0, 1, 0, b.h));
        HYB_OK(tha_hyb_conv_tail(stream, rows, st, L.in_conv_state_off, b.hf, W, 0, W, L.in_conv_taps));
      }
    } else if (seq && h_ready) h_ready = false;
    else if (seq && (L.pre_add_embed || L.pre_vec))   // a pass's re-entry addends and the mixer's norm in one pass over x
      HYB_OK(tha_hyb_add_norm(stream, dt, b.x, nullptr, 0.f, nullptr, 0.f, L.pre_add_embed ? b.x0 : nullptr, L.pre_vec, &L.norm1, m->eps, b.h, R, W));
    else if (two_norms) HYB_OK(tha_hyb_norm_pair(stream, dt, b.h, b.h2, b.x, &L.norm1, &L.norm2, m->eps, R, W));
    else HYB_OK(tha_hyb_norm(stream, dt, b.h, b.x, &L.norm1, m->eps, R, W, nullptr));
    HYB_OK(tha_hyb_linear(stream, dt, b.proj, ldp, b.h, W, 0, nullptr, L.w_in, 0, R, L.n_in, W, nullptr, 0));
    const float* right = nullptr;
    if (L.mixer == THA_MIX_ATTN || L.mixer == THA_MIX_ATTN_GDELTA) {
      const tha_attn_t& a = L.attn;
      const int rd = a.rot >= 0 ? m->rot[a.rot].dims : 0;
      // a short convolution over the projected q | k | v: the rest of the layer reads the convolved copy
      tha_attn_t ap = a;
      const float* pq = b.proj;
      long long ldq = ldp;
      if (a.conv_taps > 0) {
        const int C = (int)hyb_attn_conv_channels(a);
        HYB_OK(tha_hyb_conv(stream, dt, rows, st, a.conv_state_off, b.proj, ldp, a.o_q, C, a.conv_taps, a.conv_w, 0, 0, 1, b.conv));
        HYB_OK(tha_hyb_conv_tail(stream, rows, st, a.conv_state_off, b.proj, ldp, a.o_q, C, a.conv_taps));
        ap.o_q = 0; ap.o_k = a.heads * a.dim; ap.o_v = ap.o_k + a.kv_heads * a.dim;
        pq = b.conv; ldq = C;
      }
      HYB_OK(tha_hyb_attn_prepare(stream, &ap, rows, kv, pq, ldq, a.rot >= 0 ? b.cos_t[a.rot] : nullptr,
                                  a.rot >= 0 ? b.sin_t[a.rot] : nullptr, rd, b.q));
      int ov = a.heads * a.vdim;   // columns of the mixer's result before its output matrix
      if (a.diff) {
        // two maps per head as fp32, then their combination, the head norm and the gate
        HYB_OK(tha_hyb_attn_gated(stream, dt, &a, rows, kv, b.q, b.att, b.split_floats ? b.split : nullptr, b.split_floats, nullptr, 0));
        HYB_OK(tha_hyb_diff_combine(stream, dt, &a, b.att, b.proj, ldp, b.abuf, R));
        ov = a.heads / 2 * a.vdim;
      } else {
        HYB_OK(tha_hyb_attn_gated(stream, dt, &a, rows, kv, b.q, b.abuf, b.split_floats ? b.split : nullptr, b.split_floats, b.proj, ldp));
      }
      HYB_OK(tha_hyb_linear(stream, dt, b.left, W, b.abuf, ov, 0, nullptr, a.w_o, 0, R, W, ov, nullptr, 0));
      if (L.mixer == THA_MIX_ATTN_GDELTA) {
        const tha_gdelta_t& g = L.gdelta;
        HYB_OK(tha_hyb_gdelta_scan(stream, dt, &g, rows, st, b.proj, ldp, b.dt_raw, b.oraw, b.mbuf));
        HYB_OK(tha_hyb_linear(stream, dt, b.right, W, b.mbuf, g.heads * g.dim, 0, nullptr, g.w_o, 0, R, W, g.heads * g.dim, nullptr, 0));
        right = b.right;
      }
    } else if (L.mixer == THA_MIX_PARALLEL) {
      const tha_attn_t& a = L.attn;
      const int rd = a.rot >= 0 ? m->rot[a.rot].dims : 0;
      HYB_OK(tha_hyb_attn_prepare(stream, &a, rows, kv, b.proj, ldp, a.rot >= 0 ? b.cos_t[a.rot] : nullptr,
                                  a.rot >= 0 ? b.sin_t[a.rot] : nullptr, rd, b.q));
      HYB_OK(tha_hyb_attn(stream, dt, &a, rows, kv, b.q, b.abuf, b.split_floats ? b.split : nullptr, b.split_floats));
      HYB_OK(tha_hyb_linear(stream, dt, b.left, W, b.abuf, a.heads * a.vdim, 0, nullptr, a.w_o, 0, R, W, a.heads * a.vdim, nullptr, 0));
      const tha_mem_t& mm = L.mem;
      HYB_OK(tha_hyb_mem_scan(stream, dt, &mm, rows, st, b.proj, ldp, b.oraw, b.mbuf));
      HYB_OK(tha_hyb_linear(stream, dt, b.right, W, b.mbuf, mm.heads * mm.vdim, 0, nullptr, mm.w_o, 0, R, W, mm.heads * mm.vdim, nullptr, 0));
      right = b.right;
    } else if (L.mixer == THA_MIX_DELTA) {
      const tha_delta_t& d = L.delta;
      const int C = 2 * d.kv_heads * d.dim + d.heads * d.vdim;
      HYB_OK(tha_hyb_conv_silu(stream, rows, st, d.conv_state_off, b.proj, ldp, d.o_q, C, d.taps, d.conv, b.conv));
      HYB_OK(tha_hyb_linear(stream, dt, b.dt_raw, d.heads * d.dim, b.proj + d.o_a1, ldp, 1, nullptr, d.w_a2, 0, R, d.heads * d.dim, d.rank_a, nullptr, 0));
      HYB_OK(tha_hyb_linear(stream, dt, b.gate_raw, d.heads * d.vdim, b.proj + d.o_g1, ldp, 1, nullptr, d.w_g2, 0, R, d.heads * d.vdim, d.rank_g, nullptr, 0));
      HYB_OK(tha_hyb_delta_scan(stream, dt, &d, rows, st, b.conv, b.proj, ldp, b.dt_raw, b.gate_raw, b.oraw, b.mbuf));
      HYB_OK(tha_hyb_linear(stream, dt, b.left, W, b.mbuf, d.heads * d.vdim, 0, nullptr, d.w_o, 0, R, W, d.heads * d.vdim, nullptr, 0));
    } else if (L.mixer == THA_MIX_GLA) {
      const tha_gla_t& g = L.gla;
      HYB_OK(tha_hyb_linear(stream, dt, b.dt_raw, g.heads * g.dim, b.proj + g.o_a1, ldp, 1, nullptr, g.w_a2, 0, R, g.heads * g.dim, g.rank, nullptr, 0));
      HYB_OK(tha_hyb_gla_scan(stream, dt, &g, rows, st, b.proj, ldp, b.dt_raw, b.oraw, b.mbuf));
      HYB_OK(tha_hyb_linear(stream, dt, b.left, W, b.mbuf, g.heads * g.vdim, 0, nullptr, g.w_o, 0, R, W, g.heads * g.vdim, nullptr, 0));
    } else if (L.mixer == THA_MIX_HGRN) {
      const tha_hgrn_t& g = L.hgrn;
      HYB_OK(tha_hyb_hgrn_scan(stream, dt, &g, rows, st, b.proj, ldp, b.dt_raw, b.oraw, b.mbuf));
      HYB_OK(tha_hyb_linear(stream, dt, b.left, W, b.mbuf, g.heads * g.vdim, 0, nullptr, g.w_o, 0, R, W, g.heads * g.vdim, nullptr, 0));
    } else if (L.mixer == THA_MIX_LATENT) {
      const tha_latent_t& a = L.latent;
      const int rd = a.rot >= 0 ? m->rot[a.rot].dims : 0;
      const float* cs = a.rot >= 0 ? b.cos_t[a.rot] : nullptr;
      const float* sn = a.rot >= 0 ? b.sin_t[a.rot] : nullptr;
      const int per = a.dim + a.rot_dim, DA = a.kv_rank + a.rot_dim;
      HYB_OK(tha_hyb_latent_prepare(stream, dt, &a, rows, kv, b.proj, ldp, cs, sn, rd, b.cq));
      if (a.direct_q) {   // the queries are columns of the stacked projection
        HYB_OK(tha_hyb_latent_split_q(stream, dt, &a, R, b.proj + a.o_q, ldp, cs, sn, rd, b.qplain, b.q));
      } else {
        HYB_OK(tha_hyb_linear(stream, dt, b.qfull, a.heads * per, b.cq, a.q_rank, 0, nullptr, a.w_uq, 0, R, a.heads * per, a.q_rank, nullptr, 0));
        HYB_OK(tha_hyb_latent_split_q(stream, dt, &a, R, b.qfull, 0, cs, sn, rd, b.qplain, b.q));
      }
      // keys absorbed into the queries: q_abs[h, 0:kv_rank] = W_uk[h]^T q_plain[h]
      HYB_OK(tha_hyb_linear_heads(stream, dt, b.q, (long long)a.heads * DA, DA, b.qplain, (long long)a.heads * a.dim, a.dim, 0, a.w_uk_t,
                                  (long long)a.kv_rank * a.dim, R, a.kv_rank, a.dim, a.heads));
      // one key/value head over the cached rows [latent | rotated part]; the values are the latent itself
      tha_attn_t at = {};
      at.heads = a.heads; at.kv_heads = 1; at.dim = DA; at.vdim = a.kv_rank; at.rot = -1; at.unit_rms = 0; at.eps = a.eps;
      at.scale = a.scale; at.chunk = 0; at.cache_layer = a.cache_layer; at.values_in_keys = 1;
      at.window = a.window; at.sink = a.sink; at.fp32_scores = a.fp32_scores;
      tha_kv_t lkv = *kv;
      lkv.v_pool = kv->k_pool;
      HYB_OK(tha_hyb_attn(stream, dt, &at, rows, &lkv, b.q, b.abuf, b.split_floats ? b.split : nullptr, b.split_floats));
      // values expanded per head: o[h] = W_uv[h] o_latent[h]
      HYB_OK(tha_hyb_linear_heads(stream, dt, b.oraw, (long long)a.heads * a.vdim, a.vdim, b.abuf, (long long)a.heads * a.kv_rank, a.kv_rank, 0,
                                  a.w_uv, (long long)a.vdim * a.kv_rank, R, a.vdim, a.kv_rank, a.heads));
      HYB_OK(tha_hyb_head_gate(stream, dt, b.mbuf, b.oraw, R, a.heads, a.vdim, 0, a.eps, nullptr, 0, a.no_gate ? nullptr : b.proj + a.o_g, ldp,
                               THA_GATE_SIGMOID));
      HYB_OK(tha_hyb_linear(stream, dt, b.left, W, b.mbuf, a.heads * a.vdim, 0, nullptr, a.w_o, 0, R, W, a.heads * a.vdim, nullptr, 0));
    } else {
      return THA_STATUS_NOT_SUPPORTED;
    }
    if (streams) {
      // what follows the layer: the tap, the sum of the streams for the final norm, or the next layer's first read
      const tha_hyb_layer_t* next = li + 1 < m->n_layers && m->layers[li + 1].block == THA_BLOCK_STREAMS ? &m->layers[li + 1] : nullptr;
      float* tap = taps ? taps + (size_t)li * R * W : (float*)nullptr;
      float* sum_out = next ? (float*)nullptr : b.x;
      const bool nconv = next && next->in_conv_taps > 0;
      void* nout = next ? (nconv ? (void*)b.hf : b.h) : nullptr;
      if (L.has_ff == THA_FF_NONE) {
        HYB_OK(tha_hyb_streams(stream, dt, b.xs, n_str, nullptr, &L.streams1, b.left, nullptr, 0, nullptr, nullptr, nullptr, tap, sum_out,
                               next ? &next->streams1 : nullptr, next ? &next->norm1 : nullptr, m->eps, nconv, nout, R, W));
      } else {
        // the mixer's write and the feed-forward's read in one pass over the streams
        HYB_OK(tha_hyb_streams(stream, dt, b.xs, n_str, nullptr, &L.streams1, b.left, nullptr, 0, nullptr, nullptr, nullptr, nullptr, nullptr,
                               &L.streams2, &L.norm2, m->eps, 0, b.h2, R, W));
        HYB_OK(tha_hyb_linear(stream, dt, b.proj2, L.n_in2, b.h2, W, 0, nullptr, L.w_in2, 0, R, L.n_in2, W, nullptr, 0));
        if (L.has_ff == THA_FF_DENSE) {
          const tha_dense_ff_t& d = L.dense;
          if (d.act == THA_ACT_POLYNORM) HYB_OK(tha_hyb_polynorm(stream, dt, b.sy, b.proj2, L.n_in2, d.o_up, d.b_up, d.act_c, m->eps, R, d.ff));
          else if (d.b_up) return THA_STATUS_NOT_SUPPORTED;
          else HYB_OK(tha_hyb_ff_act(stream, dt, d.act, b.sy, b.proj2, L.n_in2, d.o_gate, d.o_up, R, d.ff, d.act_p, d.act_q));
          HYB_OK(tha_hyb_linear(stream, dt, b.sdown, W, b.sy, d.ff, 0, nullptr, d.w_down, 0, R, W, d.ff, nullptr, 0));
          HYB_OK(tha_hyb_streams(stream, dt, b.xs, n_str, nullptr, &L.streams2, b.sdown, d.b_down, 0, nullptr, nullptr, nullptr, tap, sum_out,
                                 next ? &next->streams1 : nullptr, next ? &next->norm1 : nullptr, m->eps, nconv, nout, R, W));
        } else {
          const tha_moe_t& e = L.moe;
          if (e.shared_ff > 0) return THA_STATUS_NOT_SUPPORTED;
          HYB_OK(hyb_run_experts(stream, sc, dt, R, W, e, b.h2, b.proj2, L.n_in2, b));
          HYB_OK(tha_hyb_streams(stream, dt, b.xs, n_str, nullptr, &L.streams2, nullptr, nullptr, e.top, b.weight, b.inv, b.down, tap, sum_out,
                                 next ? &next->streams1 : nullptr, next ? &next->norm1 : nullptr, m->eps, nconv, nout, R, W));
        }
      }
      h_ready = next != nullptr;
      continue;
    }
    if (seq) {
      // x += m * mixer and the feed-forward's norm of the new x in one pass; the feed-forward; then its residual add, the
      // side input and the tap in one more
      const float m_res = L.res_mult;
      const float cl = L.mixer == THA_MIX_ATTN_GDELTA ? m_res * L.mix_left : m_res, cr = m_res * L.mix_right;
      const float* ffo = nullptr;
      if (L.has_ff == THA_FF_DENSE) {
        const tha_dense_ff_t& d = L.dense;
        HYB_OK(tha_hyb_add_norm(stream, dt, b.x, b.left, cl, right, cr, nullptr, nullptr, &L.norm2, m->eps, b.h2, R, W));
        HYB_OK(tha_hyb_linear(stream, dt, b.proj2, L.n_in2, b.h2, W, 0, nullptr, L.w_in2, 0, R, L.n_in2, W, nullptr, 0));
        HYB_OK(tha_hyb_ff_act(stream, dt, d.act, b.sy, b.proj2, L.n_in2, d.o_gate, d.o_up, R, d.ff, d.act_p, d.act_q));
        HYB_OK(tha_hyb_linear(stream, dt, b.sdown, W, b.sy, d.ff, 0, nullptr, d.w_down, 0, R, W, d.ff, nullptr, 0));
        ffo = b.sdown;
      } else if (L.has_ff == THA_FF_NONE) {
        HYB_OK(tha_hyb_add_norm(stream, dt, b.x, b.left, cl, right, cr, nullptr, nullptr, nullptr, m->eps, nullptr, R, W));
      } else {
        return THA_STATUS_NOT_SUPPORTED;
      }
      const float* y = nullptr;
      if (L.side.dim > 0) {
        // the side input reads the stream after the feed-forward: x += m * ff and x in the products' number format, the gate
        // product, its activation times the token's table entries, the projection
        const tha_norm_t copy = {THA_NORM_COPY};
        HYB_OK(tha_hyb_add_norm(stream, dt, b.x, ffo, m_res, nullptr, 0.f, nullptr, nullptr, &copy, m->eps, b.h, R, W));
        ffo = nullptr;
        HYB_OK(tha_hyb_linear(stream, dt, b.sgate, L.side.dim, b.h, W, 0, nullptr, L.side.w_gate, 0, R, L.side.dim, W, nullptr, 0));
        HYB_OK(tha_hyb_side_gate(stream, dt, b.sg, b.sgate, L.side.dim, &L.side, m->side_table, m->side_cols, rows->token, R));
        HYB_OK(tha_hyb_linear(stream, dt, b.sdown, W, b.sg, L.side.dim, 0, nullptr, L.side.w_proj, 0, R, W, L.side.dim, nullptr, 0));
        y = b.sdown;
      }
      // the last pass over x: the remaining residual adds, the tap, and what comes ahead of the next layer run
      const tha_hyb_layer_t* next = li + 1 < m->n_layers && m->layers[li + 1].block == THA_BLOCK_SEQUENTIAL ? &m->layers[li + 1] : nullptr;
      HYB_OK(tha_hyb_block_finish(stream, dt, b.x, ffo, y, m_res, L.side.norm, m->eps, taps ? taps + (size_t)li * R * W : (float*)nullptr,
                                  next && next->pre_add_embed ? b.x0 : nullptr, next ? next->pre_vec : nullptr, next ? &next->norm1 : nullptr,
                                  next ? b.h : nullptr, R, W));
      h_ready = next != nullptr;
      continue;
    }
    // the feed-forward reads the mixer's normed input, or a second norm of the same x through its own stacked product
    const void* hf = b.h;
    const float* fproj = b.proj;
    long long ldf = ldp;
    if (two_norms) {
      HYB_OK(tha_hyb_linear(stream, dt, b.proj2, L.n_in2, b.h2, W, 0, nullptr, L.w_in2, 0, R, L.n_in2, W, nullptr, 0));
      hf = b.h2; fproj = b.proj2; ldf = L.n_in2;
    }
    int top = 0;
    const float* sdown = nullptr;
    const float* sgate = nullptr;
    if (L.has_ff == THA_FF_DENSE) {
      const tha_dense_ff_t& d = L.dense;
      HYB_OK(tha_hyb_ff_act(stream, dt, d.act, b.sy, fproj, ldf, d.o_gate, d.o_up, R, d.ff, 0.f, 0.f));
      HYB_OK(tha_hyb_linear(stream, dt, b.sdown, W, b.sy, d.ff, 0, nullptr, d.w_down, 0, R, W, d.ff, nullptr, 0));
      sdown = b.sdown;
    } else if (L.has_ff == THA_FF_MOE) {
      const tha_moe_t& e = L.moe;
      top = e.top;
      HYB_OK(hyb_run_experts(stream, sc, dt, R, W, e, hf, fproj, ldf, b));
      if (e.shared_ff > 0) {
        HYB_OK(tha_hyb_ff_act(stream, dt, e.act, b.sy, fproj, ldf, e.o_sgate, e.o_sup, R, e.shared_ff, e.shared_limit, e.alpha));
        HYB_OK(tha_hyb_linear(stream, dt, b.sdown, W, b.sy, e.shared_ff, 0, nullptr, e.w_sdown, 0, R, W, e.shared_ff, nullptr, 0));
        sdown = b.sdown;
        if (e.shared_scaled) sgate = fproj + e.o_sscale;
      }
    }
    THA_CUDA_OK(launch(hyb_finish_kernel, dim3(R), dim3(128), 0, s, false, b.x, W, m->eps, (const float*)b.left, right, L.left_out, L.right_out, top,
                       (const float*)b.weight, (const int*)b.inv, (const float*)b.down, sdown, sgate, ldf, L.scale_mix, L.scale_ff,
                       taps ? taps + (size_t)li * R * W : (float*)nullptr));
  }
  if (n_want > 0 && logits) {
    HYB_OK(tha_hyb_norm(stream, dt, b.hn, b.x, &m->final_norm, m->eps, n_want, W, want_rows));
    HYB_OK(tha_hyb_linear(stream, dt, logits, m->vocab, b.hn, W, 0, nullptr, m->head, 0, n_want, m->vocab, W, nullptr, 0));
    if (m->logit_softcap > 0.f) {
      const size_t n = (size_t)n_want * m->vocab;
      THA_CUDA_OK(launch(hyb_softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, false, logits, n, m->logit_softcap));
    }
  }
  return THA_STATUS_SUCCESS;
}
