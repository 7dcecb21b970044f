/* tha_hybrid.h -- C-ABI of the layer-program path: decoder models whose layers are described by data
 * (which sequence mixer, which feed-forward, every size and constant) instead of by a fixed struct.
 *
 * The llama2 path (tha_b200.h) hard-wires one layer shape.  Here a model is an array of tha_hyb_layer_t, each naming
 * its mixer(s) and feed-forward; tha_hyb_step runs ONE scheduler step over a ragged batch of rows (a row = one token
 * of one sequence at one position): prompt portions of some sequences beside single decoded tokens of others.  What a
 * sequence carries from step to step lives in two stores the host's BatchManager owns:
 *   - cache rows of the softmax-attention layers in a block pool addressed through a block table (paged KV), and
 *   - one fixed-size fp32 state slot per live sequence for the recurrent mixers (matrix memories, delta-rule
 *     memories, the tails of the short convolutions).
 * Every mechanism is also callable by itself (tha_hyb_* ops below) so that it can be tested alone and reused by
 * another layer description.
 *
 * Number formats: `dtype` selects the storage type of matrices and of the vectors that enter a matrix product
 * (THA_DT_BF16: bf16 with fp32 accumulation; THA_DT_F32: plain fp32 FMA, no reduced-precision matrix mode).  The
 * residual stream, norms, softmax, routers, gates, decays and all recurrent state are fp32 in both.
 * Small vectors (norm weights, biases, convolution taps, decay parameters) are always fp32 device arrays.
 * Matrices are row-major [out, in].  All pointers are device pointers unless named *_host.
 */
#ifndef THA_HYBRID_H
#define THA_HYBRID_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define THA_DT_BF16 0
#define THA_DT_F32 1

#define THA_MIX_PARALLEL 0 /* softmax attention and a matrix memory side by side, outputs normed and averaged */
#define THA_MIX_DELTA 1    /* gated delta rule with per-channel decay */
#define THA_MIX_GLA 2      /* gated linear attention: decayed outer-product memory, decay per key channel */
#define THA_MIX_LATENT 3   /* softmax attention whose keys and values are expanded from one cached low-rank latent */
#define THA_MIX_ATTN 4     /* softmax attention alone (tha_attn_t with its window, sink, per-head scale and gate options) */
#define THA_MIX_ATTN_GDELTA 5 /* softmax attention and a generalized delta rule side by side: mix_left * left + mix_right * right */
#define THA_MIX_HGRN 6     /* gated linear recurrence whose forget gate also decides what is written (tha_hgrn_t) */

#define THA_BLOCK_PARALLEL 0   /* x <- x + mixer(norm1 x) + ff(norm x): mixer and feed-forward read the same x */
#define THA_BLOCK_SEQUENTIAL 1 /* x <- x + m mixer(norm1 x), then x <- x + m ff(norm2 x), then the per-token side input */
#define THA_BLOCK_STREAMS 2    /* several residual streams: every sublayer reads a weighted sum of them and writes to all (tha_streams_t) */

#define THA_NORM_RMS 0     /* x / sqrt(mean(x^2) + eps) * (w_offset + w) */
#define THA_NORM_DYT 1     /* tanh(alpha * x) * w + b: element-wise, no statistics */
#define THA_NORM_LAYER 2   /* (x - mean) / sqrt(variance + eps) * w + b, variance = mean of the squared deviations */
#define THA_NORM_COPY 3    /* x itself in the product's number format (tha_hyb_add_norm, tha_hyb_block_finish) */

#define THA_FF_NONE 0
#define THA_FF_MOE 1
#define THA_FF_DENSE 2

#define THA_ACT_GLU_CLAMPED 0 /* g' = min(g, limit), u' = clamp(u, +-limit): g' sigmoid(alpha g') (u' + 1) */
#define THA_ACT_RELU2 1       /* max(u, 0)^2, no gate */
#define THA_ACT_GELU_TANH_GLU 2 /* gelu(g) u, gelu in its tanh form */
#define THA_ACT_XIELU 3       /* no gate; z > 0: softplus(p) z^2 + z / 2; z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z / 2 */
#define THA_ACT_SILU_GLU 4    /* g sigmoid(g) u */
#define THA_ACT_POLYNORM 5    /* no gate; over a row z: c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3, N(v) = v / sqrt(mean(v^2) + eps), powers by element
                                 (a reduction over the row: tha_hyb_polynorm) */

#define THA_ROUTE_TOPK_SOFTMAX 0    /* the top logits, softmax over the chosen */
#define THA_ROUTE_SOFTMAX_GROUPS 1  /* softmax over all experts; choice by score + correction inside the best groups of
                                       neighbouring experts; weights = the chosen scores (uncorrected) over their sum */

#define THA_GATE_SIGMOID 0
#define THA_GATE_SILU 1

#define THA_ROT_INTERLEAVED 0 /* rotary pairs (2i, 2i + 1) */
#define THA_ROT_HALVES 1      /* rotary pairs (i, i + dims / 2) */

/* The rows of one step.  Rows of a sequence are consecutive and in ascending position. */
typedef struct {
  int n_rows, n_seqs;
  const int* token;     /* [n_rows] */
  const int* pos;       /* [n_rows] position of the row in its sequence (from 0) */
  const int* row_seq;   /* [n_rows] index of the row's sequence in this step (0..n_seqs-1) */
  const int* seq_first; /* [n_seqs + 1] first row of each sequence; seq_first[n_seqs] == n_rows */
  const int* seq_slot;  /* [n_seqs] slot of the sequence: its block-table row and its state slot */
  int max_seq_rows;     /* longest portion of the step */
  int max_pos;          /* largest position of the step */
} tha_rows_t;

/* Paged cache: pools [block][cache layer][position in block][kv_dim] fp32, one table row of block ids per slot. */
typedef struct {
  float* k_pool;
  float* v_pool;
  const int* table;
  int table_stride; /* blocks per slot */
  int block_size;   /* positions per block, a power of two */
  int n_cache_layers;
  int kv_dim;       /* row pitch in floats (the widest K or V row of the model) */
} tha_kv_t;

/* Recurrent state: slot s starts at base + s * slot_floats. */
typedef struct {
  float* base;
  long long slot_floats;
} tha_state_store_t;

/* Rotary position tables: angle = position * inv_freq[i] (float64 on the device), cos and sin times `mag`. */
typedef struct {
  const double* inv_freq; /* [dims / 2] */
  int dims;               /* rotated dimensions of a head (pairs 2i, 2i+1), the rest pass unchanged */
  float mag;
} tha_rotary_t;

/* A norm over the width. */
typedef struct {
  int kind;          /* THA_NORM_* */
  const float* w;    /* [width] */
  const float* b;    /* [width], THA_NORM_DYT and THA_NORM_LAYER */
  float w_offset;    /* THA_NORM_RMS: 1 when the weight is stored around zero */
  float alpha;       /* THA_NORM_DYT */
} tha_norm_t;

/* Softmax attention over the cache.  A query at position p sees the keys j <= p with
 * floor(j / chunk) == floor(p / chunk) when chunk > 0, every j <= p otherwise; with window > 0 only those of them with
 * p - j < window or j < keep_first (nothing is renumbered: rotation and distances use absolute positions).
 * sink (per head): one more term exp(sink[h]) in the softmax's normalising sum; it brings no value, and neither `scale` nor
 * head_scale applies to it.
 * head_scale (per head): the scores of head h are multiplied by head_scale[h] on top of `scale`.
 * Output gate per head: head h's result is multiplied by sigmoid of column o_g + h of the stacked projection. */
typedef struct {
  int heads, kv_heads, dim, vdim;
  int rot;          /* index into the model's rotary tables, -1: none */
  int unit_rms;     /* 1: q and k are divided by their root mean square over dim after rotation */
  float eps;
  float scale;
  int chunk;
  int cache_layer;  /* which layer of the pool holds this layer's rows */
  int o_q, o_k, o_v; /* columns of the stacked input projection */
  const void* w_o;  /* [width, heads * vdim] */
  int values_in_keys; /* 1: a value row is the first vdim channels of its key row (vdim <= dim): callers pass the K pool as
                         v_pool as well, and kernels may stage one tile for both */
  /* zero-initialised, the fields below keep the behaviour described so far */
  int window, keep_first;  /* window 0: no window */
  const float* sink;       /* [heads], NULL: none */
  const float* head_scale; /* [heads], NULL: none */
  int rot_layout;          /* THA_ROT_* */
  int head_gate, o_g;      /* head_gate 1: `heads` gate columns at o_g; tha_hyb_attn_gated applies them */
  int fp32_scores;         /* 1: softmax weights are never rounded to bf16.  The tensor-core forms then multiply them with the
                              values as a bf16 pair hi + lo (16 mantissa bits) and sum the fp32 weights themselves; scores
                              accumulate in fp32 in every form */
  int v_share;             /* n > 1: key head g reads value head g / n (n key heads share one value head; kv_heads % n == 0; the
                              cache holds kv_heads / n value heads) */
  int out_f32;             /* 1: the result is written as fp32 in every number format */
  float q_temp_coef;       /* q_temp_every > 0: the query at position p is multiplied by */
  int q_temp_every;        /*   1 + q_temp_coef * ln(floor((p + 1) / q_temp_every) + 1) */
  int kv_shared;           /* 1: the layer writes no cache rows; cache_layer names the layer whose rows it reads (that layer runs
                              earlier in the step).  o_k / o_v are unused */
  /* Differential attention (diff 1): `heads` counts MAPS, two per output head, ordered per key/value group as [first maps of
   * the group's heads | second maps]; key head 2g is the first map's, 2g + 1 the second's, both read value head g (v_share 2).
   * tha_hyb_diff_combine makes o = a1 - diff_lambda a2, divides it by its root mean square over vdim, multiplies by diff_mult
   * and by the head's gate. */
  int diff;
  float diff_lambda, diff_mult;
  /* A short causal convolution (conv_taps > 0, no activation) over the projected q | k | v channels (q only with kv_shared)
   * before rotation; its taps [channels, conv_taps] in projection order; the last conv_taps - 1 projected rows are state. */
  int conv_taps;
  const float* conv_w;
  long long conv_state_off;
} tha_attn_t;

/* Generalized delta rule with a decay and a removal rate per key channel.  r, k, v, g: heads x dim columns each.
 *   decay   w = exp(-exp(-1/2) * sigmoid(W_w2 tanh(W_w1 h) + w0))      removal rate   a = sigmoid(W_a h + a_b)
 *   unit key u = k / sqrt(sum(k^2) + 1e-6) per head
 *   S' = diag(w) S - (a o u)(u^T S) + k v^T  (S on the right: the state before the token, throughout),   o = S'^T r
 * The read-out is divided by its root mean square per head, weighted (norm, [heads * dim]) and gated by sigmoid(g).
 * State per head: dim x dim floats laid out for the scan ([column pair][key channel][2], an odd last column padded). */
typedef struct {
  int heads, dim, rank;
  float eps;
  int o_r, o_k, o_v, o_g, o_a, o_w1; /* columns of the stacked input projection (w1: rank columns) */
  const void* w_w2;     /* [heads * dim, rank] */
  const float* w0;      /* [heads * dim] */
  const float* a_b;     /* [heads * dim] */
  const float* norm;    /* [heads * dim] */
  const void* w_o;      /* [width, heads * dim] */
  long long state_off;
} tha_gdelta_t;

/* Matrix memory with exponential input gate, sigmoid forget gate (both in log space, soft-capped) and a running
 * maximum that starts at 0.  State per head: S [dim, vdim], n [dim], m. */
typedef struct {
  int heads, dim, vdim;
  float gate_cap, eps;
  int o_q, o_k, o_v, o_g, o_i, o_f;
  const float* b_i; /* [heads] */
  const float* b_f; /* [heads] */
  const float* norm; /* [heads * vdim] */
  const void* w_o;  /* [width, heads * vdim] */
  long long state_off; /* floats from the slot's start */
} tha_mem_t;

/* Gated delta rule.  q / k have kv_heads heads of dim, v has heads heads of vdim; a short causal convolution
 * (taps, silu) runs over q | k | v, which are adjacent columns of the stacked projection starting at o_q.
 * State per head: S [dim, vdim]; plus the last taps-1 inputs of every convolved channel. */
typedef struct {
  int heads, kv_heads, dim, vdim, taps, rank_a, rank_g;
  float eps;
  int o_q, o_b, o_a1, o_g1; /* columns of the stacked projection (k follows q, v follows k) */
  const float* conv;   /* [channels, taps], channels = 2 * kv_heads * dim + heads * vdim */
  const void* w_a2;    /* [heads * dim, rank_a] */
  const void* w_g2;    /* [heads * vdim, rank_g] */
  const float* a_log;  /* [heads] */
  const float* dt_bias; /* [heads * dim] */
  const float* norm;   /* [vdim] */
  const void* w_o;     /* [width, heads * vdim] */
  long long state_off, conv_state_off;
} tha_delta_t;

/* Gated linear attention.  Per head S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T (q_t / sqrt(dim)), with the decay
 * a = sigmoid(z)^(1/tau) per key channel, z = W_a2 (W_a1 h) + b_a2.  The read-out is divided by its root mean square per
 * head, weighted (norm, [vdim], shared by the heads) and gated by silu(W_g h).  State per head: dim x vdim floats, laid out for the
 * scan ([column pair][key channel][2], an odd last column padded): heads * dim * (vdim rounded up to even) floats. */
typedef struct {
  int heads, dim, vdim, rank;
  float tau, eps;
  int o_q, o_k, o_v, o_g, o_a1; /* columns of the stacked input projection */
  const void* w_a2;    /* [heads * dim, rank] */
  const float* b_a2;   /* [heads * dim] */
  const float* norm;   /* [vdim] */
  const void* w_o;     /* [width, heads * vdim] */
  long long state_off;
} tha_gla_t;

/* Gated linear recurrence with a bounded forget gate.  q = silu(W_q h) (heads x dim), v = W_v h (heads x vdim),
 * f = lower + (1 - lower) * sigmoid(W_f h + f_b) per head and key channel;  S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,
 * o_t = S_t^T q_t.  The read-out is divided by its root mean square per head and weighted (norm, [vdim], shared by the
 * heads).  State per head as for tha_gla_t. */
typedef struct {
  int heads, dim, vdim;
  float eps;
  int o_q, o_f, o_v;    /* columns of the stacked input projection */
  const float* f_b;     /* [heads * dim] */
  const float* lower;   /* [heads * dim] */
  const float* norm;    /* [vdim] */
  const void* w_o;      /* [width, heads * vdim] */
  long long state_off;
} tha_hgrn_t;

/* Residual streams.  A model keeps n copies X[0..n-1] of its residual (all equal to the embedding output at the start).
 * A sublayer reads u = sum_s in[s] X[s], computes y = sublayer(norm(u)), and writes X'[t] = sum_s mix[s * n + t] X[s] + out[t] y
 * for every t at once.  "The residual stream" (taps, the final norm's input) is sum_s X[s]. */
typedef struct {
  const float* in;      /* [n] */
  const float* out;     /* [n] */
  const float* mix;     /* [n, n], indexed [from, to] */
} tha_streams_t;

/* Latent attention.  Queries: c_q = rmsnorm(W_dq h) * q_norm, q = W_uq c_q, per head [dim plain | rot_dim rotated].
 * Keys and values: W_dkv h = [kv_rank | rot_dim]; c = rmsnorm(first part) * kv_norm is the cached latent, the second part
 * (rotated) is one key part shared by all heads; per head k = W_uk c, v = W_uv c.  Only [c | rotated part] is cached
 * (kv_rank + rot_dim floats per position, in the K pool).  The score q_plain . W_uk c equals (W_uk^T q_plain) . c, so the
 * kernels attend with absorbed queries [W_uk^T q_plain | q_rot] over the cached rows as ONE key/value head of
 * kv_rank + rot_dim channels whose values are the latent itself, and expand the result with W_uv afterwards.
 * Output gate sigmoid(W_g h) on the concatenated heads. */
typedef struct {
  int heads, dim, rot_dim, vdim, q_rank, kv_rank;
  int rot;            /* index into the model's rotary tables (dims <= rot_dim), -1: none */
  float eps, scale;
  int cache_layer;
  int o_dq, o_dkv, o_g; /* columns of the stacked input projection: q_rank, kv_rank + rot_dim, heads * vdim */
  const float* q_norm;  /* [q_rank] */
  const float* kv_norm; /* [kv_rank] */
  const void* w_uq;     /* [heads * (dim + rot_dim), q_rank] */
  const void* w_uk_t;   /* [heads][kv_rank, dim]: W_uk of each head, transposed */
  const void* w_uv;     /* [heads][vdim, kv_rank] */
  const void* w_o;      /* [width, heads * vdim] */
  /* zero-initialised, the fields below keep the behaviour described above */
  int direct_q, o_q;    /* direct_q 1: no query latent; q = heads * (dim + rot_dim) columns at o_q of the stacked projection */
  int no_gate;          /* 1: no output gate */
  int window;           /* > 0: a query at p sees the keys j with 0 <= p - j < window */
  const float* sink;    /* [heads], NULL: none (see tha_attn_t) */
  int rot_layout;       /* THA_ROT_* */
  int fp32_scores;      /* see tha_attn_t */
} tha_latent_t;

/* Dense gated feed-forward: W_down act(W_gate h, W_up h). */
typedef struct {
  int ff, act;
  int o_gate, o_up;     /* columns of the feed-forward's stacked input projection (ungated activations: o_up only) */
  const void* w_down;   /* [width, ff] */
  float act_p, act_q;   /* THA_ACT_XIELU: the two stored numbers (softplus is taken by the kernel) */
  /* zero-initialised, the fields below keep the behaviour described above */
  const float* b_up;    /* [ff] added to W_up h before the activation, NULL: none */
  const float* b_down;  /* [width] added to the result, NULL: none */
  float act_c[4];       /* THA_ACT_POLYNORM: c0..c3 */
} tha_dense_ff_t;

/* Per-token side input of a layer, after its feed-forward: e = table[token, col0 : col0 + dim];
 * y = W_proj (gelu_tanh(W_gate x) * e); x <- x + m * y / sqrt(mean(y^2) + eps) * norm. */
typedef struct {
  int dim, col0;        /* dim 0: the layer has none */
  const void* w_gate;   /* [dim, width] */
  const void* w_proj;   /* [width, dim] */
  const float* norm;    /* [width] */
} tha_side_t;

/* Mixture of experts with clamped gated activation: g = min(gate, limit), u = clamp(up, -limit, limit),
 * y = g * sigmoid(alpha * g) * (u + 1).  Router: top-k logits, softmax over the chosen.  Optional shared expert. */
typedef struct {
  int experts, top, ff;
  float limit, alpha;
  int o_router;
  const void* w_gate_up; /* [experts][2 * ff, width]: an expert's gate rows, then its up rows */
  const void* w_down;    /* [experts][width, ff] */
  int shared_ff;         /* 0: none */
  float shared_limit;
  int o_sgate, o_sup;
  const void* w_sdown;   /* [width, shared_ff] */
  /* zero-initialised, the fields below keep the behaviour described above */
  int act;               /* THA_ACT_*; ungated activations: w_gate_up is [experts][ff, width] (up rows only) */
  int route;             /* THA_ROUTE_* */
  const float* correction; /* [experts], THA_ROUTE_SOFTMAX_GROUPS: added to the scores for the choice only */
  int groups, keep_groups; /* groups <= 1: every expert can be chosen */
  int shared_scaled;     /* 1: the shared expert's output is multiplied by sigmoid of column o_sscale (one number per row) */
  int o_sscale;
} tha_moe_t;

typedef struct {
  int mixer;            /* THA_MIX_* */
  tha_norm_t norm1;     /* the mixer's input norm (and the feed-forward's, unless norm2 is set) */
  const void* w_in;     /* every matrix that reads the normed input, stacked: [n_in, width] */
  int n_in;
  /* A second norm of the same x for the feed-forward (has_norm2): its matrices are stacked in w_in2 [n_in2, width] and
   * the column offsets of moe / dense refer to that product; without it they refer to w_in. */
  int has_norm2;
  tha_norm_t norm2;
  const void* w_in2;
  int n_in2;
  const float* scale_mix; /* [width] layer scale on the mixer's result, NULL: none */
  const float* scale_ff;  /* [width] layer scale on the feed-forward's result, NULL: none */
  tha_attn_t attn;      /* THA_MIX_PARALLEL */
  tha_mem_t mem;        /* THA_MIX_PARALLEL */
  const float* left_out;  /* [width] weights of the two sides' output norms */
  const float* right_out;
  tha_delta_t delta;    /* THA_MIX_DELTA */
  tha_gla_t gla;        /* THA_MIX_GLA */
  tha_latent_t latent;  /* THA_MIX_LATENT */
  int has_ff;           /* THA_FF_* */
  tha_moe_t moe;        /* THA_FF_MOE */
  tha_dense_ff_t dense; /* THA_FF_DENSE */
  /* zero-initialised, the fields below keep the behaviour described above */
  int block;            /* THA_BLOCK_*; sequential blocks: dense or no feed-forward, reading norm2 through w_in2 */
  float res_mult;       /* THA_BLOCK_SEQUENTIAL: m */
  tha_gdelta_t gdelta;  /* THA_MIX_ATTN_GDELTA (beside attn) */
  float mix_left, mix_right; /* THA_MIX_ATTN_GDELTA */
  tha_side_t side;
  /* before this run's first norm: x += the embedding output (pre_add_embed), then x += pre_vec ([width], NULL: none) */
  int pre_add_embed;
  const float* pre_vec;
  tha_hgrn_t hgrn;      /* THA_MIX_HGRN */
  /* THA_BLOCK_STREAMS: the two sublayers' stream weights; the feed-forward (dense or mixture, or none) reads norm2 through
   * w_in2.  in_conv_taps > 0: the mixer's normed input h is replaced by h + causal_conv(h) per channel (in_conv_w
   * [width, taps]); the last taps - 1 rows of h are state at in_conv_state_off. */
  tha_streams_t streams1, streams2;
  int in_conv_taps;
  const float* in_conv_w;
  long long in_conv_state_off;
} tha_hyb_layer_t;

typedef struct {
  int dtype;
  int width, vocab, n_layers;
  float eps;
  float logit_softcap;  /* 0: none */
  const void* embed;    /* [vocab, width] */
  const void* pos_embed; /* [max_positions, width] learned position vectors added to the embedding, NULL: none */
  int max_positions;
  tha_norm_t final_norm;
  const void* head;     /* [vocab, width] */
  /* host array of the layer RUNS in execution order: a layer that a model runs several times (a looped segment) appears
   * once per run with the same weight pointers and a cache layer / state offset of its own */
  const tha_hyb_layer_t* layers;
  int n_rot;
  const tha_rotary_t* rot;       /* host array */
  float embed_scale;             /* the embedding rows are multiplied by it; 0 reads as 1 */
  const void* side_table;        /* [vocab, side_cols]: the per-token side inputs of all layers, NULL: none */
  int side_cols;
  int n_streams;                 /* THA_BLOCK_STREAMS layers: copies of the residual (0 reads as 1; at most 16) */
} tha_hyb_model_t;

/* One scheduler step: every row through every layer; logits [n_want, vocab] (fp32) of the rows listed in want_rows.
 * `taps`, when not NULL, receives the residual stream after every layer: [n_layers, n_rows, width] fp32.
 * Stream-ordered; scratch is owned by the library and grows outside of any capture. */
int tha_hyb_step(void* stream, const tha_hyb_model_t* m, const tha_rows_t* rows, const tha_kv_t* kv,
                 const tha_state_store_t* st, int n_want, const int* want_rows, float* logits, float* taps);

/* ---- the mechanisms, one call each (also what tha_hyb_step is made of) ------------------------------------------- */
/* out[r, :] = x[r, :] / sqrt(mean(x[r]^2) + eps) * (w_offset + w), rows picked through `rows_idx` when not NULL;
 * out is dtype-typed (bf16 / fp32) */
int tha_hyb_rmsnorm(void* stream, int dtype, void* out, const float* x, const float* w, float w_offset, float eps,
                    int n_rows, int width, const int* rows_idx);
/* the norm `n` of rows of x (picked through rows_idx when not NULL); out is dtype-typed */
int tha_hyb_norm(void* stream, int dtype, void* out, const float* x, const tha_norm_t* n, float eps, int n_rows, int width,
                 const int* rows_idx);
/* two norms of the same rows (the two norms of a parallel block): one pass over x where the kinds allow it */
int tha_hyb_norm_pair(void* stream, int dtype, void* out1, void* out2, const float* x, const tha_norm_t* n1, const tha_norm_t* n2,
                      float eps, int n_rows, int width);
/* C[m, 0:N] = A[row(m), 0:K] . W_g[0:N, 0:K]^T, fp32 out.  a_f32: A is fp32 (else dtype-typed).  gather: row(m) =
 * a_rows[m] (NULL: m).  Groups: rows group_off[g] .. group_off[g+1]-1 use the matrix W + g * w_group_stride elements
 * (group_off NULL: one group of M rows). */
int tha_hyb_linear(void* stream, int dtype, float* C, long long ldc, const void* A, long long lda, int a_f32,
                   const int* a_rows, const void* W, long long w_group_stride, int M, int N, int K,
                   const int* group_off, int n_groups);
/* One product per head: C[m, h * c_hs + n] = sum_k A[m, h * a_hs + k] * W[h * w_hs + n * K + k], n < N, k < K, fp32 out.
 * a_f32: A is fp32 (else dtype-typed). */
int tha_hyb_linear_heads(void* stream, int dtype, float* C, long long ldc, long long c_hs, const void* A, long long lda,
                         long long a_hs, int a_f32, const void* W, long long w_hs, int M, int N, int K, int heads);
/* cos / sin [n_rows, dims/2] of the rows' positions */
int tha_hyb_rotary_table(void* stream, const tha_rotary_t* rot, const int* pos, int n_rows, float* cos_out, float* sin_out);
/* rotate q and k, unit-rms them, write k and v to the cache rows of (slot, pos), q to q_out [n_rows, heads * dim] */
int tha_hyb_attn_prepare(void* stream, const tha_attn_t* a, const tha_rows_t* rows, const tha_kv_t* kv, const float* proj,
                         long long ldp, const float* cos_t, const float* sin_t, int rot_dims, float* q_out);
/* tha_hyb_attn with the per-head output gate of a.head_gate read from proj (columns a.o_g ..); proj NULL: no gate */
int tha_hyb_attn_gated(void* stream, int dtype, const tha_attn_t* a, const tha_rows_t* rows, const tha_kv_t* kv, const float* q,
                       void* out, float* split_scratch, size_t split_scratch_floats, const float* proj, long long ldp);
/* the generalized delta rule over the rows of every sequence in order: the w1 columns of proj are replaced by their tanh,
 * w_raw [n_rows, heads * dim] receives W_w2 tanh(.) and then the decays, the a columns of proj become the removal rates;
 * the read-out goes to o_raw (fp32 [n_rows, heads * dim]) and, normed and gated, to out (dtype-typed) */
int tha_hyb_gdelta_scan(void* stream, int dtype, const tha_gdelta_t* g, const tha_rows_t* rows, const tha_state_store_t* st,
                        float* proj, long long ldp, float* w_raw, float* o_raw, void* out);
/* floats of one sequence's state of a generalized-delta-rule layer */
long long tha_hyb_gdelta_state_floats(int heads, int dim);
/* out (dtype-typed [n_rows, side->dim]) = gelu_tanh(gate_raw) * table[token, side->col0 ..]: the input of the side projection */
int tha_hyb_side_gate(void* stream, int dtype, void* out, const float* gate_raw, long long ldg, const tha_side_t* side,
                      const void* side_table, int side_cols, const int* token, int n_rows);
/* the end of a sequential block, one pass over x: x += m * ff (ff NULL: none); x += m * y / sqrt(mean(y^2) + eps) * y_norm
 * (y NULL: none); tap (nullable) receives x; then x += embed_out (nullable), x += vec (nullable), and with next_norm not
 * NULL out (dtype-typed) = that norm of x -- what comes ahead of the next layer run */
int tha_hyb_block_finish(void* stream, int dtype, float* x, const float* ff, const float* y, float m, const float* y_norm, float eps,
                         float* tap, const float* embed_out, const float* vec, const tha_norm_t* next_norm, void* out, int n_rows,
                         int width);
/* x += c_left * left + c_right * right (right NULL: none) (+ embed_out when given) (+ vec when given); then, with n not NULL,
 * out (dtype-typed) = the norm n of x (THA_NORM_COPY: x itself).  left NULL: only the optional addends. */
int tha_hyb_add_norm(void* stream, int dtype, float* x, const float* left, float c_left, const float* right, float c_right,
                     const float* embed_out, const float* vec, const tha_norm_t* n, float eps, void* out, int n_rows, int width);
/* softmax attention of every row over its visible cache rows; out dtype-typed [n_rows, heads * vdim].
 * split_scratch (nullable, fp32): room for the partial results when a step of few rows at long contexts is cut along
 * the keys (splits * n_rows * heads * (vdim + 2) floats are used, as many splits as fit, at most 16) */
int tha_hyb_attn(void* stream, int dtype, const tha_attn_t* a, const tha_rows_t* rows, const tha_kv_t* kv, const float* q,
                 void* out, float* split_scratch, size_t split_scratch_floats);
/* the matrix memory over the rows of every sequence in order, state read from and written back to the slots;
 * the two gate columns of proj are replaced by the log gates (a pass over all rows before the scan);
 * o_raw: fp32 scratch [n_rows, heads * vdim] (the read-out before the head norm);
 * out dtype-typed [n_rows, heads * vdim] = unit-rms per head * norm * sigmoid(gate) */
int tha_hyb_mem_scan(void* stream, int dtype, const tha_mem_t* m, const tha_rows_t* rows, const tha_state_store_t* st,
                     float* proj, long long ldp, float* o_raw, void* out);
/* causal convolution + silu over `channels` adjacent columns of proj starting at col0, continuing from the slot's
 * tail; out fp32 [n_rows, channels]; then the tails are advanced */
int tha_hyb_conv_silu(void* stream, const tha_rows_t* rows, const tha_state_store_t* st, long long conv_state_off,
                      const float* proj, long long ldp, int col0, int channels, int taps, const float* w, float* out);
/* the gated delta rule over the rows of every sequence in order; qkv = the convolved q | k | v, dt_raw [n_rows, heads*dim]
 * and gate_raw [n_rows, heads*vdim] the outputs of the two low-rank projections (before bias / softplus / sigmoid);
 * dt_raw is replaced by the decays and the write-strength column of proj by its sigmoid before the scan */
int tha_hyb_delta_scan(void* stream, int dtype, const tha_delta_t* d, const tha_rows_t* rows, const tha_state_store_t* st,
                       const float* qkv, float* proj, long long ldp, float* dt_raw, const float* gate_raw,
                       float* o_raw, void* out);
/* latent attention, before the query expansion: cq (dtype-typed [n_rows, q_rank]) = rmsnorm of the q_rank columns at o_dq
 * times q_norm; the cache row of (slot, pos) in the K pool = [rmsnorm of the kv_rank columns at o_dkv times kv_norm |
 * the following rot_dim columns, rotated] */
int tha_hyb_latent_prepare(void* stream, int dtype, const tha_latent_t* a, const tha_rows_t* rows, const tha_kv_t* kv,
                           const float* proj, long long ldp, const float* cos_t, const float* sin_t, int rot_dims, void* cq);
/* latent attention, after the query expansion qfull fp32 (row pitch ldq floats; 0: heads * (dim + rot_dim)): the plain
 * parts go to q_plain (dtype-typed [n_rows, heads * dim]), the rotated parts to columns kv_rank.. of q_abs (fp32 [n_rows,
 * heads * (kv_rank + rot_dim)]) whose first kv_rank columns per head the caller fills with W_uk^T q_plain */
int tha_hyb_latent_split_q(void* stream, int dtype, const tha_latent_t* a, int n_rows, const float* qfull, long long ldq,
                           const float* cos_t, const float* sin_t, int rot_dims, void* q_plain, float* q_abs);
/* out (dtype-typed [n_rows, heads * E]) = o_raw * gate_act(gate) (gate NULL: no gate), with do_norm: o_raw divided by its rms per head and
 * weighted by norm ([E], or [heads * E] with norm_per_head) first */
int tha_hyb_head_gate(void* stream, int dtype, void* out, const float* o_raw, int n_rows, int heads, int E, int do_norm,
                      float eps, const float* norm, int norm_per_head, const float* gate, long long ldg, int gate_act);
/* gated linear attention over the rows of every sequence in order: z_raw [n_rows, heads * dim] (W_a2 a1, before the bias)
 * is replaced by the decays; the read-out goes to o_raw (fp32 [n_rows, heads * vdim]) and, normed and gated, to out */
int tha_hyb_gla_scan(void* stream, int dtype, const tha_gla_t* g, const tha_rows_t* rows, const tha_state_store_t* st,
                     const float* proj, long long ldp, float* z_raw, float* o_raw, void* out);
/* router: expert ids and weights [n_rows, top]; rows sorted by expert: group_off (2 * (experts + 1) ints: the offsets,
 * then scratch), sorted_row [n_rows * top] and the position of (row, j) in that order, inv [n_rows * top] */
int tha_hyb_moe_route(void* stream, const tha_moe_t* e, const float* proj, long long ldp, int n_rows, int* expert_id,
                      float* weight, int* group_off, int* sorted_row, int* inv);
/* y = g * sigmoid(alpha g) * (u + 1) with the clamps; gu [n, ldg] holds gate at col_g and up at col_u; y dtype-typed [n, ff] */
int tha_hyb_glu_clamped(void* stream, int dtype, void* y, const float* gu, long long ldg, int col_g, int col_u, int n,
                        int ff, float limit, float alpha);
/* the same for any THA_ACT_* (ungated activations read col_u only; THA_ACT_XIELU takes its two stored numbers p, q as
 * (limit, alpha)) */
int tha_hyb_ff_act(void* stream, int dtype, int act, void* y, const float* gu, long long ldg, int col_g, int col_u, int n,
                   int ff, float limit, float alpha);

/* causal convolution over `channels` adjacent columns of proj starting at col0, continuing from the slot's tail (the last
 * taps - 1 inputs of every channel): out[r, c] = act(sum_j w[c, j] in(r - taps + 1 + j, c)) (+ in(r, c) with add_input);
 * act 0: none, 1: silu.  out fp32 [n_rows, channels] (out_f32) or dtype-typed.  The tails are NOT advanced (tha_hyb_conv_tail). */
int tha_hyb_conv(void* stream, int dtype, const tha_rows_t* rows, const tha_state_store_t* st, long long conv_state_off, const float* proj,
                 long long ldp, int col0, int channels, int taps, const float* w, int act, int add_input, int out_f32, void* out);
/* the tails of a convolution advanced by the step's rows */
int tha_hyb_conv_tail(void* stream, const tha_rows_t* rows, const tha_state_store_t* st, long long conv_state_off, const float* proj,
                      long long ldp, int col0, int channels, int taps);
/* Residual streams, one pass over the rows.  X [n_rows, n, width] fp32.  init (nullable): every stream is first set to
 * init [n_rows, width].  write (nullable): X'[t] = sum_s write->mix[s, t] X[s] + write->out[t] * y, where
 * y = dense (nullable) + bias (nullable) + sum_j weight[r, j] * down[inv[r, j]] (top picks of a mixture; top 0: none).
 * tap, sum_out (nullable, [n_rows, width]): sum_s X[s].  read (nullable): out (fp32 with out_f32, else dtype-typed) =
 * the norm of sum_s read->in[s] X[s]. */
int tha_hyb_streams(void* stream, int dtype, float* X, int n, const float* init, const tha_streams_t* write, const float* dense,
                    const float* bias, int top, const float* weight, const int* inv, const float* down, float* tap, float* sum_out,
                    const tha_streams_t* read, const tha_norm_t* norm, float eps, int out_f32, void* out, int n_rows, int width);
/* y (dtype-typed [n, ff]) = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 of z = gu[r, col_u ..] + bias (nullable) */
int tha_hyb_polynorm(void* stream, int dtype, void* y, const float* gu, long long ldg, int col_u, const float* bias, const float* c,
                     float eps, int n, int ff);
/* differential attention's combination (tha_attn_t::diff): att fp32 [n_rows, a->heads * vdim] in map order -> out dtype-typed
 * [n_rows, a->heads / 2 * vdim] in head order; gate columns at a->o_g of proj when a->head_gate */
int tha_hyb_diff_combine(void* stream, int dtype, const tha_attn_t* a, const float* att, const float* proj, long long ldp, void* out,
                         int n_rows);
/* the bounded-forget-gate recurrence over the rows of every sequence in order: the q columns of proj are replaced by their silu,
 * the f columns by 1 - f, decay [n_rows, heads * dim] receives f; read-out to o_raw (fp32), normed to out (dtype-typed) */
int tha_hyb_hgrn_scan(void* stream, int dtype, const tha_hgrn_t* g, const tha_rows_t* rows, const tha_state_store_t* st, float* proj,
                      long long ldp, float* decay, float* o_raw, void* out);

#ifdef __cplusplus
}
#endif
#endif
