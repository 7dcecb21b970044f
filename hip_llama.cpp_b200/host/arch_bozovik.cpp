// Bozovik: config.json -> layer program.
// A decoder of sequential pre-norm blocks with layer norms (weight and bias),
//     x <- x + m * mixer(norm1 x),   x <- x + m * ff(norm2 x),   x <- x + m * rms(W_proj (gelu_tanh(W_gate x) * e_token)) * w,
// whose embedding rows are multiplied by a constant and whose last step is a per-token side input: every layer owns a
// range of columns of one side table indexed by the token.
// Layer types:
//   "attention"         causal softmax attention with grouped key/value heads, rotary pairs (i, i + dims / 2), a factor per
//                       head on the scores, a constant 1 in the softmax's normalising sum (a sink fixed at zero), one sigmoid output
//                       gate per head;
//   "latent_attention"  queries straight from the layer input, keys and values expanded per head from one cached normed
//                       latent plus one rotated key part shared by the heads; sliding window; a learned sink per head;
//   "parallel"          two mixers reading the same input: softmax attention (window with kept first tokens, learned sink,
//                       gate per head) and a generalized delta rule (decay and removal rate per key channel, unit keys),
//                       summed with two constants.
// Feed-forward: none, or dense without a gate, W_down xielu(W_up h).
// "loop" runs a segment of the layer list several times with the same weights, every pass with a cache and state of its
// own; from the second pass on a pass starts by adding the embedding output to x again, and every pass then adds its own
// learned vector.  Every size and constant comes from the config; constants the design fixes live with the mechanisms.
#include <math.h>

#include "layer_model.hpp"

static void bozovik_rotary(const JsonValue& m, RotarySpec* rot, bool* on) {
  if (!m.has("rot")) return;
  const JsonValue& r = m.at("rot");
  *on = true;
  rot->dims = r.at("dims").integer();
  rot->base = r.at("base").number();
  rot->halves = true;
}

// softmax attention with grouped heads; `windowed`: the left side of a parallel mixer, else the mixer of its own
static void bozovik_attention(const JsonValue& m, const std::string& p, bool windowed, AttnSpec* out) {
  AttnSpec& a = *out;
  a.heads = m.at("heads").integer();
  a.kv_heads = m.at("kv_heads").integer();
  a.dim = m.at("dim").integer();
  a.vdim = m.at("vdim").integer();
  a.scale = (float)m.at("scale").number();
  bozovik_rotary(m, &a.rot, &a.rotary);
  a.q = p + "q"; a.k = p + "k"; a.v = p + "v"; a.g = p + "g"; a.o = p + "o";
  a.fp32_scores = true;
  if (windowed) {
    const JsonValue& k = m.at("mask");
    a.window = k.at("size").integer();
    a.keep_first = k.has("keep_first") ? k.at("keep_first").integer() : 0;
    if (a.window < 1) throw std::runtime_error("config: a window must hold at least the token itself");
    a.sink = p + "sink";
  } else {
    a.sink_zero = true;
    a.temp = p + "temp";
  }
}

static void bozovik_mixer(const JsonValue& L, const std::string& pre, LayerSpec* out) {
  LayerSpec& ls = *out;
  const std::string type = L.at("type").string();
  const JsonValue& m = L.at("mixer");
  const std::string p = pre + "mix.";
  if (type == "attention") {
    ls.mixer = THA_MIX_ATTN;
    bozovik_attention(m, p, false, &ls.attn);
  } else if (type == "parallel") {
    ls.mixer = THA_MIX_ATTN_GDELTA;
    bozovik_attention(m.at("left"), p + "left.", true, &ls.attn);
    const JsonValue& r = m.at("right");
    const std::string q = p + "right.";
    GDeltaSpec& g = ls.gdelta;
    g.heads = r.at("heads").integer();
    g.dim = r.at("dim").integer();
    g.r = q + "r"; g.k = q + "k"; g.v = q + "v"; g.g = q + "g"; g.a = q + "a"; g.a_b = q + "a.b";
    g.w1 = q + "w1"; g.w2 = q + "w2"; g.w0 = q + "w0"; g.norm = q + "norm"; g.o = q + "o";
    ls.mix_left = (float)m.at("left_scale").number();
    ls.mix_right = (float)m.at("right_scale").number();
  } else if (type == "latent_attention") {
    ls.mixer = THA_MIX_LATENT;
    LatentSpec& a = ls.latent;
    a.heads = m.at("heads").integer();
    a.dim = m.at("dim").integer();
    a.rot_dim = m.at("rot_dim").integer();
    a.vdim = m.at("vdim").integer();
    a.kv_rank = m.at("kv_rank").integer();
    a.scale = (float)m.at("scale").number();
    bozovik_rotary(m, &a.rot, &a.rotary);
    a.window = m.at("mask").at("size").integer();
    if (a.window < 1) throw std::runtime_error("config: a window must hold at least the token itself");
    a.q = p + "q"; a.dkv = p + "dkv"; a.dkv_norm = p + "dkv.norm"; a.uk = p + "uk"; a.uv = p + "uv";
    a.sink = p + "sink"; a.o = p + "o";
    a.fp32_scores = true;
  } else {
    throw std::runtime_error("config: unknown layer type '" + type + "'");
  }
}

static void bozovik_translate(const JsonValue& c, LayerProgramSpec* out) {
  LayerProgramSpec& s = *out;
  s.width = c.at("width").integer();
  s.vocab = c.at("vocab").integer();
  s.eps = (float)c.at("norm").at("eps").number();
  s.norm_kind = THA_NORM_LAYER;
  s.embed = "embed";
  s.embed_scale = (float)c.at("embedding").at("scale").number();
  s.final_norm = "final.norm";
  s.head = "head";
  const float m = (float)c.at("residual_mult").number();
  const JsonValue& layers = c.at("layers");
  if (layers.kind != JsonValue::Array) throw std::runtime_error("config: 'layers' must be a list");
  const int n = (int)layers.arr.size();
  int side_dim = 0;
  if (c.has("token_side")) {
    side_dim = c.at("token_side").at("dim").integer();
    if (side_dim < 1) throw std::runtime_error("config: 'token_side.dim' must be positive");
    s.side_table = "side.embed";
    s.side_cols = side_dim * n;
  }
  // the order of execution: the looped segment repeated in place
  int start = 0, stop = 0, times = 1;
  const bool loop = c.has("loop");
  if (loop) {
    const JsonValue& lp = c.at("loop");
    start = lp.at("start").integer();
    stop = lp.at("stop").integer();
    times = lp.at("times").integer();
    if (start < 0 || stop < start || stop > n || times < 0) throw std::runtime_error("config: 'loop' does not fit the layer list");
  }
  std::vector<int> first_run(n, -1);
  auto run = [&](int i, int pass) {   // pass >= 0: the first layer of that pass of the loop
    LayerSpec ls;
    const JsonValue& L = layers.arr[i];
    const std::string pre = "l" + std::to_string(i) + ".";
    ls.block = THA_BLOCK_SEQUENTIAL;
    ls.res_mult = m;
    ls.norm1 = pre + "norm1";
    bozovik_mixer(L, pre, &ls);
    if (L.has("mlp")) {   // absent or null: the layer has no feed-forward
      const JsonValue& f = L.at("mlp");
      const std::string kind = f.at("kind").string();
      if (kind != "dense") throw std::runtime_error("config: unknown feed-forward kind '" + kind + "'");
      ls.has_ff = true;
      ls.ff_kind = THA_FF_DENSE;
      ls.norm2 = pre + "norm2";
      ls.dense.ff = f.at("ff").integer();
      ls.dense.act = THA_ACT_XIELU;
      ls.dense.up = pre + "mlp.up"; ls.dense.down = pre + "mlp.down"; ls.dense.act_params = pre + "mlp.act";
    }
    if (side_dim > 0) {
      ls.side.dim = side_dim;
      ls.side.col0 = i * side_dim;
      ls.side.gate = pre + "side.gate"; ls.side.proj = pre + "side.proj"; ls.side.norm = pre + "side.norm";
    }
    if (pass >= 0) {
      ls.pre_add_embed = pass > 0;
      ls.pre_vec = "loop.step";
      ls.pre_vec_row = pass;
    }
    if (first_run[i] >= 0) ls.same_weights_as = first_run[i];
    else first_run[i] = (int)s.layers.size();
    s.layers.push_back(ls);
  };
  for (int i = 0; i < start; i++) run(i, -1);
  for (int t = 0; t < times; t++)
    for (int i = start; i < stop; i++) run(i, loop && i == start ? t : -1);
  for (int i = stop; i < n; i++) run(i, -1);
}

void register_bozovik() { register_architecture({"Bozovik", ModelFamily::LayerProgram, bozovik_translate}); }
