// Mozetar: config.json -> layer program.
// A decoder over several residual streams: every sublayer reads a learned weighted sum of the streams, and its result is
// written to all of them beside a learned mixing of the old ones (THA_BLOCK_STREAMS).  Norms are plain rms norms (the weight
// is stored as it is used).  The mixer's normed input h is first replaced by h + conv(h), a causal convolution per channel.
// Layer types:
//   "attention"    differential attention: two softmax maps per head over the same values, o = a1 - lambda a2, normed per head
//                  and gated per head; causal, no rotation; queries grow with the logarithm of their position;
//   "attention_2"  sliding-window softmax attention with a short convolution behind the q, k and v projections, rotary pairs
//                  (2i, 2i + 1) on the first dims of a head with frequencies stretched by wavelength; "kv_from" names an earlier
//                  layer whose cache rows the layer reads instead of projecting keys and values of its own;
//   "hgrn2"        a gated linear recurrence whose bounded forget gate f also decides what is written (1 - f).
// Feed-forward: none, dense with biases and the PolyNorm activation, or a mixture of silu-gated experts whose router takes
// softmax scores over all experts, keeps to the best groups of neighbouring experts and weighs the chosen by their scores
// over their sum.  Every size and constant comes from the config; constants the design fixes live with the mechanisms.
#include <math.h>

#include "layer_model.hpp"

static void mozetar_attention_sizes(const JsonValue& m, const std::string& p, AttnSpec* out) {
  AttnSpec& a = *out;
  a.heads = m.at("heads").integer();
  a.kv_heads = m.at("kv_heads").integer();
  a.dim = m.at("dim").integer();
  a.vdim = m.at("vdim").integer();
  a.scale = (float)m.at("scale").number();
  a.q = p + "q"; a.k = p + "k"; a.v = p + "v"; a.o = p + "o";
  a.fp32_scores = true;
}

static void mozetar_mixer(const JsonValue& L, const std::string& pre, int index, int n_layers, LayerSpec* out) {
  LayerSpec& ls = *out;
  const std::string type = L.at("type").string();
  const JsonValue& m = L.at("mixer");
  const std::string p = pre + "mix.";
  if (type == "attention") {
    ls.mixer = THA_MIX_ATTN;
    AttnSpec& a = ls.attn;
    mozetar_attention_sizes(m, p, &a);
    a.diff = true;
    a.diff_init = (float)m.at("diff").number();
    a.lq1 = p + "lq1"; a.lk1 = p + "lk1"; a.lq2 = p + "lq2"; a.lk2 = p + "lk2";
    a.g = p + "g";
    if (m.has("q_temp")) {
      a.q_temp_coef = (float)m.at("q_temp").at("coef").number();
      a.q_temp_every = m.at("q_temp").at("every").integer();
      if (a.q_temp_every < 1) throw std::runtime_error("config: 'q_temp.every' must be positive");
    }
  } else if (type == "attention_2") {
    ls.mixer = THA_MIX_ATTN;
    AttnSpec& a = ls.attn;
    mozetar_attention_sizes(m, p, &a);
    if (m.has("conv")) {   // absent: the projections are used as they are
      a.conv_taps = m.at("conv").integer();
      if (a.conv_taps < 1) throw std::runtime_error("config: 'conv' must be at least one tap");
    }
    if (m.has("rot")) {
      const JsonValue& r = m.at("rot");
      a.rotary = true;
      a.rot.dims = r.at("dims").integer();
      a.rot.base = r.at("base").number();
      if (r.has("scaling")) {
        const JsonValue& sc = r.at("scaling");
        a.rot.by_wavelength = true;
        a.rot.factor = sc.at("factor").number();
        a.rot.low = sc.at("low").number();
        a.rot.high = sc.at("high").number();
        a.rot.original = sc.at("original").number();
      }
    }
    if (m.has("mask")) {   // absent: every earlier position is seen
      a.window = m.at("mask").at("size").integer();
      if (a.window < 1) throw std::runtime_error("config: a window must hold at least the token itself");
    }
    if (m.has("kv_from")) {
      a.kv_from = m.at("kv_from").integer();
      if (a.kv_from < 0 || a.kv_from >= index) throw std::runtime_error("config: 'kv_from' must name an earlier layer");
    }
  } else if (type == "hgrn2") {
    ls.mixer = THA_MIX_HGRN;
    HgrnSpec& g = ls.hgrn;
    g.heads = m.at("heads").integer();
    g.dim = m.at("dim").integer();
    g.vdim = m.at("vdim").integer();
    g.q = p + "q"; g.f = p + "f"; g.f_b = p + "f.b"; g.lower = p + "lower"; g.v = p + "v"; g.norm = p + "norm"; g.o = p + "o";
  } else {
    throw std::runtime_error("config: unknown layer type '" + type + "'");
  }
  (void)n_layers;
}

static void mozetar_translate(const JsonValue& c, LayerProgramSpec* out) {
  LayerProgramSpec& s = *out;
  s.width = c.at("width").integer();
  s.vocab = c.at("vocab").integer();
  s.eps = (float)c.at("norm").at("eps").number();
  s.norm_kind = THA_NORM_RMS;
  s.norm_w_offset = 0.0f;
  s.n_streams = c.has("streams") ? c.at("streams").integer() : 1;
  if (s.n_streams < 1 || s.n_streams > 16) throw std::runtime_error("config: 'streams' must be between 1 and 16");
  s.embed = "embed";
  s.final_norm = "final.norm";
  s.head = "head";
  const int canon_taps = c.has("canon") ? c.at("canon").at("taps").integer() : 0;
  if (c.has("canon") && canon_taps < 1) throw std::runtime_error("config: 'canon.taps' must be at least one");
  const JsonValue& layers = c.at("layers");
  if (layers.kind != JsonValue::Array) throw std::runtime_error("config: 'layers' must be a list");
  const int n = (int)layers.arr.size();
  for (int i = 0; i < n; i++) {
    LayerSpec ls;
    const JsonValue& L = layers.arr[i];
    const std::string pre = "l" + std::to_string(i) + ".";
    ls.block = THA_BLOCK_STREAMS;
    ls.norm1 = pre + "norm1";
    ls.streams1 = {pre + "hc1.in", pre + "hc1.out", pre + "hc1.mix"};
    if (canon_taps > 0) { ls.in_conv = pre + "canon1"; ls.in_conv_taps = canon_taps; }
    mozetar_mixer(L, pre, i, n, &ls);
    if (L.has("mlp")) {   // absent or null: the layer has no feed-forward
      const JsonValue& f = L.at("mlp");
      const std::string kind = f.at("kind").string();
      const std::string q = pre + "mlp.";
      ls.has_ff = true;
      ls.norm2 = pre + "norm2";
      ls.streams2 = {pre + "hc2.in", pre + "hc2.out", pre + "hc2.mix"};
      if (kind == "dense") {
        ls.ff_kind = THA_FF_DENSE;
        ls.dense.ff = f.at("ff").integer();
        ls.dense.act = THA_ACT_POLYNORM;
        ls.dense.up = q + "up"; ls.dense.up_b = q + "up.b"; ls.dense.down = q + "down"; ls.dense.down_b = q + "down.b";
        ls.dense.act_params = q + "act";
      } else if (kind == "moe") {
        ls.ff_kind = THA_FF_MOE;
        MoeSpec& e = ls.moe;
        const JsonValue& r = f.at("router");
        e.experts = r.at("experts").integer();
        e.top = r.at("top").integer();
        e.ff = f.at("expert").at("ff").integer();
        e.act = THA_ACT_SILU_GLU;
        e.route = THA_ROUTE_SOFTMAX_GROUPS;
        if (r.has("groups")) {
          e.groups = r.at("groups").at("count").integer();
          e.keep_groups = r.at("groups").at("keep").integer();
        }
        e.router = q + "router";
        e.prefix = q;
      } else {
        throw std::runtime_error("config: unknown feed-forward kind '" + kind + "'");
      }
    }
    s.layers.push_back(ls);
  }
}

void register_mozetar() { register_architecture({"Mozetar", ModelFamily::LayerProgram, mozetar_translate}); }
