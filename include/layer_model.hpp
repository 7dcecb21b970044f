// layer_model.hpp -- models described by data: the registry of architectures, the description a config.json is
// translated into, and the loader that turns description + tensor file into device-resident tha_hyb_model_t.
//
// The llama2 family (include/models.hpp) is one fixed struct read from a llama2.c checkpoint.  A layer-program model is
// a folder with config.json and model.safetensors; its "architecture" key picks a translator from the registry, which
// names, layer by layer, the mechanisms (include/tha_hybrid.h) with their sizes, constants and tensor names.  A new
// design that combines the same mechanisms differently registers another translator; a new mechanism is added to
// tha_hybrid.h once and becomes available to every translator.
#pragma once
#include <stdint.h>

#include <map>
#include <string>
#include <vector>

#include "json_min.hpp"
#include "tha_hybrid.h"

// ---- description (host side, tensor NAMES instead of pointers) --------------------------------------------------------
struct RotarySpec {
  int dims = 0;
  double base = 10000.0;
  bool halves = false;        // pairs (i, i + dims / 2) instead of (2i, 2i + 1); the table is the same, the kernels pair by it
  bool yarn = false;          // frequency interpolation between a fast and a slow wavelength bound
  double factor = 1.0, original = 0.0, fast = 32.0, slow = 1.0;
  // stretch by wavelength l = 2 pi / f against the original context: f kept where l < original / high, f / factor where
  // l > original / low, between them (1 - s) f / factor + s f with s = (original / l - low) / (high - low); amplitude 1
  bool by_wavelength = false;
  double low = 1.0, high = 4.0;
  bool operator==(const RotarySpec& o) const {
    return dims == o.dims && base == o.base && yarn == o.yarn && factor == o.factor && original == o.original && fast == o.fast &&
           slow == o.slow && by_wavelength == o.by_wavelength && low == o.low && high == o.high;
  }
};
struct AttnSpec {
  int heads = 0, kv_heads = 0, dim = 0, vdim = 0, chunk = 0;
  bool rotary = false, unit_rms = false;
  RotarySpec rot;
  float scale = 1.0f;
  std::string q, k, v, o;
  int window = 0, keep_first = 0;        // window 0: every earlier position of the block of positions is seen
  std::string sink;                      // [heads] a learned score in the softmax denominator; empty: none
  bool sink_zero = false;                // a sink fixed at zero (a constant 1 in the normalising sum): no tensor
  std::string temp;                      // [heads] per-head factor on the scores; empty: none
  std::string g;                         // [heads, width] one sigmoid output gate per head; empty: none
  bool fp32_scores = false;              // scores and softmax weights stay fp32 in every number format
  // differential attention: q holds heads x 2 x dim rows and k kv_heads x 2 x dim rows ([first map | second map] per head), both
  // maps read the same values; o = a1 - lambda a2 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff_init, then o / rms(o)
  // times (1 - diff_init) and the head's gate
  bool diff = false;
  float diff_init = 0.f;
  std::string lq1, lk1, lq2, lk2;        // [dim] each
  float q_temp_coef = 0.f;               // q_temp_every > 0: queries times 1 + coef * ln(floor((p + 1) / every) + 1)
  int q_temp_every = 0;
  int conv_taps = 0;                     // > 0: a short causal convolution behind the q, k and v projections ("<tensor>.conv")
  int kv_from = -1;                      // >= 0: no key / value tensors; the layer reads the cache rows of that layer (index into `layers`)
};
struct HgrnSpec {
  int heads = 0, dim = 0, vdim = 0;
  std::string q, f, f_b, lower, v, norm, o;
};
struct StreamsSpec {
  std::string in, out, mix;              // [n], [n], [n, n]
};
struct GDeltaSpec {
  int heads = 0, dim = 0;
  std::string r, k, v, g, a, a_b, w1, w2, w0, norm, o;   // the rank of w1 / w2 is read from the tensors
};
struct SideSpec {
  int dim = 0, col0 = 0;                 // dim 0: none
  std::string gate, proj, norm;
};
struct MemSpec {
  int heads = 0, dim = 0, vdim = 0;
  float gate_cap = 15.0f;
  std::string q, k, v, g, o, norm, i, i_b, f, f_b;
};
struct DeltaSpec {
  int heads = 0, kv_heads = 0, dim = 0, vdim = 0, taps = 1;
  std::string q, k, v, q_conv, k_conv, v_conv, b, a_log, norm, a1, a2, dt_bias, g1, g2, o;
};
struct GlaSpec {
  int heads = 0, dim = 0, vdim = 0;
  float tau = 1.0f;
  std::string q, k, v, g, o, norm, a1, a2, a2_b;   // the rank of a1 / a2 is read from the tensors
};
struct LatentSpec {
  int heads = 0, dim = 0, rot_dim = 0, vdim = 0, q_rank = 0, kv_rank = 0;
  bool rotary = false;
  RotarySpec rot;
  float scale = 1.0f;
  std::string dq, dq_norm, uq, dkv, dkv_norm, uk, uv, g, o;
  std::string q;                         // queries straight from the layer input [heads * (dim + rot_dim), width]: no query latent
  int window = 0;                        // > 0: sliding window
  std::string sink;                      // [heads]; empty: none
  bool fp32_scores = false;
};
struct DenseSpec {
  int ff = 0, act = THA_ACT_GELU_TANH_GLU;
  std::string gate, up, down;            // ungated activations have no `gate`
  std::string act_params;                // THA_ACT_XIELU: [2]; THA_ACT_POLYNORM: [4]
  std::string up_b, down_b;              // biases; empty: none
};
struct MoeSpec {
  int experts = 0, top = 0, ff = 0, shared_ff = 0;
  float limit = 0.f, shared_limit = 0.f, alpha = 1.702f;
  std::string router, prefix;            // expert e's tensors: prefix + "e<e>.gate" / ".up" / ".down" (ungated: no ".gate")
  std::string s_gate, s_up, s_down;
  int act = THA_ACT_GLU_CLAMPED, route = THA_ROUTE_TOPK_SOFTMAX;
  std::string correction;                // THA_ROUTE_SOFTMAX_GROUPS
  int groups = 0, keep_groups = 0;
  std::string s_scale;                   // [1, width]: the shared expert is multiplied by sigmoid of this product; empty: none
};
struct LayerSpec {
  int mixer = THA_MIX_PARALLEL;
  // >= 0: this entry runs the weights of that earlier entry once more (a looped segment) with a cache layer and state of
  // its own; the other fields are copies
  int same_weights_as = -1;
  std::string norm1;
  std::string norm2;                     // a second norm of the same x for the feed-forward; empty: it reads norm1's output
  std::string scale_mix, scale_ff;       // layer scales [width]; empty: none
  GlaSpec gla;
  LatentSpec latent;
  int ff_kind = THA_FF_MOE;              // with has_ff
  DenseSpec dense;
  AttnSpec attn;
  MemSpec mem;
  std::string left_out, right_out;
  DeltaSpec delta;
  int block = THA_BLOCK_PARALLEL;
  float res_mult = 1.0f;                 // sequential blocks
  GDeltaSpec gdelta;                     // THA_MIX_ATTN_GDELTA (beside attn)
  float mix_left = 1.0f, mix_right = 1.0f;
  SideSpec side;
  bool pre_add_embed = false;            // before this run: x += the embedding output
  std::string pre_vec;                   // before this run: x += row pre_vec_row of this [rows, width] tensor; empty: none
  int pre_vec_row = 0;
  bool has_ff = false;
  MoeSpec moe;
  HgrnSpec hgrn;                         // THA_MIX_HGRN
  StreamsSpec streams1, streams2;        // THA_BLOCK_STREAMS
  std::string in_conv;                   // [width, taps]: the mixer's normed input h becomes h + conv(h); empty: none
  int in_conv_taps = 0;
};
struct LayerProgramSpec {
  int width = 0, vocab = 0;
  float eps = 1e-5f, logit_softcap = 0.f;
  // every norm over the width (the layers' and the final one): THA_NORM_RMS with weights stored around zero, or
  // THA_NORM_DYT with "<name>.alpha" (a scalar) and "<name>.b" beside the weight
  int norm_kind = THA_NORM_RMS;
  float norm_w_offset = 1.0f;            // THA_NORM_RMS: what is added to the stored weight (0: the weight is stored as it is used)
  int n_streams = 0;                     // THA_BLOCK_STREAMS layers: copies of the residual
  float embed_scale = 1.0f;
  std::string side_table;                // [vocab, side_cols]: per-token side inputs, a column range per layer; empty: none
  int side_cols = 0;
  std::string pos_embed;                 // learned position vectors [max_positions, width]; empty: none
  int max_positions = 0;                 // 0: no limit from the model
  std::string embed, final_norm, head;
  std::vector<LayerSpec> layers;
};

// ---- registry -----------------------------------------------------------------------------------------------------
enum class ModelFamily { Llama2Checkpoint, LayerProgram };
struct ArchitectureEntry {
  std::string name;
  ModelFamily family;
  // LayerProgram: fill `out` from the parsed config.json; throw std::runtime_error on a config it cannot serve
  void (*translate)(const JsonValue& config, LayerProgramSpec* out);
};
void register_architecture(const ArchitectureEntry& e);
const ArchitectureEntry* find_architecture(const std::string& name);
std::vector<std::string> registered_architectures();
// A folder with config.json -> the entry its "architecture" names (config parsed into *config); a llama2.c checkpoint
// file -> the "llama2" entry.  nullptr + *err when neither.
const ArchitectureEntry* detect_model(const std::string& path, JsonValue* config, std::string* err);

// ---- tensor file ----------------------------------------------------------------------------------------------------
struct TensorInfo { std::string dtype; std::vector<long long> shape; size_t begin = 0, end = 0; };
class SafeTensors {
 public:
  bool open(const std::string& path, std::string* err);
  ~SafeTensors();
  bool has(const std::string& name) const { return index_.count(name) > 0; }
  const TensorInfo& info(const std::string& name) const;
  size_t numel(const std::string& name) const;
  // append the tensor's values to `out` as fp32 / as raw bf16 bit patterns (rounding fp32 to nearest even)
  void read_f32(const std::string& name, std::vector<float>* out) const;
  void read_bf16(const std::string& name, std::vector<uint16_t>* out) const;

 private:
  std::map<std::string, TensorInfo> index_;
  const unsigned char* data_ = nullptr;   // start of the data section inside the mapping
  void* map_ = nullptr;
  size_t map_bytes_ = 0;
};

// ---- the loaded model ---------------------------------------------------------------------------------------------
class LayerModel {
 public:
  // dtype: THA_DT_BF16 or THA_DT_F32.  Uploads to the current device.
  static LayerModel* load(const std::string& folder, int dtype, std::string* err);
  static LayerModel* build(const LayerProgramSpec& spec, const SafeTensors& file, int dtype, std::string* err);
  ~LayerModel();

  const tha_hyb_model_t* device_model() const { return &model_; }
  const LayerProgramSpec& spec() const { return spec_; }
  int vocab() const { return spec_.vocab; }
  int max_positions() const { return spec_.pos_embed.empty() ? 0 : spec_.max_positions; }   // 0: no limit
  int n_cache_layers() const { return n_cache_layers_; }
  int kv_dim() const { return kv_dim_; }                    // widest K or V row (floats)
  bool separate_values() const { return separate_values_; } // false: every cached layer's values lie inside its key rows
  long long state_floats() const { return state_floats_; }  // recurrent state of one sequence
  size_t weight_bytes() const { return weight_bytes_; }

 private:
  LayerModel() {}
  void* upload(const void* host, size_t bytes);
  LayerProgramSpec spec_;
  tha_hyb_model_t model_ = {};
  std::vector<tha_hyb_layer_t> layers_;
  std::vector<tha_rotary_t> rot_;
  std::vector<RotarySpec> rot_specs_;
  std::vector<void*> owned_;
  int n_cache_layers_ = 0, kv_dim_ = 0;
  bool separate_values_ = false;
  long long state_floats_ = 0;
  size_t weight_bytes_ = 0;
};
