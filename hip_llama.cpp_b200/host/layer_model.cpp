// The registry of architectures, the safetensors reader and the loader of layer-program models (include/layer_model.hpp).
#include "layer_model.hpp"

#include <fcntl.h>
#include <math.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <fstream>
#include <mutex>
#include <sstream>

#include "tha_b200.h"

void register_timerax();   // host/arch_timerax.cpp
void register_numizen();   // host/arch_numizen.cpp
void register_bozovik();   // host/arch_bozovik.cpp
void register_mozetar();   // host/arch_mozetar.cpp

// ---- registry -----------------------------------------------------------------------------------------------------
static std::vector<ArchitectureEntry>& registry() {
  static std::vector<ArchitectureEntry> r;
  return r;
}
static void register_builtin() {
  static std::once_flag once;
  std::call_once(once, [] {
    registry().push_back({"llama2", ModelFamily::Llama2Checkpoint, nullptr});   // llama2.c v0 / v2 checkpoint files (host/utils.cpp)
    register_timerax();
    register_numizen();
    register_bozovik();
    register_mozetar();
  });
}
void register_architecture(const ArchitectureEntry& e) {
  for (auto& x : registry())
    if (x.name == e.name) { x = e; return; }
  registry().push_back(e);
}
const ArchitectureEntry* find_architecture(const std::string& name) {
  register_builtin();
  for (auto& x : registry())
    if (x.name == name) return &x;
  return nullptr;
}
std::vector<std::string> registered_architectures() {
  register_builtin();
  std::vector<std::string> out;
  for (auto& x : registry()) out.push_back(x.name);
  return out;
}
const ArchitectureEntry* detect_model(const std::string& path, JsonValue* config, std::string* err) {
  register_builtin();
  struct stat sb;
  if (stat(path.c_str(), &sb) != 0) { if (err) *err = "cannot open " + path; return nullptr; }
  if (!S_ISDIR(sb.st_mode)) return find_architecture("llama2");
  std::ifstream f(path + "/config.json");
  if (!f) { if (err) *err = path + "/config.json is missing"; return nullptr; }
  std::stringstream ss;
  ss << f.rdbuf();
  try {
    JsonValue c = JsonValue::parse(ss.str());
    const std::string name = c.at("architecture").string();
    const ArchitectureEntry* e = find_architecture(name);
    if (!e && err) {
      *err = "architecture '" + name + "' is not registered (known:";
      for (auto& n : registered_architectures()) *err += " " + n;
      *err += ")";
    }
    if (config) *config = c;
    return e;
  } catch (const std::exception& ex) {
    if (err) *err = ex.what();
    return nullptr;
  }
}

// ---- safetensors: 8-byte little-endian header length, JSON header, raw data ---------------------------------------
bool SafeTensors::open(const std::string& path, std::string* err) {
  const int fd = ::open(path.c_str(), O_RDONLY);
  if (fd < 0) { if (err) *err = "cannot open " + path; return false; }
  struct stat sb;
  fstat(fd, &sb);
  map_bytes_ = (size_t)sb.st_size;
  map_ = mmap(nullptr, map_bytes_, PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (map_ == MAP_FAILED || map_bytes_ < 8) { map_ = nullptr; if (err) *err = "cannot map " + path; return false; }
  const unsigned char* p = (const unsigned char*)map_;
  uint64_t n = 0;
  for (int i = 7; i >= 0; i--) n = (n << 8) | p[i];
  if (8 + n > map_bytes_) { if (err) *err = path + ": bad header length"; return false; }
  try {
    JsonValue h = JsonValue::parse(std::string((const char*)p + 8, (size_t)n));
    for (auto& kv : h.obj) {
      if (kv.first == "__metadata__") continue;
      TensorInfo t;
      t.dtype = kv.second.at("dtype").string();
      for (auto& d : kv.second.at("shape").arr) t.shape.push_back((long long)d.number());
      t.begin = (size_t)kv.second.at("data_offsets").arr.at(0).number();
      t.end = (size_t)kv.second.at("data_offsets").arr.at(1).number();
      if (8 + n + t.end > map_bytes_ || t.begin > t.end) throw std::runtime_error("tensor '" + kv.first + "' lies outside the file");
      index_[kv.first] = t;
    }
  } catch (const std::exception& ex) {
    if (err) *err = path + ": " + ex.what();
    return false;
  }
  data_ = p + 8 + n;
  return true;
}
SafeTensors::~SafeTensors() { if (map_) munmap(map_, map_bytes_); }
const TensorInfo& SafeTensors::info(const std::string& name) const {
  auto it = index_.find(name);
  if (it == index_.end()) throw std::runtime_error("tensor '" + name + "' is missing");
  return it->second;
}
size_t SafeTensors::numel(const std::string& name) const {
  size_t n = 1;
  for (long long d : info(name).shape) n *= (size_t)d;
  return n;
}
static inline float bf16_to_f32(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u; memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);   // NaN stays NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
void SafeTensors::read_f32(const std::string& name, std::vector<float>* out) const {
  const TensorInfo& t = info(name);
  const size_t n = numel(name);
  const unsigned char* p = data_ + t.begin;
  if (t.dtype == "BF16") {
    if (t.end - t.begin != 2 * n) throw std::runtime_error("tensor '" + name + "': size does not fit its shape");
    for (size_t i = 0; i < n; i++) { uint16_t b; memcpy(&b, p + 2 * i, 2); out->push_back(bf16_to_f32(b)); }
  } else if (t.dtype == "F32") {
    if (t.end - t.begin != 4 * n) throw std::runtime_error("tensor '" + name + "': size does not fit its shape");
    for (size_t i = 0; i < n; i++) { float f; memcpy(&f, p + 4 * i, 4); out->push_back(f); }
  } else if (t.dtype == "I32") {   // integer tables, read as numbers
    if (t.end - t.begin != 4 * n) throw std::runtime_error("tensor '" + name + "': size does not fit its shape");
    for (size_t i = 0; i < n; i++) { int32_t v; memcpy(&v, p + 4 * i, 4); out->push_back((float)v); }
  } else {
    throw std::runtime_error("tensor '" + name + "': dtype " + t.dtype + " is not served");
  }
}
void SafeTensors::read_bf16(const std::string& name, std::vector<uint16_t>* out) const {
  const TensorInfo& t = info(name);
  const size_t n = numel(name);
  const unsigned char* p = data_ + t.begin;
  if (t.dtype == "BF16") {
    if (t.end - t.begin != 2 * n) throw std::runtime_error("tensor '" + name + "': size does not fit its shape");
    const size_t at = out->size();
    out->resize(at + n);
    memcpy(out->data() + at, p, 2 * n);
  } else {
    std::vector<float> f;
    read_f32(name, &f);
    for (float v : f) out->push_back(f32_to_bf16(v));
  }
}

// ---- loader ---------------------------------------------------------------------------------------------------------
LayerModel::~LayerModel() {
  for (void* p : owned_) tha_free(p);
}
void* LayerModel::upload(const void* host, size_t bytes) {
  void* d = nullptr;
  if (tha_malloc(&d, bytes ? bytes : 16) != 0) throw std::runtime_error(std::string("device allocation failed: ") + tha_last_error());
  owned_.push_back(d);
  if (bytes && tha_memcpy_h2d(d, host, bytes) != 0) throw std::runtime_error(std::string("upload failed: ") + tha_last_error());
  weight_bytes_ += bytes;
  return d;
}

namespace {
// matrices of one stack, in order; rows of each
struct Stack {
  const SafeTensors& file;
  int dtype, cols;
  std::vector<float> f;
  std::vector<uint16_t> h;
  int rows = 0;
  Stack(const SafeTensors& file_, int dtype_, int cols_) : file(file_), dtype(dtype_), cols(cols_) {}
  // returns the first row of the added matrix; checks [rows_expected, cols]
  int add(const std::string& name, long long rows_expected, const std::vector<int>* order = nullptr) {
    const TensorInfo& t = file.info(name);
    const long long r = t.shape.size() == 2 ? t.shape[0] : -1, c = t.shape.size() == 2 ? t.shape[1] : -1;
    if (r != rows_expected || c != cols)
      throw std::runtime_error("tensor '" + name + "': shape [" + std::to_string(r) + ", " + std::to_string(c) + "] where [" +
                               std::to_string(rows_expected) + ", " + std::to_string(cols) + "] is expected");
    if (dtype == THA_DT_BF16) file.read_bf16(name, &h); else file.read_f32(name, &f);
    if (order) {   // row i of the stack is row (*order)[i] of the tensor
      const size_t n = (size_t)r * cols;
      if (dtype == THA_DT_BF16) {
        std::vector<uint16_t> src(h.end() - n, h.end());
        for (long long i = 0; i < r; i++) memcpy(h.data() + h.size() - n + (size_t)i * cols, src.data() + (size_t)(*order)[i] * cols, (size_t)cols * 2);
      } else {
        std::vector<float> src(f.end() - n, f.end());
        for (long long i = 0; i < r; i++) memcpy(f.data() + f.size() - n + (size_t)i * cols, src.data() + (size_t)(*order)[i] * cols, (size_t)cols * 4);
      }
    }
    const int at = rows;
    rows += (int)r;
    return at;
  }
  const void* data() const { return dtype == THA_DT_BF16 ? (const void*)h.data() : (const void*)f.data(); }
  size_t bytes() const { return dtype == THA_DT_BF16 ? h.size() * 2 : f.size() * 4; }
};
}  // namespace

LayerModel* LayerModel::load(const std::string& folder, int dtype, std::string* err) {
  JsonValue config;
  const ArchitectureEntry* e = detect_model(folder, &config, err);
  if (!e) return nullptr;
  if (e->family != ModelFamily::LayerProgram || !e->translate) { if (err) *err = "'" + e->name + "' is not a layer-program architecture"; return nullptr; }
  LayerProgramSpec spec;
  try {
    e->translate(config, &spec);
  } catch (const std::exception& ex) {
    if (err) *err = ex.what();
    return nullptr;
  }
  SafeTensors file;
  if (!file.open(folder + "/model.safetensors", err)) return nullptr;
  return build(spec, file, dtype, err);
}

LayerModel* LayerModel::build(const LayerProgramSpec& spec, const SafeTensors& file, int dtype, std::string* err) {
  LayerModel* m = new LayerModel();
  try {
    m->spec_ = spec;
    const int W = spec.width;
    auto vec = [&](const std::string& name, size_t n) -> const float* {
      std::vector<float> v;
      file.read_f32(name, &v);
      if (v.size() != n) throw std::runtime_error("tensor '" + name + "': " + std::to_string(v.size()) + " values where " + std::to_string(n) + " are expected");
      return (const float*)m->upload(v.data(), v.size() * 4);
    };
    auto mat = [&](const std::string& name, long long rows, int cols) -> const void* {
      Stack s(file, dtype, cols);
      s.add(name, rows);
      return m->upload(s.data(), s.bytes());
    };
    // a norm over the width by name: the weight, and for the dynamic tanh its bias and scalar beside it
    auto norm = [&](const std::string& name) -> tha_norm_t {
      tha_norm_t n = {};
      n.kind = spec.norm_kind;
      n.w = vec(name, W);
      n.w_offset = spec.norm_w_offset;
      if (spec.norm_kind == THA_NORM_LAYER) {
        n.w_offset = 0.0f;
        n.b = vec(name + ".b", W);
      } else if (spec.norm_kind == THA_NORM_DYT) {
        n.w_offset = 0.0f;
        n.b = vec(name + ".b", W);
        std::vector<float> a;
        file.read_f32(name + ".alpha", &a);
        if (a.size() != 1) throw std::runtime_error("tensor '" + name + ".alpha' must be one number");
        n.alpha = a[0];
      }
      return n;
    };
    // the rotary table of a setting (shared between layers with the same one): inverse frequencies in float64,
    // base^(-2i/dims), interpolated between the original and the stretched scale
    auto rotary = [&](const RotarySpec& rs) -> int {
      size_t r = 0;
      while (r < m->rot_specs_.size() && !(m->rot_specs_[r] == rs)) r++;
      if (r == m->rot_specs_.size()) {
        const int dims = rs.dims, half = dims / 2;
        std::vector<double> f(half);
        for (int i = 0; i < half; i++) f[i] = pow(rs.base, -2.0 * i / dims);
        float mag = 1.0f;
        if (rs.yarn) {
          auto where = [&](double turns) { return dims * log(rs.original / (2.0 * M_PI * turns)) / (2.0 * log(rs.base)); };
          const double lo = fmax(floor(where(rs.fast)), 0.0), hi = fmin(ceil(where(rs.slow)), dims - 1.0);
          for (int i = 0; i < half; i++) {
            const double ramp = fmin(fmax((i - lo) / fmax(hi - lo, 0.001), 0.0), 1.0);
            f[i] = f[i] / rs.factor * ramp + f[i] * (1.0 - ramp);
          }
          mag = (float)(0.1 * log(rs.factor) + 1.0);
        }
        if (rs.by_wavelength) {
          if (!(rs.high > rs.low) || !(rs.factor > 0.0) || !(rs.original > 0.0)) throw std::runtime_error("rotary scaling: needs high > low, factor > 0, original > 0");
          for (int i = 0; i < half; i++) {
            const double l = 2.0 * M_PI / f[i];
            if (l < rs.original / rs.high) continue;
            if (l > rs.original / rs.low) { f[i] = f[i] / rs.factor; continue; }
            const double t = (rs.original / l - rs.low) / (rs.high - rs.low);
            f[i] = (1.0 - t) * f[i] / rs.factor + t * f[i];
          }
        }
        tha_rotary_t R;
        R.inv_freq = (const double*)m->upload(f.data(), f.size() * 8);
        R.dims = dims;
        R.mag = mag;
        m->rot_.push_back(R);
        m->rot_specs_.push_back(rs);
      }
      return (int)r;
    };
    long long state = 0;
    size_t li_now = 0;
    m->layers_.resize(spec.layers.size());
    // softmax attention (alone, or as one side of a two-sided mixer): its matrices into the stack, its options
    auto attention = [&](const AttnSpec& a, Stack& in, tha_attn_t& A) {
      if (a.heads < 1 || a.kv_heads < 1 || a.heads % a.kv_heads) throw std::runtime_error("attention: heads must be a multiple of kv_heads");
      if (a.dim < 1 || a.vdim < 1) throw std::runtime_error("attention: dim and vdim must be positive");
      if (a.window < 0 || a.keep_first < 0) throw std::runtime_error("attention: the window and the kept first tokens cannot be negative");
      A.heads = a.heads; A.kv_heads = a.kv_heads; A.dim = a.dim; A.vdim = a.vdim;
      A.unit_rms = a.unit_rms; A.eps = spec.eps; A.scale = a.scale; A.chunk = a.chunk;
      A.window = a.window; A.keep_first = a.window > 0 ? a.keep_first : 0;
      A.fp32_scores = a.fp32_scores;
      A.rot = -1;
      if (a.rotary && a.rot.dims > 0) {
        if (a.rot.dims > a.dim || (a.rot.dims & 1)) throw std::runtime_error("attention: rotated dimensions must be even and at most dim");
        A.rot = rotary(a.rot);
        A.rot_layout = a.rot.halves ? THA_ROT_HALVES : THA_ROT_INTERLEAVED;
      }
      const int maps = a.diff ? 2 : 1;   // score maps per head: a differential head owns two query rows and two key rows
      A.heads = a.heads * maps; A.kv_heads = a.kv_heads * maps;
      const long long cq = (long long)A.heads * a.dim, ck = (long long)A.kv_heads * a.dim, cv = (long long)a.kv_heads * a.vdim;
      m->separate_values_ = true;
      if (a.kv_from >= 0) {
        // the rows of an earlier layer: same head counts and rotation, nothing of its own in the cache
        if ((size_t)a.kv_from >= li_now || spec.layers[a.kv_from].same_weights_as >= 0) throw std::runtime_error("attention: 'kv_from' must name an earlier layer");
        const LayerSpec& d = spec.layers[a.kv_from];
        if ((d.mixer != THA_MIX_ATTN) || d.attn.kv_from >= 0 || d.attn.kv_heads != a.kv_heads || d.attn.dim != a.dim || d.attn.vdim != a.vdim ||
            d.attn.diff != a.diff)
          throw std::runtime_error("attention: the layer named by 'kv_from' does not hold rows of this layer's shape");
        A.kv_shared = 1;
        A.cache_layer = m->layers_[a.kv_from].attn.cache_layer;
      } else {
        A.cache_layer = m->n_cache_layers_++;
        m->kv_dim_ = std::max(m->kv_dim_, (int)std::max(ck, cv));
      }
      if (a.diff) {
        // the q rows, stored head by head as [first map | second map], reordered per key/value group as [first maps of the
        // group's heads | second maps]: query map j then reads key head j / (heads / kv_heads), as grouped attention does
        const int gs = a.heads / a.kv_heads;
        std::vector<int> order((size_t)cq);
        for (int h = 0; h < a.heads; h++)
          for (int mp = 0; mp < 2; mp++)
            for (int d = 0; d < a.dim; d++)
              order[(size_t)(((h / gs) * 2 + mp) * gs + h % gs) * a.dim + d] = (h * 2 + mp) * a.dim + d;
        A.o_q = in.add(a.q, cq, &order);
        A.diff = 1; A.v_share = 2; A.out_f32 = 1;
        double d1 = 0.0, d2 = 0.0;
        std::vector<float> l1, k1, l2, k2;
        file.read_f32(a.lq1, &l1); file.read_f32(a.lk1, &k1); file.read_f32(a.lq2, &l2); file.read_f32(a.lk2, &k2);
        if ((int)l1.size() != a.dim || (int)k1.size() != a.dim || (int)l2.size() != a.dim || (int)k2.size() != a.dim)
          throw std::runtime_error("differential attention: the four lambda vectors must have `dim` entries");
        for (int d = 0; d < a.dim; d++) { d1 += (double)l1[d] * k1[d]; d2 += (double)l2[d] * k2[d]; }
        A.diff_lambda = (float)(exp(d1) - exp(d2) + (double)a.diff_init);
        A.diff_mult = 1.0f - a.diff_init;
      } else {
        A.o_q = in.add(a.q, cq);
      }
      if (a.kv_from < 0) {
        A.o_k = in.add(a.k, ck);
        A.o_v = in.add(a.v, cv);
      }
      A.q_temp_coef = a.q_temp_coef; A.q_temp_every = a.q_temp_every > 0 ? a.q_temp_every : 0;
      if (a.conv_taps > 0) {
        if (a.diff) throw std::runtime_error("attention: a short convolution behind differential projections is not served");
        std::vector<float> taps;
        file.read_f32(a.q + ".conv", &taps);
        if (a.kv_from < 0) { file.read_f32(a.k + ".conv", &taps); file.read_f32(a.v + ".conv", &taps); }
        const long long C = cq + (a.kv_from < 0 ? ck + cv : 0);
        if ((long long)taps.size() != C * a.conv_taps) throw std::runtime_error("attention: convolution taps do not fit [channels, " + std::to_string(a.conv_taps) + "]");
        A.conv_taps = a.conv_taps;
        A.conv_w = (const float*)m->upload(taps.data(), taps.size() * 4);
        A.conv_state_off = state;
        state += C * (a.conv_taps - 1);
      }
      if (!a.g.empty()) { A.head_gate = 1; A.o_g = in.add(a.g, a.heads); }
      if (!a.sink.empty()) A.sink = vec(a.sink, a.heads);
      else if (a.sink_zero) { std::vector<float> z(a.heads, 0.f); A.sink = (const float*)m->upload(z.data(), z.size() * 4); }
      if (!a.temp.empty()) A.head_scale = vec(a.temp, a.heads);
      if (a.diff && (A.sink || A.head_scale)) throw std::runtime_error("differential attention: sinks and per-head factors are not served");
      A.w_o = mat(a.o, W, a.heads * a.vdim);
    };
    // row `row` of a [rows, width] tensor as an fp32 device vector (uploaded once per tensor)
    std::map<std::string, const float*> pre_tables;
    auto pre_vector = [&](const std::string& name, int row) -> const float* {
      const TensorInfo& t = file.info(name);
      if (t.shape.size() != 2 || t.shape[1] != W || row < 0 || row >= t.shape[0])
        throw std::runtime_error("tensor '" + name + "': row " + std::to_string(row) + " of [rows, width] is asked for");
      auto it = pre_tables.find(name);
      if (it == pre_tables.end()) {
        std::vector<float> v;
        file.read_f32(name, &v);
        it = pre_tables.emplace(name, (const float*)m->upload(v.data(), v.size() * 4)).first;
      }
      return it->second + (size_t)row * W;
    };
    for (size_t li = 0; li < spec.layers.size(); li++) {
      li_now = li;
      const LayerSpec& ls = spec.layers[li];
      tha_hyb_layer_t& L = m->layers_[li];
      if (ls.same_weights_as >= 0) {
        // another run of an earlier entry: the same device weights, a cache layer and state of its own
        if ((size_t)ls.same_weights_as >= li) throw std::runtime_error("a repeated layer must follow the layer it repeats");
        L = m->layers_[ls.same_weights_as];
        L.pre_add_embed = ls.pre_add_embed ? 1 : 0;
        L.pre_vec = nullptr;
        if (!ls.pre_vec.empty()) L.pre_vec = pre_vector(ls.pre_vec, ls.pre_vec_row);
        if (L.in_conv_taps > 1) { L.in_conv_state_off = state; state += (long long)W * (L.in_conv_taps - 1); }
        if (L.mixer == THA_MIX_HGRN) {
          L.hgrn.state_off = state;
          state += (long long)L.hgrn.heads * L.hgrn.dim * ((L.hgrn.vdim + 7) / 8 * 8);
        }
        if ((L.mixer == THA_MIX_ATTN || L.mixer == THA_MIX_ATTN_GDELTA) && (L.attn.kv_shared || L.attn.conv_taps > 0))
          throw std::runtime_error("a repeated attention layer with a short convolution or another layer's cache rows is not served");
        if (L.mixer == THA_MIX_ATTN || L.mixer == THA_MIX_ATTN_GDELTA) {
          L.attn.cache_layer = m->n_cache_layers_++;
          if (L.mixer == THA_MIX_ATTN_GDELTA) {
            L.gdelta.state_off = state;
            state += tha_hyb_gdelta_state_floats(L.gdelta.heads, L.gdelta.dim);
          }
        } else if (L.mixer == THA_MIX_PARALLEL) {
          L.attn.cache_layer = m->n_cache_layers_++;
          L.mem.state_off = state;
          state += (long long)L.mem.heads * ((long long)L.mem.dim * L.mem.vdim + L.mem.dim + 1);
        } else if (L.mixer == THA_MIX_DELTA) {
          L.delta.state_off = state;
          state += (long long)L.delta.heads * L.delta.dim * L.delta.vdim;
          L.delta.conv_state_off = state;
          state += (2ll * L.delta.kv_heads * L.delta.dim + (long long)L.delta.heads * L.delta.vdim) * (L.delta.taps - 1);
        } else if (L.mixer == THA_MIX_GLA) {
          L.gla.state_off = state;
          state += (long long)L.gla.heads * L.gla.dim * ((L.gla.vdim + 7) / 8 * 8);   // value columns padded to eights
        } else if (L.mixer == THA_MIX_LATENT) {
          L.latent.cache_layer = m->n_cache_layers_++;
        }
        continue;
      }
      memset(&L, 0, sizeof(L));
      L.mixer = ls.mixer;
      L.block = ls.block;
      L.res_mult = ls.res_mult;
      L.pre_add_embed = ls.pre_add_embed ? 1 : 0;
      if (!ls.pre_vec.empty()) L.pre_vec = pre_vector(ls.pre_vec, ls.pre_vec_row);
      if (ls.block == THA_BLOCK_SEQUENTIAL && ls.has_ff && (ls.ff_kind != THA_FF_DENSE || ls.norm2.empty()))
        throw std::runtime_error("a sequential block serves a dense feed-forward behind a second norm, or none");
      L.norm1 = norm(ls.norm1);
      if (ls.block == THA_BLOCK_STREAMS) {
        const int n = spec.n_streams;
        if (n < 1 || n > 16) throw std::runtime_error("residual streams: 1 to 16 streams are served");
        if (spec.norm_kind != THA_NORM_RMS) throw std::runtime_error("residual streams are served with rms norms");
        if (ls.has_ff && ls.norm2.empty()) throw std::runtime_error("residual streams: the feed-forward needs a norm of its own");
        auto weights = [&](const StreamsSpec& w, tha_streams_t* out) {
          out->in = vec(w.in, n); out->out = vec(w.out, n); out->mix = vec(w.mix, (size_t)n * n);
        };
        weights(ls.streams1, &L.streams1);
        if (ls.has_ff) weights(ls.streams2, &L.streams2);
      }
      if (!ls.in_conv.empty()) {
        if (ls.block != THA_BLOCK_STREAMS) throw std::runtime_error("a convolution of the mixer's input is served in stream blocks");
        if (ls.in_conv_taps < 1) throw std::runtime_error("the input convolution needs at least one tap");
        L.in_conv_taps = ls.in_conv_taps;
        L.in_conv_w = vec(ls.in_conv, (size_t)W * ls.in_conv_taps);
        L.in_conv_state_off = state;
        state += (long long)W * (ls.in_conv_taps - 1);
      }
      if (!ls.scale_mix.empty()) L.scale_mix = vec(ls.scale_mix, W);
      if (!ls.scale_ff.empty() && ls.has_ff) L.scale_ff = vec(ls.scale_ff, W);
      Stack in(file, dtype, W);
      Stack in2(file, dtype, W);                       // what reads the second norm
      const bool two = !ls.norm2.empty() && ls.has_ff;
      Stack& fin = two ? in2 : in;                     // where the feed-forward's input matrices go
      if (ls.mixer == THA_MIX_ATTN || ls.mixer == THA_MIX_ATTN_GDELTA) {
        attention(ls.attn, in, L.attn);
        if (ls.mixer == THA_MIX_ATTN_GDELTA) {
          const GDeltaSpec& g = ls.gdelta;
          if (g.heads < 1 || g.dim < 1) throw std::runtime_error("generalized delta rule: heads and dim must be positive");
          if (g.dim > 256) throw std::runtime_error("generalized delta rule: more than 256 key channels per head are not served");
          tha_gdelta_t& G = L.gdelta;
          G.heads = g.heads; G.dim = g.dim; G.eps = spec.eps;
          const TensorInfo& w1 = file.info(g.w1);
          if (w1.shape.size() != 2) throw std::runtime_error("generalized delta rule: the decay projection must be a matrix");
          G.rank = (int)w1.shape[0];
          const long long hd = (long long)g.heads * g.dim;
          G.o_r = in.add(g.r, hd);
          G.o_k = in.add(g.k, hd);
          G.o_v = in.add(g.v, hd);
          G.o_g = in.add(g.g, hd);
          G.o_a = in.add(g.a, hd);
          G.o_w1 = in.add(g.w1, G.rank);
          G.w_w2 = mat(g.w2, hd, G.rank);
          G.w0 = vec(g.w0, (size_t)hd);
          G.a_b = vec(g.a_b, (size_t)hd);
          G.norm = vec(g.norm, (size_t)hd);
          G.w_o = mat(g.o, W, (int)hd);
          G.state_off = state;
          state += tha_hyb_gdelta_state_floats(g.heads, g.dim);
          L.mix_left = ls.mix_left; L.mix_right = ls.mix_right;
        }
      } else if (ls.mixer == THA_MIX_PARALLEL) {
        attention(ls.attn, in, L.attn);
        const MemSpec& r = ls.mem;
        tha_mem_t& M = L.mem;
        M.heads = r.heads; M.dim = r.dim; M.vdim = r.vdim; M.gate_cap = r.gate_cap; M.eps = spec.eps;
        M.o_q = in.add(r.q, (long long)r.heads * r.dim);
        M.o_k = in.add(r.k, (long long)r.heads * r.dim);
        M.o_v = in.add(r.v, (long long)r.heads * r.vdim);
        M.o_g = in.add(r.g, (long long)r.heads * r.vdim);
        M.o_i = in.add(r.i, r.heads);
        M.o_f = in.add(r.f, r.heads);
        M.b_i = vec(r.i_b, r.heads);
        M.b_f = vec(r.f_b, r.heads);
        M.norm = vec(r.norm, (size_t)r.heads * r.vdim);
        M.w_o = mat(r.o, W, r.heads * r.vdim);
        M.state_off = state;
        state += (long long)r.heads * ((long long)r.dim * r.vdim + r.dim + 1);
        L.left_out = vec(ls.left_out, W);
        L.right_out = vec(ls.right_out, W);
      } else if (ls.mixer == THA_MIX_DELTA) {
        const DeltaSpec& d = ls.delta;
        if (d.heads < 1 || d.kv_heads < 1 || d.heads % d.kv_heads || d.taps < 1) throw std::runtime_error("delta rule: heads must be a multiple of kv_heads, taps >= 1");
        tha_delta_t& D = L.delta;
        D.heads = d.heads; D.kv_heads = d.kv_heads; D.dim = d.dim; D.vdim = d.vdim; D.taps = d.taps; D.eps = spec.eps;
        const TensorInfo& a1 = file.info(d.a1);
        const TensorInfo& g1 = file.info(d.g1);
        if (a1.shape.size() != 2 || g1.shape.size() != 2) throw std::runtime_error("delta rule: the low-rank projections must be matrices");
        D.rank_a = (int)a1.shape[0];
        D.rank_g = (int)g1.shape[0];
        const long long cq = (long long)d.kv_heads * d.dim, cv = (long long)d.heads * d.vdim;
        D.o_q = in.add(d.q, cq);
        in.add(d.k, cq);
        in.add(d.v, cv);
        D.o_b = in.add(d.b, d.heads);
        D.o_a1 = in.add(d.a1, D.rank_a);
        D.o_g1 = in.add(d.g1, D.rank_g);
        std::vector<float> taps;
        file.read_f32(d.q_conv, &taps);
        file.read_f32(d.k_conv, &taps);
        file.read_f32(d.v_conv, &taps);
        if ((long long)taps.size() != (2 * cq + cv) * d.taps) throw std::runtime_error("delta rule: convolution taps do not fit [channels, " + std::to_string(d.taps) + "]");
        D.conv = (const float*)m->upload(taps.data(), taps.size() * 4);
        D.w_a2 = mat(d.a2, (long long)d.heads * d.dim, D.rank_a);
        D.w_g2 = mat(d.g2, cv, D.rank_g);
        D.a_log = vec(d.a_log, d.heads);
        D.dt_bias = vec(d.dt_bias, (size_t)d.heads * d.dim);
        D.norm = vec(d.norm, d.vdim);
        D.w_o = mat(d.o, W, (int)cv);
        D.state_off = state;
        state += (long long)d.heads * d.dim * d.vdim;
        D.conv_state_off = state;
        state += (2 * cq + cv) * (d.taps - 1);
      } else if (ls.mixer == THA_MIX_GLA) {
        const GlaSpec& g = ls.gla;
        if (g.heads < 1 || g.dim < 1 || g.vdim < 1 || !(g.tau > 0.f)) throw std::runtime_error("gated linear attention: heads, dim, vdim and tau must be positive");
        if (g.dim > 512) throw std::runtime_error("gated linear attention: more than 512 key channels per head are not served");
        tha_gla_t& G = L.gla;
        G.heads = g.heads; G.dim = g.dim; G.vdim = g.vdim; G.tau = g.tau; G.eps = spec.eps;
        const TensorInfo& a1 = file.info(g.a1);
        if (a1.shape.size() != 2) throw std::runtime_error("gated linear attention: the decay projection must be a matrix");
        G.rank = (int)a1.shape[0];
        G.o_q = in.add(g.q, (long long)g.heads * g.dim);
        G.o_k = in.add(g.k, (long long)g.heads * g.dim);
        G.o_v = in.add(g.v, (long long)g.heads * g.vdim);
        G.o_g = in.add(g.g, (long long)g.heads * g.vdim);
        G.o_a1 = in.add(g.a1, G.rank);
        G.w_a2 = mat(g.a2, (long long)g.heads * g.dim, G.rank);
        G.b_a2 = vec(g.a2_b, (size_t)g.heads * g.dim);
        G.norm = vec(g.norm, g.vdim);
        G.w_o = mat(g.o, W, g.heads * g.vdim);
        G.state_off = state;
        state += (long long)g.heads * g.dim * ((g.vdim + 7) / 8 * 8);   // value columns padded to eights
      } else if (ls.mixer == THA_MIX_HGRN) {
        const HgrnSpec& g = ls.hgrn;
        if (g.heads < 1 || g.dim < 1 || g.vdim < 1) throw std::runtime_error("gated linear recurrence: heads, dim and vdim must be positive");
        if (g.dim > 512) throw std::runtime_error("gated linear recurrence: more than 512 key channels per head are not served");
        tha_hgrn_t& G = L.hgrn;
        G.heads = g.heads; G.dim = g.dim; G.vdim = g.vdim; G.eps = spec.eps;
        G.o_q = in.add(g.q, (long long)g.heads * g.dim);
        G.o_f = in.add(g.f, (long long)g.heads * g.dim);
        G.o_v = in.add(g.v, (long long)g.heads * g.vdim);
        G.f_b = vec(g.f_b, (size_t)g.heads * g.dim);
        G.lower = vec(g.lower, (size_t)g.heads * g.dim);
        G.norm = vec(g.norm, g.vdim);
        G.w_o = mat(g.o, W, g.heads * g.vdim);
        G.state_off = state;
        state += (long long)g.heads * g.dim * ((g.vdim + 7) / 8 * 8);   // value columns padded to eights, as for gated linear attention
      } else if (ls.mixer == THA_MIX_LATENT) {
        const LatentSpec& a = ls.latent;
        const bool direct_q = !a.q.empty();
        if (a.heads < 1 || a.dim < 1 || a.vdim < 1 || (!direct_q && a.q_rank < 1) || a.kv_rank < 1 || a.rot_dim < 0 || a.window < 0)
          throw std::runtime_error("latent attention: heads, dim, vdim, q_rank and kv_rank must be positive");
        tha_latent_t& A = L.latent;
        A.heads = a.heads; A.dim = a.dim; A.rot_dim = a.rot_dim; A.vdim = a.vdim; A.q_rank = a.q_rank; A.kv_rank = a.kv_rank;
        A.eps = spec.eps; A.scale = a.scale;
        A.rot = -1;
        if (a.rotary && a.rot.dims > 0 && a.rot_dim > 0) {
          if (a.rot.dims > a.rot_dim || (a.rot.dims & 1)) throw std::runtime_error("latent attention: rotated dimensions must be even and at most rot_dim");
          A.rot = rotary(a.rot);
          A.rot_layout = a.rot.halves ? THA_ROT_HALVES : THA_ROT_INTERLEAVED;
        }
        A.cache_layer = m->n_cache_layers_++;
        m->kv_dim_ = std::max(m->kv_dim_, a.kv_rank + a.rot_dim);
        A.window = a.window;
        A.fp32_scores = a.fp32_scores;
        if (!a.sink.empty()) A.sink = vec(a.sink, a.heads);
        if (direct_q) {
          A.direct_q = 1;
          A.q_rank = 0;
          A.o_q = in.add(a.q, (long long)a.heads * (a.dim + a.rot_dim));
        } else {
          A.o_dq = in.add(a.dq, a.q_rank);
        }
        A.o_dkv = in.add(a.dkv, (long long)a.kv_rank + a.rot_dim);
        if (a.g.empty()) A.no_gate = 1;
        else A.o_g = in.add(a.g, (long long)a.heads * a.vdim);
        if (!direct_q) {
          A.q_norm = vec(a.dq_norm, a.q_rank);
          A.w_uq = mat(a.uq, (long long)a.heads * (a.dim + a.rot_dim), a.q_rank);
        }
        A.kv_norm = vec(a.dkv_norm, a.kv_rank);
        {
          // W_uk [heads * dim, kv_rank] -> per head its transpose [kv_rank, dim]: the matrix that carries a head's plain
          // query part into the latent space
          const TensorInfo& t = file.info(a.uk);
          if (t.shape.size() != 2 || t.shape[0] != (long long)a.heads * a.dim || t.shape[1] != a.kv_rank)
            throw std::runtime_error("tensor '" + a.uk + "': shape does not fit [heads * dim, kv_rank]");
          const size_t n = (size_t)a.heads * a.dim * a.kv_rank;
          if (dtype == THA_DT_BF16) {
            std::vector<uint16_t> src, dst(n);
            file.read_bf16(a.uk, &src);
            for (int h = 0; h < a.heads; h++)
              for (int d = 0; d < a.dim; d++)
                for (int c = 0; c < a.kv_rank; c++) dst[((size_t)h * a.kv_rank + c) * a.dim + d] = src[((size_t)h * a.dim + d) * a.kv_rank + c];
            A.w_uk_t = m->upload(dst.data(), n * 2);
          } else {
            std::vector<float> src, dst(n);
            file.read_f32(a.uk, &src);
            for (int h = 0; h < a.heads; h++)
              for (int d = 0; d < a.dim; d++)
                for (int c = 0; c < a.kv_rank; c++) dst[((size_t)h * a.kv_rank + c) * a.dim + d] = src[((size_t)h * a.dim + d) * a.kv_rank + c];
            A.w_uk_t = m->upload(dst.data(), n * 4);
          }
        }
        A.w_uv = mat(a.uv, (long long)a.heads * a.vdim, a.kv_rank);
        A.w_o = mat(a.o, W, a.heads * a.vdim);
      } else {
        throw std::runtime_error("unknown mixer kind");
      }
      L.has_ff = ls.has_ff ? ls.ff_kind : THA_FF_NONE;
      if (two) { L.has_norm2 = 1; L.norm2 = norm(ls.norm2); }
      if (ls.has_ff && ls.ff_kind == THA_FF_DENSE) {
        const DenseSpec& d = ls.dense;
        if (d.ff < 1) throw std::runtime_error("dense feed-forward: ff must be positive");
        L.dense.ff = d.ff;
        L.dense.act = d.act;
        if (d.act != THA_ACT_RELU2 && d.act != THA_ACT_XIELU && d.act != THA_ACT_POLYNORM) L.dense.o_gate = fin.add(d.gate, d.ff);
        L.dense.o_up = fin.add(d.up, d.ff);
        L.dense.w_down = mat(d.down, W, d.ff);
        if ((!d.up_b.empty() || !d.down_b.empty() || d.act == THA_ACT_POLYNORM) && ls.block != THA_BLOCK_STREAMS)
          throw std::runtime_error("dense feed-forward: biases and the PolyNorm activation are served in stream blocks");
        if (!d.up_b.empty()) L.dense.b_up = vec(d.up_b, d.ff);
        if (!d.down_b.empty()) L.dense.b_down = vec(d.down_b, W);
        if (d.act == THA_ACT_POLYNORM) {
          std::vector<float> c;
          file.read_f32(d.act_params, &c);
          if (c.size() != 4) throw std::runtime_error("tensor '" + d.act_params + "' must hold four numbers");
          for (int i = 0; i < 4; i++) L.dense.act_c[i] = c[i];
        }
        if (d.act == THA_ACT_XIELU) {
          std::vector<float> pq;
          file.read_f32(d.act_params, &pq);
          if (pq.size() != 2) throw std::runtime_error("tensor '" + d.act_params + "' must hold two numbers");
          L.dense.act_p = pq[0]; L.dense.act_q = pq[1];
        }
      } else if (ls.has_ff) {
        const MoeSpec& e = ls.moe;
        if (e.top < 1 || e.top > e.experts || e.top > 32) throw std::runtime_error("mixture of experts: 1 <= top <= min(experts, 32)");
        tha_moe_t& E = L.moe;
        E.experts = e.experts; E.top = e.top; E.ff = e.ff; E.limit = e.limit; E.alpha = e.alpha;
        E.act = e.act; E.route = e.route;
        if (e.route == THA_ROUTE_SOFTMAX_GROUPS) {
          const int groups = e.groups > 1 ? e.groups : 1, keep = e.groups > 1 ? e.keep_groups : 1;
          if (e.experts % groups || keep < 1 || keep > groups || e.experts > 4096)
            throw std::runtime_error("mixture of experts: groups must divide the experts (at most 4096 experts), 1 <= keep <= groups");
          if ((long long)keep * (e.experts / groups) < e.top) throw std::runtime_error("mixture of experts: the kept groups hold fewer experts than 'top'");
          E.groups = groups; E.keep_groups = keep;
          if (!e.correction.empty() && file.has(e.correction)) E.correction = vec(e.correction, e.experts);
        }
        const bool gated = e.act != THA_ACT_RELU2;
        E.o_router = fin.add(e.router, e.experts);
        Stack gu(file, dtype, W), dn(file, dtype, e.ff);
        for (int x = 0; x < e.experts; x++) {
          const std::string p = e.prefix + "e" + std::to_string(x) + ".";
          if (gated) gu.add(p + "gate", e.ff);
          gu.add(p + "up", e.ff);
          dn.add(p + "down", W);
        }
        E.w_gate_up = m->upload(gu.data(), gu.bytes());
        E.w_down = m->upload(dn.data(), dn.bytes());
        E.shared_ff = e.shared_ff;
        E.shared_limit = e.shared_limit;
        if (e.shared_ff > 0) {
          if (gated) E.o_sgate = fin.add(e.s_gate, e.shared_ff);
          E.o_sup = fin.add(e.s_up, e.shared_ff);
          E.w_sdown = mat(e.s_down, W, e.shared_ff);
          if (!e.s_scale.empty()) { E.shared_scaled = 1; E.o_sscale = fin.add(e.s_scale, 1); }
        }
      }
      if (ls.side.dim > 0) {
        if (spec.side_table.empty() || ls.side.col0 < 0 || ls.side.col0 + ls.side.dim > spec.side_cols)
          throw std::runtime_error("a layer's side input does not fit the side table");
        L.side.dim = ls.side.dim; L.side.col0 = ls.side.col0;
        L.side.w_gate = mat(ls.side.gate, ls.side.dim, W);
        L.side.w_proj = mat(ls.side.proj, W, ls.side.dim);
        L.side.norm = vec(ls.side.norm, W);
      }
      L.n_in = in.rows;
      L.w_in = m->upload(in.data(), in.bytes());
      if (two) {
        L.n_in2 = in2.rows;
        L.w_in2 = m->upload(in2.data(), in2.bytes());
      }
    }
    m->state_floats_ = state > 0 ? state : 1;
    if (m->rot_.size() > 64) throw std::runtime_error("more than 64 distinct rotary tables");
    tha_hyb_model_t& M = m->model_;
    M.dtype = dtype;
    M.width = W;
    M.vocab = spec.vocab;
    M.n_layers = (int)m->layers_.size();
    M.eps = spec.eps;
    M.logit_softcap = spec.logit_softcap;
    M.embed = mat(spec.embed, spec.vocab, W);
    M.embed_scale = spec.embed_scale;
    M.n_streams = spec.n_streams;
    if (!spec.side_table.empty()) {
      if (spec.side_cols < 1) throw std::runtime_error("a side table needs its number of columns");
      M.side_table = mat(spec.side_table, spec.vocab, spec.side_cols);
      M.side_cols = spec.side_cols;
    }
    if (!spec.pos_embed.empty()) {
      if (spec.max_positions < 1) throw std::runtime_error("a position table needs max_positions");
      M.pos_embed = mat(spec.pos_embed, spec.max_positions, W);
      M.max_positions = spec.max_positions;
    }
    M.final_norm = norm(spec.final_norm);
    M.head = mat(spec.head, spec.vocab, W);
    M.layers = m->layers_.data();
    M.n_rot = (int)m->rot_.size();
    M.rot = m->rot_.data();
    if (m->kv_dim_ < 1) m->kv_dim_ = 1;
    return m;
  } catch (const std::exception& ex) {
    if (err) *err = ex.what();
    delete m;
    return nullptr;
  }
}
