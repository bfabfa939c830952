// Plain, slow Phi-MoE forward pass in C++17 and float32: whole sequences, no cache, one function per part.
//
// Second oracle of the test-suite, written independently of tests/plain_phimoe.py (which computes in float64
// with torch) and of the engine: its own JSON reader, its own safetensors reader, plain loops.  The two plain
// implementations must agree on the tiny models' logits and on every expert choice; this one is also the timed
// CPU baseline of the tiny workloads.  The reference project (formetaohy/Flint) is Rust + WGSL and cannot be
// built here, and it has no mixture-of-experts feed-forward, so this file rests on formulas: the dense decoder's
// are taken from the reference files cited at each function (paths within that project), the sparsemixer
// routing, the LongRoPE magnitude scale and the sliding window follow the architecture's definition.
//
//   plain_phimoe logits   MODEL_DIR TOKENS.txt OUT.bin
//       one request per line of TOKENS.txt; OUT.bin gets, per request, its logits [T, V] as float32 and then
//       the chosen experts [layers, T, 2] as int32
//   plain_phimoe generate MODEL_DIR PROMPTS.txt N TEMPERATURE TOP_K TOP_P SEED
//       N tokens per prompt, each from a forward pass over the whole sequence so far; prints one line of
//       tokens per prompt and "seconds S tokens K"
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

// ---------------------------------------------------------------------------------------------- JSON
struct Json {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;
  const Json* get(const std::string& k) const {
    for (auto& kv : obj) if (kv.first == k) return &kv.second;
    return nullptr;
  }
  bool has(const std::string& k) const { const Json* j = get(k); return j && j->kind != Null; }
  const Json& at(const std::string& k) const {
    const Json* j = get(k);
    if (!j) throw std::runtime_error("missing key " + k);
    return *j;
  }
};

struct JsonParser {
  const std::string& s;
  size_t i = 0;
  explicit JsonParser(const std::string& text) : s(text) {}
  void ws() { while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i; }
  Json parse() {
    ws();
    Json j;
    if (i >= s.size()) throw std::runtime_error("json: unexpected end");
    char c = s[i];
    if (c == '{') {
      j.kind = Json::Obj;
      ++i; ws();
      if (s[i] == '}') { ++i; return j; }
      while (true) {
        ws();
        Json k = parse();
        ws();
        if (s[i] != ':') throw std::runtime_error("json: expected ':'");
        ++i;
        j.obj.emplace_back(k.str, parse());
        ws();
        if (s[i] == ',') { ++i; continue; }
        if (s[i] == '}') { ++i; break; }
        throw std::runtime_error("json: expected ',' or '}'");
      }
    } else if (c == '[') {
      j.kind = Json::Arr;
      ++i; ws();
      if (s[i] == ']') { ++i; return j; }
      while (true) {
        j.arr.push_back(parse());
        ws();
        if (s[i] == ',') { ++i; continue; }
        if (s[i] == ']') { ++i; break; }
        throw std::runtime_error("json: expected ',' or ']'");
      }
    } else if (c == '"') {
      j.kind = Json::Str;
      ++i;
      while (s[i] != '"') {
        if (s[i] == '\\') { ++i; j.str += s[i] == 'n' ? '\n' : s[i]; } else j.str += s[i];
        ++i;
      }
      ++i;
    } else if (!s.compare(i, 4, "true")) { j.kind = Json::Bool; j.b = true; i += 4; }
    else if (!s.compare(i, 5, "false")) { j.kind = Json::Bool; i += 5; }
    else if (!s.compare(i, 4, "null")) { i += 4; }
    else {
      size_t used = 0;
      j.kind = Json::Num;
      j.num = std::stod(s.substr(i, 64), &used);
      i += used;
    }
    return j;
  }
};

static std::string read_file(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot open " + path);
  std::stringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

// ---------------------------------------------------------------------------------------------- tensors
struct Tensor {
  std::vector<int64_t> shape;
  std::vector<float> v;
  int64_t rows() const { return shape.empty() ? 0 : shape[0]; }
  int64_t cols() const { return shape.size() > 1 ? shape[1] : 1; }
};

static float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

// safetensors: 8-byte little-endian header length, JSON header {name: {dtype, shape, data_offsets}}, raw data.
// A leading "model." is dropped from names.
static std::map<std::string, Tensor> read_safetensors(const std::string& path) {
  const std::string raw = read_file(path);
  uint64_t n = 0;
  std::memcpy(&n, raw.data(), 8);
  const std::string head = raw.substr(8, n);
  Json j = JsonParser(head).parse();
  std::map<std::string, Tensor> out;
  for (auto& kv : j.obj) {
    if (kv.first == "__metadata__") continue;
    Tensor t;
    int64_t count = 1;
    for (auto& d : kv.second.at("shape").arr) { t.shape.push_back((int64_t)d.num); count *= (int64_t)d.num; }
    const size_t lo = (size_t)kv.second.at("data_offsets").arr[0].num;
    const char* p = raw.data() + 8 + n + lo;
    const std::string dt = kv.second.at("dtype").str;
    t.v.resize(count);
    if (dt == "F32") std::memcpy(t.v.data(), p, count * 4);
    else if (dt == "BF16") for (int64_t i = 0; i < count; ++i) { uint16_t h; std::memcpy(&h, p + 2 * i, 2); t.v[i] = bf16_to_f32(h); }
    else throw std::runtime_error("unsupported dtype " + dt + " of " + kv.first);
    std::string name = kv.first;
    if (name.rfind("model.", 0) == 0) name = name.substr(6);
    out[name] = std::move(t);
  }
  return out;
}

struct Config {
  int H, L, nq, nkv, hd, E, I, V, window, max_pos, orig_max;
  float eps, jitter;
  double theta, partial, m_short = 1.0, m_long = 1.0;
  bool longrope = false, tied = false;
  std::string act;
  std::vector<double> short_f, long_f;
  std::vector<int> eos;
};

static Config read_config(const std::string& dir) {
  Json j = JsonParser(read_file(dir + "/config.json")).parse();
  Config c;
  c.H = (int)j.at("hidden_size").num; c.L = (int)j.at("num_hidden_layers").num;
  c.nq = (int)j.at("num_attention_heads").num; c.nkv = (int)j.at("num_key_value_heads").num;
  c.hd = j.has("head_dim") ? (int)j.at("head_dim").num : c.H / c.nq;
  c.E = (int)j.at("num_local_experts").num; c.I = (int)j.at("intermediate_size").num; c.V = (int)j.at("vocab_size").num;
  c.window = j.has("sliding_window") ? (int)j.at("sliding_window").num : 0;
  c.max_pos = (int)j.at("max_position_embeddings").num;
  c.eps = 1e-5f;
  for (const char* k : {"rms_norm_eps", "layer_norm_eps", "layer_norm_epsilon"}) if (j.has(k)) { c.eps = (float)j.at(k).num; break; }
  c.jitter = j.has("router_jitter_noise") ? (float)j.at("router_jitter_noise").num : j.has("jitter_eps") ? (float)j.at("jitter_eps").num : 0.01f;
  c.theta = j.at("rope_theta").num;
  c.partial = j.has("partial_rotary_factor") ? j.at("partial_rotary_factor").num : 1.0;
  c.act = j.has("hidden_act") ? j.at("hidden_act").str : "silu";
  c.tied = j.has("tie_word_embeddings") && j.at("tie_word_embeddings").b;
  c.orig_max = j.has("original_max_position_embeddings") ? (int)j.at("original_max_position_embeddings").num : 4096;
  if (j.has("rope_scaling")) {
    const Json& rs = j.at("rope_scaling");
    c.longrope = true;
    if (rs.has("original_max_position_embeddings")) c.orig_max = (int)rs.at("original_max_position_embeddings").num;
    for (auto& f : rs.at("short_factor").arr) c.short_f.push_back(f.num);
    for (auto& f : rs.at("long_factor").arr) c.long_f.push_back(f.num);
    const double def = c.max_pos > c.orig_max ? std::sqrt(1.0 + std::log((double)c.max_pos / c.orig_max) / std::log((double)c.orig_max)) : 1.0;
    c.m_short = rs.has("short_mscale") ? rs.at("short_mscale").num : def;
    c.m_long = rs.has("long_mscale") ? rs.at("long_mscale").num : def;
  }
  if (j.has("eos_token_id")) {
    const Json& e = j.at("eos_token_id");
    if (e.kind == Json::Num) c.eos.push_back((int)e.num);
    for (auto& x : e.arr) c.eos.push_back((int)x.num);
  }
  return c;
}

// ---------------------------------------------------------------------------------------------- parts
using Mat = std::vector<float>;      // row-major [rows, cols]

// h[r,:] = table[ids[r],:] (crates/thuban_kernel/wgsl/embed.wgsl:15-33; the scale is 1 for Phi:
// crates/thuban_architectures/src/transformer/config.rs:114)
static Mat embed(const std::vector<int>& ids, const Tensor& table) {
  const int64_t H = table.cols();
  Mat h(ids.size() * H);
  for (size_t r = 0; r < ids.size(); ++r) std::copy_n(table.v.begin() + ids[r] * H, H, h.begin() + r * H);
  return h;
}

// LayerNorm with bias: y = (x - mean) * rsqrt(var + eps) * gamma + beta (crates/thuban_kernel/wgsl/norm.wgsl:112-121,
// crates/thuban_backend/tests/support/cpu_ref.rs:54-85), the variance taken as mean((x - mean)^2)
static Mat layer_norm(const Mat& x, int T, int H, const Tensor& gamma, const Tensor* beta, float eps) {
  Mat y(x.size());
  for (int t = 0; t < T; ++t) {
    const float* r = &x[(size_t)t * H];
    float mu = 0;
    for (int i = 0; i < H; ++i) mu += r[i];
    mu /= H;
    float var = 0;
    for (int i = 0; i < H; ++i) var += (r[i] - mu) * (r[i] - mu);
    var /= H;
    const float inv = 1.0f / std::sqrt(var + eps);
    for (int i = 0; i < H; ++i) y[(size_t)t * H + i] = (r[i] - mu) * inv * gamma.v[i] + (beta ? beta->v[i] : 0.f);
  }
  return y;
}

// y[m,n] = sum_k x[m,k] W[n,k] (+ b[n]) (crates/thuban_backend/tests/support/cpu_ref.rs:11-23, crates/thuban_kernel/wgsl/bias.wgsl:11-16)
static Mat linear(const Mat& x, int M, const Tensor& w, const Tensor* b) {
  const int N = (int)w.rows(), K = (int)w.cols();
  Mat y((size_t)M * N);
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      const float* xr = &x[(size_t)m * K];
      const float* wr = &w.v[(size_t)n * K];
      float acc = 0;
      for (int k = 0; k < K; ++k) acc += xr[k] * wr[k];
      y[(size_t)m * N + n] = acc + (b ? b->v[n] : 0.f);
    }
  return y;
}

// cos/sin [T, rot/2]: inv_i = theta^(-2i/rot) / f_i, f the short factors below the original context and the long
// ones from there on, per position (crates/thuban_model/src/ops/rope.rs:52-87); the LongRoPE magnitude scale
// multiplies both.  Angles in double, stored as float.
static void rope_tables(const Config& c, int T, Mat& cs, Mat& sn, int& half) {
  const int rot = (int)(c.hd * c.partial);
  half = rot / 2;
  cs.assign((size_t)T * half, 0.f);
  sn.assign((size_t)T * half, 0.f);
  for (int p = 0; p < T; ++p)
    for (int i = 0; i < half; ++i) {
      double inv = std::pow(c.theta, -2.0 * i / rot), scale = 1.0;
      if (c.longrope) {
        const bool is_short = p < c.orig_max;
        inv /= is_short ? c.short_f[i] : c.long_f[i];
        scale = is_short ? c.m_short : c.m_long;
      }
      cs[(size_t)p * half + i] = (float)(std::cos(p * inv) * scale);
      sn[(size_t)p * half + i] = (float)(std::sin(p * inv) * scale);
    }
}

// NeoX half-split rotation in place on x [T, heads, hd]; dims from rot on pass through
// (crates/thuban_kernel/wgsl/rope.wgsl:25-39, crates/thuban_backend/tests/support/cpu_ref.rs:132-151)
static void rope_rotate(Mat& x, int T, int heads, int hd, const Mat& cs, const Mat& sn, int half) {
  for (int t = 0; t < T; ++t)
    for (int h = 0; h < heads; ++h) {
      float* v = &x[((size_t)t * heads + h) * hd];
      for (int d = 0; d < half; ++d) {
        const float c = cs[(size_t)t * half + d], s = sn[(size_t)t * half + d], a = v[d], b = v[d + half];
        v[d] = a * c - b * s;
        v[d + half] = b * c + a * s;
      }
    }
}

// Causal (and windowed) grouped-query attention over a whole sequence: the query at position p sees keys j <= p
// and, with a window, j >= p + 1 - window; scale 1/sqrt(hd); a full softmax per row
// (crates/thuban_kernel/wgsl/attn.wgsl:78-90,119-214, crates/thuban_backend/tests/support/cpu_ref.rs:182-227)
static Mat attention(const Mat& q, const Mat& k, const Mat& v, int T, int nq, int nkv, int hd, int window) {
  Mat out((size_t)T * nq * hd, 0.f);
  const int g = nq / nkv;
  const float scale = 1.0f / std::sqrt((float)hd);
  std::vector<float> s(T);
  for (int h = 0; h < nq; ++h) {
    const int kh = h / g;
    for (int p = 0; p < T; ++p) {
      const int lo = window > 0 ? std::max(0, p + 1 - window) : 0;
      float mx = -INFINITY;
      for (int j = lo; j <= p; ++j) {
        float acc = 0;
        for (int d = 0; d < hd; ++d) acc += q[((size_t)p * nq + h) * hd + d] * k[((size_t)j * nkv + kh) * hd + d];
        s[j] = acc * scale;
        mx = std::max(mx, s[j]);
      }
      float sum = 0;
      for (int j = lo; j <= p; ++j) { s[j] = std::exp(s[j] - mx); sum += s[j]; }
      for (int j = lo; j <= p; ++j) {
        const float w = s[j] / sum;
        for (int d = 0; d < hd; ++d) out[((size_t)p * nq + h) * hd + d] += w * v[((size_t)j * nkv + kh) * hd + d];
      }
    }
  }
  return out;
}

// Top-2 sparsemixer routing at inference for one row of router logits: the arg-max (lowest index on ties), its
// gate a softmax over the logits whose distance from the maximum, relative to max(|s_j|, max), is at most
// 2 * eps; then the same again with the first choice taken out.  The two gates are not renormalised.
static void sparsemixer_top2(const float* s, int E, float eps, int& i1, float& g1, int& i2, float& g2) {
  auto pick = [&](int excluded, int& idx, float& gate) {
    float m = -INFINITY;
    idx = -1;
    for (int e = 0; e < E; ++e) if (e != excluded && s[e] > m) { m = s[e]; idx = e; }
    float denom = 0;
    for (int e = 0; e < E; ++e) {
      if (e == excluded) continue;
      const float factor = std::max(std::fabs(s[e]), m);
      if (!(((m - s[e]) / factor) > 2.0f * eps)) denom += std::exp(s[e] - m);
    }
    gate = 1.0f / denom;
  };
  pick(-1, i1, g1);
  pick(i1, i2, g2);
}

// silu(g) = g / (1 + exp(-g)) or tanh-GELU (crates/thuban_kernel/wgsl/swiglu.wgsl:15-22,
// crates/thuban_backend/tests/support/cpu_ref.rs:102-108)
static float activation(float g, const std::string& name) {
  if (name == "silu") return g / (1.0f + std::exp(-g));
  if (name == "gelu_pytorch_tanh") return 0.5f * g * (1.0f + std::tanh(0.7978845608028654f * (g + 0.044715f * g * g * g)));
  throw std::runtime_error("unknown activation " + name);
}

// y = (act(x W1^T) * (x W3^T)) W2^T for one row (dense analogue: crates/thuban_model/src/ops/mlp.rs:24-79)
static std::vector<float> expert_mlp(const float* x, const Tensor& w1, const Tensor& w3, const Tensor& w2, const std::string& act) {
  const int I = (int)w1.rows(), H = (int)w1.cols();
  std::vector<float> a(I), y(H, 0.f);
  for (int i = 0; i < I; ++i) {
    float g = 0, u = 0;
    for (int k = 0; k < H; ++k) { g += x[k] * w1.v[(size_t)i * H + k]; u += x[k] * w3.v[(size_t)i * H + k]; }
    a[i] = activation(g, act) * u;
  }
  for (int n = 0; n < H; ++n) {
    float acc = 0;
    for (int i = 0; i < I; ++i) acc += a[i] * w2.v[(size_t)n * I + i];
    y[n] = acc;
  }
  return y;
}

struct Model {
  Config c;
  std::map<std::string, Tensor> w;
  const Tensor& t(const std::string& name) const {
    auto it = w.find(name);
    if (it == w.end()) throw std::runtime_error("missing tensor " + name);
    return it->second;
  }
  const Tensor* opt(const std::string& name) const {
    auto it = w.find(name);
    return it == w.end() ? nullptr : &it->second;
  }
};

// x [T, H] -> sum over the two chosen experts of gate * expert(x); chosen[t] = (i1, i2)
static Mat moe_feed_forward(const Model& m, const std::string& p, const Mat& x, int T, std::vector<int>* chosen) {
  const Config& c = m.c;
  const Mat logits = linear(x, T, m.t(p + "gate.weight"), nullptr);
  Mat out((size_t)T * c.H, 0.f);
  for (int t = 0; t < T; ++t) {
    int i1, i2;
    float g1, g2;
    sparsemixer_top2(&logits[(size_t)t * c.E], c.E, c.jitter, i1, g1, i2, g2);
    if (chosen) { chosen->push_back(i1); chosen->push_back(i2); }
    auto ex = [&](int e) {
      const std::string q = p + "experts." + std::to_string(e) + ".";
      return expert_mlp(&x[(size_t)t * c.H], m.t(q + "w1.weight"), m.t(q + "w3.weight"), m.t(q + "w2.weight"), c.act);
    };
    const std::vector<float> y1 = ex(i1), y2 = ex(i2);
    for (int n = 0; n < c.H; ++n) out[(size_t)t * c.H + n] = g1 * y1[n] + g2 * y2[n];
  }
  return out;
}

// Logits [T, V] of one whole sequence, or of its last position only (order of operations as
// crates/thuban_architectures/src/transformer/forward.rs:88-468)
static Mat forward(const Model& m, const std::vector<int>& ids, std::vector<int>* chosen, bool last_only) {
  const Config& c = m.c;
  const int T = (int)ids.size();
  Mat cs, sn;
  int half;
  rope_tables(c, T, cs, sn, half);
  Mat h = embed(ids, m.t("embed_tokens.weight"));
  for (int l = 0; l < c.L; ++l) {
    const std::string p = "layers." + std::to_string(l) + ".";
    Mat x = layer_norm(h, T, c.H, m.t(p + "input_layernorm.weight"), m.opt(p + "input_layernorm.bias"), c.eps);
    Mat q = linear(x, T, m.t(p + "self_attn.q_proj.weight"), m.opt(p + "self_attn.q_proj.bias"));
    Mat k = linear(x, T, m.t(p + "self_attn.k_proj.weight"), m.opt(p + "self_attn.k_proj.bias"));
    Mat v = linear(x, T, m.t(p + "self_attn.v_proj.weight"), m.opt(p + "self_attn.v_proj.bias"));
    rope_rotate(q, T, c.nq, c.hd, cs, sn, half);
    rope_rotate(k, T, c.nkv, c.hd, cs, sn, half);
    Mat a = attention(q, k, v, T, c.nq, c.nkv, c.hd, c.window);
    Mat o = linear(a, T, m.t(p + "self_attn.o_proj.weight"), m.opt(p + "self_attn.o_proj.bias"));
    for (size_t i = 0; i < h.size(); ++i) h[i] += o[i];
    x = layer_norm(h, T, c.H, m.t(p + "post_attention_layernorm.weight"), m.opt(p + "post_attention_layernorm.bias"), c.eps);
    Mat f = moe_feed_forward(m, p + "block_sparse_moe.", x, T, chosen);
    for (size_t i = 0; i < h.size(); ++i) h[i] += f[i];
  }
  if (last_only) {
    h = Mat(h.end() - c.H, h.end());
  }
  const int R = last_only ? 1 : T;
  Mat x = layer_norm(h, R, c.H, m.t("norm.weight"), m.opt("norm.bias"), c.eps);
  return linear(x, R, c.tied ? m.t("embed_tokens.weight") : m.t("lm_head.weight"), m.opt("lm_head.bias"));
}

// ---------------------------------------------------------------------------------------------- sampling
// The reference's order (crates/thuban_generate/src/sampler.rs:56-109): greedy if the temperature is not positive
// (first maximum wins, :209-219), else softmax((s - max) / T), sort descending, top-k, top-p (smallest prefix
// with mass >= p), renormalise, inverse-CDF draw with u = (z >> 40) / 2^24 from a splitmix64 step (:135-142).
struct Sampler {
  float temperature;
  int top_k;
  float top_p;
  uint64_t rng;
  float next_f32() {
    rng += 0x9E3779B97F4A7C15ull;
    uint64_t z = rng;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(z >> 40) / (float)(1 << 24);
  }
  int sample(const float* logits, int V) {
    if (temperature <= 0) return (int)(std::max_element(logits, logits + V) - logits);
    float mx = *std::max_element(logits, logits + V), sum = 0;
    std::vector<std::pair<float, int>> pr(V);
    for (int i = 0; i < V; ++i) { pr[i] = {std::exp((logits[i] - mx) / temperature), i}; sum += pr[i].first; }
    for (auto& x : pr) x.first /= sum;
    std::stable_sort(pr.begin(), pr.end(), [](auto& a, auto& b) { return a.first > b.first; });
    if (top_k > 0 && top_k < V) pr.resize(top_k);
    if (top_p < 1.0f) {
      float tot = 0, acc = 0;
      for (auto& x : pr) tot += x.first;
      size_t cut = pr.size();
      for (size_t i = 0; i < pr.size(); ++i) { acc += pr[i].first / tot; if (acc >= top_p) { cut = i + 1; break; } }
      pr.resize(std::max<size_t>(cut, 1));
    }
    std::vector<float> full(V, 0.f);
    float tot = 0;
    for (auto& x : pr) { full[x.second] = x.first; tot += x.first; }
    const float u = next_f32();
    float acc = 0;
    for (int i = 0; i < V; ++i) { acc += full[i] / tot; if (acc >= u) return i; }
    return V - 1;
  }
};

static std::vector<std::vector<int>> read_token_lines(const std::string& path) {
  std::vector<std::vector<int>> out;
  std::ifstream f(path);
  std::string line;
  while (std::getline(f, line)) {
    std::stringstream ss(line);
    std::vector<int> row;
    int x;
    while (ss >> x) row.push_back(x);
    if (!row.empty()) out.push_back(row);
  }
  return out;
}

int main(int argc, char** argv) {
  try {
    if (argc < 4) throw std::runtime_error("usage: plain_phimoe logits|generate MODEL_DIR TOKENS.txt ...");
    const std::string mode = argv[1], dir = argv[2];
    Model m{read_config(dir), read_safetensors(dir + "/model.safetensors")};
    const auto reqs = read_token_lines(argv[3]);
    if (mode == "logits") {
      if (argc < 5) throw std::runtime_error("logits needs OUT.bin");
      std::ofstream out(argv[4], std::ios::binary);
      for (auto& ids : reqs) {
        std::vector<int> chosen;
        const Mat lg = forward(m, ids, &chosen, false);
        out.write((const char*)lg.data(), lg.size() * 4);
        // chosen is [layer][t][2] in the order the layers ran
        out.write((const char*)chosen.data(), chosen.size() * 4);
      }
      return 0;
    }
    if (mode == "generate") {
      if (argc < 9) throw std::runtime_error("generate needs N TEMPERATURE TOP_K TOP_P SEED");
      const int n = std::atoi(argv[4]);
      uint64_t seed = std::strtoull(argv[8], nullptr, 10);
      const auto t0 = std::chrono::steady_clock::now();
      long total = 0;
      for (auto ids : reqs) {
        // the engine's seed is incremented per request (crates/thuban_generate/src/engine.rs:129,142)
        Sampler s{(float)std::atof(argv[5]), std::atoi(argv[6]), (float)std::atof(argv[7]), ++seed};
        std::string line;
        for (int i = 0; i < n; ++i) {
          const Mat lg = forward(m, ids, nullptr, true);
          const int tok = s.sample(lg.data(), m.c.V);
          if (std::find(m.c.eos.begin(), m.c.eos.end(), tok) != m.c.eos.end()) break;
          ids.push_back(tok);
          line += std::to_string(tok) + " ";
          ++total;
        }
        std::printf("%s\n", line.c_str());
      }
      const double secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
      std::printf("seconds %.6f tokens %ld\n", secs, total);
      return 0;
    }
    throw std::runtime_error("unknown mode " + mode);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "plain_phimoe: %s\n", e.what());
    return 1;
  }
}
