// TEST INFRASTRUCTURE ONLY - CPU restatement of edge-infer's speculative-decoding
// verify step. It is the checker for the CUDA path; nothing in the product calls it.
// Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may load it.
//
// Parity status: PINNED. tests/test_oracle_pin.py checks (a) this file's FP32 mode
// bit-for-bit against the unmodified reference CPU executor (oracle/_ref, built from
// the reference sources) on a Qwen2-style model (q/k/v bias, no QK-norm), and
// (b) the committed golden vectors under tests/golden/ that the same reference
// produced (tests/golden/make_golden.py).
//
// Two arithmetic modes over the same weights:
//   mode 0  "fp32"    - the reference FP32 CPU executor, loop for loop:
//                       runtime/src/qwen.cpp:293-301 (linear), 304-317 (norm),
//                       319-332 (rope), 335-424 (block order, online-softmax attention).
//                       Two gaps of that executor are filled the way the reference's
//                       CUDA decoder does it: per-head QK-norm after the q/k projections
//                       and before RoPE (runtime/include/execution/decoder.hpp:122-136),
//                       and AWQ weights dequantised on the host with the scalar
//                       kernel's formula (operators/src/cuda/kernels/awq_gemv_gemm.cu:591-599).
//   mode 1  "staged"  - the rounding points of the reference CUDA BF16 path: every
//                       operator output stored as BF16; RMSNorm rounds x*inv_rms and
//                       the weighted product (operators/src/cuda/rms_norm_cuda.cu:87-95);
//                       RoPE from the host FP32 table, sin/cos, each product and the
//                       sum rounded (operators/src/cuda/execution.cu:104-117;
//                       runtime/include/models/qwen3_model.hpp:410-436); SiLU rounded
//                       before the multiply (operators/src/cuda/silu_cuda.cu:45-56);
//                       bias joins the FP32 accumulator before the single output
//                       rounding (awq_gemv_gemm.cu:318-329; execution.cu:307-323);
//                       softmax numerators rounded to BF16 for the PV product while the
//                       denominator keeps FP32 values
//                       (operators/src/cuda/kernels/flash_attn_prefill.cu:236-252).
//                       Accumulation inside a dot product is FP64 here (the reference
//                       tests do the same: operators/tests/operators_cuda_awq_test.cu:153-162,
//                       operators_cuda_attention_precision_test.cu:80-102), so this
//                       mode is the ideal value of the staged computation, compared
//                       with a tolerance; it is not a bit-level model of MMA order.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <map>
#include <memory>
#include <string>
#include <thread>
#include <vector>

namespace {

thread_local std::string g_error;

// Splits [0, count) over the host threads. Every index is computed by exactly one thread with the
// same arithmetic as a serial loop, so results do not depend on the thread count.
int g_threads = 0;
template <typename Body>
void parallel_for(long long count, Body&& body) {
  int threads = g_threads > 0 ? g_threads : int(std::thread::hardware_concurrency());
  if (threads < 1) threads = 1;
  if (threads > count) threads = int(count > 0 ? count : 1);
  if (threads == 1) {
    for (long long i = 0; i < count; ++i) body(i);
    return;
  }
  std::vector<std::thread> pool;
  pool.reserve(threads);
  for (int t = 0; t < threads; ++t)
    pool.emplace_back([&, t] {
      const long long begin = count * t / threads, end = count * (t + 1) / threads;
      for (long long i = begin; i < end; ++i) body(i);
    });
  for (auto& th : pool) th.join();
}

inline float bf16_to_float(uint16_t bits) {
  uint32_t word = uint32_t(bits) << 16;
  float value;
  std::memcpy(&value, &word, 4);
  return value;
}

// Round-to-nearest-even FP32 -> BF16 (the conversion __float2bfloat16_rn performs).
inline uint16_t float_to_bf16(float value) {
  uint32_t word;
  std::memcpy(&word, &value, 4);
  if ((word & 0x7fffffffu) > 0x7f800000u) return uint16_t((word >> 16) | 0x0040u);  // NaN
  const uint32_t lsb = (word >> 16) & 1u;
  word += 0x7fffu + lsb;
  return uint16_t(word >> 16);
}

inline float round_bf16(float value) { return bf16_to_float(float_to_bf16(value)); }

struct Linear {
  std::vector<float> weight;  // [out][in]
  std::vector<float> bias;    // [out] or empty
  size_t in = 0, out = 0;
};

struct Config {
  uint64_t vocab, layers, heads, kv_heads, hidden, head_dim, ffn, max_pos;
  float eps, theta;
  int32_t qk_norm;
};

struct Model {
  Config c{};
  std::vector<float> embedding;  // [vocab][hidden]
  std::vector<float> output_norm;
  Linear lm_head;
  struct Layer {
    std::vector<float> attention_norm, ffn_norm, q_norm, k_norm;
    Linear q, k, v, o, gate, up, down;
  };
  std::vector<Layer> layers;
  std::vector<float> rope_table;  // [max_pos][head_dim]: [2i]=sin, [2i+1]=cos
  // KV cache [layer][capacity][kv_width] and logical length.
  size_t capacity = 0, length = 0;
  std::vector<float> k_cache, v_cache;
};

// FP32 dot product in the reference's order: bias first, then index 0..n-1, one
// rounded multiply and one rounded add per term (runtime/src/qwen.cpp:296-298).
inline float dot_fp32(const float* x, const float* w, size_t n, float start) {
  float value = start;
  for (size_t i = 0; i < n; ++i) value += x[i] * w[i];
  return value;
}

inline double dot_fp64(const float* x, const float* w, size_t n, double start) {
  double value = start;
  for (size_t i = 0; i < n; ++i) value += double(x[i]) * double(w[i]);
  return value;
}

void linear(const Linear& l, const float* in, size_t rows, float* out, int mode) {
  parallel_for((long long)l.out, [&](long long column) {
    const float* w = l.weight.data() + size_t(column) * l.in;
    const float b = l.bias.empty() ? 0.0f : l.bias[column];
    for (size_t row = 0; row < rows; ++row) {
      const float* x = in + row * l.in;
      out[row * l.out + column] =
          mode == 0 ? dot_fp32(x, w, l.in, b) : round_bf16(float(dot_fp64(x, w, l.in, b)));
    }
  });
}

// mode 0: runtime/src/qwen.cpp:304-317.  mode 1: rms_norm_cuda.cu:30-95.
void rms_norm(const float* in, const float* weight, float* out, size_t rows, size_t width,
              float eps, int mode) {
  for (size_t row = 0; row < rows; ++row) {
    const float* x = in + row * width;
    float* y = out + row * width;
    if (mode == 0) {
      float sum = 0.0f;
      for (size_t i = 0; i < width; ++i) sum += x[i] * x[i];
      const float inverse = 1.0f / std::sqrt(sum / width + eps);
      for (size_t i = 0; i < width; ++i) y[i] = x[i] * inverse * weight[i];
    } else {
      double sum = 0.0;
      for (size_t i = 0; i < width; ++i) sum += double(x[i]) * double(x[i]);
      const float inverse = float(1.0 / std::sqrt(double(float(sum)) / double(width) + double(eps)));
      for (size_t i = 0; i < width; ++i) y[i] = round_bf16(round_bf16(x[i] * inverse) * weight[i]);
    }
  }
}

// Host table of the prepared model: runtime/include/models/qwen3_model.hpp:417-425.
void build_rope_table(Model& m) {
  const size_t d = m.c.head_dim;
  m.rope_table.assign(m.c.max_pos * d, 0.0f);
  for (size_t pos = 0; pos < m.c.max_pos; ++pos)
    for (size_t i = 0; i < d / 2; ++i) {
      const float frequency = 1.0f / std::pow(m.c.theta, 2.0f * float(i) / float(d));
      const float angle = float(pos) * frequency;
      m.rope_table[pos * d + 2 * i] = std::sin(angle);
      m.rope_table[pos * d + 2 * i + 1] = std::cos(angle);
    }
}

void rope(const Model& m, float* data, size_t rows, size_t heads, size_t offset, int mode) {
  const size_t d = m.c.head_dim, half = d / 2, width = heads * d;
  for (size_t row = 0; row < rows; ++row)
    for (size_t head = 0; head < heads; ++head)
      for (size_t i = 0; i < half; ++i) {
        float* first = data + row * width + head * d + i;
        float* second = first + half;
        const float x = *first, y = *second;
        if (mode == 0) {
          // runtime/src/qwen.cpp:324-330
          const float angle = float(offset + row) * std::pow(m.c.theta, -2.0f * float(i) / m.c.head_dim);
          const float sine = std::sin(angle), cosine = std::cos(angle);
          *first = x * cosine - y * sine;
          *second = y * cosine + x * sine;
        } else {
          // operators/src/cuda/execution.cu:104-117
          const float sine = round_bf16(m.rope_table[(offset + row) * d + 2 * i]);
          const float cosine = round_bf16(m.rope_table[(offset + row) * d + 2 * i + 1]);
          *first = round_bf16(round_bf16(x * cosine) - round_bf16(y * sine));
          *second = round_bf16(round_bf16(x * sine) + round_bf16(y * cosine));
        }
      }
}

// SiLU of the staged path (operators/src/cuda/silu_cuda.cu:11-32); the tiny and the
// far-negative branches are kept so that this matches the CUDA operator over the
// whole BF16 range.
inline float silu_staged(float x) {
  uint32_t bits;
  std::memcpy(&bits, &x, 4);
  if ((bits & 0x7fffffffu) <= 0x01000000u) return x * 0.5f;
  if (x < -80.0f) {
    const double e = std::exp(double(x));
    return float(double(x) * e / (1.0 + e));
  }
  return float(double(x) / (1.0 + std::exp(-double(x))));
}

// One (row, head) of causal attention over positions 0..last.
void attention_row(const float* q, const float* keys, const float* values, size_t kv_stride,
                   size_t last, size_t d, float scale, float* out, int mode) {
  if (mode == 0) {
    // runtime/src/qwen.cpp:382-403: online softmax, FP32 state, output rescaled in place.
    float maximum = -std::numeric_limits<float>::infinity(), denominator = 0.0f;
    for (size_t c = 0; c < d; ++c) out[c] = 0.0f;
    for (size_t position = 0; position <= last; ++position) {
      const float* key = keys + position * kv_stride;
      const float* value = values + position * kv_stride;
      float score = 0.0f;
      for (size_t c = 0; c < d; ++c) score += q[c] * key[c];
      score *= scale;
      const float next_maximum = std::max(maximum, score);
      const float previous_scale = std::exp(maximum - next_maximum);
      const float probability = std::exp(score - next_maximum);
      denominator = denominator * previous_scale + probability;
      for (size_t c = 0; c < d; ++c) out[c] = out[c] * previous_scale + probability * value[c];
      maximum = next_maximum;
    }
    for (size_t c = 0; c < d; ++c) out[c] = out[c] / denominator;
    return;
  }
  // Staged: FP32 scores (scaled after the dot product), global maximum, numerators
  // rounded to BF16 for the PV sum, denominator from unrounded values, one output rounding.
  std::vector<float> scores(last + 1);
  float maximum = -std::numeric_limits<float>::infinity();
  for (size_t position = 0; position <= last; ++position) {
    scores[position] = float(dot_fp64(q, keys + position * kv_stride, d, 0.0)) * scale;
    maximum = std::max(maximum, scores[position]);
  }
  double denominator = 0.0;
  std::vector<double> accumulator(d, 0.0);
  for (size_t position = 0; position <= last; ++position) {
    const float p = float(std::exp(double(scores[position]) - double(maximum)));
    denominator += p;
    const double rounded = round_bf16(p);
    const float* value = values + position * kv_stride;
    for (size_t c = 0; c < d; ++c) accumulator[c] += rounded * double(value[c]);
  }
  for (size_t c = 0; c < d; ++c) out[c] = round_bf16(float(accumulator[c] / denominator));
}

// Greedy token of one logit row: NaN -> -inf, ties -> lowest index
// (runtime/src/qwen.cpp:462-470; operators/src/cuda/execution.cu:199-212 with a stable sort).
uint32_t argmax_row(const float* row, size_t vocab) {
  float best = 0.0f;
  uint32_t index = 0;
  for (size_t i = 0; i < vocab; ++i) {
    float value = row[i];
    if (std::isnan(value)) value = -std::numeric_limits<float>::infinity();
    if (i == 0 || value > best) {
      best = value;
      index = uint32_t(i);
    }
  }
  return index;
}

struct Workspace {
  std::vector<float> residual, normed, q, k, v, attention, projected, gate, up, ffn;
};

int forward(Model& m, const uint32_t* tokens, size_t rows, int mode, float* logits) {
  const Config& c = m.c;
  if (!rows || m.length + rows > m.capacity) {
    g_error = "oracle: rows exceed cache capacity";
    return 1;
  }
  for (size_t r = 0; r < rows; ++r)
    if (tokens[r] >= c.vocab) {
      g_error = "oracle: token exceeds vocabulary";
      return 1;
    }
  const size_t offset = m.length;
  m.length += rows;  // cache.resize(size + rows) before the forward (speculative_decoder.cpp:191)
  const size_t H = c.hidden, qw = c.heads * c.head_dim, kvw = c.kv_heads * c.head_dim, d = c.head_dim;
  Workspace w;
  w.residual.resize(rows * H);
  w.normed.resize(rows * H);
  w.q.resize(rows * qw);
  w.k.resize(rows * kvw);
  w.v.resize(rows * kvw);
  w.attention.resize(rows * qw);
  w.projected.resize(rows * H);
  w.gate.resize(rows * c.ffn);
  w.up.resize(rows * c.ffn);
  w.ffn.resize(rows * H);
  for (size_t r = 0; r < rows; ++r)
    std::memcpy(&w.residual[r * H], &m.embedding[size_t(tokens[r]) * H], H * sizeof(float));
  const size_t groups = c.heads / c.kv_heads;
  const float scale = 1.0f / std::sqrt(float(d));
  for (size_t layer = 0; layer < c.layers; ++layer) {
    const auto& L = m.layers[layer];
    rms_norm(w.residual.data(), L.attention_norm.data(), w.normed.data(), rows, H, c.eps, mode);
    linear(L.q, w.normed.data(), rows, w.q.data(), mode);
    linear(L.k, w.normed.data(), rows, w.k.data(), mode);
    linear(L.v, w.normed.data(), rows, w.v.data(), mode);
    if (c.qk_norm) {
      rms_norm(w.q.data(), L.q_norm.data(), w.q.data(), rows * c.heads, d, c.eps, mode);
      rms_norm(w.k.data(), L.k_norm.data(), w.k.data(), rows * c.kv_heads, d, c.eps, mode);
    }
    rope(m, w.q.data(), rows, c.heads, offset, mode);
    rope(m, w.k.data(), rows, c.kv_heads, offset, mode);
    float* kc = m.k_cache.data() + layer * m.capacity * kvw;
    float* vc = m.v_cache.data() + layer * m.capacity * kvw;
    std::memcpy(kc + offset * kvw, w.k.data(), rows * kvw * sizeof(float));
    std::memcpy(vc + offset * kvw, w.v.data(), rows * kvw * sizeof(float));
    parallel_for((long long)(rows * c.heads), [&](long long index) {
      const size_t r = size_t(index) / c.heads, head = size_t(index) % c.heads;
      const size_t key_base = (head / groups) * d;
      attention_row(&w.q[r * qw + head * d], kc + key_base, vc + key_base, kvw, offset + r, d, scale,
                    &w.attention[r * qw + head * d], mode);
    });
    linear(L.o, w.attention.data(), rows, w.projected.data(), mode);
    for (size_t i = 0; i < rows * H; ++i) {
      const float sum = w.residual[i] + w.projected[i];
      w.residual[i] = mode == 0 ? sum : round_bf16(sum);
    }
    rms_norm(w.residual.data(), L.ffn_norm.data(), w.normed.data(), rows, H, c.eps, mode);
    linear(L.gate, w.normed.data(), rows, w.gate.data(), mode);
    linear(L.up, w.normed.data(), rows, w.up.data(), mode);
    for (size_t i = 0; i < rows * c.ffn; ++i) {
      const float g = w.gate[i];
      if (mode == 0)
        w.gate[i] = (g / (1.0f + std::exp(-g))) * w.up[i];  // runtime/src/qwen.cpp:413-414
      else
        w.gate[i] = round_bf16(round_bf16(silu_staged(g)) * w.up[i]);
    }
    linear(L.down, w.gate.data(), rows, w.ffn.data(), mode);
    for (size_t i = 0; i < rows * H; ++i) {
      const float sum = w.residual[i] + w.ffn[i];
      w.residual[i] = mode == 0 ? sum : round_bf16(sum);
    }
  }
  rms_norm(w.residual.data(), m.output_norm.data(), w.normed.data(), rows, H, c.eps, mode);
  linear(m.lm_head, w.normed.data(), rows, logits, mode);
  return 0;
}

Linear* find_linear(Model& m, const std::string& name, size_t& layer_out) {
  if (name == "lm_head") return &m.lm_head;
  static const char* prefixes[] = {"w_gate", "w_up", "w_down", "wq", "wk", "wv", "wo"};
  for (const char* p : prefixes) {
    const std::string prefix(p);
    if (name.rfind(prefix, 0) == 0 && name.size() > prefix.size() &&
        name.find_first_not_of("0123456789", prefix.size()) == std::string::npos) {
      const size_t layer = std::stoul(name.substr(prefix.size()));
      if (layer >= m.layers.size()) return nullptr;
      layer_out = layer;
      auto& L = m.layers[layer];
      if (prefix == "wq") return &L.q;
      if (prefix == "wk") return &L.k;
      if (prefix == "wv") return &L.v;
      if (prefix == "wo") return &L.o;
      if (prefix == "w_gate") return &L.gate;
      if (prefix == "w_up") return &L.up;
      return &L.down;
    }
  }
  return nullptr;
}

// Bias keys of the reference's weight schema (runtime/include/models/qwen3_model.hpp:363-408).
Linear* find_bias_owner(Model& m, const std::string& name) {
  if (name == "lm_head.bias") return &m.lm_head;
  if (name.rfind("layers.", 0) != 0) return nullptr;
  const auto end = name.find('.', 7);
  if (end == std::string::npos) return nullptr;
  const size_t layer = std::stoul(name.substr(7, end - 7));
  if (layer >= m.layers.size()) return nullptr;
  auto& L = m.layers[layer];
  const std::string suffix = name.substr(end + 1);
  if (suffix == "self_attn.q_proj.bias") return &L.q;
  if (suffix == "self_attn.k_proj.bias") return &L.k;
  if (suffix == "self_attn.v_proj.bias") return &L.v;
  if (suffix == "self_attn.o_proj.bias") return &L.o;
  if (suffix == "mlp.gate_proj.bias") return &L.gate;
  if (suffix == "mlp.up_proj.bias") return &L.up;
  if (suffix == "mlp.down_proj.bias") return &L.down;
  return nullptr;
}

std::vector<float>* find_vector(Model& m, const std::string& name) {
  if (name == "rms_out_w") return &m.output_norm;
  static const char* prefixes[] = {"rms_att_w", "rms_ffn_w", "q_norm", "k_norm"};
  for (const char* p : prefixes) {
    const std::string prefix(p);
    if (name.rfind(prefix, 0) == 0 && name.size() > prefix.size()) {
      const size_t layer = std::stoul(name.substr(prefix.size()));
      if (layer >= m.layers.size()) return nullptr;
      auto& L = m.layers[layer];
      if (prefix == "rms_att_w") return &L.attention_norm;
      if (prefix == "rms_ffn_w") return &L.ffn_norm;
      if (prefix == "q_norm") return &L.q_norm;
      return &L.k_norm;
    }
  }
  return nullptr;
}

}  // namespace

extern "C" {

const char* vo_last_error() { return g_error.c_str(); }

uint16_t vo_float_to_bf16(float value) { return float_to_bf16(value); }
float vo_bf16_to_float(uint16_t bits) { return bf16_to_float(bits); }

void vo_round_bf16_inplace(float* data, uint64_t count) {
  for (uint64_t i = 0; i < count; ++i) data[i] = round_bf16(data[i]);
}

void* vo_create(const Config* config, uint64_t capacity) {
  auto m = std::make_unique<Model>();
  m->c = *config;
  m->layers.resize(config->layers);
  m->capacity = capacity;
  const size_t kvw = config->kv_heads * config->head_dim;
  m->k_cache.assign(config->layers * capacity * kvw, 0.0f);
  m->v_cache.assign(config->layers * capacity * kvw, 0.0f);
  build_rope_table(*m);
  return m.release();
}

void vo_destroy(void* h) { delete static_cast<Model*>(h); }

// Dense tensor, FP32 values. Linear weights are [out][in] (each output's inputs contiguous).
int vo_set_dense(void* h, const char* name_c, const float* data, uint64_t rows, uint64_t cols) {
  Model& m = *static_cast<Model*>(h);
  const std::string name(name_c);
  size_t layer = 0;
  if (name == "token_embeddings.weight") {
    m.embedding.assign(data, data + rows * cols);
    return 0;
  }
  if (Linear* l = find_linear(m, name, layer)) {
    l->out = rows;
    l->in = cols;
    l->weight.assign(data, data + rows * cols);
    return 0;
  }
  if (Linear* l = find_bias_owner(m, name)) {
    l->bias.assign(data, data + rows * cols);
    return 0;
  }
  if (auto* v = find_vector(m, name)) {
    v->assign(data, data + rows * cols);
    return 0;
  }
  g_error = "oracle: unknown tensor " + name;
  return 1;
}

// AWQ triple in the reference's N-major packing: qweight int32 [out][in/8] with nibble
// k%8 at bit 4*(k%8); scales BF16 [out][padded_groups]; zeros int32 [out][ceil(groups/8)].
// Dequantised as awq_gemv_gemm.cu:591-599; round_bf16 != 0 keeps the rows>1 rounding (:599).
int vo_set_awq(void* h, const char* name_c, const int32_t* qweight, const uint16_t* scales,
               const int32_t* zeros, uint64_t out, uint64_t in, int32_t group, int32_t padded_groups,
               int32_t round_weights) {
  Model& m = *static_cast<Model*>(h);
  size_t layer = 0;
  Linear* l = find_linear(m, name_c, layer);
  if (!l || in % group) {
    g_error = std::string("oracle: bad AWQ tensor ") + name_c;
    return 1;
  }
  l->out = out;
  l->in = in;
  l->weight.resize(out * in);
  const size_t weight_stride = (in + 7) / 8, zero_stride = (in / group + 7) / 8;
  for (size_t column = 0; column < out; ++column)
    for (size_t feature = 0; feature < in; ++feature) {
      const size_t g = feature / group;
      const uint32_t value = (uint32_t(qweight[column * weight_stride + feature / 8]) >> ((feature % 8) * 4)) & 15u;
      const uint32_t zero = (uint32_t(zeros[column * zero_stride + g / 8]) >> ((g % 8) * 4)) & 15u;
      float weight = (float(value) - float(zero)) * bf16_to_float(scales[column * padded_groups + g]);
      if (round_weights) weight = round_bf16(weight);
      l->weight[column * in + feature] = weight;
    }
  return 0;
}

uint64_t vo_size(void* h) { return static_cast<Model*>(h)->length; }

int vo_resize(void* h, uint64_t length) {
  Model& m = *static_cast<Model*>(h);
  if (length > m.capacity) {
    g_error = "oracle: resize beyond capacity";
    return 1;
  }
  m.length = length;
  return 0;
}

// Appends `rows` tokens at the current length and returns logits [rows][vocab].
int vo_forward(void* h, const uint32_t* tokens, int32_t rows, int32_t mode, float* logits) {
  return forward(*static_cast<Model*>(h), tokens, size_t(rows), mode, logits);
}

int vo_read_kv(void* h, uint64_t layer, float* k, float* v) {
  Model& m = *static_cast<Model*>(h);
  const size_t kvw = m.c.kv_heads * m.c.head_dim;
  std::memcpy(k, m.k_cache.data() + layer * m.capacity * kvw, m.length * kvw * sizeof(float));
  std::memcpy(v, m.v_cache.data() + layer * m.capacity * kvw, m.length * kvw * sizeof(float));
  return 0;
}

void vo_argmax(const float* logits, uint64_t rows, uint64_t vocab, uint32_t* tokens) {
  for (uint64_t r = 0; r < rows; ++r) tokens[r] = argmax_row(logits + r * vocab, vocab);
}

// Top-2 gap of each row (NaN treated as -inf), for the "gap exceeds tolerance" parity gate.
void vo_top2_gap(const float* logits, uint64_t rows, uint64_t vocab, float* gaps) {
  for (uint64_t r = 0; r < rows; ++r) {
    float first = -std::numeric_limits<float>::infinity(), second = first;
    for (uint64_t i = 0; i < vocab; ++i) {
      float value = logits[r * vocab + i];
      if (std::isnan(value)) value = -std::numeric_limits<float>::infinity();
      if (value > first) {
        second = first;
        first = value;
      } else if (value > second) {
        second = value;
      }
    }
    gaps[r] = first - second;
  }
}

// Greedy acceptance of one verify step (runtime/src/speculative_decoder.cpp:214-223):
// inputs = [pending, d1..dk], targets = greedy token of each of the k+1 rows. Emits
// targets[0..m] where m is the number of leading drafts with targets[i] == inputs[i+1].
// Returns the number of emitted tokens (= retained KV rows).
int32_t vo_accept(const uint32_t* inputs, const uint32_t* targets, int32_t rows) {
  int32_t emitted = 0;
  for (int32_t i = 0; i < rows; ++i) {
    ++emitted;
    if (i + 1 >= rows || targets[i] != inputs[i + 1]) break;
  }
  return emitted;
}

// ---- standalone operators in the staged arithmetic (FP32 arrays holding BF16 values) ----

// out[rows][n] = round_bf16(bias + sum_k x[k] * W[n][k]); W given dense [n][k].
void vo_op_linear(const float* x, const float* w, const float* bias, uint64_t rows, uint64_t n,
                  uint64_t k, float* out) {
  Linear l;
  l.in = k;
  l.out = n;
  l.weight.assign(w, w + n * k);
  if (bias) l.bias.assign(bias, bias + n);
  linear(l, x, rows, out, 1);
}

void vo_op_rms_norm(const float* x, const float* weight, uint64_t rows, uint64_t width, float eps,
                    float* out) {
  rms_norm(x, weight, out, rows, width, eps, 1);
}

// In-place RoPE of [rows][heads][head_dim] at positions offset.. from a table built
// for (theta, head_dim, max_pos) as the prepared model does.
void vo_op_rope(float* data, uint64_t rows, uint64_t heads, uint64_t head_dim, uint64_t offset,
                float theta, uint64_t max_pos) {
  Model m;
  m.c.head_dim = head_dim;
  m.c.theta = theta;
  m.c.max_pos = max_pos;
  build_rope_table(m);
  rope(m, data, rows, heads, offset, 1);
}

void vo_op_rope_table(float* table, uint64_t head_dim, float theta, uint64_t max_pos) {
  Model m;
  m.c.head_dim = head_dim;
  m.c.theta = theta;
  m.c.max_pos = max_pos;
  build_rope_table(m);
  std::memcpy(table, m.rope_table.data(), m.rope_table.size() * sizeof(float));
}

void vo_op_silu_multiply(const float* gate, const float* up, uint64_t count, float* out) {
  for (uint64_t i = 0; i < count; ++i) out[i] = round_bf16(round_bf16(silu_staged(gate[i])) * up[i]);
}

void vo_op_add(const float* a, const float* b, uint64_t count, float* out) {
  for (uint64_t i = 0; i < count; ++i) out[i] = round_bf16(a[i] + b[i]);
}

// Causal attention of q [rows][heads][d] at absolute offset over k, v [length][kv_heads][d]
// (length >= offset + rows); out [rows][heads][d]. mode as in vo_forward.
void vo_op_attention(const float* q, const float* k, const float* v, uint64_t rows, uint64_t heads,
                     uint64_t kv_heads, uint64_t d, uint64_t offset, int32_t mode, float* out) {
  const size_t groups = heads / kv_heads, kvw = kv_heads * d, qw = heads * d;
  const float scale = 1.0f / std::sqrt(float(d));
  parallel_for((long long)(rows * heads), [&](long long index) {
    const size_t r = size_t(index) / heads, head = size_t(index) % heads;
    const size_t base = (head / groups) * d;
    attention_row(q + r * qw + head * d, k + base, v + base, kvw, offset + r, d, scale, out + r * qw + head * d,
                  mode);
  });
}

// Host threads the oracle may use (0 = all). Results do not depend on it; bench.py uses it to time one core.
void vo_set_threads(int32_t threads) { g_threads = threads; }

}  // extern "C"
