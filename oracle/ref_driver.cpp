// TEST INFRASTRUCTURE ONLY. Thin C entry points around the UNMODIFIED edge-infer
// reference library, compiled by oracle/Makefile from the reference's own source
// tree into oracle/_ref/libedge_ref.so. Nothing here is shipped or measured as the
// product; the tests use it to pin the CPU restatement in oracle/verify_oracle.cpp and,
// on a GPU box, to compare logits with the reference CUDA path.
//
// Entry points used (reference paths):
//   QwenModel<float> CPU executor        runtime/include/qwen.hpp:18-128, runtime/src/qwen.cpp:335-424
//   QwenModel<float>::sample_cpu         runtime/src/qwen.cpp:451-470
//   KVCache<T>                           runtime/include/inference.hpp:31-138
//   Qwen3Model<bf16> / Qwen3Session<bf16> runtime/include/models/qwen3_model.hpp, runtime/src/qwen3.cpp
//   op::cuda::sample                     operators/src/cuda/execution.cu:463-498
//   op::cuda::{rms_norm, add, silu_multiply, rope_precomputed, store_kv, awq_linear, linear,
//              attention_prefill}       operators/include/operators/cuda/execution.hpp:55-124
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "common.hpp"
#include "qwen.hpp"

extern "C" {

struct ref_config {
  uint64_t vocab, layers, heads, kv_heads, hidden, head_dim, ffn, max_pos;
  float eps, theta;
  int32_t qk_norm, group_size;
  uint32_t eos;
};

// Host tensors. `transposed` means the data is physically [shape[1], shape[0]]
// row-major and is presented to the reference as the logical [shape[0], shape[1]]
// transposed view (the layout HF checkpoints give: [out, in] for a linear).
struct ref_tensor {
  const char* name;
  const void* data;
  uint64_t shape[2];
  int32_t rank;
  int32_t transposed;
};

}  // extern "C"

namespace {

thread_local std::string g_error;

ModelConfig make_config(const ref_config& c) {
  ModelConfig m;
  m["vocab_size"] = double(c.vocab);
  m["n_layers"] = double(c.layers);
  m["n_heads"] = double(c.heads);
  m["n_kv_heads"] = double(c.kv_heads);
  m["hidden_size"] = double(c.hidden);
  m["head_dim"] = double(c.head_dim);
  m["intermediate_size"] = double(c.ffn);
  m["max_position_embeddings"] = double(c.max_pos);
  m["bos_token_id"] = 0;
  m["eos_token_id"] = double(c.eos);
  m["rms_norm_eps"] = c.eps;
  m["rope_theta"] = c.theta;
  m["qk_norm"] = c.qk_norm;
  m["group_size"] = c.group_size;
  return m;
}

template <typename T>
Tensor<T> host_tensor(const ref_tensor& t) {
  std::vector<size_t> shape;
  size_t count = 1;
  for (int i = 0; i < t.rank; ++i) count *= t.shape[i];
  std::vector<T> values(count);
  std::memcpy(values.data(), t.data, count * sizeof(T));
  if (t.rank == 2 && t.transposed) {
    Tensor<T> physical(std::move(values), {size_t(t.shape[1]), size_t(t.shape[0])});
    return physical.transpose(0, 1);
  }
  for (int i = 0; i < t.rank; ++i) shape.push_back(t.shape[i]);
  return Tensor<T>(std::move(values), shape);
}

struct CpuHandle {
  std::shared_ptr<QwenModel<float>> model;
  std::unique_ptr<KVCache<float>> cache;
  ref_config config;
};

struct CudaHandle {
  std::shared_ptr<Qwen3Model<__nv_bfloat16>> model;
  std::unique_ptr<Qwen3Session<__nv_bfloat16>> session;
  std::unique_ptr<KVCache<__nv_bfloat16>> cache;
  Tensor<uint32_t> tokens, sampled;
  op::cuda::SamplingPlan plan;
  op::cuda::ExecutionContext context;
  CudaWorkspaceArena scratch;
  ref_config config;
};

template <typename F>
int guarded(F&& body) {
  try {
    body();
    return 0;
  } catch (const std::exception& e) {
    g_error = e.what();
    return 1;
  } catch (...) {
    g_error = "unknown exception";
    return 1;
  }
}

}  // namespace

extern "C" {

const char* ref_last_error() { return g_error.c_str(); }

// ---------------------------------------------------------------- CPU FP32
void* ref_cpu_create(const ref_config* config, const ref_tensor* tensors, int count,
                     uint64_t capacity) {
  CpuHandle* handle = nullptr;
  const int status = guarded([&] {
    QwenModel<float>::Parameters parameters;
    for (int i = 0; i < count; ++i) parameters.emplace(tensors[i].name, host_tensor<float>(tensors[i]));
    auto owned = std::make_unique<CpuHandle>();
    owned->config = *config;
    owned->model = std::make_shared<QwenModel<float>>(parameters, make_config(*config));
    owned->cache = std::make_unique<KVCache<float>>(config->layers, capacity,
                                                    config->kv_heads * config->head_dim, Device::CPU);
    handle = owned.release();
  });
  return status ? nullptr : handle;
}

void ref_cpu_destroy(void* h) { delete static_cast<CpuHandle*>(h); }

uint64_t ref_cpu_size(void* h) { return static_cast<CpuHandle*>(h)->cache->size(); }

int ref_cpu_resize(void* h, uint64_t length) {
  return guarded([&] { static_cast<CpuHandle*>(h)->cache->resize(length); });
}

// cache.resize(size + rows); prefill_generic(tokens) -> logits [rows, vocab] (FP32).
int ref_cpu_forward(void* h, const uint32_t* tokens, int rows, float* logits) {
  return guarded([&] {
    auto* handle = static_cast<CpuHandle*>(h);
    std::vector<uint32_t> ids(tokens, tokens + rows);
    Tensor<uint32_t> input(std::move(ids), {size_t(rows)});
    handle->cache->resize(handle->cache->size() + rows);
    auto out = handle->model->prefill_generic(&input, handle->cache.get());
    std::memcpy(logits, out.data, size_t(rows) * handle->config.vocab * sizeof(float));
  });
}

// Greedy token of every row through the reference's own sample_cpu (top_k = 1).
int ref_cpu_greedy(void* h, const float* logits, int rows, uint32_t* tokens) {
  return guarded([&] {
    auto* handle = static_cast<CpuHandle*>(h);
    const size_t vocab = handle->config.vocab;
    for (int r = 0; r < rows; ++r) {
      TensorView<const float, 2> row{logits + size_t(r) * vocab, {1, vocab}, {vocab, 1}};
      tokens[r] = handle->model->sample_cpu(row, 1.0f, 1.0f, 1);
    }
  });
}

// Copies K and V rows [0, size) of one layer (FP32, [size, kv_heads*head_dim]).
int ref_cpu_read_kv(void* h, uint64_t layer, float* k, float* v) {
  return guarded([&] {
    auto* handle = static_cast<CpuHandle*>(h);
    auto kv = handle->cache->k_view(layer), vv = handle->cache->v_view(layer);
    std::memcpy(k, kv.data, kv.numel() * sizeof(float));
    std::memcpy(v, vv.data, vv.numel() * sizeof(float));
  });
}

// ---------------------------------------------------------------- CUDA BF16
// dense: BF16 tensors (uint16 payload); qweights/zeros: int32; scales: BF16.
void* ref_cuda_create(const ref_config* config, const ref_tensor* dense, int n_dense,
                      const ref_tensor* qweights, int n_q, const ref_tensor* scales, int n_s,
                      const ref_tensor* zeros, int n_z, uint64_t capacity) {
  CudaHandle* handle = nullptr;
  const int status = guarded([&] {
    using T = __nv_bfloat16;
    Qwen3Model<T>::Parameters parameters, scale_parameters;
    Qwen3Model<T>::IntegerParameters q_parameters, z_parameters;
    for (int i = 0; i < n_dense; ++i) parameters.emplace(dense[i].name, host_tensor<T>(dense[i]));
    for (int i = 0; i < n_s; ++i) scale_parameters.emplace(scales[i].name, host_tensor<T>(scales[i]));
    for (int i = 0; i < n_q; ++i) q_parameters.emplace(qweights[i].name, host_tensor<int32_t>(qweights[i]));
    for (int i = 0; i < n_z; ++i) z_parameters.emplace(zeros[i].name, host_tensor<int32_t>(zeros[i]));
    auto owned = std::make_unique<CudaHandle>();
    owned->config = *config;
    const auto model_config = make_config(*config);
    owned->model = n_q ? std::make_shared<Qwen3Model<T>>(parameters, q_parameters, scale_parameters,
                                                          z_parameters, model_config)
                       : std::make_shared<Qwen3Model<T>>(parameters, model_config);
    owned->session = std::make_unique<Qwen3Session<T>>(owned->model, false);
    owned->cache = std::make_unique<KVCache<T>>(config->layers, capacity,
                                                config->kv_heads * config->head_dim, Device::CUDA);
    owned->tokens = Tensor<uint32_t>({size_t(capacity)}, Device::CUDA);
    owned->sampled = Tensor<uint32_t>({size_t(capacity)}, Device::CUDA);
    owned->context = op::cuda::prepare_execution_context(nullptr, owned->session->stream());
    owned->plan = op::cuda::prepare_sampling(owned->context, config->vocab);
    owned->scratch.reserve(owned->plan.total_bytes);
    handle = owned.release();
  });
  return status ? nullptr : handle;
}

void ref_cuda_destroy(void* h) { delete static_cast<CudaHandle*>(h); }

uint64_t ref_cuda_size(void* h) { return static_cast<CudaHandle*>(h)->cache->size(); }

int ref_cuda_resize(void* h, uint64_t length) {
  return guarded([&] { static_cast<CudaHandle*>(h)->cache->resize(length); });
}

// cache.resize(size + rows); Qwen3Session::prefill_eager; op::cuda::sample(top_k=1).
// logits: host BF16 [rows, vocab] (may be null); greedy: host uint32 [rows].
int ref_cuda_forward(void* h, const uint32_t* tokens, int rows, uint16_t* logits, uint32_t* greedy) {
  return guarded([&] {
    using T = __nv_bfloat16;
    auto* handle = static_cast<CudaHandle*>(h);
    const size_t vocab = handle->config.vocab;
    CUDA_CHECK(cudaMemcpy(handle->tokens.data_ptr(), tokens, rows * sizeof(uint32_t), cudaMemcpyHostToDevice));
    auto input = Tensor<uint32_t>::from_external_buffer(handle->tokens.data_ptr(), {size_t(rows)}, Device::CUDA);
    handle->cache->resize(handle->cache->size() + rows);
    auto out = handle->session->prefill_eager(&input, handle->cache.get());
    TensorView<unsigned char, 1> scratch{handle->scratch.template ptr_at<unsigned char>(0),
                                         {handle->plan.total_bytes}, {1}};
    op::cuda::sample<T>(handle->context, out.as_const(), {handle->sampled.data_ptr(), {size_t(rows)}, {1}},
                        {}, scratch, handle->plan, 1.0f, 1.0f, 1, nullptr);
    CUDA_CHECK(cudaStreamSynchronize(handle->context.stream));
    if (logits)
      CUDA_CHECK(cudaMemcpy(logits, out.data, size_t(rows) * vocab * sizeof(T), cudaMemcpyDeviceToHost));
    CUDA_CHECK(cudaMemcpy(greedy, handle->sampled.data_ptr(), rows * sizeof(uint32_t), cudaMemcpyDeviceToHost));
  });
}

// ---------------------------------------------------------------- CUDA operators
// The reference's own direct operators on caller-owned DEVICE buffers (BF16 unless noted), on the
// default stream, followed by a stream synchronisation. Used to compare single operators on
// identical device inputs on the same GPU.
namespace {
using B = __nv_bfloat16;
op::cuda::ExecutionContext& operator_context() {
  static cublasHandle_t handle = [] {
    cublasHandle_t h = nullptr;
    if (cublasCreate(&h) != CUBLAS_STATUS_SUCCESS) throw std::runtime_error("cublasCreate failed");
    return h;
  }();
  static op::cuda::ExecutionContext context = op::cuda::prepare_execution_context(handle, nullptr);
  op::cuda::bind_execution_context(context);
  return context;
}
void finish_operator() { CUDA_CHECK(cudaStreamSynchronize(nullptr)); }
}  // namespace

int ref_op_rms_norm(const void* in, const void* weight, void* out, uint64_t rows, uint64_t features, float eps) {
  return guarded([&] {
    op::cuda::rms_norm<B>(operator_context(), {static_cast<const B*>(in), size_t(rows * features)},
                          {static_cast<const B*>(weight), size_t(features)},
                          {static_cast<B*>(out), size_t(rows * features)}, rows, features, eps);
    finish_operator();
  });
}

int ref_op_add(const void* a, const void* b, void* out, uint64_t count) {
  return guarded([&] {
    op::cuda::add<B>(operator_context(), {static_cast<const B*>(a), size_t(count)},
                     {static_cast<const B*>(b), size_t(count)}, {static_cast<B*>(out), size_t(count)});
    finish_operator();
  });
}

int ref_op_silu_multiply(const void* gate, const void* up, void* out, uint64_t count) {
  return guarded([&] {
    op::cuda::silu_multiply<B>({static_cast<const B*>(gate), size_t(count)}, {static_cast<const B*>(up), size_t(count)},
                               {static_cast<B*>(out), size_t(count)}, nullptr);
    finish_operator();
  });
}

// data: [rows, heads, head_dim] contiguous, rotated in place; table: float [positions, head_dim].
int ref_op_rope_precomputed(void* data, uint64_t rows, uint64_t heads, uint64_t head_dim, const float* table,
                            uint64_t positions, uint64_t offset) {
  return guarded([&] {
    TensorView<B, 3> view{static_cast<B*>(data), {size_t(rows), size_t(heads), size_t(head_dim)},
                          {size_t(heads * head_dim), size_t(head_dim), 1}};
    TensorView<const float, 2> cache{table, {size_t(positions), size_t(head_dim)}, {size_t(head_dim), 1}};
    op::cuda::rope_precomputed<B>(operator_context(), view, cache, offset);
    finish_operator();
  });
}

// source: [rows, width]; cache: [capacity, width]; rows are written at `offset`.
int ref_op_store_kv(const void* source, void* cache, uint64_t rows, uint64_t width, uint64_t capacity, uint64_t offset) {
  return guarded([&] {
    TensorView<const B, 2> src{static_cast<const B*>(source), {size_t(rows), size_t(width)}, {size_t(width), 1}};
    TensorView<B, 2> dst{static_cast<B*>(cache), {size_t(capacity), size_t(width)}, {size_t(width), 1}};
    op::cuda::store_kv<B>(operator_context(), src, dst, offset);
    finish_operator();
  });
}

// qweight int32 [N, K/8], scales BF16 [N, padded_groups], zeros int32 [N, ceil(K/group/8)], bias BF16 [N] or null.
int ref_op_awq_linear(const void* x, uint64_t rows, uint64_t K, uint64_t N, const int32_t* qweight, const void* scales,
                      uint64_t padded_groups, const int32_t* zeros, uint64_t group_size, const void* bias, void* out) {
  return guarded([&] {
    const size_t groups = (K + group_size - 1) / group_size;
    TensorView<const int32_t, 2> q{qweight, {size_t(N), size_t((K + 7) / 8)}, {size_t((K + 7) / 8), 1}};
    TensorView<const B, 2> s{static_cast<const B*>(scales), {size_t(N), size_t(padded_groups)}, {size_t(padded_groups), 1}};
    TensorView<const int32_t, 2> z{zeros, {size_t(N), (groups + 7) / 8}, {(groups + 7) / 8, 1}};
    TensorView<const B, 1> b{};
    if (bias) b = TensorView<const B, 1>{static_cast<const B*>(bias), {size_t(N)}, {1}};
    const auto weight = op::cuda::prepare_awq<B>(q, s, z, group_size, K, b);
    TensorView<const B, 2> input{static_cast<const B*>(x), {size_t(rows), size_t(K)}, {size_t(K), 1}};
    TensorView<B, 2> output{static_cast<B*>(out), {size_t(rows), size_t(N)}, {size_t(N), 1}};
    op::cuda::awq_linear<B>(operator_context(), input, weight, output);
    finish_operator();
  });
}

// weight: BF16 physically [N, K] row-major (the checkpoint layout), presented as the logical [K, N] view.
int ref_op_linear(const void* x, uint64_t rows, uint64_t K, uint64_t N, const void* weight, const void* bias, void* out) {
  return guarded([&] {
    TensorView<const B, 2> w{static_cast<const B*>(weight), {size_t(K), size_t(N)}, {1, size_t(K)}};
    TensorView<const B, 1> b{};
    if (bias) b = TensorView<const B, 1>{static_cast<const B*>(bias), {size_t(N)}, {1}};
    const auto prepared = op::cuda::prepare_dense<B>(w, b);
    TensorView<const B, 2> input{static_cast<const B*>(x), {size_t(rows), size_t(K)}, {size_t(K), 1}};
    TensorView<B, 2> output{static_cast<B*>(out), {size_t(rows), size_t(N)}, {size_t(N), 1}};
    op::cuda::linear<B>(operator_context(), input, prepared, output);
    finish_operator();
  });
}

// q, out: [rows, heads, 128]; k, v: [length, kv_heads, 128] with length = offset + rows.
int ref_op_attention_prefill(const void* q, const void* k, const void* v, void* out, uint64_t rows, uint64_t heads,
                             uint64_t kv_heads, uint64_t head_dim, uint64_t length, uint64_t offset) {
  return guarded([&] {
    TensorView<const B, 3> qv{static_cast<const B*>(q), {size_t(rows), size_t(heads), size_t(head_dim)},
                              {size_t(heads * head_dim), size_t(head_dim), 1}};
    TensorView<const B, 3> kv{static_cast<const B*>(k), {size_t(length), size_t(kv_heads), size_t(head_dim)},
                              {size_t(kv_heads * head_dim), size_t(head_dim), 1}};
    TensorView<const B, 3> vv{static_cast<const B*>(v), {size_t(length), size_t(kv_heads), size_t(head_dim)},
                              {size_t(kv_heads * head_dim), size_t(head_dim), 1}};
    TensorView<B, 3> ov{static_cast<B*>(out), {size_t(rows), size_t(heads), size_t(head_dim)},
                        {size_t(heads * head_dim), size_t(head_dim), 1}};
    op::cuda::attention_prefill<B>(operator_context(), qv, kv, vv, ov, offset);
    finish_operator();
  });
}

}  // extern "C"
