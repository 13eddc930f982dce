// Drop-in for the reference's operators/include/operators/cuda/execution.hpp on the verify path: the same
// namespace (op::cuda), names, argument order and exception types, over the C ABI of libedge_infer_b200.so
// (edge_infer_b200.h). A maintainer who puts this include directory before the reference's gets the sm_100a
// kernels behind the calls the decoder already makes (runtime/include/execution/decoder.hpp:110-171).
//
// Views: with the reference's own headers on the include path (core/include/tensor_view.hpp,
// operators/include/operators/core/array_view.hpp) its TensorView / op::ArrayView are used as they are;
// otherwise the two aggregates are defined here with the same members in the same order.
//
// What differs from the reference, and how it shows:
//  * BF16 only. T is any 16-bit element type (the library sees pointers); a 32-bit T does not compile.
//  * The cuBLAS handle of prepare_execution_context is accepted and ignored; bind_execution_context does nothing.
//  * linear / awq_linear take no scratch here, as in the reference: shapes whose input features exceed one K
//    slice (4096 for int4 weights, 16384 for BF16) then run the any-shape kernel, not the streaming one. Callers
//    that can supply scratch use the *_scratch overloads (no counterpart in the reference).
//  * attention_prefill takes no scratch either: it uses the library's built-in split buffer
//    (ei_attention_prefill_static_bf16) and throws std::invalid_argument for shapes beyond it.
//  * sample is greedy only: the request policy is validated as the reference validates it
//    (operators/src/cuda/execution.cu:455-475) and a request that is not greedy (top_k != 1 with a positive
//    temperature) is rejected with std::invalid_argument before anything is written - the speculative decoder
//    itself rejects such requests (runtime/src/speculative_decoder.cpp:233-234). `probabilities` must be empty.
//  * Not on the verify path and not declared: multiply, silu, rope (uncached), attention_decode, attention_graph,
//    token_probability.
#pragma once

#include <algorithm>
#include <array>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <type_traits>

#include "../../edge_infer_b200.h"

#if defined(__has_include)
#if __has_include("tensor_view.hpp") && __has_include("operators/core/array_view.hpp")
#include "operators/core/array_view.hpp"
#include "tensor_view.hpp"
#define EDGE_INFER_B200_REFERENCE_VIEWS 1
#endif
#endif

#ifndef EDGE_INFER_B200_REFERENCE_VIEWS
// Borrowed descriptors, laid out as the reference's (data pointer, extents, strides in elements).
template <typename T, std::size_t Rank>
struct TensorView {
  T* data = nullptr;
  std::array<std::size_t, Rank> shape{};
  std::array<std::size_t, Rank> stride{};

  // Packed row-major view of `extents`.
  static TensorView contiguous(T* storage, std::array<std::size_t, Rank> extents) {
    TensorView view{storage, extents, {}};
    std::size_t step = 1;
    for (std::size_t axis = Rank; axis-- > 0;) {
      view.stride[axis] = step;
      step *= extents[axis];
    }
    return view;
  }
  std::size_t numel() const {
    std::size_t count = 1;
    for (std::size_t extent : shape) count *= extent;
    return count;
  }
};
namespace op {
template <typename T>
struct ArrayView {
  T* data = nullptr;
  std::size_t size = 0;
};
}  // namespace op
#endif

// The handle and stream types of the reference's signatures, without requiring the CUDA headers.
struct cublasContext;
typedef struct cublasContext* cublasHandle_t;
struct CUstream_st;
typedef struct CUstream_st* cudaStream_t;
struct curandStateXORWOW;
typedef struct curandStateXORWOW curandState;

namespace op::cuda {

namespace detail {
// A failed call becomes the exception type the reference would have thrown.
inline void check(ei_status status) {
  if (status == EI_OK) return;
  const std::string what = ei_last_error();
  switch (status) {
    case EI_INVALID_ARGUMENT: throw std::invalid_argument(what);
    case EI_OUT_OF_RANGE: throw std::out_of_range(what);
    case EI_OVERFLOW: throw std::overflow_error(what);
    case EI_LOGIC: throw std::logic_error(what);
    case EI_LENGTH: throw std::length_error(what);
    default: throw std::runtime_error(what);  // EI_RUNTIME, EI_POISONED
  }
}
template <typename T>
inline void* erase(T* p) {
  return const_cast<void*>(static_cast<const void*>(p));
}
template <typename T>
inline ei_view1 view(const TensorView<T, 1>& v) {
  static_assert(sizeof(T) != 4 || !std::is_floating_point_v<T>, "only the 16-bit instantiations exist");
  return ei_view1{erase(v.data), {v.shape[0]}, {v.stride[0]}};
}
template <typename T>
inline ei_view2 view(const TensorView<T, 2>& v) {
  return ei_view2{erase(v.data), {v.shape[0], v.shape[1]}, {v.stride[0], v.stride[1]}};
}
template <typename T>
inline ei_view3 view(const TensorView<T, 3>& v) {
  return ei_view3{erase(v.data), {v.shape[0], v.shape[1], v.shape[2]}, {v.stride[0], v.stride[1], v.stride[2]}};
}
template <typename T>
inline ei_array view(const ::op::ArrayView<T>& v) {
  return ei_array{erase(v.data), v.size};
}
template <typename T>
constexpr void require_bf16() {
  static_assert(sizeof(T) == 2, "this library provides the BF16 instantiations of the direct operators only");
}
}  // namespace detail

// execution.hpp:18-26 of the reference, member for member.
struct ExecutionContext {
  cublasHandle_t handle = nullptr;
  cudaStream_t stream = nullptr;
  int device = 0;
  int multiprocessors = 1;
  int max_threads_per_block = 1024;
  std::size_t shared_memory_limit = 0;
  const void* attention_padding = nullptr;
};
namespace detail {
inline ei_context native(const ExecutionContext& c) {
  ei_context out{};
  out.handle = c.handle;
  out.stream = c.stream;
  out.device = c.device;
  out.multiprocessors = c.multiprocessors;
  out.max_threads_per_block = c.max_threads_per_block;
  out.shared_memory_limit = c.shared_memory_limit;
  return out;
}
}  // namespace detail

// execution.hpp:28-31. Queries the current device once; the handle is kept but never used.
inline ExecutionContext prepare_execution_context(cublasHandle_t handle, cudaStream_t stream) {
  ei_context native{};
  detail::check(ei_prepare_execution_context(stream, &native));
  ExecutionContext context;
  context.handle = handle;
  context.stream = stream;
  context.device = native.device;
  context.multiprocessors = native.multiprocessors;
  context.max_threads_per_block = native.max_threads_per_block;
  context.shared_memory_limit = native.shared_memory_limit;
  return context;
}
inline void bind_execution_context(const ExecutionContext&) {}

template <typename T>
using DenseLinearWeight = ei_dense_weight;  // execution.hpp:34-41
template <typename T>
using AwqLinearWeight = ei_awq_weight;      // execution.hpp:44-53

// execution.hpp:55-64.
template <typename T>
DenseLinearWeight<T> prepare_dense(TensorView<const T, 2> weight, TensorView<const T, 1> bias = {}) {
  detail::require_bf16<T>();
  DenseLinearWeight<T> out{};
  detail::check(ei_prepare_dense_bf16(detail::view(weight), detail::view(bias), &out));
  return out;
}
template <typename T>
AwqLinearWeight<T> prepare_awq(TensorView<const std::int32_t, 2> qweight, TensorView<const T, 2> scales,
                               TensorView<const std::int32_t, 2> zeros, std::size_t group_size,
                               std::size_t input_features, TensorView<const T, 1> bias = {}) {
  detail::require_bf16<T>();
  AwqLinearWeight<T> out{};
  detail::check(ei_prepare_awq_bf16(detail::view(qweight), detail::view(scales), detail::view(zeros), group_size,
                                    input_features, detail::view(bias), &out));
  return out;
}

// execution.hpp:65-70.
template <typename T>
void linear(const ExecutionContext& context, TensorView<const T, 2> input, const DenseLinearWeight<T>& weight,
            TensorView<T, 2> output) {
  detail::require_bf16<T>();
  const ei_context c = detail::native(context);
  detail::check(ei_linear_bf16(&c, detail::view(input), &weight, detail::view(output), nullptr, 0));
}
template <typename T>
void awq_linear(const ExecutionContext& context, TensorView<const T, 2> input, const AwqLinearWeight<T>& weight,
                TensorView<T, 2> output) {
  detail::require_bf16<T>();
  const ei_context c = detail::native(context);
  detail::check(ei_awq_linear_bf16(&c, detail::view(input), &weight, detail::view(output), nullptr, 0));
}
// No counterpart in the reference: the same two with caller-owned scratch (ei_linear_scratch_bytes), which lets
// wide inputs be split over blocks, and the fused gate|up projection with the SwiGLU product.
inline std::size_t linear_scratch_bytes(std::size_t rows, std::size_t input_features, std::size_t output_features) {
  return ei_linear_scratch_bytes(rows, input_features, output_features);
}
template <typename T>
void linear_scratch(const ExecutionContext& context, TensorView<const T, 2> input, const DenseLinearWeight<T>& weight,
                    TensorView<T, 2> output, void* scratch, std::size_t scratch_bytes) {
  const ei_context c = detail::native(context);
  detail::check(ei_linear_bf16(&c, detail::view(input), &weight, detail::view(output), scratch, scratch_bytes));
}
template <typename T>
void awq_linear_scratch(const ExecutionContext& context, TensorView<const T, 2> input,
                        const AwqLinearWeight<T>& weight, TensorView<T, 2> output, void* scratch,
                        std::size_t scratch_bytes) {
  const ei_context c = detail::native(context);
  detail::check(ei_awq_linear_bf16(&c, detail::view(input), &weight, detail::view(output), scratch, scratch_bytes));
}
template <typename T>
void awq_gate_up_silu(const ExecutionContext& context, TensorView<const T, 2> input,
                      const AwqLinearWeight<T>& gate_then_up, TensorView<T, 2> output) {
  const ei_context c = detail::native(context);
  detail::check(ei_awq_gate_up_silu_bf16(&c, detail::view(input), &gate_then_up, detail::view(output)));
}

// execution.hpp:72-74, direct.hpp:36-40, execution.hpp:85-90.
template <typename T>
void add(const ExecutionContext& context, ::op::ArrayView<const T> a, ::op::ArrayView<const T> b,
         ::op::ArrayView<T> output) {
  detail::require_bf16<T>();
  const ei_context c = detail::native(context);
  detail::check(ei_add_bf16(&c, detail::view(a), detail::view(b), detail::view(output)));
}
template <typename T>
void silu_multiply(::op::ArrayView<const T> gate, ::op::ArrayView<const T> up, ::op::ArrayView<T> output,
                   cudaStream_t stream = nullptr) {
  detail::require_bf16<T>();
  ei_context c{};
  c.stream = stream;
  c.multiprocessors = 128;  // only bounds the grid of this elementwise kernel; the reference's form has no context
  detail::check(ei_silu_multiply_bf16(&c, detail::view(gate), detail::view(up), detail::view(output)));
}
template <typename T>
void rms_norm(const ExecutionContext& context, ::op::ArrayView<const T> input, ::op::ArrayView<const T> weight,
              ::op::ArrayView<T> output, std::size_t rows, std::size_t features, float epsilon) {
  detail::require_bf16<T>();
  const ei_context c = detail::native(context);
  detail::check(ei_rms_norm_bf16(&c, detail::view(input), detail::view(weight), detail::view(output), rows, features,
                                 epsilon));
}
// execution.hpp:92-107.
template <typename T>
void gather(const ExecutionContext& context, TensorView<const std::uint32_t, 1> ids, TensorView<const T, 2> table,
            TensorView<T, 2> output) {
  detail::require_bf16<T>();
  const ei_context c = detail::native(context);
  detail::check(ei_gather_bf16(&c, detail::view(ids), detail::view(table), detail::view(output)));
}
template <typename T>
void rope_precomputed(const ExecutionContext& context, TensorView<T, 3> input, TensorView<const float, 2> cache,
                      std::size_t offset = 0, const std::size_t* offsets = nullptr, const int* pingpong = nullptr) {
  detail::require_bf16<T>();
  const ei_context c = detail::native(context);
  const ei_view2 table{detail::erase(cache.data), {cache.shape[0], cache.shape[1]}, {cache.stride[0], cache.stride[1]}};
  detail::check(ei_rope_precomputed_bf16(&c, detail::view(input), table, offset, offsets, pingpong));
}
template <typename T>
void store_kv(const ExecutionContext& context, TensorView<const T, 2> source, TensorView<T, 2> capacity,
              std::size_t offset, const std::size_t* device_offset = nullptr) {
  detail::require_bf16<T>();
  const ei_context c = detail::native(context);
  detail::check(ei_store_kv_bf16(&c, detail::view(source), detail::view(capacity), offset, device_offset));
}

// execution.hpp:117-122: causal attention of q's rows at absolute position `offset` over k / v.
template <typename T>
void attention_prefill(const ExecutionContext& context, TensorView<const T, 3> q, TensorView<const T, 3> k,
                       TensorView<const T, 3> v, TensorView<T, 3> output, std::size_t offset) {
  detail::require_bf16<T>();
  const ei_context c = detail::native(context);
  detail::check(ei_attention_prefill_static_bf16(&c, detail::view(q), detail::view(k), detail::view(v),
                                                 detail::view(output), offset));
}
// No counterpart in the reference: caller-owned split scratch (ei_attention_scratch_bytes), and the captured-graph
// form whose offset is read from device memory at launch (generalises attention_graph's device lengths, :123-130).
inline std::size_t attention_scratch_bytes(std::size_t q_rows, std::size_t query_heads, std::size_t head_dim,
                                           std::size_t kv_length) {
  return ei_attention_scratch_bytes(q_rows, query_heads, head_dim, kv_length);
}
template <typename T>
void attention_prefill_scratch(const ExecutionContext& context, TensorView<const T, 3> q, TensorView<const T, 3> k,
                               TensorView<const T, 3> v, TensorView<T, 3> output, std::size_t offset, void* scratch,
                               std::size_t scratch_bytes) {
  const ei_context c = detail::native(context);
  detail::check(ei_attention_prefill_bf16(&c, detail::view(q), detail::view(k), detail::view(v), detail::view(output),
                                          offset, scratch, scratch_bytes));
}
template <typename T>
void attention_verify(const ExecutionContext& context, TensorView<const T, 3> q, TensorView<const T, 3> k_capacity,
                      TensorView<const T, 3> v_capacity, TensorView<T, 3> output, const std::int32_t* device_offset,
                      void* scratch, std::size_t scratch_bytes) {
  const ei_context c = detail::native(context);
  detail::check(ei_attention_verify_bf16(&c, detail::view(q), detail::view(k_capacity), detail::view(v_capacity),
                                         detail::view(output), device_offset, scratch, scratch_bytes));
}

// execution.hpp:132-151. The plan's only live member is total_bytes (per-block argmax partials); the offsets of
// the reference's sort buffers stay zero.
struct SamplingPlan {
  std::size_t vocabulary = 0;
  std::size_t scaled_offset = 0;
  std::size_t sorted_offset = 0;
  std::size_t indices_offset = 0;
  std::size_t sorted_indices_offset = 0;
  std::size_t sort_offset = 0;
  std::size_t sort_bytes = 0;
  std::size_t total_bytes = 0;
};
inline SamplingPlan prepare_sampling(const ExecutionContext&, std::size_t vocabulary) {
  if (vocabulary < 1 || vocabulary > std::size_t(0x7fffffff))
    throw std::invalid_argument("sampling vocabulary must lie between 1 and 2^31 - 1");
  SamplingPlan plan;
  plan.vocabulary = vocabulary;
  plan.total_bytes = ei_sample_scratch_bytes(16, vocabulary);
  return plan;
}
inline void validate_sampling_policy(std::size_t vocabulary, float temperature, float top_p, std::size_t top_k,
                                     bool has_rng) {
  const std::size_t candidates = std::min(top_k, vocabulary);
  const bool well_formed = vocabulary >= 1 && top_k >= 1 && std::isfinite(temperature) && std::isfinite(top_p) &&
                           top_p > 0.0f && top_p <= 1.0f && candidates <= 1024;
  if (!well_formed) throw std::invalid_argument("sampling policy is outside the supported parameters");
  if (temperature > 0.0f && candidates > 1 && !has_rng)
    throw std::invalid_argument("stochastic sampling needs caller-owned random state");
}
template <typename T>
void sample(const ExecutionContext& context, TensorView<const T, 2> logits, TensorView<std::uint32_t, 1> tokens,
            TensorView<float, 1> probabilities, TensorView<unsigned char, 1> workspace, const SamplingPlan& plan,
            float temperature, float top_p, std::size_t top_k, curandState* states) {
  detail::require_bf16<T>();
  validate_sampling_policy(plan.vocabulary, temperature, top_p, top_k, states != nullptr);
  const bool greedy = temperature <= 0.0f || std::min(top_k, plan.vocabulary) == 1;
  if (!greedy) throw std::invalid_argument("only greedy sampling (top_k == 1 or temperature <= 0) is provided");
  if (probabilities.data != nullptr) throw std::invalid_argument("token probabilities are not provided");
  if (plan.vocabulary != logits.shape[1] || workspace.data == nullptr || workspace.numel() < plan.total_bytes)
    throw std::invalid_argument("sampling plan, logits and workspace do not fit together");
  const ei_context c = detail::native(context);
  detail::check(ei_sample_greedy_bf16(&c, detail::view(logits), detail::view(tokens), workspace.data, workspace.numel()));
}

}  // namespace op::cuda
