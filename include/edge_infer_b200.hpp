// C++17 face of the C ABI in edge_infer_b200.h: the reference's direct-operator API under its own names.
//
// The reference declares its operators as function templates in namespace op::cuda over the aggregates
// TensorView<T, Rank> / ArrayView<T> (operators/include/operators/cuda/execution.hpp:28-157,
// core/include/tensor_view.hpp:18-26, operators/include/operators/core/array_view.hpp:8-17) and reports errors
// with exceptions. This header gives the same names, argument order and exception types on top of
// libedge_infer_b200.so for T = __nv_bfloat16 (any 16-bit element type works: the library only sees pointers).
// The aggregates below have the reference's memory layout, so a caller that already holds the reference's
// views can reinterpret them; a caller without the reference's headers can use these as they are.
//
// Differences from the reference, all visible in the signatures: scratch is caller-owned (linear, awq_linear,
// attention_prefill and sample take it; sizes from the *_scratch_bytes functions), the execution context has no
// cuBLAS handle, and only the BF16 instantiations exist.
#pragma once

#include <array>
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "edge_infer_b200.h"

namespace edge_infer_b200 {

template <typename T, std::size_t Rank>
struct TensorView {
  T* data = nullptr;
  std::array<std::size_t, Rank> shape{};
  std::array<std::size_t, Rank> stride{};  // in elements
};
template <typename T>
struct ArrayView {
  T* data = nullptr;
  std::size_t size = 0;
};
static_assert(sizeof(TensorView<void*, 2>) == sizeof(ei_view2), "views cross the ABI by value");
static_assert(sizeof(ArrayView<void*>) == sizeof(ei_array), "views cross the ABI by value");

// Rethrows a failed call as the exception type the reference would have thrown.
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

namespace detail {
template <typename T>
inline void* erase(T* p) {
  return const_cast<void*>(static_cast<const void*>(p));
}
template <typename T>
inline ei_view1 view(const TensorView<T, 1>& v) {
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
inline ei_array view(const ArrayView<T>& v) {
  return ei_array{erase(v.data), v.size};
}
}  // namespace detail

namespace op::cuda {

using ExecutionContext = ei_context;          // execution.hpp:18-26
template <typename T>
using DenseLinearWeight = ei_dense_weight;    // execution.hpp:34-41
template <typename T>
using AwqLinearWeight = ei_awq_weight;        // execution.hpp:44-53

// execution.hpp:28-29. The handle argument is accepted and ignored.
inline ExecutionContext prepare_execution_context(void* /*handle*/, void* stream) {
  ExecutionContext context{};
  check(ei_prepare_execution_context(stream, &context));
  return context;
}

// execution.hpp:55-57: weight is the logical [in, out] view.
template <typename T>
DenseLinearWeight<T> prepare_dense(TensorView<const T, 2> weight, TensorView<const T, 1> bias = {}) {
  DenseLinearWeight<T> out{};
  check(ei_prepare_dense_bf16(detail::view(weight), detail::view(bias), &out));
  return out;
}
// execution.hpp:58-64.
template <typename T>
AwqLinearWeight<T> prepare_awq(TensorView<const std::int32_t, 2> qweight, TensorView<const T, 2> scales,
                               TensorView<const std::int32_t, 2> zeros, std::size_t group_size,
                               std::size_t input_features, TensorView<const T, 1> bias = {}) {
  AwqLinearWeight<T> out{};
  check(ei_prepare_awq_bf16(detail::view(qweight), detail::view(scales), detail::view(zeros), group_size,
                            input_features, detail::view(bias), &out));
  return out;
}

inline std::size_t linear_scratch_bytes(std::size_t rows, std::size_t input_features, std::size_t output_features) {
  return ei_linear_scratch_bytes(rows, input_features, output_features);
}
// execution.hpp:65-67 (+ scratch).
template <typename T>
void linear(const ExecutionContext& context, TensorView<const T, 2> input, const DenseLinearWeight<T>& weight,
            TensorView<T, 2> output, void* scratch = nullptr, std::size_t scratch_bytes = 0) {
  check(ei_linear_bf16(&context, detail::view(input), &weight, detail::view(output), scratch, scratch_bytes));
}
// execution.hpp:68-70 (+ scratch).
template <typename T>
void awq_linear(const ExecutionContext& context, TensorView<const T, 2> input, const AwqLinearWeight<T>& weight,
                TensorView<T, 2> output, void* scratch = nullptr, std::size_t scratch_bytes = 0) {
  check(ei_awq_linear_bf16(&context, detail::view(input), &weight, detail::view(output), scratch, scratch_bytes));
}
// No counterpart in the reference: gate and up projections with the SwiGLU product in one kernel.
template <typename T>
void awq_gate_up_silu(const ExecutionContext& context, TensorView<const T, 2> input,
                      const AwqLinearWeight<T>& gate_then_up, TensorView<T, 2> output) {
  check(ei_awq_gate_up_silu_bf16(&context, detail::view(input), &gate_then_up, detail::view(output)));
}

// execution.hpp:72-74.
template <typename T>
void add(const ExecutionContext& context, ArrayView<const T> a, ArrayView<const T> b, ArrayView<T> output) {
  check(ei_add_bf16(&context, detail::view(a), detail::view(b), detail::view(output)));
}
// direct.hpp:36-40.
template <typename T>
void silu_multiply(const ExecutionContext& context, ArrayView<const T> gate, ArrayView<const T> up,
                   ArrayView<T> output) {
  check(ei_silu_multiply_bf16(&context, detail::view(gate), detail::view(up), detail::view(output)));
}
// execution.hpp:85-90.
template <typename T>
void rms_norm(const ExecutionContext& context, ArrayView<const T> input, ArrayView<const T> weight,
              ArrayView<T> output, std::size_t rows, std::size_t features, float epsilon) {
  check(ei_rms_norm_bf16(&context, detail::view(input), detail::view(weight), detail::view(output), rows, features,
                         epsilon));
}
// execution.hpp:92-94.
template <typename T>
void gather(const ExecutionContext& context, TensorView<const std::uint32_t, 1> ids, TensorView<const T, 2> table,
            TensorView<T, 2> output) {
  check(ei_gather_bf16(&context, detail::view(ids), detail::view(table), detail::view(output)));
}
// execution.hpp:98-103.
template <typename T>
void rope_precomputed(const ExecutionContext& context, TensorView<T, 3> input, TensorView<const float, 2> cache,
                      std::size_t offset = 0, const std::size_t* offsets = nullptr, const int* pingpong = nullptr) {
  check(ei_rope_precomputed_bf16(&context, detail::view(input), detail::view(cache), offset, offsets, pingpong));
}
// execution.hpp:104-107.
template <typename T>
void store_kv(const ExecutionContext& context, TensorView<const T, 2> source, TensorView<T, 2> capacity,
              std::size_t offset, const std::size_t* device_offset = nullptr) {
  check(ei_store_kv_bf16(&context, detail::view(source), detail::view(capacity), offset, device_offset));
}

inline std::size_t attention_scratch_bytes(std::size_t q_rows, std::size_t query_heads, std::size_t head_dim,
                                           std::size_t kv_length) {
  return ei_attention_scratch_bytes(q_rows, query_heads, head_dim, kv_length);
}
// execution.hpp:117-122 (+ scratch).
template <typename T>
void attention_prefill(const ExecutionContext& context, TensorView<const T, 3> q, TensorView<const T, 3> k,
                       TensorView<const T, 3> v, TensorView<T, 3> output, std::size_t offset, void* scratch,
                       std::size_t scratch_bytes) {
  check(ei_attention_prefill_bf16(&context, detail::view(q), detail::view(k), detail::view(v), detail::view(output),
                                  offset, scratch, scratch_bytes));
}
// Captured-graph form: k / v describe the cache capacity, the offset is read from device memory at launch
// (the generalisation of attention_graph's device lengths, execution.hpp:123-130).
template <typename T>
void attention_verify(const ExecutionContext& context, TensorView<const T, 3> q, TensorView<const T, 3> k_capacity,
                      TensorView<const T, 3> v_capacity, TensorView<T, 3> output, const std::int32_t* device_offset,
                      void* scratch, std::size_t scratch_bytes) {
  check(ei_attention_verify_bf16(&context, detail::view(q), detail::view(k_capacity), detail::view(v_capacity),
                                 detail::view(output), device_offset, scratch, scratch_bytes));
}

inline std::size_t sample_scratch_bytes(std::size_t rows, std::size_t vocabulary) {
  return ei_sample_scratch_bytes(rows, vocabulary);
}
// execution.hpp:146-151 with top_k == 1: greedy token per row.
template <typename T>
void sample_greedy(const ExecutionContext& context, TensorView<const T, 2> logits,
                   TensorView<std::uint32_t, 1> tokens, void* scratch, std::size_t scratch_bytes) {
  check(ei_sample_greedy_bf16(&context, detail::view(logits), detail::view(tokens), scratch, scratch_bytes));
}

}  // namespace op::cuda

// Session with the verbs of Qwen3Session<T> (runtime/include/qwen3.hpp:32-59) plus the verify step of
// SpeculativeDecoder<T>::verify_greedy (runtime/src/speculative_decoder.cpp:200-224).
class Session {
 public:
  Session(ei_model* model, std::size_t capacity, bool graph) { check(ei_session_create(model, capacity, graph, &session_)); }
  ~Session() { ei_session_destroy(session_); }
  Session(const Session&) = delete;
  Session& operator=(const Session&) = delete;

  const void* prefill(const std::uint32_t* tokens, std::size_t rows, void* all_logits = nullptr) {
    const void* last = nullptr;
    check(ei_session_prefill(session_, tokens, rows, &last, all_logits));
    return last;  // borrowed BF16 [1, vocab], valid until the next operation
  }
  const void* decode(std::uint32_t token) {
    const void* logits = nullptr;
    check(ei_session_decode(session_, token, &logits));
    return logits;
  }
  // tokens = [pending, d1..dk]; returns the emitted count and the greedy token of every row.
  ei_verify_result verify(const std::uint32_t* tokens, std::size_t rows) {
    ei_verify_result result{};
    check(ei_session_verify(session_, tokens, rows, &result, nullptr));
    return result;
  }
  void reset() { check(ei_session_reset(session_)); }
  std::size_t context_size() const {
    std::size_t value = 0;
    check(ei_session_context_size(session_, &value));
    return value;
  }
  std::size_t context_capacity() const {
    std::size_t value = 0;
    check(ei_session_context_capacity(session_, &value));
    return value;
  }
  void synchronize() { check(ei_session_synchronize(session_)); }
  void* stream() const { return ei_session_stream(session_); }
  ei_session* native() const { return session_; }

 private:
  ei_session* session_ = nullptr;
};

// The reference's SpeculativeDecoder<T> (runtime/src/speculative_decoder.cpp:227-306) over a target and a draft
// Session: greedy only; rounds run on the device, the host synchronises in drain().
class SpeculativeDecoder {
 public:
  SpeculativeDecoder(Session& target, Session& draft, std::size_t drafts_per_round) {
    check(ei_speculative_create(target.native(), draft.native(), drafts_per_round, &decoder_));
  }
  ~SpeculativeDecoder() { ei_speculative_destroy(decoder_); }
  SpeculativeDecoder(const SpeculativeDecoder&) = delete;
  SpeculativeDecoder& operator=(const SpeculativeDecoder&) = delete;

  std::uint32_t prefill(const std::uint32_t* tokens, std::size_t rows) {
    std::uint32_t first = 0;
    check(ei_speculative_prefill(decoder_, tokens, rows, &first));
    return first;  // the first generated token
  }
  void enqueue(std::size_t rounds) { check(ei_speculative_enqueue(decoder_, rounds)); }
  // Waits; returns how many tokens have been generated since the prefill and copies up to `capacity` of them.
  std::size_t drain(std::uint32_t* tokens, std::size_t capacity) {
    std::size_t count = 0;
    check(ei_speculative_drain(decoder_, tokens, capacity, &count, nullptr));
    return count;
  }
  void truncate(std::size_t generated) { check(ei_speculative_truncate(decoder_, generated)); }

 private:
  ei_speculative* decoder_ = nullptr;
};

}  // namespace edge_infer_b200
