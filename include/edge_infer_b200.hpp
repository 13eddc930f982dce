// C++17 face of the runtime part of the C ABI in edge_infer_b200.h: Session (the verbs of the reference's
// Qwen3Session<T>) and SpeculativeDecoder. The direct operators live in operators/cuda/execution.hpp, under the
// reference's own names in namespace op::cuda; this header includes it and makes the same names reachable as
// edge_infer_b200::op::cuda for callers that prefer one namespace.
#pragma once

#include "operators/cuda/execution.hpp"

namespace edge_infer_b200 {

namespace op = ::op;
using ::TensorView;
using ::op::ArrayView;
using ::op::cuda::detail::check;

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
