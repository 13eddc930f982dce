// Greedy token selection, acceptance and KV commit, all on the device.
//
// The reference finds the greedy token by sorting the whole vocabulary once per row
// (operators/src/cuda/execution.cu:463-498) and then compares and rolls back on the host
// (runtime/src/speculative_decoder.cpp:208-223). Here a row's argmax is a single streaming pass
// with the reference's tie and NaN rules (NaN counts as -inf, equal values go to the lowest
// index - what its stable descending sort yields), and one block applies the acceptance rule and
// commits the context length, so the step needs no host synchronisation before its end.
#include "kernels.cuh"

namespace ei {
namespace {

constexpr int kArgmaxThreads = 256;

__device__ __forceinline__ void take_better(float& best, int& index, float value, int candidate) {
  if (value > best || (value == best && candidate < index)) {
    best = value;
    index = candidate;
  }
}

// kWide: partials laid out [row][parts] for any number of rows; otherwise [part][16] for at most 16 rows.
template <bool kWide>
__global__ void __launch_bounds__(kArgmaxThreads) argmax_partial_kernel(const bf16* logits, int vocab,
                                                                        size_t row_stride, float* best_value,
                                                                        int* best_index) {
  __shared__ float values[kArgmaxThreads / 32];
  __shared__ int indices[kArgmaxThreads / 32];
  grid_dependency_wait();
  const int row = blockIdx.y;
  const bf16* x = logits + size_t(row) * row_stride;
  // Contiguous slice per block; the slice boundaries are multiples of 8 elements.
  const int per_block = ((vocab + gridDim.x - 1) / gridDim.x + 7) & ~7;
  const int begin = min(vocab, int(blockIdx.x) * per_block), end = min(vocab, begin + per_block);
  float best = -INFINITY;
  int index = 0x7fffffff;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  if (aligned) {
    for (int i = begin + threadIdx.x * 8; i < end; i += kArgmaxThreads * 8) {
      if (i + 8 <= end) {
        const uint4 v = *reinterpret_cast<const uint4*>(x + i);
        const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float a = bf16_lo(words[j]), b = bf16_hi(words[j]);
          if (isnan(a)) a = -INFINITY;
          if (isnan(b)) b = -INFINITY;
          take_better(best, index, a, i + 2 * j);
          take_better(best, index, b, i + 2 * j + 1);
        }
      } else {
        for (int j = i; j < end; ++j) {
          float a = __bfloat162float(x[j]);
          if (isnan(a)) a = -INFINITY;
          take_better(best, index, a, j);
        }
      }
    }
  } else {
    for (int i = begin + threadIdx.x; i < end; i += kArgmaxThreads) {
      float a = __bfloat162float(x[i]);
      if (isnan(a)) a = -INFINITY;
      take_better(best, index, a, i);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, best, o);
    const int other_index = __shfl_xor_sync(0xffffffffu, index, o);
    take_better(best, index, other, other_index);
  }
  if ((threadIdx.x & 31) == 0) {
    values[threadIdx.x >> 5] = best;
    indices[threadIdx.x >> 5] = index;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kArgmaxThreads / 32; ++w) take_better(best, index, values[w], indices[w]);
    const size_t at = kWide ? size_t(row) * gridDim.x + blockIdx.x : size_t(blockIdx.x) * 16 + row;
    best_value[at] = best;
    best_index[at] = index;
  }
}

// Greedy acceptance (reference runtime/src/speculative_decoder.cpp:214-223): emit chosen[0..m] where m is the
// number of leading drafts with chosen[i] == inputs[i+1]; commit m+1 rows; the last emitted token is pending.
__device__ void accept_commit(const uint32_t* chosen, int rows, const uint32_t* step_tokens, Control* control,
                              int32_t* context_length, uint32_t* pending, ei_verify_result* result,
                              const TokenSink* sink = nullptr) {
  int emitted = 0;
  for (int i = 0; i < rows; ++i) {
    ++emitted;
    if (i + 1 >= rows || chosen[i] != step_tokens[i + 1]) break;
  }
  ei_verify_result local;
  for (int i = 0; i < 16; ++i) local.tokens[i] = i < rows ? chosen[i] : 0u;
  if (control) {
    const bool skipped = (control->status & 1) != 0;  // capacity guard tripped: nothing was written
    if (skipped) emitted = 0;
    if (sink && sink->tokens) {
      // Token i of this step is the one after the first context + 1 + i tokens of the sequence.
      for (int i = 0; i < emitted; ++i) {
        const long long at = (long long)control->context + 1 + i - sink->base;
        if (at >= 0 && at < sink->count) sink->tokens[at] = chosen[i];
      }
    }
    control->context += emitted;
    if (emitted) control->pending = chosen[emitted - 1];
    control->steps += 1;
    control->emitted_total += (unsigned long long)emitted;
    local.emitted = emitted;
    local.context = control->context;
    control->last = local;
    if (result) *result = local;
  } else {
    *context_length += emitted;
    *pending = chosen[emitted - 1];
    local.emitted = emitted;
    local.context = *context_length;
    *result = local;
  }
}

__global__ void accept_kernel(const uint32_t* inputs, const uint32_t* targets, int rows, int32_t* context_length,
                              uint32_t* pending, ei_verify_result* result) {
  if (threadIdx.x || blockIdx.x) return;
  uint32_t chosen[16];
  for (int i = 0; i < rows; ++i) chosen[i] = targets[i];
  accept_commit(chosen, rows, inputs, nullptr, context_length, pending, result);
}

// One block, one warp per row. Partials are laid out [part][16].
__global__ void __launch_bounds__(512) finalize_kernel(const float* best_value, const int* best_index, int parts,
                                                       int rows, uint32_t* targets, const uint32_t* step_tokens,
                                                       Control* control, int32_t* context_length,
                                                       uint32_t* pending, ei_verify_result* result,
                                                       const TokenSink* sink) {
  __shared__ uint32_t chosen[16];
  grid_dependency_wait();
  const int row = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (row < rows) {
    float best = -INFINITY;
    int index = 0x7fffffff;
    for (int part = lane; part < parts; part += 32)
      take_better(best, index, best_value[part * 16 + row], best_index[part * 16 + row]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_index = __shfl_xor_sync(0xffffffffu, index, o);
      take_better(best, index, other, other_index);
    }
    if (lane == 0) {
      // A row whose logits are all NaN / -inf keeps index 0, as the sort-based reference would.
      chosen[row] = index == 0x7fffffff ? 0u : uint32_t(index);
      if (targets) targets[row] = chosen[row];
    }
  }
  __syncthreads();
  if (threadIdx.x != 0 || !step_tokens) return;
  accept_commit(chosen, rows, step_tokens, control, context_length, pending, result, sink);
}

// Wide batch: one block per session, one warp per row of that session. Partials are laid out [row][parts].
__global__ void __launch_bounds__(512) finalize_wide_kernel(const float* best_value, const int* best_index, int parts,
                                                            int rows, uint32_t* targets, const uint32_t* step_tokens,
                                                            const SessionSlot* slots) {
  __shared__ uint32_t chosen[16];
  grid_dependency_wait();
  const int session = blockIdx.x, row = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (row < rows) {
    const size_t base = (size_t(session) * rows + row) * parts;
    float best = -INFINITY;
    int index = 0x7fffffff;
    for (int part = lane; part < parts; part += 32) take_better(best, index, best_value[base + part], best_index[base + part]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_index = __shfl_xor_sync(0xffffffffu, index, o);
      take_better(best, index, other, other_index);
    }
    if (lane == 0) {
      chosen[row] = index == 0x7fffffff ? 0u : uint32_t(index);
      targets[size_t(session) * rows + row] = chosen[row];
    }
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  accept_commit(chosen, rows, step_tokens + size_t(session) * rows, slots[session].control, nullptr, nullptr, nullptr);
}

__global__ void adopt_control_kernel(Control* mine, const Control* theirs) {
  if (threadIdx.x || blockIdx.x) return;
  mine->context = theirs->context;
  mine->pending = theirs->pending;
  mine->status |= theirs->status;
}

}  // namespace

int sample_partial_blocks(size_t vocabulary, int multiprocessors) {
  const size_t by_size = (vocabulary + 2047) / 2048;  // at least 2048 logits per block
  return int(std::max<size_t>(1, std::min<size_t>(by_size, size_t(multiprocessors))));
}

void launch_argmax_partials(const bf16* logits, size_t rows, size_t vocab, size_t row_stride, float* best_value,
                            int* best_index, int blocks, cudaStream_t stream, bool pdl) {
  launch(argmax_partial_kernel<false>, dim3(blocks, unsigned(rows)), dim3(kArgmaxThreads), 0, stream, pdl, logits,
         int(vocab), row_stride, best_value, best_index);
}

void launch_argmax_partials_wide(const bf16* logits, size_t rows, size_t vocab, size_t row_stride, float* best_value,
                                 int* best_index, int parts, cudaStream_t stream, bool pdl) {
  launch(argmax_partial_kernel<true>, dim3(parts, unsigned(rows)), dim3(kArgmaxThreads), 0, stream, pdl, logits,
         int(vocab), row_stride, best_value, best_index);
}

void launch_finalize_wide(const float* best_value, const int* best_index, int parts, int rows_per_session,
                          int sessions, uint32_t* targets, const uint32_t* step_tokens, const SessionSlot* slots,
                          cudaStream_t stream, bool pdl) {
  launch(finalize_wide_kernel, dim3(sessions), dim3(512), 0, stream, pdl, best_value, best_index, parts,
         rows_per_session, targets, step_tokens, slots);
}

void launch_accept(const uint32_t* inputs, const uint32_t* targets, int rows, int32_t* context_length,
                   uint32_t* pending, ei_verify_result* result, cudaStream_t stream) {
  accept_kernel<<<1, 32, 0, stream>>>(inputs, targets, rows, context_length, pending, result);
  check_launch();
}

void launch_finalize(const float* best_value, const int* best_index, int parts, int rows, uint32_t* targets,
                     const uint32_t* step_tokens, Control* control, int32_t* context_length, uint32_t* pending,
                     ei_verify_result* result, cudaStream_t stream, bool pdl, const TokenSink* sink) {
  launch(finalize_kernel, dim3(1), dim3(512), 0, stream, pdl, best_value, best_index, parts, rows, targets,
         step_tokens, control, context_length, pending, result, sink);
}

void launch_adopt_control(Control* mine, const Control* theirs, cudaStream_t stream) {
  adopt_control_kernel<<<1, 32, 0, stream>>>(mine, theirs);
  check_launch();
}

}  // namespace ei
