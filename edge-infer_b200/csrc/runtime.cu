// Prepared model and session: the runtime contract around the verify step.
//
// Mirrors the reference's split between immutable shared weights (Qwen3Model,
// runtime/include/models/qwen3_model.hpp) and one session that owns every mutable resource
// (Qwen3Session, runtime/include/qwen3.hpp:16-148, runtime/src/qwen3.cpp): stream, workspace,
// control block, managed KV cache, prefill / decode / reset, failure -> drain or poison.
// What differs is the step itself: one fused kernel sequence per layer, the context length,
// pending token, acceptance and KV commit kept on the device, the whole step replayed from a
// CUDA graph per row count, and a single host synchronisation at its end.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "abi_util.cuh"
#include "kernels.cuh"
#include "smallm_gemm.cuh"

namespace ei {
namespace {

constexpr size_t kAlign = 256;
constexpr int kMaxRows = 16;

size_t aligned(size_t bytes) { return (bytes + kAlign - 1) & ~(kAlign - 1); }

struct PreparedLinear {
  bool quantized = false;
  int in = 0, out = 0;
  const int32_t* qweight = nullptr;
  const bf16* scales = nullptr;
  const int32_t* zeros = nullptr;
  int padded_groups = 0, zero_stride = 0, group_size = 0;
  const bf16* dense = nullptr;  // [out, in]
  const bf16* bias = nullptr;
  size_t bytes = 0;  // weight bytes one call streams
};

__global__ void commit_rows_kernel(Control* control, int rows) {
  grid_dependency_wait();
  if (threadIdx.x || blockIdx.x) return;
  if (control->status & 1) return;
  control->context += rows;
}

// Copies the control block of every session of a wide batch into one array (read back with one copy).
__global__ void gather_controls_kernel(const SessionSlot* slots, int count, Control* out) {
  grid_dependency_wait();
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j < count) out[j] = *slots[j].control;
}

__global__ void silu_pair_rows_kernel(const bf16* gate_up, int rows, int ffn, bf16* out) {
  grid_dependency_wait();
  const int total = rows * ffn;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int row = i / ffn, n = i - row * ffn;
    out[i] = __float2bfloat16_rn(silu_multiply_value(__bfloat162float(gate_up[size_t(row) * 2 * ffn + n]),
                                                     __bfloat162float(gate_up[size_t(row) * 2 * ffn + ffn + n])));
  }
}

// The same over eight features per thread (ffn a multiple of 8, 16-byte aligned rows): the prompt path's form.
__global__ void silu_pair_rows_vec_kernel(const bf16* gate_up, int rows, int ffn, bf16* out) {
  grid_dependency_wait();
  const int per_row = ffn / 8;
  const long long total = (long long)rows * per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int row = int(i / per_row), n = int(i - (long long)row * per_row) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(gate_up + size_t(row) * 2 * ffn + n);
    const uint4 u = *reinterpret_cast<const uint4*>(gate_up + size_t(row) * 2 * ffn + ffn + n);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t packed[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      packed[j] = pack_bf16(silu_multiply_value(bf16_lo(gw[j]), bf16_lo(uw[j])),
                            silu_multiply_value(bf16_hi(gw[j]), bf16_hi(uw[j])));
    *reinterpret_cast<uint4*>(out + size_t(row) * ffn + n) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
}

// residual += projection (BF16, already rounded with bias), then RMSNorm: the unfused fallback of
// launch_residual_norm for shapes the streaming GEMM does not take.
__global__ void __launch_bounds__(512) residual_norm_bf16_kernel(const bf16* projection, int hidden, bf16* residual,
                                                                const bf16* norm_weight, float eps, bf16* normed) {
  __shared__ float shared[32];
  grid_dependency_wait();
  const int row = blockIdx.x;
  float sum = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float value = round_bf16(__bfloat162float(residual[size_t(row) * hidden + i]) +
                                   __bfloat162float(projection[size_t(row) * hidden + i]));
    residual[size_t(row) * hidden + i] = __float2bfloat16_rn(value);
    sum = fmaf(value, value, sum);
  }
  sum = warp_sum(sum);
  if ((threadIdx.x & 31) == 0) shared[threadIdx.x >> 5] = sum;
  __syncthreads();
  float total = 0.0f;
  for (int w = 0; w < int(blockDim.x >> 5); ++w) total += shared[w];
  const float inv = rsqrtf(__fdividef(total, float(hidden)) + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    normed[size_t(row) * hidden + i] = __float2bfloat16_rn(
        round_bf16(__bfloat162float(residual[size_t(row) * hidden + i]) * inv) * __bfloat162float(norm_weight[i]));
}

}  // namespace
}  // namespace ei

using namespace ei;

struct ei_model {
  ei_model_config config{};
  int device = 0;
  unsigned char* arena = nullptr;
  size_t arena_bytes = 0;
  const bf16* embedding = nullptr;
  const bf16* output_norm = nullptr;
  PreparedLinear lm_head;
  struct Layer {
    PreparedLinear qkv, o, gate_up, down;
    const bf16 *attention_norm = nullptr, *ffn_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr;
  };
  std::vector<Layer> layers;
  float* rope_table = nullptr;
  size_t weight_bytes = 0;
  int multiprocessors = 1;  // queried at creation
  size_t smem_limit = 227 * 1024;
  // Activations of a prompt segment (up to kPromptSegment rows through every projection at once): one set per
  // model, created by the first long prompt and lent, under the mutex, to one prefill at a time.
  struct PromptWorkspace {
    std::mutex mutex;
    unsigned char* arena = nullptr;
    size_t rows = 0;
    bf16 *residual = nullptr, *normed = nullptr, *qkv = nullptr, *attention = nullptr, *gate_up = nullptr,
         *act = nullptr, *projection = nullptr;
    float* partial = nullptr;         // FP32 sums of the o / down projections: [K slices][rows][hidden]
    size_t partial_bytes = 0;
    uint32_t *tokens = nullptr, *step_tokens = nullptr;
    uint32_t* host_tokens = nullptr;  // pinned
  } prompt;
  bool prompt_ready = false;  // every projection of every layer has a shape the prompt GEMM takes
};

namespace {

struct Source {
  const ei_named_tensor* dense = nullptr;
  const ei_named_tensor* qweight = nullptr;
  const ei_named_tensor* scales = nullptr;
  const ei_named_tensor* zeros = nullptr;
};

size_t element_bytes(int kind) { return kind == 0 || kind == 2 ? 2 : 4; }
size_t tensor_bytes(const ei_named_tensor& t) {
  size_t count = 1;
  for (int i = 0; i < t.rank; ++i) count *= t.shape[i];
  return count * element_bytes(t.kind);
}

struct Builder {
  ei_model& model;
  std::map<std::string, Source> sources;
  size_t offset = 0;

  const Source* find(const std::string& name) const {
    auto it = sources.find(name);
    return it == sources.end() ? nullptr : &it->second;
  }
  void* place(const void* data, size_t bytes) {
    void* dst = model.arena + offset;
    EI_CUDA(cudaMemcpy(dst, data, bytes, cudaMemcpyDefault));
    offset += aligned(bytes);
    return dst;
  }
  void* reserve(size_t bytes) {
    void* dst = model.arena + offset;
    offset += aligned(bytes);
    return dst;
  }
  const bf16* vector(const std::string& name, size_t width) {
    const Source* s = find(name);
    if (!s || !s->dense || s->dense->rank != 1 || s->dense->shape[0] != width)
      throw std::invalid_argument("Qwen3 weight shape mismatch: " + name);
    return static_cast<const bf16*>(place(s->dense->data, width * 2));
  }

  // Concatenates projections that share their input along the output axis (rows of the N-major
  // layout), so that one launch streams them all.
  PreparedLinear fused(const std::vector<std::string>& names, const std::vector<std::string>& bias_names, size_t in,
                       const std::vector<size_t>& outs) {
    const auto& c = model.config;
    PreparedLinear result;
    result.in = int(in);
    size_t total_out = 0;
    for (size_t o : outs) total_out += o;
    result.out = int(total_out);
    const Source* first = find(names[0]);
    if (!first) throw std::invalid_argument("Qwen3 weight not found: " + names[0]);
    result.quantized = c.quant_type == 1 && first->qweight;
    if (result.quantized) {
      if (in % size_t(c.group_size)) throw std::invalid_argument("Qwen3 AWQ input width must be divisible by group_size");
      const size_t groups = in / c.group_size;
      const size_t padded = first->scales ? first->scales->shape[1] : 0;
      const size_t zero_stride = (groups + 7) / 8, weight_stride = (in + 7) / 8;
      auto* qweight = static_cast<int32_t*>(reserve(total_out * weight_stride * 4));
      auto* scales = static_cast<bf16*>(reserve(total_out * padded * 2));
      auto* zeros = static_cast<int32_t*>(reserve(total_out * zero_stride * 4));
      size_t row = 0;
      for (size_t i = 0; i < names.size(); ++i) {
        const Source* s = find(names[i]);
        if (!s || !s->qweight || !s->scales || !s->zeros || s->qweight->shape[0] != outs[i] ||
            s->qweight->shape[1] != weight_stride || s->scales->shape[0] != outs[i] || s->scales->shape[1] != padded ||
            padded < groups || s->zeros->shape[0] != outs[i] || s->zeros->shape[1] != zero_stride)
          throw std::invalid_argument("Qwen3 AWQ weight shape mismatch: " + names[i]);
        EI_CUDA(cudaMemcpy(qweight + row * weight_stride, s->qweight->data, outs[i] * weight_stride * 4, cudaMemcpyDefault));
        EI_CUDA(cudaMemcpy(scales + row * padded, s->scales->data, outs[i] * padded * 2, cudaMemcpyDefault));
        EI_CUDA(cudaMemcpy(zeros + row * zero_stride, s->zeros->data, outs[i] * zero_stride * 4, cudaMemcpyDefault));
        row += outs[i];
      }
      result.qweight = qweight;
      result.scales = scales;
      result.zeros = zeros;
      result.padded_groups = int(padded);
      result.zero_stride = int(zero_stride);
      result.group_size = c.group_size;
      result.bytes = total_out * (in / 2 + groups * 2 + zero_stride * 4);
    } else {
      auto* dense = static_cast<bf16*>(reserve(total_out * in * 2));
      size_t row = 0;
      for (size_t i = 0; i < names.size(); ++i) {
        const Source* s = find(names[i]);
        if (!s || !s->dense || s->dense->rank != 2 || s->dense->shape[0] != outs[i] || s->dense->shape[1] != in)
          throw std::invalid_argument("Qwen3 weight shape mismatch: " + names[i]);
        EI_CUDA(cudaMemcpy(dense + row * in, s->dense->data, outs[i] * in * 2, cudaMemcpyDefault));
        row += outs[i];
      }
      result.dense = dense;
      result.bytes = total_out * in * 2;
    }
    bool any_bias = false;
    for (const auto& b : bias_names) any_bias = any_bias || (find(b) && find(b)->dense);
    if (any_bias) {
      auto* bias = static_cast<bf16*>(reserve(total_out * 2));
      EI_CUDA(cudaMemset(bias, 0, total_out * 2));
      size_t row = 0;
      for (size_t i = 0; i < names.size(); ++i) {
        const Source* s = find(bias_names[i]);
        if (s && s->dense) {
          if (s->dense->rank != 1 || s->dense->shape[0] != outs[i])
            throw std::invalid_argument("Qwen3 weight shape mismatch: " + bias_names[i]);
          EI_CUDA(cudaMemcpy(bias + row, s->dense->data, outs[i] * 2, cudaMemcpyDefault));
        }
        row += outs[i];
      }
      result.bias = bias;
      result.bytes += total_out * 2;
    }
    return result;
  }
};

void validate_config(const ei_model_config& c) {
  auto positive = [](uint64_t v) { return v >= 1 && v <= uint64_t(std::numeric_limits<int>::max()); };
  if (!positive(c.vocab_size) || !positive(c.n_layers) || !positive(c.n_heads) || !positive(c.n_kv_heads) ||
      !positive(c.hidden_size) || !positive(c.head_dim) || !positive(c.intermediate_size) ||
      !positive(c.max_position_embeddings))
    throw std::invalid_argument("Invalid Qwen3 config: extents must be positive and fit int");
  if (c.n_heads % c.n_kv_heads || c.head_dim % 2 || !std::isfinite(c.rms_norm_eps) || c.rms_norm_eps <= 0 ||
      !std::isfinite(c.rope_theta) || c.rope_theta <= 0)
    throw std::invalid_argument("Invalid Qwen3 attention or normalization config");
  if (c.hidden_size > 10240 || c.head_dim > 10240)
    throw std::invalid_argument("Qwen3 normalization width exceeds the supported kernel range");
  if (c.head_dim != 128)
    throw std::invalid_argument("The verify path supports head_dim 128 only");
  if (c.quant_type == 1 && c.group_size != 128)
    throw std::invalid_argument("The verify path supports AWQ group_size 128 only");
}

}  // namespace

struct ei_session {
  ei_model* model = nullptr;
  size_t capacity = 0;
  bool use_graph = false;
  cudaStream_t stream = nullptr;
  unsigned char* arena = nullptr;
  // workspace
  bf16 *residual = nullptr, *normed = nullptr, *qkv = nullptr, *attention = nullptr, *act = nullptr,
       *gate_up = nullptr, *projection = nullptr, *logits = nullptr;
  float* partial = nullptr;
  float* attention_scratch = nullptr;
  float* best_value = nullptr;
  int* best_index = nullptr;
  uint32_t *tokens = nullptr, *step_tokens = nullptr, *targets = nullptr;
  Control* control = nullptr;
  DraftSource* draft_source = nullptr;
  DraftSource draft_host{nullptr, 0, 0};
  TokenSink* token_sink = nullptr;  // device; all zero unless a speculative decoder owns the session
  bf16 *k_cache = nullptr, *v_cache = nullptr;
  // pinned host staging
  uint32_t* host_tokens = nullptr;
  Control* host_control = nullptr;
  // plans
  int attention_chunk = 64, attention_splits = 1;
  // state
  size_t context = 0;
  size_t bound = 0;  // upper bound of the context length after every step enqueued so far (full acceptance)
  bool history_ready = false, poisoned = false;
  int inject_launch = 0, inject_completion = 0;
  uint32_t inject_attention_polls = 0;  // the same hook for the next attention launch (its K / V tile copies)
  uint32_t inject_wait_polls = 0;  // test hook: the next weight-streaming GEMM gets this poll limit and a copy
                                   // expectation it cannot meet, so that its bounded waits run out
  size_t launches = 0, launches_per_step[kMaxRows + 1] = {};
  size_t prefill_target_row = 0;  // where in `targets` the last prefill left the greedy token of its last row
  // graphs: [kind][rows]; kind 0 verify (host tokens), 1 verify (device drafts), 2 decode (commit all)
  cudaGraphExec_t graphs[3][kMaxRows + 1] = {};
};

// A fixed set of sessions of one model that are verified together: their rows are stacked into one
// [sessions * rows, hidden] forward, so every weight is streamed once for all of them; attention, KV append
// and acceptance stay per session. The first session lends its workspace and stream.
struct ei_batch {
  std::vector<ei_session*> sessions;
  cudaGraphExec_t graphs[kMaxRows + 1] = {};  // by rows per session
  // Wide form (more than 16 stacked rows): the sessions' slots on the device, and buffers sized on first use
  // for sessions * rows stacked rows.
  SessionSlot* slots = nullptr;
  CUtensorMap* maps = nullptr;      // [sessions][2]: TMA descriptions of every session's K and V cache, all layers
  unsigned char* wide_arena = nullptr;
  size_t wide_rows = 0;
  bf16* logits = nullptr;           // [stacked rows, vocab]
  float* attention_scratch = nullptr;
  size_t scratch_stride = 0;        // floats per session
  float* best_value = nullptr;      // [stacked rows][kWideParts]
  int* best_index = nullptr;
  uint32_t* targets = nullptr;      // [stacked rows]
  Control* controls = nullptr;      // [sessions] gathered after a step
  Control* host_controls = nullptr; // pinned
};
constexpr int kWideParts = 8;       // argmax partials per row of the wide form
constexpr size_t kMaxBatchSessions = 1024;

// A target session and a draft session that generate together without host round trips: per round the draft
// session decodes drafts_per_round + 1 tokens, each from the token the previous step left on the device, the
// target session verifies [pending, d1..dk] in one forward, and the draft session adopts the target's context
// length and pending token. One device array holds the token of every position for both: the draft session
// writes its proposals into it, the target session reads them from it and overwrites them with what it emits.
struct ei_speculative {
  ei_session* target = nullptr;
  ei_session* draft = nullptr;
  size_t drafts = 0;             // k: drafts verified per round (rows = k + 1)
  size_t capacity = 0;           // of both sessions
  uint32_t* tokens = nullptr;    // device [capacity + kMaxRows + 1]: token of every absolute position
  size_t token_count = 0;
  cudaEvent_t drafted = nullptr, verified = nullptr;
  size_t prompt_rows = 0;
  size_t bound = 0;              // upper bound of the context length after everything enqueued so far
  bool started = false;
};

namespace {

enum StepKind { kVerifyHost = 0, kVerifyDevice = 1, kCommitAllWithHead = 2, kCommitAllNoHead = 3 };

void tick(ei_session& s) {
  ++s.launches;
  if (s.inject_launch > 0 && --s.inject_launch == 0)
    throw std::runtime_error("injected launch failure (test hook)");
}

void require_usable(const ei_session& s) {
  if (s.poisoned) throw PoisonedError("Session is unusable after failed CUDA stream completion");
}

void synchronize(ei_session& s) {
  cudaError_t status = cudaStreamSynchronize(s.stream);
  if (status == cudaSuccess && s.inject_completion) {
    s.inject_completion = 0;
    status = cudaErrorUnknown;  // reported after a real wait; the context itself is intact
  }
  if (status != cudaSuccess) {
    s.poisoned = true;
    throw std::runtime_error(std::string("CUDA stream completion failed: ") + cudaGetErrorString(status));
  }
}

// After a failed submission: drain this session's own stream; on success forget the history
// (partially written KV is never restored), on failure poison. Mirrors runtime/src/qwen3.cpp:142-161.
void drain_failed(ei_session& s) noexcept {
  if (s.poisoned) return;
  if (cudaStreamSynchronize(s.stream) != cudaSuccess) {
    s.poisoned = true;
    return;
  }
  Control zero{};
  if (cudaMemcpyAsync(s.control, &zero, sizeof(Control), cudaMemcpyHostToDevice, s.stream) != cudaSuccess ||
      cudaStreamSynchronize(s.stream) != cudaSuccess) {
    s.poisoned = true;
    return;
  }
  s.context = 0;
  s.bound = 0;
  s.history_ready = false;
}

void run_linear(ei_session& s, const PreparedLinear& w, const bf16* x, int rows, int epilogue, bf16* out,
                int out_stride, bool pdl, int* ksplit_out = nullptr) {
  const ei_model& m = *s.model;
  const bool aligned_ok = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  GemmPlan plan;
  const bool layout_ok = w.quantized ? w.group_size == 128 : true;
  if (aligned_ok && layout_ok)
    plan = plan_gemm(w.quantized, rows, w.out, w.in, epilogue, m.multiprocessors, m.smem_limit,
                     epilogue == kEpiPartial);
  if (!plan.fast) throw std::invalid_argument("internal: linear shape has no streaming plan");
  GemmParams p{};
  p.x = x;
  p.x_stride = w.in;
  p.M = rows;
  p.K = w.in;
  p.N = w.out;
  p.qweight = w.qweight;
  p.scales = w.scales;
  p.zeros = w.zeros;
  p.padded_groups = w.padded_groups;
  p.zero_stride = w.zero_stride;
  p.w = w.dense;
  p.ldw = w.in;
  p.bias = epilogue == kEpiPartial ? nullptr : w.bias;
  p.out = out;
  p.out_stride = out_stride;
  p.epilogue = epilogue;
  p.ksplit = plan.ksplit;
  p.partial = s.partial;
  p.best_value = s.best_value;
  p.best_index = s.best_index;
  p.status = &s.control->status;
  if (s.inject_wait_polls) {
    p.wait_limit = s.inject_wait_polls;
    p.fault_tx = 16;
    s.inject_wait_polls = 0;  // one launch only
  }
  tick(s);
  launch_gemm(plan, w.quantized, p, s.stream, pdl);
  if (ksplit_out) *ksplit_out = plan.ksplit;
  if (epilogue == kEpiArgmax && ksplit_out) *ksplit_out = plan.grid;
}

bool has_plan(const ei_session& s, const PreparedLinear& w, int rows, int epilogue) {
  const ei_model& m = *s.model;
  if (w.quantized && w.group_size != 128) return false;
  return plan_gemm(w.quantized, rows, w.out, w.in, epilogue, m.multiprocessors, m.smem_limit, epilogue == kEpiPartial).fast;
}

void run_generic(ei_session& s, const PreparedLinear& w, const bf16* x, int rows, bf16* out, bool pdl) {
  (void)pdl;
  const size_t count = size_t(rows) * w.out;
  const unsigned blocks = unsigned(std::min<size_t>((count + 255) / 256, size_t(s.model->multiprocessors) * 32));
  tick(s);
  if (w.quantized)
    awq_generic_kernel<<<blocks, 256, 0, s.stream>>>(x, w.in, w.qweight, w.scales, w.zeros, w.bias, out, w.out, rows,
                                                    w.out, w.in, w.group_size, w.padded_groups);
  else
    dense_generic_kernel<<<blocks, 256, 0, s.stream>>>(x, w.in, w.dense, 1, w.in, w.bias, out, w.out, rows, w.out, w.in);
  check_launch();
}

// projection -> residual add -> RMSNorm with `norm_weight`.
void run_projection_residual_norm(ei_session& s, const PreparedLinear& w, const bf16* x, int rows,
                                  const bf16* norm_weight, bool pdl) {
  const auto& c = s.model->config;
  if (has_plan(s, w, rows, kEpiPartial)) {
    int ksplit = 1;
    run_linear(s, w, x, rows, kEpiPartial, nullptr, 0, pdl, &ksplit);
    ResidualNormParams p{};
    p.partial = s.partial;
    p.ksplit = ksplit;
    p.rows = rows;
    p.hidden = int(c.hidden_size);
    p.bias = w.bias;
    p.residual = s.residual;
    p.norm_weight = norm_weight;
    p.eps = c.rms_norm_eps;
    p.normed = s.normed;
    tick(s);
    launch_residual_norm(p, s.stream, pdl);
  } else {
    run_generic(s, w, x, rows, s.projection, pdl);
    tick(s);
    launch(residual_norm_bf16_kernel, dim3(rows), dim3(512), 0, s.stream, pdl, (const bf16*)s.projection,
           int(c.hidden_size), s.residual, norm_weight, c.rms_norm_eps, s.normed);
  }
}

constexpr size_t kPromptSegment = 2048;  // rows of a long prompt that go through the layers together

bool prompt_linear_ok(const PreparedLinear& w) {
  if (w.quantized && (w.in / 8) % 4) return false;
  const void* weights = w.quantized ? static_cast<const void*>(w.qweight) : static_cast<const void*>(w.dense);
  return (reinterpret_cast<uintptr_t>(weights) & 15) == 0 &&
         prompt_gemm_eligible(w.quantized, w.group_size, w.out, w.in, nullptr, w.in, nullptr, w.out);
}

void ensure_prompt_workspace(ei_model& m) {
  auto& ws = m.prompt;
  if (ws.arena) return;
  const auto& c = m.config;
  const size_t rows = std::min<size_t>(kPromptSegment, c.max_position_embeddings);
  const size_t H = c.hidden_size, F = c.intermediate_size, Q = c.n_heads * 128;
  const size_t qkv_width = (c.n_heads + 2 * c.n_kv_heads) * 128;
  size_t offset = 0;
  auto take = [&](size_t bytes) {
    const size_t at = offset;
    offset += aligned(bytes);
    return at;
  };
  const size_t o_residual = take(rows * H * 2), o_normed = take(rows * H * 2), o_qkv = take(rows * qkv_width * 2);
  const size_t o_attention = take(rows * Q * 2), o_gate_up = take(rows * 2 * F * 2), o_act = take(rows * F * 2);
  const size_t o_projection = take(rows * H * 2), o_tokens = take(rows * 4), o_step = take(rows * 4);
  // Room for the FP32 sums of a full segment, or for 16 K slices of a short one.
  const size_t partial_bytes = std::max(rows, size_t(16) * std::min<size_t>(rows, 256)) * H * sizeof(float);
  const size_t o_partial = take(partial_bytes);
  unsigned char* base = nullptr;
  EI_CUDA(cudaMalloc(reinterpret_cast<void**>(&base), offset));
  if (cudaMallocHost(reinterpret_cast<void**>(&ws.host_tokens), rows * 4) != cudaSuccess) {
    cudaFree(base);
    throw std::runtime_error("Prompt staging buffer could not be allocated");
  }
  ws.residual = reinterpret_cast<bf16*>(base + o_residual);
  ws.normed = reinterpret_cast<bf16*>(base + o_normed);
  ws.qkv = reinterpret_cast<bf16*>(base + o_qkv);
  ws.attention = reinterpret_cast<bf16*>(base + o_attention);
  ws.gate_up = reinterpret_cast<bf16*>(base + o_gate_up);
  ws.act = reinterpret_cast<bf16*>(base + o_act);
  ws.projection = reinterpret_cast<bf16*>(base + o_projection);
  ws.tokens = reinterpret_cast<uint32_t*>(base + o_tokens);
  ws.step_tokens = reinterpret_cast<uint32_t*>(base + o_step);
  ws.partial = reinterpret_cast<float*>(base + o_partial);
  ws.partial_bytes = partial_bytes;
  ws.rows = rows;
  ws.arena = base;
}

// ksplit == 0: BF16 output with bias; otherwise FP32 partial sums of `ksplit` K slices in the workspace.
void run_prompt_linear(ei_session& s, const PreparedLinear& w, const bf16* x, int rows, bf16* out, bool pdl,
                       int ksplit = 0) {
  GemmParams p{};
  p.epilogue = ksplit ? kEpiPartial : kEpiStore;
  p.ksplit = ksplit;
  p.partial = s.model->prompt.partial;
  p.x = x;
  p.x_stride = w.in;
  p.M = rows;
  p.K = w.in;
  p.N = w.out;
  p.qweight = w.qweight;
  p.scales = w.scales;
  p.zeros = w.zeros;
  p.padded_groups = w.padded_groups;
  p.zero_stride = w.zero_stride;
  p.w = w.dense;
  p.ldw = w.in;
  p.bias = w.bias;
  p.out = out;
  p.out_stride = w.out;
  p.status = &s.control->status;
  if (s.inject_wait_polls) {
    p.wait_limit = s.inject_wait_polls;
    p.fault_tx = 16;
    s.inject_wait_polls = 0;  // one launch only
  }
  tick(s);
  launch_prompt_gemm(w.quantized, p, s.stream, pdl);
}

// A projection with a BF16 output over all rows of a segment. Few output tiles (the q|k|v projection of a short
// segment) would leave most SMs idle: K is then split over blocks that leave FP32 sums, and a second kernel adds
// them, joins the bias and rounds once.
void run_prompt_linear_store(ei_session& s, const PreparedLinear& w, const bf16* x, int rows, bf16* out, bool pdl) {
  ei_model& m = *s.model;
  auto& ws = m.prompt;
  const int ksplit = w.out % 4 == 0 ? prompt_gemm_ksplit(rows, w.out, w.in, m.multiprocessors, ws.partial_bytes) : 1;
  if (ksplit < 2) {
    run_prompt_linear(s, w, x, rows, out, pdl);
    return;
  }
  run_prompt_linear(s, w, x, rows, nullptr, pdl, ksplit);
  tick(s);
  launch(splitk_store_kernel, dim3(std::min(m.multiprocessors * 8, (rows * w.out + 255) / 256)), dim3(256), 0, s.stream,
         pdl, (const float*)ws.partial, ksplit, rows, w.out, w.bias, out, w.out);
}

// projection -> residual add -> RMSNorm over all rows of a segment: the projection leaves FP32 sums (K split
// over blocks when few token tiles would leave SMs idle) that the residual + norm kernel finishes, as in the
// verify step.
void run_prompt_projection_residual_norm(ei_session& s, const PreparedLinear& w, const bf16* x, int rows,
                                         const bf16* norm_weight, bool pdl) {
  ei_model& m = *s.model;
  auto& ws = m.prompt;
  const auto& c = m.config;
  if (w.out % 4 == 0 && size_t(rows) * w.out * sizeof(float) <= ws.partial_bytes) {
    const int ksplit = prompt_gemm_ksplit(rows, w.out, w.in, m.multiprocessors, ws.partial_bytes);
    run_prompt_linear(s, w, x, rows, nullptr, pdl, ksplit);
    ResidualNormParams p{};
    p.partial = ws.partial;
    p.ksplit = ksplit;
    p.rows = rows;
    p.hidden = int(c.hidden_size);
    p.bias = w.bias;
    p.residual = ws.residual;
    p.norm_weight = norm_weight;
    p.eps = c.rms_norm_eps;
    p.normed = ws.normed;
    tick(s);
    launch_residual_norm(p, s.stream, pdl);
  } else {
    run_prompt_linear(s, w, x, rows, ws.projection, pdl);
    tick(s);
    launch(residual_norm_bf16_kernel, dim3(rows), dim3(512), 0, s.stream, pdl, (const bf16*)ws.projection,
           int(c.hidden_size), ws.residual, norm_weight, c.rms_norm_eps, ws.normed);
  }
}

// One forward of `rows` prompt tokens (any number up to the workspace's) at the device-side context length:
// every projection is one tcgen05 GEMM over all rows, attention one launch over all rows. All rows are
// committed; with `head`, the last row alone goes through the vocabulary head (logits in s.logits, its greedy
// token in s.targets[0]).
void enqueue_prompt_segment(ei_session& s, int rows, bool head) {
  ei_model& m = *s.model;
  auto& ws = m.prompt;
  const auto& c = m.config;
  const int heads = int(c.n_heads), kv_heads = int(c.n_kv_heads), hidden = int(c.hidden_size), ffn = int(c.intermediate_size);
  const int qkv_width = (heads + 2 * kv_heads) * 128, kv_width = kv_heads * 128;
  const bool pdl = true;

  EmbedParams e{};
  e.tokens = ws.tokens;
  e.control = s.control;
  e.step_tokens = ws.step_tokens;
  e.table = m.embedding;
  e.vocab = int(c.vocab_size);
  e.hidden = hidden;
  e.rows = rows;
  e.capacity = int(s.capacity);
  e.norm_weight = m.layers[0].attention_norm;
  e.eps = c.rms_norm_eps;
  e.residual = ws.residual;
  e.normed = ws.normed;
  tick(s);
  launch_embed_norm(e, s.stream, false);

  const int elementwise_blocks = m.multiprocessors * 8;
  for (size_t layer = 0; layer < m.layers.size(); ++layer) {
    const auto& L = m.layers[layer];
    run_prompt_linear_store(s, L.qkv, ws.normed, rows, ws.qkv, pdl);
    QkvParams q{};
    q.qkv = ws.qkv;
    q.rows = rows;
    q.heads = heads;
    q.kv_heads = kv_heads;
    q.qkv_stride = qkv_width;
    q.q_norm = c.qk_norm ? L.q_norm : nullptr;
    q.k_norm = c.qk_norm ? L.k_norm : nullptr;
    q.eps = c.rms_norm_eps;
    q.rope_table = m.rope_table;
    q.max_positions = int(c.max_position_embeddings);
    q.control = s.control;
    q.capacity = int(s.capacity);
    q.k_cache = s.k_cache + layer * s.capacity * kv_width;
    q.v_cache = s.v_cache + layer * s.capacity * kv_width;
    tick(s);
    launch_qk_norm_rope_store(q, s.stream, pdl);

    AttentionParams a{};
    a.q = ws.qkv;
    a.q_stride = qkv_width;
    a.k = q.k_cache;
    a.v = q.v_cache;
    a.kv_stride = kv_width;
    a.rows = rows;
    a.heads = heads;
    a.kv_heads = kv_heads;
    a.capacity = int(s.capacity);
    a.device_offset = &s.control->context;
    a.status = &s.control->status;
    a.out = ws.attention;
    a.out_stride = heads * 128;
    tick(s);
    launch_prompt_attention(a, s.stream, pdl);

    run_prompt_projection_residual_norm(s, L.o, ws.attention, rows, L.ffn_norm, pdl);

    run_prompt_linear(s, L.gate_up, ws.normed, rows, ws.gate_up, pdl);
    tick(s);
    if (ffn % 8 == 0)
      launch(silu_pair_rows_vec_kernel, dim3(elementwise_blocks), dim3(256), 0, s.stream, pdl, (const bf16*)ws.gate_up,
             rows, ffn, ws.act);
    else
      launch(silu_pair_rows_kernel, dim3(elementwise_blocks), dim3(256), 0, s.stream, pdl, (const bf16*)ws.gate_up, rows,
             ffn, ws.act);
    const bf16* next_norm = layer + 1 < m.layers.size() ? m.layers[layer + 1].attention_norm : m.output_norm;
    run_prompt_projection_residual_norm(s, L.down, ws.act, rows, next_norm, pdl);
  }

  if (head) {
    const bf16* last = ws.normed + size_t(rows - 1) * hidden;
    int parts = 0;
    if (has_plan(s, m.lm_head, 1, kEpiArgmax)) {
      run_linear(s, m.lm_head, last, 1, kEpiArgmax, s.logits, int(c.vocab_size), pdl, &parts);
    } else {
      run_generic(s, m.lm_head, last, 1, s.logits, pdl);
      parts = std::min(kSampleMaxParts, sample_partial_blocks(c.vocab_size, m.multiprocessors));
      tick(s);
      launch_argmax_partials(s.logits, 1, c.vocab_size, c.vocab_size, s.best_value, s.best_index, parts, s.stream, pdl);
    }
    tick(s);
    launch_finalize(s.best_value, s.best_index, parts, 1, s.targets, nullptr, nullptr, nullptr, nullptr, nullptr,
                    s.stream, pdl);
  }
  tick(s);
  launch(commit_rows_kernel, dim3(1), dim3(32), 0, s.stream, pdl, s.control, rows);
}

// Enqueues one forward of `rows` tokens at the device-side context length.
void enqueue_step(ei_session& s, int rows, StepKind kind, bf16* logits_out) {
  const ei_model& m = *s.model;
  const auto& c = m.config;
  const int heads = int(c.n_heads), kv_heads = int(c.n_kv_heads), hidden = int(c.hidden_size), ffn = int(c.intermediate_size);
  const int qkv_width = (heads + 2 * kv_heads) * 128, kv_width = kv_heads * 128;
  const bool pdl = true;
  const size_t before = s.launches;

  EmbedParams e{};
  e.tokens = kind == kVerifyDevice ? nullptr : s.tokens;
  e.source = kind == kVerifyDevice ? s.draft_source : nullptr;
  e.control = s.control;
  e.step_tokens = s.step_tokens;
  e.table = m.embedding;
  e.vocab = int(c.vocab_size);
  e.hidden = hidden;
  e.rows = rows;
  e.capacity = int(s.capacity);
  e.norm_weight = m.layers[0].attention_norm;
  e.eps = c.rms_norm_eps;
  e.residual = s.residual;
  e.normed = s.normed;
  tick(s);
  launch_embed_norm(e, s.stream, false);

  for (size_t layer = 0; layer < m.layers.size(); ++layer) {
    const auto& L = m.layers[layer];
    if (has_plan(s, L.qkv, rows, kEpiStore))
      run_linear(s, L.qkv, s.normed, rows, kEpiStore, s.qkv, qkv_width, pdl);
    else
      run_generic(s, L.qkv, s.normed, rows, s.qkv, pdl);
    QkvParams q{};
    q.qkv = s.qkv;
    q.rows = rows;
    q.heads = heads;
    q.kv_heads = kv_heads;
    q.qkv_stride = qkv_width;
    q.q_norm = c.qk_norm ? L.q_norm : nullptr;
    q.k_norm = c.qk_norm ? L.k_norm : nullptr;
    q.eps = c.rms_norm_eps;
    q.rope_table = m.rope_table;
    q.max_positions = int(c.max_position_embeddings);
    q.control = s.control;
    q.capacity = int(s.capacity);
    q.k_cache = s.k_cache + layer * s.capacity * kv_width;
    q.v_cache = s.v_cache + layer * s.capacity * kv_width;
    tick(s);
    launch_qk_norm_rope_store(q, s.stream, pdl);

    AttentionParams a{};
    a.q = s.qkv;
    a.q_stride = qkv_width;
    a.k = q.k_cache;
    a.v = q.v_cache;
    a.kv_stride = kv_width;
    a.rows = rows;
    a.heads = heads;
    a.kv_heads = kv_heads;
    a.capacity = int(s.capacity);
    a.device_offset = &s.control->context;
    a.status = &s.control->status;
    a.chunk = s.attention_chunk;
    a.max_splits = s.attention_splits;
    a.scratch = s.attention_scratch;
    a.out = s.attention;
    a.out_stride = heads * 128;
    if (s.inject_attention_polls) {
      a.wait_limit = s.inject_attention_polls;
      a.fault_tx = 16;
      s.inject_attention_polls = 0;  // one launch only
    }
    tick(s);
    tick(s);
    launch_verify_attention(a, s.stream, pdl);

    run_projection_residual_norm(s, L.o, s.attention, rows, L.ffn_norm, pdl);

    if (has_plan(s, L.gate_up, rows, kEpiSiluPair)) {
      run_linear(s, L.gate_up, s.normed, rows, kEpiSiluPair, s.act, ffn, pdl);
    } else {
      if (has_plan(s, L.gate_up, rows, kEpiStore))
        run_linear(s, L.gate_up, s.normed, rows, kEpiStore, s.gate_up, 2 * ffn, pdl);
      else
        run_generic(s, L.gate_up, s.normed, rows, s.gate_up, pdl);
      tick(s);
      launch(silu_pair_rows_kernel, dim3(std::min(1024, (rows * ffn + 255) / 256)), dim3(256), 0, s.stream, pdl,
             (const bf16*)s.gate_up, rows, ffn, s.act);
    }
    const bf16* next_norm = layer + 1 < m.layers.size() ? m.layers[layer + 1].attention_norm : m.output_norm;
    run_projection_residual_norm(s, L.down, s.act, rows, next_norm, pdl);
  }

  if (kind == kCommitAllNoHead) {
    tick(s);
    launch(commit_rows_kernel, dim3(1), dim3(32), 0, s.stream, pdl, s.control, rows);
  } else {
    bf16* logits = logits_out ? logits_out : s.logits;
    int parts = 0;
    if (has_plan(s, m.lm_head, rows, kEpiArgmax)) {
      run_linear(s, m.lm_head, s.normed, rows, kEpiArgmax, logits, int(c.vocab_size), pdl, &parts);
    } else {
      run_generic(s, m.lm_head, s.normed, rows, logits, pdl);
      parts = std::min(kSampleMaxParts, sample_partial_blocks(c.vocab_size, m.multiprocessors));
      tick(s);
      launch_argmax_partials(logits, rows, c.vocab_size, c.vocab_size, s.best_value, s.best_index, parts, s.stream, pdl);
    }
    tick(s);
    if (kind == kCommitAllWithHead) {
      launch_finalize(s.best_value, s.best_index, parts, rows, s.targets, nullptr, nullptr, nullptr, nullptr, nullptr,
                      s.stream, pdl);
      tick(s);
      launch(commit_rows_kernel, dim3(1), dim3(32), 0, s.stream, pdl, s.control, rows);
    } else {
      launch_finalize(s.best_value, s.best_index, parts, rows, s.targets, s.step_tokens, s.control, nullptr, nullptr,
                      nullptr, s.stream, pdl, s.token_sink);
    }
  }
  s.launches_per_step[rows] = s.launches - before;
}

// Runs a step either eagerly or by replaying its graph (captured on first use after an eager warm run).
void submit_step(ei_session& s, int rows, StepKind kind) {
  if (!s.use_graph || kind == kCommitAllNoHead || s.inject_wait_polls || s.inject_attention_polls) {
    enqueue_step(s, rows, kind, nullptr);
    return;
  }
  cudaGraphExec_t& exec = s.graphs[int(kind)][rows];
  if (!exec) {
    // Warm run outside capture: sets kernel attributes, loads modules, and does real work.
    enqueue_step(s, rows, kind, nullptr);
    // Capture a second, identical submission without executing it.
    const int saved_inject = s.inject_launch;
    s.inject_launch = 0;
    cudaGraph_t graph = nullptr;
    EI_CUDA(cudaStreamBeginCapture(s.stream, cudaStreamCaptureModeThreadLocal));
    try {
      enqueue_step(s, rows, kind, nullptr);
    } catch (...) {
      cudaStreamEndCapture(s.stream, &graph);
      if (graph) cudaGraphDestroy(graph);
      s.inject_launch = saved_inject;
      throw;
    }
    s.inject_launch = saved_inject;
    EI_CUDA(cudaStreamEndCapture(s.stream, &graph));
    const cudaError_t status = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    EI_CUDA(status);
    return;  // the warm run already executed this step
  }
  tick(s);
  EI_CUDA(cudaGraphLaunch(exec, s.stream));
}

// One verify step of every session of the batch, `rows` tokens each, on the leader's stream and workspace.
void enqueue_batch_step(ei_batch& batch, int rows) {
  ei_session& lead = *batch.sessions[0];
  const ei_model& m = *lead.model;
  const auto& c = m.config;
  const int count = int(batch.sessions.size()), total = count * rows;
  const int heads = int(c.n_heads), kv_heads = int(c.n_kv_heads), hidden = int(c.hidden_size), ffn = int(c.intermediate_size);
  const int qkv_width = (heads + 2 * kv_heads) * 128, kv_width = kv_heads * 128;
  const bool pdl = true;

  for (int j = 0; j < count; ++j) {
    ei_session& s = *batch.sessions[j];
    EmbedParams e{};
    e.tokens = lead.tokens + j * rows;
    e.control = s.control;
    e.step_tokens = lead.step_tokens + j * rows;
    e.table = m.embedding;
    e.vocab = int(c.vocab_size);
    e.hidden = hidden;
    e.rows = rows;
    e.capacity = int(s.capacity);
    e.norm_weight = m.layers[0].attention_norm;
    e.eps = c.rms_norm_eps;
    e.residual = lead.residual + size_t(j) * rows * hidden;
    e.normed = lead.normed + size_t(j) * rows * hidden;
    tick(lead);
    launch_embed_norm(e, lead.stream, false);
  }
  const size_t scratch_floats = attention_scratch_bytes(rows, heads, lead.capacity) / sizeof(float);
  for (size_t layer = 0; layer < m.layers.size(); ++layer) {
    const auto& L = m.layers[layer];
    if (has_plan(lead, L.qkv, total, kEpiStore))
      run_linear(lead, L.qkv, lead.normed, total, kEpiStore, lead.qkv, qkv_width, pdl);
    else
      run_generic(lead, L.qkv, lead.normed, total, lead.qkv, pdl);
    for (int j = 0; j < count; ++j) {
      ei_session& s = *batch.sessions[j];
      QkvParams q{};
      q.qkv = lead.qkv + size_t(j) * rows * qkv_width;
      q.rows = rows;
      q.heads = heads;
      q.kv_heads = kv_heads;
      q.qkv_stride = qkv_width;
      q.q_norm = c.qk_norm ? L.q_norm : nullptr;
      q.k_norm = c.qk_norm ? L.k_norm : nullptr;
      q.eps = c.rms_norm_eps;
      q.rope_table = m.rope_table;
      q.max_positions = int(c.max_position_embeddings);
      q.control = s.control;
      q.capacity = int(s.capacity);
      q.k_cache = s.k_cache + layer * s.capacity * kv_width;
      q.v_cache = s.v_cache + layer * s.capacity * kv_width;
      tick(lead);
      launch_qk_norm_rope_store(q, lead.stream, pdl);
    }
    for (int j = 0; j < count; ++j) {
      ei_session& s = *batch.sessions[j];
      AttentionParams a{};
      a.q = lead.qkv + size_t(j) * rows * qkv_width;
      a.q_stride = qkv_width;
      a.k = s.k_cache + layer * s.capacity * kv_width;
      a.v = s.v_cache + layer * s.capacity * kv_width;
      a.kv_stride = kv_width;
      a.rows = rows;
      a.heads = heads;
      a.kv_heads = kv_heads;
      a.capacity = int(s.capacity);
      a.device_offset = &s.control->context;
      a.status = &s.control->status;
      a.chunk = s.attention_chunk;
      a.max_splits = s.attention_splits;
      a.scratch = lead.attention_scratch + size_t(j) * scratch_floats;
      a.out = lead.attention + size_t(j) * rows * heads * 128;
      a.out_stride = heads * 128;
      tick(lead);
      tick(lead);
      launch_verify_attention(a, lead.stream, pdl);
    }
    run_projection_residual_norm(lead, L.o, lead.attention, total, L.ffn_norm, pdl);
    if (has_plan(lead, L.gate_up, total, kEpiSiluPair)) {
      run_linear(lead, L.gate_up, lead.normed, total, kEpiSiluPair, lead.act, ffn, pdl);
    } else {
      if (has_plan(lead, L.gate_up, total, kEpiStore))
        run_linear(lead, L.gate_up, lead.normed, total, kEpiStore, lead.gate_up, 2 * ffn, pdl);
      else
        run_generic(lead, L.gate_up, lead.normed, total, lead.gate_up, pdl);
      tick(lead);
      launch(silu_pair_rows_kernel, dim3(std::min(1024, (total * ffn + 255) / 256)), dim3(256), 0, lead.stream, pdl,
             (const bf16*)lead.gate_up, total, ffn, lead.act);
    }
    const bf16* next_norm = layer + 1 < m.layers.size() ? m.layers[layer + 1].attention_norm : m.output_norm;
    run_projection_residual_norm(lead, L.down, lead.act, total, next_norm, pdl);
  }
  int parts = 0;
  if (has_plan(lead, m.lm_head, total, kEpiArgmax)) {
    run_linear(lead, m.lm_head, lead.normed, total, kEpiArgmax, lead.logits, int(c.vocab_size), pdl, &parts);
  } else {
    run_generic(lead, m.lm_head, lead.normed, total, lead.logits, pdl);
    parts = std::min(kSampleMaxParts, sample_partial_blocks(c.vocab_size, m.multiprocessors));
    tick(lead);
    launch_argmax_partials(lead.logits, total, c.vocab_size, c.vocab_size, lead.best_value, lead.best_index, parts,
                           lead.stream, pdl);
  }
  // Greedy token, acceptance and commit per session, on its own rows of the per-block partials.
  for (int j = 0; j < count; ++j) {
    ei_session& s = *batch.sessions[j];
    tick(lead);
    launch_finalize(lead.best_value + j * rows, lead.best_index + j * rows, parts, rows, lead.targets + j * rows,
                    lead.step_tokens + j * rows, s.control, nullptr, nullptr, nullptr, lead.stream, pdl);
  }
}

void ensure_wide_buffers(ei_batch& batch, size_t rows) {
  ei_session& lead = *batch.sessions[0];
  const auto& c = lead.model->config;
  const size_t count = batch.sessions.size(), total = count * rows;
  if (batch.wide_arena && batch.wide_rows >= total) return;
  if (batch.wide_arena) {
    EI_CUDA(cudaStreamSynchronize(lead.stream));
    cudaFree(batch.wide_arena);
    batch.wide_arena = nullptr;
  }
  // Split partials for the sessions' full capacity and 16 rows each, so that a later call with more rows per
  // session only regrows the row-sized buffers.
  const size_t scratch_stride = attention_scratch_bytes(kMaxRows, c.n_heads, lead.capacity) / sizeof(float);
  size_t offset = 0;
  auto take = [&](size_t bytes) {
    const size_t at = offset;
    offset += aligned(bytes);
    return at;
  };
  const size_t o_logits = take(total * c.vocab_size * 2), o_scratch = take(count * scratch_stride * sizeof(float));
  const size_t o_value = take(total * kWideParts * sizeof(float)), o_index = take(total * kWideParts * sizeof(int));
  const size_t o_targets = take(total * 4), o_controls = take(count * sizeof(Control));
  EI_CUDA(cudaMalloc(reinterpret_cast<void**>(&batch.wide_arena), offset));
  unsigned char* base = batch.wide_arena;
  batch.logits = reinterpret_cast<bf16*>(base + o_logits);
  batch.attention_scratch = reinterpret_cast<float*>(base + o_scratch);
  batch.scratch_stride = scratch_stride;
  batch.best_value = reinterpret_cast<float*>(base + o_value);
  batch.best_index = reinterpret_cast<int*>(base + o_index);
  batch.targets = reinterpret_cast<uint32_t*>(base + o_targets);
  batch.controls = reinterpret_cast<Control*>(base + o_controls);
  batch.wide_rows = total;
}

// One verify step of every session of the batch in the wide form: the stacked rows (any number up to the
// prompt workspace's) go through every projection as one tcgen05 GEMM, so the weights are read once for all
// sessions; embedding, norm / RoPE / KV append, attention, greedy choice, acceptance and commit run as single
// launches that find each row's session in the slot array. Runs on the leader's stream and the model's prompt
// workspace.
void enqueue_wide_batch_step(ei_batch& batch, int rows) {
  ei_session& lead = *batch.sessions[0];
  ei_model& m = *lead.model;
  auto& ws = m.prompt;
  const auto& c = m.config;
  const int count = int(batch.sessions.size()), total = count * rows;
  const int heads = int(c.n_heads), kv_heads = int(c.n_kv_heads), hidden = int(c.hidden_size), ffn = int(c.intermediate_size);
  const int qkv_width = (heads + 2 * kv_heads) * 128, kv_width = kv_heads * 128;
  const bool pdl = true;

  EmbedParams e{};
  e.tokens = ws.tokens;
  e.step_tokens = ws.step_tokens;
  e.table = m.embedding;
  e.vocab = int(c.vocab_size);
  e.hidden = hidden;
  e.rows = total;
  e.norm_weight = m.layers[0].attention_norm;
  e.eps = c.rms_norm_eps;
  e.residual = ws.residual;
  e.normed = ws.normed;
  e.slots = batch.slots;
  e.rows_per_session = rows;
  tick(lead);
  launch_embed_norm(e, lead.stream, false);

  for (size_t layer = 0; layer < m.layers.size(); ++layer) {
    const auto& L = m.layers[layer];
    run_prompt_linear_store(lead, L.qkv, ws.normed, total, ws.qkv, pdl);
    QkvParams q{};
    q.qkv = ws.qkv;
    q.rows = total;
    q.heads = heads;
    q.kv_heads = kv_heads;
    q.qkv_stride = qkv_width;
    q.q_norm = c.qk_norm ? L.q_norm : nullptr;
    q.k_norm = c.qk_norm ? L.k_norm : nullptr;
    q.eps = c.rms_norm_eps;
    q.rope_table = m.rope_table;
    q.max_positions = int(c.max_position_embeddings);
    q.slots = batch.slots;
    q.rows_per_session = rows;
    q.layer = int(layer);
    tick(lead);
    launch_qk_norm_rope_store(q, lead.stream, pdl);

    AttentionParams a{};
    a.q = ws.qkv;
    a.q_stride = qkv_width;
    a.kv_stride = kv_width;
    a.rows = rows;
    a.heads = heads;
    a.kv_heads = kv_heads;
    // Many sessions fill the GPU by themselves: longer chunks than the single-session step's (fewer partials to
    // write and merge, the per-block set-up paid once per eight tiles), still at most 64 splits.
    a.chunk = std::max(512, lead.attention_chunk);
    a.max_splits = int((lead.capacity + a.chunk - 1) / a.chunk);
    a.scratch = batch.attention_scratch;
    a.scratch_stride = batch.scratch_stride;
    a.out = ws.attention;
    a.out_stride = heads * 128;
    a.slots = batch.slots;
    a.maps = batch.maps;
    a.status = &lead.control->status;
    a.sessions = count;
    a.layer = int(layer);
    tick(lead);
    tick(lead);
    launch_verify_attention(a, lead.stream, pdl);

    run_prompt_projection_residual_norm(lead, L.o, ws.attention, total, L.ffn_norm, pdl);
    run_prompt_linear(lead, L.gate_up, ws.normed, total, ws.gate_up, pdl);
    tick(lead);
    if (ffn % 8 == 0)
      launch(silu_pair_rows_vec_kernel, dim3(m.multiprocessors * 8), dim3(256), 0, lead.stream, pdl,
             (const bf16*)ws.gate_up, total, ffn, ws.act);
    else
      launch(silu_pair_rows_kernel, dim3(m.multiprocessors * 8), dim3(256), 0, lead.stream, pdl,
             (const bf16*)ws.gate_up, total, ffn, ws.act);
    const bf16* next_norm = layer + 1 < m.layers.size() ? m.layers[layer + 1].attention_norm : m.output_norm;
    run_prompt_projection_residual_norm(lead, L.down, ws.act, total, next_norm, pdl);
  }
  run_prompt_linear(lead, m.lm_head, ws.normed, total, batch.logits, pdl);
  tick(lead);
  launch_argmax_partials_wide(batch.logits, total, c.vocab_size, c.vocab_size, batch.best_value, batch.best_index,
                              kWideParts, lead.stream, pdl);
  tick(lead);
  launch_finalize_wide(batch.best_value, batch.best_index, kWideParts, rows, count, batch.targets, ws.step_tokens,
                       batch.slots, lead.stream, pdl);
  tick(lead);
  launch(gather_controls_kernel, dim3((count + 127) / 128), dim3(128), 0, lead.stream, pdl,
         (const SessionSlot*)batch.slots, count, batch.controls);
}

void submit_batch_step(ei_batch& batch, int rows) {
  ei_session& lead = *batch.sessions[0];
  if (!lead.use_graph) {
    enqueue_batch_step(batch, rows);
    return;
  }
  cudaGraphExec_t& exec = batch.graphs[rows];
  if (!exec) {
    enqueue_batch_step(batch, rows);  // warm run: real work, kernel attributes, first-use set-up
    cudaGraph_t graph = nullptr;
    EI_CUDA(cudaStreamBeginCapture(lead.stream, cudaStreamCaptureModeThreadLocal));
    try {
      enqueue_batch_step(batch, rows);
    } catch (...) {
      cudaStreamEndCapture(lead.stream, &graph);
      if (graph) cudaGraphDestroy(graph);
      throw;
    }
    EI_CUDA(cudaStreamEndCapture(lead.stream, &graph));
    const cudaError_t status = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    EI_CUDA(status);
    return;  // the warm run already executed this step
  }
  tick(lead);
  EI_CUDA(cudaGraphLaunch(exec, lead.stream));
}

void read_control(ei_session& s) {
  EI_CUDA(cudaMemcpyAsync(s.host_control, s.control, sizeof(Control), cudaMemcpyDeviceToHost, s.stream));
  synchronize(s);
  s.context = size_t(s.host_control->context);
  s.bound = s.context;
}

// A step that would pass the capacity refuses itself on the device (status bit 0): it and every step chained
// behind it wrote nothing, so the history stays valid. Thrown outside the drain-and-forget path.
struct CapacityRefusal : LengthError {
  using LengthError::LengthError;
};

void check_status(ei_session& s) {
  if (s.host_control->status) {
    const int status = s.host_control->status;
    // Clear the flag on the device.
    const int zero = 0;
    EI_CUDA(cudaMemcpyAsync(&s.control->status, &zero, sizeof(int), cudaMemcpyHostToDevice, s.stream));
    synchronize(s);
    if (status & 2) throw std::invalid_argument("Session token id exceeds vocabulary");
    if (status & 4) throw std::runtime_error("A bounded wait inside a kernel gave up");
    throw CapacityRefusal("Session context capacity exhausted");
  }
}

}  // namespace

extern "C" {

ei_status ei_model_create(const ei_model_config* config, const ei_named_tensor* tensors, size_t count, ei_model** out) {
  return guarded([&] {
    if (!config || !tensors || !count || !out) throw std::invalid_argument("Model creation requires a config and tensors");
    validate_config(*config);
    auto model = std::make_unique<ei_model>();
    model->config = *config;
    EI_CUDA(cudaGetDevice(&model->device));
    int value = 0;
    EI_CUDA(cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, model->device));
    model->multiprocessors = value;
    EI_CUDA(cudaDeviceGetAttribute(&value, cudaDevAttrMaxSharedMemoryPerBlockOptin, model->device));
    model->smem_limit = size_t(value);
    Builder builder{*model};
    size_t bytes = 0;
    for (size_t i = 0; i < count; ++i) {
      const auto& t = tensors[i];
      if (!t.name || !t.data || t.rank < 1 || t.rank > 2 || t.kind < 0 || t.kind > 3)
        throw std::invalid_argument("Empty or malformed Qwen3 weight");
      Source& s = builder.sources[t.name];
      const ei_named_tensor** slot = t.kind == 0 ? &s.dense : t.kind == 1 ? &s.qweight : t.kind == 2 ? &s.scales : &s.zeros;
      if (*slot) throw std::invalid_argument(std::string("Duplicate Qwen3 parameter: ") + t.name);
      *slot = &t;
      bytes += aligned(tensor_bytes(t)) + kAlign;
    }
    const auto& c = model->config;
    const size_t H = c.hidden_size, V = c.vocab_size, F = c.intermediate_size;
    const size_t qw = c.n_heads * c.head_dim, kvw = c.n_kv_heads * c.head_dim;
    bytes += c.n_layers * (aligned((qw + 2 * kvw) * 2) + aligned(2 * F * 2) + 8 * kAlign);  // fused bias vectors
    const size_t rope_bytes = c.max_position_embeddings * c.head_dim * sizeof(float);
    bytes += aligned(rope_bytes);
    EI_CUDA(cudaMalloc(reinterpret_cast<void**>(&model->arena), bytes));
    model->arena_bytes = bytes;
    try {
      const Source* embedding = builder.find("token_embeddings.weight");
      if (!embedding || !embedding->dense || embedding->dense->rank != 2 || embedding->dense->shape[0] != V ||
          embedding->dense->shape[1] != H)
        throw std::invalid_argument("Qwen3 weight shape mismatch: token_embeddings.weight");
      model->embedding = static_cast<const bf16*>(builder.place(embedding->dense->data, V * H * 2));
      model->output_norm = builder.vector("rms_out_w", H);
      if (builder.find("lm_head")) {
        model->lm_head = builder.fused({"lm_head"}, {"lm_head.bias"}, H, {V});
      } else {  // tied embeddings
        model->lm_head.in = int(H);
        model->lm_head.out = int(V);
        model->lm_head.dense = model->embedding;
        model->lm_head.bytes = V * H * 2;
      }
      model->weight_bytes = model->lm_head.bytes;
      model->layers.resize(c.n_layers);
      for (size_t i = 0; i < c.n_layers; ++i) {
        const std::string n = std::to_string(i), prefix = "layers." + n + ".";
        auto& L = model->layers[i];
        L.attention_norm = builder.vector("rms_att_w" + n, H);
        L.ffn_norm = builder.vector("rms_ffn_w" + n, H);
        if (c.qk_norm) {
          L.q_norm = builder.vector("q_norm" + n, c.head_dim);
          L.k_norm = builder.vector("k_norm" + n, c.head_dim);
        }
        L.qkv = builder.fused({"wq" + n, "wk" + n, "wv" + n},
                              {prefix + "self_attn.q_proj.bias", prefix + "self_attn.k_proj.bias",
                               prefix + "self_attn.v_proj.bias"},
                              H, {qw, kvw, kvw});
        L.o = builder.fused({"wo" + n}, {prefix + "self_attn.o_proj.bias"}, qw, {H});
        L.gate_up = builder.fused({"w_gate" + n, "w_up" + n}, {prefix + "mlp.gate_proj.bias", prefix + "mlp.up_proj.bias"},
                                  H, {F, F});
        L.down = builder.fused({"w_down" + n}, {prefix + "mlp.down_proj.bias"}, F, {H});
        model->weight_bytes += L.qkv.bytes + L.o.bytes + L.gate_up.bytes + L.down.bytes;
      }
      std::vector<float> table(c.max_position_embeddings * c.head_dim);
      if (ei_build_rope_table(table.data(), c.max_position_embeddings, c.head_dim, c.rope_theta) != EI_OK)
        throw std::invalid_argument(g_last_error);
      model->rope_table = static_cast<float*>(builder.place(table.data(), rope_bytes));
      model->prompt_ready = true;
      for (const auto& L : model->layers)
        model->prompt_ready = model->prompt_ready && prompt_linear_ok(L.qkv) && prompt_linear_ok(L.o) &&
                              prompt_linear_ok(L.gate_up) && prompt_linear_ok(L.down);
      EI_CUDA(cudaDeviceSynchronize());
    } catch (...) {
      cudaFree(model->arena);
      throw;
    }
    *out = model.release();
  });
}

void ei_model_destroy(ei_model* model) {
  if (!model) return;
  int previous = model->device;
  cudaGetDevice(&previous);
  if (previous != model->device) cudaSetDevice(model->device);
  cudaFree(model->arena);
  if (model->prompt.arena) cudaFree(model->prompt.arena);
  if (model->prompt.host_tokens) cudaFreeHost(model->prompt.host_tokens);
  if (previous != model->device) cudaSetDevice(previous);
  delete model;
}

ei_status ei_model_config_of(const ei_model* model, ei_model_config* out) {
  return guarded([&] {
    if (!model || !out) throw std::invalid_argument("model is null");
    *out = model->config;
  });
}

size_t ei_model_weight_bytes(const ei_model* model) { return model ? model->weight_bytes : 0; }

ei_status ei_session_create(ei_model* model, size_t capacity, int graph, ei_session** out) {
  return guarded([&] {
    if (!model || !out || !capacity || capacity > model->config.max_position_embeddings)
      throw std::invalid_argument("Session capacity must be positive and within the model limit");
    int device = 0;
    EI_CUDA(cudaGetDevice(&device));
    if (device != model->device) throw std::invalid_argument("Session must be created on its model CUDA device");
    const auto& c = model->config;
    auto s = std::make_unique<ei_session>();
    s->model = model;
    s->capacity = capacity;
    s->use_graph = graph != 0;
    const size_t H = c.hidden_size, V = c.vocab_size, F = c.intermediate_size;
    const size_t qkv_width = (c.n_heads + 2 * c.n_kv_heads) * 128, kv_width = c.n_kv_heads * 128;
    s->attention_chunk = attention_chunk_for(capacity);
    s->attention_splits = int((capacity + s->attention_chunk - 1) / s->attention_chunk);
    size_t offset = 0;
    auto take = [&](size_t bytes) {
      const size_t at = offset;
      offset += aligned(bytes);
      return at;
    };
    const size_t o_residual = take(kMaxRows * H * 2), o_normed = take(kMaxRows * H * 2);
    const size_t o_qkv = take(kMaxRows * qkv_width * 2), o_attention = take(kMaxRows * c.n_heads * 128 * 2);
    const size_t o_act = take(kMaxRows * F * 2), o_gate_up = take(kMaxRows * 2 * F * 2);
    const size_t o_projection = take(kMaxRows * H * 2), o_logits = take(kMaxRows * V * 2);
    const size_t o_partial = take(size_t(16) * kMaxRows * H * sizeof(float));
    const size_t o_scratch = take(attention_scratch_bytes(kMaxRows, c.n_heads, capacity));
    const size_t o_best_value = take(size_t(kSampleMaxParts) * 16 * sizeof(float));
    const size_t o_best_index = take(size_t(kSampleMaxParts) * 16 * sizeof(int));
    const size_t o_tokens = take(kMaxRows * 4), o_step = take(kMaxRows * 4), o_targets = take(kMaxRows * 4);
    const size_t o_control = take(sizeof(Control)), o_source = take(sizeof(DraftSource));
    const size_t o_sink = take(sizeof(TokenSink));
    const size_t kv_bytes = c.n_layers * capacity * kv_width * 2;
    const size_t o_k = take(kv_bytes), o_v = take(kv_bytes);
    EI_CUDA(cudaMalloc(reinterpret_cast<void**>(&s->arena), offset));
    unsigned char* base = s->arena;
    s->residual = reinterpret_cast<bf16*>(base + o_residual);
    s->normed = reinterpret_cast<bf16*>(base + o_normed);
    s->qkv = reinterpret_cast<bf16*>(base + o_qkv);
    s->attention = reinterpret_cast<bf16*>(base + o_attention);
    s->act = reinterpret_cast<bf16*>(base + o_act);
    s->gate_up = reinterpret_cast<bf16*>(base + o_gate_up);
    s->projection = reinterpret_cast<bf16*>(base + o_projection);
    s->logits = reinterpret_cast<bf16*>(base + o_logits);
    s->partial = reinterpret_cast<float*>(base + o_partial);
    s->attention_scratch = reinterpret_cast<float*>(base + o_scratch);
    s->best_value = reinterpret_cast<float*>(base + o_best_value);
    s->best_index = reinterpret_cast<int*>(base + o_best_index);
    s->tokens = reinterpret_cast<uint32_t*>(base + o_tokens);
    s->step_tokens = reinterpret_cast<uint32_t*>(base + o_step);
    s->targets = reinterpret_cast<uint32_t*>(base + o_targets);
    s->control = reinterpret_cast<Control*>(base + o_control);
    s->draft_source = reinterpret_cast<DraftSource*>(base + o_source);
    s->token_sink = reinterpret_cast<TokenSink*>(base + o_sink);
    s->k_cache = reinterpret_cast<bf16*>(base + o_k);
    s->v_cache = reinterpret_cast<bf16*>(base + o_v);
    try {
      EI_CUDA(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking));
      EI_CUDA(cudaMallocHost(reinterpret_cast<void**>(&s->host_tokens), kMaxRows * 4));
      EI_CUDA(cudaMallocHost(reinterpret_cast<void**>(&s->host_control), sizeof(Control)));
      EI_CUDA(cudaMemsetAsync(s->control, 0, sizeof(Control), s->stream));
      EI_CUDA(cudaMemsetAsync(s->draft_source, 0, sizeof(DraftSource), s->stream));
      EI_CUDA(cudaMemsetAsync(s->token_sink, 0, sizeof(TokenSink), s->stream));
      EI_CUDA(cudaStreamSynchronize(s->stream));
    } catch (...) {
      ei_session_destroy(s.release());
      throw;
    }
    *out = s.release();
  });
}

void ei_session_destroy(ei_session* s) {
  if (!s) return;
  int previous = s->model->device;
  cudaGetDevice(&previous);
  if (previous != s->model->device) cudaSetDevice(s->model->device);
  if (s->stream) cudaStreamSynchronize(s->stream);
  for (auto& kind : s->graphs)
    for (auto& exec : kind)
      if (exec) cudaGraphExecDestroy(exec);
  if (s->host_tokens) cudaFreeHost(s->host_tokens);
  if (s->host_control) cudaFreeHost(s->host_control);
  if (s->arena) cudaFree(s->arena);
  if (s->stream) cudaStreamDestroy(s->stream);
  if (previous != s->model->device) cudaSetDevice(previous);
  delete s;
}

static void require_device(const ei_session& s) {
  int device = 0;
  EI_CUDA(cudaGetDevice(&device));
  if (device != s.model->device) throw std::invalid_argument("Session CUDA device changed");
}

ei_status ei_session_prefill(ei_session* session, const uint32_t* host_tokens, size_t rows, const void** last_logits,
                             void* all_logits) {
  return guarded([&] {
    if (!session) throw std::invalid_argument("session is null");
    ei_session& s = *session;
    require_usable(s);
    if (!host_tokens || !rows) throw std::invalid_argument("Host input requires tokens; decode takes one token");
    if (rows > s.capacity) throw LengthError("Host input exceeds session capacity");
    require_device(s);
    const size_t vocab = s.model->config.vocab_size;
    for (size_t i = 0; i < rows; ++i)
      if (host_tokens[i] >= vocab) throw std::invalid_argument("Token exceeds vocabulary");
    // Long prompts go through the layers in segments of up to kPromptSegment rows, on the model's prompt
    // workspace, which this call holds until its stream has drained.
    const bool wide = rows > size_t(kPromptMinRows) && !all_logits && s.model->prompt_ready;
    std::unique_lock<std::mutex> workspace(s.model->prompt.mutex, std::defer_lock);
    if (wide) workspace.lock();
    try {
      // A prefill replaces the history (the reference resizes the managed cache to `rows`).
      EI_CUDA(cudaMemsetAsync(s.control, 0, sizeof(Control), s.stream));
      s.context = 0;
      s.bound = 0;
      s.history_ready = false;
      s.prefill_target_row = wide ? 0 : (rows - 1) % kMaxRows;
      if (wide) {
        ensure_prompt_workspace(*s.model);
        auto& ws = s.model->prompt;
        for (size_t first = 0; first < rows; first += ws.rows) {
          const size_t count = std::min(ws.rows, rows - first);
          synchronize(s);  // the pinned staging buffer is reused by every segment
          std::memcpy(ws.host_tokens, host_tokens + first, count * 4);
          EI_CUDA(cudaMemcpyAsync(ws.tokens, ws.host_tokens, count * 4, cudaMemcpyHostToDevice, s.stream));
          enqueue_prompt_segment(s, int(count), first + count >= rows);
        }
      }
      for (size_t first = wide ? rows : 0; first < rows; first += kMaxRows) {
        const int chunk = int(std::min<size_t>(kMaxRows, rows - first));
        const bool last = first + chunk >= rows;
        synchronize(s);  // the pinned staging buffer is reused by every chunk
        std::memcpy(s.host_tokens, host_tokens + first, size_t(chunk) * 4);
        EI_CUDA(cudaMemcpyAsync(s.tokens, s.host_tokens, size_t(chunk) * 4, cudaMemcpyHostToDevice, s.stream));
        if (all_logits) {
          enqueue_step(s, chunk, kCommitAllWithHead, static_cast<bf16*>(all_logits) + first * vocab);
          if (last)
            EI_CUDA(cudaMemcpyAsync(s.logits, static_cast<bf16*>(all_logits) + (rows - 1) * vocab, vocab * 2,
                                    cudaMemcpyDeviceToDevice, s.stream));
        } else if (last) {
          enqueue_step(s, chunk, kCommitAllWithHead, nullptr);
          if (chunk > 1)
            EI_CUDA(cudaMemcpyAsync(s.logits, s.logits + size_t(chunk - 1) * vocab, vocab * 2, cudaMemcpyDeviceToDevice,
                                    s.stream));
        } else {
          enqueue_step(s, chunk, kCommitAllNoHead, nullptr);
        }
      }
      read_control(s);
      check_status(s);
    } catch (const CapacityRefusal&) {
      throw;  // refused on the device before any write: the history stays
    } catch (...) {
      drain_failed(s);
      throw;
    }
    s.history_ready = true;
    if (last_logits) *last_logits = s.logits;
  });
}

ei_status ei_session_decode(ei_session* session, uint32_t token, const void** logits) {
  return guarded([&] {
    if (!session) throw std::invalid_argument("session is null");
    ei_session& s = *session;
    require_usable(s);
    if (!s.history_ready) throw std::logic_error("Decode requires successful prefill");
    if (s.context >= s.capacity) throw LengthError("Host input exceeds session capacity");
    require_device(s);
    if (token >= s.model->config.vocab_size) throw std::invalid_argument("Token exceeds vocabulary");
    try {
      s.host_tokens[0] = token;
      EI_CUDA(cudaMemcpyAsync(s.tokens, s.host_tokens, 4, cudaMemcpyHostToDevice, s.stream));
      submit_step(s, 1, kCommitAllWithHead);
      read_control(s);
      check_status(s);
    } catch (const CapacityRefusal&) {
      throw;  // refused on the device before any write: the history stays
    } catch (...) {
      drain_failed(s);
      throw;
    }
    if (logits) *logits = s.logits;
  });
}

ei_status ei_session_verify(ei_session* session, const uint32_t* host_tokens, size_t rows, ei_verify_result* result,
                            const void** logits) {
  return guarded([&] {
    if (!session) throw std::invalid_argument("session is null");
    ei_session& s = *session;
    require_usable(s);
    if (!host_tokens || !rows || rows > kMaxRows || !result)
      throw std::invalid_argument("Verify takes 1..16 tokens [pending, drafts...] and a result");
    if (!s.history_ready) throw std::logic_error("Verify requires successful prefill");
    if (s.context + rows > s.capacity) throw LengthError("Verify rows exceed session capacity");
    require_device(s);
    const size_t vocab = s.model->config.vocab_size;
    for (size_t i = 0; i < rows; ++i)
      if (host_tokens[i] >= vocab) throw std::invalid_argument("Token exceeds vocabulary");
    try {
      std::memcpy(s.host_tokens, host_tokens, rows * 4);
      EI_CUDA(cudaMemcpyAsync(s.tokens, s.host_tokens, rows * 4, cudaMemcpyHostToDevice, s.stream));
      submit_step(s, int(rows), kVerifyHost);
      read_control(s);
      check_status(s);
    } catch (const CapacityRefusal&) {
      throw;  // refused on the device before any write: the history stays
    } catch (...) {
      drain_failed(s);
      throw;
    }
    *result = s.host_control->last;
    if (logits) *logits = s.logits;
  });
}

ei_status ei_batch_create(ei_session* const* sessions, size_t count, ei_batch** out) {
  return guarded([&] {
    if (!sessions || !count || count > kMaxBatchSessions || !out)
      throw std::invalid_argument("A batch takes 1..1024 sessions");
    auto batch = std::make_unique<ei_batch>();
    for (size_t j = 0; j < count; ++j) {
      ei_session* s = sessions[j];
      if (!s) throw std::invalid_argument("session is null");
      if (s->model != sessions[0]->model) throw std::invalid_argument("Batched sessions must share one model");
      if (s->capacity != sessions[0]->capacity)
        throw std::invalid_argument("Batched sessions must have the same context capacity");
      for (size_t i = 0; i < j; ++i)
        if (sessions[i] == s) throw std::invalid_argument("A session appears twice in the batch");
      batch->sessions.push_back(s);
    }
    require_device(*sessions[0]);
    std::vector<SessionSlot> slots(count);
    for (size_t j = 0; j < count; ++j)
      slots[j] = SessionSlot{sessions[j]->control, sessions[j]->k_cache, sessions[j]->v_cache, int(sessions[j]->capacity), 0};
    const auto& c = sessions[0]->model->config;
    const size_t kv_width = c.n_kv_heads * 128;
    std::vector<CUtensorMap> maps(2 * count);
    for (size_t j = 0; j < count; ++j) {
      const ei_session& s = *sessions[j];
      encode_kv_map(&maps[2 * j], s.k_cache, s.capacity, kv_width, int(c.n_kv_heads), c.n_layers, s.capacity * kv_width);
      encode_kv_map(&maps[2 * j + 1], s.v_cache, s.capacity, kv_width, int(c.n_kv_heads), c.n_layers, s.capacity * kv_width);
    }
    EI_CUDA(cudaMalloc(reinterpret_cast<void**>(&batch->slots), count * sizeof(SessionSlot)));
    if (cudaMalloc(reinterpret_cast<void**>(&batch->maps), maps.size() * sizeof(CUtensorMap)) != cudaSuccess ||
        cudaMemcpy(batch->maps, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemcpy(batch->slots, slots.data(), count * sizeof(SessionSlot), cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMallocHost(reinterpret_cast<void**>(&batch->host_controls), count * sizeof(Control)) != cudaSuccess) {
      cudaFree(batch->slots);
      if (batch->maps) cudaFree(batch->maps);
      throw std::runtime_error("Batch state could not be placed on the device");
    }
    *out = batch.release();
  });
}

void ei_batch_destroy(ei_batch* batch) {
  if (!batch) return;
  for (auto& exec : batch->graphs)
    if (exec) cudaGraphExecDestroy(exec);
  if (!batch->sessions.empty()) cudaStreamSynchronize(batch->sessions[0]->stream);
  if (batch->slots) cudaFree(batch->slots);
  if (batch->maps) cudaFree(batch->maps);
  if (batch->wide_arena) cudaFree(batch->wide_arena);
  if (batch->host_controls) cudaFreeHost(batch->host_controls);
  delete batch;
}

ei_status ei_batch_verify(ei_batch* batch, const uint32_t* host_tokens, size_t rows, ei_verify_result* results) {
  return guarded([&] {
    if (!batch) throw std::invalid_argument("batch is null");
    const size_t count = batch->sessions.size();
    ei_session& lead = *batch->sessions[0];
    const bool wide = rows * count > kMaxRows;
    const size_t room = lead.model->prompt_ready && prompt_linear_ok(lead.model->lm_head)
                            ? std::min<size_t>(kPromptSegment, lead.model->config.max_position_embeddings) : kMaxRows;
    if (!host_tokens || !results || !rows || rows > kMaxRows || rows * count > room)
      throw std::invalid_argument(
          "A batched verify takes 1..16 rows per session, one result per session, and sessions * rows <= 16 stacked "
          "rows - or <= 2048 for models whose projections the prompt GEMM takes");
    require_device(lead);
    const size_t vocab = lead.model->config.vocab_size;
    for (ei_session* s : batch->sessions) {
      require_usable(*s);
      if (!s->history_ready) throw std::logic_error("Verify requires successful prefill");
      if (s->context + rows > s->capacity) throw LengthError("Verify rows exceed session capacity");
    }
    for (size_t i = 0; i < rows * count; ++i)
      if (host_tokens[i] >= vocab) throw std::invalid_argument("Token exceeds vocabulary");
    // The wide form borrows the model's prompt workspace until the leader's stream has drained.
    std::unique_lock<std::mutex> workspace(lead.model->prompt.mutex, std::defer_lock);
    if (wide) workspace.lock();
    try {
      // Work queued on the other sessions' own streams must be done before the shared step touches their state.
      for (size_t j = 1; j < count; ++j) synchronize(*batch->sessions[j]);
      if (wide) {
        ensure_prompt_workspace(*lead.model);
        ensure_wide_buffers(*batch, rows);
        auto& ws = lead.model->prompt;
        synchronize(lead);  // the pinned staging buffers are reused by every call
        std::memcpy(ws.host_tokens, host_tokens, rows * count * 4);
        EI_CUDA(cudaMemcpyAsync(ws.tokens, ws.host_tokens, rows * count * 4, cudaMemcpyHostToDevice, lead.stream));
        enqueue_wide_batch_step(*batch, int(rows));
        EI_CUDA(cudaMemcpyAsync(batch->host_controls, batch->controls, count * sizeof(Control), cudaMemcpyDeviceToHost,
                                lead.stream));
        synchronize(lead);
        for (size_t j = 0; j < count; ++j) *batch->sessions[j]->host_control = batch->host_controls[j];
      } else {
        std::memcpy(lead.host_tokens, host_tokens, rows * count * 4);
        EI_CUDA(cudaMemcpyAsync(lead.tokens, lead.host_tokens, rows * count * 4, cudaMemcpyHostToDevice, lead.stream));
        submit_batch_step(*batch, int(rows));
        for (ei_session* s : batch->sessions)
          EI_CUDA(cudaMemcpyAsync(s->host_control, s->control, sizeof(Control), cudaMemcpyDeviceToHost, lead.stream));
        synchronize(lead);
      }
      for (ei_session* s : batch->sessions) s->context = size_t(s->host_control->context);
      for (ei_session* s : batch->sessions)
        if (s->host_control->status) {
          const int status = s->host_control->status, zero = 0;
          EI_CUDA(cudaMemcpyAsync(&s->control->status, &zero, sizeof(int), cudaMemcpyHostToDevice, lead.stream));
          synchronize(lead);
          if (status & 2) throw std::invalid_argument("Session token id exceeds vocabulary");
          if (status & 4) throw std::runtime_error("A bounded wait inside a kernel gave up");
          throw LengthError("Session context capacity exhausted");
        }
    } catch (...) {
      for (ei_session* s : batch->sessions) drain_failed(*s);
      throw;
    }
    for (size_t j = 0; j < count; ++j) results[j] = batch->sessions[j]->host_control->last;
  });
}

ei_status ei_session_verify_enqueue(ei_session* session, const uint32_t* device_drafts, size_t draft_count,
                                    size_t draft_base, size_t rows) {
  return guarded([&] {
    if (!session) throw std::invalid_argument("session is null");
    ei_session& s = *session;
    require_usable(s);
    if (!rows || rows > kMaxRows || (rows > 1 && !device_drafts))
      throw std::invalid_argument("Verify takes 1..16 rows and a device draft array");
    if (!s.history_ready) throw std::logic_error("Verify requires successful prefill");
    // The host does not know the context length between drains: it bounds it by full acceptance and refuses,
    // before anything is submitted, a step that could pass the capacity.
    if (s.bound + rows > s.capacity) throw LengthError("Verify rows could exceed session capacity; drain first");
    require_device(s);
    try {
      if (s.draft_host.drafts != device_drafts || s.draft_host.base != (long long)draft_base ||
          s.draft_host.count != (long long)draft_count) {
        synchronize(s);
        s.draft_host = DraftSource{device_drafts, (long long)draft_base, (long long)draft_count};
        EI_CUDA(cudaMemcpyAsync(s.draft_source, &s.draft_host, sizeof(s.draft_host), cudaMemcpyHostToDevice, s.stream));
        synchronize(s);
      }
      submit_step(s, int(rows), kVerifyDevice);
      s.bound += rows;
    } catch (...) {
      drain_failed(s);
      throw;
    }
  });
}

ei_status ei_session_drain(ei_session* session, ei_verify_result* last, uint64_t* emitted_total) {
  return guarded([&] {
    if (!session) throw std::invalid_argument("session is null");
    ei_session& s = *session;
    require_usable(s);
    try {
      read_control(s);
      const unsigned long long total = s.host_control->emitted_total;
      if (last) *last = s.host_control->last;
      if (emitted_total) *emitted_total = total;
      // Reset the per-drain counters on the device.
      const int zero_steps = 0;
      const unsigned long long zero_total = 0;
      EI_CUDA(cudaMemcpyAsync(&s.control->steps, &zero_steps, sizeof(int), cudaMemcpyHostToDevice, s.stream));
      EI_CUDA(cudaMemcpyAsync(&s.control->emitted_total, &zero_total, sizeof(zero_total), cudaMemcpyHostToDevice, s.stream));
      synchronize(s);
      check_status(s);
    } catch (const CapacityRefusal&) {
      throw;  // refused on the device before any write: the history stays
    } catch (...) {
      drain_failed(s);
      throw;
    }
  });
}

ei_status ei_session_truncate(ei_session* session, size_t length) {
  return guarded([&] {
    if (!session) throw std::invalid_argument("session is null");
    ei_session& s = *session;
    require_usable(s);
    if (length > s.capacity) throw std::runtime_error("KVCache: Attempted to resize beyond max_seq_len");
    const int32_t value = int32_t(length);
    EI_CUDA(cudaMemcpyAsync(&s.control->context, &value, sizeof(value), cudaMemcpyHostToDevice, s.stream));
    synchronize(s);
    s.context = length;
    s.bound = length;
  });
}

ei_status ei_session_set_pending(ei_session* session, uint32_t token) {
  return guarded([&] {
    if (!session) throw std::invalid_argument("session is null");
    ei_session& s = *session;
    require_usable(s);
    if (token >= s.model->config.vocab_size) throw std::invalid_argument("Token exceeds vocabulary");
    EI_CUDA(cudaMemcpyAsync(&s.control->pending, &token, sizeof(token), cudaMemcpyHostToDevice, s.stream));
    synchronize(s);
  });
}

ei_status ei_session_reset(ei_session* session) {
  return guarded([&] {
    if (!session) throw std::invalid_argument("session is null");
    ei_session& s = *session;
    require_usable(s);
    synchronize(s);
    EI_CUDA(cudaMemsetAsync(s.control, 0, sizeof(Control), s.stream));
    synchronize(s);
    s.context = 0;
    s.bound = 0;
    s.history_ready = false;
  });
}

ei_status ei_session_context_size(const ei_session* session, size_t* out) {
  return guarded([&] {
    if (!session || !out) throw std::invalid_argument("session is null");
    require_usable(*session);
    *out = session->context;
  });
}

ei_status ei_session_context_capacity(const ei_session* session, size_t* out) {
  return guarded([&] {
    if (!session || !out) throw std::invalid_argument("session is null");
    require_usable(*session);
    *out = session->capacity;
  });
}

ei_status ei_session_synchronize(ei_session* session) {
  return guarded([&] {
    if (!session) throw std::invalid_argument("session is null");
    synchronize(*session);
  });
}

void* ei_session_stream(const ei_session* session) { return session ? session->stream : nullptr; }

ei_status ei_session_read_kv(ei_session* session, size_t layer, void* host_k, void* host_v) {
  return guarded([&] {
    if (!session || !host_k || !host_v) throw std::invalid_argument("session or output is null");
    ei_session& s = *session;
    require_usable(s);
    const auto& c = s.model->config;
    if (layer >= c.n_layers) throw std::out_of_range("KVCache: Layer index out of range");
    const size_t kv_width = c.n_kv_heads * 128;
    synchronize(s);
    EI_CUDA(cudaMemcpy(host_k, s.k_cache + layer * s.capacity * kv_width, s.context * kv_width * 2, cudaMemcpyDeviceToHost));
    EI_CUDA(cudaMemcpy(host_v, s.v_cache + layer * s.capacity * kv_width, s.context * kv_width * 2, cudaMemcpyDeviceToHost));
  });
}

ei_status ei_session_write_kv(ei_session* session, size_t layer, size_t first, size_t rows, const void* k,
                              const void* v) {
  return guarded([&] {
    if (!session || !k || !v) throw std::invalid_argument("session or source is null");
    ei_session& s = *session;
    require_usable(s);
    require_device(s);
    const auto& c = s.model->config;
    if (layer >= c.n_layers) throw std::out_of_range("KVCache: Layer index out of range");
    if (first > s.capacity || rows > s.capacity - first) throw LengthError("KV rows exceed session capacity");
    const size_t kv_width = c.n_kv_heads * 128;
    const size_t at = (layer * s.capacity + first) * kv_width;
    EI_CUDA(cudaMemcpyAsync(s.k_cache + at, k, rows * kv_width * 2, cudaMemcpyDefault, s.stream));
    EI_CUDA(cudaMemcpyAsync(s.v_cache + at, v, rows * kv_width * 2, cudaMemcpyDefault, s.stream));
    synchronize(s);
  });
}

ei_status ei_session_adopt_history(ei_session* session, size_t length, uint32_t pending) {
  return guarded([&] {
    if (!session) throw std::invalid_argument("session is null");
    ei_session& s = *session;
    require_usable(s);
    require_device(s);
    if (length > s.capacity) throw LengthError("History exceeds session capacity");
    if (pending >= s.model->config.vocab_size) throw std::invalid_argument("Token exceeds vocabulary");
    Control control{};
    control.context = int32_t(length);
    control.pending = pending;
    synchronize(s);
    EI_CUDA(cudaMemcpyAsync(s.control, &control, sizeof(Control), cudaMemcpyHostToDevice, s.stream));
    synchronize(s);
    s.context = length;
    s.bound = length;
    s.history_ready = true;
  });
}

ei_status ei_session_read_logits(ei_session* session, size_t rows, void* host_logits) {
  return guarded([&] {
    if (!session || !host_logits || !rows || rows > kMaxRows) throw std::invalid_argument("session, rows or output is invalid");
    ei_session& s = *session;
    require_usable(s);
    synchronize(s);
    EI_CUDA(cudaMemcpy(host_logits, s.logits, rows * s.model->config.vocab_size * 2, cudaMemcpyDeviceToHost));
  });
}

size_t ei_session_launches_per_step(const ei_session* session, size_t rows) {
  return session && rows <= kMaxRows ? session->launches_per_step[rows] : 0;
}

ei_status ei_speculative_create(ei_session* target, ei_session* draft, size_t drafts_per_round, ei_speculative** out) {
  return guarded([&] {
    if (!target || !draft || !out || target == draft)
      throw std::invalid_argument("A speculative decoder takes a target and a distinct draft session");
    if (!drafts_per_round || drafts_per_round + 1 > kMaxRows)
      throw std::invalid_argument("Invalid draft capacity");
    if (target->model->device != draft->model->device)
      throw std::invalid_argument("Target and draft sessions must live on one device");
    if (target->model->config.vocab_size != draft->model->config.vocab_size)
      throw std::invalid_argument("Target and draft models must share a vocabulary");
    require_usable(*target);
    require_usable(*draft);
    require_device(*target);
    auto spec = std::make_unique<ei_speculative>();
    spec->target = target;
    spec->draft = draft;
    spec->drafts = drafts_per_round;
    spec->capacity = std::min(target->capacity, draft->capacity);
    spec->token_count = spec->capacity + kMaxRows + 1;
    try {
      EI_CUDA(cudaMalloc(reinterpret_cast<void**>(&spec->tokens), spec->token_count * sizeof(uint32_t)));
      EI_CUDA(cudaMemset(spec->tokens, 0, spec->token_count * sizeof(uint32_t)));
      EI_CUDA(cudaEventCreateWithFlags(&spec->drafted, cudaEventDisableTiming));
      EI_CUDA(cudaEventCreateWithFlags(&spec->verified, cudaEventDisableTiming));
      // Both sessions record what they emit in the shared array; the target also takes its drafts from it.
      const TokenSink sink{spec->tokens, 0, (long long)spec->token_count};
      const DraftSource source{spec->tokens, 0, (long long)spec->token_count};
      for (ei_session* s : {target, draft}) {
        synchronize(*s);
        EI_CUDA(cudaMemcpyAsync(s->token_sink, &sink, sizeof(sink), cudaMemcpyHostToDevice, s->stream));
        s->draft_host = source;
        EI_CUDA(cudaMemcpyAsync(s->draft_source, &source, sizeof(source), cudaMemcpyHostToDevice, s->stream));
        synchronize(*s);
      }
    } catch (...) {
      ei_speculative_destroy(spec.release());
      throw;
    }
    *out = spec.release();
  });
}

void ei_speculative_destroy(ei_speculative* spec) {
  if (!spec) return;
  // Detach the sessions from the array before it is freed.
  const TokenSink none{nullptr, 0, 0};
  const DraftSource empty{nullptr, 0, 0};
  for (ei_session* s : {spec->target, spec->draft}) {
    if (!s || s->poisoned) continue;
    if (cudaStreamSynchronize(s->stream) != cudaSuccess) continue;
    cudaMemcpyAsync(s->token_sink, &none, sizeof(none), cudaMemcpyHostToDevice, s->stream);
    cudaMemcpyAsync(s->draft_source, &empty, sizeof(empty), cudaMemcpyHostToDevice, s->stream);
    s->draft_host = empty;
    cudaStreamSynchronize(s->stream);
  }
  if (spec->drafted) cudaEventDestroy(spec->drafted);
  if (spec->verified) cudaEventDestroy(spec->verified);
  if (spec->tokens) cudaFree(spec->tokens);
  delete spec;
}

ei_status ei_speculative_prefill(ei_speculative* spec, const uint32_t* host_tokens, size_t rows, uint32_t* first_token) {
  return guarded([&] {
    if (!spec) throw std::invalid_argument("speculative decoder is null");
    if (!host_tokens || !rows) throw std::invalid_argument("Prompt must be nonempty");
    if (rows + 1 > spec->capacity) throw LengthError("Prompt exceeds speculative context capacity");
    ei_session& t = *spec->target;
    ei_session& d = *spec->draft;
    spec->started = false;
    // Both sessions take the whole prompt; the target's greedy token after it is the first generated token and
    // the pending token of both (ref: runtime/src/speculative_decoder.cpp:244-276).
    for (ei_session* s : {&t, &d})
      if (ei_session_prefill(s, host_tokens, rows, nullptr, nullptr) != EI_OK)
        throw std::runtime_error("Speculative prefill failed: " + g_last_error);
    try {
      const size_t last_row = t.prefill_target_row;
      uint32_t first = 0;
      EI_CUDA(cudaMemcpyAsync(t.host_tokens, t.targets + last_row, sizeof(uint32_t), cudaMemcpyDeviceToHost, t.stream));
      synchronize(t);
      first = t.host_tokens[0];
      if (first >= t.model->config.vocab_size) throw std::runtime_error("Target sampled an invalid token id");
      for (ei_session* s : {&t, &d}) {
        EI_CUDA(cudaMemcpyAsync(&s->control->pending, &first, sizeof(first), cudaMemcpyHostToDevice, s->stream));
        synchronize(*s);
      }
      EI_CUDA(cudaMemcpyAsync(spec->tokens, host_tokens, rows * sizeof(uint32_t), cudaMemcpyHostToDevice, t.stream));
      EI_CUDA(cudaMemcpyAsync(spec->tokens + rows, &first, sizeof(first), cudaMemcpyHostToDevice, t.stream));
      synchronize(t);
      if (first_token) *first_token = first;
    } catch (...) {
      drain_failed(t);
      drain_failed(d);
      throw;
    }
    spec->prompt_rows = rows;
    spec->bound = rows;
    spec->started = true;
  });
}

ei_status ei_speculative_enqueue(ei_speculative* spec, size_t rounds) {
  return guarded([&] {
    if (!spec) throw std::invalid_argument("speculative decoder is null");
    if (!spec->started) throw std::logic_error("Speculative generation requires successful prefill");
    ei_session& t = *spec->target;
    ei_session& d = *spec->draft;
    require_usable(t);
    require_usable(d);
    require_device(t);
    const size_t rows = spec->drafts + 1;
    // The host does not know the context length between drains: it bounds it by full acceptance. Checked for
    // all rounds before any is submitted, so a refusal leaves the decoder as it was.
    if (spec->bound + rounds * rows > spec->capacity) throw LengthError("Speculative rounds exceed session capacity");
    try {
      for (size_t round = 0; round < rounds; ++round) {
        // k + 1 draft steps, each fed by the token the previous one left on the device: d1..dk are verified, the
        // last step only appends the draft cache row of dk (ref: generate_draft_tokens, speculative_decoder.cpp:176-187).
        for (size_t step = 0; step < rows; ++step) submit_step(d, 1, kVerifyDevice);
        EI_CUDA(cudaEventRecord(spec->drafted, d.stream));
        EI_CUDA(cudaStreamWaitEvent(t.stream, spec->drafted, 0));
        submit_step(t, int(rows), kVerifyDevice);  // ref: verify_greedy, speculative_decoder.cpp:200-224
        EI_CUDA(cudaEventRecord(spec->verified, t.stream));
        EI_CUDA(cudaStreamWaitEvent(d.stream, spec->verified, 0));
        // Both sessions keep the pending input plus every accepted one (speculative_decoder.cpp:219-223).
        launch_adopt_control(d.control, t.control, d.stream);
        spec->bound += rows;
      }
    } catch (...) {
      drain_failed(t);
      drain_failed(d);
      spec->started = false;
      throw;
    }
  });
}

ei_status ei_speculative_drain(ei_speculative* spec, uint32_t* host_tokens, size_t capacity, size_t* count,
                               ei_verify_result* last) {
  return guarded([&] {
    if (!spec) throw std::invalid_argument("speculative decoder is null");
    if (!spec->started) throw std::logic_error("Speculative generation requires successful prefill");
    ei_session& t = *spec->target;
    ei_session& d = *spec->draft;
    require_usable(t);
    require_usable(d);
    try {
      read_control(d);  // the draft stream ends every round: waiting for it waits for the target too
      read_control(t);
      check_status(t);
      check_status(d);
      spec->bound = t.context;
      // Generated so far: the tokens of positions prompt_rows .. context (the last one is pending).
      const size_t generated = t.context + 1 - spec->prompt_rows;
      if (count) *count = generated;
      if (host_tokens && capacity) {
        const size_t copy = std::min(generated, capacity);
        EI_CUDA(cudaMemcpyAsync(host_tokens, spec->tokens + spec->prompt_rows, copy * sizeof(uint32_t),
                                cudaMemcpyDeviceToHost, t.stream));
        synchronize(t);
      }
      if (last) *last = t.host_control->last;
    } catch (...) {
      drain_failed(t);
      drain_failed(d);
      spec->started = false;
      throw;
    }
  });
}

ei_status ei_speculative_truncate(ei_speculative* spec, size_t generated) {
  return guarded([&] {
    if (!spec) throw std::invalid_argument("speculative decoder is null");
    if (!spec->started) throw std::logic_error("Speculative generation requires successful prefill");
    ei_session& t = *spec->target;
    ei_session& d = *spec->draft;
    read_control(d);
    read_control(t);
    // Keep `generated` generated tokens: the last of them becomes pending, the ones before it stay in both caches
    // (ref: EOS truncation, speculative_decoder.cpp:302-304).
    if (!generated || spec->prompt_rows + generated - 1 > t.context)
      throw std::invalid_argument("Truncation keeps between one and all generated tokens");
    const int32_t context = int32_t(spec->prompt_rows + generated - 1);
    uint32_t pending = 0;
    EI_CUDA(cudaMemcpyAsync(t.host_tokens, spec->tokens + context, sizeof(uint32_t), cudaMemcpyDeviceToHost, t.stream));
    synchronize(t);
    pending = t.host_tokens[0];
    for (ei_session* s : {&t, &d}) {
      EI_CUDA(cudaMemcpyAsync(&s->control->context, &context, sizeof(context), cudaMemcpyHostToDevice, s->stream));
      EI_CUDA(cudaMemcpyAsync(&s->control->pending, &pending, sizeof(pending), cudaMemcpyHostToDevice, s->stream));
      synchronize(*s);
      s->context = size_t(context);
    }
    spec->bound = size_t(context);
  });
}

ei_status ei_session_inject_wait_timeout(ei_session* session, uint32_t polls) {
  return guarded([&] {
    if (!session || !polls) throw std::invalid_argument("session is null or the poll limit is zero");
    session->inject_wait_polls = polls;
  });
}

ei_status ei_session_inject_attention_wait_timeout(ei_session* session, uint32_t polls) {
  return guarded([&] {
    if (!session || !polls) throw std::invalid_argument("session is null or polls is zero");
    session->inject_attention_polls = polls;
  });
}

ei_status ei_session_inject_failure(ei_session* session, int nth_launch, int completion) {
  return guarded([&] {
    if (!session) throw std::invalid_argument("session is null");
    session->inject_launch = nth_launch;
    session->inject_completion = completion;
  });
}

}  // extern "C"
