// C-ABI entry points of the direct operators: validation (same conditions and error
// classes as the reference's op::cuda functions, rejected before any write) and dispatch to
// the sm_100a kernels. No entry point allocates; scratch is the caller's.
#include "abi_util.cuh"
#include "kernels.cuh"
#include "smallm_gemm.cuh"

#include <cmath>
#include <mutex>
#include <string>
#include <limits>

namespace ei {

thread_local std::string g_last_error;

namespace {

// ---- argument checks ------------------------------------------------------------------------------------
// Every operator rejects a malformed call with std::invalid_argument (EI_INVALID_ARGUMENT across the ABI)
// before it writes anything, as the reference's operators do (operators/src/cuda/execution.cu:23-58).

[[noreturn]] void reject(const std::string& what) { throw std::invalid_argument(what); }

// Extents cross the ABI as size_t and index the kernels as int.
int kernel_extent(size_t extent, const char* name) {
  if (extent < 1 || extent > size_t(std::numeric_limits<int>::max()))
    reject(std::string(name) + " must lie between 1 and 2^31 - 1");
  return int(extent);
}

template <typename View>
constexpr int rank_of(const View& v) {
  return int(sizeof(v.shape) / sizeof(v.shape[0]));
}

template <typename View>
size_t elements(const View& v) {
  size_t product = 1;
  for (int axis = 0; axis < rank_of(v); ++axis) product *= v.shape[axis];
  return product;
}

// Packed: walking the axes from the innermost outwards, each axis steps over exactly what lies inside it.
// An axis of extent 1 is never stepped along, so its stride is not looked at.
template <typename View>
bool packed(const View& v) {
  size_t step = 1;
  for (int axis = rank_of(v) - 1; axis >= 0; --axis) {
    if (v.shape[axis] > 1 && v.stride[axis] != step) return false;
    step *= v.shape[axis];
  }
  return true;
}

// An operand the kernels index as one dense array.
template <typename View>
void expect_packed(const View& v, const char* name) {
  if (v.data == nullptr) reject(std::string(name) + " has no storage");
  if (elements(v) == 0) reject(std::string(name) + " is empty");
  if (!packed(v)) reject(std::string(name) + " must be a packed row-major view");
}

// [rows, heads, width] with every head row packed and the heads of a row adjacent; rows may be strided
// (a slice of a wider projection output, a window of a cache).
void expect_head_rows(const ei_view3& v, const char* name) {
  if (v.data == nullptr || elements(v) == 0) reject(std::string(name) + " has no storage or is empty");
  const bool heads_adjacent = v.stride[2] == 1 && v.stride[1] == v.shape[2];
  const bool rows_disjoint = v.stride[0] >= v.shape[1] * v.shape[2];
  if (!heads_adjacent || !rows_disjoint) reject(std::string(name) + " must keep the heads of a row packed and adjacent");
  kernel_extent(v.shape[0], "rows");
  kernel_extent(v.shape[1], "heads");
  kernel_extent(v.shape[2], "head width");
}

// A bias is optional; when present it has one packed value per output feature.
void expect_bias(const ei_view1& bias, size_t outputs, const char* name) {
  if (bias.data == nullptr) return;
  if (bias.shape[0] != outputs) reject(std::string(name) + " must have one value per output feature");
  if (outputs > 1 && bias.stride[0] != 1) reject(std::string(name) + " must be packed");
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

cudaStream_t stream_of(const ei_context* ctx) {
  if (!ctx) throw std::invalid_argument("execution context is null");
  return static_cast<cudaStream_t>(ctx->stream);
}

size_t smem_limit_of(const ei_context* ctx) {
  return ctx->shared_memory_limit ? ctx->shared_memory_limit : size_t(227) * 1024;
}

// Rows are processed 16 at a time; each group streams the weights once.
template <typename Launch>
void for_row_groups(size_t rows, Launch&& body) {
  for (size_t first = 0; first < rows; first += 16) body(first, std::min<size_t>(16, rows - first));
}

}  // namespace
}  // namespace ei

using namespace ei;

namespace {
// The prompt kernel for an operator call: K split over blocks when the caller's scratch allows it and the grid
// would otherwise leave most SMs idle; the slices are added (with the bias, rounded once) by a second kernel.
void run_prompt_operator(const ei_context* ctx, bool awq, GemmParams p, void* scratch, size_t scratch_bytes,
                         cudaStream_t stream) {
  const int ksplit = (scratch && p.N % 4 == 0 && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0)
                         ? prompt_gemm_ksplit(p.M, p.N, p.K, ctx->multiprocessors, scratch_bytes) : 1;
  if (ksplit < 2) {
    launch_prompt_gemm(awq, p, stream, false);
    return;
  }
  bf16* out = p.out;
  const bf16* bias = p.bias;
  p.epilogue = kEpiPartial;
  p.ksplit = ksplit;
  p.partial = static_cast<float*>(scratch);
  launch_prompt_gemm(awq, p, stream, false);
  splitk_store_kernel<<<std::min(ctx->multiprocessors * 8, (p.M * p.N + 255) / 256), 256, 0, stream>>>(
      p.partial, ksplit, p.M, p.N, bias, out, p.out_stride);
  check_launch();
}
}  // namespace

extern "C" {

const char* ei_last_error(void) { return g_last_error.c_str(); }
const char* ei_version(void) { return "edge_infer_b200 0.1 (sm_100a)"; }

ei_status ei_prepare_execution_context(void* stream, ei_context* out) {
  return guarded([&] {
    if (!out) throw std::invalid_argument("context output is null");
    ei_context ctx{};
    ctx.stream = stream;
    EI_CUDA(cudaGetDevice(&ctx.device));
    int value = 0;
    EI_CUDA(cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, ctx.device));
    ctx.multiprocessors = value;
    EI_CUDA(cudaDeviceGetAttribute(&value, cudaDevAttrMaxThreadsPerBlock, ctx.device));
    ctx.max_threads_per_block = value;
    EI_CUDA(cudaDeviceGetAttribute(&value, cudaDevAttrMaxSharedMemoryPerBlockOptin, ctx.device));
    ctx.shared_memory_limit = size_t(value);
    *out = ctx;
  });
}

ei_status ei_prepare_dense_bf16(ei_view2 weight, ei_view1 bias, ei_dense_weight* out) {
  return guarded([&] {
    // `weight` is the logical [inputs, outputs] matrix; what matters to the kernels is along which axis its
    // storage is contiguous.
    if (out == nullptr) reject("dense weight output is null");
    if (weight.data == nullptr) reject("dense weight has no storage");
    ei_dense_weight prepared{};
    prepared.data = weight.data;
    prepared.input_features = kernel_extent(weight.shape[0], "input features");
    prepared.output_features = kernel_extent(weight.shape[1], "output features");
    const bool inputs_contiguous = weight.stride[0] == 1 && weight.stride[1] >= weight.shape[0];   // [out, in] storage
    const bool outputs_contiguous = weight.stride[1] == 1 && weight.stride[0] >= weight.shape[1];  // [in, out] storage
    if (inputs_contiguous) {
      prepared.operation = 1;
      prepared.leading_dimension = kernel_extent(weight.stride[1], "weight pitch");
    } else if (outputs_contiguous) {
      prepared.operation = 0;
      prepared.leading_dimension = kernel_extent(weight.stride[0], "weight pitch");
    } else {
      reject("a dense weight must be contiguous along its input or its output axis");
    }
    expect_bias(bias, weight.shape[1], "dense bias");
    prepared.bias = bias.data;
    *out = prepared;
  });
}

ei_status ei_prepare_awq_bf16(ei_view2 qweight, ei_view2 scales, ei_view2 zeros, size_t group_size,
                              size_t input_features, ei_view1 bias, ei_awq_weight* out) {
  return guarded([&] {
    // N-major packing of the reference (operators/src/cuda/kernels/awq_gemv_gemm.cu:591-599): one row per output
    // feature in all three arrays; eight nibbles per word, one scale per group (the row may be padded), eight
    // zero points per word.
    if (out == nullptr) reject("AWQ weight output is null");
    expect_packed(qweight, "AWQ packed weights");
    expect_packed(scales, "AWQ scales");
    expect_packed(zeros, "AWQ zero points");
    ei_awq_weight prepared{};
    prepared.input_features = kernel_extent(input_features, "input features");
    prepared.output_features = kernel_extent(qweight.shape[0], "output features");
    prepared.group_size = kernel_extent(group_size, "group size");
    prepared.padded_groups = kernel_extent(scales.shape[1], "scale row length");
    if (input_features % group_size != 0) reject("AWQ input features must be a whole number of groups");
    const size_t outputs = qweight.shape[0], groups = input_features / group_size;
    if (qweight.shape[1] != (input_features + 7) / 8) reject("AWQ packed weights must hold eight inputs per word");
    if (scales.shape[0] != outputs || scales.shape[1] < groups) reject("AWQ scales must cover every output and group");
    if (zeros.shape[0] != outputs || zeros.shape[1] != (groups + 7) / 8)
      reject("AWQ zero points must hold eight groups per word for every output");
    expect_bias(bias, outputs, "AWQ bias");
    prepared.qweight = static_cast<const int32_t*>(qweight.data);
    prepared.scales = scales.data;
    prepared.zeros = static_cast<const int32_t*>(zeros.data);
    prepared.bias = bias.data;
    *out = prepared;
  });
}

size_t ei_linear_scratch_bytes(size_t rows, size_t input_features, size_t output_features) {
  (void)input_features;
  // Up to 32 rows: worst case split of the input features over blocks, 16 FP32 partial copies of a 16-row group.
  // More rows (the prompt kernel): up to four K slices of all rows, used when the grid would otherwise be small.
  if (rows > size_t(kPromptMinRows)) return size_t(4) * rows * output_features * sizeof(float);
  return size_t(16) * std::min<size_t>(rows, 16) * output_features * sizeof(float);
}

ei_status ei_linear_bf16(const ei_context* ctx, ei_view2 input, const ei_dense_weight* weight, ei_view2 output,
                         void* scratch, size_t scratch_bytes) {
  return guarded([&] {
    cudaStream_t stream = stream_of(ctx);
    expect_packed(input, "input");
    expect_packed(output, "output");
    kernel_extent(input.shape[0], "rows");
    if (!weight || !weight->data || input.shape[1] != size_t(weight->input_features) ||
        output.shape[0] != input.shape[0] || output.shape[1] != size_t(weight->output_features))
      throw std::invalid_argument("Direct dense linear input/output dimensions or handle are invalid");
    const int K = weight->input_features, N = weight->output_features;
    const bool fast_layout = weight->operation == 1 && aligned16(weight->data) && weight->leading_dimension % 8 == 0 &&
                             aligned16(input.data);
    // Many rows: one pass on the tensor cores instead of one weight stream per 16 rows.
    if (input.shape[0] > kPromptMinRows && fast_layout &&
        prompt_gemm_eligible(false, 0, N, K, input.data, K, output.data, N)) {
      GemmParams p{};
      p.x = static_cast<const bf16*>(input.data); p.x_stride = K; p.M = int(input.shape[0]); p.K = K; p.N = N;
      p.w = static_cast<const bf16*>(weight->data); p.ldw = weight->leading_dimension;
      p.bias = static_cast<const bf16*>(weight->bias);
      p.out = static_cast<bf16*>(output.data); p.out_stride = N;
      run_prompt_operator(ctx, false, p, scratch, scratch_bytes, stream);
      return;
    }
    for_row_groups(input.shape[0], [&](size_t first, size_t rows) {
      const bf16* x = static_cast<const bf16*>(input.data) + first * K;
      bf16* out = static_cast<bf16*>(output.data) + first * N;
      GemmPlan plan;
      if (fast_layout)
        plan = plan_gemm(false, int(rows), N, K, kEpiStore, ctx->multiprocessors, smem_limit_of(ctx), scratch != nullptr);
      if (plan.fast && plan.ksplit > 1 && scratch_bytes < size_t(plan.ksplit) * rows * N * sizeof(float))
        plan.fast = false;
      if (plan.fast) {
        GemmParams p{};
        p.x = x; p.x_stride = K; p.M = int(rows); p.K = K; p.N = N;
        p.w = static_cast<const bf16*>(weight->data); p.ldw = weight->leading_dimension;
        p.bias = static_cast<const bf16*>(weight->bias);
        p.out = out; p.out_stride = N;
        p.ksplit = plan.ksplit;
        p.epilogue = plan.ksplit > 1 ? kEpiPartial : kEpiStore;
        p.partial = static_cast<float*>(scratch);
        launch_gemm(plan, false, p, stream, false);
        if (plan.ksplit > 1) {
          splitk_store_kernel<<<std::min(1024, (int(rows) * N + 255) / 256), 256, 0, stream>>>(
              p.partial, plan.ksplit, int(rows), N, p.bias, out, N);
          check_launch();
        }
      } else {
        const long long stride_k = weight->operation == 1 ? 1 : weight->leading_dimension;
        const long long stride_n = weight->operation == 1 ? weight->leading_dimension : 1;
        const size_t count = rows * size_t(N);
        dense_generic_kernel<<<unsigned(std::min<size_t>((count + 255) / 256, size_t(ctx->multiprocessors) * 32)), 256, 0,
                               stream>>>(x, K, static_cast<const bf16*>(weight->data), stride_k, stride_n,
                                         static_cast<const bf16*>(weight->bias), out, N, int(rows), N, K);
        check_launch();
      }
    });
  });
}

ei_status ei_awq_linear_bf16(const ei_context* ctx, ei_view2 input, const ei_awq_weight* weight, ei_view2 output,
                             void* scratch, size_t scratch_bytes) {
  return guarded([&] {
    cudaStream_t stream = stream_of(ctx);
    expect_packed(input, "input");
    expect_packed(output, "output");
    kernel_extent(input.shape[0], "rows");
    if (!weight || !weight->qweight || !weight->scales || !weight->zeros ||
        input.shape[1] != size_t(weight->input_features) || output.shape[0] != input.shape[0] ||
        output.shape[1] != size_t(weight->output_features))
      throw std::invalid_argument("Direct AWQ linear input/output dimensions are invalid");
    const int K = weight->input_features, N = weight->output_features;
    const bool fast_layout = weight->group_size == 128 && aligned16(weight->qweight) && aligned16(input.data);
    if (input.shape[0] > kPromptMinRows && fast_layout && (K / 8) % 4 == 0 &&
        prompt_gemm_eligible(true, weight->group_size, N, K, input.data, K, output.data, N)) {
      GemmParams p{};
      p.x = static_cast<const bf16*>(input.data); p.x_stride = K; p.M = int(input.shape[0]); p.K = K; p.N = N;
      p.qweight = weight->qweight;
      p.scales = static_cast<const bf16*>(weight->scales);
      p.zeros = weight->zeros;
      p.padded_groups = weight->padded_groups;
      p.zero_stride = (K / 128 + 7) / 8;
      p.bias = static_cast<const bf16*>(weight->bias);
      p.out = static_cast<bf16*>(output.data); p.out_stride = N;
      run_prompt_operator(ctx, true, p, scratch, scratch_bytes, stream);
      return;
    }
    for_row_groups(input.shape[0], [&](size_t first, size_t rows) {
      const bf16* x = static_cast<const bf16*>(input.data) + first * K;
      bf16* out = static_cast<bf16*>(output.data) + first * N;
      GemmPlan plan;
      if (fast_layout)
        plan = plan_gemm(true, int(rows), N, K, kEpiStore, ctx->multiprocessors, smem_limit_of(ctx), scratch != nullptr);
      if (plan.fast && plan.ksplit > 1 && scratch_bytes < size_t(plan.ksplit) * rows * N * sizeof(float))
        plan.fast = false;
      if (plan.fast) {
        GemmParams p{};
        p.x = x; p.x_stride = K; p.M = int(rows); p.K = K; p.N = N;
        p.qweight = weight->qweight;
        p.scales = static_cast<const bf16*>(weight->scales);
        p.zeros = weight->zeros;
        p.padded_groups = weight->padded_groups;
        p.zero_stride = (K / 128 + 7) / 8;
        p.bias = static_cast<const bf16*>(weight->bias);
        p.out = out; p.out_stride = N;
        p.ksplit = plan.ksplit;
        p.epilogue = plan.ksplit > 1 ? kEpiPartial : kEpiStore;
        p.partial = static_cast<float*>(scratch);
        launch_gemm(plan, true, p, stream, false);
        if (plan.ksplit > 1) {
          splitk_store_kernel<<<std::min(1024, (int(rows) * N + 255) / 256), 256, 0, stream>>>(
              p.partial, plan.ksplit, int(rows), N, p.bias, out, N);
          check_launch();
        }
      } else {
        const size_t count = rows * size_t(N);
        awq_generic_kernel<<<unsigned(std::min<size_t>((count + 255) / 256, size_t(ctx->multiprocessors) * 32)), 256, 0,
                             stream>>>(x, K, weight->qweight, static_cast<const bf16*>(weight->scales), weight->zeros,
                                       static_cast<const bf16*>(weight->bias), out, N, int(rows), N, K,
                                       weight->group_size, weight->padded_groups);
        check_launch();
      }
    });
  });
}

ei_status ei_awq_gate_up_silu_bf16(const ei_context* ctx, ei_view2 input, const ei_awq_weight* weight,
                                   ei_view2 output) {
  return guarded([&] {
    cudaStream_t stream = stream_of(ctx);
    expect_packed(input, "input");
    expect_packed(output, "output");
    if (!weight || !weight->qweight || !weight->scales || !weight->zeros || weight->output_features % 2 ||
        input.shape[1] != size_t(weight->input_features) || output.shape[0] != input.shape[0] ||
        output.shape[1] != size_t(weight->output_features / 2))
      throw std::invalid_argument("Fused gate/up projection input/output dimensions are invalid");
    const int K = weight->input_features, N = weight->output_features, rows = int(input.shape[0]);
    GemmPlan plan;
    if (rows <= 16 && weight->group_size == 128 && aligned16(weight->qweight) && aligned16(input.data))
      plan = plan_gemm(true, rows, N, K, kEpiSiluPair, ctx->multiprocessors, smem_limit_of(ctx), false);
    if (!plan.fast)
      throw std::invalid_argument(
          "Fused gate/up projection needs rows <= 16, group_size 128, K % 256 == 0 and 16-byte aligned operands");
    GemmParams p{};
    p.x = static_cast<const bf16*>(input.data); p.x_stride = K; p.M = rows; p.K = K; p.N = N;
    p.qweight = weight->qweight;
    p.scales = static_cast<const bf16*>(weight->scales);
    p.zeros = weight->zeros;
    p.padded_groups = weight->padded_groups;
    p.zero_stride = (K / 128 + 7) / 8;
    p.bias = static_cast<const bf16*>(weight->bias);
    p.out = static_cast<bf16*>(output.data); p.out_stride = N / 2;
    p.ksplit = 1;
    p.epilogue = kEpiSiluPair;
    launch_gemm(plan, true, p, stream, false);
  });
}

ei_status ei_add_bf16(const ei_context* ctx, ei_array a, ei_array b, ei_array out) {
  return guarded([&] {
    cudaStream_t stream = stream_of(ctx);
    if (a.size != b.size || a.size != out.size)
      throw std::runtime_error("Add operator: input and output views must have the same size");
    if (!a.size) return;
    if (!a.data || !b.data || !out.data) throw std::invalid_argument("Add operator: null storage");
    launch_add(static_cast<const bf16*>(a.data), static_cast<const bf16*>(b.data), static_cast<bf16*>(out.data),
               a.size, ctx->multiprocessors, stream);
  });
}

ei_status ei_silu_multiply_bf16(const ei_context* ctx, ei_array gate, ei_array up, ei_array out) {
  return guarded([&] {
    cudaStream_t stream = stream_of(ctx);
    if (up.size != gate.size || out.size != gate.size)
      throw std::runtime_error("SiLU multiply operator: input and output views must have the same size");
    if (!gate.size) return;
    if (gate.size > size_t(std::numeric_limits<int>::max()))
      throw std::runtime_error("SiLU multiply CUDA view extent exceeds the kernel index range");
    launch_silu_multiply(static_cast<const bf16*>(gate.data), static_cast<const bf16*>(up.data),
                         static_cast<bf16*>(out.data), gate.size, ctx->multiprocessors, stream);
  });
}

ei_status ei_rms_norm_bf16(const ei_context* ctx, ei_array input, ei_array weight, ei_array out, size_t rows,
                           size_t features, float epsilon) {
  return guarded([&] {
    cudaStream_t stream = stream_of(ctx);
    if (out.size != input.size)
      throw std::runtime_error("RMSNorm operator: input and output views must have the same size");
    if (!input.size) return;
    if (!features || features > 10240)
      throw std::runtime_error("RMSNorm CUDA feature_dim must be between 1 and 10240");
    if (rows > size_t(std::numeric_limits<int>::max()))
      throw std::runtime_error("RMSNorm CUDA row count exceeds the kernel index range");
    if (input.size % features || input.size / features != rows || weight.size != features)
      throw std::runtime_error("RMSNorm CUDA view extents do not match rows and feature_dim");
    launch_rms_norm(static_cast<const bf16*>(input.data), static_cast<const bf16*>(weight.data),
                    static_cast<bf16*>(out.data), rows, features, epsilon, stream, false);
  });
}

ei_status ei_gather_bf16(const ei_context* ctx, ei_view1 ids, ei_view2 table, ei_view2 out) {
  return guarded([&] {
    cudaStream_t stream = stream_of(ctx);
    expect_packed(ids, "token ids");
    expect_packed(table, "embedding table");
    expect_packed(out, "output");
    if (out.shape[0] != ids.shape[0] || out.shape[1] != table.shape[1])
      throw std::invalid_argument("Direct gather input/output shapes differ");
    launch_gather(static_cast<const uint32_t*>(ids.data), static_cast<const bf16*>(table.data),
                  static_cast<bf16*>(out.data), out.shape[0], table.shape[1], table.shape[0], ctx->multiprocessors,
                  stream);
  });
}

ei_status ei_rope_precomputed_bf16(const ei_context* ctx, ei_view3 input, ei_view2 table, size_t offset,
                                   const size_t* offsets, const int* pingpong) {
  return guarded([&] {
    cudaStream_t stream = stream_of(ctx);
    expect_head_rows(input, "RoPE input");
    expect_packed(table, "RoPE table");
    if (table.shape[1] != input.shape[2] || input.shape[2] % 2 ||
        input.shape[2] / 2 > size_t(ctx->max_threads_per_block ? ctx->max_threads_per_block : 1024))
      throw std::invalid_argument("Direct cached RoPE has incompatible cache or offsets");
    if (!offsets && (offset > table.shape[0] || input.shape[0] > table.shape[0] - offset))
      throw std::out_of_range("Direct cached RoPE positions exceed table capacity");
    launch_rope(static_cast<bf16*>(input.data), input.shape[0], input.shape[1], input.shape[2], input.stride[0],
                static_cast<const float*>(table.data), table.stride[0], offset, offsets, pingpong, ctx->multiprocessors,
                stream);
  });
}

ei_status ei_build_rope_table(float* host_table, size_t max_positions, size_t head_dim, float theta) {
  return guarded([&] {
    if (!host_table || !max_positions || !head_dim || head_dim % 2 || !std::isfinite(theta) || theta <= 0.0f)
      throw std::invalid_argument("RoPE table requires positive extents, an even head width and a positive theta");
    for (size_t pos = 0; pos < max_positions; ++pos)
      for (size_t i = 0; i < head_dim / 2; ++i) {
        const float frequency = 1.0f / std::pow(theta, 2.0f * static_cast<float>(i) / static_cast<float>(head_dim));
        const float angle = static_cast<float>(pos) * frequency;
        host_table[pos * head_dim + 2 * i] = std::sin(angle);
        host_table[pos * head_dim + 2 * i + 1] = std::cos(angle);
      }
  });
}

ei_status ei_store_kv_bf16(const ei_context* ctx, ei_view2 source, ei_view2 capacity, size_t offset,
                           const size_t* device_offset) {
  return guarded([&] {
    cudaStream_t stream = stream_of(ctx);
    expect_packed(source, "KV source");
    expect_packed(capacity, "KV cache");
    if (source.shape[1] != capacity.shape[1] || offset > capacity.shape[0] ||
        source.shape[0] > capacity.shape[0] - offset)
      throw std::invalid_argument("Direct KV store source or offset exceeds cache capacity");
    launch_store_kv(static_cast<const bf16*>(source.data), static_cast<bf16*>(capacity.data), source.shape[0],
                    source.shape[1], capacity.shape[0], offset, device_offset, ctx->multiprocessors, stream);
  });
}

size_t ei_attention_scratch_bytes(size_t q_rows, size_t query_heads, size_t head_dim, size_t kv_length) {
  (void)head_dim;
  return attention_scratch_bytes(q_rows, query_heads, kv_length);
}

static void run_attention(const ei_context* ctx, ei_view3 q, ei_view3 k, ei_view3 v, ei_view3 out, size_t offset,
                          const int32_t* device_offset, void* scratch, size_t scratch_bytes) {
  cudaStream_t stream = stream_of(ctx);
  expect_head_rows(q, "attention queries");
  expect_head_rows(k, "attention keys");
  expect_head_rows(v, "attention values");
  expect_head_rows(out, "attention output");
  auto same_shape = [](const ei_view3& a, const ei_view3& b) {
    return a.shape[0] == b.shape[0] && a.shape[1] == b.shape[1] && a.shape[2] == b.shape[2];
  };
  if (!same_shape(k, v)) reject("attention keys and values must have one shape");
  if (!same_shape(q, out)) reject("attention output must have the queries' shape");
  if (q.shape[2] != k.shape[2]) reject("attention queries and keys must share the head width");
  if (q.shape[1] % k.shape[1] != 0) reject("query heads must be a whole multiple of KV heads");
  if (!device_offset && (offset > k.shape[0] || q.shape[0] > k.shape[0] - offset))
    throw std::invalid_argument("Direct prefill attention offset exceeds live KV extent");
  const size_t group = q.shape[1] / k.shape[1];
  if (q.shape[2] != 128 || q.shape[0] * group > 112 || k.stride[0] != v.stride[0] || !aligned16(q.data) ||
      !aligned16(k.data) || !aligned16(v.data) || !aligned16(out.data) || (q.stride[0] * 2) % 16 ||
      (k.stride[0] * 2) % 16 || (out.stride[0] * 2) % 16)
    throw std::invalid_argument(
        "Verify attention supports head_dim 128, rows * (heads / kv_heads) <= 112 and 16-byte aligned rows");
  const size_t length = device_offset ? k.shape[0] : offset + q.shape[0];
  if (!scratch || scratch_bytes < attention_scratch_bytes(q.shape[0], q.shape[1], length))
    throw std::invalid_argument("Verify attention scratch capacity is insufficient");
  AttentionParams p{};
  p.q = static_cast<const bf16*>(q.data);
  p.q_stride = int(q.stride[0]);
  p.k = static_cast<const bf16*>(k.data);
  p.v = static_cast<const bf16*>(v.data);
  p.kv_stride = int(k.stride[0]);
  p.rows = int(q.shape[0]);
  p.heads = int(q.shape[1]);
  p.kv_heads = int(k.shape[1]);
  p.capacity = int(k.shape[0]);
  p.device_offset = device_offset;
  p.host_offset = int(offset);
  p.chunk = attention_chunk_for(length);
  p.max_splits = int((length + p.chunk - 1) / p.chunk);
  p.scratch = static_cast<float*>(scratch);
  p.out = static_cast<bf16*>(out.data);
  p.out_stride = int(out.stride[0]);
  launch_verify_attention(p, stream, false);
}

ei_status ei_attention_prefill_bf16(const ei_context* ctx, ei_view3 q, ei_view3 k, ei_view3 v, ei_view3 out,
                                    size_t offset, void* scratch, size_t scratch_bytes) {
  return guarded([&] { run_attention(ctx, q, k, v, out, offset, nullptr, scratch, scratch_bytes); });
}

ei_status ei_attention_verify_bf16(const ei_context* ctx, ei_view3 q, ei_view3 k_capacity, ei_view3 v_capacity,
                                   ei_view3 out, const int32_t* device_offset, void* scratch,
                                   size_t scratch_bytes) {
  return guarded([&] {
    if (!device_offset) throw std::invalid_argument("Verify attention requires a device offset");
    run_attention(ctx, q, k_capacity, v_capacity, out, 0, device_offset, scratch, scratch_bytes);
  });
}

// ---- attention for callers that cannot provide scratch ---------------------------------------------------
// Some hosts have nowhere to get device memory from at the point where they call an operator: a plugin
// slot whose interface carries only the operator's tensors, a serving process that handed all device
// memory to its own pool at start-up (a later driver allocation may fail, and it synchronises the whole
// device), or a stateless hook that cannot keep a buffer between calls. For them the split-KV partials
// live in an array that is part of the library image itself, so it exists on every device as soon as the
// library is loaded and is never allocated or freed.
constexpr size_t kStaticAttentionScratchBytes = size_t(EI_ATTENTION_STATIC_SCRATCH_BYTES);
static __device__ __align__(256) unsigned char static_attention_scratch[kStaticAttentionScratchBytes];

// Device address of the array on the current device; resolved on the first call per device.
static void* static_attention_scratch_address() {
  constexpr int kMaxDevices = 64;
  static std::mutex mutex;
  static void* address[kMaxDevices] = {};
  int device = 0;
  EI_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) throw std::invalid_argument("Device ordinal is out of range");
  std::lock_guard<std::mutex> lock(mutex);
  if (!address[device]) {
    void* resolved = nullptr;
    const cudaError_t status = cudaGetSymbolAddress(&resolved, static_attention_scratch);
    if (status != cudaSuccess || !resolved)
      throw std::runtime_error(std::string("Built-in attention scratch could not be resolved: ") +
                               cudaGetErrorString(status));
    address[device] = resolved;
  }
  return address[device];
}

ei_status ei_attention_prefill_static_bf16(const ei_context* ctx, ei_view3 q, ei_view3 k, ei_view3 v, ei_view3 out,
                                           size_t offset) {
  return guarded([&] {
    // The array is resolved for the CURRENT device: a context prepared on another one would be served the
    // wrong device's array.
    int current = -1;
    EI_CUDA(cudaGetDevice(&current));
    if (!ctx || ctx->device != current)
      throw std::invalid_argument("The execution context belongs to another CUDA device than the current one");
    const size_t length = offset + q.shape[0];
    const size_t needed = attention_scratch_bytes(q.shape[0], q.shape[1], length);
    if (needed > kStaticAttentionScratchBytes)
      throw std::invalid_argument("Attention of " + std::to_string(q.shape[0]) + " rows x " +
                                  std::to_string(q.shape[1]) + " heads over " + std::to_string(length) +
                                  " positions needs " + std::to_string(needed) +
                                  " bytes of split scratch, more than the " +
                                  std::to_string(kStaticAttentionScratchBytes) +
                                  " built into the library; call ei_attention_prefill_bf16 with caller-owned scratch");
    // Nothing in the array has to start at zero: every partial the merge reads is written by this call.
    run_attention(ctx, q, k, v, out, offset, nullptr, static_attention_scratch_address(),
                  kStaticAttentionScratchBytes);
  });
}

size_t ei_sample_scratch_bytes(size_t rows, size_t vocabulary) {
  (void)rows;
  (void)vocabulary;
  return size_t(kSampleMaxParts) * 16 * (sizeof(float) + sizeof(int));  // partial (value, index) per block and row
}

ei_status ei_sample_greedy_bf16(const ei_context* ctx, ei_view2 logits, ei_view1 tokens, void* scratch,
                                size_t scratch_bytes) {
  return guarded([&] {
    cudaStream_t stream = stream_of(ctx);
    expect_packed(logits, "logits");
    expect_packed(tokens, "tokens");
    kernel_extent(logits.shape[1], "vocabulary");
    if (tokens.shape[0] != logits.shape[0] || !scratch || scratch_bytes < ei_sample_scratch_bytes(0, 0))
      throw std::invalid_argument("Direct sampling parameters, plan or output capacities are invalid");
    const int blocks = std::min(kSampleMaxParts, sample_partial_blocks(logits.shape[1], ctx->multiprocessors));
    float* best_value = static_cast<float*>(scratch);
    int* best_index = reinterpret_cast<int*>(best_value + kSampleMaxParts * 16);
    for_row_groups(logits.shape[0], [&](size_t first, size_t rows) {
      launch_argmax_partials(static_cast<const bf16*>(logits.data) + first * logits.stride[0], rows, logits.shape[1],
                             logits.stride[0], best_value, best_index, blocks, stream, false);
      launch_finalize(best_value, best_index, blocks, int(rows), static_cast<uint32_t*>(tokens.data) + first, nullptr,
                      nullptr, nullptr, nullptr, nullptr, stream, false);
    });
  });
}

ei_status ei_verify_accept(const ei_context* ctx, const uint32_t* inputs, const uint32_t* targets, size_t rows,
                           int32_t* context_length, uint32_t* pending, ei_verify_result* result) {
  return guarded([&] {
    cudaStream_t stream = stream_of(ctx);
    if (!inputs || !targets || !rows || rows > 16 || !context_length || !pending || !result)
      throw std::invalid_argument("Verify acceptance requires 1..16 rows and non-null device pointers");
    launch_accept(inputs, targets, int(rows), context_length, pending, result, stream);
  });
}

}  // extern "C"
