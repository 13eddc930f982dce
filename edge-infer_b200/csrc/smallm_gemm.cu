// Dispatch, planning and fallbacks for the small-M weight-streaming GEMM.
#include "awq_stream.cuh"

#include <algorithm>

namespace ei {

__global__ void splitk_store_kernel(const float* partial, int ksplit, int M, int N, const bf16* bias,
                                    bf16* out, int out_stride) {
  grid_dependency_wait();
  const int total = M * N;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int row = i / N, n = i - row * N;
    float sum = 0.0f;
    for (int s = 0; s < ksplit; ++s) sum += partial[(size_t(s) * M + row) * N + n];
    if (bias) sum += __bfloat162float(bias[n]);
    out[size_t(row) * out_stride + n] = __float2bfloat16_rn(sum);
  }
}

__global__ void awq_generic_kernel(const bf16* x, int x_stride, const int32_t* qweight, const bf16* scales,
                                   const int32_t* zeros, const bf16* bias, bf16* out, int out_stride,
                                   int rows, int N, int K, int group_size, int padded_groups) {
  const size_t count = size_t(rows) * N;
  const int weight_stride = (K + 7) / 8, zero_stride = (K / group_size + 7) / 8;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
       i += size_t(gridDim.x) * blockDim.x) {
    const int row = int(i / N), n = int(i % N);
    float sum = bias ? __bfloat162float(bias[n]) : 0.0f;
    for (int k = 0; k < K; ++k) {
      const int grp = k / group_size;
      const uint32_t value = (uint32_t(qweight[size_t(n) * weight_stride + k / 8]) >> ((k % 8) * 4)) & 15u;
      const uint32_t zero = (uint32_t(zeros[size_t(n) * zero_stride + grp / 8]) >> ((grp % 8) * 4)) & 15u;
      const float weight = round_bf16(__fmul_rn(float(value) - float(zero),
                                                __bfloat162float(scales[size_t(n) * padded_groups + grp])));
      sum = fmaf(__bfloat162float(x[size_t(row) * x_stride + k]), weight, sum);
    }
    out[size_t(row) * out_stride + n] = __float2bfloat16_rn(sum);
  }
}

__global__ void dense_generic_kernel(const bf16* x, int x_stride, const bf16* w, long long stride_k,
                                     long long stride_n, const bf16* bias, bf16* out, int out_stride,
                                     int rows, int N, int K) {
  const size_t count = size_t(rows) * N;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
       i += size_t(gridDim.x) * blockDim.x) {
    const int row = int(i / N), n = int(i % N);
    float sum = bias ? __bfloat162float(bias[n]) : 0.0f;
    for (int k = 0; k < K; ++k)
      sum = fmaf(__bfloat162float(x[size_t(row) * x_stride + k]),
                 __bfloat162float(w[k * stride_k + n * stride_n]), sum);
    out[size_t(row) * out_stride + n] = __float2bfloat16_rn(sum);
  }
}

namespace {

// Two buffers of per-warp FP32 partials: 16 warps x 136 floats each.
constexpr size_t kPartBytes = size_t(2) * kGemmWarps * 136 * sizeof(float);

template <bool kAwq, bool kHigh, int kUnits, int kDepth>
void launch_instance(const GemmPlan& plan, const GemmParams& params, cudaStream_t stream, bool pdl) {
  auto kernel = smallm_gemm_kernel<kAwq, kHigh, kUnits, kDepth>;
  static thread_local int configured_device = -1;
  int device = 0;
  EI_CUDA(cudaGetDevice(&device));
  if (configured_device != device) {
    // Opt in to the full shared-memory carve-out once per device and thread.
    EI_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured_device = device;
  }
  launch(kernel, dim3(plan.grid), dim3(kGemmThreads), plan.smem, stream, pdl, params);
}

// Deeper prefetch where only the low eight rows hold fragments (half the pinned registers).
template <bool kAwq, int kUnits, int kDepthHigh, int kDepthLow>
void launch_high(const GemmPlan& plan, const GemmParams& params, cudaStream_t stream, bool pdl) {
  if (plan.high)
    launch_instance<kAwq, true, kUnits, kDepthHigh>(plan, params, stream, pdl);
  else
    launch_instance<kAwq, false, kUnits, kDepthLow>(plan, params, stream, pdl);
}

}  // namespace

GemmPlan plan_gemm(bool awq, int M, int N, int K, int epilogue, int multiprocessors, size_t smem_limit,
                   bool allow_split) {
  GemmPlan plan;
  const int unit_k = awq ? 256 : 64;
  if (M < 1 || M > 16 || N % 8 || K % unit_k) return plan;
  const bool pair = epilogue == kEpiSiluPair;
  if (pair && N % 16) return plan;
  plan.high = M > 8;
  // Units one warp may own: int4 pins its fragments in registers (one unit); BF16 reads them from shared memory.
  const int max_units = awq ? 1 : 4;
  const int units_total = K / unit_k;
  const int ks = (units_total + kGemmWarps * max_units - 1) / (kGemmWarps * max_units);
  if (ks > 1 && (!allow_split || (epilogue != kEpiStore && epilogue != kEpiPartial))) return plan;
  if (ks > 16) return plan;
  const int units = (units_total + ks - 1) / ks;  // the largest slice
  int per_warp = (units + kGemmWarps - 1) / kGemmWarps;
  if (per_warp == 3) per_warp = 4;
  const int chunks = pair ? N / 16 : N / 8;
  const int groups = std::max(1, std::min(multiprocessors / ks, chunks));
  size_t smem = kPartBytes + size_t(units) * unit_k * 16 * (plan.high ? 2 : 1);
  if (awq) {
    if (epilogue == kEpiArgmax) return plan;  // the vocabulary head is a dense matrix
    plan.tiles_per_block = ((chunks + groups - 1) / groups) * (pair ? 2 : 1);
    smem = awq_stream_layout(units, plan.tiles_per_block).total;
  }
  if (smem > smem_limit) return plan;
  plan.fast = true;
  plan.ksplit = ks;
  plan.units_per_warp = per_warp;
  plan.smem = smem;
  plan.grid = groups * ks;
  return plan;
}

void launch_gemm(const GemmPlan& plan, bool awq, const GemmParams& p, cudaStream_t stream, bool pdl) {
  const int U = plan.units_per_warp;
  if (awq) {
    static thread_local int configured_device = -1;
    int device = 0;
    EI_CUDA(cudaGetDevice(&device));
    if (configured_device != device) {
      EI_CUDA(cudaFuncSetAttribute(awq_stream_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
      EI_CUDA(cudaFuncSetAttribute(awq_stream_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
      configured_device = device;
    }
    if (plan.high)
      launch(awq_stream_kernel<true>, dim3(plan.grid), dim3(kGemmThreads), plan.smem, stream, pdl, p, plan.tiles_per_block);
    else
      launch(awq_stream_kernel<false>, dim3(plan.grid), dim3(kGemmThreads), plan.smem, stream, pdl, p, plan.tiles_per_block);
    return;
  } else {
    if (U == 1) return launch_high<false, 1, 6, 6>(plan, p, stream, pdl);
    if (U == 2) return launch_high<false, 2, 4, 4>(plan, p, stream, pdl);
    if (U == 4) return launch_high<false, 4, 2, 2>(plan, p, stream, pdl);
  }
  throw std::invalid_argument("small-M GEMM plan has no kernel instance");
}

}  // namespace ei
