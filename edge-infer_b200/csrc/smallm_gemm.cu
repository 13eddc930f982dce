// Dispatch, planning and fallbacks for the small-M weight-streaming GEMM.
#include "smallm_gemm.cuh"

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

size_t part_bytes(int tiles_per_item) { return size_t(2) * kGemmWarps * tiles_per_item * 128 * sizeof(float); }

template <bool kAwq, bool kHigh, int kTiles, int kUnits, int kDepth>
void launch_instance(const GemmPlan& plan, const GemmParams& params, cudaStream_t stream, bool pdl) {
  auto kernel = smallm_gemm_kernel<kAwq, kHigh, kTiles, kUnits, kDepth>;
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

template <bool kAwq, int kTiles, int kUnits, int kDepth>
void launch_high(const GemmPlan& plan, const GemmParams& params, cudaStream_t stream, bool pdl) {
  if (plan.high)
    launch_instance<kAwq, true, kTiles, kUnits, kDepth>(plan, params, stream, pdl);
  else
    launch_instance<kAwq, false, kTiles, kUnits, kDepth>(plan, params, stream, pdl);
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
  const int max_units = awq ? 2 : (pair ? 2 : 4);
  const int tiles = N / 8;
  static const int candidates[] = {1, 2, 3, 4, 6, 8, 12, 16};
  for (int ks : candidates) {
    if (K % (ks * unit_k)) continue;
    const int kslice = K / ks;
    const int units = kslice / unit_k;
    const int per_warp = (units + kGemmWarps - 1) / kGemmWarps;
    if (per_warp > max_units) continue;
    int tiles_per_item = pair ? 2 : (awq ? (per_warp == 1 ? 2 : 1) : 1);
    // A second tile per item only pays when every block still gets several items.
    if (!pair && tiles_per_item == 2 && tiles / 2 < 4 * multiprocessors / ks) tiles_per_item = 1;
    const size_t smem = size_t(kslice) * 16 * (plan.high ? 2 : 1) + part_bytes(tiles_per_item);
    if (smem > smem_limit) continue;
    if (ks > 1 && (!allow_split || (epilogue != kEpiStore && epilogue != kEpiPartial))) return plan;
    plan.fast = true;
    plan.ksplit = ks;
    plan.units_per_warp = per_warp == 3 ? 4 : per_warp;
    plan.tiles_per_item = tiles_per_item;
    plan.smem = smem;
    const int items = pair ? tiles / 2 : (tiles + tiles_per_item - 1) / tiles_per_item;
    const int groups = std::max(1, std::min(multiprocessors / ks, items));
    plan.grid = groups * ks;
    return plan;
  }
  return plan;
}

void launch_gemm(const GemmPlan& plan, bool awq, const GemmParams& p, cudaStream_t stream, bool pdl) {
  const int T = plan.tiles_per_item, U = plan.units_per_warp;
  if (awq) {
    if (T == 2 && U == 1) return launch_high<true, 2, 1, 3>(plan, p, stream, pdl);
    if (T == 1 && U == 1) return launch_high<true, 1, 1, 4>(plan, p, stream, pdl);
    if (T == 1 && U == 2) return launch_high<true, 1, 2, 2>(plan, p, stream, pdl);
    if (T == 2 && U == 2) return launch_high<true, 2, 2, 2>(plan, p, stream, pdl);
  } else {
    if (T == 1 && U == 1) return launch_high<false, 1, 1, 4>(plan, p, stream, pdl);
    if (T == 1 && U == 2) return launch_high<false, 1, 2, 3>(plan, p, stream, pdl);
    if (T == 1 && U == 4) return launch_high<false, 1, 4, 2>(plan, p, stream, pdl);
    if (T == 2 && U == 1) return launch_high<false, 2, 1, 3>(plan, p, stream, pdl);
    if (T == 2 && U == 2) return launch_high<false, 2, 2, 2>(plan, p, stream, pdl);
  }
  throw std::invalid_argument("small-M GEMM plan has no kernel instance");
}

}  // namespace ei
