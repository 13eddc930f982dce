// Dispatch, planning and fallbacks for the small-M weight-streaming GEMM.
#include "awq_tma.cuh"
#include "dense_tma.cuh"
#include "prompt_gemm.cuh"

#include <algorithm>
#include <stdexcept>
#include <string>

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

template <bool kHigh, int kUnits, int kDepth>
void launch_instance(const GemmPlan& plan, const GemmParams& params, cudaStream_t stream, bool pdl) {
  auto kernel = smallm_gemm_kernel<kHigh, kUnits, kDepth>;
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
template <int kUnits, int kDepthHigh, int kDepthLow>
void launch_high(const GemmPlan& plan, const GemmParams& params, cudaStream_t stream, bool pdl) {
  if (plan.high)
    launch_instance<true, kUnits, kDepthHigh>(plan, params, stream, pdl);
  else
    launch_instance<false, kUnits, kDepthLow>(plan, params, stream, pdl);
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
  int groups = std::max(1, std::min(multiprocessors / ks, chunks));
  if (epilogue == kEpiArgmax) groups = std::min(groups, 256);  // one argmax partial per block: the buffers hold 256
  size_t smem = kPartBytes + size_t(units) * unit_k * 16 * (plan.high ? 2 : 1);
  if (awq) {
    if (epilogue == kEpiArgmax) return plan;  // the vocabulary head is a dense matrix
    plan.tiles_per_block = ((chunks + groups - 1) / groups) * (pair ? 2 : 1);
    // Feasible if one phase of tiles fits in flight even when scales and zero points are staged up front.
    AwqLaunch worst{plan.tiles_per_block, kAwqPhaseTiles, std::min(kAwqSliceUnits, units_total), 0, 0, 0, 0, 0};
    smem = awq_layout(worst).total;
    plan.smem_limit = smem_limit;
  }
  if (smem > smem_limit) return plan;
  plan.smem_limit = smem_limit;
  plan.fast = true;
  plan.ksplit = ks;
  plan.units_per_warp = per_warp;
  plan.smem = smem;
  plan.grid = groups * ks;
  return plan;
}

namespace {

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime so that the library does not link libcuda.
EncodeTiled tensor_map_encoder() {
  static const EncodeTiled encoder = [] {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
    const cudaError_t status = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &found);
    if (status != cudaSuccess || found != cudaDriverEntryPointSuccess || !entry)
      throw std::runtime_error("The CUDA driver does not provide cuTensorMapEncodeTiled");
    return reinterpret_cast<EncodeTiled>(entry);
  }();
  return encoder;
}

}  // namespace

void encode_map(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base, const cuuint64_t* dims,
                const cuuint64_t* strides, const cuuint32_t* box, CUtensorMapSwizzle swizzle, const char* what) {
  const cuuint32_t ones[5] = {1, 1, 1, 1, 1};
  const CUresult result = tensor_map_encoder()(map, type, cuuint32_t(rank), const_cast<void*>(base), dims, strides, box,
                                               ones, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (result != CUDA_SUCCESS)
    throw std::runtime_error(std::string("Tensor map for ") + what + " could not be encoded: " +
                             std::to_string(int(result)));
}

namespace {

bool aligned_16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <bool kHigh, bool kPair, bool kTmaSz, bool kFull>
void launch_awq_instance(int grid, size_t smem, cudaStream_t stream, bool pdl, const AwqTensorMaps& maps,
                         const GemmParams& p, const AwqLaunch& cfg) {
  auto kernel = awq_tma_kernel<kHigh, kPair, kTmaSz, kFull>;
  static thread_local int configured_device = -1;
  int device = 0;
  EI_CUDA(cudaGetDevice(&device));
  if (configured_device != device) {
    EI_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured_device = device;
  }
  launch(kernel, dim3(grid), dim3(kGemmThreads), smem, stream, pdl, maps, p, cfg);
}

// The instances that exist: TMA-staged scales with or without full slices, and the up-front fallback.
template <bool kHigh, bool kPair>
void dispatch_awq_staging(bool tma_sz, bool full, int grid, size_t smem, cudaStream_t stream, bool pdl,
                          const AwqTensorMaps& maps, const GemmParams& p, const AwqLaunch& cfg) {
  if (tma_sz && full) return launch_awq_instance<kHigh, kPair, true, true>(grid, smem, stream, pdl, maps, p, cfg);
  if (tma_sz) return launch_awq_instance<kHigh, kPair, true, false>(grid, smem, stream, pdl, maps, p, cfg);
  return launch_awq_instance<kHigh, kPair, false, false>(grid, smem, stream, pdl, maps, p, cfg);
}
void dispatch_awq(bool high, bool pair, bool tma_sz, bool full, int grid, size_t smem, cudaStream_t stream, bool pdl,
                  const AwqTensorMaps& maps, const GemmParams& p, const AwqLaunch& cfg) {
  if (high && pair) return dispatch_awq_staging<true, true>(tma_sz, full, grid, smem, stream, pdl, maps, p, cfg);
  if (high) return dispatch_awq_staging<true, false>(tma_sz, full, grid, smem, stream, pdl, maps, p, cfg);
  if (pair) return dispatch_awq_staging<false, true>(tma_sz, full, grid, smem, stream, pdl, maps, p, cfg);
  return dispatch_awq_staging<false, false>(tma_sz, full, grid, smem, stream, pdl, maps, p, cfg);
}

void launch_awq(const GemmPlan& plan, const GemmParams& p, cudaStream_t stream, bool pdl) {
  const int units_total = p.K / 256;
  AwqLaunch cfg{};
  cfg.tiles_per_block = plan.tiles_per_block;
  cfg.units_box = std::min(kAwqSliceUnits, units_total);
  const bool pair = p.epilogue == kEpiSiluPair;
  cfg.sz_boxes = pair ? 2 : 1;
  cfg.sz_rows = plan.tiles_per_block / cfg.sz_boxes * 8;
  // TMA needs 16-byte aligned bases and row pitches, and boxes of at most 256 rows.
  cfg.tma_sz = aligned_16(p.scales) && aligned_16(p.zeros) && p.padded_groups % 8 == 0 && p.zero_stride % 4 == 0 &&
               cfg.sz_rows <= 256;
  cfg.scale_box = cfg.tma_sz ? std::min(32, p.padded_groups) : 0;
  cfg.zero_box = cfg.tma_sz ? std::min(4, p.zero_stride) : 0;
  if (!cfg.tma_sz) cfg.sz_boxes = cfg.sz_rows = 0;
  cfg.stages = kAwqMaxStages;
  cfg.wait_limit = p.wait_limit;
  cfg.extra_tx = p.fault_tx;
  while (cfg.stages > kAwqPhaseTiles && awq_layout(cfg).total > plan.smem_limit) cfg.stages -= kAwqPhaseTiles;
  const size_t smem = awq_layout(cfg).total;
  if (smem > plan.smem_limit) throw std::invalid_argument("small-M int4 GEMM does not fit in shared memory");

  AwqTensorMaps maps{};
  {
    // Packed weights as [unit of 256 inputs][row][32 words]: a box is one tile, staged as [unit][row][128 B].
    const cuuint64_t dims[3] = {32, cuuint64_t(p.N), cuuint64_t(units_total)};
    const cuuint64_t strides[2] = {cuuint64_t(p.K / 8) * 4, 128};
    const cuuint32_t box[3] = {32, 8, cuuint32_t(cfg.units_box)};
    encode_map(&maps.weights, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, p.qweight, dims, strides, box,
               CU_TENSOR_MAP_SWIZZLE_128B, "weights");
  }
  if (cfg.tma_sz) {
    const cuuint64_t scale_dims[2] = {cuuint64_t(p.padded_groups), cuuint64_t(p.N)};
    const cuuint64_t scale_strides[1] = {cuuint64_t(p.padded_groups) * 2};
    const cuuint32_t scale_box[2] = {cuuint32_t(cfg.scale_box), cuuint32_t(cfg.sz_rows)};
    encode_map(&maps.scales, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, p.scales, scale_dims, scale_strides, scale_box,
               CU_TENSOR_MAP_SWIZZLE_NONE, "scales");
    const cuuint64_t zero_dims[2] = {cuuint64_t(p.zero_stride), cuuint64_t(p.N)};
    const cuuint64_t zero_strides[1] = {cuuint64_t(p.zero_stride) * 4};
    const cuuint32_t zero_box[2] = {cuuint32_t(cfg.zero_box), cuuint32_t(cfg.sz_rows)};
    encode_map(&maps.zeros, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, p.zeros, zero_dims, zero_strides, zero_box,
               CU_TENSOR_MAP_SWIZZLE_NONE, "zero points");
  }

  const bool full = units_total % kAwqSliceUnits == 0;
  dispatch_awq(plan.high, pair, cfg.tma_sz != 0, full && cfg.tma_sz != 0, plan.grid, smem, stream, pdl, maps, p, cfg);
}

// The TMA-fed BF16 kernel takes weights whose rows are 16-byte aligned and K in steps of a warp's 256 inputs.
bool dense_tma_eligible(const GemmPlan& plan, const GemmParams& p) {
  if (p.K % kDenseWarpInputs || !aligned_16(p.w) || p.ldw % 8 || !aligned_16(p.x) || p.x_stride % 8) return false;
  const int parts_total = p.K / kDenseWarpInputs;
  if ((parts_total + plan.ksplit - 1) / plan.ksplit > kGemmWarps) return false;
  const DenseLaunch smallest{2, std::min(64, ((parts_total + plan.ksplit - 1) / plan.ksplit) * 4)};
  return dense_layout(smallest).total <= plan.smem_limit;
}

void launch_dense_tma(const GemmPlan& plan, const GemmParams& p, cudaStream_t stream, bool pdl) {
  const int parts_total = p.K / kDenseWarpInputs;
  DenseLaunch cfg{};
  cfg.units_box = std::min(64, ((parts_total + plan.ksplit - 1) / plan.ksplit) * 4);  // the largest slice
  cfg.stages = kDenseMaxStages;
  cfg.wait_limit = p.wait_limit;
  cfg.extra_tx = p.fault_tx;
  while (cfg.stages > 2 && dense_layout(cfg).total > plan.smem_limit) --cfg.stages;
  const size_t smem = dense_layout(cfg).total;
  CUtensorMap weights{};
  {
    // BF16 weights as [unit of 64 inputs][row][64 values]: a box is one tile, staged as [unit][row][128 B].
    const cuuint64_t dims[3] = {64, cuuint64_t(p.N), cuuint64_t(p.K / 64)};
    const cuuint64_t strides[2] = {cuuint64_t(p.ldw) * 2, 128};
    const cuuint32_t box[3] = {64, 8, cuuint32_t(cfg.units_box)};
    encode_map(&weights, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, p.w, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
               "dense weights");
  }
  static thread_local int configured_device = -1;
  int device = 0;
  EI_CUDA(cudaGetDevice(&device));
  if (configured_device != device) {
    EI_CUDA(cudaFuncSetAttribute(dense_tma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    EI_CUDA(cudaFuncSetAttribute(dense_tma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured_device = device;
  }
  if (plan.high)
    launch(dense_tma_kernel<true>, dim3(plan.grid), dim3(kGemmThreads), smem, stream, pdl, weights, p, cfg);
  else
    launch(dense_tma_kernel<false>, dim3(plan.grid), dim3(kGemmThreads), smem, stream, pdl, weights, p, cfg);
}

}  // namespace

void launch_gemm(const GemmPlan& plan, bool awq, const GemmParams& p, cudaStream_t stream, bool pdl) {
  if (awq) return launch_awq(plan, p, stream, pdl);
  if (dense_tma_eligible(plan, p)) return launch_dense_tma(plan, p, stream, pdl);
  const int U = plan.units_per_warp;
  if (U == 1) return launch_high<1, 6, 6>(plan, p, stream, pdl);
  if (U == 2) return launch_high<2, 4, 4>(plan, p, stream, pdl);
  if (U == 4) return launch_high<4, 2, 2>(plan, p, stream, pdl);
  throw std::invalid_argument("small-M GEMM plan has no kernel instance");
}

}  // namespace ei
