// Host side of the prompt GEMM: eligibility, tensor maps, launch.
#include "prompt_gemm.cuh"

#include <algorithm>
#include <stdexcept>

namespace ei {

namespace {
bool aligned_16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
}  // namespace

bool prompt_gemm_eligible(bool awq, int group_size, int N, int K, const void* x, int x_stride, const void* out,
                          int out_stride) {
  if (N < 16 || N % 16 || K < kPromptBlockK || K % kPromptBlockK) return false;
  if (awq && (group_size != 128 || K % 128)) return false;
  return aligned_16(x) && x_stride % 8 == 0 && aligned_16(out) && out_stride % 8 == 0;
}

// A block with two token tiles dequantises every weight once for 256 rows and reads less per flop; a block with
// one tile is not half as long but about three quarters (measured: the dequantisation and the operand traffic do
// not shrink with the rows). What decides is how the grid falls into waves of one block per SM: the cost of a
// choice is waves x block time, ties going to two tiles.
int prompt_gemm_tiles(int rows, int N, int multiprocessors) {
  const int n_tiles = (N + kPromptFeatures - 1) / kPromptFeatures;
  const int token_tiles = (rows + kPromptTokens - 1) / kPromptTokens;
  if (token_tiles < 2) return 1;
  auto waves = [&](int per_block) {
    const int blocks = n_tiles * ((token_tiles + per_block - 1) / per_block);
    return (blocks + multiprocessors - 1) / multiprocessors;
  };
  return waves(1) * 3 < waves(2) * 4 ? 1 : 2;
}

// Slices of K that bring the grid to about one block per SM, each slice at least 8 K blocks long, within the
// room of the partial buffer.
int prompt_gemm_ksplit(int rows, int N, int K, int multiprocessors, size_t partial_bytes) {
  const int per_block = prompt_gemm_tiles(rows, N, multiprocessors) * kPromptTokens;
  const int blocks = ((N + kPromptFeatures - 1) / kPromptFeatures) * ((rows + per_block - 1) / per_block);
  int ksplit = std::max(1, multiprocessors / std::max(1, blocks));
  ksplit = std::min(ksplit, std::max(1, K / (8 * kPromptBlockK)));
  ksplit = std::min(ksplit, 16);
  if (K % 128) ksplit = 1;
  while (ksplit > 1 && size_t(ksplit) * rows * N * sizeof(float) > partial_bytes) --ksplit;
  return ksplit;
}

void launch_prompt_gemm(bool awq, const GemmParams& p, cudaStream_t stream, bool pdl) {
  if (p.M < 1) throw std::invalid_argument("prompt GEMM needs at least one row");
  PromptMaps maps{};
  {
    const cuuint64_t dims[2] = {cuuint64_t(p.K), cuuint64_t(p.M)};
    const cuuint64_t strides[1] = {cuuint64_t(p.x_stride) * 2};
    const cuuint32_t box[2] = {kPromptBlockK, kPromptTokens};
    encode_map(&maps.x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.x, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
               "prompt activations");
  }
  if (awq) {
    if (!aligned_16(p.qweight) || (p.K / 8) % 4) throw std::invalid_argument("prompt GEMM: packed weight rows must be 16-byte aligned");
    const cuuint64_t dims[2] = {cuuint64_t(p.K / 8), cuuint64_t(p.N)};
    const cuuint64_t strides[1] = {cuuint64_t(p.K / 8) * 4};
    const cuuint32_t box[2] = {kPromptBlockK / 8, kPromptFeatures};
    encode_map(&maps.weights, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, p.qweight, dims, strides, box,
               CU_TENSOR_MAP_SWIZZLE_NONE, "prompt int4 weights");
  } else {
    if (!aligned_16(p.w) || p.ldw % 8) throw std::invalid_argument("prompt GEMM: weight rows must be 16-byte aligned");
    const cuuint64_t dims[2] = {cuuint64_t(p.K), cuuint64_t(p.N)};
    const cuuint64_t strides[1] = {cuuint64_t(p.ldw) * 2};
    const cuuint32_t box[2] = {kPromptBlockK, kPromptFeatures};
    encode_map(&maps.weights, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.w, dims, strides, box,
               CU_TENSOR_MAP_SWIZZLE_128B, "prompt weights");
  }
  static thread_local int configured_device = -1, multiprocessors = 0;
  int device = 0;
  EI_CUDA(cudaGetDevice(&device));
  if (configured_device != device) {
    EI_CUDA(cudaDeviceGetAttribute(&multiprocessors, cudaDevAttrMultiProcessorCount, device));
    EI_CUDA(cudaFuncSetAttribute(prompt_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(kPromptSharedBytes)));
    EI_CUDA(cudaFuncSetAttribute(prompt_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(kPromptSharedBytes)));
    configured_device = device;
  }
  const int ksplit = p.epilogue == kEpiPartial ? std::max(1, p.ksplit) : 1;
  if (p.epilogue != kEpiStore && p.epilogue != kEpiPartial)
    throw std::invalid_argument("prompt GEMM stores BF16 outputs or FP32 partial sums");
  if (ksplit > 1 && (p.K % 128 || ksplit > p.K / 128)) throw std::invalid_argument("prompt GEMM: K split too fine");
  if (p.epilogue == kEpiPartial && (!p.partial || (reinterpret_cast<uintptr_t>(p.partial) & 15) || p.N % 4))
    throw std::invalid_argument("prompt GEMM: partial sums need a 16-byte aligned buffer");
  GemmParams q = p;
  q.ksplit = ksplit;
  if (q.prompt_tiles != 1 && q.prompt_tiles != 2) q.prompt_tiles = prompt_gemm_tiles(p.M, p.N, multiprocessors);
  const int rows_per_block = kPromptTokens * q.prompt_tiles;
  const dim3 grid((p.N + kPromptFeatures - 1) / kPromptFeatures, (p.M + rows_per_block - 1) / rows_per_block, ksplit);
  if (awq)
    launch(prompt_gemm_kernel<true>, grid, dim3(kPromptThreads), kPromptSharedBytes, stream, pdl, maps, q);
  else
    launch(prompt_gemm_kernel<false>, grid, dim3(kPromptThreads), kPromptSharedBytes, stream, pdl, maps, q);
}

}  // namespace ei
