// mbarrier and tensor-memory-accelerator (TMA) helpers shared by the kernels that stage their operands with
// cp.async.bulk.tensor: bounded waits, tiled loads, and the host-side tensor-map encoder.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace ei {

constexpr uint32_t kTmaWaitLimit = 1u << 22;  // polls of ~100 ns before a bounded wait gives up

#if defined(__CUDACC__)
__device__ __forceinline__ uint32_t smem_address(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbarrier_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_address(bar)), "r"(count));
}
__device__ __forceinline__ void mbarrier_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_address(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbarrier_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 100;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_address(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbarrier_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_address(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// Bounded wait; false if the phase did not complete within the limit. The non-blocking test comes first: a
// try_wait with a time hint costs a few hundred cycles even when the phase has long completed, which is the
// normal case here (the ring runs ahead of the arithmetic).
__device__ __forceinline__ bool mbarrier_wait(uint64_t* bar, uint32_t parity, uint32_t limit = kTmaWaitLimit) {
  if (mbarrier_test_wait(bar, parity)) return true;
  for (uint32_t polls = 0; polls < limit; ++polls)
    if (mbarrier_try_wait(bar, parity)) return true;
  return false;
}
// Tiled TMA loads; coordinates run from the innermost dimension outwards. x times the element size must be
// a multiple of 16 bytes (the callers below only pass multiples of whole slices).
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
          "r"(smem_address(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_address(bar))
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], "
      "[%5];" ::"r"(smem_address(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(smem_address(bar))
      : "memory");
}
__device__ __forceinline__ void tma_load_5d(void* dst, const CUtensorMap* map, int x, int y, int z, int w, int v,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, "
      "%6}], [%7];" ::"r"(smem_address(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(w), "r"(v), "r"(smem_address(bar))
      : "memory");
}
#endif  // __CUDACC__

// Encodes a tiled tensor map of rank <= 5 (element strides 1; 256-byte L2 promotion; out-of-range elements read
// as zero). Throws std::runtime_error with `what` in the message if the driver refuses the description.
void encode_map(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base, const cuuint64_t* dims,
                const cuuint64_t* strides, const cuuint32_t* box, CUtensorMapSwizzle swizzle, const char* what);

}  // namespace ei
