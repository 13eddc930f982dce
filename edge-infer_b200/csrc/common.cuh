// Shared device/host helpers for the sm_100a verify-step kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/edge_infer_b200.h"

namespace ei {

// Exceptions mirror the reference operator API's error types
// (operators/src/cuda/execution.cu:15-58); the C-ABI layer maps them to ei_status.
struct LengthError : std::length_error {
  using std::length_error::length_error;
};

inline void check_cuda(cudaError_t status, const char* what) {
  if (status != cudaSuccess)
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(status));
}
#define EI_CUDA(call) ::ei::check_cuda((call), #call)

inline void check_launch() { check_cuda(cudaGetLastError(), "kernel launch"); }

using bf16 = __nv_bfloat16;

constexpr int kWarp = 32;

// ----------------------------------------------------------------------- device helpers
#if defined(__CUDACC__)

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}
__device__ __forceinline__ float bf16_lo(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t pair) { return __uint_as_float(pair & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float round_bf16(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}
__device__ __forceinline__ uint16_t bf16_bits(float x) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(x));
}

// 128-bit read-only load that does not allocate in L1 (streamed weights).
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_cached(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The same MMA starting a sum: the accumulator input is zero, so the destination needs no clearing first.
__device__ __forceinline__ void mma_bf16_16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                     uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// Programmatic dependent launch: wait until the kernels this one depends on have
// completed and flushed (no-op when launched without the attribute).
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
// Allow the dependent kernel to begin launching (its own wait still orders data).
// Rule kept by every kernel of this library: trigger only after the kernel's own grid_dependency_wait().
// Then, whenever the code a successor runs before ITS wait executes, everything up to this kernel's
// predecessor has completed, so such code may read weights, tables and anything written two or more
// kernels earlier (the context length, settled KV rows) - and nothing newer. Triggering at entry would let
// a chain of kernels run ahead of work that is still in flight.
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

#endif  // __CUDACC__

// ----------------------------------------------------------------------- launch helper
// Launches with the programmatic-stream-serialization attribute when `pdl` is set, so a
// kernel's independent prologue (weight prefetch) overlaps the tail of its predecessor.
template <typename... KernelArgs, typename... Args>
inline void launch(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                   cudaStream_t stream, bool pdl, Args&&... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = pdl ? 1 : 0;
  check_cuda(cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...), "cudaLaunchKernelEx");
}

}  // namespace ei
