// Row arithmetic shared by the kernels that normalise and rotate head vectors: the reference's rounding points and
// summation orders in one place.
#pragma once

#include "common.cuh"

namespace ei {

// 1 / sqrt(mean + eps) as the reference computes it (its build divides with the fast reciprocal-multiply).
__device__ __forceinline__ float inverse_rms(float sum_of_squares, int width, float eps) {
  return rsqrtf(__fdividef(sum_of_squares, float(width)) + eps);
}

// One rotation pair of half-split RoPE with the reference's BF16 staging (operators/src/cuda/execution.cu:79-122):
// sine, cosine, both products and the sum are rounded.
__device__ __forceinline__ void rotate_pair(float x, float y, float sine, float cosine, float& first,
                                            float& second) {
  sine = round_bf16(sine);
  cosine = round_bf16(cosine);
  first = round_bf16(round_bf16(x * cosine) - round_bf16(y * sine));
  second = round_bf16(round_bf16(x * sine) + round_bf16(y * cosine));
}

// Inverse RMS of a 128-wide head row with the sum of squares in the order of the reference's norm kernel
// (operators/src/cuda/rms_norm_cuda.cu:27-72 run over [rows * heads, 128]: one element per thread, a shuffle tree
// over each block of 32 elements - offsets 16, 8, 4, 2, 1 - and the four block sums combined as
// (p0 + p2) + (p1 + p3)), so that it has the reference's bits. Lane l of the warp holds elements 2l, 2l+1
// (x0, x1) and 64+2l, 64+2l+1 (y0, y1).
__device__ __forceinline__ float head_inverse_rms(float x0, float x1, float y0, float y1, float eps) {
  float a = x0 * x0, b = x1 * x1, a2 = y0 * y0, b2 = y1 * y1;
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) {  // element offsets 16, 8, 4, 2 inside a block of 32 elements = 16 lanes
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
    a2 += __shfl_xor_sync(0xffffffffu, a2, o);
    b2 += __shfl_xor_sync(0xffffffffu, b2, o);
  }
  const float q = (a + b) + (a2 + b2);  // lanes 0-15: p0 + p2, lanes 16-31: p1 + p3
  const float total = q + __shfl_xor_sync(0xffffffffu, q, 16);
  return rsqrtf(__fdividef(total, 128.0f) + eps);
}

}  // namespace ei
