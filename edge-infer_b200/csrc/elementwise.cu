// Normalisation, rotary embedding, residual and KV-append kernels of the verify step.
//
// BF16 rounding contracts follow the reference CUDA operators so that the staged values
// agree: RMSNorm rounds x * inv_rms to BF16 and then the weighted product
// (operators/src/cuda/rms_norm_cuda.cu:87-95), and its sum of squares is taken in the reference kernel's own
// order (1024 threads, thread t owns elements t, t + 1024, ...; a shuffle tree per warp, then one over the 32 warp
// sums; the mean by the fast division its build uses), so that the inverse RMS has the same bits (:27-72); RoPE rounds the table's sine and cosine, each of
// the four products and both sums (operators/src/cuda/execution.cu:104-117); the residual
// add is one rounded FP32 sum of two BF16 values (operators/src/cuda/add_cuda.cu:42-62).
#include "kernels.cuh"
#include "smallm_gemm.cuh"

namespace ei {
namespace {

constexpr int kNormThreads = 1024;      // the reference's block size: the order of the sum depends on it
constexpr int kNormMaxPerThread = 10;   // 10240 / 1024, the reference's width limit

// Sum over the block of every thread's value, in the order of the reference kernel: the shuffle tree of a warp
// (lane 0's result of offsets 16, 8, 4, 2, 1), then the same tree over the 32 warp sums. Every thread gets it.
__device__ __forceinline__ float block_sum(float v, float* shared) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) shared[warp] = v;
  __syncthreads();
  const float total = warp_sum(shared[lane]);
  __syncthreads();
  return total;
}

// 1 / sqrt(mean + eps) as the reference computes it (its build divides with the fast reciprocal-multiply).
__device__ __forceinline__ float inverse_rms(float sum_of_squares, int width, float eps) {
  return rsqrtf(__fdividef(sum_of_squares, float(width)) + eps);
}

__global__ void __launch_bounds__(kNormThreads) rms_norm_kernel(const bf16* in, const bf16* weight,
                                                               bf16* out, int width, float eps) {
  __shared__ float shared[32];
  grid_dependency_wait();
  const bf16* x = in + size_t(blockIdx.x) * width;
  bf16* y = out + size_t(blockIdx.x) * width;
  float values[kNormMaxPerThread];
  float sum = 0.0f;
#pragma unroll
  for (int j = 0; j < kNormMaxPerThread; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
    values[j] = i < width ? __bfloat162float(x[i]) : 0.0f;
    if (i < width) sum = fmaf(values[j], values[j], sum);
  }
  const float inv = inverse_rms(block_sum(sum, shared), width, eps);
  grid_launch_dependents();
#pragma unroll
  for (int j = 0; j < kNormMaxPerThread; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
    if (i < width) y[i] = __float2bfloat16_rn(round_bf16(values[j] * inv) * __bfloat162float(weight[i]));
  }
}

__global__ void add_kernel(const bf16* a, const bf16* b, bf16* out, size_t count) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += size_t(gridDim.x) * blockDim.x)
    out[i] = __float2bfloat16_rn(__bfloat162float(a[i]) + __bfloat162float(b[i]));
}

__global__ void silu_multiply_kernel(const bf16* gate, const bf16* up, bf16* out, size_t count) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += size_t(gridDim.x) * blockDim.x)
    out[i] = __float2bfloat16_rn(silu_multiply_value(__bfloat162float(gate[i]), __bfloat162float(up[i])));
}

__global__ void gather_kernel(const uint32_t* ids, const bf16* table, bf16* out, size_t count, size_t width,
                              size_t vocabulary) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += size_t(gridDim.x) * blockDim.x) {
    const uint32_t token = ids[i / width];
    out[i] = token < vocabulary ? table[size_t(token) * width + i % width] : __float2bfloat16_rn(0.0f);
  }
}

__device__ __forceinline__ void rotate_pair(float x, float y, float sine, float cosine, float& first,
                                            float& second) {
  sine = round_bf16(sine);
  cosine = round_bf16(cosine);
  first = round_bf16(round_bf16(x * cosine) - round_bf16(y * sine));
  second = round_bf16(round_bf16(x * sine) + round_bf16(y * cosine));
}

__global__ void rope_kernel(bf16* data, size_t row_stride, size_t head_dim, const float* table,
                            size_t table_stride, size_t offset, const size_t* offsets, const int* pingpong) {
  const size_t pair = threadIdx.x, half = head_dim / 2;
  if (pair >= half) return;
  const size_t position = blockIdx.x + (offsets ? offsets[pingpong ? *pingpong : 0] : offset);
  bf16* head = data + size_t(blockIdx.x) * row_stride + size_t(blockIdx.y) * head_dim;
  float first, second;
  rotate_pair(__bfloat162float(head[pair]), __bfloat162float(head[pair + half]),
              table[position * table_stride + 2 * pair], table[position * table_stride + 2 * pair + 1], first,
              second);
  head[pair] = __float2bfloat16_rn(first);
  head[pair + half] = __float2bfloat16_rn(second);
}

__global__ void store_kv_kernel(const bf16* source, bf16* cache, size_t count, size_t rows, size_t width,
                                size_t capacity, size_t offset, const size_t* device_offset) {
  const size_t start_row = device_offset ? *device_offset : offset;
  if (start_row > capacity || rows > capacity - start_row) return;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += size_t(gridDim.x) * blockDim.x)
    cache[start_row * width + i] = source[i];
}

__global__ void __launch_bounds__(kNormThreads) embed_norm_kernel(const EmbedParams p) {
  __shared__ float shared[32];
  __shared__ uint32_t token_shared;
  grid_dependency_wait();
  const int row = blockIdx.x;
  if (threadIdx.x == 0) {
    uint32_t token;
    if (p.tokens) {
      token = p.tokens[row];
    } else if (row == 0) {
      token = p.control->pending;
    } else {
      const DraftSource source = *p.source;
      const long long index = (long long)p.control->context + row - source.base;
      token = (source.drafts && index >= 0 && index < source.count) ? source.drafts[index] : 0u;
    }
    p.step_tokens[row] = token;
    if (token >= uint32_t(p.vocab)) atomicOr(&p.control->status, 2);
    if (row == 0 && p.control->context + p.rows > p.capacity) atomicOr(&p.control->status, 1);
    token_shared = token;
  }
  __syncthreads();
  const uint32_t token = token_shared;
  const bf16* source = p.table + size_t(token < uint32_t(p.vocab) ? token : 0) * p.hidden;
  bf16* residual = p.residual + size_t(row) * p.hidden;
  bf16* normed = p.normed + size_t(row) * p.hidden;
  float values[kNormMaxPerThread];
  float sum = 0.0f;
#pragma unroll
  for (int j = 0; j < kNormMaxPerThread; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
    float value = 0.0f;
    if (i < p.hidden) {
      const bf16 raw = token < uint32_t(p.vocab) ? source[i] : __float2bfloat16_rn(0.0f);
      residual[i] = raw;
      value = __bfloat162float(raw);
    }
    values[j] = value;
    if (i < p.hidden) sum = fmaf(value, value, sum);
  }
  const float inv = inverse_rms(block_sum(sum, shared), p.hidden, p.eps);
  grid_launch_dependents();
#pragma unroll
  for (int j = 0; j < kNormMaxPerThread; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
    if (i < p.hidden)
      normed[i] = __float2bfloat16_rn(round_bf16(values[j] * inv) * __bfloat162float(p.norm_weight[i]));
  }
}

// projection = round(sum of the K-slice partials + bias); residual = round(residual + projection);
// normed = RMSNorm(residual). Thread t owns features t, t + 1024, ... as the reference's norm kernel does, and
// every load of a thread (residual, bias, norm weights before the dependency wait; the partial slices after it)
// is issued before its first use, so a row costs about one memory latency instead of one per slice.
template <int kPerThread>
__global__ void __launch_bounds__(kNormThreads) residual_norm_kernel(const ResidualNormParams p) {
  __shared__ float shared[32];
  const int row = blockIdx.x;
  bf16* residual = p.residual + size_t(row) * p.hidden;
  bf16* normed = p.normed + size_t(row) * p.hidden;
  const size_t slice = size_t(p.rows) * p.hidden;
  const float* partial = p.partial + size_t(row) * p.hidden;
  float old_residual[kPerThread], bias[kPerThread], weight[kPerThread];
#pragma unroll
  for (int j = 0; j < kPerThread; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
    old_residual[j] = bias[j] = weight[j] = 0.0f;
    if (i < p.hidden) {
      old_residual[j] = __bfloat162float(residual[i]);
      if (p.bias) bias[j] = __bfloat162float(p.bias[i]);
      weight[j] = __bfloat162float(p.norm_weight[i]);
    }
  }
  grid_dependency_wait();
  grid_launch_dependents();
  float values[kPerThread];
  float sum = 0.0f;
  float slices[kPerThread][4];
#pragma unroll
  for (int j = 0; j < kPerThread; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
#pragma unroll
    for (int s = 0; s < 4; ++s) slices[j][s] = (i < p.hidden && s < p.ksplit) ? partial[s * slice + i] : 0.0f;
  }
#pragma unroll
  for (int j = 0; j < kPerThread; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
    values[j] = 0.0f;
    if (i < p.hidden) {
      float projection = ((slices[j][0] + slices[j][1]) + slices[j][2]) + slices[j][3];
      for (int s = 4; s < p.ksplit; ++s) projection += partial[s * slice + i];
      const float v = round_bf16(old_residual[j] + round_bf16(projection + bias[j]));
      residual[i] = __float2bfloat16_rn(v);
      values[j] = v;
      sum = fmaf(v, v, sum);
    }
  }
  const float inv = inverse_rms(block_sum(sum, shared), p.hidden, p.eps);
#pragma unroll
  for (int j = 0; j < kPerThread; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
    if (i < p.hidden) normed[i] = __float2bfloat16_rn(round_bf16(values[j] * inv) * weight[j]);
  }
}

int blocks_for(size_t count, int multiprocessors) {
  return int(std::max<size_t>(1, std::min<size_t>((count + 255) / 256, size_t(multiprocessors) * 32)));
}

}  // namespace

void launch_rms_norm(const bf16* in, const bf16* weight, bf16* out, size_t rows, size_t width, float eps,
                     cudaStream_t stream, bool pdl) {
  launch(rms_norm_kernel, dim3(unsigned(rows)), dim3(kNormThreads), 0, stream, pdl, in, weight, out,
         int(width), eps);
}

void launch_add(const bf16* a, const bf16* b, bf16* out, size_t count, cudaStream_t stream) {
  add_kernel<<<blocks_for(count, 148), 256, 0, stream>>>(a, b, out, count);
  check_launch();
}

void launch_silu_multiply(const bf16* gate, const bf16* up, bf16* out, size_t count, cudaStream_t stream) {
  silu_multiply_kernel<<<blocks_for(count, 148), 256, 0, stream>>>(gate, up, out, count);
  check_launch();
}

void launch_gather(const uint32_t* ids, const bf16* table, bf16* out, size_t rows, size_t width,
                   size_t vocabulary, int multiprocessors, cudaStream_t stream) {
  gather_kernel<<<blocks_for(rows * width, multiprocessors), 256, 0, stream>>>(ids, table, out, rows * width,
                                                                             width, vocabulary);
  check_launch();
}

void launch_rope(bf16* data, size_t rows, size_t heads, size_t head_dim, size_t row_stride, const float* table,
                 size_t table_stride, size_t offset, const size_t* offsets, const int* pingpong,
                 cudaStream_t stream) {
  rope_kernel<<<dim3(unsigned(rows), unsigned(heads)), unsigned(head_dim / 2), 0, stream>>>(
      data, row_stride, head_dim, table, table_stride, offset, offsets, pingpong);
  check_launch();
}

void launch_store_kv(const bf16* source, bf16* cache, size_t rows, size_t width, size_t capacity, size_t offset,
                     const size_t* device_offset, int multiprocessors, cudaStream_t stream) {
  store_kv_kernel<<<blocks_for(rows * width, multiprocessors), 256, 0, stream>>>(
      source, cache, rows * width, rows, width, capacity, offset, device_offset);
  check_launch();
}

void launch_embed_norm(const EmbedParams& p, cudaStream_t stream, bool pdl) {
  launch(embed_norm_kernel, dim3(p.rows), dim3(kNormThreads), 0, stream, pdl, p);
}

void launch_residual_norm(const ResidualNormParams& p, cudaStream_t stream, bool pdl) {
  if (p.hidden <= kNormThreads * 4)
    launch(residual_norm_kernel<4>, dim3(p.rows), dim3(kNormThreads), 0, stream, pdl, p);
  else
    launch(residual_norm_kernel<kNormMaxPerThread>, dim3(p.rows), dim3(kNormThreads), 0, stream, pdl, p);
}

}  // namespace ei
