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
#include "head_math.cuh"
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

// ---- the direct operators' copy-shaped kernels: 16 bytes per thread where the operands allow it ------------

// Embedding lookup: row r of `out` is row ids[r] of `table`, or zeros for an id outside the table. A thread moves
// one 16-byte piece (8 values) of a row; `pieces` = pieces per row (rows are 16-byte aligned multiples of 8 values).
__global__ void gather_rows_vec_kernel(const uint32_t* ids, const uint4* table, uint4* out, size_t rows, size_t pieces,
                                       size_t vocabulary) {
  const size_t total = rows * pieces;
  for (size_t at = size_t(blockIdx.x) * blockDim.x + threadIdx.x; at < total; at += size_t(gridDim.x) * blockDim.x) {
    const size_t row = at / pieces, piece = at - row * pieces;
    const uint32_t token = ids[row];
    out[at] = token < vocabulary ? table[size_t(token) * pieces + piece] : make_uint4(0, 0, 0, 0);
  }
}
// Any width or alignment: one value per thread.
__global__ void gather_rows_kernel(const uint32_t* ids, const bf16* table, bf16* out, size_t rows, size_t width,
                                   size_t vocabulary) {
  const size_t total = rows * width;
  for (size_t at = size_t(blockIdx.x) * blockDim.x + threadIdx.x; at < total; at += size_t(gridDim.x) * blockDim.x) {
    const size_t row = at / width, column = at - row * width;
    const uint32_t token = ids[row];
    out[at] = token < vocabulary ? table[size_t(token) * width + column] : __float2bfloat16_rn(0.0f);
  }
}

// Half-split RoPE in place over [rows, heads, width]: a thread owns rotation pair `pair` of one head row,
// i.e. elements pair and pair + width / 2; the table row of position p holds (sine, cosine) of pair i at
// [2 i, 2 i + 1]. The first row's position comes from the host or, in a captured graph, from device memory.
__global__ void rope_pairs_kernel(bf16* data, size_t rows, size_t heads, size_t width, size_t row_stride,
                                  const float* table, size_t table_stride, size_t host_offset,
                                  const size_t* device_offsets, const int* which_offset) {
  const size_t half = width / 2, total = rows * heads * half;
  const size_t first_position = device_offsets ? device_offsets[which_offset ? *which_offset : 0] : host_offset;
  for (size_t at = size_t(blockIdx.x) * blockDim.x + threadIdx.x; at < total; at += size_t(gridDim.x) * blockDim.x) {
    const size_t pair = at % half, head = (at / half) % heads, row = at / (half * heads);
    bf16* values = data + row * row_stride + head * width;
    const float2 trig = *reinterpret_cast<const float2*>(table + (first_position + row) * table_stride + 2 * pair);
    float first, second;
    rotate_pair(__bfloat162float(values[pair]), __bfloat162float(values[pair + half]), trig.x, trig.y, first, second);
    values[pair] = __float2bfloat16_rn(first);
    values[pair + half] = __float2bfloat16_rn(second);
  }
}

// KV append: `rows` packed rows of `width` values land at cache row `first` (host value or device word). A
// request that would pass the capacity writes nothing.
template <typename Piece>
__global__ void append_rows_kernel(const Piece* source, Piece* cache, size_t pieces, size_t pieces_per_row, size_t rows,
                                   size_t capacity, size_t host_first, const size_t* device_first) {
  const size_t first = device_first ? *device_first : host_first;
  if (first > capacity || rows > capacity - first) return;
  Piece* target = cache + first * pieces_per_row;
  for (size_t at = size_t(blockIdx.x) * blockDim.x + threadIdx.x; at < pieces; at += size_t(gridDim.x) * blockDim.x)
    target[at] = source[at];
}

__global__ void __launch_bounds__(kNormThreads) embed_norm_kernel(const EmbedParams p) {
  __shared__ float shared[32];
  __shared__ uint32_t token_shared;
  grid_dependency_wait();
  const int row = blockIdx.x;
  if (threadIdx.x == 0) {
    Control* control = p.control;
    int local = row, step_rows = p.rows, capacity = p.capacity;
    if (p.slots) {
      const int session = row / p.rows_per_session;
      local = row - session * p.rows_per_session;
      step_rows = p.rows_per_session;
      control = p.slots[session].control;
      capacity = p.slots[session].capacity;
    }
    uint32_t token;
    if (p.tokens) {
      token = p.tokens[row];
    } else if (local == 0) {
      token = control->pending;
    } else {
      const DraftSource source = *p.source;
      const long long index = (long long)control->context + local - source.base;
      token = (source.drafts && index >= 0 && index < source.count) ? source.drafts[index] : 0u;
    }
    p.step_tokens[row] = token;
    if (token >= uint32_t(p.vocab)) atomicOr(&control->status, 2);
    if (local == 0 && control->context + step_rows > capacity) atomicOr(&control->status, 1);
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

// One warp per (row, head); lane l owns rotation pairs 2l and 2l+1, i.e. elements
// {2l, 2l+1} of the first half and {64+2l, 64+2l+1} of the second.
__global__ void __launch_bounds__(128) qk_norm_rope_store_kernel(const QkvParams p) {
  const int warp_global = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int per_row = p.heads + 2 * p.kv_heads;
  if (warp_global >= p.rows * per_row) return;
  const int row = warp_global / per_row, slot = warp_global - row * per_row;
  // Read before waiting for the projection: the context length (written by the previous step), the norm
  // weights and the rotation table do not come from it, so their latency overlaps its tail.
  const Control* control = p.control;
  bf16 *k_cache = p.k_cache, *v_cache = p.v_cache;
  int local = row, step_rows = p.rows, capacity = p.capacity;
  if (p.slots) {
    const int session = row / p.rows_per_session;
    const SessionSlot owner = p.slots[session];
    local = row - session * p.rows_per_session;
    step_rows = p.rows_per_session;
    control = owner.control;
    capacity = owner.capacity;
    const size_t layer_offset = size_t(p.layer) * size_t(capacity) * p.kv_heads * 128;
    k_cache = owner.k_cache + layer_offset;
    v_cache = owner.v_cache + layer_offset;
  }
  const int context = control->context;
  const int position = context + local;
  if (context + step_rows > capacity || position >= p.max_positions) {  // status set by the embed kernel
    grid_dependency_wait();  // every block leaves here: complete only after the predecessor has
    return;
  }
  const bool is_value = slot >= p.heads + p.kv_heads;
  const bool is_query = slot < p.heads;
  const bf16* norm = is_query ? p.q_norm : p.k_norm;
  uint32_t wl = 0, wh = 0;
  float4 trig = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  if (!is_value) {
    if (norm) {
      wl = *reinterpret_cast<const uint32_t*>(norm + 2 * lane);
      wh = *reinterpret_cast<const uint32_t*>(norm + 64 + 2 * lane);
    }
    trig = *reinterpret_cast<const float4*>(p.rope_table + size_t(position) * 128 + 4 * lane);
  }
  grid_dependency_wait();
  grid_launch_dependents();
  bf16* head = p.qkv + size_t(row) * p.qkv_stride + size_t(slot) * 128;
  if (is_value) {  // value head: append as is
    const int kvh = slot - p.heads - p.kv_heads;
    const uint2 v = *reinterpret_cast<const uint2*>(head + lane * 4);
    *reinterpret_cast<uint2*>(v_cache + (size_t(position) * p.kv_heads + kvh) * 128 + lane * 4) = v;
    return;
  }
  const uint32_t lo = *reinterpret_cast<const uint32_t*>(head + 2 * lane);
  const uint32_t hi = *reinterpret_cast<const uint32_t*>(head + 64 + 2 * lane);
  float x0 = bf16_lo(lo), x1 = bf16_hi(lo), y0 = bf16_lo(hi), y1 = bf16_hi(hi);
  if (norm) {
    const float inv = head_inverse_rms(x0, x1, y0, y1, p.eps);
    x0 = round_bf16(round_bf16(x0 * inv) * bf16_lo(wl));
    x1 = round_bf16(round_bf16(x1 * inv) * bf16_hi(wl));
    y0 = round_bf16(round_bf16(y0 * inv) * bf16_lo(wh));
    y1 = round_bf16(round_bf16(y1 * inv) * bf16_hi(wh));
  }
  float a0, b0, a1, b1;
  rotate_pair(x0, y0, trig.x, trig.y, a0, b0);
  rotate_pair(x1, y1, trig.z, trig.w, a1, b1);
  const uint32_t out_lo = pack_bf16(a0, a1), out_hi = pack_bf16(b0, b1);
  if (is_query) {
    *reinterpret_cast<uint32_t*>(head + 2 * lane) = out_lo;
    *reinterpret_cast<uint32_t*>(head + 64 + 2 * lane) = out_hi;
  } else {
    bf16* dst = k_cache + (size_t(position) * p.kv_heads + (slot - p.heads)) * 128;
    *reinterpret_cast<uint32_t*>(dst + 2 * lane) = out_lo;
    *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = out_hi;
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

// Vectorised form for hidden % 4 == 0: 1024 threads, each owning up to three groups of four consecutive
// features. Its sum of squares is taken in this layout's own order, not the reference kernel's: the inverse RMS
// may differ from the reference's in the last FP32 bit (the element-order form above costs 3 us more per launch,
// measured, for a difference far below that of the projections' accumulation orders). Every load of a thread (partial slices, bias, residual) is issued before the first use, so a
// row costs about one memory latency instead of one per slice.
constexpr int kRowThreads = 1024;
constexpr int kRowMaxGroups = 3;  // 1024 threads * 4 values * 3 groups >= 10240

__device__ __forceinline__ float4 load4_bf16(const bf16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  return make_float4(bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y));
}
__device__ __forceinline__ void store4_bf16(bf16* p, float4 v) {
  uint2 raw;
  raw.x = pack_bf16(v.x, v.y);
  raw.y = pack_bf16(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = raw;
}

// kRowGroups: groups of 4096 values a row needs (1 for hidden <= 4096), so that small rows keep few registers.
template <int kRowGroups>
__global__ void __launch_bounds__(kRowThreads) residual_norm_vec_kernel(const ResidualNormParams p) {
  __shared__ float shared[32];
  const int row = blockIdx.x;
  bf16* residual = p.residual + size_t(row) * p.hidden;
  bf16* normed = p.normed + size_t(row) * p.hidden;
  const size_t slice = size_t(p.rows) * p.hidden;
  const float* partial = p.partial + size_t(row) * p.hidden;
  const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  // Before waiting for the projection: the residual stream (last written several kernels ago), the bias and
  // the norm weights do not come from it.
  float4 old_residual[kRowGroups], bias[kRowGroups], weight[kRowGroups];
#pragma unroll
  for (int j = 0; j < kRowGroups; ++j) {
    const int i = (threadIdx.x + j * kRowThreads) * 4;
    old_residual[j] = bias[j] = weight[j] = zero;
    if (i < p.hidden) {
      old_residual[j] = load4_bf16(residual + i);
      if (p.bias) bias[j] = load4_bf16(p.bias + i);
      weight[j] = load4_bf16(p.norm_weight + i);
    }
  }
  grid_dependency_wait();
  grid_launch_dependents();
  float4 values[kRowGroups];
  float sum = 0.0f;
#pragma unroll
  for (int j = 0; j < kRowGroups; ++j) {
    const int i = (threadIdx.x + j * kRowThreads) * 4;
    values[j] = zero;
    if (i < p.hidden) {
      const float4 a0 = *reinterpret_cast<const float4*>(partial + i);
      const float4 a1 = p.ksplit > 1 ? *reinterpret_cast<const float4*>(partial + slice + i) : zero;
      const float4 a2 = p.ksplit > 2 ? *reinterpret_cast<const float4*>(partial + 2 * slice + i) : zero;
      const float4 a3 = p.ksplit > 3 ? *reinterpret_cast<const float4*>(partial + 3 * slice + i) : zero;
      const float4 r = old_residual[j], b = bias[j];
      float4 projection = make_float4(a0.x + a1.x, a0.y + a1.y, a0.z + a1.z, a0.w + a1.w);
      projection = make_float4(projection.x + a2.x, projection.y + a2.y, projection.z + a2.z, projection.w + a2.w);
      projection = make_float4(projection.x + a3.x, projection.y + a3.y, projection.z + a3.z, projection.w + a3.w);
      for (int s = 4; s < p.ksplit; ++s) {
        const float4 more = *reinterpret_cast<const float4*>(partial + s * slice + i);
        projection = make_float4(projection.x + more.x, projection.y + more.y, projection.z + more.z, projection.w + more.w);
      }
      float4 v;
      v.x = round_bf16(r.x + round_bf16(projection.x + b.x));
      v.y = round_bf16(r.y + round_bf16(projection.y + b.y));
      v.z = round_bf16(r.z + round_bf16(projection.z + b.z));
      v.w = round_bf16(r.w + round_bf16(projection.w + b.w));
      store4_bf16(residual + i, v);
      values[j] = v;
      sum = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, sum))));
    }
  }
  const float inv = inverse_rms(block_sum(sum, shared), p.hidden, p.eps);
#pragma unroll
  for (int j = 0; j < kRowGroups; ++j) {
    const int i = (threadIdx.x + j * kRowThreads) * 4;
    if (i < p.hidden) {
      const float4 w = weight[j];
      float4 out;
      out.x = round_bf16(values[j].x * inv) * w.x;
      out.y = round_bf16(values[j].y * inv) * w.y;
      out.z = round_bf16(values[j].z * inv) * w.z;
      out.w = round_bf16(values[j].w * inv) * w.w;
      store4_bf16(normed + i, out);
    }
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

void launch_add(const bf16* a, const bf16* b, bf16* out, size_t count, int multiprocessors, cudaStream_t stream) {
  add_kernel<<<blocks_for(count, multiprocessors), 256, 0, stream>>>(a, b, out, count);
  check_launch();
}

void launch_silu_multiply(const bf16* gate, const bf16* up, bf16* out, size_t count, int multiprocessors,
                          cudaStream_t stream) {
  silu_multiply_kernel<<<blocks_for(count, multiprocessors), 256, 0, stream>>>(gate, up, out, count);
  check_launch();
}

namespace {
bool sixteen_byte_aligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
}  // namespace

void launch_gather(const uint32_t* ids, const bf16* table, bf16* out, size_t rows, size_t width,
                   size_t vocabulary, int multiprocessors, cudaStream_t stream) {
  if (width % 8 == 0 && sixteen_byte_aligned(table) && sixteen_byte_aligned(out)) {
    const size_t pieces = width / 8;
    gather_rows_vec_kernel<<<blocks_for(rows * pieces, multiprocessors), 256, 0, stream>>>(
        ids, reinterpret_cast<const uint4*>(table), reinterpret_cast<uint4*>(out), rows, pieces, vocabulary);
  } else {
    gather_rows_kernel<<<blocks_for(rows * width, multiprocessors), 256, 0, stream>>>(ids, table, out, rows, width,
                                                                                   vocabulary);
  }
  check_launch();
}

void launch_rope(bf16* data, size_t rows, size_t heads, size_t head_dim, size_t row_stride, const float* table,
                 size_t table_stride, size_t offset, const size_t* offsets, const int* pingpong, int multiprocessors,
                 cudaStream_t stream) {
  rope_pairs_kernel<<<blocks_for(rows * heads * (head_dim / 2), multiprocessors), 256, 0, stream>>>(
      data, rows, heads, head_dim, row_stride, table, table_stride, offset, offsets, pingpong);
  check_launch();
}

void launch_store_kv(const bf16* source, bf16* cache, size_t rows, size_t width, size_t capacity, size_t offset,
                     const size_t* device_offset, int multiprocessors, cudaStream_t stream) {
  if (width % 8 == 0 && sixteen_byte_aligned(source) && sixteen_byte_aligned(cache)) {
    const size_t per_row = width / 8;
    append_rows_kernel<uint4><<<blocks_for(rows * per_row, multiprocessors), 256, 0, stream>>>(
        reinterpret_cast<const uint4*>(source), reinterpret_cast<uint4*>(cache), rows * per_row, per_row, rows, capacity,
        offset, device_offset);
  } else {
    append_rows_kernel<bf16><<<blocks_for(rows * width, multiprocessors), 256, 0, stream>>>(
        source, cache, rows * width, width, rows, capacity, offset, device_offset);
  }
  check_launch();
}

void launch_embed_norm(const EmbedParams& p, cudaStream_t stream, bool pdl) {
  launch(embed_norm_kernel, dim3(p.rows), dim3(kNormThreads), 0, stream, pdl, p);
}

void launch_qk_norm_rope_store(const QkvParams& p, cudaStream_t stream, bool pdl) {
  const int warps = p.rows * (p.heads + 2 * p.kv_heads);
  launch(qk_norm_rope_store_kernel, dim3((warps + 3) / 4), dim3(128), 0, stream, pdl, p);
}

void launch_residual_norm(const ResidualNormParams& p, cudaStream_t stream, bool pdl) {
  if (p.hidden % 4 != 0) {
    launch(residual_norm_kernel<kNormMaxPerThread>, dim3(p.rows), dim3(kNormThreads), 0, stream, pdl, p);
  } else if (p.hidden <= kRowThreads * 4) {
    launch(residual_norm_vec_kernel<1>, dim3(p.rows), dim3(kRowThreads), 0, stream, pdl, p);
  } else if (p.hidden <= kRowThreads * 8) {
    launch(residual_norm_vec_kernel<2>, dim3(p.rows), dim3(kRowThreads), 0, stream, pdl, p);
  } else {
    launch(residual_norm_vec_kernel<kRowMaxGroups>, dim3(p.rows), dim3(kRowThreads), 0, stream, pdl, p);
  }
}

}  // namespace ei
