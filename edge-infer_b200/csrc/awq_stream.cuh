// int4 (AWQ, group 128) small-M GEMM with bulk-copy staging: out[M,N] = x[M,K] * dequant(W)[N,K]^T (+ bias).
//
// A tile is 8 output features = 8 consecutive rows of the N-major packed weight matrix. Each row slice is
// brought into shared memory by one asynchronous bulk copy (cp.async.bulk, the 1-D form of TMA) that
// completes on an mbarrier; a ring of kStages tiles is always in flight per block, so HBM streams
// continuously and independently of the warps' register scoreboards, and the loop issues no global loads.
// Row slices land with a 16-byte skew between rows, which makes the warps' 128-bit reads conflict-free.
// The group scales and zero points of every tile the block will touch are fetched once into shared memory
// before the kernel waits for its predecessor, as are the first kStages tiles: weights do not depend on it.
//
// The <= 16 activation rows never change while the block runs and warp w always works on input features
// [256 w, 256 w + 256) of the block's K slice, so its A fragments are loaded once, in the register order
// mma.sync wants, and stay in registers: the inner loop is nibble extraction, the exact BF16 dequantisation
// (see dequant_pair) and mma.sync.m16n8k16 with FP32 accumulation. Per tile the 16 warps add their partial
// accumulators through shared memory in a fixed order. K beyond 4096 is split over blocks (ksplit) that write
// FP32 partials for a separate fixed-order reduction.
//
// Every wait on an mbarrier is bounded: if a copy does not complete within the limit the block records the
// failure in GemmParams::status and leaves without touching its outputs again.
#pragma once

#include "smallm_gemm.cuh"

namespace ei {

constexpr int kAwqStages = 8;
constexpr int kAwqRowSkew = 16;          // bytes added to each staged row
constexpr uint32_t kAwqWaitLimit = 1u << 22;  // polls of ~100 ns before a wait gives up

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
// Bounded wait; false if the phase did not complete within the limit.
__device__ __forceinline__ bool mbarrier_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t polls = 0; polls < kAwqWaitLimit; ++polls)
    if (mbarrier_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void bulk_copy_to_shared(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_address(dst)),
               "l"(src), "r"(bytes), "r"(smem_address(bar))
               : "memory");
}

struct AwqStreamLayout {
  int row_bytes;     // staged bytes per weight row (slice) incl. skew
  int stage_bytes;   // 8 rows
  int groups;        // scale groups of the slice
  int sz_tile_bytes; // scales + zero nibbles of one tile: 8 rows x groups x (2 + 1) bytes, 16-byte padded
  size_t part_offset, barrier_offset, sz_offset, stage_offset, total;
};

__host__ __device__ inline AwqStreamLayout awq_stream_layout(int units, int tiles_per_block) {
  AwqStreamLayout l;
  l.row_bytes = units * 128 + kAwqRowSkew;
  l.stage_bytes = 8 * l.row_bytes;
  l.groups = units * 2;
  l.sz_tile_bytes = ((8 * l.groups * 3) + 15) & ~15;
  l.part_offset = 0;
  l.barrier_offset = size_t(4) * kGemmWarps * 136 * sizeof(float);  // two buffers x two tiles of partials
  l.sz_offset = l.barrier_offset + 128;
  l.stage_offset = (l.sz_offset + size_t(tiles_per_block) * l.sz_tile_bytes + 127) & ~size_t(127);
  l.total = l.stage_offset + size_t(kAwqStages) * l.stage_bytes;
  return l;
}

template <bool kHigh>
__global__ void __launch_bounds__(kGemmThreads, 1) awq_stream_kernel(const GemmParams p, int tiles_per_block) {
  constexpr int kBlock = 136;
  extern __shared__ __align__(128) unsigned char smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
  const int slice = blockIdx.x % p.ksplit;
  const int group = blockIdx.x / p.ksplit;
  const int groups = gridDim.x / p.ksplit;
  const int units_total = p.K / 256;
  const int unit_begin = int((long long)slice * units_total / p.ksplit);
  const int units = int((long long)(slice + 1) * units_total / p.ksplit) - unit_begin;
  const int tiles = p.N / 8;
  const bool pair = p.epilogue == kEpiSiluPair;
  const int chunks = pair ? tiles / 2 : tiles;
  const int per_chunk = pair ? 2 : 1;
  const int item_begin = int((long long)group * chunks / groups) * per_chunk;
  const int item_end = int((long long)(group + 1) * chunks / groups) * per_chunk;
  const int item_count = item_end - item_begin;
  auto tile_of = [&](int item) -> int { return pair ? (item >> 1) + (item & 1) * (tiles / 2) : item; };

  const AwqStreamLayout layout = awq_stream_layout(units, tiles_per_block);
  float* part = reinterpret_cast<float*>(smem + layout.part_offset);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + layout.barrier_offset);
  unsigned char* sz = smem + layout.sz_offset;
  unsigned char* stages = smem + layout.stage_offset;
  const uint32_t slice_row_bytes = uint32_t(units) * 128;
  const unsigned char* weight_rows = reinterpret_cast<const unsigned char*>(p.qweight) + size_t(unit_begin) * 128;
  const size_t weight_row_stride = size_t(p.K / 8) * 4;

  // Lanes 0-7 of warp 0 each copy one row of the tile; lane 0 announces the bytes first.
  auto issue = [&](int index) {
    if (index >= item_count) return;
    const int stage = index % kAwqStages;
    const int tile = tile_of(item_begin + index);
    if (lane == 0) mbarrier_expect_tx(&full[stage], 8 * slice_row_bytes);
    __syncwarp();
    if (lane < 8)
      bulk_copy_to_shared(stages + size_t(stage) * layout.stage_bytes + lane * layout.row_bytes,
                          weight_rows + (size_t(tile) * 8 + lane) * weight_row_stride, slice_row_bytes, &full[stage]);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kAwqStages; ++s) mbarrier_init(&full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 0)
    for (int s = 0; s < kAwqStages; ++s) issue(s);

  // Scales (BF16) and zero nibbles (one byte each) of every tile of this block: [item][row][group].
  // Four elements per thread per round, all eight loads issued before the first store, so a round costs one
  // memory latency.
  {
    const int per_tile = 8 * layout.groups;
    const int total = item_count * per_tile;
    for (int first = threadIdx.x; first < total; first += 4 * blockDim.x) {
      unsigned short scale[4];
      uint32_t zero_word[4];
      int shift[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int idx = first + k * blockDim.x;
        scale[k] = 0;
        zero_word[k] = 0;
        shift[k] = 0;
        if (idx < total) {
          const int index = idx / per_tile, rem = idx - index * per_tile;
          const int r = rem / layout.groups, grp = unit_begin * 2 + (rem - r * layout.groups);
          const size_t n = size_t(tile_of(item_begin + index)) * 8 + r;
          scale[k] = __ldg(reinterpret_cast<const unsigned short*>(p.scales) + n * p.padded_groups + grp);
          zero_word[k] = uint32_t(__ldg(p.zeros + n * p.zero_stride + (grp >> 3)));
          shift[k] = (grp & 7) * 4;
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int idx = first + k * blockDim.x;
        if (idx < total) {
          const int index = idx / per_tile, rem = idx - index * per_tile;
          unsigned char* dst = sz + size_t(index) * layout.sz_tile_bytes;
          reinterpret_cast<unsigned short*>(dst)[rem] = scale[k];
          dst[per_tile * 2 + rem] = static_cast<unsigned char>((zero_word[k] >> shift[k]) & 15u);
        }
      }
    }
  }
  grid_dependency_wait();

  // A fragments of this warp's 256 inputs, pinned in registers.
  const bool live = warp < units;
  CellFragments<kHigh> frag[8];
  {
    const int k = (unit_begin + (live ? warp : 0)) * 256 + c * 64;
#pragma unroll
    for (int cell = 0; cell < 8; ++cell)
      load_cell<true, kHigh>(frag[cell], p.x, p.x_stride, live ? p.M : 0, g, k + cell * 8);
  }
  __syncthreads();  // scales / zeros visible
  grid_launch_dependents();

  // Reduction role of this lane: warp r owns accumulator elements e in [8r, 8r + 8); a lane is (part, element).
  const int e = warp * 8 + (lane & 7);
  const int part_index = lane >> 3;
  const int rl = e >> 2, reg = e & 3;
  const int row = (rl >> 2) + (reg >= 2 ? 8 : 0);
  const int col = (rl & 3) * 2 + (reg & 1);
  const int lane_group = warp * 2 + (c >> 1);  // this lane's scale group within the slice

  // One tile: 8 words per lane, two accumulator chains so consecutive MMAs do not wait on each other.
  auto compute_tile = [&](int index, float (&acc)[4]) {
    float other[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
    if (!live) return;
    const int stage = index % kAwqStages;
    const unsigned char* tile_sz = sz + size_t(index) * layout.sz_tile_bytes;
    const uint32_t scale2 = uint32_t(reinterpret_cast<const unsigned short*>(tile_sz)[g * layout.groups + lane_group]) * 0x10001u;
    const uint32_t zero2 = (0x4300u | tile_sz[8 * layout.groups * 2 + g * layout.groups + lane_group]) * 0x10001u;
    const unsigned char* src = stages + size_t(stage) * layout.stage_bytes + g * layout.row_bytes + warp * 128 + c * 32;
    const uint4 w0 = *reinterpret_cast<const uint4*>(src);
    const uint4 w1 = *reinterpret_cast<const uint4*>(src + 16);
#pragma unroll
    for (int cell = 0; cell < 8; ++cell) {
      const uint4 wv = cell < 4 ? w0 : w1;
      const int q = cell & 3;
      const uint32_t word = q == 0 ? wv.x : q == 1 ? wv.y : q == 2 ? wv.z : wv.w;
      const uint32_t b0 = dequant_pair(word, zero2, scale2);
      const uint32_t b1 = dequant_pair(word >> 4, zero2, scale2);
      const uint32_t b2 = dequant_pair(word >> 8, zero2, scale2);
      const uint32_t b3 = dequant_pair(word >> 12, zero2, scale2);
      mma_cell<kHigh>(acc, frag[cell], 0, b0, b1);
      mma_cell<kHigh>(other, frag[cell], 1, b2, b3);
    }
    acc[0] += other[0]; acc[1] += other[1]; acc[2] += other[2]; acc[3] += other[3];
  };

  auto wait_tile = [&](int index) -> bool {
#ifdef EI_EXP_NOWAIT
    return true;
#else
    return mbarrier_wait(&full[index % kAwqStages], (index / kAwqStages) & 1);
#endif
  };

  // Two tiles per block-wide barrier.
  for (int index = 0; index < item_count; index += 2) {
    const bool second = index + 1 < item_count;
    float acc0[4], acc1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    bool ok = wait_tile(index);
    if (ok) compute_tile(index, acc0);
    if (ok && second) {
      ok = wait_tile(index + 1);
      if (ok) compute_tile(index + 1, acc1);
    }
    if (!ok) {
      if (p.status) atomicOr(p.status, 4);
      return;  // every thread of the block sees the same incomplete phase and leaves here
    }
    float* mine = part + ((size_t((index >> 1) & 1) * 2) * kGemmWarps + warp) * kBlock;
    *reinterpret_cast<float4*>(mine + lane * 4) = make_float4(acc0[0], acc0[1], acc0[2], acc0[3]);
    *reinterpret_cast<float4*>(mine + kGemmWarps * kBlock + lane * 4) = make_float4(acc1[0], acc1[1], acc1[2], acc1[3]);
    __syncthreads();
    // Every warp has finished reading these two stages: refill them with the tiles kStages ahead.
    if (warp == 0) {
      issue(index + kAwqStages);
      issue(index + 1 + kAwqStages);
    }
    float sums[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const float* src = part + ((size_t((index >> 1) & 1) * 2 + t) * kGemmWarps + part_index) * kBlock + e;
      float sum = 0.0f;
#pragma unroll
      for (int w = 0; w < 4; ++w) sum += src[size_t(w) * 4 * kBlock];
      sum += __shfl_xor_sync(0xffffffffu, sum, 16);
      sum += __shfl_xor_sync(0xffffffffu, sum, 8);
      sums[t] = sum;
    }
    if (part_index == 0 && row < p.M) {
      if (pair) {
        // (index, index + 1) = (gate tile, up tile) of the same outputs.
        const int out_n = tile_of(item_begin + index) * 8 + col;
        float gate = sums[0], up = sums[1];
        if (p.bias) {
          gate += __bfloat162float(p.bias[out_n]);
          up += __bfloat162float(p.bias[out_n + p.N / 2]);
        }
        p.out[size_t(row) * p.out_stride + out_n] =
            __float2bfloat16_rn(silu_multiply_value(round_bf16(gate), round_bf16(up)));
      } else {
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (t == 1 && !second) break;
          const int n = tile_of(item_begin + index + t) * 8 + col;
          float sum = sums[t];
          if (p.epilogue == kEpiPartial) {
            p.partial[(size_t(slice) * p.M + row) * p.N + n] = sum;
          } else {
            if (p.bias) sum += __bfloat162float(p.bias[n]);
            p.out[size_t(row) * p.out_stride + n] = __float2bfloat16_rn(sum);
          }
        }
      }
    }
  }
}

}  // namespace ei
