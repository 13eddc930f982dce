// BF16 small-M GEMM fed by TMA: out[M,N] = x[M,K] * W[N,K]^T (+ bias), M <= 16, K a multiple of 256.
//
// Same skeleton as the int4 kernel (awq_tma.cuh) without the dequantisation: a tile is 8 output features over
// one K slice of up to 4096 inputs, brought into shared memory by one tiled TMA copy (rank-3 map
// [unit of 64 inputs][row][128 bytes], 128-byte swizzle, 64 KiB for a full slice) through a ring of stages on
// mbarriers with bounded waits. Warp w owns inputs [256 w, 256 w + 256) of the slice; its activation fragments
// are loaded once, 64 contiguous bytes per row and load, and stay in registers (the register-prefetching
// kernel in smallm_gemm.cuh keeps them in shared memory and reads them again for every MMA, which at more
// than 8 rows costs a quarter of the HBM rate on the vocabulary head). The loop is 8 128-bit shared-memory
// loads and 16 mma.sync.m16n8k16 per tile and warp; a lane's 16-byte chunk feeds two MMAs, and because the
// activation fragments take their inputs from the same positions, any fixed assignment of a chunk's eight
// inputs to MMA k-slots is valid. Per tile the 16 warps add their partial accumulators through shared memory
// in a fixed order; K beyond 4096 is split over blocks (ksplit) that write FP32 partials.
#pragma once

#include <cuda.h>

#include "awq_tma.cuh"

namespace ei {

constexpr int kDenseMaxStages = 8;
constexpr int kDenseWarpInputs = 256;  // inputs of the slice one warp owns: four 64-input units

struct DenseLaunch {
  int stages;           // tiles in flight per block
  int units_box;        // 64-input units the weight box covers (<= 64)
  uint32_t wait_limit;  // polls before a wait gives up (0: kAwqWaitLimit)
  uint32_t extra_tx;    // test hook: bytes the first copy is expected to deliver beyond what it does (0 in production)
};

struct DenseLayout {
  int tile_bytes;
  size_t stage_offset, part_offset, barrier_offset, total;
};
__host__ __device__ inline DenseLayout dense_layout(const DenseLaunch& cfg) {
  DenseLayout l;
  l.tile_bytes = cfg.units_box * 1024;
  l.stage_offset = 0;
  l.part_offset = size_t(cfg.stages) * l.tile_bytes;
  l.barrier_offset = l.part_offset + size_t(2) * kGemmWarps * 136 * sizeof(float);
  l.total = l.barrier_offset + 128 + 1024;  // + slack to reach a 1024-byte boundary
  return l;
}

template <bool kHigh>
__global__ void __launch_bounds__(kGemmThreads, 1)
    dense_tma_kernel(const __grid_constant__ CUtensorMap weights, const GemmParams p, const DenseLaunch cfg) {
  constexpr int kBlock = 136;
  constexpr int kParts = 4;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_address(smem_raw) & 1023u)) & 1023u);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
  const int slice = blockIdx.x % p.ksplit;
  const int group = blockIdx.x / p.ksplit;
  const int groups = gridDim.x / p.ksplit;
  // Slices in steps of one warp's 256 inputs.
  const int parts_total = p.K / kDenseWarpInputs;
  const int part_begin = int((long long)slice * parts_total / p.ksplit);
  const int parts = int((long long)(slice + 1) * parts_total / p.ksplit) - part_begin;
  const int tiles = p.N / 8;
  const bool pair = p.epilogue == kEpiSiluPair;
  const int chunks = pair ? tiles / 2 : tiles;
  const int per_chunk = pair ? 2 : 1;
  const int item_begin = int((long long)group * chunks / groups) * per_chunk;
  const int item_end = int((long long)(group + 1) * chunks / groups) * per_chunk;
  const int item_count = item_end - item_begin;
  auto tile_of = [&](int item) -> int { return pair ? (item >> 1) + (item & 1) * (tiles / 2) : item; };

  const DenseLayout layout = dense_layout(cfg);
  unsigned char* stages = smem + layout.stage_offset;
  float* part = reinterpret_cast<float*>(smem + layout.part_offset);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + layout.barrier_offset);
  volatile int* failed = reinterpret_cast<volatile int*>(full + kDenseMaxStages);  // set by a thread whose wait ran out
  const uint32_t wait_limit = cfg.wait_limit ? cfg.wait_limit : kAwqWaitLimit;

  auto issue = [&](int index) {
    if (index >= item_count) return;
    const int slot = index % cfg.stages;
    mbarrier_expect_tx(&full[slot], uint32_t(layout.tile_bytes) + (index == 0 ? cfg.extra_tx : 0u));
    tma_load_3d(stages + size_t(slot) * layout.tile_bytes, &weights, 0, tile_of(item_begin + index) * 8,
                part_begin * 4, &full[slot]);
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < cfg.stages; ++s) mbarrier_init(&full[s], 1);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    issue(0);  // weights do not depend on the preceding kernel; more now would delay the activation loads below
  }
  __syncthreads();  // barriers initialised: synchronise while the block would wait for its predecessor anyway
  grid_dependency_wait();
  grid_launch_dependents();

  // A fragments of this warp's 256 inputs: cell (unit u, half h) of lane (g, c) holds inputs
  // [64 u + 32 h + 8 c, + 8) of rows g and g + 8: the four lanes of a row read 64 contiguous bytes per load.
  const bool live = warp < parts;
  uint4 lo[8], hi[8];
  {
    const int k = (part_begin + (live ? warp : 0)) * kDenseWarpInputs + c * 8;
#pragma unroll
    for (int cell = 0; cell < 8; ++cell) {
      lo[cell] = make_uint4(0, 0, 0, 0);
      hi[cell] = make_uint4(0, 0, 0, 0);
      if (live && g < p.M) lo[cell] = *reinterpret_cast<const uint4*>(p.x + size_t(g) * p.x_stride + k + cell * 32);
      if (kHigh && live && g + 8 < p.M)
        hi[cell] = *reinterpret_cast<const uint4*>(p.x + size_t(g + 8) * p.x_stride + k + cell * 32);
    }
  }
  asm volatile("" ::: "memory");  // the activation loads are issued before the rest of the ring is requested
  if (threadIdx.x == 0)
    for (int s = 1; s < cfg.stages; ++s) issue(s);

  // Reduction role of this lane: warp r owns accumulator elements e in [8r, 8r + 8); a lane is (part, element).
  const int e = warp * 8 + (lane & 7);
  const int part_index = lane >> 3;
  const int rl = e >> 2, reg = e & 3;
  const int row = (rl >> 2) + (reg >= 2 ? 8 : 0);
  const int col = (rl & 3) * 2 + (reg & 1);
  float best_value = -INFINITY;
  int best_index = 0x7fffffff;
  float gate_sum = 0.0f;  // fused SwiGLU: the gate tile's sum waits here for the up tile

  // Rows g of units 4 warp .. 4 warp + 3 in a staged tile [unit][row][128 B]; 16-byte chunk j of row r sits at
  // chunk (j ^ r), and bits 4-6 of lane_base hold g, so chunk (4 h + c) of unit u is at
  // (lane_base + u * 1024) ^ ((4 h + c) << 4).
  const uint32_t stages_address = smem_address(stages);
  const uint32_t lane_base = uint32_t(warp * 4096 + g * 128 + (g << 4));
  auto shared_u128 = [](uint32_t address) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(address));
    return v;
  };

  int slot = 0;
  uint32_t parity = 0;
  // Giving up is the block's decision: a thread whose wait ran out raises the flag before the tile's block-wide
  // barrier; every thread reads it after the barrier and acts on it at the top of the next tile.
  int gave_up = 0, tiles_done = 0;
  for (int index = 0; index < item_count && !gave_up; ++index) {
    const int item = item_begin + index;
    const bool ok = mbarrier_wait(&full[slot], parity, wait_limit);
    if (!ok) *failed = 1;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, other[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (live && ok) {
      const uint32_t tile_address = stages_address + uint32_t(slot) * uint32_t(layout.tile_bytes) + lane_base;
      uint4 w[8];
#pragma unroll
      for (int cell = 0; cell < 8; ++cell)
        w[cell] = shared_u128((tile_address + uint32_t(cell >> 1) * 1024u) ^ uint32_t((((cell & 1) << 2) + c) << 4));
#pragma unroll
      for (int cell = 0; cell < 8; ++cell) {
        if (kHigh) {
          mma_bf16_16816(acc, lo[cell].x, hi[cell].x, lo[cell].y, hi[cell].y, w[cell].x, w[cell].y);
          mma_bf16_16816(other, lo[cell].z, hi[cell].z, lo[cell].w, hi[cell].w, w[cell].z, w[cell].w);
        } else {
          mma_bf16_16816(acc, lo[cell].x, 0u, lo[cell].y, 0u, w[cell].x, w[cell].y);
          mma_bf16_16816(other, lo[cell].z, 0u, lo[cell].w, 0u, w[cell].z, w[cell].w);
        }
      }
      acc[0] += other[0]; acc[1] += other[1]; acc[2] += other[2]; acc[3] += other[3];
    }
    if (++slot == cfg.stages) {
      slot = 0;
      parity ^= 1;
    }
    float* mine = part + (size_t(index & 1) * kGemmWarps + warp) * kBlock;
    *reinterpret_cast<float4*>(mine + lane * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    __syncthreads();
    // Every warp has finished reading this stage: refill it with the tile `stages` ahead.
    if (threadIdx.x == 0) issue(index + cfg.stages);
    gave_up = *failed;
    tiles_done = index + 1;

    // Fixed-order reduction by all 16 warps: part q adds the partials of warps q, q + 4, q + 8, q + 12 in that
    // order and the parts are combined by two shuffles, so an output sees the same additions in every run.
    float sum = 0.0f;
    {
      const float* src = part + (size_t(index & 1) * kGemmWarps + part_index) * kBlock + e;
#pragma unroll
      for (int w = 0; w < kGemmWarps / kParts; ++w) sum += src[size_t(w) * kParts * kBlock];
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 16);
    sum += __shfl_xor_sync(0xffffffffu, sum, 8);
    if (part_index == 0 && row < p.M) {
      const int n = tile_of(item) * 8 + col;
      if (pair) {
        if ((item & 1) == 0) {
          gate_sum = sum;
        } else {
          float gate = gate_sum, up = sum;
          const int out_n = n - p.N / 2;
          if (p.bias) {
            gate += __bfloat162float(p.bias[out_n]);
            up += __bfloat162float(p.bias[n]);
          }
          p.out[size_t(row) * p.out_stride + out_n] =
              __float2bfloat16_rn(silu_multiply_value(round_bf16(gate), round_bf16(up)));
        }
      } else if (p.epilogue == kEpiPartial) {
        p.partial[(size_t(slice) * p.M + row) * p.N + n] = sum;
      } else {
        if (p.bias) sum += __bfloat162float(p.bias[n]);
        const bf16 rounded = __float2bfloat16_rn(sum);
        p.out[size_t(row) * p.out_stride + n] = rounded;
        if (p.epilogue == kEpiArgmax) {
          float value = __bfloat162float(rounded);
          if (isnan(value)) value = -INFINITY;
          if (value > best_value || (value == best_value && n < best_index)) {
            best_value = value;
            best_index = n;
          }
        }
      }
    }
  }

  if (gave_up) {
    if (threadIdx.x == 0) {
      if (p.status) atomicOr(p.status, 4);
      // A block never leaves while a copy into its shared memory may be in flight: give every tile still in
      // the ring its chance to land (bounded again).
      for (int back = max(0, tiles_done - 1); back < min(item_count, tiles_done - 1 + cfg.stages); ++back)
        mbarrier_wait(&full[back % cfg.stages], uint32_t((back / cfg.stages) & 1), wait_limit);
    }
    __syncthreads();
    return;
  }

  if (p.epilogue == kEpiArgmax) {
    // An element owner always sees the same output row; fold the 8 owners of each row.
    __syncthreads();
    float* values = part;
    int* indices = reinterpret_cast<int*>(part + 128);
    if (part_index == 0) {
      values[e] = best_value;
      indices[e] = best_index;
    }
    __syncthreads();
    if (threadIdx.x < 16) {
      const int want = threadIdx.x;
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int v = 0; v < 128; ++v) {
        const int vl = v >> 2, vr = v & 3;
        if ((vl >> 2) + (vr >= 2 ? 8 : 0) != want) continue;
        const float value = values[v];
        const int index = indices[v];
        if (value > bv || (value == bv && index < bi)) {
          bv = value;
          bi = index;
        }
      }
      p.best_value[blockIdx.x * 16 + want] = bv;
      p.best_index[blockIdx.x * 16 + want] = bi;
    }
  }
}

}  // namespace ei
