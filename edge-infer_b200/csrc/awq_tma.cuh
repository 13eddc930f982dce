// int4 (AWQ, group 128) small-M GEMM fed by TMA: out[M,N] = x[M,K] * dequant(W)[N,K]^T (+ bias).
//
// A tile is 8 output features = 8 consecutive rows of the N-major packed weight matrix, over one K slice of
// up to 4096 inputs. One thread brings a whole tile into shared memory with a single tiled TMA copy
// (cp.async.bulk.tensor) that completes on an mbarrier; a ring of tiles is always in flight per block, so HBM streams continuously, independently of
// the warps' register scoreboards, and the loop issues no global loads at all. The group scales and packed zero points of all rows the block will touch come in up front, by one
// box each (a TMA copy costs about 100 ns of the copy engine's time whatever its size, so few large copies).
//
// The weight matrix is described to TMA as a rank-3 tensor [unit of 256 inputs][row][128 bytes], so that the
// staged tile is [unit][row][128 B] and the 128-byte swizzle places the 16-byte chunk j of row r at chunk
// (j ^ r): the eight rows a quarter-warp reads in one load then fall into eight distinct bank groups.
//
// The <= 16 activation rows never change while the block runs and warp w always works on inputs
// [256 w, 256 w + 256) of the block's K slice, so its A fragments are loaded once, in the register order
// mma.sync wants, and stay in registers: the inner loop is nibble extraction, the exact BF16 dequantisation
// (see dequant_pair) and mma.sync.m16n8k16 with FP32 accumulation. Per tile the 16 warps add their partial
// accumulators through shared memory in a fixed order. K beyond 4096 is split over blocks (ksplit) that write
// FP32 partials for a separate fixed-order reduction.
//
// Scale and zero-point rows that TMA cannot address (row pitch not a multiple of 16 bytes) are instead
// fetched once, with ordinary loads, for every tile the block will touch, before the kernel waits for its
// predecessor.
//
// Every wait on an mbarrier is bounded, and the decision is the block's, not a thread's: a thread whose wait
// ran out raises a shared flag that all threads read after the phase's block-wide barrier, so either all go on or all record the failure in
// GemmParams::status, wait (bounded again) for the copies still in flight and leave without touching the
// outputs again.
#pragma once

#include "smallm_gemm.cuh"
#include "tma.cuh"

namespace ei {

constexpr int kAwqMaxStages = 12;
constexpr int kAwqSliceUnits = 16;            // 256-input units per K slice: one per warp
constexpr uint32_t kAwqWaitLimit = kTmaWaitLimit;  // polls of ~100 ns before a wait gives up

struct AwqTensorMaps {
  CUtensorMap weights;  // u32 [units][N][32], box [units_box][8][32], 128-byte swizzle
  CUtensorMap scales;   // bf16 [N][padded_groups], box [8][scale_box]
  CUtensorMap zeros;    // i32 [N][zero_stride], box [8][zero_box]
};

struct AwqLaunch {
  int tiles_per_block;  // tiles (items) the busiest block walks
  int stages;           // tiles in flight per block
  int units_box;        // units the weight box covers (<= 16)
  int tma_sz;           // 1: scales/zeros ride with the tile by TMA; 0: fetched up front by ordinary loads
  int scale_box;        // groups per staged scale row
  int zero_box;         // words per staged zero row
  int sz_boxes;         // TMA boxes of scale / zero rows per block: 1, or 2 in pair mode (gate rows, up rows)
  int sz_rows;          // rows per such box (<= 256)
  uint32_t wait_limit;  // polls before a wait gives up (0: kAwqWaitLimit)
  uint32_t extra_tx;    // test hook: bytes added to what the first weight copy is expected to deliver, so that
                        // its barrier never completes and the bounded waits run out (0 in production)
};

constexpr int kAwqPhaseTiles = 2;  // tiles a warp accumulates between two block-wide barriers
constexpr int kAwqEarlyPhases = 1; // phases (pairs of tiles) requested before the kernel waits for its predecessor

struct AwqLayout {
  int weight_bytes;   // staged weight bytes of a tile: units_box KiB
  int sz_tile_bytes;  // up-front mode: scales + zero nibbles of one tile, 16-byte padded
  int sz_scale_bytes; // TMA mode: bytes of all staged scale rows (the zero-point rows follow)
  size_t stage_offset, part_offset, barrier_offset, sz_offset, total;
};

// Offsets are relative to the first 1024-byte boundary of the dynamic shared memory (the swizzle needs it);
// `total` includes the slack to reach that boundary.
__host__ __device__ inline AwqLayout awq_layout(const AwqLaunch& cfg) {
  AwqLayout l;
  l.weight_bytes = cfg.units_box * 1024;
  l.sz_tile_bytes = cfg.tma_sz ? 0 : ((8 * cfg.units_box * 2 * 3) + 15) & ~15;
  l.sz_scale_bytes = cfg.sz_boxes * cfg.sz_rows * cfg.scale_box * 2;
  l.stage_offset = 0;
  l.part_offset = size_t(cfg.stages) * l.weight_bytes;
  l.barrier_offset = l.part_offset + size_t(2) * kAwqPhaseTiles * kGemmWarps * 136 * sizeof(float);
  l.sz_offset = l.barrier_offset + 128;
  const size_t sz_bytes = cfg.tma_sz ? size_t(l.sz_scale_bytes) + size_t(cfg.sz_boxes) * cfg.sz_rows * cfg.zero_box * 4
                                     : size_t(cfg.tiles_per_block) * l.sz_tile_bytes;
  l.total = l.sz_offset + sz_bytes + 1024;
  return l;
}

// kPair: SwiGLU pair epilogue; kTmaSz: scales / zero points staged by TMA boxes; kFull: every warp owns a unit
// of the K slice (slices of 4096 inputs). The three are compile-time so that the loop, which is issue-bound,
// carries no branch or uniform-register arithmetic for them.
template <bool kHigh, bool kPair, bool kTmaSz, bool kFull>
__global__ void __launch_bounds__(kGemmThreads, 1)
    awq_tma_kernel(const __grid_constant__ AwqTensorMaps maps, const GemmParams p, const AwqLaunch cfg) {
  constexpr int kBlock = 136;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_address(smem_raw) & 1023u)) & 1023u);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
  const int slice = blockIdx.x % p.ksplit;
  const int group = blockIdx.x / p.ksplit;
  const int groups = gridDim.x / p.ksplit;
  const int units_total = p.K / 256;
  const int unit_begin = slice * kAwqSliceUnits;
  const int units = min(kAwqSliceUnits, units_total - unit_begin);
  const int tiles = p.N / 8;
  constexpr bool pair = kPair;
  const int chunks = pair ? tiles / 2 : tiles;
  const int per_chunk = pair ? 2 : 1;
  const int item_begin = int((long long)group * chunks / groups) * per_chunk;
  const int item_end = int((long long)(group + 1) * chunks / groups) * per_chunk;
  const int item_count = item_end - item_begin;
  auto tile_of = [&](int item) -> int { return pair ? (item >> 1) + (item & 1) * (tiles / 2) : item; };

  const AwqLayout layout = awq_layout(cfg);
  unsigned char* stages = smem + layout.stage_offset;
  float* part = reinterpret_cast<float*>(smem + layout.part_offset);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + layout.barrier_offset);
  uint64_t* sz_full = full + kAwqMaxStages;
  volatile int* failed = reinterpret_cast<volatile int*>(sz_full + 1);  // set by a thread whose wait ran out
  unsigned char* sz = smem + layout.sz_offset;
  const int scale_pitch = cfg.scale_box * 2, zero_pitch = cfg.zero_box * 4;

  // One thread brings in the two tiles of a phase, one copy each, on one barrier (a wait costs a few hundred
  // cycles even when the data has long arrived, so there is one per phase, not one per tile). One copy for
  // both tiles (a 16-row box, or a rank-4 box over the gate and the up half) was measured slower to deliver.
  const int ring_phases = cfg.stages / kAwqPhaseTiles;
  const int phase_bytes = kAwqPhaseTiles * layout.weight_bytes;
  const uint32_t wait_limit = cfg.wait_limit ? cfg.wait_limit : kAwqWaitLimit;
  auto issue = [&](int phase) {
    const int index = phase * kAwqPhaseTiles;
    if (index >= item_count) return;
    const int slot = phase % ring_phases, tiles_here = min(kAwqPhaseTiles, item_count - index);
    mbarrier_expect_tx(&full[slot], uint32_t(tiles_here * layout.weight_bytes) + (phase == 0 ? cfg.extra_tx : 0u));
    for (int t = 0; t < tiles_here; ++t)
      tma_load_3d(stages + size_t(slot) * phase_bytes + size_t(t) * layout.weight_bytes, &maps.weights, 0,
                  tile_of(item_begin + index + t) * 8, unit_begin, &full[slot]);
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < ring_phases; ++s) mbarrier_init(&full[s], 1);
    mbarrier_init(sz_full, 1);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (kTmaSz) {
      // Group scales and packed zero points of every row this block will touch: one box each (two in pair
      // mode: the gate rows and the up rows). Rows past the matrix read as zero and are never used.
      mbarrier_expect_tx(sz_full, uint32_t(cfg.sz_boxes * cfg.sz_rows * (scale_pitch + zero_pitch)));
      for (int b = 0; b < cfg.sz_boxes; ++b) {
        const int row = pair ? ((item_begin >> 1) + b * (tiles / 2)) * 8 : item_begin * 8;
        tma_load_2d(sz + size_t(b) * cfg.sz_rows * scale_pitch, &maps.scales, unit_begin * 2, row, sz_full);
        tma_load_2d(sz + layout.sz_scale_bytes + size_t(b) * cfg.sz_rows * zero_pitch, &maps.zeros, unit_begin / 4, row,
                    sz_full);
      }
    }
    // Only a few tiles now: requests made here are served before the activation loads below, and a full
    // ring from every block would put those loads behind tens of megabytes of weight traffic.
    for (int ph = 0; ph < kAwqEarlyPhases && ph < ring_phases; ++ph) issue(ph);
  }

  if (!kTmaSz) {
    // Scales (BF16) and zero nibbles (one byte each) of every tile of this block: [item][row][group].
    // Four elements per thread per round, all eight loads issued before the first store, so a round costs
    // one memory latency.
    const int slice_groups = cfg.units_box * 2;
    const int per_tile = 8 * slice_groups;
    const int total = item_count * per_tile;
    const int last_group = p.K / 128 - 1;
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
          const int r = rem / slice_groups, grp = min(unit_begin * 2 + (rem - r * slice_groups), last_group);
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
  // Barriers initialised, up-front scales / zeros visible: the block synchronises here, while it would wait for
  // its predecessor anyway, so that nothing after the activation loads below needs a block-wide barrier.
  __syncthreads();
  grid_dependency_wait();
  grid_launch_dependents();

  // A fragments of this warp's 256 inputs, pinned in registers.
  const bool live = kFull || warp < units;
  CellFragments<kHigh> frag[8];
  {
    // Cell `cell` of lane (g, c) holds inputs [32 cell + 8 c, + 8) of the unit: the four lanes of a row read
    // 64 contiguous bytes per load, so a warp-wide load touches 8 lines instead of 32.
    const int k = (unit_begin + (live ? warp : 0)) * 256 + c * 8;
#pragma unroll
    for (int cell = 0; cell < 8; ++cell)
      load_cell<kHigh>(frag[cell], p.x, p.x_stride, live ? p.M : 0, g, k + cell * 32);
  }
  asm volatile("" ::: "memory");  // the activation loads are issued before the rest of the ring is requested
  // One thread requests the phases one after another: they then arrive in the order they are needed. Requested
  // side by side by several warps (measured), their bytes interleave and the first phase lands microseconds late.
  if (threadIdx.x == 0)
    for (int ph = kAwqEarlyPhases; ph < ring_phases; ++ph) issue(ph);
  bool sz_ok = true;
  if (kTmaSz) sz_ok = mbarrier_wait(sz_full, 0, wait_limit);

  // With at most eight rows the operands trade places: the two tiles of a phase (16 features) are the A operand of
  // one MMA and the rows the B operand, so an MMA covers 256 weights instead of 128 and a phase has one accumulator
  // fragment (features x rows) instead of two (rows x features, half of them empty).
  constexpr bool kSwap = !kHigh;
  // Reduction role of this lane: warp r owns accumulator elements e in [8r, 8r + 8); a lane is (part, element).
  const int e = warp * 8 + (lane & 7);
  const int part_index = lane >> 3;
  const int rl = e >> 2, reg = e & 3;
  // Element (lane rl, register reg) of a fragment: (row, col) of the output it belongs to, and for the swapped
  // form the tile of the phase (`swap_tile`): there the fragment's rows are features and its columns output rows.
  const int row = kSwap ? (rl & 3) * 2 + (reg & 1) : (rl >> 2) + (reg >= 2 ? 8 : 0);
  const int col = kSwap ? (rl >> 2) : (rl & 3) * 2 + (reg & 1);
  const int swap_tile = reg >> 1;
  const int unit_group = warp * 2;  // the unit's two scale groups within the slice: cells 0-3 and cells 4-7
  // Everything a tile's addresses depend on is folded into per-lane constants here, so that the loop does no
  // division and little integer arithmetic (the loop is issue-bound: every instruction in it counts).
  // Row g of unit `warp` in a staged tile; the lane's word of cell j is word c of 16-byte chunk (j ^ g), and
  // because bits 4-6 of this offset hold g, that word sits at (lane_word ^ (j << 4)).
  const uint32_t stages_address = smem_address(stages);
  const uint32_t lane_word = uint32_t(warp * 1024 + g * 128 + (g << 4) + c * 4);
  // Scales / zero points of this lane's row and groups: TMA mode [box][row][group], up-front mode [item][...].
  const uint32_t sz_address = smem_address(sz);
  const uint32_t lane_scale = kTmaSz ? sz_address + g * scale_pitch + unit_group * 2
                                         : sz_address + (g * cfg.units_box * 2 + unit_group) * 2;
  const uint32_t lane_zero = kTmaSz ? sz_address + layout.sz_scale_bytes + g * zero_pitch + (unit_group >> 3) * 4
                                        : sz_address + 8 * cfg.units_box * 2 * 2 + g * cfg.units_box * 2 + unit_group;
  const int zero_shift = kTmaSz ? (unit_group & 7) * 4 : 0;
  // Row of tile t (0 or 1) of phase `step` in the staged scale / zero rows.
  const int phase_rows = pair ? 8 : 16, second_rows = pair ? cfg.sz_rows : 8;

  auto shared_u32 = [](uint32_t address) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(address));
    return v;
  };

  // One tile: 8 words per lane, two accumulator chains so consecutive MMAs do not wait on each other.
  // `tile_address`: the staged tile; `step`, `t`: phase and tile within the phase.
  auto compute_tile = [&](uint32_t tile_address, int step, int t, float (&acc)[4]) {
    float other[4];
    if (!live) {
      acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
      return;
    }
    uint32_t scale2[2], zero2[2];
    if (kTmaSz) {
      const int sz_row = step * phase_rows + t * second_rows;
      const uint32_t zero_word = shared_u32(lane_zero + sz_row * zero_pitch);
      const uint32_t scales = shared_u32(lane_scale + sz_row * scale_pitch);
      scale2[0] = (scales & 0xffffu) * 0x10001u;
      scale2[1] = (scales >> 16) * 0x10001u;
      zero2[0] = (0x4300u | ((zero_word >> zero_shift) & 15u)) * 0x10001u;
      zero2[1] = (0x4300u | ((zero_word >> (zero_shift + 4)) & 15u)) * 0x10001u;
    } else {
      const uint32_t offset = uint32_t(step * kAwqPhaseTiles + t) * layout.sz_tile_bytes;
      const uint32_t scales = shared_u32(lane_scale + offset);
      uint32_t nibbles;
      asm volatile("ld.shared.u16 %0, [%1];" : "=r"(nibbles) : "r"(lane_zero + offset));
      scale2[0] = (scales & 0xffffu) * 0x10001u;
      scale2[1] = (scales >> 16) * 0x10001u;
      zero2[0] = (0x4300u | (nibbles & 15u)) * 0x10001u;
      zero2[1] = (0x4300u | ((nibbles >> 8) & 15u)) * 0x10001u;
    }
    uint32_t words[8];
#pragma unroll
    for (int cell = 0; cell < 8; ++cell) words[cell] = shared_u32((tile_address + lane_word) ^ uint32_t(cell << 4));
#pragma unroll
    for (int cell = 0; cell < 8; ++cell) {
      const uint32_t word = words[cell], z = zero2[cell >> 2], sc = scale2[cell >> 2];
      const uint32_t b0 = dequant_pair(word, z, sc);
      const uint32_t b1 = dequant_pair(word >> 4, z, sc);
      const uint32_t b2 = dequant_pair(word >> 8, z, sc);
      const uint32_t b3 = dequant_pair(word >> 12, z, sc);
      if (cell == 0) {  // the first MMA of each chain starts from zero: no clearing of the accumulators
        mma_cell<kHigh, true>(acc, frag[cell], 0, b0, b1);
        mma_cell<kHigh, true>(other, frag[cell], 1, b2, b3);
      } else {
        mma_cell<kHigh>(acc, frag[cell], 0, b0, b1);
        mma_cell<kHigh>(other, frag[cell], 1, b2, b3);
      }
    }
    acc[0] += other[0]; acc[1] += other[1]; acc[2] += other[2]; acc[3] += other[3];
  };

  // Swapped form: both tiles of the phase at once. Lane (g, c) dequantises its word of row g of either tile; the
  // A operand takes (tile 0 row g, tile 1 row g) as rows g and g + 8, the B operand the activation fragments.
  auto compute_phase = [&](uint32_t tile_address, int step, bool second, float (&acc)[4]) {
    float other[4];
    if (!live) {
      acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
      return;
    }
    uint32_t scale2[2][2], zero2[2][2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      if (kTmaSz) {
        const int sz_row = step * phase_rows + t * second_rows;
        const uint32_t zero_word = shared_u32(lane_zero + sz_row * zero_pitch);
        const uint32_t scales = shared_u32(lane_scale + sz_row * scale_pitch);
        scale2[t][0] = (scales & 0xffffu) * 0x10001u;
        scale2[t][1] = (scales >> 16) * 0x10001u;
        zero2[t][0] = (0x4300u | ((zero_word >> zero_shift) & 15u)) * 0x10001u;
        zero2[t][1] = (0x4300u | ((zero_word >> (zero_shift + 4)) & 15u)) * 0x10001u;
      } else {
        const uint32_t offset = uint32_t(step * kAwqPhaseTiles + t) * layout.sz_tile_bytes;
        const uint32_t scales = shared_u32(lane_scale + offset);
        uint32_t nibbles;
        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(nibbles) : "r"(lane_zero + offset));
        scale2[t][0] = (scales & 0xffffu) * 0x10001u;
        scale2[t][1] = (scales >> 16) * 0x10001u;
        zero2[t][0] = (0x4300u | (nibbles & 15u)) * 0x10001u;
        zero2[t][1] = (0x4300u | ((nibbles >> 8) & 15u)) * 0x10001u;
      }
    }
    uint32_t words[2][8];
#pragma unroll
    for (int cell = 0; cell < 8; ++cell) {
      words[0][cell] = shared_u32((tile_address + lane_word) ^ uint32_t(cell << 4));
      // A phase without a second tile (the last one of an odd count) feeds zeros: its half of the fragment is
      // never emitted, and zeros keep the arithmetic finite.
      words[1][cell] = second ? shared_u32((tile_address + uint32_t(layout.weight_bytes) + lane_word) ^ uint32_t(cell << 4))
                              : 0u;
    }
#pragma unroll
    for (int cell = 0; cell < 8; ++cell) {
      const int half = cell >> 2;
      const uint32_t w0 = words[0][cell], w1 = words[1][cell];
      const uint32_t a0 = dequant_pair(w0, zero2[0][half], scale2[0][half]);
      const uint32_t a1 = dequant_pair(w1, zero2[1][half], scale2[1][half]);
      const uint32_t a2 = dequant_pair(w0 >> 4, zero2[0][half], scale2[0][half]);
      const uint32_t a3 = dequant_pair(w1 >> 4, zero2[1][half], scale2[1][half]);
      const uint32_t c0 = dequant_pair(w0 >> 8, zero2[0][half], scale2[0][half]);
      const uint32_t c1 = dequant_pair(w1 >> 8, zero2[1][half], scale2[1][half]);
      const uint32_t c2 = dequant_pair(w0 >> 12, zero2[0][half], scale2[0][half]);
      const uint32_t c3 = dequant_pair(w1 >> 12, zero2[1][half], scale2[1][half]);
      if (cell == 0) {
        mma_bf16_16816_first(acc, a0, a1, a2, a3, frag[cell].a[0][0], frag[cell].a[0][1]);
        mma_bf16_16816_first(other, c0, c1, c2, c3, frag[cell].a[1][0], frag[cell].a[1][1]);
      } else {
        mma_bf16_16816(acc, a0, a1, a2, a3, frag[cell].a[0][0], frag[cell].a[0][1]);
        mma_bf16_16816(other, c0, c1, c2, c3, frag[cell].a[1][0], frag[cell].a[1][1]);
      }
    }
    acc[0] += other[0]; acc[1] += other[1]; acc[2] += other[2]; acc[3] += other[3];
  };

  // Reduction of one phase (kAwqPhaseTiles tiles): the partials were read into `loaded` right after the
  // phase's barrier; the additions happen one tile of computation later, so the shared-memory latency is
  // hidden behind that tile's arithmetic. After the shuffles all four parts of a warp hold the same sums:
  // part q keeps those of phases q, q + 4, q + 8, ... and the epilogue runs once every four phases with all 32
  // lanes busy instead of every phase with 8 (this loop is issue-bound: the epilogue's instructions count).
  float held[kAwqPhaseTiles] = {0.0f, 0.0f};
  auto emit = [&](int first_step, int last_step) {  // epilogue of phases first_step + part_index <= last_step
    const int step = first_step + part_index;
    if (kSwap) {
      // held[0] is this lane's element of the phase's single fragment: feature `col` of tile `swap_tile`, row `row`.
      // In pair mode the gate value sits in registers 0-1 and its up value two registers on: two lanes further.
      const float partner = __shfl_down_sync(0xffffffffu, held[0], 2);
      if (step > last_step || row >= p.M) return;
      const int index = step * kAwqPhaseTiles;
      if (pair) {
        if (swap_tile) return;
        const int out_n = tile_of(item_begin + index) * 8 + col;
        float gate = held[0], up = partner;
        if (p.bias) {
          gate += __bfloat162float(p.bias[out_n]);
          up += __bfloat162float(p.bias[out_n + p.N / 2]);
        }
        p.out[size_t(row) * p.out_stride + out_n] =
            __float2bfloat16_rn(silu_multiply_value(round_bf16(gate), round_bf16(up)));
        return;
      }
      if (index + swap_tile >= item_count) return;
      const int n = tile_of(item_begin + index + swap_tile) * 8 + col;
      float sum = held[0];
      if (p.epilogue == kEpiPartial) {
        p.partial[(size_t(slice) * p.M + row) * p.N + n] = sum;
      } else {
        if (p.bias) sum += __bfloat162float(p.bias[n]);
        p.out[size_t(row) * p.out_stride + n] = __float2bfloat16_rn(sum);
      }
      return;
    }
    if (step > last_step || row >= p.M) return;
    const int index = step * kAwqPhaseTiles;
    if (pair) {
      // (index, index + 1) = (gate tile, up tile) of the same outputs.
      const int out_n = tile_of(item_begin + index) * 8 + col;
      float gate = held[0], up = held[1];
      if (p.bias) {
        gate += __bfloat162float(p.bias[out_n]);
        up += __bfloat162float(p.bias[out_n + p.N / 2]);
      }
      p.out[size_t(row) * p.out_stride + out_n] =
          __float2bfloat16_rn(silu_multiply_value(round_bf16(gate), round_bf16(up)));
    } else {
#pragma unroll
      for (int t = 0; t < kAwqPhaseTiles; ++t) {
        if (index + t >= item_count) break;
        const int n = tile_of(item_begin + index + t) * 8 + col;
        float sum = held[t];
        if (p.epilogue == kEpiPartial) {
          p.partial[(size_t(slice) * p.M + row) * p.N + n] = sum;
        } else {
          if (p.bias) sum += __bfloat162float(p.bias[n]);
          p.out[size_t(row) * p.out_stride + n] = __float2bfloat16_rn(sum);
        }
      }
    }
  };
  auto finish = [&](int step, const float (&loaded)[kAwqPhaseTiles][4]) {
#pragma unroll
    for (int t = 0; t < (kSwap ? 1 : kAwqPhaseTiles); ++t) {
      float sum = 0.0f;
#pragma unroll
      for (int w = 0; w < 4; ++w) sum += loaded[t][w];
      sum += __shfl_xor_sync(0xffffffffu, sum, 16);
      sum += __shfl_xor_sync(0xffffffffu, sum, 8);
      if (part_index == (step & 3)) held[t] = sum;
    }
    if ((step & 3) == 3) emit(step - 3, step);
  };

  // kAwqPhaseTiles tiles per block-wide barrier; the partial buffers alternate between phases.
  static_assert(kAwqPhaseTiles == 2, "the loop below is written for two tiles per phase");
  float loaded[kAwqPhaseTiles][4];
  int pending = -1;  // phase whose partials sit in `loaded`
  int slot = 0;          // ring position of the current phase
  uint32_t parity = 0;   // of the current pass over the ring
  int gave_up = 0, steps_done = 0;
  for (int index = 0, step = 0; index < item_count && !gave_up; index += kAwqPhaseTiles, ++step) {
    const int phase = step & 1;
    float acc[kAwqPhaseTiles][4];
    // Warp-uniform: the shuffles of the reduction below are taken by whole warps or not at all.
    const bool ok = __all_sync(0xffffffffu, sz_ok && mbarrier_wait(&full[slot], parity, wait_limit));
    const uint32_t tile_address = stages_address + uint32_t(slot) * uint32_t(phase_bytes);
    if (kSwap) {
      if (ok) compute_phase(tile_address, step, kPair || index + 1 < item_count, acc[0]);
      if (ok && pending >= 0) finish(pending, loaded);
    } else {
      if (ok) compute_tile(tile_address, step, 0, acc[0]);
      if (ok && pending >= 0) finish(pending, loaded);
      if (ok && (kPair || index + 1 < item_count))  // pairs come whole
        compute_tile(tile_address + layout.weight_bytes, step, 1, acc[1]);
      else
        acc[1][0] = acc[1][1] = acc[1][2] = acc[1][3] = 0.0f;
    }
    if (++slot == ring_phases) {
      slot = 0;
      parity ^= 1;
    }
    float* mine = part + (size_t(phase) * kAwqPhaseTiles * kGemmWarps + warp) * kBlock + lane * 4;
    if (ok) {
#pragma unroll
      for (int t = 0; t < (kSwap ? 1 : kAwqPhaseTiles); ++t)
        *reinterpret_cast<float4*>(mine + size_t(t) * kGemmWarps * kBlock) = make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
    }
    // The decision to give up is the block's: a thread whose wait ran out raises the flag before the phase's
    // block-wide barrier and every thread reads it after (below, with the partials, and acts on it at the top of
    // the next phase, so the read costs the phase nothing).
    if (!ok) *failed = 1;
    __syncthreads();
    // Every warp has finished reading these stages: refill them with the tiles `stages` ahead.
    if (threadIdx.x == 0) issue(step + ring_phases);  // lands in the slot this phase has just left
#pragma unroll
    for (int t = 0; t < (kSwap ? 1 : kAwqPhaseTiles); ++t) {
      const float* src = part + ((size_t(phase) * kAwqPhaseTiles + t) * kGemmWarps + part_index) * kBlock + e;
#pragma unroll
      for (int w = 0; w < 4; ++w) loaded[t][w] = src[size_t(w) * 4 * kBlock];
    }
    gave_up = *failed;
    pending = step;
    steps_done = step + 1;
  }
  if (gave_up) {
    if (threadIdx.x == 0) {
      if (p.status) atomicOr(p.status, 4);
      // A block never leaves while a copy into its shared memory may be in flight: give every phase still in
      // the ring its chance to land (bounded again).
      for (int back = max(0, steps_done - 1); back < steps_done - 1 + ring_phases; ++back)
        if (back * kAwqPhaseTiles < item_count)
          mbarrier_wait(&full[back % ring_phases], uint32_t((back / ring_phases) & 1), wait_limit);
    }
    __syncthreads();
    return;
  }
  if (pending >= 0) {
    finish(pending, loaded);
    if ((pending & 3) != 3) emit(pending & ~3, pending);
  }
}

}  // namespace ei
