// Causal verify attention for q_len = k + 1 <= 16 query rows over a session's KV cache
// (head_dim 128, grouped-query heads).
//
// The path is bound by KV bytes, so each KV byte is fetched once: a block owns one KV head and
// one chunk of the sequence, and serves every query row of every query head of that KV group
// (rows * heads/kv_heads <= 112 stacked rows, one 16-row MMA tile per warp). K and V tiles of
// 64 tokens are brought into shared memory by TMA (one tiled copy each for K and V, issued by one thread,
// completing on an mbarrier; a ring of three tiles per block, every wait bounded) in the 128-byte-swizzled
// layout [half of the head][token][128 B], which makes the fragment loads conflict-free. Scores, running maxima and sums
// stay in FP32; numerators are rounded to BF16 only as the A operand of the PV product while the
// denominator adds the unrounded values - the staging of the reference kernel
// (operators/src/cuda/kernels/flash_attn_prefill.cu:236-252). Chunks write (o, m, l) partials to
// caller scratch and a second kernel merges the live chunks in FP32 and rounds once.
// The position of the first query row is read from device memory, so a captured graph can be
// replayed while the context grows; blocks beyond the live length return immediately.
#include "kernels.cuh"

#include <algorithm>
#include <cfloat>
#include <stdexcept>

namespace ei {
namespace {

constexpr int kTile = 64;          // tokens per shared-memory tile
constexpr int kDim = 128;
constexpr int kPartial = 132;      // floats per (split, row, head): 128 outputs, m, l, padding
constexpr int kTileBytes = kTile * kDim * 2;

constexpr int kStages = 3;                     // K/V tiles in flight per block
constexpr int kStageBytes = 2 * kTileBytes;    // one K tile and one V tile
constexpr size_t kAttentionShared = size_t(kStages) * kStageBytes + 1024 /* alignment */ + 64;

struct AttentionShared {
  uint64_t full[kStages];
  int failed;
};

// Byte offset of (token, 16-byte chunk of the 256-byte head row) inside a staged tile: the two 128-byte halves
// of the rows are stored one after the other, and inside a half the chunk index is XORed with (token & 7).
__device__ __forceinline__ int tile_offset(int token, int chunk) {
  return (chunk >> 3) * (kTile * 128) + token * 128 + (((chunk & 7) ^ (token & 7)) << 4);
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                                  const void* smem_ptr) {
  const uint32_t address = static_cast<uint32_t>(__cvta_generic_to_shared(smem_ptr));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(address));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* smem_ptr) {
  const uint32_t address = static_cast<uint32_t>(__cvta_generic_to_shared(smem_ptr));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(address));
}

// kDirect = false: the verify step. Block (split, kv head) covers one chunk of the sequence for all <= 16 query
// rows and writes (o, m, l) partials for the merge kernel.
// kDirect = true: a prompt of many rows. Block (query block, kv head) covers 16 consecutive query rows over their
// whole causal history and writes the normalised output itself; blocks with the longest histories start first.
template <bool kDirect>
__global__ void __launch_bounds__(224) verify_attention_kernel(const __grid_constant__ AttentionParams p) {
  extern __shared__ unsigned char attention_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(attention_smem_raw) + 1023) &
                                                         ~uintptr_t(1023));
  AttentionShared* sh = reinterpret_cast<AttentionShared*>(smem + size_t(kStages) * kStageBytes);
  // The context length was written by the previous step; the preceding kernel of this step only appends the
  // new rows [offset, offset + rows). A chunk that ends before them can start fetching at once.
  // Wide batch (split form only): grid slice z is a session with its own cache, context length, queries, scratch.
  const SessionSlot* owner = (!kDirect && p.slots) ? p.slots + blockIdx.z : nullptr;
  const int capacity = owner ? owner->capacity : p.capacity;
  const int first_offset = owner ? owner->control->context : (p.device_offset ? *p.device_offset : p.host_offset);
  // The KV heads of one stretch of tokens are neighbours in the grid, so the blocks that read the same cache rows
  // (one 256-byte piece each) run at about the same time.
  const int kv_head = blockIdx.x;
  if (first_offset < 0 || first_offset + p.rows > capacity) {
    // The whole grid leaves: it still waits for its predecessor first, so that a successor never sees this
    // kernel complete before the kernels ahead of it have.
    grid_dependency_wait();
    return;
  }
  const int first_row = kDirect ? (int(gridDim.y) - 1 - int(blockIdx.y)) * 16 : 0;
  const int rows = kDirect ? min(16, p.rows - first_row) : p.rows;
  const int offset = first_offset + first_row;
  const int length = offset + rows;
  const int split = kDirect ? 0 : blockIdx.y;
  const int start = kDirect ? 0 : split * p.chunk;
  if (start >= length) return;  // other blocks of the grid wait
  const int end = kDirect ? length : min(start + p.chunk, length);
  const int group = p.heads / p.kv_heads;
  const int stacked = rows * group;  // query rows served by this block
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;

  const CUtensorMap* k_map = owner ? p.maps + 2 * blockIdx.z : &p.k_map;
  const CUtensorMap* v_map = owner ? p.maps + 2 * blockIdx.z + 1 : &p.v_map;
  const int layer = owner ? p.layer : 0;
  const bf16* q_base = p.q + (owner ? size_t(blockIdx.z) * p.rows * p.q_stride : 0);
  float* scratch = p.scratch + (owner ? size_t(blockIdx.z) * p.scratch_stride : 0);
  const uint32_t wait_limit = p.wait_limit ? p.wait_limit : kTmaWaitLimit;
  const int tiles = (end - start + kTile - 1) / kTile;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) mbarrier_init(&sh->full[s], 1);
    sh->failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // One thread requests a tile: the K and the V box of 64 tokens of this KV head, one stage of the ring.
  auto request = [&](int tile) {
    const int stage = tile % kStages;
    unsigned char* base = smem + size_t(stage) * kStageBytes;
    mbarrier_expect_tx(&sh->full[stage], uint32_t(kStageBytes) + (tile == 0 ? p.fault_tx : 0u));
    tma_load_5d(base, k_map, 0, start + tile * kTile, 0, kv_head, layer, &sh->full[stage]);
    tma_load_5d(base + kTileBytes, v_map, 0, start + tile * kTile, 0, kv_head, layer, &sh->full[stage]);
  };

  const bool settled = end <= offset;  // no row of this chunk is written by the preceding kernel
  if (!settled) grid_dependency_wait();
  if (threadIdx.x == 0)
    for (int tile = 0; tile < min(kStages, tiles); ++tile) request(tile);
  if (settled) grid_dependency_wait();  // the queries come from the preceding kernel
  // Only now: a kernel that triggers after its own wait lets its successor's prologue see everything up to the
  // kernel before this one as complete, which is what the early fetch above relies on.
  grid_launch_dependents();

  // Stacked row i = r * group + hq  ->  query row r, query head kv_head * group + hq.
  const int i_lo = warp * 16 + g, i_hi = i_lo + 8;
  const bool live_lo = i_lo < stacked, live_hi = i_hi < stacked;
  const int r_lo = live_lo ? i_lo / group : 0, r_hi = live_hi ? i_hi / group : 0;
  const int h_lo = kv_head * group + (live_lo ? i_lo % group : 0);
  const int h_hi = kv_head * group + (live_hi ? i_hi % group : 0);
  uint32_t qa[8][4];
  {
    const bf16* q_lo = q_base + size_t(first_row + r_lo) * p.q_stride + size_t(h_lo) * kDim;
    const bf16* q_hi = q_base + size_t(first_row + r_hi) * p.q_stride + size_t(h_hi) * kDim;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      qa[kk][0] = live_lo ? *reinterpret_cast<const uint32_t*>(q_lo + kk * 16 + 2 * c) : 0u;
      qa[kk][1] = live_hi ? *reinterpret_cast<const uint32_t*>(q_hi + kk * 16 + 2 * c) : 0u;
      qa[kk][2] = live_lo ? *reinterpret_cast<const uint32_t*>(q_lo + kk * 16 + 8 + 2 * c) : 0u;
      qa[kk][3] = live_hi ? *reinterpret_cast<const uint32_t*>(q_hi + kk * 16 + 8 + 2 * c) : 0u;
    }
  }
  // Last visible token of each row (causal): offset + r.
  const int limit_lo = offset + r_lo, limit_hi = offset + r_hi;
  const float scale = rsqrtf(float(kDim));

  float o[16][4];
#pragma unroll
  for (int d = 0; d < 16; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;

  int tile = 0;
  bool gave_up = false;
  for (; tile < tiles; ++tile) {
    const int stage = tile % kStages;
    if (!mbarrier_wait(&sh->full[stage], (tile / kStages) & 1, wait_limit)) sh->failed = 1;
    unsigned char* ks = smem + size_t(stage) * kStageBytes;
    unsigned char* vs = ks + kTileBytes;
    const int first = start + tile * kTile;
    if (end - first < kTile) {
      // The last tile reaches past the live rows: what the copy brought for them is whatever the cache holds
      // there (rows of rejected drafts, or memory never written). Their scores are masked below; their V rows
      // are cleared so that a non-finite leftover cannot reach the PV product through a zero weight.
      const int live = end - first;
      for (int i = threadIdx.x; i < (kTile - live) * 16; i += blockDim.x) {
        const int token = live + (i >> 4), chunk = i & 15;
        *reinterpret_cast<uint4*>(vs + tile_offset(token, chunk)) = make_uint4(0, 0, 0, 0);
      }
      __syncthreads();
    }

    // S = Q K^T: n-tile j covers tokens 8j..8j+7. One ldmatrix.x4 brings the K fragments of two k-steps (four
    // 16-byte chunks of eight token rows: lane l addresses row l & 7 of chunk l >> 3); the eight accumulators take
    // their k-steps in ascending order, interleaved so that consecutive MMAs do not depend on each other.
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
    for (int pair = 0; pair < 4; ++pair) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, ks + tile_offset(j * 8 + (lane & 7), 4 * pair + (lane >> 3)));
        mma_bf16_16816(s[j], qa[2 * pair][0], qa[2 * pair][1], qa[2 * pair][2], qa[2 * pair][3], b0, b1);
        mma_bf16_16816(s[j], qa[2 * pair + 1][0], qa[2 * pair + 1][1], qa[2 * pair + 1][2], qa[2 * pair + 1][3], b2, b3);
      }
    }
    // Scale, mask (causal and beyond-the-end), running maximum.
    float tile_max_lo = -INFINITY, tile_max_hi = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int t0 = first + j * 8 + 2 * c, t1 = t0 + 1;
      s[j][0] = t0 <= limit_lo ? s[j][0] * scale : -INFINITY;
      s[j][1] = t1 <= limit_lo ? s[j][1] * scale : -INFINITY;
      s[j][2] = t0 <= limit_hi ? s[j][2] * scale : -INFINITY;
      s[j][3] = t1 <= limit_hi ? s[j][3] * scale : -INFINITY;
      tile_max_lo = fmaxf(tile_max_lo, fmaxf(s[j][0], s[j][1]));
      tile_max_hi = fmaxf(tile_max_hi, fmaxf(s[j][2], s[j][3]));
    }
    tile_max_lo = fmaxf(tile_max_lo, __shfl_xor_sync(0xffffffffu, tile_max_lo, 1));
    tile_max_lo = fmaxf(tile_max_lo, __shfl_xor_sync(0xffffffffu, tile_max_lo, 2));
    tile_max_hi = fmaxf(tile_max_hi, __shfl_xor_sync(0xffffffffu, tile_max_hi, 1));
    tile_max_hi = fmaxf(tile_max_hi, __shfl_xor_sync(0xffffffffu, tile_max_hi, 2));
    const float new_lo = fmaxf(m_lo, tile_max_lo), new_hi = fmaxf(m_hi, tile_max_hi);
    // A row with nothing visible yet keeps m = -inf; use 0 as the exponent base so exp() gives 0.
    const float base_lo = new_lo == -INFINITY ? 0.0f : new_lo;
    const float base_hi = new_hi == -INFINITY ? 0.0f : new_hi;
    const float rescale_lo = __expf(m_lo - base_lo), rescale_hi = __expf(m_hi - base_hi);
    m_lo = new_lo;
    m_hi = new_hi;
    float sum_lo = 0.0f, sum_hi = 0.0f;
    uint32_t pa[8][2];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float p0 = __expf(s[j][0] - base_lo), p1 = __expf(s[j][1] - base_lo);
      const float p2 = __expf(s[j][2] - base_hi), p3 = __expf(s[j][3] - base_hi);
      sum_lo += p0 + p1;
      sum_hi += p2 + p3;
      pa[j][0] = pack_bf16(p0, p1);
      pa[j][1] = pack_bf16(p2, p3);
    }
    l_lo = l_lo * rescale_lo + sum_lo;  // per-lane partial; the quad is summed at the end
    l_hi = l_hi * rescale_hi + sum_hi;
#pragma unroll
    for (int d = 0; d < 16; ++d) {
      o[d][0] *= rescale_lo;
      o[d][1] *= rescale_lo;
      o[d][2] *= rescale_hi;
      o[d][3] *= rescale_hi;
    }
    // O += P V : k-step t covers tokens 16t..16t+15, n-tile d covers dims 8d..8d+7.
#pragma unroll
    for (int t = 0; t < 4; ++t) {
#pragma unroll
      for (int d = 0; d < 16; d += 2) {
        const int matrix = lane >> 3, row = lane & 7;
        const int token = t * 16 + (matrix & 1) * 8 + row;
        const int chunk = d + (matrix >> 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, vs + tile_offset(token, chunk));
        mma_bf16_16816(o[d], pa[2 * t][0], pa[2 * t][1], pa[2 * t + 1][0], pa[2 * t + 1][1], b0, b1);
        mma_bf16_16816(o[d + 1], pa[2 * t][0], pa[2 * t][1], pa[2 * t + 1][0], pa[2 * t + 1][1], b2, b3);
      }
    }
    __syncthreads();  // every warp is done with this stage
    gave_up = sh->failed != 0;  // written before the barrier by any thread whose wait ran out: block-uniform
    if (gave_up) break;
    if (threadIdx.x == 0 && tile + kStages < tiles) request(tile + kStages);
  }
  if (gave_up) {
    // Copies still in flight write into this block's shared memory: wait for them (bounded) before leaving. The
    // copy of tile 0 carries the test hook's unmet expectation when that is armed and is known not to complete.
    if (threadIdx.x == 0) {
      for (int t = max(tile, p.fault_tx ? 1 : 0); t < min(tile + kStages, tiles); ++t)
        mbarrier_wait(&sh->full[t % kStages], (t / kStages) & 1, wait_limit);
      if (p.status) atomicOr(p.status, 4);
    }
    return;
  }

  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

  if (kDirect) {
    const float inverse_lo = l_lo > 0.0f ? 1.0f / l_lo : 0.0f, inverse_hi = l_hi > 0.0f ? 1.0f / l_hi : 0.0f;
    if (live_lo) {
      bf16* dst = p.out + size_t(first_row + r_lo) * p.out_stride + size_t(h_lo) * kDim;
#pragma unroll
      for (int d = 0; d < 16; ++d)
        *reinterpret_cast<uint32_t*>(dst + d * 8 + 2 * c) = pack_bf16(o[d][0] * inverse_lo, o[d][1] * inverse_lo);
    }
    if (live_hi) {
      bf16* dst = p.out + size_t(first_row + r_hi) * p.out_stride + size_t(h_hi) * kDim;
#pragma unroll
      for (int d = 0; d < 16; ++d)
        *reinterpret_cast<uint32_t*>(dst + d * 8 + 2 * c) = pack_bf16(o[d][2] * inverse_hi, o[d][3] * inverse_hi);
    }
    return;
  }
  const size_t slots = size_t(p.rows) * p.heads;
  if (live_lo) {
    float* dst = scratch + (size_t(split) * slots + size_t(r_lo) * p.heads + h_lo) * kPartial;
#pragma unroll
    for (int d = 0; d < 16; ++d) *reinterpret_cast<float2*>(dst + d * 8 + 2 * c) = make_float2(o[d][0], o[d][1]);
    if (c == 0) {
      dst[128] = m_lo;
      dst[129] = l_lo;
    }
  }
  if (live_hi) {
    float* dst = scratch + (size_t(split) * slots + size_t(r_hi) * p.heads + h_hi) * kPartial;
#pragma unroll
    for (int d = 0; d < 16; ++d) *reinterpret_cast<float2*>(dst + d * 8 + 2 * c) = make_float2(o[d][2], o[d][3]);
    if (c == 0) {
      dst[128] = m_hi;
      dst[129] = l_hi;
    }
  }
}

// One block of four warps per (row, head). The live splits (at most 64) are read in parallel: thread s
// fetches split s's maximum and sum, the block agrees on the global maximum, then warp w accumulates
// splits w, w+4, ... and the four partial sums are added in warp order. The order of every addition is
// fixed, so replays give identical bits.
__global__ void __launch_bounds__(128) attention_merge_kernel(const AttentionParams p) {
  __shared__ float weights[64];
  __shared__ float warp_values[4];
  __shared__ float4 partial_out[4][32];
  // The context length was written by the previous step (or by the host): it does not come from the kernel
  // this one waits for, so it is read first and the wait hides its latency.
  const SessionSlot* owner = p.slots ? p.slots + blockIdx.y : nullptr;
  const int offset = owner ? owner->control->context : (p.device_offset ? *p.device_offset : p.host_offset);
  grid_dependency_wait();
  grid_launch_dependents();
  const int slot = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = p.rows * p.heads;
  const int length = offset + p.rows;
  if (offset < 0 || length > (owner ? owner->capacity : p.capacity)) return;  // after the wait above
  const float* scratch = p.scratch + (owner ? size_t(blockIdx.y) * p.scratch_stride : 0);
  bf16* out = p.out + (owner ? size_t(blockIdx.y) * p.rows * p.out_stride : 0);
  const int splits = min(64, (length + p.chunk - 1) / p.chunk);
  // This warp's splits (w, w + 4, ...) are requested together with the maxima and sums, so that the block pays
  // one trip to memory instead of two.
  float4 values[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int s = warp + 4 * i;
    values[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (s < splits)
      values[i] = *reinterpret_cast<const float4*>(scratch + (size_t(s) * slots + slot) * kPartial + 4 * lane);
  }
  float m = -INFINITY, l = 0.0f;
  if (int(threadIdx.x) < splits) {
    const float* src = scratch + (size_t(threadIdx.x) * slots + slot) * kPartial;
    m = src[128];
    l = src[129];
  }
  float maximum = warp_max(m);
  if (lane == 0) warp_values[warp] = maximum;
  __syncthreads();
  maximum = fmaxf(fmaxf(warp_values[0], warp_values[1]), fmaxf(warp_values[2], warp_values[3]));
  const float weight = m == -INFINITY ? 0.0f : __expf(m - maximum);  // a split with nothing visible counts 0
  if (threadIdx.x < 64) weights[threadIdx.x] = weight;
  float denominator = warp_sum(l * weight);
  __syncthreads();
  if (lane == 0) warp_values[warp] = denominator;
  float4 accumulator = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int s = warp + 4 * i;
    if (s < splits) {
      const float w = weights[s];
      accumulator.x += values[i].x * w;
      accumulator.y += values[i].y * w;
      accumulator.z += values[i].z * w;
      accumulator.w += values[i].w * w;
    }
  }
  partial_out[warp][lane] = accumulator;
  __syncthreads();
  if (warp != 0) return;
  denominator = (warp_values[0] + warp_values[1]) + (warp_values[2] + warp_values[3]);
  const float4 a = partial_out[0][lane], b = partial_out[1][lane], c = partial_out[2][lane], d = partial_out[3][lane];
  const float inverse = denominator > 0.0f ? 1.0f / denominator : 0.0f;
  const int row = slot / p.heads, head = slot - row * p.heads;
  bf16* dst = out + size_t(row) * p.out_stride + size_t(head) * kDim + 4 * lane;
  uint2 packed;
  packed.x = pack_bf16(((a.x + b.x) + (c.x + d.x)) * inverse, ((a.y + b.y) + (c.y + d.y)) * inverse);
  packed.y = pack_bf16(((a.z + b.z) + (c.z + d.z)) * inverse, ((a.w + b.w) + (c.w + d.w)) * inverse);
  *reinterpret_cast<uint2*>(dst) = packed;
}

// The merge for a wide batch: one WARP per (session, row, head) and no block-wide barrier, four per block. With
// thousands of (row, head) slots a block per slot costs one launch wave after another of blocks that each wait on
// two trips to memory; here a warp requests all of its slot's partials (lane l owns outputs 4l .. 4l + 3) before it
// combines them in split order.
__global__ void __launch_bounds__(128) attention_merge_wide_kernel(const AttentionParams p) {
  grid_dependency_wait();
  grid_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int slots = p.rows * p.heads;
  const int slot_global = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (slot_global >= slots * p.sessions) return;
  const int session = slot_global / slots, slot = slot_global - session * slots;
  const SessionSlot owner = p.slots[session];
  const int offset = owner.control->context, length = offset + p.rows;
  if (offset < 0 || length > owner.capacity) return;
  const int splits = min(64, (length + p.chunk - 1) / p.chunk);
  const float* base = p.scratch + size_t(session) * p.scratch_stride + size_t(slot) * kPartial;
  const size_t step = size_t(slots) * kPartial;
  float maximum = -INFINITY;
  for (int s = lane; s < splits; s += 32) maximum = fmaxf(maximum, base[s * step + 128]);
  maximum = warp_max(maximum);
  float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  float denominator = 0.0f;
  for (int first = 0; first < splits; first += 8) {
    float4 values[8];
    float m[8], l[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int s = first + i;
      values[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      m[i] = -INFINITY;
      l[i] = 0.0f;
      if (s < splits) {
        const float* src = base + s * step;
        values[i] = *reinterpret_cast<const float4*>(src + 4 * lane);
        m[i] = src[128];
        l[i] = src[129];
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float weight = m[i] == -INFINITY ? 0.0f : __expf(m[i] - maximum);  // a split with nothing visible counts 0
      sum.x = fmaf(values[i].x, weight, sum.x);
      sum.y = fmaf(values[i].y, weight, sum.y);
      sum.z = fmaf(values[i].z, weight, sum.z);
      sum.w = fmaf(values[i].w, weight, sum.w);
      denominator = fmaf(l[i], weight, denominator);
    }
  }
  const float inverse = denominator > 0.0f ? 1.0f / denominator : 0.0f;
  const int row = slot / p.heads, head = slot - row * p.heads;
  bf16* dst = p.out + (size_t(session) * p.rows + row) * p.out_stride + size_t(head) * kDim + 4 * lane;
  uint2 packed;
  packed.x = pack_bf16(sum.x * inverse, sum.y * inverse);
  packed.y = pack_bf16(sum.z * inverse, sum.w * inverse);
  *reinterpret_cast<uint2*>(dst) = packed;
}

}  // namespace

int attention_chunk_for(size_t kv_length) {
  // At most 64 splits; chunks are whole tiles.
  const size_t tiles = (kv_length + kTile - 1) / kTile;
  const size_t tiles_per_chunk = std::max<size_t>(1, (tiles + 63) / 64);
  return int(tiles_per_chunk * kTile);
}

size_t attention_scratch_bytes(size_t rows, size_t heads, size_t kv_length) {
  const size_t chunk = attention_chunk_for(kv_length);
  const size_t splits = (kv_length + chunk - 1) / chunk;
  return splits * rows * heads * kPartial * sizeof(float);
}

namespace {
void configure_attention_kernels() {
  static thread_local int configured_device = -1;
  int device = 0;
  EI_CUDA(cudaGetDevice(&device));
  if (configured_device == device) return;
  EI_CUDA(cudaFuncSetAttribute(verify_attention_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               int(kAttentionShared)));
  EI_CUDA(cudaFuncSetAttribute(verify_attention_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               int(kAttentionShared)));
  configured_device = device;
}

// The parameters with the single session's tensor maps filled in (a wide batch brings its own).
AttentionParams with_maps(const AttentionParams& p) {
  AttentionParams q = p;
  if (!q.slots) {
    encode_kv_map(&q.k_map, q.k, size_t(q.capacity), size_t(q.kv_stride), q.kv_heads, 1, 0);
    encode_kv_map(&q.v_map, q.v, size_t(q.capacity), size_t(q.kv_stride), q.kv_heads, 1, 0);
  } else if (!q.maps) {
    throw std::invalid_argument("A wide attention launch needs the sessions' tensor maps");
  }
  return q;
}
}  // namespace

void encode_kv_map(CUtensorMap* map, const bf16* base, size_t tokens, size_t token_stride, int kv_heads, size_t layers,
                   size_t layer_stride) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) || token_stride % 8 || layer_stride % 8)
    throw std::invalid_argument("K / V rows must be 16-byte aligned");
  const cuuint64_t dims[5] = {64, cuuint64_t(tokens), 2, cuuint64_t(kv_heads), cuuint64_t(std::max<size_t>(1, layers))};
  const cuuint64_t strides[4] = {cuuint64_t(token_stride) * 2, 128, 256,
                                 cuuint64_t(layers > 1 ? layer_stride : token_stride * std::max<size_t>(1, tokens)) * 2};
  const cuuint32_t box[5] = {64, cuuint32_t(kTile), 2, 1, 1};
  encode_map(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
             "K / V cache");
}

void launch_verify_attention(const AttentionParams& p, cudaStream_t stream, bool pdl) {
  const int group = p.heads / p.kv_heads;
  const int warps = (p.rows * group + 15) / 16;
  configure_attention_kernels();
  const AttentionParams q = with_maps(p);
  const unsigned sessions = q.slots ? unsigned(q.sessions) : 1u;
  launch(verify_attention_kernel<false>, dim3(q.kv_heads, q.max_splits, sessions), dim3(warps * 32), kAttentionShared,
         stream, pdl, q);
  if (q.slots)
    launch(attention_merge_wide_kernel, dim3((q.rows * q.heads * q.sessions + 3) / 4), dim3(128), 0, stream, pdl, q);
  else
    launch(attention_merge_kernel, dim3(q.rows * q.heads, sessions), dim3(128), 0, stream, pdl, q);
}

void launch_prompt_attention(const AttentionParams& p, cudaStream_t stream, bool pdl) {
  const int group = p.heads / p.kv_heads;
  configure_attention_kernels();
  const AttentionParams q = with_maps(p);
  launch(verify_attention_kernel<true>, dim3(q.kv_heads, (q.rows + 15) / 16), dim3(group * 32), kAttentionShared,
         stream, pdl, q);
}

}  // namespace ei
