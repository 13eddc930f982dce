// Prompt (prefill) GEMM for sm_100a on the 5th-generation tensor cores: out[T,N] = x[T,K] * W[N,K]^T (+ bias) for
// T in the hundreds or thousands, W int4 (AWQ, group 128) or BF16.
//
// With many rows the projection is no longer bound by weight bytes but by arithmetic, so the small-M streaming
// kernels (one pass over the weights per 16 rows) are the wrong tool: here every weight is dequantised once per
// 256 tokens and multiplied on tcgen05.
//
// A block owns a tile of 256 output features and up to 256 tokens (two token tiles of 128, the M of one MMA), and
// walks K in blocks of 64 inputs through a ring of stages:
//   * one thread (warp 8) issues the TMA copies of a stage: the activations of both token tiles as
//     [128 tokens][64 inputs] BF16 boxes with the 128-byte swizzle (the K-major operand layout of tcgen05.mma),
//     and the weights - BF16 weights as one [256 features][64 inputs] swizzled box, int4 weights as a raw
//     [256 rows][32 bytes] box;
//   * for int4, warps 0-7 turn the raw box into the BF16 K-major swizzled operand in shared memory with the
//     exact dequantisation of the small-M kernels (dequant_pair: round_bf16((w - z) * scale)), fence the writes
//     towards the asynchronous proxy and arrive on the stage's `ready` barrier;
//   * one thread (warp 9) issues, per stage and token tile, four tcgen05.mma (M 128, N 256, K 16) that
//     accumulate in tensor memory - 2 token tiles x 256 FP32 columns = all 512 columns - and commits the stage's
//     `empty` barrier, which hands the stage back to the copy thread;
//   * after the last K block warps 0-7 read the accumulators with tcgen05.ld (warp w: lanes 32 (w % 4) ..., token
//     tile w / 4), add the bias in FP32, round once to BF16 and store whole output rows through shared memory -
//     or, for a projection whose sum the
//     residual + norm kernel finishes, store FP32 partial sums, K split over blockIdx.z so that few token tiles
//     still fill the SMs.
// Rows beyond T and features beyond N are zero-filled by TMA and masked in the epilogue.
//
// Every wait on an mbarrier is bounded. A role whose wait runs out raises a flag in shared memory that every
// other wait polls, so all roles leave their loops; the copy thread then waits (bounded) for its copies in
// flight, the MMA thread for the MMAs it issued, bit 2 of GemmParams::status is set and the tensor memory is
// freed before the block returns.
#pragma once

#include "awq_tma.cuh"

namespace ei {

constexpr int kPromptTokens = 128;     // tokens per token tile = M of one MMA
constexpr int kPromptTokenTiles = 2;   // token tiles per block
constexpr int kPromptFeatures = 256;   // output features per block = N of one MMA
constexpr int kPromptBlockK = 64;      // inputs per stage: one 128-byte swizzle row of BF16
constexpr int kPromptStages = 3;
constexpr int kPromptWorkerWarps = 8;
constexpr int kPromptThreads = (kPromptWorkerWarps + 2) * 32;
constexpr int kPromptTileBytes = kPromptTokens * kPromptBlockK * 2;                 // 16 KiB per token tile
constexpr int kPromptWeightBytes = kPromptFeatures * kPromptBlockK * 2;             // 32 KiB BF16 operand
constexpr int kPromptRawBytes = kPromptFeatures * (kPromptBlockK / 2);              // 8 KiB of int4
constexpr int kPromptStageBytes = kPromptTokenTiles * kPromptTileBytes + kPromptWeightBytes + kPromptRawBytes;
constexpr size_t kPromptSharedBytes = size_t(kPromptStages) * kPromptStageBytes + 1024 /* alignment */ + 256;

struct PromptMaps {
  CUtensorMap x;        // bf16 [T][K], box [128][64], 128-byte swizzle
  CUtensorMap weights;  // int4: u32 [N][K/8], box [256][8]; BF16: bf16 [N][K], box [256][64], 128-byte swizzle
};

struct PromptShared {
  uint64_t full[kPromptStages], ready[kPromptStages], empty[kPromptStages], done;
  uint32_t tmem_base;
  volatile int abort;
};

// ---- tcgen05 wrappers ----------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* shared_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_address(shared_result)),
               "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_address(bar))
               : "memory");
}
// D[tmem_d] (+)= A[desc_a] * B[desc_b]^T, both operands K-major in shared memory, FP32 accumulation.
__device__ __forceinline__ void umma_bf16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_load16(uint32_t address, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
      "[%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(address)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major, 128-byte-swizzled operand: rows 128 bytes apart, groups of eight
// rows 1024 bytes apart; bits [46,48) carry the descriptor version of this architecture, bits [61,64) the swizzle.
__device__ __forceinline__ uint64_t umma_kmajor_sw128_desc(uint32_t shared_address) {
  return uint64_t((shared_address & 0x3ffffu) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) |
         (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
// Instruction descriptor: D FP32, A and B BF16, both K-major, N = 256, M = 128.
constexpr uint32_t kPromptInstruction =
    (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t(kPromptFeatures) >> 3) << 17) | ((uint32_t(kPromptTokens) >> 4) << 24);

// Bounded wait that also gives up as soon as another role of the block has.
__device__ __forceinline__ bool prompt_wait(PromptShared* sh, uint64_t* bar, uint32_t parity, uint32_t limit) {
  if (mbarrier_test_wait(bar, parity)) return true;
  for (uint32_t polls = 0; polls < limit; ++polls) {
    if (mbarrier_try_wait(bar, parity)) return true;
    if (sh->abort) return false;
  }
  sh->abort = 1;
  return false;
}
__device__ __forceinline__ void mbarrier_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_address(bar)) : "memory");
}

template <bool kAwq>
__global__ void __launch_bounds__(kPromptThreads, 1)
    prompt_gemm_kernel(const __grid_constant__ PromptMaps maps, const GemmParams p) {
  extern __shared__ unsigned char prompt_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(prompt_smem_raw) + 1023) &
                                                         ~uintptr_t(1023));
  PromptShared* sh = reinterpret_cast<PromptShared*>(smem + size_t(kPromptStages) * kPromptStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // p.prompt_tiles (1 or 2) token tiles per block: chosen on the host so that the grid's waves are well filled.
  const int tiles_per_block = p.prompt_tiles == 1 ? 1 : kPromptTokenTiles;
  const int n0 = blockIdx.x * kPromptFeatures, t0 = blockIdx.y * (kPromptTokens * tiles_per_block);
  const int token_tiles = min(tiles_per_block, (p.M - t0 + kPromptTokens - 1) / kPromptTokens);
  // K slice of this block (blockIdx.z of p.ksplit): whole quantisation groups, i.e. pairs of K blocks.
  const int slice = blockIdx.z;
  const int pairs_total = p.K / (2 * kPromptBlockK);
  const int kb_begin = p.ksplit > 1 ? int((long long)slice * pairs_total / p.ksplit) * 2 : 0;
  const int kb_end = p.ksplit > 1 ? int((long long)(slice + 1) * pairs_total / p.ksplit) * 2 : p.K / kPromptBlockK;
  const int k_blocks = kb_end - kb_begin;
  const uint32_t limit = p.wait_limit ? p.wait_limit : kAwqWaitLimit;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPromptStages; ++s) {
      mbarrier_init(&sh->full[s], 1);
      mbarrier_init(&sh->ready[s], kPromptWorkerWarps);
      mbarrier_init(&sh->empty[s], 1);
    }
    mbarrier_init(&sh->done, 1);
    sh->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kPromptWorkerWarps + 1) tmem_alloc(&sh->tmem_base, 512);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem = sh->tmem_base;
  grid_dependency_wait();
  grid_launch_dependents();

  auto stage_base = [&](int s) { return smem + size_t(s) * kPromptStageBytes; };
  constexpr int kWeightOffset = kPromptTokenTiles * kPromptTileBytes;
  constexpr int kRawOffset = kWeightOffset + kPromptWeightBytes;

  if (warp == kPromptWorkerWarps) {
    // ---- copy thread ----
    if (lane == 0) {
      const uint32_t bytes = uint32_t(token_tiles) * kPromptTileBytes + (kAwq ? kPromptRawBytes : kPromptWeightBytes);
      int issued = 0;
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % kPromptStages;
        if (kb >= kPromptStages && !prompt_wait(sh, &sh->empty[s], ((kb / kPromptStages) - 1) & 1, limit)) break;
        mbarrier_expect_tx(&sh->full[s], bytes + (kb == 0 ? p.fault_tx : 0u));
        unsigned char* base = stage_base(s);
        for (int mt = 0; mt < token_tiles; ++mt)
          tma_load_2d(base + mt * kPromptTileBytes, &maps.x, (kb_begin + kb) * kPromptBlockK, t0 + mt * kPromptTokens,
                      &sh->full[s]);
        if (kAwq)
          tma_load_2d(base + kRawOffset, &maps.weights, (kb_begin + kb) * (kPromptBlockK / 8), n0, &sh->full[s]);
        else
          tma_load_2d(base + kWeightOffset, &maps.weights, (kb_begin + kb) * kPromptBlockK, n0, &sh->full[s]);
        issued = kb + 1;
      }
      if (sh->abort) {
        // Copies still in flight write into this block's shared memory: wait for them (bounded) before leaving.
        // The copy of K block 0 carries the test hook's unmet expectation and is known never to complete.
        for (int kb = max(p.fault_tx ? 1 : 0, issued - kPromptStages); kb < issued; ++kb) {
          const int s = kb % kPromptStages;
          for (uint32_t polls = 0; polls < limit; ++polls)
            if (mbarrier_try_wait(&sh->full[s], (kb / kPromptStages) & 1)) break;
        }
      }
    }
  } else if (warp == kPromptWorkerWarps + 1) {
    // ---- MMA thread ----
    if (lane == 0) {
      bool issued = false;
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % kPromptStages;
        if (!prompt_wait(sh, kAwq ? &sh->ready[s] : &sh->full[s], (kb / kPromptStages) & 1, limit)) break;
        tcgen05_fence_after();
        const uint32_t base = smem_address(stage_base(s));
        const uint64_t b_desc = umma_kmajor_sw128_desc(base + kWeightOffset);
        for (int mt = 0; mt < token_tiles; ++mt) {
          const uint64_t a_desc = umma_kmajor_sw128_desc(base + mt * kPromptTileBytes);
#pragma unroll
          for (int j = 0; j < kPromptBlockK / 16; ++j)  // 16 inputs = 32 bytes further along the swizzled row
            umma_bf16_ss(tmem + mt * kPromptFeatures, a_desc + uint64_t(j * 2), b_desc + uint64_t(j * 2),
                         kPromptInstruction, (kb > 0 || j > 0) ? 1u : 0u);
        }
        tcgen05_commit(&sh->empty[s]);
        issued = true;
      }
      tcgen05_commit(&sh->done);  // arrives when every MMA issued so far has completed
      if (sh->abort && issued) {
        for (uint32_t polls = 0; polls < limit; ++polls)
          if (mbarrier_try_wait(&sh->done, 0)) break;
      }
    }
  } else {
    // ---- workers: dequantisation (int4 only), then the epilogue ----
    if (kAwq) {
      // Thread t converts (row t / 2, half t % 2) and (row 128 + t / 2, half t % 2) of every stage: a half is 32
      // inputs = 16 raw bytes = four 16-byte chunks of the operand row.
      const int half = threadIdx.x & 1;
      int rows[2], live_rows[2];
      rows[0] = threadIdx.x >> 1;
      rows[1] = 128 + rows[0];
#pragma unroll
      for (int i = 0; i < 2; ++i) live_rows[i] = min(n0 + rows[i], p.N - 1);
      // Scales and zero points of a group are requested one group (two K blocks) before they are used.
      uint32_t scale2[2] = {0, 0}, zero_word[2] = {0, 0}, scale_next[2], zero_next[2];
      const int group_begin = kb_begin >> 1, group_end = kb_end >> 1;
      auto request = [&](int g) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          scale_next[i] = uint32_t(__bfloat16_as_ushort(p.scales[size_t(live_rows[i]) * p.padded_groups + g])) * 0x10001u;
          zero_next[i] = ((g & 7) == 0 || g == group_begin) ? uint32_t(p.zeros[size_t(live_rows[i]) * p.zero_stride + (g >> 3)]) : zero_word[i];
        }
      };
      request(group_begin);
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % kPromptStages;
        const int grp = (kb_begin + kb) >> 1;  // 128 inputs per group, 64 per K block
        if ((kb & 1) == 0) {
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            scale2[i] = scale_next[i];
            zero_word[i] = zero_next[i];
          }
          if (grp + 1 < group_end) request(grp + 1);
        }
        // The loop is left by whole warps: the barrier and the vote below are warp-wide.
        const bool arrived = prompt_wait(sh, &sh->full[s], (kb / kPromptStages) & 1, limit);
        if (!__all_sync(0xffffffffu, arrived)) break;
        unsigned char* base = stage_base(s);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int row = rows[i];
          const uint4 raw = *reinterpret_cast<const uint4*>(base + kRawOffset + row * 32 + half * 16);
          const uint32_t zero2 = (0x4300u | ((zero_word[i] >> ((grp & 7) * 4)) & 15u)) * 0x10001u;
          const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            // dequant_pair gives (k, k + 4) pairs; the operand wants the eight inputs of a word in order.
            const uint32_t p0 = dequant_pair(words[w], zero2, scale2[i]);
            const uint32_t p1 = dequant_pair(words[w] >> 4, zero2, scale2[i]);
            const uint32_t p2 = dequant_pair(words[w] >> 8, zero2, scale2[i]);
            const uint32_t p3 = dequant_pair(words[w] >> 12, zero2, scale2[i]);
            uint4 o;
            o.x = __byte_perm(p0, p1, 0x5410);
            o.y = __byte_perm(p2, p3, 0x5410);
            o.z = __byte_perm(p0, p1, 0x7632);
            o.w = __byte_perm(p2, p3, 0x7632);
            const int chunk = (half * 4 + w) ^ (row & 7);
            *reinterpret_cast<uint4*>(base + kWeightOffset + row * 128 + chunk * 16) = o;
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbarrier_arrive(&sh->ready[s]);
      }
    }
    // ---- epilogue ----
    const bool complete = __all_sync(0xffffffffu, prompt_wait(sh, &sh->done, 0, limit) && !sh->abort);
    tcgen05_fence_after();
    const int quarter = warp & 3, mt = warp >> 2;
    if (complete && mt < token_tiles) {
      // The accumulators come out of tensor memory one token per lane, which would make every store of a warp hit
      // 32 different output rows. They go through shared memory instead (the ring's stages are free by now; a
      // padded row pitch keeps both directions conflict-free), 128 columns at a time, and leave as whole rows:
      // sixteen lanes write 256 contiguous bytes of a BF16 row (thirty-two lanes 512 bytes of an FP32 one).
      const bool partial = p.epilogue == kEpiPartial;
      constexpr int kPitch = 528;  // bytes per staged row: 512 of FP32 (or 256 of BF16) plus 16
      unsigned char* staged = smem + size_t(warp) * 32 * kPitch;
      const int first_token = t0 + mt * kPromptTokens + quarter * 32;
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        if (n0 + half * 128 >= p.N) break;  // block-uniform
#pragma unroll 1
        for (int cb = 0; cb < 8; ++cb) {
          float v[16];
          tmem_load16(tmem + (uint32_t(quarter * 32) << 16) + mt * kPromptFeatures + half * 128 + cb * 16, v);
          if (partial) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<float4*>(staged + lane * kPitch + cb * 64 + i * 16) =
                  make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          } else {
            uint32_t packed[8];
            const int column = n0 + half * 128 + cb * 16;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float a = v[2 * i], b = v[2 * i + 1];
              if (p.bias && column + 2 * i + 1 < p.N) {
                a += __bfloat162float(p.bias[column + 2 * i]);
                b += __bfloat162float(p.bias[column + 2 * i + 1]);
              }
              packed[i] = pack_bf16(a, b);
            }
            *reinterpret_cast<uint4*>(staged + lane * kPitch + cb * 32) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            *reinterpret_cast<uint4*>(staged + lane * kPitch + cb * 32 + 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
          }
        }
        __syncwarp();
        if (partial) {
          // One staged row (128 floats) per instruction.
          const int column = n0 + half * 128 + lane * 4;
#pragma unroll 4
          for (int r = 0; r < 32; ++r) {
            const int token = first_token + r;
            if (token < p.M && column < p.N)
              *reinterpret_cast<float4*>(p.partial + (size_t(slice) * p.M + token) * p.N + column) =
                  *reinterpret_cast<const float4*>(staged + r * kPitch + lane * 16);
          }
        } else {
          // Two staged rows (128 BF16 values each) per instruction.
          const int column = n0 + half * 128 + (lane & 15) * 8;
#pragma unroll 4
          for (int r = lane >> 4; r < 32; r += 2) {
            const int token = first_token + r;
            if (token < p.M && column < p.N)
              *reinterpret_cast<uint4*>(p.out + size_t(token) * p.out_stride + column) =
                  *reinterpret_cast<const uint4*>(staged + r * kPitch + (lane & 15) * 16);
          }
        }
        __syncwarp();
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  if (warp == kPromptWorkerWarps + 1) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
  if (threadIdx.x == 0 && sh->abort && p.status) atomicOr(p.status, 4);
}

}  // namespace ei
