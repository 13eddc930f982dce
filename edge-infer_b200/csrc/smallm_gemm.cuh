// Small-M (<= 16 rows) weight-streaming GEMM for sm_100a: out[M,N] = x[M,K] * W[N,K]^T (+ bias).
//
// The path is HBM-bound: every weight byte is read exactly once per call, straight from
// global memory into registers with 128-bit loads (each quad of lanes reads 128 contiguous
// bytes of one weight row), dequantised in registers and fed to mma.sync.m16n8k16 as the B
// operand. The <= 16 activation rows are staged once per block in shared memory in the exact
// order the A fragments need, so a fragment is one conflict-free 128-bit shared load.
// Weights never pass through shared memory, which is why the register-operand MMA is used
// rather than a shared-memory-operand tensor-core path: with 16 rows the tensor pipe is
// nearly idle either way and the instruction budget goes to the int4 -> BF16 conversion.
//
// Work decomposition: persistent blocks of 16 warps. A "tile" is 8 output features; an item
// is kTiles tiles processed together (they share the A fragments). Within an item the K range
// is cut into units (256 inputs for int4, 64 for BF16) dealt round-robin to the 16 warps;
// warps write FP32 partial accumulators to shared memory and 128 * kTiles threads add them in
// warp order, so results do not depend on scheduling. Loads for the next kDepth items are
// kept in flight in registers while the current one is computed. An optional split of K over
// blocks writes FP32 partials to caller scratch for a separate fixed-order reduction.
//
// Rounding contract (reference operators/src/cuda/kernels/awq_gemv_gemm.cu:119-127, 318-329):
// int4 weights are dequantised as round_bf16((w - z) * scale) - here computed as an exact BF16
// subtraction followed by one correctly rounded BF16 multiply, which gives the same bits -
// products accumulate in FP32, the bias joins the FP32 sum and the result is rounded once.
#pragma once

#include "common.cuh"

namespace ei {

enum GemmEpilogue : int {
  kEpiStore = 0,     // out = round_bf16(sum + bias)
  kEpiPartial = 1,   // partial[slice][row][n] = sum (FP32, no bias)
  kEpiSiluPair = 2,  // item = (gate tile t, up tile t + T/2): out = round(round(silu(g)) * u)
  kEpiArgmax = 3     // kEpiStore + per-block running argmax of every row
};

struct GemmParams {
  const bf16* x;          // [M, K], row stride x_stride
  int x_stride;
  int M, K, N;
  const int32_t* qweight; // AWQ: [N, K/8]
  const bf16* scales;     //      [N, padded_groups]
  const int32_t* zeros;   //      [N, zero_stride]
  int padded_groups, zero_stride;
  const bf16* w;          // dense: row n at w + n * ldw (K contiguous)
  int ldw;
  const bf16* bias;       // [N] or null
  bf16* out;              // [M, out_stride]
  int out_stride;
  int epilogue;
  int ksplit;             // blocks along K (>= 1); > 1 requires kEpiPartial
  float* partial;         // [ksplit, M, N]
  float* best_value;      // kEpiArgmax: [grid, 16]
  int* best_index;        //             [grid, 16]
};

constexpr int kGemmWarps = 16;
constexpr int kGemmThreads = kGemmWarps * 32;

__device__ __forceinline__ float silu_value(float x) {
  // Same branches as the reference operator (operators/src/cuda/silu_cuda.cu:11-32).
  if ((__float_as_uint(x) & 0x7fffffffu) <= 0x01000000u) {
    const float zero = __uint_as_float(__float_as_uint(x) & 0x80000000u);
    return __fmaf_ieee_rn(x, 0.5f, zero);
  }
  if (x < -80.0f) {
    const double e = exp(static_cast<double>(x));
    const double a = static_cast<double>(x) * e / (1.0 + e);
    float r;
    asm("cvt.rn.f32.f64 %0, %1;" : "=f"(r) : "d"(a));
    return r;
  }
  return x / (1.0f + expf(-x));
}

__device__ __forceinline__ float silu_multiply_value(float gate, float up) {
  const float activated = round_bf16(silu_value(gate));
  const float zero = __uint_as_float((__float_as_uint(activated) ^ __float_as_uint(up)) & 0x80000000u);
  return round_bf16(__fmaf_ieee_rn(activated, up, zero));
}

// Shared-memory image of the activations: 16-byte cells of 8 consecutive inputs of one row.
// Cell (row r < 8, kb) lives at ((kb * 8 + (r ^ swizzle(kb))) * 16; rows 8..15 in a second
// array of the same shape. kShift picks the kb bits that differ between the four lanes of a
// quad so that a quarter-warp's 128-bit loads fall into eight distinct bank groups.
template <int kShift>
__device__ __forceinline__ int x_cell(int kb, int r) {
  return (kb * 8 + (r ^ (((kb >> kShift) & 3) << 1))) * 16;
}

template <bool kAwq>
__device__ __forceinline__ void stage_activations(const GemmParams& p, unsigned char* lo,
                                                  unsigned char* hi, bool has_hi, int k0, int kslice) {
  constexpr int kShift = kAwq ? 3 : 1;
  const int cells = kslice / 8;
  const int halves = has_hi ? 2 : 1;
  for (int idx = threadIdx.x; idx < cells * 8 * halves; idx += blockDim.x) {
    const int half = idx / (cells * 8);
    const int rem = idx - half * cells * 8;
    const int r = rem & 7, kb = rem >> 3;
    const int row = r + half * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < p.M) v = *reinterpret_cast<const uint4*>(p.x + size_t(row) * p.x_stride + k0 + kb * 8);
    if (kAwq) {
      // (k0k1, k2k3, k4k5, k6k7) -> (k0k4, k1k5, k2k6, k3k7): the pair order int4 extraction yields.
      uint4 t;
      t.x = __byte_perm(v.x, v.z, 0x5410);
      t.y = __byte_perm(v.x, v.z, 0x7632);
      t.z = __byte_perm(v.y, v.w, 0x5410);
      t.w = __byte_perm(v.y, v.w, 0x7632);
      v = t;
    }
    *reinterpret_cast<uint4*>((half ? hi : lo) + x_cell<kShift>(kb, r)) = v;
  }
}

// Registers of one prefetched item for one warp.
template <bool kAwq, int kTiles, int kUnits>
struct ItemRegs {
  uint4 w[kTiles][kUnits][2];
  uint32_t scale[kAwq ? kTiles : 1][kAwq ? kUnits : 1];  // BF16 scale replicated in both halves
  uint32_t zero[kAwq ? kTiles : 1][kAwq ? kUnits : 1];   // BF16 (128 + z) replicated in both halves
};

template <bool kAwq, bool kHigh, int kTiles, int kUnits, int kDepth>
__global__ void __launch_bounds__(kGemmThreads, 1) smallm_gemm_kernel(const GemmParams p) {
  constexpr int kUnitK = kAwq ? 256 : 64;
  constexpr int kShift = kAwq ? 3 : 1;
  extern __shared__ __align__(16) unsigned char smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
  const int slice = blockIdx.x % p.ksplit;
  const int group = blockIdx.x / p.ksplit;
  const int groups = gridDim.x / p.ksplit;
  const int kslice = p.K / p.ksplit;
  const int k0 = slice * kslice;
  const int units = kslice / kUnitK;
  const int tiles = p.N / 8;
  const bool pair = p.epilogue == kEpiSiluPair;
  const int items = pair ? tiles / 2 : (tiles + kTiles - 1) / kTiles;
  const int item_begin = int((long long)group * items / groups);
  const int item_end = int((long long)(group + 1) * items / groups);

  unsigned char* x_lo = smem;
  unsigned char* x_hi = smem + size_t(kslice) * 16;  // (kslice / 8) cells * 8 rows * 16 B
  float* part = reinterpret_cast<float*>(smem + size_t(kslice) * 16 * (kHigh ? 2 : 1));
  // part[2][kGemmWarps][kTiles][32][4]

  auto tile_of = [&](int item, int t) -> int {
    if (pair) return t == 0 ? item : item + tiles / 2;
    const int tile = item * kTiles + t;
    return tile < tiles ? tile : -1;
  };

  ItemRegs<kAwq, kTiles, kUnits> regs[kDepth];

  auto prefetch = [&](ItemRegs<kAwq, kTiles, kUnits>& r, int item) {
#pragma unroll
    for (int t = 0; t < kTiles; ++t) {
      const int tile = item < item_end ? tile_of(item, t) : -1;
#pragma unroll
      for (int j = 0; j < kUnits; ++j) {
        const int u = warp + kGemmWarps * j;
        if (tile >= 0 && u < units) {
          const size_t n = size_t(tile) * 8 + g;
          const int k = k0 + u * kUnitK + c * (kUnitK / 4);
          if (kAwq) {
            const int32_t* src = p.qweight + n * size_t(p.K / 8) + k / 8;
            r.w[t][j][0] = ldg_stream(src);
            r.w[t][j][1] = ldg_stream(src + 4);
            const int grp = k >> 7;
            const uint32_t s = __ldg(reinterpret_cast<const unsigned short*>(p.scales) + n * p.padded_groups + grp);
            const uint32_t zw = uint32_t(__ldg(p.zeros + n * p.zero_stride + (grp >> 3)));
            r.scale[t][j] = s * 0x10001u;
            r.zero[t][j] = (0x4300u | ((zw >> ((grp & 7) * 4)) & 15u)) * 0x10001u;
          } else {
            const bf16* src = p.w + n * size_t(p.ldw) + k;
            r.w[t][j][0] = ldg_stream(src);
            r.w[t][j][1] = ldg_stream(src + 8);
          }
        } else {
          r.w[t][j][0] = make_uint4(0, 0, 0, 0);
          r.w[t][j][1] = make_uint4(0, 0, 0, 0);
          if (kAwq) {
            r.scale[t][j] = 0;
            r.zero[t][j] = 0x43004300u;
          }
        }
      }
    }
  };

  // Weights do not depend on the preceding kernel: get them moving before waiting for it.
#pragma unroll
  for (int s = 0; s < kDepth; ++s) prefetch(regs[s], item_begin + s);
  grid_dependency_wait();
  stage_activations<kAwq>(p, x_lo, x_hi, kHigh, k0, kslice);
  __syncthreads();
  grid_launch_dependents();

  float best_value = -INFINITY;
  int best_index = 0x7fffffff;

  for (int base = item_begin; base < item_end; base += kDepth) {
#pragma unroll
    for (int s = 0; s < kDepth; ++s) {
      const int item = base + s;
      if (item >= item_end) break;
      float acc[kTiles][4];
#pragma unroll
      for (int t = 0; t < kTiles; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f;
#pragma unroll
      for (int j = 0; j < kUnits; ++j) {
        const int u = warp + kGemmWarps * j;
        if (u < units) {
          const int kb_base = (u * kUnitK + c * (kUnitK / 4)) >> 3;
#pragma unroll
          for (int v = 0; v < 2; ++v) {
#pragma unroll
            for (int q = 0; q < (kAwq ? 4 : 1); ++q) {
              const int kb = kb_base + (kAwq ? v * 4 + q : v);
              const int cell = x_cell<kShift>(kb, g);
              const uint4 xa = *reinterpret_cast<const uint4*>(x_lo + cell);
              uint4 xb = make_uint4(0, 0, 0, 0);
              if (kHigh) xb = *reinterpret_cast<const uint4*>(x_hi + cell);
#pragma unroll
              for (int t = 0; t < kTiles; ++t) {
                uint32_t b0, b1, b2, b3;
                if (kAwq) {
                  const uint4 wv = regs[s].w[t][j][v];
                  const uint32_t word = q == 0 ? wv.x : q == 1 ? wv.y : q == 2 ? wv.z : wv.w;
                  const __nv_bfloat162 zero = *reinterpret_cast<const __nv_bfloat162*>(&regs[s].zero[t][j]);
                  const __nv_bfloat162 scale = *reinterpret_cast<const __nv_bfloat162*>(&regs[s].scale[t][j]);
                  uint32_t e0 = (word & 0x000f000fu) | 0x43004300u;
                  uint32_t e1 = ((word >> 4) & 0x000f000fu) | 0x43004300u;
                  uint32_t e2 = ((word >> 8) & 0x000f000fu) | 0x43004300u;
                  uint32_t e3 = ((word >> 12) & 0x000f000fu) | 0x43004300u;
                  __nv_bfloat162 d0 = __hmul2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&e0), zero), scale);
                  __nv_bfloat162 d1 = __hmul2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&e1), zero), scale);
                  __nv_bfloat162 d2 = __hmul2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&e2), zero), scale);
                  __nv_bfloat162 d3 = __hmul2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&e3), zero), scale);
                  b0 = *reinterpret_cast<uint32_t*>(&d0);
                  b1 = *reinterpret_cast<uint32_t*>(&d1);
                  b2 = *reinterpret_cast<uint32_t*>(&d2);
                  b3 = *reinterpret_cast<uint32_t*>(&d3);
                } else {
                  const uint4 wv = regs[s].w[t][j][v];
                  b0 = wv.x; b1 = wv.y; b2 = wv.z; b3 = wv.w;
                }
                mma_bf16_16816(acc[t], xa.x, xb.x, xa.y, xb.y, b0, b1);
                mma_bf16_16816(acc[t], xa.z, xb.z, xa.w, xb.w, b2, b3);
              }
            }
          }
        }
      }
      // This register set is free again: refill it with the item kDepth ahead.
      prefetch(regs[s], item + kDepth);

      float* mine = part + ((size_t(item & 1) * kGemmWarps + warp) * kTiles) * 128;
#pragma unroll
      for (int t = 0; t < kTiles; ++t)
        *reinterpret_cast<float4*>(mine + t * 128 + lane * 4) = make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
      __syncthreads();

      const int reducers = (pair ? 1 : kTiles) * 128;
      if (int(threadIdx.x) < reducers) {
        const int t = threadIdx.x >> 7;
        const int e = threadIdx.x & 127;
        const int rl = e >> 2, reg = e & 3;
        const int row = (rl >> 2) + (reg >= 2 ? 8 : 0);
        const int col = (rl & 3) * 2 + (reg & 1);
        const float* src = part + size_t(item & 1) * kGemmWarps * kTiles * 128 + e;
        if (pair) {
          float gate = 0.0f, up = 0.0f;
#pragma unroll
          for (int w = 0; w < kGemmWarps; ++w) {
            gate += src[(w * kTiles + 0) * 128];
            up += src[(w * kTiles + 1) * 128];
          }
          if (row < p.M) {
            const int n = item * 8 + col;
            if (p.bias) {
              gate += __bfloat162float(p.bias[n]);
              up += __bfloat162float(p.bias[n + p.N / 2]);
            }
            p.out[size_t(row) * p.out_stride + n] =
                __float2bfloat16_rn(silu_multiply_value(round_bf16(gate), round_bf16(up)));
          }
        } else {
          const int tile = tile_of(item, t);
          float sum = 0.0f;
#pragma unroll
          for (int w = 0; w < kGemmWarps; ++w) sum += src[(w * kTiles + t) * 128];
          if (tile >= 0 && row < p.M && (kHigh || reg < 2)) {
            const int n = tile * 8 + col;
            if (p.epilogue == kEpiPartial) {
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
      }
    }
  }

  if (p.epilogue == kEpiArgmax) {
    // Reducer thread (t, e) always owns the same output row; fold the kTiles * 8 owners of a row.
    __syncthreads();
    float* values = part;
    int* indices = reinterpret_cast<int*>(part + kTiles * 128);
    if (int(threadIdx.x) < kTiles * 128) {
      values[threadIdx.x] = best_value;
      indices[threadIdx.x] = best_index;
    }
    __syncthreads();
    if (threadIdx.x < 16) {
      const int row = threadIdx.x;
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int t = 0; t < kTiles; ++t)
        for (int e = 0; e < 128; ++e) {
          const int rl = e >> 2, reg = e & 3;
          if ((rl >> 2) + (reg >= 2 ? 8 : 0) != row) continue;
          const float value = values[t * 128 + e];
          const int index = indices[t * 128 + e];
          if (value > bv || (value == bv && index < bi)) {
            bv = value;
            bi = index;
          }
        }
      p.best_value[blockIdx.x * 16 + row] = bv;
      p.best_index[blockIdx.x * 16 + row] = bi;
    }
  }
}

// Fixed-order reduction of split-K partials for a plain linear: out = round_bf16(sum_s partial + bias).
__global__ void splitk_store_kernel(const float* partial, int ksplit, int M, int N, const bf16* bias,
                                    bf16* out, int out_stride);

// Any-shape fallbacks (one thread per output, sequential FP32 fma in input order like the
// reference's scalar kernel, operators/src/cuda/kernels/awq_gemv_gemm.cu:579-604).
__global__ void awq_generic_kernel(const bf16* x, int x_stride, const int32_t* qweight, const bf16* scales,
                                   const int32_t* zeros, const bf16* bias, bf16* out, int out_stride,
                                   int rows, int N, int K, int group_size, int padded_groups);
__global__ void dense_generic_kernel(const bf16* x, int x_stride, const bf16* w, long long stride_k,
                                     long long stride_n, const bf16* bias, bf16* out, int out_stride,
                                     int rows, int N, int K);

struct GemmPlan {
  bool fast = false;
  bool high = false;
  int tiles_per_item = 1, units_per_warp = 1, depth = 2;
  int ksplit = 1, grid = 1;
  size_t smem = 0;
};

// Chooses the kernel instance, the K split and the grid for a shape. `allow_split` permits
// ksplit > 1 (the caller provides FP32 scratch of ksplit * M * N floats).
GemmPlan plan_gemm(bool awq, int M, int N, int K, int epilogue, int multiprocessors,
                   size_t smem_limit, bool allow_split);
void launch_gemm(const GemmPlan& plan, bool awq, const GemmParams& params, cudaStream_t stream, bool pdl);

}  // namespace ei
