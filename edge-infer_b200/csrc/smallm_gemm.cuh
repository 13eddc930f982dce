// Small-M (<= 16 rows) weight-streaming GEMMs for sm_100a: out[M,N] = x[M,K] * W[N,K]^T (+ bias).
//
// This header holds what the two kernels share (parameters, plan, epilogues, the exact int4 dequantisation,
// the activation fragments) and the kernel for dense BF16 weights; the int4 kernel is in awq_tma.cuh.
//
// Dense BF16 kernel (the vocabulary head and every projection of unquantised models). The path is HBM-bound:
//  * every weight byte is read exactly once, straight from global memory into registers with 128-bit loads
//    that bypass L1 (each quad of lanes reads 128 contiguous bytes of one weight row); the loads of the next
//    kDepth items are kept in flight in registers while the current item is computed, and nothing is computed
//    from a loaded word before its item is consumed (a dependent instruction would stall the in-order issue of
//    the loads behind it);
//  * the <= 16 activation rows are staged once per block in swizzled shared memory and read as A fragments;
//    the weights are the B operand of mma.sync.m16n8k16 with FP32 accumulation.
//
// Work decomposition: persistent blocks of 16 warps. An item is one tile of 8 output features; K is dealt to
// the warps in units of 64 inputs. Per item the warps write their FP32 partial accumulators to shared memory
// and all 512 threads add them in a fixed order (4 partials per thread, parts combined by shuffles), so
// results do not depend on scheduling. Input features beyond 64 units per block are split over blocks
// (ksplit) that write FP32 partials to caller scratch for a separate fixed-order reduction.
//
// Rounding contract (reference operators/src/cuda/kernels/awq_gemv_gemm.cu:119-127, 318-329,
// operators/src/cuda/execution.cu:299-324): int4 weights are dequantised as round_bf16((w - z) * scale) -
// computed as an exact BF16 subtraction followed by one correctly rounded BF16 multiply, which gives the same
// bits - products accumulate in FP32, the bias joins the FP32 sum and the result is rounded once.
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
  int* status;            // optional device word; bit 2 is set if a bounded wait on a bulk copy gave up
  uint32_t wait_limit;    // polls before a bounded wait gives up (0: the kernel's default)
  int prompt_tiles;       // prompt GEMM only: token tiles of 128 rows per block (0: chosen by the launch function)
  uint32_t fault_tx;      // test hook: bytes the first weight copy is expected to deliver beyond what it does,
                          // so that the bounded waits run out (0 in production)
};

constexpr int kGemmWarps = 16;
constexpr int kGemmThreads = kGemmWarps * 32;

__device__ __forceinline__ float silu_value(float x) {
  // Same branches as the reference operator (operators/src/cuda/silu_cuda.cu:11-32), whose build uses
  // fast-math for the exponential and the division of the main branch.
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
  return __fdividef(x, 1.0f + __expf(-x));
}

__device__ __forceinline__ float silu_multiply_value(float gate, float up) {
  const float activated = round_bf16(silu_value(gate));
  const float zero = __uint_as_float((__float_as_uint(activated) ^ __float_as_uint(up)) & 0x80000000u);
  return round_bf16(__fmaf_ieee_rn(activated, up, zero));
}

// Two int4 weights (bits 0-3 of each 16-bit half of `shifted`) -> two BF16 values round_bf16((w - z) * scale):
// one LOP3 plants each nibble in the mantissa of 128.0 (0x4300 | w = 128 + w exactly), one packed subtract of
// (128 + z) is exact, one packed multiply rounds once - the value the reference computes in FP32 and rounds.
__device__ __forceinline__ uint32_t dequant_pair(uint32_t shifted, uint32_t zero2, uint32_t scale2) {
  uint32_t planted, difference, product;
  asm("lop3.b32 %0, %1, 0x000f000f, 0x43004300, 0xea;" : "=r"(planted) : "r"(shifted));
  asm("sub.bf16x2 %0, %1, %2;" : "=r"(difference) : "r"(planted), "r"(zero2));
  asm("mul.bf16x2 %0, %1, %2;" : "=r"(product) : "r"(difference), "r"(scale2));
  return product;
}

// With BF16 weights a warp covers up to four 64-input units, too many fragments to pin in registers: the
// activations sit in shared memory as 16-byte cells of 8 consecutive inputs of one row. Cell (row r < 8, kb) lives at (kb * 8 + (r ^ swizzle(kb))) * 16, rows 8..15 in a second
// array of the same shape; the swizzle uses the kb bits that differ between the four lanes of a quad so that
// a quarter-warp's 128-bit loads fall into eight distinct bank groups.
__device__ __forceinline__ int x_cell(int kb, int r) { return (kb * 8 + (r ^ (((kb >> 1) & 3) << 1))) * 16; }

__device__ __forceinline__ void stage_activations(const GemmParams& p, unsigned char* lo, unsigned char* hi,
                                                  bool has_hi, int k_begin, int k_count) {
  const int cells = k_count / 8;
  const int halves = has_hi ? 2 : 1;
  for (int idx = threadIdx.x; idx < cells * 8 * halves; idx += blockDim.x) {
    const int half = idx / (cells * 8);
    const int rem = idx - half * cells * 8;
    const int r = rem & 7, kb = rem >> 3;  // eight lanes write the eight rows of one kb: distinct bank groups
    const int row = r + half * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < p.M) v = *reinterpret_cast<const uint4*>(p.x + size_t(row) * p.x_stride + k_begin + kb * 8);
    *reinterpret_cast<uint4*>((half ? hi : lo) + x_cell(kb, r)) = v;
  }
}

// Registers of one prefetched item (one tile) for one warp. Raw loaded words only.
template <int kUnits>
struct ItemRegs {
  uint4 w[kUnits][2];
};

// A fragments of one 8-input cell of the int4 kernel: two MMAs' worth of (a0, a1, a2, a3). The 8 inputs are
// taken in the order (0,4 | 1,5) and (2,6 | 3,7): the pair order the nibble extraction yields.
template <bool kHigh>
struct CellFragments {
  uint32_t a[2][kHigh ? 4 : 2];
};

// Loads the fragments of one cell for lane (g, c): 8 consecutive inputs of rows g and g + 8 starting at k.
template <bool kHigh>
__device__ __forceinline__ void load_cell(CellFragments<kHigh>& f, const bf16* x, int x_stride, int M, int g, int k) {
  uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
  if (g < M) lo = *reinterpret_cast<const uint4*>(x + size_t(g) * x_stride + k);
  if (kHigh && g + 8 < M) hi = *reinterpret_cast<const uint4*>(x + size_t(g + 8) * x_stride + k);
  // (k0k1, k2k3, k4k5, k6k7) -> (k0k4, k1k5, k2k6, k3k7)
  uint4 t;
  t.x = __byte_perm(lo.x, lo.z, 0x5410); t.y = __byte_perm(lo.x, lo.z, 0x7632);
  t.z = __byte_perm(lo.y, lo.w, 0x5410); t.w = __byte_perm(lo.y, lo.w, 0x7632);
  lo = t;
  if (kHigh) {
    t.x = __byte_perm(hi.x, hi.z, 0x5410); t.y = __byte_perm(hi.x, hi.z, 0x7632);
    t.z = __byte_perm(hi.y, hi.w, 0x5410); t.w = __byte_perm(hi.y, hi.w, 0x7632);
    hi = t;
    f.a[0][0] = lo.x; f.a[0][1] = hi.x; f.a[0][2] = lo.y; f.a[0][3] = hi.y;
    f.a[1][0] = lo.z; f.a[1][1] = hi.z; f.a[1][2] = lo.w; f.a[1][3] = hi.w;
  } else {
    f.a[0][0] = lo.x; f.a[0][1] = lo.y;
    f.a[1][0] = lo.z; f.a[1][1] = lo.w;
  }
}

template <bool kHigh, bool kFirst = false>
__device__ __forceinline__ void mma_cell(float (&acc)[4], const CellFragments<kHigh>& f, int which, uint32_t b0,
                                         uint32_t b1) {
  if (kFirst) {
    if (kHigh)
      mma_bf16_16816_first(acc, f.a[which][0], f.a[which][1], f.a[which][2], f.a[which][3], b0, b1);
    else
      mma_bf16_16816_first(acc, f.a[which][0], 0u, f.a[which][1], 0u, b0, b1);
  } else {
    if (kHigh)
      mma_bf16_16816(acc, f.a[which][0], f.a[which][1], f.a[which][2], f.a[which][3], b0, b1);
    else
      mma_bf16_16816(acc, f.a[which][0], 0u, f.a[which][1], 0u, b0, b1);
  }
}

template <bool kHigh, int kUnits, int kDepth>
__global__ void __launch_bounds__(kGemmThreads, 1) smallm_gemm_kernel(const GemmParams p) {
  constexpr int kUnitK = 64;
  constexpr int kParts = 4;             // reduction parts per output: a warp's lanes are 4 parts x 8 elements
  constexpr int kBlock = 136;           // floats per warp in the partial buffer: 128 + 8 keeps loads conflict-free
  extern __shared__ __align__(16) unsigned char smem[];
  float* part = reinterpret_cast<float*>(smem);  // [2][kGemmWarps][kBlock]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
  const int slice = blockIdx.x % p.ksplit;
  const int group = blockIdx.x / p.ksplit;
  const int groups = gridDim.x / p.ksplit;
  const int units_total = p.K / kUnitK;
  const int unit_begin = int((long long)slice * units_total / p.ksplit);
  const int units = int((long long)(slice + 1) * units_total / p.ksplit) - unit_begin;
  const int tiles = p.N / 8;
  // An item is one tile. The fused SwiGLU epilogue walks (gate tile i, up tile i) as two consecutive items.
  const bool pair = p.epilogue == kEpiSiluPair;
  const int chunks = pair ? tiles / 2 : tiles;
  const int per_chunk = pair ? 2 : 1;
  const int item_begin = int((long long)group * chunks / groups) * per_chunk;
  const int item_end = int((long long)(group + 1) * chunks / groups) * per_chunk;
  auto tile_of = [&](int item) -> int { return pair ? (item >> 1) + (item & 1) * (tiles / 2) : item; };

  // Per-lane bases of everything the lane ever loads for unit j; a tile only adds a row offset.
  const unsigned char* w_base[kUnits];
  bool live[kUnits];
#pragma unroll
  for (int j = 0; j < kUnits; ++j) {
    const int u = warp + kGemmWarps * j;
    live[j] = u < units;
    const int k = (unit_begin + (live[j] ? u : 0)) * kUnitK + c * (kUnitK / 4);
    w_base[j] = reinterpret_cast<const unsigned char*>(p.w + size_t(g) * p.ldw + k);
  }
  const size_t w_tile_stride = size_t(8) * p.ldw * 2;  // bytes per tile

  ItemRegs<kUnits> regs[kDepth];
  auto prefetch = [&](ItemRegs<kUnits>& r, int item) {
    const bool valid = item < item_end;
    const int tile = valid ? tile_of(item) : 0;
#pragma unroll
    for (int j = 0; j < kUnits; ++j) {
      if (valid && live[j]) {
        const unsigned char* src = w_base[j] + size_t(tile) * w_tile_stride;
        r.w[j][0] = ldg_stream(src);
        r.w[j][1] = ldg_stream(src + 16);
      } else {
        r.w[j][0] = make_uint4(0, 0, 0, 0);
        r.w[j][1] = make_uint4(0, 0, 0, 0);
      }
    }
  };

  // Weights do not depend on the preceding kernel: get them moving before waiting for it.
#pragma unroll
  for (int s = 0; s < kDepth; ++s) prefetch(regs[s], item_begin + s);
  grid_dependency_wait();

  // Activations staged in shared memory behind the partials.
  unsigned char* x_lo = smem + size_t(2) * kGemmWarps * kBlock * sizeof(float);
  unsigned char* x_hi = x_lo + size_t(units) * kUnitK * 16;
  stage_activations(p, x_lo, x_hi, kHigh, unit_begin * kUnitK, units * kUnitK);
  __syncthreads();
  grid_launch_dependents();

  // Reduction role of this lane: warp r owns accumulator elements e in [8r, 8r + 8); a lane is (part, element).
  const int e = warp * 8 + (lane & 7);
  const int part_index = lane >> 3;
  const int rl = e >> 2, reg = e & 3;
  const int row = (rl >> 2) + (reg >= 2 ? 8 : 0);
  const int col = (rl & 3) * 2 + (reg & 1);
  float best_value = -INFINITY;
  int best_index = 0x7fffffff;
  float gate_sum = 0.0f;  // fused SwiGLU: the gate tile's sum waits here for the up tile

  const bool high_row = g + 8 < p.M;  // this lane's second fragment row exists (9 rows: only one lane group)
  for (int base = item_begin; base < item_end; base += kDepth) {
#pragma unroll
    for (int s = 0; s < kDepth; ++s) {
      const int item = base + s;
      if (item >= item_end) break;
      float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int j = 0; j < kUnits; ++j) {
#pragma unroll
        for (int v = 0; v < 2; ++v) {
          const uint4 wv = regs[s].w[j][v];
          if (live[j]) {
            // Cell of (unit, lane, v); both cells of a lane share the swizzle term.
            const int u = warp + kGemmWarps * j;
            const int cell = x_cell((u * kUnitK + c * (kUnitK / 4)) >> 3, g) + v * 128;
            const uint4 xa = *reinterpret_cast<const uint4*>(x_lo + cell);
            uint4 xb = make_uint4(0, 0, 0, 0);
            if (kHigh && high_row) xb = *reinterpret_cast<const uint4*>(x_hi + cell);  // rows >= M are zero
            mma_bf16_16816(acc, xa.x, xb.x, xa.y, xb.y, wv.x, wv.y);
            mma_bf16_16816(acc, xa.z, xb.z, xa.w, xb.w, wv.z, wv.w);
          }
        }
      }
      // This register set is free again: refill it with the item kDepth ahead.
      prefetch(regs[s], item + kDepth);

      // part[buffer][warp][e] with e = lane * 4 + reg (conflict-free 128-bit stores).
      float* mine = part + (size_t(item & 1) * kGemmWarps + warp) * kBlock;
      *reinterpret_cast<float4*>(mine + lane * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      __syncthreads();

      // Fixed-order reduction by all 16 warps: part p adds the partials of warps p, p + 4, p + 8, p + 12 in
      // that order and the parts are combined by two shuffles, so an output sees the same additions in every
      // run. The 136-float stride puts the 32 lanes of each load in 32 different banks.
      float sum = 0.0f;
      {
        const float* src = part + (size_t(item & 1) * kGemmWarps + part_index) * kBlock + e;
#pragma unroll
        for (int w = 0; w < kGemmWarps / kParts; ++w) sum += src[size_t(w) * kParts * kBlock];
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 16);
      sum += __shfl_xor_sync(0xffffffffu, sum, 8);
      if (part_index == 0 && row < p.M) {
        const int tile = tile_of(item);
        const int n = tile * 8 + col;
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
  int units_per_warp = 1;
  int tiles_per_block = 0;  // int4 path: tiles (items) the busiest block walks
  size_t smem_limit = 0;    // int4 path: dynamic shared memory a block may opt in to
  int ksplit = 1, grid = 1;
  size_t smem = 0;
};

// Chooses the kernel instance, the K split and the grid for a shape. `allow_split` permits
// ksplit > 1 (the caller provides FP32 scratch of ksplit * M * N floats).
GemmPlan plan_gemm(bool awq, int M, int N, int K, int epilogue, int multiprocessors,
                   size_t smem_limit, bool allow_split);
void launch_gemm(const GemmPlan& plan, bool awq, const GemmParams& params, cudaStream_t stream, bool pdl);

// ---- prompt GEMM (prompt_gemm.cuh): many rows at once on tcgen05 ----
constexpr int kPromptMinRows = 32;  // more rows than this take the prompt kernel where the shape allows
// True if the prompt kernel takes this shape (features in steps of 16, inputs in steps of a K block - of a
// quantisation group for int4 - and 16-byte aligned rows).
bool prompt_gemm_eligible(bool awq, int group_size, int N, int K, const void* x, int x_stride, const void* out,
                          int out_stride);
// epilogue kEpiStore: out[T, N] = x[T, K] * W^T (+ bias), rounded once to BF16. kEpiPartial: FP32 partial sums
// partial[ksplit][T][N] without bias, K split over ksplit blocks (whole groups of 128 inputs each).
// Uses p.x, x_stride, M (= T), K, N, the weight fields of its kind, bias, out, out_stride, epilogue, ksplit,
// partial, status, wait_limit, fault_tx.
int prompt_gemm_ksplit(int rows, int N, int K, int multiprocessors, size_t partial_bytes);
// Token tiles per block (1 or 2) that fill the grid's waves best for this shape.
int prompt_gemm_tiles(int rows, int N, int multiprocessors);
void launch_prompt_gemm(bool awq, const GemmParams& p, cudaStream_t stream, bool pdl);


}  // namespace ei
