// W8A8 K-group-scaled GEMM for a handful of rows (M <= 8): weight streaming on CUDA cores.
//
// With so few rows the operation is a read of the weights once from HBM; the tensor cores and
// their set-up (tensor maps, TMEM, 200 KB of staging per CTA) buy nothing and cost several
// microseconds per launch.  Here a warp owns a few output columns (weight rows of B[N, K]) and
// walks each of them with whole-warp loads: 32 lanes x 16 bytes = 512 contiguous bytes per
// instruction, eight instructions in flight.  Every lane multiplies its 16 weights with the
// activation rows by `dp4a`; the lanes that share a K group (group_size / 16 of them) add up
// their exact INT32 sums by shuffles and one of them leaves the group's dot in shared memory.
// When the CTA's columns are done one thread per (row, column) folds the groups in order,
// total = fmaf(float(dot_g), sa[m, g] * sb[g, n], total), which is the arithmetic of the
// tensor-core kernels and of the reference (src/grain_gemm/kernels/triton.py:28-51), bit for
// bit.  The host picks the columns per warp so that all CTAs of the launch are resident at once.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace gg {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kGemvMaxColumnsPerWarp = 8;
constexpr int kGemvMaxRows = 8;

struct GemvParams {
  const int8_t* a;          // [M, K], K contiguous, rows 16-byte aligned
  const int8_t* b;          // [N, K], K contiguous, rows 16-byte aligned
  const float* scale_a;     // [M, Q]
  const float* scale_b;     // [Q, N]
  void* c;                  // [M, N]
  int m, n, k, group_size, out_dtype;
  long long a_sm, b_sn, sa_sm, sa_sg, sb_sg, sb_sn, ldc;
  int columns_per_warp;     // 1 .. kGemvMaxColumnsPerWarp; a CTA owns 8 times as many columns
};

__device__ __forceinline__ uint4 ldg_stream_16(const void* address) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(address));
  return v;
}

__device__ __forceinline__ int dot16(const uint4& w, const uint4& x) {
  int sum = __dp4a(static_cast<int>(w.x), static_cast<int>(x.x), 0);
  sum = __dp4a(static_cast<int>(w.y), static_cast<int>(x.y), sum);
  sum = __dp4a(static_cast<int>(w.z), static_cast<int>(x.z), sum);
  sum = __dp4a(static_cast<int>(w.w), static_cast<int>(x.w), sum);
  return sum;
}

// One whole-warp step: 16 weights per lane against every activation row, the lanes of a K group
// add up and the group's first lane stores the dot.
template <int kRows, int kLanesPerGroup>
__device__ __forceinline__ void gemv_step(const GemvParams& p, const uint4& w, int chunk, int chunks,
                                          int lane, int* dots, int groups) {
  const bool valid = chunk < chunks;
  const long long offset = static_cast<long long>(valid ? chunk : 0) << 4;
  int sum[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    // Rows at or beyond M repeat the last row (their results are never stored).
    const int row = r < p.m ? r : p.m - 1;
    const uint4 x = __ldg(reinterpret_cast<const uint4*>(p.a + static_cast<long long>(row) * p.a_sm + offset));
    sum[r] = valid ? dot16(w, x) : 0;
  }
#pragma unroll
  for (int delta = kLanesPerGroup >> 1; delta > 0; delta >>= 1) {
#pragma unroll
    for (int r = 0; r < kRows; ++r) sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], delta);
  }
  if (valid && (lane & (kLanesPerGroup - 1)) == 0) {
    const int group = chunk / kLanesPerGroup;
#pragma unroll
    for (int r = 0; r < kRows; ++r) dots[r * groups + group] = sum[r];
  }
}

template <int kRows, int kLanesPerGroup>
__global__ void __launch_bounds__(kGemvThreads, kRows <= 2 ? 4 : 2) gemm_gemv_kernel(const GemvParams p) {
  extern __shared__ int gemv_dots[];             // [C][kRows][Q], C = columns of this CTA
  const int groups = (p.k + p.group_size - 1) / p.group_size;
  const int columns = kGemvWarps * p.columns_per_warp;
  const int first_column = blockIdx.x * columns;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunks = p.k >> 4;                              // 16-byte chunks of K
  const int blocks_per_column = (chunks + 255) >> 8;        // blocks of eight whole-warp loads
  const int warp_first = first_column + warp * p.columns_per_warp;
  const int warp_columns = max(0, min(p.columns_per_warp, p.n - warp_first));
  const int blocks = warp_columns * blocks_per_column;

  // The first eight loads of weights are requested before anything else.
  const int8_t* weights = p.b + static_cast<long long>(warp_first) * p.b_sn;
  uint4 w[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int chunk = j * 32 + lane;
    w[j] = blocks > 0 && chunk < chunks ? ldg_stream_16(weights + (static_cast<long long>(chunk) << 4))
                                        : make_uint4(0u, 0u, 0u, 0u);
  }

  // The scales of this CTA's columns and rows wait in shared memory, so that the ordered fold
  // at the end does not pay a memory latency per group.
  float* column_scales = reinterpret_cast<float*>(gemv_dots + columns * kRows * groups);   // [Q][C]
  float* row_scales = column_scales + groups * columns;                                    // [kRows][Q]
  for (int i = threadIdx.x; i < groups * columns; i += kGemvThreads) {
    const int g = i / columns;
    const int col = first_column + (i - g * columns);
    column_scales[i] = col < p.n ? p.scale_b[static_cast<long long>(g) * p.sb_sg +
                                              static_cast<long long>(col) * p.sb_sn]
                                 : 0.0f;
  }
  for (int i = threadIdx.x; i < groups * kRows; i += kGemvThreads) {
    const int r = i / groups, g = i - r * groups;
    row_scales[i] = r < p.m ? p.scale_a[static_cast<long long>(r) * p.sa_sm + g * p.sa_sg] : 0.0f;
  }

  int column = 0, block_in_column = 0;
  for (int block = 0; block < blocks; ++block) {
    int* dots = gemv_dots + (warp * p.columns_per_warp + column) * kRows * groups;
    const int base = block_in_column * 256 + lane;
    // Where the next block's weights are (the same column or the next one).
    if (++block_in_column == blocks_per_column) {
      block_in_column = 0;
      ++column;
    }
    const bool more = block + 1 < blocks;
    const int8_t* next = p.b + static_cast<long long>(warp_first + (more ? column : 0)) * p.b_sn;
    const int next_base = block_in_column * 256 + lane;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      // Whole-warp condition: the shuffles inside always see 32 lanes.
      if (base - lane + j * 32 < chunks) {
        gemv_step<kRows, kLanesPerGroup>(p, w[j], base + j * 32, chunks, lane, dots, groups);
      }
      // The register is free again: its next load goes out at once, so that eight loads stay
      // in flight per lane throughout.
      const int chunk = next_base + j * 32;
      w[j] = more && chunk < chunks ? ldg_stream_16(next + (static_cast<long long>(chunk) << 4))
                                    : make_uint4(0u, 0u, 0u, 0u);
    }
  }
  __syncthreads();

  // Ordered fold: one thread per (row, column).
  for (int item = threadIdx.x; item < kRows * columns; item += kGemvThreads) {
    const int r = item / columns;
    const int c = item - r * columns;
    const int col = first_column + c;
    if (r < p.m && col < p.n) {
      float total = 0.0f;
      for (int g = 0; g < groups; ++g) {
        const float scale = __fmul_rn(row_scales[r * groups + g], column_scales[g * columns + c]);
        total = __fmaf_rn(__int2float_rn(gemv_dots[(c * kRows + r) * groups + g]), scale, total);
      }
      const long long index = static_cast<long long>(r) * p.ldc + col;
      if (p.out_dtype == 0) static_cast<float*>(p.c)[index] = total;
      else if (p.out_dtype == 1) static_cast<__nv_bfloat16*>(p.c)[index] = __float2bfloat16_rn(total);
      else static_cast<__half*>(p.c)[index] = __float2half_rn(total);
    }
  }
}

}  // namespace gg
