// CUDA-core grouped W8A8 GEMM for operands the TMA path cannot take: arbitrary positive
// strides, unaligned bases, K that is not a multiple of 16, row-major B.  Same arithmetic
// as the tensor-core kernel (exact INT32 group dot, FP32 scale product rounded once, one
// fmaf per group in group order, one cast), following
// src/grain_gemm/kernels/triton.py:28-51 of the reference.  Also serves the MoE path as
// the ragged, optionally row-gathered GEMM of src/grain_gemm/kernels/moe.py:359-393 when
// the tensor-core MoE kernels are not applicable.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"

namespace gg {

struct GemmSimtParams {
  const int8_t* a;
  const int8_t* b;
  const float* scale_a;
  const float* scale_b;
  void* c;
  int m, n, k;
  long long a_sm, a_sk, b_sk, b_sn;
  long long sa_sm, sa_sg, sb_sg, sb_sn;
  long long ldc;
  int group_size;
  int* partials;  // optional [M, N, Q] INT32 dump of the group dots
  // Ragged mode (all null / zero for a plain GEMM).
  const long long* order;     // [S] sorted slot -> flattened assignment, gather when non-null
  int top_k;                  // assignment / top_k = source row
  const int* expert_offsets;  // [E+1]
  const int* tile_expert;     // [tiles_m]
  const int* tile_row;        // [tiles_m]
  long long b_expert_stride;  // elements between experts in b
  long long sb_expert_stride; // elements between experts in scale_b
};

template <typename OutT>
__device__ __forceinline__ OutT cast_out(float v);
template <>
__device__ __forceinline__ float cast_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half cast_out<__half>(float v) { return __float2half_rn(v); }

constexpr int kSimtTile = 32;
constexpr int kSimtMaxGroup = 256;
constexpr int kSimtPitch = kSimtMaxGroup + 4;  // odd number of 32-bit words per row

template <typename OutT, bool kRagged>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const GemmSimtParams p) {
  __shared__ __align__(16) int8_t a_tile[kSimtTile][kSimtPitch];
  __shared__ __align__(16) int8_t b_tile[kSimtTile][kSimtPitch];
  __shared__ long long a_row_offset[kSimtTile];
  __shared__ long long sa_row_offset[kSimtTile];
  __shared__ int a_row_valid[kSimtTile];

  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  // One-dimensional grid (row tiles can exceed the 65535 limit of grid.y): column tile fastest.
  const int tiles_n = (p.n + kSimtTile - 1) / kSimtTile;
  const int tile_m = blockIdx.x / tiles_n;
  const int n0 = (blockIdx.x - tile_m * tiles_n) * kSimtTile;
  int row0, row_limit;
  const int8_t* b = p.b;
  const float* sb = p.scale_b;
  if constexpr (kRagged) {
    const int expert = p.tile_expert[tile_m];
    if (expert < 0) return;
    row0 = p.tile_row[tile_m];
    row_limit = p.expert_offsets[expert + 1];
    b += static_cast<long long>(expert) * p.b_expert_stride;
    sb += static_cast<long long>(expert) * p.sb_expert_stride;
  } else {
    row0 = tile_m * kSimtTile;
    row_limit = p.m;
  }
  if (tid < kSimtTile) {
    const int row = row0 + tid;
    const bool valid = row < row_limit;
    long long source = row;
    if constexpr (kRagged) {
      if (valid && p.order != nullptr) source = p.order[row] / p.top_k;
    }
    a_row_valid[tid] = valid;
    a_row_offset[tid] = valid ? source * p.a_sm : 0;
    sa_row_offset[tid] = valid ? source * p.sa_sm : 0;
  }
  __syncthreads();

  const int groups = (p.k + p.group_size - 1) / p.group_size;
  const int words = p.group_size / 4;
  float total[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  const int r0 = ty * 2, c0 = tx * 2;

  for (int g = 0; g < groups; ++g) {
    const int k0 = g * p.group_size;
    for (int idx = tid; idx < kSimtTile * p.group_size; idx += 256) {
      // A: consecutive threads walk K; B: consecutive threads walk K as well, which is the
      // contiguous direction of Linear-format weights.
      const int r = idx / p.group_size, kk = idx - r * p.group_size;
      const int k = k0 + kk;
      int8_t av = 0, bv = 0;
      if (k < p.k) {
        if (a_row_valid[r]) av = p.a[a_row_offset[r] + k * p.a_sk];
        if (n0 + r < p.n) bv = b[k * p.b_sk + static_cast<long long>(n0 + r) * p.b_sn];
      }
      a_tile[r][kk] = av;
      b_tile[r][kk] = bv;
    }
    __syncthreads();
    int dot[2][2] = {{0, 0}, {0, 0}};
    const int* a0 = reinterpret_cast<const int*>(a_tile[r0]);
    const int* a1 = reinterpret_cast<const int*>(a_tile[r0 + 1]);
    const int* b0 = reinterpret_cast<const int*>(b_tile[c0]);
    const int* b1 = reinterpret_cast<const int*>(b_tile[c0 + 1]);
    for (int w = 0; w < words; ++w) {
      const int x0 = a0[w], x1 = a1[w], y0 = b0[w], y1 = b1[w];
      dot[0][0] = __dp4a(x0, y0, dot[0][0]);
      dot[0][1] = __dp4a(x0, y1, dot[0][1]);
      dot[1][0] = __dp4a(x1, y0, dot[1][0]);
      dot[1][1] = __dp4a(x1, y1, dot[1][1]);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int col = n0 + c0 + j;
        if (a_row_valid[r0 + i] && col < p.n) {
          const float sa = p.scale_a[sa_row_offset[r0 + i] + g * p.sa_sg];
          const float sbv = sb[g * p.sb_sg + col * p.sb_sn];
          const float scale = __fmul_rn(sa, sbv);
          total[i][j] = __fmaf_rn(__int2float_rn(dot[i][j]), scale, total[i][j]);
          if (p.partials != nullptr) {
            p.partials[(static_cast<long long>(row0 + r0 + i) * p.n + col) * groups + g] =
                dot[i][j];
          }
        }
      }
    }
    __syncthreads();
  }
  OutT* c = reinterpret_cast<OutT*>(p.c);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int col = n0 + c0 + j;
      if (a_row_valid[r0 + i] && col < p.n) {
        c[static_cast<long long>(row0 + r0 + i) * p.ldc + col] = cast_out<OutT>(total[i][j]);
      }
    }
  }
}

// Second half of the split-K path: folds the INT32 group dots partials[Q][M][N] in group
// order, C[m,n] = cast(fold_g fmaf(float(p_g), sa[m,g]*sb[g,n], total)); one thread per output.
template <typename OutT>
__global__ void __launch_bounds__(256)
fold_partials_kernel(const int* __restrict__ partials, const float* __restrict__ scale_a,
                     const float* __restrict__ scale_b, OutT* __restrict__ c, int m, int n,
                     int groups, long long sa_sm, long long sa_sg, long long sb_sg, long long sb_sn,
                     long long ldc) {
  const int col = blockIdx.x * 256 + threadIdx.x;
  const int row = blockIdx.y;
  if (col >= n) return;
  float total = 0.0f;
  const long long plane = static_cast<long long>(m) * n;
  const int* source = partials + static_cast<long long>(row) * n + col;
  // Sixteen groups' loads are issued before their fused adds (which stay in group order).
  int g = 0;
  for (; g + 16 <= groups; g += 16) {
    int dot[16];
    float scale[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      dot[j] = source[(g + j) * plane];
      scale[j] = __fmul_rn(scale_a[row * sa_sm + (g + j) * sa_sg], scale_b[(g + j) * sb_sg + col * sb_sn]);
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) total = __fmaf_rn(__int2float_rn(dot[j]), scale[j], total);
  }
  for (; g < groups; ++g) {
    const float scale = __fmul_rn(scale_a[row * sa_sm + g * sa_sg], scale_b[g * sb_sg + col * sb_sn]);
    total = __fmaf_rn(__int2float_rn(source[g * plane]), scale, total);
  }
  c[static_cast<long long>(row) * ldc + col] = cast_out<OutT>(total);
}

}  // namespace gg
