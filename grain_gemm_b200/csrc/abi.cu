// extern "C" entry points of libgrain_b200.so (declared in include/grain_gemm_b200.h):
// argument checks, tensor-map encoding, variant selection and kernel launches.
// Nothing here allocates or synchronises (gg_device_status excepted, which reads back a word).

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "../../include/grain_gemm_b200.h"
#include "gemm_gemv.cuh"
#include "gemm_simt.cuh"
#include "gemm_tc.cuh"
#include "moe_ep.cuh"
#include "moe_gate_up_tc.cuh"
#include "moe_route.cuh"

namespace gg {

constexpr int kAbiVersion = 4;

// ---------------------------------------------------------------- host helpers

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &query) !=
            cudaSuccess ||
        query != cudaDriverEntryPointSuccess) {
      ptr = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// Tensor map over a row-major int8 matrix [rows, cols] with row pitch `pitch` bytes; boxes of
// 128 bytes x box_rows with the 128-byte swizzle; out-of-range elements read as zero.
static int encode_int8_rows(CUtensorMap* map, const void* base, long long rows, long long cols,
                            long long pitch, int box_rows) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return static_cast<int>(cudaErrorNotSupported);
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch)};
  const cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t element_strides[2] = {1u, 1u};
  const CUresult result = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base),
                                 dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return result == CUDA_SUCCESS ? 0 : -10000 - static_cast<int>(result);
}

static int sm_count() {
  // Immutable device property, cached per device.
  static int cached[64] = {0};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
  if (cached[device] == 0) {
    int count = 0;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        count <= 0) {
      count = 148;
    }
    cached[device] = count;
  }
  return cached[device];
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct GemmArgs {
  const void *a, *b, *scale_a, *scale_b;
  void* c;
  int m, n, k;
  long long a_sm, a_sk, b_sk, b_sn, sa_sm, sa_sg, sb_sg, sb_sn, ldc;
  int group_size, out_dtype;
};

static bool valid_group(int g) { return g == 32 || g == 64 || g == 128 || g == 256; }

// The automatic choice gives one row to the weight-streaming kernel whatever the weights' size,
// two rows up to this many weight bytes (measured: beyond it split-K is faster for two rows).
constexpr long long kGemvTwoRowBytes = 32ll << 20;

static bool tensor_core_layout(const GemmArgs& g) {
  return g.a_sk == 1 && g.b_sk == 1 && g.a_sm % 16 == 0 && g.b_sn % 16 == 0 && g.a_sm >= g.k &&
         g.b_sn >= g.k && aligned16(g.a) && aligned16(g.b);
}

// Split-K plan for skinny M: N tiles of 256 columns times k_splits K ranges fill the SMs; the
// INT32 group dots go through `workspace` and are folded in group order by a second kernel,
// so the result is bit-identical to the single-pass kernels.
struct SplitKPlan {
  int splits, groups_per_split;
  size_t workspace_bytes;
};

static SplitKPlan splitk_plan(int m, int n, int k, int group_size) {
  SplitKPlan plan = {1, 0, 0};
  const int groups = (k + group_size - 1) / group_size;
  const int unit = group_size >= 128 ? 1 : 128 / group_size;   // ranges start on 128-byte slabs
  if (m > 32 || n <= 0 || groups < 2 * unit) return plan;
  // Finest ranges: the kernel hands every group's INT32 dots to the fold anyway, so a work item
  // of one 128-byte-aligned range costs nothing extra, and tiles x ranges items spread evenly
  // over all SMs whatever N is (a skinny GEMM is bound by how many SMs pull weights at once).
  const int splits = (groups + unit - 1) / unit;
  if (splits < 2) return plan;
  plan.splits = splits;
  plan.groups_per_split = unit;
  plan.workspace_bytes = static_cast<size_t>(groups) * m * n * sizeof(int);
  return plan;
}

// The weight-streaming kernel takes the tensor-core kernels' operand layout and whole 16-byte
// chunks of K.
static int gemv_rows(int m) { return m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : 8; }

static size_t gemv_smem_bytes(const GemmArgs& g, int columns) {
  const size_t rows = static_cast<size_t>(gemv_rows(g.m));
  const size_t groups = static_cast<size_t>((g.k + g.group_size - 1) / g.group_size);
  return groups * (rows * columns + columns + rows) * sizeof(int);
}

// The kernel instantiation for (rows, lanes per K group): every combination exists.
typedef void (*GemvKernel)(const GemvParams);

template <int kRows>
static GemvKernel gemv_kernel_for_group(int group_size) {
  switch (group_size) {
    case 32: return gemm_gemv_kernel<kRows, 2>;
    case 64: return gemm_gemv_kernel<kRows, 4>;
    case 128: return gemm_gemv_kernel<kRows, 8>;
    default: return gemm_gemv_kernel<kRows, 16>;
  }
}

static GemvKernel gemv_kernel(int rows, int group_size) {
  switch (rows) {
    case 1: return gemv_kernel_for_group<1>(group_size);
    case 2: return gemv_kernel_for_group<2>(group_size);
    case 4: return gemv_kernel_for_group<4>(group_size);
    default: return gemv_kernel_for_group<8>(group_size);
  }
}

// CTAs of the kernel that one SM holds (registers decide; asked once per row count).
static int gemv_ctas_per_sm(int rows) {
  static int cached[4] = {0, 0, 0, 0};
  const int index = rows == 1 ? 0 : rows == 2 ? 1 : rows == 4 ? 2 : 3;
  if (cached[index] == 0) {
    int blocks = 0;
    const cudaError_t error = cudaOccupancyMaxActiveBlocksPerMultiprocessor(
        &blocks, gemv_kernel(rows, 256), kGemvThreads, 4096);
    if (error != cudaSuccess) (void)cudaGetLastError();
    cached[index] = error == cudaSuccess && blocks > 0 ? blocks : 2;
  }
  return cached[index];
}

// Columns per warp (0 = not eligible): the fewest for which all CTAs of the launch are resident
// at once, as long as a CTA's per-group dots and scales fit 96 KB of shared memory.
static int gemv_columns_per_warp(const GemmArgs& g) {
  if (!tensor_core_layout(g) || g.m < 1 || g.m > kGemvMaxRows || g.k % 16 != 0) return 0;
  const long long resident = static_cast<long long>(sm_count()) * gemv_ctas_per_sm(gemv_rows(g.m));
  int per_warp = 1;
  while (per_warp < kGemvMaxColumnsPerWarp &&
         (g.n + kGemvWarps * per_warp - 1) / (kGemvWarps * per_warp) > resident) {
    ++per_warp;
  }
  while (per_warp > 1 && gemv_smem_bytes(g, kGemvWarps * per_warp) > 96 * 1024) --per_warp;
  return gemv_smem_bytes(g, kGemvWarps * per_warp) <= 96 * 1024 ? per_warp : 0;
}

static bool gemv_eligible(const GemmArgs& g) { return gemv_columns_per_warp(g) != 0; }

static int launch_gemv(const GemmArgs& g, cudaStream_t stream) {
  const int per_warp = gemv_columns_per_warp(g);
  if (per_warp == 0) return static_cast<int>(cudaErrorInvalidValue);
  GemvParams p = {};
  p.a = static_cast<const int8_t*>(g.a);
  p.b = static_cast<const int8_t*>(g.b);
  p.scale_a = static_cast<const float*>(g.scale_a);
  p.scale_b = static_cast<const float*>(g.scale_b);
  p.c = g.c;
  p.m = g.m; p.n = g.n; p.k = g.k;
  p.group_size = g.group_size;
  p.out_dtype = g.out_dtype;
  p.a_sm = g.a_sm; p.b_sn = g.b_sn;
  p.sa_sm = g.sa_sm; p.sa_sg = g.sa_sg; p.sb_sg = g.sb_sg; p.sb_sn = g.sb_sn;
  p.ldc = g.ldc;
  p.columns_per_warp = per_warp;
  const int columns = kGemvWarps * per_warp;
  const size_t smem = gemv_smem_bytes(g, columns);
  const unsigned grid = static_cast<unsigned>((g.n + columns - 1) / columns);
  const GemvKernel kernel = gemv_kernel(gemv_rows(g.m), g.group_size);
  if (smem > 48 * 1024) {
    const cudaError_t error = cudaFuncSetAttribute(
        kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (error != cudaSuccess) return static_cast<int>(error);
  }
  kernel<<<grid, kGemvThreads, smem, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

static int select_variant(const GemmArgs& g) {
  if (!tensor_core_layout(g)) return GG_VARIANT_SIMT;
  const bool gemv_rows_ok =
      g.m == 1 || (g.m == 2 && static_cast<long long>(g.n) * g.k <= kGemvTwoRowBytes);
  if (gemv_rows_ok && gemv_eligible(g)) return GG_VARIANT_GEMV;
  const int sms = sm_count();
  const long long tiles_256 = static_cast<long long>((g.m + 127) / 128) * ((g.n + 255) / 256);
  if (splitk_plan(g.m, g.n, g.k, g.group_size).splits >= 2) return GG_VARIANT_TC_SPLITK;
  if (g.m > 128 && tiles_256 >= sms) return GG_VARIANT_TC_PAIR_N256;
  if (tiles_256 >= sms) return GG_VARIANT_TC_N256;
  const long long tiles_128 = static_cast<long long>((g.m + 127) / 128) * ((g.n + 127) / 128);
  if (tiles_128 >= sms) return GG_VARIANT_TC_N128;
  return GG_VARIANT_TC_N64;
}

template <typename OutT, bool kRagged>
static int launch_simt(const GemmSimtParams& p, int row_tiles, cudaStream_t stream) {
  const long long blocks = static_cast<long long>((p.n + kSimtTile - 1) / kSimtTile) * row_tiles;
  if (blocks <= 0) return 0;
  if (blocks > 0x7fffffffLL) return static_cast<int>(cudaErrorInvalidValue);
  gemm_simt_kernel<OutT, kRagged><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

template <bool kRagged>
static int launch_simt_dtype(const GemmSimtParams& p, int row_tiles, int out_dtype,
                             cudaStream_t stream) {
  switch (out_dtype) {
    case GG_OUT_FP32: return launch_simt<float, kRagged>(p, row_tiles, stream);
    case GG_OUT_BF16: return launch_simt<__nv_bfloat16, kRagged>(p, row_tiles, stream);
    case GG_OUT_FP16: return launch_simt<__half, kRagged>(p, row_tiles, stream);
    default: return static_cast<int>(cudaErrorInvalidValue);
  }
}

static GemmSimtParams simt_params(const GemmArgs& g) {
  GemmSimtParams p = {};
  p.a = static_cast<const int8_t*>(g.a);
  p.b = static_cast<const int8_t*>(g.b);
  p.scale_a = static_cast<const float*>(g.scale_a);
  p.scale_b = static_cast<const float*>(g.scale_b);
  p.c = g.c;
  p.m = g.m; p.n = g.n; p.k = g.k;
  p.a_sm = g.a_sm; p.a_sk = g.a_sk; p.b_sk = g.b_sk; p.b_sn = g.b_sn;
  p.sa_sm = g.sa_sm; p.sa_sg = g.sa_sg; p.sb_sg = g.sb_sg; p.sb_sn = g.sb_sn;
  p.ldc = g.ldc;
  p.group_size = g.group_size;
  return p;
}

template <int kCtaGroup, int BN, int kStages, typename OutT, bool kGrouped, int kPromoWarps,
          int kARows = 128>
static int launch_tc_kernel(const CUtensorMap& map_a, const CUtensorMap& map_b,
                            const GemmTcParams& p, cudaStream_t stream) {
  using Shape = GemmTcShape<kCtaGroup, BN, kStages, kPromoWarps, kARows>;
  auto kernel = gemm_tc_kernel<kCtaGroup, BN, kStages, OutT, kGrouped, kPromoWarps, false, kARows>;
  cudaError_t error =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape::kSmemBytes);
  if (error != cudaSuccess) return static_cast<int>(error);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(sm_count() / kCtaGroup * kCtaGroup);
  config.blockDim = dim3(Shape::kThreads);
  config.dynamicSmemBytes = Shape::kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = kCtaGroup;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  // The kernel is persistent: every CTA (pair) of the grid must be resident at once, or the
  // late ones only start when an early one has finished all of its tiles.  How many pairs fit
  // depends on the part: a cluster cannot span GPCs, and B200s differ in how their 148 SMs are
  // spread over GPCs (one with an odd number of SMs strands one SM for pairs).  Immutable per
  // device and kernel, so asked once.
  int workers_max = sm_count() / kCtaGroup;
  if constexpr (kCtaGroup > 1) {
    static int cached[64] = {0};
    int device = 0;
    if (cudaGetDevice(&device) == cudaSuccess && device >= 0 && device < 64) {
      if (cached[device] == 0) {
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess || clusters <= 0) {
          clusters = workers_max;
        }
        cached[device] = clusters;
      }
      if (cached[device] < workers_max) workers_max = cached[device];
    }
  }
  const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
  const int workers = static_cast<int>(tiles < workers_max ? tiles : workers_max);
  if (workers <= 0) return 0;
  config.gridDim = dim3(workers * kCtaGroup);
  error = cudaLaunchKernelEx(&config, kernel, map_a, map_b, p);
  return static_cast<int>(error);
}

template <int kCtaGroup, int BN, int kStages, bool kGrouped, int kPromoWarps = 8, int kARows = 128>
static int launch_tc_dtype(const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmTcParams& p,
                           int out_dtype, cudaStream_t stream) {
  switch (out_dtype) {
    case GG_OUT_FP32:
      if constexpr (kGrouped) return static_cast<int>(cudaErrorInvalidValue);
      else return launch_tc_kernel<kCtaGroup, BN, kStages, float, kGrouped, kPromoWarps, kARows>(map_a, map_b, p, stream);
    case GG_OUT_BF16:
      return launch_tc_kernel<kCtaGroup, BN, kStages, __nv_bfloat16, kGrouped, kPromoWarps, kARows>(map_a, map_b, p, stream);
    case GG_OUT_FP16:
      return launch_tc_kernel<kCtaGroup, BN, kStages, __half, kGrouped, kPromoWarps, kARows>(map_a, map_b, p, stream);
    default: return static_cast<int>(cudaErrorInvalidValue);
  }
}

static int launch_gemm_tc(const GemmArgs& g, int variant, cudaStream_t stream) {
  const bool pair = variant == GG_VARIANT_TC_PAIR_N256 || variant == GG_VARIANT_TC_PAIR_N128;
  const int bn = (variant == GG_VARIANT_TC_N256 || variant == GG_VARIANT_TC_PAIR_N256) ? 256
                 : (variant == GG_VARIANT_TC_N128 || variant == GG_VARIANT_TC_PAIR_N128) ? 128
                                                                                         : 64;
  CUtensorMap map_a, map_b;
  int status = encode_int8_rows(&map_a, g.a, g.m, g.k, g.a_sm, 128);
  if (status) return status;
  status = encode_int8_rows(&map_b, g.b, g.n, g.k, g.b_sn, pair ? bn / 2 : bn);
  if (status) return status;
  GemmTcParams p = {};
  p.scale_a = static_cast<const float*>(g.scale_a);
  p.scale_b = static_cast<const float*>(g.scale_b);
  p.c = g.c;
  p.m = g.m; p.n = g.n; p.k = g.k;
  p.sa_sm = g.sa_sm; p.sa_sg = g.sa_sg; p.sb_sg = g.sb_sg; p.sb_sn = g.sb_sn;
  p.ldc = g.ldc;
  p.group_size = g.group_size;
  p.k_splits = 1;
  p.band_rows = 16;
  p.tiles_m = (g.m + (pair ? 255 : 127)) / (pair ? 256 : 128);
  p.tiles_n = (g.n + bn - 1) / bn;
  const int out_bytes = g.out_dtype == GG_OUT_FP32 ? 4 : 2;
  p.c_vector_ok = aligned16(g.c) && (g.ldc * out_bytes) % 16 == 0;
  switch (variant) {
    case GG_VARIANT_TC_N256: return launch_tc_dtype<1, 256, 4, false>(map_a, map_b, p, g.out_dtype, stream);
    case GG_VARIANT_TC_N128: return launch_tc_dtype<1, 128, 6, false>(map_a, map_b, p, g.out_dtype, stream);
    case GG_VARIANT_TC_N64: return launch_tc_dtype<1, 64, 8, false>(map_a, map_b, p, g.out_dtype, stream);
    case GG_VARIANT_TC_PAIR_N256: return launch_tc_dtype<2, 256, 6, false>(map_a, map_b, p, g.out_dtype, stream);
    case GG_VARIANT_TC_PAIR_N128: return launch_tc_dtype<2, 128, 8, false>(map_a, map_b, p, g.out_dtype, stream);
    default: return static_cast<int>(cudaErrorInvalidValue);
  }
}

static int launch_gemm_splitk(const GemmArgs& g, void* workspace, size_t workspace_bytes,
                              cudaStream_t stream) {
  const SplitKPlan plan = splitk_plan(g.m, g.n, g.k, g.group_size);
  if (plan.splits < 2 || workspace == nullptr || workspace_bytes < plan.workspace_bytes ||
      !aligned16(workspace)) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  CUtensorMap map_a, map_b;
  int status = encode_int8_rows(&map_a, g.a, g.m, g.k, g.a_sm, 32);
  if (status) return status;
  status = encode_int8_rows(&map_b, g.b, g.n, g.k, g.b_sn, 256);
  if (status) return status;
  GemmTcParams p = {};
  p.m = g.m; p.n = g.n; p.k = g.k;
  p.group_size = g.group_size;
  p.tiles_m = 1;
  p.band_rows = 8;
  p.tiles_n = (g.n + 255) / 256;
  p.k_splits = plan.splits;
  p.groups_per_split = plan.groups_per_split;
  p.partials = static_cast<int*>(workspace);
  using Shape = GemmTcShape<1, 256, 6, 8, 32>;
  auto kernel = gemm_tc_kernel<1, 256, 6, float, false, 8, true, 32>;
  cudaError_t error =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape::kSmemBytes);
  if (error != cudaSuccess) return static_cast<int>(error);
  const int items = p.tiles_n * p.k_splits;
  const int grid = items < sm_count() ? items : sm_count();
  kernel<<<grid, Shape::kThreads, Shape::kSmemBytes, stream>>>(map_a, map_b, p);
  error = cudaGetLastError();
  if (error != cudaSuccess) return static_cast<int>(error);
  const int groups = (g.k + g.group_size - 1) / g.group_size;
  const dim3 fold_grid((g.n + 255) / 256, g.m);
  const int* partials = static_cast<const int*>(workspace);
  const float* sa = static_cast<const float*>(g.scale_a);
  const float* sb = static_cast<const float*>(g.scale_b);
  switch (g.out_dtype) {
    case GG_OUT_FP32:
      fold_partials_kernel<float><<<fold_grid, 256, 0, stream>>>(
          partials, sa, sb, static_cast<float*>(g.c), g.m, g.n, groups, g.sa_sm, g.sa_sg, g.sb_sg,
          g.sb_sn, g.ldc);
      break;
    case GG_OUT_BF16:
      fold_partials_kernel<__nv_bfloat16><<<fold_grid, 256, 0, stream>>>(
          partials, sa, sb, static_cast<__nv_bfloat16*>(g.c), g.m, g.n, groups, g.sa_sm, g.sa_sg,
          g.sb_sg, g.sb_sn, g.ldc);
      break;
    default:
      fold_partials_kernel<__half><<<fold_grid, 256, 0, stream>>>(
          partials, sa, sb, static_cast<__half*>(g.c), g.m, g.n, groups, g.sa_sm, g.sa_sg, g.sb_sg,
          g.sb_sn, g.ldc);
      break;
  }
  return static_cast<int>(cudaGetLastError());
}

static int run_gemm(const GemmArgs& g, int variant, cudaStream_t stream, void* workspace = nullptr,
                    size_t workspace_bytes = 0) {
  if (g.m < 0 || g.n < 0 || g.k < 0 || !valid_group(g.group_size) || g.out_dtype < 0 ||
      g.out_dtype > 2 || g.a_sm <= 0 || g.a_sk <= 0 || g.b_sk <= 0 || g.b_sn <= 0 || g.ldc < g.n) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (g.m == 0 || g.n == 0) return 0;
  if (g.k == 0) return static_cast<int>(cudaErrorInvalidValue);  // callers zero-fill instead
  if (!g.a || !g.b || !g.scale_a || !g.scale_b || !g.c) return static_cast<int>(cudaErrorInvalidValue);
  if (variant == GG_VARIANT_AUTO) {
    variant = select_variant(g);
    // Without a workspace the skinny shapes stay on the single-pass kernels.
    if (variant == GG_VARIANT_TC_SPLITK && workspace == nullptr) variant = GG_VARIANT_TC_N64;
  }
  if (variant == GG_VARIANT_TC_SPLITK) {
    if (!tensor_core_layout(g)) return static_cast<int>(cudaErrorInvalidValue);
    return launch_gemm_splitk(g, workspace, workspace_bytes, stream);
  }
  if (variant == GG_VARIANT_SIMT) {
    return launch_simt_dtype<false>(simt_params(g), (g.m + kSimtTile - 1) / kSimtTile, g.out_dtype,
                                    stream);
  }
  if (variant == GG_VARIANT_GEMV) return launch_gemv(g, stream);
  if (variant < GG_VARIANT_TC_N256 || variant > GG_VARIANT_TC_PAIR_N128 || !tensor_core_layout(g)) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  return launch_gemm_tc(g, variant, stream);
}

template <typename RoundT, bool kGather>
static int launch_gate_up_tc(const CUtensorMap& map_x, const CUtensorMap& map_w,
                             const GateUpParams& p, int grid, cudaStream_t stream) {
  auto kernel = moe_gate_up_tc_kernel<RoundT, kGather>;
  const cudaError_t error = cudaFuncSetAttribute(
      kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GateUpShape::kSmemBytes);
  if (error != cudaSuccess) return static_cast<int>(error);
  kernel<<<grid, 384, GateUpShape::kSmemBytes, stream>>>(map_x, map_w, p);
  return static_cast<int>(cudaGetLastError());
}

// One warp waits, with the kernels' own bounded wait, on a barrier that nothing ever
// completes: the wait gives up after `limit_ns`, records (kSiteSelfTest << 8) | 1 in the device
// status word and the kernel returns normally.  *result = 1 if the wait reported success.
__global__ void wait_timeout_probe_kernel(unsigned long long limit_ns, int* result) {
  __shared__ uint64_t barrier;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&barrier, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const bool completed = mbar_wait_warp(&barrier, 0u, kSiteSelfTest, &abort_flag, limit_ns);
  if (threadIdx.x == 0) *result = completed ? 1 : 0;
}

}  // namespace gg

// ------------------------------------------------------------------ extern "C"

extern "C" {

int gg_abi_version(void) { return gg::kAbiVersion; }

const char* gg_error_string(int status) {
  if (status == 0) return "success";
  if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
  if (status == GG_STATUS_STATIC_SCRATCH_TOO_SMALL) {
    return "problem too large for the library's static scratch (use the entry point that takes "
           "a caller workspace)";
  }
  if (status <= -10000) {
    static thread_local char text[64];
    snprintf(text, sizeof(text), "tensor map encoding failed (CUresult %d)", -10000 - status);
    return text;
  }
  return "unknown status";
}

const char* grain_cuda_error_string(int status) { return gg_error_string(status); }

int gg_int8_gemm(const void* a, const void* b, const void* scale_a, const void* scale_b, void* c,
                 int m, int n, int k, long long a_sm, long long a_sk, long long b_sk,
                 long long b_sn, long long sa_sm, long long sa_sg, long long sb_sg, long long sb_sn,
                 long long ldc, int group_size, int out_dtype, int variant, void* stream) {
  const gg::GemmArgs g = {a, b, scale_a, scale_b, c, m, n, k, a_sm, a_sk, b_sk, b_sn,
                          sa_sm, sa_sg, sb_sg, sb_sn, ldc, group_size, out_dtype};
  return gg::run_gemm(g, variant, static_cast<cudaStream_t>(stream));
}

size_t gg_int8_gemm_workspace_bytes(int m, int n, int k, int group_size) {
  if (m <= 0 || n <= 0 || k <= 0 || !gg::valid_group(group_size)) return 0;
  return gg::splitk_plan(m, n, k, group_size).workspace_bytes;
}

int gg_int8_gemm_ws(const void* a, const void* b, const void* scale_a, const void* scale_b, void* c,
                    int m, int n, int k, long long a_sm, long long a_sk, long long b_sk,
                    long long b_sn, long long sa_sm, long long sa_sg, long long sb_sg,
                    long long sb_sn, long long ldc, int group_size, int out_dtype, int variant,
                    void* workspace, size_t workspace_bytes, void* stream) {
  const gg::GemmArgs g = {a, b, scale_a, scale_b, c, m, n, k, a_sm, a_sk, b_sk, b_sn,
                          sa_sm, sa_sg, sb_sg, sb_sn, ldc, group_size, out_dtype};
  return gg::run_gemm(g, variant, static_cast<cudaStream_t>(stream), workspace, workspace_bytes);
}

int gg_int8_gemm_select(const void* a, const void* b, const void* c, int m, int n, int k,
                        long long a_sm, long long a_sk, long long b_sk, long long b_sn,
                        long long ldc, int group_size, int out_dtype) {
  const gg::GemmArgs g = {a, b, nullptr, nullptr, const_cast<void*>(c), m, n, k, a_sm, a_sk, b_sk,
                          b_sn, 0, 0, 0, 0, ldc, group_size, out_dtype};
  return gg::select_variant(g);
}

int gg_int8_gemm_partials(const void* a, const void* b, const void* scale_a, const void* scale_b,
                          void* c_fp32, void* partials, int m, int n, int k, long long a_sm,
                          long long a_sk, long long b_sk, long long b_sn, long long sa_sm,
                          long long sa_sg, long long sb_sg, long long sb_sn, int group_size,
                          void* stream) {
  if (m <= 0 || n <= 0 || k <= 0 || !gg::valid_group(group_size) || !partials || !c_fp32) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  const gg::GemmArgs g = {a, b, scale_a, scale_b, c_fp32, m, n, k, a_sm, a_sk, b_sk, b_sn,
                          sa_sm, sa_sg, sb_sg, sb_sn, n, group_size, GG_OUT_FP32};
  gg::GemmSimtParams p = gg::simt_params(g);
  p.partials = static_cast<int*>(partials);
  return gg::launch_simt_dtype<false>(p, (m + gg::kSimtTile - 1) / gg::kSimtTile, GG_OUT_FP32,
                                      static_cast<cudaStream_t>(stream));
}

int grain_cute_g256(const void* a, const void* b, const void* scale_a, const void* scale_b,
                    void* c, int m, int n, int k, int config, void* stream) {
  (void)config;
  if (m <= 0 || n <= 0 || k <= 0 || k % 256) return static_cast<int>(cudaErrorInvalidValue);
  const int groups = k / 256;
  const gg::GemmArgs g = {a, b, scale_a, scale_b, c, m, n, k, k, 1, 1, k,
                          groups, 1, n, 1, n, 256, GG_OUT_BF16};
  return gg::run_gemm(g, GG_VARIANT_AUTO, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------- MoE

size_t gg_moe_route_workspace_bytes(int tokens, int top_k, int experts) {
  const long long slots = static_cast<long long>(tokens) * top_k;
  if (slots <= gg::kRouteChunk) return 0;
  const long long chunks = (slots + gg::kRouteChunk - 1) / gg::kRouteChunk;
  return static_cast<size_t>(chunks * (experts + 2)) * sizeof(int);
}

int gg_moe_route(const void* ids, int ids_are_i64, const void* mask, int tokens, int top_k,
                 int experts, void* effective_ids, void* order, void* inverse, void* counts,
                 void* offsets, void* statistics, void* workspace, size_t workspace_bytes,
                 void* stream_ptr) {
  if (tokens < 0 || top_k <= 0 || experts <= 0 || !counts || !offsets || !statistics) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  gg::RouteParams p = {};
  p.ids = ids;
  p.ids_are_i64 = ids_are_i64;
  p.mask = static_cast<const uint8_t*>(mask);
  p.tokens = tokens; p.top_k = top_k; p.experts = experts;
  p.effective_ids = effective_ids;
  p.order = static_cast<long long*>(order);
  p.inverse = static_cast<int*>(inverse);
  p.counts = static_cast<int*>(counts);
  p.offsets = static_cast<int*>(offsets);
  p.statistics = static_cast<int*>(statistics);
  p.workspace = static_cast<int*>(workspace);
  const long long slots = static_cast<long long>(tokens) * top_k;
  const size_t smem = static_cast<size_t>(experts + 2) * sizeof(int);
  if (smem > 200 * 1024) return static_cast<int>(cudaErrorInvalidValue);
  if (slots > 0 && (!ids || !effective_ids || !order || !inverse)) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  cudaError_t error;
  if (slots <= gg::kRouteChunk) {
    if (smem > 48 * 1024) {
      error = cudaFuncSetAttribute(gg::route_single_kernel,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (error != cudaSuccess) return static_cast<int>(error);
    }
    gg::route_single_kernel<<<1, gg::kRouteChunk, smem, stream>>>(p);
    return static_cast<int>(cudaGetLastError());
  }
  if (slots <= gg::kRouteMediumSlots && experts + 1 <= gg::kRouteMediumKeys) {
    const size_t medium = (static_cast<size_t>(33) * (experts + 1) + 33) * sizeof(int);
    if (medium > 48 * 1024) {
      error = cudaFuncSetAttribute(gg::route_medium_kernel,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(medium));
      if (error != cudaSuccess) return static_cast<int>(error);
    }
    gg::route_medium_kernel<<<1, 1024, medium, stream>>>(p);
    return static_cast<int>(cudaGetLastError());
  }
  if (workspace_bytes < gg_moe_route_workspace_bytes(tokens, top_k, experts) || !workspace) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  const int chunks = static_cast<int>((slots + gg::kRouteChunk - 1) / gg::kRouteChunk);
  if (smem > 48 * 1024) {
    for (const void* kernel : {reinterpret_cast<const void*>(gg::route_histogram_kernel),
                               reinterpret_cast<const void*>(gg::route_scan_kernel),
                               reinterpret_cast<const void*>(gg::route_place_kernel)}) {
      error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(smem));
      if (error != cudaSuccess) return static_cast<int>(error);
    }
  }
  gg::route_histogram_kernel<<<chunks, gg::kRouteChunk, smem, stream>>>(p);
  gg::route_scan_kernel<<<1, 1024, smem, stream>>>(p, chunks);
  gg::route_place_kernel<<<chunks, gg::kRouteChunk, smem, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

// ---- routing without any allocation -----------------------------------------------------
//
// Scratch for gg_moe_route_noalloc lives in the library image: every GPU that loads the
// library carries these 2 MiB until the process exits.
static constexpr size_t kStaticRouteScratchInts = 512 * 1024;
static __device__ __align__(256) int g_static_route_scratch[kStaticRouteScratchInts];

// Device address of the static scratch for the current device.  In host code the array's
// name is only a handle; the address a kernel can use comes from cudaGetSymbolAddress, asked
// once per device while that device is current.
static int static_route_scratch(int** out) {
  static int* address[64] = {nullptr};
  static std::mutex guard;
  int device = 0;
  cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) return static_cast<int>(error);
  if (device < 0 || device >= 64) return static_cast<int>(cudaErrorInvalidDevice);
  std::lock_guard<std::mutex> lock(guard);
  if (address[device] == nullptr) {
    void* pointer = nullptr;
    error = cudaGetSymbolAddress(&pointer, g_static_route_scratch);
    if (error != cudaSuccess) return static_cast<int>(error);
    address[device] = static_cast<int*>(pointer);
  }
  *out = address[device];
  return 0;
}

int gg_moe_route_noalloc(const void* ids, int ids_are_i64, const void* mask, int tokens, int top_k,
                         int experts, void* effective_ids, void* order, void* inverse, void* counts,
                         void* offsets, void* statistics, void* stream) {
  if (tokens < 0 || top_k <= 0 || experts <= 0) return static_cast<int>(cudaErrorInvalidValue);
  const size_t needed = gg_moe_route_workspace_bytes(tokens, top_k, experts);
  if (needed > kStaticRouteScratchInts * sizeof(int)) return GG_STATUS_STATIC_SCRATCH_TOO_SMALL;
  if (!counts || !offsets || !statistics ||
      (static_cast<long long>(tokens) * top_k > 0 && (!ids || !effective_ids || !order || !inverse))) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  int* scratch = nullptr;
  const int status = static_route_scratch(&scratch);
  if (status) return status;
  return gg_moe_route(ids, ids_are_i64, mask, tokens, top_k, experts, effective_ids, order, inverse,
                      counts, offsets, statistics, scratch, kStaticRouteScratchInts * sizeof(int),
                      stream);
}

size_t gg_moe_route_noalloc_capacity_bytes(void) { return kStaticRouteScratchInts * sizeof(int); }

int gg_moe_tile_capacity(int assignments, int experts, int tile_rows) {
  if (assignments < 0 || experts <= 0 || tile_rows <= 0) return 0;
  return (assignments + tile_rows - 1) / tile_rows + experts;
}

int gg_moe_tiles(const void* offsets, int experts, int tile_rows, int capacity, void* tile_expert,
                 void* tile_row, void* stream) {
  if (!offsets || !tile_expert || !tile_row || experts <= 0 || tile_rows <= 0 || capacity <= 0) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  gg::moe_tiles_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int*>(offsets), experts, tile_rows, capacity, static_cast<int*>(tile_expert),
      static_cast<int*>(tile_row));
  return static_cast<int>(cudaGetLastError());
}

size_t gg_moe_gate_up_scratch_bytes(int assignments, int hidden, int intermediate, int tile_rows,
                                    int row_gather) {
  const size_t slots = static_cast<size_t>(assignments > 0 ? assignments : 0);
  if (tile_rows == 128) {
    const size_t table = 65536 * sizeof(float);
    if (row_gather) return table;
    const size_t rows = slots * static_cast<size_t>(hidden > 0 ? hidden : 0);
    const size_t scales = slots * static_cast<size_t>(hidden > 0 ? hidden / 256 : 0) * 4;
    return ((rows + 255) & ~static_cast<size_t>(255)) + ((scales + 255) & ~static_cast<size_t>(255)) +
           table;
  }
  return slots * 2 * intermediate * 2;
}

int gg_moe_silu_table(void* table, int out_dtype, void* stream_ptr) {
  if (!table || (out_dtype != GG_OUT_BF16 && out_dtype != GG_OUT_FP16)) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  gg::silu_table_kernel<<<256, 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<float*>(table), out_dtype == GG_OUT_FP16 ? 1 : 0);
  return static_cast<int>(cudaGetLastError());
}

int gg_moe_gate_up(const void* x, const void* scale_x, const void* w1, const void* scale_w1,
                   const void* order, const void* offsets, const void* tile_expert,
                   const void* tile_row, int tile_capacity, int tile_rows, void* q, void* s,
                   void* gate_up_scratch, int tokens, int top_k, int experts, int hidden,
                   int intermediate, int interleaved, int out_dtype, int row_gather,
                   void* stream_ptr) {
  if (tokens <= 0 || top_k <= 0 || experts <= 0 || hidden <= 0 || intermediate <= 0 ||
      hidden % 256 || intermediate % 256 || tile_capacity <= 0 ||
      (out_dtype != GG_OUT_BF16 && out_dtype != GG_OUT_FP16) || !x || !scale_x || !w1 ||
      !scale_w1 || !order || !offsets || !tile_expert || !tile_row || !q || !s) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const long long slots = static_cast<long long>(tokens) * top_k;
  if (tile_rows == 128) {
    if (!gg::aligned16(x) || !gg::aligned16(w1) || !gg::aligned16(q) || !gate_up_scratch ||
        !gg::aligned16(gate_up_scratch)) {
      return static_cast<int>(cudaErrorInvalidValue);
    }
    uint8_t* scratch = static_cast<uint8_t*>(gate_up_scratch);
    gg::GateUpParams p = {};
    CUtensorMap map_x, map_w;
    int status;
    if (row_gather) {
      p.silu_table = reinterpret_cast<float*>(scratch);
      p.row_scale = static_cast<const float*>(scale_x);
      status = gg::encode_int8_rows(&map_x, x, tokens, hidden, hidden, 1);
    } else {
      // Activation rows and their scales in sorted-slot order first.
      int8_t* sorted_x = reinterpret_cast<int8_t*>(scratch);
      const size_t row_bytes = (static_cast<size_t>(slots) * hidden + 255) & ~static_cast<size_t>(255);
      float* sorted_scale = reinterpret_cast<float*>(scratch + row_bytes);
      const size_t scale_bytes =
          (static_cast<size_t>(slots) * (hidden / 256) * 4 + 255) & ~static_cast<size_t>(255);
      p.silu_table = reinterpret_cast<float*>(scratch + row_bytes + scale_bytes);
      p.row_scale = sorted_scale;
      const long long blocks = (slots + 7) / 8;
      const int limit = gg::sm_count() * 8;
      gg::gather_rows_kernel<<<static_cast<int>(blocks < limit ? blocks : limit), 256, 0, stream>>>(
          static_cast<const int8_t*>(x), static_cast<const float*>(scale_x),
          static_cast<const long long*>(order), static_cast<const int*>(offsets), experts, top_k,
          hidden, sorted_x, sorted_scale);
      const cudaError_t error = cudaGetLastError();
      if (error != cudaSuccess) return static_cast<int>(error);
      status = gg::encode_int8_rows(&map_x, sorted_x, slots, hidden, hidden, 128);
    }
    if (status) return status;
    status = gg_moe_silu_table(const_cast<float*>(p.silu_table), out_dtype, stream_ptr);
    if (status) return status;
    status = gg::encode_int8_rows(&map_w, w1, static_cast<long long>(experts) * 2 * intermediate,
                                  hidden, hidden, 128);
    if (status) return status;
    p.order = static_cast<const long long*>(order);
    p.top_k = top_k;
    p.scale_w = static_cast<const float*>(scale_w1);
    p.expert_offsets = static_cast<const int*>(offsets);
    p.tile_expert = static_cast<const int*>(tile_expert);
    p.tile_row = static_cast<const int*>(tile_row);
    p.q = static_cast<int8_t*>(q);
    p.s = static_cast<float*>(s);
    p.hidden = hidden; p.intermediate = intermediate;
    p.max_tiles = tile_capacity; p.interleaved = interleaved;
    const long long items = static_cast<long long>(tile_capacity) * (intermediate / 256);
    const int grid = static_cast<int>(items < gg::sm_count() ? items : gg::sm_count());
    if (row_gather) {
      if (out_dtype == GG_OUT_BF16) {
        return gg::launch_gate_up_tc<__nv_bfloat16, true>(map_x, map_w, p, grid, stream);
      }
      return gg::launch_gate_up_tc<__half, true>(map_x, map_w, p, grid, stream);
    }
    if (out_dtype == GG_OUT_BF16) {
      return gg::launch_gate_up_tc<__nv_bfloat16, false>(map_x, map_w, p, grid, stream);
    }
    return gg::launch_gate_up_tc<__half, false>(map_x, map_w, p, grid, stream);
  }
  if (tile_rows != gg::kSimtTile || !gate_up_scratch) return static_cast<int>(cudaErrorInvalidValue);
  // CUDA-core path: ragged gathered GEMM into the scratch matrix, then SwiGLU + requantisation.
  gg::GemmSimtParams p = {};
  p.a = static_cast<const int8_t*>(x);
  p.b = static_cast<const int8_t*>(w1);
  p.scale_a = static_cast<const float*>(scale_x);
  p.scale_b = static_cast<const float*>(scale_w1);
  p.c = gate_up_scratch;
  p.m = static_cast<int>(slots); p.n = 2 * intermediate; p.k = hidden;
  p.a_sm = hidden; p.a_sk = 1; p.b_sk = 1; p.b_sn = hidden;
  p.sa_sm = hidden / 256; p.sa_sg = 1; p.sb_sg = 2 * intermediate; p.sb_sn = 1;
  p.ldc = 2 * intermediate;
  p.group_size = 256;
  p.order = static_cast<const long long*>(order);
  p.top_k = top_k;
  p.expert_offsets = static_cast<const int*>(offsets);
  p.tile_expert = static_cast<const int*>(tile_expert);
  p.tile_row = static_cast<const int*>(tile_row);
  p.b_expert_stride = static_cast<long long>(2) * intermediate * hidden;
  p.sb_expert_stride = static_cast<long long>(hidden / 256) * 2 * intermediate;
  int status = gg::launch_simt_dtype<true>(p, tile_capacity, out_dtype, stream);
  if (status) return status;
  const long long items = slots * (intermediate / 256);
  const unsigned blocks = static_cast<unsigned>((items + 7) / 8);
  const int* valid = static_cast<const int*>(offsets) + experts;
  if (out_dtype == GG_OUT_BF16) {
    gg::swiglu_quantize_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(gate_up_scratch), slots, valid, intermediate, interleaved,
        static_cast<int8_t*>(q), static_cast<float*>(s));
  } else {
    gg::swiglu_quantize_kernel<__half><<<blocks, 256, 0, stream>>>(
        static_cast<const __half*>(gate_up_scratch), slots, valid, intermediate, interleaved,
        static_cast<int8_t*>(q), static_cast<float*>(s));
  }
  return static_cast<int>(cudaGetLastError());
}

int gg_moe_down(const void* q, const void* s, const void* w2, const void* scale_w2,
                const void* offsets, const void* tile_expert, const void* tile_row,
                int tile_capacity, int tile_rows, void* expert_out, const void* row_destination,
                int assignments, int experts, int hidden, int intermediate, int out_dtype,
                void* stream_ptr) {
  if (assignments <= 0 || experts <= 0 || hidden <= 0 || intermediate <= 0 || intermediate % 256 ||
      tile_capacity <= 0 || (out_dtype != GG_OUT_BF16 && out_dtype != GG_OUT_FP16) || !q || !s ||
      !w2 || !scale_w2 || !offsets || !tile_expert || !tile_row ||
      (!expert_out && !row_destination) || (row_destination && tile_rows != 128)) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (tile_rows == 128) {
    if (!gg::aligned16(q) || !gg::aligned16(w2) || !gg::aligned16(expert_out) || hidden % 8 ||
        !gg::aligned16(row_destination)) {
      return static_cast<int>(cudaErrorInvalidValue);
    }
    const unsigned long long* destinations = static_cast<const unsigned long long*>(row_destination);
    CUtensorMap map_a, map_b;
    int status = gg::encode_int8_rows(&map_a, q, assignments, intermediate, intermediate, 128);
    if (status) return status;
    const int bn = hidden >= 256 ? 256 : hidden >= 128 ? 128 : 64;
    status = gg::encode_int8_rows(&map_b, w2, static_cast<long long>(experts) * hidden, intermediate,
                                  intermediate, bn);
    if (status) return status;
    gg::GemmTcParams p = {};
    p.scale_a = static_cast<const float*>(s);
    p.scale_b = static_cast<const float*>(scale_w2);
    p.c = expert_out;
    p.m = assignments; p.n = hidden; p.k = intermediate;
    p.sa_sm = intermediate / 256; p.sa_sg = 1; p.sb_sg = hidden; p.sb_sn = 1;
    p.ldc = hidden;
    p.group_size = 256;
    p.k_splits = 1;
    p.band_rows = 8;
    p.tiles_m = tile_capacity;
    p.tiles_n = (hidden + bn - 1) / bn;
    p.c_vector_ok = 1;
    p.expert_offsets = static_cast<const int*>(offsets);
    p.tile_expert = static_cast<const int*>(tile_expert);
    p.tile_row = static_cast<const int*>(tile_row);
    p.b_rows_per_expert = hidden;
    p.sb_expert_stride = static_cast<long long>(intermediate / 256) * hidden;
    p.row_destination = destinations;
    if (bn == 256) return gg::launch_tc_dtype<1, 256, 4, true>(map_a, map_b, p, out_dtype, stream);
    if (bn == 128) return gg::launch_tc_dtype<1, 128, 6, true>(map_a, map_b, p, out_dtype, stream);
    return gg::launch_tc_dtype<1, 64, 8, true>(map_a, map_b, p, out_dtype, stream);
  }
  if (tile_rows != gg::kSimtTile) return static_cast<int>(cudaErrorInvalidValue);
  gg::GemmSimtParams p = {};
  p.a = static_cast<const int8_t*>(q);
  p.b = static_cast<const int8_t*>(w2);
  p.scale_a = static_cast<const float*>(s);
  p.scale_b = static_cast<const float*>(scale_w2);
  p.c = expert_out;
  p.m = assignments; p.n = hidden; p.k = intermediate;
  p.a_sm = intermediate; p.a_sk = 1; p.b_sk = 1; p.b_sn = intermediate;
  p.sa_sm = intermediate / 256; p.sa_sg = 1; p.sb_sg = hidden; p.sb_sn = 1;
  p.ldc = hidden;
  p.group_size = 256;
  p.expert_offsets = static_cast<const int*>(offsets);
  p.tile_expert = static_cast<const int*>(tile_expert);
  p.tile_row = static_cast<const int*>(tile_row);
  p.b_expert_stride = static_cast<long long>(hidden) * intermediate;
  p.sb_expert_stride = static_cast<long long>(intermediate / 256) * hidden;
  return gg::launch_simt_dtype<true>(p, tile_capacity, out_dtype, stream);
}

// ---------------------------------------------------------------- expert-parallel exchange

int gg_ep_plan(const void* ids, int ids_are_i64, const void* mask, int tokens, int top_k,
               int experts, int world, int local_experts, void* position, void* counts,
               void* home_inverse, void* stream_ptr) {
  if (tokens < 0 || top_k <= 0 || experts <= 0 || world <= 0 || world > 1024 ||
      local_experts <= 0 || static_cast<long long>(local_experts) * world != experts || !counts) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (tokens > 0 && (!ids || !position || !home_inverse)) return static_cast<int>(cudaErrorInvalidValue);
  gg::EpPlanParams p = {};
  p.ids = ids; p.ids_are_i64 = ids_are_i64;
  p.mask = static_cast<const uint8_t*>(mask);
  p.tokens = tokens; p.top_k = top_k; p.experts = experts; p.world = world;
  p.local_experts = local_experts;
  p.position = static_cast<int*>(position);
  p.counts = static_cast<int*>(counts);
  p.home_inverse = static_cast<int*>(home_inverse);
  gg::ep_plan_kernel<<<world, 1024, 0, static_cast<cudaStream_t>(stream_ptr)>>>(p);
  return static_cast<int>(cudaGetLastError());
}

int gg_ep_dispatch(const void* x, const void* scale_x, const void* ids, int ids_are_i64,
                   const void* mask, const void* position, int tokens, int top_k, int experts,
                   int world, int local_experts, int hidden, int rank, int capacity,
                   const void* recv_x, const void* recv_scale, const void* recv_ids,
                   const void* recv_src, void* error, void* stream_ptr) {
  if (tokens < 0 || top_k <= 0 || experts <= 0 || world <= 0 || local_experts <= 0 ||
      static_cast<long long>(local_experts) * world != experts || hidden <= 0 || hidden % 256 ||
      rank < 0 || rank >= world || capacity <= 0 || tokens > capacity || !recv_x || !recv_scale ||
      !recv_ids || !recv_src || !error) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (tokens == 0) return 0;
  if (!x || !scale_x || !ids || !position || !gg::aligned16(x)) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  gg::EpDispatchParams p = {};
  p.x = static_cast<const int8_t*>(x);
  p.scale_x = static_cast<const float*>(scale_x);
  p.ids = ids; p.ids_are_i64 = ids_are_i64;
  p.mask = static_cast<const uint8_t*>(mask);
  p.position = static_cast<const int*>(position);
  p.tokens = tokens; p.top_k = top_k; p.experts = experts; p.world = world;
  p.local_experts = local_experts; p.hidden = hidden; p.rank = rank; p.capacity = capacity;
  p.recv_x = static_cast<const unsigned long long*>(recv_x);
  p.recv_scale = static_cast<const unsigned long long*>(recv_scale);
  p.recv_ids = static_cast<const unsigned long long*>(recv_ids);
  p.recv_src = static_cast<const unsigned long long*>(recv_src);
  p.error = static_cast<int*>(error);
  const long long pairs = static_cast<long long>(tokens) * world;
  const long long blocks = (pairs + 7) / 8;
  const int limit = gg::sm_count() * 8;
  gg::ep_dispatch_kernel<<<static_cast<int>(blocks < limit ? blocks : limit), 256, 0,
                           static_cast<cudaStream_t>(stream_ptr)>>>(p);
  return static_cast<int>(cudaGetLastError());
}

int gg_ep_row_mask(const void* counts_all, int world, int rank, int capacity, void* row_mask,
                   void* stream_ptr) {
  if (!counts_all || !row_mask || world <= 0 || rank < 0 || rank >= world || capacity <= 0) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  const long long rows = static_cast<long long>(world) * capacity;
  const long long blocks = (rows + 255) / 256;
  const int limit = gg::sm_count() * 4;
  gg::ep_row_mask_kernel<<<static_cast<int>(blocks < limit ? blocks : limit), 256, 0,
                           static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<const int*>(counts_all), world, rank, capacity, static_cast<uint8_t*>(row_mask));
  return static_cast<int>(cudaGetLastError());
}

int gg_ep_row_destination(const void* order, const void* offsets, int experts, int top_k,
                          int capacity, int world, int hidden, int out_dtype, const void* recv_src,
                          const void* home_out, void* row_destination, void* error,
                          void* stream_ptr) {
  if (!order || !offsets || !recv_src || !home_out || !row_destination || !error || experts <= 0 ||
      top_k <= 0 || capacity <= 0 || world <= 0 || hidden <= 0 ||
      (out_dtype != GG_OUT_BF16 && out_dtype != GG_OUT_FP16)) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  const long long slots = static_cast<long long>(world) * capacity * top_k;
  const long long blocks = (slots + 255) / 256;
  const int limit = gg::sm_count() * 8;
  gg::ep_row_destination_kernel<<<static_cast<int>(blocks < limit ? blocks : limit), 256, 0,
                                  static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<const long long*>(order), static_cast<const int*>(offsets), experts, top_k,
      capacity, world, hidden, 2, static_cast<const int*>(recv_src),
      static_cast<const unsigned long long*>(home_out), slots,
      static_cast<unsigned long long*>(row_destination), static_cast<int*>(error));
  return static_cast<int>(cudaGetLastError());
}

// ---- peer-addressable device memory (set-up time, not on the hot path) -------------------

int gg_peer_alloc(size_t bytes, void** pointer) {
  if (!pointer || bytes == 0) return static_cast<int>(cudaErrorInvalidValue);
  void* memory = nullptr;
  cudaError_t error = cudaMalloc(&memory, bytes);
  if (error != cudaSuccess) return static_cast<int>(error);
  error = cudaMemset(memory, 0, bytes);
  if (error != cudaSuccess) {
    cudaFree(memory);
    return static_cast<int>(error);
  }
  *pointer = memory;
  return 0;
}

int gg_peer_free(void* pointer) { return static_cast<int>(cudaFree(pointer)); }

int gg_peer_export(void* pointer, void* handle) {
  if (!pointer || !handle) return static_cast<int>(cudaErrorInvalidValue);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
  return static_cast<int>(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle), pointer));
}

int gg_peer_import(const void* handle, void** pointer) {
  if (!handle || !pointer) return static_cast<int>(cudaErrorInvalidValue);
  cudaIpcMemHandle_t copy;
  memcpy(&copy, handle, sizeof(copy));
  return static_cast<int>(cudaIpcOpenMemHandle(pointer, copy, cudaIpcMemLazyEnablePeerAccess));
}

int gg_peer_release(void* pointer) { return static_cast<int>(cudaIpcCloseMemHandle(pointer)); }

int gg_moe_topk(const void* logits, int in_dtype, int tokens, int experts, int top_k, void* weights,
                void* ids, int ids_are_i64, void* stream_ptr) {
  if (tokens < 0 || experts <= 0 || experts > 1024 || top_k <= 0 || top_k > experts ||
      (in_dtype != GG_OUT_FP32 && in_dtype != GG_OUT_BF16 && in_dtype != GG_OUT_FP16)) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (tokens == 0) return 0;
  if (!logits || !weights || !ids) return static_cast<int>(cudaErrorInvalidValue);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const int grid = (tokens + 7) / 8;
  float* w = static_cast<float*>(weights);
  if (in_dtype == GG_OUT_FP32) {
    gg::router_topk_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(logits), tokens,
                                                             experts, top_k, w, ids, ids_are_i64);
  } else if (in_dtype == GG_OUT_BF16) {
    gg::router_topk_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(logits), tokens, experts, top_k, w, ids, ids_are_i64);
  } else {
    gg::router_topk_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(logits),
                                                              tokens, experts, top_k, w, ids,
                                                              ids_are_i64);
  }
  return static_cast<int>(cudaGetLastError());
}

int gg_moe_route_topk(const void* logits, int in_dtype, const void* mask, int tokens, int experts,
                      int top_k, void* weights, void* ids, int ids_are_i64, void* effective_ids,
                      void* order, void* inverse, void* counts, void* offsets, void* statistics,
                      void* stream_ptr) {
  const long long slots = static_cast<long long>(tokens) * top_k;
  if (tokens <= 0 || experts <= 0 || experts > 1024 || top_k <= 0 || top_k > experts ||
      slots > gg::kRouteChunk ||
      (in_dtype != GG_OUT_FP32 && in_dtype != GG_OUT_BF16 && in_dtype != GG_OUT_FP16) || !logits ||
      !weights || !ids || !effective_ids || !order || !inverse || !counts || !offsets || !statistics) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  gg::RouteParams p = {};
  p.ids = ids;
  p.ids_are_i64 = ids_are_i64;
  p.mask = static_cast<const uint8_t*>(mask);
  p.tokens = tokens; p.top_k = top_k; p.experts = experts;
  p.effective_ids = effective_ids;
  p.order = static_cast<long long*>(order);
  p.inverse = static_cast<int*>(inverse);
  p.counts = static_cast<int*>(counts);
  p.offsets = static_cast<int*>(offsets);
  p.statistics = static_cast<int*>(statistics);
  const size_t smem = static_cast<size_t>(experts + 2) * sizeof(int);
  float* w = static_cast<float*>(weights);
  if (in_dtype == GG_OUT_FP32) {
    gg::route_topk_single_kernel<float><<<1, gg::kRouteChunk, smem, stream>>>(
        static_cast<const float*>(logits), w, p);
  } else if (in_dtype == GG_OUT_BF16) {
    gg::route_topk_single_kernel<__nv_bfloat16><<<1, gg::kRouteChunk, smem, stream>>>(
        static_cast<const __nv_bfloat16*>(logits), w, p);
  } else {
    gg::route_topk_single_kernel<__half><<<1, gg::kRouteChunk, smem, stream>>>(
        static_cast<const __half*>(logits), w, p);
  }
  return static_cast<int>(cudaGetLastError());
}

int gg_quantize_rows(const void* x, int in_dtype, long long rows, int width, int group_size,
                     void* q, void* s, void* stream_ptr) {
  const bool group_ok = group_size == 32 || group_size == 64 || group_size == 128 || group_size == 256;
  if (rows < 0 || width <= 0 || width % 256 || !group_ok ||
      (in_dtype != GG_OUT_FP32 && in_dtype != GG_OUT_BF16 && in_dtype != GG_OUT_FP16)) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (rows == 0) return 0;
  if (!x || !q || !s || !gg::aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 7)) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const long long items = rows * (width / 256);
  const long long blocks = (items + 7) / 8;
  if (blocks > 0x7fffffffLL) return static_cast<int>(cudaErrorInvalidValue);
  const int grid = static_cast<int>(blocks);
  int8_t* codes = static_cast<int8_t*>(q);
  float* scales = static_cast<float*>(s);
  if (in_dtype == GG_OUT_FP32) {
    gg::quantize_rows_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(x), rows,
                                                               width, group_size, codes, scales);
  } else if (in_dtype == GG_OUT_BF16) {
    gg::quantize_rows_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), rows, width, group_size, codes, scales);
  } else {
    gg::quantize_rows_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(x), rows,
                                                                width, group_size, codes, scales);
  }
  return static_cast<int>(cudaGetLastError());
}

int gg_moe_combine(const void* expert_out, const void* weights, const void* inverse, void* out,
                   int tokens, int top_k, int hidden, int out_dtype, void* stream_ptr) {
  if (tokens < 0 || top_k <= 0 || hidden <= 0 || !weights || !inverse || !out ||
      (out_dtype != GG_OUT_BF16 && out_dtype != GG_OUT_FP16)) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (tokens == 0) return 0;
  if (!expert_out) return static_cast<int>(cudaErrorInvalidValue);
  // Rows move as 16-byte vectors when H is a multiple of 8 and both bases are aligned;
  // anything else takes the element-wise loop.
  const int vector_ok = hidden % 8 == 0 && gg::aligned16(expert_out) && gg::aligned16(out);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const size_t smem = static_cast<size_t>(top_k) * 8;
  if (smem > 48 * 1024) return static_cast<int>(cudaErrorInvalidValue);
  // Threads per token: the 16-byte chunks of a row spread evenly over whole passes
  // (H = 7168: 896 chunks, 4 passes of 224 threads instead of 3.5 of 256).
  const int chunks = (hidden + 7) / 8;
  const int passes = (chunks + 255) / 256;
  int threads = ((chunks + passes - 1) / passes + 31) / 32 * 32;
  if (threads > 256) threads = 256;
  if (threads < 32) threads = 32;
  if (out_dtype == GG_OUT_BF16) {
    gg::combine_kernel<__nv_bfloat16><<<tokens, threads, smem, stream>>>(
        static_cast<const __nv_bfloat16*>(expert_out), static_cast<const float*>(weights),
        static_cast<const int*>(inverse), static_cast<__nv_bfloat16*>(out), top_k, hidden, vector_ok);
  } else {
    gg::combine_kernel<__half><<<tokens, threads, smem, stream>>>(
        static_cast<const __half*>(expert_out), static_cast<const float*>(weights),
        static_cast<const int*>(inverse), static_cast<__half*>(out), top_k, hidden, vector_ok);
  }
  return static_cast<int>(cudaGetLastError());
}

int gg_report_to_host(const void* values, int count, void* host_words, void* stream_ptr) {
  if (count <= 0) return 0;
  if (count > 1024 || !values || !host_words) return static_cast<int>(cudaErrorInvalidValue);
  // The destination must be page-locked host memory the device can address; its device-side
  // address is asked for rather than assumed.
  void* mapped = nullptr;
  cudaError_t error = cudaHostGetDevicePointer(&mapped, host_words, 0);
  if (error != cudaSuccess) {
    (void)cudaGetLastError();
    return static_cast<int>(error);
  }
  gg::report_to_host_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<const int*>(values), count, static_cast<int*>(mapped));
  return static_cast<int>(cudaGetLastError());
}

int gg_selftest_wait_timeout(long long limit_ns, void* result, void* stream_ptr) {
  if (limit_ns <= 0 || limit_ns > 100000000ll || !result) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  gg::wait_timeout_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<unsigned long long>(limit_ns), static_cast<int*>(result));
  return static_cast<int>(cudaGetLastError());
}

int gg_device_status(int* status, void* stream_ptr) {
  if (!status) return static_cast<int>(cudaErrorInvalidValue);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  unsigned int words[4] = {0, 0, 0, 0};
  cudaError_t error = cudaMemcpyFromSymbolAsync(words, gg::g_device_status, sizeof(words), 0,
                                                cudaMemcpyDeviceToHost, stream);
  if (error != cudaSuccess) return static_cast<int>(error);
  error = cudaStreamSynchronize(stream);
  if (error != cudaSuccess) return static_cast<int>(error);
  *status = static_cast<int>(words[0]);
  if (words[0] != 0) {
    const unsigned int zeros[4] = {0, 0, 0, 0};
    error = cudaMemcpyToSymbolAsync(gg::g_device_status, zeros, sizeof(zeros), 0,
                                    cudaMemcpyHostToDevice, stream);
    if (error != cudaSuccess) return static_cast<int>(error);
    error = cudaStreamSynchronize(stream);
  }
  return static_cast<int>(error);
}

}  // extern "C"
