// W8A8 GEMM with per-row x per-column K-group FP32 scales on the 5th-generation tensor cores.
//
//   C[m,n] = cast( fold over groups g = 0..Q-1, in order, starting from 0:
//                  fmaf( float(sum_{k in g} A[m,k]*B[k,n]),  sa[m,g]*sb[g,n],  total ) )
//
// which is the arithmetic of the reference's portable kernel
// (src/grain_gemm/kernels/triton.py:28-51): exact INT32 group dot, the scale product rounded
// to FP32 once, one fused multiply-add per group, one final cast.
//
// Kernel shape (persistent, warp specialised, 384 threads):
//   producer    TMA warp: A tile [128 rows x 128 B of K] and B tile [BN/ctas rows x 128 B]
//               per stage, 128-byte swizzle, kStages-deep ring guarded by full/empty mbarriers.
//   warp 9      MMA issuer: tcgen05.mma kind::i8, K = 32 per instruction, INT32 accumulators in
//               TMEM, two accumulator buffers of BN columns.  The first MMA of every K group
//               overwrites the buffer, the last one commits it to the promotion warps.
//   scale warp  cp.async of each group's scale_b columns and scale_a rows into a shared-memory
//               ring, a whole ring ahead of the promotion warps
//   warps 0-7   promotion: drain the group's INT32 tile with tcgen05.ld in a matrix-fragment
//               layout (a thread owns 4 rows x 32 columns of its warp's 32 x 128 region),
//               multiply by sa*sb, add into FP32 registers while the tensor core works on the
//               next group; at the end of the tile cast, exchange inside quads and store.
// kCtaGroup == 2 pairs two CTAs (a 2-CTA cluster) on a 256 x BN tile: each CTA loads its own
// 128 rows of A and its own half of B, the leader CTA issues cta_group::2 MMAs that read both
// CTAs' shared memory and write both CTAs' TMEM.
//
// Any M and N (rows/columns beyond the edge are zero-filled by TMA and never stored), any
// K that is a multiple of 16 (TMA row pitch), G in {32, 64, 128, 256}; a partial last group
// is zero-filled by TMA and uses scale index Q-1.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "ptx.cuh"

namespace gg {

// Register split between the eight promotion warps and the four auxiliary warps (setmaxnreg).
#ifndef GG_PROMO_REGS
#define GG_PROMO_REGS 216
#endif
#ifndef GG_AUX_REGS
#define GG_AUX_REGS 64
#endif

struct GemmTcParams {
  const float* scale_a;
  const float* scale_b;
  void* c;
  int m, n, k;
  long long sa_sm, sa_sg, sb_sg, sb_sn;
  long long ldc;
  int group_size;
  int tiles_m, tiles_n;
  int c_vector_ok;   // rows of C start on 16-byte boundaries
  // Grouped (per-expert) mode, used by the MoE down projection; null for a plain GEMM.
  const int* expert_offsets;   // [E+1] first sorted slot of each expert
  const int* tile_expert;      // [tiles_m] expert of each row tile, -1 = unused
  const int* tile_row;         // [tiles_m] first row of each row tile
  long long b_rows_per_expert; // N (rows of the Linear weight per expert)
  long long sb_expert_stride;  // elements between experts in scale_b
  // Optional (grouped mode): device address of the first element of every output row.  When
  // set, row r is stored at row_destination[r] instead of c + r * ldc; the addresses may lie in
  // another GPU's memory (peer mapping), which is how the expert-parallel Down projection
  // returns each result row to the token's home rank while the GEMM is still running.
  const unsigned long long* row_destination;
  // Split-K dump mode: the K groups are divided over k_splits work items per output tile and
  // the INT32 group dots go to partials[Q][M][N] instead of being promoted (a second kernel
  // then folds them in group order).  k_splits == 1 and partials == null otherwise.
  int band_rows;               // row tiles per scheduling band
  int k_splits;
  int groups_per_split;
  int* partials;
};

// K range of one work item (the whole K unless split-K is on).
struct TileWork {
  int tm, tn;
  int group_begin, groups;   // K groups [group_begin, group_begin + groups)
  int k_begin;               // first K element (a multiple of 128)
  int ksteps, slabs;         // MMAs (K = 32) and 128-byte slabs in the range
  bool whole_g256;           // G = 256 and the range is whole groups: fast issue path
};

template <int kCtaGroup, int BN, int kStages, int kPromoWarps = 8, int kARows = 128>
struct GemmTcShape {
  static constexpr int kBM = 128;                       // rows per CTA
  static constexpr int kBK = 128;                       // bytes of K per stage
  static constexpr int kBRows = BN / kCtaGroup;         // B rows loaded by each CTA
  // Rows of A actually fetched per stage.  Skinny problems (M <= kARows) fetch only that many:
  // the MMA still reads 128 rows, the rest being whatever follows in the stage (the B tile),
  // which only feeds accumulator rows that are never stored.
  static constexpr int kABytes = kARows * kBK;
  static_assert(kARows % 8 == 0 && kARows <= 128 && (kARows == 128 || kBRows >= 128),
                "a short A tile needs the B tile behind it to cover the 128 rows the MMA reads");
  static constexpr int kBBytes = kBRows * kBK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemColumns = 2 * BN;
  // Ring of per-group scale vectors (the short-A shape is the split-K dump kernel, which
  // stages no scales and needs the room for its operand stages).
  static constexpr int kScaleSlots = kARows == 128 ? 8 : 4;
  static constexpr int kScaleSlotFloats = BN + 128;     // scale_b columns, then scale_a rows
  static constexpr int kScaleBytes = kScaleSlots * kScaleSlotFloats * 4;
  static constexpr int kBarrierBytes = (2 * kStages + 4 + 2 * kScaleSlots) * 8 + 16;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kScaleBytes + kBarrierBytes;
  static constexpr int kThreads = (kPromoWarps + 4) * 32;   // + producer, MMA, two spares
  static constexpr int kColumnsPerThread = BN / (kPromoWarps / 4);
  static constexpr int kDrainWidth = kPromoWarps == 16 ? 16 : 32;  // columns per tcgen05.ld
  static constexpr int kPromoRegisters = kPromoWarps == 16 ? 104 : GG_PROMO_REGS;
  static constexpr int kAuxRegisters = kPromoWarps == 16 ? 48 : GG_AUX_REGS;
  // setmaxnreg can only hand the promotion warps registers that the four other warps of the
  // same CTA released: (promo - launch) * promo threads <= (launch - aux) * 128, where launch
  // is the per-thread count the kernel starts with under its launch bound.
  static constexpr int kLaunchRegisters = kPromoWarps == 16 ? 96 : 168;
  static_assert((kPromoRegisters - kLaunchRegisters) * kPromoWarps * 32 <=
                    (kLaunchRegisters - kAuxRegisters) * 128,
                "register reallocation exceeds what the auxiliary warps release");
  static_assert(kPromoWarps == 8 || kPromoWarps == 16, "promotion warps come in groups of four");
  static_assert(kColumnsPerThread % kDrainWidth == 0, "tile too narrow for the warp count");
  static_assert(BN == 64 || BN == 128 || BN == 256, "unsupported tile width");
};

__device__ __forceinline__ void tile_coordinates(int tile, int tiles_m, int tiles_n, int& tm,
                                                 int& tn, int band_rows = 8) {
  // Bands of row tiles: consecutive CTAs share B columns and a few A rows in L2.
  const int band_size = band_rows * tiles_n;
  const int band = tile / band_size;
  const int first_m = band * band_rows;
  const int band_m = min(tiles_m - first_m, band_rows);
  const int local = tile - band * band_size;
  tm = first_m + local % band_m;
  tn = local / band_m;
}

__device__ __forceinline__ TileWork decode_tile(const GemmTcParams& p, int tile, int tiles_m) {
  TileWork w;
  int split = 0;
  if (p.k_splits > 1) {
    const int per_split = tiles_m * p.tiles_n;
    split = tile / per_split;
    tile -= split * per_split;
  }
  tile_coordinates(tile, tiles_m, p.tiles_n, w.tm, w.tn, p.band_rows);
  const int total_groups = (p.k + p.group_size - 1) / p.group_size;
  w.group_begin = split * p.groups_per_split;
  const int group_end = p.k_splits > 1 ? min(total_groups, w.group_begin + p.groups_per_split)
                                       : total_groups;
  w.groups = group_end - w.group_begin;
  w.k_begin = w.group_begin * p.group_size;
  const int k_length = min(p.k, group_end * p.group_size) - w.k_begin;
  w.ksteps = (k_length + 31) / 32;
  w.slabs = (k_length + 127) / 128;
  w.whole_g256 = p.group_size == 256 && (k_length & 255) == 0;
  return w;
}

// TMEM drain layouts.  A promotion warp reads its 32 lanes x 32 columns of a block as two
// fragments of 16 lanes; with r = lane / 4 and q = lane % 4 a thread receives rows r, r + 8
// (and r + 16, r + 24 from the second fragment) and eight columns of the block:
//   kFragmentPairs (tcgen05.ld.16x256b.x4): the pairs 8j + 2q, 8j + 2q + 1   (j = 0..3)
//   kFragmentQuads (tcgen05.ld.16x128b.x8): the columns 4k + q               (k = 0..7)
// Both need the same scales per thread (4 row scales, 8 column scales per block), far fewer
// than the row-per-thread 32x32b shape, whose broadcast scale loads saturate the shared-memory
// return path.  Measured on B200 with eight warps draining 128 lanes x 256 columns: 16x256b
// delivers 256 B/clk/SM, 16x128b 507 B/clk/SM (32x32b 940 B/clk/SM), so the quad layout halves
// the time the drain keeps TMEM's read port busy.
enum FragmentLayout { kFragmentPairs = 0, kFragmentQuads = 1 };

// The accumulator pair j (j = 0..3) of a thread holds the block's columns
//   pairs layout: 8j + 2q, 8j + 2q + 1        quads layout: 8j + q, 8j + 4 + q.
// Position of block column `c` (0..31) in the scale ring: thread q reads its eight column
// scales, in accumulator-pair order, as two 16-byte vectors at q * 8.
template <FragmentLayout kLayout>
__device__ __forceinline__ int ring_column_position(int c) {
  if constexpr (kLayout == kFragmentPairs) return ((c >> 1) & 3) * 8 + (c >> 3) * 2 + (c & 1);
  else return (c & 3) * 8 + (c >> 3) * 2 + ((c >> 2) & 1);
}
// Position of row `r` (0..31 within its warp's 32 rows): the thread with row index
// lane / 4 = r % 8 reads its four rows r % 8 + 8j as one 16-byte vector.
__device__ __forceinline__ int ring_row_position(int r) { return (r & 7) * 4 + (r >> 3); }

// The eight column scales (four pairs) of this thread for one 32-column block.
__device__ __forceinline__ void load_column_scales(const float* block_base, int quad,
                                                   float2 (&sb)[4]) {
  const uint32_t address = smem_u32(block_base + quad * 8);
  const float4 lo = lds_f32x4(address);
  const float4 hi = lds_f32x4(address + 16);
  sb[0] = make_float2(lo.x, lo.y);
  sb[1] = make_float2(lo.z, lo.w);
  sb[2] = make_float2(hi.x, hi.y);
  sb[3] = make_float2(hi.z, hi.w);
}
// The four row scales of this thread (rows fragment_row + 8j of the warp's 32 rows), each
// doubled into the register pair the packed multiply takes; built once per K group.
__device__ __forceinline__ void load_row_scales(const float* warp_rows_base, int fragment_row,
                                                float2 (&sa)[4]) {
  const float4 v = lds_f32x4(smem_u32(warp_rows_base + fragment_row * 4));
  sa[0] = make_float2(v.x, v.x);
  sa[1] = make_float2(v.y, v.y);
  sa[2] = make_float2(v.z, v.z);
  sa[3] = make_float2(v.w, v.w);
}

template <FragmentLayout kLayout>
__device__ __forceinline__ void tmem_ld_fragment(uint32_t taddr, uint32_t (&r)[16]) {
  if constexpr (kLayout == kFragmentPairs) tmem_ld_16x256b_x4(taddr, r);
  else tmem_ld_16x128b_x8(taddr, r);
}

// Promotion of one 16-row x 32-column fragment: this thread holds rows r ("low") and r + 8
// ("high") and four column pairs; `sb` are the scales of those pairs, read once per 32-column
// block and used for both 16-row fragments.  Registers: pairs layout 4j + {0,1} = low pair j,
// 4j + {2,3} = high pair j; quads layout 4j + {0,2} = low pair j, 4j + {1,3} = high pair j.
template <FragmentLayout kLayout>
__device__ __forceinline__ void promote_fragment(const uint32_t (&partial)[16], float2 sa_low2,
                                                 float2 sa_high2, const float2 (&sb)[4],
                                                 float2* acc_low, float2* acc_high) {
  constexpr int kLowY = kLayout == kFragmentPairs ? 1 : 2;
  constexpr int kHighX = kLayout == kFragmentPairs ? 2 : 1;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 low = make_float2(__int2float_rn(static_cast<int>(partial[4 * j + 0])),
                                   __int2float_rn(static_cast<int>(partial[4 * j + kLowY])));
    const float2 high = make_float2(__int2float_rn(static_cast<int>(partial[4 * j + kHighX])),
                                    __int2float_rn(static_cast<int>(partial[4 * j + 3])));
    acc_low[j] = __ffma2_rn(low, __fmul2_rn(sa_low2, sb[j]), acc_low[j]);
    acc_high[j] = __ffma2_rn(high, __fmul2_rn(sa_high2, sb[j]), acc_high[j]);
  }
}

// Two outputs as one 32-bit word, the first in the low half.
template <typename OutT>
__device__ __forceinline__ uint32_t pack_pair(float2 v) {
  if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
    const __nv_bfloat162 packed = __floats2bfloat162_rn(v.x, v.y);
    return *reinterpret_cast<const uint32_t*>(&packed);
  } else {
    const __half2 packed = __floats2half2_rn(v.x, v.y);
    return *reinterpret_cast<const uint32_t*>(&packed);
  }
}

// 4x4 transpose inside every quad of lanes: lane q (= lane & 3) enters with its words
// w[0..3] and leaves with word q of lanes 0, 1, 2, 3 of its quad, in that order.
__device__ __forceinline__ void quad_transpose(uint32_t (&w)[4], int q) {
  const bool odd = (q & 1) != 0;
  uint32_t s0 = odd ? w[0] : w[1];
  uint32_t s1 = odd ? w[2] : w[3];
  s0 = __shfl_xor_sync(0xffffffffu, s0, 1);
  s1 = __shfl_xor_sync(0xffffffffu, s1, 1);
  if (odd) { w[0] = s0; w[2] = s1; } else { w[1] = s0; w[3] = s1; }
  const bool upper = (q & 2) != 0;
  uint32_t t0 = upper ? w[0] : w[2];
  uint32_t t1 = upper ? w[1] : w[3];
  t0 = __shfl_xor_sync(0xffffffffu, t0, 2);
  t1 = __shfl_xor_sync(0xffffffffu, t1, 2);
  if (upper) { w[0] = t0; w[1] = t1; } else { w[2] = t0; w[3] = t1; }
}

template <int kCtaGroup, int BN, int kStages, typename OutT, bool kGrouped, int kPromoWarps,
          bool kDump = false, int kARows = 128>
__global__ void __launch_bounds__((kPromoWarps + 4) * 32, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const GemmTcParams p) {
  using Shape = GemmTcShape<kCtaGroup, BN, kStages, kPromoWarps, kARows>;
  constexpr int kNC = Shape::kColumnsPerThread;   // columns owned by one promotion thread
  constexpr int kProducerWarp = kPromoWarps, kMmaWarp = kPromoWarps + 1;
  constexpr int kScaleWarp = kPromoWarps + 2;
  constexpr FragmentLayout kLayout = kFragmentQuads;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stage_base = smem;
  float* scale_ring = reinterpret_cast<float*>(smem + kStages * Shape::kStageBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * Shape::kStageBytes +
                                                   Shape::kScaleBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full_bar = empty_bar + kStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint64_t* scale_full_bar = tmem_empty_bar + 2;
  uint64_t* scale_empty_bar = scale_full_bar + Shape::kScaleSlots;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(scale_empty_bar + Shape::kScaleSlots);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = kCtaGroup == 2 ? cluster_ctarank() : 0u;
  const int worker = blockIdx.x / kCtaGroup;
  const int workers = gridDim.x / kCtaGroup;
  // (total_tiles follows the set-up below: the grouped kernel first finds how many row tiles
  // of its list are in use.)
  const int steps_per_group = p.group_size / 32;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full_bar[i], 1);
      mbar_init(&tmem_empty_bar[i], kPromoWarps * kCtaGroup);
    }
    for (int i = 0; i < Shape::kScaleSlots; ++i) {
      mbar_init(&scale_full_bar[i], 32);            // every lane of the scale warp
      mbar_init(&scale_empty_bar[i], kPromoWarps);  // one arrival per promotion warp
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  // Grouped problems: the row-tile list has room for the worst case and its used entries come
  // first; the kernel walks only those.  (An expert-parallel rank's list is sized for every
  // row it could receive, several times what it does receive.)
  __shared__ int used_row_tiles;
  if constexpr (kGrouped) {
    if (threadIdx.x == 32) {
      int low = 0, high = p.tiles_m;
      while (low < high) {
        const int middle = (low + high) >> 1;
        if (p.tile_expert[middle] >= 0) low = middle + 1;
        else high = middle;
      }
      used_row_tiles = low;
    }
  }
  if constexpr (kCtaGroup == 2) cluster_sync_all();
  if (warp == kMmaWarp) tmem_alloc<kCtaGroup>(tmem_holder, Shape::kTmemColumns);
  tcgen05_fence_before();
  __syncthreads();
  if constexpr (kCtaGroup == 2) cluster_sync_all();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  int tiles_m = p.tiles_m;
  if constexpr (kGrouped) tiles_m = used_row_tiles;
  const int total_tiles = tiles_m * p.tiles_n * p.k_splits;
  // The last four warps (producer, MMA issuer, two spares) give registers to the promotion warps.
  if (warp >= kPromoWarps) {
  setmaxnreg_dec<Shape::kAuxRegisters>();
  if (warp == kProducerWarp) {
    // ------------------------------------------------------------ TMA producer
    // The whole warp walks the ring (see mbar_wait_warp); one elected lane issues the copies.
    const bool leader = elect_one();
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (int tile = worker; tile < total_tiles && ok; tile += workers) {
      const TileWork work = decode_tile(p, tile, tiles_m);
      const int tm = work.tm, tn = work.tn;
      int row_a, row_b;
      if constexpr (kGrouped) {
        const int expert = p.tile_expert[tm];
        if (expert < 0) continue;
        row_a = p.tile_row[tm] + static_cast<int>(cta_rank) * Shape::kBM;
        row_b = expert * static_cast<int>(p.b_rows_per_expert) + tn * BN +
                static_cast<int>(cta_rank) * Shape::kBRows;
      } else {
        row_a = (tm * kCtaGroup + static_cast<int>(cta_rank)) * Shape::kBM;
        row_b = tn * BN + static_cast<int>(cta_rank) * Shape::kBRows;
      }
      for (int slab = 0, x = work.k_begin; slab < work.slabs; ++slab, x += Shape::kBK) {
        if (!mbar_wait_warp(&empty_bar[stage], phase ^ 1u, kSiteProducerEmpty, abort_flag)) {
          ok = false;
          break;
        }
        if (leader) {
          uint8_t* a_dst = stage_base + stage * Shape::kStageBytes;
          uint8_t* b_dst = a_dst + Shape::kABytes;
          if constexpr (kCtaGroup == 1) {
            mbar_expect_tx(&full_bar[stage], Shape::kStageBytes);
            tma_load_2d(a_dst, &map_a, &full_bar[stage], x, row_a);
            tma_load_2d(b_dst, &map_b, &full_bar[stage], x, row_b);
          } else {
            if (cta_rank == 0) mbar_expect_tx(&full_bar[stage], 2 * Shape::kStageBytes);
            tma_load_2d_pair(a_dst, &map_a, &full_bar[stage], x, row_a);
            tma_load_2d_pair(b_dst, &map_b, &full_bar[stage], x, row_b);
          }
        }
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issuer
    // The warp of the pair's leader CTA walks the loop converged; one elected lane issues every
    // MMA and commit.  (A loop run by a single lane of a diverged warp has to move each
    // descriptor into uniform registers per instruction and issues about a third slower.)
    if (cta_rank == 0) {
      const bool leader = elect_one();
      constexpr uint32_t idesc = make_idesc_i8(Shape::kBM * kCtaGroup, BN);
      const uint32_t a_low_base = smem_desc_low(smem_u32(stage_base));
      uint32_t stage = 0, phase = 0;                 // shared-memory ring position
      uint32_t buffer = 0, empty_parity = 1;         // TMEM ring position
      int step = 0;                                  // MMAs issued into the open group
      bool ok = true;
      for (int tile = worker; tile < total_tiles && ok; tile += workers) {
        const TileWork work = decode_tile(p, tile, tiles_m);
        if constexpr (kGrouped) {
          if (p.tile_expert[work.tm] < 0) continue;
        }
        if (work.whole_g256) {
          // G = 256 with whole groups: two slabs per group, no per-MMA bookkeeping.
          for (int slab = 0; slab < work.slabs; ++slab) {
            if (!mbar_wait_warp(&full_bar[stage], phase, kSiteMmaFull, abort_flag)) {
              ok = false;
              break;
            }
            tcgen05_fence_after();
            const bool group_start = (slab & 1) == 0;
            if (group_start) {
              if (!mbar_wait_warp(&tmem_empty_bar[buffer], empty_parity, kSiteMmaTmemEmpty,
                                  abort_flag)) {
                ok = false;
                break;
              }
              tcgen05_fence_after();
            }
            const uint32_t a_low = a_low_base + stage * (Shape::kStageBytes >> 4);
            const uint32_t b_low = a_low + (Shape::kABytes >> 4);
            const uint32_t tmem_d = tmem_base + buffer * BN;
            if (leader) {
              umma_i8<kCtaGroup>(tmem_d, a_low, b_low, idesc, group_start ? 0u : 1u);
              umma_i8<kCtaGroup>(tmem_d, a_low + 2, b_low + 2, idesc, 1u);
              umma_i8<kCtaGroup>(tmem_d, a_low + 4, b_low + 4, idesc, 1u);
              umma_i8<kCtaGroup>(tmem_d, a_low + 6, b_low + 6, idesc, 1u);
              if constexpr (kCtaGroup == 1) umma_commit(&empty_bar[stage]);
              else umma_commit_pair(&empty_bar[stage], 3);
              if (!group_start) {
                if constexpr (kCtaGroup == 1) umma_commit(&tmem_full_bar[buffer]);
                else umma_commit_pair(&tmem_full_bar[buffer], 3);
              }
            }
            if (!group_start) {
              buffer ^= 1u;
              if (buffer == 0) empty_parity ^= 1u;
            }
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          continue;
        }
        int remaining = work.ksteps;
        for (int slab = 0; slab < work.slabs && ok; ++slab) {
          if (!mbar_wait_warp(&full_bar[stage], phase, kSiteMmaFull, abort_flag)) {
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t a_low = a_low_base + stage * (Shape::kStageBytes >> 4);
          const uint32_t b_low = a_low + (Shape::kABytes >> 4);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (remaining > 0) {
              if (step == 0) {
                if (!mbar_wait_warp(&tmem_empty_bar[buffer], empty_parity, kSiteMmaTmemEmpty,
                                    abort_flag)) {
                  ok = false;
                  break;
                }
                tcgen05_fence_after();
              }
              if (leader) {
                umma_i8<kCtaGroup>(tmem_base + buffer * BN, a_low + 2 * j, b_low + 2 * j, idesc,
                                   step != 0 ? 1u : 0u);
              }
              ++step;
              --remaining;
              if (step == steps_per_group || remaining == 0) {
                if (leader) {
                  if constexpr (kCtaGroup == 1) umma_commit(&tmem_full_bar[buffer]);
                  else umma_commit_pair(&tmem_full_bar[buffer], 3);
                }
                step = 0;
                buffer ^= 1u;
                if (buffer == 0) empty_parity ^= 1u;
              }
            }
          }
          if (leader && ok) {
            if constexpr (kCtaGroup == 1) umma_commit(&empty_bar[stage]);
            else umma_commit_pair(&empty_bar[stage], 3);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == kScaleWarp && !kDump) {
    // ------------------------------------------------------------ scale staging warp
    // Copies each group's scale_b columns and scale_a rows into a shared-memory ring with
    // asynchronous 4-byte copies (cp.async) that land directly in the order the promotion
    // threads read; each lane's copies signal the slot's barrier when they have arrived.
    // Nothing passes through registers, so the warp runs a whole ring ahead of the promotion
    // warps and a global-memory latency of several K groups stays hidden (a version that
    // held one group in registers left the promotion warps waiting for scales).
    constexpr int kColumnsPerLane = BN / 32;
    uint32_t slot = 0, phase = 0;
    bool ok = true;
    for (int tile = worker; tile < total_tiles && ok; tile += workers) {
      const TileWork work = decode_tile(p, tile, tiles_m);
      int row0, row_limit;
      const float* sb_base = p.scale_b;
      if constexpr (kGrouped) {
        const int expert = p.tile_expert[work.tm];
        if (expert < 0) continue;
        row0 = p.tile_row[work.tm] + static_cast<int>(cta_rank) * Shape::kBM;
        row_limit = p.expert_offsets[expert + 1];
        sb_base += static_cast<long long>(expert) * p.sb_expert_stride;
      } else {
        row0 = (work.tm * kCtaGroup + static_cast<int>(cta_rank)) * Shape::kBM;
        row_limit = p.m;
      }
      const int n0 = work.tn * BN;
      // Per-lane sources and destinations do not change within the tile.
      const float* sb_source[kColumnsPerLane];
      const float* sa_source[4];
      bool sb_valid[kColumnsPerLane], sa_valid[4];
#pragma unroll
      for (int i = 0; i < kColumnsPerLane; ++i) {
        const int col = n0 + lane + 32 * i;
        sb_valid[i] = col < p.n;
        sb_source[i] = sb_base + (sb_valid[i] ? col * p.sb_sn : 0);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = row0 + lane + 32 * i;
        sa_valid[i] = r < row_limit;
        sa_source[i] = p.scale_a + (sa_valid[i] ? r * p.sa_sm : 0);
      }
      const int column_position = ring_column_position<kLayout>(lane);
      const int row_position = ring_row_position(lane);
      for (int g = 0; g < work.groups; ++g) {
        const bool got = mbar_test(&scale_empty_bar[slot], phase ^ 1u) ||
                         mbar_wait(&scale_empty_bar[slot], phase ^ 1u, kSiteScaleEmpty, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          ok = false;
          break;
        }
        const long long group = work.group_begin + g;
        float* destination = scale_ring + slot * Shape::kScaleSlotFloats;
#pragma unroll
        for (int i = 0; i < kColumnsPerLane; ++i) {
          cp_async_f32(destination + 32 * i + column_position, sb_source[i] + group * p.sb_sg,
                       sb_valid[i]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          cp_async_f32(destination + BN + 32 * i + row_position, sa_source[i] + group * p.sa_sg,
                       sa_valid[i]);
        }
        cp_async_arrive(&scale_full_bar[slot]);
        if (++slot == Shape::kScaleSlots) {
          slot = 0;
          phase ^= 1u;
        }
      }
    }
    cp_async_wait_all();
  }
  } else {
    setmaxnreg_inc<Shape::kPromoRegisters>();
    // ------------------------------------------------------------ promotion warps
    const int half = warp >> 2;           // which slice of the BN columns
    const int quarter = warp & 3;         // TMEM lane quarter this warp may read
    const int row_in_cta = quarter * 32 + lane;
    const int col_base = half * kNC;
    uint32_t group_sequence = 0;
    uint32_t scale_slot = 0, scale_phase = 0;
    bool ok = true;
    OutT* c = reinterpret_cast<OutT*>(p.c);
    // A failed wait clears `ok` but the loops keep their shape, so that every thread still
    // reaches every named barrier the others wait on.
    for (int tile = worker; tile < total_tiles; tile += workers) {
      const TileWork work = decode_tile(p, tile, tiles_m);
      const int tm = work.tm, tn = work.tn;
      const int groups = work.groups;
      int row, row_limit;
      const float* sb_base = p.scale_b;
      if constexpr (kGrouped) {
        const int expert = p.tile_expert[tm];
        if (expert < 0) continue;
        row = p.tile_row[tm] + static_cast<int>(cta_rank) * Shape::kBM + row_in_cta;
        row_limit = p.expert_offsets[expert + 1];
        sb_base += static_cast<long long>(expert) * p.sb_expert_stride;
      } else {
        row = (tm * kCtaGroup + static_cast<int>(cta_rank)) * Shape::kBM + row_in_cta;
        row_limit = p.m;
      }
      const int n0 = tn * BN;
      const bool row_ok = row < row_limit;
      // Rows of this warp: 32 consecutive ones of the tile, the same for every lane.
      const bool warp_has_rows = row - row_in_cta + quarter * 32 < row_limit;
      if constexpr (kDump) {
        // Split-K: hand the exact INT32 group dots to the folding kernel.
        for (int g = 0; g < groups; ++g, ++group_sequence) {
          const uint32_t buffer = group_sequence & 1u;
          if (ok) {
            ok = mbar_wait_warp(&tmem_full_bar[buffer], (group_sequence >> 1) & 1u,
                                kSiteEpilogueTmemFull, abort_flag);
          }
          tcgen05_fence_after();
          const uint32_t taddr =
              tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buffer * BN + col_base;
          int* destination = p.partials +
                             (static_cast<long long>(work.group_begin + g) * p.m + row) * p.n + n0 +
                             col_base;
          // Rows at or beyond M hold zero-filled operands; a warp whose 32 rows are all
          // beyond M skips the drain altogether.
          if (ok && warp_has_rows) {
#pragma unroll
            for (int chunk = 0; chunk < kNC / 32; ++chunk) {
              uint32_t partial[32];
              tmem_ld_32x32b_x32(taddr + chunk * 32, partial);
              tmem_ld_wait();
              if (row_ok) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                  const int col = n0 + col_base + chunk * 32 + j;
                  if (col + 4 <= p.n && (p.n & 3) == 0) {
                    *reinterpret_cast<uint4*>(destination + chunk * 32 + j) =
                        make_uint4(partial[j], partial[j + 1], partial[j + 2], partial[j + 3]);
                  } else {
                    for (int i = 0; i < 4; ++i) {
                      if (col + i < p.n) destination[chunk * 32 + j + i] = static_cast<int>(partial[j + i]);
                    }
                  }
                }
              }
            }
          }
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty_bar[buffer]);
        }
        continue;
      }
      // Fragment layout: this thread owns rows (lane / 4) + 8 * s, s = 0..3, of its warp's 32
      // rows, and in every 8-column group the two columns 2 * (lane % 4), +1.
      constexpr int kBlocks = kNC / 32;          // 32-column blocks in this warp's columns
      constexpr int kPairs = kNC / 8;            // column pairs per owned row
      float2 acc[4][kPairs];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
#pragma unroll
        for (int i = 0; i < kPairs; ++i) acc[r][i] = make_float2(0.0f, 0.0f);
      }
      static_assert(!kDump || kCtaGroup == 1, "split-K dump runs on single CTAs");
      const int fragment_row = lane >> 2;

      // `ok` is the same in every lane (mbar_wait_warp votes), so the .sync.aligned TMEM
      // instructions below always see a converged warp, also after a wait has run out.
      for (int g = 0; g < groups; ++g, ++group_sequence) {
        // This group's scales, staged by the scale warp.
        if (ok) {
          ok = mbar_wait_warp(&scale_full_bar[scale_slot], scale_phase, kSiteScaleFull, abort_flag);
        }
        const float* scale_slot_base = scale_ring + scale_slot * Shape::kScaleSlotFloats;
        float2 sa[4];
        load_row_scales(scale_slot_base + BN + quarter * 32, fragment_row, sa);
        const uint32_t buffer = group_sequence & 1u;
        if (ok) {
          ok = mbar_wait_warp(&tmem_full_bar[buffer], (group_sequence >> 1) & 1u,
                              kSiteEpilogueTmemFull, abort_flag);
        }
        tcgen05_fence_after();
        const float* sb_columns = scale_slot_base + col_base;
        const uint32_t taddr_low =
            tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buffer * BN + col_base;
        const uint32_t taddr_high = taddr_low + (16u << 16);
        // Fragments alternate between the two 16-row halves of each 32-column block; the load
        // of the next fragment is in flight while the current one is promoted.
        uint32_t partial_a[16], partial_b[16];
        float2 sb[4];
        if (ok && !warp_has_rows) {
          // None of this warp's 32 rows exists (a skinny problem, the ragged end of an expert):
          // nothing to promote, the buffer goes straight back.
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (kCtaGroup == 1) mbar_arrive(&tmem_empty_bar[buffer]);
            else mbar_arrive_cluster(&tmem_empty_bar[buffer], 0);
          }
        } else if (ok) {
          tmem_ld_fragment<kLayout>(taddr_low, partial_a);
#pragma unroll
          for (int fragment = 0; fragment < 2 * kBlocks; ++fragment) {
            const int block = fragment >> 1;
            const int high_half = fragment & 1;
            if (!high_half) load_column_scales(sb_columns + block * 32, lane & 3, sb);
            tmem_ld_wait();
            if (fragment + 1 < 2 * kBlocks) {
              const uint32_t next = ((fragment + 1) & 1 ? taddr_high : taddr_low) +
                                    ((fragment + 1) >> 1) * 32;
              if (fragment & 1) tmem_ld_fragment<kLayout>(next, partial_a);
              else tmem_ld_fragment<kLayout>(next, partial_b);
            } else {
              // All of this warp's TMEM accesses for the buffer are done: hand it back.
              tcgen05_fence_before();
              __syncwarp();
              if (lane == 0) {
                if constexpr (kCtaGroup == 1) mbar_arrive(&tmem_empty_bar[buffer]);
                else mbar_arrive_cluster(&tmem_empty_bar[buffer], 0);
              }
            }
            if (fragment & 1) {
              promote_fragment<kLayout>(partial_b, sa[2], sa[3], sb, &acc[2][block * 4],
                                      &acc[3][block * 4]);
            } else {
              promote_fragment<kLayout>(partial_a, sa[0], sa[1], sb, &acc[0][block * 4],
                                      &acc[1][block * 4]);
            }
          }
        }
        // Every lane has consumed the slot's values (they fed the arithmetic above).
        __syncwarp();
        if (lane == 0) mbar_arrive(&scale_empty_bar[scale_slot]);
        if (++scale_slot == Shape::kScaleSlots) {
          scale_slot = 0;
          scale_phase ^= 1u;
        }
      }
      // The fragment layout leaves each lane with columns spread over the block.  A 4x4
      // exchange inside every quad gives lane q the eight consecutive columns 8q..8q+7 of each
      // 32-column block (after it, accumulator pair i of the quads layout holds columns
      // 8q + i and 8q + 4 + i), so that a row leaves as 16-byte stores: a quarter of the store
      // instructions and of the memory-pipe wavefronts of pair stores.
      if (ok) {
        const int quad = lane & 3;
        const int first_row = row - row_in_cta + quarter * 32 + fragment_row;
        const bool aligned = p.c_vector_ok != 0;
        // Destination addresses of this thread's four rows and of the four rows of the lane it
        // exchanges with, fetched in one batch before the first store: a load issued between
        // the stores would wait behind them (the compiler must assume they alias), one round
        // trip per row instead of one per tile.
        [[maybe_unused]] unsigned long long own_destination[4] = {0ull, 0ull, 0ull, 0ull};
        [[maybe_unused]] unsigned long long other_destination[4] = {0ull, 0ull, 0ull, 0ull};
        if constexpr (kGrouped) {
          if (p.row_destination != nullptr) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              const int out_row = first_row + 8 * r;
              const int partner_row = out_row + (fragment_row < 4 ? 4 : -4);
              if (out_row < row_limit) own_destination[r] = __ldg(p.row_destination + out_row);
              if (partner_row < row_limit) other_destination[r] = __ldg(p.row_destination + partner_row);
            }
          }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int out_row = first_row + 8 * r;
          bool row_stored = out_row < row_limit;
          OutT* c_row = c + static_cast<long long>(out_row) * p.ldc;
          if constexpr (kGrouped) {
            if (p.row_destination != nullptr) {
              // The table holds the address of the row's first element; 0 = do not store.
              row_stored = own_destination[r] != 0ull;
              c_row = reinterpret_cast<OutT*>(own_destination[r]);
            }
          }
          if constexpr (kGrouped && sizeof(OutT) == 2 && kBlocks % 2 == 0) {
            // Rows that leave for another GPU's memory: lanes 16 apart (rows 4 apart) swap one
            // of two neighbouring blocks, so that a store instruction covers four rows with 128
            // contiguous bytes each instead of eight rows with 64; a link carries full cache
            // lines better than halves.  All conditions are the same in every lane.
            if (p.row_destination != nullptr && aligned && n0 + col_base + kNC <= p.n) {
              const bool low = fragment_row < 4;
              const unsigned long long partner_destination = other_destination[r];
#pragma unroll
              for (int block = 0; block < kBlocks; block += 2) {
                uint32_t w[2][4];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
#pragma unroll
                  for (int i = 0; i < 4; ++i) w[half][i] = pack_pair<OutT>(acc[r][(block + half) * 4 + i]);
                  quad_transpose(w[half], quad);
                  if constexpr (kLayout == kFragmentQuads) {
                    const uint32_t v0 = w[half][0], v1 = w[half][1], v2 = w[half][2], v3 = w[half][3];
                    w[half][0] = __byte_perm(v0, v1, 0x5410);
                    w[half][1] = __byte_perm(v2, v3, 0x5410);
                    w[half][2] = __byte_perm(v0, v1, 0x7632);
                    w[half][3] = __byte_perm(v2, v3, 0x7632);
                  }
                }
                // Low lanes keep block `block` and give away the next one, high lanes the reverse.
                uint32_t received[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  received[i] = __shfl_xor_sync(0xffffffffu, low ? w[1][i] : w[0][i], 16);
                }
                const int col = n0 + col_base + (block + (low ? 0 : 1)) * 32 + 8 * quad;
                // First the rows of the low lanes, then the rows of the high lanes.
                const unsigned long long first = low ? reinterpret_cast<unsigned long long>(c_row)
                                                     : partner_destination;
                const unsigned long long second = low ? partner_destination
                                                      : reinterpret_cast<unsigned long long>(c_row);
                const bool first_stored = low ? row_stored : partner_destination != 0ull;
                const bool second_stored = low ? partner_destination != 0ull : row_stored;
                const uint4 own = low ? make_uint4(w[0][0], w[0][1], w[0][2], w[0][3])
                                      : make_uint4(w[1][0], w[1][1], w[1][2], w[1][3]);
                const uint4 other = make_uint4(received[0], received[1], received[2], received[3]);
                if (first_stored) {
                  *reinterpret_cast<uint4*>(reinterpret_cast<OutT*>(first) + col) = low ? own : other;
                }
                if (second_stored) {
                  *reinterpret_cast<uint4*>(reinterpret_cast<OutT*>(second) + col) = low ? other : own;
                }
              }
              continue;
            }
          }
#pragma unroll
          for (int block = 0; block < kBlocks; ++block) {
            const int col = n0 + col_base + block * 32 + 8 * quad;
            if constexpr (sizeof(OutT) == 2) {
              uint32_t w[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) w[i] = pack_pair<OutT>(acc[r][block * 4 + i]);
              quad_transpose(w, quad);
              if constexpr (kLayout == kFragmentQuads) {
                const uint32_t v0 = w[0], v1 = w[1], v2 = w[2], v3 = w[3];
                w[0] = __byte_perm(v0, v1, 0x5410);
                w[1] = __byte_perm(v2, v3, 0x5410);
                w[2] = __byte_perm(v0, v1, 0x7632);
                w[3] = __byte_perm(v2, v3, 0x7632);
              }
              if (row_stored) {
                if (aligned && col + 8 <= p.n) {
                  *reinterpret_cast<uint4*>(c_row + col) = make_uint4(w[0], w[1], w[2], w[3]);
                } else {
                  unsigned short* out = reinterpret_cast<unsigned short*>(c_row);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    if (col + 2 * j < p.n) out[col + 2 * j] = static_cast<unsigned short>(w[j] & 0xffffu);
                    if (col + 2 * j + 1 < p.n) out[col + 2 * j + 1] = static_cast<unsigned short>(w[j] >> 16);
                  }
                }
              }
            } else {
              uint32_t wx[4], wy[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                wx[i] = __float_as_uint(acc[r][block * 4 + i].x);
                wy[i] = __float_as_uint(acc[r][block * 4 + i].y);
              }
              quad_transpose(wx, quad);
              quad_transpose(wy, quad);
              if (row_stored) {
                if (aligned && col + 8 <= p.n) {
                  uint4* out = reinterpret_cast<uint4*>(c_row + col);
                  if constexpr (kLayout == kFragmentQuads) {
                    out[0] = make_uint4(wx[0], wx[1], wx[2], wx[3]);
                    out[1] = make_uint4(wy[0], wy[1], wy[2], wy[3]);
                  } else {
                    out[0] = make_uint4(wx[0], wy[0], wx[1], wy[1]);
                    out[1] = make_uint4(wx[2], wy[2], wx[3], wy[3]);
                  }
                } else {
                  uint32_t* out = reinterpret_cast<uint32_t*>(c_row);
                  constexpr int kStepX = kLayout == kFragmentQuads ? 1 : 2;
                  constexpr int kOffsetY = kLayout == kFragmentQuads ? 4 : 1;
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    if (col + kStepX * j < p.n) out[col + kStepX * j] = wx[j];
                    if (col + kStepX * j + kOffsetY < p.n) out[col + kStepX * j + kOffsetY] = wy[j];
                  }
                }
              }
            }
          }
        }
      }
    }
    if constexpr (kGrouped) {
      // Rows stored into another GPU's memory are consumed there after a collective that
      // follows this kernel in the stream.
      if (p.row_destination != nullptr) __threadfence_system();
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if constexpr (kCtaGroup == 2) cluster_sync_all();
  if (warp == kMmaWarp) tmem_dealloc<kCtaGroup>(tmem_base, Shape::kTmemColumns);
}

}  // namespace gg
