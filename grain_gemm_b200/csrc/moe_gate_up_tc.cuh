// Gathered Gate/Up projection fused with output rounding, SwiGLU and G256 requantisation.
//
// For every sorted slot (row) of every expert and every 256-channel group of the intermediate
// dimension I:
//   gate/up[c] = round_out( fold_g fmaf(float(dot_i32(x[token], W1[e][c], group g)),
//                                       scale_x[token,g] * scale_w[e,g,c], total) )
//   h[c]      = silu(gate[c]) * up[c]                       (FP32, every operation rounded)
//   scale     = max(max_c |h[c]|, 1e-12) / 127 ;  q[c] = clamp(nearbyint(h[c]/scale), +-127)
// i.e. src/grain_gemm/kernels/moe.py:359-393 (ragged GEMM with SOURCE_IS_TOKEN) followed by
// :564-601 (SwiGLU + requantisation) of the reference, without the [S, 2I] intermediate.
// Token rows reach shared memory in one of two ways (template parameter kGather): straight from
// x[T, H] by token index with TMA row gathers (tile::gather4, 32 per 128-row operand slab, no
// copy of the activations in expert order), or as one tiled TMA box per slab from a copy of the
// rows in sorted-slot order that gather_rows_kernel writes first.  Both give the same bits;
// on B200 the copy is faster (the TMA unit takes about as long for a four-row gather as for a
// whole box), so it is what the Python layer picks by default.
//
// Work item = (128-row tile of one expert, 256-channel group), processed as two sub-tiles of
// 128 channels; a sub-tile is one N = 256 accumulator (128 gate + 128 up columns) in TMEM.
//   warp 8    TMA producer: per stage the activation rows (one box, or 32 row gathers) and two weight boxes
//   warp 9    MMA issuer (tcgen05.mma kind::i8, two TMEM buffers)
//   warp 10   scale staging (cp.async of each K group's column and row scales into a shared-memory ring)
//   warps 0-7 promotion per K group, then SwiGLU (silu by table lookup); the first sub-tile's h
//             is parked in shared memory until the second sub-tile supplies the other half of
//             the row maximum.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm_tc.cuh"
#include "moe_route.cuh"
#include "ptx.cuh"

namespace gg {

struct GateUpParams {
  const float* row_scale;     // gathered: scale_x [T, H/256]; pre-sorted: [S, H/256] by sorted slot
  const long long* order;     // [S] sorted slot -> flattened assignment (gathered mode)
  int top_k;                  // assignment / top_k = token
  const float* silu_table;    // [65536] silu of every value of the output type, by bit pattern
  const float* scale_w;       // [E, H/256, 2I]
  const int* expert_offsets;  // [E+1]
  const int* tile_expert;     // [max_tiles]
  const int* tile_row;        // [max_tiles]
  int8_t* q;                  // [S, I]
  float* s;                   // [S, I/256]
  int hidden, intermediate, max_tiles, interleaved;
};

struct GateUpShape {
  static constexpr int kStages = 3;
  static constexpr int kABytes = 128 * 128;
  static constexpr int kBBytes = 256 * 128;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStashBytes = 256 * 64 * 4;   // 64 parked FP32 values per promotion thread
  static constexpr int kRingFloats = 256 + 128;   // column scales then row scales of one group
  static constexpr int kScaleSlots = 8;
  static constexpr int kScaleBytes = kScaleSlots * kRingFloats * 4;
  static constexpr int kAmaxBytes = 2 * 4 * 128 * 4;   // two item parities x (sub, half) x 128 rows
  static constexpr int kBarrierBytes = (2 * kStages + 4 + 2 * kScaleSlots) * 8 + 16;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kStashBytes + kScaleBytes +
                                    kAmaxBytes + kBarrierBytes;
};

// Work item -> (row tile, channel group).  Items of one expert are consecutive and ordered
// channel-group-major: neighbouring CTAs work on different row tiles of the same expert
// against the same 256-channel weight block, so that block is read from DRAM once and served
// from L2 to the other row tiles.  Returns false for items past the last used tile.
__device__ __forceinline__ bool gate_up_item(const GateUpParams& p, int item, int channel_groups,
                                             int& tile, int& jg, int& expert) {
  const int probe = item / channel_groups;
  expert = p.tile_expert[probe];
  if (expert < 0) return false;
  const int begin = p.expert_offsets[expert];
  const int rows = p.expert_offsets[expert + 1] - begin;
  const int first = probe - (p.tile_row[probe] - begin) / 128;
  const int span = (rows + 127) / 128;
  const int local = item - first * channel_groups;
  jg = local / span;
  tile = first + local - jg * span;
  return true;
}

// The two 16-bit floats of a packed pair as FP32 (exact).
template <typename T>
__device__ __forceinline__ float2 unpack_pair(uint32_t packed) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    return make_float2(__uint_as_float(packed << 16), __uint_as_float(packed & 0xffff0000u));
  } else {
    return __half22float2(*reinterpret_cast<const __half2*>(&packed));
  }
}

// Token row of the tile row `row` (gathered mode); rows past the expert's last one read token 0,
// whose data only feeds accumulator rows that are never stored.
__device__ __forceinline__ int gate_up_source_row(const GateUpParams& p, int row, int row_end) {
  return row < row_end ? static_cast<int>(p.order[row] / p.top_k) : 0;
}

// kGather: map_x covers the original activations x[T, H] and the producer fetches each tile's
// rows by token index with TMA row gathers (no copy of the rows in sorted order exists);
// otherwise map_x covers a pre-sorted copy [S, H] and the tile is one tiled box.
template <typename RoundT, bool kGather>
__global__ void __launch_bounds__(384, 1)
moe_gate_up_tc_kernel(const __grid_constant__ CUtensorMap map_x,
                      const __grid_constant__ CUtensorMap map_w, const GateUpParams p) {
  using Shape = GateUpShape;
  constexpr int kStages = Shape::kStages;
  constexpr int BN = 256;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stage_base = smem;
  // The first sub-tile's h waits here for the second sub-tile's half of the row maximum.
  float* stash = reinterpret_cast<float*>(smem + kStages * Shape::kStageBytes);
  float* sb_ring = stash + Shape::kStashBytes / 4;
  float* amax_part = sb_ring + Shape::kScaleSlots * Shape::kRingFloats;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(amax_part + 2 * 4 * 128);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full_bar = empty_bar + kStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint64_t* scale_full_bar = tmem_empty_bar + 2;
  uint64_t* scale_empty_bar = scale_full_bar + Shape::kScaleSlots;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(scale_empty_bar + Shape::kScaleSlots);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int channel_groups = p.intermediate / 256;
  const int groups = p.hidden / 256;
  const int slabs = p.hidden / 128;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full_bar[i], 1);   // the producer's arrive.expect_tx; the TMA bytes complete it
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full_bar[i], 1);
      mbar_init(&tmem_empty_bar[i], 8);
    }
    for (int i = 0; i < Shape::kScaleSlots; ++i) {
      mbar_init(&scale_full_bar[i], 32);   // every lane of the scale warp
      mbar_init(&scale_empty_bar[i], 8);   // one arrival per promotion warp
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 8 && lane == 0) {
    prefetch_tensormap(&map_x);
    prefetch_tensormap(&map_w);
  }
  // The row-tile list has room for the worst case and its used entries come first; the kernel
  // walks only those.  (An expert-parallel rank's list is sized for every row it could
  // receive, several times what it does receive.)
  __shared__ int used_row_tiles;
  if (threadIdx.x == 32) {
    int low = 0, high = p.max_tiles;
    while (low < high) {
      const int middle = (low + high) >> 1;
      if (p.tile_expert[middle] >= 0) low = middle + 1;
      else high = middle;
    }
    used_row_tiles = low;
  }
  if (warp == 9) tmem_alloc<1>(tmem_holder, 512);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const int total_items = used_row_tiles * channel_groups;
  constexpr FragmentLayout kLayout = kFragmentPairs;

  // Warps 8-11 (producer, MMA issuer, two spares) give registers to the promotion warps.
  if (warp >= 8) {
  setmaxnreg_dec<GG_AUX_REGS>();
  if (warp != 9) {
    // ------------------------------------------------------------ TMA producer (warp 8)
    // Three boxes per stage: 128 sorted activation rows, 128 gate and 128 up weight rows.
    // The warp walks the ring converged; one elected lane issues the tiled loads.  Warp 11 idles.
    if (warp == 8) {
      const bool leader = elect_one();
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        int tile, jg, expert;
        if (!gate_up_item(p, item, channel_groups, tile, jg, expert)) continue;
        const int row0 = p.tile_row[tile];
        [[maybe_unused]] int source[4];   // token rows of tile rows 4 * lane .. 4 * lane + 3
        if constexpr (kGather) {
          const int row_end = p.expert_offsets[expert + 1];
#pragma unroll
          for (int i = 0; i < 4; ++i) source[i] = gate_up_source_row(p, row0 + 4 * lane + i, row_end);
        }
        for (int sub = 0; sub < 2 && ok; ++sub) {
          const int channel0 = jg * 256 + sub * 128;
          const int w_base = expert * 2 * p.intermediate;
          const int row_gate = p.interleaved ? w_base + 2 * channel0 : w_base + channel0;
          const int row_up = p.interleaved ? row_gate + 128 : w_base + p.intermediate + channel0;
          for (int slab = 0, x = 0; slab < slabs; ++slab, x += 128) {
            if (!mbar_wait_warp(&empty_bar[stage], phase ^ 1u, kSiteProducerEmpty, abort_flag)) {
              ok = false;
              break;
            }
            uint8_t* a_dst = stage_base + stage * Shape::kStageBytes;
            uint8_t* b_dst = a_dst + Shape::kABytes;
            if (leader) {
              mbar_expect_tx(&full_bar[stage], Shape::kStageBytes);
              if constexpr (!kGather) tma_load_2d(a_dst, &map_x, &full_bar[stage], x, row0);
              tma_load_2d(b_dst, &map_w, &full_bar[stage], x, row_gate);
              tma_load_2d(b_dst + 128 * 128, &map_w, &full_bar[stage], x, row_up);
            }
            if constexpr (kGather) {
              // Every lane fetches its four rows: 32 gathers of 512 bytes fill the A tile.
              tma_gather4_rows(a_dst + lane * 512, &map_x, &full_bar[stage], x, source[0], source[1],
                               source[2], source[3]);
            }
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    } else if (warp == 10) {
      // ---------------------------------------------------------- scale staging warp
      // Copies each group's 256 column scales (by accumulator column) and 128 row scales into a
      // shared-memory ring with asynchronous 4-byte copies that land in the order the
      // promotion threads read; the copies themselves signal the slot's barrier, so the warp
      // runs a whole ring ahead and global-memory latency stays hidden.
      uint32_t slot = 0, phase = 0;
      bool ok = true;
      const int column_position = ring_column_position<kLayout>(lane);
      const int row_position = ring_row_position(lane);
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        int tile, jg, expert;
        if (!gate_up_item(p, item, channel_groups, tile, jg, expert)) continue;
        const int row0 = p.tile_row[tile];
        const int row_end = p.expert_offsets[expert + 1];
        const float* sb_base = p.scale_w + static_cast<long long>(expert) * groups * 2 * p.intermediate;
        const float* sa_source[4];   // row of row_scale for tile rows lane + 32 * i
        bool sa_valid[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = row0 + lane + 32 * i;
          sa_valid[i] = r < row_end;
          const long long source_row = kGather ? gate_up_source_row(p, r, row_end) : (sa_valid[i] ? r : 0);
          sa_source[i] = p.row_scale + source_row * groups;
        }
        for (int sub = 0; sub < 2 && ok; ++sub) {
          const int channel0 = jg * 256 + sub * 128;
          const float* sb_source[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int c = lane + 32 * i;   // accumulator column
            const int sb_col = p.interleaved ? 2 * channel0 + c
                                             : (i < 4 ? channel0 + c : p.intermediate + channel0 + c - 128);
            sb_source[i] = sb_base + sb_col;
          }
          for (int g = 0; g < groups; ++g) {
            const bool got = mbar_test(&scale_empty_bar[slot], phase ^ 1u) ||
                             mbar_wait(&scale_empty_bar[slot], phase ^ 1u, kSiteScaleEmpty, abort_flag);
            if (!__all_sync(0xffffffffu, got)) {
              ok = false;
              break;
            }
            float* destination = sb_ring + slot * Shape::kRingFloats;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              cp_async_f32(destination + 32 * i + column_position,
                           sb_source[i] + static_cast<long long>(g) * 2 * p.intermediate, true);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              cp_async_f32(destination + BN + 32 * i + row_position, sa_source[i] + g, sa_valid[i]);
            }
            cp_async_arrive(&scale_full_bar[slot]);
            if (++slot == Shape::kScaleSlots) {
              slot = 0;
              phase ^= 1u;
            }
          }
        }
      }
      cp_async_wait_all();
    }
  } else {
    // ------------------------------------------------------------ MMA issuer
    // The warp walks the loop converged and one elected lane issues, which keeps the
    // descriptor arithmetic in the uniform datapath.
    {
      const bool leader = elect_one();
      constexpr uint32_t idesc = make_idesc_i8(128, BN);
      const uint32_t a_low_base = smem_desc_low(smem_u32(stage_base));
      uint32_t stage = 0, phase = 0;
      uint32_t buffer = 0, empty_parity = 1;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        if (p.tile_expert[item / channel_groups] < 0) continue;
        for (int sub = 0; sub < 2 && ok; ++sub) {
          for (int slab = 0; slab < slabs; ++slab) {
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
              umma_i8<1>(tmem_d, a_low, b_low, idesc, group_start ? 0u : 1u);
              umma_i8<1>(tmem_d, a_low + 2, b_low + 2, idesc, 1u);
              umma_i8<1>(tmem_d, a_low + 4, b_low + 4, idesc, 1u);
              umma_i8<1>(tmem_d, a_low + 6, b_low + 6, idesc, 1u);
              umma_commit(&empty_bar[stage]);
              if (!group_start) umma_commit(&tmem_full_bar[buffer]);
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
        }
      }
    }
  }
  } else {
    setmaxnreg_inc<GG_PROMO_REGS>();
    // ------------------------------------------------------------ promotion + SwiGLU warps
    // Fragment layout (tmem_ld_16x256b_x4): warp (quarter, half) drains TMEM lanes
    // 32*quarter.. of four 32-column blocks; a thread owns tile rows
    // 32*quarter + lane/4 + 8r (r = 0..3) and, in every block, the column pairs
    // 8i + 2*(lane%4), +1 (i = 0..3).  Split layout: blocks 0,1 are 64 gate columns of this
    // half, blocks 2,3 the matching up columns; interleaved: each pair is (gate, up) of one
    // channel.
    const int half = warp >> 2;
    const int quarter = warp & 3;
    const int tid = threadIdx.x;
    const int fragment_row = lane >> 2;
    const int quad = lane & 3;
    uint32_t group_sequence = 0;
    uint32_t scale_slot = 0, scale_phase = 0;
    bool ok = true;
    float4* stash4 = reinterpret_cast<float4*>(stash) + tid;   // element j at stash4[j * 256]
    // The row-maximum exchange buffer alternates between two copies from one work item to the
    // next: a warp may start the next item (and write its sub-tile 0 maxima) while its partner
    // half is still reading this item's; the barrier of the next item keeps it from getting
    // two items ahead.
    uint32_t item_parity = 0;
    int block_column[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      block_column[b] = p.interleaved ? half * 128 + 32 * b
                                      : (b < 2 ? half * 64 + 32 * b : 128 + half * 64 + 32 * (b - 2));
    }
    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
      int tile, jg, expert;
      if (!gate_up_item(p, item, channel_groups, tile, jg, expert)) continue;
      const int row0 = p.tile_row[tile];
      const int row_end = p.expert_offsets[expert + 1];
      const int first_row = row0 + quarter * 32 + fragment_row;   // + 8r
      float amax_first[4] = {0.0f, 0.0f, 0.0f, 0.0f};

      for (int sub = 0; sub < 2; ++sub) {
        float2 acc[4][16];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[r][i] = make_float2(0.0f, 0.0f);
        }
        for (int g = 0; g < groups; ++g, ++group_sequence) {
          // This group's scales, staged by the scale warp: [0, 256) column scales by
          // accumulator column, [256, 384) row scales by tile row (both in the order the
          // promotion threads read them).  `ok` is the same in every lane.
          if (ok) {
            ok = mbar_wait_warp(&scale_full_bar[scale_slot], scale_phase, kSiteScaleFull, abort_flag);
          }
          const float* slot = sb_ring + scale_slot * Shape::kRingFloats;
          float2 sa[4];
          load_row_scales(slot + BN + quarter * 32, fragment_row, sa);
          const uint32_t buffer = group_sequence & 1u;
          if (ok) {
            ok = mbar_wait_warp(&tmem_full_bar[buffer], (group_sequence >> 1) & 1u,
                                kSiteEpilogueTmemFull, abort_flag);
          }
          tcgen05_fence_after();
          const uint32_t taddr_low =
              tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buffer * BN;
          const uint32_t taddr_high = taddr_low + (16u << 16);
          uint32_t partial_a[16], partial_b[16];
          float2 sb[4];
          if (ok) {
            tmem_ld_16x256b_x4(taddr_low + block_column[0], partial_a);
#pragma unroll
            for (int fragment = 0; fragment < 8; ++fragment) {
              const int block = fragment >> 1;
              if ((fragment & 1) == 0) load_column_scales(slot + block_column[block], quad, sb);
              tmem_ld_wait();
              if (fragment + 1 < 8) {
                const uint32_t next = ((fragment + 1) & 1 ? taddr_high : taddr_low) +
                                      block_column[(fragment + 1) >> 1];
                if (fragment & 1) tmem_ld_16x256b_x4(next, partial_a);
                else tmem_ld_16x256b_x4(next, partial_b);
              } else {
                // All of this warp's TMEM accesses for the buffer are done: hand it back.
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tmem_empty_bar[buffer]);
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

        // SwiGLU on the rounded gate/up values.  h[r][k] is channel (of this sub-tile's 128)
        //   split:       half*64 + (k/8)*32 + 8*((k%8)/2) + 2*quad + k%2
        //   interleaved: half*64 + (k/4)*16 + 4*(k%4) + quad
        // gate and up are rounded to the output type first (pack_pair), so silu(gate) is a
        // lookup by the gate's 16-bit pattern in a table built with the formula itself.
        float h[4][16];
        float amax[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          float row_amax = 0.0f;
          if (p.interleaved) {
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              const uint32_t pair = pack_pair<RoundT>(acc[r][k]);   // (gate, up) of one channel
              h[r][k] = __fmul_rn(__ldg(p.silu_table + (pair & 0xffffu)), unpack_pair<RoundT>(pair).y);
            }
          } else {
#pragma unroll
            for (int b = 0; b < 2; ++b) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const uint32_t gate = pack_pair<RoundT>(acc[r][b * 4 + i]);
                const float2 up = unpack_pair<RoundT>(pack_pair<RoundT>(acc[r][(2 + b) * 4 + i]));
                h[r][b * 8 + 2 * i] = __fmul_rn(__ldg(p.silu_table + (gate & 0xffffu)), up.x);
                h[r][b * 8 + 2 * i + 1] = __fmul_rn(__ldg(p.silu_table + (gate >> 16)), up.y);
              }
            }
          }
#pragma unroll
          for (int k = 0; k < 16; ++k) row_amax = fmaxf(row_amax, fabsf(h[r][k]));
          // The four lanes of a quad hold the row's other channels of this half.
          row_amax = fmaxf(row_amax, __shfl_xor_sync(0xffffffffu, row_amax, 1));
          row_amax = fmaxf(row_amax, __shfl_xor_sync(0xffffffffu, row_amax, 2));
          amax[r] = row_amax;
          if (quad == 0) {
            amax_part[((item_parity * 2 + sub) * 2 + half) * 128 + quarter * 32 + fragment_row + 8 * r] = row_amax;
          }
        }
        if (sub == 0) {
#pragma unroll
          for (int r = 0; r < 4; ++r) {
#pragma unroll
            for (int k = 0; k < 16; k += 4) {
              stash4[(r * 4 + k / 4) * 256] = make_float4(h[r][k], h[r][k + 1], h[r][k + 2], h[r][k + 3]);
            }
            amax_first[r] = amax[r];
          }
        } else {
          named_barrier_sync(1, 256);
          const bool all_ok = ok;
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int tile_row = quarter * 32 + fragment_row + 8 * r;
            float row_max = fmaxf(amax[r], amax_first[r]);
            row_max = fmaxf(row_max, amax_part[((item_parity * 2 + 0) * 2 + (half ^ 1)) * 128 + tile_row]);
            row_max = fmaxf(row_max, amax_part[((item_parity * 2 + 1) * 2 + (half ^ 1)) * 128 + tile_row]);
            const float scale = quantize_scale(row_max);
            const bool by_fma = quantize_division_is_safe(row_max);
            const float y = __frcp_rn(scale);
            const int row = first_row + 8 * r;
            const bool row_stored = all_ok && row < row_end;
            int8_t* q_row = p.q + static_cast<long long>(row) * p.intermediate + jg * 256;
#pragma unroll
            for (int piece = 0; piece < 2; ++piece) {
              // piece 0: parked first sub-tile (channels 0..127), piece 1: registers.
              float v[16];
#pragma unroll
              for (int k = 0; k < 16; k += 4) {
                if (piece == 0) {
                  const float4 parked = stash4[(r * 4 + k / 4) * 256];
                  v[k] = parked.x; v[k + 1] = parked.y; v[k + 2] = parked.z; v[k + 3] = parked.w;
                } else {
                  v[k] = h[r][k]; v[k + 1] = h[r][k + 1]; v[k + 2] = h[r][k + 2]; v[k + 3] = h[r][k + 3];
                }
              }
              uint32_t code[16];
              if (by_fma) {
#pragma unroll
                for (int k = 0; k < 16; ++k)
                  code[k] = static_cast<uint32_t>(quantize_value_by_fma(v[k], scale, y)) & 0xffu;
              } else {
#pragma unroll
                for (int k = 0; k < 16; ++k)
                  code[k] = static_cast<uint32_t>(quantize_value(v[k], scale)) & 0xffu;
              }
              int8_t* q_piece = q_row + piece * 128 + half * 64;
              if (p.interleaved) {
                // Lane `quad` holds channels 16*blk + 4i + quad; after the exchange it holds the
                // four consecutive channels 16*blk + 4*quad .. +3.
#pragma unroll
                for (int blk = 0; blk < 4; ++blk) {
                  uint32_t w[4] = {code[blk * 4], code[blk * 4 + 1], code[blk * 4 + 2], code[blk * 4 + 3]};
                  quad_transpose(w, quad);
                  if (row_stored) {
                    *reinterpret_cast<uint32_t*>(q_piece + blk * 16 + 4 * quad) =
                        w[0] | (w[1] << 8) | (w[2] << 16) | (w[3] << 24);
                  }
                }
              } else {
                // Lane `quad` holds channel pairs 32*b + 8i + 2*quad, +1; after the exchange it
                // holds the eight consecutive channels 32*b + 8*quad .. +7.
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                  uint32_t w[4];
#pragma unroll
                  for (int i = 0; i < 4; ++i) w[i] = code[b * 8 + 2 * i] | (code[b * 8 + 2 * i + 1] << 8);
                  quad_transpose(w, quad);
                  if (row_stored) {
                    *reinterpret_cast<uint2*>(q_piece + b * 32 + 8 * quad) =
                        make_uint2(w[0] | (w[1] << 16), w[2] | (w[3] << 16));
                  }
                }
              }
            }
            if (row_stored && half == 0 && quad == 0) {
              p.s[static_cast<long long>(row) * channel_groups + jg] = scale;
            }
          }
        }
      }
      item_parity ^= 1u;
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc<1>(tmem_base, 512);
}

}  // namespace gg
