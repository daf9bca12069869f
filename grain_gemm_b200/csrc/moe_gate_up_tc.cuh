// Gathered Gate/Up projection fused with output rounding, SwiGLU and G256 requantisation.
//
// For every sorted slot (row) of every expert and every 256-channel group of the intermediate
// dimension I:
//   gate/up[c] = round_out( fold_g fmaf(float(dot_i32(x[token], W1[e][c], group g)),
//                                       scale_x[token,g] * scale_w[e,g,c], total) )
//   h[c]      = silu(gate[c]) * up[c]                       (FP32, every operation rounded)
//   scale     = max(max_c |h[c]|, 1e-12) / 127 ;  q[c] = clamp(nearbyint(h[c]/scale), +-127)
// i.e. src/grain_gemm/kernels/moe.py:359-393 (ragged GEMM with SOURCE_IS_TOKEN) followed by
// :564-601 (SwiGLU + requantisation) of the reference, without the [S, 2I] intermediate and
// without an expert-expanded copy of x: the token rows are gathered by the sorted route index
// straight into the swizzled shared-memory operand tile.
//
// Work item = (128-row tile of one expert, 256-channel group), processed as two sub-tiles of
// 128 channels; a sub-tile is one N = 256 accumulator (128 gate + 128 up columns) in TMEM.
//   warps 8, 10, 11   producers: 16-byte cp.async gather of the x rows (96 threads); lane 0 of
//             warp 8 also issues the TMA loads of the two weight boxes
//   warp 9    MMA issuer (tcgen05.mma kind::i8, two TMEM buffers)
//   warps 0-7 promotion per K group, then SwiGLU; the first sub-tile's h is parked in a per-CTA
//             global scratch (L2 resident) until the second sub-tile supplies the other half of
//             the row maximum.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm_tc.cuh"
#include "moe_route.cuh"
#include "ptx.cuh"

namespace gg {

struct GateUpParams {
  const int8_t* x;            // [T, H]
  const float* scale_x;       // [T, H/256]
  const float* scale_w;       // [E, H/256, 2I]
  const long long* order;     // [S]
  const int* expert_offsets;  // [E+1]
  const int* tile_expert;     // [max_tiles]
  const int* tile_row;        // [max_tiles]
  int8_t* q;                  // [S, I]
  float* s;                   // [S, I/256]
  float* stash;               // [CTAs, 128, 128] parking space for the first sub-tile's h
  int top_k, hidden, intermediate, max_tiles, interleaved;
};

struct GateUpShape {
  static constexpr int kStages = 4;
  static constexpr int kABytes = 128 * 128;
  static constexpr int kBBytes = 256 * 128;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStashPitch = 128;   // floats per parked row
  static constexpr int kStashBytesPerCta = 128 * kStashPitch * 4;   // in global memory (L2)
  static constexpr int kScaleBytes = 2 * 256 * 4;
  static constexpr int kAmaxBytes = 4 * 128 * 4;
  static constexpr int kTokenBytes = 128 * 4;
  static constexpr int kBarrierBytes = (2 * kStages + 4) * 8 + 16;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kScaleBytes + kAmaxBytes +
                                    kTokenBytes + kBarrierBytes;
};

__device__ __forceinline__ void cp_async_16_zfill(uint32_t smem_dst, const void* src, bool valid) {
  const uint32_t bytes = valid ? 16u : 0u;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(src), "r"(bytes)
               : "memory");
}
// Makes `bar` receive one (pre-counted) arrival once all cp.async issued so far by this
// thread have completed.
__device__ __forceinline__ void cp_async_arrive_on(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

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

template <typename RoundT>
__device__ __forceinline__ float round_through(float v) {
  return static_cast<float>(cast_out<RoundT>(v));
}

template <typename RoundT>
__global__ void __launch_bounds__(384, 1)
moe_gate_up_tc_kernel(const __grid_constant__ CUtensorMap map_w, const GateUpParams p) {
  using Shape = GateUpShape;
  constexpr int kStages = Shape::kStages;
  constexpr int BN = 256;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stage_base = smem;
  float* sb_ring = reinterpret_cast<float*>(smem + kStages * Shape::kStageBytes);
  // The first sub-tile's h waits in global memory (it stays in L2) for the second sub-tile's
  // half of the row maximum; keeping it out of shared memory buys a fourth operand stage.
  float* stash = p.stash + static_cast<size_t>(blockIdx.x) * 128 * Shape::kStashPitch;
  float* amax_part = sb_ring + 2 * BN;
  int* tile_tokens = reinterpret_cast<int*>(amax_part + 4 * 128);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tile_tokens + 128);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full_bar = empty_bar + kStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int channel_groups = p.intermediate / 256;
  const int total_items = p.max_tiles * channel_groups;
  const int groups = p.hidden / 256;
  const int slabs = p.hidden / 128;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full_bar[i], 97);  // 96 gather threads + the TMA transaction arrival
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full_bar[i], 1);
      mbar_init(&tmem_empty_bar[i], 8);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 8 && lane == 0) prefetch_tensormap(&map_w);
  if (warp == 9) tmem_alloc<1>(tmem_holder, 512);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  // Warps 8-11 (producer, MMA issuer, two spares) give registers to the promotion warps.
  if (warp >= 8) {
  setmaxnreg_dec<64>();
  if (warp != 9) {
    // ------------------------------------------------------------ producers (warps 8, 10, 11)
    // 96 gather threads: thread g copies 16-byte chunk (g & 7) of rows (g >> 3) + 12 * i.
    // Lane 0 of warp 8 also issues the TMA loads of the two weight boxes.
    const int gather_id = (warp == 8 ? 0 : warp - 9) * 32 + lane;
    const int chunk = gather_id & 7;
    const int row_group = gather_id >> 3;
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    const bool tma_leader = warp == 8 && elect_one();
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      int tile, jg, expert;
      if (!gate_up_item(p, item, channel_groups, tile, jg, expert)) continue;
      const int row0 = p.tile_row[tile];
      const int row_end = p.expert_offsets[expert + 1];
      const int8_t* source[11];
      uint32_t valid_mask = 0;
#pragma unroll
      for (int i = 0; i < 11; ++i) {
        const int r = row_group + 12 * i;
        const int row = row0 + r;
        const bool valid = r < 128 && row < row_end;
        const long long token = valid ? p.order[row] / p.top_k : 0;
        source[i] = p.x + token * p.hidden + chunk * 16;
        valid_mask |= valid ? (1u << i) : 0u;
      }
      for (int sub = 0; sub < 2 && ok; ++sub) {
        const int channel0 = jg * 256 + sub * 128;
        const int w_base = expert * 2 * p.intermediate;
        const int row_gate = p.interleaved ? w_base + 2 * channel0 : w_base + channel0;
        const int row_up = p.interleaved ? row_gate + 128 : w_base + p.intermediate + channel0;
        for (int slab = 0, x = 0; slab < slabs; ++slab, x += 128) {
          // Every lane waits; the vote keeps the warp's control flow uniform on failure.
          const bool got = mbar_test(&empty_bar[stage], phase ^ 1u) ||
                           mbar_wait(&empty_bar[stage], phase ^ 1u, kSiteProducerEmpty, abort_flag);
          if (!__all_sync(0xffffffffu, got)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = stage_base + stage * Shape::kStageBytes;
          if (tma_leader) {
            uint8_t* b_dst = a_dst + Shape::kABytes;
            mbar_expect_tx(&full_bar[stage], Shape::kBBytes);
            tma_load_2d(b_dst, &map_w, &full_bar[stage], x, row_gate);
            tma_load_2d(b_dst + 128 * 128, &map_w, &full_bar[stage], x, row_up);
          }
          const uint32_t a_smem = smem_u32(a_dst);
#pragma unroll
          for (int i = 0; i < 11; ++i) {
            const int r = row_group + 12 * i;
            if (r < 128) {
              cp_async_16_zfill(a_smem + r * 128 + ((chunk ^ (r & 7)) << 4), source[i] + x,
                                (valid_mask >> i) & 1u);
            }
          }
          // The barrier receives this thread's arrival when its copies above have landed;
          // the thread itself goes straight on to the next slab.
          cp_async_arrive_on(&full_bar[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
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
            // The x rows were written by cp.async (generic proxy); order them before the
            // tensor core's reads (async proxy).
            fence_proxy_async();
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
    setmaxnreg_inc<216>();
    // ------------------------------------------------------------ promotion + SwiGLU warps
    const int half = warp >> 2;
    const int quarter = warp & 3;
    const int tid = threadIdx.x;
    const int row_in_tile = quarter * 32 + lane;
    uint32_t group_sequence = 0;
    bool ok = true;
    float* stash_row = stash + row_in_tile * Shape::kStashPitch + half * 64;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
      int tile, jg, expert;
      if (!gate_up_item(p, item, channel_groups, tile, jg, expert)) continue;
      const int row = p.tile_row[tile] + row_in_tile;
      const bool row_ok = row < p.expert_offsets[expert + 1];
      const long long token = row_ok ? p.order[row] / p.top_k : 0;
      const float* sa_row = p.scale_x + token * groups;
      const float* sb_base = p.scale_w + static_cast<long long>(expert) * groups * 2 * p.intermediate;
      float amax_first = 0.0f;

      for (int sub = 0; sub < 2; ++sub) {
        const int channel0 = jg * 256 + sub * 128;
        // Accumulator column `tid` of this sub-tile corresponds to this weight column.
        const int sb_col = p.interleaved ? 2 * channel0 + tid
                                         : (tid < 128 ? channel0 + tid
                                                      : p.intermediate + channel0 + tid - 128);
        float2 acc2[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) acc2[i] = make_float2(0.0f, 0.0f);
        sb_ring[tid] = sb_base[sb_col];
        float sa_next = row_ok ? sa_row[0] : 0.0f;
        named_barrier_sync(1, 256);

        for (int g = 0; g < groups; ++g, ++group_sequence) {
          const float sa = sa_next;
          float sb_next = 0.0f;
          if (g + 1 < groups) {
            sb_next = sb_base[static_cast<long long>(g + 1) * 2 * p.intermediate + sb_col];
            if (row_ok) sa_next = sa_row[g + 1];
          }
          const uint32_t buffer = group_sequence & 1u;
          if (ok && !mbar_wait(&tmem_full_bar[buffer], (group_sequence >> 1) & 1u,
                               kSiteEpilogueTmemFull, abort_flag)) {
            ok = false;
          }
          tcgen05_fence_after();
          const float* sb_slot = sb_ring + (g & 1) * BN;
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buffer * BN;
          // Split layout: chunks 0,1 are this thread's gate columns, 2,3 its up columns.
          const int column0 = p.interleaved ? half * 128 : half * 64;
          const int column1 = column0 + 32;
          const int column2 = p.interleaved ? half * 128 + 64 : 128 + half * 64;
          const int column3 = column2 + 32;
          uint32_t partial_a[32], partial_b[32];
          if (ok) {
            tmem_ld_32x32b_x32(taddr + column0, partial_a);
            tmem_ld_wait();
            tmem_ld_32x32b_x32(taddr + column1, partial_b);
            promote<32>(partial_a, sa, sb_slot + column0, acc2);
            tmem_ld_wait();
            tmem_ld_32x32b_x32(taddr + column2, partial_a);
            promote<32>(partial_b, sa, sb_slot + column1, acc2 + 16);
            tmem_ld_wait();
            tmem_ld_32x32b_x32(taddr + column3, partial_b);
            promote<32>(partial_a, sa, sb_slot + column2, acc2 + 32);
            tmem_ld_wait();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty_bar[buffer]);
            promote<32>(partial_b, sa, sb_slot + column3, acc2 + 48);
          }
          sb_ring[((g + 1) & 1) * BN + tid] = sb_next;
          named_barrier_sync(1, 256);
        }

        // SwiGLU on the rounded gate/up values.  Accumulator i is column i of this thread's
        // 128: split layout = gate c at i = c and up c at i = 64 + c; interleaved = 2c, 2c + 1.
        float acc[64];
        float amax = 0.0f;
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 8) {
          float gate[8], up[8], denominator[8];
          bool safe = true;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int c = c0 + j;
            const float gate_split = (c & 1) ? acc2[c / 2].y : acc2[c / 2].x;
            const float up_split = (c & 1) ? acc2[32 + c / 2].y : acc2[32 + c / 2].x;
            gate[j] = round_through<RoundT>(p.interleaved ? acc2[c].x : gate_split);
            up[j] = round_through<RoundT>(p.interleaved ? acc2[c].y : up_split);
            denominator[j] = __fadd_rn(1.0f, expf(-gate[j]));
            safe = safe && swiglu_division_is_safe(gate[j], denominator[j]);
          }
          if (safe) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float y = reciprocal_by_fma(denominator[j]);
              acc[c0 + j] = __fmul_rn(divide_by_fma(gate[j], denominator[j], y), up[j]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              acc[c0 + j] = __fmul_rn(__fdiv_rn(gate[j], denominator[j]), up[j]);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(acc[c0 + j]));
        }
        amax_part[(sub * 2 + half) * 128 + row_in_tile] = amax;
        if (sub == 0) {
#pragma unroll
          for (int c = 0; c < 64; c += 4)
            *reinterpret_cast<float4*>(stash_row + c) =
                make_float4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
          amax_first = amax;
        } else {
          named_barrier_sync(1, 256);
          float row_max = fmaxf(amax, amax_first);
          row_max = fmaxf(row_max, amax_part[(0 * 2 + (half ^ 1)) * 128 + row_in_tile]);
          row_max = fmaxf(row_max, amax_part[(1 * 2 + (half ^ 1)) * 128 + row_in_tile]);
          const float scale = quantize_scale(row_max);
          if (row_ok && ok) {
            int8_t* q_row = p.q + static_cast<long long>(row) * p.intermediate + jg * 256;
            const bool by_fma = quantize_division_is_safe(row_max);
            const float y = __frcp_rn(scale);
#pragma unroll
            for (int piece = 0; piece < 2; ++piece) {
              // piece 0: parked first sub-tile (channels half*64..), piece 1: registers.
              uint4* dst = reinterpret_cast<uint4*>(q_row + piece * 128 + half * 64);
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                float h16[16];
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                  const int c = v * 16 + w * 4;
                  if (piece == 0) {
                    const float4 parked = *reinterpret_cast<const float4*>(stash_row + c);
                    h16[w * 4] = parked.x; h16[w * 4 + 1] = parked.y;
                    h16[w * 4 + 2] = parked.z; h16[w * 4 + 3] = parked.w;
                  } else {
#pragma unroll
                    for (int b = 0; b < 4; ++b) h16[w * 4 + b] = acc[c + b];
                  }
                }
                uint32_t words[4] = {0u, 0u, 0u, 0u};
                if (by_fma) {
#pragma unroll
                  for (int b = 0; b < 16; ++b)
                    words[b / 4] |= (static_cast<uint32_t>(quantize_value_by_fma(h16[b], scale, y)) & 0xffu)
                                    << (8 * (b % 4));
                } else {
#pragma unroll
                  for (int b = 0; b < 16; ++b)
                    words[b / 4] |= (static_cast<uint32_t>(quantize_value(h16[b], scale)) & 0xffu)
                                    << (8 * (b % 4));
                }
                dst[v] = make_uint4(words[0], words[1], words[2], words[3]);
              }
            }
            if (half == 0) p.s[static_cast<long long>(row) * channel_groups + jg] = scale;
          }
        }
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc<1>(tmem_base, 512);
}

}  // namespace gg
