// MoE routing metadata, SwiGLU requantisation and top-k combine kernels.
//
// Routing restates src/grain_gemm/kernels/moe.py:48-171,222-291 of the reference as a stable
// counting sort: key = expert id when the token is enabled and 0 <= id < E (tested at the
// ids' own width, so INT64 ids cannot wrap), else E; `order` lists all assignments sorted by
// key with ties in original order (invalid tail included); `inverse` is the sorted slot or
// -1; counts/offsets per expert; statistics = (enabled out-of-range ids, max count, total).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm_simt.cuh"
#include "ptx.cuh"

namespace gg {

constexpr int kRouteChunk = 1024;

struct RouteParams {
  const void* ids;
  int ids_are_i64;
  const uint8_t* mask;  // [T] or null
  int tokens, top_k, experts;
  void* effective_ids;  // same width as ids
  long long* order;     // [S]
  int* inverse;         // [S]
  int* counts;          // [E]
  int* offsets;         // [E+1]
  int* statistics;      // [3]
  int* workspace;       // [chunks * (E + 1) + chunks] for the multi-chunk path
};

__device__ __forceinline__ int route_key(const RouteParams& p, long long s, bool& invalid) {
  const long long id = p.ids_are_i64 ? reinterpret_cast<const long long*>(p.ids)[s]
                                     : static_cast<long long>(reinterpret_cast<const int*>(p.ids)[s]);
  const bool enabled = p.mask == nullptr || p.mask[s / p.top_k] != 0;
  const bool in_range = id >= 0 && id < p.experts;
  invalid = enabled && !in_range;
  const int key = (enabled && in_range) ? static_cast<int>(id) : p.experts;
  if (p.ids_are_i64) reinterpret_cast<long long*>(p.effective_ids)[s] = key;
  else reinterpret_cast<int*>(p.effective_ids)[s] = key;
  return key;
}

// Stable placement of one chunk: `cursor[key]` holds the next free slot of each key for this
// chunk; warps take turns in index order, lanes of a warp rank themselves among equal keys.
__device__ __forceinline__ void route_place_chunk(const RouteParams& p, long long s, bool present,
                                                  int key, int* cursor) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int turn = 0; turn < kRouteChunk / 32; ++turn) {
    if (warp == turn) {
      const unsigned active = __ballot_sync(0xffffffffu, present);
      if (present) {
        const unsigned same = __match_any_sync(active, key);
        const int rank = __popc(same & ((1u << lane) - 1u));
        const int leader = __ffs(same) - 1;
        int first = 0;
        if (lane == leader) {
          first = cursor[key];
          cursor[key] = first + __popc(same);
        }
        first = __shfl_sync(same, first, leader);
        const int slot = first + rank;
        p.order[slot] = s;
        p.inverse[s] = key < p.experts ? slot : -1;
      }
    }
    __syncthreads();
  }
}

// Scan of the per-key totals held in bins[0..E]; leaves bins[key] = first slot of the key and
// writes counts, offsets and statistics.  Called by one thread.
__device__ __forceinline__ void route_finish_totals(const RouteParams& p, int* bins, int invalid) {
  int running = 0, maximum = 0;
  p.offsets[0] = 0;
  for (int e = 0; e <= p.experts; ++e) {
    const int count = bins[e];
    bins[e] = running;
    running += count;
    if (e < p.experts) {
      p.counts[e] = count;
      p.offsets[e + 1] = running;
      maximum = max(maximum, count);
    }
  }
  p.statistics[0] = invalid;
  p.statistics[1] = maximum;
  p.statistics[2] = p.offsets[p.experts];
}

// Whole routing problem in one CTA (S <= 1024): keys, histogram, scan and placement.
__device__ __forceinline__ void route_single_body(const RouteParams& p, int* bins) {
  const long long slots = static_cast<long long>(p.tokens) * p.top_k;
  for (int i = threadIdx.x; i < p.experts + 2; i += blockDim.x) bins[i] = 0;
  __syncthreads();
  const long long s = threadIdx.x;
  const bool present = s < slots;
  int key = p.experts;
  if (present) {
    bool invalid;
    key = route_key(p, s, invalid);
    atomicAdd(&bins[key], 1);
    if (invalid) atomicAdd(&bins[p.experts + 1], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) route_finish_totals(p, bins, bins[p.experts + 1]);
  __syncthreads();
  route_place_chunk(p, s, present, key, bins);
}

__global__ void __launch_bounds__(kRouteChunk) route_single_kernel(const RouteParams p) {
  extern __shared__ int bins[];  // [E + 2]; the last entry counts invalid ids
  route_single_body(p, bins);
}

// Routing problems of up to kRouteMediumSlots assignments and kRouteMediumKeys - 1 experts in
// ONE CTA of 32 warps, instead of three launches with serial sections.  Every warp owns a
// contiguous range of the assignments and walks it in rounds of 32:
//   1. keys and a private per-warp histogram (lanes with equal keys elect a leader);
//   2. per key an exclusive prefix over the warps, then a block-wide exclusive scan over the
//      keys: base[warp][key] = first slot of that key for that warp;
//   3. the same walk again: slot = base + rank among equal keys of the round, bases advance.
// Warps are ordered, rounds are ordered and lanes are ordered, so the sort is stable, like the
// chunked kernels (and the reference's argsort with stable=True).
constexpr int kRouteMediumRounds = 8;
constexpr int kRouteMediumSlots = 32 * 32 * kRouteMediumRounds;   // 8192 assignments
constexpr int kRouteMediumKeys = 512;                              // experts + 1 at most

__global__ void __launch_bounds__(1024) route_medium_kernel(const RouteParams p) {
  extern __shared__ int medium_smem[];     // [32][keys] per-warp histograms / bases, then scratch
  const int keys = p.experts + 1;
  int* warp_bins = medium_smem;
  int* key_total = medium_smem + 32 * keys;        // [keys] totals, then first slots
  int* scan_scratch = key_total + keys;            // [32] warp totals of the block scan
  int* invalid_total = scan_scratch + 32;          // [1]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long slots = static_cast<long long>(p.tokens) * p.top_k;
  for (int i = threadIdx.x; i < 32 * keys; i += 1024) warp_bins[i] = 0;
  if (threadIdx.x == 0) *invalid_total = 0;
  __syncthreads();

  const int per_warp = static_cast<int>((slots + 31) / 32 + 31) / 32 * 32;   // multiple of 32
  const long long warp_begin = static_cast<long long>(warp) * per_warp;
  int* bins = warp_bins + warp * keys;
  int key[kRouteMediumRounds];
  int invalid_count = 0;
#pragma unroll
  for (int r = 0; r < kRouteMediumRounds; ++r) {
    const long long s = warp_begin + r * 32 + lane;
    const bool present = r * 32 < per_warp && s < slots;
    key[r] = -1;
    if (present) {
      bool invalid;
      key[r] = route_key(p, s, invalid);
      invalid_count += invalid ? 1 : 0;
    }
    const unsigned active = __ballot_sync(0xffffffffu, present);
    if (present) {
      const unsigned same = __match_any_sync(active, key[r]);
      if (lane == __ffs(same) - 1) bins[key[r]] += __popc(same);
    }
    __syncwarp();
  }
  for (int offset = 16; offset > 0; offset >>= 1) {
    invalid_count += __shfl_xor_sync(0xffffffffu, invalid_count, offset);
  }
  if (lane == 0 && invalid_count) atomicAdd(invalid_total, invalid_count);
  __syncthreads();

  // Per key: exclusive prefix over the warps and the key's total.
  for (int k = threadIdx.x; k < keys; k += 1024) {
    int running = 0;
    for (int w = 0; w < 32; ++w) {
      const int count = warp_bins[w * keys + k];
      warp_bins[w * keys + k] = running;
      running += count;
    }
    key_total[k] = running;
  }
  __syncthreads();
  // Block-wide exclusive scan of key_total (keys <= 512: one value per thread of 16 warps).
  int value = threadIdx.x < keys ? key_total[threadIdx.x] : 0;
  int inclusive = value;
  for (int offset = 1; offset < 32; offset <<= 1) {
    const int other = __shfl_up_sync(0xffffffffu, inclusive, offset);
    if (lane >= offset) inclusive += other;
  }
  if (lane == 31) scan_scratch[warp] = inclusive;
  __syncthreads();
  if (warp == 0) {
    const int total = scan_scratch[lane];
    int scanned = total;
    for (int offset = 1; offset < 32; offset <<= 1) {
      const int other = __shfl_up_sync(0xffffffffu, scanned, offset);
      if (lane >= offset) scanned += other;
    }
    scan_scratch[lane] = scanned - total;
  }
  __syncthreads();
  const int first_slot = scan_scratch[warp] + inclusive - value;
  if (threadIdx.x < keys) {
    key_total[threadIdx.x] = first_slot;
    if (threadIdx.x < p.experts) {
      p.counts[threadIdx.x] = value;
      p.offsets[threadIdx.x + 1] = first_slot + value;
    }
    if (threadIdx.x == 0) p.offsets[0] = 0;
  }
  // Largest expert count (statistics[1]).
  int largest = threadIdx.x < p.experts ? value : 0;
  for (int offset = 16; offset > 0; offset >>= 1) {
    largest = max(largest, __shfl_xor_sync(0xffffffffu, largest, offset));
  }
  __syncthreads();                       // scan_scratch is read above, rewritten below
  if (lane == 0) scan_scratch[warp] = largest;
  __syncthreads();
  if (threadIdx.x == 0) {
    int maximum = 0;
    for (int w = 0; w < 32; ++w) maximum = max(maximum, scan_scratch[w]);
    p.statistics[0] = *invalid_total;
    p.statistics[1] = maximum;
    p.statistics[2] = key_total[p.experts];     // first slot of the ignored tail = valid total
  }

  // Placement: the same walk, against base[warp][key] = first slot of the key + warp prefix.
#pragma unroll
  for (int r = 0; r < kRouteMediumRounds; ++r) {
    const long long s = warp_begin + r * 32 + lane;
    const bool present = key[r] >= 0;
    const unsigned active = __ballot_sync(0xffffffffu, present);
    if (present) {
      const unsigned same = __match_any_sync(active, key[r]);
      const int leader = __ffs(same) - 1;
      int first = 0;
      if (lane == leader) {
        first = key_total[key[r]] + bins[key[r]];
        bins[key[r]] += __popc(same);
      }
      first = __shfl_sync(same, first, leader);
      const int slot = first + __popc(same & ((1u << lane) - 1u));
      p.order[slot] = s;
      p.inverse[s] = key[r] < p.experts ? slot : -1;
    }
    __syncwarp();
  }
}

__global__ void __launch_bounds__(kRouteChunk) route_histogram_kernel(const RouteParams p) {
  extern __shared__ int bins[];
  const long long slots = static_cast<long long>(p.tokens) * p.top_k;
  const int chunks = gridDim.x;
  for (int i = threadIdx.x; i < p.experts + 2; i += blockDim.x) bins[i] = 0;
  __syncthreads();
  const long long s = static_cast<long long>(blockIdx.x) * kRouteChunk + threadIdx.x;
  if (s < slots) {
    bool invalid;
    const int key = route_key(p, s, invalid);
    atomicAdd(&bins[key], 1);
    if (invalid) atomicAdd(&bins[p.experts + 1], 1);
  }
  __syncthreads();
  int* histogram = p.workspace + static_cast<long long>(blockIdx.x) * (p.experts + 1);
  for (int i = threadIdx.x; i <= p.experts; i += blockDim.x) histogram[i] = bins[i];
  if (threadIdx.x == 0) p.workspace[static_cast<long long>(chunks) * (p.experts + 1) + blockIdx.x] =
      bins[p.experts + 1];
}

// One CTA: turns the per-chunk histograms into per-chunk first slots (in place).
__global__ void __launch_bounds__(1024) route_scan_kernel(const RouteParams p, int chunks) {
  extern __shared__ int bins[];  // [E + 1]
  const int stride = p.experts + 1;
  for (int key = threadIdx.x; key <= p.experts; key += blockDim.x) {
    int total = 0;
    for (int c = 0; c < chunks; ++c) total += p.workspace[static_cast<long long>(c) * stride + key];
    bins[key] = total;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int invalid = 0;
    const int* invalid_counts = p.workspace + static_cast<long long>(chunks) * stride;
    for (int c = 0; c < chunks; ++c) invalid += invalid_counts[c];
    route_finish_totals(p, bins, invalid);
  }
  __syncthreads();
  for (int key = threadIdx.x; key <= p.experts; key += blockDim.x) {
    int running = bins[key];
    for (int c = 0; c < chunks; ++c) {
      int* cell = p.workspace + static_cast<long long>(c) * stride + key;
      const int count = *cell;
      *cell = running;
      running += count;
    }
  }
}

__global__ void __launch_bounds__(kRouteChunk) route_place_kernel(const RouteParams p) {
  extern __shared__ int bins[];
  const long long slots = static_cast<long long>(p.tokens) * p.top_k;
  const int* first = p.workspace + static_cast<long long>(blockIdx.x) * (p.experts + 1);
  for (int i = threadIdx.x; i <= p.experts; i += blockDim.x) bins[i] = first[i];
  __syncthreads();
  const long long s = static_cast<long long>(blockIdx.x) * kRouteChunk + threadIdx.x;
  const bool present = s < slots;
  int key = p.experts;
  if (present) {
    key = p.ids_are_i64 ? static_cast<int>(reinterpret_cast<const long long*>(p.effective_ids)[s])
                        : reinterpret_cast<const int*>(p.effective_ids)[s];
  }
  route_place_chunk(p, s, present, key, bins);
}

// Hands a few integers (routing statistics, error flags) to the host by storing them into
// page-locked host memory the device can address.  Unlike a device-to-host copy this does not
// queue behind other transfers on the copy engine, so a caller that streams large results to
// the host at the same time still learns the values as soon as the producing kernel is done,
// and the stream does not wait for the copy engine either.
__global__ void __launch_bounds__(32)
report_to_host_kernel(const int* __restrict__ values, int count, int* host_words) {
  for (int i = threadIdx.x; i < count; i += 32) host_words[i] = values[i];
  __threadfence_system();
}

// Row-tile list for the grouped kernels: every expert's sorted rows are cut into tiles of
// `tile_rows`; tile_expert/tile_row have room for ceil(S / tile_rows) + E entries, unused
// entries get expert -1.  One CTA: a block-wide exclusive scan of the experts' tile counts,
// 1024 experts at a time.
__global__ void __launch_bounds__(1024)
moe_tiles_kernel(const int* __restrict__ offsets, int experts, int tile_rows, int max_tiles,
                 int* __restrict__ tile_expert, int* __restrict__ tile_row) {
  __shared__ int warp_total[32];
  __shared__ int carry;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < experts; base += 1024) {
    const int e = base + threadIdx.x;
    int begin = 0, tiles = 0;
    if (e < experts) {
      begin = offsets[e];
      tiles = (offsets[e + 1] - begin + tile_rows - 1) / tile_rows;
    }
    int inclusive = tiles;
    for (int offset = 1; offset < 32; offset <<= 1) {
      const int other = __shfl_up_sync(0xffffffffu, inclusive, offset);
      if (lane >= offset) inclusive += other;
    }
    if (lane == 31) warp_total[warp] = inclusive;
    __syncthreads();
    if (warp == 0) {
      const int total = warp_total[lane];
      int scanned = total;
      for (int offset = 1; offset < 32; offset <<= 1) {
        const int other = __shfl_up_sync(0xffffffffu, scanned, offset);
        if (lane >= offset) scanned += other;
      }
      warp_total[lane] = scanned - total;
    }
    __syncthreads();
    const int first = carry + warp_total[warp] + inclusive - tiles;
    for (int t = 0; t < tiles; ++t) {
      tile_expert[first + t] = e;
      tile_row[first + t] = begin + t * tile_rows;
    }
    __syncthreads();
    if (threadIdx.x == 1023) carry = first + tiles;
    __syncthreads();
  }
  for (int t = carry + threadIdx.x; t < max_tiles; t += blockDim.x) {
    tile_expert[t] = -1;
    tile_row[t] = 0;
  }
}

// ------------------------------------------------------------------ SwiGLU + requantisation

// SiLU table of the fused Gate/Up kernel: gate values reach SwiGLU rounded to the 16-bit
// output type, so silu(gate) = div_rn(gate, 1 + exp(-gate)) has only 65536 possible
// arguments.  Entry b holds the result for the value whose bit pattern is b, computed here with
// exactly the operations of swiglu_value, hence bit-identical to evaluating the formula
// (the idea of the reference's experiments/thor_interleaved_mega/exact_silu_lut.cuh:1-36).
__global__ void __launch_bounds__(256)
silu_table_kernel(float* __restrict__ silu_table, int half_output) {
  const int bits = blockIdx.x * 256 + threadIdx.x;
  if (bits >= 65536) return;
  const float gate = half_output ? __half2float(__ushort_as_half(static_cast<unsigned short>(bits)))
                                 : __uint_as_float(static_cast<uint32_t>(bits) << 16);
  silu_table[bits] = __fdiv_rn(gate, __fadd_rn(1.0f, expf(-gate)));
}

// Activation rows and their scales in sorted-slot order, for the valid slots only:
// sorted_x[slot, :] = x[order[slot] / top_k, :] and likewise for the row scales (the
// pre-sorted mode of the fused Gate/Up kernel, kept for measurements against the row-gather
// mode).  One warp per slot; a row is `hidden` bytes (a multiple of 256) moved as 16-byte vectors.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const int8_t* __restrict__ x, const float* __restrict__ scale_x,
                   const long long* __restrict__ order, const int* __restrict__ offsets,
                   int experts, int top_k, int hidden, int8_t* __restrict__ sorted_x,
                   float* __restrict__ sorted_scale) {
  const int valid = offsets[experts];
  const int lane = threadIdx.x & 31;
  const int groups = hidden / 256;
  const int vectors = hidden / 16;
  for (long long slot = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5); slot < valid;
       slot += static_cast<long long>(gridDim.x) * 8) {
    const long long token = order[slot] / top_k;
    const uint4* source = reinterpret_cast<const uint4*>(x + token * hidden);
    uint4* destination = reinterpret_cast<uint4*>(sorted_x + slot * hidden);
    for (int i = lane; i < vectors; i += 32) destination[i] = source[i];
    for (int g = lane; g < groups; g += 32) {
      sorted_scale[slot * groups + g] = scale_x[token * groups + g];
    }
  }
}

// h = silu(gate) * up with every operation rounded separately (no FMA contraction), as in
// src/grain_gemm/kernels/moe.py:594 of the reference (div_rn(g, 1 + exp(-g)) * u).
__device__ __forceinline__ float swiglu_value(float gate, float up) {
  const float denominator = __fadd_rn(1.0f, expf(-gate));
  return __fmul_rn(__fdiv_rn(gate, denominator), up);
}

// q = clamp(nearbyint(h / scale), -127, 127) with scale = max(amax, 1e-12) / 127
// (src/grain_gemm/kernels/moe.py:321-328).
__device__ __forceinline__ float quantize_scale(float amax) {
  return __fdiv_rn(fmaxf(amax, 1.0e-12f), 127.0f);
}
__device__ __forceinline__ int quantize_value(float h, float scale) {
  const float rounded = nearbyintf(__fdiv_rn(h, scale));
  return static_cast<int>(fminf(fmaxf(rounded, -127.0f), 127.0f));
}

// The library division carries a branch to a slow path, which keeps the compiler from
// interleaving the long dependent chains of many divisions.  The fused Gate/Up epilogue
// therefore requantises (h / scale, one scale per row) with the classical FMA sequence, which
// is branch-free and, by Markstein's theorem, still correctly rounded: with y = RN(1/d)
// (__frcp_rn), q within 1 ulp of n/d and r = fma(-d, q, n) exact, fma(r, y, q) is the
// correctly rounded quotient.  It needs every intermediate to stay normal; the caller tests
// the row's range and falls back to the library division outside it, so codes always equal
// those of __fdiv_rn.
__device__ __forceinline__ float divide_by_fma(float n, float d, float y) {
  float q = __fmul_rn(n, y);
  q = __fmaf_rn(__fmaf_rn(-d, q, n), y, q);  // now within 1 ulp
  return __fmaf_rn(__fmaf_rn(-d, q, n), y, q);
}
// Row scales for which h / scale may use the sequence with y = __frcp_rn(scale): quotients
// of magnitude >= 1/4 then have normal residuals, and smaller ones round to 0 either way.
__device__ __forceinline__ bool quantize_division_is_safe(float row_max) {
  return row_max < 1.0e30f;  // also false for NaN and infinity
}
__device__ __forceinline__ int quantize_value_by_fma(float h, float scale, float y) {
  const float rounded = nearbyintf(divide_by_fma(h, scale, y));
  return static_cast<int>(fminf(fmaxf(rounded, -127.0f), 127.0f));
}

// Router front-end: per token, the top_k largest of E logits (ties to the lower expert id,
// ids in descending order of logit, like torch.topk on distinct values) and their routing
// weights softmax(logits)[id] renormalised over the selection, i.e.
//   w_i = exp(l_i - l_max) / sum_{j selected} exp(l_j - l_max),
// the logits -> softmax -> top-k -> renormalise step in front of routing (the reference leaves
// it to the caller: benchmarks/bench_moe_ffn.py:283-285, docs/moe_ffn.md:5-7).  One warp per
// token; expert e lives in lane e % 32, slot e / 32 (E <= 1024).  Logits must be finite.
template <typename InT>
__device__ __forceinline__ void router_topk_token(const InT* __restrict__ row, int experts, int top_k,
                                                  float* __restrict__ weights,
                                                  void* __restrict__ ids, int ids_are_i64,
                                                  long long token, int lane) {
  constexpr float kLowest = -3.402823466e+38f;
  float value[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int e = lane + 32 * i;
    value[i] = e < experts ? static_cast<float>(row[e]) : kLowest;
  }
  float first = 0.0f, total = 0.0f, mine = 0.0f;   // lane r keeps the r-th weight
  int mine_id = 0;
  for (int r = 0; r < top_k; ++r) {
    float best = kLowest;
    int best_id = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (value[i] > best) {   // slots ascend in expert id: the first maximum wins a tie
        best = value[i];
        best_id = lane + 32 * i;
      }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, offset);
      const int other_id = __shfl_xor_sync(0xffffffffu, best_id, offset);
      if (other > best || (other == best && other_id < best_id)) {
        best = other;
        best_id = other_id;
      }
    }
    if (r == 0) first = best;
    const float weight = expf(best - first);
    total += weight;
    if (lane == (r & 31)) {
      mine = weight;
      mine_id = best_id;
    }
    if ((best_id & 31) == lane) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (i == (best_id >> 5)) value[i] = kLowest;
      }
    }
    if ((r & 31) == 31 || r == top_k - 1) {
      // Flush up to 32 selections; weights are divided by the final total below.
      const int base = r & ~31;
      if (lane <= (r & 31)) {
        const long long slot = token * top_k + base + lane;
        weights[slot] = mine;
        if (ids_are_i64) reinterpret_cast<long long*>(ids)[slot] = mine_id;
        else reinterpret_cast<int*>(ids)[slot] = mine_id;
      }
    }
  }
  __syncwarp();
  for (int r = lane; r < top_k; r += 32) {
    const long long slot = token * top_k + r;
    weights[slot] = __fdiv_rn(weights[slot], total);
  }
}

template <typename InT>
__global__ void __launch_bounds__(256)
router_topk_kernel(const InT* __restrict__ logits, int tokens, int experts, int top_k,
                   float* __restrict__ weights, void* __restrict__ ids, int ids_are_i64) {
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (token >= tokens) return;
  router_topk_token(logits + static_cast<long long>(token) * experts, experts, top_k, weights, ids,
                    ids_are_i64, token, lane);
}

// Router front-end and routing in one launch for decode-sized problems (T * R <= 1024,
// E <= 1024): the warps of one CTA select every token's experts, and the same CTA then
// sorts the assignments it has just written (row N3 of the next rows: the ids never leave the
// SM's caches between top-k and the histogram).  p.ids is the id output of the first half and
// the input of the second.
template <typename InT>
__global__ void __launch_bounds__(kRouteChunk)
route_topk_single_kernel(const InT* __restrict__ logits, float* __restrict__ weights,
                         const RouteParams p) {
  extern __shared__ int bins[];  // [E + 2]
  const int lane = threadIdx.x & 31;
  for (int token = threadIdx.x >> 5; token < p.tokens; token += kRouteChunk / 32) {
    router_topk_token(logits + static_cast<long long>(token) * p.experts, p.experts, p.top_k,
                      weights, const_cast<void*>(p.ids), p.ids_are_i64, token, lane);
  }
  __syncthreads();   // the ids written above are read back by other warps of this CTA
  route_single_body(p, bins);
}

// Entry quantiser: symmetric per-row, per-K-group INT8 quantisation of floating rows,
// restating quantize_rows (src/grain_gemm/kernels/moe.py:321-356):
//   scale = div_rn(max(amax, 1e-12), 127);  q = clamp(nearbyint(div_rn(v, scale)), +-127).
// Eight consecutive values per lane (16 bytes of BF16/FP16, 32 of FP32); a group of G values
// is G/8 neighbouring lanes, so a warp covers 256/G groups of one row at a time.  HBM bound:
// sizeof(InT) bytes read and one byte (+ 4/G) written per element.
template <typename InT>
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const InT* __restrict__ x, long long rows, int width, int group,
                     int8_t* __restrict__ q, float* __restrict__ s) {
  const int lane = threadIdx.x & 31;
  const int chunks = width / 256;                 // 256-value chunks per row (width % 256 == 0)
  const long long item = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (item >= rows * chunks) return;
  const long long row = item / chunks;
  const int column = static_cast<int>(item - row * chunks) * 256 + lane * 8;
  const InT* source = x + row * width + column;
  float v[8];
  if constexpr (sizeof(InT) == 4) {
    const float4 a = *reinterpret_cast<const float4*>(source);
    const float4 b = *reinterpret_cast<const float4*>(source + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 raw = *reinterpret_cast<const uint4*>(source);
    const InT* values = reinterpret_cast<const InT*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = static_cast<float>(values[i]);
  }
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  for (int offset = group / 16; offset > 0; offset >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
  }
  const float scale = quantize_scale(amax);
  uint32_t packed[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    packed[i >> 2] |= (static_cast<uint32_t>(quantize_value(v[i], scale)) & 0xffu) << (8 * (i & 3));
  }
  *reinterpret_cast<uint2*>(q + row * width + column) = make_uint2(packed[0], packed[1]);
  if ((lane & (group / 8 - 1)) == 0) s[row * (width / group) + column / group] = scale;
}

// Stand-alone SwiGLU + G256 requantisation over a [rows, 2I] gate/up matrix (the unfused
// path).  One warp per (row, 256-channel group); rows at or beyond *valid_rows get q = 0 and
// scale = 1e-12/127.
template <typename InT>
__global__ void __launch_bounds__(256)
swiglu_quantize_kernel(const InT* __restrict__ gate_up, long long rows,
                       const int* __restrict__ valid_rows_ptr, int intermediate, int interleaved,
                       int8_t* __restrict__ q, float* __restrict__ s) {
  const int groups = intermediate / 256;
  const long long item = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (item >= rows * groups) return;
  const long long row = item / groups;
  const int group = static_cast<int>(item - row * groups);
  const int lane = threadIdx.x & 31;
  const long long valid_rows = valid_rows_ptr ? *valid_rows_ptr : rows;
  int8_t* q_row = q + row * intermediate + group * 256;
  if (row >= valid_rows) {
    for (int j = lane; j < 256; j += 32) q_row[j] = 0;
    if (lane == 0) s[row * groups + group] = __fdiv_rn(1.0e-12f, 127.0f);
    return;
  }
  const InT* in = gate_up + row * 2 * intermediate;
  float h[8];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int channel = group * 256 + i * 32 + lane;
    const float gate = static_cast<float>(in[interleaved ? 2 * channel : channel]);
    const float up = static_cast<float>(in[interleaved ? 2 * channel + 1 : intermediate + channel]);
    h[i] = swiglu_value(gate, up);
    amax = fmaxf(amax, fabsf(h[i]));
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1)
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
  const float scale = quantize_scale(amax);
#pragma unroll
  for (int i = 0; i < 8; ++i) q_row[i * 32 + lane] = static_cast<int8_t>(quantize_value(h[i], scale));
  if (lane == 0) s[row * groups + group] = scale;
}

// ------------------------------------------------------------------ top-k combine

// out[t,:] = cast( sum over the token's slots r, in slot order, with inverse >= 0 of
//                  float(expert_out[inverse[t*R+r], :]) * weights[t,r] )
// product and sum are separate FP32 operations (src/grain_gemm/kernels/moe.py:634-653).
// One CTA per token, 8 columns per thread per step.
template <typename T>
__global__ void __launch_bounds__(256)
combine_kernel(const T* __restrict__ expert_out, const float* __restrict__ weights,
               const int* __restrict__ inverse, T* __restrict__ out, int top_k, int hidden,
               int vector_ok) {
  extern __shared__ int slot_smem[];  // [R] slots then [R] weights
  float* weight_smem = reinterpret_cast<float*>(slot_smem + top_k);
  const long long token = blockIdx.x;
  for (int r = threadIdx.x; r < top_k; r += blockDim.x) {
    const int slot = inverse[token * top_k + r];
    slot_smem[r] = slot;
    weight_smem[r] = slot >= 0 ? weights[token * top_k + r] : 0.0f;
  }
  __syncthreads();
  if (vector_ok) {
    for (int col = threadIdx.x * 8; col < hidden; col += blockDim.x * 8) {
      float total[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      // Eight rows are fetched before any is added, so that a thread keeps eight 16-byte loads
      // in flight; the additions stay in slot order.
      for (int r0 = 0; r0 < top_k; r0 += 8) {
        uint4 packed[8];
        int slot[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          slot[j] = r0 + j < top_k ? slot_smem[r0 + j] : -1;
          if (slot[j] >= 0) {
            packed[j] = *reinterpret_cast<const uint4*>(
                expert_out + static_cast<long long>(slot[j]) * hidden + col);
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (slot[j] < 0) continue;
          const float w = weight_smem[r0 + j];
          const T* values = reinterpret_cast<const T*>(&packed[j]);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            total[i] = __fadd_rn(total[i], __fmul_rn(static_cast<float>(values[i]), w));
        }
      }
      uint4 packed_out;
      T* outputs = reinterpret_cast<T*>(&packed_out);
#pragma unroll
      for (int i = 0; i < 8; ++i) outputs[i] = cast_out<T>(total[i]);
      *reinterpret_cast<uint4*>(out + token * hidden + col) = packed_out;
    }
  } else {
    for (int col = threadIdx.x; col < hidden; col += blockDim.x) {
      float total = 0.0f;
      for (int r = 0; r < top_k; ++r) {
        const int slot = slot_smem[r];
        if (slot < 0) continue;
        total = __fadd_rn(total, __fmul_rn(static_cast<float>(
                                               expert_out[static_cast<long long>(slot) * hidden + col]),
                                           weight_smem[r]));
      }
      out[token * hidden + col] = cast_out<T>(total);
    }
  }
}

}  // namespace gg
