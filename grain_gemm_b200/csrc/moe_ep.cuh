// Expert-parallel exchange kernels: token dispatch and result return over peer memory.
//
// The reference is a single-GPU library (its moe_ffn runs "one GPU and no communication",
// benchmarks/results/thor/moe_ffn_original_x_emc2750.md:26-27); expert parallelism is added on
// top of its stages without changing their arithmetic.  Experts are split contiguously over W
// ranks, tokens are sharded per rank.  Every rank owns a receive area that all ranks can
// address (peer mappings of device memory, plain loads and stores over NVLink):
//
//   recv_x    [W * C, H]   int8   token rows; source rank s writes rows [s * C, s * C + n_s)
//   recv_scale[W * C, H/256] f32  their scales
//   recv_ids  [W * C, R]   int32  per slot the local expert index, or E_local ("not mine")
//   recv_src  [W * C]      int32  the token's index on its home rank
//   home_out  [C * R, H]   out    expert outputs of this rank's own tokens, by flattened
//                                 (token, slot); written by the ranks that own the experts
//
// with C the token capacity per rank.  A source's rows for a destination start at a fixed
// offset (s * C), so nothing has to be agreed on before the rows are sent; the per-pair counts
// travel afterwards in one small all-gather that also orders "all rows have arrived" before
// the expert kernels start.  Rows beyond a source's count are masked out of the local routing.
// The Down projection then stores each output row straight into the home rank's home_out
// (see GemmTcParams::row_destination), so the return trip overlaps the GEMM tile by tile.
#pragma once

#include <stdint.h>

namespace gg {

struct EpPlanParams {
  const void* ids;        // [T, R] global expert ids
  int ids_are_i64;
  const uint8_t* mask;    // [T] or null
  int tokens, top_k, experts, world, local_experts;
  int* position;          // [T, W] index of the token among this rank's rows for rank d, or -1
  int* counts;            // [W + 1] rows for each rank; [W] = enabled ids outside [0, E)
  int* home_inverse;      // [T * R] the flattened assignment itself when valid, else -1
};

__device__ __forceinline__ long long ep_read_id(const EpPlanParams& p, long long slot) {
  return p.ids_are_i64 ? reinterpret_cast<const long long*>(p.ids)[slot]
                       : static_cast<long long>(reinterpret_cast<const int*>(p.ids)[slot]);
}

// One CTA per destination rank d: a running count over the tokens that have at least one
// valid expert on d gives every such token its row index in the (this rank -> d) list, in
// token order.  CTA 0 also fills home_inverse and counts the invalid ids.
__global__ void __launch_bounds__(1024) ep_plan_kernel(const EpPlanParams p) {
  __shared__ int warp_total[32];
  __shared__ int running;
  __shared__ int invalid;
  const int d = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    running = 0;
    invalid = 0;
  }
  __syncthreads();
  for (int base = 0; base < p.tokens; base += 1024) {
    const int t = base + threadIdx.x;
    bool member = false;
    if (t < p.tokens) {
      const bool enabled = p.mask == nullptr || p.mask[t] != 0;
      int bad = 0;
      for (int r = 0; r < p.top_k; ++r) {
        const long long id = ep_read_id(p, static_cast<long long>(t) * p.top_k + r);
        const bool in_range = id >= 0 && id < p.experts;
        const bool valid = enabled && in_range;
        if (valid && id / p.local_experts == d) member = true;
        if (d == 0) {
          p.home_inverse[static_cast<long long>(t) * p.top_k + r] =
              valid ? static_cast<int>(static_cast<long long>(t) * p.top_k + r) : -1;
          if (enabled && !in_range) ++bad;
        }
      }
      if (bad) atomicAdd(&invalid, bad);
    }
    const unsigned ballot = __ballot_sync(0xffffffffu, member);
    if (lane == 0) warp_total[warp] = __popc(ballot);
    __syncthreads();
    int before = running;
    for (int w = 0; w < warp; ++w) before += warp_total[w];
    if (t < p.tokens) {
      p.position[static_cast<long long>(t) * p.world + d] =
          member ? before + __popc(ballot & ((1u << lane) - 1u)) : -1;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int total = 0;
      for (int w = 0; w < 32; ++w) total += warp_total[w];
      running += total;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    p.counts[d] = running;
    if (d == 0) p.counts[p.world] = invalid;
  }
}

struct EpDispatchParams {
  const int8_t* x;        // [T, H]
  const float* scale_x;   // [T, H/256]
  const void* ids;        // [T, R]
  int ids_are_i64;
  const uint8_t* mask;
  const int* position;    // [T, W]
  int tokens, top_k, experts, world, local_experts, hidden, rank, capacity;
  // Receive areas of every rank (device addresses valid on this GPU), [W] each.
  const unsigned long long* recv_x;
  const unsigned long long* recv_scale;
  const unsigned long long* recv_ids;
  const unsigned long long* recv_src;
  int* error;             // set to 1 when a row index falls outside the capacity
};

// One warp per (token, destination rank) pair that exists: copies the token row, its scales,
// the per-slot local expert indices and the token's home index into the destination's area.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const EpDispatchParams p) {
  const int lane = threadIdx.x & 31;
  const long long pairs = static_cast<long long>(p.tokens) * p.world;
  const int groups = p.hidden / 256;
  const int vectors = p.hidden / 16;
  for (long long pair = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5); pair < pairs;
       pair += static_cast<long long>(gridDim.x) * 8) {
    const int position = p.position[pair];
    if (position < 0) continue;
    const int token = static_cast<int>(pair / p.world);
    const int d = static_cast<int>(pair - static_cast<long long>(token) * p.world);
    if (position >= p.capacity) {
      if (lane == 0) *p.error = 1;
      continue;
    }
    const long long row = static_cast<long long>(p.rank) * p.capacity + position;
    const uint4* source = reinterpret_cast<const uint4*>(p.x + static_cast<long long>(token) * p.hidden);
    uint4* destination = reinterpret_cast<uint4*>(p.recv_x[d]) + row * vectors;
    for (int i = lane; i < vectors; i += 32) destination[i] = source[i];
    float* scale_destination = reinterpret_cast<float*>(p.recv_scale[d]) + row * groups;
    for (int g = lane; g < groups; g += 32) {
      scale_destination[g] = p.scale_x[static_cast<long long>(token) * groups + g];
    }
    int* id_destination = reinterpret_cast<int*>(p.recv_ids[d]) + row * p.top_k;
    const bool enabled = p.mask == nullptr || p.mask[token] != 0;
    for (int r = lane; r < p.top_k; r += 32) {
      const long long slot = static_cast<long long>(token) * p.top_k + r;
      const long long id = p.ids_are_i64 ? reinterpret_cast<const long long*>(p.ids)[slot]
                                         : static_cast<long long>(reinterpret_cast<const int*>(p.ids)[slot]);
      const bool mine = enabled && id >= 0 && id < p.experts && id / p.local_experts == d;
      id_destination[r] = mine ? static_cast<int>(id - static_cast<long long>(d) * p.local_experts)
                               : p.local_experts;
    }
    if (lane == 0) reinterpret_cast<int*>(p.recv_src[d])[row] = token;
  }
  // The rows are consumed by another GPU after a collective that follows this kernel.
  __threadfence_system();
}

// row_mask[s * C + i] = i < counts_all[s][rank]: which rows of the receive area hold a token
// of this step.  counts_all is the all-gathered [W, W + 1] count matrix.
__global__ void __launch_bounds__(256)
ep_row_mask_kernel(const int* __restrict__ counts_all, int world, int rank, int capacity,
                   uint8_t* __restrict__ row_mask) {
  const long long rows = static_cast<long long>(world) * capacity;
  for (long long row = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x; row < rows;
       row += static_cast<long long>(gridDim.x) * 256) {
    const int source = static_cast<int>(row / capacity);
    const int index = static_cast<int>(row - static_cast<long long>(source) * capacity);
    row_mask[row] = index < counts_all[source * (world + 1) + rank] ? 1 : 0;
  }
}

// Destination of every sorted output row of the Down projection: the row of assignment
// (received token m, slot r) goes to home_out of the token's home rank at flattened index
// src_token * R + r.  Rows beyond the valid prefix get 0 (they are never stored).
__global__ void __launch_bounds__(256)
ep_row_destination_kernel(const long long* __restrict__ order, const int* __restrict__ offsets,
                          int experts, int top_k, int capacity, int world, int hidden,
                          int element_bytes, const int* __restrict__ recv_src,
                          const unsigned long long* __restrict__ home_out, long long slots,
                          unsigned long long* __restrict__ row_destination, int* error) {
  const int valid = offsets[experts];
  for (long long slot = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x; slot < slots;
       slot += static_cast<long long>(gridDim.x) * 256) {
    unsigned long long destination = 0;
    if (slot < valid) {
      const long long assignment = order[slot];
      const long long m = assignment / top_k;
      const int r = static_cast<int>(assignment - m * top_k);
      const int source = static_cast<int>(m / capacity);
      const int token = recv_src[m];
      if (source >= 0 && source < world && token >= 0 && token < capacity) {
        destination = home_out[source] +
                      (static_cast<unsigned long long>(token) * top_k + r) * hidden * element_bytes;
      } else {
        *error = 1;
      }
    }
    row_destination[slot] = destination;
  }
}

}  // namespace gg
