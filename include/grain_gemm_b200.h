/*
 * C ABI of libgrain_b200.so: the B200 (sm_100a) implementation of GrainGEMM's two hot
 * paths, the W8A8 K-group-scaled GEMM and the inference MoE FFN stages.
 *
 * Conventions (the reference's, src/grain_gemm/kernels/csrc/sm110/int8_g256_moe_gather.cu:380-440):
 *  - plain pointers and sizes only; every pointer is device memory of the current device
 *    unless stated otherwise; the caller owns all memory, outputs and workspaces included;
 *  - every launch goes to `stream` (a cudaStream_t passed as void*); no entry point
 *    synchronises, allocates or keeps state between calls, except where stated;
 *  - return value: 0 = success; > 0 = cudaError_t; -10000 - r = CUresult r from the tensor-map
 *    encoder; gg_error_string() decodes all of them.
 * Paths quoted below are relative to the reference project.
 */
#ifndef GRAIN_GEMM_B200_H
#define GRAIN_GEMM_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Output element types. */
#define GG_OUT_FP32 0
#define GG_OUT_BF16 1
#define GG_OUT_FP16 2

/* Kernel variants for gg_int8_gemm (GG_VARIANT_AUTO picks by layout and shape). */
#define GG_VARIANT_AUTO 0
#define GG_VARIANT_SIMT 1        /* CUDA-core kernel: any strides, any K */
#define GG_VARIANT_TC_N256 2     /* tcgen05, one CTA per 128 x 256 tile */
#define GG_VARIANT_TC_N128 3     /* tcgen05, one CTA per 128 x 128 tile */
#define GG_VARIANT_TC_N64 4      /* tcgen05, one CTA per 128 x 64 tile */
#define GG_VARIANT_TC_PAIR_N256 5 /* tcgen05 cta_group::2, CTA pair per 256 x 256 tile */
#define GG_VARIANT_TC_PAIR_N128 6 /* tcgen05 cta_group::2, CTA pair per 256 x 128 tile */
#define GG_VARIANT_TC_SPLITK 7   /* tcgen05, M <= 32: K split over CTAs, INT32 dots folded in order */
#define GG_VARIANT_GEMV 8        /* CUDA cores (dp4a), M <= 8, K % 16 == 0: weights streamed once, no workspace */

/* ABI version of this header; the Python loader refuses a library that reports another. */
int gg_abi_version(void);

/* Text for a status returned by any entry point.  Replaces grain_cuda_error_string /
 * grain_moe_gather_error_string (csrc/sm110/int8_g256_cute.cu:300, int8_g256_moe_gather.cu:437). */
const char* gg_error_string(int status);

/*
 * C[M,N] = A[M,K] @ B[K,N] with FP32 scales scale_a[M, ceil(K/G)] and scale_b[ceil(K/G), N]:
 * exact INT32 dot per K group, then total = fmaf(float(dot), sa*sb, total) in group order,
 * one cast to out_dtype.  All strides are in elements and must be positive; c is row-major
 * with row pitch ldc.  group_size in {32, 64, 128, 256}.
 * Replaces the launch behind int8_gemm (src/grain_gemm/gemm.py:212-219): the Triton kernel
 * src/grain_gemm/kernels/triton.py:54-63 and grain_cute_g256 (csrc/sm110/int8_g256_cute.cu:264).
 * The tensor-core variants need A rows and B columns contiguous in K (a_sk == 1, b_sk == 1),
 * 16-byte aligned bases and row pitches that are multiples of 16; anything else runs the
 * CUDA-core variant (or fails with cudaErrorInvalidValue when a tensor-core variant was forced).
 */
int gg_int8_gemm(const void* a, const void* b, const void* scale_a, const void* scale_b, void* c,
                 int m, int n, int k,
                 long long a_sm, long long a_sk, long long b_sk, long long b_sn,
                 long long sa_sm, long long sa_sg, long long sb_sg, long long sb_sn,
                 long long ldc, int group_size, int out_dtype, int variant, void* stream);

/*
 * gg_int8_gemm with a caller-provided workspace, which skinny problems (M <= 32) use to split
 * K over all SMs: the exact INT32 group dots are written to the workspace and a second kernel
 * folds them in group order, so the result is bit-identical to the single-pass kernels.
 * gg_int8_gemm_workspace_bytes returns the size to provide (0 when no workspace is used);
 * passing NULL falls back to the single-pass kernels.
 */
size_t gg_int8_gemm_workspace_bytes(int m, int n, int k, int group_size);
int gg_int8_gemm_ws(const void* a, const void* b, const void* scale_a, const void* scale_b, void* c,
                    int m, int n, int k,
                    long long a_sm, long long a_sk, long long b_sk, long long b_sn,
                    long long sa_sm, long long sa_sg, long long sb_sg, long long sb_sn,
                    long long ldc, int group_size, int out_dtype, int variant,
                    void* workspace, size_t workspace_bytes, void* stream);

/* Variant gg_int8_gemm would run for these arguments (GG_VARIANT_*), without launching.
 * Backs get_kernel_config (src/grain_gemm/gemm.py:84-178). */
int gg_int8_gemm_select(const void* a, const void* b, const void* c, int m, int n, int k,
                        long long a_sm, long long a_sk, long long b_sk, long long b_sn,
                        long long ldc, int group_size, int out_dtype);

/* Same GEMM on the CUDA-core kernel, additionally writing the INT32 group dots to
 * partials[M, N, ceil(K/G)] (test aid for the "INT32 partials bit-exact" contract). */
int gg_int8_gemm_partials(const void* a, const void* b, const void* scale_a, const void* scale_b,
                          void* c_fp32, void* partials, int m, int n, int k,
                          long long a_sm, long long a_sk, long long b_sk, long long b_sn,
                          long long sa_sm, long long sa_sg, long long sb_sg, long long sb_sn,
                          int group_size, void* stream);

/* The reference's native GEMM entry point with its exact signature
 * (csrc/sm110/int8_g256_cute.cu:264-266; ctypes declaration src/grain_gemm/kernels/cuda.py:85-88):
 * G = 256, BF16 output, A [M,K] contiguous, B stored as Linear [N,K] contiguous, contiguous
 * scales.  `config` is accepted and ignored (the library chooses the tile). */
int grain_cute_g256(const void* a, const void* b, const void* scale_a, const void* scale_b,
                    void* c, int m, int n, int k, int config, void* stream);
const char* grain_cuda_error_string(int status);

/* ---- MoE stages (src/grain_gemm/moe.py:253-346) ------------------------------------------ */

/* Bytes of scratch gg_moe_route needs for T tokens, top-k R and E experts (may be 0). */
size_t gg_moe_route_workspace_bytes(int tokens, int top_k, int experts);

/*
 * Routing metadata, replacing prepare_routes (src/grain_gemm/kernels/moe.py:222-291).
 * ids: [T,R] int32 or int64 (ids_are_i64); mask: [T] bytes or NULL.
 * effective_ids [T*R] (same width as ids), order [T*R] int64, inverse [T*R] int32,
 * counts [E] int32, offsets [E+1] int32, statistics [3] int32 =
 * (enabled ids outside [0,E), largest count, number of valid assignments).
 */
int gg_moe_route(const void* ids, int ids_are_i64, const void* mask, int tokens, int top_k,
                 int experts, void* effective_ids, void* order, void* inverse, void* counts,
                 void* offsets, void* statistics, void* workspace, size_t workspace_bytes,
                 void* stream);

/*
 * gg_moe_route for callers that cannot allocate device memory.  This entry point has no
 * counterpart in the reference.  Some hosts of this library are not allowed to call
 * cudaMalloc (or an allocator built on it) at the point where routing runs: an inference
 * server that hands out all of its device memory at start-up and forbids later growth, a
 * plugin whose host gives it no allocator, or a latency-critical loop that must not hit the
 * implicit device-wide synchronisation of an allocation.  They cannot provide the
 * `workspace` that gg_moe_route asks for, so this variant keeps the scratch inside the
 * library, in a fixed array in device memory that is part of the loaded module:
 *  - capacity gg_moe_route_noalloc_capacity_bytes() = 2 MiB per GPU, held by every GPU that
 *    loads the library until the process exits;
 *  - the problem must satisfy gg_moe_route_workspace_bytes(T, R, E) <= that capacity
 *    (for example 131072 assignments with up to 4094 experts); anything larger returns
 *    GG_STATUS_STATIC_SCRATCH_TOO_SMALL and launches nothing;
 *  - it calls no cudaMalloc, cudaFree or any other allocating routine; inputs and outputs
 *    are still the caller's;
 *  - the first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current) and remembers it; make that first
 *    call before starting any stream capture on the device;
 *  - every call on a device shares the one array, which keeps whatever the previous call
 *    left in it.  The routing kernels overwrite every scratch word they later read, so
 *    nothing has to be cleared between calls, but two calls whose kernels overlap on the
 *    GPU (different streams, or different host threads on one device) race on it: issue
 *    them on one stream or order them with events.
 * Outputs are identical to gg_moe_route's.
 */
#define GG_STATUS_STATIC_SCRATCH_TOO_SMALL (-20001)
int gg_moe_route_noalloc(const void* ids, int ids_are_i64, const void* mask, int tokens, int top_k,
                         int experts, void* effective_ids, void* order, void* inverse, void* counts,
                         void* offsets, void* statistics, void* stream);
size_t gg_moe_route_noalloc_capacity_bytes(void);

/* Entries tile_expert / tile_row must hold for S assignments, E experts, tiles of tile_rows. */
int gg_moe_tile_capacity(int assignments, int experts, int tile_rows);

/* Cuts every expert's sorted rows into tiles of tile_rows rows; the used entries come first,
 * unused entries get expert -1 (gg_moe_gate_up and gg_moe_down rely on that order: they walk
 * the list up to its first unused entry).
 * Replaces prepare_ragged_tiles (src/grain_gemm/kernels/moe.py:294-318). */
int gg_moe_tiles(const void* offsets, int experts, int tile_rows, int capacity, void* tile_expert,
                 void* tile_row, void* stream);

/*
 * Router front-end (the step before gg_moe_route): per token the top_k largest of `experts`
 * logits (<= 1024; ties to the lower id; ids in descending order of logit) and their weights
 * softmax(logits)[id] renormalised over the selection.  logits[tokens, experts] contiguous of
 * dtype in_dtype (GG_OUT_FP32/BF16/FP16 name the element type), finite; weights[tokens, top_k]
 * fp32; ids[tokens, top_k] int32 or int64.  The reference leaves this step to the caller
 * (benchmarks/bench_moe_ffn.py:283-285, docs/moe_ffn.md:5-7).
 */
int gg_moe_topk(const void* logits, int in_dtype, int tokens, int experts, int top_k, void* weights,
                void* ids, int ids_are_i64, void* stream);

/*
 * gg_moe_topk followed by gg_moe_route in ONE launch, for decode-sized problems
 * (tokens * top_k <= 1024, experts <= 1024; anything larger returns cudaErrorInvalidValue and the
 * caller makes the two calls): the CTA that selects the experts sorts the assignments it has
 * just written.  Arguments and results as for the two entry points (ids is an output here).
 */
int gg_moe_route_topk(const void* logits, int in_dtype, const void* mask, int tokens, int experts,
                      int top_k, void* weights, void* ids, int ids_are_i64, void* effective_ids,
                      void* order, void* inverse, void* counts, void* offsets, void* statistics,
                      void* stream);

/*
 * Entry quantiser (the step before both paths): x[rows, width] of dtype in_dtype (GG_OUT_FP32,
 * GG_OUT_BF16 or GG_OUT_FP16 name the element type), contiguous, width a multiple of 256,
 * 16-byte aligned; writes q[rows, width] int8 and s[rows, width/group_size] fp32 with
 * scale = max(amax, 1e-12) / 127 and q = clamp(nearbyint(x / scale), +-127), every division
 * correctly rounded.  group_size is 32, 64, 128 or 256.
 * Replaces quantize_rows (src/grain_gemm/kernels/moe.py:321-356).
 */
int gg_quantize_rows(const void* x, int in_dtype, long long rows, int width, int group_size,
                     void* q, void* s, void* stream);

/*
 * Fills table[65536] (fp32, device) with silu(v) = v / (1 + exp(-v)) for every value v of
 * out_dtype (GG_OUT_BF16 or GG_OUT_FP16), indexed by v's 16-bit pattern, computed with the
 * operations of the SwiGLU formula itself (expf, one correctly rounded division).  The fused
 * Gate/Up kernel looks silu up here; gg_moe_gate_up fills its own copy on every call, this
 * entry point exposes the table to tests and to callers that want to inspect it.  The idea is
 * the reference's experiments/thor_interleaved_mega/exact_silu_lut.cuh:1-36.
 */
int gg_moe_silu_table(void* table, int out_dtype, void* stream);

/*
 * Gate/Up projection + rounding to out_dtype + SwiGLU + G256 requantisation over the sorted
 * slots: q[S,I] int8 and s[S,I/256] fp32; rows are gathered from x[T,H] by order[slot] / R.
 * w1: Linear [E,2I,H] contiguous int8; scale_w1: [E,H/256,2I] fp32.  interleaved != 0 means
 * the 2I dimension is ordered [g0,u0,g1,u1,...].  tile_rows must be the value given to
 * gg_moe_tiles: 128 selects the fused tensor-core kernel (needs 16-byte aligned x and w1),
 * 32 the CUDA-core path.  The fused kernel has two ways to fetch the token rows of a tile:
 *   row_gather != 0  straight from x[T,H] and scale_x by token index (order[slot] / R): 32 TMA
 *                    row gathers (cp.async.bulk.tensor tile::gather4, four rows each, per-CTA,
 *                    no multicast) fill a 128-row operand slab in shared memory; no copy of the
 *                    activations in expert order exists anywhere;
 *   row_gather == 0  a small copy kernel first writes the rows and their scales in sorted-slot
 *                    order into the scratch, so that a slab is one tiled TMA box.  Measured on
 *                    B200 this is the faster of the two (the TMA unit processes a gather of
 *                    four rows no faster than a whole 128-row box), so the Python layer uses
 *                    it by default.
 * Both give identical bits.  gate_up_scratch must hold gg_moe_gate_up_scratch_bytes() bytes
 * (16-byte aligned): the 256 KiB SiLU table, preceded for row_gather == 0 by the sorted rows
 * [S,H] and scales [S,H/256]; for the CUDA-core path the [S,2I] gate/up matrix of out_dtype.
 * Replaces ragged_gemm + swiglu_quantize (src/grain_gemm/moe.py:298-304) and
 * grain_moe_gather_launch / grain_moe_interleaved_launch
 * (csrc/sm110/int8_g256_moe_gather.cu:380, int8_g256_moe_interleaved.cu:372).
 */
size_t gg_moe_gate_up_scratch_bytes(int assignments, int hidden, int intermediate, int tile_rows,
                                    int row_gather);
int gg_moe_gate_up(const void* x, const void* scale_x, const void* w1, const void* scale_w1,
                   const void* order, const void* offsets, const void* tile_expert,
                   const void* tile_row, int tile_capacity, int tile_rows, void* q, void* s,
                   void* gate_up_scratch, int tokens, int top_k, int experts, int hidden,
                   int intermediate, int interleaved, int out_dtype, int row_gather, void* stream);

/*
 * Down projection over the sorted slots: expert_out[S,H] (out_dtype) from q[S,I], s[S,I/256],
 * w2 Linear [E,H,I] contiguous int8, scale_w2 [E,I/256,H].  Rows at or beyond offsets[E] are
 * not written.  tile_rows 128 = tensor cores, 32 = CUDA cores.
 * row_destination (optional, tensor-core path only): a device array of S 64-bit addresses; row r
 * is then stored at row_destination[r] (the address of its first element, 16-byte aligned;
 * 0 = skip the row) instead of expert_out + r * H, and expert_out may be NULL.  The addresses
 * may point into another GPU's memory mapped on this one: the expert-parallel layer uses this to
 * return every result row to the token's home rank from inside the GEMM.
 * Replaces the second ragged_gemm (src/grain_gemm/moe.py:305-308) and grain_cutlass_moe_g256
 * (csrc/sm110/int8_g256_moe.cu:287).
 */
int gg_moe_down(const void* q, const void* s, const void* w2, const void* scale_w2,
                const void* offsets, const void* tile_expert, const void* tile_row,
                int tile_capacity, int tile_rows, void* expert_out, const void* row_destination,
                int assignments, int experts, int hidden, int intermediate, int out_dtype,
                void* stream);

/*
 * out[T,H] = cast( sum_r float(expert_out[inverse[t*R+r]]) * weights[t,r] ), slots with
 * inverse < 0 skipped, FP32 product and sum unfused.  Replaces combine
 * (src/grain_gemm/kernels/moe.py:656-676).
 */
int gg_moe_combine(const void* expert_out, const void* weights, const void* inverse, void* out,
                   int tokens, int top_k, int hidden, int out_dtype, void* stream);

/* ---- Expert parallelism over peer memory --------------------------------------------------
 *
 * The reference is single-GPU ("one GPU and no communication",
 * benchmarks/results/thor/moe_ffn_original_x_emc2750.md:26-27); these entry points have no
 * counterpart there.  Experts are split contiguously over `world` ranks (local_experts each),
 * tokens are sharded per rank.  Every rank owns a receive area that all ranks of the node can
 * address (gg_peer_* below), laid out for a token capacity C per rank:
 *   recv_x [world*C, H] int8, recv_scale [world*C, H/256] fp32, recv_ids [world*C, R] int32,
 *   recv_src [world*C] int32, home_out [C*R, H] out_dtype.
 * Rank s writes its rows for rank d at rows [s*C, s*C + n) of d's area, so no offsets have to
 * be agreed on first; the counts travel afterwards in one all-gather that also orders "all rows
 * have arrived" before the expert kernels.  All kernels bound every remote index and set *error
 * instead of touching memory outside the areas.
 */

/* Per destination rank d and token t: position[t*world + d] = index of t among this rank's rows
 * for d (token order) or -1; counts[world + 1] = rows per destination, then the number of enabled
 * ids outside [0, experts); home_inverse[t*R + r] = t*R + r for a valid assignment, else -1 (the
 * `inverse` gg_moe_combine takes when home_out is indexed by flattened assignment). */
int gg_ep_plan(const void* ids, int ids_are_i64, const void* mask, int tokens, int top_k,
               int experts, int world, int local_experts, void* position, void* counts,
               void* home_inverse, void* stream);

/* Copies every (token, destination) pair's row, scales, per-slot local expert indices
 * (local_experts = "not on this rank") and home token index into the destination's receive
 * area.  recv_* are device arrays of `world` 64-bit addresses (valid on this GPU). */
int gg_ep_dispatch(const void* x, const void* scale_x, const void* ids, int ids_are_i64,
                   const void* mask, const void* position, int tokens, int top_k, int experts,
                   int world, int local_experts, int hidden, int rank, int capacity,
                   const void* recv_x, const void* recv_scale, const void* recv_ids,
                   const void* recv_src, void* error, void* stream);

/* row_mask[s*C + i] = i < counts_all[s][rank] for the all-gathered counts [world, world + 1]. */
int gg_ep_row_mask(const void* counts_all, int world, int rank, int capacity, void* row_mask,
                   void* stream);

/* row_destination[slot] for gg_moe_down: the row of assignment (received token m, slot r) goes
 * to home_out[m / C] + ((recv_src[m] * R + r) * H) elements; 0 beyond the valid prefix. */
int gg_ep_row_destination(const void* order, const void* offsets, int experts, int top_k,
                          int capacity, int world, int hidden, int out_dtype, const void* recv_src,
                          const void* home_out, void* row_destination, void* error, void* stream);

/* Device memory that other processes of the node can map (CUDA IPC; set-up time only: these
 * allocate, map or free and are not meant for the hot path).  gg_peer_alloc returns zeroed
 * memory from cudaMalloc; gg_peer_export fills a 64-byte handle another process passes to
 * gg_peer_import, which maps the allocation (peer access is enabled lazily) and returns an
 * address valid in that process; gg_peer_release unmaps, gg_peer_free frees. */
int gg_peer_alloc(size_t bytes, void** pointer);
int gg_peer_free(void* pointer);
int gg_peer_export(void* pointer, void* handle64);
int gg_peer_import(const void* handle64, void** pointer);
int gg_peer_release(void* pointer);

/*
 * Reads (and clears) the device status word that kernels set when one of their bounded
 * waits ran out.  Synchronises `stream`.  *status = 0 when every kernel completed normally;
 * otherwise (site << 8) | 1 with `site` naming the wait that gave up first.
 */
int gg_device_status(int* status, void* stream);

/*
 * Stores count (1 .. 1024) 32-bit words from device memory into page-locked host memory from
 * a kernel on `stream` (no counterpart in the reference, which reads its routing statistics back
 * with a blocking copy, src/grain_gemm/moe.py:258-260).  host_words
 * must come from cudaHostAlloc / cudaHostRegister (torch pinned memory does); the call asks
 * the driver for its device-side address and returns the driver's error if there is none.  A
 * copy engine busy with other transfers does not delay it.  The caller orders its read with an
 * event recorded after the call.
 */
int gg_report_to_host(const void* values, int count, void* host_words, void* stream);

/*
 * Self-test of that mechanism (no counterpart in the reference, whose device waits are
 * unbounded): launches one warp that waits, with the kernels' own bounded wait, on a barrier
 * nothing ever completes.  The wait gives up after limit_ns nanoseconds (1 .. 100 000 000), the
 * kernel returns normally, *result (a device int) is 0 and gg_device_status then reports
 * GG_SELFTEST_WAIT_STATUS once.  Nothing traps or hangs: the wait is bounded by construction.
 */
#define GG_SELFTEST_WAIT_STATUS ((15 << 8) | 1)
int gg_selftest_wait_timeout(long long limit_ns, void* result, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* GRAIN_GEMM_B200_H */
