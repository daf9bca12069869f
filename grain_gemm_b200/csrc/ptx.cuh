// Thin inline-PTX wrappers for the sm_100a features the kernels use:
// mbarrier, TMA tiled loads, tcgen05 (alloc / mma / commit / ld), register reallocation and barriers.
// Every wait is bounded: a wait that runs out returns false and the caller unwinds.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gg {

// Device status word written by kernels whose bounded waits ran out.
// 0 = ok; otherwise (site << 8) | code of the first failure seen.
__device__ unsigned int g_device_status[4];

enum WaitSite : unsigned int {
  kSiteProducerEmpty = 1,
  kSiteMmaFull = 2,
  kSiteMmaTmemEmpty = 3,
  kSiteEpilogueTmemFull = 4,
  kSiteDrain = 5,
  kSiteScaleEmpty = 8,
  kSiteScaleFull = 9,
  kSiteSelfTest = 15,
};

__device__ __forceinline__ void report_timeout(unsigned int site) {
  atomicCAS(&g_device_status[0], 0u, (site << 8) | 1u);
  atomicAdd(&g_device_status[1], 1u);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t lane_id() {
  uint32_t l;
  asm volatile("mov.u32 %0, %laneid;" : "=r"(l));
  return l;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}


__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Arrive on the barrier at the same shared-memory offset in CTA `cta` of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint64_t* bar, uint32_t cta) {
  asm volatile(
      "{\n\t"
      ".reg .b32 remote;\n\t"
      "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
      "mbarrier.arrive.shared::cluster.b64 _, [remote];\n\t"
      "}" ::"r"(smem_u32(bar)), "r"(cta)
      : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

// Upper bound, in nanoseconds, for which one try_wait may keep the thread suspended before it
// reports "not yet"; keeps waiting warps from burning issue slots on polling.
#ifndef GG_TRY_WAIT_SUSPEND_NS
#define GG_TRY_WAIT_SUSPEND_NS 20000
#endif
constexpr uint32_t kTryWaitSuspendNs = GG_TRY_WAIT_SUSPEND_NS;

// Single non-blocking probe of a phase parity.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Longest time a wait may take before the kernel gives up (nanoseconds of %globaltimer).
constexpr uint64_t kWaitLimitNs = 2000000000ull;

// Bounded wait on a phase parity.  Returns false (after reporting `site`) when the
// barrier has not flipped within `limit_ns`, or when another thread of the CTA has already
// given up (*abort_flag != 0).  The clock is read only after a probe has failed and come
// back from its suspension, every 64 such failures, so a wait that succeeds costs nothing.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned int site,
                                          volatile int* abort_flag,
                                          uint64_t limit_ns = kWaitLimitNs) {
  const uint32_t addr = smem_u32(bar);
  uint64_t start = 0;
  for (uint32_t spin = 0;; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(addr), "r"(parity), "r"(kTryWaitSuspendNs)
        : "memory");
    if (done) return true;
    if ((spin & 0x3fu) == 0x3fu) {
      if (*abort_flag) return false;
      const uint64_t now = global_timer_ns();
      if (start == 0) {
        start = now;
      } else if (now - start > limit_ns) {
        *abort_flag = 1;
        report_timeout(site);
        return false;
      }
    }
  }
}

// Warp-collective wait: every lane probes, then waits if needed; the verdict is the same in
// all lanes.  Issuing warps stay converged this way, so that descriptor and address
// arithmetic around their tcgen05.mma / TMA instructions runs in the uniform datapath; only
// the issue itself is left to one elected lane.  The promotion warps use it too: their
// tcgen05.ld / tcgen05.wait are .sync.aligned and must see the whole warp take one path,
// also after a wait has run out.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, unsigned int site,
                                               volatile int* abort_flag,
                                               uint64_t limit_ns = kWaitLimitNs) {
  const bool got = mbar_test(bar, parity) || mbar_wait(bar, parity, site, abort_flag, limit_ns);
  return __all_sync(0xffffffffu, got);
}

// 16-byte shared-memory load by 32-bit shared address (a pointer that went through integer
// arithmetic is a generic pointer to the compiler, which then emits generic loads).
__device__ __forceinline__ float4 lds_f32x4(uint32_t smem_address) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(smem_address));
  return v;
}

// ---------------------------------------------------------------- cp.async (scale staging)

// Asynchronous 4-byte copy global -> shared; `valid == false` writes zero without reading.
__device__ __forceinline__ void cp_async_f32(float* smem_dst, const float* src, bool valid) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(smem_dst)), "l"(src),
               "r"(valid ? 4 : 0)
               : "memory");
}

// One arrival on `bar` once all cp.async issued so far by this thread have landed (the
// arrival is already part of the barrier's expected count).
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.wait_all;" ::: "memory");
}

// ---------------------------------------------------------------- TMA

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 2-D tiled load into this CTA's shared memory, completion on this CTA's barrier.
// x is the innermost (byte) coordinate and must be a multiple of 16.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Row gather: four rows y0..y3 of a 2-D tensor (128 bytes each at byte column x; the tensor map
// has a box of 128 bytes x 1 row) land as four consecutive 128-byte rows at smem_dst, with the
// tensor map's swizzle applied by shared-memory address, so 32 such copies at 512-byte steps
// fill a 128-row operand tile exactly like one tiled load of 128 consecutive rows.
// A per-CTA load: no multicast.  x must be a multiple of 16.
__device__ __forceinline__ void tma_gather4_rows(void* smem_dst, const CUtensorMap* map,
                                                 uint64_t* bar, int32_t x, int32_t y0, int32_t y1,
                                                 int32_t y2, int32_t y3) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y0), "r"(y1), "r"(y2),
      "r"(y3)
      : "memory");
}

// Pair variant: the data lands in this CTA's shared memory, the bytes are counted on the
// barrier of the pair's leader CTA (rank 0) at the same offset.  Each CTA issues its own
// load for its own half of the tile.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map,
                                                 uint64_t* bar, int32_t x, int32_t y) {
  const uint32_t leader_bar = smem_u32(bar) & 0xFEFFFFFFu;
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}

// ---------------------------------------------------------------- tcgen05

template <int kCtaGroup>
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t columns) {
  if constexpr (kCtaGroup == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(smem_result)),
                 "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  } else {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(smem_result)),
                 "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
}

template <int kCtaGroup>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
  if constexpr (kCtaGroup == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns)
                 : "memory");
  } else {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns)
                 : "memory");
  }
}

__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}


// Instruction descriptor for kind::i8: signed 8-bit A and B, both K-major, INT32 accumulate.
__host__ __device__ constexpr uint32_t make_idesc_i8(int m, int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// High word of the shared-memory descriptor above (stride byte offset 1024, version 1,
// SWIZZLE_128B) and its low word for a given shared address; the issuing loop keeps the low
// word in a register and adds 2 per 32 bytes of K.
constexpr uint32_t kSmemDescHighSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t smem_desc_low(uint32_t smem_addr) {
  return ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16);
}

template <int kCtaGroup>
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint32_t desc_a_low, uint32_t desc_b_low,
                                        uint32_t idesc, uint32_t accumulate) {
  if constexpr (kCtaGroup == 1) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %5};\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %3, p;\n\t"
        "}" ::"r"(tmem_d),
        "r"(desc_a_low), "r"(desc_b_low), "r"(idesc), "r"(accumulate), "r"(kSmemDescHighSw128)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %5};\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %3, p;\n\t"
        "}" ::"r"(tmem_d),
        "r"(desc_a_low), "r"(desc_b_low), "r"(idesc), "r"(accumulate), "r"(kSmemDescHighSw128)
        : "memory");
  }
}

// Make `bar` (in this CTA) complete one arrival when all tcgen05.mma issued so far by this
// thread have finished.  Implies tcgen05.fence::before_thread_sync.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// Pair variant: arrives on the barrier at this offset in every CTA named by cta_mask.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
      " [%0], %1;" ::"r"(smem_u32(bar)),
      "h"(cta_mask)
      : "memory");
}

// Load 32 consecutive 32-bit columns of this warp's 32 TMEM lanes: thread i gets lane
// (taddr.lane + i), registers j = column (taddr.col + j).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}


// 16 TMEM lanes x 32 columns in the matrix-fragment layout: with q = lane % 4 and
// r = lane / 4, register 4i+0/4i+1 hold row r, columns 8i+2q and 8i+2q+1; registers 4i+2/4i+3
// hold row r+8, same columns (i = 0..3).  taddr.lane selects the first of the 16 lanes.
__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}


__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 16 TMEM lanes x 32 columns as 4-column groups: with q = lane % 4 and r = lane / 4, register
// 2k holds row r, column 4k + q and register 2k + 1 holds row r + 8, same column (k = 0..7).
// Drains TMEM at twice the rate of the 16x256b shape (507 against 256 B/clk/SM measured).
__device__ __forceinline__ void tmem_ld_16x128b_x8(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x128b.x8.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// ---------------------------------------------------------------- misc

// Register reallocation between warpgroups (all four warps of a warpgroup execute it).
template <int kRegisters>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegisters));
}
template <int kRegisters>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegisters));
}

__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::
                   : "memory");
}

}  // namespace gg
