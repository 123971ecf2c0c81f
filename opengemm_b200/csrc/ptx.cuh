// Thin inline-PTX layer for sm_100a: mbarriers with bounded waits, TMA loads
// and stores (no cluster multicast anywhere), tensor memory management,
// tcgen05.mma / cp / commit / ld, and cluster helpers.
//
// Replaces the reference's three PTX headers (opengemm/src/common/ptx.cuh:8-239,
// opengemm/src/mm/ptx.cuh:121-330, opengemm/src/smm/ptx.cuh:12-203) with one
// layer shared by the dense and the block-scaled paths.  Unlike the
// reference, whose waits spin forever (common/ptx.cuh:111-135), every wait
// here gives up after a wall-clock limit and reports it.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace og {

// MMA instruction families (the PTX `.kind::` qualifier).
enum Kind : int {
  KIND_F16 = 0,       // f16 / bf16 inputs, f32 accumulate
  KIND_TF32 = 1,      // tf32 inputs
  KIND_I8 = 2,        // s8 / u8 inputs, s32 accumulate
  KIND_F8F6F4 = 3,    // e4m3 / e5m2 / e3m2 / e2m3 / e2m1 in 8-bit containers
  KIND_MXF8F6F4 = 4,  // block-scaled fp8, one ue8m0 scale per 32 values
  KIND_MXF4 = 5,      // block-scaled packed fp4, ue8m0 per 32
  KIND_NVF4 = 6,      // block-scaled packed fp4, ue4m3 per 16 (kind::mxf4nvf4, scale_vec::4X)
};
__host__ __device__ constexpr bool kind_scaled(int kind) { return kind >= KIND_MXF8F6F4; }

// Codes written to the launch's status word when a wait gives up.
enum WaitSite : int {
  SITE_NONE = 0,
  SITE_PRODUCER_EMPTY = 1,
  SITE_MMA_FULL = 2,
  SITE_MMA_ACC_EMPTY = 3,
  SITE_EPI_ACC_FULL = 4,
  SITE_DRAIN = 5,
  SITE_PARTIAL_FLAG = 6,
  SITE_CLC = 7,
  SITE_TMEM_READY = 8,
  SITE_CLUSTER_K = 9,
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xFFFFFFFF;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---- cluster ----------------------------------------------------------------

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}

// The address of the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}

// ---- mbarrier ---------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cta.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Arrive on a barrier that may live in another CTA of the cluster; `bar` is a
// shared::cluster address (from map_to_cta).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar)
               : "memory");
}

// One attempt: the hardware parks the thread until the phase completes or the
// hint (nanoseconds) runs out, so a waiting role does not burn issue slots and
// power spinning - on a power-capped part that is tensor-core clock.
constexpr uint32_t WAIT_PARK_NS = 500000;
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity), "r"(WAIT_PARK_NS)
      : "memory");
  return done != 0;
}

// What every role needs to give up cleanly: a CTA-wide abort flag in shared
// memory, the launch's status word in global memory (may be null) and the
// limit in nanoseconds.
struct WaitCtx {
  volatile int* abort_flag;
  int* status;
  uint64_t limit_ns;
};

// Wait for the phase with this parity to complete.  Returns false when the
// limit ran out, or when another role of this CTA already gave up; the
// caller then leaves its loop and heads for the common teardown.
//
// The waits next to the data (a stage's full / empty barrier, a scheduler
// answer) give up after the limit; the waits for a whole accumulator, which
// sit behind an entire K loop of those, allow twice as long, so that a stall
// is reported where it arose rather than where it was felt.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& ctx,
                                          int site) {
  if (mbar_try_wait(bar, parity)) return true;
  // Not there yet.  Every further attempt may park the thread for up to
  // WAIT_PARK_NS, so the clock and the abort flag are looked at once per
  // attempt: a limit of a few milliseconds is kept to within one parking time.
  const uint64_t start = global_timer_ns();
  const uint64_t limit = (site == SITE_EPI_ACC_FULL || site == SITE_MMA_ACC_EMPTY) ? 2 * ctx.limit_ns : ctx.limit_ns;
#pragma unroll 1
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*ctx.abort_flag) return false;
    if (global_timer_ns() - start > limit) {
      *ctx.abort_flag = 1;
      if (ctx.status) atomicCAS(ctx.status, 0, site | (int(blockIdx.x) << 8));
      return false;
    }
  }
}

// Publish `value` in a global flag word after this warp's earlier global
// stores: the warp has synchronised (the caller's __syncwarp), so lane 0's
// release store orders all of them before the flag for any thread of the GPU
// that reads the flag with acquire semantics.
__device__ __forceinline__ void flag_release(int* flag, int value) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}

__device__ __forceinline__ int flag_acquire(const int* flag) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
  return v;
}

// Wait (whole warp) until a global flag word equals `want`: lane 0 polls, the
// others join it.  Bounded like mbar_wait; false means give up.
__device__ __forceinline__ bool wait_flag(const int* flag, int want, const WaitCtx& ctx) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) {
    const uint64_t start = global_timer_ns();
    while (flag_acquire(flag) != want) {
      if (*ctx.abort_flag || global_timer_ns() - start > ctx.limit_ns) {
        if (!*ctx.abort_flag) {
          *ctx.abort_flag = 1;
          if (ctx.status) atomicCAS(ctx.status, 0, SITE_PARTIAL_FLAG | (int(blockIdx.x) << 8));
        }
        ok = 0;
        break;
      }
    }
  }
  ok = __shfl_sync(0xFFFFFFFFu, ok, 0);  // also orders the other lanes' loads after lane 0's acquire
  return ok != 0;
}

// ---- TMA (tensor and bulk copies; never multicast) ----------------------------

__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// 2-D tile load into this CTA's shared memory.  With CTA_GROUP == 2 the
// completion bytes may be credited to a barrier in the pair's other CTA, so
// `bar` is then a shared::cluster address.
template <int CTA_GROUP>
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int x, int y,
                                            uint32_t bar) {
  if constexpr (CTA_GROUP == 1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(tmap), "r"(x), "r"(y), "r"(bar)
        : "memory");
  } else {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(tmap), "r"(x), "r"(y), "r"(bar)
        : "memory");
  }
}

__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   tmap),
               "r"(src), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Wait until at most N of this thread's store groups still READ shared memory.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// Make generic-proxy shared-memory writes visible to the async proxy (TMA).
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void pdl_wait_prior_grids() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---- cluster launch control ----------------------------------------------------

// Ask the hardware to cancel a cluster of this grid that has not started yet.
// The 16-byte answer lands in this CTA's shared memory at `response` and
// completes 16 bytes on `bar` (no fan-out to other CTAs).
__device__ __forceinline__ void clc_try_cancel(uint32_t response, uint32_t bar) {
  asm volatile(
      "clusterlaunchcontrol.try_cancel.async.shared::cta.mbarrier::complete_tx::bytes.b128 [%0], [%1];" ::"r"(
          response),
      "r"(bar)
      : "memory");
}

// Decode an answer: the first CTA id (x) of the cancelled cluster, or -1 when
// nothing was left to cancel.
__device__ __forceinline__ int clc_decode(uint4 answer) {
  uint32_t ok, x;
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b128 h;\n\t"
      "mov.b128 h, {%2, %3, %4, %5};\n\t"
      "clusterlaunchcontrol.query_cancel.is_canceled.pred.b128 p, h;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "mov.u32 %1, 0;\n\t"
      "@p clusterlaunchcontrol.query_cancel.get_first_ctaid::x.b32.b128 %1, h;\n\t}"
      : "=r"(ok), "=r"(x)
      : "r"(answer.x), "r"(answer.y), "r"(answer.z), "r"(answer.w));
  return ok ? int(x) : -1;
}

__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}

// Store 16 bytes into another CTA's shared memory (`addr` from map_to_cta).
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// ---- tensor memory ------------------------------------------------------------

template <int CTA_GROUP>
__device__ __forceinline__ void tmem_alloc(uint32_t result_smem, uint32_t cols) {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     result_smem),
                 "r"(cols)
                 : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     result_smem),
                 "r"(cols)
                 : "memory");
}

template <int CTA_GROUP>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

template <int CTA_GROUP>
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols)
                 : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Ties every later use of 32 registers that an earlier tcgen05.ld filled to
// this point of the program.  Placed after tcgen05.wait::ld when other work
// was scheduled between the load and the wait, it keeps the compiler from
// reading (or moving) those registers before the wait has made them valid.
__device__ __forceinline__ void tmem_ld_settle_32(uint32_t* v) {
  asm volatile(""
               : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]),
                 "+r"(v[7]), "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]),
                 "+r"(v[14]), "+r"(v[15]), "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]),
                 "+r"(v[21]), "+r"(v[22]), "+r"(v[23]), "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]),
                 "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
               :
               : "memory");
}

// ---- shared-memory matrix descriptors ----------------------------------------

// K-major operand tile whose rows are 128 bytes, 128-byte swizzled: groups of
// eight rows are 1024 bytes apart.  Bits: start>>4 [0,14), stride-byte-offset>>4
// [32,46), descriptor version 1 at bit 46, swizzle mode 2 (128 B) at [61,64).
__device__ __forceinline__ uint64_t operand_desc(uint32_t smem_addr) {
  return uint64_t((smem_addr & 0x3FFFFu) >> 4) | (uint64_t(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}

// A 512-byte scale atom: 32 rows of 16 bytes, unswizzled, eight-row groups
// 128 bytes apart.
__device__ __forceinline__ uint64_t scale_desc(uint32_t smem_addr) {
  return uint64_t((smem_addr & 0x3FFFFu) >> 4) | (uint64_t(128 >> 4) << 32) | (1ull << 46);
}

// ---- tcgen05.mma / cp / commit ----------------------------------------------

template <int KIND, int CTA_GROUP>
__device__ __forceinline__ void mma_dense(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
#define OG_MMA(KSTR, G)                                                                   \
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"                          \
               "tcgen05.mma.cta_group::" G ".kind::" KSTR " [%0], %1, %2, %3, p;\n\t}" :: \
                   "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)     \
               : "memory")
  if constexpr (CTA_GROUP == 1) {
    if constexpr (KIND == KIND_F16) OG_MMA("f16", "1");
    else if constexpr (KIND == KIND_TF32) OG_MMA("tf32", "1");
    else if constexpr (KIND == KIND_I8) OG_MMA("i8", "1");
    else OG_MMA("f8f6f4", "1");
  } else {
    if constexpr (KIND == KIND_F16) OG_MMA("f16", "2");
    else if constexpr (KIND == KIND_TF32) OG_MMA("tf32", "2");
    else if constexpr (KIND == KIND_I8) OG_MMA("i8", "2");
    else OG_MMA("f8f6f4", "2");
  }
#undef OG_MMA
}

template <int KIND, int CTA_GROUP>
__device__ __forceinline__ void mma_scaled(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                           uint32_t accumulate) {
#define OG_SMMA(KSTR, G)                                                                       \
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"                               \
               "tcgen05.mma.cta_group::" G ".kind::" KSTR " [%0], %1, %2, %3, [%4], [%5], p;"  \
               "\n\t}" ::"r"(d_tmem),                                                          \
               "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem),             \
               "r"(accumulate)                                                                 \
               : "memory")
  if constexpr (CTA_GROUP == 1) {
    if constexpr (KIND == KIND_MXF8F6F4) OG_SMMA("mxf8f6f4.block_scale.scale_vec::1X", "1");
    else if constexpr (KIND == KIND_MXF4) OG_SMMA("mxf4.block_scale.scale_vec::2X", "1");
    else OG_SMMA("mxf4nvf4.block_scale.scale_vec::4X", "1");
  } else {
    if constexpr (KIND == KIND_MXF8F6F4) OG_SMMA("mxf8f6f4.block_scale.scale_vec::1X", "2");
    else if constexpr (KIND == KIND_MXF4) OG_SMMA("mxf4.block_scale.scale_vec::2X", "2");
    else OG_SMMA("mxf4nvf4.block_scale.scale_vec::4X", "2");
  }
#undef OG_SMMA
}

// Copy one 512-byte scale atom from shared memory into four tensor-memory
// columns, replicated over the four 32-lane quarters.
template <int CTA_GROUP>
__device__ __forceinline__ void scale_copy(uint32_t tmem_addr, uint64_t desc) {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(desc)
                 : "memory");
  else
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(desc)
                 : "memory");
}

// Arrive on `bar` once every tcgen05 operation this thread issued so far has
// completed.  In a pair the arrival goes to the same barrier in both CTAs
// (an mbarrier arrive fanned out inside the cluster; not a TMA load).
template <int CTA_GROUP>
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::
                     "r"(bar)
                 : "memory");
  else
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
        " [%0], %1;" ::"r"(bar),
        "h"(uint16_t(3))
        : "memory");
}

// ---- tensor memory -> registers ----------------------------------------------

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives row
// (lane base + t), columns [col, col+32).
__device__ __forceinline__ void tmem_ld_32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

// ---- small data-path helpers --------------------------------------------------

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t v;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(v) : "f"(hi), "f"(lo));
  return v;
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t v;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(v) : "f"(hi), "f"(lo));
  return v;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}

}  // namespace og
