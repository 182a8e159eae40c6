// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (MMA, TMEM
// alloc/ld/st, commit, fences), plus the shared-memory / instruction descriptor encoders.
//
// Every wait in this file is bounded: a wait that runs out returns false and the caller is
// expected to raise the CTA-wide abort flag, leave its loop and fall through to the common
// exit (TMEM free + return). Nothing here traps, asserts or spins without a limit.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fo {

// Wall-clock bound of a single wait (ns). Legitimate waits are micro- to milliseconds.
constexpr uint64_t kWaitLimitNs = 2000000000ull;
constexpr uint32_t kWaitParkNs = 20000u;  // suspend-time hint of one parked test

// Device status codes written to the status word that every launch receives.
enum DevStatus : int {
  kDevOk = 0,
  kDevWaitTimeout = 1,   // a bounded mbarrier wait ran out
  kDevBadIndex = 2,      // a work-list / indptr entry was out of range
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xffffffff;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// The test with a suspend-time hint: the hardware parks the thread until the phase completes or the hint
// (nanoseconds) runs out. A parked warp takes no issue slots from the warps of its scheduler that work and
// wakes as soon as the phase completes; polling loops (with or without nanosleep) measured 4-6 % slower
// on the attention kernel.
__device__ __forceinline__ bool mbar_try_wait_parked(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}

// Bounded wait for the phase with the given parity. `abort_flag` is a CTA-shared word: when any
// role raises it every other waiter gives up at its next check, so the whole CTA drains to its exit.
// The clock and the flag are only looked at when a parked test has run out of its hint.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait_parked(bar, parity, kWaitParkNs)) return true;
  const uint64_t t0 = global_timer_ns();
  while (true) {
    if (mbar_try_wait_parked(bar, parity, kWaitParkNs)) return true;
    if (*abort_flag != 0) return false;
    if (global_timer_ns() - t0 > kWaitLimitNs) {
      *abort_flag = 1;
      return false;
    }
  }
}

// Bounded wait that polls instead of parking: for the one thread whose wake-up time is on the critical path of a
// pipeline (an MMA issuer waiting for its operand). The clock and the abort flag are looked at every 64 polls.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  uint64_t t0 = 0;
  for (uint32_t n = 0;; ++n) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((n & 63u) == 63u) {
      if (*abort_flag != 0) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// The same for a whole warp that goes on to warp-collective instructions (tcgen05.ld, __syncwarp): lane 0
// waits and the outcome is broadcast, so that a wait that runs out never leaves the lanes of a warp on
// different sides of it. All 32 lanes must call it.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// ---------------------------------------------------------------------------------------------
// TMA tiled loads (no multicast anywhere in this library)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x,
                                            int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], "
      "[%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// TMA tiled store (shared -> global), bulk-group completion.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tmap, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* tmap, const void* smem_src, int x, int y,
                                             int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05: TMEM allocation
// ---------------------------------------------------------------------------------------------
// Warp-collective. `slot` is a shared-memory word that receives the TMEM base address.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// tcgen05: descriptors
// ---------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor (64 bit). Fields: start address >> 4 in [0,14), leading byte
// offset >> 4 in [16,30), stride byte offset >> 4 in [32,46), version = 1 in [46,48),
// layout (swizzle) type in [61,64) with 2 = 128-byte swizzle.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// Instruction descriptor for kind::f16 with bf16 (or f16) inputs and fp32 accumulation.
// a_mn / b_mn: 0 = operand is K-major in shared memory, 1 = MN-major.
__host__ __device__ constexpr uint32_t make_idesc_f16(int M, int N, bool in_bf16, int a_mn, int b_mn) {
  return (1u << 4)                                   // D format: f32
         | ((in_bf16 ? 1u : 0u) << 7)                // A format
         | ((in_bf16 ? 1u : 0u) << 10)               // B format
         | (static_cast<uint32_t>(a_mn) << 15)       // A major
         | (static_cast<uint32_t>(b_mn) << 16)       // B major
         | (static_cast<uint32_t>(N >> 3) << 17)     // N / 8
         | (static_cast<uint32_t>(M >> 4) << 24);    // M / 16
}

// ---------------------------------------------------------------------------------------------
// tcgen05: MMA issue (single thread) and commit
// ---------------------------------------------------------------------------------------------
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Variants with the accumulate flag fixed at compile time (no predicate set-up on the issuing thread).
template <bool kAccumulate>
__device__ __forceinline__ void umma_ss_c(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
  if (kAccumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.eq.b32 p, 0, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc)
        : "memory");
  } else {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, 0, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc)
        : "memory");
  }
}
template <bool kAccumulate>
__device__ __forceinline__ void umma_ts_c(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
  if (kAccumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.eq.b32 p, 0, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc)
        : "memory");
  } else {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, 0, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc)
        : "memory");
  }
}
// ---------------------------------------------------------------------------------------------
// Batched issue. A single thread feeds the tensor pipe, so the instruction count between two
// tcgen05.mma matters: rebuilding 64-bit descriptors and predicates in C++ costs ~100 clocks per MMA,
// more than a 128x128x16 MMA takes to execute (64). These helpers issue a whole K = 64 / K = 128
// group from one asm block; the descriptors' high words are constant and only the low words (which
// hold the 14-bit start address) vary.
// ---------------------------------------------------------------------------------------------
#define FO_MMA_SS(LA, LB, P) \
  "mov.b64 da, {" LA ", %1}; mov.b64 db, {" LB ", %2}; tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, " P ";\n"
#define FO_MMA_TS(TA, LB, P) \
  "mov.b64 db, {" LB ", %1}; tcgen05.mma.cta_group::1.kind::f16 [%0], [" TA "], db, %2, " P ";\n"

// 8 x (D[tmem] (+)= A[smem] * B[smem]); the first instruction accumulates iff `acc_first`.
__device__ __forceinline__ void umma_ss_x8(uint32_t d_tmem, uint32_t a_hi, uint32_t b_hi, uint32_t idesc,
                                           uint32_t acc_first, const uint32_t (&la)[8], const uint32_t (&lb)[8]) {
  asm volatile(
      "{\n"
      ".reg .pred p0, p1;\n"
      ".reg .b64 da, db;\n"
      "setp.ne.b32 p0, %4, 0;\n"
      "setp.eq.b32 p1, 0, 0;\n"
      FO_MMA_SS("%5", "%13", "p0") FO_MMA_SS("%6", "%14", "p1") FO_MMA_SS("%7", "%15", "p1")
      FO_MMA_SS("%8", "%16", "p1") FO_MMA_SS("%9", "%17", "p1") FO_MMA_SS("%10", "%18", "p1")
      FO_MMA_SS("%11", "%19", "p1") FO_MMA_SS("%12", "%20", "p1")
      "}\n" ::"r"(d_tmem),
      "r"(a_hi), "r"(b_hi), "r"(idesc), "r"(acc_first), "r"(la[0]), "r"(la[1]), "r"(la[2]), "r"(la[3]), "r"(la[4]),
      "r"(la[5]), "r"(la[6]), "r"(la[7]), "r"(lb[0]), "r"(lb[1]), "r"(lb[2]), "r"(lb[3]), "r"(lb[4]), "r"(lb[5]),
      "r"(lb[6]), "r"(lb[7])
      : "memory");
}
// 4 x (D[tmem] (+)= A[smem] * B[smem])
__device__ __forceinline__ void umma_ss_x4(uint32_t d_tmem, uint32_t a_hi, uint32_t b_hi, uint32_t idesc,
                                           uint32_t acc_first, const uint32_t* la, const uint32_t* lb) {
  asm volatile(
      "{\n"
      ".reg .pred p0, p1;\n"
      ".reg .b64 da, db;\n"
      "setp.ne.b32 p0, %4, 0;\n"
      "setp.eq.b32 p1, 0, 0;\n"
      FO_MMA_SS("%5", "%9", "p0") FO_MMA_SS("%6", "%10", "p1") FO_MMA_SS("%7", "%11", "p1") FO_MMA_SS("%8", "%12", "p1")
      "}\n" ::"r"(d_tmem),
      "r"(a_hi), "r"(b_hi), "r"(idesc), "r"(acc_first), "r"(la[0]), "r"(la[1]), "r"(la[2]), "r"(la[3]), "r"(lb[0]),
      "r"(lb[1]), "r"(lb[2]), "r"(lb[3])
      : "memory");
}
// 8 x (D[tmem] (+)= A[tmem] * B[smem]); A advances by ta[i] columns.
__device__ __forceinline__ void umma_ts_x8(uint32_t d_tmem, uint32_t b_hi, uint32_t idesc, uint32_t acc_first,
                                           const uint32_t (&ta)[8], const uint32_t (&lb)[8]) {
  asm volatile(
      "{\n"
      ".reg .pred p0, p1;\n"
      ".reg .b64 db;\n"
      "setp.ne.b32 p0, %3, 0;\n"
      "setp.eq.b32 p1, 0, 0;\n"
      FO_MMA_TS("%4", "%12", "p0") FO_MMA_TS("%5", "%13", "p1") FO_MMA_TS("%6", "%14", "p1") FO_MMA_TS("%7", "%15", "p1")
      FO_MMA_TS("%8", "%16", "p1") FO_MMA_TS("%9", "%17", "p1") FO_MMA_TS("%10", "%18", "p1") FO_MMA_TS("%11", "%19", "p1")
      "}\n" ::"r"(d_tmem),
      "r"(b_hi), "r"(idesc), "r"(acc_first), "r"(ta[0]), "r"(ta[1]), "r"(ta[2]), "r"(ta[3]), "r"(ta[4]), "r"(ta[5]),
      "r"(ta[6]), "r"(ta[7]), "r"(lb[0]), "r"(lb[1]), "r"(lb[2]), "r"(lb[3]), "r"(lb[4]), "r"(lb[5]), "r"(lb[6]),
      "r"(lb[7])
      : "memory");
}

// 4 x (D[tmem] (+)= A[tmem] * B[smem]); A advances by ta[i] columns.
__device__ __forceinline__ void umma_ts_x4(uint32_t d_tmem, uint32_t b_hi, uint32_t idesc, uint32_t acc_first,
                                           const uint32_t* ta, const uint32_t* lb) {
  asm volatile(
      "{\n"
      ".reg .pred p0, p1;\n"
      ".reg .b64 db;\n"
      "setp.ne.b32 p0, %3, 0;\n"
      "setp.eq.b32 p1, 0, 0;\n"
      FO_MMA_TS("%4", "%8", "p0") FO_MMA_TS("%5", "%9", "p1") FO_MMA_TS("%6", "%10", "p1") FO_MMA_TS("%7", "%11", "p1")
      "}\n" ::"r"(d_tmem),
      "r"(b_hi), "r"(idesc), "r"(acc_first), "r"(ta[0]), "r"(ta[1]), "r"(ta[2]), "r"(ta[3]), "r"(lb[0]), "r"(lb[1]),
      "r"(lb[2]), "r"(lb[3])
      : "memory");
}

// Arrive (count 1) on `bar` once every tcgen05 op issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05: TMEM <-> registers. Shape 32x32b: thread t of the warp touches TMEM lane
// (lane base of the warp's quadrant) + t, N consecutive 32-bit columns.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// small math helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Packed fp32 pairs (one instruction for two lanes of work) and the three-input max: the softmax warps
// are bound by instruction issue, so halving the instruction count of their inner loops matters.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

}  // namespace fo
