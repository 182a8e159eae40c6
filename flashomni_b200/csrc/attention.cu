// Block-sparse prefill attention on tcgen05 / TMEM / TMA, driven by compacted work lists.
//
// What it computes (reference: include/flashomni/attention/prefill.cuh:1203-1531): for every work
// item (b, h, qb) -- an active 128-row q-block of one head -- and its ascending list of kept
// 128-row kv-blocks,  O[rows, h, :] = softmax_over_kept(Q K^T * sm_scale) V,  fp32 accumulation,
// base-2 online softmax, output rounded to the input dtype. q-blocks that are not in the list are
// never written. An item with an empty list writes zeros (lse = -5e4), like the reference.
//
// One persistent CTA per SM walks its items (dealt round-robin in longest-first order) as ONE
// sequence of kv blocks g = 0, 1, 2, ... and software-pipelines it three deep:
//
//   round r:   tensor pipe   S[(r+1)&1] = Q K_{r+1}^T   interleaved with   O += P[(r-1)&1] V_{r-1}
//              softmax warps block r: S[r&1] -> P[r&1]
//
// TMEM (512 columns): S0, S1 (fp32, 128 each), O (fp32, 128), P0, P1 (16 bit, 64 each). Because S is
// double-buffered and P does not alias S, the QK and PV batches of a round are independent of each
// other and of the softmax of the block in between; they are issued by two different threads, because
// a thread that issues a batch is held until the batch has drained.
// Warps: 0-15 softmax / O-rescale / epilogue (4 threads per q row: TMEM lane = row, 32 columns
// each), 16 TMA producer (double-buffered Q tile + two-slot FIFOs of 32 KB K and V tiles, K running two
// blocks ahead of V), 17 QK issuer, 18 PV issuer. Every mbarrier wait is bounded.
#include <cuda_fp16.h>

#include "internal.h"

#ifndef FO_POLY_EVERY
#define FO_POLY_EVERY 4
#endif

namespace fo {
namespace {

constexpr int kBQ = 128, kBKV = 128, kD = 128;
constexpr int kTileBytes = 128 * kD * 2;    // 32 KB: a 128-row tile of Q, K or V
constexpr int kHalfBytes = kTileBytes / 2;  // one 64-column half (one swizzle-atom column)
constexpr int kRingK = 2, kRingV = 2;  // separate FIFOs of 32 KB tiles for K and V
constexpr int kRing = kRingK + kRingV;
constexpr int kQBufs = 2;
constexpr int kSoftmaxWarps = 16;
constexpr int kWarpProducer = kSoftmaxWarps;
constexpr int kWarpQK = kSoftmaxWarps + 1;      // issues S = Q K^T
constexpr int kWarpPV = kSoftmaxWarps + 2;      // issues O += P V
constexpr int kWarpMma = kWarpQK;               // owner of the TMEM allocation
constexpr int kThreads = (kWarpPV + 1) * 32;    // 608
constexpr int kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 256, kColP = 384;
#ifndef FO_TWO_BLOCK_STEPS
#define FO_TWO_BLOCK_STEPS 0
#endif
constexpr bool kTwoBlockSteps = FO_TWO_BLOCK_STEPS != 0;  // softmax handles two blocks of an item per step
constexpr int kPolyEvery = FO_POLY_EVERY;   // 1 in (2 * kPolyEvery) exponentials is computed by polynomial
constexpr float kRescaleThreshold = 8.0f;  // lazy rescale: keep the old max while exp2 stays <= 2^8

struct Tail {
  uint64_t q_full[kQBufs], q_empty[kQBufs];
  uint64_t k_full[kRingK], k_empty[kRingK], v_full[kRingV], v_empty[kRingV];
  uint64_t s_full[2], s_free[2];  // S buffer written by QK / copied to registers by the softmax
  uint64_t p_full[2], pv_done[2];  // indexed by block parity, so that no waiter can fall two phases behind
  uint64_t o_full, o_free;
  uint64_t xbar;          // barrier among the softmax warps (bounded, unlike bar.sync)
  uint32_t tmem_base;
  int abort_flag;
  float xmax[2][4][128];  // [block parity][column quarter][row]: partial row maxima
  float xsum[4][128];     // [column quarter][row]: partial row sums
};
constexpr int kSmemBytes = (kQBufs + kRing) * kTileBytes + 1024 + static_cast<int>(sizeof(Tail));

#ifdef FO_ATTN_TRACE
// Development aid (only with -DFO_ATTN_TRACE): CTA 0 records clock64() at pipeline events.
__device__ long long g_trace[8][512];
__device__ __forceinline__ void trace(int ev, int idx) {
  if (blockIdx.x == 0 && idx >= 0 && idx < 512) g_trace[ev][idx] = clock64();
}
#define FO_TRACE(ev, idx) trace(ev, idx)
#else
#define FO_TRACE(ev, idx)
#endif


// Walks the CTA's share of the schedule as a flat sequence of kv blocks.
struct BlockSeq {
  int pos, stride, n_items;
  int item_no;   // index among this CTA's non-empty items (selects the Q buffer, o_full / o_free phases)
  int b, h, qb, n, j;
  int kvb, kvb_next;  // kv-block index of the current block; the next one is fetched a block early
  const int32_t* kv;
  __device__ __forceinline__ void init(int start, int stride_, int n_items_) {
    pos = start; stride = stride_; n_items = n_items_; item_no = -1; n = 0; j = 0; kv = nullptr;
    b = h = qb = 0; kvb = kvb_next = 0;
  }
  // Advances to the next block; `on_empty(b, h, qb)` is called for every item without kv blocks that
  // is passed on the way. Returns false at the end of the sequence.
  template <class F>
  __device__ __forceinline__ bool next(const AttnArgs& a, F&& on_empty) {
    if (j + 1 < n) {
      ++j;
      kvb = kvb_next;
      if (j + 1 < n) kvb_next = kv[j + 1];
      return true;
    }
    while (pos < n_items) {
      const int it = a.order[pos];
      pos += stride;
      const int4 rec = *reinterpret_cast<const int4*>(a.items + 4 * it);
      if (rec.w <= 0) { on_empty(rec.x, rec.y, rec.z); continue; }
      b = rec.x; h = rec.y; qb = rec.z; n = rec.w; j = 0;
      kv = a.kv_idx + a.kv_ptr[it];
      kvb = kv[0];
      if (n > 1) kvb_next = kv[1];
      ++item_no;
      return true;
    }
    n = 0; j = 0;
    return false;
  }
  __device__ __forceinline__ bool first() const { return j == 0; }
  __device__ __forceinline__ bool last() const { return j == n - 1; }
};

template <bool kBf16>
__global__ void __launch_bounds__(kThreads, 1) attention_kernel(const __grid_constant__ AttnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* smem_q = smem;                           // kQBufs tiles
  uint8_t* smem_ring = smem + kQBufs * kTileBytes;  // kRing tiles
  Tail* tail = reinterpret_cast<Tail*>(smem + (kQBufs + kRing) * kTileBytes);
  volatile int* abort_flag = &tail->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kQBufs; ++i) { mbar_init(&tail->q_full[i], 1); mbar_init(&tail->q_empty[i], 1); }
    for (int i = 0; i < kRingK; ++i) { mbar_init(&tail->k_full[i], 1); mbar_init(&tail->k_empty[i], 1); }
    for (int i = 0; i < kRingV; ++i) { mbar_init(&tail->v_full[i], 1); mbar_init(&tail->v_empty[i], 1); }
    mbar_init(&tail->s_full[0], 1);
    mbar_init(&tail->s_full[1], 1);
    mbar_init(&tail->s_free[0], kSoftmaxWarps);
    mbar_init(&tail->s_free[1], kSoftmaxWarps);
    for (int i = 0; i < 2; ++i) { mbar_init(&tail->p_full[i], kSoftmaxWarps); mbar_init(&tail->pv_done[i], 1); }
    mbar_init(&tail->o_full, 1);
    mbar_init(&tail->o_free, kSoftmaxWarps);
    mbar_init(&tail->xbar, kSoftmaxWarps);
    tail->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kWarpProducer && lane == 0) {
    tma_prefetch_desc(&a.tmap_q);
    tma_prefetch_desc(&a.tmap_k);
    tma_prefetch_desc(&a.tmap_v);
  }
  if (warp == kWarpMma) {
    tmem_alloc(&tail->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tail->tmem_base;

  int n_items = a.counters[0];
  if (n_items < 0) n_items = 0;
  const int sched_start = static_cast<int>(blockIdx.x), sched_stride = static_cast<int>(gridDim.x);
  auto ignore_empty = [](int, int, int) {};

  if (warp == kWarpProducer) {
    // ------------------------------------------------------------------ TMA producer
    // Push order: K_0, K_1, then (K_t, V_{t-2}) for t = 2, 3, ... and the last two V (K runs two blocks ahead).
    if (lane == 0) {
      BlockSeq seq;
      seq.init(sched_start, sched_stride, n_items);
      uint32_t nk = 0, nv = 0;           // K / V tiles pushed so far
      uint32_t q_uses[kQBufs] = {0, 0};  // loads issued per Q buffer
      int hist_row[3] = {0, 0, 0}, hist_head[3] = {0, 0, 0};  // kv row / kv head of blocks t, t-1, t-2
      int pending_v = 0;                 // number of blocks whose V has not been pushed yet (0..2)
      int kv_row0 = 0;                   // first kv row of the current item's request
      bool ok = true;
      auto push = [&](bool is_v, int head, int row) -> bool {
        const uint32_t n = is_v ? nv : nk;
        const int slot = static_cast<int>(n % (is_v ? kRingV : kRingK));
        const uint32_t phase = (n / (is_v ? kRingV : kRingK)) & 1u;
        uint64_t* empty = is_v ? &tail->v_empty[slot] : &tail->k_empty[slot];
        uint64_t* full = is_v ? &tail->v_full[slot] : &tail->k_full[slot];
        if (!mbar_wait(empty, phase ^ 1u, abort_flag)) return false;
        uint8_t* dst = smem_ring + (is_v ? kRingK + slot : slot) * kTileBytes;
        const CUtensorMap* tm = is_v ? &a.tmap_v : &a.tmap_k;
        mbar_expect_tx(full, kTileBytes);
        tma_load_3d(dst, tm, full, 0, head, row);
        tma_load_3d(dst + kHalfBytes, tm, full, 64, head, row);
        if (is_v) ++nv; else ++nk;
        return true;
      };
      while (ok) {
        const bool have = seq.next(a, ignore_empty);
        if (have) {
          const int hq = seq.h - a.head_begin;
          const int hk = hq / a.group_size;
          if (seq.first()) kv_row0 = a.kv_indptr[seq.b];
          if (seq.first()) {  // new item: its Q tile goes to buffer item_no & 1
            const int qb_i = seq.item_no & 1;
            if (!mbar_wait(&tail->q_empty[qb_i], (q_uses[qb_i] & 1u) ^ 1u, abort_flag)) { ok = false; break; }
            ++q_uses[qb_i];
            const int q_row = a.qo_indptr[seq.b] + seq.qb * kBQ;
            uint8_t* dst = smem_q + qb_i * kTileBytes;
            mbar_expect_tx(&tail->q_full[qb_i], kTileBytes);
            tma_load_3d(dst, &a.tmap_q, &tail->q_full[qb_i], 0, hq, q_row);
            tma_load_3d(dst + kHalfBytes, &a.tmap_q, &tail->q_full[qb_i], 64, hq, q_row);
          }
          hist_row[2] = hist_row[1]; hist_row[1] = hist_row[0];
          hist_head[2] = hist_head[1]; hist_head[1] = hist_head[0];
          hist_row[0] = kv_row0 + seq.kvb * kBKV;
          hist_head[0] = hk;
          if (!push(false, hist_head[0], hist_row[0])) { ok = false; break; }
          if (pending_v == 2) {
            if (!push(true, hist_head[2], hist_row[2])) { ok = false; break; }
          } else {
            ++pending_v;
          }
        } else {
          // drain: V of the last (up to two) blocks, oldest first
          if (pending_v == 2) ok = push(true, hist_head[1], hist_row[1]);
          if (ok && pending_v >= 1) ok = push(true, hist_head[0], hist_row[0]);
          break;
        }
      }
    }
  } else if (warp == kWarpQK) {
    // ------------------------------------------------------------------ QK issuer: S[g&1] = Q K_g^T
    // Two threads feed the tensor pipe (this one and the PV issuer): an issuing thread is blocked while
    // its batch drains, so with a single issuer the pipe would idle during that thread's bookkeeping.
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(kBQ, kBKV, kBf16, 0, 0);
      // descriptors: constant high word (K-major, 128-byte swizzle), low word holds the address
      const uint64_t d0 = make_smem_desc_sw128(smem_u32(smem_q), 16, 1024);
      const uint32_t hi = static_cast<uint32_t>(d0 >> 32);
      const uint32_t q_lo0 = static_cast<uint32_t>(d0);
      const uint32_t k_lo0 = static_cast<uint32_t>(make_smem_desc_sw128(smem_u32(smem_ring), 16, 1024));
      BlockSeq seq;
      seq.init(sched_start, sched_stride, n_items);
      uint32_t g = 0, nk = 0;
      uint32_t q_uses[kQBufs] = {0, 0};
      bool ok = true;
      while (ok && seq.next(a, ignore_empty)) {
        const uint32_t sb = g & 1u;
        const int qb_i = seq.item_no & 1;
        // S[sb] is free once the softmax has copied block g-2 into registers
        if (g >= 2u && !mbar_wait(&tail->s_free[sb], ((g - 2u) >> 1) & 1u, abort_flag)) { ok = false; break; }
        if (seq.first()) {
          if (!mbar_wait(&tail->q_full[qb_i], q_uses[qb_i] & 1u, abort_flag)) { ok = false; break; }
          ++q_uses[qb_i];
        }
        const int slot = static_cast<int>(nk % kRingK);
        if (!mbar_wait(&tail->k_full[slot], (nk / kRingK) & 1u, abort_flag)) { ok = false; break; }
        ++nk;
        tc_fence_after_sync();
        const uint32_t q_lo = q_lo0 + static_cast<uint32_t>((qb_i * kTileBytes) >> 4);
        const uint32_t k_lo = k_lo0 + static_cast<uint32_t>((slot * kTileBytes) >> 4);
        uint32_t la[8], lb[8];
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // 16 elements further along K: +32 B inside a 64-column half, +16 KB for the second half
          const uint32_t off = static_cast<uint32_t>(((kk >> 2) * kHalfBytes + (kk & 3) * 32) >> 4);
          la[kk] = q_lo + off;
          lb[kk] = k_lo + off;
        }
        umma_ss_x8(tmem_base + kColS + sb * 128u, hi, hi, idesc_qk, 0u, la, lb);
        umma_commit(&tail->s_full[sb]);
        umma_commit(&tail->k_empty[slot]);
        if (seq.last()) umma_commit(&tail->q_empty[qb_i]);
        ++g;
      }
    }
  } else if (warp == kWarpPV) {
    // ------------------------------------------------------------------ PV issuer: O (+)= P[g&1] V_g
    if (lane == 0) {
      constexpr uint32_t idesc_pv = make_idesc_f16(kBQ, kD, kBf16, 0, 1);
      // V is MN-major: its two 64-column halves are 16 KB apart (leading byte offset)
      const uint64_t d0 = make_smem_desc_sw128(smem_u32(smem_ring + kRingK * kTileBytes), kHalfBytes, 1024);
      const uint32_t hi = static_cast<uint32_t>(d0 >> 32), v_lo0 = static_cast<uint32_t>(d0);
      BlockSeq seq;
      seq.init(sched_start, sched_stride, n_items);
      uint32_t g = 0, nv = 0, items_started = 0;
      bool ok = true;
      while (ok && seq.next(a, ignore_empty)) {
        const uint32_t sb = g & 1u;
        if (!mbar_wait(&tail->p_full[sb], (g >> 1) & 1u, abort_flag)) { ok = false; break; }
        if (seq.first() && items_started > 0) {  // O must have been drained by the previous item's epilogue
          if (!mbar_wait(&tail->o_free, (items_started - 1u) & 1u, abort_flag)) { ok = false; break; }
        }
        const int slot = static_cast<int>(nv % kRingV);
        if (!mbar_wait(&tail->v_full[slot], (nv / kRingV) & 1u, abort_flag)) { ok = false; break; }
        ++nv;
        tc_fence_after_sync();
        const uint32_t tmem_p = tmem_base + kColP + sb * 64u;
        const uint32_t v_lo = v_lo0 + static_cast<uint32_t>((slot * kTileBytes) >> 4);
        uint32_t ta[8], lb[8];
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // 16 kv rows further = 16 * 128 B in the V tile, 8 columns further in the 16-bit P tile
          ta[kk] = tmem_p + static_cast<uint32_t>(kk * 8);
          lb[kk] = v_lo + static_cast<uint32_t>((kk * 2048) >> 4);
        }
        umma_ts_x8(tmem_base + kColO, hi, idesc_pv, seq.first() ? 0u : 1u, ta, lb);
        umma_commit(&tail->pv_done[sb]);
        umma_commit(&tail->v_empty[slot]);
        if (seq.last()) umma_commit(&tail->o_full);
        if (seq.first()) ++items_started;
        ++g;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue warps 0..15
    // Four threads per q row: thread (quadrant = warp & 3, column quarter cq = warp >> 2) owns columns
    // [32cq, 32cq+32) of S, P and O for row 32*quadrant + lane.
    const int cq = warp >> 2;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t col0 = static_cast<uint32_t>(32 * cq);
    const uint32_t tmem_s0 = tmem_base + lane_base + kColS + col0;
    const uint32_t tmem_p0 = tmem_base + lane_base + kColP + (col0 >> 1);
    const uint32_t tmem_o = tmem_base + lane_base + kColO + col0;
    const int r_in_tile = (warp & 3) * 32 + lane;
    const bool tracer = (threadIdx.x == 0);
    (void)tracer;
    uint16_t* o16 = reinterpret_cast<uint16_t*>(a.o);
    bool ok = true;
    uint32_t xbar_phase = 0;
    // Barrier among the 16 softmax warps built on an mbarrier, so that it is bounded like every other
    // wait of the kernel (a warp that gave up elsewhere cannot leave the others parked forever).
    auto softmax_bar = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(&tail->xbar);
      const bool r = mbar_wait(&tail->xbar, xbar_phase, abort_flag);
      xbar_phase ^= 1u;
      return r;
    };

    struct RowCtx {  // where an item's rows live in global memory
      uint16_t* orow;
      float* lse;
      bool row_ok;
    };
    auto row_ctx = [&](int b, int h, int qb) -> RowCtx {
      RowCtx c;
      const int hq = h - a.head_begin;
      const int q0 = a.qo_indptr[b];
      const int q_len = a.qo_indptr[b + 1] - q0;
      const int row_in_req = qb * kBQ + r_in_tile;
      c.row_ok = row_in_req < q_len;
      const int64_t grow = static_cast<int64_t>(q0) + row_in_req;
      c.orow = o16 + grow * a.o_stride_n + static_cast<int64_t>(hq) * a.o_stride_h + col0;
      c.lse = (a.lse != nullptr && cq == 0) ? a.lse + grow * a.lse_stride_n + hq : nullptr;
      return c;
    };
    auto on_empty = [&](int b, int h, int qb) {  // active q-block that keeps nothing: zeros, lse = -5e4
      const RowCtx c = row_ctx(b, h, qb);
      if (c.row_ok) {
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(c.orow)[i] = z;
        if (c.lse != nullptr) *c.lse = -5e4f;
      }
    };

    BlockSeq seq;
    seq.init(sched_start, sched_stride, n_items);
    uint32_t g = 0;           // global block index
    uint32_t s_uses[2] = {0, 0};
    uint32_t items_done = 0;  // epilogues completed
    float m_used = -INFINITY;
    uint64_t l2 = 0;  // running row sum of this thread's columns, as a packed pair of partial sums
    // an item whose last block has been handed over and whose O is still being accumulated
    bool pend = false;
    float pend_l = 0.f, pend_m = 0.f;
    RowCtx pend_ctx;
    pend_ctx.orow = nullptr; pend_ctx.lse = nullptr; pend_ctx.row_ok = false;

    auto epilogue = [&]() -> bool {
      // the four quarters of a row exchange their partial sums
      float* xs = tail->xsum[0];
      xs[cq * kBQ + r_in_tile] = pend_l;
      if (!softmax_bar()) return false;
      const float lsum = xs[r_in_tile] + xs[kBQ + r_in_tile] + xs[2 * kBQ + r_in_tile] + xs[3 * kBQ + r_in_tile];
      if (!mbar_wait(&tail->o_full, items_done & 1u, abort_flag)) return false;
      tc_fence_after_sync();
      const float inv_l = lsum > 0.f ? __frcp_rn(lsum) : 0.f;
      uint32_t v[32];
      tmem_ld_x32(tmem_o, v);
      tmem_wait_ld();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tail->o_free);  // O may be overwritten by the next item
      if (pend_ctx.row_ok) {
        uint4 outv[4];
        uint32_t* o32 = reinterpret_cast<uint32_t*>(outv);
#pragma unroll
        for (int t = 0; t < 16; ++t) {
          const float x0 = __uint_as_float(v[2 * t]) * inv_l, x1 = __uint_as_float(v[2 * t + 1]) * inv_l;
          o32[t] = kBf16 ? pack_bf16x2(x0, x1) : pack_f16x2(x0, x1);
        }
        uint4* dst = reinterpret_cast<uint4*>(pend_ctx.orow);
#pragma unroll
        for (int t = 0; t < 4; ++t) dst[t] = outv[t];
        if (pend_ctx.lse != nullptr) *pend_ctx.lse = (lsum > 0.f) ? (log2f(lsum) + pend_m) : -5e4f;
      }
      ++items_done;
      pend = false;
      return softmax_bar();  // xsum is reused by the next epilogue
    };

    int kv_len = 0;
    uint32_t step_no = 0;
    // One softmax step handles up to two consecutive blocks of an item (both S buffers): one max
    // exchange, one rescale decision and one hand-over for 256 kv columns.
    while (ok && seq.next(a, on_empty)) {
      if (seq.first()) {
        m_used = -INFINITY;
        l2 = 0;
        kv_len = a.kv_indptr[seq.b + 1] - a.kv_indptr[seq.b];
      }
      const bool step_first = seq.first();
      const int valid0 = kv_len - seq.kvb * kBKV - static_cast<int>(col0);  // valid columns of my quarter
      const bool two = kTwoBlockSteps && !seq.last();
      int valid1 = 0;
      if (two) {
        seq.next(a, on_empty);  // stays inside the item
        valid1 = kv_len - seq.kvb * kBKV - static_cast<int>(col0);
      }
      const uint32_t b0 = g & 1u, b1 = b0 ^ 1u;
      if (!mbar_wait(&tail->s_full[b0], s_uses[b0] & 1u, abort_flag)) { ok = false; break; }
      ++s_uses[b0];
      if (two) {
        if (!mbar_wait(&tail->s_full[b1], s_uses[b1] & 1u, abort_flag)) { ok = false; break; }
        ++s_uses[b1];
      }
      if (tracer) FO_TRACE(4, static_cast<int>(g));  // S ready seen by softmax
      tc_fence_after_sync();
      uint32_t s0[32], s1[32];
      tmem_ld_x32(tmem_s0 + b0 * 128u, s0);
      if (two) tmem_ld_x32(tmem_s0 + b1 * 128u, s1);
      tmem_wait_ld();
      if (tracer) FO_TRACE(0, static_cast<int>(g));  // S in registers
      // both S buffers are in registers: the QK of the blocks after next may overwrite them
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&tail->s_free[b0]);
        if (two) mbar_arrive(&tail->s_free[b1]);
      }
      float mx = -INFINITY;
      if (valid0 >= 32) {
#pragma unroll
        for (int t = 0; t < 16; ++t) mx = fmax3(mx, __uint_as_float(s0[2 * t]), __uint_as_float(s0[2 * t + 1]));
      } else {
#pragma unroll
        for (int t = 0; t < 32; ++t)
          if (t < valid0) mx = fmaxf(mx, __uint_as_float(s0[t]));
      }
      if (two) {
        if (valid1 >= 32) {
#pragma unroll
          for (int t = 0; t < 16; ++t) mx = fmax3(mx, __uint_as_float(s1[2 * t]), __uint_as_float(s1[2 * t + 1]));
        } else {
#pragma unroll
          for (int t = 0; t < 32; ++t)
            if (t < valid1) mx = fmaxf(mx, __uint_as_float(s1[t]));
        }
      }
      if (tracer) FO_TRACE(1, static_cast<int>(g));  // local max done
      float* xm = tail->xmax[step_no & 1u][0];
      xm[cq * kBQ + r_in_tile] = mx;
      if (!softmax_bar()) { ok = false; break; }
      if (tracer) FO_TRACE(5, static_cast<int>(g));  // max exchanged
      mx = fmaxf(fmaxf(xm[r_in_tile], xm[kBQ + r_in_tile]), fmaxf(xm[2 * kBQ + r_in_tile], xm[3 * kBQ + r_in_tile]));
      const float m_new = fmaxf(m_used, mx * a.sm_scale_log2);
      // ---- lazy rescale of l and O (warp-uniform decision; the TMEM round trip is warp-collective).
      // O is rescaled only after the PV of the previous block has completed.
      const bool need = (m_new - m_used) > kRescaleThreshold;  // true on an item's first block
      if (step_first) {
        m_used = m_new;
      } else if (__any_sync(0xffffffffu, need)) {
        // PV of block g-1 is completion number (g-1)/2 on the barrier of its parity
        if (!mbar_wait(&tail->pv_done[(g - 1u) & 1u], ((g - 1u) >> 1) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const float alpha = need ? ex2_approx(m_used - m_new) : 1.0f;
        if (need) m_used = m_new;
        l2 = ffma2(l2, pack_f32x2(alpha, alpha), 0ull);
        uint32_t v[32];
        tmem_ld_x32(tmem_o, v);
        tmem_wait_ld();
#pragma unroll
        for (int t = 0; t < 32; ++t) v[t] = __float_as_uint(__uint_as_float(v[t]) * alpha);
        tmem_st_x32(tmem_o, v);
      }
      // ---- P = exp2(S*scale - m_used), row sum, P (16 bit) to its own TMEM buffers
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
      const uint64_t scale2 = pack_f32x2(a.sm_scale_log2, a.sm_scale_log2);
      const uint64_t negm2 = pack_f32x2(neg_m, neg_m);
      auto exp_block = [&](const uint32_t (&s)[32], int valid, uint32_t (&pk)[16]) {
        if (valid >= 32) {
          // packed path: one FMA and one add per PAIR of columns; one pair in kPolyEvery takes the
          // polynomial exp2 (FMA pipe) for its second element, the rest use MUFU
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            const uint64_t x2 = ffma2(pack_f32x2(__uint_as_float(s[2 * t]), __uint_as_float(s[2 * t + 1])), scale2, negm2);
            float x0, x1;
            unpack_f32x2(x2, x0, x1);
            const float p0 = ex2_approx(x0);
            const float p1 = (t % kPolyEvery == 0) ? ex2_poly(x1) : ex2_approx(x1);
            l2 = fadd2(l2, pack_f32x2(p0, p1));
            pk[t] = kBf16 ? pack_bf16x2(p0, p1) : pack_f16x2(p0, p1);
          }
        } else {
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            float p0 = ex2_approx(fmaf(__uint_as_float(s[2 * t]), a.sm_scale_log2, neg_m));
            float p1 = ex2_approx(fmaf(__uint_as_float(s[2 * t + 1]), a.sm_scale_log2, neg_m));
            if (2 * t >= valid) p0 = 0.f;
            if (2 * t + 1 >= valid) p1 = 0.f;
            l2 = fadd2(l2, pack_f32x2(p0, p1));
            pk[t] = kBf16 ? pack_bf16x2(p0, p1) : pack_f16x2(p0, p1);
          }
        }
      };
      {
        uint32_t pk[16];
        exp_block(s0, valid0, pk);
        if (tracer) FO_TRACE(2, static_cast<int>(g));  // exponentials done
        // P[b0] was last read by the PV of block g-2
        if (g >= 2u && !mbar_wait(&tail->pv_done[b0], ((g - 2u) >> 1) & 1u, abort_flag)) { ok = false; break; }
        if (tracer) FO_TRACE(3, static_cast<int>(g));  // pv_done seen
        tmem_st_x16(tmem_p0 + b0 * 64u, pk);
      }
      if (two) {
        uint32_t pk[16];
        exp_block(s1, valid1, pk);
        if (g >= 1u && !mbar_wait(&tail->pv_done[b1], ((g - 1u) >> 1) & 1u, abort_flag)) { ok = false; break; }
        tmem_st_x16(tmem_p0 + b1 * 64u, pk);
      }
      tmem_wait_st();
      if (tracer) FO_TRACE(7, static_cast<int>(g));  // P stored
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&tail->p_full[b0]);
        if (two) mbar_arrive(&tail->p_full[b1]);
      }
      if (tracer) FO_TRACE(6, static_cast<int>(g));  // P handed over
      g += two ? 2u : 1u;
      ++step_no;
      // the previous item's epilogue runs one step late, so that its last PV overlaps this softmax
      if (pend) {
        if (!epilogue()) { ok = false; break; }
      }
      if (seq.last()) {
        pend = true;
        {
          float la, lb;
          unpack_f32x2(l2, la, lb);
          pend_l = la + lb;
        }
        pend_m = m_used;
        pend_ctx = row_ctx(seq.b, seq.h, seq.qb);
      }
    }
    if (ok && pend) epilogue();
  }

  // ------------------------------------------------------------------ common exit
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    if (threadIdx.x == 0) atomicExch(a.status, kDevWaitTimeout);
    __syncthreads();
  }
  if (warp == kWarpMma) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

#ifdef FO_ATTN_TRACE
extern "C" __attribute__((visibility("default"))) int fo_trace_dump(long long* host_dst) {
  return static_cast<int>(cudaMemcpyFromSymbol(host_dst, g_trace, sizeof(g_trace)));
}
#endif

cudaError_t launch_attention(const AttnArgs& a, int max_ctas, cudaStream_t stream) {
  if (max_ctas <= 0) return cudaSuccess;
  cudaError_t e;
  if (a.is_bf16) {
    e = cudaFuncSetAttribute(attention_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    attention_kernel<true><<<max_ctas, kThreads, kSmemBytes, stream>>>(a);
  } else {
    e = cudaFuncSetAttribute(attention_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    attention_kernel<false><<<max_ctas, kThreads, kSmemBytes, stream>>>(a);
  }
  return cudaGetLastError();
}

}  // namespace fo
