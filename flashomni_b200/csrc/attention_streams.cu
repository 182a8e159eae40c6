// Block-sparse prefill attention on tcgen05 / TMEM / TMA for launches with FEW work units: two streams of units per
// SM, kv lists cut into parts, partial results merged by the part that delivers last. (attention.cu holds the
// kernel for launches with many units: one unit at a time per SM, two softmax groups on alternate kv blocks.)
//
// What it computes (reference: include/flashomni/attention/prefill.cuh:1203-1531): for every work
// item (b, h, qb) -- an active 128-row q-block of one head -- and its ascending list of kept
// 128-row kv-blocks,  O[rows, h, :] = softmax_over_kept(Q K^T * sm_scale) V,  fp32 accumulation,
// base-2 online softmax, output rounded to the input dtype. q-blocks that are not in the list are
// never written. An item with an empty list writes zeros (lse = -5e4), like the reference.
//
// One persistent CTA per SM runs TWO independent streams of items, A and B. A stream owns a q tile in
// shared memory, one K and one V tile slot, an S and an O accumulator in TMEM (S_A, S_B, O_A, O_B = 512
// columns), a softmax warpgroup, a TMA producer thread and an MMA issuer thread, and walks its items as one
// sequence of kv blocks:
//
//   issuer     S = Q K_j^T                      ... O (+)= P V_j,  then S = Q K_{j+1}^T ...
//   softmax             S -> registers -> P (16 bit, written over S)
//
// Inside a stream these steps depend on each other (P lives in S's columns, so the next Q K^T follows the
// P V that reads it); the tensor pipe and the exponential unit are kept busy by the OTHER stream, which is
// in the opposite phase. Nothing is shared between the streams but the hardware: no running maximum handed
// between groups, no exchange between threads of a row (one thread owns a whole row of S: TMEM lane = row).
// Items are positions of the work list's processing order, handed out dynamically: the first 2 x grid
// positions go to the streams in launch order, the rest are drawn from a device-wide cursor by the stream's
// producer and passed to its other roles through a small shared-memory queue.
// Warps: 0-3 softmax A, 4-7 softmax B (`setmaxnreg` gives them 224 registers: a row of S is held in
// registers, read from TMEM once), 8 / 9 TMA producers of A / B (Q, K, V tiles of 32 KB; K and V one slot
// each), 10 / 11 MMA issuers of A / B. Whole q-blocks leave through a 16 KB staging area per stream (two
// rounds of 64 columns, 128-byte swizzle) and TMA stores. Every mbarrier wait is bounded.
#include <cuda_fp16.h>

#include "internal.h"

#ifndef FO_ROT_STEP
#define FO_ROT_STEP 5
#endif

namespace fo {
namespace {

constexpr int kBQ = 128, kBKV = 128, kD = 128;
constexpr int kTileBytes = 128 * kD * 2;    // 32 KB: a 128-row tile of Q, K or V
constexpr int kHalfBytes = kTileBytes / 2;  // one 64-column half (one swizzle-atom column)
constexpr int kStreams = 2;
constexpr int kWgWarps = 4;                 // warps of a softmax warpgroup (one thread per q row)
constexpr int kSoftmaxWarps = kStreams * kWgWarps;
constexpr int kWarpProducer = kSoftmaxWarps;          // + stream
constexpr int kWarpIssuer = kSoftmaxWarps + kStreams;  // + stream
constexpr int kWarpTmem = kWarpIssuer;                 // owner of the TMEM allocation
constexpr int kThreads = (kSoftmaxWarps + 2 * kStreams) * 32;  // 384
constexpr int kRegsSoftmax = 224, kRegsOther = 56;  // register split between the warpgroups (setmaxnreg)
// setmaxnreg.inc waits until the registers are free in the pool the CTA was launched with (threads x the
// per-thread count the compiler settles on for this block size): a split that asks for more never returns.
constexpr int kRegsAtLaunch = (65536 / kThreads) / 8 * 8;
static_assert(kSoftmaxWarps * 32 * kRegsSoftmax + (kThreads - kSoftmaxWarps * 32) * kRegsOther <= kThreads * kRegsAtLaunch,
              "register split exceeds the CTA's register pool");
constexpr int kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 256;  // + 128 * stream; P (16 bit) occupies the first 64 columns of S
constexpr int kRotStep = FO_ROT_STEP;       // q-block qb starts its kv list at entry (qb * kRotStep) mod length
constexpr int kItemQ = 4;                   // entries of a stream's item queue
constexpr int kItemReaders = kWgWarps + 1;  // the stream's softmax warps and its MMA issuer
constexpr float kRescaleThreshold = 8.0f;   // lazy rescale: keep the old max while exp2 stays <= 2^8
#ifndef FO_SPLIT_P
#define FO_SPLIT_P 1
#endif
constexpr bool kSplitP = FO_SPLIT_P != 0;  // hand P to the P V in two halves
constexpr int kStageBytes = 128 * 128;      // output staging of a stream: 128 rows x 64 columns

struct StreamBars {
  // One mbarrier per EVENT, waited for by every role that depends on it (a tcgen05.commit between two MMA batches
  // costs tensor-pipe time, so a turn commits twice: once behind its P V, once behind its Q K^T).
  uint64_t q_full, k_full, v_full;  // TMA loads landed
  uint64_t s_full;    // Q K^T of a block complete: S may be read; the K slot (and after an item's last block the Q slot) is free
  uint64_t p_half[2]; // P written by the softmax warps, kv columns 0-63 / 64-127 of the block (count = warps)
  uint64_t pv_done;   // P V of a block complete: the V slot is free, O may be rescaled, after an item's last block O is final
  uint64_t o_free;    // O copied to registers by the epilogue (count = warps)
  uint64_t wg_bar;    // bounded barrier of the stream's softmax warpgroup (count = warps)
  uint64_t iq_full[kItemQ], iq_empty[kItemQ];  // item queue: the producer draws work-list positions for the stream
  int item_q[kItemQ];
  int merge_go;       // this stream's part of a split item delivered last and merges the item's partial results
};
struct Tail {
  StreamBars st[kStreams];
  uint32_t tmem_base;
  int abort_flag;
  int pipe_token;   // held by the issuer whose MMAs go into the tensor pipe next
};

constexpr int kSmemBytes = kStreams * 3 * kTileBytes + kStreams * kStageBytes + 1024 + static_cast<int>(sizeof(Tail));
static_assert(kSmemBytes <= 227 * 1024, "shared memory of one CTA");

// The kept kv blocks of an item are visited in rotated order (the online softmax does not care):
// q-block qb starts at entry (qb * kRotStep) mod length of its list.
__device__ __forceinline__ int rot_of(int qb, int n) {
  return static_cast<int>(static_cast<unsigned>(qb * kRotStep) % static_cast<unsigned>(n));
}

// A whole warp waits (every lane takes the acquire) and agrees on the outcome, so that a wait that runs out
// never leaves the lanes of a warp on different sides of a warp-collective instruction.
__device__ __forceinline__ bool wait_all(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag) ? 1 : 0) != 0;
}

// Work-list positions are handed out dynamically: one position per stream is fixed at launch (ItemDraw::init), the following ones are drawn from a device-wide cursor by the stream's producer, which passes them
// to the other roles through a small shared-memory queue (entry k in slot k % kItemQ, -1 ends the sequence).
struct ItemDraw {  // the drawing role (one thread)
  StreamBars* sb;
  int32_t* cursor;
  volatile int* abort_flag;
  int n_items, n_pub;
  int p0, p1, p2;  // current, published next, drawn (still in flight) after next: the atomic never sits between two items
  bool started, ended;
  __device__ __forceinline__ int draw() {
    const int p = atomicAdd(cursor, 1) + kStreams * static_cast<int>(gridDim.x);
    return p < n_items ? p : -1;
  }
  __device__ __forceinline__ bool publish(int v) {
    if (ended) return true;
    const int slot = n_pub % kItemQ;
    if (!mbar_wait(&sb->iq_empty[slot], (static_cast<uint32_t>(n_pub / kItemQ) & 1u) ^ 1u, abort_flag)) return false;
    sb->item_q[slot] = v;
    mbar_arrive(&sb->iq_full[slot]);
    ++n_pub;
    if (v < 0) ended = true;
    return true;
  }
  __device__ __forceinline__ void init(StreamBars* s, int stream, int32_t* cur, volatile int* ab, int n) {
    sb = s; cursor = cur; abort_flag = ab; n_items = n; n_pub = 0; started = false; ended = false;
    // Units come longest first. Stream 0 of CTA c starts with unit c, stream 1 with unit 2 * CTAs - 1 - c: the SM
    // that got the longest unit of the first round gets the shortest of the second.
    const int first = stream == 0 ? static_cast<int>(blockIdx.x)
                                  : kStreams * static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
    p0 = first < n ? first : -1;
    p1 = p2 = -1;
    bool ok = publish(p0);
    if (ok && p0 >= 0) {
      p1 = draw();
      ok = publish(p1);
      if (ok && p1 >= 0) p2 = draw();
    }
    if (!ok) p0 = -1;
  }
  __device__ __forceinline__ int next() {
    if (!started) { started = true; return p0; }
    p0 = p1;
    if (p0 < 0) return -1;
    p1 = p2;
    if (!publish(p1)) return -1;
    p2 = p1 >= 0 ? draw() : -1;
    return p0;
  }
};

template <bool kWholeWarp>
struct ItemRead {  // the reading roles: one thread, or all lanes of a softmax warp
  StreamBars* sb;
  volatile int* abort_flag;
  int k;
  __device__ __forceinline__ void init(StreamBars* s, volatile int* ab) { sb = s; abort_flag = ab; k = 0; }
  __device__ __forceinline__ int next() {
    const int slot = k % kItemQ;
    if (kWholeWarp) {
      if (!wait_all(&sb->iq_full[slot], static_cast<uint32_t>(k / kItemQ) & 1u, abort_flag)) return -1;
    } else {
      if (!mbar_wait(&sb->iq_full[slot], static_cast<uint32_t>(k / kItemQ) & 1u, abort_flag)) return -1;
    }
    const int v = sb->item_q[slot];
    if (kWholeWarp) {
      __syncwarp();
      if ((threadIdx.x & 31) == 0) mbar_arrive(&sb->iq_empty[slot]);
    } else {
      mbar_arrive(&sb->iq_empty[slot]);
    }
    ++k;
    return v;
  }
};

// The walk of a stream's items as a flat sequence of kv blocks. kNeedKv: the role needs the kv-block indices
// (the producer); the others only need the shape of the sequence (and the softmax warps which step, if any, is
// the ragged last block of its request). No global load sits between two blocks of an item.
template <class Src, bool kNeedKv, bool kNeedRagged>
struct BlockSeq {
  Src src;
  int item_no;   // index among this stream's non-empty units
  int h, n, j;                   // head inside the q / o tensors, kv blocks of the unit, current block
  int q_row0, q_valid, kv_row0;  // first row of the q-block in q / o, its existing rows, first kv row of the request
  int slot, part, nparts;        // partial slot, part number and count (a whole item: nparts = 1)
  int kvb, kvb_next;  // kv-block index of the current block; the next one is fetched a block early
  int rot;            // rotation of the visiting order inside the item's kv list
  int ragged_j, ragged_valid;  // visiting step of the request's partial last kv block (-1: none) and its columns
  const int32_t* kv;
  __device__ __forceinline__ void init() {
    item_no = -1; n = 0; j = 0; kv = nullptr; slot = 0; part = 0; nparts = 1;
    h = q_row0 = q_valid = kv_row0 = 0; kvb = kvb_next = 0; rot = 0; ragged_j = -1; ragged_valid = 0;
  }
  // Advances to the next block; `on_empty(q_row0, q_valid, h)` is called for every item without kv blocks that
  // is passed on the way. Returns false at the end of the sequence.
  template <class F>
  __device__ __forceinline__ bool next(const AttnArgs& a, F&& on_empty) {
    if (j + 1 < n) {
      ++j;
      if (kNeedKv) {
        kvb = kvb_next;
        if (j + 1 < n) kvb_next = kv[at(j + 1)];
      }
      return true;
    }
    while (true) {
      const int pos = src.next();
      if (pos < 0) break;
      // the unit's record: everything this role needs, in one 32-byte load
      const int4* up = reinterpret_cast<const int4*>(a.units + 8 * static_cast<int64_t>(pos));
      const int4 u0 = up[0], u1 = up[1];
      if (u0.x <= 0) { on_empty(u0.w, u1.x, u0.z - a.head_begin); continue; }
      n = u0.x; j = 0;
      h = u0.z - a.head_begin;
      q_row0 = u0.w; q_valid = u1.x; kv_row0 = u1.y;
      slot = static_cast<int>(static_cast<unsigned>(u1.w) >> 16); part = (u1.w >> 8) & 0xff; nparts = u1.w & 0xff;
      rot = rot_of(q_row0 >> 7, n);
      if (kNeedKv) {
        kv = a.kv_idx + u0.y;
        kvb = kv[at(0)];
        if (n > 1) kvb_next = kv[at(1)];
      }
      if (kNeedRagged) {
        ragged_j = -1;
        if (u1.z != 0) {  // the unit's last entry is the request's partial kv block
          ragged_j = n - 1 - rot;
          if (ragged_j < 0) ragged_j += n;
          ragged_valid = u1.z;
        }
      }
      ++item_no;
      return true;
    }
    n = 0; j = 0;
    return false;
  }
  __device__ __forceinline__ int at(int jj) const {
    const int t = jj + rot;
    return t >= n ? t - n : t;
  }
  __device__ __forceinline__ bool first() const { return j == 0; }
  __device__ __forceinline__ bool last() const { return j == n - 1; }
  __device__ __forceinline__ int valid() const { return j == ragged_j ? ragged_valid : kBKV; }
};

template <bool kBf16, bool kSoftCap>
__global__ void __launch_bounds__(kThreads, 1) attention_streams_kernel(const __grid_constant__ AttnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  // per stream: Q, K, V tiles; then the two staging areas; then the barriers
  uint8_t* smem_stage = smem + kStreams * 3 * kTileBytes;
  Tail* tail = reinterpret_cast<Tail*>(smem_stage + kStreams * kStageBytes);
  volatile int* abort_flag = &tail->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int x = 0; x < kStreams; ++x) {
      StreamBars* sb = &tail->st[x];
      mbar_init(&sb->q_full, 1);
      mbar_init(&sb->k_full, 1);
      mbar_init(&sb->v_full, 1);
      mbar_init(&sb->s_full, 1);
      mbar_init(&sb->p_half[0], kWgWarps);
      mbar_init(&sb->p_half[1], kWgWarps);
      mbar_init(&sb->pv_done, 1);
      mbar_init(&sb->o_free, kWgWarps);
      mbar_init(&sb->wg_bar, kWgWarps);
      for (int i = 0; i < kItemQ; ++i) { mbar_init(&sb->iq_full[i], 1); mbar_init(&sb->iq_empty[i], kItemReaders); }
    }
    tail->abort_flag = 0;
    tail->pipe_token = 0;
    fence_barrier_init();
  }
  if (warp == kWarpProducer && lane == 0) {
    tma_prefetch_desc(&a.tmap_q);
    tma_prefetch_desc(&a.tmap_k);
    tma_prefetch_desc(&a.tmap_v);
    tma_prefetch_desc(&a.tmap_o);
  }
  if (warp == kWarpTmem) {
    tmem_alloc(&tail->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tail->tmem_base;

  // The lists may be incomplete: a compaction or unit builder that ran out of room records it in its status word
  // and leaves records unwritten. Nothing of such a list is dereferenced; the launch only reports it.
  const bool list_bad = a.unit_counters[3] != kDevOk || a.unit_counters[1] > a.partial_slots;
  int n_items = a.unit_counters[0];  // units: whole items or parts of items
  if (list_bad || n_items < 0) n_items = 0;
  if (n_items > a.max_units) n_items = a.max_units;
  auto ignore_empty = [](int, int, int) {};

  if (warp >= kSoftmaxWarps) {
    // ================================================================== producers and issuers (one thread each)
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
    const int X = (warp - kSoftmaxWarps) & 1;
    StreamBars* sb = &tail->st[X];
    uint8_t* smem_q = smem + X * 3 * kTileBytes;
    uint8_t* smem_k = smem_q + kTileBytes;
    uint8_t* smem_v = smem_k + kTileBytes;
    if (warp < kWarpIssuer) {
      // ---------------------------------------------------------------- TMA producer of the stream's Q, K and V tiles
      if (lane == 0) {
        BlockSeq<ItemDraw, true, false> seq;
        seq.init();
        seq.src.init(sb, X, a.status + 1, abort_flag, n_items);
        uint32_t g = 0;
        int kv_row0 = 0;
        while (seq.next(a, ignore_empty)) {
          const int hk = seq.h;               // a unit's head is the kv head; its q tile holds the
          const int hq = hk * a.group_size;   // group's q heads of 128 / group tokens, token-major
          // the K slot (and, for a new item, the Q slot) is free once the Q K^T of the stream's previous block is done
          if (!mbar_wait(&sb->s_full, (g & 1u) ^ 1u, abort_flag)) break;
          if (seq.first()) {
            kv_row0 = seq.kv_row0;
            const int q_row = seq.q_row0;
            mbar_expect_tx(&sb->q_full, kTileBytes);
            tma_load_3d(smem_q, &a.tmap_q, &sb->q_full, 0, hq, q_row);
            tma_load_3d(smem_q + kHalfBytes, &a.tmap_q, &sb->q_full, 64, hq, q_row);
          }
          const int row = kv_row0 + seq.kvb * kBKV;
          mbar_expect_tx(&sb->k_full, kTileBytes);
          tma_load_3d(smem_k, &a.tmap_k, &sb->k_full, 0, hk, row);
          tma_load_3d(smem_k + kHalfBytes, &a.tmap_k, &sb->k_full, 64, hk, row);
          // the V slot is free once the P V of the previous block is done
          if (!mbar_wait(&sb->pv_done, (g & 1u) ^ 1u, abort_flag)) break;
          mbar_expect_tx(&sb->v_full, kTileBytes);
          tma_load_3d(smem_v, &a.tmap_v, &sb->v_full, 0, hk, row);
          tma_load_3d(smem_v + kHalfBytes, &a.tmap_v, &sb->v_full, 64, hk, row);
          ++g;
        }
      }
    } else {
      // ---------------------------------------------------------------- MMA issuer of the stream
      if (lane == 0) {
        constexpr uint32_t idesc_qk = make_idesc_f16(kBQ, kBKV, kBf16, 0, 0);
        constexpr uint32_t idesc_pv = make_idesc_f16(kBQ, kD, kBf16, 0, 1);
        // descriptors: constant high word, low word holds the address. Q and K are K-major (128-byte swizzle);
        // V is MN-major: its two 64-column halves are 16 KB apart (leading byte offset)
        const uint64_t dq = make_smem_desc_sw128(smem_u32(smem_q), 16, 1024);
        const uint32_t hi_k = static_cast<uint32_t>(dq >> 32);
        const uint32_t q_lo = static_cast<uint32_t>(dq);
        const uint32_t k_lo = static_cast<uint32_t>(make_smem_desc_sw128(smem_u32(smem_k), 16, 1024));
        const uint64_t dv = make_smem_desc_sw128(smem_u32(smem_v), kHalfBytes, 1024);
        const uint32_t hi_v = static_cast<uint32_t>(dv >> 32), v_lo = static_cast<uint32_t>(dv);
        const uint32_t tmem_s = tmem_base + kColS + static_cast<uint32_t>(X) * 128u;
        const uint32_t tmem_o = tmem_base + kColO + static_cast<uint32_t>(X) * 128u;
        uint32_t la[8], lb[8], ta[8], lv[8];
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // Q K^T: 16 elements further along K = +32 B inside a 64-column half, +16 KB for the second half
          const uint32_t off = static_cast<uint32_t>(((kk >> 2) * kHalfBytes + (kk & 3) * 32) >> 4);
          la[kk] = q_lo + off;
          lb[kk] = k_lo + off;
          // P V: 16 kv rows further = 16 * 128 B in the V tile, 8 columns further in the 16-bit P tile
          ta[kk] = tmem_s + static_cast<uint32_t>(kk * 8);
          lv[kk] = v_lo + static_cast<uint32_t>((kk * 2048) >> 4);
        }
        BlockSeq<ItemRead<false>, false, false> seq;
        seq.init();
        seq.src.init(sb, abort_flag);
        // The tensor pipe serves the two streams' issuers in turns: a turn is the P V of a block followed at once by
        // the Q K^T of the stream's next block (or the first Q K^T of an item), taken under a CTA-wide token. The
        // stream that comes second starts its softmax a turn later, which puts the streams in opposite phases (one in
        // its exponentials while the other one's MMAs run) instead of leaving both on the exponential unit together.
        auto take_pipe = [&]() -> bool {
          const uint64_t t0 = global_timer_ns();
          while (atomicCAS(&tail->pipe_token, 0, 1) != 0) {
            if (*abort_flag != 0) return false;
            if (global_timer_ns() - t0 > kWaitLimitNs) { *abort_flag = 1; return false; }
          }
          return true;
        };
        auto give_pipe = [&]() { atomicExch(&tail->pipe_token, 0); };
        // The token goes back while the last four MMAs of the turn are still being issued: an issuing thread is held
        // until the pipe has room, so the other stream's first MMAs queue up behind these instead of after a gap.
        auto issue_qk = [&]() {
          tc_fence_after_sync();
          // S is free: its last reader was the P V of the previous block, issued by this thread before
          umma_ss_x4(tmem_s, hi_k, hi_k, idesc_qk, 0u, la, lb);
          give_pipe();
          umma_ss_x4(tmem_s, hi_k, hi_k, idesc_qk, 1u, la + 4, lb + 4);
          umma_commit(&sb->s_full);
        };
        uint32_t g = 0;
        while (seq.next(a, ignore_empty)) {
          const uint32_t item = static_cast<uint32_t>(seq.item_no);
          if (seq.first()) {  // the item's first Q K^T (the later ones ride behind the previous block's P V)
            if (!mbar_wait(&sb->q_full, item & 1u, abort_flag)) break;
            if (!mbar_wait(&sb->k_full, g & 1u, abort_flag)) break;
            if (!take_pipe()) break;
            issue_qk();
          }
          // everything but P first (long since there), so that only P is waited for on the critical path
          if (!mbar_wait(&sb->v_full, g & 1u, abort_flag)) break;
          if (!seq.last() && !mbar_wait(&sb->k_full, (g + 1u) & 1u, abort_flag)) break;
          if (seq.first() && item > 0u) {  // O must have been drained by the previous item's epilogue
            if (!mbar_wait(&sb->o_free, (item - 1u) & 1u, abort_flag)) break;
          }
          if (kSplitP) {
            // P V in two halves of four MMAs: the first half runs while the softmax warps still compute the second
            if (!mbar_wait_spin(&sb->p_half[0], g & 1u, abort_flag)) break;
            if (!take_pipe()) break;
            tc_fence_after_sync();
            umma_ts_x4(tmem_o, hi_v, idesc_pv, seq.first() ? 0u : 1u, ta, lv);
            if (!mbar_wait_spin(&sb->p_half[1], g & 1u, abort_flag)) { give_pipe(); break; }
            tc_fence_after_sync();
            umma_ts_x4(tmem_o, hi_v, idesc_pv, 1u, ta + 4, lv + 4);
          } else {
            if (!mbar_wait_spin(&sb->p_half[1], g & 1u, abort_flag)) break;
            if (!take_pipe()) break;
            tc_fence_after_sync();
            umma_ts_x8(tmem_o, hi_v, idesc_pv, seq.first() ? 0u : 1u, ta, lv);
          }
          umma_commit(&sb->pv_done);
          if (!seq.last()) issue_qk(); else give_pipe();
          ++g;
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    // ================================================================== softmax / epilogue warpgroup of stream X
    // Thread (warp w of the group, lane) owns q row 32 w + lane = its TMEM lane: the whole row of S, of P and of O.
    const int X = warp / kWgWarps;
    const int wq = warp % kWgWarps;
    StreamBars* sb = &tail->st[X];
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t tmem_s = tmem_base + lane_base + kColS + static_cast<uint32_t>(X) * 128u;
    const uint32_t tmem_o = tmem_base + lane_base + kColO + static_cast<uint32_t>(X) * 128u;
    const int row = wq * 32 + lane;
    uint8_t* stage = smem_stage + X * kStageBytes;
    uint16_t* o16 = reinterpret_cast<uint16_t*>(a.o);
    uint32_t wg_phase = 0;
    bool ok = true;

    // bounded barrier of the four warps of this group
    auto wg_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(&sb->wg_bar);
      const bool r = wait_all(&sb->wg_bar, wg_phase, abort_flag);
      wg_phase ^= 1u;
      return r;
    };

    struct RowCtx {  // where an item's row lives in global memory
      uint16_t* orow;
      float* lse;
      bool row_ok;
      bool whole;   // no row of the q-block is past the end of its request
      int grow0;    // first row of the q-block in the q / o tensors
    };
    // Row r of a tile is token q_row0 + r / group, q head h * group + r % group (group = 1: the row itself).
    const int grp = a.group_size;
    auto row_ctx = [&](int q_row0, int q_valid, int h) -> RowCtx {
      RowCtx c;
      c.row_ok = static_cast<int>(row) < q_valid * grp;
      c.whole = q_valid * grp == kBQ;
      c.grow0 = q_row0;
      const int64_t grow = static_cast<int64_t>(q_row0) + static_cast<int>(row) / grp;
      const int hq = h * grp + static_cast<int>(row) % grp;
      c.orow = o16 + grow * a.o_stride_n + static_cast<int64_t>(hq) * a.o_stride_h;
      c.lse = a.lse != nullptr ? a.lse + grow * a.lse_stride_n + hq : nullptr;
      return c;
    };
    auto on_empty = [&](int q_row0, int q_valid, int hq) {  // active q-block that keeps nothing: zeros, lse = -5e4
      const RowCtx c = row_ctx(q_row0, q_valid, hq);
      if (c.row_ok) {
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int i = 0; i < 16; ++i) reinterpret_cast<uint4*>(c.orow)[i] = z;
        if (c.lse != nullptr) *c.lse = -5e4f;
      }
    };

    BlockSeq<ItemRead<true>, false, true> seq;
    seq.init();
    seq.src.init(sb, abort_flag);
    uint32_t g = 0;            // blocks of this stream so far
    float m_run = -INFINITY;   // the maximum the row's sum and O refer to
    uint64_t l2a = 0, l2b = 0; // row sum (two packed pairs of partial sums)
    bool stage_busy = false;   // a TMA store of this stream may still be reading the staging area

    while (ok && seq.next(a, on_empty)) {
      if (seq.first()) {
        m_run = -INFINITY;
        l2a = 0;
        l2b = 0;
      }
      // ---- S -> registers (the whole row, once)
      if (!wait_all(&sb->s_full, g & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t s[128];
      tmem_ld_x32(tmem_s, s);
      tmem_ld_x32(tmem_s + 32u, s + 32);
      tmem_ld_x32(tmem_s + 64u, s + 64);
      tmem_ld_x32(tmem_s + 96u, s + 96);
      tmem_wait_ld();
      if constexpr (kSoftCap) {  // logit = cap * tanh(q.k * sm_scale / cap); the factor cap is part of sm_scale_log2
#pragma unroll
        for (int t = 0; t < 128; ++t) s[t] = __float_as_uint(tanh_approx(__uint_as_float(s[t]) * a.soft_cap_pre));
      }
      const int valid = seq.valid();
      if (valid < kBKV) {
#pragma unroll
        for (int t = 0; t < 128; ++t)
          if (t >= valid) s[t] = 0xff800000u;  // -inf: excluded from the maximum, exp2 gives 0
      }
      float mx;
      {
        float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int t = 0; t < 16; ++t) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            mxs[i] = fmax3(mxs[i], __uint_as_float(s[8 * t + 2 * i]), __uint_as_float(s[8 * t + 2 * i + 1]));
        }
        mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));
      }
      const float m_new = fmaxf(m_run, mx * a.sm_scale_log2);
      // lazy rescale: the row keeps its old reference maximum while the new one is at most 2^8 above it
      const bool need = (m_new - m_run) > kRescaleThreshold;
      const bool rescale = !seq.first() && __any_sync(0xffffffffu, need);
      const float m_used = (seq.first() || need) ? m_new : m_run;
      if (rescale) {
        // O is rescaled after the P V of the previous block has completed (and before this block's P is handed over)
        if (!wait_all(&sb->pv_done, (g - 1u) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const float alpha = need ? ex2_approx(m_run - m_new) : 1.0f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_x32(tmem_o + 32u * c, v);
          tmem_wait_ld();
#pragma unroll
          for (int t = 0; t < 32; ++t) v[t] = __float_as_uint(__uint_as_float(v[t]) * alpha);
          tmem_st_x32(tmem_o + 32u * c, v);
        }
      }
      if (m_run != m_used) {  // the row sum follows the maximum in use (first block: the sum is zero anyway)
        const float beta = (m_run == -INFINITY) ? 0.f : ex2_approx(m_run - m_used);
        const uint64_t beta2 = pack_f32x2(beta, beta);
        l2a = ffma2(l2a, beta2, 0ull);
        l2b = ffma2(l2b, beta2, 0ull);
        m_run = m_used;
      }
      // ---- P = exp2(S * scale - m_used), row sum, P (16 bit) over the first 64 columns of S: one FMA and one
      // add per PAIR of columns
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
      const uint64_t scale2 = pack_f32x2(a.sm_scale_log2, a.sm_scale_log2);
      const uint64_t negm2 = pack_f32x2(neg_m, neg_m);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int t = 0; t < 16; ++t) {
          const int e = 32 * c + 2 * t;
          const uint64_t x2 = ffma2(pack_f32x2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])), scale2, negm2);
          float x0, x1;
          unpack_f32x2(x2, x0, x1);
          const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
          if (t & 1) l2b = fadd2(l2b, pack_f32x2(p0, p1)); else l2a = fadd2(l2a, pack_f32x2(p0, p1));
          pk[t] = kBf16 ? pack_bf16x2(p0, p1) : pack_f16x2(p0, p1);
        }
        tmem_st_x16(tmem_s + 16u * c, pk);
        if (kSplitP ? (c & 1) : (c == 3)) {  // a half of P (64 kv columns) is complete: its four MMAs may start
          tmem_wait_st();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sb->p_half[c >> 1]);
        }
      }
      ++g;

      if (seq.last()) {
        // ---- epilogue of the unit. A whole item: O / l -> 16 bit -> global. A part of a split item: the fp32 O, the
        // row maxima and the row sums go to the item's partial slots; the part that delivers last merges them.
        const RowCtx c = row_ctx(seq.q_row0, seq.q_valid, seq.h);
        float la, lb, lc, ld;
        unpack_f32x2(l2a, la, lb);
        unpack_f32x2(l2b, lc, ld);
        const float lsum = (la + lb) + (lc + ld);
        // Writes one round (64 columns, packed to 16 bit) of the q-block: whole q-blocks through the stream's staging
        // area (128-byte swizzle) and a TMA store, a q-block cut by the end of its request row by row.
        auto store_round = [&](int r, const uint4 (&outv)[8]) -> bool {
          if (c.whole) {
            if (stage_busy) {  // the previous store must have read the staging area
              if (wq == 0 && lane == 0) tma_store_wait_read<0>();
              if (!wg_sync()) return false;
              stage_busy = false;
            }
            uint8_t* rowp = stage + row * 128;
            const uint32_t swz = static_cast<uint32_t>(row & 7);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<uint4*>(rowp + ((static_cast<uint32_t>(q) ^ swz) << 4)) = outv[q];
            fence_proxy_async_smem();
            if (!wg_sync()) return false;
            if (wq == 0 && lane == 0) {
              tma_store_3d(&a.tmap_o, stage, 64 * r, seq.h * grp, c.grow0);
              tma_store_commit();
            }
            stage_busy = true;
          } else if (c.row_ok) {
            uint4* dst = reinterpret_cast<uint4*>(c.orow + 64 * r);
#pragma unroll
            for (int q = 0; q < 8; ++q) dst[q] = outv[q];
          }
          return true;
        };
        if (!wait_all(&sb->pv_done, (g - 1u) & 1u, abort_flag)) { ok = false; break; }  // the unit's last P V
        tc_fence_after_sync();
        if (seq.nparts <= 1) {
          const float inv_l = lsum > 0.f ? __frcp_rn(lsum) : 0.f;
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            uint32_t v[64];
            tmem_ld_x32(tmem_o + 64u * r, v);
            tmem_ld_x32(tmem_o + 64u * r + 32u, v + 32);
            tmem_wait_ld();
            if (r == 1) {  // O may be overwritten by the next unit
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&sb->o_free);
            }
            uint4 outv[8];
            uint32_t* w = reinterpret_cast<uint32_t*>(outv);
#pragma unroll
            for (int t = 0; t < 32; ++t) {
              const float x0 = __uint_as_float(v[2 * t]) * inv_l;
              const float x1 = __uint_as_float(v[2 * t + 1]) * inv_l;
              w[t] = kBf16 ? pack_bf16x2(x0, x1) : pack_f16x2(x0, x1);
            }
            if (!store_round(r, outv)) { ok = false; break; }
          }
          if (!ok) break;
          if (c.row_ok && c.lse != nullptr) *c.lse = (lsum > 0.f) ? (log2f(lsum) + m_run) : -5e4f;
        } else {
          // ---- partial result: O as [column group of 4][row][4] (a warp's store covers 512 contiguous bytes)
          float* ps = a.partials + static_cast<size_t>(seq.slot) * kPartialFloats;
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t v[32];
            tmem_ld_x32(tmem_o + 32u * cc, v);
            tmem_wait_ld();
            if (cc == 3) {  // O may be overwritten by the next unit
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&sb->o_free);
            }
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<uint4*>(ps + (static_cast<size_t>(8 * cc + q) * 128 + row) * 4) =
                  make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          }
          ps[128 * 128 + row] = m_run;
          ps[128 * 128 + 128 + row] = lsum;
          __threadfence();
          if (!wg_sync()) { ok = false; break; }
          if (wq == 0 && lane == 0) {
            int* cnt = a.arrive + (seq.slot - seq.part);  // a split item counts at its first slot
            const int old = atomicAdd(cnt, 1);
            const int mine = old == seq.nparts - 1 ? 1 : 0;
            if (mine) *cnt = 0;  // the counter is back at zero for the next launch
            __threadfence();
            sb->merge_go = mine;
          }
          if (!wg_sync()) { ok = false; break; }
          if (sb->merge_go != 0) {
            // ---- this part delivered last: O = sum_p O_p 2^(m_p - m) / sum_p l_p 2^(m_p - m), m = max_p m_p
            const float* base = a.partials + static_cast<size_t>(seq.slot - seq.part) * kPartialFloats;
            float m_all = -INFINITY;
            for (int pp = 0; pp < seq.nparts; ++pp)
              m_all = fmaxf(m_all, __ldcg(base + static_cast<size_t>(pp) * kPartialFloats + 128 * 128 + row));
            float l_all = 0.f;
            for (int pp = 0; pp < seq.nparts; ++pp) {
              const float* pq = base + static_cast<size_t>(pp) * kPartialFloats;
              const float mp = __ldcg(pq + 128 * 128 + row);
              const float wgt = (mp == -INFINITY) ? 0.f : ex2_approx(mp - m_all);
              l_all = fmaf(__ldcg(pq + 128 * 128 + 128 + row), wgt, l_all);
            }
            const float inv_l = l_all > 0.f ? __frcp_rn(l_all) : 0.f;
#pragma unroll 1
            for (int r = 0; r < 2; ++r) {
              float acc[64];
#pragma unroll
              for (int t = 0; t < 64; ++t) acc[t] = 0.f;
              for (int pp = 0; pp < seq.nparts; ++pp) {
                const float* pq = base + static_cast<size_t>(pp) * kPartialFloats;
                const float mp = __ldcg(pq + 128 * 128 + row);
                const float wgt = (mp == -INFINITY) ? 0.f : ex2_approx(mp - m_all);
#pragma unroll
                for (int q = 0; q < 16; ++q) {
                  const float4 x = __ldcg(reinterpret_cast<const float4*>(pq + (static_cast<size_t>(16 * r + q) * 128 + row) * 4));
                  acc[4 * q] = fmaf(x.x, wgt, acc[4 * q]);
                  acc[4 * q + 1] = fmaf(x.y, wgt, acc[4 * q + 1]);
                  acc[4 * q + 2] = fmaf(x.z, wgt, acc[4 * q + 2]);
                  acc[4 * q + 3] = fmaf(x.w, wgt, acc[4 * q + 3]);
                }
              }
              uint4 outv[8];
              uint32_t* w = reinterpret_cast<uint32_t*>(outv);
#pragma unroll
              for (int t = 0; t < 32; ++t)
                w[t] = kBf16 ? pack_bf16x2(acc[2 * t] * inv_l, acc[2 * t + 1] * inv_l)
                             : pack_f16x2(acc[2 * t] * inv_l, acc[2 * t + 1] * inv_l);
              if (!store_round(r, outv)) { ok = false; break; }
            }
            if (!ok) break;
            if (c.row_ok && c.lse != nullptr) *c.lse = (l_all > 0.f) ? (log2f(l_all) + m_all) : -5e4f;
          }
        }
      }
    }
    if (wq == 0 && lane == 0) tma_store_wait_all<0>();
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
  if (list_bad && blockIdx.x == 0 && threadIdx.x == 0) atomicCAS(a.status, kDevOk, kDevBadIndex);
  if (warp == kWarpTmem) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  // the last CTA to get here puts the cursor and the arrival count back to zero for the next launch
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(a.status + 2, 1) == static_cast<int>(gridDim.x) - 1) {
      atomicExch(a.status + 1, 0);
      atomicExch(a.status + 2, 0);
    }
  }
}

template <bool kBf16, bool kSoftCap>
cudaError_t launch_one(const AttnArgs& a, int ctas, cudaStream_t stream) {
  const cudaError_t e = cudaFuncSetAttribute(attention_streams_kernel<kBf16, kSoftCap>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kSmemBytes);
  if (e != cudaSuccess) return e;
  attention_streams_kernel<kBf16, kSoftCap><<<ctas, kThreads, kSmemBytes, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_attention_streams(const AttnArgs& a, int max_ctas, cudaStream_t stream) {
  if (max_ctas <= 0) return cudaSuccess;
  const bool cap = a.soft_cap_pre > 0.f;
  if (a.is_bf16) return cap ? launch_one<true, true>(a, max_ctas, stream) : launch_one<true, false>(a, max_ctas, stream);
  return cap ? launch_one<false, true>(a, max_ctas, stream) : launch_one<false, false>(a, max_ctas, stream);
}

}  // namespace fo
