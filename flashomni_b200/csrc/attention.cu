// Block-sparse prefill attention on tcgen05 / TMEM / TMA, driven by compacted work lists: the kernel for launches
// with MANY work units (several per SM). Launches with few units take attention_streams.cu instead.
//
// What it computes (reference: include/flashomni/attention/prefill.cuh:1203-1531): for every work
// item (b, h, qb) -- an active 128-row q-block of one head -- and its ascending list of kept
// 128-row kv-blocks,  O[rows, h, :] = softmax_over_kept(Q K^T * sm_scale) V,  fp32 accumulation,
// base-2 online softmax, output rounded to the input dtype. q-blocks that are not in the list are
// never written. An item with an empty list writes zeros (lse = -5e4), like the reference.
//
// One persistent CTA per SM walks its items as ONE sequence of kv blocks g = 0, 1, 2, ... and
// software-pipelines it:
//
//   tensor pipe     S[g&1] = Q K_g^T   (QK issuer)   and   O (+)= P[g&1] V_g   (PV issuer)
//   softmax group   g&1:  S[g&1] -> registers -> P[g&1]
//
// Items are positions of the work list's processing order, handed out dynamically: position i < grid
// size goes to CTA i, the rest are drawn from a device-wide cursor by the K producer and passed to the
// other roles through a small shared-memory queue.
// TMEM (512 columns): S0, S1 (fp32, 128 each), O (fp32, 128), P0, P1 (16 bit, 64 each). S is
// double-buffered and P does not alias S, so the QK and PV batches are independent of each other and
// of the softmax in between; they are issued by two different threads, because a thread that issues a
// batch is held until the batch has drained.
// The softmax is split into two groups of eight warps that take alternate blocks (group = g & 1), two
// threads per q row with 64 columns each: while one group is in its exponentials the other one loads,
// reduces and hands over. S is read twice (row maximum, then exponentials) instead of being held in
// registers across the exchanges; the two halves of a row meet through shared memory; the running
// maximum passes from block to block through shared memory (m_pub / m_ready); each thread keeps its
// own partial row sum, and the four of a row are merged, with the output, in the epilogue (whole
// q-blocks leave through a per-warp staging area and TMA box stores).
// Warps: 0-7 softmax group 0, 8-15 softmax group 1 (TMEM lane = q row; `setmaxnreg` gives them 112
// registers), 16 TMA producer of Q (double-buffered) and K (two-slot FIFO of 32 KB tiles) and drawer of
// work-list positions, 17 QK issuer, 18 PV issuer, 19 TMA producer of V (its own two-slot FIFO).
// Every mbarrier wait is bounded.
#include <cuda_fp16.h>

#include "internal.h"

#ifndef FO_ROT_STEP
#define FO_ROT_STEP 5
#endif

namespace fo {
namespace {

constexpr int kBQ = 128, kBKV = 128;
constexpr int kTileBytes = 128 * 128 * 2;   // 32 KB: the slot of a 128-row tile of Q, K or V (head_dim 64 fills half of it)
constexpr int kHalfBytes = kTileBytes / 2;  // one 64-column half (one swizzle-atom column)
constexpr int kRingK = 2, kRingV = 2;  // separate FIFOs of 32 KB tiles for K and V
constexpr int kRing = kRingK + kRingV;
constexpr int kQBufs = 2;
constexpr int kGroupWarps = 8;                  // warps of one softmax group (two threads per q row)
constexpr int kSoftmaxWarps = 2 * kGroupWarps;
constexpr int kWarpProducer = kSoftmaxWarps;
constexpr int kWarpQK = kSoftmaxWarps + 1;      // issues S = Q K^T
constexpr int kWarpPV = kSoftmaxWarps + 2;      // issues O += P V
constexpr int kWarpProducerV = kSoftmaxWarps + 3;
constexpr int kWarpMma = kWarpQK;               // owner of the TMEM allocation
constexpr int kThreads = (kSoftmaxWarps + 4) * 32;  // 640: four softmax warpgroups and the producer / issuer warpgroup
constexpr int kRegsSoftmax = 112, kRegsOther = 32;  // register split between the warpgroups (setmaxnreg)
// setmaxnreg.inc waits until the registers are free in the pool the CTA was launched with (threads x the
// per-thread count the compiler settles on for this block size): a split that asks for more never returns.
constexpr int kRegsAtLaunch = (65536 / kThreads) / 8 * 8;
static_assert(kSoftmaxWarps * 32 * kRegsSoftmax + (kThreads - kSoftmaxWarps * 32) * kRegsOther <= kThreads * kRegsAtLaunch,
              "register split exceeds the CTA's register pool");
constexpr int kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 256, kColP = 384;
constexpr int kRotStep = FO_ROT_STEP;       // q-block qb starts its kv list at entry (qb * kRotStep) mod length
constexpr int kItemQ = 8;                   // entries of the item queue
constexpr int kItemReaders = kSoftmaxWarps + 3;  // softmax warps, V producer, the two MMA issuers
constexpr float kRescaleThreshold = 8.0f;  // lazy rescale: keep the old max while exp2 stays <= 2^8

struct Tail {
  uint64_t q_full[kQBufs], q_empty[kQBufs];
  uint64_t k_full[kRingK], k_empty[kRingK], v_full[kRingV], v_empty[kRingV];
  uint64_t s_full[2], s_free[2];  // S buffer written by QK / copied to registers by its softmax group
  uint64_t p_full[2], pv_done[2];  // indexed by block parity, so that no waiter can fall two phases behind
  uint64_t m_ready[2];             // running maximum after a block of this parity has been published
  uint64_t stats_ready[2];         // indexed by item parity: both groups have published (m, l) of the item
  uint64_t o_full, o_free;
  uint64_t iq_full[kItemQ], iq_empty[kItemQ];  // item queue: the K producer draws work-list positions for the CTA
  uint64_t ep_bar;                 // all softmax warps, in the epilogue of a part of a split item
  int item_q[kItemQ];
  uint32_t tmem_base;
  int abort_flag;
  int merge_go;                    // this CTA's part of a split item delivered last and merges the partial results
  uint64_t pair_bar[2][4];   // [group][quadrant]: the two warps that share 32 rows
  float m_pub[2][128];       // [block parity][row]: running maximum in use after that block
  float xmax[2][2][2][128];  // [group][parity of the group's block count][column half][row]: half-row maxima
  float stats_m[2][4][128];  // [item parity][2 * group + half][row]: the maximum the partial sum refers to
  float stats_l[2][4][128];  // [item parity][2 * group + half][row]: partial row sum
};



constexpr int kOutStageBytes = 16 * 64;  // per softmax warp: 16 rows x 32 output columns
constexpr int kSmemBytes = (kQBufs + kRing) * kTileBytes + kSoftmaxWarps * kOutStageBytes + 1024 +
                           static_cast<int>(sizeof(Tail));
static_assert(kSmemBytes <= 227 * 1024, "shared memory of one CTA");

// The kept kv blocks of an item are visited in rotated order (the online softmax does not care):
// q-block qb starts at entry (qb * kRotStep) mod length of its list.
__device__ __forceinline__ int rot_of(int qb, int n) {
  return static_cast<int>(static_cast<unsigned>(qb * kRotStep) % static_cast<unsigned>(n));
}

// Work-list positions are handed out dynamically: position i < gridDim.x goes to CTA i, the following ones are
// drawn from a device-wide cursor by the CTA's K producer, which passes them to the other roles through a small
// shared-memory queue (entry k in slot k % kItemQ, -1 ends the sequence). A CTA that got short items draws more.
struct ItemDraw {  // the drawing role (one thread)
  Tail* tail;
  int32_t* cursor;
  volatile int* abort_flag;
  int n_items, n_pub;
  int p0, p1, p2;  // current, published next, drawn (still in flight) after next: the atomic never sits between two items
  bool started, ended;
  __device__ __forceinline__ int draw() {
    const int p = atomicAdd(cursor, 1) + static_cast<int>(gridDim.x);
    return p < n_items ? p : -1;
  }
  __device__ __forceinline__ bool publish(int v) {
    if (ended) return true;
    const int slot = n_pub % kItemQ;
    if (!mbar_wait(&tail->iq_empty[slot], (static_cast<uint32_t>(n_pub / kItemQ) & 1u) ^ 1u, abort_flag)) return false;
    tail->item_q[slot] = v;
    mbar_arrive(&tail->iq_full[slot]);
    ++n_pub;
    if (v < 0) ended = true;
    return true;
  }
  __device__ __forceinline__ void init(Tail* t, int32_t* cur, volatile int* ab, int n) {
    tail = t; cursor = cur; abort_flag = ab; n_items = n; n_pub = 0; started = false; ended = false;
    p0 = static_cast<int>(blockIdx.x) < n ? static_cast<int>(blockIdx.x) : -1;
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
  Tail* tail;
  volatile int* abort_flag;
  int k;
  __device__ __forceinline__ void init(Tail* t, volatile int* ab) { tail = t; abort_flag = ab; k = 0; }
  __device__ __forceinline__ int next() {
    const int slot = k % kItemQ;
    if (!mbar_wait(&tail->iq_full[slot], static_cast<uint32_t>(k / kItemQ) & 1u, abort_flag)) return -1;
    const int v = tail->item_q[slot];
    if (kWholeWarp) {
      __syncwarp();
      if ((threadIdx.x & 31) == 0) mbar_arrive(&tail->iq_empty[slot]);
    } else {
      mbar_arrive(&tail->iq_empty[slot]);
    }
    ++k;
    return v;
  }
};

// The same walk for the softmax groups, which do not need the kv-block indices: only which step of an
// item (if any) is the ragged last block of its request. No global load sits between two blocks.
template <bool kWithKv>
struct GroupSeq {
  ItemRead<true> src;
  const int32_t* kv;
  int rot, kvb, kvb_next, causal_base, req;
  __device__ __forceinline__ int at(int jj) const {
    const int t = jj + rot;
    return t >= n ? t - n : t;
  }
  int h, n, j;            // head inside the q / o tensors, kv blocks of the unit, current block
  int q_row0, q_valid;    // first row of the q-block in q / o, its existing rows
  int ragged_j, ragged_valid;  // visiting step of the request's partial last kv block (-1: none) and its columns
  int parts;              // slot << 16 | part << 8 | number of parts (a whole item: one part)
  __device__ __forceinline__ void init(Tail* tail, volatile int* abort_flag) {
    src.init(tail, abort_flag); n = 0; j = 0;
    h = q_row0 = q_valid = 0; ragged_j = -1; ragged_valid = 0; parts = 1;
    kv = nullptr; rot = 0; kvb = kvb_next = 0; causal_base = 0; req = 0;
  }
  template <class F>
  __device__ __forceinline__ bool next(const AttnArgs& a, F&& on_empty) {
    if (j + 1 < n) {
      ++j;
      if (kWithKv) {
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
      if (u0.x <= 0) { on_empty(u0.w, u1.x & 0xffff, (u0.z & 0xffff) - a.head_begin); continue; }
      n = u0.x; j = 0;
      h = (u0.z & 0xffff) - a.head_begin; q_row0 = u0.w; q_valid = u1.x & 0xffff; parts = u1.w;
      req = u0.z >> 16;
      causal_base = u1.z;
      ragged_j = -1;
      if ((u1.x >> 16) != 0) {  // the unit's last entry is the request's partial kv block
        ragged_j = n - 1 - rot_of(q_row0 >> 7, n);
        if (ragged_j < 0) ragged_j += n;
        ragged_valid = u1.x >> 16;
      }
      if (kWithKv) {  // the kv-block indices too (a causal mask needs the block's position)
        kv = a.kv_idx + u0.y;
        rot = rot_of(q_row0 >> 7, n);
        kvb = kv[at(0)];
        if (n > 1) kvb_next = kv[at(1)];
      }
      return true;
    }
    n = 0; j = 0;
    return false;
  }
  __device__ __forceinline__ bool first() const { return j == 0; }
  __device__ __forceinline__ bool last() const { return j == n - 1; }
  __device__ __forceinline__ int valid() const { return j == ragged_j ? ragged_valid : kBKV; }
};

// Walks the CTA's share of the schedule as a flat sequence of kv blocks.
template <class Src>
struct BlockSeq {
  Src src;
  int item_no;   // index among this CTA's non-empty units (selects the Q buffer, o_full / o_free phases)
  int h, n, j;
  int q_row0, kv_row0;  // first row of the q-block in q / o, first kv row of the request
  int kvb, kvb_next;  // kv-block index of the current block; the next one is fetched a block early
  int rot;            // rotation of the visiting order inside the unit's kv list
  const int32_t* kv;
  __device__ __forceinline__ void init() {
    item_no = -1; n = 0; j = 0; kv = nullptr;
    h = q_row0 = kv_row0 = 0; kvb = kvb_next = 0; rot = 0;
  }
  // Advances to the next block; `on_empty(q_row0, q_valid, h)` is called for every item without kv blocks that
  // is passed on the way. Returns false at the end of the sequence.
  template <class F>
  __device__ __forceinline__ bool next(const AttnArgs& a, F&& on_empty) {
    if (j + 1 < n) {
      ++j;
      kvb = kvb_next;
      if (j + 1 < n) kvb_next = kv[at(j + 1)];
      return true;
    }
    while (true) {
      const int pos = src.next();
      if (pos < 0) break;
      const int4* up = reinterpret_cast<const int4*>(a.units + 8 * static_cast<int64_t>(pos));
      const int4 u0 = up[0], u1 = up[1];
      if (u0.x <= 0) { on_empty(u0.w, u1.x & 0xffff, (u0.z & 0xffff) - a.head_begin); continue; }
      n = u0.x; j = 0;
      h = (u0.z & 0xffff) - a.head_begin; q_row0 = u0.w; kv_row0 = u1.y;
      kv = a.kv_idx + u0.y;
      rot = rot_of(q_row0 >> 7, n);
      kvb = kv[at(0)];
      if (n > 1) kvb_next = kv[at(1)];
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
};

// kParts: the launch may hold parts of split items (partial results and their merge in the epilogue); the
// instantiation without carries none of that code.
// Up to 64 bits of the little-endian bit stream `seg` starting at bit `pos` (nine independent byte loads; bytes at
// or beyond `limit` read as zero), the bits from `nbits` on cleared.
__device__ __forceinline__ uint64_t load_mask_bits64(const uint8_t* seg, int64_t pos, int64_t limit, int nbits) {
  const int64_t byte0 = pos >> 3;
  const int sh = static_cast<int>(pos & 7);
  uint64_t lo = 0, hi = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t bi = byte0 + i;
    const uint64_t v = (bi < limit) ? seg[bi] : 0u;
    lo |= v << (8 * i);
  }
  if (byte0 + 8 < limit) hi = seg[byte0 + 8];
  uint64_t r = sh ? ((lo >> sh) | (hi << (64 - sh))) : lo;
  if (nbits < 64) r &= (1ull << nbits) - 1ull;
  return r;
}

// kD: head dimension, 128, 64 or 256. With 64 a tile is one 64-column half: the second TMA box, the upper four of the
// eight Q K^T MMAs and the upper 64 columns of O are left out; everything else is the same code. With 256 a tile
// is four halves (64 KB), so Q, K and V have one slot each instead of two (a load waits for the MMA that read the
// slot), Q K^T is sixteen MMAs, O takes 256 TMEM columns and P is written over the S it came from (S is in
// registers by then): the QK of a group's next block waits for the PV of its previous one instead of for the
// softmax. Correct and slower per FLOP than 128; whole items only.
// kMask 1 (causal): a kv position is visible to a q token only up to token + kv_len - q_len (the reference's
// MaskMode::kCausal, prefill.cuh:746-751). kMask 2 (custom): position (i, j) of a request is visible iff bit
// i * kv_len + j of the request's packed mask is set (MaskMode::kCustom, variants.cuh:76-87). In both the softmax
// warps also read the kv-block indices.
template <bool kBf16, bool kSoftCap, bool kParts, int kD, int kMask>
__global__ void __launch_bounds__(kThreads, 1) attention_kernel(const __grid_constant__ AttnArgs a) {
  static_assert(kD == 128 || kD == 64 || kD == 256, "head dimension");
  static_assert(!(kParts && kD == 256), "head dimension 256 runs whole items only");
  constexpr int kLoadBytes = 128 * kD * 2;   // bytes of one tile load
  constexpr int kHalves = kD / 64;           // 64-column boxes per tile
  constexpr bool kWide = kD == 256;
  constexpr int kTB = kWide ? 2 * kTileBytes : kTileBytes;                               // bytes of a tile slot
  constexpr int kQB = kWide ? 1 : kQBufs, kRK = kWide ? 1 : kRingK, kRV = kWide ? 1 : kRingV;   // slots of Q, K, V
  static_assert((kQB + kRK + kRV) * kTB <= (kQBufs + kRing) * kTileBytes, "tile slots");
  constexpr int kOW = kWide ? 64 : 32;       // columns of O per softmax thread in the epilogue
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* smem_q = smem;                           // kQBufs tiles
  uint8_t* smem_ring = smem + kQB * kTB;  // K slots, then V slots
  uint8_t* smem_ostage = smem + (kQBufs + kRing) * kTileBytes;  // output staging of the softmax warps
  Tail* tail = reinterpret_cast<Tail*>(smem_ostage + kSoftmaxWarps * kOutStageBytes);
  volatile int* abort_flag = &tail->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kQBufs; ++i) { mbar_init(&tail->q_full[i], 1); mbar_init(&tail->q_empty[i], 1); }
    for (int i = 0; i < kRingK; ++i) { mbar_init(&tail->k_full[i], 1); mbar_init(&tail->k_empty[i], 1); }
    for (int i = 0; i < kRingV; ++i) { mbar_init(&tail->v_full[i], 1); mbar_init(&tail->v_empty[i], 1); }
    mbar_init(&tail->s_full[0], 1);
    mbar_init(&tail->s_full[1], 1);
    mbar_init(&tail->s_free[0], kGroupWarps);
    mbar_init(&tail->s_free[1], kGroupWarps);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tail->p_full[i], kGroupWarps);
      mbar_init(&tail->pv_done[i], 1);
      mbar_init(&tail->m_ready[i], kGroupWarps);
      mbar_init(&tail->stats_ready[i], kSoftmaxWarps);
    }
    mbar_init(&tail->o_full, 1);
    mbar_init(&tail->o_free, kSoftmaxWarps);
    mbar_init(&tail->ep_bar, kSoftmaxWarps);
    for (int i = 0; i < kItemQ; ++i) { mbar_init(&tail->iq_full[i], 1); mbar_init(&tail->iq_empty[i], kItemReaders); }
    for (int i = 0; i < 8; ++i) mbar_init(&tail->pair_bar[i >> 2][i & 3], 2);
    tail->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kWarpProducer && lane == 0) {
    tma_prefetch_desc(&a.tmap_q);
    tma_prefetch_desc(&a.tmap_k);
    tma_prefetch_desc(&a.tmap_v);
    tma_prefetch_desc(&a.tmap_o16);
  }
  if (warp == kWarpMma) {
    tmem_alloc(&tail->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tail->tmem_base;

  // The list may be shorter than counters[0] says: a compaction that ran out of room records it in counters[2]
  // and leaves records unwritten. Nothing of such a list is dereferenced; the launch only reports it.
  const bool list_bad = a.unit_counters[3] != kDevOk || a.unit_counters[1] > (kParts ? a.partial_slots : 0);
  int n_items = a.unit_counters[0];
  if (list_bad || n_items < 0) n_items = 0;
  if (n_items > a.max_units) n_items = a.max_units;
  auto ignore_empty = [](int, int, int) {};

  // The softmax warps take the registers that the producer / issuer warpgroup does not need.
  if (warp >= kSoftmaxWarps) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
  if (warp == kWarpProducer) {
    // ------------------------------------------------------------------ TMA producer of Q and K tiles
    // K and V have their own producer threads: a K tile is requested as soon as its slot has been
    // read by the QK two blocks earlier, whatever the state of the V FIFO (and the other way round).
    if (lane == 0) {
      BlockSeq<ItemDraw> seq;
      seq.init();
      seq.src.init(tail, a.status + 1, abort_flag, n_items);
      uint32_t nk = 0;                   // K tiles pushed so far
      uint32_t q_uses[kQBufs] = {0, 0};  // loads issued per Q buffer
      int kv_row0 = 0;                   // first kv row of the current item's request
      bool ok = true;
      while (ok && seq.next(a, ignore_empty)) {
        const int hk = seq.h;                 // a unit's head is the kv head; its q tile holds the
        const int hq = hk * a.group_size;     // group's q heads of 128 / group tokens, token-major
        if (seq.first()) {  // new item: its Q tile goes to buffer item_no & 1
          kv_row0 = seq.kv_row0;
          const int qb_i = seq.item_no % kQB;
          if (!mbar_wait(&tail->q_empty[qb_i], (q_uses[qb_i] & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          ++q_uses[qb_i];
          const int q_row = seq.q_row0;
          uint8_t* dst = smem_q + qb_i * kTB;
          mbar_expect_tx(&tail->q_full[qb_i], kLoadBytes);
#pragma unroll
          for (int i = 0; i < kHalves; ++i) tma_load_3d(dst + i * kHalfBytes, &a.tmap_q, &tail->q_full[qb_i], 64 * i, hq, q_row);
        }
        const int slot = static_cast<int>(nk % kRK);
        if (!mbar_wait(&tail->k_empty[slot], ((nk / kRK) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        ++nk;
        uint8_t* dst = smem_ring + slot * kTB;
        const int row = kv_row0 + seq.kvb * kBKV;
        mbar_expect_tx(&tail->k_full[slot], kLoadBytes);
#pragma unroll
        for (int i = 0; i < kHalves; ++i) tma_load_3d(dst + i * kHalfBytes, &a.tmap_k, &tail->k_full[slot], 64 * i, hk, row);
      }
    }
  } else if (warp == kWarpProducerV) {
    // ------------------------------------------------------------------ TMA producer of V tiles
    if (lane == 0) {
      BlockSeq<ItemRead<false>> seq;
      seq.init();
      seq.src.init(tail, abort_flag);
      uint32_t nv = 0;
      int kv_row0 = 0;
      bool ok = true;
      while (ok && seq.next(a, ignore_empty)) {
        const int hk = seq.h;
        if (seq.first()) kv_row0 = seq.kv_row0;
        const int slot = static_cast<int>(nv % kRV);
        if (!mbar_wait(&tail->v_empty[slot], ((nv / kRV) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        ++nv;
        uint8_t* dst = smem_ring + (kRK + slot) * kTB;
        const int row = kv_row0 + seq.kvb * kBKV;
        mbar_expect_tx(&tail->v_full[slot], kLoadBytes);
#pragma unroll
        for (int i = 0; i < kHalves; ++i) tma_load_3d(dst + i * kHalfBytes, &a.tmap_v, &tail->v_full[slot], 64 * i, hk, row);
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
      BlockSeq<ItemRead<false>> seq;
      seq.init();
      seq.src.init(tail, abort_flag);
      uint32_t g = 0, nk = 0;
      uint32_t q_uses[kQBufs] = {0, 0};
      bool ok = true;
      while (ok && seq.next(a, ignore_empty)) {
        const uint32_t sb = g & 1u;
        const int qb_i = seq.item_no % kQB;
        // S[sb] is free once the softmax has copied block g-2 into registers (head dimension 256: once the PV of
        // block g-2 has read the P that was written over it)
        if (g >= 2u && !mbar_wait(kWide ? &tail->pv_done[sb] : &tail->s_free[sb], ((g - 2u) >> 1) & 1u, abort_flag)) { ok = false; break; }
        if (seq.first()) {
          if (!mbar_wait(&tail->q_full[qb_i], q_uses[qb_i] & 1u, abort_flag)) { ok = false; break; }
          ++q_uses[qb_i];
        }
        const int slot = static_cast<int>(nk % kRK);
        if (!mbar_wait(&tail->k_full[slot], (nk / kRK) & 1u, abort_flag)) { ok = false; break; }
        ++nk;
        tc_fence_after_sync();
        const uint32_t q_lo = q_lo0 + static_cast<uint32_t>((qb_i * kTB) >> 4);
        const uint32_t k_lo = k_lo0 + static_cast<uint32_t>((slot * kTB) >> 4);
        uint32_t la[8], lb[8];
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // 16 elements further along K: +32 B inside a 64-column half, +16 KB for the second half
          const uint32_t off = static_cast<uint32_t>(((kk >> 2) * kHalfBytes + (kk & 3) * 32) >> 4);
          la[kk] = q_lo + off;
          lb[kk] = k_lo + off;
        }
        if constexpr (kD >= 128) umma_ss_x8(tmem_base + kColS + sb * 128u, hi, hi, idesc_qk, 0u, la, lb);
        else umma_ss_x4(tmem_base + kColS + sb * 128u, hi, hi, idesc_qk, 0u, la, lb);
        if constexpr (kWide) {  // the other two 64-column halves of Q and K, accumulated onto the first two
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t off = static_cast<uint32_t>((((kk >> 2) + 2) * kHalfBytes + (kk & 3) * 32) >> 4);
            la[kk] = q_lo + off;
            lb[kk] = k_lo + off;
          }
          umma_ss_x8(tmem_base + kColS + sb * 128u, hi, hi, idesc_qk, 1u, la, lb);
        }
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
      const uint64_t d0 = make_smem_desc_sw128(smem_u32(smem_ring + kRK * kTB), kHalfBytes, 1024);
      const uint32_t hi = static_cast<uint32_t>(d0 >> 32), v_lo0 = static_cast<uint32_t>(d0);
      BlockSeq<ItemRead<false>> seq;
      seq.init();
      seq.src.init(tail, abort_flag);
      uint32_t g = 0, nv = 0, items_started = 0;
      bool ok = true;
      while (ok && seq.next(a, ignore_empty)) {
        const uint32_t sb = g & 1u;
        if (!mbar_wait(&tail->p_full[sb], (g >> 1) & 1u, abort_flag)) { ok = false; break; }
        if (seq.first() && items_started > 0) {  // O must have been drained by the previous item's epilogue
          if (!mbar_wait(&tail->o_free, (items_started - 1u) & 1u, abort_flag)) { ok = false; break; }
        }
        const int slot = static_cast<int>(nv % kRV);
        if (!mbar_wait(&tail->v_full[slot], (nv / kRV) & 1u, abort_flag)) { ok = false; break; }
        ++nv;
        tc_fence_after_sync();
        const uint32_t tmem_p = tmem_base + (kWide ? kColS + sb * 128u : kColP + sb * 64u);
        const uint32_t v_lo = v_lo0 + static_cast<uint32_t>((slot * kTB) >> 4);
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
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    // ------------------------------------------------------------------ softmax / epilogue warps 0..15
    // Group X = warp / 8 takes the blocks with g & 1 == X. Two threads per q row: thread
    // (quadrant = warp & 3, half ch = (warp >> 2) & 1, lane) owns row 32 * quadrant + lane (its TMEM lane)
    // and the columns [64 ch, 64 ch + 64) of S[X], P[X] and (in a rescale) O; in the epilogue the 16 warps
    // cover O in 32-column quarters.
    const uint32_t X = static_cast<uint32_t>(warp >> 3), Y = X ^ 1u;
    const uint32_t ch = static_cast<uint32_t>((warp >> 2) & 1);
    const int quad = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tmem_s = tmem_base + lane_base + kColS + X * 128u + ch * 64u;
    const uint32_t tmem_p = tmem_base + lane_base + (kWide ? kColS + X * 128u : kColP + X * 64u) + ch * 32u;
    const uint32_t tmem_o = tmem_base + lane_base + kColO;
    const uint32_t ocol = static_cast<uint32_t>(kOW) * (2u * X + ch);  // this thread's quarter of O in the epilogue
    const bool has_cols = ocol < static_cast<uint32_t>(kD);  // head_dim 64: the second group's threads own no column of O
    const int row = quad * 32 + lane;
    uint64_t* pair_bar = &tail->pair_bar[X][quad];
    uint32_t pair_phase = 0;
    uint16_t* o16 = reinterpret_cast<uint16_t*>(a.o);
    bool ok = true;

    struct RowCtx {  // where an item's row lives in global memory (this thread's 32-column quarter)
      uint16_t* orow;
      float* lse;
      bool row_ok;
    };
    // Row r of a tile is token q_row0 + r / group, q head h * group + r % group (group = 1: the row itself).
    const int grp = a.group_size;
    auto row_ctx = [&](int q_row0, int q_valid, int h) -> RowCtx {
      RowCtx c;
      c.row_ok = static_cast<int>(row) < q_valid * grp;
      const int64_t grow = static_cast<int64_t>(q_row0) + static_cast<int>(row) / grp;
      const int hq = h * grp + static_cast<int>(row) % grp;
      c.orow = o16 + grow * a.o_stride_n + static_cast<int64_t>(hq) * a.o_stride_h + ocol;
      c.lse = (a.lse != nullptr && ocol == 0u) ? a.lse + grow * a.lse_stride_n + hq : nullptr;
      return c;
    };
    auto on_empty = [&](int q_row0, int q_valid, int hq) {  // active q-block that keeps nothing: zeros, lse = -5e4
      const RowCtx c = row_ctx(q_row0, q_valid, hq);
      if (c.row_ok && has_cols) {
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int i = 0; i < kOW / 8; ++i) reinterpret_cast<uint4*>(c.orow)[i] = z;
        if (c.lse != nullptr) *c.lse = -5e4f;
      }
    };

    GroupSeq<kMask != 0> seq;
    seq.init(tail, abort_flag);
    uint32_t g = 0;          // global block index (both parities)
    uint32_t my_blocks = 0;  // blocks this group has processed
    uint32_t items_seen = 0; // items whose last block has been passed
    float m_ref = -INFINITY; // the maximum this thread's partial sum refers to
    uint64_t l2a = 0, l2b = 0;  // partial row sum over this thread's columns of the group's blocks
    // an item whose statistics have been published and whose O is still being accumulated
    int cm_kv_len = 0, cm_base = 0;   // custom mask: the request's kv length, byte offset of its matrix,
    int64_t cm_row_bit = 0;           // and the bit offset of this thread's row inside it
    bool pend = false;
    uint32_t pend_item = 0;
    int pend_q_row0 = 0, pend_q_valid = 0, pend_h = 0, pend_parts = 1;
    uint32_t ep_phase = 0;
    // bounded barrier of the softmax warps (only the epilogue of a part of a split item uses it)
    auto ep_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(&tail->ep_bar);
      const bool r = __all_sync(0xffffffffu, mbar_wait(&tail->ep_bar, ep_phase, abort_flag) ? 1 : 0) != 0;
      ep_phase ^= 1u;
      return r;
    };

    auto epilogue = [&]() -> bool {
      const uint32_t ip = pend_item & 1u;
      if (!mbar_wait(&tail->stats_ready[ip], (pend_item >> 1) & 1u, abort_flag)) return false;
      float lsum = 0.f, m_fin = -INFINITY;
#pragma unroll
      for (int i = 0; i < 4; ++i) m_fin = fmaxf(m_fin, tail->stats_m[ip][i][row]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float mi = tail->stats_m[ip][i][row];
        const float ci = (mi == m_fin) ? 1.f : ex2_approx(mi - m_fin);
        lsum = fmaf(tail->stats_l[ip][i][row], ci, lsum);
      }
      if (!mbar_wait(&tail->o_full, pend_item & 1u, abort_flag)) return false;
      tc_fence_after_sync();
      uint32_t v[32];
      [[maybe_unused]] uint32_t v_hi[kWide ? 32 : 1];  // head dimension 256: the thread's second 32 columns
      if (has_cols) {
        tmem_ld_x32(tmem_o + ocol, v);
        if constexpr (kWide) tmem_ld_x32(tmem_o + ocol + 32u, v_hi);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int t = 0; t < 32; ++t) v[t] = 0u;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tail->o_free);  // O may be overwritten by the next item
      const RowCtx pend_ctx = row_ctx(pend_q_row0, pend_q_valid, pend_h);
      const int nparts = pend_parts & 0xff;
      float m_out = m_fin, l_out = lsum;
      if constexpr (kParts) {
        if (nparts > 1) {
          // ---- a part of a split item: the fp32 O (relative to m_fin), m_fin and the row sum go to the part's slot
          // as [column group of 4][row][4] (a warp's store covers 512 contiguous bytes); the part that delivers last
          // merges all of them, in ascending order whichever part it is (the result does not depend on it):
          // O = sum_p O_p 2^(m_p - m) / sum_p l_p 2^(m_p - m), m = max_p m_p.
          const int slot = static_cast<int>(static_cast<uint32_t>(pend_parts) >> 16), part = (pend_parts >> 8) & 0xff;
          float* ps = a.partials + static_cast<size_t>(slot) * kPartialFloats;
          if (has_cols) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<uint4*>(ps + (static_cast<size_t>(ocol / 4u + q) * 128 + row) * 4) =
                  make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          }
          if (ocol == 0u) {
            ps[128 * 128 + row] = m_fin;
            ps[128 * 128 + 128 + row] = lsum;
          }
          __threadfence();
          if (!ep_sync()) return false;
          if (warp == 0 && lane == 0) {
            int* cnt = a.arrive + (slot - part);  // a split item counts at its first slot
            const int old = atomicAdd(cnt, 1);
            const int mine = old == nparts - 1 ? 1 : 0;
            if (mine) *cnt = 0;  // the counter is back at zero for the next launch
            __threadfence();
            tail->merge_go = mine;
          }
          if (!ep_sync()) return false;
          if (tail->merge_go == 0) {  // another part will merge
            pend = false;
            return true;
          }
          const float* base = a.partials + static_cast<size_t>(slot - part) * kPartialFloats;
          float m_all = -INFINITY;
          for (int pp = 0; pp < nparts; ++pp)
            m_all = fmaxf(m_all, __ldcg(base + static_cast<size_t>(pp) * kPartialFloats + 128 * 128 + row));
          float l_all = 0.f;
#pragma unroll
          for (int t = 0; t < 32; ++t) v[t] = 0u;  // v becomes the accumulator (fp32 bit patterns)
          for (int pp = 0; pp < nparts; ++pp) {
            const float* pq = base + static_cast<size_t>(pp) * kPartialFloats;
            const float mp = __ldcg(pq + 128 * 128 + row);
            const float wgt = (mp == -INFINITY) ? 0.f : ex2_approx(mp - m_all);
            l_all = fmaf(__ldcg(pq + 128 * 128 + 128 + row), wgt, l_all);
            if (!has_cols) continue;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 x = __ldcg(reinterpret_cast<const float4*>(pq + (static_cast<size_t>(ocol / 4u + q) * 128 + row) * 4));
              v[4 * q] = __float_as_uint(fmaf(x.x, wgt, __uint_as_float(v[4 * q])));
              v[4 * q + 1] = __float_as_uint(fmaf(x.y, wgt, __uint_as_float(v[4 * q + 1])));
              v[4 * q + 2] = __float_as_uint(fmaf(x.z, wgt, __uint_as_float(v[4 * q + 2])));
              v[4 * q + 3] = __float_as_uint(fmaf(x.w, wgt, __uint_as_float(v[4 * q + 3])));
            }
          }
          m_out = m_all;
          l_out = l_all;
        }
      }
      const float inv_out = l_out > 0.f ? __frcp_rn(l_out) : 0.f;
      const bool whole = pend_q_valid * grp == kBQ;  // no row of the q-block is past the request
#pragma unroll
      for (int hh = 0; hh < kOW / 32; ++hh) {  // 32 columns at a time
        uint4 outv[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t w[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            uint32_t r0 = v[8 * q + 2 * t], r1 = v[8 * q + 2 * t + 1];
            if constexpr (kWide) {
              if (hh == 1) { r0 = v_hi[8 * q + 2 * t]; r1 = v_hi[8 * q + 2 * t + 1]; }
            }
            const float x0 = __uint_as_float(r0) * inv_out;
            const float x1 = __uint_as_float(r1) * inv_out;
            w[t] = kBf16 ? pack_bf16x2(x0, x1) : pack_f16x2(x0, x1);
          }
          outv[q] = make_uint4(w[0], w[1], w[2], w[3]);
        }
        if (!has_cols) {
          // head_dim 64: this thread's quarter of O does not exist
        } else if (whole) {
          // Through a 1 KB staging area per warp (16 rows x 64 bytes, plain row-major) and a TMA store of one
          // 16-row x 32-column box: a store instruction of a warp would otherwise write 32 scattered 16-byte pieces.
          uint8_t* stg = smem_ostage + warp * kOutStageBytes;
          const int grow0 = pend_q_row0 + (quad * 32) / grp;
#pragma unroll
          for (int ph = 0; ph < 2; ++ph) {
            if (lane == 0) tma_store_wait_read<0>();  // the staging area is free once its last store has read it
            __syncwarp();
            if ((lane >> 4) == ph) {
              const int r = lane & 15;
#pragma unroll
              for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(stg + r * 64 + c * 16) = outv[c];
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_3d(&a.tmap_o16, stg, static_cast<int>(ocol) + 32 * hh, pend_h * grp, grow0 + (ph * 16) / grp);
              tma_store_commit();
            }
          }
        } else if (pend_ctx.row_ok) {
          uint4* dst = reinterpret_cast<uint4*>(pend_ctx.orow) + 4 * hh;
#pragma unroll
          for (int q = 0; q < 4; ++q) dst[q] = outv[q];
        }
      }
      if (pend_ctx.row_ok && pend_ctx.lse != nullptr) *pend_ctx.lse = (l_out > 0.f) ? (log2f(l_out) + m_out) : -5e4f;
      pend = false;
      return true;
    };

    while (ok && seq.next(a, on_empty)) {
      if (seq.first()) {
        if constexpr (kMask == 2) {  // both groups: the row's bit offset inside the request's matrix
          const int q0 = a.qo_indptr[seq.req];
          cm_kv_len = a.kv_indptr[seq.req + 1] - a.kv_indptr[seq.req];
          cm_base = a.mask_indptr[seq.req];
          cm_row_bit = static_cast<int64_t>(seq.q_row0 - q0 + row / grp) * cm_kv_len;
        }
        m_ref = -INFINITY;
        l2a = 0;
        l2b = 0;
      }
      if ((g & 1u) == X) {
        // ---- this thread's half row of S[X] goes to registers once and stays there until the exponentials; S[X] is
        // handed back at once, so that the QK of this group's next block (about 1 800 clocks from here to a
        // visible S while other batches are in the pipe) runs under this block's softmax
        if (!mbar_wait(&tail->s_full[X], my_blocks & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        int valid = seq.valid() - static_cast<int>(64u * ch);  // of my columns, how many exist
        if constexpr (kMask == 1) {
          // ... and how many this row's token may attend to: kv positions up to causal_base + token
          const int lim = seq.causal_base + row / grp - seq.kvb * kBKV + 1;
          const int vc = (lim > kBKV ? kBKV : lim) - static_cast<int>(64u * ch);
          valid = valid < vc ? valid : vc;
        }
        uint32_t s[64];
        tmem_ld_x32(tmem_s, s);
        tmem_ld_x32(tmem_s + 32u, s + 32);
        tmem_wait_ld();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tail->s_free[X]);
        if (valid < 64) {
#pragma unroll
          for (int t = 0; t < 64; ++t)
            if (t >= valid) s[t] = 0xff800000u;  // -inf: exp2 gives 0
        }
        if constexpr (kMask == 2) {  // custom mask: one bit per column of this thread's half row
          const int col0 = seq.kvb * kBKV + static_cast<int>(64u * ch);
          int nb = cm_kv_len - col0;
          nb = nb > 64 ? 64 : nb;
          const uint64_t mbits =
              nb > 0 ? load_mask_bits64(a.custom_mask + cm_base, cm_row_bit + col0, a.custom_mask_bytes - cm_base, nb) : 0ull;
#pragma unroll
          for (int t = 0; t < 64; ++t)
            if (!((mbits >> t) & 1ull)) s[t] = 0xff800000u;
        }
        float mx;
        {
          float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int t = 0; t < 8; ++t) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              mxs[i] = fmax3(mxs[i], __uint_as_float(s[8 * t + 2 * i]), __uint_as_float(s[8 * t + 2 * i + 1]));
          }
          mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));
        }
        // ---- the two halves of a row exchange their maxima (the warps `warp` and `warp ^ 4`)
        tail->xmax[X][my_blocks & 1u][ch][row] = mx;
        __syncwarp();
        if (lane == 0) mbar_arrive(pair_bar);
        if (!mbar_wait(pair_bar, pair_phase, abort_flag)) { ok = false; break; }
        pair_phase ^= 1u;
        mx = fmaxf(mx, tail->xmax[X][my_blocks & 1u][ch ^ 1u][row]);
        // ---- the running maximum after block g-1 comes from the other group (every block waits, so
        // that the two groups stay within one phase of each other)
        if (g >= 1u && !mbar_wait(&tail->m_ready[Y], ((g - 1u) >> 1) & 1u, abort_flag)) { ok = false; break; }
        const float m_prev = seq.first() ? -INFINITY : tail->m_pub[Y][row];
        // with a soft cap the logit is cap * tanh(s * sm_scale / cap): monotonic, so the maximum is transformed once
        if constexpr (kSoftCap) mx = (mx == -INFINITY) ? mx : tanh_approx(mx * a.soft_cap_pre);
        const float m_new = fmaxf(m_prev, mx * a.sm_scale_log2);
        // lazy rescale (the decision is the same in both warps of a row: same rows, same values)
        const bool need = (m_new - m_prev) > kRescaleThreshold;
        const bool rescale = !seq.first() && __any_sync(0xffffffffu, need);
        const float m_used = (seq.first() || (rescale && need)) ? m_new : m_prev;
        if (ch == 0u) tail->m_pub[X][row] = m_used;
        __syncwarp();
        if (lane == 0) mbar_arrive(&tail->m_ready[X]);
        // this thread's partial sum follows the maximum in use
        if (m_ref != m_used) {
          const float beta = ex2_approx(m_ref - m_used);
          const uint64_t beta2 = pack_f32x2(beta, beta);
          l2a = ffma2(l2a, beta2, 0ull);
          l2b = ffma2(l2b, beta2, 0ull);
          m_ref = m_used;
        }
        // P[X] was last read by the PV of this group's previous block
        if (my_blocks >= 1u && !mbar_wait(&tail->pv_done[X], (my_blocks - 1u) & 1u, abort_flag)) { ok = false; break; }
        // ---- pass 2: P = exp2(S * scale - m_used), row sum, P (16 bit) to TMEM: one FMA and one add per
        // PAIR of columns
        const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
        const uint64_t scale2 = pack_f32x2(a.sm_scale_log2, a.sm_scale_log2);
        const uint64_t negm2 = pack_f32x2(neg_m, neg_m);
        if constexpr (kSoftCap) {
#pragma unroll
          for (int t = 0; t < 64; ++t)  // masked columns stay at -inf
            if (s[t] != 0xff800000u) s[t] = __float_as_uint(tanh_approx(__uint_as_float(s[t]) * a.soft_cap_pre));
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
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
          tmem_st_x16(tmem_p + 16u * c, pk);
        }
        tmem_wait_st();
        if (rescale) {
          // (after the exponentials, when S has left the registers, and before P is handed over: the PV of this
          // block must see the rescaled O) O is rescaled only after the PV of block g-1 has completed; that PV may be the first of
          // its item and wait for the previous item's epilogue, so this thread's share of it goes first
          if (pend && !epilogue()) { ok = false; break; }
          if (!mbar_wait(&tail->pv_done[Y], ((g - 1u) >> 1) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const float alpha = need ? ex2_approx(m_prev - m_new) : 1.0f;
#pragma unroll
          for (int c = 0; c < kD / 64; ++c) {  // this thread's half of the row of O: kD / 2 columns
            uint32_t v[32];
            tmem_ld_x32(tmem_o + static_cast<uint32_t>(kD / 2) * ch + 32u * c, v);
            tmem_wait_ld();
#pragma unroll
            for (int t = 0; t < 32; ++t) v[t] = __float_as_uint(__uint_as_float(v[t]) * alpha);
            tmem_st_x32(tmem_o + static_cast<uint32_t>(kD / 2) * ch + 32u * c, v);
          }
          tmem_wait_st();
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tail->p_full[X]);
        ++my_blocks;
        // the previous item's epilogue runs after this group's first block of the next item, so that
        // the item's last PV overlaps a softmax step (running it before the block, in the wait for S,
        // frees O earlier for the next item's first PV but measured 9 % slower: it delays the group's
        // own chain, which is the longer one)
        if (pend && !epilogue()) { ok = false; break; }
      }
      if (seq.last()) {
        if (pend && !epilogue()) { ok = false; break; }
        const uint32_t ip = items_seen & 1u;
        float la, lb, lc, ld;
        unpack_f32x2(l2a, la, lb);
        unpack_f32x2(l2b, lc, ld);
        tail->stats_m[ip][2u * X + ch][row] = m_ref;
        tail->stats_l[ip][2u * X + ch][row] = (la + lb) + (lc + ld);
        __syncwarp();
        if (lane == 0) mbar_arrive(&tail->stats_ready[ip]);
        pend = true;
        pend_item = items_seen;
        pend_q_row0 = seq.q_row0; pend_q_valid = seq.q_valid; pend_h = seq.h; pend_parts = seq.parts;
        ++items_seen;
      }
      ++g;
    }
    if (ok && pend) epilogue();
    if (lane == 0) tma_store_wait_all<0>();
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
  if (warp == kWarpMma) {
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

}  // namespace


namespace {
template <bool kBf16, bool kSoftCap, bool kParts, int kD, int kMask = 0>
cudaError_t launch_one(const AttnArgs& a, int ctas, cudaStream_t stream) {
  const cudaError_t e = cudaFuncSetAttribute(attention_kernel<kBf16, kSoftCap, kParts, kD, kMask>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return e;
  attention_kernel<kBf16, kSoftCap, kParts, kD, kMask><<<ctas, kThreads, kSmemBytes, stream>>>(a);
  return cudaGetLastError();
}
template <bool kBf16, bool kSoftCap>
cudaError_t launch_two(const AttnArgs& a, int ctas, cudaStream_t stream) {
  if (a.head_dim == 256) {  // whole items only
    if (a.partial_slots > 0) return cudaErrorInvalidValue;
    if (a.mask_mode == 1) return launch_one<kBf16, kSoftCap, false, 256, 1>(a, ctas, stream);
    if (a.mask_mode == 2) return launch_one<kBf16, kSoftCap, false, 256, 2>(a, ctas, stream);
    return launch_one<kBf16, kSoftCap, false, 256>(a, ctas, stream);
  }
  if (a.mask_mode != 0) {  // whole items only (the caller gives no room for partial results)
    if (a.partial_slots > 0) return cudaErrorInvalidValue;
    if (a.mask_mode == 1)
      return a.head_dim == 64 ? launch_one<kBf16, kSoftCap, false, 64, 1>(a, ctas, stream)
                              : launch_one<kBf16, kSoftCap, false, 128, 1>(a, ctas, stream);
    return a.head_dim == 64 ? launch_one<kBf16, kSoftCap, false, 64, 2>(a, ctas, stream)
                            : launch_one<kBf16, kSoftCap, false, 128, 2>(a, ctas, stream);
  }
  // room for partial results means that the unit builder may have cut lists: the instantiation with the merge
  if (a.head_dim == 64)
    return a.partial_slots > 0 ? launch_one<kBf16, kSoftCap, true, 64>(a, ctas, stream)
                               : launch_one<kBf16, kSoftCap, false, 64>(a, ctas, stream);
  return a.partial_slots > 0 ? launch_one<kBf16, kSoftCap, true, 128>(a, ctas, stream)
                             : launch_one<kBf16, kSoftCap, false, 128>(a, ctas, stream);
}
}  // namespace

cudaError_t launch_attention(const AttnArgs& a, int max_ctas, cudaStream_t stream) {
  if (max_ctas <= 0) return cudaSuccess;
  const bool cap = a.soft_cap_pre > 0.f;
  if (a.is_bf16) return cap ? launch_two<true, true>(a, max_ctas, stream) : launch_two<true, false>(a, max_ctas, stream);
  return cap ? launch_two<false, true>(a, max_ctas, stream) : launch_two<false, false>(a, max_ctas, stream);
}

}  // namespace fo
