// GEMM-Q / GEMM-O on tcgen05: one persistent, warp-specialised kernel.
//
//   Y[b, rows(iy), cols(ix)] = init + sum_{k-blocks of the tile} X[b, rows, kblk] * W[cols, kblk]^T
//
// GEMM-Q (reference: include/flashomni/gemm/w16a16/gemm.cuh:27-228): the tile list holds only the
// active 128x128 output tiles; every tile runs the whole K range; init = bias[cols] or 0; tiles
// that are not listed are never touched.
// GEMM-O (reference: include/flashomni/gemm/w16a16/gemm_reduction.cuh:27-276): every output tile is
// produced; its K loop visits only the K-slices of the heads selected for its row block (compacted
// list, ascending); init = cache[b, rows, cols] or bias[cols] or 0.
//
// A CTA works on "pair tiles": one 128-row A tile against TWO 128-column blocks of W (any two: for
// GEMM-Q they are two active heads of the same row block), issued as one UMMA of N = 256 so that
// the A operand is read from shared memory once per 256 output columns. A leftover single block
// runs as N = 128.
//
// CTA = 192 threads: warps 0-3 epilogue, warp 4 TMA producer, warp 5 MMA issuer. K step 64 (one
// 128-byte swizzle atom), 4-stage ring of (A 16 KB + B 32 KB), two 256-column TMEM accumulators so
// the epilogue of tile i overlaps the main loop of tile i+1. The epilogue converts 64-column slabs
// (TMEM -> registers -> +init -> 16-bit) into a swizzled shared-memory slab and hands each slab to a
// TMA store, so global writes are full 128-byte lines and asynchronous. The tiles of the sparse modes
// (unequal lengths) are handed to the persistent CTAs through a device-wide cursor, in list order; the
// equal tiles of a dense launch keep fixed round-robin shares.
#include <cuda_fp16.h>

#include "internal.h"

namespace fo {
namespace {

constexpr int kBM = 128, kBNH = 128, kBK = 64;
constexpr int kStages = 4;
constexpr int kABytes = kBM * kBK * 2;        // 16 KB
constexpr int kBHalfBytes = kBNH * kBK * 2;   // 16 KB per 128-column block of W
constexpr int kStageBytes = kABytes + 2 * kBHalfBytes;
constexpr int kSlabCols = 64;
constexpr int kSlabBytes = kBM * kSlabCols * 2;  // 16 KB
constexpr int kSlabBufs = 2;
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr int kMaxHeadsSmem = 128;
constexpr int kTileQ = 8;   // entries of the tile queue (the producer runs at most a few tiles ahead of the epilogue)

struct Tail {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t tq_full[kTileQ];   // tile queue: the producer warp draws tile numbers and hands them to the other roles
  uint64_t tq_empty[kTileQ];
  int tile_q[kTileQ];
  uint32_t tmem_base;
  int abort_flag;
  int epi_go;                   // outcome of the epilogue warps' vote of the current round
  int heads[2][kMaxHeadsSmem];  // GEMM-O: head lists of the current and the next tile, staged for the producer
};
constexpr int kSmemBytes = kStages * kStageBytes + kSlabBufs * kSlabBytes + 1024 + static_cast<int>(sizeof(Tail));


struct TileInfo {
  int a_row;             // first row of the A tile in [batch*m]
  int w_row0, w_row1;    // first rows of the two W blocks (= first output columns); w_row1 < 0: single
  int nkb;               // number of 64-wide K blocks
  const int32_t* heads;  // GEMM-O: selected heads of the row block (null for GEMM-Q)
};

__device__ __forceinline__ int pairs_per_row(const GemmArgs& a) { return (a.n / kBNH + 1) / 2; }

__device__ __forceinline__ int num_tiles(const GemmArgs& a) {
  if (a.mode == kGemmQ && a.tiles != nullptr) {
    const int cap = a.batch * (a.m / kBM) * (a.n / kBNH);  // a list holds at most one record per 128x128 tile
    const int n = *a.n_tiles_ptr;
    return n < cap ? (n < 0 ? 0 : n) : cap;
  }
  return a.batch * (a.m / kBM) * pairs_per_row(a);
}

__device__ __forceinline__ TileInfo get_tile(const GemmArgs& a, int t) {
  TileInfo ti;
  const int nct = a.n / kBNH;
  if (a.mode == kGemmQ && a.tiles != nullptr) {
    const int4 rec = *reinterpret_cast<const int4*>(a.tiles + 4 * t);  // (b, iy, ix0, ix1)
    ti.a_row = rec.x * a.m + rec.y * kBM;
    ti.w_row0 = rec.z * kBNH;
    ti.w_row1 = rec.w >= 0 ? rec.w * kBNH : -1;
    ti.nkb = (a.k + kBK - 1) / kBK;  // a last partial K block reads zeros past k (TMA fill)
    ti.heads = nullptr;
    return ti;
  }
  const int npr = pairs_per_row(a);
  const int j = t % npr;
  const int rr = t / npr;
  ti.w_row0 = (2 * j) * kBNH;
  ti.w_row1 = (2 * j + 1 < nct) ? (2 * j + 1) * kBNH : -1;
  if (a.mode == kGemmQ) {  // dense: row blocks in natural order
    ti.a_row = rr * kBM;
    ti.nkb = (a.k + kBK - 1) / kBK;  // a last partial K block reads zeros past k (TMA fill)
    ti.heads = nullptr;
  } else {
    const int r = a.row_order[rr];
    ti.a_row = r * kBM;
    const int h0 = a.row_indptr[r], h1 = a.row_indptr[r + 1];
    ti.heads = a.row_heads + h0;
    ti.nkb = (h1 - h0) * a.kb_per_head;
  }
  return ti;
}

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <bool kBf16>
__global__ void __launch_bounds__(kThreads, 1) gemm_kernel(const __grid_constant__ GemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* smem_slab = smem + kStages * kStageBytes;
  Tail* tail = reinterpret_cast<Tail*>(smem_slab + kSlabBufs * kSlabBytes);
  volatile int* abort_flag = &tail->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&tail->full[s], 1);
      mbar_init(&tail->empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tail->acc_full[i], 1);
      mbar_init(&tail->acc_empty[i], 4);
    }
    for (int i = 0; i < kTileQ; ++i) {
      mbar_init(&tail->tq_full[i], 1);
      mbar_init(&tail->tq_empty[i], 5);  // the MMA thread and the four epilogue warps
    }
    tail->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&a.tmap_a);
    tma_prefetch_desc(&a.tmap_b);
    tma_prefetch_desc(&a.tmap_y);
  }
  if (warp == 5) {
    tmem_alloc(&tail->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tail->tmem_base;

  const int n_tiles = num_tiles(a);
  // Tiles are handed out in list order through a device-wide cursor (the GEMM-O rows are sorted
  // longest first, the GEMM-Q list ends with its half-size tiles), so that a CTA that finishes early
  // takes the next tile instead of idling at the end of a fixed share. Tile i < gridDim.x goes to CTA i; the cursor counts the tiles after those.
  // Entry k of a CTA's sequence travels through slot k % kTileQ; -1 ends the sequence.
  auto read_slot = [&](int k) -> int {  // one thread of a consumer role; -2 when the wait gave up
    const int slot = k % kTileQ;
    if (!mbar_wait(&tail->tq_full[slot], static_cast<uint32_t>(k / kTileQ) & 1u, abort_flag)) return -2;
    const int t = tail->tile_q[slot];
    mbar_arrive(&tail->tq_empty[slot]);
    return t;
  };

  if (warp == 4) {
    // ------------------------------------------------------------- TMA producer
    // All lanes stage the tile's head list in shared memory (one coalesced read instead of one
    // dependent global load per K block); lane 0 then issues the copies.
    // The head list of tile i+1 is fetched into registers while lane 0 feeds tile i, so that the
    // dependent global loads (row order -> row indptr -> heads) never sit between two tiles.
    int stage = 0;
    uint32_t phase = 0;
    int ok = 1;
    TileInfo nxt;
    nxt.a_row = nxt.w_row0 = nxt.nkb = 0; nxt.w_row1 = -1; nxt.heads = nullptr;
    int hreg[kMaxHeadsSmem / 32];
    auto fetch_heads = [&](const TileInfo& ti) {
      if (ti.heads == nullptr) return;
      const int nh = ti.nkb / a.kb_per_head;
#pragma unroll
      for (int i = 0; i < kMaxHeadsSmem / 32; ++i) hreg[i] = (lane + 32 * i < nh && nh <= kMaxHeadsSmem) ? ti.heads[lane + 32 * i] : 0;
    };
    auto stash_heads = [&](int par) {
#pragma unroll
      for (int i = 0; i < kMaxHeadsSmem / 32; ++i) tail->heads[par][lane + 32 * i] = hreg[i];
    };
    int n_pub = 0;  // entries published so far (lane 0)
    auto publish = [&](int t) -> bool {  // lane 0
      const int slot = n_pub % kTileQ;
      if (!mbar_wait(&tail->tq_empty[slot], (static_cast<uint32_t>(n_pub / kTileQ) & 1u) ^ 1u, abort_flag)) return false;
      tail->tile_q[slot] = t;
      mbar_arrive(&tail->tq_full[slot]);
      ++n_pub;
      return true;
    };
    int n_drawn = 0;
    auto draw = [&]() -> int {  // lane 0: the next tile of the device-wide sequence
      // equal tiles (dense: no cursor) keep the fixed round-robin share and skip the atomic
      ++n_drawn;
      const int t = a.cursor != nullptr ? atomicAdd(a.cursor, 1) + static_cast<int>(gridDim.x)
                                        : static_cast<int>(blockIdx.x) + n_drawn * static_cast<int>(gridDim.x);
      return t < n_tiles ? t : -1;
    };
    // t_cur is being loaded, t_n1 is known and published, t_n2 is drawn while t_cur runs (two tiles of
    // lead, so that the atomic's round trip never sits between two tiles)
    int t_cur = static_cast<int>(blockIdx.x) < n_tiles ? static_cast<int>(blockIdx.x) : -1;
    int t_n1 = -1;
    if (lane == 0) {
      ok = publish(t_cur) ? 1 : 0;
      if (ok && t_cur >= 0) {
        t_n1 = draw();
        ok = publish(t_n1) ? 1 : 0;
      }
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    t_n1 = __shfl_sync(0xffffffffu, t_n1, 0);
    if (t_cur >= 0) {
      nxt = get_tile(a, t_cur);
      fetch_heads(nxt);
      stash_heads(0);
    }
    __syncwarp();
    int par = 0;
    while (t_cur >= 0 && ok) {
      int t_n2 = -1;
      if (lane == 0 && t_n1 >= 0) t_n2 = draw();
      TileInfo ti = nxt;
      if (ti.heads != nullptr && ti.nkb / a.kb_per_head <= kMaxHeadsSmem) ti.heads = tail->heads[par];
      const bool more = t_n1 >= 0;
      if (more) {
        nxt = get_tile(a, t_n1);
        fetch_heads(nxt);
      }
      if (lane == 0) {
        const uint32_t bytes = ti.w_row1 >= 0 ? kStageBytes : (kABytes + kBHalfBytes);
        // K columns are generated without divisions: (head list entry, K block inside the head)
        int hh = 0, sub = 0;
        int kcol = (ti.heads != nullptr && ti.nkb > 0) ? ti.heads[0] * a.kb_per_head * kBK : 0;
        for (int j = 0; j < ti.nkb; ++j) {
          if (!mbar_wait(&tail->empty[stage], phase ^ 1u, abort_flag)) { ok = 0; break; }
          uint8_t* sa = smem + stage * kStageBytes;
          mbar_expect_tx(&tail->full[stage], bytes);
          tma_load_2d(sa, &a.tmap_a, &tail->full[stage], kcol, ti.a_row);
          tma_load_2d(sa + kABytes, &a.tmap_b, &tail->full[stage], kcol, ti.w_row0);
          if (ti.w_row1 >= 0)
            tma_load_2d(sa + kABytes + kBHalfBytes, &a.tmap_b, &tail->full[stage], kcol, ti.w_row1);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
          // next K block
          if (ti.heads == nullptr) {
            kcol += kBK;
          } else if (++sub < a.kb_per_head) {
            kcol += kBK;
          } else {
            sub = 0;
            ++hh;
            if (j + 1 < ti.nkb) kcol = ti.heads[hh] * a.kb_per_head * kBK;
          }
        }
        if (ok && more && !publish(t_n2)) ok = 0;
      }
      __syncwarp();
      if (more) stash_heads(par ^ 1);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      stage = __shfl_sync(0xffffffffu, stage, 0);
      phase = __shfl_sync(0xffffffffu, phase, 0);
      t_n2 = __shfl_sync(0xffffffffu, t_n2, 0);
      t_cur = t_n1;
      t_n1 = t_n2;
      par ^= 1;
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc256 = make_idesc_f16(kBM, 2 * kBNH, kBf16, 0, 0);
      constexpr uint32_t idesc128 = make_idesc_f16(kBM, kBNH, kBf16, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      // every operand tile is K-major with 128-byte swizzle: same descriptor high word, low word = address
      const uint64_t desc0 = make_smem_desc_sw128(smem_u32(smem), 16, 1024);
      const uint32_t desc_hi = static_cast<uint32_t>(desc0 >> 32), desc_lo0 = static_cast<uint32_t>(desc0);
      TileInfo nxt;
      nxt.a_row = nxt.w_row0 = nxt.nkb = 0; nxt.w_row1 = -1; nxt.heads = nullptr;
      int k_seq = 0;
      int t_cur = read_slot(0);
      if (t_cur >= 0) nxt = get_tile(a, t_cur);
      for (; t_cur >= 0 && ok; ++k_seq) {
        const TileInfo ti = nxt;  // the next tile's record is fetched while this one runs
        const int t_nxt = read_slot(k_seq + 1);
        if (t_nxt >= 0) nxt = get_tile(a, t_nxt);
        if (t_nxt == -2) ok = false;
        t_cur = t_nxt;
        const uint32_t idesc = ti.w_row1 >= 0 ? idesc256 : idesc128;
        if (!mbar_wait(&tail->acc_empty[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * 2 * kBNH);
        for (int j = 0; j < ti.nkb; ++j) {
          if (!mbar_wait(&tail->full[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          // descriptor low words of the 4 K = 16 steps (advancing 32 bytes inside the swizzle atom = +2)
          const uint32_t a_lo = desc_lo0 + static_cast<uint32_t>((stage * kStageBytes) >> 4);
          const uint32_t b_lo = a_lo + static_cast<uint32_t>(kABytes >> 4);
          const uint32_t la[4] = {a_lo, a_lo + 2u, a_lo + 4u, a_lo + 6u};
          const uint32_t lb[4] = {b_lo, b_lo + 2u, b_lo + 4u, b_lo + 6u};
          umma_ss_x4(d_tmem, desc_hi, desc_hi, idesc, j != 0 ? 1u : 0u, la, lb);
          umma_commit(&tail->empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&tail->acc_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue warps 0..3
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t slab_count = 0;  // slabs handed to TMA stores so far (selects the staging buffer)
    const uint16_t* init16 = reinterpret_cast<const uint16_t*>(a.init);
    const int r_in_tile = warp * 32 + lane;
    const uint32_t swz = static_cast<uint32_t>(r_in_tile & 7);
    TileInfo nxt;
    nxt.a_row = nxt.w_row0 = nxt.nkb = 0; nxt.w_row1 = -1; nxt.heads = nullptr;
    auto read_slot_warp = [&](int k) -> int {  // lane 0 reads, the warp shares the value
      int t = 0;
      if (lane == 0) t = read_slot(k);
      return __shfl_sync(0xffffffffu, t, 0);
    };
    int k_seq = 0;
    int t_cur = read_slot_warp(0);
    if (t_cur >= 0) nxt = get_tile(a, t_cur);
    // The four warps leave this loop together: every round ends in a vote (two CTA-local barriers around one
    // shared word), so a wait that ran out in one warp can never leave the others behind at `epi_bar`.
    for (;; ++k_seq) {
      const TileInfo ti = nxt;
      const int t_this = t_cur;
      bool fail = t_this == -2;
      if (t_this >= 0) {
        const int t_nxt = read_slot_warp(k_seq + 1);
        if (t_nxt >= 0) nxt = get_tile(a, t_nxt);
        t_cur = t_nxt;
      }
      const int64_t row = static_cast<int64_t>(ti.a_row) + r_in_tile;
      const int nslab = ti.w_row1 >= 0 ? 4 : 2;
      // init values of slab 0 are fetched before the accumulator is waited for
      uint4 initv[8];
      auto load_init = [&](int s) {
        const int col0 = ((s >> 1) == 0 ? ti.w_row0 : ti.w_row1) + (s & 1) * kSlabCols;
        if (a.init_mode == kInitBias1D) {
          const uint4* p = reinterpret_cast<const uint4*>(init16 + col0);
#pragma unroll
          for (int i = 0; i < 8; ++i) initv[i] = __ldg(p + i);
        } else if (a.init_mode == kInitFull) {
          const uint4* p = reinterpret_cast<const uint4*>(init16 + row * a.n + col0);
#pragma unroll
          for (int i = 0; i < 8; ++i) initv[i] = __ldg(p + i);
        }
      };
      if (t_this >= 0) {
        load_init(0);
        if (!mbar_wait_warp(&tail->acc_full[acc], acc_phase, abort_flag)) fail = true;
      }
      if (fail && lane == 0) *abort_flag = 1;
      epi_bar();
      if (threadIdx.x == 0) tail->epi_go = (*abort_flag == 0) ? 1 : 0;
      epi_bar();
      if (tail->epi_go == 0 || t_this < 0) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + static_cast<uint32_t>(acc * 2 * kBNH);
#pragma unroll 1
      for (int s = 0; s < nslab; ++s) {
        const int col0 = ((s >> 1) == 0 ? ti.w_row0 : ti.w_row1) + (s & 1) * kSlabCols;
        uint32_t v0[32], v1[32];
        if (ti.nkb > 0) {
          tmem_ld_x32(taddr + static_cast<uint32_t>(s * kSlabCols), v0);
          tmem_ld_x32(taddr + static_cast<uint32_t>(s * kSlabCols + 32), v1);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) { v0[i] = 0u; v1[i] = 0u; }
        }
        if (s == nslab - 1) {  // accumulator fully read: hand it back to the MMA warp
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tail->acc_empty[acc]);
        }
        uint4 outv[8];
        uint32_t* o32 = reinterpret_cast<uint32_t*>(outv);
        const uint32_t* a32 = reinterpret_cast<const uint32_t*>(initv);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float lo = __uint_as_float(i < 16 ? v0[2 * i] : v1[2 * i - 32]);
          float hi = __uint_as_float(i < 16 ? v0[2 * i + 1] : v1[2 * i - 31]);
          if (a.init_mode != kInitNone) {
            if (kBf16) {
              lo += __uint_as_float(a32[i] << 16);
              hi += __uint_as_float(a32[i] & 0xFFFF0000u);
            } else {
              const __half2 h2 = *reinterpret_cast<const __half2*>(&a32[i]);
              lo += __low2float(h2);
              hi += __high2float(h2);
            }
          }
          o32[i] = kBf16 ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
        }
        if (s + 1 < nslab) load_init(s + 1);  // next slab's init loads fly during the store hand-off
        // staging buffer of this slab must no longer be read by the store issued two slabs ago
        uint8_t* buf = smem_slab + (slab_count & 1u) * kSlabBytes;
        if (threadIdx.x == 0) tma_store_wait_read<1>();
        epi_bar();
        uint8_t* rowp = buf + r_in_tile * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(rowp + ((static_cast<uint32_t>(c) ^ swz) << 4)) = outv[c];
        fence_proxy_async_smem();
        epi_bar();
        if (threadIdx.x == 0) {
          tma_store_2d(&a.tmap_y, buf, col0, ti.a_row);
          tma_store_commit();
        }
        ++slab_count;
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (threadIdx.x == 0) tma_store_wait_all<0>();
  }

  // ------------------------------------------------------------- common exit
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    // give copies that may still be in flight time to land before the CTA's smem is released
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    if (threadIdx.x == 0) atomicExch(a.status, kDevWaitTimeout);
    __syncthreads();
  }
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  // the last CTA to get here puts the tile cursor (and its own arrival count, the word after it) back to zero,
  // so the next launch over the same workspace needs no reset in between
  if (threadIdx.x == 0 && a.cursor != nullptr) {
    __threadfence();
    if (atomicAdd(a.cursor + 1, 1) == static_cast<int>(gridDim.x) - 1) {
      atomicExch(a.cursor, 0);
      atomicExch(a.cursor + 1, 0);
    }
  }
}

}  // namespace


cudaError_t launch_gemm(const GemmArgs& a, int max_ctas, cudaStream_t stream) {
  const int cap = a.batch * (a.m / kBM) * ((a.mode == kGemmQ && a.tiles != nullptr) ? a.n / kBNH : (a.n / kBNH + 1) / 2);
  if (cap <= 0) return cudaSuccess;
  const int grid = cap < max_ctas ? cap : max_ctas;
  cudaError_t e;
  if (a.is_bf16) {
    e = cudaFuncSetAttribute(gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    gemm_kernel<true><<<grid, kThreads, kSmemBytes, stream>>>(a);
  } else {
    e = cudaFuncSetAttribute(gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    gemm_kernel<false><<<grid, kThreads, kSmemBytes, stream>>>(a);
  }
  return cudaGetLastError();
}

}  // namespace fo
