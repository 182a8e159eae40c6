// Dense projection GEMM with 256x256 (or 256x192) output tiles: Y[rows, n] = X[rows, k] W[n, k]^T (+ bias).
//
// Why a second GEMM kernel: the path from L2 to the SMs is what limits the 128x256 tiles of gemm.cu (48 KB
// of operands per 512 tensor clocks = 94 B/clk per SM against about 84 B/clk that all SMs can pull from L2 at
// once). A 256x256 tile needs 64 KB per 1024 tensor clocks (62.5 B/clk): two 128-row halves of X share one
// 256-column block of W in shared memory. Only the dense mode uses it (a sparse GEMM-Q would need two row
// blocks with the same active heads); shapes whose N is not a multiple of 256 or 192 fall back to gemm.cu.
// The 192-column variant (56 KB per 768 tensor clocks, 73 B/clk) exists for shapes whose tiles fill the SMs
// badly at 256 columns: a narrow projection (one GPU's share of the heads) gets 4/3 as many tiles, each 3/4 as
// long, and the launch lasts as long as its fullest SM (tall_tile_cols picks the width).
//
// One persistent CTA per SM, 384 threads. Warp 8: TMA producer, 3 stages of 64 KB (X top, X bottom, W, W).
// Warps 9 and 10: MMA issuers, per K block of 64 four 128x256x16 MMAs into the top accumulator (TMEM columns
// 0-255) by the one and four into the bottom one (256-511) by the other. Both accumulators belong to the same
// tile, so the read-out of a tile cannot overlap the next tile's MMAs; to keep that gap short the epilogue has
// one warpgroup per half (warps 0-3 top, 4-7 bottom: TMEM lane quadrant = warp % 4), reads the whole
// accumulator into registers first and stores it through a small per-warp staging area (TMA stores of 16 x 64
// boxes) while the next tile's MMAs already run. A shape whose row count is an odd multiple of 128 leaves the
// bottom half of its last row pair empty. Every mbarrier wait is bounded.
#include <cuda_fp16.h>

#include "internal.h"

namespace fo {
namespace {

constexpr int kBM = 128, kBK = 64;
constexpr int kStages = 3;
constexpr int kHalfBytes = kBM * kBK * 2;          // 16 KB: a 128-row K block of X or W
constexpr int kStageBytesMax = 4 * kHalfBytes;     // X top | X bottom | W rows 0-127 | W rows 128-(kBN-1)
constexpr int kEpiWarps = 8;
constexpr int kWarpProducer = kEpiWarps, kWarpMma = kEpiWarps + 1;  // warps 9 and 10 issue the MMAs of one half each
constexpr int kThreads = (kEpiWarps + 4) * 32;     // 384: three warpgroups (warp 11 only takes part in the set-up)
constexpr int kRegsEpilogue = 208, kRegsOther = 40;  // setmaxnreg split: the epilogue holds a 256-column row in registers
static_assert(kEpiWarps * 32 * kRegsEpilogue + 4 * 32 * kRegsOther <= kThreads * ((65536 / kThreads) / 8 * 8),
              "register split exceeds the CTA's register pool");
constexpr int kTmemCols = 512;

struct Tail {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];    // [half]
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int kStageWarpBytes = 16 * 128;          // store staging per epilogue warp
constexpr int kSmemBytes = kStages * kStageBytesMax + kEpiWarps * kStageWarpBytes + 1024 + static_cast<int>(sizeof(Tail));


template <bool kBf16, int kBN>
__global__ void __launch_bounds__(kThreads, 1) gemm_tall_kernel(const __grid_constant__ GemmArgs a) {
  static_assert(kBN == 256 || kBN == 192, "tile width");
  constexpr int kStageBytes = 2 * kHalfBytes + kBN * kBK * 2;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* smem_stage = smem + kStages * kStageBytesMax;
  Tail* tail = reinterpret_cast<Tail*>(smem_stage + kEpiWarps * kStageWarpBytes);
  volatile int* abort_flag = &tail->abort_flag;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&tail->full[s], 1);
      mbar_init(&tail->empty[s], 2);  // both issuers have read the stage
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tail->acc_full[i], 1);
      mbar_init(&tail->acc_empty[i], 4);
    }
    tail->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kWarpProducer && lane == 0) {
    tma_prefetch_desc(&a.tmap_a);
    tma_prefetch_desc(&a.tmap_b);
    if (kBN != 256) tma_prefetch_desc(&a.tmap_b64);
    tma_prefetch_desc(&a.tmap_y);
  }
  if (warp == kWarpMma) {
    tmem_alloc(&tail->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tail->tmem_base;

  const int col_tiles = a.n / kBN;
  const int total_rows = a.batch * a.m;  // a multiple of 128; an odd last row block leaves the bottom half of its
                                         // tile empty (the loads past the end return zeros, nothing is stored)
  const int n_tiles = ((total_rows + 2 * kBM - 1) / (2 * kBM)) * col_tiles;
  const int nkb = a.k / kBK;
  // tile t: row pair t / col_tiles, column block t % col_tiles (CTAs that run together share X rows and W columns)

  if (warp >= kEpiWarps) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
  if (warp == kWarpProducer) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        const int a_row = (t / col_tiles) * 2 * kBM;
        const int w_row = (t % col_tiles) * kBN;
        for (int j = 0; j < nkb; ++j) {
          if (!mbar_wait(&tail->empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* s = smem + stage * kStageBytes;
          mbar_expect_tx(&tail->full[stage], kStageBytes);
          tma_load_2d(s, &a.tmap_a, &tail->full[stage], j * kBK, a_row);
          tma_load_2d(s + kHalfBytes, &a.tmap_a, &tail->full[stage], j * kBK, a_row + kBM);
          tma_load_2d(s + 2 * kHalfBytes, &a.tmap_b, &tail->full[stage], j * kBK, w_row);
          if (kBN == 256) tma_load_2d(s + 3 * kHalfBytes, &a.tmap_b, &tail->full[stage], j * kBK, w_row + kBM);
          else tma_load_2d(s + 3 * kHalfBytes, &a.tmap_b64, &tail->full[stage], j * kBK, w_row + kBM);  // 64 rows
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == kWarpMma || warp == kWarpMma + 1) {
    // Two issuing threads, one per half of the tile: a thread that issues a batch of MMAs is held until the
    // batch has drained, so a single issuer would leave the tensor pipe idle during its own bookkeeping
    // (barrier wait, descriptors, commit) between two K blocks.
    if (lane == 0) {
      const int half = warp - kWarpMma;
      constexpr uint32_t idesc = make_idesc_f16(kBM, kBN, kBf16, 0, 0);
      const uint64_t desc0 = make_smem_desc_sw128(smem_u32(smem), 16, 1024);
      const uint32_t desc_hi = static_cast<uint32_t>(desc0 >> 32), desc_lo0 = static_cast<uint32_t>(desc0);
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(half * 256);
      int stage = 0;
      uint32_t phase = 0, tile_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        for (int j = 0; j < nkb; ++j) {
          if (!mbar_wait(&tail->full[stage], phase, abort_flag)) { ok = false; break; }
          if (j == 0) {  // the previous tile's half must have been read out of TMEM
            if (!mbar_wait(&tail->acc_empty[half], tile_phase ^ 1u, abort_flag)) { ok = false; break; }
          }
          tc_fence_after_sync();
          const uint32_t lo = desc_lo0 + static_cast<uint32_t>((stage * kStageBytes) >> 4);
          const uint32_t x = lo + static_cast<uint32_t>((half * kHalfBytes) >> 4), b = lo + (2 * kHalfBytes >> 4);
          const uint32_t la[4] = {x, x + 2u, x + 4u, x + 6u};
          const uint32_t lb[4] = {b, b + 2u, b + 4u, b + 6u};
          umma_ss_x4(d_tmem, desc_hi, desc_hi, idesc, j != 0 ? 1u : 0u, la, lb);
          umma_commit(&tail->empty[stage]);
          if (j == nkb - 1) umma_commit(&tail->acc_full[half]);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        tile_phase ^= 1u;
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsEpilogue));
    // ------------------------------------------------------------- epilogue: warpgroup `half` drains its accumulator
    const int half = warp >> 2;
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + static_cast<uint32_t>(half * 256);
    const uint16_t* bias16 = reinterpret_cast<const uint16_t*>(a.init);
    uint32_t tile_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
      const int w_row = (t % col_tiles) * kBN;
      if (!mbar_wait_warp(&tail->acc_full[half], tile_phase, abort_flag)) { ok = false; break; }
      tile_phase ^= 1u;
      tc_fence_after_sync();
      // The accumulator is read out and rounded to 16 bits completely (128 registers per thread) before anything
      // is stored: the next tile's MMAs may start as soon as the last TMEM load has returned, and the stores
      // run beside them.
      uint32_t pk[kBN / 64][32];
#pragma unroll
      for (int q = 0; q < kBN / 64; ++q) {
        uint32_t v0[32], v1[32];
        tmem_ld_x32(taddr + static_cast<uint32_t>(q * 64), v0);
        tmem_ld_x32(taddr + static_cast<uint32_t>(q * 64 + 32), v1);
        tmem_wait_ld();
        if (q == kBN / 64 - 1) {  // accumulator fully read: the next tile may overwrite it
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tail->acc_empty[half]);
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float lo = __uint_as_float(i < 16 ? v0[2 * i] : v1[2 * i - 32]);
          float hi = __uint_as_float(i < 16 ? v0[2 * i + 1] : v1[2 * i - 31]);
          if (a.init_mode == kInitBias1D) {
            const uint32_t bb = *reinterpret_cast<const uint32_t*>(bias16 + w_row + q * 64 + 2 * i);
            if (kBf16) {
              lo += __uint_as_float(bb << 16);
              hi += __uint_as_float(bb & 0xFFFF0000u);
            } else {
              const __half2 h2 = *reinterpret_cast<const __half2*>(&bb);
              lo += __low2float(h2);
              hi += __high2float(h2);
            }
          }
          pk[q][i] = kBf16 ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
        }
      }
      if ((t / col_tiles) * 2 * kBM + half * kBM >= total_rows) continue;  // empty half of the last row pair
      // Stores: through a 2 KB staging area per warp (16 rows x 128 bytes in the 128-byte swizzle pattern) handed
      // to a TMA store of one 16 x 64 box, instead of 32 scattered 16-byte pieces per store instruction
      // (scattered stores of one tile took as long as a quarter of its MMAs and held up the operand loads of
      // the next tile).
      uint8_t* stg = smem_stage + warp * kStageWarpBytes;
      const int row0 = (t / col_tiles) * 2 * kBM + half * kBM + (warp & 3) * 32;  // first row of this warp
#pragma unroll
      for (int s = 0; s < kBN / 64; ++s) {
#pragma unroll
        for (int ph = 0; ph < 2; ++ph) {
          // the staging area is free once the store issued from it has read it
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
          if ((lane >> 4) == ph) {
            const int r = lane & 15;
#pragma unroll
            for (int c = 0; c < 8; ++c)
              *reinterpret_cast<uint4*>(stg + r * 128 + ((c ^ (r & 7)) << 4)) =
                  make_uint4(pk[s][4 * c], pk[s][4 * c + 1], pk[s][4 * c + 2], pk[s][4 * c + 3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&a.tmap_y, stg, w_row + s * 64, row0 + ph * 16);
            tma_store_commit();
          }
        }
      }
    }
  }

  if (warp < kEpiWarps && lane == 0) tma_store_wait_all<0>();
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
  if (warp == kWarpMma) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace


// Tile width for a dense launch: 256 or 192 columns (0: leave the launch to the 128x256 tiles of gemm.cu). All
// kernels deal equal tiles in fixed shares, so a launch lasts as long as its fullest SM: rounds of tiles times the
// tile's length, in units of a 128x256 tile of this kernel (a 256x256 tile is 2, a 256x192 tile 1.5; the 128x256
// tiles of gemm.cu run at about 0.93 of this kernel's rate). The other kernel gets the launch only when it is
// clearly ahead; between the two widths of this kernel the wider wins ties.
int tall_tile_cols(const GemmArgs& a, int sm_count) {
  const bool fits = a.mode == kGemmQ && a.tiles == nullptr && (a.init_mode == kInitNone || a.init_mode == kInitBias1D) &&
                    (static_cast<int64_t>(a.batch) * a.m) % kBM == 0 && static_cast<int64_t>(a.batch) * a.m >= 2 * kBM &&
                    a.k % kBK == 0 && a.k > 0 && a.n > 0;
  if (!fits) return 0;
  const bool ok256 = a.n % 256 == 0, ok192 = a.n % 192 == 0;
  if (!ok256 && !ok192) return 0;
  if (sm_count <= 0) return ok256 ? 256 : 192;
  const int64_t rows = static_cast<int64_t>(a.batch) * a.m;
  const int64_t row_pairs = (rows + 2 * kBM - 1) / (2 * kBM);
  auto rounds = [&](int64_t t) { return static_cast<double>((t + sm_count - 1) / sm_count); };
  const double c256 = ok256 ? rounds(row_pairs * (a.n / 256)) * 2.0 : 1e30;
  const double c192 = ok192 ? rounds(row_pairs * (a.n / 192)) * 1.5 : 1e30;
  const int cols = c192 < c256 ? 192 : 256;
  const double c_tall = c192 < c256 ? c192 : c256;
  // the other kernel: 128-row tiles of two column blocks (a last single block of an odd count rated as a pair)
  const double c_wide = rounds((rows / kBM) * ((a.n + 255) / 256)) / 0.93;
  if (c_wide * 1.05 < c_tall) return 0;
  return cols;
}

bool gemm_tall_applies(const GemmArgs& a, int sm_count) { return tall_tile_cols(a, sm_count) != 0; }

namespace {
template <bool kBf16, int kBN>
cudaError_t launch_tall(const GemmArgs& a, int grid, cudaStream_t stream) {
  const cudaError_t e = cudaFuncSetAttribute(gemm_tall_kernel<kBf16, kBN>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return e;
  gemm_tall_kernel<kBf16, kBN><<<grid, kThreads, kSmemBytes, stream>>>(a);
  return cudaGetLastError();
}
}  // namespace

cudaError_t launch_gemm_tall(const GemmArgs& a, int max_ctas, cudaStream_t stream) {
  const int cols = tall_tile_cols(a, max_ctas);
  if (cols == 0) return cudaErrorInvalidValue;
  const int64_t tiles = ((static_cast<int64_t>(a.batch) * a.m + 2 * kBM - 1) / (2 * kBM)) * (a.n / cols);
  if (tiles <= 0) return cudaSuccess;
  const int grid = tiles < max_ctas ? static_cast<int>(tiles) : max_ctas;
  if (cols == 256) return a.is_bf16 ? launch_tall<true, 256>(a, grid, stream) : launch_tall<false, 256>(a, grid, stream);
  return a.is_bf16 ? launch_tall<true, 192>(a, grid, stream) : launch_tall<false, 192>(a, grid, stream);
}

}  // namespace fo
