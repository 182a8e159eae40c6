// GEMM-Q / GEMM-O on tcgen05: one persistent, warp-specialised kernel.
//
//   Y[b, rows(iy), cols(ix)] = init + sum_{k-blocks of the tile} X[b, rows, kblk] * W[cols, kblk]^T
//
// GEMM-Q (reference: include/flashomni/gemm/w16a16/gemm.cuh:27-228): the tile list holds only the
// active (b, iy, ix) output tiles; every tile runs the whole K range; init = bias[cols] or 0; tiles
// that are not listed are never touched.
// GEMM-O (reference: include/flashomni/gemm/w16a16/gemm_reduction.cuh:27-276): every output tile is
// produced; its K loop visits only the K-slices of the heads selected for its row block (compacted
// list, ascending); init = cache[b, rows, cols] or bias[cols] or 0.
//
// CTA = 192 threads: warps 0-3 epilogue (TMEM -> registers -> global), warp 4 TMA producer,
// warp 5 MMA issuer. 128x128 output tile, K step 64 (one 128-byte swizzle atom), 6-stage ring of
// (A 16 KB + B 16 KB), two 128-column TMEM accumulators so the epilogue of tile i overlaps the
// main loop of tile i+1. Tiles are dealt round-robin to the persistent CTAs.
#include <cuda_fp16.h>

#include "internal.h"

namespace fo {
namespace {

constexpr int kBM = 128, kBN = 128, kBK = 64;
constexpr int kStages = 6;
constexpr int kABytes = kBM * kBK * 2;
constexpr int kBBytes = kBN * kBK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kThreads = 192;
constexpr int kTmemCols = 256;

struct Tail {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + static_cast<int>(sizeof(Tail));

struct TileInfo {
  int a_row;            // first row of the A tile in [batch*m]
  int w_row;            // first row of the W tile (= first output column)
  int nkb;              // number of 64-wide K blocks
  const int32_t* heads; // GEMM-O: selected heads of the row block (null for GEMM-Q)
};

__device__ __forceinline__ int num_tiles(const GemmArgs& a) {
  const int cap = a.batch * (a.m / kBM) * (a.n / kBN);
  if (a.mode == kGemmQ && a.tiles != nullptr) {
    const int n = *a.n_tiles_ptr;
    return n < cap ? (n < 0 ? 0 : n) : cap;
  }
  return cap;
}

__device__ __forceinline__ TileInfo get_tile(const GemmArgs& a, int t) {
  TileInfo ti;
  if (a.mode == kGemmQ) {
    int b, iy, ix;
    if (a.tiles != nullptr) {
      b = a.tiles[3 * t + 0]; iy = a.tiles[3 * t + 1]; ix = a.tiles[3 * t + 2];
    } else {  // dense: t enumerates (b, iy, ix) in row-major order
      const int nct = a.n / kBN, mt = a.m / kBM;
      ix = t % nct;
      iy = (t / nct) % mt;
      b = t / (nct * mt);
    }
    ti.a_row = b * a.m + iy * kBM;
    ti.w_row = ix * kBN;
    ti.nkb = a.k / kBK;
    ti.heads = nullptr;
  } else {
    const int nct = a.n / kBN;
    const int r = a.row_order[t / nct];
    ti.a_row = r * kBM;
    ti.w_row = (t % nct) * kBN;
    const int h0 = a.row_indptr[r], h1 = a.row_indptr[r + 1];
    ti.heads = a.row_heads + h0;
    ti.nkb = (h1 - h0) * a.kb_per_head;
  }
  return ti;
}

__device__ __forceinline__ int kcol_of(const GemmArgs& a, const TileInfo& ti, int j) {
  if (ti.heads == nullptr) return j * kBK;
  const int hh = j / a.kb_per_head;
  return (ti.heads[hh] * a.kb_per_head + (j - hh * a.kb_per_head)) * kBK;
}

template <bool kBf16>
__global__ void __launch_bounds__(kThreads, 1) gemm_kernel(const __grid_constant__ GemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  Tail* tail = reinterpret_cast<Tail*>(smem + kStages * kStageBytes);
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
    tail->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&a.tmap_a);
    tma_prefetch_desc(&a.tmap_b);
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

  if (warp == 4) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        const TileInfo ti = get_tile(a, t);
        for (int j = 0; j < ti.nkb; ++j) {
          if (!mbar_wait(&tail->empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          const int kcol = kcol_of(a, ti, j);
          uint8_t* sa = smem + stage * kStageBytes;
          mbar_expect_tx(&tail->full[stage], kStageBytes);
          tma_load_2d(sa, &a.tmap_a, &tail->full[stage], kcol, ti.a_row);
          tma_load_2d(sa + kABytes, &a.tmap_b, &tail->full[stage], kcol, ti.w_row);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kBM, kBN, kBf16, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        const TileInfo ti = get_tile(a, t);
        if (!mbar_wait(&tail->acc_empty[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kBN);
        for (int j = 0; j < ti.nkb; ++j) {
          if (!mbar_wait(&tail->full[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * kStageBytes);
          const uint64_t adesc = make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sa + kABytes, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) {
            // advancing 16 elements (32 bytes) along K inside the swizzle atom: +2 in the address field
            umma_ss(d_tmem, adesc + static_cast<uint64_t>(kk * 2), bdesc + static_cast<uint64_t>(kk * 2), idesc,
                    (j | kk) != 0 ? 1u : 0u);
          }
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
    bool ok = true;
    const uint16_t* init16 = reinterpret_cast<const uint16_t*>(a.init);
    uint16_t* y16 = reinterpret_cast<uint16_t*>(a.y);
    for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
      const TileInfo ti = get_tile(a, t);
      if (!mbar_wait(&tail->acc_full[acc], acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const int64_t row = static_cast<int64_t>(ti.a_row) + warp * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + static_cast<uint32_t>(acc * kBN);
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t v[32];
        if (ti.nkb > 0) {
          tmem_ld_x32(taddr + static_cast<uint32_t>(c * 32), v);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        const int col0 = ti.w_row + c * 32;
        uint4 add[4];
        if (a.init_mode == kInitBias1D) {
          const uint4* p = reinterpret_cast<const uint4*>(init16 + col0);
#pragma unroll
          for (int i = 0; i < 4; ++i) add[i] = __ldg(p + i);
        } else if (a.init_mode == kInitFull) {
          const uint4* p = reinterpret_cast<const uint4*>(init16 + row * a.n + col0);
#pragma unroll
          for (int i = 0; i < 4; ++i) add[i] = __ldg(p + i);
        }
        uint4 outv[4];
        uint32_t* o32 = reinterpret_cast<uint32_t*>(outv);
        const uint32_t* a32 = reinterpret_cast<const uint32_t*>(add);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float lo = __uint_as_float(v[2 * i]), hi = __uint_as_float(v[2 * i + 1]);
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
        uint4* dst = reinterpret_cast<uint4*>(y16 + row * a.n + col0);
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i] = outv[i];
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tail->acc_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
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
}

}  // namespace

cudaError_t launch_gemm(const GemmArgs& a, int max_ctas, cudaStream_t stream) {
  const int cap = a.batch * (a.m / kBM) * (a.n / kBN);
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
