// Block-sparse prefill attention on tcgen05 / TMEM / TMA, driven by compacted work lists.
//
// What it computes (reference: include/flashomni/attention/prefill.cuh:1203-1531): for every work
// item (b, h, qb) -- an active 128-row q-block of one head -- and its ascending list of kept
// 128-row kv-blocks,  O[rows, h, :] = softmax_over_kept(Q K^T * sm_scale) V,  fp32 accumulation,
// base-2 online softmax, output rounded to the input dtype. q-blocks that are not in the list are
// never written. An item with an empty list writes zeros (lse = -5e4), like the reference.
//
// CTA = 192 threads, two CTAs per SM: warps 0-3 softmax / correction / epilogue (one thread per
// q row, TMEM lane = row), warp 4 TMA producer, warp 5 MMA issuer. TMEM per CTA: S (128 fp32
// columns, P in bf16 aliases its first 64 columns) + O (128 fp32 columns). Shared memory per
// CTA: Q tile 32 KB + a two-slot ring of 32 KB tiles that K and V blocks alternate through.
// While one CTA of the SM is in its softmax, the other one's MMAs keep the tensor pipe busy.
// CTAs are persistent; items are dealt round-robin in longest-first order.
#include <cuda_fp16.h>

#include "internal.h"

namespace fo {
namespace {

constexpr int kBQ = 128, kBKV = 128, kD = 128;
constexpr int kTileBytes = 128 * kD * 2;   // 32 KB: a 128-row tile of Q, K or V
constexpr int kHalfBytes = kTileBytes / 2; // one 64-column half (one swizzle-atom column)
constexpr int kRing = 2;
constexpr int kThreads = 192;
constexpr int kTmemCols = 256;
constexpr uint32_t kColS = 0, kColO = 128;
constexpr float kRescaleThreshold = 8.0f;  // lazy rescale: keep the old max while exp2 stays <= 2^8

struct Tail {
  uint64_t q_full, q_empty;
  uint64_t ring_full[kRing], ring_empty[kRing];
  uint64_t s_full, p_full, o_full;
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int kSmemBytes = (1 + kRing) * kTileBytes + 1024 + static_cast<int>(sizeof(Tail));

struct Item {
  int b, h, qb, n;
  const int32_t* kv;
};

__device__ __forceinline__ Item load_item(const AttnArgs& a, int i) {
  const int it = a.order[i];
  Item r;
  r.b = a.items[4 * it + 0];
  r.h = a.items[4 * it + 1];
  r.qb = a.items[4 * it + 2];
  r.n = a.items[4 * it + 3];
  r.kv = a.kv_idx + a.kv_ptr[it];
  return r;
}

template <bool kBf16>
__global__ void __launch_bounds__(kThreads, 2) attention_kernel(const __grid_constant__ AttnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* smem_q = smem;
  uint8_t* smem_ring = smem + kTileBytes;
  Tail* tail = reinterpret_cast<Tail*>(smem + (1 + kRing) * kTileBytes);
  volatile int* abort_flag = &tail->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(&tail->q_full, 1);
    mbar_init(&tail->q_empty, 1);
    for (int s = 0; s < kRing; ++s) {
      mbar_init(&tail->ring_full[s], 1);
      mbar_init(&tail->ring_empty[s], 1);
    }
    mbar_init(&tail->s_full, 1);
    mbar_init(&tail->p_full, 4);
    mbar_init(&tail->o_full, 1);
    tail->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&a.tmap_q);
    tma_prefetch_desc(&a.tmap_k);
    tma_prefetch_desc(&a.tmap_v);
  }
  if (warp == 5) {
    tmem_alloc(&tail->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tail->tmem_base;

  int n_items = a.counters[0];
  if (n_items < 0) n_items = 0;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int slot = 0;
      uint32_t ring_phase = 0, q_phase = 0;
      bool ok = true;
      for (int i = blockIdx.x; i < n_items && ok; i += gridDim.x) {
        const Item it = load_item(a, i);
        if (it.n <= 0) continue;
        const int hq = it.h - a.head_begin;
        const int hk = hq / a.group_size;
        const int q_row = a.qo_indptr[it.b] + it.qb * kBQ;
        const int kv_row0 = a.kv_indptr[it.b];
        if (!mbar_wait(&tail->q_empty, q_phase ^ 1u, abort_flag)) { ok = false; break; }
        q_phase ^= 1u;
        mbar_expect_tx(&tail->q_full, kTileBytes);
        tma_load_3d(smem_q, &a.tmap_q, &tail->q_full, 0, hq, q_row);
        tma_load_3d(smem_q + kHalfBytes, &a.tmap_q, &tail->q_full, 64, hq, q_row);
        for (int j = 0; j < it.n && ok; ++j) {
          const int row = kv_row0 + it.kv[j] * kBKV;
#pragma unroll
          for (int which = 0; which < 2; ++which) {  // 0: K block, 1: V block
            if (!mbar_wait(&tail->ring_empty[slot], ring_phase ^ 1u, abort_flag)) { ok = false; break; }
            uint8_t* dst = smem_ring + slot * kTileBytes;
            const CUtensorMap* tm = which == 0 ? &a.tmap_k : &a.tmap_v;
            mbar_expect_tx(&tail->ring_full[slot], kTileBytes);
            tma_load_3d(dst, tm, &tail->ring_full[slot], 0, hk, row);
            tma_load_3d(dst + kHalfBytes, tm, &tail->ring_full[slot], 64, hk, row);
            if (++slot == kRing) { slot = 0; ring_phase ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(kBQ, kBKV, kBf16, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_f16(kBQ, kD, kBf16, 0, 1);
      const uint32_t tmem_s = tmem_base + kColS;
      const uint32_t tmem_o = tmem_base + kColO;
      const uint32_t q_addr = smem_u32(smem_q);
      int slot = 0;
      uint32_t ring_phase = 0, q_phase = 0, p_phase = 0;
      bool ok = true;
      for (int i = blockIdx.x; i < n_items && ok; i += gridDim.x) {
        const Item it = load_item(a, i);
        if (it.n <= 0) continue;
        if (!mbar_wait(&tail->q_full, q_phase, abort_flag)) { ok = false; break; }
        q_phase ^= 1u;
        for (int j = 0; j < it.n; ++j) {
          // ---- S = Q K_j^T
          if (!mbar_wait(&tail->ring_full[slot], ring_phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          {
            const uint32_t k_addr = smem_u32(smem_ring + slot * kTileBytes);
#pragma unroll
            for (int kk = 0; kk < kD / 16; ++kk) {
              const uint32_t off = static_cast<uint32_t>((kk >> 2) * kHalfBytes + (kk & 3) * 32);
              umma_ss(tmem_s, make_smem_desc_sw128(q_addr + off, 16, 1024),
                      make_smem_desc_sw128(k_addr + off, 16, 1024), idesc_qk, kk != 0 ? 1u : 0u);
            }
            umma_commit(&tail->ring_empty[slot]);
            umma_commit(&tail->s_full);
            if (j == it.n - 1) umma_commit(&tail->q_empty);
            if (++slot == kRing) { slot = 0; ring_phase ^= 1u; }
          }
          // ---- O (+)= P_j V_j
          if (!mbar_wait(&tail->p_full, p_phase, abort_flag)) { ok = false; break; }
          p_phase ^= 1u;
          if (!mbar_wait(&tail->ring_full[slot], ring_phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          {
            const uint32_t v_addr = smem_u32(smem_ring + slot * kTileBytes);
#pragma unroll
            for (int kk = 0; kk < kBKV / 16; ++kk) {
              // V is MN-major: 16 kv rows further = 16 * 128 B; the two 64-column halves are 16 KB apart
              umma_ts(tmem_o, tmem_s + static_cast<uint32_t>(kk * 8),
                      make_smem_desc_sw128(v_addr + static_cast<uint32_t>(kk * 2048), kHalfBytes, 1024),
                      idesc_pv, (j | kk) != 0 ? 1u : 0u);
            }
            umma_commit(&tail->ring_empty[slot]);
            if (j == it.n - 1) umma_commit(&tail->o_full);
            if (++slot == kRing) { slot = 0; ring_phase ^= 1u; }
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue warps
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t tmem_s = tmem_base + lane_base + kColS;
    const uint32_t tmem_o = tmem_base + lane_base + kColO;
    const int r_in_tile = warp * 32 + lane;
    uint32_t s_phase = 0, o_phase = 0;
    bool ok = true;
    uint16_t* o16 = reinterpret_cast<uint16_t*>(a.o);
    for (int i = blockIdx.x; i < n_items && ok; i += gridDim.x) {
      const Item it = load_item(a, i);
      const int hq = it.h - a.head_begin;
      const int q0 = a.qo_indptr[it.b];
      const int q_len = a.qo_indptr[it.b + 1] - q0;
      const int kv_len = a.kv_indptr[it.b + 1] - a.kv_indptr[it.b];
      const int row_in_req = it.qb * kBQ + r_in_tile;
      const bool row_ok = row_in_req < q_len;
      const int64_t grow = static_cast<int64_t>(q0) + row_in_req;
      uint16_t* orow = o16 + grow * a.o_stride_n + static_cast<int64_t>(hq) * a.o_stride_h;

      if (it.n <= 0) {
        if (row_ok) {
          const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
          for (int c = 0; c < kD / 8; ++c) reinterpret_cast<uint4*>(orow)[c] = z;
          if (a.lse != nullptr) a.lse[grow * a.lse_stride_n + hq] = -5e4f;
        }
        continue;
      }

      float m_used = -INFINITY;  // running max (scaled, log2 domain) that the exponentials refer to
      float l = 0.f;
      for (int j = 0; j < it.n; ++j) {
        if (!mbar_wait(&tail->s_full, s_phase, abort_flag)) { ok = false; break; }
        s_phase ^= 1u;
        tc_fence_after_sync();
        const int kvb = it.kv[j];
        const int valid = kv_len - kvb * kBKV;  // columns of this block inside the request (>= 128: all)
        // ---- pass 1: row max
        float mx = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < kBKV / 32; ++c) {
          uint32_t v[32];
          tmem_ld_x32(tmem_s + static_cast<uint32_t>(c * 32), v);
          tmem_wait_ld();
          if (valid >= kBKV) {
#pragma unroll
            for (int t = 0; t < 32; ++t) mx = fmaxf(mx, __uint_as_float(v[t]));
          } else {
#pragma unroll
            for (int t = 0; t < 32; ++t)
              if (c * 32 + t < valid) mx = fmaxf(mx, __uint_as_float(v[t]));
          }
        }
        const float m_new = fmaxf(m_used, mx * a.sm_scale_log2);
        // ---- lazy rescale of l and O (warp-uniform decision; TMEM round trip is warp-collective)
        const bool need = (m_new - m_used) > kRescaleThreshold;  // true on the first block (m_used = -inf)
        if (j == 0) {
          m_used = m_new;
        } else if (__any_sync(0xffffffffu, need)) {
          const float alpha = need ? ex2_approx(m_used - m_new) : 1.0f;
          if (need) m_used = m_new;
          l *= alpha;
#pragma unroll 1
          for (int c = 0; c < kD / 32; ++c) {
            uint32_t v[32];
            tmem_ld_x32(tmem_o + static_cast<uint32_t>(c * 32), v);
            tmem_wait_ld();
#pragma unroll
            for (int t = 0; t < 32; ++t) v[t] = __float_as_uint(__uint_as_float(v[t]) * alpha);
            tmem_st_x32(tmem_o + static_cast<uint32_t>(c * 32), v);
          }
        }
        // ---- pass 2: P = exp2(S*scale - m_used), row sum, write P (16-bit) over the S columns
        const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
#pragma unroll 1
        for (int c = 0; c < kBKV / 32; ++c) {
          uint32_t v[32];
          tmem_ld_x32(tmem_s + static_cast<uint32_t>(c * 32), v);
          tmem_wait_ld();
          uint32_t pk[16];
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            float p0 = ex2_approx(fmaf(__uint_as_float(v[2 * t]), a.sm_scale_log2, neg_m));
            float p1 = ex2_approx(fmaf(__uint_as_float(v[2 * t + 1]), a.sm_scale_log2, neg_m));
            if (valid < kBKV) {
              if (c * 32 + 2 * t >= valid) p0 = 0.f;
              if (c * 32 + 2 * t + 1 >= valid) p1 = 0.f;
            }
            l += p0 + p1;
            pk[t] = kBf16 ? pack_bf16x2(p0, p1) : pack_f16x2(p0, p1);
          }
          tmem_st_x16(tmem_s + static_cast<uint32_t>(c * 16), pk);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tail->p_full);
      }
      if (!ok) break;
      // ---- epilogue: O / l -> global
      if (!mbar_wait(&tail->o_full, o_phase, abort_flag)) { ok = false; break; }
      o_phase ^= 1u;
      tc_fence_after_sync();
      const float inv_l = l > 0.f ? __frcp_rn(l) : 0.f;
#pragma unroll 1
      for (int c = 0; c < kD / 32; ++c) {
        uint32_t v[32];
        tmem_ld_x32(tmem_o + static_cast<uint32_t>(c * 32), v);
        tmem_wait_ld();
        if (row_ok) {
          uint4 outv[4];
          uint32_t* o32 = reinterpret_cast<uint32_t*>(outv);
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            const float x0 = __uint_as_float(v[2 * t]) * inv_l, x1 = __uint_as_float(v[2 * t + 1]) * inv_l;
            o32[t] = kBf16 ? pack_bf16x2(x0, x1) : pack_f16x2(x0, x1);
          }
          uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
          for (int t = 0; t < 4; ++t) dst[t] = outv[t];
        }
      }
      if (row_ok && a.lse != nullptr) {
        a.lse[grow * a.lse_stride_n + hq] = (l > 0.f) ? (log2f(l) + m_used) : -5e4f;
      }
      tc_fence_before_sync();
    }
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
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

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
