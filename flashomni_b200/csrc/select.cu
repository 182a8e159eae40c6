// Block selection: from pooled attention scores [B, H, n, n] to the packed masks of the hot path
// (sparse_info bits [b][qb][h], sparse_kv_info bits [b][qb][h][kvb], little-endian, one byte segment per
// request). The reference does this with torch ops and Triton fill kernels on an unpacked [B, H, nq, nkv]
// layout that callers then transpose and bit-pack (benchmark/test_attn_score.py:93-133,
// benchmark/utils.py:83-84); here one pass writes the packed form directly.
//
// Per row of scores: mass_j = floor(2^31 * exp(x_j - max)) with a fixed polynomial exponential whose
// multiplies and adds are rounded separately (the CPU statement of the same arithmetic is bit-identical),
// integer total, limit = floor(threshold * total) in fp64, and the blocks taken in ascending (mass, index)
// order while the cumulative mass stays <= limit are switched off. No sort: the largest key
// K = (mass << 16 | index) with mass(keys <= K) <= limit is found bit by bit (48 warp reductions).
#include "internal.h"

namespace fo {
namespace {

constexpr int kSelWarps = 4;           // rows per CTA
constexpr int kSelMaxBlocks = 2048;    // longest row (shared memory: 4 B per entry and warp)

__device__ __forceinline__ uint32_t det_exp2_mass(float x, float row_max) {
  const float d = __fsub_rn(x, row_max);
  float t = __fmul_rn(d, 1.4426950408889634f);
  if (t < -64.0f) return 0u;
  const float n = rintf(t);
  const float f = __fsub_rn(t, n);
  float p = 0.0013333558f;
  p = __fadd_rn(__fmul_rn(p, f), 0.0096181291f);
  p = __fadd_rn(__fmul_rn(p, f), 0.0555041087f);
  p = __fadd_rn(__fmul_rn(p, f), 0.2402265070f);
  p = __fadd_rn(__fmul_rn(p, f), 0.6931471806f);
  p = __fadd_rn(__fmul_rn(p, f), 1.0f);
  const float e = scalbnf(p, static_cast<int>(n));          // exact: p in [0.70, 1.42], n >= -64
  const float s = __fmul_rn(e, 2147483648.0f);               // exact (power of two)
  const uint32_t m = __float2uint_rz(s);
  return m > 0x80000000u ? 0x80000000u : m;
}

// keep flags of one row, 32 entries at a time: calls emit(k, word) with bit i of `word` = keep of entry
// 32 k + i (entries past `len` are 0). All 32 lanes must call; `mass` is this warp's shared-memory row.
template <class Emit>
__device__ __forceinline__ void select_row(const float* __restrict__ x, int len, float threshold, uint32_t* mass,
                                           Emit&& emit) {
  const int lane = threadIdx.x & 31;
  float mx = -INFINITY;
  for (int j = lane; j < len; j += 32) mx = fmaxf(mx, x[j]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  unsigned long long total = 0;
  for (int j = lane; j < len; j += 32) {
    const uint32_t m = det_exp2_mass(x[j], mx);
    mass[j] = m;
    total += m;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
  __syncwarp();
  unsigned long long K = 0;
  bool any_off = threshold >= 0.f;
  if (any_off) {
    const unsigned long long limit = __double2ull_rd(__dmul_rn(static_cast<double>(threshold), static_cast<double>(total)));
    for (int bit = 47; bit >= 0; --bit) {  // keys are below 2^48: mass <= 2^31, index < 2^16
      const unsigned long long cand = K | (1ull << bit);
      unsigned long long m_le = 0;
      for (int j = lane; j < len; j += 32) {
        const unsigned long long key = (static_cast<unsigned long long>(mass[j]) << 16) | static_cast<unsigned>(j);
        if (key <= cand) m_le += mass[j];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m_le += __shfl_xor_sync(0xffffffffu, m_le, o);
      if (m_le <= limit) K = cand;
    }
  }
  for (int k = 0; k * 32 < len; ++k) {
    const int j = k * 32 + lane;
    bool keep = false;
    if (j < len) {
      const unsigned long long key = (static_cast<unsigned long long>(mass[j]) << 16) | static_cast<unsigned>(j);
      keep = !(any_off && key <= K);
    }
    emit(k, __ballot_sync(0xffffffffu, keep));
  }
  __syncwarp();
}

// t2i[b][j] = sum over heads (outer) and text rows (inner) of score[b][h][q][t2t + j], sequential fp32.
// A CTA takes 32 columns j: its 256 threads fetch the (head, text row) values of those columns 8 pairs at a time
// into shared memory (every load of a pass in flight together), then one warp adds them up per column in the
// stated order, pass after pass.
constexpr int kT2iPairs = 64;   // (head, text row) pairs per pass
__global__ void __launch_bounds__(256) select_t2i_kernel(SelectArgs a) {
  __shared__ float s_v[kT2iPairs][33];
  const int n_img = a.n - a.t2t;
  const int b = blockIdx.y;
  const int j0 = blockIdx.x * 32;
  const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;   // 8 groups of 32 columns' worth of threads
  const int pairs = a.heads * a.t2t;
  float acc = 0.f;
  for (int p0 = 0; p0 < pairs; p0 += kT2iPairs) {
#pragma unroll
    for (int u = 0; u < kT2iPairs / 8; ++u) {
      const int p = p0 + u * 8 + grp;
      const int h = p / a.t2t, q = p - h * a.t2t;
      float v = 0.f;
      if (p < pairs && j0 + lane < n_img)
        v = a.score[((static_cast<int64_t>(b) * a.heads + h) * a.n + q) * a.n + a.t2t + j0 + lane];
      s_v[u * 8 + grp][lane] = v;
    }
    __syncthreads();
    if (grp == 0) {
      const int np = pairs - p0 < kT2iPairs ? pairs - p0 : kT2iPairs;
      for (int u = 0; u < np; ++u) acc = __fadd_rn(acc, s_v[u][lane]);
    }
    __syncthreads();
  }
  if (grp == 0 && j0 + lane < n_img) a.t2i[static_cast<int64_t>(b) * a.n + j0 + lane] = acc;
}

// One CTA per request: which image q-blocks stay on (bytes q_keep[b][qb], text blocks always 1). The same
// integer arithmetic as select_row, with the sums taken over the whole CTA (exact, so the order does not matter).
constexpr int kSelQThreads = 128;
// `round` alternates between two sets of partials, so one barrier per sum is enough: a set is rewritten two sums
// later, after a barrier that every reader of it has passed.
__device__ __forceinline__ unsigned long long cta_sum_u64(unsigned long long v, unsigned long long (*s_part)[kSelQThreads / 32],
                                                          int round) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  unsigned long long* part = s_part[round & 1];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  unsigned long long t = 0;
#pragma unroll
  for (int w = 0; w < kSelQThreads / 32; ++w) t += part[w];
  return t;
}
__global__ void __launch_bounds__(kSelQThreads) select_q_kernel(SelectArgs a) {
  __shared__ uint32_t s_mass[kSelMaxBlocks];
  __shared__ unsigned long long s_part[2][kSelQThreads / 32];
  __shared__ float s_max[kSelQThreads / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = blockIdx.x;
  uint8_t* keep = a.q_keep + static_cast<int64_t>(b) * a.n;
  for (int q = tid; q < a.t2t && q < a.n; q += kSelQThreads) keep[q] = 1;
  const int n_img = a.n - a.t2t;
  if (n_img <= 0) return;
  if (a.t2t == 0) {  // no text rows to score the image blocks with: everything stays on
    for (int q = tid; q < a.n; q += kSelQThreads) keep[q] = 1;
    return;
  }
  const float* x = a.t2i + static_cast<int64_t>(b) * a.n;
  const float threshold = a.q_thr[b];
  float mx = -INFINITY;
  for (int j = tid; j < n_img; j += kSelQThreads) mx = fmaxf(mx, x[j]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) s_max[warp] = mx;
  __syncthreads();
#pragma unroll
  for (int w = 0; w < kSelQThreads / 32; ++w) mx = fmaxf(mx, s_max[w]);
  unsigned long long mine = 0;
  for (int j = tid; j < n_img; j += kSelQThreads) {
    const uint32_t m = det_exp2_mass(x[j], mx);
    s_mass[j] = m;
    mine += m;
  }
  const unsigned long long total = cta_sum_u64(mine, s_part, 0);
  unsigned long long K = 0;
  const bool any_off = threshold >= 0.f;
  if (any_off) {
    const unsigned long long limit = __double2ull_rd(__dmul_rn(static_cast<double>(threshold), static_cast<double>(total)));
    for (int bit = 47; bit >= 0; --bit) {
      const unsigned long long cand = K | (1ull << bit);
      unsigned long long m_le = 0;
      for (int j = tid; j < n_img; j += kSelQThreads) {
        const unsigned long long key = (static_cast<unsigned long long>(s_mass[j]) << 16) | static_cast<unsigned>(j);
        if (key <= cand) m_le += s_mass[j];
      }
      m_le = cta_sum_u64(m_le, s_part, bit);   // 47 first: the other set than the total's
      if (m_le <= limit) K = cand;
    }
  }
  for (int j = tid; j < n_img; j += kSelQThreads) {
    const unsigned long long key = (static_cast<unsigned long long>(s_mass[j]) << 16) | static_cast<unsigned>(j);
    keep[a.t2t + j] = static_cast<uint8_t>((any_off && key <= K) ? 0 : 1);
  }
}

// sparse_info bytes (bit qb * H + h = q_keep[b][qb]) and the two byte indptrs.
__global__ void select_pack_q_kernel(SelectArgs a) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i <= a.batch) {
    a.info_indptr[i] = static_cast<int32_t>(i * a.info_seg_bytes);
    a.kv_info_indptr[i] = static_cast<int32_t>(i * a.kv_seg_bytes);
  }
  if (i >= static_cast<int64_t>(a.batch) * a.info_seg_bytes) return;
  const int b = static_cast<int>(i / a.info_seg_bytes);
  const int64_t byte = i - static_cast<int64_t>(b) * a.info_seg_bytes;
  const int64_t nbits = static_cast<int64_t>(a.n) * a.heads;
  uint32_t v = 0;
  for (int t = 0; t < 8; ++t) {
    const int64_t bit = byte * 8 + t;
    if (bit < nbits && a.q_keep[static_cast<int64_t>(b) * a.n + bit / a.heads]) v |= 1u << t;
  }
  a.sparse_info[i] = static_cast<uint8_t>(v);
}

// One warp per (b, h, qb): the kept kv-blocks of the row, OR-ed into the packed stream (zeroed before).
__global__ void __launch_bounds__(kSelWarps * 32) select_kv_kernel(SelectArgs a) {
  __shared__ uint32_t s_mass[kSelWarps][kSelMaxBlocks];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kSelWarps + warp;
  const int64_t rows = static_cast<int64_t>(a.batch) * a.heads * a.n;
  if (row >= rows) return;
  const int q = static_cast<int>(row % a.n);
  const int h = static_cast<int>((row / a.n) % a.heads);
  const int b = static_cast<int>(row / (static_cast<int64_t>(a.n) * a.heads));
  if (a.zero_inactive && a.q_keep[static_cast<int64_t>(b) * a.n + q] == 0) return;
  uint32_t* words = reinterpret_cast<uint32_t*>(a.sparse_kv_info);
  const int64_t bit0 = static_cast<int64_t>(b) * a.kv_seg_bytes * 8 + (static_cast<int64_t>(q) * a.heads + h) * a.n;
  auto emit = [&](int k, uint32_t word) {
    if (lane != 0 || word == 0u) return;
    const int64_t bit = bit0 + static_cast<int64_t>(k) * 32;
    const int sh = static_cast<int>(bit & 31);
    atomicOr(words + (bit >> 5), word << sh);
    if (sh != 0 && (word >> (32 - sh)) != 0u) atomicOr(words + (bit >> 5) + 1, word >> (32 - sh));
  };
  if (q < a.t2t) {  // text rows keep every kv-block
    for (int k = 0; k * 32 < a.n; ++k) {
      const int rem = a.n - k * 32;
      emit(k, rem >= 32 ? 0xffffffffu : ((1u << rem) - 1u));
    }
    return;
  }
  const float* x = a.score + ((static_cast<int64_t>(b) * a.heads + h) * a.n + q) * a.n;
  select_row(x, a.n, a.kv_thr[h], s_mass[warp], emit);
}

}  // namespace

cudaError_t launch_select_blocks(const SelectArgs& a, cudaStream_t stream) {
  if (a.n > kSelMaxBlocks) return cudaErrorInvalidValue;
  cudaError_t e = cudaMemsetAsync(a.sparse_kv_info, 0, static_cast<size_t>(a.kv_words) * 4, stream);
  if (e != cudaSuccess) return e;
  const int n_img = a.n - a.t2t;
  if (n_img > 0 && a.t2t > 0) {
    dim3 g((n_img + 31) / 32, a.batch);
    select_t2i_kernel<<<g, 256, 0, stream>>>(a);
  }
  select_q_kernel<<<a.batch, kSelQThreads, 0, stream>>>(a);
  const int64_t info_bytes = static_cast<int64_t>(a.batch) * a.info_seg_bytes;
  const int64_t threads = info_bytes > a.batch + 1 ? info_bytes : a.batch + 1;
  select_pack_q_kernel<<<static_cast<int>((threads + 255) / 256), 256, 0, stream>>>(a);
  const int64_t rows = static_cast<int64_t>(a.batch) * a.heads * a.n;
  select_kv_kernel<<<static_cast<int>((rows + kSelWarps - 1) / kSelWarps), kSelWarps * 32, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace fo
