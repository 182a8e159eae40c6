// Mask path: bit packing (packbits / segment_packbits) and the compaction of the packed
// block masks into the work lists the attention and GEMM kernels consume.
//
// Bit layout (same as include/flashomni/attention/prefill.cuh:1284-1294,1385-1394 and
// include/flashomni/gemm/w16a16/gemm.cuh:50-58 of the reference): per request b the segment starts
// at byte `indptr[b]`; q-block bit index = qb*H + h; kv-block bit index = (qb*H + h)*nkv + kvb;
// bit i of a segment = (seg[i >> 3] >> (i & 7)) & 1.
//
// All kernels here are integer / byte work bound by HBM and launch latency; they never touch
// memory outside the extents given (reads are clamped to the packed buffers' byte sizes) and
// report malformed input through a status word instead of faulting.
#include "internal.h"

namespace fo {

// ---------------------------------------------------------------------------------------------
// packbits
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack8(const uint8_t* p, int64_t avail, bool little, bool aligned8) {
  // Packs up to 8 input bytes (non-zero -> 1). `avail` = number of valid inputs (1..8).
  uint32_t out = 0;
  if (aligned8 && avail >= 8) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const uint32_t w[2] = {v.x, v.y};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t byte = (w[i >> 2] >> ((i & 3) * 8)) & 0xFFu;
      const uint32_t bit = byte != 0u;
      out |= bit << (little ? i : 7 - i);
    }
  } else {
    const int n = avail < 8 ? static_cast<int>(avail) : 8;
    for (int i = 0; i < n; ++i) {
      const uint32_t bit = p[i] != 0;
      out |= bit << (little ? i : 7 - i);
    }
  }
  return out;
}

// Four output bytes from 32 input bytes held in two 16-byte words: per 32-bit word the "byte is non-zero" flags are
// gathered with one multiply (flag of byte i at bit 8 i; the product with 2^24 + 2^17 + 2^10 + 2^3 puts flag i at bit
// 24 + i, all partial products land on distinct bits).
__device__ __forceinline__ uint32_t nibble_of(uint32_t w) {
  const uint32_t t = ((((w & 0x7f7f7f7fu) + 0x7f7f7f7fu) | w) & 0x80808080u) >> 7;
  return (t * 0x01020408u) >> 24;
}
__device__ __forceinline__ uint32_t pack32(const uint4& a, const uint4& b, bool little) {
  uint32_t r = (nibble_of(a.x) | (nibble_of(a.y) << 4)) | ((nibble_of(a.z) | (nibble_of(a.w) << 4)) << 8) |
               ((nibble_of(b.x) | (nibble_of(b.y) << 4)) << 16) | ((nibble_of(b.z) | (nibble_of(b.w) << 4)) << 24);
  if (!little) r = __byte_perm(__brev(r), 0, 0x0123);  // reverse the bits inside every byte, keep the byte order
  return r;
}

// One thread per four output bytes (32 inputs, two 16-byte loads in flight) where alignment and length allow it,
// byte by byte otherwise.
__global__ void packbits_kernel(const uint8_t* __restrict__ x, int64_t n, int little, uint8_t* __restrict__ y) {
  const int64_t nbytes = (n + 7) >> 3;
  const int64_t nwords = (nbytes + 3) >> 2;
  const bool x16 = (reinterpret_cast<uintptr_t>(x) & 15u) == 0, y4 = (reinterpret_cast<uintptr_t>(y) & 3u) == 0;
  const bool x8 = (reinterpret_cast<uintptr_t>(x) & 7u) == 0;
  for (int64_t w = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; w < nwords;
       w += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t i0 = w * 4;
    if (x16 && y4 && (i0 + 4) * 8 <= n) {
      const uint4 a = *reinterpret_cast<const uint4*>(x + i0 * 8), b = *reinterpret_cast<const uint4*>(x + i0 * 8 + 16);
      *reinterpret_cast<uint32_t*>(y + i0) = pack32(a, b, little != 0);
    } else {
      for (int64_t i = i0; i < i0 + 4 && i < nbytes; ++i)
        y[i] = static_cast<uint8_t>(pack8(x + i * 8, n - i * 8, little != 0, x8));
    }
  }
}

// The same per segment; the segment of an output byte is found by binary search over the byte indptr.
__device__ __forceinline__ int seg_of(const int32_t* __restrict__ new_indptr, int num_segments, int64_t i) {
  int lo = 0, hi = num_segments;  // new_indptr[lo] <= i < new_indptr[lo + 1]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (static_cast<int64_t>(new_indptr[mid]) <= i) lo = mid; else hi = mid;
  }
  return lo;
}
__global__ void segment_packbits_kernel(const uint8_t* __restrict__ x, const int32_t* __restrict__ indptr,
                                        const int32_t* __restrict__ new_indptr, int num_segments,
                                        int64_t out_bytes, int little, uint8_t* __restrict__ y) {
  const int64_t nwords = (out_bytes + 3) >> 2;
  const bool y4 = (reinterpret_cast<uintptr_t>(y) & 3u) == 0;
  for (int64_t w = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; w < nwords;
       w += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t i0 = w * 4;
    const int lo = seg_of(new_indptr, num_segments, i0);
    const int64_t seg_in0 = indptr[lo], seg_in1 = indptr[lo + 1];
    const int64_t src0 = seg_in0 + (i0 - new_indptr[lo]) * 8;
    // fast path: the four bytes lie in one segment, all 32 inputs exist, loads and the store are aligned
    if (y4 && i0 + 4 <= out_bytes && i0 + 4 <= static_cast<int64_t>(new_indptr[lo + 1]) && src0 + 32 <= seg_in1 &&
        (reinterpret_cast<uintptr_t>(x + src0) & 15u) == 0) {
      const uint4 a = *reinterpret_cast<const uint4*>(x + src0), b = *reinterpret_cast<const uint4*>(x + src0 + 16);
      *reinterpret_cast<uint32_t*>(y + i0) = pack32(a, b, little != 0);
      continue;
    }
    for (int64_t i = i0; i < i0 + 4 && i < out_bytes; ++i) {
      const int sg = seg_of(new_indptr, num_segments, i);
      const int64_t src = static_cast<int64_t>(indptr[sg]) + (i - new_indptr[sg]) * 8;
      const int64_t avail = static_cast<int64_t>(indptr[sg + 1]) - src;
      if (avail <= 0) { y[i] = 0; continue; }
      const bool aligned = (reinterpret_cast<uintptr_t>(x + src) & 7u) == 0;
      y[i] = static_cast<uint8_t>(pack8(x + src, avail, little != 0, aligned));
    }
  }
}

cudaError_t launch_packbits(const uint8_t* x, int64_t n, int little, uint8_t* y, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  const int64_t nwords = (((n + 7) >> 3) + 3) >> 2;
  const int threads = 256;
  int64_t blocks = (nwords + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  packbits_kernel<<<static_cast<int>(blocks), threads, 0, stream>>>(x, n, little, y);
  return cudaGetLastError();
}

cudaError_t launch_segment_packbits(const uint8_t* x, const int32_t* indptr, const int32_t* new_indptr,
                                    int num_segments, int64_t out_bytes, int little, uint8_t* y,
                                    cudaStream_t stream) {
  if (out_bytes <= 0 || num_segments <= 0) return cudaSuccess;
  const int64_t nwords = (out_bytes + 3) >> 2;
  const int threads = 256;
  int64_t blocks = (nwords + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  segment_packbits_kernel<<<static_cast<int>(blocks), threads, 0, stream>>>(x, indptr, new_indptr, num_segments,
                                                                            out_bytes, little, y);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Bit-stream helpers
// ---------------------------------------------------------------------------------------------
// 32 bits of the little-endian bit stream `seg` starting at bit `pos`; bytes at or beyond `limit`
// (the number of readable bytes from `seg`) read as zero.
__device__ __forceinline__ uint32_t load_bits32(const uint8_t* seg, int64_t pos, int64_t limit) {
  const int64_t byte0 = pos >> 3;
  const int sh = static_cast<int>(pos & 7);
  uint64_t acc = 0;
#pragma unroll
  for (int i = 0; i < 5; ++i) {
    const int64_t bi = byte0 + i;
    const uint64_t v = (bi < limit) ? seg[bi] : 0u;
    acc |= v << (8 * i);
  }
  return static_cast<uint32_t>(acc >> sh);
}
__device__ __forceinline__ int get_bit(const uint8_t* seg, int64_t pos, int64_t limit) {
  const int64_t bi = pos >> 3;
  if (bi >= limit) return 0;
  return (seg[bi] >> (pos & 7)) & 1;
}

// up to 64 bits of the stream starting at bit `pos` (9 independent byte loads, clamped like load_bits32)
__device__ __forceinline__ uint64_t load_bits64(const uint8_t* seg, int64_t pos, int64_t limit, int nbits) {
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

// ---------------------------------------------------------------------------------------------
// Attention mask compaction
// ---------------------------------------------------------------------------------------------
// Candidate c enumerates (b, qb, hl) in ascending (b, qb, hl) order, hl in [0, head_count).
struct Cand {
  int b, qb, h;       // h = head_begin + hl (index used for mask bits)
  int nq, nkv;
  bool valid;
};

constexpr int kMaxBatchSmem = 1024;
constexpr int64_t kCompactL2Bytes = 48ll << 20;   // K + V bytes of the heads of one group (a share of the 126 MB L2)
constexpr int64_t kCompactFineBuckets = 8192;  // groups * (max_nkv + 1) up to which items are ordered by length inside a group

// Fills smem prefix of candidates per request. Thread 0 computes (B is small), all read after sync.
__device__ __forceinline__ void build_cand_prefix(const CompactArgs& a, int64_t* s_prefix) {
  if (threadIdx.x == 0) {
    int64_t acc = 0;
    s_prefix[0] = 0;
    for (int b = 0; b < a.batch; ++b) {
      const int64_t ql = static_cast<int64_t>(a.qo_indptr[b + 1]) - a.qo_indptr[b];
      const int64_t nq = ql > 0 ? (ql + a.sbq - 1) / a.sbq : 0;
      acc += nq * a.head_count;
      s_prefix[b + 1] = acc;
    }
  }
  __syncthreads();
}

__device__ __forceinline__ Cand decode_cand(const CompactArgs& a, const int64_t* s_prefix, int64_t c) {
  Cand r;
  int lo = 0, hi = a.batch;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (s_prefix[mid] <= c) lo = mid; else hi = mid;
  }
  r.b = lo;
  const int64_t local = c - s_prefix[lo];
  r.qb = static_cast<int>(local / a.head_count);
  r.h = a.head_begin + static_cast<int>(local % a.head_count);
  const int64_t ql = static_cast<int64_t>(a.qo_indptr[lo + 1]) - a.qo_indptr[lo];
  const int64_t kl = static_cast<int64_t>(a.kv_indptr[lo + 1]) - a.kv_indptr[lo];
  r.nq = static_cast<int>((ql + a.sbq - 1) / a.sbq);
  r.nkv = kl > 0 ? static_cast<int>((kl + a.sbkv - 1) / a.sbkv) : 0;
  r.valid = c < s_prefix[a.batch];
  return r;
}

// Pass 1: one warp per candidate. cnt[c] = number of kept kv-blocks if the q-block is active, else -1.
__global__ void compact_count_kernel(CompactArgs a) {
  __shared__ int64_t s_prefix[kMaxBatchSmem + 1];
  build_cand_prefix(a, s_prefix);
  const int lane = threadIdx.x & 31;
  const int64_t warps_per_grid = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t c = blockIdx.x * static_cast<int64_t>(blockDim.x >> 5) + (threadIdx.x >> 5); c < a.n_cand;
       c += warps_per_grid) {
    const Cand cd = decode_cand(a, s_prefix, c);
    int result;
    if (a.is_full) {
      result = cd.nkv;
    } else {
      const int64_t ioff = a.info_indptr[cd.b];
      const int64_t koff = a.kv_info_indptr[cd.b];
      const int64_t qbit = static_cast<int64_t>(cd.qb) * a.num_heads + cd.h;
      const int active = get_bit(a.sparse_info + ioff, qbit, a.info_bytes - ioff);
      if (!active) {
        result = -1;
      } else {
        const int64_t row0 = qbit * cd.nkv;
        int cnt = 0;
        for (int w = lane * 32; w < cd.nkv; w += 32 * 32) {
          uint32_t bits = load_bits32(a.sparse_kv_info + koff, row0 + w, a.kv_info_bytes - koff);
          const int rem = cd.nkv - w;
          if (rem < 32) bits &= (1u << rem) - 1u;
          cnt += __popc(bits);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
        result = cnt;
      }
    }
    if (lane == 0) a.cnt[c] = result;
  }
}

// Pass 2: single CTA. Exclusive scans of the active flags (item index) and of the kept counts
// (offset into kv_idx), then the processing order: items grouped by (request, head), q-blocks ascending
// inside a group, by a stable counting sort: W warps own contiguous candidate slices, each with its own
// histogram in shared memory; bucket starts are (items of smaller keys) + (same bucket, earlier
// slices); every warp then places its slice in ascending candidate order, 32 at a time.
__global__ void __launch_bounds__(1024) compact_scan_kernel(CompactArgs a, int sort_warps, int by_length, int heads_per_group) {
  extern __shared__ __align__(16) int s_whist[];  // [sort_warps + 1][batch * head_count]; first the scan's staging
  __shared__ int s_warp_items[32];
  __shared__ long long s_warp_kept[32];
  __shared__ int s_carry_items;
  __shared__ long long s_carry_kept;
  __shared__ int64_t s_prefix[kMaxBatchSmem + 1];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) { s_carry_items = 0; s_carry_kept = 0; }
  __syncthreads();
  // kScanPer consecutive candidates per thread and pass: a thread scans its own run, the CTA scans the run totals
  constexpr int kScanPer = 8;
  constexpr int kPassCand = 1024 * kScanPer, kPassPad = kPassCand + kPassCand / 32;
  // staging of a pass, over the dynamic shared memory that the sort below uses afterwards
  long long* s_off = reinterpret_cast<long long*>(s_whist);           // [kPassPad] kept-list offsets
  int* s_val = reinterpret_cast<int*>(s_off + kPassPad);              // [kPassPad] candidate counts
  int* s_pos = s_val + kPassPad;                                      // [kPassPad] item positions
  for (int64_t base = 0; base < a.n_cand; base += static_cast<int64_t>(blockDim.x) * kScanPer) {
    const int64_t c0 = base + static_cast<int64_t>(tid) * kScanPer;
    // The counts of a pass come in with coalesced loads and the results leave with coalesced stores; between them
    // they sit in shared memory, where a thread finds its eight consecutive entries (index i at i + i / 32: the
    // accesses of a warp then fall on 32 different banks).
    const int64_t pass_n = (a.n_cand - base) < kPassCand ? (a.n_cand - base) : kPassCand;
    for (int i = tid; i < pass_n; i += blockDim.x) s_val[i + (i >> 5)] = a.cnt[base + i];
    __syncthreads();
    int vals[kScanPer];
#pragma unroll
    for (int k = 0; k < kScanPer; ++k) {
      const int i = tid * kScanPer + k;
      vals[k] = (c0 + k < a.n_cand) ? s_val[i + (i >> 5)] : -1;
    }
    int run_i = 0;
    long long run_k = 0;
#pragma unroll
    for (int k = 0; k < kScanPer; ++k) {
      run_i += vals[k] >= 0;
      run_k += vals[k] >= 0 ? vals[k] : 0;
    }
    int xi = run_i;
    long long xk = run_k;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int yi = __shfl_up_sync(0xffffffffu, xi, o);
      const long long yk = __shfl_up_sync(0xffffffffu, xk, o);
      if (lane >= o) { xi += yi; xk += yk; }
    }
    if (lane == 31) { s_warp_items[warp] = xi; s_warp_kept[warp] = xk; }
    __syncthreads();
    if (warp == 0) {
      int wi = s_warp_items[lane];
      long long wk = s_warp_kept[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int yi = __shfl_up_sync(0xffffffffu, wi, o);
        const long long yk = __shfl_up_sync(0xffffffffu, wk, o);
        if (lane >= o) { wi += yi; wk += yk; }
      }
      s_warp_items[lane] = wi;  // inclusive over warps
      s_warp_kept[lane] = wk;
    }
    __syncthreads();
    int pre_i = s_carry_items + (warp ? s_warp_items[warp - 1] : 0) + xi - run_i;
    long long pre_k = s_carry_kept + (warp ? s_warp_kept[warp - 1] : 0) + xk - run_k;
#pragma unroll
    for (int k = 0; k < kScanPer; ++k) {
      if (c0 + k < a.n_cand) {
        const bool flag = vals[k] >= 0;
        const int i = tid * kScanPer + k;
        s_pos[i + (i >> 5)] = flag ? pre_i : -1;
        s_off[i + (i >> 5)] = pre_k;
        pre_i += flag;
        pre_k += flag ? vals[k] : 0;
      }
    }
    __syncthreads();
    for (int i = tid; i < pass_n; i += blockDim.x) {
      a.item_pos[base + i] = s_pos[i + (i >> 5)];
      a.kv_off[base + i] = s_off[i + (i >> 5)];
    }
    if (tid == 0) {
      s_carry_items += s_warp_items[31];
      s_carry_kept += s_warp_kept[31];
    }
    __syncthreads();
  }
  const int n_items = s_carry_items;
  const long long total_kept = s_carry_kept;
  if (tid == 0) {
    a.counters[0] = n_items;
    a.counters[1] = static_cast<int>(total_kept > 0x7fffffffLL ? 0x7fffffff : total_kept);
    a.counters[2] = (total_kept > a.max_kept || n_items > a.max_items) ? kDevBadIndex : kDevOk;
    a.counters[3] = a.max_nkv;
    a.kv_ptr[n_items <= a.max_items ? n_items : 0] = static_cast<int>(total_kept);
  }
  // ---- processing order: stable counting sort by (request, group of heads), so that the CTAs that run at the
  // same time work on the same few heads and share their K / V tiles in L2. A group is `heads_per_group`
  // consecutive heads: as many as keep their K and V in L2 together (launch_attn_compact).
  // With `by_length` the items of a group are ordered by descending list length (ties: canonical order):
  // the items drawn last are then the short ones of the group and the launch ends without a long straggler.
  const int per_group = by_length ? a.max_nkv + 1 : 1;
  const int grp_per_req = (a.head_count + heads_per_group - 1) / heads_per_group;
  const int nb = a.batch * grp_per_req * per_group;
  if (!by_length) {
    // Single heads with their q-blocks ascending: the candidates read in (request, head, q-block) order instead of
    // (request, q-block, head); the running count of active ones is the position. One more scan, no sort.
    build_cand_prefix(a, s_prefix);
    if (a.head_count <= 512) {
      // Threads laid out head-fastest: thread (chunk k, head h) walks the q-blocks of its chunk for its head, so the
      // threads of a chunk read consecutive positions (one row of heads at a time). Count, prefix per head over the
      // chunks and over the heads, then the same walk again writing the positions out.
      int* s_cnt = reinterpret_cast<int*>(s_whist);          // [chunks][H] counts, then exclusive starts
      const int H = a.head_count;
      const int chunks = static_cast<int>(blockDim.x) / H;
      int* s_tot = s_cnt + chunks * H;                       // [H] items of a head, then the head's start
      const int h = tid % H, ck = tid / H;
      int req_base = 0;
      for (int b = 0; b < a.batch; ++b) {
        const int64_t c_req = s_prefix[b];
        const int nq = static_cast<int>((s_prefix[b + 1] - s_prefix[b]) / H);
        const int qpc = (nq + chunks - 1) / chunks;
        const int q0 = ck * qpc, q1 = (q0 + qpc < nq) ? q0 + qpc : nq;
        int mine = 0;
        if (ck < chunks)
          for (int qb = q0; qb < q1; ++qb) mine += a.item_pos[c_req + static_cast<int64_t>(qb) * H + h] >= 0;
        if (ck < chunks) s_cnt[ck * H + h] = mine;
        __syncthreads();
        if (tid < H) {   // exclusive prefix over the chunks of head `tid`
          int run = 0;
          for (int k = 0; k < chunks; ++k) {
            const int t = s_cnt[k * H + tid];
            s_cnt[k * H + tid] = run;
            run += t;
          }
          s_tot[tid] = run;
        }
        __syncthreads();
        if (warp == 0) {  // exclusive prefix over the heads
          int carry = 0;
          for (int h0 = 0; h0 < H; h0 += 32) {
            const int v = (h0 + lane < H) ? s_tot[h0 + lane] : 0;
            int x = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
              const int y = __shfl_up_sync(0xffffffffu, x, o);
              if (lane >= o) x += y;
            }
            if (h0 + lane < H) s_tot[h0 + lane] = carry + x - v;
            carry += __shfl_sync(0xffffffffu, x, 31);
          }
          if (lane == 0) s_carry_items = carry;   // items of this request
        }
        __syncthreads();
        if (ck < chunks) {
          int pos = req_base + s_tot[h] + s_cnt[ck * H + h];
          for (int qb = q0; qb < q1; ++qb) {
            const int ip = a.item_pos[c_req + static_cast<int64_t>(qb) * H + h];
            if (ip >= 0) {
              if (pos < a.max_items) a.order[pos] = ip;
              ++pos;
            }
          }
        }
        req_base += s_carry_items;
        __syncthreads();
      }
      return;
    }
    if (tid == 0) s_carry_items = 0;
    __syncthreads();
    for (int64_t base = 0; base < a.n_cand; base += static_cast<int64_t>(blockDim.x) * kScanPer) {
      const int64_t j0 = base + static_cast<int64_t>(tid) * kScanPer;
      int ip[kScanPer];
#pragma unroll
      for (int k = 0; k < kScanPer; ++k) {
        const int64_t j = j0 + k;
        ip[k] = -1;
        if (j < a.n_cand) {
          int lo = 0, hi = a.batch;
          while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_prefix[mid] <= j) lo = mid; else hi = mid;
          }
          const int64_t local = j - s_prefix[lo];
          const int64_t nq = (s_prefix[lo + 1] - s_prefix[lo]) / a.head_count;
          const int64_t h = local / nq, qb = local % nq;
          ip[k] = a.item_pos[s_prefix[lo] + qb * a.head_count + h];
        }
      }
      int run = 0;
#pragma unroll
      for (int k = 0; k < kScanPer; ++k) run += ip[k] >= 0;
      int x = run;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
      }
      if (lane == 31) s_warp_items[warp] = x;
      __syncthreads();
      if (warp == 0) {
        int w = s_warp_items[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int y = __shfl_up_sync(0xffffffffu, w, o);
          if (lane >= o) w += y;
        }
        s_warp_items[lane] = w;
      }
      __syncthreads();
      int pos = s_carry_items + (warp ? s_warp_items[warp - 1] : 0) + x - run;
#pragma unroll
      for (int k = 0; k < kScanPer; ++k) {
        if (ip[k] >= 0) {
          if (pos < a.max_items) a.order[pos] = ip[k];
          ++pos;
        }
      }
      __syncthreads();
      if (tid == 0) s_carry_items += s_warp_items[31];
      __syncthreads();
    }
    return;
  }
  if (sort_warps <= 0) {  // too many (request, group, length) buckets for the shared-memory histograms: canonical order
    for (int i = tid; i < n_items && i < a.max_items; i += blockDim.x) a.order[i] = i;
    return;
  }
  int* s_total = s_whist + sort_warps * nb;  // [nb] bucket totals, then bucket starts
  for (int i = tid; i < (sort_warps + 1) * nb; i += blockDim.x) s_whist[i] = 0;
  build_cand_prefix(a, s_prefix);
  auto key_of = [&](int64_t c, int len) -> int {   // len = cnt[c], already fetched by the caller
    int lo = 0, hi = a.batch;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_prefix[mid] <= c) lo = mid; else hi = mid;
    }
    const int grp = lo * grp_per_req + static_cast<int>((c - s_prefix[lo]) % a.head_count) / heads_per_group;
    if (!by_length) return grp;
    len = len < 0 ? 0 : (len > a.max_nkv ? a.max_nkv : len);
    return grp * per_group + (a.max_nkv - len);
  };
  const int64_t slice = ((a.n_cand + sort_warps - 1) / sort_warps + 31) / 32 * 32;
  const int64_t my0 = static_cast<int64_t>(warp) * slice;
  const int64_t my1 = (my0 + slice < a.n_cand) ? my0 + slice : a.n_cand;
  constexpr int kAhead = 4;  // candidate counts fetched ahead: the loads of four steps are in flight together
  if (warp < sort_warps) {
    int* h = s_whist + warp * nb;
    for (int64_t c0 = my0 + lane; c0 < my1; c0 += 32 * kAhead) {
      int v[kAhead];
#pragma unroll
      for (int k = 0; k < kAhead; ++k) v[k] = (c0 + 32 * k < my1) ? a.cnt[c0 + 32 * k] : -1;
#pragma unroll
      for (int k = 0; k < kAhead; ++k)
        if (v[k] >= 0) atomicAdd(&h[key_of(c0 + 32 * k, v[k])], 1);
    }
  }
  __syncthreads();
  // per bucket: exclusive prefix over the slices; the bucket total goes to s_total
  for (int k = tid; k < nb; k += blockDim.x) {
    int run = 0;
    for (int w = 0; w < sort_warps; ++w) {
      const int t = s_whist[w * nb + k];
      s_whist[w * nb + k] = run;
      run += t;
    }
    s_total[k] = run;
  }
  __syncthreads();
  // bucket starts in ascending key order (exclusive scan by warp 0)
  if (warp == 0) {
    int carry = 0;
    for (int k0 = 0; k0 < nb; k0 += 32) {
      const int k = k0 + lane;
      const int v = (k < nb) ? s_total[k] : 0;
      int x = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
      }
      if (k < nb) s_total[k] = carry + x - v;
      carry += __shfl_sync(0xffffffffu, x, 31);
    }
  }
  __syncthreads();
  for (int i = tid; i < sort_warps * nb; i += blockDim.x) s_whist[i] += s_total[i % nb];
  __syncthreads();
  if (warp < sort_warps) {
    int* h = s_whist + warp * nb;
    for (int64_t base0 = my0; base0 < my1; base0 += 32 * kAhead) {
      int cv[kAhead], ip[kAhead];
#pragma unroll
      for (int k = 0; k < kAhead; ++k) {
        const int64_t c = base0 + 32 * k + lane;
        cv[k] = (c < my1) ? a.cnt[c] : -1;
        ip[k] = (c < my1) ? a.item_pos[c] : -1;
      }
#pragma unroll
      for (int k = 0; k < kAhead; ++k) {
      const int64_t base = base0 + 32 * k;
      if (base >= my1) break;
      const int64_t c = base + lane;
      const bool flag = (c < my1) && cv[k] >= 0;
      const int v = flag ? key_of(c, cv[k]) : -1 - lane;
      const unsigned grp = __match_any_sync(0xffffffffu, v);
      const int rank_in_grp = __popc(grp & ((1u << lane) - 1u));
      const int leader = __ffs(grp) - 1;
      int start = 0;
      if (flag && lane == leader) {
        start = h[v];
        h[v] = start + __popc(grp);
      }
      start = __shfl_sync(0xffffffffu, start, leader);
      if (flag) {
        const int pos = start + rank_in_grp;
        if (pos < a.max_items) a.order[pos] = ip[k];
      }
      __syncwarp();
      }
    }
  }
}

// Pass 3: one warp per candidate; writes the item record and expands its kept kv-blocks (ascending).
__global__ void compact_fill_kernel(CompactArgs a) {
  __shared__ int64_t s_prefix[kMaxBatchSmem + 1];
  build_cand_prefix(a, s_prefix);
  const int lane = threadIdx.x & 31;
  const int64_t warps_per_grid = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t c = blockIdx.x * static_cast<int64_t>(blockDim.x >> 5) + (threadIdx.x >> 5); c < a.n_cand;
       c += warps_per_grid) {
    const int pos = a.item_pos[c];
    if (pos < 0 || pos >= a.max_items) continue;
    const Cand cd = decode_cand(a, s_prefix, c);
    const long long off = a.kv_off[c];
    const int kept = a.cnt[c];
    if (off + kept > a.max_kept) continue;  // flagged by the scan pass
    if (lane == 0) {
      a.items[4 * pos + 0] = cd.b;
      a.items[4 * pos + 1] = cd.h;
      a.items[4 * pos + 2] = cd.qb;
      a.items[4 * pos + 3] = kept;
      a.kv_ptr[pos] = static_cast<int>(off);
    }
    int written = 0;
    if (a.is_full) {
      for (int j = lane; j < cd.nkv; j += 32) a.kv_idx[off + j] = j;
    } else {
      const int64_t koff = a.kv_info_indptr[cd.b];
      const int64_t row0 = (static_cast<int64_t>(cd.qb) * a.num_heads + cd.h) * cd.nkv;
      for (int w0 = 0; w0 < cd.nkv; w0 += 32 * 32) {
        const int w = w0 + lane * 32;
        uint32_t bits = 0;
        if (w < cd.nkv) {
          bits = load_bits32(a.sparse_kv_info + koff, row0 + w, a.kv_info_bytes - koff);
          const int rem = cd.nkv - w;
          if (rem < 32) bits &= (1u << rem) - 1u;
        }
        const int pc = __popc(bits);
        int x = pc;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int y = __shfl_up_sync(0xffffffffu, x, o);
          if (lane >= o) x += y;
        }
        int dst = written + x - pc;
        while (bits) {
          const int bpos = __ffs(bits) - 1;
          bits &= bits - 1;
          a.kv_idx[off + dst++] = w + bpos;
        }
        written += __shfl_sync(0xffffffffu, x, 31);
      }
    }
  }
}

cudaError_t launch_attn_compact(const CompactArgs& a, cudaStream_t stream) {
  if (a.batch > kMaxBatchSmem) return cudaErrorInvalidValue;
  if (a.n_cand <= 0) {
    return cudaMemsetAsync(a.counters, 0, 4 * sizeof(int), stream);
  }
  const int threads = 256, wpb = threads / 32;
  int64_t blocks = (a.n_cand + wpb - 1) / wpb;
  if (blocks > 148 * 8) blocks = 148 * 8;
  // Groups of heads: as many consecutive heads as keep their K and V tiles in L2 together (kCompactL2Bytes for
  // 128-row x 128-column 16-bit blocks, max_nkv of them per head and tensor), evenly sized. Inside a group the
  // items are ordered by descending list length while the histograms (groups x lengths) stay below
  // kCompactFineBuckets; otherwise the groups are single heads with their q-blocks ascending.
  // Sort histograms: as many warps as fit in ~160 KB of shared memory, plus one row of bucket totals; with more
  // groups than fit, the kernel leaves the items in canonical order.
  int64_t hpg = kCompactL2Bytes / (static_cast<int64_t>(a.max_nkv > 0 ? a.max_nkv : 1) * 65536);
  hpg = hpg < 1 ? 1 : (hpg > a.head_count ? a.head_count : hpg);
  const int64_t grp_per_req = (a.head_count + hpg - 1) / hpg;
  hpg = (a.head_count + grp_per_req - 1) / grp_per_req;
  int by_length = static_cast<int64_t>(a.batch) * grp_per_req * (a.max_nkv + 1) <= kCompactFineBuckets ? 1 : 0;
  if (!by_length) hpg = 1;
  const int64_t groups = static_cast<int64_t>(a.batch) * ((a.head_count + hpg - 1) / hpg);
  const int64_t nb = by_length ? groups * (a.max_nkv + 1) : groups;
  int64_t sort_warps = nb > 0 ? (160 * 1024) / (nb * 4) - 1 : 0;
  if (sort_warps > 32) sort_warps = 32;
  if (sort_warps < 1) sort_warps = 0;
  size_t scan_smem = static_cast<size_t>((sort_warps + 1) * nb * 4) * (sort_warps > 0 ? 1 : 0);
  const size_t stage_smem = static_cast<size_t>(8192 + 8192 / 32) * 16;   // the scan's staging: 8 + 4 + 4 bytes per candidate
  if (scan_smem < stage_smem) scan_smem = stage_smem;
  {
    cudaError_t ea = cudaFuncSetAttribute(compact_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 164 * 1024);
    if (ea != cudaSuccess) return ea;
  }
  compact_count_kernel<<<static_cast<int>(blocks), threads, 0, stream>>>(a);
  compact_scan_kernel<<<1, 1024, scan_smem, stream>>>(a, static_cast<int>(sort_warps), by_length, static_cast<int>(hpg));
  compact_fill_kernel<<<static_cast<int>(blocks), threads, 0, stream>>>(a);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Attention work units (self-contained records; split of long kv lists)
// ---------------------------------------------------------------------------------------------
// Walks the items in processing order and writes one 32-byte record per unit of work, holding everything the
// attention kernel's roles need (no chain of dependent loads at a unit boundary):
//   [0] n          kv blocks of the unit (0: an active q-block that keeps nothing)
//   [1] kv_off     offset of the unit's first entry in kv_idx
//   [2] h | b << 16   mask head (< 65536), request (< 32768)
//   [3] q_row0     first row of the q-block in the q / o tensors
//   [4] q_valid | ragged << 16   rows (tokens) of the q-block that exist (1..sbq); columns of the request's partial
//                  last kv block if the unit's list ends with it, else 0
//   [5] kv_row0    first kv row of the request
//   [6] causal     qb * sbq + kv_len - q_len: the last kv position that the q-block's first token may attend to
//                  under a causal mask (token t of the block: causal + t)
//   [7] slot << 16 | part << 8 | n_parts   (a whole item: n_parts = 1, slot = 0xffff)
// A kv list is cut into n_parts = ceil(n_kept / chunk_max) parts of (almost) equal length only when there is room for
// partial results (max_slots > 0) and the launch has more than min_items and at most num_streams items: chunk_max = max(min_chunk,
// ceil(total_kept / num_streams), ceil(max_nkv / 255)); otherwise every item is one unit.
// unit_counters: n_units, partial slots in use, chunk_max, status. arrive[slot] = 0 for every slot.
constexpr int kUnitSortMax = 2048;

__global__ void __launch_bounds__(1024) attn_units_kernel(UnitArgs a) {
  __shared__ int s_warp_u[32], s_warp_p[32];
  __shared__ int s_carry_u, s_carry_p;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool list_ok = a.counters[2] == kDevOk;
  int n_items = a.counters[0];
  if (!list_ok || n_items < 0) n_items = 0;
  if (n_items > a.max_items) n_items = static_cast<int>(a.max_items);
  const long long total_kept = a.counters[1];
  int chunk_max = 0x7fffffff;
  if (n_items > a.min_items && a.max_slots > 0 && n_items <= a.num_streams) {
    long long c = (total_kept + a.num_streams - 1) / a.num_streams;
    if (c < a.min_chunk) c = a.min_chunk;
    const long long c255 = (static_cast<long long>(a.max_nkv) + 254) / 255;
    if (c < c255) c = c255;
    chunk_max = static_cast<int>(c);
  }
  for (int64_t i = tid; i < a.max_slots; i += blockDim.x) a.arrive[i] = 0;
  if (tid == 0) { s_carry_u = 0; s_carry_p = 0; }
  __syncthreads();
  for (int base = 0; base < n_items; base += blockDim.x) {
    const int pos = base + tid;
    int it = 0, n = 0, np = 0;
    int4 rec = make_int4(0, 0, 0, 0);
    if (pos < n_items) {
      it = a.order[pos];
      rec = *reinterpret_cast<const int4*>(a.items + 4 * it);  // (b, mask head, qb, n_kept)
      n = rec.w > 0 ? rec.w : 0;
      np = n > chunk_max ? (n + chunk_max - 1) / chunk_max : 1;
    }
    const int sp = np > 1 ? np : 0;
    int xu = np, xp = sp;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int yu = __shfl_up_sync(0xffffffffu, xu, o);
      const int yp = __shfl_up_sync(0xffffffffu, xp, o);
      if (lane >= o) { xu += yu; xp += yp; }
    }
    if (lane == 31) { s_warp_u[warp] = xu; s_warp_p[warp] = xp; }
    __syncthreads();
    if (warp == 0) {
      int wu = s_warp_u[lane], wp = s_warp_p[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int yu = __shfl_up_sync(0xffffffffu, wu, o);
        const int yp = __shfl_up_sync(0xffffffffu, wp, o);
        if (lane >= o) { wu += yu; wp += yp; }
      }
      s_warp_u[lane] = wu;
      s_warp_p[lane] = wp;
    }
    __syncthreads();
    const int off_u = s_carry_u + (warp ? s_warp_u[warp - 1] : 0) + xu - np;
    const int off_p = s_carry_p + (warp ? s_warp_p[warp - 1] : 0) + xp - sp;
    if (pos < n_items) {
      const int q0 = a.qo_indptr[rec.x], q_len = a.qo_indptr[rec.x + 1] - q0;
      const int k0 = a.kv_indptr[rec.x], kv_len = a.kv_indptr[rec.x + 1] - k0;
      const int kvp = a.kv_ptr[it];
      int q_valid = q_len - rec.z * a.sbq;
      q_valid = q_valid > a.sbq ? a.sbq : (q_valid < 0 ? 0 : q_valid);
      int ragged = 0;
      const int tail_cols = kv_len % a.sbkv;
      // lists are ascending: only the item's last entry can be the request's partial block
      if (tail_cols != 0 && n > 0 && a.kv_idx[kvp + n - 1] == kv_len / a.sbkv) ragged = tail_cols;
      for (int p = 0; p < np; ++p) {
        const int j0 = static_cast<int>(static_cast<long long>(n) * p / np);
        const int j1 = static_cast<int>(static_cast<long long>(n) * (p + 1) / np);
        if (off_u + p < a.max_units) {
          int4* dst = reinterpret_cast<int4*>(a.units + 8 * static_cast<int64_t>(off_u + p));
          const int sp_word = np > 1 ? (((off_p + p) & 0xffff) << 16) | (p << 8) | np : (0xffff << 16) | 1;
          dst[0] = make_int4(j1 - j0, kvp + j0, rec.y | (rec.x << 16), q0 + rec.z * a.sbq);
          dst[1] = make_int4(q_valid | ((p == np - 1 ? ragged : 0) << 16), k0, rec.z * a.sbq + kv_len - q_len, sp_word);
        }
      }
    }
    __syncthreads();
    if (tid == 0) { s_carry_u += s_warp_u[31]; s_carry_p += s_warp_p[31]; }
    __syncthreads();
  }
  // When lists were cut, the units are put in descending order of their length (stable: equal lengths keep the
  // order above), so that the CTAs, which draw units in list order, take the short ones last. Every thread holds
  // its records in registers before any is written back.
  const int n_units = s_carry_u;
  if (chunk_max != 0x7fffffff && n_units <= kUnitSortMax && n_units <= a.max_units) {
    __shared__ int s_len[kUnitSortMax];
    int4 r0[kUnitSortMax / 1024], r1[kUnitSortMax / 1024];
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kUnitSortMax / 1024; ++k) {
      const int u = tid + k * 1024;
      if (u < n_units) {
        const int4* src = reinterpret_cast<const int4*>(a.units + 8 * static_cast<int64_t>(u));
        r0[k] = src[0];
        r1[k] = src[1];
        s_len[u] = r0[k].x;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kUnitSortMax / 1024; ++k) {
      const int u = tid + k * 1024;
      if (u < n_units) {
        const int len = r0[k].x;
        int pos = 0;
        for (int v = 0; v < n_units; ++v) {
          const int lv = s_len[v];
          pos += (lv > len || (lv == len && v < u)) ? 1 : 0;
        }
        int4* dst = reinterpret_cast<int4*>(a.units + 8 * static_cast<int64_t>(pos));
        dst[0] = r0[k];
        dst[1] = r1[k];
      }
    }
  }
  if (tid == 0) {
    a.unit_counters[0] = s_carry_u;
    a.unit_counters[1] = s_carry_p;
    a.unit_counters[2] = chunk_max;
    a.unit_counters[3] = (!list_ok || s_carry_u > a.max_units || s_carry_p > a.max_slots || s_carry_p > 0xffff) ? kDevBadIndex : kDevOk;
  }
}

// The same records when no list can be cut (no room for partial results): every item is exactly one unit at its
// position in the processing order, so the items are independent of one another: one thread per item, any number
// of CTAs.
__global__ void __launch_bounds__(256) attn_units_whole_kernel(UnitArgs a) {
  const bool list_ok = a.counters[2] == kDevOk;
  int n_items = a.counters[0];
  if (!list_ok || n_items < 0) n_items = 0;
  if (n_items > a.max_items) n_items = static_cast<int>(a.max_items);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    a.unit_counters[0] = n_items;
    a.unit_counters[1] = 0;
    a.unit_counters[2] = 0x7fffffff;
    a.unit_counters[3] = (!list_ok || n_items > a.max_units) ? kDevBadIndex : kDevOk;
  }
  for (int64_t pos = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; pos < n_items && pos < a.max_units;
       pos += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int it = a.order[pos];
    const int4 rec = *reinterpret_cast<const int4*>(a.items + 4 * it);  // (b, mask head, qb, n_kept)
    const int n = rec.w > 0 ? rec.w : 0;
    const int q0 = a.qo_indptr[rec.x], q_len = a.qo_indptr[rec.x + 1] - q0;
    const int k0 = a.kv_indptr[rec.x], kv_len = a.kv_indptr[rec.x + 1] - k0;
    const int kvp = a.kv_ptr[it];
    int q_valid = q_len - rec.z * a.sbq;
    q_valid = q_valid > a.sbq ? a.sbq : (q_valid < 0 ? 0 : q_valid);
    int ragged = 0;
    const int tail_cols = kv_len % a.sbkv;
    if (tail_cols != 0 && n > 0 && a.kv_idx[kvp + n - 1] == kv_len / a.sbkv) ragged = tail_cols;
    int4* dst = reinterpret_cast<int4*>(a.units + 8 * pos);
    dst[0] = make_int4(n, kvp, rec.y | (rec.x << 16), q0 + rec.z * a.sbq);
    dst[1] = make_int4(q_valid | (ragged << 16), k0, rec.z * a.sbq + kv_len - q_len, (0xffff << 16) | 1);
  }
}

cudaError_t launch_attn_units(const UnitArgs& a, cudaStream_t stream) {
  if (a.max_slots <= 0) {
    int64_t blocks = (a.max_items + 255) / 256;
    if (blocks > 148 * 4) blocks = 148 * 4;
    if (blocks < 1) blocks = 1;
    attn_units_whole_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(a);
    return cudaGetLastError();
  }
  attn_units_kernel<<<1, 1024, 0, stream>>>(a);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// GEMM work lists (single CTA: the candidate counts are a few thousand at most)
// ---------------------------------------------------------------------------------------------
// GEMM-Q: tile records (b, iy, ix0, ix1). Per row block (b, iy) the active column blocks are taken two
// at a time in ascending order; a leftover single block has ix1 = -1. All two-block records come first,
// the single-block records after them, each part in ascending (b, iy) order: the GEMM hands tiles to its
// CTAs in list order, and the half-size tiles at the end fill the last wave. The last `k` two-block records
// are cut into two single-block records each, k chosen so that the launch ends earliest when `n_ctas` CTAs draw
// the records in list order (gemm_q_split_rule: a two-block tile costs 20 time units, a single-block tile 13).
// counters[0] = number of records, counters[1] = number of active 128x128 tiles, counters[3] = number
// of two-block records. The kernel walks the row blocks twice: totals first, then the records.
constexpr int kPairCost = 20, kSingleCost = 13;

// Time at which the last CTA ends when `n` CTAs draw `pairs` two-block tiles and then `singles` single-block tiles
// in list order, every tile going to the CTA that is free first.
__device__ __forceinline__ int gemm_q_makespan(int pairs, int singles, int n) {
  const int full = pairs / n, r = pairs % n;
  int t_a = full * kPairCost, c_a = n - r;        // CTAs free after the full rounds
  int t_b = (full + 1) * kPairCost, c_b = r;      // CTAs that run one more two-block tile
  int end = (full + (r ? 1 : 0)) * kPairCost;
  int m = singles;
  while (m > 0) {
    if (c_a > 0 && (c_b == 0 || t_a <= t_b)) {
      m -= c_a;
      t_a += kSingleCost;
      end = end > t_a ? end : t_a;
    } else {
      m -= c_b;
      t_b += kSingleCost;
      end = end > t_b ? end : t_b;
    }
  }
  return end;
}

__global__ void __launch_bounds__(1024) gemm_q_tiles_kernel(GemmListArgs a) {
  __shared__ int s_warp[32];
  __shared__ int s_warp_t[32];
  __shared__ int s_carry, s_carry_t, s_pairs_total, s_best;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int mt = a.m / 128, nt = a.n / 128;
  const int rows = a.batch * mt;
  for (int pass = 0; pass < 2; ++pass) {
    if (tid == 0) { s_carry = 0; s_carry_t = 0; }
    __syncthreads();
    const int pairs_total = pass == 0 ? 0 : s_pairs_total;
    const int n_split = pass == 0 ? 0 : (s_best & 0xffff);   // two-block records cut into singles
    const int pairs_kept = pairs_total - n_split;
    for (int base = 0; base < rows; base += blockDim.x) {
      const int r = base + tid;
      int cnt = 0;
      const uint8_t* seg = nullptr;
      int64_t limit = 0, bit0 = 0;
      uint64_t rowbits = 0;
      bool fast = false;
      if (r < rows) {
        const int b = r / mt, iy = r % mt;
        if (a.is_full) {
          cnt = nt;
        } else {
          const int64_t ioff = a.info_indptr[b];
          seg = a.sparse_info + ioff;
          limit = a.info_bytes - ioff;
          const int64_t qb = (static_cast<int64_t>(a.num_text_tokens) + static_cast<int64_t>(iy) * 128) / a.sparse_q_size;
          bit0 = qb * a.num_heads + a.head_begin;
          if (a.head_dim == 128 && nt <= 64) {  // one bit per column block: fetch the row's bits at once
            rowbits = load_bits64(seg, bit0, limit, nt);
            cnt = __popcll(rowbits);
            fast = true;
          } else {
            for (int ix = 0; ix < nt; ++ix) cnt += get_bit(seg, bit0 + (ix * 128) / a.head_dim, limit);
          }
        }
      }
      // x: two-block records, xt: single-block records (inclusive scans over the CTA)
      const int npair = cnt >> 1, nsingle = cnt & 1;
      int x = npair, xt = nsingle;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, o);
        const int yt = __shfl_up_sync(0xffffffffu, xt, o);
        if (lane >= o) { x += y; xt += yt; }
      }
      if (lane == 31) { s_warp[warp] = x; s_warp_t[warp] = xt; }
      __syncthreads();
      if (warp == 0) {
        int w = s_warp[lane], wt = s_warp_t[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int y = __shfl_up_sync(0xffffffffu, w, o);
          const int yt = __shfl_up_sync(0xffffffffu, wt, o);
          if (lane >= o) { w += y; wt += yt; }
        }
        s_warp[lane] = w;
        s_warp_t[lane] = wt;
      }
      __syncthreads();
      if (pass == 1 && r < rows && cnt > 0) {
        int pos = s_carry + (warp ? s_warp[warp - 1] : 0) + x - npair;
        const int spos = pairs_total + n_split + s_carry_t + (warp ? s_warp_t[warp - 1] : 0) + xt - nsingle;
        const int b = r / mt, iy = r % mt;
        int first = -1;
        for (int ix = 0; ix < nt; ++ix) {
          const int on = a.is_full ? 1 : (fast ? static_cast<int>((rowbits >> ix) & 1ull)
                                                 : get_bit(seg, bit0 + (ix * 128) / a.head_dim, limit));
          if (!on) continue;
          if (first < 0) {
            first = ix;
          } else {
            if (pos < pairs_kept) {
              if (pos < a.max_tiles) *reinterpret_cast<int4*>(a.tiles + 4 * pos) = make_int4(b, iy, first, ix);
            } else {
              const int sp = pairs_kept + 2 * (pos - pairs_kept);
              if (sp + 1 < a.max_tiles) {
                *reinterpret_cast<int4*>(a.tiles + 4 * sp) = make_int4(b, iy, first, -1);
                *reinterpret_cast<int4*>(a.tiles + 4 * sp + 4) = make_int4(b, iy, ix, -1);
              }
            }
            ++pos;
            first = -1;
          }
        }
        if (first >= 0 && spos < a.max_tiles) *reinterpret_cast<int4*>(a.tiles + 4 * spos) = make_int4(b, iy, first, -1);
      }
      __syncthreads();
      if (tid == 0) { s_carry += s_warp[31]; s_carry_t += s_warp_t[31]; }
      __syncthreads();
    }
    if (pass == 0) {
      if (tid == 0) { s_pairs_total = s_carry; s_best = 0x7fffffff; }
      __syncthreads();
      // thread k rates the list with its last k two-block records cut; the smallest (end time, k) wins
      const int P = s_carry, S = s_carry_t, n = a.n_ctas > 0 ? a.n_ctas : 1;
      if (tid <= P && tid <= n && P + S + tid <= a.max_tiles) {
        const int t = gemm_q_makespan(P - tid, S + 2 * tid, n);
        atomicMin(&s_best, ((t < 32767 ? t : 32767) << 16) | tid);
      }
      __syncthreads();
      if (tid == 0 && s_best == 0x7fffffff) s_best = 0;  // a list that does not fit is reported below, uncut
      __syncthreads();
    }
  }
  if (tid == 0) {
    const int n_split = s_best & 0xffff;
    const int n_rec = s_carry + s_carry_t + n_split;
    a.counters[0] = n_rec;
    a.counters[1] = 2 * s_carry + s_carry_t;
    a.counters[2] = n_rec > a.max_tiles ? kDevBadIndex : kDevOk;
    a.counters[3] = s_carry - n_split;
    a.counters[4] = kDevOk;  // status word of the GEMM kernel that follows
    a.counters[5] = 0;       // its tile cursor
    a.counters[6] = 0;       // and the count of CTAs that have finished
  }
}

// GEMM-O: per 128-row block the ascending list of selected local heads, plus the row blocks sorted
// by descending list length (stable). counters[0] = number of row blocks, counters[1] = total heads.
__global__ void __launch_bounds__(1024) gemm_o_rows_kernel(GemmListArgs a) {
  __shared__ int s_warp[32];
  __shared__ int s_carry;
  extern __shared__ int s_hist[];  // local_heads + 2 buckets
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int mt = a.m / 128;
  const int rows = a.batch * mt;
  const int local_heads = a.k / a.head_dim;
  const int want = a.is_for_cache ? 0 : 1;
  if (tid == 0) s_carry = 0;
  for (int i = tid; i <= local_heads; i += blockDim.x) s_hist[i] = 0;
  __syncthreads();
  for (int base = 0; base < rows; base += blockDim.x) {
    const int r = base + tid;
    int cnt = 0;
    uint64_t rowbits = 0;
    if (r < rows) {
      const int b = r / mt, iy = r % mt;
      const int64_t ioff = a.info_indptr[b];
      const int64_t qb = (static_cast<int64_t>(a.num_text_tokens) + static_cast<int64_t>(iy) * 128) / a.sparse_q_size;
      const int64_t bit0 = qb * a.num_heads + a.head_begin;
      if (local_heads <= 64) {  // fetch the row's bits at once
        rowbits = load_bits64(a.sparse_info + ioff, bit0, a.info_bytes - ioff, local_heads);
        if (!want) rowbits = ~rowbits & (local_heads < 64 ? ((1ull << local_heads) - 1ull) : ~0ull);
        cnt = __popcll(rowbits);
      } else {
        for (int h = 0; h < local_heads; ++h)
          cnt += get_bit(a.sparse_info + ioff, bit0 + h, a.info_bytes - ioff) == want;
      }
    }
    int x = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) s_warp[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int w = s_warp[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += y;
      }
      s_warp[lane] = w;
    }
    __syncthreads();
    const int off = s_carry + (warp ? s_warp[warp - 1] : 0) + x - cnt;
    if (r < rows) {
      a.row_indptr[r] = off;
      atomicAdd(&s_hist[cnt], 1);
      const int b = r / mt, iy = r % mt;
      const int64_t ioff = a.info_indptr[b];
      const int64_t qb = (static_cast<int64_t>(a.num_text_tokens) + static_cast<int64_t>(iy) * 128) / a.sparse_q_size;
      const int64_t bit0 = qb * a.num_heads + a.head_begin;
      int w = off;
      if (local_heads <= 64) {
        uint64_t bits = rowbits;
        while (bits) {
          a.row_heads[w++] = __ffsll(static_cast<long long>(bits)) - 1;
          bits &= bits - 1;
        }
      } else {
        for (int h = 0; h < local_heads; ++h)
          if (get_bit(a.sparse_info + ioff, bit0 + h, a.info_bytes - ioff) == want) a.row_heads[w++] = h;
      }
    }
    __syncthreads();
    if (tid == 0) s_carry += s_warp[31];
    __syncthreads();
  }
  if (tid == 0) {
    a.row_indptr[rows] = s_carry;
    a.counters[0] = rows;
    a.counters[1] = s_carry;
    a.counters[2] = kDevOk;
    a.counters[4] = kDevOk;  // status word of the GEMM kernel that follows
    a.counters[5] = 0;       // its tile cursor
    a.counters[6] = 0;       // and the count of CTAs that have finished
    // bucket starts, descending count
    int acc = 0;
    for (int k = local_heads; k >= 0; --k) { const int v = s_hist[k]; s_hist[k] = acc; acc += v; }
  }
  __syncthreads();
  if (warp == 0) {
    for (int base = 0; base < rows; base += 32) {
      const int r = base + lane;
      const bool ok = r < rows;
      const int cnt = ok ? (a.row_indptr[r + 1] - a.row_indptr[r]) : -1 - lane;
      const unsigned grp = __match_any_sync(0xffffffffu, cnt);
      const int rank = __popc(grp & ((1u << lane) - 1u));
      const int leader = __ffs(grp) - 1;
      int start = 0;
      if (ok && lane == leader) { start = s_hist[cnt]; s_hist[cnt] = start + __popc(grp); }
      start = __shfl_sync(0xffffffffu, start, leader);
      if (ok) a.row_order[start + rank] = r;
      __syncwarp();
    }
  }
}

cudaError_t launch_gemm_q_tiles(const GemmListArgs& a, cudaStream_t stream) {
  gemm_q_tiles_kernel<<<1, 1024, 0, stream>>>(a);
  return cudaGetLastError();
}
cudaError_t launch_gemm_o_rows(const GemmListArgs& a, cudaStream_t stream) {
  const int local_heads = a.k / a.head_dim;
  gemm_o_rows_kernel<<<1, 1024, (local_heads + 2) * sizeof(int), stream>>>(a);
  return cudaGetLastError();
}

}  // namespace fo
