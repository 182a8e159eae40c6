// C ABI of libflashomni_b200.so: argument validation, tensor-map encoding, launches.
// See include/flashomni_b200.h for the contract of every entry point.
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <string>

#include "../../include/flashomni_b200.h"
#include "internal.h"

namespace fo {
namespace {

thread_local std::string g_last_error;
std::atomic<long long> g_kernel_launches{0};  // kernels this library has launched (or recorded into a capture)
inline void count_launches(int n) { g_kernel_launches.fetch_add(n, std::memory_order_relaxed); }

int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}
int fail_cuda(const char* what, cudaError_t e) {
  g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
  return FO_ERR_CUDA;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// A tensor map is a pure function of (base, extents, strides, box, swizzle): encoded maps are kept in a small
// per-thread table and reused when a call passes the same tensors again (a step that runs the same buffers every
// time never re-encodes).
namespace {
struct TmapKey {
  const void* base;
  uint64_t dims[5];
  uint64_t strides[5];
  uint32_t box[5];
  int32_t rank;
  int32_t swizzle;
};
struct TmapSlot {
  TmapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int kTmapSlots = 64;
thread_local TmapSlot t_tmaps[kTmapSlots];
}  // namespace

int encode_tmap_16bit(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128) {
  if (rank < 1 || rank > 5) return -2;
  TmapKey key;
  memset(&key, 0, sizeof(key));
  key.base = base;
  key.rank = rank;
  key.swizzle = swizzle128 ? 1 : 0;
  uint64_t h = reinterpret_cast<uint64_t>(base) * 0x9E3779B97F4A7C15ull + static_cast<uint64_t>(rank * 2 + key.swizzle);
  for (int i = 0; i < rank; ++i) {
    key.dims[i] = dims[i];
    key.strides[i] = i > 0 ? strides_bytes[i] : 0;
    key.box[i] = box[i];
    h = (h ^ (dims[i] + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2))) * 0xff51afd7ed558ccdull;
    h ^= key.strides[i] * 0xc4ceb9fe1a85ec53ull + box[i];
  }
  TmapSlot& slot = t_tmaps[(h >> 32) % kTmapSlots];
  if (slot.used && memcmp(&slot.key, &key, sizeof(key)) == 0) {
    *out = slot.map;
    return 0;
  }
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bdim[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i];
  }
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base),
                        gdim, gstr, bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  slot.key = key;
  slot.map = *out;
  slot.used = true;
  return 0;
}

}  // namespace fo

using namespace fo;

extern "C" {

const char* fo_last_error(void) { return g_last_error.c_str(); }
int fo_abi_version(void) { return FO_ABI_VERSION; }
long long fo_launch_count(void) { return g_kernel_launches.load(std::memory_order_relaxed); }

// ------------------------------------------------------------------------------------------ packbits
int fo_packbits(const uint8_t* x, int64_t n, int little, uint8_t* y, void* stream) {
  if (n < 0) return fail(FO_ERR_INVALID_ARG, "fo_packbits: n < 0");
  if (n == 0) return FO_OK;
  if (x == nullptr || y == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_packbits: null pointer");
  const cudaError_t e = launch_packbits(x, n, little, y, static_cast<cudaStream_t>(stream));
  count_launches(1);
  return e == cudaSuccess ? FO_OK : fail_cuda("fo_packbits", e);
}

int fo_segment_packbits(const uint8_t* x, const int32_t* indptr, const int32_t* new_indptr, int32_t num_segments,
                        int64_t out_bytes, int little, uint8_t* y, void* stream) {
  if (num_segments < 0 || out_bytes < 0) return fail(FO_ERR_INVALID_ARG, "fo_segment_packbits: negative size");
  if (num_segments == 0 || out_bytes == 0) return FO_OK;
  if (x == nullptr || y == nullptr || indptr == nullptr || new_indptr == nullptr)
    return fail(FO_ERR_INVALID_ARG, "fo_segment_packbits: null pointer");
  const cudaError_t e = launch_segment_packbits(x, indptr, new_indptr, num_segments, out_bytes, little, y,
                                                static_cast<cudaStream_t>(stream));
  count_launches(1);
  return e == cudaSuccess ? FO_OK : fail_cuda("fo_segment_packbits", e);
}

// ------------------------------------------------------------------------------------------ compaction
size_t fo_mask_compact_scratch_bytes(int64_t n_cand, int32_t max_nkv) {
  if (n_cand < 0) n_cand = 0;
  if (max_nkv < 0) max_nkv = 0;
  // cnt int32[n] | item_pos int32[n] | kv_off int64[n] | hist int32[max_nkv+1], each 16-byte aligned
  const size_t n = static_cast<size_t>(n_cand);
  size_t b = 0;
  b += (n * 4 + 15) & ~static_cast<size_t>(15);
  b += (n * 4 + 15) & ~static_cast<size_t>(15);
  b += (n * 8 + 15) & ~static_cast<size_t>(15);
  b += ((static_cast<size_t>(max_nkv) + 1) * 4 + 15) & ~static_cast<size_t>(15);
  return b + 16;
}

int fo_mask_compact(const uint8_t* sparse_info, int64_t sparse_info_bytes, const uint8_t* sparse_kv_info,
                    int64_t sparse_kv_info_bytes, const int32_t* sparse_info_indptr,
                    const int32_t* sparse_kv_info_indptr, const int32_t* qo_indptr, const int32_t* kv_indptr,
                    int32_t batch, int32_t num_heads, int32_t head_begin, int32_t head_count, int32_t sbq,
                    int32_t sbkv, int32_t is_full, int64_t n_cand, int32_t max_nkv, int64_t max_items,
                    int64_t max_kept, int32_t* items, int32_t* kv_ptr, int32_t* kv_idx, int32_t* order,
                    int32_t* counters, void* scratch, size_t scratch_bytes, void* stream) {
  if (batch <= 0 || num_heads <= 0 || head_count <= 0 || head_begin < 0 || head_begin + head_count > num_heads)
    return fail(FO_ERR_INVALID_ARG, "fo_mask_compact: bad batch / head window");
  if (sbq <= 0 || sbkv <= 0) return fail(FO_ERR_INVALID_ARG, "fo_mask_compact: block sizes must be positive");
  if (qo_indptr == nullptr || kv_indptr == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_mask_compact: null indptr");
  if (!is_full && (sparse_info == nullptr || sparse_kv_info == nullptr || sparse_info_indptr == nullptr ||
                   sparse_kv_info_indptr == nullptr))
    return fail(FO_ERR_INVALID_ARG,
                "fo_mask_compact: sparse_info / sparse_kv_info / their indptrs are required unless is_full");
  if (items == nullptr || kv_ptr == nullptr || kv_idx == nullptr || order == nullptr || counters == nullptr)
    return fail(FO_ERR_INVALID_ARG, "fo_mask_compact: null output");
  if (n_cand < 0 || max_nkv < 0 || max_items < n_cand || max_kept < 0)
    return fail(FO_ERR_INVALID_ARG, "fo_mask_compact: capacities must cover n_cand");
  if (batch > 1024) return fail(FO_ERR_UNSUPPORTED, "fo_mask_compact: batch > 1024");
  if (num_heads > 65535) return fail(FO_ERR_UNSUPPORTED, "fo_mask_compact: more than 65535 heads");
  if (scratch == nullptr || scratch_bytes < fo_mask_compact_scratch_bytes(n_cand, max_nkv) || !aligned16(scratch))
    return fail(FO_ERR_WORKSPACE, "fo_mask_compact: scratch too small or misaligned");
  CompactArgs a;
  memset(&a, 0, sizeof(a));
  a.sparse_info = sparse_info;
  a.sparse_kv_info = sparse_kv_info;
  a.info_indptr = sparse_info_indptr;
  a.kv_info_indptr = sparse_kv_info_indptr;
  a.qo_indptr = qo_indptr;
  a.kv_indptr = kv_indptr;
  a.info_bytes = sparse_info_bytes;
  a.kv_info_bytes = sparse_kv_info_bytes;
  a.batch = batch;
  a.num_heads = num_heads;
  a.head_begin = head_begin;
  a.head_count = head_count;
  a.sbq = sbq;
  a.sbkv = sbkv;
  a.is_full = is_full;
  a.max_nkv = max_nkv;
  a.n_cand = n_cand;
  a.max_items = max_items;
  a.max_kept = max_kept;
  a.items = items;
  a.kv_ptr = kv_ptr;
  a.kv_idx = kv_idx;
  a.order = order;
  a.counters = counters;
  uint8_t* p = static_cast<uint8_t*>(scratch);
  const size_t n = static_cast<size_t>(n_cand);
  a.cnt = reinterpret_cast<int32_t*>(p);
  p += (n * 4 + 15) & ~static_cast<size_t>(15);
  a.item_pos = reinterpret_cast<int32_t*>(p);
  p += (n * 4 + 15) & ~static_cast<size_t>(15);
  a.kv_off = reinterpret_cast<long long*>(p);
  p += (n * 8 + 15) & ~static_cast<size_t>(15);
  a.hist = reinterpret_cast<int32_t*>(p);
  const cudaError_t e = launch_attn_compact(a, static_cast<cudaStream_t>(stream));
  count_launches(a.n_cand > 0 ? 3 : 0);
  return e == cudaSuccess ? FO_OK : fail_cuda("fo_mask_compact", e);
}

size_t fo_attn_partial_bytes(int64_t partial_slots) {
  return partial_slots > 0 ? static_cast<size_t>(partial_slots) * kPartialFloats * sizeof(float) : 0;
}

int fo_attn_units(const int32_t* items, const int32_t* kv_ptr, const int32_t* kv_idx, const int32_t* order,
                  const int32_t* counters, const int32_t* qo_indptr, const int32_t* kv_indptr, int64_t max_items,
                  int32_t max_nkv, int32_t sbq, int32_t sbkv, int32_t min_items, int32_t num_streams, int32_t min_chunk, int64_t max_units,
                  int64_t max_slots, int32_t* units, int32_t* unit_counters, int32_t* arrive, void* stream) {
  if (items == nullptr || kv_ptr == nullptr || kv_idx == nullptr || order == nullptr || counters == nullptr ||
      qo_indptr == nullptr || kv_indptr == nullptr || units == nullptr || unit_counters == nullptr ||
      (max_slots > 0 && arrive == nullptr))
    return fail(FO_ERR_INVALID_ARG, "fo_attn_units: null pointer");
  if (max_items <= 0 || max_units < max_items || max_slots < 0 || num_streams <= 0 || min_chunk <= 0 || max_nkv < 0 ||
      sbq <= 0 || sbkv <= 0)
    return fail(FO_ERR_INVALID_ARG, "fo_attn_units: max_units must cover max_items; sizes must be positive");
  if (!aligned16(units)) return fail(FO_ERR_INVALID_ARG, "fo_attn_units: units must be 16-byte aligned");
  UnitArgs a;
  memset(&a, 0, sizeof(a));
  a.items = items;
  a.kv_ptr = kv_ptr;
  a.kv_idx = kv_idx;
  a.order = order;
  a.counters = counters;
  a.qo_indptr = qo_indptr;
  a.kv_indptr = kv_indptr;
  a.max_items = max_items;
  a.max_units = max_units;
  a.max_slots = max_slots;
  a.num_streams = num_streams;
  a.min_items = min_items < 0 ? 0 : min_items;
  a.min_chunk = min_chunk;
  a.max_nkv = max_nkv;
  a.sbq = sbq;
  a.sbkv = sbkv;
  a.units = units;
  a.unit_counters = unit_counters;
  a.arrive = arrive;
  const cudaError_t e = launch_attn_units(a, static_cast<cudaStream_t>(stream));
  count_launches(1);
  return e == cudaSuccess ? FO_OK : fail_cuda("fo_attn_units", e);
}

// ------------------------------------------------------------------------------------------ attention
namespace {
int sparse_attn_impl(const void* q, const void* k, const void* v, void* o, float* lse, int32_t dtype,
                     int64_t total_q, int64_t total_kv, int32_t num_qo_heads, int32_t num_kv_heads,
                     int32_t head_dim, int64_t q_stride_n, int64_t q_stride_h, int64_t k_stride_n,
                     int64_t k_stride_h, int64_t v_stride_n, int64_t v_stride_h, int64_t o_stride_n,
                     int64_t o_stride_h, int32_t sbq, int32_t sbkv, const int32_t* kv_idx,
                     const int32_t* units, const int32_t* unit_counters, int64_t max_units, int32_t* arrive,
                     float* partials, int64_t partial_slots, int32_t head_begin, float sm_scale,
                     float logits_soft_cap, int32_t mask_mode, const uint8_t* custom_mask, int64_t custom_mask_bytes,
                     const int32_t* mask_indptr, const int32_t* qo_indptr, const int32_t* kv_indptr, int32_t* status,
                     void* stream) {
  if (mask_mode == 2 && (custom_mask == nullptr || mask_indptr == nullptr || qo_indptr == nullptr || kv_indptr == nullptr ||
                         custom_mask_bytes <= 0))
    return fail(FO_ERR_INVALID_ARG, "fo_sparse_attn_fwd_custom_mask: mask, its indptr and the request indptrs are required");
  if (!(logits_soft_cap >= 0.f) || !(sm_scale > 0.f))
    return fail(FO_ERR_INVALID_ARG, "fo_sparse_attn_fwd: sm_scale must be positive and logits_soft_cap >= 0");
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr)
    return fail(FO_ERR_INVALID_ARG, "fo_sparse_attn_fwd: null q/k/v/o");
  if (kv_idx == nullptr || units == nullptr || unit_counters == nullptr || status == nullptr)
    return fail(FO_ERR_INVALID_ARG, "fo_sparse_attn_fwd: null work list / status");
  if (!aligned16(units)) return fail(FO_ERR_INVALID_ARG, "fo_sparse_attn_fwd: units must be 16-byte aligned");
  if (partial_slots < 0 || (partial_slots > 0 && (partials == nullptr || !aligned16(partials) || arrive == nullptr)))
    return fail(FO_ERR_INVALID_ARG, "fo_sparse_attn_fwd: partial-result scratch missing or misaligned");
  if (dtype != FO_DTYPE_F16 && dtype != FO_DTYPE_BF16) return fail(FO_ERR_INVALID_ARG, "fo_sparse_attn_fwd: bad dtype");
  if (head_dim != 128 && head_dim != 64 && head_dim != 256)
    return fail(FO_ERR_UNSUPPORTED, "fo_sparse_attn_fwd: head_dim must be 64, 128 or 256");
  if (head_dim == 256 && partial_slots > 0)
    return fail(FO_ERR_UNSUPPORTED, "fo_sparse_attn_fwd: head_dim 256 runs whole items only (partial_slots must be 0)");
  if (sbq != 128 || sbkv != 128)
    return fail(FO_ERR_UNSUPPORTED, "fo_sparse_attn_fwd: only 128-row q and kv sparse blocks are implemented");
  if (num_qo_heads <= 0 || num_kv_heads <= 0 || num_qo_heads % num_kv_heads != 0)
    return fail(FO_ERR_INVALID_ARG, "fo_sparse_attn_fwd: num_qo_heads must be a multiple of num_kv_heads");
  if (total_q <= 0 || total_kv <= 0 || max_units <= 0) return FO_OK;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o))
    return fail(FO_ERR_INVALID_ARG, "fo_sparse_attn_fwd: q/k/v/o must be 16-byte aligned");
  const int64_t strides[] = {q_stride_n, q_stride_h, k_stride_n, k_stride_h, v_stride_n, v_stride_h, o_stride_n, o_stride_h};
  for (int64_t s : strides)
    if (s <= 0 || (s % 8) != 0)
      return fail(FO_ERR_INVALID_ARG, "fo_sparse_attn_fwd: strides must be positive multiples of 8 elements");

  // With several q heads per kv head a q tile is 128 rows of (token, q head of the group) pairs, token-major, as the
  // reference packs them (include/flashomni/attention/prefill.cuh:1283-1291): a box of group heads x 128 / group tokens.
  const uint32_t group = static_cast<uint32_t>(num_qo_heads / num_kv_heads);
  if (group > 16 || (16 % group) != 0)
    return fail(FO_ERR_UNSUPPORTED, "fo_sparse_attn_fwd: num_qo_heads / num_kv_heads must be 1, 2, 4, 8 or 16");
  AttnArgs a;
  memset(&a, 0, sizeof(a));
  {
    const uint32_t box[3] = {64, 1, 128};
    const uint32_t qbox[3] = {64, group, 128 / group};
    const uint64_t qd[3] = {static_cast<uint64_t>(head_dim), static_cast<uint64_t>(num_qo_heads), static_cast<uint64_t>(total_q)};
    const uint64_t qs[3] = {0, static_cast<uint64_t>(q_stride_h) * 2, static_cast<uint64_t>(q_stride_n) * 2};
    const uint64_t kd[3] = {static_cast<uint64_t>(head_dim), static_cast<uint64_t>(num_kv_heads), static_cast<uint64_t>(total_kv)};
    const uint64_t ks[3] = {0, static_cast<uint64_t>(k_stride_h) * 2, static_cast<uint64_t>(k_stride_n) * 2};
    const uint64_t vs[3] = {0, static_cast<uint64_t>(v_stride_h) * 2, static_cast<uint64_t>(v_stride_n) * 2};
    int r = encode_tmap_16bit(&a.tmap_q, q, 3, qd, qs, qbox);
    if (r == 0) r = encode_tmap_16bit(&a.tmap_k, k, 3, kd, ks, box);
    if (r == 0) r = encode_tmap_16bit(&a.tmap_v, v, 3, kd, vs, box);
    const uint64_t os[3] = {0, static_cast<uint64_t>(o_stride_h) * 2, static_cast<uint64_t>(o_stride_n) * 2};
    if (r == 0) r = encode_tmap_16bit(&a.tmap_o, o, 3, qd, os, qbox);  // stores of 64 columns x 128 rows
    const uint32_t obox16[3] = {32, group, 16 / group};
    if (r == 0) r = encode_tmap_16bit(&a.tmap_o16, o, 3, qd, os, obox16, false);
    if (r != 0) {
      char buf[96];
      snprintf(buf, sizeof(buf), "fo_sparse_attn_fwd: cuTensorMapEncodeTiled failed (%d)", r);
      return fail(FO_ERR_CUDA, buf);
    }
  }
  a.o = o;
  a.lse = lse;
  a.o_stride_n = o_stride_n;
  a.o_stride_h = o_stride_h;
  a.lse_stride_n = num_qo_heads;
  a.kv_idx = kv_idx;
  a.units = units;
  a.unit_counters = unit_counters;
  a.max_units = static_cast<int>(max_units > 0x7fffffffLL ? 0x7fffffffLL : max_units);
  a.arrive = arrive;
  a.partials = partials;
  a.partial_slots = static_cast<int>(partial_slots > 0x7fffffffLL ? 0x7fffffffLL : partial_slots);
  a.head_begin = head_begin;
  a.head_dim = head_dim;
  a.mask_mode = mask_mode;
  a.custom_mask = custom_mask;
  a.custom_mask_bytes = custom_mask_bytes;
  a.mask_indptr = mask_indptr;
  a.qo_indptr = qo_indptr;
  a.kv_indptr = kv_indptr;
  a.group_size = static_cast<int>(group);
  a.is_bf16 = dtype == FO_DTYPE_BF16;
  if (logits_soft_cap > 0.f) {
    a.soft_cap_pre = sm_scale / logits_soft_cap;
    a.sm_scale_log2 = logits_soft_cap * 1.4426950408889634f;
  } else {
    a.soft_cap_pre = 0.f;
    a.sm_scale_log2 = sm_scale * 1.4426950408889634f;
  }
  a.status = status;
  int64_t ctas = static_cast<int64_t>(sm_count());  // one persistent CTA per SM
  if (ctas > max_units) ctas = max_units;
  const cudaError_t e = launch_attention(a, static_cast<int>(ctas), static_cast<cudaStream_t>(stream));
  count_launches(1);
  return e == cudaSuccess ? FO_OK : fail_cuda("fo_sparse_attn_fwd", e);
}
}  // namespace

int fo_sparse_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int32_t dtype,
                       int64_t total_q, int64_t total_kv, int32_t num_qo_heads, int32_t num_kv_heads,
                       int32_t head_dim, int64_t q_stride_n, int64_t q_stride_h, int64_t k_stride_n,
                       int64_t k_stride_h, int64_t v_stride_n, int64_t v_stride_h, int64_t o_stride_n,
                       int64_t o_stride_h, int32_t sbq, int32_t sbkv, const int32_t* kv_idx,
                       const int32_t* units, const int32_t* unit_counters, int64_t max_units, int32_t* arrive,
                       float* partials, int64_t partial_slots, int32_t head_begin, float sm_scale, int32_t* status,
                       void* stream) {
  return sparse_attn_impl(q, k, v, o, lse, dtype, total_q, total_kv, num_qo_heads, num_kv_heads, head_dim, q_stride_n,
                          q_stride_h, k_stride_n, k_stride_h, v_stride_n, v_stride_h, o_stride_n, o_stride_h, sbq, sbkv,
                          kv_idx, units, unit_counters, max_units, arrive, partials,
                          partial_slots, head_begin, sm_scale, 0.f, 0, nullptr, 0, nullptr, nullptr, nullptr, status, stream);
}

int fo_sparse_attn_fwd_softcap(const void* q, const void* k, const void* v, void* o, float* lse, int32_t dtype,
                               int64_t total_q, int64_t total_kv, int32_t num_qo_heads, int32_t num_kv_heads,
                               int32_t head_dim, int64_t q_stride_n, int64_t q_stride_h, int64_t k_stride_n,
                               int64_t k_stride_h, int64_t v_stride_n, int64_t v_stride_h, int64_t o_stride_n,
                               int64_t o_stride_h, int32_t sbq, int32_t sbkv, const int32_t* kv_idx,
                               const int32_t* units, const int32_t* unit_counters, int64_t max_units, int32_t* arrive,
                               float* partials, int64_t partial_slots, int32_t head_begin, float sm_scale,
                               float logits_soft_cap, int32_t* status, void* stream) {
  return sparse_attn_impl(q, k, v, o, lse, dtype, total_q, total_kv, num_qo_heads, num_kv_heads, head_dim, q_stride_n,
                          q_stride_h, k_stride_n, k_stride_h, v_stride_n, v_stride_h, o_stride_n, o_stride_h, sbq, sbkv,
                          kv_idx, units, unit_counters, max_units, arrive, partials,
                          partial_slots, head_begin, sm_scale, logits_soft_cap, 0, nullptr, 0, nullptr, nullptr, nullptr, status, stream);
}

int fo_sparse_attn_fwd_causal(const void* q, const void* k, const void* v, void* o, float* lse, int32_t dtype,
                              int64_t total_q, int64_t total_kv, int32_t num_qo_heads, int32_t num_kv_heads,
                              int32_t head_dim, int64_t q_stride_n, int64_t q_stride_h, int64_t k_stride_n,
                              int64_t k_stride_h, int64_t v_stride_n, int64_t v_stride_h, int64_t o_stride_n,
                              int64_t o_stride_h, int32_t sbq, int32_t sbkv, const int32_t* kv_idx,
                              const int32_t* units, const int32_t* unit_counters, int64_t max_units, int32_t head_begin,
                              float sm_scale, float logits_soft_cap, int32_t* status, void* stream) {
  return sparse_attn_impl(q, k, v, o, lse, dtype, total_q, total_kv, num_qo_heads, num_kv_heads, head_dim, q_stride_n,
                          q_stride_h, k_stride_n, k_stride_h, v_stride_n, v_stride_h, o_stride_n, o_stride_h, sbq, sbkv,
                          kv_idx, units, unit_counters, max_units, nullptr, nullptr, 0, head_begin, sm_scale,
                          logits_soft_cap, 1, nullptr, 0, nullptr, nullptr, nullptr, status, stream);
}

int fo_sparse_attn_fwd_custom_mask(const void* q, const void* k, const void* v, void* o, float* lse, int32_t dtype,
                                   int64_t total_q, int64_t total_kv, int32_t num_qo_heads, int32_t num_kv_heads,
                                   int32_t head_dim, int64_t q_stride_n, int64_t q_stride_h, int64_t k_stride_n,
                                   int64_t k_stride_h, int64_t v_stride_n, int64_t v_stride_h, int64_t o_stride_n,
                                   int64_t o_stride_h, int32_t sbq, int32_t sbkv, const int32_t* kv_idx,
                                   const int32_t* units, const int32_t* unit_counters, int64_t max_units,
                                   int32_t head_begin, float sm_scale, float logits_soft_cap, const uint8_t* custom_mask,
                                   int64_t custom_mask_bytes, const int32_t* mask_indptr, const int32_t* qo_indptr,
                                   const int32_t* kv_indptr, int32_t* status, void* stream) {
  return sparse_attn_impl(q, k, v, o, lse, dtype, total_q, total_kv, num_qo_heads, num_kv_heads, head_dim, q_stride_n,
                          q_stride_h, k_stride_n, k_stride_h, v_stride_n, v_stride_h, o_stride_n, o_stride_h, sbq, sbkv,
                          kv_idx, units, unit_counters, max_units, nullptr, nullptr, 0, head_begin, sm_scale,
                          logits_soft_cap, 2, custom_mask, custom_mask_bytes, mask_indptr, qo_indptr, kv_indptr, status,
                          stream);
}

int fo_cast_fp8(const void* src, int64_t n, int32_t fp8_kind, int32_t dtype, void* dst, void* stream) {
  if (n < 0) return fail(FO_ERR_INVALID_ARG, "fo_cast_fp8: n < 0");
  if (n == 0) return FO_OK;
  if (src == nullptr || dst == nullptr || !aligned16(src) || !aligned16(dst))
    return fail(FO_ERR_INVALID_ARG, "fo_cast_fp8: null or misaligned pointer (16 bytes)");
  if ((fp8_kind != 0 && fp8_kind != 1) || (dtype != FO_DTYPE_F16 && dtype != FO_DTYPE_BF16))
    return fail(FO_ERR_INVALID_ARG, "fo_cast_fp8: fp8_kind must be 0 (e4m3) or 1 (e5m2), dtype f16 or bf16");
  const cudaError_t e = launch_cast_fp8(src, n, fp8_kind, dtype == FO_DTYPE_BF16, dst, sm_count(), static_cast<cudaStream_t>(stream));
  count_launches(1);
  return e == cudaSuccess ? FO_OK : fail_cuda("fo_cast_fp8", e);
}

// ------------------------------------------------------------------------------------------ GEMMs
int fo_gemm_dense_tile_rows(int32_t batch, int32_t m, int32_t n, int32_t k, int32_t has_full_init, int32_t sm_count) {
  if (batch <= 0 || m <= 0 || n <= 0 || k <= 0) return 0;
  GemmArgs g;
  memset(&g, 0, sizeof(g));
  g.mode = kGemmQ;
  g.init_mode = has_full_init ? kInitFull : kInitNone;
  g.batch = batch;
  g.m = m;
  g.n = n;
  g.k = k;
  return gemm_tall_applies(g, sm_count) ? 256 : 128;
}

int fo_gemm_dense_tile_cols(int32_t batch, int32_t m, int32_t n, int32_t k, int32_t has_full_init, int32_t sm_count) {
  if (batch <= 0 || m <= 0 || n <= 0 || k <= 0) return 0;
  GemmArgs g;
  memset(&g, 0, sizeof(g));
  g.mode = kGemmQ;
  g.init_mode = has_full_init ? kInitFull : kInitNone;
  g.batch = batch;
  g.m = m;
  g.n = n;
  g.k = k;
  const int c = tall_tile_cols(g, sm_count);
  return c != 0 ? c : 256;
}

size_t fo_gemm_workspace_bytes(int32_t batch, int32_t m, int32_t n, int32_t k, int32_t head_dim) {
  if (batch <= 0 || m <= 0 || n <= 0 || k <= 0 || head_dim <= 0) return 64;
  const size_t mt = static_cast<size_t>(m) / 128, nt = static_cast<size_t>(n) / 128;
  const size_t rows = static_cast<size_t>(batch) * mt;
  const size_t lh = static_cast<size_t>(k) / static_cast<size_t>(head_dim);
  const size_t words_q = 8 + 4 * rows * nt;
  const size_t words_o = 8 + (rows + 1) + rows * (lh > 0 ? lh : 1) + rows;
  const size_t words = words_q > words_o ? words_q : words_o;
  return ((words * 4 + 255) / 256) * 256;
}

namespace {

struct GemmShape {
  int32_t batch, m, n, k, num_heads, head_begin, head_dim, sparse_q_size, num_text_tokens;
};

int check_lists_common(const char* who, const GemmShape& s, bool need_mask, const uint8_t* sparse_info,
                       const int32_t* indptr, void* ws, size_t ws_bytes) {
  if (s.batch <= 0 || s.m <= 0 || s.n <= 0 || s.k <= 0) return fail(FO_ERR_INVALID_ARG, std::string(who) + ": empty shape");
  if (s.m % 128 != 0 || s.n % 128 != 0)
    return fail(FO_ERR_INVALID_ARG, std::string(who) + ": m and n must be multiples of 128");
  if (s.num_heads <= 0 || s.head_dim <= 0 || s.head_begin < 0 || s.sparse_q_size <= 0 || s.num_text_tokens < 0)
    return fail(FO_ERR_INVALID_ARG, std::string(who) + ": bad head / block parameters");
  if (need_mask && (sparse_info == nullptr || indptr == nullptr))
    return fail(FO_ERR_INVALID_ARG, std::string(who) + ": sparse_info and sparse_info_indptr are required");
  if (ws == nullptr || !aligned16(ws) ||
      ws_bytes < fo_gemm_workspace_bytes(s.batch, s.m, s.n, s.k, s.head_dim))
    return fail(FO_ERR_WORKSPACE, std::string(who) + ": workspace too small or misaligned");
  return FO_OK;
}

GemmListArgs make_list_args(const GemmShape& s, const uint8_t* sparse_info, int64_t info_bytes,
                            const int32_t* indptr, void* ws) {
  GemmListArgs a;
  memset(&a, 0, sizeof(a));
  a.sparse_info = sparse_info;
  a.info_indptr = indptr;
  a.info_bytes = info_bytes;
  a.batch = s.batch;
  a.m = s.m;
  a.n = s.n;
  a.k = s.k;
  a.num_heads = s.num_heads;
  a.head_begin = s.head_begin;
  a.head_dim = s.head_dim;
  a.sparse_q_size = s.sparse_q_size;
  a.num_text_tokens = s.num_text_tokens;
  int32_t* w = static_cast<int32_t*>(ws);
  a.counters = w;
  const int rows = s.batch * (s.m / 128);
  const int lh = s.k / s.head_dim;
  a.tiles = w + 8;
  a.max_tiles = rows * (s.n / 128);
  a.n_ctas = sm_count();
  a.row_indptr = w + 8;
  a.row_heads = w + 8 + rows + 1;
  a.row_order = w + 8 + rows + 1 + rows * (lh > 0 ? lh : 1);
  return a;
}

}  // namespace

int fo_gemm_q_worklist(int32_t batch, int32_t m, int32_t n, int32_t num_heads, int32_t head_begin,
                       int32_t head_dim, int32_t sparse_q_size, int32_t num_text_tokens, int32_t is_full,
                       const uint8_t* sparse_info, int64_t sparse_info_bytes, const int32_t* sparse_info_indptr,
                       void* workspace, size_t workspace_bytes, void* stream) {
  const GemmShape s = {batch, m, n, head_dim > 0 ? head_dim : 1, num_heads, head_begin, head_dim, sparse_q_size, num_text_tokens};
  int rc = check_lists_common("fo_gemm_q_worklist", s, !is_full, sparse_info, sparse_info_indptr, workspace, workspace_bytes);
  if (rc != FO_OK) return rc;
  if (128 % head_dim != 0 && head_dim % 128 != 0)
    return fail(FO_ERR_UNSUPPORTED, "fo_gemm_q_worklist: head_dim must divide or be a multiple of 128");
  GemmListArgs a = make_list_args(s, sparse_info, sparse_info_bytes, sparse_info_indptr, workspace);
  a.is_full = is_full;
  const cudaError_t e = launch_gemm_q_tiles(a, static_cast<cudaStream_t>(stream));
  count_launches(1);
  return e == cudaSuccess ? FO_OK : fail_cuda("fo_gemm_q_worklist", e);
}

int fo_gemm_o_worklist(int32_t batch, int32_t m, int32_t k, int32_t num_heads, int32_t head_begin,
                       int32_t head_dim, int32_t sparse_q_size, int32_t num_text_tokens, int32_t is_for_cache,
                       const uint8_t* sparse_info, int64_t sparse_info_bytes, const int32_t* sparse_info_indptr,
                       void* workspace, size_t workspace_bytes, void* stream) {
  const GemmShape s = {batch, m, 128, k, num_heads, head_begin, head_dim, sparse_q_size, num_text_tokens};
  int rc = check_lists_common("fo_gemm_o_worklist", s, true, sparse_info, sparse_info_indptr, workspace, workspace_bytes);
  if (rc != FO_OK) return rc;
  if (k % head_dim != 0) return fail(FO_ERR_INVALID_ARG, "fo_gemm_o_worklist: k must be a multiple of head_dim");
  GemmListArgs a = make_list_args(s, sparse_info, sparse_info_bytes, sparse_info_indptr, workspace);
  a.is_for_cache = is_for_cache;
  const cudaError_t e = launch_gemm_o_rows(a, static_cast<cudaStream_t>(stream));
  count_launches(1);
  return e == cudaSuccess ? FO_OK : fail_cuda("fo_gemm_o_worklist", e);
}

namespace {

int encode_gemm_maps(const char* who, GemmArgs& g, const void* x, const void* w, const void* y, int64_t rows_a,
                     int64_t n, int64_t k) {
  const uint32_t box[2] = {64, 128};
  const uint64_t ad[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(rows_a)};
  const uint64_t bd[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n)};
  const uint64_t yd[2] = {static_cast<uint64_t>(n), static_cast<uint64_t>(rows_a)};
  const uint64_t st[2] = {0, static_cast<uint64_t>(k) * 2};
  const uint64_t yst[2] = {0, static_cast<uint64_t>(n) * 2};
  int r = encode_tmap_16bit(&g.tmap_a, x, 2, ad, st, box);
  if (r == 0) r = encode_tmap_16bit(&g.tmap_b, w, 2, bd, st, box);
  if (r == 0) r = encode_tmap_16bit(&g.tmap_y, y, 2, yd, yst, box);
  if (r != 0) {
    char buf[96];
    snprintf(buf, sizeof(buf), "%s: cuTensorMapEncodeTiled failed (%d)", who, r);
    return fail(FO_ERR_CUDA, buf);
  }
  return FO_OK;
}

}  // namespace

namespace {
// `prepared`: the work list is already in the workspace (built by fo_gemm_q_worklist on any stream ordered
// before this call); nothing is reset here (the kernel leaves the tile cursor at zero when it ends).
int gemm_q_impl(const void* x, const void* w, void* y, const void* bias, int32_t dtype, int32_t batch, int32_t m,
                int32_t n, int32_t k, int32_t num_heads, int32_t head_begin, int32_t head_dim,
                int32_t sparse_q_size, int32_t num_text_tokens, int32_t is_full, const uint8_t* sparse_info,
                int64_t sparse_info_bytes, const int32_t* sparse_info_indptr, void* workspace,
                size_t workspace_bytes, void* stream, bool prepared) {
  if (x == nullptr || w == nullptr || y == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_gemm_q: null x/w/y");
  if (dtype != FO_DTYPE_F16 && dtype != FO_DTYPE_BF16) return fail(FO_ERR_INVALID_ARG, "fo_gemm_q: bad dtype");
  const GemmShape s = {batch, m, n, k, num_heads, head_begin, head_dim, sparse_q_size, num_text_tokens};
  int rc = check_lists_common("fo_gemm_q", s, !is_full && !prepared, sparse_info, sparse_info_indptr, workspace, workspace_bytes);
  if (rc != FO_OK) return rc;
  if (k % 32 != 0) return fail(FO_ERR_INVALID_ARG, "fo_gemm_q: k must be a multiple of 32");
  if (128 % head_dim != 0 && head_dim % 128 != 0)
    return fail(FO_ERR_UNSUPPORTED, "fo_gemm_q: head_dim must divide or be a multiple of 128");
  if (!aligned16(x) || !aligned16(w) || !aligned16(y) || (bias != nullptr && !aligned16(bias)))
    return fail(FO_ERR_INVALID_ARG, "fo_gemm_q: pointers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int32_t* wsw = static_cast<int32_t*>(workspace);
  GemmArgs g;
  memset(&g, 0, sizeof(g));
  rc = encode_gemm_maps("fo_gemm_q", g, x, w, y, static_cast<int64_t>(batch) * m, n, k);
  if (rc != FO_OK) return rc;
  cudaError_t e;
  if (!is_full) {
    GemmListArgs la = make_list_args(s, sparse_info, sparse_info_bytes, sparse_info_indptr, workspace);
    la.is_full = 0;
    // A prepared list needs nothing here: the kernel leaves its cursor at zero when it ends, and the status word
    // (set only when a bounded wait runs out) stays as it is until the next list is built.
    e = prepared ? cudaSuccess : launch_gemm_q_tiles(la, st);
    if (e != cudaSuccess) return fail_cuda("fo_gemm_q (work list)", e);
    count_launches(prepared ? 0 : 1);
    g.tiles = la.tiles;
    g.n_tiles_ptr = la.counters;
  }
  g.y = y;
  g.init = bias;
  g.init_mode = bias != nullptr ? kInitBias1D : kInitNone;
  g.mode = kGemmQ;
  g.is_bf16 = dtype == FO_DTYPE_BF16;
  g.batch = batch;
  g.m = m;
  g.n = n;
  g.k = k;
  g.kb_per_head = 1;
  g.status = wsw + 4;
  g.cursor = is_full ? nullptr : wsw + 5;  // equal tiles keep a fixed share
  if (gemm_tall_applies(g, sm_count())) {
    // the tall-tile kernel stores 16-row x 64-column boxes (one per-warp staging area at a time)
    const uint32_t ybox[2] = {64, 16};
    const uint64_t yd[2] = {static_cast<uint64_t>(n), static_cast<uint64_t>(batch) * m};
    const uint64_t yst[2] = {0, static_cast<uint64_t>(n) * 2};
    if (encode_tmap_16bit(&g.tmap_y, y, 2, yd, yst, ybox) != 0)
      return fail(FO_ERR_CUDA, "fo_gemm_q: cuTensorMapEncodeTiled failed (output boxes)");
    if (tall_tile_cols(g, sm_count()) == 192) {
      const uint32_t wbox[2] = {64, 64};
      const uint64_t wd[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n)};
      const uint64_t wst[2] = {0, static_cast<uint64_t>(k) * 2};
      if (encode_tmap_16bit(&g.tmap_b64, w, 2, wd, wst, wbox) != 0)
        return fail(FO_ERR_CUDA, "fo_gemm_q: cuTensorMapEncodeTiled failed (64-row weight boxes)");
    }
    e = launch_gemm_tall(g, sm_count(), st);
  } else {
    e = launch_gemm(g, sm_count(), st);
  }
  count_launches(1);
  return e == cudaSuccess ? FO_OK : fail_cuda("fo_gemm_q", e);
}
}  // namespace

int fo_gemm_q(const void* x, const void* w, void* y, const void* bias, int32_t dtype, int32_t batch, int32_t m,
              int32_t n, int32_t k, int32_t num_heads, int32_t head_begin, int32_t head_dim,
              int32_t sparse_q_size, int32_t num_text_tokens, int32_t is_full, const uint8_t* sparse_info,
              int64_t sparse_info_bytes, const int32_t* sparse_info_indptr, void* workspace,
              size_t workspace_bytes, void* stream) {
  return gemm_q_impl(x, w, y, bias, dtype, batch, m, n, k, num_heads, head_begin, head_dim, sparse_q_size,
                     num_text_tokens, is_full, sparse_info, sparse_info_bytes, sparse_info_indptr, workspace,
                     workspace_bytes, stream, false);
}

int fo_gemm_q_prepared(const void* x, const void* w, void* y, const void* bias, int32_t dtype, int32_t batch,
                       int32_t m, int32_t n, int32_t k, int32_t head_dim, void* workspace, size_t workspace_bytes,
                       void* stream) {
  return gemm_q_impl(x, w, y, bias, dtype, batch, m, n, k, 1, 0, head_dim, 128, 0, 0, nullptr, 0, nullptr, workspace,
                     workspace_bytes, stream, true);
}

namespace {
int gemm_o_impl(const void* x, const void* w, void* y, const void* init, int32_t init_is_full, int32_t dtype,
                int32_t batch, int32_t m, int32_t n, int32_t k, int32_t num_heads, int32_t head_begin,
                int32_t head_dim, int32_t sparse_q_size, int32_t num_text_tokens, int32_t is_for_cache,
                const uint8_t* sparse_info, int64_t sparse_info_bytes, const int32_t* sparse_info_indptr,
                void* workspace, size_t workspace_bytes, void* stream, bool prepared) {
  if (x == nullptr || w == nullptr || y == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_gemm_o: null x/w/y");
  if (dtype != FO_DTYPE_F16 && dtype != FO_DTYPE_BF16) return fail(FO_ERR_INVALID_ARG, "fo_gemm_o: bad dtype");
  const GemmShape s = {batch, m, n, k, num_heads, head_begin, head_dim, sparse_q_size, num_text_tokens};
  int rc = check_lists_common("fo_gemm_o", s, !prepared, sparse_info, sparse_info_indptr, workspace, workspace_bytes);
  if (rc != FO_OK) return rc;
  if (head_dim % 64 != 0) return fail(FO_ERR_UNSUPPORTED, "fo_gemm_o: head_dim must be a multiple of 64");
  if (k % head_dim != 0) return fail(FO_ERR_INVALID_ARG, "fo_gemm_o: k must be a multiple of head_dim");
  if (!aligned16(x) || !aligned16(w) || !aligned16(y) || (init != nullptr && !aligned16(init)))
    return fail(FO_ERR_INVALID_ARG, "fo_gemm_o: pointers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int32_t* wsw = static_cast<int32_t*>(workspace);
  GemmArgs g;
  memset(&g, 0, sizeof(g));
  rc = encode_gemm_maps("fo_gemm_o", g, x, w, y, static_cast<int64_t>(batch) * m, n, k);
  if (rc != FO_OK) return rc;
  GemmListArgs la = make_list_args(s, sparse_info, sparse_info_bytes, sparse_info_indptr, workspace);
  la.is_for_cache = is_for_cache;
  cudaError_t e = prepared ? cudaSuccess : launch_gemm_o_rows(la, st);
  if (e != cudaSuccess) return fail_cuda("fo_gemm_o (work list)", e);
  count_launches(prepared ? 1 : 2);
  g.y = y;
  g.init = init;
  g.init_mode = init == nullptr ? kInitNone : (init_is_full ? kInitFull : kInitBias1D);
  g.mode = kGemmO;
  g.is_bf16 = dtype == FO_DTYPE_BF16;
  g.batch = batch;
  g.m = m;
  g.n = n;
  g.k = k;
  g.kb_per_head = head_dim / 64;
  g.row_indptr = la.row_indptr;
  g.row_heads = la.row_heads;
  g.row_order = la.row_order;
  g.status = wsw + 4;
  g.cursor = wsw + 5;
  e = launch_gemm(g, sm_count(), st);
  return e == cudaSuccess ? FO_OK : fail_cuda("fo_gemm_o", e);
}
}  // namespace

int fo_gemm_o(const void* x, const void* w, void* y, const void* init, int32_t init_is_full, int32_t dtype,
              int32_t batch, int32_t m, int32_t n, int32_t k, int32_t num_heads, int32_t head_begin,
              int32_t head_dim, int32_t sparse_q_size, int32_t num_text_tokens, int32_t is_for_cache,
              const uint8_t* sparse_info, int64_t sparse_info_bytes, const int32_t* sparse_info_indptr,
              void* workspace, size_t workspace_bytes, void* stream) {
  return gemm_o_impl(x, w, y, init, init_is_full, dtype, batch, m, n, k, num_heads, head_begin, head_dim,
                     sparse_q_size, num_text_tokens, is_for_cache, sparse_info, sparse_info_bytes,
                     sparse_info_indptr, workspace, workspace_bytes, stream, false);
}

int fo_gemm_o_prepared(const void* x, const void* w, void* y, const void* init, int32_t init_is_full, int32_t dtype,
                       int32_t batch, int32_t m, int32_t n, int32_t k, int32_t head_dim, void* workspace,
                       size_t workspace_bytes, void* stream) {
  return gemm_o_impl(x, w, y, init, init_is_full, dtype, batch, m, n, k, 1, 0, head_dim, 128, 0, 0, nullptr, 0,
                     nullptr, workspace, workspace_bytes, stream, true);
}

size_t fo_select_blocks_scratch_bytes(int32_t batch, int32_t num_blocks) {
  if (batch < 0 || num_blocks < 0) return 0;
  const size_t n = static_cast<size_t>(batch) * static_cast<size_t>(num_blocks);
  return ((n * 4 + 15) & ~static_cast<size_t>(15)) + ((n + 15) & ~static_cast<size_t>(15)) + 16;
}

int32_t fo_select_blocks(const float* pooled_score, int32_t batch, int32_t num_heads, int32_t num_blocks,
                         int32_t num_text_blocks, const float* q_threshold, const float* kv_threshold,
                         int32_t zero_inactive, uint8_t* sparse_info, int64_t sparse_info_bytes,
                         uint8_t* sparse_kv_info, int64_t sparse_kv_info_bytes, int32_t* info_indptr,
                         int32_t* kv_info_indptr, void* scratch, size_t scratch_bytes, void* stream) {
  if (batch <= 0 || num_heads <= 0 || num_blocks <= 0 || num_text_blocks < 0 || num_text_blocks > num_blocks)
    return fail(FO_ERR_INVALID_ARG, "fo_select_blocks: bad sizes");
  if (num_blocks > 2048) return fail(FO_ERR_UNSUPPORTED, "fo_select_blocks: at most 2048 blocks per request");
  if (pooled_score == nullptr || q_threshold == nullptr || kv_threshold == nullptr || sparse_info == nullptr ||
      sparse_kv_info == nullptr || info_indptr == nullptr || kv_info_indptr == nullptr)
    return fail(FO_ERR_INVALID_ARG, "fo_select_blocks: null pointer");
  SelectArgs a;
  memset(&a, 0, sizeof(a));
  a.info_seg_bytes = (static_cast<int64_t>(num_blocks) * num_heads + 7) / 8;
  a.kv_seg_bytes = (static_cast<int64_t>(num_blocks) * num_heads * num_blocks + 7) / 8;
  a.kv_words = (static_cast<int64_t>(batch) * a.kv_seg_bytes + 3) / 4;
  if (a.kv_seg_bytes * batch > 0x7fffffffLL)
    return fail(FO_ERR_UNSUPPORTED, "fo_select_blocks: packed kv mask above 2 GiB (int32 byte indptr)");
  if (sparse_info_bytes < a.info_seg_bytes * batch || sparse_kv_info_bytes < a.kv_words * 4)
    return fail(FO_ERR_INVALID_ARG, "fo_select_blocks: output buffers too small (the kv stream is written in 4-byte words)");
  if ((reinterpret_cast<uintptr_t>(sparse_kv_info) & 3u) != 0)
    return fail(FO_ERR_INVALID_ARG, "fo_select_blocks: sparse_kv_info must be 4-byte aligned");
  if (scratch == nullptr || scratch_bytes < fo_select_blocks_scratch_bytes(batch, num_blocks) || !aligned16(scratch))
    return fail(FO_ERR_WORKSPACE, "fo_select_blocks: scratch too small or misaligned");
  a.score = pooled_score;
  a.q_thr = q_threshold;
  a.kv_thr = kv_threshold;
  a.batch = batch;
  a.heads = num_heads;
  a.n = num_blocks;
  a.t2t = num_text_blocks;
  a.zero_inactive = zero_inactive;
  a.sparse_info = sparse_info;
  a.sparse_kv_info = sparse_kv_info;
  a.info_indptr = info_indptr;
  a.kv_info_indptr = kv_info_indptr;
  const size_t n = static_cast<size_t>(batch) * static_cast<size_t>(num_blocks);
  a.t2i = static_cast<float*>(scratch);
  a.q_keep = static_cast<uint8_t*>(scratch) + ((n * 4 + 15) & ~static_cast<size_t>(15));
  const cudaError_t e = launch_select_blocks(a, static_cast<cudaStream_t>(stream));
  count_launches(3);
  return e == cudaSuccess ? FO_OK : fail_cuda("fo_select_blocks", e);
}

int32_t fo_strided_gather(int32_t n_src, const void* const* src, const int64_t* src_row_stride_bytes,
                          const int64_t* n_rows, void* const* dst, const int64_t* dst_row_stride_bytes,
                          int64_t row_bytes, void* stream) {
  if (n_src < 0 || n_src > kMaxGatherSources)
    return fail(FO_ERR_INVALID_ARG, "fo_strided_gather: between 0 and 16 sources");
  if (n_src == 0) return FO_OK;
  if (src == nullptr || dst == nullptr || src_row_stride_bytes == nullptr || dst_row_stride_bytes == nullptr ||
      n_rows == nullptr)
    return fail(FO_ERR_INVALID_ARG, "fo_strided_gather: null array");
  if (row_bytes <= 0 || row_bytes % 16 != 0)
    return fail(FO_ERR_INVALID_ARG, "fo_strided_gather: row_bytes must be a positive multiple of 16");
  GatherArgs a;
  memset(&a, 0, sizeof(a));
  a.n_src = n_src;
  a.row_vecs = row_bytes / 16;
  for (int i = 0; i < n_src; ++i) {
    if (n_rows[i] < 0) return fail(FO_ERR_INVALID_ARG, "fo_strided_gather: negative row count");
    if (n_rows[i] > 0 && (src[i] == nullptr || dst[i] == nullptr || !aligned16(src[i]) || !aligned16(dst[i]) ||
                          src_row_stride_bytes[i] % 16 != 0 || dst_row_stride_bytes[i] % 16 != 0 ||
                          src_row_stride_bytes[i] < row_bytes || dst_row_stride_bytes[i] < row_bytes))
      return fail(FO_ERR_INVALID_ARG, "fo_strided_gather: pointers and strides must be 16-byte aligned, strides >= row_bytes");
    a.src[i] = static_cast<const uint8_t*>(src[i]);
    a.dst[i] = static_cast<uint8_t*>(dst[i]);
    a.src_stride[i] = src_row_stride_bytes[i];
    a.dst_stride[i] = dst_row_stride_bytes[i];
    a.vec_prefix[i + 1] = a.vec_prefix[i] + n_rows[i] * a.row_vecs;
  }
  const cudaError_t e = launch_strided_gather(a, sm_count(), static_cast<cudaStream_t>(stream));
  count_launches(a.vec_prefix[a.n_src] > 0 ? 1 : 0);
  return e == cudaSuccess ? FO_OK : fail_cuda("fo_strided_gather", e);
}

int32_t fo_reduce_rows(int32_t n_src, const void* const* src, int64_t src_row_stride_bytes, const void* init,
                       int64_t init_row_stride_bytes, void* dst, int64_t dst_row_stride_bytes, int64_t n_rows,
                       int64_t row_bytes, int32_t dtype, void* stream) {
  if (n_src <= 0 || n_src > kMaxGatherSources) return fail(FO_ERR_INVALID_ARG, "fo_reduce_rows: between 1 and 16 sources");
  if (dtype != FO_DTYPE_F16 && dtype != FO_DTYPE_BF16) return fail(FO_ERR_INVALID_ARG, "fo_reduce_rows: bad dtype");
  if (n_rows < 0 || row_bytes <= 0 || row_bytes % 16 != 0)
    return fail(FO_ERR_INVALID_ARG, "fo_reduce_rows: row_bytes must be a positive multiple of 16");
  if (n_rows == 0) return FO_OK;
  if (src == nullptr || dst == nullptr || !aligned16(dst) || dst_row_stride_bytes % 16 != 0 ||
      src_row_stride_bytes % 16 != 0 || dst_row_stride_bytes < row_bytes || src_row_stride_bytes < row_bytes ||
      (init != nullptr && (!aligned16(init) || init_row_stride_bytes % 16 != 0 || init_row_stride_bytes < row_bytes)))
    return fail(FO_ERR_INVALID_ARG, "fo_reduce_rows: pointers and strides must be 16-byte aligned, strides >= row_bytes");
  ReduceArgs a;
  memset(&a, 0, sizeof(a));
  for (int i = 0; i < n_src; ++i) {
    if (src[i] == nullptr || !aligned16(src[i])) return fail(FO_ERR_INVALID_ARG, "fo_reduce_rows: null or misaligned source");
    a.src[i] = static_cast<const uint8_t*>(src[i]);
  }
  a.init = static_cast<const uint8_t*>(init);
  a.dst = static_cast<uint8_t*>(dst);
  a.src_stride = src_row_stride_bytes;
  a.init_stride = init_row_stride_bytes;
  a.dst_stride = dst_row_stride_bytes;
  a.rows = n_rows;
  a.row_vecs = row_bytes / 16;
  a.n_src = n_src;
  const cudaError_t e = launch_reduce_rows(a, dtype == FO_DTYPE_BF16, sm_count(), static_cast<cudaStream_t>(stream));
  count_launches(1);
  return e == cudaSuccess ? FO_OK : fail_cuda("fo_reduce_rows", e);
}

int32_t fo_peer_barrier(int32_t world, int32_t rank, int32_t* const* pads, int32_t channel, int32_t num_channels,
                        int32_t* epoch, int32_t* status, int64_t timeout_ms, void* stream) {
  if (world <= 0 || world > kMaxBarrierRanks || rank < 0 || rank >= world)
    return fail(FO_ERR_INVALID_ARG, "fo_peer_barrier: world must be 1..64 and rank inside it");
  if (channel < 0 || channel >= num_channels) return fail(FO_ERR_INVALID_ARG, "fo_peer_barrier: channel out of range");
  if (pads == nullptr || epoch == nullptr || status == nullptr)
    return fail(FO_ERR_INVALID_ARG, "fo_peer_barrier: null pads / epoch / status");
  if (timeout_ms <= 0 || timeout_ms > 60000) return fail(FO_ERR_INVALID_ARG, "fo_peer_barrier: timeout_ms must be 1..60000");
  BarrierArgs a;
  memset(&a, 0, sizeof(a));
  for (int i = 0; i < world; ++i) {
    if (pads[i] == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_peer_barrier: null pad pointer");
    a.pads[i] = pads[i];
  }
  a.epoch = epoch;
  a.status = status;
  a.rank = rank;
  a.world = world;
  a.channel = channel;
  a.timeout_ns = static_cast<uint64_t>(timeout_ms) * 1000000ull;
  const cudaError_t e = launch_peer_barrier(a, static_cast<cudaStream_t>(stream));
  count_launches(1);
  return e == cudaSuccess ? FO_OK : fail_cuda("fo_peer_barrier", e);
}

}  // extern "C"
