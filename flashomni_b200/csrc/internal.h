// Internal declarations shared by the translation units of libflashomni_b200.so.
// Nothing in this header is part of the C ABI (see include/flashomni_b200.h for that).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace fo {

// ------------------------------------------------------------------ mask path
struct CompactArgs {
  const uint8_t* sparse_info;
  const uint8_t* sparse_kv_info;
  const int32_t* info_indptr;      // byte offsets per request
  const int32_t* kv_info_indptr;   // byte offsets per request
  const int32_t* qo_indptr;        // token offsets per request
  const int32_t* kv_indptr;
  int64_t info_bytes;              // readable bytes of sparse_info
  int64_t kv_info_bytes;           // readable bytes of sparse_kv_info
  int batch, num_heads, head_begin, head_count, sbq, sbkv, is_full;
  int max_nkv;                     // upper bound of kv-blocks per request (histogram size - 1)
  int64_t n_cand;                  // sum_b nq(b) * head_count
  int64_t max_items, max_kept;     // capacities of the output lists
  // outputs
  int32_t* items;                  // [max_items, 4] (b, h, qb, n_kept)
  int32_t* kv_ptr;                 // [max_items + 1]
  int32_t* kv_idx;                 // [max_kept]
  int32_t* order;                  // [max_items]
  int32_t* counters;               // [4]: n_items, total_kept, status, max_nkv
  // scratch
  int32_t* cnt;                    // [n_cand]
  int32_t* item_pos;               // [n_cand]
  long long* kv_off;               // [n_cand]
  int32_t* hist;                   // [max_nkv + 1]
};

struct GemmListArgs {
  const uint8_t* sparse_info;
  const int32_t* info_indptr;
  int64_t info_bytes;
  int batch, m, n, k, num_heads, head_begin, head_dim, sparse_q_size, num_text_tokens;
  int is_full, is_for_cache;
  int32_t* tiles;                  // GEMM-Q: [max_tiles, 4] pair records (b, iy, ix0, ix1)
  int max_tiles;
  int n_ctas;                      // CTAs of the GEMM launch that will draw the records (GEMM-Q list rule)
  int32_t* row_indptr;             // GEMM-O: [rows + 1]
  int32_t* row_heads;              // GEMM-O: [rows * local_heads]
  int32_t* row_order;              // GEMM-O: [rows]
  int32_t* counters;               // [4]
};

cudaError_t launch_packbits(const uint8_t* x, int64_t n, int little, uint8_t* y, cudaStream_t stream);
cudaError_t launch_segment_packbits(const uint8_t* x, const int32_t* indptr, const int32_t* new_indptr,
                                    int num_segments, int64_t out_bytes, int little, uint8_t* y,
                                    cudaStream_t stream);
cudaError_t launch_attn_compact(const CompactArgs& a, cudaStream_t stream);

struct UnitArgs {
  const int32_t* items;      // [max_items, 4] as written by the compaction
  const int32_t* kv_ptr;     // [max_items + 1]
  const int32_t* kv_idx;
  const int32_t* order;      // [max_items]
  const int32_t* counters;   // the compaction's counters (n_items, total_kept, status, max_nkv)
  const int32_t* qo_indptr;
  const int32_t* kv_indptr;
  int64_t max_items, max_units, max_slots;
  int min_items, num_streams, min_chunk, max_nkv, sbq, sbkv;
  int32_t* units;            // [max_units, 8]
  int32_t* unit_counters;    // [4]: n_units, partial slots in use, chunk_max, status
  int32_t* arrive;           // [max_slots]
};
cudaError_t launch_attn_units(const UnitArgs& a, cudaStream_t stream);
cudaError_t launch_cast_fp8(const void* src, int64_t n, int e5m2, int is_bf16, void* dst, int sm_count, cudaStream_t stream);
cudaError_t launch_gemm_q_tiles(const GemmListArgs& a, cudaStream_t stream);
cudaError_t launch_gemm_o_rows(const GemmListArgs& a, cudaStream_t stream);

// ------------------------------------------------------------------ GEMM
enum GemmMode : int { kGemmQ = 0, kGemmO = 1 };
enum GemmInit : int { kInitNone = 0, kInitBias1D = 1, kInitFull = 2 };

struct GemmArgs {
  CUtensorMap tmap_a;              // X as [batch*m, k], box 64 x 128, 128B swizzle
  CUtensorMap tmap_b;              // W as [n, k],       box 64 x 128, 128B swizzle
  CUtensorMap tmap_y;              // Y as [batch*m, n], box 64 x 128, 128B swizzle (TMA stores)
  CUtensorMap tmap_b64;            // W with a box of 64 x 64 (the 192-column tiles of gemm_tall.cu)
  void* y;                         // [batch, m, n]
  const void* init;                // bias [n] or cache [batch, m, n] or null
  int init_mode;
  int mode;
  int is_bf16;
  int batch, m, n, k;
  int kb_per_head;                 // GEMM-O: head_dim / 64
  const int32_t* tiles;            // GEMM-Q pair records (b, iy, ix0, ix1); null = every tile (dense)
  const int32_t* n_tiles_ptr;      // device count of GEMM-Q tiles
  const int32_t* row_indptr;       // GEMM-O lists
  const int32_t* row_heads;
  const int32_t* row_order;
  int32_t* status;                 // device status word (DevStatus)
  int32_t* cursor;                 // device-wide tile cursor, zero when the kernel starts
};
cudaError_t launch_gemm(const GemmArgs& a, int max_ctas, cudaStream_t stream);
// dense projections whose shape divides into 256x256 tiles take the tall-tile kernel (gemm_tall.cu)
bool gemm_tall_applies(const GemmArgs& a, int sm_count);
int tall_tile_cols(const GemmArgs& a, int sm_count);   // 256, 192 or 0 (not applicable)
cudaError_t launch_gemm_tall(const GemmArgs& a, int max_ctas, cudaStream_t stream);

// ------------------------------------------------------------------ block selection
struct SelectArgs {
  const float* score;        // [batch, heads, n, n]
  const float* q_thr;        // [batch]
  const float* kv_thr;       // [heads]
  int batch, heads, n, t2t, zero_inactive;
  int64_t info_seg_bytes;    // ceil(n * heads / 8)
  int64_t kv_seg_bytes;      // ceil(n * heads * n / 8)
  int64_t kv_words;          // 32-bit words of sparse_kv_info that are zeroed first
  uint8_t* sparse_info;
  uint8_t* sparse_kv_info;
  int32_t* info_indptr;      // [batch + 1]
  int32_t* kv_info_indptr;   // [batch + 1]
  float* t2i;                // scratch [batch, n]
  uint8_t* q_keep;           // scratch [batch, n]
};
cudaError_t launch_select_blocks(const SelectArgs& a, cudaStream_t stream);

// ------------------------------------------------------------------ strided gather (exchange)
constexpr int kMaxGatherSources = 16;
struct GatherArgs {
  const uint8_t* src[kMaxGatherSources];
  uint8_t* dst[kMaxGatherSources];
  int64_t src_stride[kMaxGatherSources];   // bytes between rows
  int64_t dst_stride[kMaxGatherSources];
  int64_t vec_prefix[kMaxGatherSources + 1];  // exclusive prefix of rows * row_vecs
  int64_t row_vecs;                         // 16-byte vectors per row
  int n_src;
};
cudaError_t launch_strided_gather(const GatherArgs& a, int sm_count, cudaStream_t stream);

struct ReduceArgs {
  const uint8_t* src[kMaxGatherSources];   // partial results (peer pointers allowed), rows src_stride bytes apart
  const uint8_t* init;                      // optional addend (local), rows init_stride bytes apart
  uint8_t* dst;
  int64_t src_stride, init_stride, dst_stride;
  int64_t rows, row_vecs;                   // 16-byte vectors per row
  int n_src;
};
cudaError_t launch_reduce_rows(const ReduceArgs& a, int is_bf16, int sm_count, cudaStream_t stream);

constexpr int kMaxBarrierRanks = 64;
struct BarrierArgs {
  int* pads[kMaxBarrierRanks];   // every rank's flag pad as mapped into this process: int32 [channels][world]
  int* epoch;                    // this GPU's own epoch counters: int32 [channels]
  int* status;                   // device status word
  int rank, world, channel;
  uint64_t timeout_ns;
};
cudaError_t launch_peer_barrier(const BarrierArgs& a, cudaStream_t stream);

// ------------------------------------------------------------------ attention
struct AttnArgs {
  CUtensorMap tmap_q;              // [D, H, Tq]   box 64 x 1 x 128
  CUtensorMap tmap_k;              // [D, Hkv, Tkv]
  CUtensorMap tmap_v;
  CUtensorMap tmap_o;              // [D, Hq, Tq]   box 64 x 1 x 128, 128B swizzle (stores of whole q-blocks, two-stream kernel)
  CUtensorMap tmap_o16;            // [D, Hq, Tq]   box 32 x 1 x 16, no swizzle (stores of whole q-blocks, one-tile kernel)
  void* o;                         // [Tq, H, D] (strides below, in elements)
  float* lse;                      // [Tq, H] or null
  int64_t o_stride_n, o_stride_h;
  int64_t lse_stride_n;
  const int32_t* kv_idx;           // kept kv-block indices; unit records point into it
  const int32_t* units;            // 8 words per unit (see attn_units_kernel), processing order
  const int32_t* unit_counters;    // n_units, partial slots in use, chunk_max, status
  int max_units;                   // capacity of the unit list
  int32_t* arrive;                 // per partial slot (a split item counts at its first slot): parts delivered; zero between launches
  float* partials;                 // partial results of split items: partial_slots x kPartialFloats floats
  int partial_slots;
  int head_dim;                    // 128 or 64
  int mask_mode;                   // 0: none; 1: causal (kv position <= q token + kv_len - q_len); 2: custom bit mask
  const uint8_t* custom_mask;      // mode 2: per request a [q_len, kv_len] bit matrix, row-major, little-endian bits
  int64_t custom_mask_bytes;
  const int32_t* mask_indptr;      // mode 2: byte offset of each request's matrix [batch + 1]
  const int32_t* qo_indptr;        // mode 2: request rows and lengths
  const int32_t* kv_indptr;
  int head_begin;                  // tensor head = item head - head_begin
  int group_size;                  // H / Hkv
  int is_bf16;
  float sm_scale_log2;             // sm_scale * log2(e); with a soft cap: cap * log2(e)
  float soft_cap_pre;              // 0: no soft cap; else sm_scale / cap (logits = cap * tanh(q.k * sm_scale / cap))
  int32_t* status;
};
// floats of one partial result: O (32 column groups x 128 rows x 4), then the row maxima and the row sums
constexpr int kPartialFloats = 128 * 128 + 2 * 128;
// one unit at a time per SM (launches with many units) / two streams of units per SM with split kv lists (few units)
cudaError_t launch_attention(const AttnArgs& a, int max_ctas, cudaStream_t stream);

// ------------------------------------------------------------------ host helpers
// Encodes a tiled tensor map (bf16/f16 elements, 128-byte swizzle or none). dims/strides innermost first;
// strides in bytes for dims 1..rank-1. Returns 0 on success.
int encode_tmap_16bit(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128 = true);

}  // namespace fo
