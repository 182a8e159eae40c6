/*
 * flashomni_b200 -- C ABI of the B200 (sm_100a) sparse-DiT hot path.
 *
 * One entry point per native op that the reference binds under torch.ops.flashomni_kernels
 * (csrc/flashomni_ops.cu:20-68), plus the mask-compaction step that replaces the reference's
 * in-kernel bit scanning. Conventions:
 *   - plain pointers and sizes only; every pointer that is not marked "host" is a DEVICE pointer
 *     owned by the caller; nothing here allocates or frees device memory;
 *   - the caller selects the device (cudaSetDevice / a torch device guard) before the call;
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it and no call
 *     synchronises the device;
 *   - return value: FO_OK or an error code; fo_last_error() returns a thread-local message;
 *   - malformed device-side data (bad indptr, list overflow, a wait that ran out) never faults:
 *     the kernels record a code in the status word the call was given (see each function).
 *   - dtype: FO_DTYPE_F16 or FO_DTYPE_BF16 (inputs and outputs share it; accumulation is fp32).
 *   - state between calls lives in memory the CALLER hands in, never in the library: the attention status words
 *     (unit cursor, count of finished CTAs), `arrive` and `partials`, and the GEMM `workspace` (work list, tile
 *     cursor, status word) are read and written by the launch that gets them. Two launches that share any of them
 *     must be ordered on one stream (or by events); launches on different streams need their own copies. The
 *     Python layer keeps one such set per wrapper object and one GEMM workspace per (device, stream). The only
 *     memory the library owns is the static scratch of fo_gemm_q_static (one stream at a time, see there) and a
 *     per-thread host table of encoded tensor maps.
 *
 * Bit layout of the packed masks (reference: include/flashomni/attention/prefill.cuh:1284-1294,
 * 1385-1394; include/flashomni/gemm/w16a16/gemm.cuh:50-58): request b's segment starts at byte
 * indptr[b]; q-block bit = qb*H + h; kv-block bit = (qb*H + h)*nkv + kvb; bit i = (seg[i>>3] >> (i&7)) & 1.
 * With grouped heads (Hq > Hkv) the attention reads the masks as the reference's kernel does
 * (prefill.cuh:1283-1291): H = Hkv, and a q-block is 128 PACKED rows, a packed row being a (token, q head of the
 * group) pair in token-major order, i.e. 128 / group tokens of all the q heads that share kv head h.
 */
#ifndef FLASHOMNI_B200_H_
#define FLASHOMNI_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FO_ABI_VERSION 2

#if defined(__GNUC__)
#define FO_API __attribute__((visibility("default")))
#else
#define FO_API
#endif

enum {
  FO_OK = 0,
  FO_ERR_INVALID_ARG = 1,  /* null / misaligned / inconsistent argument (the reference TORCH_CHECKs) */
  FO_ERR_UNSUPPORTED = 2,  /* shape or dtype outside what this build implements */
  FO_ERR_CUDA = 3,         /* a CUDA runtime / driver call failed; message has the CUDA error string */
  FO_ERR_WORKSPACE = 4     /* workspace / scratch too small */
};
enum { FO_DTYPE_F16 = 0, FO_DTYPE_BF16 = 1 };

/* Device status codes (written into status words by the kernels). */
enum { FO_DEV_OK = 0, FO_DEV_WAIT_TIMEOUT = 1, FO_DEV_BAD_INDEX = 2 };

/* Thread-local description of the last error returned on this thread ("" if none). */
FO_API const char* fo_last_error(void);
FO_API int fo_abi_version(void);
/* Number of kernels this library has launched (or recorded into a stream capture) in this process so far.
 * Host-side bookkeeping for benchmarks that report their launch counts; no device call. */
FO_API long long fo_launch_count(void);

/* ---- mask packing -------------------------------------------------------------------------
 * Replaces torch.ops.flashomni_kernels.packbits / segment_packbits (csrc/flashomni_ops.cu:46-51,
 * csrc/quantization.cu:24-57; kernels include/flashomni/quantization.cuh:39-109).
 * x: n bytes, non-zero = 1. y: (n+7)/8 bytes. little != 0 selects bitorder="little". */
FO_API int fo_packbits(const uint8_t* x, int64_t n, int little, uint8_t* y, void* stream);
/* indptr / new_indptr: int32 [num_segments+1] (element and byte offsets); out_bytes = new_indptr[-1]
 * as known to the host (flashomni/quantization.py:148-152). */
FO_API int fo_segment_packbits(const uint8_t* x, const int32_t* indptr, const int32_t* new_indptr,
                        int32_t num_segments, int64_t out_bytes, int little, uint8_t* y, void* stream);

/* ---- attention mask compaction (new step; no counterpart op in the reference, which re-reads
 * the bits in the kernel: prefill.cuh:1284-1294,1380-1460) -------------------------------------
 * Turns the packed masks into work lists, restricted to heads [head_begin, head_begin+head_count):
 *   items   int32 [max_items,4]  (b, h, qb, n_kept) of every active q-block, ascending (b, qb, h)
 *   kv_ptr  int32 [max_items+1]  offsets into kv_idx
 *   kv_idx  int32 [max_kept]     ascending kept kv-block indices per item
 *   order   int32 [max_items]    the processing order: item indices grouped by (b, group of heads), a group
 *                                being as many consecutive heads as keep K and V in L2 together (48 MiB /
 *                                (max_nkv * 64 KiB), evened out); inside a group by descending n_kept (ties:
 *                                list order) while batch * groups * (max_nkv + 1) <= 8192, else single-head
 *                                groups, q-blocks ascending
 *   counters int32 [4]           n_items, total_kept, status (FO_DEV_*), max_nkv
 * n_cand = sum over requests of ceil(qo_len/sbq)*head_count and max_nkv = max ceil(kv_len/sbkv) are
 * host-known (plan time). is_full != 0 ignores the masks (they may be null). scratch must hold
 * fo_mask_compact_scratch_bytes(n_cand, max_nkv) bytes. */
FO_API size_t fo_mask_compact_scratch_bytes(int64_t n_cand, int32_t max_nkv);
FO_API int fo_mask_compact(const uint8_t* sparse_info, int64_t sparse_info_bytes, const uint8_t* sparse_kv_info,
                    int64_t sparse_kv_info_bytes, const int32_t* sparse_info_indptr,
                    const int32_t* sparse_kv_info_indptr, const int32_t* qo_indptr, const int32_t* kv_indptr,
                    int32_t batch, int32_t num_heads, int32_t head_begin, int32_t head_count, int32_t sbq,
                    int32_t sbkv, int32_t is_full, int64_t n_cand, int32_t max_nkv, int64_t max_items,
                    int64_t max_kept, int32_t* items, int32_t* kv_ptr, int32_t* kv_idx, int32_t* order,
                    int32_t* counters, void* scratch, size_t scratch_bytes, void* stream);

/* ---- attention work units (no counterpart op in the reference; its planner chunks kv ranges on the host,
 * include/flashomni/attention/scheduler.cuh:35-64, and merges with attention/cascade.cuh:346-437) -----------
 * Turns the compaction's lists into the unit list the attention kernel walks, in processing order: one
 * self-contained record of eight int32 per unit,
 *   [0] n         kv blocks of the unit (0: an active q-block that keeps nothing)
 *   [1] kv_off    offset of the unit's first entry in kv_idx
 *   [2] h | b << 16   mask head (< 65536) and request (< 32768)
 *   [3] q_row0    first row of the q-block in the q / o tensors
 *   [4] q_valid | ragged << 16   rows of the q-block that exist (1..sbq); columns of the request's partial last kv
 *                 block if the unit's list ends with it, else 0
 *   [5] kv_row0   first kv row of the request
 *   [6] causal    qb * sbq + kv_len - q_len: the last kv position the q-block's first token sees under a causal mask
 *   [7] slot << 16 | part << 8 | n_parts   (a whole item: n_parts = 1, slot = 0xffff)
 * An item is one unit unless its kv list is cut: lists are cut only when max_slots > 0 and the launch has more than
 * min_items and at most num_streams items (num_streams: the unit count the caller aims at, a few per SM; min_items:
 * the number of SMs, or 0: with at most one item per SM, cutting measured slower on a power-capped part, since the
 * SMs that end early leave their share of the power to the long items), into n_parts = ceil(n_kept / chunk_max) parts of (almost) equal length, chunk_max =
 * max(min_chunk, ceil(total_kept / num_streams), ceil(max_nkv / 255)). Cuts fall between list ENTRIES, so no
 * part is ever empty and every part of a split item delivers a partial result before the merge (the reference's
 * split path cuts kv ranges and merges partials that an early-returning q-block never wrote). The parts of an item
 * use consecutive partial slots. When lists were cut (and the launch has at most 2048 units) the units are put in
 * descending order of their length (stable), so that the CTAs, which draw units in list order, take the short
 * ones last.
 *   units          int32 [max_units,8]  16-byte aligned
 *   unit_counters  int32 [4]            n_units, partial slots in use, chunk_max, status (FO_DEV_*)
 *   arrive         int32 [max_slots]    per slot: parts delivered (a split item counts at its first slot); zeroed
 *                                       here, and put back to zero by the kernel
 * max_units >= max_items + num_streams and max_slots >= num_streams + num_streams / 2 always suffice. */
FO_API int fo_attn_units(const int32_t* items, const int32_t* kv_ptr, const int32_t* kv_idx, const int32_t* order,
                         const int32_t* counters, const int32_t* qo_indptr, const int32_t* kv_indptr,
                         int64_t max_items, int32_t max_nkv, int32_t sbq, int32_t sbkv, int32_t min_items,
                         int32_t num_streams, int32_t min_chunk, int64_t max_units, int64_t max_slots, int32_t* units,
                         int32_t* unit_counters, int32_t* arrive, void* stream);
/* Bytes of partial-result scratch for `partial_slots` slots (fp32 O of a 128-row q-block plus row maxima and sums). */
FO_API size_t fo_attn_partial_bytes(int64_t partial_slots);

/* ---- block-sparse attention ------------------------------------------------------------------
 * Replaces torch.ops.flashomni_kernels.batch_sparseFA_with_ragged_kv_run
 * (csrc/batch_sparseFA.cu:67-201 -> include/flashomni/attention/prefill.cuh:1203-1636), consuming kv_idx of
 * fo_mask_compact and the units of fo_attn_units. q [total_q, Hq, D], k/v [total_kv, Hkv, D],
 * o [total_q, Hq, D] with element strides (row, head); the innermost dimension is contiguous. lse (optional,
 * may be null): float32 [total_q, Hq], base 2. Hq / Hkv here are the numbers of heads IN THE TENSORS; unit heads
 * are mask heads and map to kv head (h - head_begin) of the tensors and its q heads (h - head_begin) * group + j.
 * With group = Hq / Hkv > 1 (1, 2, 4, 8 or 16) the units are built with fo_mask_compact / fo_attn_units given
 * head_count = Hkv and sbq = 128 / group tokens; a unit's q tile is then 128 / group tokens x group q heads.
 * q-blocks that are not listed are not written. The kernel walks min(unit_counters[0], max_units) units, and none at all when unit_counters[3]
 * is not FO_DEV_OK or more partial slots are in use than `partial_slots` (the output is then untouched and
 * status[0] = FO_DEV_BAD_INDEX). The parts of a split item write fp32 partial results into `partials`
 * (fo_attn_partial_bytes(partial_slots) bytes, 16-byte aligned; null when partial_slots = 0) and the
 * part that delivers last merges them and writes the rows. One persistent CTA per SM draws the units in list
 * order, one unit at a time, with two softmax groups on alternate kv blocks. status: FOUR int32 device words
 * that the caller zeroes once: [0] is set to FO_DEV_WAIT_TIMEOUT if a bounded wait ran out;
 * [1] (unit cursor: units are handed to the CTAs dynamically) and [2] (count of finished CTAs) are used by
 * the kernel and are zero again when it ends, so launches that share the words (or `arrive`, `partials`) must
 * not overlap; [3] is reserved.
 * This build implements D = 64, 128 and 256 with 128-row q and kv blocks (D = 256: whole items only,
 * partial_slots = 0). */
FO_API int fo_sparse_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int32_t dtype,
                       int64_t total_q, int64_t total_kv, int32_t num_qo_heads, int32_t num_kv_heads,
                       int32_t head_dim, int64_t q_stride_n, int64_t q_stride_h, int64_t k_stride_n,
                       int64_t k_stride_h, int64_t v_stride_n, int64_t v_stride_h, int64_t o_stride_n,
                       int64_t o_stride_h, int32_t sbq, int32_t sbkv, const int32_t* kv_idx,
                       const int32_t* units, const int32_t* unit_counters, int64_t max_units, int32_t* arrive,
                       float* partials, int64_t partial_slots, int32_t head_begin, float sm_scale,
                       int32_t* status, void* stream);

/* The same with the reference's logits soft cap (include/flashomni/attention/variants.cuh:47-50,72-74: the
 * logit of a (q, k) pair is cap * tanh(q.k * sm_scale / cap) before the softmax). logits_soft_cap = 0 is
 * fo_sparse_attn_fwd. */
FO_API int fo_sparse_attn_fwd_softcap(const void* q, const void* k, const void* v, void* o, float* lse, int32_t dtype,
                       int64_t total_q, int64_t total_kv, int32_t num_qo_heads, int32_t num_kv_heads,
                       int32_t head_dim, int64_t q_stride_n, int64_t q_stride_h, int64_t k_stride_n,
                       int64_t k_stride_h, int64_t v_stride_n, int64_t v_stride_h, int64_t o_stride_n,
                       int64_t o_stride_h, int32_t sbq, int32_t sbkv, const int32_t* kv_idx,
                       const int32_t* units, const int32_t* unit_counters, int64_t max_units, int32_t* arrive,
                       float* partials, int64_t partial_slots, int32_t head_begin, float sm_scale,
                       float logits_soft_cap, int32_t* status, void* stream);

/* The same under a causal mask (the reference's MaskMode::kCausal, include/flashomni/attention/prefill.cuh:746-751):
 * inside the kept kv-blocks, kv position j of a request is visible to q token i only if j <= i + kv_len - q_len
 * (positions and lengths of the request; with grouped heads i is the token of the packed row). The units carry
 * the position (word [6]); whole items only, so there is no partial-result scratch. A row whose kept blocks hold no
 * visible position gets zeros and lse = -5e4, like a q-block that keeps nothing (the reference fills masked logits
 * with -5e4 instead of -inf and would return the mean of V over those positions there). logits_soft_cap = 0: no cap. */
FO_API int fo_sparse_attn_fwd_causal(const void* q, const void* k, const void* v, void* o, float* lse, int32_t dtype,
                       int64_t total_q, int64_t total_kv, int32_t num_qo_heads, int32_t num_kv_heads,
                       int32_t head_dim, int64_t q_stride_n, int64_t q_stride_h, int64_t k_stride_n,
                       int64_t k_stride_h, int64_t v_stride_n, int64_t v_stride_h, int64_t o_stride_n,
                       int64_t o_stride_h, int32_t sbq, int32_t sbkv, const int32_t* kv_idx,
                       const int32_t* units, const int32_t* unit_counters, int64_t max_units, int32_t head_begin,
                       float sm_scale, float logits_soft_cap, int32_t* status, void* stream);

/* The same under a custom mask (the reference's MaskMode::kCustom with packed_custom_mask / mask_indptr,
 * flashomni/attention.py:524-533, include/flashomni/attention/variants.cuh:76-87): inside the kept kv-blocks,
 * position (i, j) of request b is visible iff bit i * kv_len_b + j of the request's matrix is set. custom_mask holds
 * the matrices bit-packed (little-endian bits, as segment_packbits packs them), request b's starting at byte
 * mask_indptr[b]; the same matrix serves all heads. qo_indptr / kv_indptr are the request indptrs of the plan. A row
 * without any visible position gets zeros and lse = -5e4. Whole items only. logits_soft_cap = 0: no cap. */
FO_API int fo_sparse_attn_fwd_custom_mask(const void* q, const void* k, const void* v, void* o, float* lse, int32_t dtype,
                       int64_t total_q, int64_t total_kv, int32_t num_qo_heads, int32_t num_kv_heads,
                       int32_t head_dim, int64_t q_stride_n, int64_t q_stride_h, int64_t k_stride_n,
                       int64_t k_stride_h, int64_t v_stride_n, int64_t v_stride_h, int64_t o_stride_n,
                       int64_t o_stride_h, int32_t sbq, int32_t sbkv, const int32_t* kv_idx,
                       const int32_t* units, const int32_t* unit_counters, int64_t max_units, int32_t head_begin,
                       float sm_scale, float logits_soft_cap, const uint8_t* custom_mask, int64_t custom_mask_bytes,
                       const int32_t* mask_indptr, const int32_t* qo_indptr, const int32_t* kv_indptr,
                       int32_t* status, void* stream);

/* K / V stored as 8-bit floats (the reference casts its fp8 K / V fragments to the type of Q before the MMA, no
 * scales: include/flashomni/attention/prefill.cuh:602-612): n contiguous values of fp8_kind 0 (e4m3) or 1 (e5m2)
 * are cast to dtype (exact: every fp8 value is representable in f16 and bf16) into dst; the attention then runs on
 * the 16-bit copy. src and dst 16-byte aligned. */
FO_API int fo_cast_fp8(const void* src, int64_t n, int32_t fp8_kind, int32_t dtype, void* dst, void* stream);

/* ---- GEMM-Q / GEMM-O ---------------------------------------------------------------------------
 * Workspace (device, caller-owned, 16-byte aligned) of fo_gemm_workspace_bytes(...) bytes, laid out
 * as int32 words: [0..3] counters (count, aux, list status, two-block records), [4] kernel status (FO_DEV_*,
 * cleared when a list is built, set when a bounded wait of a GEMM kernel ran out, otherwise left alone),
 * [5] tile cursor and [6] count of finished CTAs of the running GEMM kernel (both zero again when it ends),
 * [8...] the work list built from the mask. The caller zeroes the workspace once before its first use; launches
 * that share a workspace must not overlap. */
FO_API size_t fo_gemm_workspace_bytes(int32_t batch, int32_t m, int32_t n, int32_t k, int32_t head_dim);

/* Host-only query (no device call): the row count of the output tiles, 256 or 128, that a dense launch
 * (is_full) of fo_gemm_q uses for this shape on a device with sm_count SMs; 0 for an empty shape. Both
 * dense kernels deal equal tiles in fixed shares, so the choice goes to the shape whose fullest SM ends first
 * (rounds of tiles times the tile's length). has_full_init: the launch adds a [batch, m, n] tensor (not reachable through fo_gemm_q). */
FO_API int fo_gemm_dense_tile_rows(int32_t batch, int32_t m, int32_t n, int32_t k, int32_t has_full_init,
                                   int32_t sm_count);
/* The column count of those tiles: 256, or 192 where the 256-row kernel runs its narrower tiles (more, shorter
 * tiles for a narrow projection whose 256-column tiles would leave SMs idle). */
FO_API int fo_gemm_dense_tile_cols(int32_t batch, int32_t m, int32_t n, int32_t k, int32_t has_full_init,
                                   int32_t sm_count);

/* Replaces torch.ops.flashomni_kernels.flashomni_gemm (csrc/gemm.cu:24-59 ->
 * include/flashomni/gemm/w16a16/gemm.cuh:27-357). x [batch, m, k], w [n, k], y [batch, m, n], all
 * contiguous; bias [n] or null. Output tile (iy, ix) of batch b is computed iff is_full or bit
 * ((num_text_tokens + iy*128)/sparse_q_size)*num_heads + head_begin + (ix*128)/head_dim of b's
 * segment is 1; other tiles of y are left untouched. head_dim = n/num_heads in the reference
 * (pass that, with head_begin = 0, for the reference behaviour). m, n multiples of 128; k of 32 (the
 * reference's rule, csrc/gemm.cu:36). */
FO_API int fo_gemm_q(const void* x, const void* w, void* y, const void* bias, int32_t dtype, int32_t batch,
              int32_t m, int32_t n, int32_t k, int32_t num_heads, int32_t head_begin, int32_t head_dim,
              int32_t sparse_q_size, int32_t num_text_tokens, int32_t is_full, const uint8_t* sparse_info,
              int64_t sparse_info_bytes, const int32_t* sparse_info_indptr, void* workspace,
              size_t workspace_bytes, void* stream);

/* Replaces torch.ops.flashomni_kernels.flashomni_gemm_reduction (csrc/gemm_reduction.cu:24-57 ->
 * include/flashomni/gemm/w16a16/gemm_reduction.cuh:27-406). Every tile of y is written:
 * y = init + sum over selected heads h of x[:, :, h*head_dim:(h+1)*head_dim] w[:, same]^T, selected =
 * bit 1 (is_for_cache = 0) or bit 0 (is_for_cache != 0) of bit ((num_text_tokens + iy*128)/
 * sparse_q_size)*num_heads + head_begin + h. init: null, or bias [n] (init_is_full = 0), or the cached
 * tensor [batch, m, n] (init_is_full != 0). head_dim = n/num_heads in the reference; k/head_dim local
 * heads are visited. m, n multiples of 128; head_dim a multiple of 64. */
FO_API int fo_gemm_o(const void* x, const void* w, void* y, const void* init, int32_t init_is_full, int32_t dtype,
              int32_t batch, int32_t m, int32_t n, int32_t k, int32_t num_heads, int32_t head_begin,
              int32_t head_dim, int32_t sparse_q_size, int32_t num_text_tokens, int32_t is_for_cache,
              const uint8_t* sparse_info, int64_t sparse_info_bytes, const int32_t* sparse_info_indptr,
              void* workspace, size_t workspace_bytes, void* stream);

/* The list builders that fo_gemm_q / fo_gemm_o run first (exposed so that the lists can be checked
 * bit for bit). They fill the same workspace layout: GEMM-Q: words [8 + 4*i ..] = (b, iy, ix0, ix1), the
 * i-th pair record: per row block (b, iy), ascending, its active 128-column blocks taken two at a
 * time (ix1 = -1 for a leftover single block), all two-block records first, then the single-block ones; the
 * last k two-block records are cut into two single-block records each, k being the value in [0, min(P, SMs)]
 * (P two-block, S single-block records before the cut) for which the launch ends earliest when one CTA per SM
 * draws the records in list order at 20 time units per two-block and 13 per single-block tile (smallest k on a
 * tie; see oracle/masks.py gemm_q_split_rule); counters[0] = record count, counters[1] = active tile count,
 * counters[3] = two-block records. GEMM-O with R = batch*m/128 row blocks and
 * L = k/head_dim local heads: words [8 .. 8+R] row_indptr, then [8+R+1 ..] row_heads (R*L words
 * reserved), then row_order (R words): row blocks by descending list length (stable). */
FO_API int fo_gemm_q_worklist(int32_t batch, int32_t m, int32_t n, int32_t num_heads, int32_t head_begin,
                       int32_t head_dim, int32_t sparse_q_size, int32_t num_text_tokens, int32_t is_full,
                       const uint8_t* sparse_info, int64_t sparse_info_bytes,
                       const int32_t* sparse_info_indptr, void* workspace, size_t workspace_bytes,
                       void* stream);
FO_API int fo_gemm_o_worklist(int32_t batch, int32_t m, int32_t k, int32_t num_heads, int32_t head_begin,
                       int32_t head_dim, int32_t sparse_q_size, int32_t num_text_tokens,
                       int32_t is_for_cache, const uint8_t* sparse_info, int64_t sparse_info_bytes,
                       const int32_t* sparse_info_indptr, void* workspace, size_t workspace_bytes,
                       void* stream);

/* ---- GEMM-Q / GEMM-O over a work list built earlier -------------------------------------------------
 * No counterpart in the reference. Same computation as fo_gemm_q (sparse) / fo_gemm_o, but the work list is
 * taken from `workspace` as fo_gemm_q_worklist / fo_gemm_o_worklist left it (same batch, m, n / k, head_dim),
 * built on any stream that is ordered before this call -- e.g. a side stream, beside the dense projections,
 * since the list depends on the mask only. Nothing is reset here: a list may be used by any number of launches,
 * one after another. */
FO_API int32_t fo_gemm_q_prepared(const void* x, const void* w, void* y, const void* bias, int32_t dtype,
                                  int32_t batch, int32_t m, int32_t n, int32_t k, int32_t head_dim,
                                  void* workspace, size_t workspace_bytes, void* stream);
FO_API int32_t fo_gemm_o_prepared(const void* x, const void* w, void* y, const void* init, int32_t init_is_full,
                                  int32_t dtype, int32_t batch, int32_t m, int32_t n, int32_t k, int32_t head_dim,
                                  void* workspace, size_t workspace_bytes, void* stream);

/* ---- block selection: pooled scores -> packed masks ------------------------------------------------
 * Replaces the mask generation of benchmark/test_attn_score.py:93-133 (torch sum / softmax / sort / cumsum /
 * searchsorted + Triton fill kernels on an unpacked [B, H, nq, nkv] layout) and the transpose + bit-pack its
 * callers add (benchmark/utils.py:83-84). pooled_score is fp32 [batch, heads, n, n] (n q-blocks = n kv-blocks,
 * the first num_text_blocks are text). q_threshold [batch] and kv_threshold [heads] are device arrays.
 *   q-blocks: text-to-image scores summed over heads and text rows, softmax over the image blocks; the blocks
 *     taken in ascending (mass, index) order while the cumulative mass stays <= threshold are switched off for
 *     every head. Nothing is switched off when there are no text blocks.
 *   kv-blocks: per (b, h, image q-block) the row softmax over all kv-blocks, same rule with the head's
 *     threshold; text q rows keep everything. With zero_inactive the rows of switched-off q-blocks are zero.
 * Outputs: sparse_info (bit qb*H + h) and sparse_kv_info (bit (qb*H + h)*n + kvb), little-endian, one segment of
 * ceil(bits / 8) bytes per request, plus the two byte indptrs [batch + 1]: exactly what fo_mask_compact and the
 * GEMM entry points read. sparse_kv_info must be 4-byte aligned and hold the total rounded up to 4 bytes.
 * The arithmetic is fixed (see oracle/select.py): results are bit-identical to that statement. */
FO_API size_t fo_select_blocks_scratch_bytes(int32_t batch, int32_t num_blocks);
FO_API int32_t fo_select_blocks(const float* pooled_score, int32_t batch, int32_t num_heads, int32_t num_blocks,
                                int32_t num_text_blocks, const float* q_threshold, const float* kv_threshold,
                                int32_t zero_inactive, uint8_t* sparse_info, int64_t sparse_info_bytes,
                                uint8_t* sparse_kv_info, int64_t sparse_kv_info_bytes, int32_t* info_indptr,
                                int32_t* kv_info_indptr, void* scratch, size_t scratch_bytes, void* stream);

/* ---- strided row gather (sequence-parallel exchange) -----------------------------------------------
 * No counterpart in the reference (it has no multi-GPU code). For source i < n_src (at most 16), copies
 * n_rows[i] rows of row_bytes bytes from src[i] (rows src_row_stride_bytes[i] apart) to dst[i] (rows
 * dst_row_stride_bytes[i] apart), all in one launch. A source may be another GPU's buffer mapped into this
 * process (a peer pointer): the kernel reads it with plain loads over NVLink and writes into local memory,
 * which turns the all-to-all of a sequence-parallel attention block plus its two layout changes into one
 * pull per rank. Pointers, strides and row_bytes must be multiples of 16. The arrays are host arrays and
 * are read before the call returns. Ordering against the producers of the sources (on other GPUs) is the
 * caller's business. */
FO_API int32_t fo_strided_gather(int32_t n_src, const void* const* src, const int64_t* src_row_stride_bytes,
                                 const int64_t* n_rows, void* const* dst, const int64_t* dst_row_stride_bytes,
                                 int64_t row_bytes, void* stream);

/* ---- sum of partial results held by several GPUs ------------------------------------------------
 * No counterpart in the reference (it has no multi-GPU code). dst[r, :] = init[r, :] + sum_i src[i][r, :] for
 * n_rows rows of row_bytes bytes of 16-bit elements (fp32 accumulation, one rounding). The sources are the
 * partial outputs of a head-partitioned GEMM-O, one per GPU, all with the same row stride; a source may be a
 * peer pointer (plain loads over NVLink). Each GPU calls this for the row slice it owns (pass pointers that
 * already point at that slice), so the partials are summed where the result is wanted and each crosses the
 * link once. init may be null. Ordering against the producers on other GPUs is the caller's business
 * (fo_peer_barrier). Pointers, strides and row_bytes must be multiples of 16; at most 16 sources. */
FO_API int32_t fo_reduce_rows(int32_t n_src, const void* const* src, int64_t src_row_stride_bytes, const void* init,
                              int64_t init_row_stride_bytes, void* dst, int64_t dst_row_stride_bytes,
                              int64_t n_rows, int64_t row_bytes, int32_t dtype, void* stream);

/* ---- barrier between the GPUs of one job ---------------------------------------------------------
 * No counterpart in the reference. One launch per GPU, each on its own device and stream; the launch ends when
 * every rank's launch of the same (channel, epoch) has started, i.e. when everything each rank had enqueued
 * before its call is complete and visible to the others. pads[r] (host array of `world` device pointers) is
 * rank r's flag pad, int32 [num_channels][world], zeroed once before the first use and mapped into this
 * process (peer memory); epoch is this GPU's own int32 [num_channels] counter array, zeroed once; the kernel
 * advances it, so a launch replayed from a CUDA graph works. Ranks must call the channels in the same order.
 * The wait is bounded by timeout_ms: when a peer does not arrive the launch writes FO_DEV_WAIT_TIMEOUT to
 * *status (device word) and returns instead of trapping; the host reads the word before trusting the step. */
FO_API int32_t fo_peer_barrier(int32_t world, int32_t rank, int32_t* const* pads, int32_t channel,
                               int32_t num_channels, int32_t* epoch, int32_t* status, int64_t timeout_ms,
                               void* stream);

/* ---- GEMM-Q without a caller workspace ------------------------------------------------------------
 * No counterpart in the reference. Same arguments and result as fo_gemm_q minus the workspace: the
 * tile list, counters and status word live in a 1 MiB array that is part of the library image (one
 * copy per GPU that loads the library, kept until exit), so this path performs no device allocation
 * of any kind. It is meant for hosts that may not allocate when the op runs -- a server whose arena
 * owns all device memory, a plugin that must stay out of its framework's allocator, a latency-bound
 * loop that cannot risk the synchronisation an allocation can cause.
 * Problems whose fo_gemm_workspace_bytes(...) exceeds fo_gemm_q_static_max_bytes() are refused with
 * FO_ERR_WORKSPACE. The first call on a device looks up the array's device address; issue it before
 * starting any stream capture. All calls on a device share the array: do not let two of them overlap
 * on the GPU. Errors of this entry point are described by fo_gemm_q_static_last_error(); the kernel
 * status word is not readable by the caller (use fo_gemm_q where that matters). */
FO_API size_t fo_gemm_q_static_max_bytes(void);
FO_API const char* fo_gemm_q_static_last_error(void);
FO_API int fo_gemm_q_static(const void* x, const void* w, void* y, const void* bias, int32_t dtype, int32_t batch,
                     int32_t m, int32_t n, int32_t k, int32_t num_heads, int32_t head_begin, int32_t head_dim,
                     int32_t sparse_q_size, int32_t num_text_tokens, int32_t is_full,
                     const uint8_t* sparse_info, int64_t sparse_info_bytes, const int32_t* sparse_info_indptr,
                     void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASHOMNI_B200_H_ */
