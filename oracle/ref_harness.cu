// Test infrastructure: a C-ABI harness around the REFERENCE's own CUDA kernels, compiled from the
// reference headers where they lie (never copied into this repository), so that the kernels of this
// project can be compared with them on a GPU and timed beside them.
//
// Entry points call, unchanged:
//   flashomni::BatchSparseFAWithRaggedKVDispatched  (include/flashomni/attention/prefill.cuh:1535-1636)
//   flashomni::FLASHOMNIGEMMRun                     (include/flashomni/gemm/w16a16/gemm.cuh:230-357)
//   flashomni::FLASHOMNIGEMMReductionRun            (include/flashomni/gemm/w16a16/gemm_reduction.cuh:278-406)
//   flashomni::quantization::SegmentPackBits        (include/flashomni/quantization.cuh:97-109)
// The reference's torch bindings (csrc/*.cu) are not used: they need generated headers. The work-list
// arrays of its planner (request / q-tile / kv-tile indices, o_indptr, kv_chunk_size) are passed in by
// the caller for the un-split case, which is the only case the benchmark shapes reach
// (include/flashomni/attention/scheduler.cuh:35-64,264-271).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include <flashomni/attention/default_sparseFA_params.cuh>
#include <flashomni/attention/prefill.cuh>
#include <flashomni/attention/variants.cuh>
#include <flashomni/gemm/w16a16/gemm.cuh>
#include <flashomni/gemm/w16a16/gemm_reduction.cuh>
#include <flashomni/quantization.cuh>

using namespace flashomni;

// TQ: the kernel's q tile (CTA_TILE_Q). The reference has no 128-row configuration for head dimension 256
// (prefill.cuh:1601 rejects it), so that one runs with 64-row tiles, as the reference's own dispatch would.
template <typename T, int HD, MaskMode MM = MaskMode::kNone, int TQ = 128>
static int run_attn(uint8_t* custom_mask, int32_t* mask_indptr, void* q, void* k, void* v, void* o, float* lse, uint8_t* sparse_info, uint8_t* sparse_kv_info,
                    int32_t* info_indptr, int32_t* kv_info_indptr, int32_t* q_indptr, int32_t* kv_indptr,
                    int32_t* request_indices, int32_t* qo_tile_indices, int32_t* kv_tile_indices, int32_t* o_indptr,
                    int32_t* kv_chunk_size_ptr, uint32_t padded_batch, uint32_t num_qo_heads, uint32_t num_kv_heads,
                    uint32_t q_stride_n, uint32_t q_stride_h, uint32_t k_stride_n, uint32_t k_stride_h,
                    uint32_t v_stride_n, uint32_t v_stride_h, float sm_scale, int is_full, uint32_t max_rows,
                    cudaStream_t stream) {
  using Params = BatchRaggedSparseFAParams<T, T, T, int32_t>;
  using Variant = DefaultAttention</*use_custom_mask=*/MM == MaskMode::kCustom, /*use_logits_soft_cap=*/false, /*use_alibi=*/false>;
  Params p;
  p.q = static_cast<T*>(q);
  p.k = static_cast<T*>(k);
  p.v = static_cast<T*>(v);
  p.o = static_cast<T*>(o);
  p.lse = lse;
  p.maybe_custom_mask = custom_mask;
  p.maybe_mask_indptr = mask_indptr;
  p.sparse_info = sparse_info;
  p.sparse_kv_info = sparse_kv_info;
  p.sparse_info_indptr = info_indptr;
  p.sparse_kv_info_indptr = kv_info_indptr;
  p.sparse_block_size_for_q = 128;
  p.sparse_block_size_for_kv = 128;
  p.is_full = is_full != 0;
  p.q_indptr = q_indptr;
  p.kv_indptr = kv_indptr;
  p.group_size = uint_fastdiv(num_qo_heads / num_kv_heads);
  p.num_qo_heads = num_qo_heads;
  p.num_kv_heads = num_kv_heads;
  p.q_stride_n = q_stride_n;
  p.q_stride_h = q_stride_h;
  p.k_stride_n = k_stride_n;
  p.k_stride_h = k_stride_h;
  p.v_stride_n = v_stride_n;
  p.v_stride_h = v_stride_h;
  p.logits_soft_cap = 0.f;
  p.sm_scale = sm_scale;
  p.rope_rcp_scale = 1.f;
  p.rope_rcp_theta = 1e-4f;
  p.request_indices = request_indices;
  p.qo_tile_indices = qo_tile_indices;
  p.kv_tile_indices = kv_tile_indices;
  p.merge_indptr = nullptr;
  p.o_indptr = o_indptr;
  p.kv_chunk_size_ptr = kv_chunk_size_ptr;
  p.block_valid_mask = nullptr;
  p.max_total_num_rows = max_rows;
  p.total_num_rows = nullptr;
  p.padded_batch_size = padded_batch;
  p.partition_kv = false;
  cudaError_t e = BatchSparseFAWithRaggedKVDispatched<TQ, HD, HD, PosEncodingMode::kNone, false, MM,
                                                      Variant, Params>(p, nullptr, nullptr, stream);
  return static_cast<int>(e);
}

extern "C" {

__attribute__((visibility("default"))) int ref_sparse_attn(
    void* q, void* k, void* v, void* o, float* lse, uint8_t* sparse_info, uint8_t* sparse_kv_info,
    int32_t* info_indptr, int32_t* kv_info_indptr, int32_t* q_indptr, int32_t* kv_indptr, int32_t* request_indices,
    int32_t* qo_tile_indices, int32_t* kv_tile_indices, int32_t* o_indptr, int32_t* kv_chunk_size_ptr,
    uint32_t padded_batch, uint32_t num_qo_heads, uint32_t num_kv_heads, uint32_t q_stride_n, uint32_t q_stride_h,
    uint32_t k_stride_n, uint32_t k_stride_h, uint32_t v_stride_n, uint32_t v_stride_h, float sm_scale, int is_full,
    uint32_t max_rows, int is_bf16, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    return run_attn<nv_bfloat16, 128>(nullptr, nullptr, q, k, v, o, lse, sparse_info, sparse_kv_info, info_indptr, kv_info_indptr, q_indptr,
                                 kv_indptr, request_indices, qo_tile_indices, kv_tile_indices, o_indptr,
                                 kv_chunk_size_ptr, padded_batch, num_qo_heads, num_kv_heads, q_stride_n, q_stride_h,
                                 k_stride_n, k_stride_h, v_stride_n, v_stride_h, sm_scale, is_full, max_rows, st);
  return run_attn<half, 128>(nullptr, nullptr, q, k, v, o, lse, sparse_info, sparse_kv_info, info_indptr, kv_info_indptr, q_indptr, kv_indptr,
                        request_indices, qo_tile_indices, kv_tile_indices, o_indptr, kv_chunk_size_ptr, padded_batch,
                        num_qo_heads, num_kv_heads, q_stride_n, q_stride_h, k_stride_n, k_stride_h, v_stride_n,
                        v_stride_h, sm_scale, is_full, max_rows, st);
}

// The same with head dimension 64 (one of the reference's AOT head dimensions, setup.py:30).
__attribute__((visibility("default"))) int ref_sparse_attn_hd64(
    void* q, void* k, void* v, void* o, float* lse, uint8_t* sparse_info, uint8_t* sparse_kv_info,
    int32_t* info_indptr, int32_t* kv_info_indptr, int32_t* q_indptr, int32_t* kv_indptr, int32_t* request_indices,
    int32_t* qo_tile_indices, int32_t* kv_tile_indices, int32_t* o_indptr, int32_t* kv_chunk_size_ptr,
    uint32_t padded_batch, uint32_t num_qo_heads, uint32_t num_kv_heads, uint32_t q_stride_n, uint32_t q_stride_h,
    uint32_t k_stride_n, uint32_t k_stride_h, uint32_t v_stride_n, uint32_t v_stride_h, float sm_scale, int is_full,
    uint32_t max_rows, int is_bf16, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    return run_attn<nv_bfloat16, 64>(nullptr, nullptr, q, k, v, o, lse, sparse_info, sparse_kv_info, info_indptr, kv_info_indptr, q_indptr,
                                 kv_indptr, request_indices, qo_tile_indices, kv_tile_indices, o_indptr,
                                 kv_chunk_size_ptr, padded_batch, num_qo_heads, num_kv_heads, q_stride_n, q_stride_h,
                                 k_stride_n, k_stride_h, v_stride_n, v_stride_h, sm_scale, is_full, max_rows, st);
  return run_attn<half, 64>(nullptr, nullptr, q, k, v, o, lse, sparse_info, sparse_kv_info, info_indptr, kv_info_indptr, q_indptr, kv_indptr,
                        request_indices, qo_tile_indices, kv_tile_indices, o_indptr, kv_chunk_size_ptr, padded_batch,
                        num_qo_heads, num_kv_heads, q_stride_n, q_stride_h, k_stride_n, k_stride_h, v_stride_n,
                        v_stride_h, sm_scale, is_full, max_rows, st);
}

// The same with head dimension 256 (one of the reference's AOT head dimensions, setup.py:30), q tiles of 64 rows.
__attribute__((visibility("default"))) int ref_sparse_attn_hd256(
    void* q, void* k, void* v, void* o, float* lse, uint8_t* sparse_info, uint8_t* sparse_kv_info,
    int32_t* info_indptr, int32_t* kv_info_indptr, int32_t* q_indptr, int32_t* kv_indptr, int32_t* request_indices,
    int32_t* qo_tile_indices, int32_t* kv_tile_indices, int32_t* o_indptr, int32_t* kv_chunk_size_ptr,
    uint32_t padded_batch, uint32_t num_qo_heads, uint32_t num_kv_heads, uint32_t q_stride_n, uint32_t q_stride_h,
    uint32_t k_stride_n, uint32_t k_stride_h, uint32_t v_stride_n, uint32_t v_stride_h, float sm_scale, int is_full,
    uint32_t max_rows, int is_bf16, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    return run_attn<nv_bfloat16, 256, MaskMode::kNone, 64>(nullptr, nullptr, q, k, v, o, lse, sparse_info, sparse_kv_info, info_indptr, kv_info_indptr, q_indptr,
                                 kv_indptr, request_indices, qo_tile_indices, kv_tile_indices, o_indptr,
                                 kv_chunk_size_ptr, padded_batch, num_qo_heads, num_kv_heads, q_stride_n, q_stride_h,
                                 k_stride_n, k_stride_h, v_stride_n, v_stride_h, sm_scale, is_full, max_rows, st);
  return run_attn<half, 256, MaskMode::kNone, 64>(nullptr, nullptr, q, k, v, o, lse, sparse_info, sparse_kv_info, info_indptr, kv_info_indptr, q_indptr, kv_indptr,
                        request_indices, qo_tile_indices, kv_tile_indices, o_indptr, kv_chunk_size_ptr, padded_batch,
                        num_qo_heads, num_kv_heads, q_stride_n, q_stride_h, k_stride_n, k_stride_h, v_stride_n,
                        v_stride_h, sm_scale, is_full, max_rows, st);
}

// Head dimension 128 under the reference's causal mask mode (MaskMode::kCausal, prefill.cuh:746-751).
__attribute__((visibility("default"))) int ref_sparse_attn_causal(
    void* q, void* k, void* v, void* o, float* lse, uint8_t* sparse_info, uint8_t* sparse_kv_info,
    int32_t* info_indptr, int32_t* kv_info_indptr, int32_t* q_indptr, int32_t* kv_indptr, int32_t* request_indices,
    int32_t* qo_tile_indices, int32_t* kv_tile_indices, int32_t* o_indptr, int32_t* kv_chunk_size_ptr,
    uint32_t padded_batch, uint32_t num_qo_heads, uint32_t num_kv_heads, uint32_t q_stride_n, uint32_t q_stride_h,
    uint32_t k_stride_n, uint32_t k_stride_h, uint32_t v_stride_n, uint32_t v_stride_h, float sm_scale, int is_full,
    uint32_t max_rows, int is_bf16, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    return run_attn<nv_bfloat16, 128, MaskMode::kCausal>(nullptr, nullptr, q, k, v, o, lse, sparse_info, sparse_kv_info, info_indptr, kv_info_indptr, q_indptr,
                                 kv_indptr, request_indices, qo_tile_indices, kv_tile_indices, o_indptr,
                                 kv_chunk_size_ptr, padded_batch, num_qo_heads, num_kv_heads, q_stride_n, q_stride_h,
                                 k_stride_n, k_stride_h, v_stride_n, v_stride_h, sm_scale, is_full, max_rows, st);
  return run_attn<half, 128, MaskMode::kCausal>(nullptr, nullptr, q, k, v, o, lse, sparse_info, sparse_kv_info, info_indptr, kv_info_indptr, q_indptr, kv_indptr,
                        request_indices, qo_tile_indices, kv_tile_indices, o_indptr, kv_chunk_size_ptr, padded_batch,
                        num_qo_heads, num_kv_heads, q_stride_n, q_stride_h, k_stride_n, k_stride_h, v_stride_n,
                        v_stride_h, sm_scale, is_full, max_rows, st);
}

// Head dimension 128 under the reference's custom mask mode (MaskMode::kCustom, variants.cuh:76-87).
__attribute__((visibility("default"))) int ref_sparse_attn_custom(
    uint8_t* custom_mask, int32_t* mask_indptr, void* q, void* k, void* v, void* o, float* lse, uint8_t* sparse_info, uint8_t* sparse_kv_info,
    int32_t* info_indptr, int32_t* kv_info_indptr, int32_t* q_indptr, int32_t* kv_indptr, int32_t* request_indices,
    int32_t* qo_tile_indices, int32_t* kv_tile_indices, int32_t* o_indptr, int32_t* kv_chunk_size_ptr,
    uint32_t padded_batch, uint32_t num_qo_heads, uint32_t num_kv_heads, uint32_t q_stride_n, uint32_t q_stride_h,
    uint32_t k_stride_n, uint32_t k_stride_h, uint32_t v_stride_n, uint32_t v_stride_h, float sm_scale, int is_full,
    uint32_t max_rows, int is_bf16, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    return run_attn<nv_bfloat16, 128, MaskMode::kCustom>(custom_mask, mask_indptr, q, k, v, o, lse, sparse_info, sparse_kv_info, info_indptr, kv_info_indptr, q_indptr,
                                 kv_indptr, request_indices, qo_tile_indices, kv_tile_indices, o_indptr,
                                 kv_chunk_size_ptr, padded_batch, num_qo_heads, num_kv_heads, q_stride_n, q_stride_h,
                                 k_stride_n, k_stride_h, v_stride_n, v_stride_h, sm_scale, is_full, max_rows, st);
  return run_attn<half, 128, MaskMode::kCustom>(custom_mask, mask_indptr, q, k, v, o, lse, sparse_info, sparse_kv_info, info_indptr, kv_info_indptr, q_indptr, kv_indptr,
                        request_indices, qo_tile_indices, kv_tile_indices, o_indptr, kv_chunk_size_ptr, padded_batch,
                        num_qo_heads, num_kv_heads, q_stride_n, q_stride_h, k_stride_n, k_stride_h, v_stride_n,
                        v_stride_h, sm_scale, is_full, max_rows, st);
}

__attribute__((visibility("default"))) int ref_gemm_q(void* x, void* w, void* y, void* bias, uint32_t batch, uint32_t m,
                                                      uint32_t n, uint32_t k, uint32_t sparse_q_size,
                                                      uint32_t num_heads, uint32_t head_dim, uint8_t* sparse_info,
                                                      uint32_t* info_indptr, uint32_t num_text_tokens, int is_full,
                                                      int is_bf16, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    return static_cast<int>(flashomni::gemm::FLASHOMNIGEMMRun<cute::bfloat16_t>(
        static_cast<cute::bfloat16_t*>(x), static_cast<cute::bfloat16_t*>(w), static_cast<cute::bfloat16_t*>(y),
        static_cast<cute::bfloat16_t*>(bias), m, n, k, sparse_q_size, batch, num_heads, head_dim, sparse_info,
        info_indptr, num_text_tokens, is_full != 0, st));
  return static_cast<int>(flashomni::gemm::FLASHOMNIGEMMRun<cute::half_t>(
      static_cast<cute::half_t*>(x), static_cast<cute::half_t*>(w), static_cast<cute::half_t*>(y),
      static_cast<cute::half_t*>(bias), m, n, k, sparse_q_size, batch, num_heads, head_dim, sparse_info, info_indptr,
      num_text_tokens, is_full != 0, st));
}

__attribute__((visibility("default"))) int ref_gemm_o(void* x, void* w, void* y, void* bias, uint32_t batch, uint32_t m,
                                                      uint32_t n, uint32_t k, uint32_t sparse_q_size,
                                                      uint32_t num_heads, uint32_t head_dim, uint8_t* sparse_info,
                                                      uint32_t* info_indptr, uint32_t num_text_tokens,
                                                      int is_for_cached, int is_bf16, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    return static_cast<int>(flashomni::gemm::FLASHOMNIGEMMReductionRun<cute::bfloat16_t>(
        static_cast<cute::bfloat16_t*>(x), static_cast<cute::bfloat16_t*>(w), static_cast<cute::bfloat16_t*>(y),
        static_cast<cute::bfloat16_t*>(bias), m, n, k, sparse_q_size, batch, num_heads, head_dim, sparse_info,
        info_indptr, num_text_tokens, is_for_cached != 0, st));
  return static_cast<int>(flashomni::gemm::FLASHOMNIGEMMReductionRun<cute::half_t>(
      static_cast<cute::half_t*>(x), static_cast<cute::half_t*>(w), static_cast<cute::half_t*>(y),
      static_cast<cute::half_t*>(bias), m, n, k, sparse_q_size, batch, num_heads, head_dim, sparse_info, info_indptr,
      num_text_tokens, is_for_cached != 0, st));
}

__attribute__((visibility("default"))) int ref_segment_packbits(uint8_t* x, int32_t* indptr, int32_t* new_indptr,
                                                                uint32_t batch, int little, uint8_t* y, void* stream) {
  return static_cast<int>(quantization::SegmentPackBits(
      reinterpret_cast<bool*>(x), y, indptr, new_indptr, batch,
      little ? quantization::BitOrder::kLittle : quantization::BitOrder::kBig, static_cast<cudaStream_t>(stream)));
}

}  // extern "C"
