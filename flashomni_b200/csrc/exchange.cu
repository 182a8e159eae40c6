// Strided row gather from several source buffers, some of which may be another GPU's memory mapped into
// this process (peer pointers): the data path of the sequence-parallel exchange. Every rank PULLS the
// slices it needs with plain 16-byte loads over NVLink and writes them, already in their final layout,
// into its own memory -- one kernel instead of a permute copy, a library all-to-all and a second permute.
// Only loads cross the link; nothing here waits on another GPU (the callers order the steps with their
// own barriers).
#include "internal.h"

namespace fo {
namespace {

__global__ void __launch_bounds__(256) strided_gather_kernel(const __grid_constant__ GatherArgs a) {
  const int64_t total = a.vec_prefix[a.n_src];
  const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    int s = 0;
#pragma unroll 1
    while (s + 1 < a.n_src && i >= a.vec_prefix[s + 1]) ++s;
    const int64_t local = i - a.vec_prefix[s];
    const int64_t row = local / a.row_vecs;
    const int64_t col = local - row * a.row_vecs;
    const uint4 v = *reinterpret_cast<const uint4*>(a.src[s] + row * a.src_stride[s] + col * 16);
    *reinterpret_cast<uint4*>(a.dst[s] + row * a.dst_stride[s] + col * 16) = v;
  }
}

}  // namespace

cudaError_t launch_strided_gather(const GatherArgs& a, int sm_count, cudaStream_t stream) {
  const int64_t total = a.vec_prefix[a.n_src];
  if (total <= 0) return cudaSuccess;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count) * 8;
  if (blocks > cap) blocks = cap;
  strided_gather_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace fo
