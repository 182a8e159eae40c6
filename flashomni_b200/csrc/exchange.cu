// Strided row gather from several source buffers, some of which may be another GPU's memory mapped into
// this process (peer pointers): the data path of the sequence-parallel exchange. Every rank PULLS the
// slices it needs with plain 16-byte loads over NVLink and writes them, already in their final layout,
// into its own memory -- one kernel instead of a permute copy, a library all-to-all and a second permute.
// Only loads cross the link; nothing here waits on another GPU (the callers order the steps with their
// own barriers).
#include "internal.h"

namespace fo {
namespace {

// grid (x, source): a warp copies whole rows (no index divisions), four rows per pass so that several loads
// are in flight per lane.
__global__ void __launch_bounds__(256) strided_gather_kernel(const __grid_constant__ GatherArgs a) {
  const int s = blockIdx.y;
  const int64_t rows = (a.vec_prefix[s + 1] - a.vec_prefix[s]) / a.row_vecs;
  const uint8_t* __restrict__ src = a.src[s];
  uint8_t* __restrict__ dst = a.dst[s];
  const int64_t ss = a.src_stride[s], ds = a.dst_stride[s];
  const int lane = threadIdx.x & 31;
  const int64_t warp = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  const int rv = static_cast<int>(a.row_vecs);
  for (int64_t r0 = warp * 4; r0 < rows; r0 += nwarps * 4) {
    for (int v = lane; v < rv; v += 32) {
      uint4 x[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (r0 + i < rows) x[i] = *reinterpret_cast<const uint4*>(src + (r0 + i) * ss + v * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (r0 + i < rows) *reinterpret_cast<uint4*>(dst + (r0 + i) * ds + v * 16) = x[i];
    }
  }
}

}  // namespace

cudaError_t launch_strided_gather(const GatherArgs& a, int sm_count, cudaStream_t stream) {
  const int64_t total = a.vec_prefix[a.n_src];
  if (total <= 0 || a.n_src <= 0) return cudaSuccess;
  int64_t max_rows = 0;
  for (int i = 0; i < a.n_src; ++i) {
    const int64_t r = (a.vec_prefix[i + 1] - a.vec_prefix[i]) / a.row_vecs;
    if (r > max_rows) max_rows = r;
  }
  // 8 warps per CTA, 4 rows per warp and pass; enough CTAs per source to fill the GPU a few times over
  int64_t bx = (max_rows + 31) / 32;
  const int64_t cap = (static_cast<int64_t>(sm_count) * 8 + a.n_src - 1) / a.n_src;
  if (bx > cap) bx = cap;
  if (bx < 1) bx = 1;
  dim3 grid(static_cast<unsigned>(bx), static_cast<unsigned>(a.n_src));
  strided_gather_kernel<<<grid, 256, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace fo
