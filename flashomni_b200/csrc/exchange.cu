// Strided row gather from several source buffers, some of which may be another GPU's memory mapped into
// this process (peer pointers): the data path of the sequence-parallel exchange. Every rank PULLS the
// slices it needs with plain 16-byte loads over NVLink and writes them, already in their final layout,
// into its own memory -- one kernel instead of a permute copy, a library all-to-all and a second permute.
// Only loads cross the link; nothing here waits on another GPU (the callers order the steps with their
// own barriers).
#include <cuda_fp16.h>
#include <cuda_fp8.h>

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

// out[r, :] = init[r, :] + sum over the sources of src_s[r, :] for the rows of one slice, 16-bit elements, fp32
// accumulation, one rounding at the end. The sources are the partial results of several GPUs (peer pointers, read
// with plain loads over NVLink); each GPU reduces the row slice it owns, so every partial crosses the link once.
template <bool kBf16>
__global__ void __launch_bounds__(256) reduce_rows_kernel(const __grid_constant__ ReduceArgs a) {
  const int64_t total = a.rows * a.row_vecs;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / a.row_vecs, v = i % a.row_vecs;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    uint4 x[kMaxGatherSources];
#pragma unroll
    for (int s = 0; s < kMaxGatherSources; ++s)
      if (s < a.n_src) x[s] = *reinterpret_cast<const uint4*>(a.src[s] + r * a.src_stride + v * 16);
    uint4 in = make_uint4(0u, 0u, 0u, 0u);
    if (a.init != nullptr) in = *reinterpret_cast<const uint4*>(a.init + r * a.init_stride + v * 16);
    auto add = [&](const uint4& q) {
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (kBf16) {
          acc[2 * j] += __uint_as_float(w[j] << 16);
          acc[2 * j + 1] += __uint_as_float(w[j] & 0xFFFF0000u);
        } else {
          const __half2 h2 = *reinterpret_cast<const __half2*>(&w[j]);
          acc[2 * j] += __low2float(h2);
          acc[2 * j + 1] += __high2float(h2);
        }
      }
    };
    if (a.init != nullptr) add(in);
#pragma unroll
    for (int s = 0; s < kMaxGatherSources; ++s)
      if (s < a.n_src) add(x[s]);
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) ow[j] = kBf16 ? pack_bf16x2(acc[2 * j], acc[2 * j + 1]) : pack_f16x2(acc[2 * j], acc[2 * j + 1]);
    *reinterpret_cast<uint4*>(a.dst + r * a.dst_stride + v * 16) = o;
  }
}

// Barrier between the GPUs of a job, one launch per GPU (each on its own device): thread t tells rank t that
// this rank has arrived (a release store of the new epoch into rank t's flag pad, over NVLink) and then waits
// until rank t's arrival shows up in this rank's own pad. The epoch lives in this GPU's memory and advances by
// one per launch, so a launch replayed from a CUDA graph still uses a fresh value. The wait is bounded: when it
// runs out the launch records FO_DEV_WAIT_TIMEOUT in the status word and returns; nothing traps.
__global__ void __launch_bounds__(64) peer_barrier_kernel(const __grid_constant__ BarrierArgs a) {
  __shared__ int s_epoch;
  const int t = threadIdx.x;
  if (t == 0) {
    s_epoch = a.epoch[a.channel] + 1;
    a.epoch[a.channel] = s_epoch;
  }
  __syncthreads();
  const int epoch = s_epoch;
  if (t >= a.world) return;
  __threadfence_system();
  if (t != a.rank) {
    int* remote = a.pads[t] + a.channel * a.world + a.rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const int* mine = a.pads[a.rank] + a.channel * a.world + t;
    const uint64_t t0 = global_timer_ns();
    while (true) {
      int seen;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if (seen - epoch >= 0) break;
      if (global_timer_ns() - t0 > a.timeout_ns) {
        atomicExch(a.status, kDevWaitTimeout);
        break;
      }
      __nanosleep(200);
    }
  }
  __threadfence_system();
}

// 8-bit floating point (e4m3 or e5m2) to the 16-bit type the attention computes in: what the reference does to its
// fp8 K / V fragments before the MMA (a plain cast, no scales; include/flashomni/attention/prefill.cuh:602-612),
// done once per tensor here. Every fp8 value is exactly representable in f16 and in bf16.
template <bool kE5m2, bool kBf16>
__global__ void __launch_bounds__(256) cast_fp8_kernel(const uint8_t* __restrict__ src, int64_t n, uint16_t* __restrict__ dst) {
  const int64_t nvec = n / 16;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint4 x = *reinterpret_cast<const uint4*>(src + i * 16);
    const uint32_t w[4] = {x.x, x.y, x.z, x.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const __nv_fp8x2_storage_t p = static_cast<__nv_fp8x2_storage_t>((w[j >> 1] >> ((j & 1) * 16)) & 0xffffu);
      const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(p, kE5m2 ? __NV_E5M2 : __NV_E4M3);
      const __half2 h2 = *reinterpret_cast<const __half2*>(&hr);
      o[j] = kBf16 ? pack_bf16x2(__low2float(h2), __high2float(h2)) : *reinterpret_cast<const uint32_t*>(&h2);
    }
    uint4* d = reinterpret_cast<uint4*>(dst + i * 16);
    d[0] = make_uint4(o[0], o[1], o[2], o[3]);
    d[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
  // tail of fewer than 16 values
  if (blockIdx.x == 0) {
    for (int64_t i = nvec * 16 + threadIdx.x; i < n; i += blockDim.x) {
      const __half_raw hr = __nv_cvt_fp8_to_halfraw(src[i], kE5m2 ? __NV_E5M2 : __NV_E4M3);
      const __half h = *reinterpret_cast<const __half*>(&hr);
      if (kBf16) dst[i] = static_cast<uint16_t>(pack_bf16x2(__half2float(h), 0.f) & 0xffffu);
      else dst[i] = *reinterpret_cast<const uint16_t*>(&h);
    }
  }
}

}  // namespace

cudaError_t launch_cast_fp8(const void* src, int64_t n, int e5m2, int is_bf16, void* dst, int sm_count, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  int64_t blocks = (n / 16 + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count) * 8;
  blocks = blocks > cap ? cap : (blocks < 1 ? 1 : blocks);
  const uint8_t* s = static_cast<const uint8_t*>(src);
  uint16_t* d = static_cast<uint16_t*>(dst);
  const unsigned g = static_cast<unsigned>(blocks);
  if (e5m2) {
    if (is_bf16) cast_fp8_kernel<true, true><<<g, 256, 0, stream>>>(s, n, d);
    else cast_fp8_kernel<true, false><<<g, 256, 0, stream>>>(s, n, d);
  } else {
    if (is_bf16) cast_fp8_kernel<false, true><<<g, 256, 0, stream>>>(s, n, d);
    else cast_fp8_kernel<false, false><<<g, 256, 0, stream>>>(s, n, d);
  }
  return cudaGetLastError();
}

cudaError_t launch_reduce_rows(const ReduceArgs& a, int is_bf16, int sm_count, cudaStream_t stream) {
  const int64_t total = a.rows * a.row_vecs;
  if (total <= 0) return cudaSuccess;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count) * 8;
  if (blocks > cap) blocks = cap;
  if (is_bf16) reduce_rows_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a);
  else reduce_rows_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_peer_barrier(const BarrierArgs& a, cudaStream_t stream) {
  peer_barrier_kernel<<<1, 64, 0, stream>>>(a);
  return cudaGetLastError();
}

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
