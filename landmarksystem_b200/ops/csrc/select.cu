// Row selection without a host round trip: stream compaction of a sample mask (the reference's
// `app_mask.nonzero()` + index gathers, benchmarks/nerf/gridnerf/gridnerf.py:846-871, make the host wait
// for the element count), plus the gathers / scatters that move per-sample rows between the full
// [rays x samples] layout and the compacted one.  Every consumer takes the device-side count, so buffer
// shapes are static (capacity = number of samples) and the whole training step can be captured in a
// CUDA graph.
#include "common.cuh"

namespace lmb {

// idx[pos] = i and coords_out[pos] = xyzb[i] for every i with mask[i] != 0; *count ends as the number of
// selected rows.  A block of 256 threads takes 1024 consecutive elements (four per thread, one 32-bit mask load),
// ranks its selected rows with a block-wide scan and reserves its output range with ONE atomic: a launch over 2^25
// samples issues 2^15 atomics on the counter instead of one per warp (2^20), which is what bounded the kernel.
// Rows of one block stay adjacent and in order.
constexpr int kCompactPerThread = 4;

__global__ void __launch_bounds__(256)
compact_kernel(const unsigned char* __restrict__ mask, long long n, const float4* __restrict__ xyzb, int* __restrict__ idx,
               float4* __restrict__ coords_out, int* __restrict__ count, int mask_aligned) {
  __shared__ int warp_sum[8];
  __shared__ int block_base;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long i0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * kCompactPerThread;
  unsigned sel = 0;
  if (mask_aligned && i0 + kCompactPerThread <= n) {
    const uchar4 m = *reinterpret_cast<const uchar4*>(mask + i0);
    sel = (m.x != 0 ? 1u : 0u) | (m.y != 0 ? 2u : 0u) | (m.z != 0 ? 4u : 0u) | (m.w != 0 ? 8u : 0u);
  } else {
#pragma unroll
    for (int k = 0; k < kCompactPerThread; ++k)
      if (i0 + k < n && mask[i0 + k] != 0) sel |= 1u << k;
  }
  const int mine = __popc(sel);
  int incl = mine;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += v;
  }
  if (lane == 31) warp_sum[warp] = incl;
  __syncthreads();
  if (threadIdx.x == 0) {
    int total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const int t = warp_sum[w];
      warp_sum[w] = total;
      total += t;
    }
    block_base = total > 0 ? atomicAdd(count, total) : 0;
  }
  __syncthreads();
  int pos = block_base + warp_sum[warp] + incl - mine;
#pragma unroll
  for (int k = 0; k < kCompactPerThread; ++k) {
    if (sel & (1u << k)) {
      idx[pos] = (int)(i0 + k);
      coords_out[pos] = xyzb[i0 + k];
      ++pos;
    }
  }
}

// payload[j] = (coords[j].xyz, dirs[idx[j] / S]), owner[j] = (int)coords[j].w for the first *count rows: the rows a
// rank sends to the owners of the blocks its colour samples fall into
__global__ void __launch_bounds__(256)
build_payload6_kernel(const float4* __restrict__ coords, const float* __restrict__ dirs, const int* __restrict__ idx,
                      const int* __restrict__ count_ptr, long long max_n, int S, float* __restrict__ payload,
                      int* __restrict__ owner) {
  const long long n = resolve_count(count_ptr, max_n);
  const long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const float4 c = coords[j];
  const float* d = dirs + (long long)(idx[j] / S) * 3;
  float* o = payload + j * 6;
  o[0] = c.x; o[1] = c.y; o[2] = c.z; o[3] = d[0]; o[4] = d[1]; o[5] = d[2];
  owner[j] = (int)c.w;
}

// kScatter: out[idx[j], :] = vals[j, :] (rows whose block id coords[j].w < 0 contribute zeros; out is pre-zeroed)
// else    : vals[j, :] = out[idx[j], :] (same rule) - the adjoint
template <bool kScatter>
__global__ void __launch_bounds__(256)
rows3_kernel(float* __restrict__ vals, const int* __restrict__ idx, const float4* __restrict__ coords,
             const int* __restrict__ count_ptr, long long max_n, float* __restrict__ full) {
  const long long n = resolve_count(count_ptr, max_n);
  const long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const bool live = coords[j].w >= 0.f;
  float* f = full + (long long)idx[j] * 3;
  float* v = vals + j * 3;
  if (kScatter) {
    if (live) { f[0] = v[0]; f[1] = v[1]; f[2] = v[2]; }
  } else {
    v[0] = live ? f[0] : 0.f; v[1] = live ? f[1] : 0.f; v[2] = live ? f[2] : 0.f;
  }
}

}  // namespace lmb

using namespace lmb;

// mask: uint8/bool [n]; xyzb: float [n, 4]; idx: int32 [n]; coords_out: float [n, 4]; count: int32 [1]
LMB_API int lmb_compact_rows(const unsigned char* mask, long long n, const float* xyzb, int* idx, float* coords_out, int* count,
                             cudaStream_t stream) {
  LMB_CUDA_TRY(cudaMemsetAsync(count, 0, sizeof(int), stream));
  if (n <= 0) return 0;
  const int aligned = (reinterpret_cast<uintptr_t>(mask) & 3u) == 0 ? 1 : 0;
  compact_kernel<<<ceil_div(n, 256 * kCompactPerThread), 256, 0, stream>>>(mask, n, (const float4*)xyzb, idx, (float4*)coords_out,
                                                                           count, aligned);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_scatter_rows3(const float* vals, const int* idx, const float* coords, const int* count_ptr, long long max_n,
                              float* out, cudaStream_t stream) {
  if (max_n <= 0) return 0;
  rows3_kernel<true><<<ceil_div(max_n, 256), 256, 0, stream>>>(const_cast<float*>(vals), idx, (const float4*)coords, count_ptr,
                                                              max_n, out);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_gather_rows3(const float* full, const int* idx, const float* coords, const int* count_ptr, long long max_n,
                             float* vals, cudaStream_t stream) {
  if (max_n <= 0) return 0;
  rows3_kernel<false><<<ceil_div(max_n, 256), 256, 0, stream>>>(vals, idx, (const float4*)coords, count_ptr, max_n,
                                                               const_cast<float*>(full));
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_build_payload6(const float* coords, const float* dirs, const int* idx, const int* count_ptr, long long max_n,
                               int S, float* payload, int* owner, cudaStream_t stream) {
  if (max_n <= 0) return 0;
  build_payload6_kernel<<<ceil_div(max_n, 256), 256, 0, stream>>>((const float4*)coords, dirs, idx, count_ptr, max_n, S, payload,
                                                                 owner);
  LMB_LAUNCH_CHECK();
  return 0;
}
