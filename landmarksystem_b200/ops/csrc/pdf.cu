// Inverse-CDF resampling along rays: piecewise-constant PDF from per-bin weights -> new sample positions.
// One block per ray keeps the ray's CDF and bin edges in shared memory (block scan), then every thread draws
// samples by binary search and linear interpolation inside the bin.  Replaces the cumsum / searchsorted / four
// gathers / where chain of landmark/nerf_components/ray_samplers/pdf_sampler.py:60-116 (and the same pattern in
// proposal_network_sampler.py:387-501).
#include "common.cuh"

namespace lmb {

constexpr int kPdfThreads = 128;

// bins: [R, B+1]; weights: [R, B]; u: [R, n] in [0,1) or null (deterministic: linspace(0,1,n)); out: [R, n]
__global__ void __launch_bounds__(kPdfThreads)
pdf_resample_kernel(const float* __restrict__ bins, const float* __restrict__ weights, const float* __restrict__ u, int B, int n,
                    float eps, float* __restrict__ out) {
  extern __shared__ float sh[];
  float* cdf = sh;                 // B + 1
  float* edge = sh + B + 1;        // B + 1
  __shared__ float warp_sums[kPdfThreads / 32];
  __shared__ float carry_sh;
  const long long ray = blockIdx.x;
  const float* w = weights + ray * B;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i <= B; i += kPdfThreads) edge[i] = bins[ray * (B + 1) + i];
  if (tid == 0) { cdf[0] = 0.f; carry_sh = 0.f; }
  __syncthreads();
  // inclusive scan of (w + eps) in chunks of 128: warp scans + carry
  for (int base = 0; base < B; base += kPdfThreads) {
    const int i = base + tid;
    float v = i < B ? w[i] + eps : 0.f;
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += t;
    }
    if (lane == 31) warp_sums[warp] = v;
    __syncthreads();
    float offset = carry_sh;
    for (int k = 0; k < warp; ++k) offset += warp_sums[k];
    if (i < B) cdf[i + 1] = v + offset;
    __syncthreads();
    if (tid == kPdfThreads - 1) carry_sh = v + offset;
    __syncthreads();
  }
  const float total = carry_sh;
  for (int i = tid + 1; i <= B; i += kPdfThreads) cdf[i] /= total;
  __syncthreads();
  for (int j = tid; j < n; j += kPdfThreads) {
    const float uj = u ? u[ray * n + j] : (n > 1 ? (float)j / (float)(n - 1) : 0.f);
    int lo = 0, hi = B + 1;                       // first index with cdf[idx] > uj  (searchsorted, right = True)
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (cdf[mid] > uj) hi = mid; else lo = mid + 1;
    }
    const int below = max(lo - 1, 0), above = min(lo, B);
    const float c0 = cdf[below], c1 = cdf[above];
    float denom = c1 - c0;
    if (denom < 1e-5f) denom = 1.f;
    out[ray * n + j] = edge[below] + (uj - c0) / denom * (edge[above] - edge[below]);
  }
}

}  // namespace lmb

using namespace lmb;

LMB_API int lmb_pdf_resample(const float* bins, const float* weights, const float* u, long long R, int B, int n, float eps,
                             float* out, cudaStream_t stream) {
  if (R <= 0 || n <= 0) return 0;
  if (B < 1 || (size_t)(2 * (B + 1)) * sizeof(float) > 48 * 1024) return (int)cudaErrorInvalidValue;
  pdf_resample_kernel<<<(unsigned)R, kPdfThreads, 2 * (B + 1) * sizeof(float), stream>>>(bins, weights, u, B, n, eps, out);
  LMB_LAUNCH_CHECK();
  return 0;
}
