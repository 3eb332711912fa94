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

// ---- proposal-network resampling -----------------------------------------------------------------------------
// One warp per ray: histogram (padded weights) -> clamped CDF -> inverse-CDF samples for the given u -> optional
// merge with the existing edges.  Both sequences are ascending, so the merge is a rank computation (two binary
// searches) instead of the concatenate + sort of landmark/nerf_components/ray_samplers/proposal_network_sampler.py:437-478.
constexpr int kPropWarps = 2;
constexpr int kPropMax = 1025;          // edges per ray held in shared memory

// w [R, E]; existing [R, E+1]; u [R, B] ascending; out [R, B] or, merged, [R, B + E + 1]
__global__ void __launch_bounds__(kPropWarps * 32)
prop_resample_kernel(const float* __restrict__ w, const float* __restrict__ existing, const float* __restrict__ u, long long R,
                     int E, int B, float hist_pad, float eps, int merge, float* __restrict__ out) {
  __shared__ float cdf_s[kPropWarps][kPropMax], edge_s[kPropWarps][kPropMax], new_s[kPropWarps][kPropMax];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const long long r = (long long)blockIdx.x * kPropWarps + wid;
  if (r >= R) return;
  float* cdf = cdf_s[wid]; float* edge = edge_s[wid]; float* fresh = new_s[wid];
  const float* wr = w + r * E;
  float total = 0.f;
  for (int i = lane; i < E; i += 32) total += wr[i] + hist_pad;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
  const float padding = fmaxf(eps - total, 0.f);
  const float add = hist_pad + padding / (float)E, inv = 1.f / (total + padding);
  float carry = 0.f;
  for (int base = 0; base < E; base += 32) {
    const int i = base + lane;
    float v = i < E ? (wr[i] + add) * inv : 0.f;
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += t;
    }
    if (i < E) cdf[i + 1] = fminf(carry + v, 1.f);
    carry += __shfl_sync(0xffffffffu, v, 31);
  }
  if (lane == 0) cdf[0] = 0.f;
  for (int i = lane; i <= E; i += 32) edge[i] = existing[r * (E + 1) + i];
  __syncwarp();
  const int out_w = merge ? B + E + 1 : B;
  float* orow = out + r * out_w;
  for (int k = lane; k < B; k += 32) {
    const float uk = u[r * B + k];
    int a = 0, b = E + 1;                                   // #cdf entries <= u
    while (a < b) { const int mid = (a + b) >> 1; if (cdf[mid] <= uk) a = mid + 1; else b = mid; }
    const int below = min(max(a - 1, 0), E), above = min(a, E);
    const float c0 = cdf[below], c1 = cdf[above];
    float t = (uk - c0) / (c1 - c0);
    if (t != t) t = 0.f;                                    // 0 / 0
    t = fminf(fmaxf(t, 0.f), 1.f);
    const float v = edge[below] + t * (edge[above] - edge[below]);
    if (merge) fresh[k] = v; else orow[k] = v;
  }
  if (!merge) return;
  __syncwarp();
  // rank of a new value: its index + #existing <= it; rank of an existing edge: its index + #new < it
  for (int k = lane; k < B; k += 32) {
    const float v = fresh[k];
    int a = 0, b = E + 1;
    while (a < b) { const int mid = (a + b) >> 1; if (edge[mid] <= v) a = mid + 1; else b = mid; }
    orow[k + a] = v;
  }
  for (int j = lane; j <= E; j += 32) {
    const float v = edge[j];
    int a = 0, b = B;
    while (a < b) { const int mid = (a + b) >> 1; if (fresh[mid] < v) a = mid + 1; else b = mid; }
    orow[j + a] = v;
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

LMB_API int lmb_prop_resample(const float* w, const float* existing, const float* u, long long R, int E, int B, float hist_pad,
                              float eps, int merge, float* out, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (E + 1 > kPropMax || B > kPropMax || E <= 0 || B <= 0) return (int)cudaErrorInvalidValue;
  prop_resample_kernel<<<ceil_div(R, kPropWarps), kPropWarps * 32, 0, stream>>>(w, existing, u, R, E, B, hist_pad, eps, merge, out);
  LMB_LAUNCH_CHECK();
  return 0;
}
