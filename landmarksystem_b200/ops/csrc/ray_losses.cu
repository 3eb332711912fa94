// Per-ray regularisers of the mip-NeRF-360 family, one warp per ray, loss and gradient in one pass.
//
//   distortion:  L_r = sum_ij w_i w_j |m_i - m_j| + 1/3 sum_i w_i^2 d_i        (m sorted along the ray)
//   interlevel:  L_r = sum_i max(0, w_i - W_i)^2 / (w_i + eps),   W_i = proposal weight that overlaps fine interval i
//
// The reference evaluates the first with the external eff_distloss package (benchmarks/nerf/gridnerf/gridnerf.py:24) or
// with an S x S matrix per ray (landmark/nerf_components/utils/loss_utils.py:85-121) and the second with
// searchsorted + gathers (loss_utils.py:124-177).  Here both are prefix sums held in registers / shared memory:
// O(S) work per ray, no intermediate tensors, and the gradient comes out of the same pass.
#include "common.cuh"

namespace lmb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_inclusive_scan(float v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float u = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += u;
  }
  return v;
}

// w, m, d: [R, S].  loss: [R].  dw: [R, S] = dL_r / dw_i (may be null).
__global__ void __launch_bounds__(256)
distortion_kernel(const float* __restrict__ w, const float* __restrict__ m, const float* __restrict__ d, long long R, int S,
                  float* __restrict__ loss, float* __restrict__ dw) {
  const int lane = threadIdx.x & 31;
  const long long r = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (r >= R) return;
  const float* wr = w + r * S; const float* mr = m + r * S; const float* dr = d + r * S;
  float w_tot = 0.f, b_tot = 0.f;
  for (int i = lane; i < S; i += 32) { const float wi = wr[i]; w_tot += wi; b_tot += wi * mr[i]; }
  w_tot = warp_sum(w_tot); b_tot = warp_sum(b_tot);
  float carry_a = 0.f, carry_b = 0.f, acc = 0.f;
  for (int base = 0; base < S; base += 32) {
    const int i = base + lane;
    const bool ok = i < S;
    const float wi = ok ? wr[i] : 0.f, mi = ok ? mr[i] : 0.f, di = ok ? dr[i] : 0.f;
    const float inc_a = warp_inclusive_scan(wi, lane), inc_b = warp_inclusive_scan(wi * mi, lane);
    const float A = carry_a + inc_a - wi, B = carry_b + inc_b - wi * mi;     // sums over j < i
    acc += 2.f * wi * (mi * A - B) + (1.f / 3.f) * wi * wi * di;
    if (dw != nullptr && ok) {
      const float after_w = w_tot - A - wi, after_b = b_tot - B - wi * mi;   // sums over j > i
      dw[r * S + i] = 2.f * ((mi * A - B) + (after_b - mi * after_w)) + (2.f / 3.f) * wi * di;
    }
    carry_a += __shfl_sync(0xffffffffu, inc_a, 31);
    carry_b += __shfl_sync(0xffffffffu, inc_b, 31);
  }
  acc = warp_sum(acc);
  if (lane == 0) loss[r] = acc;
}

constexpr int kMaxEnv = 1024;      // proposal intervals per ray held in shared memory
constexpr int kInterWarps = 4;

// t [R, S+1] fine edges, w [R, S] fine weights (constants); t_env [R, E+1], w_env [R, E] proposal histogram.
// loss [R]; dw_env [R, E] = dL_r / dw_env (may be null).
__global__ void __launch_bounds__(kInterWarps * 32)
interlevel_kernel(const float* __restrict__ t, const float* __restrict__ w, const float* __restrict__ t_env,
                  const float* __restrict__ w_env, long long R, int S, int E, float eps, float* __restrict__ loss,
                  float* __restrict__ dw_env) {
  __shared__ float cum[kInterWarps][kMaxEnv + 1];     // exclusive prefix sums of w_env
  __shared__ float edge[kInterWarps][kMaxEnv + 1];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const long long r = (long long)blockIdx.x * kInterWarps + wid;
  if (r >= R) return;
  float* cy = cum[wid]; float* te = edge[wid];
  const float* ter = t_env + r * (E + 1); const float* wer = w_env + r * E;
  float carry = 0.f;
  for (int base = 0; base < E; base += 32) {
    const int j = base + lane;
    const float v = j < E ? wer[j] : 0.f;
    const float inc = warp_inclusive_scan(v, lane);
    if (j < E) cy[j + 1] = carry + inc;
    carry += __shfl_sync(0xffffffffu, inc, 31);
  }
  if (lane == 0) cy[0] = 0.f;
  for (int j = lane; j <= E; j += 32) te[j] = ter[j];
  __syncwarp();
  const float* tr = t + r * (S + 1); const float* wr = w + r * S;
  float acc = 0.f;
  // pass 1: the loss
  for (int base = 0; base < S; base += 32) {
    const int i = base + lane;
    if (i < S) {
      const float t0 = tr[i], t1 = tr[i + 1], wi = wr[i];
      // lo = (#starts <= t0) - 1 over starts = te[0..E-1];  hi = #ends <= t1 over ends = te[1..E]; both clamped to [0, E-1]
      int a = 0, b = E;
      while (a < b) { const int mid = (a + b) >> 1; if (te[mid] <= t0) a = mid + 1; else b = mid; }
      int lo = a - 1; lo = lo < 0 ? 0 : (lo > E - 1 ? E - 1 : lo);
      a = 0; b = E;
      while (a < b) { const int mid = (a + b) >> 1; if (te[mid + 1] <= t1) a = mid + 1; else b = mid; }
      const int hi = a > E - 1 ? E - 1 : a;
      const float outer = cy[hi + 1] - cy[lo];
      const float diff = fmaxf(wi - outer, 0.f);
      acc += diff * diff / (wi + eps);
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) loss[r] = acc;
  if (dw_env == nullptr) return;
  __syncwarp();
  // pass 2: dw_env[j] = sum over the fine intervals whose range [lo, hi] covers j of -2 diff / (w + eps); the ranges are
  // recomputed rather than stored (two binary searches in shared memory)
  float* out = dw_env + r * E;
  for (int j = lane; j < E; j += 32) out[j] = 0.f;
  __syncwarp();
  for (int base = 0; base < S; base += 32) {
    const int i = base + lane;
    if (i < S) {
      const float t0 = tr[i], t1 = tr[i + 1], wi = wr[i];
      int a = 0, b = E;
      while (a < b) { const int mid = (a + b) >> 1; if (te[mid] <= t0) a = mid + 1; else b = mid; }
      int lo = a - 1; lo = lo < 0 ? 0 : (lo > E - 1 ? E - 1 : lo);
      a = 0; b = E;
      while (a < b) { const int mid = (a + b) >> 1; if (te[mid + 1] <= t1) a = mid + 1; else b = mid; }
      const int hi = a > E - 1 ? E - 1 : a;
      const float diff = fmaxf(wi - (cy[hi + 1] - cy[lo]), 0.f);
      if (diff > 0.f && hi >= lo) {
        const float g = -2.f * diff / (wi + eps);
        for (int j = lo; j <= hi; ++j) atomicAdd(&out[j], g);       // ranges span a handful of proposal bins
      }
    }
  }
}

}  // namespace lmb

using namespace lmb;

LMB_API int lmb_distortion_loss(const float* w, const float* m, const float* d, long long R, int S, float* loss, float* dw,
                                cudaStream_t stream) {
  if (R <= 0 || S <= 0) return 0;
  distortion_kernel<<<ceil_div(R * 32, 256), 256, 0, stream>>>(w, m, d, R, S, loss, dw);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_interlevel_loss(const float* t, const float* w, const float* t_env, const float* w_env, long long R, int S, int E,
                                float eps, float* loss, float* dw_env, cudaStream_t stream) {
  if (R <= 0 || S <= 0 || E <= 0) return 0;
  if (E > kMaxEnv) return (int)cudaErrorInvalidValue;
  interlevel_kernel<<<ceil_div(R, kInterWarps), kInterWarps * 32, 0, stream>>>(t, w, t_env, w_env, R, S, E, eps, loss, dw_env);
  LMB_LAUNCH_CHECK();
  return 0;
}
