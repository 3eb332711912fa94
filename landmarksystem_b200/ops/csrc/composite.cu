// Volume-rendering composite, forward and backward, one warp per ray.
//
//   alpha_i = 1 - exp(-sigma_i * dist_i);  T_i = prod_{j<i} (1 - alpha_j + 1e-10);  w_i = alpha_i * T_i
//   rgb = sum_i w_i c_i (+ (1 - sum_i w_i) * bg);  depth = sum_i w_i z_i;  acc = sum_i w_i
//
// Same math as the reference's torch ops (landmark/nerf_components/model_components/renderers/
// volume_renderer.py:20-67) but the exclusive cumprod is a warp shuffle scan, so a ray's samples
// are read once and nothing of size [R, S+1] is materialised.
#include "common.cuh"

namespace lmb {

constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ float warp_excl_prod(float v, float& total) {
  float x = v;
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    float y = __shfl_up_sync(kFull, x, d);
    if (lane >= d) x *= y;
  }
  total = __shfl_sync(kFull, x, 31);
  float e = __shfl_up_sync(kFull, x, 1);
  return lane == 0 ? 1.f : e;
}

__device__ __forceinline__ float warp_incl_sum(float v, float& total) {
  float x = v;
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    float y = __shfl_up_sync(kFull, x, d);
    if (lane >= d) x += y;
  }
  total = __shfl_sync(kFull, x, 31);
  return x;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(kFull, v, d);
  return v;
}

__global__ void __launch_bounds__(256)
weights_fwd_kernel(const float* __restrict__ sigma, const float* __restrict__ dists, int R, int S,
                   float* __restrict__ weights, float* __restrict__ bg_trans) {
  const int ray = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (ray >= R) return;
  const long long base = (long long)ray * S;
  float carry = 1.f;
  for (int s0 = 0; s0 < S; s0 += 32) {
    const int s = s0 + lane;
    float a = 0.f;
    if (s < S) a = 1.f - __expf(-sigma[base + s] * dists[base + s]);
    float tot;
    float T = carry * warp_excl_prod(s < S ? (1.f - a + 1e-10f) : 1.f, tot);
    if (s < S) weights[base + s] = a * T;
    carry *= tot;
  }
  if (lane == 0 && bg_trans) bg_trans[ray] = carry;
}

__global__ void __launch_bounds__(256)
weights_bwd_kernel(const float* __restrict__ sigma, const float* __restrict__ dists,
                   const float* __restrict__ dweights, const float* __restrict__ dbg, int R, int S,
                   float* __restrict__ dsigma) {
  const int ray = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (ray >= R) return;
  const long long base = (long long)ray * S;
  // pass 1: total = sum_k dw_k w_k (+ dbg * T_end), needs the forward scan once
  float carry = 1.f, total = 0.f;
  for (int s0 = 0; s0 < S; s0 += 32) {
    const int s = s0 + lane;
    float a = 0.f, dw = 0.f;
    if (s < S) { a = 1.f - __expf(-sigma[base + s] * dists[base + s]); dw = dweights[base + s]; }
    float tot;
    float T = carry * warp_excl_prod(s < S ? (1.f - a + 1e-10f) : 1.f, tot);
    total += warp_sum(dw * a * T);
    carry *= tot;
  }
  if (dbg) total += dbg[ray] * carry;
  // pass 2: d alpha_i = dw_i T_i - (sum_{k>i} dw_k w_k + dbg T_end) / t_i
  carry = 1.f;
  float prefix = 0.f;
  for (int s0 = 0; s0 < S; s0 += 32) {
    const int s = s0 + lane;
    float a = 0.f, dw = 0.f, d = 0.f;
    if (s < S) { d = dists[base + s]; a = 1.f - __expf(-sigma[base + s] * d); dw = dweights[base + s]; }
    const float t = 1.f - a + 1e-10f;
    float tot, stot;
    float T = carry * warp_excl_prod(s < S ? t : 1.f, tot);
    float incl = prefix + warp_incl_sum(dw * a * T, stot);
    if (s < S) {
      float suffix = total - incl;
      float dalpha = dw * T - suffix / t;
      dsigma[base + s] = dalpha * d * (1.f - a);
    }
    carry *= tot;
    prefix += stot;
  }
}

// rgbs: [R, S, 3].  out_rgb is NOT clamped (clamping stays in the caller so autograd sees it).
__global__ void __launch_bounds__(256)
render_fwd_kernel(const float* __restrict__ weights, const float* __restrict__ rgbs, const float* __restrict__ z_vals,
                  int R, int S, float bg, float* __restrict__ out_rgb, float* __restrict__ out_depth,
                  float* __restrict__ out_acc) {
  const int ray = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (ray >= R) return;
  const long long base = (long long)ray * S;
  float r = 0.f, g = 0.f, b = 0.f, dep = 0.f, acc = 0.f;
  for (int s = lane; s < S; s += 32) {
    const float w = weights[base + s];
    if (w != 0.f) {
      const float* c = rgbs + (base + s) * 3;
      r += w * c[0]; g += w * c[1]; b += w * c[2];
      dep += w * z_vals[base + s];
      acc += w;
    }
  }
  r = warp_sum(r); g = warp_sum(g); b = warp_sum(b); dep = warp_sum(dep); acc = warp_sum(acc);
  if (lane == 0) {
    const float rest = bg * (1.f - acc);
    out_rgb[ray * 3 + 0] = r + rest; out_rgb[ray * 3 + 1] = g + rest; out_rgb[ray * 3 + 2] = b + rest;
    if (out_depth) out_depth[ray] = dep;
    if (out_acc) out_acc[ray] = acc;
  }
}

__global__ void __launch_bounds__(256)
render_bwd_kernel(const float* __restrict__ weights, const float* __restrict__ rgbs, const float* __restrict__ drgb_map,
                  int R, int S, float bg, float* __restrict__ dweights, float* __restrict__ drgbs) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)R * S) return;
  const int ray = (int)(i / S);
  const float d0 = drgb_map[ray * 3], d1 = drgb_map[ray * 3 + 1], d2 = drgb_map[ray * 3 + 2];
  const float w = weights[i];
  const float* c = rgbs + i * 3;
  dweights[i] = d0 * (c[0] - bg) + d1 * (c[1] - bg) + d2 * (c[2] - bg);
  drgbs[i * 3] = w * d0; drgbs[i * 3 + 1] = w * d1; drgbs[i * 3 + 2] = w * d2;
}

}  // namespace lmb

using namespace lmb;

LMB_API int lmb_weights_fwd(const float* sigma, const float* dists, int R, int S, float* weights, float* bg_trans,
                            cudaStream_t stream) {
  if (R <= 0 || S <= 0) return 0;
  weights_fwd_kernel<<<ceil_div((long long)R * 32, 256), 256, 0, stream>>>(sigma, dists, R, S, weights, bg_trans);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_weights_bwd(const float* sigma, const float* dists, const float* dweights, const float* dbg, int R,
                            int S, float* dsigma, cudaStream_t stream) {
  if (R <= 0 || S <= 0) return 0;
  weights_bwd_kernel<<<ceil_div((long long)R * 32, 256), 256, 0, stream>>>(sigma, dists, dweights, dbg, R, S, dsigma);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_render_fwd(const float* weights, const float* rgbs, const float* z_vals, int R, int S, float bg,
                           float* out_rgb, float* out_depth, float* out_acc, cudaStream_t stream) {
  if (R <= 0 || S <= 0) return 0;
  render_fwd_kernel<<<ceil_div((long long)R * 32, 256), 256, 0, stream>>>(weights, rgbs, z_vals, R, S, bg, out_rgb,
                                                                         out_depth, out_acc);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_render_bwd(const float* weights, const float* rgbs, const float* drgb_map, int R, int S, float bg,
                           float* dweights, float* drgbs, cudaStream_t stream) {
  if (R <= 0 || S <= 0) return 0;
  render_bwd_kernel<<<ceil_div((long long)R * S, 256), 256, 0, stream>>>(weights, rgbs, drgb_map, R, S, bg, dweights,
                                                                        drgbs);
  LMB_LAUNCH_CHECK();
  return 0;
}
