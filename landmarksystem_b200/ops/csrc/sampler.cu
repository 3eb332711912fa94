// Fused ray sampling front end: per (ray, sample) one thread computes the sample distance, the world position,
// the inside-AABB test, the spatial block the sample falls into and its block-local coordinates.
//
// The reference does this with ~30 elementwise PyTorch kernels over [rays, samples, 3] tensors
// (landmark/nerf_components/ray_samplers/uniform_sampler.py:42-98, scene/scene_manager.py:63-124); the
// world positions are only an intermediate and are never written here.
#include "common.cuh"

namespace lmb {

struct SamplerArgs {
  float near, far, step;        // distance clamp of the first sample, spacing
  float norm_lo, norm_size;     // normalised coordinate range of the whole scene box
  int nx, ny;                   // block partition of the scene footprint
  int rel_x, rel_y, lx, ly;     // resident window: origin block and extent (ids are window-relative)
  int S;
  int hull;                     // 1: S samples linearly spaced from `near` to the ground-plane hit (render-time sampling)
};

// rays: [R, stride] (origin 3, direction 3, ...); jitter: [R] in [0,1) or null; aabb: device float[6] (min, max)
// z: [R, S]; dists: [R, S] (last 0); xyzb: [R*S, 4] = block-local xyz in [-1,1] + window-relative block id (-1:
// outside the box or the window); valid: [R*S] uint8 inside-the-box flags.
__global__ void __launch_bounds__(256)
uniform_sampler_kernel(const float* __restrict__ rays, int stride, long long R, const float* __restrict__ jitter,
                       const float* __restrict__ aabb, SamplerArgs a, float* __restrict__ z, float* __restrict__ dists,
                       float4* __restrict__ xyzb, unsigned char* __restrict__ valid) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= R * a.S) return;
  const long long r = i / a.S;
  const int k = (int)(i - r * a.S);
  const float* ray = rays + r * stride;
  const float lo[3] = {aabb[0], aabb[1], aabb[2]}, hi[3] = {aabb[3], aabb[4], aabb[5]};
  float o[3], d[3], tmin = -3.4e38f;
#pragma unroll
  for (int c = 0; c < 3; ++c) {
    o[c] = ray[c]; d[c] = ray[3 + c];
    const float safe = d[c] == 0.f ? 1e-6f : d[c];
    // IEEE division / no fused multiply-add: the first sample sits exactly on the box face, so the inside test must
    // see the same bits as the unfused reference arithmetic (a one-ulp difference flips it)
    tmin = fmaxf(tmin, fminf(__fdiv_rn(__fsub_rn(hi[c], o[c]), safe), __fdiv_rn(__fsub_rn(lo[c], o[c]), safe)));
  }
  tmin = fminf(fmaxf(tmin, a.near), a.far);
  float zk, dk;
  if (a.hull) {
    // near -> where the ray meets the ground plane z = lo_z (rays that look up: `far`), linspace over S samples
    const float dz = d[2];
    float hit = -((o[2] - lo[2]) / (dz == 0.f ? 1e-6f : dz));
    if (dz >= 0.f) hit = a.far;
    const float inv = a.S > 1 ? 1.f / (float)(a.S - 1) : 0.f;
    const float t0 = (float)k * inv, t1 = (float)(k + 1) * inv;
    zk = a.near * (1.f - t0) + hit * t0;
    dk = k + 1 < a.S ? (a.near * (1.f - t1) + hit * t1) - zk : 0.f;
  } else {
    zk = __fadd_rn(tmin, __fmul_rn(a.step, __fadd_rn((float)k, jitter ? jitter[r] : 0.f)));
    dk = k + 1 < a.S ? a.step : 0.f;
  }
  z[i] = zk;
  dists[i] = dk;
  float p[3];
  bool inside = true;
#pragma unroll
  for (int c = 0; c < 3; ++c) {
    p[c] = __fadd_rn(o[c], __fmul_rn(d[c], zk));
    inside = inside && !(p[c] < lo[c]) && !(p[c] > hi[c]);
  }
  // scene-normalised coordinates, then block and block-local coordinates
  float n[3];
#pragma unroll
  for (int c = 0; c < 3; ++c) n[c] = (p[c] - lo[c]) * (a.norm_size / (hi[c] - lo[c])) + a.norm_lo;
  const float u = (n[0] - a.norm_lo) / (a.norm_size / (float)a.nx), v = (n[1] - a.norm_lo) / (a.norm_size / (float)a.ny);
  const float bx = fminf(fmaxf(floorf(u), 0.f), (float)(a.nx - 1)), by = fminf(fmaxf(floorf(v), 0.f), (float)(a.ny - 1));
  const int rx = (int)bx - a.rel_x, ry = (int)by - a.rel_y;
  const bool resident = rx >= 0 && rx < a.lx && ry >= 0 && ry < a.ly;
  const float block = (inside && resident) ? (float)(rx * a.ly + ry) : -1.f;
  xyzb[i] = make_float4((u - bx) * 2.f - 1.f, (v - by) * 2.f - 1.f, (n[2] - a.norm_lo) / a.norm_size * 2.f - 1.f, block);
  valid[i] = inside ? 1 : 0;
}

}  // namespace lmb

using namespace lmb;

LMB_API int lmb_uniform_sampler(const float* rays, int stride, long long R, int S, const float* jitter, const float* aabb,
                                float near, float far, float step, float norm_lo, float norm_size, int nx, int ny, int rel_x,
                                int rel_y, int lx, int ly, int hull, float* z, float* dists, float* xyzb,
                                unsigned char* valid, cudaStream_t stream) {
  if (R <= 0 || S <= 0) return 0;
  SamplerArgs a{near, far, step, norm_lo, norm_size, nx, ny, rel_x, rel_y, lx, ly, S, hull};
  uniform_sampler_kernel<<<ceil_div(R * S, 256), 256, 0, stream>>>(rays, stride, R, jitter, aabb, a, z, dists, (float4*)xyzb,
                                                                  valid);
  LMB_LAUNCH_CHECK();
  return 0;
}
