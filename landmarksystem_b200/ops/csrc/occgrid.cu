// Occupancy-grid ray marching (Instant-NGP style), one thread per ray.
//
// The grid has `levels` cascades of `res`^3 binary cells; cascade l covers the region of interest
// scaled by 2^l about its centre.  A ray advances in steps dt = clamp(t * cone_angle, step, inf); a
// step whose midpoint lies in an occupied cell of the finest cascade that contains it becomes a
// sample [t, t + dt]; empty cells are skipped by jumping to the cell's exit (in whole steps, so the
// sample lattice of a ray does not depend on what was skipped).  The reference obtains this from
// nerfacc's OccGridEstimator.sampling (landmark/nerf_components/ray_samplers/volumetric_sampler.py:92-104).
// Output is written directly in the padded [R, max_samples] layout the compositing kernels consume,
// so no packed->padded conversion pass is needed.
#include "common.cuh"

namespace lmb {

struct OccGrid {
  const unsigned char* cells;   // [levels, res, res, res] (z fastest? no: x slowest) -> index ((l*res + ix)*res + iy)*res + iz
  float lo[3], hi[3];           // region of interest of cascade 0
  int res, levels;
};

__device__ __forceinline__ bool ray_aabb(const float* o, const float* d, const float* lo, const float* hi, float& t0, float& t1) {
  t0 = -3.4e38f; t1 = 3.4e38f;
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    const float inv = 1.f / (fabsf(d[k]) > 1e-12f ? d[k] : (d[k] >= 0 ? 1e-12f : -1e-12f));
    float a = (lo[k] - o[k]) * inv, b = (hi[k] - o[k]) * inv;
    if (a > b) { float s = a; a = b; b = s; }
    t0 = fmaxf(t0, a); t1 = fminf(t1, b);
  }
  return t1 > t0;
}

template <bool kWrite>
__global__ void __launch_bounds__(128)
occ_march_kernel(int R, const float* __restrict__ rays_o, const float* __restrict__ rays_d, const float* __restrict__ jitter,
                 OccGrid g, float near_t, float far_t, float step, float cone_angle, int max_samples,
                 int* __restrict__ counts, float* __restrict__ t_starts, float* __restrict__ t_ends) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  const float o[3] = {rays_o[3 * r], rays_o[3 * r + 1], rays_o[3 * r + 2]};
  const float d[3] = {rays_d[3 * r], rays_d[3 * r + 1], rays_d[3 * r + 2]};
  // outermost cascade bounds
  float c[3], h[3], olo[3], ohi[3];
  const float grow = (float)(1 << (g.levels - 1));
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    c[k] = 0.5f * (g.lo[k] + g.hi[k]); h[k] = 0.5f * (g.hi[k] - g.lo[k]);
    olo[k] = c[k] - h[k] * grow; ohi[k] = c[k] + h[k] * grow;
  }
  float t0, t1;
  int n = 0;
  if (ray_aabb(o, d, olo, ohi, t0, t1)) {
    t0 = fmaxf(t0, near_t); t1 = fminf(t1, far_t);
    float t = t0;
    if (jitter) t += jitter[r] * fmaxf(t * cone_angle, step);
    int guard = 0;
    while (t < t1 && n < max_samples && guard < 100000) {
      ++guard;
      const float dt = fmaxf(t * cone_angle, step);
      const float tm = t + 0.5f * dt;
      float p[3], m = 0.f;
#pragma unroll
      for (int k = 0; k < 3; ++k) { p[k] = o[k] + tm * d[k]; m = fmaxf(m, fabsf(p[k] - c[k]) / h[k]); }
      // finest cascade containing p: m <= 2^l
      int l = 0;
      while (l < g.levels - 1 && m > (float)(1 << l)) ++l;
      if (m > (float)(1 << l)) { t += dt; continue; }          // outside every cascade
      const float s = (float)(1 << l);
      int idx[3];
      float u[3];
#pragma unroll
      for (int k = 0; k < 3; ++k) {
        u[k] = ((p[k] - c[k]) / (h[k] * s) * 0.5f + 0.5f) * g.res;     // cell coordinates in [0, res]
        idx[k] = min(max((int)u[k], 0), g.res - 1);
      }
      const long long cell = (((long long)l * g.res + idx[0]) * g.res + idx[1]) * g.res + idx[2];
      if (g.cells[cell]) {
        if (kWrite) { t_starts[(long long)r * max_samples + n] = t; t_ends[(long long)r * max_samples + n] = t + dt; }
        ++n;
        t += dt;
      } else {
        // distance (in t) to leave this cell; advance in whole steps past it
        float texit = 3.4e38f;
#pragma unroll
        for (int k = 0; k < 3; ++k) {
          if (fabsf(d[k]) < 1e-12f) continue;
          const float edge = d[k] > 0 ? (float)(idx[k] + 1) : (float)idx[k];
          const float world = c[k] + ((edge / g.res - 0.5f) * 2.f) * h[k] * s;
          texit = fminf(texit, (world - o[k]) / d[k]);
        }
        do { t += fmaxf(t * cone_angle, step); } while (t + 0.5f * fmaxf(t * cone_angle, step) < texit && t < t1);
      }
    }
  }
  counts[r] = n;
}

}  // namespace lmb

using namespace lmb;

LMB_API int lmb_occ_march(int R, const float* rays_o, const float* rays_d, const float* jitter, const unsigned char* cells,
                          const float* roi /* lo xyz, hi xyz (host) */, int res, int levels, float near_t, float far_t,
                          float step, float cone_angle, int max_samples, int* counts, float* t_starts, float* t_ends,
                          cudaStream_t stream) {
  if (R <= 0) return 0;
  OccGrid g;
  g.cells = cells; g.res = res; g.levels = levels;
  for (int k = 0; k < 3; ++k) { g.lo[k] = roi[k]; g.hi[k] = roi[3 + k]; }
  occ_march_kernel<true><<<ceil_div(R, 128), 128, 0, stream>>>(R, rays_o, rays_d, jitter, g, near_t, far_t, step, cone_angle,
                                                              max_samples, counts, t_starts, t_ends);
  LMB_LAUNCH_CHECK();
  return 0;
}
