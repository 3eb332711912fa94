// 3D Gaussian splatting rasteriser: projection + SH colour, (tile, depth) key generation, per-tile
// ranges, tile alpha-blending, and the backward of all of it.
//
// Functional counterpart of the rasteriser extension the reference calls
// (GaussianRasterizationSettings / GaussianRasterizer with an extra visible_filter;
// benchmarks/nerf/origin_gs/gs_model.py:82-97,148-162,211-220) whose source is not part of the
// reference tree.  The math is the published EWA splatting formulation: 3-D covariance R S S^T R^T,
// perspective Jacobian, 0.3 px low-pass, 3-sigma extent, front-to-back alpha compositing with
// alpha < 1/255 skipped, alpha clamped to 0.99 and termination at T < 1e-4.
// Conventions: matrices are row-vector style ([x y z 1] @ M), 16x16 pixel tiles, channel-first
// image output [3, H, W].  Backward reduces per-Gaussian gradients across the warp with shuffles
// before touching global memory (one atomic per warp and Gaussian instead of one per pixel).
#include "common.cuh"

namespace lmb {

constexpr int kTile = 16;
constexpr int kTilePixels = kTile * kTile;

struct GSCamera {
  float view[16];      // world -> view, row-vector convention (transposed world-to-camera)
  float proj[16];      // world -> clip (view @ projection)
  float campos[3];
  float tanfovx, tanfovy;
  int W, H;
  float scale_modifier;
  int sh_degree;       // active degree
  int sh_coeffs;       // coefficients stored per Gaussian ((max_degree + 1)^2)
};

__device__ __forceinline__ float3 xform43(const float* m, float3 p) {   // [p 1] @ M, first 3 comps
  return make_float3(m[0] * p.x + m[4] * p.y + m[8] * p.z + m[12], m[1] * p.x + m[5] * p.y + m[9] * p.z + m[13],
                     m[2] * p.x + m[6] * p.y + m[10] * p.z + m[14]);
}
__device__ __forceinline__ float4 xform44(const float* m, float3 p) {
  return make_float4(m[0] * p.x + m[4] * p.y + m[8] * p.z + m[12], m[1] * p.x + m[5] * p.y + m[9] * p.z + m[13],
                     m[2] * p.x + m[6] * p.y + m[10] * p.z + m[14], m[3] * p.x + m[7] * p.y + m[11] * p.z + m[15]);
}

__device__ __forceinline__ void quat_to_rot(float4 q, float* R) {   // q = (w, x, y, z), unit
  const float r = q.x, x = q.y, y = q.z, z = q.w;
  R[0] = 1.f - 2.f * (y * y + z * z); R[1] = 2.f * (x * y - r * z); R[2] = 2.f * (x * z + r * y);
  R[3] = 2.f * (x * y + r * z); R[4] = 1.f - 2.f * (x * x + z * z); R[5] = 2.f * (y * z - r * x);
  R[6] = 2.f * (x * z - r * y); R[7] = 2.f * (y * z + r * x); R[8] = 1.f - 2.f * (x * x + y * y);
}

// Sigma = R diag(s)^2 R^T, upper triangle (xx, xy, xz, yy, yz, zz)
__device__ __forceinline__ void cov3d_from(float3 s, float4 q, float* c) {
  float R[9];
  quat_to_rot(q, R);
  const float sx = s.x * s.x, sy = s.y * s.y, sz = s.z * s.z;
  c[0] = R[0] * R[0] * sx + R[1] * R[1] * sy + R[2] * R[2] * sz;
  c[1] = R[0] * R[3] * sx + R[1] * R[4] * sy + R[2] * R[5] * sz;
  c[2] = R[0] * R[6] * sx + R[1] * R[7] * sy + R[2] * R[8] * sz;
  c[3] = R[3] * R[3] * sx + R[4] * R[4] * sy + R[5] * R[5] * sz;
  c[4] = R[3] * R[6] * sx + R[4] * R[7] * sy + R[5] * R[8] * sz;
  c[5] = R[6] * R[6] * sx + R[7] * R[7] * sy + R[8] * R[8] * sz;
}

// T = J * Wr (2x3), where Wr[i][j] = d view_i / d world_j.  Returns cov2D (a, b, c) before the low-pass.
__device__ __forceinline__ void project_cov(const GSCamera& cam, float3 t, const float* c3, float fx, float fy,
                                            float* T, float& a, float& b, float& c) {
  const float limx = 1.3f * cam.tanfovx, limy = 1.3f * cam.tanfovy;
  const float txz = fminf(limx, fmaxf(-limx, t.x / t.z)) * t.z;
  const float tyz = fminf(limy, fmaxf(-limy, t.y / t.z)) * t.z;
  const float j00 = fx / t.z, j02 = -fx * txz / (t.z * t.z), j11 = fy / t.z, j12 = -fy * tyz / (t.z * t.z);
  const float* v = cam.view;   // Wr[i][j] = v[j*4 + i]
  T[0] = j00 * v[0] + j02 * v[2]; T[1] = j00 * v[4] + j02 * v[6]; T[2] = j00 * v[8] + j02 * v[10];
  T[3] = j11 * v[1] + j12 * v[2]; T[4] = j11 * v[5] + j12 * v[6]; T[5] = j11 * v[9] + j12 * v[10];
  // cov2D = T Sigma T^T
  const float s0 = c3[0] * T[0] + c3[1] * T[1] + c3[2] * T[2];
  const float s1 = c3[1] * T[0] + c3[3] * T[1] + c3[4] * T[2];
  const float s2 = c3[2] * T[0] + c3[4] * T[1] + c3[5] * T[2];
  const float u0 = c3[0] * T[3] + c3[1] * T[4] + c3[2] * T[5];
  const float u1 = c3[1] * T[3] + c3[3] * T[4] + c3[4] * T[5];
  const float u2 = c3[2] * T[3] + c3[4] * T[4] + c3[5] * T[5];
  a = T[0] * s0 + T[1] * s1 + T[2] * s2;
  b = T[3] * s0 + T[4] * s1 + T[5] * s2;
  c = T[3] * u0 + T[4] * u1 + T[5] * u2;
}

__constant__ float kSH_C1 = 0.4886025119029199f;
__constant__ float kSH_C2[5] = {1.0925484305920792f, -1.0925484305920792f, 0.31539156525252005f, -1.0925484305920792f, 0.5462742152960396f};
__constant__ float kSH_C3[7] = {-0.5900435899266435f, 2.890611442640554f, -0.4570457994644658f, 0.3731763325901154f, -0.4570457994644658f, 1.445305721320277f, -0.5900435899266435f};

__device__ __forceinline__ void sh_basis(int deg, float3 d, float* B) {
  const float x = d.x, y = d.y, z = d.z;
  B[0] = 0.28209479177387814f;
  if (deg > 0) {
    B[1] = -kSH_C1 * y; B[2] = kSH_C1 * z; B[3] = -kSH_C1 * x;
    if (deg > 1) {
      const float xx = x * x, yy = y * y, zz = z * z, xy = x * y, yz = y * z, xz = x * z;
      B[4] = kSH_C2[0] * xy; B[5] = kSH_C2[1] * yz; B[6] = kSH_C2[2] * (2.f * zz - xx - yy);
      B[7] = kSH_C2[3] * xz; B[8] = kSH_C2[4] * (xx - yy);
      if (deg > 2) {
        B[9] = kSH_C3[0] * y * (3.f * xx - yy); B[10] = kSH_C3[1] * xy * z; B[11] = kSH_C3[2] * y * (4.f * zz - xx - yy);
        B[12] = kSH_C3[3] * z * (2.f * zz - 3.f * xx - 3.f * yy); B[13] = kSH_C3[4] * x * (4.f * zz - xx - yy);
        B[14] = kSH_C3[5] * z * (xx - yy); B[15] = kSH_C3[6] * x * (xx - 3.f * yy);
      }
    }
  }
}

// d(basis)/d(dir) for the backward of the view-dependent colour
__device__ __forceinline__ void sh_basis_grad(int deg, float3 d, float* Bx, float* By, float* Bz) {
  const float x = d.x, y = d.y, z = d.z;
  Bx[0] = By[0] = Bz[0] = 0.f;
  if (deg > 0) {
    Bx[1] = 0.f; By[1] = -kSH_C1; Bz[1] = 0.f;
    Bx[2] = 0.f; By[2] = 0.f; Bz[2] = kSH_C1;
    Bx[3] = -kSH_C1; By[3] = 0.f; Bz[3] = 0.f;
    if (deg > 1) {
      Bx[4] = kSH_C2[0] * y; By[4] = kSH_C2[0] * x; Bz[4] = 0.f;
      Bx[5] = 0.f; By[5] = kSH_C2[1] * z; Bz[5] = kSH_C2[1] * y;
      Bx[6] = kSH_C2[2] * -2.f * x; By[6] = kSH_C2[2] * -2.f * y; Bz[6] = kSH_C2[2] * 4.f * z;
      Bx[7] = kSH_C2[3] * z; By[7] = 0.f; Bz[7] = kSH_C2[3] * x;
      Bx[8] = kSH_C2[4] * 2.f * x; By[8] = kSH_C2[4] * -2.f * y; Bz[8] = 0.f;
      if (deg > 2) {
        const float xx = x * x, yy = y * y, zz = z * z;
        Bx[9] = kSH_C3[0] * 6.f * x * y; By[9] = kSH_C3[0] * (3.f * xx - 3.f * yy); Bz[9] = 0.f;
        Bx[10] = kSH_C3[1] * y * z; By[10] = kSH_C3[1] * x * z; Bz[10] = kSH_C3[1] * x * y;
        Bx[11] = kSH_C3[2] * -2.f * x * y; By[11] = kSH_C3[2] * (4.f * zz - xx - 3.f * yy); Bz[11] = kSH_C3[2] * 8.f * y * z;
        Bx[12] = kSH_C3[3] * -6.f * x * z; By[12] = kSH_C3[3] * -6.f * y * z; Bz[12] = kSH_C3[3] * (6.f * zz - 3.f * xx - 3.f * yy);
        Bx[13] = kSH_C3[4] * (4.f * zz - 3.f * xx - yy); By[13] = kSH_C3[4] * -2.f * x * y; Bz[13] = kSH_C3[4] * 8.f * x * z;
        Bx[14] = kSH_C3[5] * 2.f * x * z; By[14] = kSH_C3[5] * -2.f * y * z; Bz[14] = kSH_C3[5] * (xx - yy);
        Bx[15] = kSH_C3[6] * (3.f * xx - 3.f * yy); By[15] = kSH_C3[6] * -6.f * x * y; Bz[15] = 0.f;
      }
    }
  }
}

__device__ __forceinline__ void tile_rect(float2 p, int r, int tiles_x, int tiles_y, int& x0, int& y0, int& x1, int& y1) {
  x0 = min(tiles_x, max(0, (int)((p.x - r) / kTile)));
  y0 = min(tiles_y, max(0, (int)((p.y - r) / kTile)));
  x1 = min(tiles_x, max(0, (int)((p.x + r + kTile - 1) / kTile)));
  y1 = min(tiles_y, max(0, (int)((p.y + r + kTile - 1) / kTile)));
}

// ---- preprocess ------------------------------------------------------------------------------------------
// visible: optional per-Gaussian byte mask (0 = skip).  shs: [N, sh_coeffs, 3] or null (then colors_pre [N,3]).
// cov3d_pre: optional [N, 6].  Outputs are per Gaussian; radii == 0 marks "not rendered".
__global__ void __launch_bounds__(256)
gs_preprocess_kernel(int N, const float* __restrict__ means, const float* __restrict__ scales, const float* __restrict__ rots,
                     const float* __restrict__ opac, const float* __restrict__ shs, const float* __restrict__ colors_pre,
                     const float* __restrict__ cov3d_pre, const unsigned char* __restrict__ visible, GSCamera cam,
                     int* __restrict__ radii, float2* __restrict__ xy, float* __restrict__ depth, float* __restrict__ cov3d,
                     float4* __restrict__ conic_op, float* __restrict__ rgb, unsigned char* __restrict__ clamped,
                     uint32_t* __restrict__ tiles_touched, int radius_only) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N) return;
  radii[i] = 0;
  if (tiles_touched) tiles_touched[i] = 0;
  if (visible && !visible[i]) return;
  const float3 p = make_float3(means[3 * i], means[3 * i + 1], means[3 * i + 2]);
  const float3 t = xform43(cam.view, p);
  if (t.z <= 0.2f) return;
  const float4 ph = xform44(cam.proj, p);
  const float pw = 1.f / (ph.w + 1e-7f);
  const float2 ndc = make_float2(ph.x * pw, ph.y * pw);
  float c3[6];
  if (cov3d_pre) {
#pragma unroll
    for (int k = 0; k < 6; ++k) c3[k] = cov3d_pre[6 * i + k];
  } else {
    const float3 s = make_float3(scales[3 * i] * cam.scale_modifier, scales[3 * i + 1] * cam.scale_modifier,
                                 scales[3 * i + 2] * cam.scale_modifier);
    float4 q = make_float4(rots[4 * i], rots[4 * i + 1], rots[4 * i + 2], rots[4 * i + 3]);
    cov3d_from(s, q, c3);
  }
  const float fx = cam.W / (2.f * cam.tanfovx), fy = cam.H / (2.f * cam.tanfovy);
  float T[6], a, b, c;
  project_cov(cam, t, c3, fx, fy, T, a, b, c);
  a += 0.3f; c += 0.3f;
  const float det = a * c - b * b;
  if (det == 0.f) return;
  const float inv = 1.f / det;
  const float mid = 0.5f * (a + c);
  const float lam = mid + sqrtf(fmaxf(0.1f, mid * mid - det));
  const int r = (int)ceilf(3.f * sqrtf(lam));
  const float2 pix = make_float2(((ndc.x + 1.f) * cam.W - 1.f) * 0.5f, ((ndc.y + 1.f) * cam.H - 1.f) * 0.5f);
  const int tiles_x = (cam.W + kTile - 1) / kTile, tiles_y = (cam.H + kTile - 1) / kTile;
  int x0, y0, x1, y1;
  tile_rect(pix, r, tiles_x, tiles_y, x0, y0, x1, y1);
  if ((x1 - x0) * (y1 - y0) == 0) return;
  radii[i] = r;
  if (radius_only) return;
  if (cov3d) {
#pragma unroll
    for (int k = 0; k < 6; ++k) cov3d[6 * i + k] = c3[k];
  }
  float col[3];
  if (shs) {
    float3 d = make_float3(p.x - cam.campos[0], p.y - cam.campos[1], p.z - cam.campos[2]);
    const float n = rsqrtf(d.x * d.x + d.y * d.y + d.z * d.z);
    d.x *= n; d.y *= n; d.z *= n;
    float B[16];
    sh_basis(cam.sh_degree, d, B);
    const int nb = (cam.sh_degree + 1) * (cam.sh_degree + 1);
    const float* sh = shs + (long long)i * cam.sh_coeffs * 3;
#pragma unroll
    for (int ch = 0; ch < 3; ++ch) {
      float v = 0.5f;
      for (int k = 0; k < nb; ++k) v += B[k] * sh[k * 3 + ch];
      clamped[3 * i + ch] = v < 0.f;
      col[ch] = fmaxf(v, 0.f);
    }
  } else {
#pragma unroll
    for (int ch = 0; ch < 3; ++ch) col[ch] = colors_pre[3 * i + ch];
  }
  rgb[3 * i] = col[0]; rgb[3 * i + 1] = col[1]; rgb[3 * i + 2] = col[2];
  depth[i] = t.z;
  xy[i] = pix;
  conic_op[i] = make_float4(c * inv, -b * inv, a * inv, opac[i]);
  tiles_touched[i] = (uint32_t)((x1 - x0) * (y1 - y0));
}

__global__ void __launch_bounds__(256)
gs_make_keys_kernel(int N, const float2* __restrict__ xy, const float* __restrict__ depth, const int* __restrict__ radii,
                    const uint32_t* __restrict__ offsets, int W, int H, long long capacity, uint64_t* __restrict__ keys,
                    uint32_t* __restrict__ vals) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N || radii[i] <= 0) return;
  const int tiles_x = (W + kTile - 1) / kTile, tiles_y = (H + kTile - 1) / kTile;
  int x0, y0, x1, y1;
  tile_rect(xy[i], radii[i], tiles_x, tiles_y, x0, y0, x1, y1);
  long long off = offsets[i];
  const uint64_t dbits = (uint64_t)__float_as_uint(depth[i]);
  for (int y = y0; y < y1; ++y)
    for (int x = x0; x < x1; ++x) {
      if (off >= capacity) return;
      keys[off] = ((uint64_t)(y * tiles_x + x) << 32) | dbits;
      vals[off] = (uint32_t)i;
      ++off;
    }
}

__global__ void __launch_bounds__(256)
gs_tile_ranges_kernel(const uint64_t* __restrict__ keys, const int* __restrict__ count_ptr, long long capacity,
                      uint2* __restrict__ ranges) {
  const long long n = resolve_count(count_ptr, capacity);
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint32_t tile = (uint32_t)(keys[i] >> 32);
  if (i == 0) ranges[tile].x = 0;
  else {
    const uint32_t prev = (uint32_t)(keys[i - 1] >> 32);
    if (prev != tile) { ranges[prev].y = (uint32_t)i; ranges[tile].x = (uint32_t)i; }
  }
  if (i == n - 1) ranges[tile].y = (uint32_t)n;
}

// total = offsets[N-1] + tiles_touched[N-1], clamped to capacity, kept on the device
__global__ void gs_total_kernel(int N, const uint32_t* offsets, const uint32_t* touched, long long capacity, int* total,
                                int* overflow) {
  long long t = (long long)offsets[N - 1] + touched[N - 1];
  if (t > capacity) { *overflow = 1; t = capacity; }
  *total = (int)t;
}

// ---- tile blending, forward ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(kTilePixels)
gs_render_fwd_kernel(const uint2* __restrict__ ranges, const uint32_t* __restrict__ point_list, int W, int H,
                     const float2* __restrict__ xy, const float* __restrict__ rgb, const float4* __restrict__ conic_op,
                     const float* __restrict__ bg, float* __restrict__ out_color, float* __restrict__ final_T,
                     uint32_t* __restrict__ n_contrib) {
  __shared__ uint32_t s_id[kTilePixels];
  __shared__ float2 s_xy[kTilePixels];
  __shared__ float4 s_co[kTilePixels];
  __shared__ float s_rgb[kTilePixels * 3];
  const int tiles_x = (W + kTile - 1) / kTile;
  const int px = blockIdx.x * kTile + threadIdx.x, py = blockIdx.y * kTile + threadIdx.y;
  const bool inside = px < W && py < H;
  const float2 pixf = make_float2((float)px, (float)py);
  const uint2 range = ranges[blockIdx.y * tiles_x + blockIdx.x];
  const int tid = threadIdx.y * kTile + threadIdx.x;
  bool done = !inside;
  float T = 1.f, C[3] = {0.f, 0.f, 0.f};
  uint32_t contributor = 0, last = 0;
  const int rounds = (int)((range.y - range.x + kTilePixels - 1) / kTilePixels);
  int todo = (int)(range.y - range.x);
  for (int r = 0; r < rounds; ++r, todo -= kTilePixels) {
    if (__syncthreads_count(done) == kTilePixels) break;
    const uint32_t k = range.x + r * kTilePixels + tid;
    if (k < range.y) {
      const uint32_t id = point_list[k];
      s_id[tid] = id; s_xy[tid] = xy[id]; s_co[tid] = conic_op[id];
      s_rgb[3 * tid] = rgb[3 * id]; s_rgb[3 * tid + 1] = rgb[3 * id + 1]; s_rgb[3 * tid + 2] = rgb[3 * id + 2];
    }
    __syncthreads();
    for (int j = 0; !done && j < min(kTilePixels, todo); ++j) {
      ++contributor;
      const float2 d = make_float2(s_xy[j].x - pixf.x, s_xy[j].y - pixf.y);
      const float4 co = s_co[j];
      const float power = -0.5f * (co.x * d.x * d.x + co.z * d.y * d.y) - co.y * d.x * d.y;
      if (power > 0.f) continue;
      const float alpha = fminf(0.99f, co.w * __expf(power));
      if (alpha < 1.f / 255.f) continue;
      const float test_T = T * (1.f - alpha);
      if (test_T < 1e-4f) { done = true; continue; }
      const float w = alpha * T;
      C[0] += s_rgb[3 * j] * w; C[1] += s_rgb[3 * j + 1] * w; C[2] += s_rgb[3 * j + 2] * w;
      T = test_T;
      last = contributor;
    }
  }
  if (inside) {
    const long long pix = (long long)py * W + px;
    final_T[pix] = T;
    n_contrib[pix] = last;
#pragma unroll
    for (int ch = 0; ch < 3; ++ch) out_color[(long long)ch * H * W + pix] = C[ch] + T * bg[ch];
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}

// ---- tile blending, backward ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(kTilePixels)
gs_render_bwd_kernel(const uint2* __restrict__ ranges, const uint32_t* __restrict__ point_list, int W, int H,
                     const float* __restrict__ bg, const float2* __restrict__ xy, const float4* __restrict__ conic_op,
                     const float* __restrict__ rgb, const float* __restrict__ final_T, const uint32_t* __restrict__ n_contrib,
                     const float* __restrict__ dL_dpix, float* __restrict__ dL_dmean2D, float* __restrict__ dL_dconic,
                     float* __restrict__ dL_dopacity, float* __restrict__ dL_dcolor) {
  __shared__ uint32_t s_id[kTilePixels];
  __shared__ float2 s_xy[kTilePixels];
  __shared__ float4 s_co[kTilePixels];
  __shared__ float s_rgb[kTilePixels * 3];
  const int tiles_x = (W + kTile - 1) / kTile;
  const int px = blockIdx.x * kTile + threadIdx.x, py = blockIdx.y * kTile + threadIdx.y;
  const bool inside = px < W && py < H;
  const long long pix = (long long)py * W + px;
  const float2 pixf = make_float2((float)px, (float)py);
  const uint2 range = ranges[blockIdx.y * tiles_x + blockIdx.x];
  const int tid = threadIdx.y * kTile + threadIdx.x;
  const int lane = tid & 31;
  const int rounds = (int)((range.y - range.x + kTilePixels - 1) / kTilePixels);
  int todo = (int)(range.y - range.x);
  const float T_final = inside ? final_T[pix] : 0.f;
  float T = T_final;
  uint32_t contributor = (uint32_t)todo;
  const uint32_t last = inside ? n_contrib[pix] : 0;
  float accum[3] = {0.f, 0.f, 0.f}, dpix[3] = {0.f, 0.f, 0.f}, last_color[3] = {0.f, 0.f, 0.f};
  float last_alpha = 0.f;
  if (inside) {
#pragma unroll
    for (int ch = 0; ch < 3; ++ch) dpix[ch] = dL_dpix[(long long)ch * H * W + pix];
  }
  const float ddelx_dx = 0.5f * W, ddely_dy = 0.5f * H;
  for (int r = 0; r < rounds; ++r, todo -= kTilePixels) {
    __syncthreads();
    const long long k = (long long)range.y - 1 - (long long)r * kTilePixels - tid;   // back to front
    if (k >= (long long)range.x) {
      const uint32_t id = point_list[k];
      s_id[tid] = id; s_xy[tid] = xy[id]; s_co[tid] = conic_op[id];
      s_rgb[3 * tid] = rgb[3 * id]; s_rgb[3 * tid + 1] = rgb[3 * id + 1]; s_rgb[3 * tid + 2] = rgb[3 * id + 2];
    }
    __syncthreads();
    const int batch = min(kTilePixels, todo);
    for (int j = 0; j < batch; ++j) {
      --contributor;
      float g_col[3] = {0.f, 0.f, 0.f}, g_mx = 0.f, g_my = 0.f, g_ca = 0.f, g_cb = 0.f, g_cc = 0.f, g_op = 0.f;
      bool active = inside && contributor < last;
      float2 d; float4 co; float G = 0.f, alpha = 0.f;
      if (active) {
        d = make_float2(s_xy[j].x - pixf.x, s_xy[j].y - pixf.y);
        co = s_co[j];
        const float power = -0.5f * (co.x * d.x * d.x + co.z * d.y * d.y) - co.y * d.x * d.y;
        if (power > 0.f) active = false;
        else {
          G = __expf(power);
          alpha = fminf(0.99f, co.w * G);
          if (alpha < 1.f / 255.f) active = false;
        }
      }
      if (active) {
        T = T / (1.f - alpha);
        const float dchannel_dcolor = alpha * T;
        float dL_dalpha = 0.f;
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) {
          const float c = s_rgb[3 * j + ch];
          accum[ch] = last_alpha * last_color[ch] + (1.f - last_alpha) * accum[ch];
          last_color[ch] = c;
          dL_dalpha += (c - accum[ch]) * dpix[ch];
          g_col[ch] = dchannel_dcolor * dpix[ch];
        }
        dL_dalpha *= T;
        last_alpha = alpha;
        float bg_dot = 0.f;
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) bg_dot += bg[ch] * dpix[ch];
        dL_dalpha += (-T_final / (1.f - alpha)) * bg_dot;
        const float dL_dG = co.w * dL_dalpha * (co.w * G <= 0.99f ? 1.f : 0.f);
        const float gdx = G * d.x, gdy = G * d.y;
        const float dG_ddelx = -gdx * co.x - gdy * co.y, dG_ddely = -gdy * co.z - gdx * co.y;
        g_mx = dL_dG * dG_ddelx * ddelx_dx;
        g_my = dL_dG * dG_ddely * ddely_dy;
        g_ca = -0.5f * gdx * d.x * dL_dG;
        g_cb = -0.5f * gdx * d.y * dL_dG;
        g_cc = -0.5f * gdy * d.y * dL_dG;
        g_op = G * dL_dalpha * (co.w * G <= 0.99f ? 1.f : 0.f);
      }
      if (__any_sync(0xffffffffu, active)) {
        g_col[0] = warp_sum(g_col[0]); g_col[1] = warp_sum(g_col[1]); g_col[2] = warp_sum(g_col[2]);
        g_mx = warp_sum(g_mx); g_my = warp_sum(g_my); g_ca = warp_sum(g_ca); g_cb = warp_sum(g_cb);
        g_cc = warp_sum(g_cc); g_op = warp_sum(g_op);
        if (lane == 0) {
          const uint32_t id = s_id[j];
          atomicAdd(&dL_dcolor[3 * id], g_col[0]); atomicAdd(&dL_dcolor[3 * id + 1], g_col[1]);
          atomicAdd(&dL_dcolor[3 * id + 2], g_col[2]);
          atomicAdd(&dL_dmean2D[2 * id], g_mx); atomicAdd(&dL_dmean2D[2 * id + 1], g_my);
          atomicAdd(&dL_dconic[3 * id], g_ca); atomicAdd(&dL_dconic[3 * id + 1], g_cb); atomicAdd(&dL_dconic[3 * id + 2], g_cc);
          atomicAdd(&dL_dopacity[id], g_op);
        }
      }
    }
  }
}

// ---- preprocess backward -----------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gs_preprocess_bwd_kernel(int N, const float* __restrict__ means, const float* __restrict__ scales, const float* __restrict__ rots,
                         const float* __restrict__ shs, const float* __restrict__ cov3d, const int* __restrict__ radii,
                         const unsigned char* __restrict__ clamped, GSCamera cam, const float* __restrict__ dL_dmean2D,
                         const float* __restrict__ dL_dconic, const float* __restrict__ dL_dcolor_in,
                         float* __restrict__ dL_dmeans, float* __restrict__ dL_dscales, float* __restrict__ dL_drots,
                         float* __restrict__ dL_dshs, float* __restrict__ dL_dcolors_pre, int have_scale_rot) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N || radii[i] <= 0) return;
  const float3 p = make_float3(means[3 * i], means[3 * i + 1], means[3 * i + 2]);
  const float3 t = xform43(cam.view, p);
  const float fx = cam.W / (2.f * cam.tanfovx), fy = cam.H / (2.f * cam.tanfovy);
  float c3[6];
#pragma unroll
  for (int k = 0; k < 6; ++k) c3[k] = cov3d[6 * i + k];
  float T[6], a, b, c;
  project_cov(cam, t, c3, fx, fy, T, a, b, c);
  a += 0.3f; c += 0.3f;
  const float denom = a * c - b * b;
  const float denom2inv = 1.f / (denom * denom + 1e-7f);
  const float gcx = dL_dconic[3 * i], gcy = dL_dconic[3 * i + 1], gcz = dL_dconic[3 * i + 2];
  float dL_da = 0.f, dL_db = 0.f, dL_dc = 0.f;
  float dL_dcov[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  float dT[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (denom2inv != 0.f) {
    // conic = (c, -b, a) / denom
    dL_da = denom2inv * (-c * c * gcx + 2.f * b * c * gcy + (denom - a * c) * gcz);
    dL_dc = denom2inv * (-a * a * gcz + 2.f * a * b * gcy + (denom - a * c) * gcx);
    dL_db = denom2inv * 2.f * (b * c * gcx - (denom + 2.f * b * b) * gcy + a * b * gcz);
    // cov2D = T Sigma T^T  ->  d/dSigma
    dL_dcov[0] = T[0] * T[0] * dL_da + T[0] * T[3] * dL_db + T[3] * T[3] * dL_dc;
    dL_dcov[3] = T[1] * T[1] * dL_da + T[1] * T[4] * dL_db + T[4] * T[4] * dL_dc;
    dL_dcov[5] = T[2] * T[2] * dL_da + T[2] * T[5] * dL_db + T[5] * T[5] * dL_dc;
    dL_dcov[1] = 2.f * T[0] * T[1] * dL_da + (T[0] * T[4] + T[1] * T[3]) * dL_db + 2.f * T[3] * T[4] * dL_dc;
    dL_dcov[2] = 2.f * T[0] * T[2] * dL_da + (T[0] * T[5] + T[2] * T[3]) * dL_db + 2.f * T[3] * T[5] * dL_dc;
    dL_dcov[4] = 2.f * T[2] * T[1] * dL_da + (T[1] * T[5] + T[2] * T[4]) * dL_db + 2.f * T[4] * T[5] * dL_dc;
    // d/dT
    const float S0[3] = {c3[0], c3[1], c3[2]}, S1[3] = {c3[1], c3[3], c3[4]}, S2[3] = {c3[2], c3[4], c3[5]};
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      const float st0 = S0[k] * T[0] + S1[k] * T[1] + S2[k] * T[2];   // (Sigma T0^T)_k
      const float st1 = S0[k] * T[3] + S1[k] * T[4] + S2[k] * T[5];
      dT[k] = 2.f * st0 * dL_da + st1 * dL_db;
      dT[3 + k] = 2.f * st1 * dL_dc + st0 * dL_db;
    }
  }
  // T = J Wr ; J entries: j00 = fx/tz, j02 = -fx*txz/tz^2, j11 = fy/tz, j12 = -fy*tyz/tz^2
  const float* v = cam.view;
  const float dJ00 = v[0] * dT[0] + v[4] * dT[1] + v[8] * dT[2];
  const float dJ02 = v[2] * dT[0] + v[6] * dT[1] + v[10] * dT[2];
  const float dJ11 = v[1] * dT[3] + v[5] * dT[4] + v[9] * dT[5];
  const float dJ12 = v[2] * dT[3] + v[6] * dT[4] + v[10] * dT[5];
  const float limx = 1.3f * cam.tanfovx, limy = 1.3f * cam.tanfovy;
  const float rx = t.x / t.z, ry = t.y / t.z;
  const float txz = fminf(limx, fmaxf(-limx, rx)) * t.z, tyz = fminf(limy, fmaxf(-limy, ry)) * t.z;
  const float x_grad_mul = (rx < -limx || rx > limx) ? 0.f : 1.f;
  const float y_grad_mul = (ry < -limy || ry > limy) ? 0.f : 1.f;
  const float tz = 1.f / t.z, tz2 = tz * tz, tz3 = tz2 * tz;
  const float dL_dtx = x_grad_mul * -fx * tz2 * dJ02;
  const float dL_dty = y_grad_mul * -fy * tz2 * dJ12;
  const float dL_dtz = -fx * tz2 * dJ00 - fy * tz2 * dJ11 + (2.f * fx * txz) * tz3 * dJ02 + (2.f * fy * tyz) * tz3 * dJ12;
  // view = [p 1] @ V -> d p_j = sum_i V[j*4+i] d t_i
  float3 dmean = make_float3(v[0] * dL_dtx + v[1] * dL_dty + v[2] * dL_dtz, v[4] * dL_dtx + v[5] * dL_dty + v[6] * dL_dtz,
                             v[8] * dL_dtx + v[9] * dL_dty + v[10] * dL_dtz);
  // screen-space mean gradient through the projection
  {
    const float4 mh = xform44(cam.proj, p);
    const float mw = 1.f / (mh.w + 1e-7f);
    const float* m = cam.proj;
    const float gx = dL_dmean2D[2 * i], gy = dL_dmean2D[2 * i + 1];
    const float mul1 = (m[0] * p.x + m[4] * p.y + m[8] * p.z + m[12]) * mw * mw;
    const float mul2 = (m[1] * p.x + m[5] * p.y + m[9] * p.z + m[13]) * mw * mw;
    dmean.x += (m[0] * mw - m[3] * mul1) * gx + (m[1] * mw - m[3] * mul2) * gy;
    dmean.y += (m[4] * mw - m[7] * mul1) * gx + (m[5] * mw - m[7] * mul2) * gy;
    dmean.z += (m[8] * mw - m[11] * mul1) * gx + (m[9] * mw - m[11] * mul2) * gy;
  }
  // colour
  if (shs) {
    float3 dir0 = make_float3(p.x - cam.campos[0], p.y - cam.campos[1], p.z - cam.campos[2]);
    const float n2 = dir0.x * dir0.x + dir0.y * dir0.y + dir0.z * dir0.z;
    const float invn = rsqrtf(n2);
    const float3 d = make_float3(dir0.x * invn, dir0.y * invn, dir0.z * invn);
    float B[16], Bx[16], By[16], Bz[16];
    sh_basis(cam.sh_degree, d, B);
    sh_basis_grad(cam.sh_degree, d, Bx, By, Bz);
    const int nb = (cam.sh_degree + 1) * (cam.sh_degree + 1);
    const float* sh = shs + (long long)i * cam.sh_coeffs * 3;
    float* dsh = dL_dshs + (long long)i * cam.sh_coeffs * 3;
    float3 ddir = make_float3(0.f, 0.f, 0.f);
#pragma unroll
    for (int ch = 0; ch < 3; ++ch) {
      const float g = clamped[3 * i + ch] ? 0.f : dL_dcolor_in[3 * i + ch];
      for (int k = 0; k < nb; ++k) {
        dsh[k * 3 + ch] = B[k] * g;
        const float s = sh[k * 3 + ch] * g;
        ddir.x += Bx[k] * s; ddir.y += By[k] * s; ddir.z += Bz[k] * s;
      }
    }
    // backward of normalisation: (I - d d^T) / |dir0|
    const float dot = d.x * ddir.x + d.y * ddir.y + d.z * ddir.z;
    dmean.x += (ddir.x - d.x * dot) * invn; dmean.y += (ddir.y - d.y * dot) * invn; dmean.z += (ddir.z - d.z * dot) * invn;
  } else if (dL_dcolors_pre) {
#pragma unroll
    for (int ch = 0; ch < 3; ++ch) dL_dcolors_pre[3 * i + ch] = dL_dcolor_in[3 * i + ch];
  }
  dL_dmeans[3 * i] = dmean.x; dL_dmeans[3 * i + 1] = dmean.y; dL_dmeans[3 * i + 2] = dmean.z;
  if (!have_scale_rot) return;
  // Sigma = M M^T with M = R diag(s): dL/dM = 2 * dSigma_sym * M
  const float3 s = make_float3(scales[3 * i] * cam.scale_modifier, scales[3 * i + 1] * cam.scale_modifier,
                               scales[3 * i + 2] * cam.scale_modifier);
  const float4 q0 = make_float4(rots[4 * i], rots[4 * i + 1], rots[4 * i + 2], rots[4 * i + 3]);
  float R[9];
  quat_to_rot(q0, R);
  // symmetric dSigma with off-diagonals halved (each appears twice in the full matrix)
  const float D[9] = {dL_dcov[0], 0.5f * dL_dcov[1], 0.5f * dL_dcov[2], 0.5f * dL_dcov[1], dL_dcov[3], 0.5f * dL_dcov[4],
                      0.5f * dL_dcov[2], 0.5f * dL_dcov[4], dL_dcov[5]};
  const float sv[3] = {s.x, s.y, s.z};
  float dM[9];   // dL/dM, M[r][c] = R[r][c] * s[c]
#pragma unroll
  for (int r = 0; r < 3; ++r)
#pragma unroll
    for (int cc = 0; cc < 3; ++cc) {
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < 3; ++k) acc += D[r * 3 + k] * R[k * 3 + cc] * sv[cc];
      dM[r * 3 + cc] = 2.f * acc;
    }
  float ds[3], dR[9];
#pragma unroll
  for (int cc = 0; cc < 3; ++cc) {
    ds[cc] = (R[cc] * dM[cc] + R[3 + cc] * dM[3 + cc] + R[6 + cc] * dM[6 + cc]) * cam.scale_modifier;
#pragma unroll
    for (int r = 0; r < 3; ++r) dR[r * 3 + cc] = dM[r * 3 + cc] * sv[cc];
  }
  dL_dscales[3 * i] = ds[0]; dL_dscales[3 * i + 1] = ds[1]; dL_dscales[3 * i + 2] = ds[2];
  const float r = q0.x, x = q0.y, y = q0.z, z = q0.w;
  float4 dq;
  dq.x = 2.f * (-z * dR[1] + y * dR[2] + z * dR[3] - x * dR[5] - y * dR[6] + x * dR[7]);
  dq.y = 2.f * (y * dR[1] + z * dR[2] + y * dR[3] - 2.f * x * dR[4] - r * dR[5] + z * dR[6] + r * dR[7] - 2.f * x * dR[8]);
  dq.z = 2.f * (-2.f * y * dR[0] + x * dR[1] + r * dR[2] + x * dR[3] + z * dR[5] - r * dR[6] + z * dR[7] - 2.f * y * dR[8]);
  dq.w = 2.f * (-2.f * z * dR[0] - r * dR[1] + x * dR[2] + r * dR[3] - 2.f * z * dR[4] + y * dR[5] + x * dR[6] + y * dR[7]);
  dL_drots[4 * i] = dq.x; dL_drots[4 * i + 1] = dq.y; dL_drots[4 * i + 2] = dq.z; dL_drots[4 * i + 3] = dq.w;
}

}  // namespace lmb

using namespace lmb;

LMB_API int lmb_gs_preprocess(int N, const float* means, const float* scales, const float* rots, const float* opac,
                              const float* shs, const float* colors_pre, const float* cov3d_pre,
                              const unsigned char* visible, const GSCamera* cam, int* radii, float* xy, float* depth,
                              float* cov3d, float* conic_op, float* rgb, unsigned char* clamped, uint32_t* tiles_touched,
                              int radius_only, cudaStream_t stream) {
  if (N <= 0) return 0;
  gs_preprocess_kernel<<<ceil_div(N, 256), 256, 0, stream>>>(N, means, scales, rots, opac, shs, colors_pre, cov3d_pre, visible,
                                                            *cam, radii, (float2*)xy, depth, cov3d, (float4*)conic_op, rgb,
                                                            clamped, tiles_touched, radius_only);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_gs_make_keys(int N, const float* xy, const float* depth, const int* radii, const uint32_t* offsets,
                             const uint32_t* touched, int W, int H, long long capacity, uint64_t* keys, uint32_t* vals,
                             int* total, int* overflow, cudaStream_t stream) {
  if (N <= 0) return 0;
  gs_total_kernel<<<1, 1, 0, stream>>>(N, offsets, touched, capacity, total, overflow);
  gs_make_keys_kernel<<<ceil_div(N, 256), 256, 0, stream>>>(N, (const float2*)xy, depth, radii, offsets, W, H, capacity, keys, vals);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_gs_tile_ranges(const uint64_t* keys, const int* count_ptr, long long capacity, uint32_t* ranges, int n_tiles,
                               cudaStream_t stream) {
  LMB_CUDA_TRY(cudaMemsetAsync(ranges, 0, (size_t)n_tiles * 8, stream));
  if (capacity <= 0) return 0;
  gs_tile_ranges_kernel<<<ceil_div(capacity, 256), 256, 0, stream>>>(keys, count_ptr, capacity, (uint2*)ranges);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_gs_render_fwd(const uint32_t* ranges, const uint32_t* point_list, int W, int H, const float* xy,
                              const float* rgb, const float* conic_op, const float* bg, float* out_color, float* final_T,
                              uint32_t* n_contrib, cudaStream_t stream) {
  dim3 grid((W + kTile - 1) / kTile, (H + kTile - 1) / kTile), block(kTile, kTile);
  gs_render_fwd_kernel<<<grid, block, 0, stream>>>((const uint2*)ranges, point_list, W, H, (const float2*)xy, rgb,
                                                  (const float4*)conic_op, bg, out_color, final_T, n_contrib);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_gs_render_bwd(const uint32_t* ranges, const uint32_t* point_list, int W, int H, const float* bg, const float* xy,
                              const float* conic_op, const float* rgb, const float* final_T, const uint32_t* n_contrib,
                              const float* dL_dpix, float* dL_dmean2D, float* dL_dconic, float* dL_dopacity, float* dL_dcolor,
                              cudaStream_t stream) {
  dim3 grid((W + kTile - 1) / kTile, (H + kTile - 1) / kTile), block(kTile, kTile);
  gs_render_bwd_kernel<<<grid, block, 0, stream>>>((const uint2*)ranges, point_list, W, H, bg, (const float2*)xy,
                                                  (const float4*)conic_op, rgb, final_T, n_contrib, dL_dpix, dL_dmean2D,
                                                  dL_dconic, dL_dopacity, dL_dcolor);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_gs_preprocess_bwd(int N, const float* means, const float* scales, const float* rots, const float* shs,
                                  const float* cov3d, const int* radii, const unsigned char* clamped, const GSCamera* cam,
                                  const float* dL_dmean2D, const float* dL_dconic, const float* dL_dcolor, float* dL_dmeans,
                                  float* dL_dscales, float* dL_drots, float* dL_dshs, float* dL_dcolors_pre,
                                  int have_scale_rot, cudaStream_t stream) {
  if (N <= 0) return 0;
  gs_preprocess_bwd_kernel<<<ceil_div(N, 256), 256, 0, stream>>>(N, means, scales, rots, shs, cov3d, radii, clamped, *cam,
                                                               dL_dmean2D, dL_dconic, dL_dcolor, dL_dmeans, dL_dscales,
                                                               dL_drots, dL_dshs, dL_dcolors_pre, have_scale_rot);
  LMB_LAUNCH_CHECK();
  return 0;
}
