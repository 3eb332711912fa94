// Per-sample glue of the hash-grid radiance fields (Instant-NGP, Nerfacto) as kernels:
//
//  * sh_encode_kernel        directions -> real spherical-harmonics basis, degree <= 4.  The reference gets this from
//                            tiny-cuda-nn's "SphericalHarmonics" encoding
//                            (landmark/nerf_components/model_components/fields/encodings/sh_encoding.py:31-38).
//  * ngp_positions_kernel    valid-sample index -> world position -> block-local hash-grid coordinate + inside flag
//                            (benchmarks/nerf/instant_ngp/instant_ngp.py:225-260 builds these with tensor ops).
//  * ngp_head_rows_kernel    density-head output -> sigma (truncated exp) and the colour head's bf16 input row
//                            [SH(dir) | geometry features | appearance embedding | zero tail] in one pass
//                            (instant_ngp.py:262-289: trunc_exp, SH encode, embedding lookup, concatenate).
//  * ngp_head_rows_bwd_kernel the matching backward: gradient of the density-head output, and the appearance
//                            embedding's gradient reduced per ray inside the warp before it touches memory.
//  * occ_* kernels           the occupancy grid's periodic refresh: jittered cell centres, EMA-max update, mean and
//                            threshold (nerfacc's OccGridEstimator.update_every_n_steps in the reference,
//                            instant_ngp.py:316-326).
#include "common.cuh"

namespace lmb {

// ---------------------------------------------------------------------------------------------------------------------
// Real spherical harmonics, the same ordering and constants as the 3DGS colour SH (l = 0..4, m = -l..l).
template <int kLevels>
__device__ __forceinline__ void sh_basis(float x, float y, float z, float* o) {
  o[0] = 0.28209479177387814f;
  if (kLevels > 1) {
    o[1] = -0.4886025119029199f * y;
    o[2] = 0.4886025119029199f * z;
    o[3] = -0.4886025119029199f * x;
  }
  if (kLevels > 2) {
    const float xx = x * x, yy = y * y, zz = z * z, xy = x * y, yz = y * z, xz = x * z;
    o[4] = 1.0925484305920792f * xy;
    o[5] = -1.0925484305920792f * yz;
    o[6] = 0.31539156525252005f * (2.f * zz - xx - yy);
    o[7] = -1.0925484305920792f * xz;
    o[8] = 0.5462742152960396f * (xx - yy);
    if (kLevels > 3) {
      o[9] = -0.5900435899266435f * y * (3.f * xx - yy);
      o[10] = 2.890611442640554f * xy * z;
      o[11] = -0.4570457994644658f * y * (4.f * zz - xx - yy);
      o[12] = 0.3731763325901154f * z * (2.f * zz - 3.f * xx - 3.f * yy);
      o[13] = -0.4570457994644658f * x * (4.f * zz - xx - yy);
      o[14] = 1.445305721320277f * z * (xx - yy);
      o[15] = -0.5900435899266435f * x * (xx - 3.f * yy);
    }
    if (kLevels > 4) {
      o[16] = 2.5033429417967046f * xy * (xx - yy);
      o[17] = -1.7701307697799304f * yz * (3.f * xx - yy);
      o[18] = 0.9461746957575601f * xy * (7.f * zz - 1.f);
      o[19] = -0.6690465435572892f * yz * (7.f * zz - 3.f);
      o[20] = 0.10578554691520431f * (zz * (35.f * zz - 30.f) + 3.f);
      o[21] = -0.6690465435572892f * xz * (7.f * zz - 3.f);
      o[22] = 0.47308734787878004f * (xx - yy) * (7.f * zz - 1.f);
      o[23] = -1.7701307697799304f * xz * (xx - 3.f * yy);
      o[24] = 0.6258357354491761f * (xx * (xx - 3.f * yy) - yy * (3.f * xx - yy));
    }
  }
}

template <int kLevels>
__global__ void __launch_bounds__(256)
sh_encode_kernel(long long n, const float* __restrict__ dirs, int unit_range, float* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float x = dirs[3 * i], y = dirs[3 * i + 1], z = dirs[3 * i + 2];
  if (unit_range) { x = 2.f * x - 1.f; y = 2.f * y - 1.f; z = 2.f * z - 1.f; }
  float o[kLevels * kLevels];
  sh_basis<kLevels>(x, y, z, o);
  float* dst = out + i * (kLevels * kLevels);
  if (kLevels == 4) {
#pragma unroll
    for (int k = 0; k < 4; ++k)
      reinterpret_cast<float4*>(dst)[k] = make_float4(o[4 * k], o[4 * k + 1], o[4 * k + 2], o[4 * k + 3]);
  } else {
#pragma unroll
    for (int k = 0; k < kLevels * kLevels; ++k) dst[k] = o[k];
  }
}

// ---------------------------------------------------------------------------------------------------------------------
struct NgpBox {
  float lo[3], inv_extent[3];
  int nx, ny;          // plane division of the hash tables
  int only_block;      // >= 0: keep samples of this block only and address table 0 (spatial-block training); -1: all
};

// idx == nullptr: sample m is flat sample m (every sample valid).
__global__ void __launch_bounds__(256)
ngp_positions_kernel(long long m_total, const long long* __restrict__ idx, int samples_per_ray,
                     const float* __restrict__ origins, const float* __restrict__ dirs, const float* __restrict__ z_flat,
                     NgpBox box, float* __restrict__ xyzb, unsigned char* __restrict__ inside_out) {
  const long long m = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= m_total) return;
  const long long flat = idx ? idx[m] : m;
  const long long ray = flat / samples_per_ray;
  const float t = z_flat[flat];
  float u[3];
  bool inside = true;
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    const float p = origins[3 * ray + k] + dirs[3 * ray + k] * t;
    u[k] = (p - box.lo[k]) * box.inv_extent[k];
    inside = inside && (u[k] > 0.f) && (u[k] < 1.f);
  }
  float block = 0.f;
  if (box.nx * box.ny > 1) {
    const float a = u[0] * box.nx, b = u[1] * box.ny;
    const float bx = fminf(fmaxf(floorf(a), 0.f), (float)(box.nx - 1));
    const float by = fminf(fmaxf(floorf(b), 0.f), (float)(box.ny - 1));
    u[0] = a - bx; u[1] = b - by;
    block = bx * box.ny + by;
    if (box.only_block >= 0) {
      inside = inside && (block == (float)box.only_block);
      block = 0.f;
    }
  }
  const float keep = inside ? 1.f : 0.f;
  reinterpret_cast<float4*>(xyzb)[m] = make_float4(u[0] * keep, u[1] * keep, u[2] * keep, block);
  inside_out[m] = inside ? 1 : 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// Colour-head input rows.  Row layout (bf16): [0,16) SH basis of the ray's unit direction, [16, 16+G) geometry features,
// [16+G, 16+G+A) appearance embedding of the ray, zeros up to `width` (a multiple of 8).  `h` is the density head's
// output [M, 1+G] fp32: column 0 is the raw density, sigma = exp(h0); the backward uses exp(clamp(h0, -15, 15)) (the
// truncated exponential of the hash-grid fields).
// One thread per row; the row leaves as 16-byte stores.
constexpr int kRowMaxWidth = 64;

__device__ __forceinline__ float trunc_exp_grad(float v) { return expf(fminf(fmaxf(v, -15.f), 15.f)); }

__global__ void __launch_bounds__(256)
ngp_head_rows_kernel(long long m_total, const long long* __restrict__ idx, int samples_per_ray,
                     const float* __restrict__ dirs, const float* __restrict__ h, int geo, const unsigned char* __restrict__ inside,
                     const float* __restrict__ app_ray, int app, int width, __nv_bfloat16* __restrict__ rows,
                     float* __restrict__ sigma) {
  const long long m = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= m_total) return;
  const long long ray = (idx ? idx[m] : m) / samples_per_ray;
  float x = dirs[3 * ray], y = dirs[3 * ray + 1], z = dirs[3 * ray + 2];
  const float inv = rsqrtf(fmaxf(x * x + y * y + z * z, 1e-30f));
  x *= inv; y *= inv; z *= inv;
  float sh[16];
  sh_basis<4>(x, y, z, sh);
  const float keep = inside[m] ? 1.f : 0.f;
  const float* hm = h + m * (1 + geo);
  sigma[m] = expf(hm[0]) * keep;
  __nv_bfloat16* dst = rows + m * width;
#pragma unroll
  for (int k = 0; k < 16; k += 8) {
    F8 v;
#pragma unroll
    for (int j = 0; j < 8; ++j) v.v[j] = sh[k + j];
    store8(dst + k, v);
  }
  for (int k = 16; k < width; k += 8) {
    F8 v;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = k + j - 16;
      float val = 0.f;
      if (c < geo) val = hm[1 + c] * keep;
      else if (c < geo + app && app_ray) val = app_ray[ray * app + (c - geo)];
      v.v[j] = val;
    }
    store8(dst + k, v);
  }
}

// Backward.  d_rows [M, width] bf16 (gradient of the colour head's input), d_sigma [M] fp32.
//   d_h[m, 0]     = d_sigma[m] * exp(clamp(h0, -15, 15)) * inside     (the truncated exp passes its gradient everywhere)
//   d_h[m, 1 + k] = d_rows[m, 16 + k] * inside
//   d_app[ray, k] += d_rows[m, 16 + G + k]   summed over the ray's samples: rows of one ray are consecutive, so a
//   segmented reduction over the warp's 32 rows leaves one atomic per (ray, channel) per warp.
__global__ void __launch_bounds__(256)
ngp_head_rows_bwd_kernel(long long m_total, const long long* __restrict__ idx, int samples_per_ray,
                         const __nv_bfloat16* __restrict__ d_rows, const float* __restrict__ d_sigma,
                         const float* __restrict__ h, int geo, const unsigned char* __restrict__ inside, int app, int width,
                         float* __restrict__ d_h, float* __restrict__ d_app) {
  const long long m = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = m < m_total;
  const int lane = threadIdx.x & 31;
  long long ray = -1;
  const __nv_bfloat16* src = d_rows + m * width;
  if (live) {
    ray = (idx ? idx[m] : m) / samples_per_ray;
    const float keep = inside[m] ? 1.f : 0.f;
    float* dh = d_h + m * (1 + geo);
    dh[0] = d_sigma[m] * trunc_exp_grad(h[m * (1 + geo)]) * keep;
#pragma unroll 1
    for (int k = 0; k < geo; ++k) dh[1 + k] = __bfloat162float(src[16 + k]) * keep;
  }
  if (d_app == nullptr) return;
  const long long prev_ray = __shfl_up_sync(0xffffffffu, ray, 1);
  const bool head = live && (lane == 0 || prev_ray != ray);
  // eight appearance channels at a time: segmented suffix sums over equal, consecutive ray ids
  for (int c0 = 0; c0 < app; c0 += 8) {
    float ga[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) ga[k] = (live && c0 + k < app) ? __bfloat162float(src[16 + geo + c0 + k]) : 0.f;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const long long other_ray = __shfl_down_sync(0xffffffffu, ray, off);
      const bool take = (lane + off < 32) && (other_ray == ray);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float o = __shfl_down_sync(0xffffffffu, ga[k], off);
        if (take) ga[k] += o;
      }
    }
    if (head) {
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (c0 + k < app) atomicAdd(d_app + ray * app + c0 + k, ga[k]);
    }
  }
}

// The same backward for the shape the shipped configurations use - 15 geometry features, rows of 64 columns (up to
// 33 appearance channels): the row's gradient arrives as six 16-byte loads and d_h leaves as four, all register
// indices are compile-time constants.
__global__ void __launch_bounds__(256)
ngp_head_rows_bwd_g15w64_kernel(long long m_total, const long long* __restrict__ idx, int samples_per_ray,
                                const __nv_bfloat16* __restrict__ d_rows, const float* __restrict__ d_sigma,
                                const float* __restrict__ h, const unsigned char* __restrict__ inside, int app,
                                float* __restrict__ d_h, float* __restrict__ d_app) {
  constexpr int kGeo = 15, kWidth = 64;
  const long long m = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = m < m_total;
  const int lane = threadIdx.x & 31;
  long long ray = -1;
  float v[48];                                     // columns 16 .. 63 of the row
#pragma unroll
  for (int i = 0; i < 48; ++i) v[i] = 0.f;
  if (live) {
    ray = (idx ? idx[m] : m) / samples_per_ray;
    const __nv_bfloat16* src = d_rows + m * kWidth + 16;
#pragma unroll
    for (int c = 0; c < 6; ++c) {
      const F8 f = load8(src + 8 * c);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[8 * c + j] = f.v[j];
    }
    const float keep = inside[m] ? 1.f : 0.f;
    float4* dh = reinterpret_cast<float4*>(d_h + m * 16);
    dh[0] = make_float4(d_sigma[m] * trunc_exp_grad(h[m * 16]) * keep, v[0] * keep, v[1] * keep, v[2] * keep);
    dh[1] = make_float4(v[3] * keep, v[4] * keep, v[5] * keep, v[6] * keep);
    dh[2] = make_float4(v[7] * keep, v[8] * keep, v[9] * keep, v[10] * keep);
    dh[3] = make_float4(v[11] * keep, v[12] * keep, v[13] * keep, v[14] * keep);
  }
  if (d_app == nullptr) return;
  const long long prev_ray = __shfl_up_sync(0xffffffffu, ray, 1);
  const bool head = live && (lane == 0 || prev_ray != ray);
  bool take[5];
#pragma unroll
  for (int s = 0; s < 5; ++s) {
    const long long other_ray = __shfl_down_sync(0xffffffffu, ray, 1 << s);
    take[s] = (lane + (1 << s) < 32) && (other_ray == ray);
  }
#pragma unroll
  for (int k = 0; k < 33; ++k) {
    if (k < app) {                                 // uniform across the grid
      float g = v[kGeo + k];
#pragma unroll
      for (int s = 0; s < 5; ++s) {
        const float o = __shfl_down_sync(0xffffffffu, g, 1 << s);
        if (take[s]) g += o;
      }
      if (head) atomicAdd(d_app + ray * app + k, g);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Occupancy grid refresh.
struct OccRoi { float centre[3], half[3]; };

__device__ __forceinline__ unsigned hash_u32(unsigned v) {
  v ^= v >> 16; v *= 0x7feb352dU; v ^= v >> 15; v *= 0x846ca68bU; v ^= v >> 16;
  return v;
}

// Cell index -> jittered world position inside the cell (cascade `level` spans the region scaled by 2^level), and the
// cell's decayed previous value.  idx == nullptr: cell i is cell i.
__global__ void __launch_bounds__(256)
occ_cells_kernel(long long n, const long long* __restrict__ idx, int res, OccRoi roi, float level_scale, unsigned seed,
                 int jitter, const float* __restrict__ occs_level, float decay, float* __restrict__ xyz,
                 float* __restrict__ decayed) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long cell = idx ? idx[i] : i;
  const int c[3] = {(int)(cell / ((long long)res * res)), (int)((cell / res) % res), (int)(cell % res)};
  unsigned s = hash_u32(seed ^ hash_u32((unsigned)i * 3u + 0x9e3779b9u));
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    s = hash_u32(s + (unsigned)k);
    const float r = jitter ? (float)(s >> 8) * (1.f / 16777216.f) : 0.5f;
    const float u = ((float)c[k] + r) / (float)res;
    xyz[3 * i + k] = roi.centre[k] + (2.f * u - 1.f) * roi.half[k] * level_scale;
  }
  decayed[i] = occs_level[cell] * decay;
}

// Pass 1 of the update: every sampled cell takes its decayed value (duplicates store the same number).
__global__ void __launch_bounds__(256)
occ_store_decayed_kernel(long long n, const long long* __restrict__ idx, const float* __restrict__ decayed,
                         float* __restrict__ occs_level) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  occs_level[idx ? idx[i] : i] = decayed[i];
}

// Pass 2: maximum with the fresh estimates.  Values are non-negative, so the integer maximum orders them; a cell that
// was sampled twice ends with the larger estimate whatever the order.
__global__ void __launch_bounds__(256)
occ_max_kernel(long long n, const long long* __restrict__ idx, const float* __restrict__ fresh, float* __restrict__ occs_level) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = fmaxf(fresh[i], 0.f);
  atomicMax(reinterpret_cast<int*>(occs_level + (idx ? idx[i] : i)), __float_as_int(v));
}

__global__ void __launch_bounds__(256)
occ_sum_kernel(long long n, const float* __restrict__ occs, double* __restrict__ sum) {
  double acc = 0.0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    acc += occs[i];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, off);
  __shared__ double part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += part[w];
    atomicAdd(sum, t);
  }
}

// binaries = occs > min(mean, threshold); the mean comes from the device-side sum, so the refresh needs no host read.
__global__ void __launch_bounds__(256)
occ_threshold_kernel(long long n, const float* __restrict__ occs, const double* __restrict__ sum, float threshold,
                     unsigned char* __restrict__ binaries) {
  const float thre = fminf((float)(*sum / (double)n), threshold);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    binaries[i] = occs[i] > thre ? 1 : 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// Opacity culling of marched samples (nerfacc's sampling with a density callback and alpha_thre > 0, as the reference
// calls it in landmark/nerf_components/ray_samplers/volumetric_sampler.py:92-104): a sample survives if its opacity is
// at least `alpha_thre` and the transmittance in front of it at least `early_stop_eps`; survivors move to the front of
// the ray's row in order.  One warp per ray: opacity per lane, transmittance by a multiplicative warp scan with a
// carry, positions by ballot.  In place: a row is read 32 samples at a time and written at or before where it is read.
__global__ void __launch_bounds__(256)
occ_cull_kernel(int R, int S, const float* __restrict__ sigma, float* __restrict__ ts, float* __restrict__ te,
                int* __restrict__ counts, float alpha_thre, float early_stop_eps, int* __restrict__ src) {
  const int ray = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  if (ray >= R) return;
  const int n = counts[ray];
  const long long base = (long long)ray * S;
  float carry = 1.f;       // transmittance in front of this group of 32 samples
  int kept = 0;
  for (int s0 = 0; s0 < n; s0 += 32) {
    const int s = s0 + lane;
    const bool valid = s < n;
    float a = 0.f, t0 = 0.f, t1 = 0.f;
    if (valid) {
      t0 = ts[base + s]; t1 = te[base + s];
      a = 1.f - expf(-sigma[base + s] * (t1 - t0));
    }
    float incl = 1.f - a;                                      // inclusive product of (1 - alpha) over the lanes so far
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float v = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl *= v;
    }
    float before = __shfl_up_sync(0xffffffffu, incl, 1);
    before = carry * (lane == 0 ? 1.f : before);
    const bool keep = valid && a >= alpha_thre && before >= early_stop_eps;
    const unsigned won = __ballot_sync(0xffffffffu, keep);
    __syncwarp();                                              // every lane has read its sample before any lane writes
    if (keep) {
      const int pos = kept + __popc(won & ((1u << lane) - 1u));
      ts[base + pos] = t0; te[base + pos] = t1;
      if (src) src[base + pos] = s;              // where the survivor sat before: lets a caller reuse per-sample results
    }
    kept += __popc(won);
    carry *= __shfl_sync(0xffffffffu, incl, 31);
  }
  __syncwarp();
  for (int s = kept + lane; s < n; s += 32) { ts[base + s] = 0.f; te[base + s] = 0.f; }
  if (lane == 0) counts[ray] = kept;
}

// ---------------------------------------------------------------------------------------------------------------------
// Rows of the sampler's density query for the samples that survived the culling.  Survivor m sits at flat slot idx[m]
// of the compacted [R, S] block; before the compaction it sat at slot source[idx[m]] of the same ray, and the query
// wrote row where[that flat slot] (where == nullptr: the query covered every slot, the row is the flat slot).  Two row
// sets are gathered at once (hash features and head outputs), 16 bytes per thread.
__global__ void __launch_bounds__(256)
ngp_gather_cached_kernel(long long n, const long long* __restrict__ idx, int samples_per_ray, const int* __restrict__ source,
                         const long long* __restrict__ where, const uint4* __restrict__ a_src, int a_pieces,
                         const uint4* __restrict__ b_src, int b_pieces, uint4* __restrict__ a_dst, uint4* __restrict__ b_dst) {
  const int pieces = a_pieces + b_pieces;
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long m = t / pieces;
  if (m >= n) return;
  const int piece = (int)(t - m * pieces);
  const long long flat = idx[m];
  long long row = (flat / samples_per_ray) * samples_per_ray + source[flat];
  if (where != nullptr) row = where[row];
  if (piece < a_pieces) a_dst[m * a_pieces + piece] = __ldg(a_src + row * a_pieces + piece);
  else b_dst[m * b_pieces + (piece - a_pieces)] = __ldg(b_src + row * b_pieces + (piece - a_pieces));
}

}  // namespace lmb

using namespace lmb;

LMB_API int lmb_sh_encode(long long n, const float* dirs, int unit_range, int levels, float* out, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int grid = ceil_div(n, 256);
  switch (levels) {
    case 1: sh_encode_kernel<1><<<grid, 256, 0, stream>>>(n, dirs, unit_range, out); break;
    case 2: sh_encode_kernel<2><<<grid, 256, 0, stream>>>(n, dirs, unit_range, out); break;
    case 3: sh_encode_kernel<3><<<grid, 256, 0, stream>>>(n, dirs, unit_range, out); break;
    case 4: sh_encode_kernel<4><<<grid, 256, 0, stream>>>(n, dirs, unit_range, out); break;
    case 5: sh_encode_kernel<5><<<grid, 256, 0, stream>>>(n, dirs, unit_range, out); break;
    default: return (int)cudaErrorInvalidValue;
  }
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_ngp_positions(long long m, const long long* idx, int samples_per_ray, const float* origins, const float* dirs,
                              const float* z_flat, const float* aabb_lo, const float* aabb_hi, int nx, int ny, int only_block,
                              float* xyzb, unsigned char* inside, cudaStream_t stream) {
  if (m <= 0) return 0;
  NgpBox box;
  for (int k = 0; k < 3; ++k) {
    box.lo[k] = aabb_lo[k];
    box.inv_extent[k] = 1.f / (aabb_hi[k] - aabb_lo[k]);
  }
  box.nx = nx; box.ny = ny; box.only_block = only_block;
  ngp_positions_kernel<<<ceil_div(m, 256), 256, 0, stream>>>(m, idx, samples_per_ray, origins, dirs, z_flat, box, xyzb, inside);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_ngp_head_rows(long long m, const long long* idx, int samples_per_ray, const float* dirs, const float* h, int geo,
                              const unsigned char* inside, const float* app_ray, int app, int width, __nv_bfloat16* rows,
                              float* sigma, cudaStream_t stream) {
  if (m <= 0) return 0;
  if (width % 8 != 0 || width > kRowMaxWidth || 16 + geo + app > width) return (int)cudaErrorInvalidValue;
  ngp_head_rows_kernel<<<ceil_div(m, 256), 256, 0, stream>>>(m, idx, samples_per_ray, dirs, h, geo, inside, app_ray, app, width,
                                                            rows, sigma);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_ngp_head_rows_bwd(long long m, const long long* idx, int samples_per_ray, const __nv_bfloat16* d_rows,
                                  const float* d_sigma, const float* h, int geo, const unsigned char* inside, int app, int width,
                                  float* d_h, float* d_app, cudaStream_t stream) {
  if (m <= 0) return 0;
  if (16 + geo + app > width) return (int)cudaErrorInvalidValue;
  if (geo == 15 && width == 64)
    ngp_head_rows_bwd_g15w64_kernel<<<ceil_div(m, 256), 256, 0, stream>>>(m, idx, samples_per_ray, d_rows, d_sigma, h, inside, app,
                                                                         d_h, d_app);
  else
    ngp_head_rows_bwd_kernel<<<ceil_div(m, 256), 256, 0, stream>>>(m, idx, samples_per_ray, d_rows, d_sigma, h, geo, inside, app,
                                                                  width, d_h, d_app);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_occ_cells(long long n, const long long* idx, int res, const float* roi6, int level, unsigned seed, int jitter,
                          const float* occs_level, float decay, float* xyz, float* decayed, cudaStream_t stream) {
  if (n <= 0) return 0;
  OccRoi roi;
  for (int k = 0; k < 3; ++k) {
    roi.centre[k] = 0.5f * (roi6[k] + roi6[3 + k]);
    roi.half[k] = 0.5f * (roi6[3 + k] - roi6[k]);
  }
  occ_cells_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(n, idx, res, roi, (float)(1 << level), seed, jitter, occs_level, decay, xyz,
                                                        decayed);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_occ_update(long long n, const long long* idx, const float* decayed, const float* fresh, float* occs_level,
                           cudaStream_t stream) {
  if (n <= 0) return 0;
  occ_store_decayed_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(n, idx, decayed, occs_level);
  LMB_LAUNCH_CHECK();
  occ_max_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(n, idx, fresh, occs_level);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_occ_binarise(long long n, const float* occs, float threshold, double* sum_scratch, unsigned char* binaries,
                             cudaStream_t stream) {
  if (n <= 0) return 0;
  LMB_CUDA_TRY(cudaMemsetAsync(sum_scratch, 0, sizeof(double), stream));
  const int grid = (int)fminf((float)ceil_div(n, 256), 148.f * 8.f);
  occ_sum_kernel<<<grid, 256, 0, stream>>>(n, occs, sum_scratch);
  LMB_LAUNCH_CHECK();
  occ_threshold_kernel<<<grid, 256, 0, stream>>>(n, occs, sum_scratch, threshold, binaries);
  LMB_LAUNCH_CHECK();
  return 0;
}

// sigma: fp32 [R, S] (values past counts[r] ignored); ts / te: fp32 [R, S], compacted in place; counts: int32 [R], updated
// src (may be null): int32 [R, S], slot of every survivor before the compaction
LMB_API int lmb_occ_cull(int R, int S, const float* sigma, float* ts, float* te, int* counts, float alpha_thre,
                         float early_stop_eps, int* src, cudaStream_t stream) {
  if (R <= 0) return 0;
  occ_cull_kernel<<<ceil_div((long long)R * 32, 256), 256, 0, stream>>>(R, S, sigma, ts, te, counts, alpha_thre, early_stop_eps, src);
  LMB_LAUNCH_CHECK();
  return 0;
}

// a / b: two row-major arrays with rows of a_bytes / b_bytes (multiples of 16); idx: int64 [n]; source: int32 [R * S];
// where: int64 [R * S] or null
LMB_API int lmb_ngp_gather_cached(long long n, const long long* idx, int samples_per_ray, const int* source, const long long* where,
                                  const void* a_src, int a_bytes, const void* b_src, int b_bytes, void* a_dst, void* b_dst,
                                  cudaStream_t stream) {
  if (n <= 0) return 0;
  if (a_bytes % 16 || b_bytes % 16 || a_bytes <= 0 || b_bytes <= 0) return (int)cudaErrorInvalidValue;
  const int pieces = (a_bytes + b_bytes) / 16;
  ngp_gather_cached_kernel<<<ceil_div(n * pieces, 256), 256, 0, stream>>>(n, idx, samples_per_ray, source, where, (const uint4*)a_src,
                                                                         a_bytes / 16, (const uint4*)b_src, b_bytes / 16,
                                                                         (uint4*)a_dst, (uint4*)b_dst);
  LMB_LAUNCH_CHECK();
  return 0;
}
