// Multiresolution hash-grid encoding (Instant-NGP style), forward and backward.
//
// Level l: pos = x * scale_l + 0.5; the 8 corners of the enclosing cell are looked up in the level's
// table (dense index when the grid fits, XOR-of-primes spatial hash otherwise) and blended
// trilinearly.  The reference gets this op from tiny-cuda-nn (landmark/nerf_components/
// model_components/fields/encodings/hash_encoding.py:82-107).  One thread handles one
// (sample, level) pair; consecutive threads walk the levels of one sample, so the coarse (dense,
// L2-resident) levels and the fine (hashed, HBM-resident) levels of neighbouring samples are in
// flight together and a sample's output row is written as one contiguous segment.
#include "common.cuh"

namespace lmb {

struct HashMeta {
  float scale[32];
  int res[32];
  long long offset[33];
  int n_levels, n_features;
};

__device__ __forceinline__ uint32_t grid_index(uint32_t ix, uint32_t iy, uint32_t iz, uint32_t res, uint32_t entries) {
  // dense when res^3 fits (res <= 1625 keeps res^3 inside 32 bits; larger grids always hash)
  if (res <= 1625u && res * res * res <= entries) return ix + iy * res + iz * res * res;
  return ((ix * 1u) ^ (iy * 2654435761u) ^ (iz * 805459861u)) % entries;
}

template <typename T, typename OutT, int F>
__global__ void __launch_bounds__(256)
hashgrid_fwd_kernel(const float* __restrict__ x, long long n, const T* __restrict__ table, HashMeta m,
                    OutT* __restrict__ out) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int L = m.n_levels;
  const long long i = tid / L;
  const int l = (int)(tid - i * L);
  if (i >= n) return;
  const float scale = m.scale[l];
  const uint32_t res = (uint32_t)m.res[l];
  const uint32_t entries = (uint32_t)(m.offset[l + 1] - m.offset[l]);
  const T* tab = table + m.offset[l] * F;
  float p[3], w[3];
  uint32_t p0[3];
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    p[d] = x[i * 3 + d] * scale + 0.5f;
    float fl = floorf(p[d]);
    w[d] = p[d] - fl;
    p0[d] = (uint32_t)max((int)fl, 0);
  }
  float acc[F];
#pragma unroll
  for (int f = 0; f < F; ++f) acc[f] = 0.f;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint32_t ix = min(p0[0] + (c & 1), res - 1), iy = min(p0[1] + ((c >> 1) & 1), res - 1),
                   iz = min(p0[2] + ((c >> 2) & 1), res - 1);
    const float wt = ((c & 1) ? w[0] : 1.f - w[0]) * ((c & 2) ? w[1] : 1.f - w[1]) * ((c & 4) ? w[2] : 1.f - w[2]);
    const T* e = tab + (long long)grid_index(ix, iy, iz, res, entries) * F;
#pragma unroll
    for (int f = 0; f < F; ++f) acc[f] += wt * (float)e[f];
  }
  OutT* o = out + i * (long long)(L * F) + l * F;
#pragma unroll
  for (int f = 0; f < F; ++f) o[f] = (OutT)acc[f];
}

template <typename GT, int F>
__global__ void __launch_bounds__(256)
hashgrid_bwd_kernel(const float* __restrict__ x, long long n, HashMeta m, const GT* __restrict__ dout,
                    float* __restrict__ grad) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int L = m.n_levels;
  const long long i = tid / L;
  const int l = (int)(tid - i * L);
  if (i >= n) return;
  const GT* g = dout + i * (long long)(L * F) + l * F;
  float gv[F];
  bool any = false;
#pragma unroll
  for (int f = 0; f < F; ++f) { gv[f] = (float)g[f]; any |= gv[f] != 0.f; }
  if (!any) return;
  const float scale = m.scale[l];
  const uint32_t res = (uint32_t)m.res[l];
  const uint32_t entries = (uint32_t)(m.offset[l + 1] - m.offset[l]);
  float* tab = grad + m.offset[l] * F;
  float w[3];
  uint32_t p0[3];
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    float p = x[i * 3 + d] * scale + 0.5f;
    float fl = floorf(p);
    w[d] = p - fl;
    p0[d] = (uint32_t)max((int)fl, 0);
  }
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint32_t ix = min(p0[0] + (c & 1), res - 1), iy = min(p0[1] + ((c >> 1) & 1), res - 1),
                   iz = min(p0[2] + ((c >> 2) & 1), res - 1);
    const float wt = ((c & 1) ? w[0] : 1.f - w[0]) * ((c & 2) ? w[1] : 1.f - w[1]) * ((c & 4) ? w[2] : 1.f - w[2]);
    float* e = tab + (long long)grid_index(ix, iy, iz, res, entries) * F;
    if (F == 2) {
      asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(e), "f"(wt * gv[0]), "f"(wt * gv[1]) : "memory");
    } else if (F == 4) {
      red_add_v4(e, wt * gv[0], wt * gv[1], wt * gv[2], wt * gv[3]);
    } else {
#pragma unroll
      for (int f = 0; f < F; ++f) atomicAdd(e + f, wt * gv[f]);
    }
  }
}

}  // namespace lmb

using namespace lmb;

#define LMB_DISPATCH_F(F_, ...)            \
  switch (F_) {                            \
    case 1: { constexpr int F = 1; __VA_ARGS__; break; } \
    case 2: { constexpr int F = 2; __VA_ARGS__; break; } \
    case 4: { constexpr int F = 4; __VA_ARGS__; break; } \
    case 8: { constexpr int F = 8; __VA_ARGS__; break; } \
    default: return (int)cudaErrorInvalidValue; \
  }

LMB_API int lmb_hashgrid_fwd(const float* x, long long n, const void* table, int table_dtype, const HashMeta* meta,
                             void* out, int out_dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int blocks = ceil_div(n * meta->n_levels, 256);
  LMB_DISPATCH_F(meta->n_features, {
    if (table_dtype == 0 && out_dtype == 0)
      hashgrid_fwd_kernel<float, float, F><<<blocks, 256, 0, stream>>>(x, n, (const float*)table, *meta, (float*)out);
    else if (table_dtype == 1 && out_dtype == 0)
      hashgrid_fwd_kernel<__nv_bfloat16, float, F><<<blocks, 256, 0, stream>>>(x, n, (const __nv_bfloat16*)table, *meta, (float*)out);
    else if (table_dtype == 0 && out_dtype == 1)
      hashgrid_fwd_kernel<float, __nv_bfloat16, F><<<blocks, 256, 0, stream>>>(x, n, (const float*)table, *meta, (__nv_bfloat16*)out);
    else
      hashgrid_fwd_kernel<__nv_bfloat16, __nv_bfloat16, F><<<blocks, 256, 0, stream>>>(x, n, (const __nv_bfloat16*)table, *meta, (__nv_bfloat16*)out);
  });
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_hashgrid_bwd(const float* x, long long n, const HashMeta* meta, const void* dout, int dout_dtype,
                             float* grad, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int blocks = ceil_div(n * meta->n_levels, 256);
  LMB_DISPATCH_F(meta->n_features, {
    if (dout_dtype == 0) hashgrid_bwd_kernel<float, F><<<blocks, 256, 0, stream>>>(x, n, *meta, (const float*)dout, grad);
    else hashgrid_bwd_kernel<__nv_bfloat16, F><<<blocks, 256, 0, stream>>>(x, n, *meta, (const __nv_bfloat16*)dout, grad);
  });
  LMB_LAUNCH_CHECK();
  return 0;
}
