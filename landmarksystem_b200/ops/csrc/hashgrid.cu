// Multiresolution hash-grid encoding (Instant-NGP style), forward and backward.
//
// Level l: pos = x * scale_l + 0.5; the 8 corners of the enclosing cell are looked up in the level's
// table (dense index when the grid fits, XOR-of-primes spatial hash otherwise) and blended
// trilinearly.  The reference gets this op from tiny-cuda-nn (landmark/nerf_components/
// model_components/fields/encodings/hash_encoding.py:82-107).
//
// Work layout: one thread handles one sample and a group of kLevelGroup consecutive levels; blockIdx.y is the level
// group and varies slowest.  A warp is therefore 32 consecutive samples (neighbours along a ray) at the same levels:
//  * on the coarse levels neighbouring samples sit in the same cell, so their corner loads coalesce into a few
//    sectors, and in the backward their contributions are summed inside the warp (segmented over runs of equal cells)
//    before one lane per run touches memory;
//  * the tables of one level group (4 x 2^22 entries at most) are the only ones in flight while the grid sweeps the
//    samples, instead of all 16 levels competing for the L2;
//  * a thread's outputs are 4 levels x F features = one full 32-byte sector of the sample's row.
#include "common.cuh"

namespace lmb {

struct HashMeta {
  float scale[32];
  int res[32];
  long long offset[33];
  int n_levels, n_features;
};

constexpr int kLevelGroup = 4;
// The backward sweeps two levels at a time: their fp32 gradient tables (2 x 2^22 entries x 8 bytes = 64 MB at the
// benchmark shape) stay resident in the 126 MB L2 while the grid walks the samples, so the reductions on the hashed
// levels complete in the L2 instead of fetching and writing back a DRAM sector each.  Measured on the Instant-NGP
// benchmark step (42 M samples, 16 levels): 105.6 ms with four levels per sweep, 91.5 ms with two, 92.1 ms with one.
constexpr int kBwdLevelGroup = 2;
constexpr int kWarpReduceMaxRes = 512;   // levels up to this resolution pre-reduce their gradients inside the warp

struct LevelIndex {
  uint32_t res, entries, mask;
  bool dense, pow2;
  __device__ __forceinline__ LevelIndex(uint32_t res_, uint32_t entries_) : res(res_), entries(entries_) {
    // dense when res^3 fits (res <= 1625 keeps res^3 inside 32 bits; larger grids always hash)
    dense = res <= 1625u && res * res * res <= entries;
    pow2 = (entries & (entries - 1u)) == 0u;
    mask = entries - 1u;
  }
  __device__ __forceinline__ uint32_t operator()(uint32_t ix, uint32_t iy, uint32_t iz) const {
    if (dense) return ix + iy * res + iz * res * res;
    const uint32_t h = (ix * 1u) ^ (iy * 2654435761u) ^ (iz * 805459861u);
    return pow2 ? (h & mask) : (h % entries);
  }
};

template <typename T, int F>
__device__ __forceinline__ void load_entry(const T* e, float* v) {
  if constexpr (sizeof(T) == 4 && F == 2) {
    const float2 t = __ldg(reinterpret_cast<const float2*>(e));
    v[0] = t.x; v[1] = t.y;
  } else if constexpr (sizeof(T) == 4 && F == 4) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(e));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else if constexpr (sizeof(T) == 2 && F == 2) {
    const unsigned u = __ldg(reinterpret_cast<const unsigned*>(e));
    const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u));
    v[0] = t.x; v[1] = t.y;
  } else if constexpr (sizeof(T) == 2 && F == 8) {
    const F8 t = load8(reinterpret_cast<const __nv_bfloat16*>(e));
#pragma unroll
    for (int f = 0; f < 8; ++f) v[f] = t.v[f];
  } else {
#pragma unroll
    for (int f = 0; f < F; ++f) v[f] = (float)e[f];
  }
}

template <typename T, typename OutT, int F>
__global__ void __launch_bounds__(256)
hashgrid_fwd_kernel(const float* __restrict__ x, long long n, const T* __restrict__ table, HashMeta m,
                    OutT* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int L = m.n_levels;
  const int l0 = blockIdx.y * kLevelGroup;
  const float xs[3] = {x[i * 3], x[i * 3 + 1], x[i * 3 + 2]};
  float acc[kLevelGroup][F];
#pragma unroll
  for (int g = 0; g < kLevelGroup; ++g) {
    const int l = l0 + g;
#pragma unroll
    for (int f = 0; f < F; ++f) acc[g][f] = 0.f;
    if (l >= L) continue;
    const float scale = m.scale[l];
    const LevelIndex index((uint32_t)m.res[l], (uint32_t)(m.offset[l + 1] - m.offset[l]));
    const T* tab = table + m.offset[l] * F;
    float w[3];
    uint32_t p0[3];
#pragma unroll
    for (int d = 0; d < 3; ++d) {
      const float p = xs[d] * scale + 0.5f;
      const float fl = floorf(p);
      w[d] = p - fl;
      p0[d] = (uint32_t)max((int)fl, 0);
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint32_t ix = min(p0[0] + (c & 1), index.res - 1), iy = min(p0[1] + ((c >> 1) & 1), index.res - 1),
                     iz = min(p0[2] + ((c >> 2) & 1), index.res - 1);
      const float wt = ((c & 1) ? w[0] : 1.f - w[0]) * ((c & 2) ? w[1] : 1.f - w[1]) * ((c & 4) ? w[2] : 1.f - w[2]);
      float e[F];
      load_entry<T, F>(tab + (long long)index(ix, iy, iz) * F, e);
#pragma unroll
      for (int f = 0; f < F; ++f) acc[g][f] += wt * e[f];
    }
  }
  OutT* o = out + i * (long long)(L * F) + l0 * F;
  if (F == 2 && L % kLevelGroup == 0) {
    // 4 levels x 2 features: one 32-byte (fp32) or 16-byte (bf16) piece of the row, aligned because L*F is a multiple of 8
    if constexpr (sizeof(OutT) == 4) {
      reinterpret_cast<float4*>(o)[0] = make_float4(acc[0][0], acc[0][F > 1 ? 1 : 0], acc[1][0], acc[1][F > 1 ? 1 : 0]);
      reinterpret_cast<float4*>(o)[1] = make_float4(acc[2][0], acc[2][F > 1 ? 1 : 0], acc[3][0], acc[3][F > 1 ? 1 : 0]);
    } else {
      F8 v;
#pragma unroll
      for (int g = 0; g < kLevelGroup; ++g) { v.v[2 * g] = acc[g][0]; v.v[2 * g + 1] = acc[g][F > 1 ? 1 : 0]; }
      store8(reinterpret_cast<__nv_bfloat16*>(o), v);
    }
  } else {
#pragma unroll
    for (int g = 0; g < kLevelGroup; ++g)
      if (l0 + g < L) {
#pragma unroll
        for (int f = 0; f < F; ++f) o[g * F + f] = (OutT)acc[g][f];
      }
  }
}

template <int F>
__device__ __forceinline__ void red_entry(float* e, const float* v) {
  if constexpr (F == 2) {
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(e), "f"(v[0]), "f"(v[1]) : "memory");
  } else if constexpr (F == 4) {
    red_add_v4(e, v[0], v[1], v[2], v[3]);
  } else if constexpr (F == 8) {
    red_add_v4(e, v[0], v[1], v[2], v[3]);
    red_add_v4(e + 4, v[4], v[5], v[6], v[7]);
  } else {
#pragma unroll
    for (int f = 0; f < F; ++f) atomicAdd(e + f, v[f]);
  }
}

template <typename GT, int F, int LG>
__global__ void __launch_bounds__(256)
hashgrid_bwd_kernel(const float* __restrict__ x, long long n, HashMeta m, const GT* __restrict__ dout,
                    float* __restrict__ grad) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = i < n;
  const int lane = threadIdx.x & 31;
  const int L = m.n_levels;
  const int l0 = blockIdx.y * LG;
  float xs[3] = {0.f, 0.f, 0.f};
  if (live) { xs[0] = x[i * 3]; xs[1] = x[i * 3 + 1]; xs[2] = x[i * 3 + 2]; }
#pragma unroll 1
  for (int g = 0; g < LG; ++g) {
    const int l = l0 + g;
    if (l >= L) break;                                      // uniform
    float gv[F];
    bool any = false;
    if (live) {
      const GT* gp = dout + i * (long long)(L * F) + l * F;
#pragma unroll
      for (int f = 0; f < F; ++f) { gv[f] = (float)gp[f]; any |= gv[f] != 0.f; }
    } else {
#pragma unroll
      for (int f = 0; f < F; ++f) gv[f] = 0.f;
    }
    const float scale = m.scale[l];
    const LevelIndex index((uint32_t)m.res[l], (uint32_t)(m.offset[l + 1] - m.offset[l]));
    float* tab = grad + m.offset[l] * F;
    float w[3];
    uint32_t p0[3];
#pragma unroll
    for (int d = 0; d < 3; ++d) {
      const float p = xs[d] * scale + 0.5f;
      const float fl = floorf(p);
      w[d] = p - fl;
      p0[d] = (uint32_t)max((int)fl, 0);
    }
    if ((int)index.res <= kWarpReduceMaxRes) {
      // Runs of consecutive lanes in the same cell (res <= 512: the cell packs into 30 bits, and positions past the grid clamp to
      // the last cell in the key as they do in the index; a lane without a gradient gets a key of its own) are summed with a segmented suffix reduction; the first lane of a run writes.
      const uint32_t key = (live && any) ? (min(p0[0], 1023u) | (min(p0[1], 1023u) << 10) | (min(p0[2], 1023u) << 20))
                                          : (0xC0000000u | (uint32_t)lane);
      const uint32_t prev = __shfl_up_sync(0xffffffffu, key, 1);
      const bool head = lane == 0 || prev != key;
      const unsigned heads = __ballot_sync(0xffffffffu, head);
      const int seg = __popc(heads & (0xffffffffu >> (31 - lane)));
      bool take[5];
#pragma unroll
      for (int s = 0; s < 5; ++s) {
        const int other = __shfl_down_sync(0xffffffffu, seg, 1 << s);
        take[s] = (lane + (1 << s) < 32) && other == seg;
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float wt = ((c & 1) ? w[0] : 1.f - w[0]) * ((c & 2) ? w[1] : 1.f - w[1]) * ((c & 4) ? w[2] : 1.f - w[2]);
        float v[F];
#pragma unroll
        for (int f = 0; f < F; ++f) {
          v[f] = wt * gv[f];
#pragma unroll
          for (int s = 0; s < 5; ++s) {
            const float o = __shfl_down_sync(0xffffffffu, v[f], 1 << s);
            if (take[s]) v[f] += o;
          }
        }
        if (head && live && any) {
          const uint32_t ix = min(p0[0] + (c & 1), index.res - 1), iy = min(p0[1] + ((c >> 1) & 1), index.res - 1),
                         iz = min(p0[2] + ((c >> 2) & 1), index.res - 1);
          red_entry<F>(tab + (long long)index(ix, iy, iz) * F, v);
        }
      }
    } else if (live && any) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint32_t ix = min(p0[0] + (c & 1), index.res - 1), iy = min(p0[1] + ((c >> 1) & 1), index.res - 1),
                       iz = min(p0[2] + ((c >> 2) & 1), index.res - 1);
        const float wt = ((c & 1) ? w[0] : 1.f - w[0]) * ((c & 2) ? w[1] : 1.f - w[1]) * ((c & 4) ? w[2] : 1.f - w[2]);
        float v[F];
#pragma unroll
        for (int f = 0; f < F; ++f) v[f] = wt * gv[f];
        red_entry<F>(tab + (long long)index(ix, iy, iz) * F, v);
      }
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
  const dim3 blocks(ceil_div(n, 256), ceil_div(meta->n_levels, kLevelGroup));
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
  const dim3 blocks(ceil_div(n, 256), ceil_div(meta->n_levels, kBwdLevelGroup));
  LMB_DISPATCH_F(meta->n_features, {
    if (dout_dtype == 0)
      hashgrid_bwd_kernel<float, F, kBwdLevelGroup><<<blocks, 256, 0, stream>>>(x, n, *meta, (const float*)dout, grad);
    else
      hashgrid_bwd_kernel<__nv_bfloat16, F, kBwdLevelGroup><<<blocks, 256, 0, stream>>>(x, n, *meta, (const __nv_bfloat16*)dout, grad);
  });
  LMB_LAUNCH_CHECK();
  return 0;
}
