// Shared helpers for the sm_100a kernel library: exported-symbol macro, launch checks,
// bf16 <-> fp32 vector conversion, and vectorised global reductions.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define LMB_API extern "C" __attribute__((visibility("default")))

#define LMB_LAUNCH_CHECK()                                   \
  do {                                                       \
    cudaError_t e_ = cudaGetLastError();                     \
    if (e_ != cudaSuccess) return (int)e_;                   \
  } while (0)

#define LMB_CUDA_TRY(x)                                      \
  do {                                                       \
    cudaError_t e_ = (x);                                    \
    if (e_ != cudaSuccess) return (int)e_;                   \
  } while (0)

namespace lmb {

constexpr int kMaxLevels = 4;

__host__ __device__ inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// 8 consecutive channels as fp32, loaded from fp32 or bf16 storage.
struct F8 { float v[8]; };

__device__ __forceinline__ F8 load8(const float* p) {
  F8 r;
  float4 a = __ldg(reinterpret_cast<const float4*>(p));
  float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  r.v[0] = a.x; r.v[1] = a.y; r.v[2] = a.z; r.v[3] = a.w;
  r.v[4] = b.x; r.v[5] = b.y; r.v[6] = b.z; r.v[7] = b.w;
  return r;
}

__device__ __forceinline__ F8 load8(const __nv_bfloat16* p) {
  F8 r;
  uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    r.v[2 * i] = f.x; r.v[2 * i + 1] = f.y;
  }
  return r;
}

__device__ __forceinline__ void store8(float* p, const F8& r) {
  reinterpret_cast<float4*>(p)[0] = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(r.v[4], r.v[5], r.v[6], r.v[7]);
}

__device__ __forceinline__ void store8(__nv_bfloat16* p, const F8& r) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(r.v[2 * i], r.v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

// One 16-byte L2 reduction instead of four scalar atomics (sm_90+).
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

__device__ __forceinline__ void red_add8(float* addr, const F8& g, float w) {
  red_add_v4(addr, g.v[0] * w, g.v[1] * w, g.v[2] * w, g.v[3] * w);
  red_add_v4(addr + 4, g.v[4] * w, g.v[5] * w, g.v[6] * w, g.v[7] * w);
}

// Device-side element count: kernels take (count_ptr, max_count) so that a data-dependent
// size never needs a host synchronisation; count_ptr == nullptr means "use max_count".
__device__ __forceinline__ long long resolve_count(const int* count_ptr, long long max_count) {
  if (count_ptr == nullptr) return max_count;
  long long c = *count_ptr;
  return c < max_count ? c : max_count;
}

}  // namespace lmb
