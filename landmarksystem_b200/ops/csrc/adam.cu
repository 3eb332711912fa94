// Fused Adam for feature grids and MLPs: one pass over (grad, master, m, v) that also writes the
// bf16 shadow copy the lookup kernels read and clears the gradient for the next step.
//
// The reference uses torch.optim.Adam (benchmarks/nerf/gridnerf/gridnerf_trainer.py:127-154) plus a
// separate zero_grad; for 10^9-parameter plane grids the update is purely HBM-bound, so every extra
// pass costs milliseconds.  Bytes per parameter here: read 16 (g, p, m, v), write 12 + 2 + 4.
#include "common.cuh"
#include <cmath>

namespace lmb {

struct AdamArgs {
  float lr, beta1, beta2, eps, bias1, bias2, grad_scale, weight_decay;
  // Optional device-resident schedule {learning rate, step number (1-based) of the step being applied}:
  // when set it overrides lr / bias1 / bias2, so a launch recorded in a CUDA graph follows the schedule
  // on every replay.  l2_beta* = log2(beta*).
  const float* dyn;
  float l2_beta1, l2_beta2;
  // mode 0: Adam, p -= lr/bias1 * m / (sqrt(v)/sqrt(bias2) + eps).  Modes 1 and 2 take the step size `A` from the host
  // (rectified Adam): 1: p -= A * m / (sqrt(v) + eps);  2: p -= A * m (variance not yet tractable).
  int mode;
  float A;
};

struct AdamStep { float step, vscale; bool adaptive; };
__device__ __forceinline__ AdamStep adam_step_of(const AdamArgs& a) {
  AdamStep s;
  if (a.mode == 0) { s.step = a.lr / a.bias1; s.vscale = rsqrtf(a.bias2); s.adaptive = true; }
  else { s.step = a.A; s.vscale = 1.f; s.adaptive = a.mode == 1; }
  return s;
}

__device__ __forceinline__ void resolve_dyn(AdamArgs& a) {
  if (a.dyn != nullptr) {
    const float step = a.dyn[1];
    a.lr = a.dyn[0];
    a.bias1 = 1.f - exp2f(a.l2_beta1 * step);
    a.bias2 = 1.f - exp2f(a.l2_beta2 * step);
  }
}

template <bool kShadow>
__global__ void __launch_bounds__(256)
adam_kernel(float4* __restrict__ p, float4* __restrict__ g, float4* __restrict__ m, float4* __restrict__ v,
            uint2* __restrict__ shadow, long long n4, AdamArgs a) {
  resolve_dyn(a);
  const AdamStep st = adam_step_of(a);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 gg = g[i], pp = p[i], mm = m[i], vv = v[i];
    float* G = &gg.x; float* P = &pp.x; float* M = &mm.x; float* V = &vv.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float gr = G[k] * a.grad_scale + a.weight_decay * P[k];
      M[k] = a.beta1 * M[k] + (1.f - a.beta1) * gr;
      V[k] = a.beta2 * V[k] + (1.f - a.beta2) * gr * gr;
      P[k] -= st.step * M[k] / (st.adaptive ? sqrtf(V[k]) * st.vscale + a.eps : 1.f);
    }
    p[i] = pp; m[i] = mm; v[i] = vv;
    g[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (kShadow) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(pp.x, pp.y), hi = __floats2bfloat162_rn(pp.z, pp.w);
      uint2 u;
      u.x = *reinterpret_cast<unsigned*>(&lo); u.y = *reinterpret_cast<unsigned*>(&hi);
      shadow[i] = u;
    }
  }
}

__global__ void adam_tail_kernel(float* p, float* g, float* m, float* v, __nv_bfloat16* shadow, long long start,
                                 long long n, AdamArgs a) {
  long long i = start + blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  resolve_dyn(a);
  float gr = g[i] * a.grad_scale + a.weight_decay * p[i];
  float mm = a.beta1 * m[i] + (1.f - a.beta1) * gr;
  float vv = a.beta2 * v[i] + (1.f - a.beta2) * gr * gr;
  const AdamStep st = adam_step_of(a);
  float pp = p[i] - st.step * mm / (st.adaptive ? sqrtf(vv) * st.vscale + a.eps : 1.f);
  p[i] = pp; m[i] = mm; v[i] = vv; g[i] = 0.f;
  if (shadow) shadow[i] = __float2bfloat16_rn(pp);
}

__global__ void adam_dyn_advance_kernel(float* dyn, float decay) {
  dyn[0] *= decay;
  dyn[1] += 1.f;
}

__global__ void __launch_bounds__(256) cast_bf16_kernel(const float4* __restrict__ src, uint2* __restrict__ dst, long long n4) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 pp = src[i];
    __nv_bfloat162 lo = __floats2bfloat162_rn(pp.x, pp.y), hi = __floats2bfloat162_rn(pp.z, pp.w);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&lo); u.y = *reinterpret_cast<unsigned*>(&hi);
    dst[i] = u;
  }
}

}  // namespace lmb

using namespace lmb;

static int adam_launch(float* p, float* g, float* m, float* v, void* shadow_bf16, long long n, const AdamArgs& a,
                       cudaStream_t stream) {
  const long long n4 = n / 4;
  if (n4 > 0) {
    long long want = (n4 + 255) / 256;
    int blocks = (int)(want < 148LL * 16 ? want : 148LL * 16);
    if (shadow_bf16)
      adam_kernel<true><<<blocks, 256, 0, stream>>>((float4*)p, (float4*)g, (float4*)m, (float4*)v, (uint2*)shadow_bf16, n4, a);
    else
      adam_kernel<false><<<blocks, 256, 0, stream>>>((float4*)p, (float4*)g, (float4*)m, (float4*)v, nullptr, n4, a);
    LMB_LAUNCH_CHECK();
  }
  if (n4 * 4 < n) {
    adam_tail_kernel<<<1, 32, 0, stream>>>(p, g, m, v, (__nv_bfloat16*)shadow_bf16, n4 * 4, n, a);
    LMB_LAUNCH_CHECK();
  }
  return 0;
}

// step >= 1.  shadow may be null.  All pointers 16-byte aligned (torch allocations are).
LMB_API int lmb_adam_step(float* p, float* g, float* m, float* v, void* shadow_bf16, long long n, float lr,
                          float beta1, float beta2, float eps, int step, float grad_scale, float weight_decay,
                          cudaStream_t stream) {
  if (n <= 0) return 0;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.grad_scale = grad_scale; a.weight_decay = weight_decay;
  a.bias1 = 1.f - powf(beta1, (float)step);
  a.bias2 = 1.f - powf(beta2, (float)step);
  a.dyn = nullptr; a.l2_beta1 = a.l2_beta2 = 0.f; a.mode = 0; a.A = 0.f;
  return adam_launch(p, g, m, v, shadow_bf16, n, a, stream);
}

// Rectified Adam (Liu et al. 2020; the optimiser of the reference's Nerfacto trainer,
// benchmarks/nerf/nerfacto/nerfacto_trainer.py:139): the variance rectification term depends only on the step number,
// so it is folded into the step size on the host and the device pass is the same single sweep as Adam's.
LMB_API int lmb_radam_step(float* p, float* g, float* m, float* v, void* shadow_bf16, long long n, float lr,
                           float beta1, float beta2, float eps, int step, float grad_scale, float weight_decay,
                           cudaStream_t stream) {
  if (n <= 0) return 0;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.grad_scale = grad_scale; a.weight_decay = weight_decay;
  a.bias1 = a.bias2 = 1.f; a.dyn = nullptr; a.l2_beta1 = a.l2_beta2 = 0.f;
  const double b1 = 1.0 - pow((double)beta1, step), b2t = pow((double)beta2, step), b2 = 1.0 - b2t;
  const double rho_inf = 2.0 / (1.0 - (double)beta2) - 1.0;
  const double rho_t = rho_inf - 2.0 * step * b2t / b2;
  if (rho_t > 5.0) {
    const double rect = sqrt((rho_t - 4.0) * (rho_t - 2.0) * rho_inf / ((rho_inf - 4.0) * (rho_inf - 2.0) * rho_t));
    a.mode = 1; a.A = (float)(lr * rect * sqrt(b2) / b1);
  } else {
    a.mode = 2; a.A = (float)(lr / b1);
  }
  return adam_launch(p, g, m, v, shadow_bf16, n, a, stream);
}

// Same update with the learning rate and step number read from device memory (dyn = {lr, step}); the
// launch can be replayed from a CUDA graph while lmb_adam_dyn_advance moves the schedule.
LMB_API int lmb_adam_step_dyn(float* p, float* g, float* m, float* v, void* shadow_bf16, long long n, const float* dyn,
                              float beta1, float beta2, float eps, float grad_scale, float weight_decay, cudaStream_t stream) {
  if (n <= 0) return 0;
  AdamArgs a;
  a.lr = 0.f; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.grad_scale = grad_scale; a.weight_decay = weight_decay;
  a.bias1 = a.bias2 = 1.f;
  a.dyn = dyn; a.l2_beta1 = (float)log2((double)beta1); a.l2_beta2 = (float)log2((double)beta2); a.mode = 0; a.A = 0.f;
  return adam_launch(p, g, m, v, shadow_bf16, n, a, stream);
}

// dyn[0] *= decay (next step's learning rate); dyn[1] += 1 (next step's number)
LMB_API int lmb_adam_dyn_advance(float* dyn, float decay, cudaStream_t stream) {
  adam_dyn_advance_kernel<<<1, 1, 0, stream>>>(dyn, decay);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_cast_bf16(const float* src, void* dst, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 4 != 0) return (int)cudaErrorInvalidValue;
  long long n4 = n / 4, want = (n4 + 255) / 256;
  int blocks = (int)(want < 148LL * 16 ? want : 148LL * 16);
  cast_bf16_kernel<<<blocks, 256, 0, stream>>>((const float4*)src, (uint2*)dst, n4);
  LMB_LAUNCH_CHECK();
  return 0;
}
