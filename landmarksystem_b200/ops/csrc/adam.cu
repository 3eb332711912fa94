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

// ---- dense Adam of a channels-last plane fused with its regularisers -------------------------------------------
// Every shipped GridNeRF configuration of the reference adds an L1 term on the density planes and a total-variation
// term on all planes (landmark/nerf_components/model_components/fields/encodings/tensor_vm_encoding.py:249-296,
// benchmarks/nerf/gridnerf/gridnerf_trainer.py:260-272).  Their gradients are dense, so every texel is updated every
// step and the update is bound by the bytes of one sweep over (gradient, parameter, moments).  Here that sweep also
// evaluates the regulariser gradient from the parameter and its four plane neighbours - no gradient tensor of the
// regularisers is ever written or read.  Neighbour values must be the OLD ones while texels are being overwritten, so
// the parameter is ping-ponged between two buffers: the sweep reads buffer `in` (centre + neighbours, the neighbours
// come from L1/L2) and writes buffer `out`; the roles swap every step (step parity, read from the device-resident
// schedule when there is one, so a launch recorded in a CUDA graph keeps alternating).
//   TV term  = w_tv * 1e-2 * 2 * (sum (p[i+1,j]-p[i,j])^2 / count_h + sum (p[i,j+1]-p[i,j])^2 / count_w)
//   L1 term  = w_l1 * mean |p|
// Bytes per parameter: read 16 (g, p, m, v), write 12 + 2 + 4 - the same as the plain fused Adam.
struct PlaneReg {
  int B, H, W, C;
  const float* tv_w_dev;   // device-resident TV weight (decays every step) or nullptr
  float tv_w;              // host value used when tv_w_dev == nullptr
  float tv_h, tv_w_scale;  // 0.04 / count_h, 0.04 / count_w (times the caller's loss scale)
  float l1;                // w_l1 / numel (times the caller's loss scale)
  float* loss;             // optional {TV value, L1 value} accumulators (unscaled by the caller's loss scale)
  float inv_loss_scale;
  int host_step;           // step number when there is no device-resident schedule
};

__device__ __forceinline__ float4 ld4(const float4* p) { return *p; }

__global__ void __launch_bounds__(256)
adam_plane_reg_kernel(float4* __restrict__ buf_odd, float4* __restrict__ buf_even, float4* __restrict__ g, float4* __restrict__ m,
                      float4* __restrict__ v, uint2* __restrict__ shadow, long long n4, AdamArgs a, PlaneReg r) {
  resolve_dyn(a);
  const AdamStep st = adam_step_of(a);
  const int step = a.dyn != nullptr ? (int)a.dyn[1] : r.host_step;
  const float4* in = (step & 1) ? buf_odd : buf_even;       // the buffer that holds the current values
  float4* out = (step & 1) ? buf_even : buf_odd;
  const float wtv = r.tv_w_dev != nullptr ? *r.tv_w_dev : r.tv_w;
  const float ch = wtv * r.tv_h, cw = wtv * r.tv_w_scale;
  const int c4 = r.C >> 2;
  const long long row4 = (long long)r.W * c4;
  float tv_h_sum = 0.f, tv_w_sum = 0.f, l1_sum = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const long long texel = i / c4;
    const int x = (int)(texel % r.W);
    const int y = (int)((texel / r.W) % r.H);
    float4 pp = ld4(in + i), gg = g[i], mm = m[i], vv = v[i];
    const bool has_l = x > 0, has_r = x + 1 < r.W, has_u = y > 0, has_d = y + 1 < r.H;
    const float4 pl = has_l ? ld4(in + i - c4) : pp, pr = has_r ? ld4(in + i + c4) : pp;
    const float4 pu = has_u ? ld4(in + i - row4) : pp, pd = has_d ? ld4(in + i + row4) : pp;
    float* G = &gg.x; float* P = &pp.x; float* M = &mm.x; float* V = &vv.x;
    const float* L = &pl.x; const float* R = &pr.x; const float* U = &pu.x; const float* D = &pd.x;
    float4 po;
    float* O = &po.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float dr = R[k] - P[k], dd = D[k] - P[k];           // forward differences (zero at the far edges)
      tv_w_sum += dr * dr; tv_h_sum += dd * dd;
      l1_sum += fabsf(P[k]);
      const float sgn = P[k] > 0.f ? 1.f : (P[k] < 0.f ? -1.f : 0.f);
      const float reg = cw * ((P[k] - L[k]) - dr) + ch * ((P[k] - U[k]) - dd) + r.l1 * sgn;
      const float gr = G[k] * a.grad_scale + reg + a.weight_decay * P[k];
      M[k] = a.beta1 * M[k] + (1.f - a.beta1) * gr;
      V[k] = a.beta2 * V[k] + (1.f - a.beta2) * gr * gr;
      O[k] = P[k] - st.step * M[k] / (st.adaptive ? sqrtf(V[k]) * st.vscale + a.eps : 1.f);
    }
    out[i] = po; m[i] = mm; v[i] = vv;
    g[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    __nv_bfloat162 lo = __floats2bfloat162_rn(po.x, po.y), hi = __floats2bfloat162_rn(po.z, po.w);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&lo); u.y = *reinterpret_cast<unsigned*>(&hi);
    shadow[i] = u;
  }
  if (r.loss != nullptr) {
    __shared__ float red[3][8];
    float vals[3] = {tv_h_sum * ch + tv_w_sum * cw, l1_sum * r.l1, 0.f};
#pragma unroll
    for (int q = 0; q < 2; ++q)
      for (int o = 16; o > 0; o >>= 1) vals[q] += __shfl_xor_sync(0xffffffffu, vals[q], o);
    if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = vals[0]; red[1][threadIdx.x >> 5] = vals[1]; }
    __syncthreads();
    if (threadIdx.x < 2) {
      float t = 0.f;
      for (int wq = 0; wq < 8; ++wq) t += red[threadIdx.x][wq];
      // value = sum of squares * (w * 0.02 / count): the gradient coefficient carries an extra factor 2
      atomicAdd(r.loss + threadIdx.x, t * r.inv_loss_scale * (threadIdx.x == 0 ? 0.5f : 1.f));
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

// Dense Adam of one channels-last plane [B, H, W, C] (C a multiple of 4) fused with its TV / L1 regularisers; see
// adam_plane_reg_kernel.  buf_odd / buf_even: the two parameter buffers - buf_odd holds the current values when the
// step number being applied is odd.  dyn: device-resident {lr, step} (then lr / step are ignored) or null.
// tv_weight_dev: device float (the decaying TV weight) or null (then tv_weight).  loss_scale multiplies the
// regulariser gradients (the factor the caller applies to its total loss); loss_out: optional float[2]
// accumulators that receive the TV and L1 loss values of this plane.
LMB_API int lmb_adam_plane_reg(float* buf_odd, float* buf_even, float* g, float* m, float* v, void* shadow_bf16, int B, int H, int W,
                               int C, const float* dyn, float lr, int step, float beta1, float beta2, float eps, float grad_scale,
                               const float* tv_weight_dev, float tv_weight, float l1_weight, float loss_scale, float* loss_out,
                               cudaStream_t stream) {
  const long long n = (long long)B * H * W * C;
  if (n <= 0) return 0;
  if (C % 4 != 0 || shadow_bf16 == nullptr || buf_odd == buf_even) return (int)cudaErrorInvalidValue;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.grad_scale = grad_scale; a.weight_decay = 0.f;
  a.bias1 = 1.f - powf(beta1, (float)step);
  a.bias2 = 1.f - powf(beta2, (float)step);
  a.dyn = dyn; a.l2_beta1 = (float)log2((double)beta1); a.l2_beta2 = (float)log2((double)beta2); a.mode = 0; a.A = 0.f;
  PlaneReg r;
  r.B = B; r.H = H; r.W = W; r.C = C;
  r.tv_w_dev = tv_weight_dev; r.tv_w = tv_weight;
  const double count_h = (double)C * (H > 1 ? H - 1 : 1) * W * B, count_w = (double)C * H * (W > 1 ? W - 1 : 1) * B;
  r.tv_h = (float)(0.04 / count_h * loss_scale); r.tv_w_scale = (float)(0.04 / count_w * loss_scale);
  r.l1 = (float)((double)l1_weight / (double)n * loss_scale);
  r.loss = loss_out; r.inv_loss_scale = loss_scale != 0.f ? 1.f / loss_scale : 0.f;
  r.host_step = step;
  const long long n4 = n / 4, want = (n4 + 255) / 256;
  const int blocks = (int)(want < 148LL * 16 ? want : 148LL * 16);
  adam_plane_reg_kernel<<<blocks, 256, 0, stream>>>((float4*)buf_odd, (float4*)buf_even, (float4*)g, (float4*)m, (float4*)v,
                                                    (uint2*)shadow_bf16, n4, a, r);
  LMB_LAUNCH_CHECK();
  return 0;
}
