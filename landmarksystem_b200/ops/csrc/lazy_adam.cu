// Lazy (deferred) Adam for feature planes: exact Adam semantics at a fraction of the memory traffic.
//
// A training step touches only the texels its samples fall on (about a quarter of a 4096^2 plane for
// 10^6 samples), yet a dense Adam pass reads and writes every parameter and both moments each step
// (34 bytes per parameter; 36 GB per step for a 10^9-parameter grid, which dominated the step).  With
// zero gradient the Adam recurrence of an element needs nothing but its own state,
//     m <- b1 m,  v <- b2 v,  p <- p - lr_k / (1 - b1^k) * m / (sqrt(v / (1 - b2^k)) + eps),
// so an untouched texel can be left alone and caught up later by replaying the skipped steps in
// registers.  Per step:
//   mark     every texel the step's samples will read gets need = 1                         (vm_mark)
//   prepare  needed texels that are behind get their bf16 shadow value brought to "after step t-1"
//            (reads p, m, v; writes only the 2-byte shadow)
//   step     after backward, needed texels replay their skipped steps, apply step t with the real
//            gradient, store p / m / v / shadow once, clear the gradient and record last_step = t
//   flush    brings every texel up to date (before checkpoints, evaluation, resizing).
// The learning-rate schedule is the trainers' geometric decay: lr_k = lr_t * decay^(k - t).
#include "common.cuh"
#include <cmath>

namespace lmb {

struct LazySched {
  float lr_ref;    // learning rate of step t_ref
  int t_ref;
  float decay;     // lr_{k+1} = lr_k * decay
  float beta1, beta2, eps;
  float l2_decay, l2_beta1, l2_beta2;   // log2 of the three bases (host, double precision)
  int t;           // step being prepared / applied, or (flush) the last completed step (1-based)
  const float* dyn;  // optional device-resident {lr of the step being applied, its number}: overrides lr_ref, t_ref, t
};

__device__ __forceinline__ void resolve_dyn(LazySched& s) {
  if (s.dyn != nullptr) {
    s.lr_ref = s.dyn[0];
    s.t_ref = s.t = (int)s.dyn[1];
  }
}

struct Replay {
  float lr, b1p, b2p;   // lr_k, beta1^k, beta2^k of the NEXT step to replay
};

__device__ __forceinline__ Replay replay_start(const LazySched& s, int k) {
  Replay r;
  r.lr = s.lr_ref * exp2f(s.l2_decay * (float)(k - s.t_ref));
  r.b1p = exp2f(s.l2_beta1 * (float)k);
  r.b2p = exp2f(s.l2_beta2 * (float)k);
  return r;
}

// advance one zero-gradient step for 4 elements
__device__ __forceinline__ void zero_grad_step(float4& p, float4& m, float4& v, const LazySched& s, Replay& r) {
  const float step = r.lr / (1.f - r.b1p);
  const float inv_sqrt_b2 = rsqrtf(1.f - r.b2p);
  float* P = &p.x; float* M = &m.x; float* V = &v.x;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    M[k] *= s.beta1;
    V[k] *= s.beta2;
    P[k] -= step * M[k] / (sqrtf(V[k]) * inv_sqrt_b2 + s.eps);
  }
  r.lr *= s.decay; r.b1p *= s.beta1; r.b2p *= s.beta2;
}

__device__ __forceinline__ uint2 to_bf16x4(const float4& p) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(p.x, p.y), hi = __floats2bfloat162_rn(p.z, p.w);
  uint2 u;
  u.x = *reinterpret_cast<unsigned*>(&lo); u.y = *reinterpret_cast<unsigned*>(&hi);
  return u;
}

// Kernels walk the plane's one-byte flags in texel order, one warp per 32 texels: the warp compacts the
// flagged texels of its chunk with a ballot and spreads their (texel, 4-channel group) work items over its
// lanes, so every texel's channels are read and written as one contiguous run and addresses only ever
// increase (the flags themselves are 1/64th .. 1/192th of the parameter bytes).
// need: 0 idle, 1 marked, 2 prepared.
constexpr int kMaxReplay = 192;   // beta1^192 < 2e-9: later zero-gradient steps cannot change an fp32 parameter

// number of zero-gradient steps to run explicitly / to fold into a moment decay afterwards
__device__ __forceinline__ void replay_plan(int last, int upto, int& n_explicit, int& n_rest) {
  const int n = (last == 0 || upto <= last) ? 0 : upto - last;   // never stepped: both moments are zero and stay zero
  n_explicit = n < kMaxReplay ? n : kMaxReplay;
  n_rest = n - n_explicit;
}
__device__ __forceinline__ void decay_moments(float4& mm, float4& vv, const LazySched& s, int n_rest) {
  if (n_rest > 0) {                               // the remaining steps only decay the moments
    const float d1 = exp2f(s.l2_beta1 * (float)n_rest), d2 = exp2f(s.l2_beta2 * (float)n_rest);
    mm.x *= d1; mm.y *= d1; mm.z *= d1; mm.w *= d1;
    vv.x *= d2; vv.y *= d2; vv.z *= d2; vv.w *= d2;
  }
}

template <bool kPrepare>
__global__ void __launch_bounds__(256)
lazy_scan_kernel(unsigned char* __restrict__ need, int* __restrict__ last_step, float4* __restrict__ p, float4* __restrict__ g,
                 float4* __restrict__ m, float4* __restrict__ v, uint2* __restrict__ shadow, int c4, long long n_texels,
                 LazySched s, float grad_scale) {
  resolve_dyn(s);
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long chunk = warp0; chunk * 32 < n_texels; chunk += n_warps) {
    const long long texel = chunk * 32 + lane;
    const unsigned char flag = texel < n_texels ? need[texel] : 0;
    const int last = flag ? last_step[texel] : 0;
    const bool mine = kPrepare ? (flag == 1) : (flag != 0);
    const bool work = kPrepare ? (mine && last > 0 && last < s.t - 1) : mine;
    const unsigned mask = __ballot_sync(0xffffffffu, work);
    const int total = __popc(mask) * c4;
    // Every lane runs every statement below (loads, stores and arithmetic are predicated on `on`): the
    // replay loop has ONE trip count per warp, so lanes never split and each memory instruction is issued
    // once per warp with all its addresses together.
    for (int w0 = 0; w0 < total; w0 += 32) {
      const int w = w0 + lane;
      const bool on = w < total;
      const int which = on ? w / c4 : 0, grp = w - which * c4;
      const int src = __fns(mask, 0, which + 1);                 // lane that owns the which-th flagged texel
      const int last_t = __shfl_sync(0xffffffffu, last, src);
      const long long e = (chunk * 32 + src) * c4 + grp;
      const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
      float4 pp = on ? p[e] : zero, mm = on ? m[e] : zero, vv = on ? v[e] : zero;
      float4 gg = zero;
      if (!kPrepare && on) gg = g[e];
      int n_explicit, n_rest;
      replay_plan(on ? last_t : 0, s.t - 1, n_explicit, n_rest);
      const int n_warp = __reduce_max_sync(0xffffffffu, n_explicit);
      Replay r = replay_start(s, last_t + 1);
      for (int k = 0; k < n_warp; ++k) {
        float4 p2 = pp, m2 = mm, v2 = vv;
        Replay r2 = r;
        zero_grad_step(p2, m2, v2, s, r2);
        if (k < n_explicit) { pp = p2; mm = m2; vv = v2; r = r2; }   // selects, not branches
      }
      decay_moments(mm, vv, s, n_rest);
      if (kPrepare) {
        if (on) shadow[e] = to_bf16x4(pp);
      } else {
        Replay rt = replay_start(s, s.t);
        const float step = rt.lr / (1.f - rt.b1p);
        const float inv_sqrt_b2 = rsqrtf(1.f - rt.b2p);
        const float* G = &gg.x; float* P = &pp.x; float* M = &mm.x; float* V = &vv.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float gr = G[k] * grad_scale;
          M[k] = s.beta1 * M[k] + (1.f - s.beta1) * gr;
          V[k] = s.beta2 * V[k] + (1.f - s.beta2) * gr * gr;
          P[k] -= step * M[k] / (sqrtf(V[k]) * inv_sqrt_b2 + s.eps);
        }
        if (on) {
          g[e] = zero;
          p[e] = pp; m[e] = mm; v[e] = vv;
          if (shadow) shadow[e] = to_bf16x4(pp);
        }
      }
    }
    __syncwarp();
    if (mine) {
      if (kPrepare) need[texel] = 2;
      else { need[texel] = 0; last_step[texel] = s.t; }
    }
  }
}

// flush: every texel of the plane that is behind step s.t replays up to it (no gradient); one thread
// per (texel, group), last_step is advanced by a second launch
__global__ void __launch_bounds__(256)
lazy_flush_kernel(const int* __restrict__ last_step, float4* __restrict__ p, float4* __restrict__ m, float4* __restrict__ v,
                  uint2* __restrict__ shadow, int c4, long long n_texels, LazySched s) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long texel = e / c4;
  if (texel >= n_texels) return;
  const int last = last_step[texel];
  if (last >= s.t || last == 0) return;
  float4 pp = p[e], mm = m[e], vv = v[e];
  int n_explicit, n_rest;
  replay_plan(last, s.t, n_explicit, n_rest);
  Replay r = replay_start(s, last + 1);
  for (int k = 0; k < n_explicit; ++k) zero_grad_step(pp, mm, vv, s, r);
  decay_moments(mm, vv, s, n_rest);
  p[e] = pp; m[e] = mm; v[e] = vv;
  if (shadow) shadow[e] = to_bf16x4(pp);
}
__global__ void __launch_bounds__(256) lazy_flush_commit_kernel(int* __restrict__ last_step, long long n_texels, int t) {
  const long long texel = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (texel < n_texels && last_step[texel] < t) last_step[texel] = t;
}

// Flag the 4 corner texels of every sample on one plane level (same tap rule as the lookup kernel).
__global__ void __launch_bounds__(256)
vm_mark_kernel(const float4* __restrict__ coords, const int* __restrict__ count_ptr, long long max_n, int B, int H, int W,
               unsigned char* __restrict__ need) {
  const long long n_valid = resolve_count(count_ptr, max_n);
  const long long n = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= n_valid) return;
  const float4 q = __ldg(coords + n);
  const int b = (int)q.w;
  if (b < 0 || b >= B) return;
  const float fx = (q.x + 1.f) * 0.5f * (float)(W - 1), fy = (q.y + 1.f) * 0.5f * (float)(H - 1);
  const int x0 = (int)floorf(fx), y0 = (int)floorf(fy);
#pragma unroll
  for (int corner = 0; corner < 4; ++corner) {
    const int x = min(max(x0 + (corner & 1), 0), W - 1), y = min(max(y0 + (corner >> 1), 0), H - 1);
    unsigned char* f = need + ((long long)b * H + y) * W + x;
    if (*f == 0) *f = 1;
  }
}

}  // namespace lmb

using namespace lmb;

static LazySched make_sched(float lr_ref, int t_ref, float decay, float beta1, float beta2, float eps, int t,
                            const float* dyn = nullptr) {
  LazySched s;
  s.dyn = dyn;
  s.lr_ref = lr_ref; s.t_ref = t_ref; s.decay = decay; s.beta1 = beta1; s.beta2 = beta2; s.eps = eps; s.t = t;
  s.l2_decay = (float)log2((double)decay); s.l2_beta1 = (float)log2((double)beta1); s.l2_beta2 = (float)log2((double)beta2);
  return s;
}

static int scan_grid(long long n_texels) {
  const long long blocks = (n_texels + 255) / 256;     // one warp per 32 texels, 8 warps per block
  return (int)(blocks < 148 * 32 ? (blocks > 0 ? blocks : 1) : 148 * 32);
}

// need: uint8 [B*H*W]
LMB_API int lmb_vm_mark(const float* coords, const int* count_ptr, long long max_n, int B, int H, int W, unsigned char* need,
                        cudaStream_t stream) {
  if (max_n <= 0) return 0;
  vm_mark_kernel<<<ceil_div(max_n, 256), 256, 0, stream>>>((const float4*)coords, count_ptr, max_n, B, H, W, need);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_lazy_adam_prepare(unsigned char* need, int* last_step, const float* p, const float* m, const float* v,
                                  void* shadow, int C, long long n_texels, float lr_ref, int t_ref, float decay, float beta1,
                                  float beta2, float eps, int t, const float* dyn, cudaStream_t stream) {
  if (C % 4) return (int)cudaErrorInvalidValue;
  if (n_texels <= 0) return 0;
  lazy_scan_kernel<true><<<scan_grid(n_texels), 256, 0, stream>>>(need, last_step, (float4*)p, nullptr, (float4*)m, (float4*)v,
                                                                 (uint2*)shadow, C / 4, n_texels,
                                                                 make_sched(lr_ref, t_ref, decay, beta1, beta2, eps, t, dyn), 1.f);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_lazy_adam_step(unsigned char* need, int* last_step, float* p, float* g, float* m, float* v, void* shadow,
                               int C, long long n_texels, float lr_ref, int t_ref, float decay, float beta1, float beta2,
                               float eps, int t, float grad_scale, const float* dyn, cudaStream_t stream) {
  if (C % 4) return (int)cudaErrorInvalidValue;
  if (n_texels <= 0) return 0;
  lazy_scan_kernel<false><<<scan_grid(n_texels), 256, 0, stream>>>(need, last_step, (float4*)p, (float4*)g, (float4*)m,
                                                                  (float4*)v, (uint2*)shadow, C / 4, n_texels,
                                                                  make_sched(lr_ref, t_ref, decay, beta1, beta2, eps, t, dyn),
                                                                  grad_scale);
  LMB_LAUNCH_CHECK();
  return 0;
}

// Bring every texel up to step t (zero-gradient replay); call between steps (no flags set).
LMB_API int lmb_lazy_adam_flush(int* last_step, float* p, float* m, float* v, void* shadow, int C, long long n_texels,
                                float lr_ref, int t_ref, float decay, float beta1, float beta2, float eps, int t,
                                cudaStream_t stream) {
  if (C % 4) return (int)cudaErrorInvalidValue;
  if (n_texels <= 0) return 0;
  const int c4 = C / 4;
  lazy_flush_kernel<<<ceil_div(n_texels * c4, 256), 256, 0, stream>>>(last_step, (float4*)p, (float4*)m, (float4*)v,
                                                                     (uint2*)shadow, c4, n_texels,
                                                                     make_sched(lr_ref, t_ref, decay, beta1, beta2, eps, t));
  LMB_LAUNCH_CHECK();
  lazy_flush_commit_kernel<<<ceil_div(n_texels, 256), 256, 0, stream>>>(last_step, n_texels, t);
  LMB_LAUNCH_CHECK();
  return 0;
}
