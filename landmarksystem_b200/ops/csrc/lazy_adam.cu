// Lazy (deferred) Adam for feature planes: exact Adam semantics at a fraction of the memory traffic.
//
// A training step touches only the texels its samples fall on (about a quarter of a 4096^2 plane for
// 10^6 samples), yet a dense Adam pass reads and writes every parameter and both moments each step
// (34 bytes per parameter; 36 GB per step for a 10^9-parameter grid, which dominated the step).  With
// zero gradient the Adam recurrence of an element needs nothing but its own state,
//     m <- b1 m,  v <- b2 v,  p <- p - lr_k / (1 - b1^k) * m / (sqrt(v / (1 - b2^k)) + eps),
// so an untouched texel can be left alone and caught up later by replaying the skipped steps in
// registers.  Per step:
//   mark     every texel the step's samples will read is claimed (need = 1) and appended to a list (vm_mark)
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
};

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

// The texels a step touches are kept as a compact list (filled by vm_mark, which claims a texel with an
// atomic compare-and-swap on its flag), so prepare / step cost scales with the touched set and never scan
// the plane.  need: 0 idle, 1 marked, 2 prepared.  One thread per (list entry, 4-channel group).
__global__ void __launch_bounds__(256)
lazy_prepare_kernel(const int* __restrict__ need, const int* __restrict__ last_step, const int* __restrict__ list,
                    const int* __restrict__ list_count, const float4* __restrict__ p, const float4* __restrict__ m,
                    const float4* __restrict__ v, uint2* __restrict__ shadow, int c4, LazySched s) {
  const long long total = (long long)(*list_count) * c4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int texel = list[i / c4];
    if (need[texel] != 1) continue;
    const int last = last_step[texel];
    if (last >= s.t - 1) continue;
    const long long e = (long long)texel * c4 + (i % c4);
    float4 pp = p[e], mm = m[e], vv = v[e];
    Replay r = replay_start(s, last + 1);
    for (int k = last + 1; k < s.t; ++k) zero_grad_step(pp, mm, vv, s, r);
    shadow[e] = to_bf16x4(pp);
  }
}

// after prepare: marked -> prepared (a separate launch, so every channel group has seen need == 1)
__global__ void __launch_bounds__(256)
lazy_mark_prepared_kernel(int* __restrict__ need, const int* __restrict__ list, const int* __restrict__ list_count) {
  const int total = *list_count;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int texel = list[i];
    if (need[texel] == 1) need[texel] = 2;
  }
}

__device__ __forceinline__ void lazy_apply(long long e, int last, float4* p, float4* g, float4* m, float4* v, uint2* shadow,
                                           const LazySched& s, float grad_scale, bool flush) {
  const int upto = flush ? s.t : s.t - 1;        // zero-gradient steps to replay: last+1 .. upto
  float4 pp = p[e], mm = m[e], vv = v[e];
  Replay r = replay_start(s, last + 1);
  for (int k = last + 1; k <= upto; ++k) zero_grad_step(pp, mm, vv, s, r);
  if (!flush) {
    float4 gg = g[e];
    const float step = r.lr / (1.f - r.b1p);
    const float inv_sqrt_b2 = rsqrtf(1.f - r.b2p);
    float* G = &gg.x; float* P = &pp.x; float* M = &mm.x; float* V = &vv.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gr = G[k] * grad_scale;
      M[k] = s.beta1 * M[k] + (1.f - s.beta1) * gr;
      V[k] = s.beta2 * V[k] + (1.f - s.beta2) * gr * gr;
      P[k] -= step * M[k] / (sqrtf(V[k]) * inv_sqrt_b2 + s.eps);
    }
    g[e] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  p[e] = pp; m[e] = mm; v[e] = vv;
  if (shadow) shadow[e] = to_bf16x4(pp);
}

// step t over the touched list
__global__ void __launch_bounds__(256)
lazy_step_kernel(const int* __restrict__ last_step, const int* __restrict__ list, const int* __restrict__ list_count,
                 float4* __restrict__ p, float4* __restrict__ g, float4* __restrict__ m, float4* __restrict__ v,
                 uint2* __restrict__ shadow, int c4, LazySched s, float grad_scale) {
  const long long total = (long long)(*list_count) * c4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int texel = list[i / c4];
    lazy_apply((long long)texel * c4 + (i % c4), last_step[texel], p, g, m, v, shadow, s, grad_scale, false);
  }
}

// second half of a step: bookkeeping per touched texel (separate so that all channel groups have read
// last_step before it changes)
__global__ void __launch_bounds__(256)
lazy_commit_kernel(int* __restrict__ need, int* __restrict__ last_step, const int* __restrict__ list,
                   const int* __restrict__ list_count, int t) {
  const int total = *list_count;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int texel = list[i];
    last_step[texel] = t;
    need[texel] = 0;
  }
}

// flush: every texel of the plane that is behind step s.t replays up to it (no gradient)
__global__ void __launch_bounds__(256)
lazy_flush_kernel(const int* __restrict__ last_step, float4* __restrict__ p, float4* __restrict__ m, float4* __restrict__ v,
                  uint2* __restrict__ shadow, int c4, long long n_texels, LazySched s) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long texel = e / c4;
  if (texel >= n_texels) return;
  const int last = last_step[texel];
  if (last >= s.t) return;
  lazy_apply(e, last, p, nullptr, m, v, shadow, s, 1.f, true);
}
__global__ void __launch_bounds__(256) lazy_flush_commit_kernel(int* __restrict__ last_step, long long n_texels, int t) {
  const long long texel = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (texel < n_texels && last_step[texel] < t) last_step[texel] = t;
}

// Claim the 4 corner texels of every sample on one plane level (same tap rule as the lookup kernel) and
// append newly claimed ones to the list; list positions are handed out per warp (one atomic per warp).
__global__ void __launch_bounds__(256)
vm_mark_kernel(const float4* __restrict__ coords, const int* __restrict__ count_ptr, long long max_n, int B, int H, int W,
               int* __restrict__ need, int* __restrict__ list, int* __restrict__ list_count, int list_cap) {
  const long long n_valid = resolve_count(count_ptr, max_n);
  const long long n = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31;
  bool active = n < n_valid;
  float4 q = make_float4(0.f, 0.f, 0.f, -1.f);
  if (active) q = __ldg(coords + n);
  const int b = (int)q.w;
  active = active && b >= 0 && b < B;
  const float fx = (q.x + 1.f) * 0.5f * (float)(W - 1), fy = (q.y + 1.f) * 0.5f * (float)(H - 1);
  const int x0 = (int)floorf(fx), y0 = (int)floorf(fy);
#pragma unroll
  for (int corner = 0; corner < 4; ++corner) {
    int texel = -1;
    if (active) {
      const int x = min(max(x0 + (corner & 1), 0), W - 1), y = min(max(y0 + (corner >> 1), 0), H - 1);
      const int t = (b * H + y) * W + x;
      if (need[t] == 0 && atomicCAS(need + t, 0, 1) == 0) texel = t;
    }
    const unsigned won = __ballot_sync(0xffffffffu, texel >= 0);
    if (won) {
      int base = 0;
      if (lane == __ffs(won) - 1) base = atomicAdd(list_count, __popc(won));
      base = __shfl_sync(0xffffffffu, base, __ffs(won) - 1);
      if (texel >= 0) {
        const int pos = base + __popc(won & ((1u << lane) - 1u));
        if (pos < list_cap) list[pos] = texel;
      }
    }
  }
}

}  // namespace lmb

using namespace lmb;

static LazySched make_sched(float lr_ref, int t_ref, float decay, float beta1, float beta2, float eps, int t) {
  LazySched s;
  s.lr_ref = lr_ref; s.t_ref = t_ref; s.decay = decay; s.beta1 = beta1; s.beta2 = beta2; s.eps = eps; s.t = t;
  s.l2_decay = (float)log2((double)decay); s.l2_beta1 = (float)log2((double)beta1); s.l2_beta2 = (float)log2((double)beta2);
  return s;
}

static int list_grid(long long work) {
  const long long blocks = (work + 255) / 256;
  return (int)(blocks < 148 * 16 ? (blocks > 0 ? blocks : 1) : 148 * 16);
}

// need: int32 [B*H*W]; list: int32 [list_cap] with *list_count entries in use (list_cap >= 4 * max_n per call
// outstanding guarantees no overflow; entries past the capacity are dropped and reported by lmb_lazy_list_ok).
LMB_API int lmb_vm_mark(const float* coords, const int* count_ptr, long long max_n, int B, int H, int W, int* need, int* list,
                        int* list_count, int list_cap, cudaStream_t stream) {
  if (max_n <= 0) return 0;
  vm_mark_kernel<<<ceil_div(max_n, 256), 256, 0, stream>>>((const float4*)coords, count_ptr, max_n, B, H, W, need, list,
                                                          list_count, list_cap);
  LMB_LAUNCH_CHECK();
  return 0;
}

// work_hint: upper bound of list entries (sizes the grid; the kernels read the true count on the device)
LMB_API int lmb_lazy_adam_prepare(int* need, const int* last_step, const int* list, const int* list_count, long long work_hint,
                                  const float* p, const float* m, const float* v, void* shadow, int C, float lr_ref, int t_ref,
                                  float decay, float beta1, float beta2, float eps, int t, cudaStream_t stream) {
  if (C % 4) return (int)cudaErrorInvalidValue;
  const int c4 = C / 4;
  lazy_prepare_kernel<<<list_grid(work_hint * c4), 256, 0, stream>>>(need, last_step, list, list_count, (const float4*)p,
                                                                    (const float4*)m, (const float4*)v, (uint2*)shadow, c4,
                                                                    make_sched(lr_ref, t_ref, decay, beta1, beta2, eps, t));
  LMB_LAUNCH_CHECK();
  lazy_mark_prepared_kernel<<<list_grid(work_hint), 256, 0, stream>>>(need, list, list_count);
  LMB_LAUNCH_CHECK();
  return 0;
}

// One optimiser step over the touched list; clears the list afterwards.
LMB_API int lmb_lazy_adam_step(int* need, int* last_step, const int* list, int* list_count, long long work_hint, float* p,
                               float* g, float* m, float* v, void* shadow, int C, float lr_ref, int t_ref, float decay,
                               float beta1, float beta2, float eps, int t, float grad_scale, cudaStream_t stream) {
  if (C % 4) return (int)cudaErrorInvalidValue;
  const int c4 = C / 4;
  lazy_step_kernel<<<list_grid(work_hint * c4), 256, 0, stream>>>(last_step, list, list_count, (float4*)p, (float4*)g,
                                                                 (float4*)m, (float4*)v, (uint2*)shadow, c4,
                                                                 make_sched(lr_ref, t_ref, decay, beta1, beta2, eps, t),
                                                                 grad_scale);
  LMB_LAUNCH_CHECK();
  lazy_commit_kernel<<<list_grid(work_hint), 256, 0, stream>>>(need, last_step, list, list_count, t);
  LMB_LAUNCH_CHECK();
  LMB_CUDA_TRY(cudaMemsetAsync(list_count, 0, sizeof(int), stream));
  return 0;
}

// Bring every texel up to step t (zero-gradient replay); call between steps (empty list).
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
