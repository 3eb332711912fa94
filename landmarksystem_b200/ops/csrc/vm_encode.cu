// VM (vector-matrix) feature-grid lookup for GridNeRF-style fields, forward and backward.
//
// A sample carries block-local coordinates (x, y, z) in [-1, 1] and the index b of the spatial
// block that owns it.  For every resolution level l the feature is
//     bilinear(plane_l[b], x, y)  *  linear(line_l[b], z)          (element-wise over C channels)
// with align_corners=True / zero-padding semantics, and levels are concatenated: out[n, l*C + c].
// This is the math of the reference's 5-D/4-D F.grid_sample pair followed by the product
// (landmark/nerf_components/model_components/fields/encodings/tensor_vm_encoding.py:129-197) and of
// its channels-last kernel (landmark/ops/kernel/densityappfeature/grid_sampler_3d_ndhwc_kernel.cu:206-369),
// re-designed around the memory system: planes are stored channels-last [B, H, W, C] so one texel
// is one or three 32-byte sectors, each thread moves 8 channels with a single 16-byte load, and the
// plane * line product and the level concat are fused so no intermediate ever reaches HBM.
#include "common.cuh"

namespace lmb {

struct VMLevels {
  const void* plane[kMaxLevels];  // [B, H, W, C]
  const void* line[kMaxLevels];   // [B, Z, C]
  float* gplane[kMaxLevels];      // fp32 gradient accumulators, same shapes (backward only)
  float* gline[kMaxLevels];
  int H[kMaxLevels], W[kMaxLevels], Z[kMaxLevels];
  int L, C, B;
};

struct Corner2 {
  int i0, i1;
  float w0, w1;  // weights already zeroed for out-of-range taps
};

__device__ __forceinline__ Corner2 taps(float u, int size) {
  // u in [-1, 1] -> continuous index in [0, size-1] (align_corners=True); zero padding outside.
  float f = (u + 1.f) * 0.5f * (float)(size - 1);
  float fl = floorf(f);
  int i0 = (int)fl;
  float t = f - fl;
  Corner2 c;
  c.i0 = i0; c.i1 = i0 + 1;
  c.w0 = (i0 >= 0 && i0 < size) ? 1.f - t : 0.f;
  c.w1 = (c.i1 >= 0 && c.i1 < size) ? t : 0.f;
  c.i0 = min(max(c.i0, 0), size - 1);
  c.i1 = min(max(c.i1, 0), size - 1);
  return c;
}

template <typename T, typename OutT>
__global__ void __launch_bounds__(256)
vm_encode_fwd_kernel(const float4* __restrict__ coords, const int* __restrict__ count_ptr, long long max_n,
                     VMLevels lv, OutT* __restrict__ out, int out_stride) {
  const int CH = lv.C >> 3;
  const long long n_valid = resolve_count(count_ptr, max_n);
  // grid-stride: the grid is capped, so a launch sized for a worst-case row capacity costs nothing when
  // the device-side count is small
  for (long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x; tid < n_valid * CH;
       tid += (long long)gridDim.x * blockDim.x) {
  long long n = tid / CH;
  int ch = (int)(tid - n * CH);
  float4 q = __ldg(coords + n);
  int b = (int)q.w;
  if (b < 0 || b >= lv.B) {
    F8 z;
#pragma unroll
    for (int i = 0; i < 8; ++i) z.v[i] = 0.f;
    for (int l = 0; l < lv.L; ++l) store8(out + n * out_stride + l * lv.C + ch * 8, z);
    continue;
  }
  for (int l = 0; l < lv.L; ++l) {
    const int H = lv.H[l], W = lv.W[l], Z = lv.Z[l];
    Corner2 cx = taps(q.x, W), cy = taps(q.y, H), cz = taps(q.z, Z);
    const T* pl = reinterpret_cast<const T*>(lv.plane[l]) + ((long long)b * H * W) * lv.C + ch * 8;
    const T* ln = reinterpret_cast<const T*>(lv.line[l]) + ((long long)b * Z) * lv.C + ch * 8;
    F8 p00 = load8(pl + ((long long)cy.i0 * W + cx.i0) * lv.C);
    F8 p01 = load8(pl + ((long long)cy.i0 * W + cx.i1) * lv.C);
    F8 p10 = load8(pl + ((long long)cy.i1 * W + cx.i0) * lv.C);
    F8 p11 = load8(pl + ((long long)cy.i1 * W + cx.i1) * lv.C);
    F8 l0 = load8(ln + (long long)cz.i0 * lv.C);
    F8 l1 = load8(ln + (long long)cz.i1 * lv.C);
    const float w00 = cy.w0 * cx.w0, w01 = cy.w0 * cx.w1, w10 = cy.w1 * cx.w0, w11 = cy.w1 * cx.w1;
    F8 f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float pv = w00 * p00.v[i] + w01 * p01.v[i] + w10 * p10.v[i] + w11 * p11.v[i];
      float lvv = cz.w0 * l0.v[i] + cz.w1 * l1.v[i];
      f.v[i] = pv * lvv;
    }
    store8(out + n * out_stride + l * lv.C + ch * 8, f);
  }
  }
}

// Backward: recompute the taps and both interpolants, then push d(plane) and d(line) with
// 16-byte vector reductions into the fp32 accumulators.
template <typename T, typename GT>
__global__ void __launch_bounds__(256)
vm_encode_bwd_kernel(const float4* __restrict__ coords, const int* __restrict__ count_ptr, long long max_n,
                     VMLevels lv, const GT* __restrict__ dout, int out_stride) {
  const int CH = lv.C >> 3;
  const long long n_valid = resolve_count(count_ptr, max_n);
  for (long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x; tid < n_valid * CH;
       tid += (long long)gridDim.x * blockDim.x) {
  long long n = tid / CH;
  int ch = (int)(tid - n * CH);
  float4 q = __ldg(coords + n);
  int b = (int)q.w;
  if (b < 0 || b >= lv.B) continue;
  for (int l = 0; l < lv.L; ++l) {
    const int H = lv.H[l], W = lv.W[l], Z = lv.Z[l];
    Corner2 cx = taps(q.x, W), cy = taps(q.y, H), cz = taps(q.z, Z);
    const long long pbase = ((long long)b * H * W) * lv.C + ch * 8;
    const long long lbase = ((long long)b * Z) * lv.C + ch * 8;
    const T* pl = reinterpret_cast<const T*>(lv.plane[l]) + pbase;
    const T* ln = reinterpret_cast<const T*>(lv.line[l]) + lbase;
    const long long o00 = ((long long)cy.i0 * W + cx.i0) * lv.C, o01 = ((long long)cy.i0 * W + cx.i1) * lv.C;
    const long long o10 = ((long long)cy.i1 * W + cx.i0) * lv.C, o11 = ((long long)cy.i1 * W + cx.i1) * lv.C;
    F8 p00 = load8(pl + o00), p01 = load8(pl + o01), p10 = load8(pl + o10), p11 = load8(pl + o11);
    F8 l0 = load8(ln + (long long)cz.i0 * lv.C), l1 = load8(ln + (long long)cz.i1 * lv.C);
    F8 g = load8(dout + n * out_stride + l * lv.C + ch * 8);
    const float w00 = cy.w0 * cx.w0, w01 = cy.w0 * cx.w1, w10 = cy.w1 * cx.w0, w11 = cy.w1 * cx.w1;
    F8 dp, dl;
    bool any = false;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float pv = w00 * p00.v[i] + w01 * p01.v[i] + w10 * p10.v[i] + w11 * p11.v[i];
      float lvv = cz.w0 * l0.v[i] + cz.w1 * l1.v[i];
      dp.v[i] = g.v[i] * lvv;
      dl.v[i] = g.v[i] * pv;
      any |= (g.v[i] != 0.f);
    }
    if (!any) continue;
    float* gp = lv.gplane[l] + pbase;
    float* gl = lv.gline[l] + lbase;
    if (w00 != 0.f) red_add8(gp + o00, dp, w00);
    if (w01 != 0.f) red_add8(gp + o01, dp, w01);
    if (w10 != 0.f) red_add8(gp + o10, dp, w10);
    if (w11 != 0.f) red_add8(gp + o11, dp, w11);
    if (cz.w0 != 0.f) red_add8(gl + (long long)cz.i0 * lv.C, dl, cz.w0);
    if (cz.w1 != 0.f) red_add8(gl + (long long)cz.i1 * lv.C, dl, cz.w1);
  }
  }
}

// ---- fused density head --------------------------------------------------------------------------
// sigma = act(relu?(sum_c w_c * feature_c)): the lookup, the 1-wide linear layer (or plain channel sum)
// and the activation of the reference's density path (benchmarks/nerf/gridnerf/gridnerf.py:177-197,
// compute_densityfeature + feature2density) in one kernel; the [N, L*C] feature matrix is never written.
// The C/8 threads of a sample are adjacent lanes (C/8 must be a power of two <= 32).
struct DensityHead {
  const float* w;     // [L*C] weights of the 1-wide linear layer, or nullptr for a plain sum
  int inner_relu;     // relu between the linear layer and the activation
  int act;            // 0 relu, 1 softplus(x + shift)
  float shift;
};

template <typename T>
__device__ __forceinline__ void vm_features(const VMLevels& lv, int l, const float4& q, int b, int ch, F8& f, F8& pv8, F8& lv8,
                                            Corner2& cx, Corner2& cy, Corner2& cz) {
  const int H = lv.H[l], W = lv.W[l], Z = lv.Z[l];
  cx = taps(q.x, W); cy = taps(q.y, H); cz = taps(q.z, Z);
  const T* pl = reinterpret_cast<const T*>(lv.plane[l]) + ((long long)b * H * W) * lv.C + ch * 8;
  const T* ln = reinterpret_cast<const T*>(lv.line[l]) + ((long long)b * Z) * lv.C + ch * 8;
  F8 p00 = load8(pl + ((long long)cy.i0 * W + cx.i0) * lv.C), p01 = load8(pl + ((long long)cy.i0 * W + cx.i1) * lv.C);
  F8 p10 = load8(pl + ((long long)cy.i1 * W + cx.i0) * lv.C), p11 = load8(pl + ((long long)cy.i1 * W + cx.i1) * lv.C);
  F8 l0 = load8(ln + (long long)cz.i0 * lv.C), l1 = load8(ln + (long long)cz.i1 * lv.C);
  const float w00 = cy.w0 * cx.w0, w01 = cy.w0 * cx.w1, w10 = cy.w1 * cx.w0, w11 = cy.w1 * cx.w1;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    pv8.v[i] = w00 * p00.v[i] + w01 * p01.v[i] + w10 * p10.v[i] + w11 * p11.v[i];
    lv8.v[i] = cz.w0 * l0.v[i] + cz.w1 * l1.v[i];
    f.v[i] = pv8.v[i] * lv8.v[i];
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
vm_density_fwd_kernel(const float4* __restrict__ coords, const int* __restrict__ count_ptr, long long max_n, VMLevels lv,
                      DensityHead head, float* __restrict__ sigma, float* __restrict__ pre) {
  const int CH = lv.C >> 3;
  const long long n_valid = resolve_count(count_ptr, max_n);
  // grid-stride with a trip count that is uniform per block (the shuffles below need whole warps)
  for (long long base = (long long)blockIdx.x * blockDim.x; base < n_valid * CH; base += (long long)gridDim.x * blockDim.x) {
  const long long tid = base + threadIdx.x;
  const long long n = tid / CH;
  const int ch = (int)(tid - n * CH);
  const bool live = n < n_valid;
  float acc = 0.f;
  if (live) {
    const float4 q = __ldg(coords + n);
    const int b = (int)q.w;
    if (b >= 0 && b < lv.B) {
      for (int l = 0; l < lv.L; ++l) {
        F8 f, pv8, lv8;
        Corner2 cx, cy, cz;
        vm_features<T>(lv, l, q, b, ch, f, pv8, lv8, cx, cy, cz);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc += f.v[i] * (head.w ? __ldg(head.w + l * lv.C + ch * 8 + i) : 1.f);
      }
    }
  }
  for (int o = CH >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (live && ch == 0) {
    const float r = head.inner_relu ? fmaxf(acc, 0.f) : acc;
    const float x = r + head.shift;
    sigma[n] = head.act == 0 ? fmaxf(r, 0.f) : (x > 20.f ? x : log1pf(__expf(x)));
    pre[n] = acc;
  }
  }
}

// dsigma [N] -> plane / line gradient accumulators (as vm_encode_bwd) and dw [L*C] (block-reduced, one
// atomic per block and channel)
template <typename T>
__global__ void __launch_bounds__(256)
vm_density_bwd_kernel(const float4* __restrict__ coords, const int* __restrict__ count_ptr, long long max_n, VMLevels lv,
                      DensityHead head, const float* __restrict__ dsigma, const float* __restrict__ pre, float* __restrict__ dw) {
  extern __shared__ float dw_sh[];               // [L*C]
  const int CH = lv.C >> 3;
  const int n_w = lv.L * lv.C;
  for (int i = threadIdx.x; i < n_w; i += blockDim.x) dw_sh[i] = 0.f;
  __syncthreads();
  const long long n_valid = resolve_count(count_ptr, max_n);
  const int lane = threadIdx.x & 31;
  for (long long base = (long long)blockIdx.x * blockDim.x; base < n_valid * CH; base += (long long)gridDim.x * blockDim.x) {
  const long long tid = base + threadIdx.x;
  const long long n = tid / CH;
  const int ch = (int)(tid - n * CH);
  bool live = n < n_valid;
  float4 q = make_float4(0.f, 0.f, 0.f, -1.f);
  float dz = 0.f;
  if (live) {
    q = __ldg(coords + n);
    const int b = (int)q.w;
    live = b >= 0 && b < lv.B;
    if (live) {
      const float z = pre[n];
      const float r = head.inner_relu ? fmaxf(z, 0.f) : z;
      const float dact = head.act == 0 ? (r > 0.f ? 1.f : 0.f) : __fdividef(1.f, 1.f + __expf(-(r + head.shift)));
      dz = dsigma[n] * dact * ((head.inner_relu && z <= 0.f) ? 0.f : 1.f);
    }
  }
  for (int l = 0; l < lv.L; ++l) {
    F8 dwp;
#pragma unroll
    for (int i = 0; i < 8; ++i) dwp.v[i] = 0.f;
    if (live && dz != 0.f) {
      const int b = (int)q.w;
      F8 f, pv8, lv8;
      Corner2 cx, cy, cz;
      vm_features<T>(lv, l, q, b, ch, f, pv8, lv8, cx, cy, cz);
      const int H = lv.H[l], W = lv.W[l], Z = lv.Z[l];
      F8 dp, dl;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float g = dz * (head.w ? __ldg(head.w + l * lv.C + ch * 8 + i) : 1.f);
        dp.v[i] = g * lv8.v[i];
        dl.v[i] = g * pv8.v[i];
        dwp.v[i] = dz * f.v[i];
      }
      float* gp = lv.gplane[l] + ((long long)b * H * W) * lv.C + ch * 8;
      float* gl = lv.gline[l] + ((long long)b * Z) * lv.C + ch * 8;
      const float w00 = cy.w0 * cx.w0, w01 = cy.w0 * cx.w1, w10 = cy.w1 * cx.w0, w11 = cy.w1 * cx.w1;
      if (w00 != 0.f) red_add8(gp + ((long long)cy.i0 * W + cx.i0) * lv.C, dp, w00);
      if (w01 != 0.f) red_add8(gp + ((long long)cy.i0 * W + cx.i1) * lv.C, dp, w01);
      if (w10 != 0.f) red_add8(gp + ((long long)cy.i1 * W + cx.i0) * lv.C, dp, w10);
      if (w11 != 0.f) red_add8(gp + ((long long)cy.i1 * W + cx.i1) * lv.C, dp, w11);
      if (cz.w0 != 0.f) red_add8(gl + (long long)cz.i0 * lv.C, dl, cz.w0);
      if (cz.w1 != 0.f) red_add8(gl + (long long)cz.i1 * lv.C, dl, cz.w1);
    }
    if (head.w != nullptr && dw != nullptr) {
      // lanes with the same channel group are CH apart: fold them, then one shared-memory atomic per warp
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float v = dwp.v[i];
        for (int o = CH; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane < CH) atomicAdd(&dw_sh[l * lv.C + (lane % CH) * 8 + i], v);
      }
    }
  }
  }
  if (head.w != nullptr && dw != nullptr) {
    __syncthreads();
    for (int i = threadIdx.x; i < n_w; i += blockDim.x)
      if (dw_sh[i] != 0.f) atomicAdd(dw + i, dw_sh[i]);
  }
}

}  // namespace lmb

using namespace lmb;

// enough blocks to fill the GPU several times over, never more than the work needs
static int capped_grid(long long work_items, int threads) {
  const long long want = (work_items + threads - 1) / threads;
  const long long cap = 148LL * 64;
  return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

// param_dtype / io_dtype: 0 = fp32, 1 = bf16.
LMB_API int lmb_vm_encode_fwd(const float* coords, const int* count_ptr, long long max_n, const VMLevels* levels,
                              int param_dtype, void* out, int out_dtype, int out_stride, cudaStream_t stream) {
  if (max_n <= 0) return 0;
  if (levels->C % 8 != 0 || levels->L < 1 || levels->L > kMaxLevels) return (int)cudaErrorInvalidValue;
  const int CH = levels->C / 8;
  const int threads = 256;
  const int blocks = capped_grid(max_n * CH, threads);
  const float4* c4 = reinterpret_cast<const float4*>(coords);
#define LAUNCH(T, O) vm_encode_fwd_kernel<T, O><<<blocks, threads, 0, stream>>>(c4, count_ptr, max_n, *levels, (O*)out, out_stride > 0 ? out_stride : levels->L * levels->C)
  if (param_dtype == 0 && out_dtype == 0) LAUNCH(float, float);
  else if (param_dtype == 0 && out_dtype == 1) LAUNCH(float, __nv_bfloat16);
  else if (param_dtype == 1 && out_dtype == 0) LAUNCH(__nv_bfloat16, float);
  else LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_vm_encode_bwd(const float* coords, const int* count_ptr, long long max_n, const VMLevels* levels,
                              int param_dtype, const void* dout, int dout_dtype, int dout_stride, cudaStream_t stream) {
  if (max_n <= 0) return 0;
  if (levels->C % 8 != 0 || levels->L < 1 || levels->L > kMaxLevels) return (int)cudaErrorInvalidValue;
  const int CH = levels->C / 8;
  const int threads = 256;
  const int blocks = capped_grid(max_n * CH, threads);
  const float4* c4 = reinterpret_cast<const float4*>(coords);
#define LAUNCH(T, G) vm_encode_bwd_kernel<T, G><<<blocks, threads, 0, stream>>>(c4, count_ptr, max_n, *levels, (const G*)dout, dout_stride > 0 ? dout_stride : levels->L * levels->C)
  if (param_dtype == 0 && dout_dtype == 0) LAUNCH(float, float);
  else if (param_dtype == 0 && dout_dtype == 1) LAUNCH(float, __nv_bfloat16);
  else if (param_dtype == 1 && dout_dtype == 0) LAUNCH(__nv_bfloat16, float);
  else LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
  LMB_LAUNCH_CHECK();
  return 0;
}

static bool density_shape_ok(const VMLevels* lv) {
  const int CH = lv->C / 8;
  return lv->C % 8 == 0 && lv->L >= 1 && lv->L <= kMaxLevels && CH >= 1 && CH <= 32 && (CH & (CH - 1)) == 0;
}

// sigma, pre: fp32 [max_n]; w: fp32 [L*C] or null (plain channel sum); act: 0 relu, 1 softplus(x + shift)
LMB_API int lmb_vm_density_fwd(const float* coords, const int* count_ptr, long long max_n, const VMLevels* levels,
                               int param_dtype, const float* w, int inner_relu, int act, float shift, float* sigma, float* pre,
                               cudaStream_t stream) {
  if (max_n <= 0) return 0;
  if (!density_shape_ok(levels)) return (int)cudaErrorInvalidValue;
  const DensityHead head{w, inner_relu, act, shift};
  const int blocks = capped_grid(max_n * (levels->C / 8), 256);
  const float4* c4 = reinterpret_cast<const float4*>(coords);
  if (param_dtype == 0) vm_density_fwd_kernel<float><<<blocks, 256, 0, stream>>>(c4, count_ptr, max_n, *levels, head, sigma, pre);
  else vm_density_fwd_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(c4, count_ptr, max_n, *levels, head, sigma, pre);
  LMB_LAUNCH_CHECK();
  return 0;
}

// dw: fp32 [L*C] accumulator (may be null when w is null)
LMB_API int lmb_vm_density_bwd(const float* coords, const int* count_ptr, long long max_n, const VMLevels* levels,
                               int param_dtype, const float* w, int inner_relu, int act, float shift, const float* dsigma,
                               const float* pre, float* dw, cudaStream_t stream) {
  if (max_n <= 0) return 0;
  if (!density_shape_ok(levels)) return (int)cudaErrorInvalidValue;
  const DensityHead head{w, inner_relu, act, shift};
  const int blocks = capped_grid(max_n * (levels->C / 8), 256);
  const size_t smem = sizeof(float) * levels->L * levels->C;
  const float4* c4 = reinterpret_cast<const float4*>(coords);
  if (param_dtype == 0)
    vm_density_bwd_kernel<float><<<blocks, 256, smem, stream>>>(c4, count_ptr, max_n, *levels, head, dsigma, pre, dw);
  else
    vm_density_bwd_kernel<__nv_bfloat16><<<blocks, 256, smem, stream>>>(c4, count_ptr, max_n, *levels, head, dsigma, pre, dw);
  LMB_LAUNCH_CHECK();
  return 0;
}
