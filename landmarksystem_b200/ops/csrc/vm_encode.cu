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

// Optional 16-column tail of every output row: the viewing direction of the row's ray (3 values) followed by 13 zeros,
// written by the row's first thread as two 16-byte stores.  The colour head reads the direction from there, so the
// row leaves this kernel complete and no separate pass has to patch three 2-byte values into every 320-byte row.
struct DirTail {
  const float* dirs;   // [rays, 3]; null: no tail
  const int* idx;      // row -> flat sample index (ray = idx / samples_per_ray); null: row n reads dirs[n]
  int samples_per_ray;
  int col;             // first tail column, a multiple of 8
};

template <typename T, typename OutT>
__global__ void __launch_bounds__(256)
vm_encode_fwd_kernel(const float4* __restrict__ coords, const int* __restrict__ count_ptr, long long max_n,
                     VMLevels lv, OutT* __restrict__ out, int out_stride, DirTail tail) {
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
  if (tail.dirs != nullptr && ch == 0) {
    const float* d = tail.dirs + (tail.idx != nullptr ? (long long)(tail.idx[n] / tail.samples_per_ray) : n) * 3;
    F8 a, z;
#pragma unroll
    for (int i = 0; i < 8; ++i) { a.v[i] = 0.f; z.v[i] = 0.f; }
    a.v[0] = d[0]; a.v[1] = d[1]; a.v[2] = d[2];
    store8(out + n * out_stride + tail.col, a);
    store8(out + n * out_stride + tail.col + 8, z);
  }
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

// ---- atomic-free (deterministic) backward ------------------------------------------------------------------
// Samples are sorted by the texel cell they fall into; one thread owns a whole run of equal cells, sums the run in
// registers in sorted (stable) order and adds the four corner sums to the gradient plane with plain loads and stores.
// Neighbouring cells share corners, so cells are 4-coloured by the parity of (x0, y0) and the colours run as separate
// launches: within a launch no two runs touch the same texel.  Lines are handled the same way with cells sorted by z0,
// two colours, and a warp per run (fixed lane assignment and shuffle tree).  The result is bit-reproducible; the
// default backward (16-byte reductions into L2) is faster and differs only in summation order.
constexpr unsigned long long kNoKey = ~0ull;

__global__ void __launch_bounds__(256)
vm_sort_keys_kernel(const float4* __restrict__ coords, const int* __restrict__ count_ptr, long long max_n, int B, int H, int W, int Z,
                    unsigned long long* __restrict__ pkeys, unsigned* __restrict__ pvals, unsigned long long* __restrict__ zkeys,
                    unsigned* __restrict__ zvals) {
  const long long n = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= max_n) return;
  const long long n_valid = resolve_count(count_ptr, max_n);
  unsigned long long pk = kNoKey, zk = kNoKey;
  if (n < n_valid) {
    const float4 q = __ldg(coords + n);
    const int b = (int)q.w;
    if (b >= 0 && b < B) {
      const float fx = (q.x + 1.f) * 0.5f * (float)(W - 1), fy = (q.y + 1.f) * 0.5f * (float)(H - 1);
      const float fz = (q.z + 1.f) * 0.5f * (float)(Z - 1);
      const int x0 = min(max((int)floorf(fx), -1), W - 1), y0 = min(max((int)floorf(fy), -1), H - 1);
      const int z0 = min(max((int)floorf(fz), -1), Z - 1);
      pk = ((unsigned long long)b * (H + 1) + (y0 + 1)) * (W + 1) + (x0 + 1);
      zk = (unsigned long long)b * (Z + 1) + (z0 + 1);
    }
  }
  pkeys[n] = pk; pvals[n] = (unsigned)n;
  zkeys[n] = zk; zvals[n] = (unsigned)n;
}

__device__ __forceinline__ void rmw_add8(float* p, const F8& a) {
  float4* q = reinterpret_cast<float4*>(p);
  float4 u = q[0], v = q[1];
  u.x += a.v[0]; u.y += a.v[1]; u.z += a.v[2]; u.w += a.v[3];
  v.x += a.v[4]; v.y += a.v[5]; v.z += a.v[6]; v.w += a.v[7];
  q[0] = u; q[1] = v;
}

template <typename T, typename GT>
__global__ void __launch_bounds__(256)
vm_bwd_sorted_plane_kernel(const float4* __restrict__ coords, VMLevels lv, int l, const GT* __restrict__ dout, int out_stride,
                           const unsigned long long* __restrict__ keys, const unsigned* __restrict__ vals, long long max_n,
                           int colour) {
  const int CH = lv.C >> 3;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long i = tid / CH;
  const int ch = (int)(tid - i * CH);
  if (i >= max_n) return;
  const unsigned long long key = keys[i];
  if (key == kNoKey || (i > 0 && keys[i - 1] == key)) return;          // not the head of a run
  const int H = lv.H[l], W = lv.W[l], Z = lv.Z[l];
  const int x0p = (int)(key % (unsigned long long)(W + 1));
  const unsigned long long t = key / (unsigned long long)(W + 1);
  const int y0p = (int)(t % (unsigned long long)(H + 1));
  const int b = (int)(t / (unsigned long long)(H + 1));
  if (((x0p & 1) | ((y0p & 1) << 1)) != colour) return;
  F8 a00, a01, a10, a11;
#pragma unroll
  for (int k = 0; k < 8; ++k) a00.v[k] = a01.v[k] = a10.v[k] = a11.v[k] = 0.f;
  const T* ln = reinterpret_cast<const T*>(lv.line[l]) + ((long long)b * Z) * lv.C + ch * 8;
  for (long long j = i; j < max_n && keys[j] == key; ++j) {
    const long long n = vals[j];
    const float4 q = __ldg(coords + n);
    const Corner2 cx = taps(q.x, W), cy = taps(q.y, H), cz = taps(q.z, Z);
    const F8 l0 = load8(ln + (long long)cz.i0 * lv.C), l1 = load8(ln + (long long)cz.i1 * lv.C);
    const F8 g = load8(dout + n * out_stride + l * lv.C + ch * 8);
    const float w00 = cy.w0 * cx.w0, w01 = cy.w0 * cx.w1, w10 = cy.w1 * cx.w0, w11 = cy.w1 * cx.w1;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float dp = g.v[k] * (cz.w0 * l0.v[k] + cz.w1 * l1.v[k]);
      a00.v[k] += dp * w00; a01.v[k] += dp * w01; a10.v[k] += dp * w10; a11.v[k] += dp * w11;
    }
  }
  const int x0 = x0p - 1, y0 = y0p - 1;
  float* gp = lv.gplane[l] + ((long long)b * H * W) * lv.C + ch * 8;
  const bool xa = x0 >= 0, xb = x0 + 1 < W, ya = y0 >= 0, yb = y0 + 1 < H;
  if (ya && xa) rmw_add8(gp + ((long long)y0 * W + x0) * lv.C, a00);
  if (ya && xb) rmw_add8(gp + ((long long)y0 * W + x0 + 1) * lv.C, a01);
  if (yb && xa) rmw_add8(gp + ((long long)(y0 + 1) * W + x0) * lv.C, a10);
  if (yb && xb) rmw_add8(gp + ((long long)(y0 + 1) * W + x0 + 1) * lv.C, a11);
}

__device__ __forceinline__ long long lower_bound_u64(const unsigned long long* a, long long n, unsigned long long v) {
  long long lo = 0, hi = n;
  while (lo < hi) {
    const long long mid = (lo + hi) >> 1;
    if (a[mid] < v) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// one warp per (z cell, channel group)
template <typename T, typename GT>
__global__ void __launch_bounds__(256)
vm_bwd_sorted_line_kernel(const float4* __restrict__ coords, VMLevels lv, int l, const GT* __restrict__ dout, int out_stride,
                          const unsigned long long* __restrict__ keys, const unsigned* __restrict__ vals, long long max_n,
                          int colour) {
  const int CH = lv.C >> 3;
  const int H = lv.H[l], W = lv.W[l], Z = lv.Z[l];
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long cell = warp / CH;
  const int ch = (int)(warp - cell * CH);
  if (cell >= (long long)lv.B * (Z + 1)) return;
  const int z0p = (int)(cell % (Z + 1));
  if ((z0p & 1) != colour) return;
  const int b = (int)(cell / (Z + 1));
  const long long start = lower_bound_u64(keys, max_n, (unsigned long long)cell);
  const long long end = lower_bound_u64(keys, max_n, (unsigned long long)cell + 1);
  F8 a0, a1;
#pragma unroll
  for (int k = 0; k < 8; ++k) a0.v[k] = a1.v[k] = 0.f;
  const T* pl = reinterpret_cast<const T*>(lv.plane[l]) + ((long long)b * H * W) * lv.C + ch * 8;
  for (long long j = start + lane; j < end; j += 32) {
    const long long n = vals[j];
    const float4 q = __ldg(coords + n);
    const Corner2 cx = taps(q.x, W), cy = taps(q.y, H), cz = taps(q.z, Z);
    const F8 p00 = load8(pl + ((long long)cy.i0 * W + cx.i0) * lv.C), p01 = load8(pl + ((long long)cy.i0 * W + cx.i1) * lv.C);
    const F8 p10 = load8(pl + ((long long)cy.i1 * W + cx.i0) * lv.C), p11 = load8(pl + ((long long)cy.i1 * W + cx.i1) * lv.C);
    const F8 g = load8(dout + n * out_stride + l * lv.C + ch * 8);
    const float w00 = cy.w0 * cx.w0, w01 = cy.w0 * cx.w1, w10 = cy.w1 * cx.w0, w11 = cy.w1 * cx.w1;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float dl = g.v[k] * (w00 * p00.v[k] + w01 * p01.v[k] + w10 * p10.v[k] + w11 * p11.v[k]);
      a0.v[k] += dl * cz.w0; a1.v[k] += dl * cz.w1;
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k)
    for (int o = 16; o > 0; o >>= 1) {
      a0.v[k] += __shfl_xor_sync(0xffffffffu, a0.v[k], o);
      a1.v[k] += __shfl_xor_sync(0xffffffffu, a1.v[k], o);
    }
  if (lane != 0 || start == end) return;
  const int z0 = z0p - 1;
  float* gl = lv.gline[l] + ((long long)b * Z) * lv.C + ch * 8;
  if (z0 >= 0) rmw_add8(gl + (long long)z0 * lv.C, a0);
  if (z0 + 1 < Z) rmw_add8(gl + (long long)(z0 + 1) * lv.C, a1);
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

// Spatial-block model parallelism: the rows of an owner's batch came from other GPUs (all-to-all dispatch); row n
// belongs to rank route_src[n], which expects its density at slot route_slot[n] of its landing buffer dest[src].
// With a route the density kernel stores sigma there itself (a peer store over NVLink) - the "combine" half of the
// exchange costs no kernel of its own.
struct DensityRoute {
  const int* src;     // nullptr: no route
  const int* slot;
  float* dest[8];
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
                      DensityHead head, float* __restrict__ sigma, float* __restrict__ pre, DensityRoute route) {
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
    const float sg = head.act == 0 ? fmaxf(r, 0.f) : (x > 20.f ? x : log1pf(__expf(x)));
    sigma[n] = sg;
    pre[n] = acc;
    if (route.src != nullptr) route.dest[route.src[n]][route.slot[n]] = sg;
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
// tail_dirs (may be null): see DirTail; tail_col must be a multiple of 8 with tail_col + 16 <= the row stride.
LMB_API int lmb_vm_encode_fwd(const float* coords, const int* count_ptr, long long max_n, const VMLevels* levels,
                              int param_dtype, void* out, int out_dtype, int out_stride, const float* tail_dirs,
                              const int* tail_idx, int tail_samples_per_ray, int tail_col, cudaStream_t stream) {
  if (max_n <= 0) return 0;
  if (levels->C % 8 != 0 || levels->L < 1 || levels->L > kMaxLevels) return (int)cudaErrorInvalidValue;
  const int CH = levels->C / 8;
  const int threads = 256;
  const int blocks = capped_grid(max_n * CH, threads);
  const float4* c4 = reinterpret_cast<const float4*>(coords);
  const int stride = out_stride > 0 ? out_stride : levels->L * levels->C;
  const DirTail tail{tail_dirs, tail_idx, tail_samples_per_ray > 0 ? tail_samples_per_ray : 1, tail_col};
  if (tail_dirs != nullptr && (tail_col % 8 != 0 || tail_col < levels->L * levels->C || tail_col + 16 > stride))
    return (int)cudaErrorInvalidValue;
#define LAUNCH(T, O) vm_encode_fwd_kernel<T, O><<<blocks, threads, 0, stream>>>(c4, count_ptr, max_n, *levels, (O*)out, stride, tail)
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
// route_src / route_slot / dest_table (all null, or int [max_n] x 2 and `world` landing-buffer addresses): see DensityRoute
LMB_API int lmb_vm_density_fwd(const float* coords, const int* count_ptr, long long max_n, const VMLevels* levels,
                               int param_dtype, const float* w, int inner_relu, int act, float shift, float* sigma, float* pre,
                               const int* route_src, const int* route_slot, const long long* dest_table, int world,
                               cudaStream_t stream) {
  if (max_n <= 0) return 0;
  if (!density_shape_ok(levels) || (route_src != nullptr && (dest_table == nullptr || world > 8))) return (int)cudaErrorInvalidValue;
  const DensityHead head{w, inner_relu, act, shift};
  DensityRoute route;
  route.src = route_src; route.slot = route_slot;
  for (int i = 0; i < 8; ++i) route.dest[i] = (route_src != nullptr && i < world) ? (float*)dest_table[i] : nullptr;
  const int blocks = capped_grid(max_n * (levels->C / 8), 256);
  const float4* c4 = reinterpret_cast<const float4*>(coords);
  if (param_dtype == 0) vm_density_fwd_kernel<float><<<blocks, 256, 0, stream>>>(c4, count_ptr, max_n, *levels, head, sigma, pre, route);
  else vm_density_fwd_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(c4, count_ptr, max_n, *levels, head, sigma, pre, route);
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

extern "C" int lmb_radix_sort_pairs(uint64_t* keys, uint32_t* vals, const int* count_ptr, long long max_n, int begin_bit, int end_bit,
                                    void* scratch, cudaStream_t stream);

static int bits_for(unsigned long long n_keys) {      // enough bits that the all-ones "no key" sorts after every real key
  int bits = 1;
  while ((1ull << bits) <= n_keys) ++bits;
  return bits;
}

// Deterministic backward.  pkeys / zkeys: uint64 [max_n]; pvals / zvals: uint32 [max_n]; sort_scratch: lmb_radix_sort_scratch_bytes(max_n).
LMB_API int lmb_vm_encode_bwd_sorted(const float* coords, const int* count_ptr, long long max_n, const VMLevels* levels,
                                     int param_dtype, const void* dout, int dout_dtype, int dout_stride, uint64_t* pkeys,
                                     uint32_t* pvals, uint64_t* zkeys, uint32_t* zvals, void* sort_scratch, cudaStream_t stream) {
  if (max_n <= 0) return 0;
  if (levels->C % 8 != 0 || levels->L < 1 || levels->L > kMaxLevels) return (int)cudaErrorInvalidValue;
  const int CH = levels->C / 8;
  const float4* c4 = reinterpret_cast<const float4*>(coords);
  const int stride = dout_stride > 0 ? dout_stride : levels->L * levels->C;
  for (int l = 0; l < levels->L; ++l) {
    const int H = levels->H[l], W = levels->W[l], Z = levels->Z[l], B = levels->B;
    vm_sort_keys_kernel<<<ceil_div(max_n, 256), 256, 0, stream>>>(c4, count_ptr, max_n, B, H, W, Z, (unsigned long long*)pkeys, pvals,
                                                                 (unsigned long long*)zkeys, zvals);
    LMB_LAUNCH_CHECK();
    int rc = lmb_radix_sort_pairs(pkeys, pvals, nullptr, max_n, 0, bits_for((unsigned long long)B * (H + 1) * (W + 1)), sort_scratch, stream);
    if (rc) return rc;
    rc = lmb_radix_sort_pairs(zkeys, zvals, nullptr, max_n, 0, bits_for((unsigned long long)B * (Z + 1)), sort_scratch, stream);
    if (rc) return rc;
    const int pblocks = ceil_div(max_n * CH, 256);
    const int lblocks = ceil_div((long long)B * (Z + 1) * CH * 32, 256);
#define LAUNCH(T, G)                                                                                                              \
    for (int colour = 0; colour < 4; ++colour)                                                                                    \
      vm_bwd_sorted_plane_kernel<T, G><<<pblocks, 256, 0, stream>>>(c4, *levels, l, (const G*)dout, stride,                       \
                                                                   (const unsigned long long*)pkeys, pvals, max_n, colour);      \
    for (int colour = 0; colour < 2; ++colour)                                                                                    \
      vm_bwd_sorted_line_kernel<T, G><<<lblocks, 256, 0, stream>>>(c4, *levels, l, (const G*)dout, stride,                        \
                                                                  (const unsigned long long*)zkeys, zvals, max_n, colour);
    if (param_dtype == 0 && dout_dtype == 0) { LAUNCH(float, float) }
    else if (param_dtype == 0 && dout_dtype == 1) { LAUNCH(float, __nv_bfloat16) }
    else if (param_dtype == 1 && dout_dtype == 0) { LAUNCH(__nv_bfloat16, float) }
    else { LAUNCH(__nv_bfloat16, __nv_bfloat16) }
#undef LAUNCH
    LMB_LAUNCH_CHECK();
  }
  return 0;
}
