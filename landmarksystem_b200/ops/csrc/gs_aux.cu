// Small fused helpers of the anchor-based Gaussian models.
//
// octree_lod_mask: per-anchor level-of-detail selection of Octree-GS in one pass (reference:
// landmark/nerf_components/model_components/fields/encodings/octreegs_encoding.py:238-294, a chain of
// ~12 elementwise torch kernels): distance from the voxel centre to the camera, predicted level
//   log2(standard_dist / (dist * resolution_scale)) / log2(fork) + extra_level,
// mapped to an integer level (floor / round / ceil / progressive) and compared with the anchor's level.
#include "common.cuh"

namespace lmb {

// mode: 0 floor, 1 round, 2 ceil, 3 progressive
__global__ void __launch_bounds__(256)
octree_lod_mask_kernel(int n, const float* __restrict__ anchor, const float* __restrict__ level,
                       const float* __restrict__ extra_level, float cx, float cy, float cz, float half_voxel, float fork,
                       float standard_dist, float resolution_scale, int max_level, int mode,
                       unsigned char* __restrict__ mask, float* __restrict__ prog_ratio,
                       unsigned char* __restrict__ transition) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float lv = level[i];
  const float off = half_voxel / powf(fork, lv);
  const float dx = anchor[3 * i] + off - cx, dy = anchor[3 * i + 1] + off - cy, dz = anchor[3 * i + 2] + off - cz;
  const float dist = sqrtf(dx * dx + dy * dy + dz * dz) * resolution_scale;
  float pred = log2f(standard_dist / dist) / log2f(fork) + extra_level[i];
  int il;
  if (mode == 3) {
    pred = fminf(fmaxf(pred + 1.f, 0.9999f), (float)max_level + 0.9999f);
    il = (int)floorf(pred);
    if (prog_ratio) prog_ratio[i] = pred - floorf(pred);
    if (transition) transition[i] = ((int)lv == il);
  } else {
    const float r = mode == 0 ? floorf(pred) : (mode == 1 ? rintf(pred) : ceilf(pred));
    il = min(max((int)r, 0), max_level);
  }
  mask[i] = (int)lv <= il;
}

// ---- Scaffold-GS anchor decode: everything after the three MLP heads -------------------------------------------
// candidate i = (anchor a, offset j): kept when its opacity is positive; kept candidates are written densely, in
// candidate order, as Gaussians: xyz = anchor + offset * scaling[:3], scale = scaling[3:] * sigmoid(sr[:3]),
// rot = normalize(sr[3:7]).  Replaces the mask / boolean-index / repeat_interleave / gather chain of
// landmark/nerf_components/model_components/fields/decoders/anchor_decoder.py:205-242 at render time.
__global__ void __launch_bounds__(256)
anchor_flag_kernel(const float* __restrict__ opacity, long long n, unsigned* __restrict__ flags) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) flags[i] = opacity[i] > 0.f ? 1u : 0u;
}

__global__ void __launch_bounds__(256)
anchor_epilogue_kernel(const float* __restrict__ anchor, const float* __restrict__ offsets, const float* __restrict__ scaling,
                       const float* __restrict__ opacity, const float* __restrict__ color, const float* __restrict__ scale_rot,
                       long long n, int k, const unsigned* __restrict__ flags, const unsigned* __restrict__ pos,
                       float* __restrict__ xyz_o, float* __restrict__ color_o, float* __restrict__ opacity_o,
                       float* __restrict__ scaling_o, float* __restrict__ rot_o, int* __restrict__ count) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (i == n - 1) *count = (int)(pos[i] + flags[i]);
  if (!flags[i]) return;
  const long long a = i / k, o = pos[i];
  const float* sc = scaling + a * 6;
  const float* sr = scale_rot + i * 7;
#pragma unroll
  for (int c = 0; c < 3; ++c) {
    xyz_o[o * 3 + c] = anchor[a * 3 + c] + offsets[i * 3 + c] * sc[c];
    color_o[o * 3 + c] = color[i * 3 + c];
    scaling_o[o * 3 + c] = sc[3 + c] * (1.f / (1.f + __expf(-sr[c])));
  }
  const float q0 = sr[3], q1 = sr[4], q2 = sr[5], q3 = sr[6];
  const float inv = 1.f / fmaxf(sqrtf(q0 * q0 + q1 * q1 + q2 * q2 + q3 * q3), 1e-12f);
  rot_o[o * 4 + 0] = q0 * inv; rot_o[o * 4 + 1] = q1 * inv; rot_o[o * 4 + 2] = q2 * inv; rot_o[o * 4 + 3] = q3 * inv;
  opacity_o[o] = opacity[i];
}

// ---- anchor growing helper: per-segment maximum --------------------------------------------------------------
// out[index[i], c] = max(out[index[i], c], values[i, c]); the reference uses torch_scatter.scatter_max in 4096-row
// chunks (landmark/nerf_components/model_components/fields/encodings/scaffoldgs_encoding.py:571).  Float maximum as
// an integer atomic: non-negative floats order like signed ints, negative floats like reversed unsigned ints.
__device__ __forceinline__ void atomic_max_float(float* addr, float v) {
  if (v >= 0.f) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v + 0.f));      // -0 becomes +0
  else atomicMin(reinterpret_cast<unsigned*>(addr), __float_as_uint(v));
}

__global__ void __launch_bounds__(256)
segment_amax_kernel(const float* __restrict__ values, const long long* __restrict__ index, long long n, int C, long long n_seg,
                    float* __restrict__ out) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n * C) return;
  const long long i = e / C, s = index[i];
  if (s < 0 || s >= n_seg) return;
  atomic_max_float(out + s * C + (e - i * C), values[e]);
}

}  // namespace lmb

using namespace lmb;

LMB_API int lmb_octree_lod_mask(int n, const float* anchor, const float* level, const float* extra_level, float cx, float cy,
                                float cz, float half_voxel, float fork, float standard_dist, float resolution_scale,
                                int max_level, int mode, unsigned char* mask, float* prog_ratio, unsigned char* transition,
                                cudaStream_t stream) {
  if (n <= 0) return 0;
  octree_lod_mask_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(n, anchor, level, extra_level, cx, cy, cz, half_voxel, fork,
                                                              standard_dist, resolution_scale, max_level, mode, mask,
                                                              prog_ratio, transition);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_exclusive_scan_u32(const uint32_t* in, uint32_t* out, long long n, void* scratch, cudaStream_t stream);

// n = anchors * k candidates.  flags, pos: uint32 [n] work arrays; scan_scratch: lmb_scan_scratch_bytes(n) bytes.
// Outputs have capacity n rows; *count = rows written.
LMB_API int lmb_anchor_epilogue(const float* anchor, const float* offsets, const float* scaling, const float* opacity,
                                const float* color, const float* scale_rot, long long n, int k, unsigned* flags, unsigned* pos,
                                void* scan_scratch, float* xyz_o, float* color_o, float* opacity_o, float* scaling_o, float* rot_o,
                                int* count, cudaStream_t stream) {
  if (n <= 0) return (int)cudaMemsetAsync(count, 0, sizeof(int), stream);
  anchor_flag_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(opacity, n, flags);
  LMB_LAUNCH_CHECK();
  const int rc = lmb_exclusive_scan_u32(flags, pos, n, scan_scratch, stream);
  if (rc) return rc;
  anchor_epilogue_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(anchor, offsets, scaling, opacity, color, scale_rot, n, k, flags, pos,
                                                              xyz_o, color_o, opacity_o, scaling_o, rot_o, count);
  LMB_LAUNCH_CHECK();
  return 0;
}

// values [n, C] fp32, index [n] int64 in [0, n_seg), out [n_seg, C] pre-filled by the caller (-inf for a plain maximum)
LMB_API int lmb_segment_amax(const float* values, const long long* index, long long n, int C, long long n_seg, float* out,
                             cudaStream_t stream) {
  if (n <= 0 || C <= 0) return 0;
  segment_amax_kernel<<<ceil_div(n * C, 256), 256, 0, stream>>>(values, index, n, C, n_seg, out);
  LMB_LAUNCH_CHECK();
  return 0;
}
