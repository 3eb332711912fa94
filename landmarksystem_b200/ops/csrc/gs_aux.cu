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
