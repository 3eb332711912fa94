// Mean squared distance to the 3 nearest neighbours of every point (initial Gaussian scales).
//
// Counterpart of simple_knn's distCUDA2 (call site landmark/nerf_components/model_components/fields/
// encodings/gaussian_encoding.py:124-136; the submodule source is absent from the reference tree).
// Points are binned into a uniform hash grid (cell size from the mean point spacing); each point
// searches rings of cells around its own cell until the ring distance exceeds its current 3rd-best
// distance.  Cell lists come from one sort of (cell id, point id) pairs with the library's radix sort.
#include "common.cuh"

namespace lmb {

struct KnnGrid {
  float3 lo;
  float inv_cell;
  int3 dims;
};

__device__ __forceinline__ int3 cell_of(const KnnGrid& g, float3 p) {
  return make_int3(min(max((int)((p.x - g.lo.x) * g.inv_cell), 0), g.dims.x - 1),
                   min(max((int)((p.y - g.lo.y) * g.inv_cell), 0), g.dims.y - 1),
                   min(max((int)((p.z - g.lo.z) * g.inv_cell), 0), g.dims.z - 1));
}

__global__ void knn_keys_kernel(int n, const float* __restrict__ pts, KnnGrid g, uint64_t* keys, uint32_t* vals) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int3 c = cell_of(g, make_float3(pts[3 * i], pts[3 * i + 1], pts[3 * i + 2]));
  keys[i] = (uint64_t)((long long)(c.z * g.dims.y + c.y) * g.dims.x + c.x);
  vals[i] = i;
}

__global__ void knn_cell_ranges_kernel(int n, const uint64_t* __restrict__ keys, uint32_t* __restrict__ cell_start,
                                       uint32_t* __restrict__ cell_end) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint64_t k = keys[i];
  if (i == 0 || keys[i - 1] != k) cell_start[k] = i;
  if (i == n - 1 || keys[i + 1] != k) cell_end[k] = i + 1;
}

__global__ void __launch_bounds__(128)
knn_query_kernel(int n, const float* __restrict__ pts, KnnGrid g, const uint32_t* __restrict__ order,
                 const uint32_t* __restrict__ cell_start, const uint32_t* __restrict__ cell_end, float* __restrict__ out) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;     // walk points in cell order for locality
  if (s >= n) return;
  const int i = order[s];
  const float3 p = make_float3(pts[3 * i], pts[3 * i + 1], pts[3 * i + 2]);
  const int3 c = cell_of(g, p);
  float best[3] = {3.4e38f, 3.4e38f, 3.4e38f};
  const float cell = 1.f / g.inv_cell;
  const int max_ring = max(g.dims.x, max(g.dims.y, g.dims.z));
  for (int ring = 0; ring <= max_ring; ++ring) {
    if (ring > 0) {
      const float reach = (ring - 1) * cell;   // closest possible distance of a point in this ring
      if (reach * reach > best[2]) break;
    }
    for (int dz = -ring; dz <= ring; ++dz) {
      const int z = c.z + dz;
      if (z < 0 || z >= g.dims.z) continue;
      for (int dy = -ring; dy <= ring; ++dy) {
        const int y = c.y + dy;
        if (y < 0 || y >= g.dims.y) continue;
        const bool shell_yz = (abs(dz) == ring) || (abs(dy) == ring);
        for (int dx = -ring; dx <= ring; dx += (shell_yz ? 1 : max(2 * ring, 1))) {
          const int x = c.x + dx;
          if (x < 0 || x >= g.dims.x) continue;
          const long long cid = (long long)(z * g.dims.y + y) * g.dims.x + x;
          for (uint32_t k = cell_start[cid]; k < cell_end[cid]; ++k) {
            const int j = order[k];
            if (j == i) continue;
            const float ddx = pts[3 * j] - p.x, ddy = pts[3 * j + 1] - p.y, ddz = pts[3 * j + 2] - p.z;
            const float d2 = ddx * ddx + ddy * ddy + ddz * ddz;
            if (d2 < best[2]) {
              if (d2 < best[0]) { best[2] = best[1]; best[1] = best[0]; best[0] = d2; }
              else if (d2 < best[1]) { best[2] = best[1]; best[1] = d2; }
              else best[2] = d2;
            }
          }
        }
      }
    }
  }
  float sum = 0.f; int cnt = 0;
#pragma unroll
  for (int k = 0; k < 3; ++k) if (best[k] < 3.0e38f) { sum += best[k]; ++cnt; }
  out[i] = cnt ? sum / 3.f : 0.f;
}

}  // namespace lmb

using namespace lmb;
extern "C" int lmb_radix_sort_pairs(uint64_t*, uint32_t*, const int*, long long, int, int, void*, cudaStream_t);

// keys/vals: n entries each; cell_start/cell_end: n_cells entries (zero-filled here); sort_ws: radix-sort scratch.
LMB_API int lmb_knn_mean_dist2(int n, const float* pts, float lo_x, float lo_y, float lo_z, float cell, int dx, int dy,
                               int dz, uint64_t* keys, uint32_t* vals, uint32_t* cell_start, uint32_t* cell_end,
                               void* sort_ws, float* out, cudaStream_t stream) {
  if (n <= 0) return 0;
  KnnGrid g;
  g.lo = make_float3(lo_x, lo_y, lo_z);
  g.inv_cell = 1.f / cell;
  g.dims = make_int3(dx, dy, dz);
  const long long n_cells = (long long)dx * dy * dz;
  LMB_CUDA_TRY(cudaMemsetAsync(cell_start, 0, n_cells * 4, stream));
  LMB_CUDA_TRY(cudaMemsetAsync(cell_end, 0, n_cells * 4, stream));
  knn_keys_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(n, pts, g, keys, vals);
  LMB_LAUNCH_CHECK();
  int bits = 1;
  while ((1LL << bits) < n_cells) ++bits;
  int rc = lmb_radix_sort_pairs(keys, vals, nullptr, n, 0, bits, sort_ws, stream);
  if (rc) return rc;
  knn_cell_ranges_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(n, keys, cell_start, cell_end);
  LMB_LAUNCH_CHECK();
  knn_query_kernel<<<ceil_div(n, 128), 128, 0, stream>>>(n, pts, g, vals, cell_start, cell_end, out);
  LMB_LAUNCH_CHECK();
  return 0;
}
