// Bilinear (align_corners) resize of channels-last grids [B, H, W, C] -> [B, H2, W2, C]: the grid upsampling step of
// the coarse-to-fine schedule (reference: F.interpolate on NCHW tensors, landmark/nerf_components/model_components/
// fields/encodings/tensor_vm_encoding.py:199-234).  Working directly on the channels-last layout avoids two full
// transposes of multi-GB planes; lines [B, Z, C] are the W = 1 case.
#include "common.cuh"

namespace lmb {

__global__ void __launch_bounds__(256)
resize_bilinear_nhwc_kernel(const float4* __restrict__ src, float4* __restrict__ dst, int B, int H, int W, int H2, int W2, int C4) {
  const long long total = (long long)B * H2 * W2 * C4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % C4);
    long long r = i / C4;
    const int x = (int)(r % W2); r /= W2;
    const int y = (int)(r % H2);
    const int b = (int)(r / H2);
    const float fy = H2 > 1 ? (float)y * (float)(H - 1) / (float)(H2 - 1) : 0.f;
    const float fx = W2 > 1 ? (float)x * (float)(W - 1) / (float)(W2 - 1) : 0.f;
    const int y0 = min((int)fy, H - 1), x0 = min((int)fx, W - 1);
    const int y1 = min(y0 + 1, H - 1), x1 = min(x0 + 1, W - 1);
    const float ty = fy - (float)y0, tx = fx - (float)x0;
    const float4* base = src + (long long)b * H * W * C4 + c;
    const float4 p00 = base[((long long)y0 * W + x0) * C4], p01 = base[((long long)y0 * W + x1) * C4];
    const float4 p10 = base[((long long)y1 * W + x0) * C4], p11 = base[((long long)y1 * W + x1) * C4];
    const float w00 = (1.f - ty) * (1.f - tx), w01 = (1.f - ty) * tx, w10 = ty * (1.f - tx), w11 = ty * tx;
    dst[i] = make_float4(w00 * p00.x + w01 * p01.x + w10 * p10.x + w11 * p11.x, w00 * p00.y + w01 * p01.y + w10 * p10.y + w11 * p11.y,
                         w00 * p00.z + w01 * p01.z + w10 * p10.z + w11 * p11.z, w00 * p00.w + w01 * p01.w + w10 * p10.w + w11 * p11.w);
  }
}

// ---- occupancy (alpha) mask rebuild ----------------------------------------------------------------------------
// alpha [X, Y, Z] (dense evaluation of the field) -> mask [Z, Y, X] = (max over the 3x3x3 neighbourhood of
// clamp(alpha, 0, 1) >= thre), plus the index bounding box of the occupied voxels (bbox = {min x, y, z, max x, y, z},
// initialised by the caller to {X, Y, Z, -1, -1, -1}).  Replaces the clamp / transpose / max_pool3d / compare / boolean
// gather / amin / amax sequence of benchmarks/nerf/gridnerf/gridnerf.py:380-413 with one pass and no dense coordinate
// tensor.
__global__ void __launch_bounds__(256)
alpha_pool_kernel(const float* __restrict__ alpha, int X, int Y, int Z, float thre, float* __restrict__ mask,
                  int* __restrict__ bbox) {
  const long long n = (long long)X * Y * Z;
  int lo[3] = {X, Y, Z}, hi[3] = {-1, -1, -1};
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    // threads walk the INPUT order (z fastest): the 27 reads of a warp are contiguous runs, only the one write is strided
    const int z = (int)(i % Z), y = (int)((i / Z) % Y), x = (int)(i / ((long long)Z * Y));
    float m = 0.f;
    for (int dx = -1; dx <= 1; ++dx) {
      const int xx = x + dx;
      if (xx < 0 || xx >= X) continue;
      for (int dy = -1; dy <= 1; ++dy) {
        const int yy = y + dy;
        if (yy < 0 || yy >= Y) continue;
        const float* row = alpha + ((long long)xx * Y + yy) * Z;
        for (int dz = -1; dz <= 1; ++dz) {
          const int zz = z + dz;
          if (zz < 0 || zz >= Z) continue;
          m = fmaxf(m, fminf(fmaxf(row[zz], 0.f), 1.f));
        }
      }
    }
    const bool on = m >= thre;
    mask[((long long)z * Y + y) * X + x] = on ? 1.f : 0.f;
    if (on) {
      lo[0] = min(lo[0], x); lo[1] = min(lo[1], y); lo[2] = min(lo[2], z);
      hi[0] = max(hi[0], x); hi[1] = max(hi[1], y); hi[2] = max(hi[2], z);
    }
  }
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    for (int o = 16; o > 0; o >>= 1) {
      lo[k] = min(lo[k], __shfl_xor_sync(0xffffffffu, lo[k], o));
      hi[k] = max(hi[k], __shfl_xor_sync(0xffffffffu, hi[k], o));
    }
    if ((threadIdx.x & 31) == 0 && hi[k] >= 0) { atomicMin(&bbox[k], lo[k]); atomicMax(&bbox[3 + k], hi[k]); }
  }
}

}  // namespace lmb

using namespace lmb;

LMB_API int lmb_resize_bilinear_nhwc(const float* src, float* dst, int B, int H, int W, int H2, int W2, int C, cudaStream_t stream) {
  if (C % 4 || B <= 0 || H <= 0 || W <= 0 || H2 <= 0 || W2 <= 0) return (int)cudaErrorInvalidValue;
  const long long total = (long long)B * H2 * W2 * (C / 4);
  const long long want = (total + 255) / 256;
  const int blocks = (int)(want < 148LL * 32 ? want : 148LL * 32);
  resize_bilinear_nhwc_kernel<<<blocks, 256, 0, stream>>>((const float4*)src, (float4*)dst, B, H, W, H2, W2, C / 4);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_alpha_pool(const float* alpha, int X, int Y, int Z, float thre, float* mask, int* bbox, cudaStream_t stream) {
  const long long n = (long long)X * Y * Z;
  if (n <= 0) return 0;
  const long long want = (n + 255) / 256;
  alpha_pool_kernel<<<(int)(want < 148 * 16 ? want : 148 * 16), 256, 0, stream>>>(alpha, X, Y, Z, thre, mask, bbox);
  LMB_LAUNCH_CHECK();
  return 0;
}
