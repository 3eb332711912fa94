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
