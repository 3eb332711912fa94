// Definitions shared by the tcgen05 fused-MLP kernels (forward: fused_mlp.cu, training backward:
// fused_mlp_bwd.cu): network description, multi-source input descriptor, shared-memory tile helpers.
#pragma once
#include <cuda.h>
#include "common.cuh"
#include "tc05.cuh"

namespace lmb {

constexpr int kTileRows = 128;
constexpr int kMaxLayers = 5;
constexpr int kMaxK = 160;            // widest activation row kept in shared memory
constexpr int kSlotCols = 160;        // TMEM columns per slot (>= widest layer output)
constexpr int kActBytes = kTileRows * kMaxK * 2;

enum Act : int { ACT_NONE = 0, ACT_RELU = 1, ACT_SIGMOID = 2, ACT_TANH = 3, ACT_EXP = 4 };

struct MLPSpec {
  int n_layers;
  int K[kMaxLayers];        // padded input width of each layer (multiple of 16, <= kMaxK)
  int N[kMaxLayers];        // padded output width (multiple of 16, <= kSlotCols)
  int act[kMaxLayers];
  int w_off[kMaxLayers];    // byte offset of the packed [K/8][N][8] bf16 weights inside the blob
  int b_off[kMaxLayers];    // byte offset of N fp32 biases inside the blob (-1: no bias)
  int blob_bytes;           // multiple of 16
  int in_width;             // row width of the input tensor (multiple of 8)
  int out_dim;              // number of valid output columns of the last layer
  int pe_stage;             // 1: GridNeRF colour expansion between layer 0 and layer 1
  int dir_col;              // column of the input row that holds the view direction (pe_stage)
  int bias_in_gemm;         // bit l: layer l's bias is a column of its weights, multiplied by a ones column that the
                            // kernels write into the layer's input (or it is zero): the epilogue adds nothing
  int hidden_cols;          // plain backward kernel: widest real hidden width (0 = as padded); at most 64 lets its
                            // 128-column epilogues stop after the first 64 columns (the rest is zero padding)
};

// Input rows may be assembled from several tensors ("sources"), each contributing a contiguous range of
// 16-byte column chunks of the A tile.  A source can live in a peer GPU's memory: the tile is then
// pulled over NVLink by the (non-multicast) TMA load itself, which fuses an all-gather of column
// slices into the first GEMM of the network.
constexpr int kMaxSources = 4;
struct alignas(64) MLPInputs {
  CUtensorMap map[kMaxSources];
  int chunk_begin[kMaxSources + 1];
  int n_src;
  // Single local source, whole-row copies: map[0] moves 64-column pieces (128-byte rows, SWIZZLE_128B), map[1] a last
  // piece of at most 32 columns (64-byte rows, SWIZZLE_64B); 128 copy requests of 128 bytes per piece instead of 128
  // requests of 16 bytes per 8-column chunk.  n128 / n64: number of pieces of either kind (0: chunked copies above).
  int n128, n64;
  const __nv_bfloat16* x0;      // source 0 (the kernel reads the view direction of the colour stage from it)
};

__device__ __forceinline__ float apply_act(float x, int act) {
  switch (act) {
    case ACT_RELU: return fmaxf(x, 0.f);
    case ACT_SIGMOID: return 1.f / (1.f + __expf(-x));
    case ACT_TANH: return tanhf(x);
    case ACT_EXP: return __expf(x);
    default: return x;
  }
}

__device__ __forceinline__ void store_chunk(unsigned char* buf, int chunk, int row, const float* v) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(buf + ((size_t)chunk * kTileRows + row) * 16) = u;
}

// relu(v) rounded to bf16, eight values -> one 16-byte chunk: `cvt.rn.relu.bf16x2.f32` clamps and packs a pair at once
__device__ __forceinline__ void store_chunk_relu(unsigned char* buf, int chunk, int row, const float* v) {
  uint4 u;
  uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    asm("cvt.rn.relu.bf16x2.f32 %0, %1, %2;" : "=r"(w[i]) : "f"(v[2 * i + 1]), "f"(v[2 * i]));
  *reinterpret_cast<uint4*>(buf + ((size_t)chunk * kTileRows + row) * 16) = u;
}

__device__ __forceinline__ float load_elem(const unsigned char* buf, int col, int row) {
  const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(buf + ((size_t)(col >> 3) * kTileRows + row) * 16);
  return __bfloat162float(p[col & 7]);
}


// cuTensorMapEncodeTiled is a driver-API function; it is resolved through the runtime at first use instead of
// linking the driver library, so the kernel library loads (and its symbols can be checked) on a machine that has
// the CUDA toolkit but no driver.
typedef CUresult (*TensorMapEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                           const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                           CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline TensorMapEncodeTiledFn tensor_map_encoder() {
  static TensorMapEncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<TensorMapEncodeTiledFn>(p);
  }
  return fn;
}

// 3-D tensor map over a row-major bf16 [rows, width] matrix: (8 elements, width/8 chunks, rows), box
// = one 16-byte chunk of 128 rows, so a tile lands in shared memory in the chunked operand layout.
// Row-major [rows, width] bf16 as a 2-D tensor with a [box_cols x 128 rows] box written in a swizzled layout
// (box_cols * 2 bytes = the swizzle span: 64 columns for SWIZZLE_128B, 32 for SWIZZLE_64B).  Columns past `width`
// and rows past `rows` read as zeros.
inline int encode_swizzled_map(CUtensorMap* map, const void* x, int width, long long rows, int box_cols) {
  const cuuint64_t gdim[2] = {(cuuint64_t)width, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)width * 2};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)kTileRows};
  const cuuint32_t estride[2] = {1, 1};
  TensorMapEncodeTiledFn encode = tensor_map_encoder();
  if (encode == nullptr) return 19999;
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), gdim, gstride, box, estride,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 10000 + (int)r;
}

inline int encode_input_map(CUtensorMap* map, const void* x, int width, long long rows) {
  const cuuint64_t gdim[3] = {8, (cuuint64_t)(width / 8), (cuuint64_t)rows};
  const cuuint64_t gstride[2] = {16, (cuuint64_t)width * 2};
  const cuuint32_t box[3] = {8, 1, (cuuint32_t)kTileRows};
  const cuuint32_t estride[3] = {1, 1, 1};
  TensorMapEncodeTiledFn encode = tensor_map_encoder();
  if (encode == nullptr) return 19999;
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(x), gdim, gstride, box,
                                      estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 10000 + (int)r;
}

}  // namespace lmb
