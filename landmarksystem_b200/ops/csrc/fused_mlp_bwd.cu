// Training backward of the GridNeRF colour head as ONE tcgen05 kernel: recompute + data gradients +
// weight gradients, with every intermediate kept on chip.
//
// Network (benchmarks/nerf/gridnerf/gridnerf.py:137-174 of the reference, nn.Sequential in
// landmark/nerf_components/model_components/fields/mlp_decoder.py:70-109):
//   f  = W0 x0                      (K0 <= 144 appearance features -> 27, no bias)
//   x1 = [f, d, sin/cos(f 2^k), sin/cos(d 2^k)]   (150 wide, k = 0, 1)
//   h1 = relu(W1 x1 + b1), h2 = relu(W2 h1 + b2), rgb = sigmoid(W3 h2 + b3)      (128, 128, 3)
// The reference runs this backward as ~20 cuBLAS GEMMs and elementwise kernels that stream every
// activation through HBM.  Here one persistent CTA per SM walks 128-row tiles; per tile it
//   1. re-runs the forward (4 MMA groups) keeping x1, h1, h2 in shared memory as bf16,
//   2. forms dz3 = dL/drgb * rgb (1 - rgb) in registers,
//   3. runs the data-gradient GEMMs dh = dz W with the forward weight blob read as an MN-major
//      (transposed) B operand - no second copy of the weights,
//   4. runs the weight-gradient GEMMs dW += dz^T h with BOTH operands read MN-major from the same
//      activation tiles (reduction over the tile's 128 rows), accumulating ACROSS TILES in tensor
//      memory; bias gradients ride along as a column of ones appended to x1 / h1,
//   5. back-propagates the sin/cos expansion in registers and writes dL/dx0 (bf16) for the grid kernel.
// Weight gradients leave the SM once per CTA (vector reductions into a small fp32 buffer).
//
// Tensor-memory map (512 columns): [0,128) working accumulator, [128,288) dW1 (out x 160),
// [288,432) dW2 (out x 128 + ones chunk), [432,448) dW3^T (in x 16), [448,512) dW0^T (in x 32, twice:
// input columns 0..127 and 16..143).  Shared memory: weights | A (x0 -> x1) | H1 (h1 -> x0 again) |
// HZ (h2 -> dz2 -> dz1, in place) | S (dz3, later df).
#include "fused_mlp.cuh"

namespace lmb {

constexpr int kBwdThreads = 128;
constexpr uint32_t kChunk = kTileRows * 16;           // bytes of one 8-column chunk of a tile
constexpr uint32_t kColWork = 0, kColDW1 = 128, kColDW2 = 288, kColDW3T = 432, kColDW0T = 448;
constexpr int kBufA = 20 * kChunk, kBufH1 = 18 * kChunk, kBufHZ = 16 * kChunk, kBufS = 4 * kChunk;

// layout (floats) of the gradient buffer the kernel reduces into
constexpr int kG_DW1 = 0;                       // [128][160]  (column 150 = db1)
constexpr int kG_DW2 = kG_DW1 + 128 * 160;      // [128][144]  (column 128 = db2)
constexpr int kG_DW3T = kG_DW2 + 128 * 144;     // [128][16]   (input-major)
constexpr int kG_DW0T = kG_DW3T + 128 * 16;     // [144][32]   (input-major)
constexpr int kG_DB3 = kG_DW0T + 144 * 32;      // [16]
constexpr int kG_TOTAL = kG_DB3 + 16;

// forward GEMM: D[128 x N] = A[128 x K] (K-major tile) * W^T (blob [K/8][N][8], K-major)
__device__ __forceinline__ void issue_fwd(uint32_t d, uint32_t a_addr, uint32_t w_addr, int K, int N) {
  const uint32_t idesc = tc05::idesc_bf16(N, false, false);
  for (int k = 0; k < K; k += 16) {
    const uint64_t da = tc05::smem_desc(a_addr + (uint32_t)(k >> 3) * kChunk, kChunk, 128);
    const uint64_t db = tc05::smem_desc(w_addr + (uint32_t)(k >> 3) * (uint32_t)(N * 16), (uint32_t)(N * 16), 128);
    tc05::mma_ss(d, da, db, idesc, k > 0);
  }
}
// data gradient: D[128 x ncols] = dZ[128 x n_out] (K-major tile) * W[n_out x k_in]; the forward blob
// [k_in/8][n_out][8] is an MN-major B operand: 8 k_in contiguous, n_out 16 bytes apart, k_in chunks
// n_out*16 bytes apart.  Output columns are k_in = 8*c0 .. 8*c0 + ncols.
__device__ __forceinline__ void issue_dgrad(uint32_t d, uint32_t a_addr, uint32_t w_addr, int n_out, int c0, int ncols) {
  const uint32_t idesc = tc05::idesc_bf16(ncols, false, true);
  const uint32_t w0 = w_addr + (uint32_t)c0 * (uint32_t)(n_out * 16);
  for (int k = 0; k < n_out; k += 16) {
    const uint64_t da = tc05::smem_desc(a_addr + (uint32_t)(k >> 3) * kChunk, kChunk, 128);
    const uint64_t db = tc05::smem_desc(w0 + (uint32_t)(k >> 3) * 128u, 128, (uint32_t)(n_out * 16));
    tc05::mma_ss(d, da, db, idesc, k > 0);
  }
}
// weight gradient: D[128 x ncols] (+)= P^T Q with P = tile [128 rows x 128 cols] at p_addr and
// Q = tile [128 rows x ncols] at q_addr, both read MN-major (reduction over the rows, 16 per MMA)
__device__ __forceinline__ void issue_wgrad(uint32_t d, uint32_t p_addr, uint32_t q_addr, int ncols, bool accumulate) {
  const uint32_t idesc = tc05::idesc_bf16(ncols, true, true);
  for (int r = 0; r < kTileRows / 16; ++r) {
    const uint64_t da = tc05::smem_desc(p_addr + (uint32_t)r * 256u, 128, kChunk);
    const uint64_t db = tc05::smem_desc(q_addr + (uint32_t)r * 256u, 128, kChunk);
    tc05::mma_ss(d, da, db, idesc, accumulate || r > 0);
  }
}

__device__ __forceinline__ void load_chunk2(const unsigned char* buf, int chunk, int row, float* v) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint4 u = *reinterpret_cast<const uint4*>(buf + ((size_t)(chunk + h) * kTileRows + row) * 16);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(p[i]);
      v[8 * h + 2 * i] = f.x; v[8 * h + 2 * i + 1] = f.y;
    }
  }
}

// Back-propagate 16 columns [N0, N0+16) of d(x1) into df; x1 = [f(27), d(3), sin(f), sin(2f) interleaved
// from 30, cos(f), cos(2f) interleaved from 84, direction terms from 138].
template <int N0>
__device__ __forceinline__ void pe_backward_cols(const float* v, const float* f, float* df) {
#pragma unroll
  for (int j = 0; j < 16; j += 2) {
    constexpr int dummy = 0; (void)dummy;
    const int c = N0 + j;                      // even column; pairs (c, c+1) never straddle a block edge
    if (c < 27) {
      df[c] += v[j];
      if (c + 1 < 27) df[c + 1] += v[j + 1];
    } else if (c >= 30 && c < 84) {
      const int i = (c - 30) >> 1;
      float s1, c1;
      __sincosf(f[i], &s1, &c1);
      df[i] += v[j] * c1 + v[j + 1] * 2.f * (1.f - 2.f * s1 * s1);
    } else if (c >= 84 && c < 138) {
      const int i = (c - 84) >> 1;
      float s1, c1;
      __sincosf(f[i], &s1, &c1);
      df[i] -= v[j] * s1 + v[j + 1] * 4.f * s1 * c1;
    }
  }
}

// status words: 0 ok, 1 weight load timed out, 2 input tile load timed out, 3 MMA completion timed out
//
// kPE = true : the colour head described above (4 GEMM layers, positional-encoding stage after the first).
// kPE = false: a plain three-layer perceptron on the same machinery - x1 [rows, 160] is the input itself (column 159
//              holds ones so that dW1[:, 159] is the bias gradient), h1 = relu(W1 x1 + b1), h2 = relu(W2 h1 + b2),
//              out = act(W3 h2 + b3) with up to 16 outputs and act = sigmoid or identity; widths are zero-padded to
//              160 -> 128 -> 128 -> 16 by the host (padded units stay at relu(0) = 0 and receive no gradient), and a
//              two-layer network passes W2 = I, b2 = 0 (relu(h1) = h1).  This covers the 64-wide density / colour heads
//              of the hash-grid models (benchmarks/nerf/instant_ngp/instant_ngp.py:120-170 of the reference, which
//              trains them through tiny-cuda-nn).  dx receives all 160 input columns.
template <bool kPE>
__global__ void __launch_bounds__(kBwdThreads, 1)
mlp_bwd_kernel(const __grid_constant__ CUtensorMap xmap, const unsigned char* __restrict__ blob, MLPSpec spec,
                   const int* __restrict__ count_ptr, long long max_rows, const float* __restrict__ dout, int dout_stride,
                   __nv_bfloat16* __restrict__ dx, float* __restrict__ gbuf, int* __restrict__ status) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (tc05::smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* wsm = smem;
  unsigned char* bufA = smem + ((spec.blob_bytes + 1023) & ~1023);
  unsigned char* bufH1 = bufA + kBufA;
  unsigned char* bufHZ = bufH1 + kBufH1;
  unsigned char* bufS = bufHZ + kBufHZ;
  __shared__ __align__(8) uint64_t bar_w, bar_in, bar_x0, bar_mma;
  __shared__ uint32_t tmem_base_sh;

  const int row = threadIdx.x;                 // tile row == TMEM lane of this thread
  const int warp = row >> 5, lane = row & 31;
  if (row == 0) {
    tc05::mbar_init(&bar_w, 1); tc05::mbar_init(&bar_in, 1); tc05::mbar_init(&bar_x0, 1); tc05::mbar_init(&bar_mma, 1);
    tc05::fence_barrier_init();
  }
  if (row < 32) tc05::tmem_alloc(&tmem_base_sh, 512);
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tmem = tmem_base_sh;
  const uint32_t tlane = tmem + ((uint32_t)(warp * 32) << 16);

  const long long n_rows = resolve_count(count_ptr, max_rows);
  const long long n_tiles = (n_rows + kTileRows - 1) / kTileRows;
  const int K0 = spec.K[0];
  const int in_chunks = spec.in_width >> 3, k0_chunks = K0 >> 3;
  const uint32_t in_bytes = (uint32_t)in_chunks * kChunk, x0_bytes = (uint32_t)k0_chunks * kChunk;
  const uint32_t aA = tc05::smem_u32(bufA), aH1 = tc05::smem_u32(bufH1), aHZ = tc05::smem_u32(bufHZ), aS = tc05::smem_u32(bufS);
  constexpr int L1 = kPE ? 1 : 0;                // index of the first 128-wide layer in the spec
  constexpr int kOut = kPE ? 3 : 16;             // output columns that can carry a gradient
  const uint32_t aW0 = tc05::smem_u32(wsm + spec.w_off[0]), aW1 = tc05::smem_u32(wsm + spec.w_off[L1]);
  const uint32_t aW2 = tc05::smem_u32(wsm + spec.w_off[L1 + 1]), aW3 = tc05::smem_u32(wsm + spec.w_off[L1 + 2]);
  const float* b1 = reinterpret_cast<const float*>(wsm + spec.b_off[L1]);
  const float* b2 = reinterpret_cast<const float*>(wsm + spec.b_off[L1 + 1]);
  const float* b3 = reinterpret_cast<const float*>(wsm + spec.b_off[L1 + 2]);
  const bool out_sigmoid = spec.act[L1 + 2] == ACT_SIGMOID;
  // biases that ride in the GEMM (a column of the weights against the ones column of the layer's input) or are zero
  const bool skip_b1 = (spec.bias_in_gemm >> L1) & 1, skip_b2 = (spec.bias_in_gemm >> (L1 + 1)) & 1;
  const int k_fwd2 = (skip_b2 && spec.K[L1 + 1] == 144) ? 144 : 128;
  // plain network with two layers only (K of the middle layer given as 0): h1 feeds the output layer directly and the
  // middle layer's recompute, mask, weight-gradient and data-gradient groups are skipped
  // hidden layers of at most 64 real units (the hash-grid heads): the padded upper halves of h1 / h2 / dz are zero and
  // stay zero, so they are written once below and the epilogues walk 64 columns instead of 128
  const int hid = (!kPE && spec.hidden_cols > 0 && spec.hidden_cols <= 64) ? 64 : 128;
  const bool two_layers = !kPE && spec.K[1] == 0;
  const uint32_t aH2 = two_layers ? aH1 : aHZ;
  const int n_out = kPE ? 3 : spec.out_dim;
  (void)aW0;

  bool in_pending = false, x0_pending = false;
  long long tile = blockIdx.x;
  if (row == 0) {
    tc05::mbar_expect_tx(&bar_w, (uint32_t)spec.blob_bytes);
    tc05::tma_bulk_g2s(wsm, blob, (uint32_t)spec.blob_bytes, &bar_w);
    if (tile < n_tiles) {
      tc05::mbar_expect_tx(&bar_in, in_bytes);
      for (int c = 0; c < in_chunks; ++c) tc05::tma_load_3d(bufA + (size_t)c * kChunk, &xmap, 0, c, (int)(tile * kTileRows), &bar_in);
    }
  }
  in_pending = tile < n_tiles;
  bool ok = tc05::mbar_wait(&bar_w, 0);
  ok = __syncthreads_and(ok);
  if (!ok && row == 0) atomicExch(status, 1);

  uint32_t ph_in = 0, ph_x0 = 0, ph_mma = 0;
  bool first = true;
  float db3[kOut];
#pragma unroll
  for (int i = 0; i < kOut; ++i) db3[i] = 0.f;

  // one MMA group: thread 0 has issued the instructions; commit, bounded wait, agree, fence
#define LMB_MMA_WAIT()                                                                        \
  {                                                                                           \
    if (row == 0) tc05::mma_commit(&bar_mma);                                                 \
    bool done_ = tc05::mbar_wait(&bar_mma, ph_mma);                                           \
    ph_mma ^= 1;                                                                              \
    if (!__syncthreads_and(done_)) { if (row == 0) atomicExch(status, 3); ok = false; break; } \
    tc05::fence_after_sync();                                                                 \
  }
  // shared-memory writes and TMEM reads of all threads are finished before thread 0 issues again
#define LMB_EPILOGUE_DONE()       \
  {                               \
    tc05::fence_before_sync();    \
    tc05::fence_async_shared();   \
    __syncthreads();              \
    if (row == 0) tc05::fence_after_sync(); \
  }

  if constexpr (!kPE) {
    // An input narrower than the 160-column operand: the copies fill chunks [0, in_chunks) of every tile, the rest is
    // written once here - zeros, and ones in column 159 (the bias column of dW1) - and never touched again.
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (int c = in_chunks; c < 20; ++c)
      *reinterpret_cast<uint4*>(bufA + ((size_t)c * kTileRows + row) * 16) = (c == 19) ? make_uint4(0, 0, 0, 0x3F800000u) : z;
    if (hid < 128) {
      for (int c = hid >> 3; c < 16; ++c) {
        *reinterpret_cast<uint4*>(bufH1 + ((size_t)c * kTileRows + row) * 16) = z;
        *reinterpret_cast<uint4*>(bufHZ + ((size_t)c * kTileRows + row) * 16) = z;
      }
    }
  }

  for (; ok && tile < n_tiles; tile += gridDim.x) {
    const long long row0 = tile * kTileRows;
    const bool valid = row0 + row < n_rows;
    const bool partial = row0 + kTileRows > n_rows;
    {
      bool got = tc05::mbar_wait(&bar_in, ph_in);
      ph_in ^= 1;
      in_pending = false;
      if (!__syncthreads_and(got)) { if (row == 0) atomicExch(status, 2); ok = false; break; }
    }
    if constexpr (kPE) {
      float dir[3];
  #pragma unroll
      for (int i = 0; i < 3; ++i) dir[i] = valid ? load_elem(bufA, spec.dir_col + i, row) : 0.f;

      // ================= forward recompute =================
      if (row == 0) { tc05::fence_after_sync(); issue_fwd(tmem + kColWork, aA, aW0, K0, 32); }
      LMB_MMA_WAIT();
      {
        float f[32];
        tc05::tmem_ld16(tlane + kColWork, f);
        tc05::tmem_ld16(tlane + kColWork + 16, f + 16);
        float x[160];
  #pragma unroll
        for (int i = 0; i < 27; ++i) {
          const float fi = valid ? f[i] : 0.f;
          x[i] = fi;
          float s1, c1;
          __sincosf(fi, &s1, &c1);
          x[30 + 2 * i] = s1; x[31 + 2 * i] = 2.f * s1 * c1;
          x[84 + 2 * i] = c1; x[85 + 2 * i] = 1.f - 2.f * s1 * s1;
        }
  #pragma unroll
        for (int i = 0; i < 3; ++i) {
          x[27 + i] = dir[i];
          float s1, c1;
          __sincosf(dir[i], &s1, &c1);
          x[138 + 2 * i] = s1; x[139 + 2 * i] = 2.f * s1 * c1;
          x[144 + 2 * i] = c1; x[145 + 2 * i] = 1.f - 2.f * s1 * s1;
        }
        x[150] = 1.f;                               // ones column: dW1[:, 150] becomes the bias gradient
  #pragma unroll
        for (int i = 151; i < 160; ++i) x[i] = 0.f;
  #pragma unroll
        for (int c = 0; c < 20; ++c) store_chunk(bufA, c, row, x + 8 * c);
      }
      LMB_EPILOGUE_DONE();
    } else {
      if (partial && !valid) {                    // rows past the end hold arbitrary bits: 0 * NaN must not reach dW1
        const uint4 z = make_uint4(0, 0, 0, 0);
        for (int c = 0; c < in_chunks; ++c) *reinterpret_cast<uint4*>(bufA + ((size_t)c * kTileRows + row) * 16) = z;
      }
      LMB_EPILOGUE_DONE();
    }

    if (row == 0) issue_fwd(tmem + kColWork, aA, aW1, 160, 128);
    LMB_MMA_WAIT();
    for (int n0 = 0; n0 < hid; n0 += 64) {                       // 64 accumulator columns per wait: load latencies overlap
      float v[64];
      tc05::tmem_ld64(tlane + kColWork + n0, v);
      if (!skip_b1) {
#pragma unroll
        for (int i = 0; i < 64; i += 4) {             // four biases per shared-memory load
          const float4 b4 = *reinterpret_cast<const float4*>(b1 + n0 + i);
          v[i] += b4.x; v[i + 1] += b4.y; v[i + 2] += b4.z; v[i + 3] += b4.w;
        }
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) store_chunk_relu(bufH1, (n0 >> 3) + c, row, v + 8 * c);   // relu inside the bf16 packing
    }
    {
      float ones[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) ones[i] = 1.f;  // ones chunk: dW2[:, 128] becomes the bias gradient
      store_chunk(bufH1, 16, row, ones);
      store_chunk(bufH1, 17, row, ones);
    }
    LMB_EPILOGUE_DONE();

    if (!two_layers) {
    if (row == 0) issue_fwd(tmem + kColWork, aH1, aW2, k_fwd2, 128);      // 144: the ones chunk of h1 times the bias column
    LMB_MMA_WAIT();
    for (int n0 = 0; n0 < hid; n0 += 64) {
      float v[64];
      tc05::tmem_ld64(tlane + kColWork + n0, v);
      if (!skip_b2) {
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
          const float4 b4 = *reinterpret_cast<const float4*>(b2 + n0 + i);
          v[i] += b4.x; v[i + 1] += b4.y; v[i + 2] += b4.z; v[i + 3] += b4.w;
        }
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) store_chunk_relu(bufHZ, (n0 >> 3) + c, row, v + 8 * c);
    }
    LMB_EPILOGUE_DONE();
    }

    if (row == 0) issue_fwd(tmem + kColWork, aH2, aW3, 128, 16);
    LMB_MMA_WAIT();
    {
      float v[16], dz[16];
      tc05::tmem_ld16(tlane + kColWork, v);
#pragma unroll
      for (int i = 0; i < 16; ++i) dz[i] = 0.f;
      if (valid) {
        const float* g = dout + (row0 + row) * (long long)dout_stride;
#pragma unroll
        for (int i = 0; i < kOut; ++i) {
          if (i < n_out) {
            const float o = __fdividef(1.f, 1.f + __expf(-(v[i] + b3[i])));
            dz[i] = out_sigmoid ? g[i] * o * (1.f - o) : g[i];
            db3[i] += dz[i];
          }
        }
      }
      store_chunk(bufS, 0, row, dz);
      store_chunk(bufS, 1, row, dz + 8);
    }
    LMB_EPILOGUE_DONE();

    // ================= layer 3 =================
    if (row == 0) {
      issue_wgrad(tmem + kColDW3T, aH2, aS, 16, !first);          // dW3^T += h2^T dz3
      issue_dgrad(tmem + kColWork, aS, aW3, 16, 0, 128);          // dh2 = dz3 W3
    }
    LMB_MMA_WAIT();
    if (!two_layers) {
    for (int n0 = 0; n0 < hid; n0 += 64) {                         // dz2 = dh2 * [h2 > 0], in place of h2
      float v[64];
      tc05::tmem_ld64(tlane + kColWork + n0, v);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float h[16];
        load_chunk2(bufHZ, (n0 >> 3) + 2 * q, row, h);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[16 * q + i] = h[i] > 0.f ? v[16 * q + i] : 0.f;
        store_chunk(bufHZ, (n0 >> 3) + 2 * q, row, v + 16 * q);
        store_chunk(bufHZ, (n0 >> 3) + 2 * q + 1, row, v + 16 * q + 8);
      }
    }
    LMB_EPILOGUE_DONE();

    // ================= layer 2 =================
    if (row == 0) {
      issue_wgrad(tmem + kColDW2, aHZ, aH1, 144, !first);         // dW2 (+ db2) += dz2^T [h1 | 1]
      issue_dgrad(tmem + kColWork, aHZ, aW2, 128, 0, 128);        // dh1 = dz2 W2
    }
    LMB_MMA_WAIT();
    }
    for (int n0 = 0; n0 < hid; n0 += 64) {                         // dz1 = dh1 * [h1 > 0] -> HZ
      float v[64];
      tc05::tmem_ld64(tlane + kColWork + n0, v);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float h[16];
        load_chunk2(bufH1, (n0 >> 3) + 2 * q, row, h);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[16 * q + i] = h[i] > 0.f ? v[16 * q + i] : 0.f;
        store_chunk(bufHZ, (n0 >> 3) + 2 * q, row, v + 16 * q);
        store_chunk(bufHZ, (n0 >> 3) + 2 * q + 1, row, v + 16 * q + 8);
      }
    }
    LMB_EPILOGUE_DONE();

    if constexpr (kPE) {
      // ================= layer 1 =================
      if (row == 0) {
        // h1 is dead: bring the input tile back (x1 replaced it in A) for the layer-0 weight gradient
        tc05::mbar_expect_tx(&bar_x0, x0_bytes);
        for (int c = 0; c < k0_chunks; ++c) tc05::tma_load_3d(bufH1 + (size_t)c * kChunk, &xmap, 0, c, (int)row0, &bar_x0);
        issue_wgrad(tmem + kColDW1, aHZ, aA, 160, !first);          // dW1 (+ db1) += dz1^T [x1 | 1]
        issue_dgrad(tmem + kColWork, aHZ, aW1, 128, 0, 128);        // d(x1)[:, 0:128] = dz1 W1
      }
      x0_pending = true;
      LMB_MMA_WAIT();
      float f[32], df[27];
      load_chunk2(bufA, 0, row, f);
      load_chunk2(bufA, 2, row, f + 16);
  #pragma unroll
      for (int i = 0; i < 27; ++i) df[i] = 0.f;
      {
        float v[64];
        tc05::tmem_ld64(tlane + kColWork + 0, v);
        pe_backward_cols<0>(v, f, df);   pe_backward_cols<16>(v + 16, f, df);
        pe_backward_cols<32>(v + 32, f, df);  pe_backward_cols<48>(v + 48, f, df);
        tc05::tmem_ld64(tlane + kColWork + 64, v);
        pe_backward_cols<64>(v, f, df);  pe_backward_cols<80>(v + 16, f, df);
        pe_backward_cols<96>(v + 32, f, df);  pe_backward_cols<112>(v + 48, f, df);
      }
      LMB_EPILOGUE_DONE();
      if (row == 0) issue_dgrad(tmem + kColWork, aHZ, aW1, 128, 16, 16);   // d(x1)[:, 128:144]
      LMB_MMA_WAIT();
      {
        float v[16];
        tc05::tmem_ld16(tlane + kColWork, v);
        pe_backward_cols<128>(v, f, df);
        float o[32];
  #pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = i < 27 ? df[i] : 0.f;
  #pragma unroll
        for (int c = 0; c < 4; ++c) store_chunk(bufS, c, row, o + 8 * c);
      }
      {
        bool got = tc05::mbar_wait(&bar_x0, ph_x0);
        ph_x0 ^= 1;
        x0_pending = false;
        if (!__syncthreads_and(got)) { if (row == 0) atomicExch(status, 2); ok = false; break; }
        if (partial && !valid) {                    // rows past the end hold arbitrary bits: 0 * NaN must not reach dW0
          const uint4 z = make_uint4(0, 0, 0, 0);
          for (int c = 0; c < k0_chunks; ++c) *reinterpret_cast<uint4*>(bufH1 + ((size_t)c * kTileRows + row) * 16) = z;
        }
      }
      LMB_EPILOGUE_DONE();

      // ================= layer 0 =================
      const long long next = tile + gridDim.x;
      if (row == 0) {
        if (next < n_tiles) {                       // x1 is dead: prefetch the next tile's input into A
          tc05::mbar_expect_tx(&bar_in, in_bytes);
          for (int c = 0; c < in_chunks; ++c) tc05::tma_load_3d(bufA + (size_t)c * kChunk, &xmap, 0, c, (int)(next * kTileRows), &bar_in);
        }
        issue_wgrad(tmem + kColDW0T, aH1, aS, 32, !first);                         // dW0^T[0:128] += x0^T df
        if (K0 > 128) issue_wgrad(tmem + kColDW0T + 32, aH1 + 2 * kChunk, aS, 32, !first);   // input columns 16..143
        issue_dgrad(tmem + kColWork, aS, aW0, 32, 0, K0 < 128 ? K0 : 128);         // d(x0)[:, 0:128] = df W0
      }
      in_pending = next < n_tiles;
      LMB_MMA_WAIT();
      __nv_bfloat16* dxr = dx + (row0 + row) * (long long)spec.in_width;
      {
        const int n_main = K0 < 128 ? K0 : 128;
        for (int n0 = 0; n0 < n_main; n0 += 16) {
          float v[16];
          tc05::tmem_ld16(tlane + kColWork + n0, v);
          if (valid) {
            uint4 u[2];
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(u);
  #pragma unroll
            for (int i = 0; i < 8; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            *reinterpret_cast<uint4*>(dxr + n0) = u[0];
            *reinterpret_cast<uint4*>(dxr + n0 + 8) = u[1];
          }
        }
      }
      LMB_EPILOGUE_DONE();
      if (K0 > 128) {
        if (row == 0) issue_dgrad(tmem + kColWork, aS, aW0, 32, 16, K0 - 128);    // d(x0)[:, 128:K0]
        LMB_MMA_WAIT();
        for (int n0 = 0; n0 < K0 - 128; n0 += 16) {
          float v[16];
          tc05::tmem_ld16(tlane + kColWork + n0, v);
          if (valid) {
            uint4 u[2];
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(u);
  #pragma unroll
            for (int i = 0; i < 8; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            *reinterpret_cast<uint4*>(dxr + 128 + n0) = u[0];
            *reinterpret_cast<uint4*>(dxr + 128 + n0 + 8) = u[1];
          }
        }
        LMB_EPILOGUE_DONE();
      }
      if (valid) {                                  // direction / padding columns carry no gradient
        const uint4 z = make_uint4(0, 0, 0, 0);
        for (int c = k0_chunks; c < in_chunks; ++c) *reinterpret_cast<uint4*>(dxr + 8 * c) = z;
      }
    } else {
      // ================= layer 1 (plain input) =================
      if (row == 0) {
        issue_wgrad(tmem + kColDW1, aHZ, aA, 160, !first);          // dW1 (+ db1) += dz1^T x1   (x1[:, 159] = 1)
        issue_dgrad(tmem + kColWork, aHZ, aW1, 128, 0, 128);        // d(x1)[:, 0:128] = dz1 W1
      }
      LMB_MMA_WAIT();
      const long long next = tile + gridDim.x;
      __nv_bfloat16* dxr = dx + (row0 + row) * (long long)spec.in_width;
      for (int n0 = 0; n0 < 128; n0 += 16) {
        float v[16];
        tc05::tmem_ld16(tlane + kColWork + n0, v);
        if (valid) {
          uint4 u[2];
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(u);
#pragma unroll
          for (int i = 0; i < 8; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
          if (n0 < spec.in_width) *reinterpret_cast<uint4*>(dxr + n0) = u[0];
          if (n0 + 8 < spec.in_width) *reinterpret_cast<uint4*>(dxr + n0 + 8) = u[1];
        }
      }
      LMB_EPILOGUE_DONE();
      if (row == 0) {
        if (next < n_tiles) {                       // x1 is dead (its weight-gradient MMAs completed): prefetch the next tile
          tc05::mbar_expect_tx(&bar_in, in_bytes);
          for (int c = 0; c < in_chunks; ++c) tc05::tma_load_3d(bufA + (size_t)c * kChunk, &xmap, 0, c, (int)(next * kTileRows), &bar_in);
        }
        issue_dgrad(tmem + kColWork, aHZ, aW1, 128, 16, 32);        // d(x1)[:, 128:160]
      }
      in_pending = next < n_tiles;
      LMB_MMA_WAIT();
      for (int n0 = 0; n0 < 32; n0 += 16) {
        float v[16];
        tc05::tmem_ld16(tlane + kColWork + n0, v);
        if (valid) {
          uint4 u[2];
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(u);
#pragma unroll
          for (int i = 0; i < 8; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
          if (128 + n0 < spec.in_width) *reinterpret_cast<uint4*>(dxr + 128 + n0) = u[0];
          if (128 + n0 + 8 < spec.in_width) *reinterpret_cast<uint4*>(dxr + 128 + n0 + 8) = u[1];
        }
      }
      LMB_EPILOGUE_DONE();
    }
    first = false;
  }
#undef LMB_MMA_WAIT
#undef LMB_EPILOGUE_DONE

  // a bounded wait gave up: let copies that are still in flight land before shared memory is released
  if (in_pending) tc05::mbar_wait(&bar_in, ph_in);
  if (x0_pending) tc05::mbar_wait(&bar_x0, ph_x0);

  // ---- weight gradients leave the SM: one vector reduction per 4 accumulator columns ----------------
  if (ok && !first) {
    tc05::fence_after_sync();
    for (int n0 = 0; n0 < 160; n0 += 16) {
      float v[16];
      tc05::tmem_ld16(tlane + kColDW1 + n0, v);
      float* g = gbuf + kG_DW1 + row * 160 + n0;
#pragma unroll
      for (int i = 0; i < 16; i += 4) red_add_v4(g + i, v[i], v[i + 1], v[i + 2], v[i + 3]);
    }
    for (int n0 = 0; n0 < 144; n0 += 16) {
      float v[16];
      tc05::tmem_ld16(tlane + kColDW2 + n0, v);
      float* g = gbuf + kG_DW2 + row * 144 + n0;
#pragma unroll
      for (int i = 0; i < 16; i += 4) red_add_v4(g + i, v[i], v[i + 1], v[i + 2], v[i + 3]);
    }
    {
      float v[16];
      tc05::tmem_ld16(tlane + kColDW3T, v);
      float* g = gbuf + kG_DW3T + row * 16;
#pragma unroll
      for (int i = 0; i < 16; i += 4) red_add_v4(g + i, v[i], v[i + 1], v[i + 2], v[i + 3]);
    }
    if constexpr (kPE) {
      for (int half = 0; half < 2; ++half) {
        float v[32];
        tc05::tmem_ld16(tlane + kColDW0T + 32 * half, v);
        tc05::tmem_ld16(tlane + kColDW0T + 32 * half + 16, v + 16);
        // second accumulator covers input columns 16..143; only 128..143 (lanes 112..127) are new
        const int col = half == 0 ? row : row + 16;
        const bool take = half == 0 ? (col < K0) : (K0 > 128 && row >= 112 && col < K0);
        if (take) {
          float* g = gbuf + kG_DW0T + col * 32;
  #pragma unroll
          for (int i = 0; i < 32; i += 4) red_add_v4(g + i, v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kOut; ++i) {
      float s = db3[i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0 && i < n_out) atomicAdd(gbuf + kG_DB3 + i, s);
    }
  }

  tc05::fence_before_sync();
  __syncthreads();
  if (row < 32) tc05::tmem_dealloc(tmem_base_sh, 512);
}

}  // namespace lmb

using namespace lmb;

// x: [max_rows, 160] bf16 rows (features, direction at spec.dir_col, zeros); dout: fp32 [max_rows, dout_stride]
// (3 used); dx: bf16 [max_rows, 160] (written for the first `count` rows); gbuf: fp32 [lmb_rgb_mlp_bwd_gbuf_floats()],
// zeroed by the caller, receives dW1|dW2|dW3^T|dW0^T|db3 in the layout documented above.
LMB_API int lmb_rgb_mlp_bwd_gbuf_floats() { return kG_TOTAL; }

LMB_API int lmb_rgb_mlp_bwd(const void* x, const int* count_ptr, long long max_rows, const void* blob, const MLPSpec* spec,
                            const float* dout, int dout_stride, void* dx, float* gbuf, int* status, cudaStream_t stream) {
  if (max_rows <= 0) return 0;
  const MLPSpec& s = *spec;
  // the kernel is specialised to the colour-head shape; anything else is refused
  if (s.n_layers != 4 || !s.pe_stage || s.in_width != 160 || s.K[0] % 16 || s.K[0] < 16 || s.K[0] > 144 || s.N[0] != 32 ||
      s.K[1] != 160 || s.N[1] != 128 || (s.K[2] != 128 && s.K[2] != 144) || s.N[2] != 128 || s.K[3] != 128 || s.N[3] != 16 || s.out_dim != 3 ||
      s.b_off[0] >= 0 || s.b_off[1] < 0 || s.b_off[2] < 0 || s.b_off[3] < 0 || s.blob_bytes % 16 ||
      s.act[1] != ACT_RELU || s.act[2] != ACT_RELU || s.act[3] != ACT_SIGMOID || s.dir_col + 3 > 160)
    return (int)cudaErrorInvalidValue;
  CUtensorMap xmap;
  int rc = encode_input_map(&xmap, x, 160, max_rows);
  if (rc) return rc;
  const size_t smem = ((s.blob_bytes + 1023) & ~1023) + (size_t)(kBufA + kBufH1 + kBufHZ + kBufS) + 1024;
  if (smem > 226 * 1024) return (int)cudaErrorInvalidValue;
  static size_t configured = 0;
  if (smem > configured) {
    LMB_CUDA_TRY(cudaFuncSetAttribute(mlp_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long tiles = (max_rows + kTileRows - 1) / kTileRows;
  const int grid = (int)(tiles < sms ? tiles : sms);
  mlp_bwd_kernel<true><<<grid, kBwdThreads, smem, stream>>>(xmap, (const unsigned char*)blob, s, count_ptr, max_rows, dout,
                                                         dout_stride, (__nv_bfloat16*)dx, gbuf, status);
  LMB_LAUNCH_CHECK();
  return 0;
}

// Plain three-layer perceptron 160 -> 128 -> 128 -> 16 (padded widths, see the kernel's header).  x: bf16
// [max_rows, x_width], x_width a multiple of 8: either 160 with ones in column 159, or at most 152 - the kernel then
// supplies the zero columns and the ones column itself, so the caller pads nothing; dout: fp32 [max_rows, dout_stride]
// (spec.out_dim used); dx: bf16 [max_rows, x_width]; gbuf as for lmb_rgb_mlp_bwd (dW1 [128][160] with db1 in column
// 159, dW2 [128][144] with db2 in column 128, dW3^T [128][16], db3 [16]; the dW0^T block stays zero).
LMB_API int lmb_mlp3_bwd(const void* x, int x_width, const int* count_ptr, long long max_rows, const void* blob,
                         const MLPSpec* spec, const float* dout, int dout_stride, void* dx, float* gbuf, int* status,
                         cudaStream_t stream) {
  if (max_rows <= 0) return 0;
  if (x_width % 8 != 0 || x_width < 8 || (x_width > 152 && x_width != 160)) return (int)cudaErrorInvalidValue;
  MLPSpec s = *spec;
  if (s.n_layers != 3 || s.pe_stage || s.in_width != 160 || s.K[0] != 160 || s.N[0] != 128 || (s.K[1] != 128 && s.K[1] != 0) || s.N[1] != 128 ||
      s.K[2] != 128 || s.N[2] != 16 || s.out_dim < 1 || s.out_dim > 16 || s.b_off[0] < 0 || s.b_off[1] < 0 || s.b_off[2] < 0 ||
      s.blob_bytes % 16 || s.act[0] != ACT_RELU || s.act[1] != ACT_RELU || (s.act[2] != ACT_SIGMOID && s.act[2] != ACT_NONE) ||
      dout_stride < s.out_dim)
    return (int)cudaErrorInvalidValue;
  s.in_width = x_width;                      // the kernel's copy width and dx row pitch; the operand stays 160 wide
  CUtensorMap xmap;
  int rc = encode_input_map(&xmap, x, x_width, max_rows);
  if (rc) return rc;
  const size_t smem = ((s.blob_bytes + 1023) & ~1023) + (size_t)(kBufA + kBufH1 + kBufHZ + kBufS) + 1024;
  if (smem > 226 * 1024) return (int)cudaErrorInvalidValue;
  static size_t configured = 0;
  if (smem > configured) {
    LMB_CUDA_TRY(cudaFuncSetAttribute(mlp_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long tiles = (max_rows + kTileRows - 1) / kTileRows;
  const int grid = (int)(tiles < sms ? tiles : sms);
  mlp_bwd_kernel<false><<<grid, kBwdThreads, smem, stream>>>(xmap, (const unsigned char*)blob, s, count_ptr, max_rows, dout,
                                                            dout_stride, (__nv_bfloat16*)dx, gbuf, status);
  LMB_LAUNCH_CHECK();
  return 0;
}
